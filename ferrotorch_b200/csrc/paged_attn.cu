// Paged KV cache on the device: block tables, append, and single-token decode attention.
//
// The reference keeps its paged cache as a host-side data structure that no kernel consumes
// (PagePool / PagedKVCache / PagedAttentionManager, ferrotorch-nn/src/paged_attention.rs:73-532)
// and its GPU decode path re-runs the whole prefix (ferrotorch-llama/src/gpu.rs:549-788).  Here
// the cache is two device arrays [num_blocks, block_size, n_kv_heads, head_dim] (bf16) and an
// int32 block table [batch, max_blocks_per_seq]; token t of sequence b lives in block
// table[b][t / block_size] at row t % block_size.
//
//   ft_kv_append        scatter new K/V rows (a prefill chunk or one decode token per sequence)
//                       into the cache through the block table.
//   ft_paged_decode     one query token per sequence: softmax(q K^T / sqrt(d)) V over the cached
//                       context, GQA (all query heads of a KV group share one pass over K/V),
//                       flash-decoding split over the context with a second combine pass.
// Decode attention is bandwidth bound (every cached byte is read once per step).  head_dim 128
// runs on the tensor-core kernel (paged_decode_tc_kernel: cp.async rows -> shared memory ->
// tcgen05.mma); head_dim 64 on the CUDA-core kernel, which reads K with
// one key per lane (full rows, no shuffles in the dot products) and V with one row per warp step.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int PD_THREADS = 128;
constexpr int PD_WARPS = PD_THREADS / 32;
constexpr int PD_MAX_G = 8;

// k_new / v_new: [T, Hkv, D] rows with token stride ld (elements).  Token i goes to sequence
// seq_ids[i] (or i / tokens_per_seq when null) at position pos[i].
__global__ void kv_append_kernel(const __nv_bfloat16* __restrict__ k_new, const __nv_bfloat16* __restrict__ v_new,
                                 __nv_bfloat16* __restrict__ k_cache, __nv_bfloat16* __restrict__ v_cache,
                                 const int* __restrict__ block_table, const int* __restrict__ pos,
                                 const int* __restrict__ seq_ids, int T, int tokens_per_seq, int Hkv, int D,
                                 long long ldk, long long ldv, int block_size, int max_blocks, int num_blocks) {
  const int row_vec = (Hkv * D) >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const int b = seq_ids ? seq_ids[t] : t / tokens_per_seq;
    const int p = pos[t];
    const int blk = block_table[static_cast<long long>(b) * max_blocks + p / block_size];
    if (blk < 0 || blk >= num_blocks) continue;  // host validates; never write out of range
    const long long dst = (static_cast<long long>(blk) * block_size + p % block_size) * Hkv * D;
    const uint4* ks = reinterpret_cast<const uint4*>(k_new + static_cast<long long>(t) * ldk);
    const uint4* vs = reinterpret_cast<const uint4*>(v_new + static_cast<long long>(t) * ldv);
    uint4* kd = reinterpret_cast<uint4*>(k_cache + dst);
    uint4* vd = reinterpret_cast<uint4*>(v_cache + dst);
    for (int i = threadIdx.x; i < row_vec; i += blockDim.x) {
      kd[i] = ks[i];
      vd[i] = vs[i];
    }
  }
}

// grid (n_splits, Hkv, B).  Each CTA covers tiles of 32 keys, strided over its warps, inside its
// slice of the context; partial (m, l, o) per (b, q head, split) go to scratch when n_splits > 1.
// Scores: lane j owns key j of the tile and reads its whole row (all loads issued before the
// math).  PV: the two half-warps take even / odd keys, each lane owns 8 (D=128) or 4 (D=64)
// output dims, V rows are read 8 keys at a time with 16-byte (8-byte) loads.
template <int D, int G>
__global__ void __launch_bounds__(PD_THREADS)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache, const int* __restrict__ block_table,
                    const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                    float* __restrict__ part_ml, int Hq, int Hkv, long long ldq, long long ldo, int block_size,
                    int max_blocks, int num_blocks, float scale_log2, int n_splits) {
  constexpr int DV = D / 16;  // dims per lane in the PV phase (half-warp covers D)
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane >> 4, hl = lane & 15;
  const int len = ctx_len[b];
  const int tiles_total = (len + 31) >> 5;
  const int tiles_per_split = (tiles_total + n_splits - 1) / n_splits;
  const int tile_lo = split * tiles_per_split, tile_hi = min(tiles_total, tile_lo + tiles_per_split);

  __shared__ __align__(16) float s_q[G][D];          // q * scale * log2(e)
  __shared__ float s_p[PD_WARPS][G][32];             // probabilities of the current tile
  __shared__ float s_m[PD_WARPS][G], s_l[PD_WARPS][G];
  __shared__ __align__(16) float s_o[PD_WARPS][G][D];

  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    s_q[g][d] = __bfloat162float(q[static_cast<long long>(b) * ldq + static_cast<long long>(kvh * G + g) * D + d]) * scale_log2;
  }
  __syncthreads();

  float m[G], l[G], o[G][DV];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DV; ++j) o[g][j] = 0.f;
  }
  const int* bt = block_table + static_cast<long long>(b) * max_blocks;
  const long long row_stride = static_cast<long long>(Hkv) * D;
  const long long head_off = static_cast<long long>(kvh) * D;

  for (int tile = tile_lo + warp; tile < tile_hi; tile += PD_WARPS) {
    const int key0 = tile << 5;
    // ---- scores: lane j owns key key0 + j; issue the whole row's loads, then the dot products
    const int key = key0 + lane;
    const bool valid = key < len;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    {
      const int kk = valid ? key : key0;
      int blk = bt[kk / block_size];
      blk = min(max(blk, 0), num_blocks - 1);
      const uint4* kr = reinterpret_cast<const uint4*>(
          k_cache + (static_cast<long long>(blk) * block_size + kk % block_size) * row_stride + head_off);
      uint4 kv[D / 8];
#pragma unroll
      for (int c = 0; c < D / 8; ++c) kv[c] = __ldg(kr + c);
#pragma unroll
      for (int c = 0; c < D / 8; ++c) {
        const float2 k0 = unpack_bf16x2(kv[c].x), k1 = unpack_bf16x2(kv[c].y), k2 = unpack_bf16x2(kv[c].z),
                     k3 = unpack_bf16x2(kv[c].w);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float4 qa = *reinterpret_cast<const float4*>(&s_q[g][c * 8]);
          const float4 qb = *reinterpret_cast<const float4*>(&s_q[g][c * 8 + 4]);
          s[g] += k0.x * qa.x + k0.y * qa.y + k1.x * qa.z + k1.y * qa.w + k2.x * qb.x + k2.y * qb.y + k3.x * qb.z + k3.y * qb.w;
        }
      }
    }
    // ---- online softmax per head across the 32 lanes
    float alpha[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float sv = valid ? s[g] : -INFINITY;
      const float mx = warp_max(sv);
      const float m_new = fmaxf(m[g], mx);
      const float pv = valid ? fast_exp2(sv - m_new) : 0.f;
      alpha[g] = fast_exp2(m[g] - m_new);  // exp2(-inf) = 0 on the first tile
      l[g] = l[g] * alpha[g] + warp_sum(pv);
      m[g] = m_new;
      s_p[warp][g][lane] = pv;
#pragma unroll
      for (int j = 0; j < DV; ++j) o[g][j] *= alpha[g];
    }
    __syncwarp();
    // ---- O += P V: half-warp `half` takes keys key0 + 2*i + half; 8 keys (per half) in flight
    const int n_keys = min(32, len - key0);
    for (int i0 = 0; i0 < 16; i0 += 8) {
      if (2 * i0 >= n_keys) break;
      uint4 vv[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j = 2 * (i0 + i) + half;
        const int kj = key0 + min(j, n_keys - 1);
        int blk = bt[kj / block_size];
        blk = min(max(blk, 0), num_blocks - 1);
        const __nv_bfloat16* vr = v_cache + (static_cast<long long>(blk) * block_size + kj % block_size) * row_stride +
                                  head_off + hl * DV;
        if constexpr (DV == 8) {
          vv[i] = __ldg(reinterpret_cast<const uint4*>(vr));
        } else {
          const uint2 t = __ldg(reinterpret_cast<const uint2*>(vr));
          vv[i] = make_uint4(t.x, t.y, 0u, 0u);
        }
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int j = 2 * (i0 + i) + half;
        if (j < n_keys) {
          float f[8];
          const float2 a0 = unpack_bf16x2(vv[i].x), a1 = unpack_bf16x2(vv[i].y);
          f[0] = a0.x; f[1] = a0.y; f[2] = a1.x; f[3] = a1.y;
          if constexpr (DV == 8) {
            const float2 a2 = unpack_bf16x2(vv[i].z), a3 = unpack_bf16x2(vv[i].w);
            f[4] = a2.x; f[5] = a2.y; f[6] = a3.x; f[7] = a3.y;
          }
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float pj = s_p[warp][g][j];
#pragma unroll
            for (int e = 0; e < DV; ++e) o[g][e] += pj * f[e];
          }
        }
      }
    }
    __syncwarp();
  }

  // ---- combine the two half-warps, then the warps of this CTA
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int e = 0; e < DV; ++e) o[g][e] += __shfl_xor_sync(0xffffffffu, o[g][e], 16);
    if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
    if (half == 0) {
#pragma unroll
      for (int e = 0; e < DV; ++e) s_o[warp][g][hl * DV + e] = o[g][e];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < PD_WARPS; ++w) mm = fmaxf(mm, s_m[w][g]);
    float ll = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < PD_WARPS; ++w) {
      const float sc = (s_m[w][g] == -INFINITY) ? 0.f : fast_exp2(s_m[w][g] - mm);
      ll += s_l[w][g] * sc;
      acc += s_o[w][g][d] * sc;
    }
    const int hq = kvh * G + g;
    if (n_splits == 1) {
      out[static_cast<long long>(b) * ldo + static_cast<long long>(hq) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
    } else {
      const long long pidx = (static_cast<long long>(b) * Hq + hq) * n_splits + split;
      part_o[pidx * D + d] = acc;
      if (d == 0) { part_ml[pidx * 2] = mm; part_ml[pidx * 2 + 1] = ll; }
    }
  }
}

template <int D>
__global__ void paged_decode_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                            __nv_bfloat16* __restrict__ out, int Hq, long long ldo, int n_splits) {
  const int hq = blockIdx.x, b = blockIdx.y;
  const long long base = (static_cast<long long>(b) * Hq + hq) * n_splits;
  float mm = -INFINITY;
  for (int s = 0; s < n_splits; ++s) mm = fmaxf(mm, part_ml[(base + s) * 2]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float ll = 0.f, acc = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(base + s) * 2];
      const float sc = (ms == -INFINITY) ? 0.f : fast_exp2(ms - mm);
      ll += part_ml[(base + s) * 2 + 1] * sc;
      acc += part_o[(base + s) * D + d] * sc;
    }
    out[static_cast<long long>(b) * ldo + static_cast<long long>(hq) * D + d] = __float2bfloat16(ll > 0.f ? acc / ll : 0.f);
  }
}


// ----------------------------------------------------------------------------- tensor-core decode
// The decode kernel for head_dim 128 (any page size).  A CTA owns one (sequence, KV head, context
// split) and walks its keys in tiles of 128; all query heads of the KV group ride along as the
// (padded) 16-wide N dimension of two small MMAs per tile:
//     S^T[key, head] = K_tile[key, :] . Q[head, :]          (M = 128 keys, N = 16, K = head_dim)
//     O^T[dim, head] += V_tile^T[dim, key] . P^T[key, head]  (M = head_dim rows, N = 16, K = 128 keys)
// so the cached K and V rows go from HBM to shared memory with 16-byte cp.async copies (a page of
// 16 tokens x one head is only 2 KB per 64-wide half, too small a box for TMA to move at
// bandwidth; four loader warps keep three 64 KB tiles in flight instead) and from there straight
// into the tensor core: no per-element CUDA-core arithmetic on the cache at all.  The four softmax warps (thread r = key r of the tile) only handle the
// 128 x G scores: tile maximum over the keys (warp shuffles + one exchange through shared
// memory), lazy rescale of O^T in tensor memory, P^T as bf16 into a small shared-memory operand.
//   warp 1: MMA issuer     warp 2: TMEM allocator     warps 4-7: softmax / epilogue
//   warps 8-11: loaders (block-table lookups, cp.async into the 128-byte-swizzled operand
//   layout, rows past the context zero-filled; 3-stage ring of {K, V} tiles)
// Partial results use the same (m, l, o) scratch layout as paged_decode_kernel, so the combine
// pass is shared.  All waits are bounded.
constexpr int PT_THREADS = 384;
constexpr int PT_LOADERS = 128;  // warps 8-11
constexpr int PT_TILE = 128;   // keys per tile
constexpr int PT_STAGES = 3;
constexpr int PT_N = 16;       // MMA N: query heads of the group, zero-padded
constexpr float PT_RESCALE = 8.f;

template <int D>
struct PtCfg {  // D = 128 (an MMA with 64 rows lays its accumulator out differently)
  static constexpr int KV_BYTES = PT_TILE * D * 2;        // one K or V tile
  static constexpr int STAGE_BYTES = 2 * KV_BYTES;
  static constexpr int CHUNK = PT_TILE * 128;             // one 64-wide column chunk of a tile
  static constexpr int Q_BYTES = PT_N * D * 2;            // Q^T operand: 16 rows x head_dim
  static constexpr int P_BYTES = PT_N * PT_TILE * 2;      // P^T operand: 16 rows x 128 keys
  static constexpr int OFF_Q = PT_STAGES * STAGE_BYTES;
  static constexpr int OFF_P = OFF_Q + Q_BYTES;           // two buffers
  static constexpr int OFF_RED = OFF_P + 2 * P_BYTES;     // [4 warps][16] floats
  static constexpr int OFF_BAR = OFF_RED + 4 * PT_N * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
};

template <int D, int G>
__global__ void __launch_bounds__(PT_THREADS, 1)
paged_decode_tc_kernel(const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                       const __nv_bfloat16* __restrict__ q, const int* __restrict__ block_table,
                       const int* __restrict__ ctx_len, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                       float* __restrict__ part_ml, int Hq, int Hkv, long long ldq, long long ldo, int block_size,
                       int max_blocks, int num_blocks, float scale_log2, int n_splits, int* status) {
  using Cfg = PtCfg<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase + Cfg::OFF_Q, sP = sbase + Cfg::OFF_P;
  float* s_red = reinterpret_cast<float*>(smem + Cfg::OFF_RED);
  enum { KV_FULL = 0, ST_EMPTY = KV_FULL + PT_STAGES, S_FULL = ST_EMPTY + PT_STAGES,
         P_FULL = S_FULL + 2, O_DONE = P_FULL + 2, NBARS = O_DONE + 1 };
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8 * NBARS);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = ctx_len[b];
  const int tiles_total = (len + PT_TILE - 1) / PT_TILE;
  const int tiles_per_split = (tiles_total + n_splits - 1) / n_splits;
  const int tile_lo = split * tiles_per_split;
  const int n_tiles = max(0, min(tiles_total, tile_lo + tiles_per_split) - tile_lo);

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < PT_STAGES; ++s) {
      mbar_init(bar(KV_FULL + s), PT_LOADERS);   // every loader thread arrives once its copies have landed
      mbar_init(bar(ST_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(P_FULL + s), 4);
    }
    mbar_init(bar(O_DONE), 1);
    fence_mbar_init();
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), 64);
    tmem_relinquish();
  }
  // Q^T operand (scaled, bf16, rows >= G zero) and zeroed P^T buffers, written by all threads
  for (int i = threadIdx.x; i < (Cfg::Q_BYTES + 2 * Cfg::P_BYTES) / 16; i += blockDim.x)
    reinterpret_cast<uint4*>(smem + Cfg::OFF_Q)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  for (int i = threadIdx.x; i < G * (D / 8); i += blockDim.x) {
    const int g = i / (D / 8), j = i - g * (D / 8);  // 16-byte chunk j of head g
    const uint4 raw = *reinterpret_cast<const uint4*>(q + static_cast<long long>(b) * ldq +
                                                      static_cast<long long>(kvh * G + g) * D + j * 8);
    const float2 a0 = unpack_bf16x2(raw.x), a1 = unpack_bf16x2(raw.y), a2 = unpack_bf16x2(raw.z),
                 a3 = unpack_bf16x2(raw.w);
    uint4 o;
    o.x = pack_bf16x2(a0.x * scale_log2, a0.y * scale_log2);
    o.y = pack_bf16x2(a1.x * scale_log2, a1.y * scale_log2);
    o.z = pack_bf16x2(a2.x * scale_log2, a2.y * scale_log2);
    o.w = pack_bf16x2(a3.x * scale_log2, a3.y * scale_log2);
    const int c = j >> 3, jj = j & 7;                // 64-wide chunk, 16-byte unit inside it
    *reinterpret_cast<uint4*>(smem + Cfg::OFF_Q + c * (PT_N * 128) + g * 128 + ((jj ^ (g & 7)) << 4)) = o;
  }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t COL_S = 0, COL_O = 32;

  if (warp >= 8) {
    // ------------------------------------------------------------------ loaders
    // Thread lt copies 16-byte unit (lt & 15) of rows (lt >> 4) + 8 i, i = 0..15, of the K tile
    // and of the V tile: 16 consecutive threads read one 256-byte cache row.
    const int lt = threadIdx.x - 256;
    const int unit = lt & 15, row0 = lt >> 4;
    const int* bt = block_table + static_cast<long long>(b) * max_blocks;
    const long long row_stride = static_cast<long long>(Hkv) * D;
    const long long col_off = static_cast<long long>(kvh) * D + unit * 8;
    const uint32_t chunk_off = static_cast<uint32_t>(unit >> 3) * Cfg::CHUNK;
    constexpr int AHEAD = PT_STAGES - 1;
    bool ok = true;
    for (int t = 0; t < n_tiles + AHEAD; ++t) {
      // First hand over tile t - AHEAD (groups are committed once per iteration, so "at most
      // AHEAD - 1 groups pending" means its copies have landed).  This must come before the
      // wait below: the MMA warp needs tile t - AHEAD + 1 ... to make progress towards freeing
      // the stage this iteration is about to wait for.
      if (t >= AHEAD) {
        asm volatile("cp.async.wait_group %0;" ::"n"(AHEAD - 1) : "memory");
        fence_proxy_async_smem();
        if (ok) mbar_arrive(bar(KV_FULL + (t - AHEAD) % PT_STAGES));
      }
      if (t < n_tiles && ok) {
        const int st = t % PT_STAGES;
        ok = mbar_wait(bar(ST_EMPTY + st), ((t / PT_STAGES) & 1) ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER);
        if (ok) {
          const int key0 = (tile_lo + t) * PT_TILE;
          const uint32_t sK = sbase + st * Cfg::STAGE_BYTES + chunk_off, sV = sK + Cfg::KV_BYTES;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int row = row0 + 8 * i;
            const int key = key0 + row;
            const int page = key / block_size;
            int blk = (key < len && page < max_blocks) ? __ldg(bt + page) : 0;
            blk = min(max(blk, 0), num_blocks - 1);
            const long long src = (static_cast<long long>(blk) * block_size + key % block_size) * row_stride + col_off;
            const uint32_t dst = static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>((unit & 7) ^ (row & 7)) << 4);
            const uint32_t nbytes = key < len ? 16u : 0u;   // rows past the context are zero-filled
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sK + dst), "l"(k_cache + src), "r"(nbytes)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(sV + dst), "l"(v_cache + src), "r"(nbytes)
                         : "memory");
          }
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(PT_TILE, PT_N, 1, 0, 0);   // keys x heads, both K-major
      constexpr uint32_t idesc_pv = make_idesc_f16(D, PT_N, 1, 1, 0);         // dims x heads, A (V^T) MN-major
      auto issue_qk = [&](int t) {
        const uint32_t sK = sbase + (t % PT_STAGES) * Cfg::STAGE_BYTES;
        const uint32_t d = tmem_base + COL_S + (t & 1) * PT_N;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t ko = (kk >> 2) * Cfg::CHUNK + (kk & 3) * 32;
          const uint32_t qo = (kk >> 2) * (PT_N * 128) + (kk & 3) * 32;
          umma_f16_ss(d, make_smem_desc_sw128(sK + ko, 16, 1024), make_smem_desc_sw128(sQ + qo, 16, 1024),
                      idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(S_FULL + (t & 1)));
      };
      bool ok = mbar_wait(bar(KV_FULL + 0), 0, abort_word, FT_ERR_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) {
          // S buffer (t+1)&1 was last read by the softmax of tile t-1, which has arrived on P_FULL
          ok = mbar_wait(bar(KV_FULL + (t + 1) % PT_STAGES), ((t + 1) / PT_STAGES) & 1, abort_word, FT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_qk(t + 1);
        }
        const int st = t % PT_STAGES;
        ok = mbar_wait(bar(P_FULL + (t & 1)), (t >> 1) & 1, abort_word, FT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t sV = sbase + st * Cfg::STAGE_BYTES + Cfg::KV_BYTES;
        const uint32_t pb = sP + (t & 1) * Cfg::P_BYTES;
#pragma unroll
        for (int kk = 0; kk < PT_TILE / 16; ++kk) {
          // A = V^T: 16 keys = 2048 bytes down each 64-wide chunk, chunks CHUNK bytes apart
          umma_f16_ss(tmem_base + COL_O, make_smem_desc_sw128(sV + kk * 2048, Cfg::CHUNK, 1024),
                      make_smem_desc_sw128(pb + (kk >> 2) * (PT_N * 128) + (kk & 3) * 32, 16, 1024), idesc_pv,
                      (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bar(O_DONE));
        umma_commit(bar(ST_EMPTY + st));
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------------ softmax / epilogue
    const int ew = warp & 3;
    const int r = ew * 32 + lane;   // key of the tile while scoring, output dim in the epilogue
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    float m_ref[G], l_part[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { m_ref[g] = -INFINITY; l_part[g] = 0.f; }
    bool ok = true;
    // Every softmax thread runs every iteration down to the named barriers, also after a failed
    // wait (later waits then fail at once), so no barrier is ever left short of arrivals.
    for (int t = 0; t < n_tiles; ++t) {
      const int sb = t & 1;
      if (ok && !mbar_wait(bar(S_FULL + sb), (t >> 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) ok = false;
      uint32_t sv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) sv[i] = 0u;
      if (ok) {
        tc_fence_after();
        tmem_ld_32x16(lane_addr + COL_S + sb * PT_N, sv);
        tmem_ld_wait();
      }
      const int key = (tile_lo + t) * PT_TILE + r;
      const bool valid = key < len;
      float s[G], mx[G];
#pragma unroll
      for (int g = 0; g < G; ++g) {
        s[g] = valid ? __uint_as_float(sv[g]) : -INFINITY;
        mx[g] = warp_max(s[g]);
      }
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) s_red[ew * PT_N + g] = mx[g];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      float alpha[G];
      bool any_rescale = false;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float tile_max = fmaxf(fmaxf(s_red[g], s_red[PT_N + g]), fmaxf(s_red[2 * PT_N + g], s_red[3 * PT_N + g]));
        alpha[g] = 1.f;
        if (tile_max > m_ref[g] + PT_RESCALE) {   // the same decision in every thread
          alpha[g] = fast_exp2(m_ref[g] - tile_max);  // m_ref = -inf on the first tile -> 0
          m_ref[g] = tile_max;
          any_rescale = true;
        }
        l_part[g] *= alpha[g];
      }
      // O of the earlier tiles (and the P buffer of tile t-2) are free once PV(t-1) has completed
      if (t > 0 && ok && !mbar_wait(bar(O_DONE), (t - 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) ok = false;
      if (t > 0 && any_rescale && ok) {
        tc_fence_after();
        uint32_t ov[16];
        tmem_ld_32x16(lane_addr + COL_O, ov);   // this thread's output dim, one column per head
        tmem_ld_wait();
#pragma unroll
        for (int g = 0; g < G; ++g) ov[g] = __float_as_uint(__uint_as_float(ov[g]) * alpha[g]);
        tmem_st_32x16(lane_addr + COL_O, ov);
        tmem_st_wait();
      }
      // P^T[head g][key r] as bf16 into the K-major operand tile (rows >= G stay zero)
      {
        uint8_t* pb = smem + Cfg::OFF_P + sb * Cfg::P_BYTES + (r >> 6) * (PT_N * 128);
        const int kc = r & 63;
#pragma unroll
        for (int g = 0; g < G; ++g) {
          const float pv = valid ? fast_exp2(s[g] - m_ref[g]) : 0.f;
          const __nv_bfloat16 pb16 = __float2bfloat16(pv);
          l_part[g] += __bfloat162float(pb16);   // the sum of what the MMA will actually use
          *reinterpret_cast<__nv_bfloat16*>(pb + g * 128 + (((kc >> 3) ^ (g & 7)) << 4) + (kc & 7) * 2) = pb16;
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(bar(P_FULL + sb));
      // s_red is rewritten in the next iteration: every thread must have read it
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if (ok && n_tiles > 0) {
      ok = mbar_wait(bar(O_DONE), (n_tiles - 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE);
      tc_fence_after();
    }
    // total l per head: sum of the per-thread partial sums
    float l_tot[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float ws = warp_sum(l_part[g]);
      if (lane == 0) s_red[ew * PT_N + g] = ws;
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
    for (int g = 0; g < G; ++g) l_tot[g] = s_red[g] + s_red[PT_N + g] + s_red[2 * PT_N + g] + s_red[3 * PT_N + g];
    if (ok && r < D) {
      uint32_t ov[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) ov[i] = 0u;
      if (n_tiles > 0) {
        tmem_ld_32x16(lane_addr + COL_O, ov);
        tmem_ld_wait();
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const int hq = kvh * G + g;
        const float acc = __uint_as_float(ov[g]);
        if (n_splits == 1) {
          out[static_cast<long long>(b) * ldo + static_cast<long long>(hq) * D + r] =
              __float2bfloat16(l_tot[g] > 0.f ? acc / l_tot[g] : 0.f);
        } else {
          const long long pidx = (static_cast<long long>(b) * Hq + hq) * n_splits + split;
          part_o[pidx * D + r] = acc;
          if (r == 0) { part_ml[pidx * 2] = m_ref[g]; part_ml[pidx * 2 + 1] = l_tot[g]; }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 64);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && status) atomicCAS(status, 0, *abort_word);
}

}  // namespace ft

using namespace ft;

FT_API int ft_kv_append(const void* k_new, const void* v_new, void* k_cache, void* v_cache, const int* block_table,
                        const int* pos, const int* seq_ids, int T, int tokens_per_seq, int Hkv, int D,
                        long long ldk, long long ldv, int block_size, int max_blocks, int num_blocks,
                        int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(k_new && v_new && k_cache && v_cache && block_table && pos, "ft_kv_append: null pointer");
  FT_REQUIRE((Hkv * D) % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && block_size > 0 && (seq_ids || tokens_per_seq > 0),
             "ft_kv_append: bad layout");
  if (T <= 0) return FT_E_OK;
  const int grid = T < sm_count(device) * 8 ? T : sm_count(device) * 8;
  kv_append_kernel<<<grid, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(k_new), static_cast<const __nv_bfloat16*>(v_new),
                                             static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
                                             block_table, pos, seq_ids, T, tokens_per_seq, Hkv, D, ldk, ldv, block_size,
                                             max_blocks, num_blocks);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// Scratch floats needed for n_splits > 1: B * Hq * n_splits * (D + 2).
FT_API long long ft_paged_decode_scratch(int B, int Hq, int D, int n_splits) {
  return n_splits > 1 ? static_cast<long long>(B) * Hq * n_splits * (D + 2) : 0;
}

// q: [B, Hq, D] (row stride ldq), out: [B, Hq, D] (row stride ldo), ctx_len: int32 [B] = number of
// cached tokens to attend to (including the current one, which must already be appended).
FT_API int ft_paged_decode(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                           const int* ctx_len, void* out, float* scratch, int B, int Hq, int Hkv, int D,
                           long long ldq, long long ldo, int block_size, int max_blocks, int num_blocks,
                           float scale, int n_splits, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(q && k_cache && v_cache && block_table && ctx_len && out, "ft_paged_decode: null pointer");
  FT_REQUIRE(D == 64 || D == 128, "ft_paged_decode: head_dim %d not supported (64, 128)", D);
  FT_REQUIRE(Hq % Hkv == 0 && Hq / Hkv <= PD_MAX_G, "ft_paged_decode: group size %d not supported (max %d)", Hq / Hkv, PD_MAX_G);
  FT_REQUIRE(n_splits >= 1 && (n_splits == 1 || scratch), "ft_paged_decode: splits need scratch");
  if (B <= 0) return FT_E_OK;
  const float sl2 = scale * 1.4426950408889634f;
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + static_cast<long long>(B) * Hq * n_splits * D : nullptr;
  dim3 grid(n_splits, Hkv, B);
  const int G = Hq / Hkv;
  const bool tensor_core = D == 128 && (G == 1 || G == 2 || G == 4 || G == 8) && block_size >= 1 &&
                           (reinterpret_cast<uintptr_t>(q) & 15) == 0 && ldq % 8 == 0 &&
                           ((reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15) == 0;
  if (tensor_core) {
    using Cfg = PtCfg<128>;
    int* status = device_status_word(device);
#define FT_PT_LAUNCH(GG)                                                                                        \
  {                                                                                                             \
    auto kern = paged_decode_tc_kernel<128, GG>;                                                                \
    static bool attr_set[64] = {false};                                                                         \
    if (!attr_set[device]) {                                                                                    \
      FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));  \
      attr_set[device] = true;                                                                                  \
    }                                                                                                           \
    kern<<<grid, PT_THREADS, Cfg::SMEM_BYTES, stream>>>(                                                        \
        static_cast<const __nv_bfloat16*>(k_cache), static_cast<const __nv_bfloat16*>(v_cache),                \
        static_cast<const __nv_bfloat16*>(q), block_table, ctx_len, static_cast<__nv_bfloat16*>(out),           \
        part_o, part_ml, Hq, Hkv, ldq, ldo, block_size, max_blocks, num_blocks, sl2, n_splits, status);         \
  }
    switch (G) {
      case 1: FT_PT_LAUNCH(1) break;
      case 2: FT_PT_LAUNCH(2) break;
      case 4: FT_PT_LAUNCH(4) break;
      default: FT_PT_LAUNCH(8) break;
    }
#undef FT_PT_LAUNCH
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
    if (n_splits > 1) {
      dim3 g2(Hq, B);
      paged_decode_combine_kernel<128><<<g2, 128, 0, stream>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out), Hq, ldo, n_splits);
      FT_CUDA_CHECK(cudaGetLastError());
      count_launch();
    }
    return FT_E_OK;
  }
#define FT_PD_LAUNCH(DD, GG)                                                                                   \
  paged_decode_kernel<DD, GG><<<grid, PD_THREADS, 0, stream>>>(                                                \
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),                        \
      static_cast<const __nv_bfloat16*>(v_cache), block_table, ctx_len, static_cast<__nv_bfloat16*>(out),      \
      part_o, part_ml, Hq, Hkv, ldq, ldo, block_size, max_blocks, num_blocks, sl2, n_splits)
#define FT_PD_BY_G(DD)                                             \
  switch (G) {                                                     \
    case 1: FT_PD_LAUNCH(DD, 1); break;                            \
    case 2: FT_PD_LAUNCH(DD, 2); break;                            \
    case 4: FT_PD_LAUNCH(DD, 4); break;                            \
    case 8: FT_PD_LAUNCH(DD, 8); break;                            \
    default:                                                       \
      set_last_error("ft_paged_decode: group size %d not supported (1, 2, 4, 8)", G); \
      return FT_E_BAD_ARG;                                         \
  }
  if (D == 128) { FT_PD_BY_G(128) } else { FT_PD_BY_G(64) }
#undef FT_PD_BY_G
#undef FT_PD_LAUNCH
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  if (n_splits > 1) {
    dim3 g2(Hq, B);
    if (D == 128)
      paged_decode_combine_kernel<128><<<g2, 128, 0, stream>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out), Hq, ldo, n_splits);
    else
      paged_decode_combine_kernel<64><<<g2, 64, 0, stream>>>(part_o, part_ml, static_cast<__nv_bfloat16*>(out), Hq, ldo, n_splits);
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  return FT_E_OK;
}
