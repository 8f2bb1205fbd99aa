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
// Decode attention is bandwidth bound (every cached byte is read once per step); the kernel
// reads K with one key per lane (full 256-byte rows, no shuffles in the dot products) and V
// with one row per warp step (coalesced), fp32 math.
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
