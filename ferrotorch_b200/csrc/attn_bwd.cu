// Flash-attention backward on tcgen05 / TMEM for sm_100a (bf16, head_dim 64/128, causal or
// full, GQA).  The reference has no GPU attention backward at all (its flash kernel is
// forward-only, ferrotorch-gpu/src/flash_attention.rs:628-687; the CPU backward is
// ferrotorch-nn/src/flash_attention.rs:59-647), so the math below is the standard
// recompute-from-LSE formulation of that CPU backward:
//     P  = exp(S * scale - lse)          S  = Q K^T
//     dP = dO V^T                        dS = P * (dP - delta) * scale,  delta = rowsum(dO * O)
//     dV = P^T dO      dK = dS^T Q       dQ = dS K
//
// Two launches of one templated kernel, each CTA owning a resident 128-row tile (TMEM lanes)
// and streaming 64-row blocks of the other side through a 2-stage TMA ring:
//   dK/dV pass: resident = keys j (K_j, V_j); streamed = queries (Q_c, dO_c) of every query
//               head in the KV group, so the GQA reduction happens in the TMEM accumulators.
//               Scores are computed transposed (S^T = K Q^T), so a thread owns a key row and
//               P^T / dS^T rows land in shared memory as K-major A operands.
//   dQ pass:    resident = queries i (Q_i, dO_i); streamed = keys (K_c, V_c); dQ += dS K_c.
// Per step: 2 score MMAs (128x64xD) into double-buffered TMEM; the softmax warps turn them into
// bf16 P / dS and write those back into tensor memory over the scores they came from (each warp
// over its own 32 score columns), and the 1-2 accumulate MMAs (128xDx64) take them from there as
// their A operand, with the streamed tile read MN-major as B.  Nothing of P / dS touches shared
// memory.  The softmax scale is applied once, to the accumulators in the epilogue.  In the dK/dV
// pass the per-query lse / delta of the next block are fetched one step ahead into shared memory.
// All waits are bounded.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int AB_R = 128;  // resident rows
constexpr int AB_C = 64;   // streamed block rows
constexpr int AB_THREADS = 384;  // 4 role warps + 8 softmax warps (2 per TMEM lane quarter)
constexpr int AB_SPLIT = 2;      // column halves of a score tile, one per softmax warpgroup

template <int HD, bool IS_DQ>
struct AttBwdCfg {
  static constexpr int R_TILE = AB_R * HD * 2;          // one resident operand
  static constexpr int C_TILE = AB_C * HD * 2;          // one streamed operand
  static constexpr int STAGES = HD == 128 ? 4 : 6;      // ring of streamed {C1, C2} pairs
  static constexpr int OFF_R = 0;
  static constexpr int OFF_C = 2 * R_TILE;
  static constexpr int OFF_LD = OFF_C + STAGES * 2 * C_TILE;           // lse/delta, 2 buffers
  static constexpr int OFF_BAR = OFF_LD + 2 * 2 * AB_C * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // TMEM columns: S[2] (64 each), dP[2] (64 each), accumulators of HD columns.  Softmax warp
  // `half` of a score buffer writes its 32 bf16 P (dS) columns, two per 32-bit column, into the
  // first 16 columns of its own 32-column half of S (dP).
  static constexpr int COL_S = 0, COL_DP = 128, COL_ACC0 = 256, COL_ACC1 = 256 + HD;
};

struct AttBwdParams {
  __nv_bfloat16* out0;  // dQ pass: dQ;  dK/dV pass: dK
  __nv_bfloat16* out1;  // dK/dV pass: dV
  long long ld0, ld1;   // token strides of out0 / out1
  const float* lse;     // [B, Hq, Sq] log-sum-exp in base 2 (+inf for fully masked rows)
  const float* delta;   // [B, Hq, Sq]
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_offset;
  float scale, scale_log2;
  int* status;
};

// delta[b, h, i] = sum_d dO[b, i, h, d] * O[b, i, h, d]; one warp per (token, head) row.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                  const float* __restrict__ lse, float* __restrict__ delta,
                                  float* __restrict__ lse2, int B, int Sq, int Hq, int D, long long ldo,
                                  long long lddo) {
  const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long total = static_cast<long long>(B) * Sq * Hq;
  if (w >= total) return;
  const int h = static_cast<int>(w % Hq);
  const long long tok = w / Hq;
  const __nv_bfloat16* op = o + tok * ldo + static_cast<long long>(h) * D;
  const __nv_bfloat16* dp = dout + tok * lddo + static_cast<long long>(h) * D;
  float s = 0.f;
  for (int d = lane * 2; d < D; d += 64) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(op + d));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dp + d));
    s += a.x * b.x + a.y * b.y;
  }
  s = warp_sum(s);
  if (lane == 0) {
    const int b_ = static_cast<int>(tok / Sq), i = static_cast<int>(tok % Sq);
    const long long idx = (static_cast<long long>(b_) * Hq + h) * Sq + i;
    delta[idx] = s;
    const float l = lse[idx];
    // base-2 log-sum-exp; a fully masked row (lse = -inf) gets +inf so that P = exp2(s - lse) = 0
    lse2[idx] = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
  }
}

// tmR1/tmR2: resident operands (dK/dV: K, V; dQ: Q, dO); tmC1/tmC2: streamed (dK/dV: Q, dO;
// dQ: K, V).  All are 3-D maps {heads*D, seq, batch} with 64-element (128-byte) boxes.
template <int HD, bool IS_DQ>
__global__ void __launch_bounds__(AB_THREADS, 1)
flash_bwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmR1, const __grid_constant__ CUtensorMap tmR2,
                         const __grid_constant__ CUtensorMap tmC1, const __grid_constant__ CUtensorMap tmC2,
                         const AttBwdParams p) {
  using Cfg = AttBwdCfg<HD, IS_DQ>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sR1 = sbase + Cfg::OFF_R, sR2 = sR1 + Cfg::R_TILE;
  const uint32_t sC = sbase + Cfg::OFF_C;    // stage s: C1 at sC + s*2*C_TILE, C2 right after
  constexpr int STAGES = Cfg::STAGES;
  enum { R_FULL = 0, C_FULL = 1, C_EMPTY = C_FULL + STAGES, S_FULL = C_EMPTY + STAGES, P_FULL = S_FULL + 2,
         ACC_FULL = P_FULL + 2, NBARS = ACC_FULL + 1 };
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8 * NBARS);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* ld_buf = reinterpret_cast<float*>(smem + Cfg::OFF_LD);  // [2 buffers][lse | delta][AB_C]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int batch = blockIdx.z;
  const int group = p.Hq / p.Hkv;
  // resident tile index; heavy tiles first under a causal mask
  int rblk, head_r;  // head_r: kv head (dK/dV) or q head (dQ)
  head_r = blockIdx.y;
  int c_begin, c_end, n_heads_iter;
  if constexpr (IS_DQ) {
    const int nb = (p.Sq + AB_R - 1) / AB_R;
    rblk = nb - 1 - blockIdx.x;
    c_begin = 0;
    int kv_end = p.Sk;
    if (p.causal) kv_end = min(p.Sk, rblk * AB_R + AB_R + p.causal_offset);
    c_end = kv_end > 0 ? (kv_end + AB_C - 1) / AB_C : 0;
    n_heads_iter = 1;
  } else {
    rblk = blockIdx.x;
    c_end = (p.Sq + AB_C - 1) / AB_C;
    c_begin = 0;
    if (p.causal) {
      const int first_q = rblk * AB_R - p.causal_offset;  // first query that sees key rblk*128
      c_begin = first_q > 0 ? first_q / AB_C : 0;
    }
    if (c_begin > c_end) c_begin = c_end;
    n_heads_iter = group;
  }
  const int r0 = rblk * AB_R;
  const int n_c = c_end - c_begin;
  const int n_iter = n_c * n_heads_iter;
  const int kv_head = IS_DQ ? head_r / group : head_r;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(bar(R_FULL), 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(C_FULL + s), 1);
      mbar_init(bar(C_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(P_FULL + s), 4 * AB_SPLIT);
    }
    mbar_init(bar(ACC_FULL), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmR1);
    tma_prefetch_desc(&tmR2);
    tma_prefetch_desc(&tmC1);
    tma_prefetch_desc(&tmC2);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // iteration t -> (query head, streamed block)
  auto iter_head = [&](int t) { return IS_DQ ? head_r : head_r * group + t / n_c; };
  auto iter_cblk = [&](int t) { return c_begin + (IS_DQ ? t : t % n_c); };

  if (warp == 0) {
    if (lane == 0 && n_iter > 0) {
      // resident operands: for dQ they belong to query head head_r, for dK/dV to kv head head_r
      mbar_expect_tx(bar(R_FULL), 2 * Cfg::R_TILE);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_3d(sR1 + c * (AB_R * 128), &tmR1, bar(R_FULL), head_r * HD + c * 64, r0, batch);
        tma_load_3d(sR2 + c * (AB_R * 128), &tmR2, bar(R_FULL), head_r * HD + c * 64, r0, batch);
      }
      for (int t = 0; t < n_iter; ++t) {
        const int st = t % STAGES;
        if (!mbar_wait(bar(C_EMPTY + st), ((t / STAGES) & 1) ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) break;
        const int hc = IS_DQ ? kv_head : iter_head(t);
        const int row = iter_cblk(t) * AB_C;
        const uint32_t c1 = sC + st * 2 * Cfg::C_TILE, c2 = c1 + Cfg::C_TILE;
        mbar_expect_tx(bar(C_FULL + st), 2 * Cfg::C_TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_3d(c1 + c * (AB_C * 128), &tmC1, bar(C_FULL + st), hc * HD + c * 64, row, batch);
          tma_load_3d(c2 + c * (AB_C * 128), &tmC2, bar(C_FULL + st), hc * HD + c * 64, row, batch);
        }
      }
      if (*abort_word) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(AB_R, AB_C, 1, 0, 0);   // 128 x 64, K-major both
      constexpr uint32_t idesc_acc = make_idesc_f16(AB_R, HD, 1, 0, 1);   // 128 x HD, B MN-major
      auto issue_scores = [&](int t) {
        const int st = t % STAGES, sb = t & 1;
        const uint32_t c1 = sC + st * 2 * Cfg::C_TILE, c2 = c1 + Cfg::C_TILE;
        const uint32_t dS_ = tmem_base + Cfg::COL_S + sb * AB_C;
        const uint32_t dP_ = tmem_base + Cfg::COL_DP + sb * AB_C;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t ro = (kk >> 2) * (AB_R * 128) + (kk & 3) * 32;
          const uint32_t co = (kk >> 2) * (AB_C * 128) + (kk & 3) * 32;
          umma_f16_ss(dS_, make_smem_desc_sw128(sR1 + ro, 16, 1024), make_smem_desc_sw128(c1 + co, 16, 1024),
                      idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t ro = (kk >> 2) * (AB_R * 128) + (kk & 3) * 32;
          const uint32_t co = (kk >> 2) * (AB_C * 128) + (kk & 3) * 32;
          umma_f16_ss(dP_, make_smem_desc_sw128(sR2 + ro, 16, 1024), make_smem_desc_sw128(c2 + co, 16, 1024),
                      idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(S_FULL + sb));
      };
      bool ok = mbar_wait(bar(R_FULL), 0, abort_word, FT_ERR_TIMEOUT_MMA) &&
                mbar_wait(bar(C_FULL + 0), 0, abort_word, FT_ERR_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int t = 0; t < n_iter && ok; ++t) {
        if (t + 1 < n_iter) {
          // The scores of step t+1 land in the buffer whose P / dS the MMAs of step t-1 read;
          // those were issued in the previous iteration and the tensor core runs in issue order.
          const int tn = t + 1;
          ok = mbar_wait(bar(C_FULL + tn % STAGES), (tn / STAGES) & 1, abort_word, FT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_scores(tn);
        }
        const int st = t % STAGES, sb = t & 1;
        if (!mbar_wait(bar(P_FULL + sb), (t >> 1) & 1, abort_word, FT_ERR_TIMEOUT_MMA)) { ok = false; break; }
        tc_fence_after();
        const uint32_t c1 = sC + st * 2 * Cfg::C_TILE, c2 = c1 + Cfg::C_TILE;
        const uint32_t aP = tmem_base + Cfg::COL_S + sb * AB_C;    // P^T (dK/dV pass)
        const uint32_t aS = tmem_base + Cfg::COL_DP + sb * AB_C;   // dS (dQ pass) / dS^T
        // the streamed tile as an MN-major B operand: 64-column chunks of [64 rows x 128 B];
        // A comes from tensor memory: k-step kk = 16 streamed rows = 8 columns, written by
        // softmax warp (kk >> 1) at the start of its own 32-column half
#pragma unroll
        for (int kk = 0; kk < AB_C / 16; ++kk) {
          const uint32_t ao = static_cast<uint32_t>(32 * (kk >> 1) + 8 * (kk & 1));
          if constexpr (IS_DQ) {
            // dQ += dS K_c
            umma_f16_ts(tmem_base + Cfg::COL_ACC0, aS + ao,
                        make_smem_desc_sw128(c1 + kk * 2048, AB_C * 128, 1024), idesc_acc,
                        (t > 0 || kk > 0) ? 1u : 0u);
          } else {
            // dK += dS^T Q_c ; dV += P^T dO_c
            umma_f16_ts(tmem_base + Cfg::COL_ACC0, aS + ao,
                        make_smem_desc_sw128(c1 + kk * 2048, AB_C * 128, 1024), idesc_acc,
                        (t > 0 || kk > 0) ? 1u : 0u);
            umma_f16_ts(tmem_base + Cfg::COL_ACC1, aP + ao,
                        make_smem_desc_sw128(c2 + kk * 2048, AB_C * 128, 1024), idesc_acc,
                        (t > 0 || kk > 0) ? 1u : 0u);
          }
        }
        umma_commit(bar(C_EMPTY + st));
      }
      if (ok) umma_commit(bar(ACC_FULL));
    }
  } else if (warp >= 4) {
    const int ew = warp & 3;             // TMEM lane quarter
    const int half = (warp - 4) >> 2;    // which 32 of the 64 score columns this warp handles
    const int r = ew * 32 + lane;
    const int grow = r0 + r;             // global row on the resident side
    const int sidx = threadIdx.x - 128;  // 0..255 among the softmax threads
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    float my_lse = INFINITY, my_delta = 0.f;
    if constexpr (IS_DQ) {
      if (grow < p.Sq) {
        const long long idx = (static_cast<long long>(batch) * p.Hq + head_r) * p.Sq + grow;
        my_lse = p.lse[idx];
        my_delta = p.delta[idx];
      }
    }
    // dK/dV pass: the statistics of the streamed queries.  Softmax threads 0..127 fetch the 64
    // lse and 64 delta values of step t+1 while step t is computed and publish them in shared
    // memory; a named barrier of the 256 softmax threads separates the writes from the reads.
    // Every softmax thread runs every iteration down to that barrier, also after a failed wait
    // (its later waits then fail at once), so the barrier can never be left short of arrivals.
    auto fetch_stat = [&](int t) -> float {
      const int j = sidx & (AB_C - 1);
      const int col = iter_cblk(t) * AB_C + j;
      if (col >= p.Sq) return sidx < AB_C ? INFINITY : 0.f;
      const long long idx = (static_cast<long long>(batch) * p.Hq + iter_head(t)) * p.Sq + col;
      return sidx < AB_C ? __ldg(p.lse + idx) : __ldg(p.delta + idx);
    };
    if constexpr (!IS_DQ) {
      if (sidx < 2 * AB_C && n_iter > 0) ld_buf[sidx] = fetch_stat(0);
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    bool ok = true;
    for (int t = 0; t < n_iter; ++t) {
      const int sb = t & 1;
      const int c0 = iter_cblk(t) * AB_C + half * 32;  // first global column of this thread
      float next_stat = 0.f;
      if constexpr (!IS_DQ) {
        if (sidx < 2 * AB_C && t + 1 < n_iter) next_stat = fetch_stat(t + 1);
      }
      // does any element of this 128 x 32 slab need masking?  (uniform per warp)
      bool need_mask;
      if constexpr (IS_DQ) {
        const int last_vis = p.causal ? min(p.Sk - 1, r0 + ew * 32 + p.causal_offset) : p.Sk - 1;
        need_mask = c0 + 31 > last_vis;
      } else {
        need_mask = (r0 + ew * 32 + 31 >= p.Sk) || (p.causal && r0 + ew * 32 + 31 > c0 + p.causal_offset);
      }
      if (ok && !mbar_wait(bar(S_FULL + sb), (t >> 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) ok = false;
      if (ok) {
        tc_fence_after();
        uint32_t a[32], b[32];
        tmem_ld_32x32(lane_addr + Cfg::COL_S + sb * AB_C + half * 32, a);
        tmem_ld_32x32(lane_addr + Cfg::COL_DP + sb * AB_C + half * 32, b);
        tmem_ld_wait();
        const float* st_lse = ld_buf + sb * 2 * AB_C + half * 32;
        const float* st_delta = st_lse + AB_C;
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          float lse4[4], delta4[4];
          if constexpr (IS_DQ) {
#pragma unroll
            for (int e = 0; e < 4; ++e) { lse4[e] = my_lse; delta4[e] = my_delta; }
          } else {
            const float4 l4 = *reinterpret_cast<const float4*>(st_lse + c);
            const float4 d4 = *reinterpret_cast<const float4*>(st_delta + c);
            lse4[0] = l4.x; lse4[1] = l4.y; lse4[2] = l4.z; lse4[3] = l4.w;
            delta4[0] = d4.x; delta4[1] = d4.y; delta4[2] = d4.z; delta4[3] = d4.w;
          }
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pe = fast_exp2(fmaf(__uint_as_float(a[c + e]), p.scale_log2, -lse4[e]));
            if (need_mask) {
              const int col = c0 + c + e;
              const bool visible = IS_DQ ? (col < p.Sk && (!p.causal || col <= grow + p.causal_offset))
                                         : (grow < p.Sk && (!p.causal || grow <= col + p.causal_offset));
              pe = visible ? pe : 0.f;
            }
            pv[e] = pe;
            dv[e] = pe * (__uint_as_float(b[c + e]) - delta4[e]);  // the softmax scale is applied in the epilogue
          }
          pk[c >> 1] = pack_bf16x2(pv[0], pv[1]);
          pk[(c >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
          dk[c >> 1] = pack_bf16x2(dv[0], dv[1]);
          dk[(c >> 1) + 1] = pack_bf16x2(dv[2], dv[3]);
        }
        // P / dS over the first 16 columns of this warp's own 32 score columns
        if constexpr (!IS_DQ) tmem_st_32x16(lane_addr + Cfg::COL_S + sb * AB_C + half * 32, pk);
        tmem_st_32x16(lane_addr + Cfg::COL_DP + sb * AB_C + half * 32, dk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(P_FULL + sb));
      }
      if constexpr (!IS_DQ) {
        if (sidx < 2 * AB_C && t + 1 < n_iter) ld_buf[(sb ^ 1) * 2 * AB_C + sidx] = next_stat;
        asm volatile("bar.sync 1, 256;" ::: "memory");
      }
    }
    // ---------------------------------------------------------------- epilogue
    if (ok && n_iter > 0) {
      ok = mbar_wait(bar(ACC_FULL), 0, abort_word, FT_ERR_TIMEOUT_EPILOGUE);
      tc_fence_after();
    }
    if (ok) {
      const int s_lim = IS_DQ ? p.Sq : p.Sk;
      const bool row_ok = grow < s_lim;
      const long long tok = static_cast<long long>(batch) * s_lim + grow;
#pragma unroll
      for (int acc = 0; acc < (IS_DQ ? 1 : 2); ++acc) {
        __nv_bfloat16* orow = (acc == 0 ? p.out0 + tok * p.ld0 : p.out1 + tok * p.ld1) +
                              static_cast<long long>(head_r) * HD;
        const uint32_t col = acc == 0 ? Cfg::COL_ACC0 : Cfg::COL_ACC1;
        const float osc = acc == 0 ? p.scale : 1.f;  // dQ and dK carry the softmax scale, dV does not
        // the two warps of a lane quarter split the HD columns
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          const int cc = half * (HD / 64) + c;  // 32-column chunk index
          uint32_t t32[32];
          if (n_iter > 0) {
            tmem_ld_32x32(lane_addr + col + cc * 32, t32);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) t32[i] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(t32[g * 8 + 0]) * osc, __uint_as_float(t32[g * 8 + 1]) * osc);
              o.y = pack_bf16x2(__uint_as_float(t32[g * 8 + 2]) * osc, __uint_as_float(t32[g * 8 + 3]) * osc);
              o.z = pack_bf16x2(__uint_as_float(t32[g * 8 + 4]) * osc, __uint_as_float(t32[g * 8 + 5]) * osc);
              o.w = pack_bf16x2(__uint_as_float(t32[g * 8 + 6]) * osc, __uint_as_float(t32[g * 8 + 7]) * osc);
              *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) = o;
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status) atomicCAS(p.status, 0, *abort_word);
}

template <int HD, bool IS_DQ>
static int launch_bwd(const CUtensorMap& r1, const CUtensorMap& r2, const CUtensorMap& c1,
                      const CUtensorMap& c2, const AttBwdParams& p, int device, cudaStream_t stream) {
  using Cfg = AttBwdCfg<HD, IS_DQ>;
  auto kern = flash_bwd_tcgen05_kernel<HD, IS_DQ>;
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set[device] = true;
  }
  dim3 grid(IS_DQ ? (p.Sq + AB_R - 1) / AB_R : (p.Sk + AB_R - 1) / AB_R, IS_DQ ? p.Hq : p.Hkv, p.B);
  kern<<<grid, AB_THREADS, Cfg::SMEM_BYTES, stream>>>(r1, r2, c1, c2, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}


// ----------------------------------------------------------------------------- fused single pass
// head_dim 128: one kernel computes dK, dV and dQ, so the scores are recomputed once (five MMA
// groups per step instead of seven over the two passes above, and one softmax instead of two).
// A CTA owns 128 keys of one KV head (K, V resident) and streams the 64-query blocks (Q_c, dO_c)
// of every query head of the group that attend to them:
//     S^T = K Q_c^T,  dP^T = V dO_c^T                         (128 keys x 64 queries, into TMEM)
//     P^T = exp2(S^T scale - lse),  dS^T = P^T (dP^T - delta)  (softmax warps; bf16 into shared memory)
//     dV += P^T dO_c,  dK += dS^T Q_c                          (accumulators in TMEM for the whole CTA)
//     dQ_c^T = K^T dS^T                                        (128 dims x 64 queries, a fresh TMEM tile)
// The dS^T tile in shared memory serves twice: as the K-major A operand of the dK product and as
// the MN-major B operand of the dQ product.  dQ_c^T is partial (this CTA's 128 keys only): four
// reduction warps read it from TMEM, transpose it into an fp32 [64 queries][128 dims] tile in
// shared memory and one TMA reduce-add per step adds that tile into an fp32 dQ accumulator in
// global memory (the memory system does the addition); a small kernel afterwards scales and
// rounds the accumulator to bf16.  The sum over key tiles therefore runs
// in arrival order: dQ can differ in its last bits from run to run (dK and dV cannot).
//   warp 0 TMA producer, warp 1 MMA issuer, warp 2 TMEM allocator,
//   warps 4-11 softmax (two per TMEM lane quarter, 32 score columns each), warps 12-15 dQ reduction
constexpr int AF_THREADS = 512;
constexpr int AF_STAGES = 2;

struct AttFusedCfg {
  static constexpr int HD = 128;
  static constexpr int R_TILE = AB_R * HD * 2;          // K or V: 32 KB
  static constexpr int C_TILE = AB_C * HD * 2;          // Q_c or dO_c: 16 KB
  static constexpr int PS_TILE = AB_R * AB_C * 2;       // P^T or dS^T: 128 rows x 128 bytes
  static constexpr int OFF_R = 0;
  static constexpr int OFF_C = 2 * R_TILE;
  static constexpr int OFF_PS = OFF_C + AF_STAGES * 2 * C_TILE;   // 2 buffers x {P^T, dS^T}
  static constexpr int DQ_TILE = AB_C * HD * 4;                   // dQ_c as fp32 [64 queries][128 dims]
  static constexpr int OFF_DQ = OFF_PS + 2 * 2 * PS_TILE;
  static constexpr int OFF_LD = OFF_DQ + DQ_TILE;                 // lse / delta, 2 buffers
  static constexpr int OFF_BAR = OFF_LD + 2 * 2 * AB_C * 4;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // TMEM columns
  static constexpr int COL_S = 0, COL_DP = 64, COL_DQ = 128 /* two buffers of 64 */, COL_DK = 256, COL_DV = 384;
};

struct AttFusedParams {
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  float* dq_acc;        // fp32 [B, Sq, Hq, D], zero on entry
  long long ldk, ldv;   // token strides of dk / dv
  const float* lse;     // base-2 log-sum-exp [B, Hq, Sq]
  const float* delta;   // [B, Hq, Sq]
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_offset;
  float scale, scale_log2;
  int* status;
};

// tmK / tmV: resident operands (128-row boxes); tmQ / tmDO: streamed (64-row boxes).
__global__ void __launch_bounds__(AF_THREADS, 1)
flash_bwd_fused_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                       const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmDO,
                       const __grid_constant__ CUtensorMap tmDQ, const AttFusedParams p) {
  using Cfg = AttFusedCfg;
  constexpr int HD = Cfg::HD;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sK = sbase + Cfg::OFF_R, sV = sK + Cfg::R_TILE;
  const uint32_t sC = sbase + Cfg::OFF_C;     // stage s: Q_c at sC + s*2*C_TILE, dO_c right after
  const uint32_t sPS = sbase + Cfg::OFF_PS;   // buffer b: P^T at sPS + b*2*PS_TILE, dS^T right after
  enum { R_FULL = 0, C_FULL = 1, C_EMPTY = C_FULL + AF_STAGES, S_FULL = C_EMPTY + AF_STAGES, S_READ = S_FULL + 1,
         P_FULL = S_READ + 1, PS_EMPTY = P_FULL + 2, DQ_FULL = PS_EMPTY + 2, DQ_EMPTY = DQ_FULL + 2,
         ACC_FULL = DQ_EMPTY + 2, NBARS = ACC_FULL + 1 };
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8 * NBARS);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* ld_buf = reinterpret_cast<float*>(smem + Cfg::OFF_LD);  // [2 buffers][lse | delta][AB_C]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int batch = blockIdx.z, kvh = blockIdx.y, rblk = blockIdx.x;
  const int group = p.Hq / p.Hkv;
  int c_end = (p.Sq + AB_C - 1) / AB_C, c_begin = 0;
  if (p.causal) {
    const int first_q = rblk * AB_R - p.causal_offset;  // first query that sees key rblk*128
    c_begin = first_q > 0 ? first_q / AB_C : 0;
  }
  if (c_begin > c_end) c_begin = c_end;
  const int r0 = rblk * AB_R;
  const int n_c = c_end - c_begin;
  const int n_iter = n_c * group;
  auto iter_head = [&](int t) { return kvh * group + t / n_c; };
  auto iter_cblk = [&](int t) { return c_begin + t % n_c; };

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(bar(R_FULL), 1);
    for (int s = 0; s < AF_STAGES; ++s) {
      mbar_init(bar(C_FULL + s), 1);
      mbar_init(bar(C_EMPTY + s), 1);
    }
    mbar_init(bar(S_FULL), 1);
    mbar_init(bar(S_READ), 4 * AB_SPLIT);      // every softmax warp has its scores in registers
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(P_FULL + s), 4 * AB_SPLIT);
      mbar_init(bar(PS_EMPTY + s), 1);
      mbar_init(bar(DQ_FULL + s), 1);
      mbar_init(bar(DQ_EMPTY + s), 4);
    }
    mbar_init(bar(ACC_FULL), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmDO);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0 && n_iter > 0) {
      mbar_expect_tx(bar(R_FULL), 2 * Cfg::R_TILE);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c) {
        tma_load_3d(sK + c * (AB_R * 128), &tmK, bar(R_FULL), kvh * HD + c * 64, r0, batch);
        tma_load_3d(sV + c * (AB_R * 128), &tmV, bar(R_FULL), kvh * HD + c * 64, r0, batch);
      }
      for (int t = 0; t < n_iter; ++t) {
        const int st = t % AF_STAGES;
        if (!mbar_wait(bar(C_EMPTY + st), ((t / AF_STAGES) & 1) ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) break;
        const int hc = iter_head(t), row = iter_cblk(t) * AB_C;
        const uint32_t c1 = sC + st * 2 * Cfg::C_TILE, c2 = c1 + Cfg::C_TILE;
        mbar_expect_tx(bar(C_FULL + st), 2 * Cfg::C_TILE);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          tma_load_3d(c1 + c * (AB_C * 128), &tmQ, bar(C_FULL + st), hc * HD + c * 64, row, batch);
          tma_load_3d(c2 + c * (AB_C * 128), &tmDO, bar(C_FULL + st), hc * HD + c * 64, row, batch);
        }
      }
      if (*abort_word) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_iter > 0) {
      constexpr uint32_t idesc_s = make_idesc_f16(AB_R, AB_C, 1, 0, 0);    // 128 keys x 64 queries, K-major both
      constexpr uint32_t idesc_acc = make_idesc_f16(AB_R, HD, 1, 0, 1);    // 128 keys x HD, A K-major, B MN-major
      constexpr uint32_t idesc_dq = make_idesc_f16(HD, AB_C, 1, 1, 1);     // HD dims x 64 queries, both MN-major
      auto issue_scores = [&](int t) {
        const uint32_t c1 = sC + (t % AF_STAGES) * 2 * Cfg::C_TILE, c2 = c1 + Cfg::C_TILE;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t ro = (kk >> 2) * (AB_R * 128) + (kk & 3) * 32;
          const uint32_t co = (kk >> 2) * (AB_C * 128) + (kk & 3) * 32;
          umma_f16_ss(tmem_base + Cfg::COL_S, make_smem_desc_sw128(sK + ro, 16, 1024),
                      make_smem_desc_sw128(c1 + co, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t ro = (kk >> 2) * (AB_R * 128) + (kk & 3) * 32;
          const uint32_t co = (kk >> 2) * (AB_C * 128) + (kk & 3) * 32;
          umma_f16_ss(tmem_base + Cfg::COL_DP, make_smem_desc_sw128(sV + ro, 16, 1024),
                      make_smem_desc_sw128(c2 + co, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(S_FULL));
      };
      bool ok = mbar_wait(bar(R_FULL), 0, abort_word, FT_ERR_TIMEOUT_MMA) &&
                mbar_wait(bar(C_FULL + 0), 0, abort_word, FT_ERR_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_scores(0);
      }
      for (int t = 0; t < n_iter && ok; ++t) {
        const int st = t % AF_STAGES, pb = t & 1;
        if (t + 1 < n_iter) {
          // the single S / dP buffer is free once every softmax warp holds the scores of step t
          ok = mbar_wait(bar(S_READ), t & 1, abort_word, FT_ERR_TIMEOUT_MMA) &&
               mbar_wait(bar(C_FULL + (t + 1) % AF_STAGES), ((t + 1) / AF_STAGES) & 1, abort_word, FT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_scores(t + 1);
        }
        ok = mbar_wait(bar(P_FULL + pb), (t >> 1) & 1, abort_word, FT_ERR_TIMEOUT_MMA) &&
             mbar_wait(bar(DQ_EMPTY + pb), ((t >> 1) & 1) ^ 1u, abort_word, FT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t c1 = sC + st * 2 * Cfg::C_TILE, c2 = c1 + Cfg::C_TILE;
        const uint32_t sPt = sPS + pb * 2 * Cfg::PS_TILE, sDSt = sPt + Cfg::PS_TILE;
#pragma unroll
        for (int kk = 0; kk < AB_C / 16; ++kk) {
          // dV += P^T dO_c ; dK += dS^T Q_c   (A: 128 keys x 64 queries K-major; B: streamed tile MN-major)
          umma_f16_ss(tmem_base + Cfg::COL_DV, make_smem_desc_sw128(sPt + kk * 32, 16, 1024),
                      make_smem_desc_sw128(c2 + kk * 2048, AB_C * 128, 1024), idesc_acc, (t > 0 || kk > 0) ? 1u : 0u);
          umma_f16_ss(tmem_base + Cfg::COL_DK, make_smem_desc_sw128(sDSt + kk * 32, 16, 1024),
                      make_smem_desc_sw128(c1 + kk * 2048, AB_C * 128, 1024), idesc_acc, (t > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bar(C_EMPTY + st));
#pragma unroll
        for (int kk = 0; kk < AB_R / 16; ++kk) {
          // dQ_c^T = K^T dS^T: A = K read MN-major (16 keys = 2048 bytes down each 64-dim chunk),
          // B = the dS^T tile read MN-major (64 queries contiguous, 16 keys = 2048 bytes)
          umma_f16_ss(tmem_base + Cfg::COL_DQ + pb * AB_C, make_smem_desc_sw128(sK + kk * 2048, AB_R * 128, 1024),
                      make_smem_desc_sw128(sDSt + kk * 2048, AB_C * 128, 1024), idesc_dq, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(DQ_FULL + pb));
        umma_commit(bar(PS_EMPTY + pb));
      }
      if (ok) umma_commit(bar(ACC_FULL));
    }
  } else if (warp >= 4 && warp < 12) {
    // ------------------------------------------------------------------ softmax
    const int ew = warp & 3;             // TMEM lane quarter
    const int half = (warp - 4) >> 2;    // which 32 of the 64 score columns this warp handles
    const int r = ew * 32 + lane;
    const int grow = r0 + r;             // global key row
    const int sidx = threadIdx.x - 128;  // 0..255 among the softmax threads
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    auto fetch_stat = [&](int t) -> float {
      const int j = sidx & (AB_C - 1);
      const int col = iter_cblk(t) * AB_C + j;
      if (col >= p.Sq) return sidx < AB_C ? INFINITY : 0.f;
      const long long idx = (static_cast<long long>(batch) * p.Hq + iter_head(t)) * p.Sq + col;
      return sidx < AB_C ? __ldg(p.lse + idx) : __ldg(p.delta + idx);
    };
    if (sidx < 2 * AB_C && n_iter > 0) ld_buf[sidx] = fetch_stat(0);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    bool ok = true;
    // Every softmax thread runs every iteration down to the named barrier, also after a failed
    // wait (its later waits then fail at once), so the barrier is never left short of arrivals.
    for (int t = 0; t < n_iter; ++t) {
      const int pb = t & 1;
      const int c0 = iter_cblk(t) * AB_C + half * 32;  // first global query column of this thread
      float next_stat = 0.f;
      if (sidx < 2 * AB_C && t + 1 < n_iter) next_stat = fetch_stat(t + 1);
      const bool need_mask = (r0 + ew * 32 + 31 >= p.Sk) || (p.causal && r0 + ew * 32 + 31 > c0 + p.causal_offset);
      if (ok && !mbar_wait(bar(S_FULL), t & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) ok = false;
      if (ok) {
        tc_fence_after();
        uint32_t a[32], b[32];
        tmem_ld_32x32(lane_addr + Cfg::COL_S + half * 32, a);
        tmem_ld_32x32(lane_addr + Cfg::COL_DP + half * 32, b);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(S_READ));
        const float* st_lse = ld_buf + pb * 2 * AB_C + half * 32;
        const float* st_delta = st_lse + AB_C;
        uint32_t pk[16], dk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 l4 = *reinterpret_cast<const float4*>(st_lse + c);
          const float4 d4 = *reinterpret_cast<const float4*>(st_delta + c);
          const float lse4[4] = {l4.x, l4.y, l4.z, l4.w}, delta4[4] = {d4.x, d4.y, d4.z, d4.w};
          float pv[4], dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float pe = fast_exp2(fmaf(__uint_as_float(a[c + e]), p.scale_log2, -lse4[e]));
            if (need_mask) {
              const int col = c0 + c + e;
              const bool visible = grow < p.Sk && (!p.causal || grow <= col + p.causal_offset);
              pe = visible ? pe : 0.f;
            }
            pv[e] = pe;
            dv[e] = pe * (__uint_as_float(b[c + e]) - delta4[e]);  // the softmax scale is applied at the end
          }
          pk[c >> 1] = pack_bf16x2(pv[0], pv[1]);
          pk[(c >> 1) + 1] = pack_bf16x2(pv[2], pv[3]);
          dk[c >> 1] = pack_bf16x2(dv[0], dv[1]);
          dk[(c >> 1) + 1] = pack_bf16x2(dv[2], dv[3]);
        }
        // the P^T / dS^T buffer of this parity was last read by the MMAs of step t - 2
        if (!mbar_wait(bar(PS_EMPTY + pb), ((t >> 1) & 1) ^ 1u, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) ok = false;
        if (ok) {
          const uint32_t ps = sPS + pb * 2 * Cfg::PS_TILE;
#pragma unroll
          for (int uu = 0; uu < 4; ++uu) {
            const int u = half * 4 + uu;
            const uint32_t off = r * 128 + ((u ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ps + off), "r"(pk[uu * 4]),
                         "r"(pk[uu * 4 + 1]), "r"(pk[uu * 4 + 2]), "r"(pk[uu * 4 + 3]) : "memory");
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(ps + Cfg::PS_TILE + off), "r"(dk[uu * 4]),
                         "r"(dk[uu * 4 + 1]), "r"(dk[uu * 4 + 2]), "r"(dk[uu * 4 + 3]) : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(P_FULL + pb));
        }
      }
      if (sidx < 2 * AB_C && t + 1 < n_iter) ld_buf[(pb ^ 1) * 2 * AB_C + sidx] = next_stat;
      asm volatile("bar.sync 1, 256;" ::: "memory");
    }
    // ---------------------------------------------------------------- dK / dV epilogue
    if (ok && n_iter > 0) {
      ok = mbar_wait(bar(ACC_FULL), 0, abort_word, FT_ERR_TIMEOUT_EPILOGUE);
      tc_fence_after();
    }
    if (ok) {
      const bool row_ok = grow < p.Sk;
      const long long tok = static_cast<long long>(batch) * p.Sk + grow;
#pragma unroll
      for (int acc = 0; acc < 2; ++acc) {
        __nv_bfloat16* orow = (acc == 0 ? p.dk + tok * p.ldk : p.dv + tok * p.ldv) + static_cast<long long>(kvh) * HD;
        const uint32_t col = acc == 0 ? Cfg::COL_DK : Cfg::COL_DV;
        const float osc = acc == 0 ? p.scale : 1.f;  // dK carries the softmax scale, dV does not
#pragma unroll
        for (int c = 0; c < HD / 64; ++c) {
          const int cc = half * (HD / 64) + c;  // 32-column chunk index
          uint32_t t32[32];
          if (n_iter > 0) {
            tmem_ld_32x32(lane_addr + col + cc * 32, t32);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) t32[i] = 0u;
          }
          if (row_ok) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 o;
              o.x = pack_bf16x2(__uint_as_float(t32[g * 8 + 0]) * osc, __uint_as_float(t32[g * 8 + 1]) * osc);
              o.y = pack_bf16x2(__uint_as_float(t32[g * 8 + 2]) * osc, __uint_as_float(t32[g * 8 + 3]) * osc);
              o.z = pack_bf16x2(__uint_as_float(t32[g * 8 + 4]) * osc, __uint_as_float(t32[g * 8 + 5]) * osc);
              o.w = pack_bf16x2(__uint_as_float(t32[g * 8 + 6]) * osc, __uint_as_float(t32[g * 8 + 7]) * osc);
              *reinterpret_cast<uint4*>(orow + cc * 32 + g * 8) = o;
            }
          }
        }
      }
    }
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ dQ reduction
    const int ew = warp & 3;
    const int d = ew * 32 + lane;        // head dim of this thread (TMEM lane of dQ^T)
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    const uint32_t sDQ = sbase + Cfg::OFF_DQ;
    bool ok = true;
    // every reduction thread runs every iteration down to the named barriers (see the softmax warps)
    for (int t = 0; t < n_iter; ++t) {
      const int pb = t & 1;
      if (ok && !mbar_wait(bar(DQ_FULL + pb), (t >> 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) ok = false;
      uint32_t v0[32], v1[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) v0[j] = v1[j] = 0u;
      if (ok) {
        tc_fence_after();
        tmem_ld_32x32(lane_addr + Cfg::COL_DQ + pb * AB_C, v0);
        tmem_ld_32x32(lane_addr + Cfg::COL_DQ + pb * AB_C + 32, v1);
        tmem_ld_wait();
        // both halves are in registers: the MMA warp may overwrite this dQ buffer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(DQ_EMPTY + pb));
      }
      // the staging tile is free once the previous step's reduce has read it
      if (threadIdx.x == 12 * 32) tma_store_wait_read<0>();
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ok) {
        // transpose: thread d writes column d of the [64 queries][128 dims] tile (a warp writes
        // 32 consecutive floats of one row: no bank conflicts)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(sDQ + static_cast<uint32_t>(j * HD + d) * 4u), "r"(v0[j]) : "memory");
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(sDQ + static_cast<uint32_t>((32 + j) * HD + d) * 4u), "r"(v1[j])
                       : "memory");
        }
        fence_proxy_async_smem();
      }
      asm volatile("bar.sync 2, 128;" ::: "memory");
      if (ok && threadIdx.x == 12 * 32) {
        // dq_acc[batch, q0 .. q0+63, head, :] += tile (queries past Sq are clipped by the tensor map)
        asm volatile(
            "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];"
            :
            : "l"(reinterpret_cast<uint64_t>(&tmDQ)), "r"(sDQ), "r"(iter_head(t) * HD), "r"(iter_cblk(t) * AB_C), "r"(batch)
            : "memory");
        tma_store_commit();
      }
    }
    if (threadIdx.x == 12 * 32) tma_store_wait<0>();   // shared memory must outlive the reduce that reads it
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status) atomicCAS(p.status, 0, *abort_word);
}

// dq[i] = bf16(acc[i] * scale) over [B*Sq, Hq*D] (dq rows have stride lddq elements).
__global__ void attn_dq_finalize_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long long rows,
                                        int width, long long lddq, float scale) {
  const int wv = width >> 2;
  const long long total = rows * wv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long rr = i / wv;
    const int c = static_cast<int>(i - rr * wv) << 2;
    const float4 v = *reinterpret_cast<const float4*>(acc + rr * width + c);
    uint2 o;
    o.x = pack_bf16x2(v.x * scale, v.y * scale);
    o.y = pack_bf16x2(v.z * scale, v.w * scale);
    *reinterpret_cast<uint2*>(dq + rr * lddq + c) = o;
  }
}

}  // namespace ft

// Gradients of ft_flash_attn_fwd.  q/k/v/o/dout/dq/dk/dv are [B, S, H, D] with packed heads and
// the given token strides (elements); lse [B, Hq, Sq] from the forward; delta_scratch: 2*B*Hq*Sq
// floats of scratch (16-byte aligned).  dq/dk/dv are fully overwritten.  dq_acc (optional):
// B*Sq*Hq*D floats of scratch; with it, head_dim 128 runs the fused single-pass kernel (dQ summed
// over key tiles by TMA reduce-adds in arrival order, so its last bits can vary from run to run);
// without it, and for head_dim 64, the two-pass kernels run (bit-reproducible).
FT_API int ft_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                             const float* lse, void* dq, void* dk, void* dv, float* delta_scratch, float* dq_acc, int B,
                             int Sq, int Sk, int Hq, int Hkv, int D, long long ldq, long long ldk,
                             long long ldv, long long ldo, long long lddq, long long lddk, long long lddv,
                             float scale, int causal, int causal_offset, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  using namespace ft;
  FT_REQUIRE(q && k && v && o && dout && lse && dq && dk && dv && delta_scratch, "ft_flash_attn_bwd: null pointer");
  FT_REQUIRE(D == 64 || D == 128, "ft_flash_attn_bwd: head_dim %d not supported (64, 128)", D);
  FT_REQUIRE(B > 0 && Sq > 0 && Sk > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "ft_flash_attn_bwd: bad shape");
  FT_REQUIRE(ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && ldo % 8 == 0 && lddq % 8 == 0 &&
                 lddk % 8 == 0 && lddv % 8 == 0,
             "ft_flash_attn_bwd: token strides must be multiples of 8 elements");
  {
    const long long rows = static_cast<long long>(B) * Sq * Hq;
    const int threads = 256;
    const long long blocks = (rows * 32 + threads - 1) / threads;
    attn_delta_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(dout), lse, delta_scratch,
        delta_scratch + rows, B, Sq, Hq, D, ldo, static_cast<long long>(Hq) * D);
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  CUtensorMap tq_r, tdo_r, tk_r, tv_r, tq_c, tdo_c, tk_c, tv_c;
  const long long lddo = static_cast<long long>(Hq) * D;
  auto mk = [&](CUtensorMap* m, const void* base, int H, int S, long long ld, int box_rows) {
    return make_tmap_3d(m, base, 2, static_cast<uint64_t>(H) * D, S, B, ld * 2,
                        static_cast<uint64_t>(S) * ld * 2, 64, box_rows, 1, 3);
  };
  int rc;
  if ((rc = mk(&tk_r, k, Hkv, Sk, ldk, AB_R))) return rc;
  if ((rc = mk(&tv_r, v, Hkv, Sk, ldv, AB_R))) return rc;
  if ((rc = mk(&tq_c, q, Hq, Sq, ldq, AB_C))) return rc;
  if ((rc = mk(&tdo_c, dout, Hq, Sq, lddo, AB_C))) return rc;
  if ((rc = mk(&tq_r, q, Hq, Sq, ldq, AB_R))) return rc;
  if ((rc = mk(&tdo_r, dout, Hq, Sq, lddo, AB_R))) return rc;
  if ((rc = mk(&tk_c, k, Hkv, Sk, ldk, AB_C))) return rc;
  if ((rc = mk(&tv_c, v, Hkv, Sk, ldv, AB_C))) return rc;

  if (dq_acc && D == 128) {
    FT_REQUIRE((reinterpret_cast<uintptr_t>(dq_acc) & 15) == 0 && lddq % 4 == 0,
               "ft_flash_attn_bwd: dq_acc must be 16-byte aligned");
    const long long n_acc = static_cast<long long>(B) * Sq * Hq * D;
    FT_CUDA_CHECK(cudaMemsetAsync(dq_acc, 0, n_acc * sizeof(float), stream));
    AttFusedParams f;
    f.dk = static_cast<__nv_bfloat16*>(dk); f.dv = static_cast<__nv_bfloat16*>(dv); f.dq_acc = dq_acc;
    f.ldk = lddk; f.ldv = lddv;
    f.lse = delta_scratch + static_cast<long long>(B) * Sq * Hq; f.delta = delta_scratch;
    f.B = B; f.Sq = Sq; f.Sk = Sk; f.Hq = Hq; f.Hkv = Hkv;
    f.causal = causal; f.causal_offset = causal_offset;
    f.scale = scale; f.scale_log2 = scale * 1.4426950408889634f;
    f.status = device_status_word(device);
    static bool attr_set[64] = {false};
    if (!attr_set[device]) {
      FT_CUDA_CHECK(cudaFuncSetAttribute(flash_bwd_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         AttFusedCfg::SMEM_BYTES));
      attr_set[device] = true;
    }
    // dq_acc as {Hq*D, Sq, B} fp32; one box = 128 dims x 64 queries, unswizzled (512-byte rows)
    CUtensorMap tdq;
    rc = make_tmap_3d(&tdq, dq_acc, 4, static_cast<uint64_t>(Hq) * D, Sq, B, static_cast<uint64_t>(Hq) * D * 4,
                      static_cast<uint64_t>(Sq) * Hq * D * 4, 128, AB_C, 1, 0);
    if (rc) return rc;
    dim3 grid((Sk + AB_R - 1) / AB_R, Hkv, B);
    flash_bwd_fused_kernel<<<grid, AF_THREADS, AttFusedCfg::SMEM_BYTES, stream>>>(tk_r, tv_r, tq_c, tdo_c, tdq, f);
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
    const long long rows_q = static_cast<long long>(B) * Sq;
    const long long work = rows_q * (static_cast<long long>(Hq) * D / 4);
    long long blocks = (work + 255) / 256;
    const long long cap = static_cast<long long>(sm_count(device)) * 16;
    if (blocks > cap) blocks = cap;
    attn_dq_finalize_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        dq_acc, static_cast<__nv_bfloat16*>(dq), rows_q, Hq * D, lddq, scale);
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
    return FT_E_OK;
  }

  AttBwdParams p;
  p.lse = delta_scratch + static_cast<long long>(B) * Sq * Hq; p.delta = delta_scratch;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.causal = causal; p.causal_offset = causal_offset;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  p.status = device_status_word(device);
  // dK / dV
  p.out0 = static_cast<__nv_bfloat16*>(dk); p.ld0 = lddk;
  p.out1 = static_cast<__nv_bfloat16*>(dv); p.ld1 = lddv;
  rc = D == 128 ? launch_bwd<128, false>(tk_r, tv_r, tq_c, tdo_c, p, device, stream)
                : launch_bwd<64, false>(tk_r, tv_r, tq_c, tdo_c, p, device, stream);
  if (rc) return rc;
  // dQ
  p.out0 = static_cast<__nv_bfloat16*>(dq); p.ld0 = lddq;
  p.out1 = nullptr; p.ld1 = 0;
  return D == 128 ? launch_bwd<128, true>(tq_r, tdo_r, tk_c, tv_c, p, device, stream)
                  : launch_bwd<64, true>(tq_r, tdo_r, tk_c, tv_c, p, device, stream);
}
