// Flash-attention forward on tcgen05 / TMEM for sm_100a: bf16, head_dim 64 or 128,
// causal or full, grouped-query attention without a materialised repeat_kv, LSE output.
//
// The reference materialises [heads, seq, seq] scores through two batched cuBLAS GEMMs, a
// mask kernel and a softmax kernel (ferrotorch-llama/src/gpu.rs:627-663) or, in its
// "flash" kernel, gives one thread one query row in fp32 CUDA cores
// (ferrotorch-gpu/src/flash_attention.rs:139-687).  Semantics kept: scale 1/sqrt(d),
// causal mask hides key j > query i (+ offset when the query block is the tail of a longer
// key sequence), max-subtracted softmax (ferrotorch-nn/src/flash_attention.rs:647-746).
//
// Two kernels: sequences of more than 128 queries run on the two-tile kernel described at
// flash_fwd2_tcgen05_kernel; shorter ones (decode-time prefill chunks, tests) on this one.
// One CTA per (128-query block, head, batch), 256 threads:
//   warp 0     TMA producer: Q once, then K/V tiles of 128 keys through 2-stage rings
//   warp 1     MMA issuer: S[j+1] = Q K[j+1]^T is issued before O += P[j] V[j] so the tensor
//              core works on the next scores while the softmax warps handle block j
//   warp 2     TMEM allocator (2 x 128 columns of S, head_dim columns of O)
//   warps 4-7  softmax: thread r owns query row r -- tcgen05.ld gives it the whole row, so
//              max/sum need no shuffles; P goes back through shared memory (128B swizzle)
//              as the A operand of the second MMA; O is rescaled in TMEM when a row max moves
// All waits are bounded and report through the device status word.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int ATT_BM = 128;
constexpr int ATT_BN = 128;
constexpr int ATT_THREADS = 256;
constexpr int ATT_KV_STAGES = 2;

template <int HD>
struct AttCfg {
  static constexpr int Q_BYTES = ATT_BM * HD * 2;
  static constexpr int KV_BYTES = ATT_BN * HD * 2;
  static constexpr int P_BYTES = ATT_BM * ATT_BN * 2;
  static constexpr int OFF_K = Q_BYTES;
  static constexpr int OFF_V = OFF_K + ATT_KV_STAGES * KV_BYTES;
  static constexpr int OFF_P = OFF_V + ATT_KV_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_P + P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 2 * ATT_BN;
};

struct AttParams {
  __nv_bfloat16* O;
  float* lse;
  long long ldo;  // token stride of O (elements)
  int B, Sq, Sk, Hq, Hkv;
  int causal, causal_offset;  // key j visible to query i iff j <= i + causal_offset
  float scale_log2;           // softmax scale * log2(e)
  int* status;
};

template <int HD>
__global__ void __launch_bounds__(ATT_THREADS, 1)
flash_fwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                         const __grid_constant__ CUtensorMap tmV, const AttParams p) {
  using Cfg = AttCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase, sK = sbase + Cfg::OFF_K, sV = sbase + Cfg::OFF_V, sP = sbase + Cfg::OFF_P;
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  // barrier slots
  enum { Q_FULL = 0, K_FULL = 1, K_EMPTY = 3, V_FULL = 5, V_EMPTY = 7, S_FULL = 9, S_EMPTY = 11,
         P_FULL = 13, O_DONE = 14, NBARS = 15 };
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8 * NBARS);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qblocks = (p.Sq + ATT_BM - 1) / ATT_BM;
  const int qb = n_qblocks - 1 - blockIdx.x;  // heaviest (latest) query blocks first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qb * ATT_BM;
  int kv_end = p.Sk;
  if (p.causal) kv_end = min(p.Sk, q0 + ATT_BM + p.causal_offset);
  const int n_blocks = kv_end > 0 ? (kv_end + ATT_BN - 1) / ATT_BN : 0;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(K_FULL + s), 1);
      mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);
      mbar_init(bar(V_EMPTY + s), 1);
      mbar_init(bar(S_FULL + s), 1);
      mbar_init(bar(S_EMPTY + s), 4);
    }
    mbar_init(bar(P_FULL), 4);
    mbar_init(bar(O_DONE), 1);
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0 && n_blocks > 0) {
      mbar_expect_tx(bar(Q_FULL), Cfg::Q_BYTES);
#pragma unroll
      for (int c = 0; c < HD / 64; ++c)
        tma_load_3d(sQ + c * (ATT_BM * 128), &tmQ, bar(Q_FULL), head * HD + c * 64, q0, batch);
      for (int j = 0; j < n_blocks; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1u;
        if (!mbar_wait(bar(K_EMPTY + st), par, abort_word, FT_ERR_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(bar(K_FULL + st), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(sK + st * Cfg::KV_BYTES + c * (ATT_BN * 128), &tmK, bar(K_FULL + st),
                      kv_head * HD + c * 64, j * ATT_BN, batch);
        if (!mbar_wait(bar(V_EMPTY + st), par, abort_word, FT_ERR_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(bar(V_FULL + st), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(sV + st * Cfg::KV_BYTES + c * (ATT_BN * 128), &tmV, bar(V_FULL + st),
                      kv_head * HD + c * 64, j * ATT_BN, batch);
      }
      if (*abort_word) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_blocks > 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(ATT_BM, ATT_BN, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(ATT_BM, HD, 1, 0, 1);
      auto issue_qk = [&](int j) {
        const int st = j & 1;
        const uint32_t kbase = sK + st * Cfg::KV_BYTES;
        const uint32_t d = tmem_base + static_cast<uint32_t>((j & 1) * ATT_BN);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (ATT_BM * 128) + (kk & 3) * 32;
          umma_f16_ss(d, make_smem_desc_sw128(sQ + off, 16, 1024),
                      make_smem_desc_sw128(kbase + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(S_FULL + (j & 1)));
        umma_commit(bar(K_EMPTY + st));
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_word, FT_ERR_TIMEOUT_MMA) &&
                mbar_wait(bar(K_FULL + 0), 0, abort_word, FT_ERR_TIMEOUT_MMA);
      if (ok) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < n_blocks && ok; ++j) {
        if (j + 1 < n_blocks) {
          const int jn = j + 1, st = jn & 1;
          ok = mbar_wait(bar(K_FULL + st), (jn >> 1) & 1, abort_word, FT_ERR_TIMEOUT_MMA) &&
               mbar_wait(bar(S_EMPTY + st), ((jn >> 1) & 1) ^ 1u, abort_word, FT_ERR_TIMEOUT_MMA);
          if (!ok) break;
          tc_fence_after();
          issue_qk(jn);
        }
        const int st = j & 1;
        ok = mbar_wait(bar(P_FULL), j & 1, abort_word, FT_ERR_TIMEOUT_MMA) &&
             mbar_wait(bar(V_FULL + st), (j >> 1) & 1, abort_word, FT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t vbase = sV + st * Cfg::KV_BYTES;
        const uint32_t d = tmem_base + Cfg::O_COL;
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk) {
          const uint32_t poff = (kk >> 2) * (ATT_BM * 128) + (kk & 3) * 32;
          umma_f16_ss(d, make_smem_desc_sw128(sP + poff, 16, 1024),
                      make_smem_desc_sw128(vbase + kk * 2048, ATT_BN * 128, 1024), idesc_pv,
                      (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(bar(O_DONE));
        umma_commit(bar(V_EMPTY + st));
      }
    }
  } else if (warp >= 4) {
    const int ew = warp & 3;
    const int r = ew * 32 + lane;  // row inside the tile == TMEM lane
    const int qrow = q0 + r;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    float m = -INFINITY, l = 0.f;
    bool ok = n_blocks > 0;
    for (int j = 0; j < n_blocks && ok; ++j) {
      const int sb = j & 1;
      if (!mbar_wait(bar(S_FULL + sb), (j >> 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      float s[ATT_BN];
#pragma unroll
      for (int c = 0; c < ATT_BN / 32; ++c) {
        uint32_t t[32];
        tmem_ld_32x32(lane_addr + sb * ATT_BN + c * 32, t);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(t[i]) * p.scale_log2;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(S_EMPTY + sb));
      const int kv0 = j * ATT_BN;
      const int limit = p.causal ? min(p.Sk - 1, qrow + p.causal_offset) : p.Sk - 1;  // last visible key
      if (kv0 + ATT_BN - 1 > limit) {
#pragma unroll
        for (int c = 0; c < ATT_BN; ++c)
          if (kv0 + c > limit) s[c] = -INFINITY;
      }
      float mx = s[0];
#pragma unroll
      for (int c = 1; c < ATT_BN; ++c) mx = fmaxf(mx, s[c]);
      const float m_new = fmaxf(m, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m - m_use);  // m = -inf on the first block -> 0
      float rowsum = 0.f;
      uint32_t pk[ATT_BN / 2];
#pragma unroll
      for (int c = 0; c < ATT_BN; c += 2) {
        const float p0 = exp2f(s[c] - m_use), p1 = exp2f(s[c + 1] - m_use);
        rowsum += p0 + p1;
        pk[c >> 1] = pack_bf16x2(p0, p1);
      }
      l = l * alpha + rowsum;
      m = m_new;
      if (j > 0) {
        // PV of the previous block must be complete before O is rescaled or P overwritten
        if (!mbar_wait(bar(O_DONE), (j - 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t t[32];
            tmem_ld_32x32(lane_addr + Cfg::O_COL + c * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
            tmem_st_32x32(lane_addr + Cfg::O_COL + c * 32, t);
          }
          tmem_st_wait();
        }
      }
      // P -> shared memory, K-major with the 128-byte swizzle the MMA descriptor expects
#pragma unroll
      for (int u = 0; u < ATT_BN / 8; ++u) {
        const uint32_t addr = sP + (u >> 3) * (ATT_BM * 128) + r * 128 + (((u & 7) ^ (r & 7)) << 4);
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(pk[u * 4]),
                     "r"(pk[u * 4 + 1]), "r"(pk[u * 4 + 2]), "r"(pk[u * 4 + 3])
                     : "memory");
      }
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL));
    }
    if (ok && n_blocks > 0) {
      ok = mbar_wait(bar(O_DONE), (n_blocks - 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE);
      tc_fence_after();
    }
    if (ok) {
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qrow < p.Sq;
      __nv_bfloat16* orow = p.O + (static_cast<long long>(batch) * p.Sq + qrow) * p.ldo +
                            static_cast<long long>(head) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t t[32];
        if (n_blocks > 0) {
          tmem_ld_32x32(lane_addr + Cfg::O_COL + c * 32, t);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(t[g * 8 + 0]) * inv_l, __uint_as_float(t[g * 8 + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(t[g * 8 + 2]) * inv_l, __uint_as_float(t[g * 8 + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(t[g * 8 + 4]) * inv_l, __uint_as_float(t[g * 8 + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(t[g * 8 + 6]) * inv_l, __uint_as_float(t[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
          }
        }
      }
      if (row_ok && p.lse)
        p.lse[(static_cast<long long>(batch) * p.Hq + head) * p.Sq + qrow] =
            l > 0.f ? (m + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status) atomicCAS(p.status, 0, *abort_word);
}

template <int HD>
static int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                      const AttParams& p, int device, cudaStream_t stream) {
  using Cfg = AttCfg<HD>;
  auto kern = flash_fwd_tcgen05_kernel<HD>;
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set[device] = true;
  }
  dim3 grid((p.Sq + ATT_BM - 1) / ATT_BM, p.Hq, p.B);
  kern<<<grid, ATT_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}


// ----------------------------------------------------------------------------- two-tile kernel
// The kernel used for sequences longer than one query tile.  One CTA owns TWO 128-query tiles
// of one head (256 rows) and walks the keys once for both:
//   warp 0      TMA producer: both Q tiles once, then K / V blocks of 128 keys (2-stage rings)
//   warp 1      MMA issuer, alternating between the tiles: O_i += P_i V, then S_i = Q_i K_next^T,
//               so while softmax group i works on its scores the tensor core runs the other tile
//   warp 2      TMEM allocator: S0 | S1 (128 fp32 columns each) and O0 | O1 (head_dim each)
//   warps 4-7   softmax group of tile 0, warps 8-11 of tile 1 (thread r owns query row r)
// P never touches shared memory: the softmax thread writes its bf16 row over the first 64
// columns of its own S tile in TMEM and the second MMA takes its A operand from there.  O is
// rescaled lazily: a row keeps its reference maximum until the true maximum has moved by more
// than 8 (a factor 256, harmless in fp32 / bf16), so after the first blocks the softmax groups
// do not touch O at all.
constexpr int ATT2_THREADS = 384;
constexpr float ATT2_RESCALE_THRESHOLD = 8.f;

template <int HD>
struct Att2Cfg {
  static constexpr int Q_BYTES = ATT_BM * HD * 2;   // one Q tile
  static constexpr int KV_BYTES = ATT_BN * HD * 2;
  static constexpr int OFF_K = 2 * Q_BYTES;
  static constexpr int OFF_V = OFF_K + ATT_KV_STAGES * KV_BYTES;
  static constexpr int OFF_BAR = OFF_V + ATT_KV_STAGES * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int S_COL = 0;       // S_i at S_COL + i * 128; P_i aliases its first 64 columns
  static constexpr int O_COL = 256;     // O_i at O_COL + i * 128
};

// p = 2^(s * scale + neg_m) for one row of 128 scores held as packed pairs; writes the bf16 pairs
// and returns the row sum (four independent partial sums of pairs).  Moving a share of the
// exponentials from the special-function unit to a polynomial on the FMA pipe was measured at
// 0 / 25 / 37 / 50 / 62 %: 908 / 904 / 902 / 880 / 811 TFLOP/s at B4 S4096 H32/8 D128, so all of
// them stay on ex2.approx.
__device__ __forceinline__ float att2_exp_row(const f32x2 (&sp)[ATT_BN / 2], float scale, float neg_m,
                                              uint32_t (&pk)[ATT_BN / 2]) {
  const f32x2 sc2 = f2_pack(scale, scale), nm2 = f2_pack(neg_m, neg_m);
  f32x2 acc[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) acc[k] = f2_pack(0.f, 0.f);
#pragma unroll
  for (int i = 0; i < ATT_BN / 2; ++i) {
    float x0, x1;
    f2_unpack(f2_fma(sp[i], sc2, nm2), x0, x1);
    const float e0 = fast_exp2(x0), e1 = fast_exp2(x1);
    acc[i & 3] = f2_add(acc[i & 3], f2_pack(e0, e1));
    pk[i] = pack_bf16x2(e0, e1);
  }
  float a, b, c, d;
  f2_unpack(f2_add(acc[0], acc[1]), a, b);
  f2_unpack(f2_add(acc[2], acc[3]), c, d);
  return (a + b) + (c + d);
}

template <int HD>
__global__ void __launch_bounds__(ATT2_THREADS, 1)
flash_fwd2_tcgen05_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const AttParams p) {
  using Cfg = Att2Cfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const uint32_t sbase = smem_u32(smem);
  const uint32_t sQ = sbase, sK = sbase + Cfg::OFF_K, sV = sbase + Cfg::OFF_V;
  const uint32_t bar0 = sbase + Cfg::OFF_BAR;
  enum { Q_FULL = 0, K_FULL = 2, K_EMPTY = 4, V_FULL = 6, V_EMPTY = 8, S_FULL = 10, P_FULL = 12,
         O_DONE = 14, NBARS = 16 };
  auto bar = [&](int i) { return bar0 + 8u * i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + Cfg::OFF_BAR + 8 * NBARS);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qpairs = (p.Sq + 2 * ATT_BM - 1) / (2 * ATT_BM);
  const int qp = n_qpairs - 1 - blockIdx.x;  // heaviest (latest) query blocks first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qp * 2 * ATT_BM;
  // number of key blocks each tile needs
  int nb[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int qi = q0 + i * ATT_BM;
    int kv_end = qi < p.Sq ? p.Sk : 0;
    if (p.causal && qi < p.Sq) kv_end = min(p.Sk, qi + ATT_BM + p.causal_offset);
    nb[i] = kv_end > 0 ? (kv_end + ATT_BN - 1) / ATT_BN : 0;
  }
  const int n_blocks = max(nb[0], nb[1]);

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar(Q_FULL + i), 1);
      mbar_init(bar(K_FULL + i), 1);
      mbar_init(bar(K_EMPTY + i), 1);
      mbar_init(bar(V_FULL + i), 1);
      mbar_init(bar(V_EMPTY + i), 1);
      mbar_init(bar(S_FULL + i), 1);
      mbar_init(bar(P_FULL + i), 4);  // one arrival per softmax warp of the tile
      mbar_init(bar(O_DONE + i), 1);
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 2) {
    tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0 && n_blocks > 0) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        if (nb[i] == 0) continue;
        mbar_expect_tx(bar(Q_FULL + i), Cfg::Q_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(sQ + i * Cfg::Q_BYTES + c * (ATT_BM * 128), &tmQ, bar(Q_FULL + i), head * HD + c * 64,
                      q0 + i * ATT_BM, batch);
      }
      for (int j = 0; j < n_blocks; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1u;
        if (!mbar_wait(bar(K_EMPTY + st), par, abort_word, FT_ERR_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(bar(K_FULL + st), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(sK + st * Cfg::KV_BYTES + c * (ATT_BN * 128), &tmK, bar(K_FULL + st),
                      kv_head * HD + c * 64, j * ATT_BN, batch);
        if (!mbar_wait(bar(V_EMPTY + st), par, abort_word, FT_ERR_TIMEOUT_PRODUCER)) break;
        mbar_expect_tx(bar(V_FULL + st), Cfg::KV_BYTES);
#pragma unroll
        for (int c = 0; c < HD / 64; ++c)
          tma_load_3d(sV + st * Cfg::KV_BYTES + c * (ATT_BN * 128), &tmV, bar(V_FULL + st),
                      kv_head * HD + c * 64, j * ATT_BN, batch);
      }
      if (*abort_word) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_blocks > 0) {
      constexpr uint32_t idesc_qk = make_idesc_f16(ATT_BM, ATT_BN, 1, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_f16(ATT_BM, HD, 1, 0, 1);
      bool ok = true;
      // S_i = Q_i K_j^T into the tile's S columns
      auto issue_qk = [&](int i, int j) {
        const uint32_t kbase = sK + (j & 1) * Cfg::KV_BYTES;
        const uint32_t qbase = sQ + i * Cfg::Q_BYTES;
        const uint32_t d = tmem_base + Cfg::S_COL + i * ATT_BN;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * (ATT_BM * 128) + (kk & 3) * 32;
          umma_f16_ss(d, make_smem_desc_sw128(qbase + off, 16, 1024),
                      make_smem_desc_sw128(kbase + off, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(S_FULL + i));
      };
      // O_i += P_i V_j with P_i read from tensor memory
      auto issue_pv = [&](int i, int j) {
        const uint32_t vbase = sV + (j & 1) * Cfg::KV_BYTES;
        const uint32_t d = tmem_base + Cfg::O_COL + i * ATT_BN;
        const uint32_t a = tmem_base + Cfg::S_COL + i * ATT_BN;
#pragma unroll
        for (int kk = 0; kk < ATT_BN / 16; ++kk)
          umma_f16_ts(d, a + kk * 8, make_smem_desc_sw128(vbase + kk * 2048, ATT_BN * 128, 1024), idesc_pv,
                      (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(O_DONE + i));
      };
      // block 0 scores of both tiles
      ok = mbar_wait(bar(K_FULL + 0), 0, abort_word, FT_ERR_TIMEOUT_MMA);
#pragma unroll
      for (int i = 0; i < 2 && ok; ++i) {
        if (nb[i] == 0) continue;
        ok = mbar_wait(bar(Q_FULL + i), 0, abort_word, FT_ERR_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        issue_qk(i, 0);
      }
      if (ok) umma_commit(bar(K_EMPTY + 0));  // stage 0 is free once the block-0 scores are done
      for (int j = 0; j < n_blocks && ok; ++j) {
        const int st = j & 1;
        const bool has_next = j + 1 < n_blocks;
        if (has_next) {
          ok = mbar_wait(bar(K_FULL + (st ^ 1)), ((j + 1) >> 1) & 1, abort_word, FT_ERR_TIMEOUT_MMA);
          if (!ok) break;
        }
        ok = mbar_wait(bar(V_FULL + st), (j >> 1) & 1, abort_word, FT_ERR_TIMEOUT_MMA);
        if (!ok) break;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          if (j < nb[i]) {
            ok = mbar_wait(bar(P_FULL + i), j & 1, abort_word, FT_ERR_TIMEOUT_MMA);
            if (!ok) break;
            tc_fence_after();
            issue_pv(i, j);
          }
          if (j + 1 < nb[i]) {
            tc_fence_after();
            issue_qk(i, j + 1);
          }
        }
        if (!ok) break;
        // every MMA that reads this V stage (and the K stage of block j + 1) has been issued
        umma_commit(bar(V_EMPTY + st));
        if (has_next) umma_commit(bar(K_EMPTY + (st ^ 1)));
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax groups
    const int ti = (warp - 4) >> 2;  // tile of this warpgroup
    const int ew = warp & 3;         // TMEM lane quarter
    const int r = ew * 32 + lane;
    const int qrow = q0 + ti * ATT_BM + r;
    const int my_nb = nb[ti];
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(ew * 32) << 16);
    const uint32_t s_addr = lane_addr + Cfg::S_COL + ti * ATT_BN;
    const uint32_t o_addr = lane_addr + Cfg::O_COL + ti * ATT_BN;
    float m_ref = -INFINITY;  // reference maximum the stored P and O are relative to
    float l = 0.f;
    bool ok = true;
    const int limit = p.causal ? min(p.Sk - 1, qrow + p.causal_offset) : p.Sk - 1;  // last visible key
    // first key block in which some row of this warp's 32 rows is masked
    const int warp_limit = p.causal ? min(p.Sk - 1, q0 + ti * ATT_BM + ew * 32 + p.causal_offset) : p.Sk - 1;
    for (int j = 0; j < my_nb && ok; ++j) {
      if (!mbar_wait(bar(S_FULL + ti), j & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      // the row as 64 packed pairs: every later step works on two keys per instruction
      f32x2 sp[ATT_BN / 2];
      {
        uint32_t t0[32], t1[32], t2[32], t3[32];
        tmem_ld_32x32(s_addr, t0);
        tmem_ld_32x32(s_addr + 32, t1);
        tmem_ld_32x32(s_addr + 64, t2);
        tmem_ld_32x32(s_addr + 96, t3);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          sp[i] = f2_pack(__uint_as_float(t0[2 * i]), __uint_as_float(t0[2 * i + 1]));
          sp[16 + i] = f2_pack(__uint_as_float(t1[2 * i]), __uint_as_float(t1[2 * i + 1]));
          sp[32 + i] = f2_pack(__uint_as_float(t2[2 * i]), __uint_as_float(t2[2 * i + 1]));
          sp[48 + i] = f2_pack(__uint_as_float(t3[2 * i]), __uint_as_float(t3[2 * i + 1]));
        }
      }
      const int kv0 = j * ATT_BN;
      const bool masked = kv0 + ATT_BN - 1 > warp_limit;   // warp-uniform
      if (masked) {
#pragma unroll
        for (int i = 0; i < ATT_BN / 2; ++i) {
          float a, b;
          f2_unpack(sp[i], a, b);
          if (kv0 + 2 * i > limit) a = -INFINITY;
          if (kv0 + 2 * i + 1 > limit) b = -INFINITY;
          sp[i] = f2_pack(a, b);
        }
      }
      float mx;
      {
        float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;   // four independent chains
#pragma unroll
        for (int i = 0; i < ATT_BN / 2; i += 4) {
          float a, b;
          f2_unpack(sp[i], a, b);
          m0 = max3(m0, a, b);
          f2_unpack(sp[i + 1], a, b);
          m1 = max3(m1, a, b);
          f2_unpack(sp[i + 2], a, b);
          m2 = max3(m2, a, b);
          f2_unpack(sp[i + 3], a, b);
          m3 = max3(m3, a, b);
        }
        mx = fmaxf(max3(m0, m1, m2), m3);
      }
      mx *= p.scale_log2;  // scale > 0, so the maximum commutes with it
      // lazy reference maximum
      float alpha = 1.f;
      if (mx > m_ref + ATT2_RESCALE_THRESHOLD) {
        alpha = fast_exp2(m_ref - mx);  // m_ref = -inf on the first block -> 0
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      uint32_t pk[ATT_BN / 2];
      const float rowsum = att2_exp_row(sp, p.scale_log2, -m_use, pk);
      l = l * alpha + rowsum;
      if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
        // O of the previous blocks is relative to the old reference: bring it to the new one
        if (!mbar_wait(bar(O_DONE + ti), (j - 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t t[32];
          tmem_ld_32x32(o_addr + c * 32, t);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = __float_as_uint(__uint_as_float(t[i]) * alpha);
          tmem_st_32x32(o_addr + c * 32, t);
        }
      }
      // P (bf16, two keys per 32-bit column) over the first 64 columns of this tile's S
      {
        uint32_t(&lo)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[0]);
        uint32_t(&hi)[32] = *reinterpret_cast<uint32_t(*)[32]>(&pk[32]);
        tmem_st_32x32(s_addr, lo);
        tmem_st_32x32(s_addr + 32, hi);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(P_FULL + ti));
    }
    if (ok && my_nb > 0) {
      ok = mbar_wait(bar(O_DONE + ti), (my_nb - 1) & 1, abort_word, FT_ERR_TIMEOUT_EPILOGUE);
      tc_fence_after();
    }
    if (ok && q0 + ti * ATT_BM < p.Sq) {
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      const bool row_ok = qrow < p.Sq;
      __nv_bfloat16* orow = p.O + (static_cast<long long>(batch) * p.Sq + qrow) * p.ldo +
                            static_cast<long long>(head) * HD;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t t[32];
        if (my_nb > 0) {
          tmem_ld_32x32(o_addr + c * 32, t);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) t[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(t[g * 8 + 0]) * inv_l, __uint_as_float(t[g * 8 + 1]) * inv_l);
            o.y = pack_bf16x2(__uint_as_float(t[g * 8 + 2]) * inv_l, __uint_as_float(t[g * 8 + 3]) * inv_l);
            o.z = pack_bf16x2(__uint_as_float(t[g * 8 + 4]) * inv_l, __uint_as_float(t[g * 8 + 5]) * inv_l);
            o.w = pack_bf16x2(__uint_as_float(t[g * 8 + 6]) * inv_l, __uint_as_float(t[g * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + c * 32 + g * 8) = o;
          }
        }
      }
      if (row_ok && p.lse)
        p.lse[(static_cast<long long>(batch) * p.Hq + head) * p.Sq + qrow] =
            l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status) atomicCAS(p.status, 0, *abort_word);
}

template <int HD>
static int launch_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                       const AttParams& p, int device, cudaStream_t stream) {
  using Cfg = Att2Cfg<HD>;
  auto kern = flash_fwd2_tcgen05_kernel<HD>;
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set[device] = true;
  }
  dim3 grid((p.Sq + 2 * ATT_BM - 1) / (2 * ATT_BM), p.Hq, p.B);
  kern<<<grid, ATT2_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

}  // namespace ft

// q: [B, Sq, Hq, D], k/v: [B, Sk, Hkv, D], o: [B, Sq, Hq, D]; ld* = token strides in elements
// (heads are packed: head stride = D), so q/k/v may be slices of one packed QKV buffer.
// lse: fp32 [B, Hq, Sq] or null.  causal_offset: key j visible to query i iff j <= i + offset
// (Sk - Sq aligns the last query with the last key).
FT_API int ft_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B,
                             int Sq, int Sk, int Hq, int Hkv, int D, long long ldq, long long ldk,
                             long long ldv, long long ldo, float scale, int causal, int causal_offset,
                             int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  using namespace ft;
  FT_REQUIRE(q && k && v && o, "ft_flash_attn_fwd: null pointer");
  FT_REQUIRE(D == 64 || D == 128, "ft_flash_attn_fwd: head_dim %d not supported (64, 128)", D);
  FT_REQUIRE(B > 0 && Sq > 0 && Sk > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "ft_flash_attn_fwd: bad shape");
  FT_REQUIRE(ldq % 8 == 0 && ldk % 8 == 0 && ldv % 8 == 0 && ldo % 8 == 0,
             "ft_flash_attn_fwd: token strides must be multiples of 8 elements");
  FT_REQUIRE((reinterpret_cast<uintptr_t>(o) & 15) == 0, "ft_flash_attn_fwd: o must be 16-byte aligned");
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_3d(&tq, q, 2, static_cast<uint64_t>(Hq) * D, Sq, B, ldq * 2,
                        static_cast<uint64_t>(Sq) * ldq * 2, 64, ATT_BM, 1, 3);
  if (rc) return rc;
  rc = make_tmap_3d(&tk, k, 2, static_cast<uint64_t>(Hkv) * D, Sk, B, ldk * 2,
                    static_cast<uint64_t>(Sk) * ldk * 2, 64, ATT_BN, 1, 3);
  if (rc) return rc;
  rc = make_tmap_3d(&tv, v, 2, static_cast<uint64_t>(Hkv) * D, Sk, B, ldv * 2,
                    static_cast<uint64_t>(Sk) * ldv * 2, 64, ATT_BN, 1, 3);
  if (rc) return rc;
  AttParams p;
  p.O = static_cast<__nv_bfloat16*>(o); p.lse = lse; p.ldo = ldo;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hkv = Hkv;
  p.causal = causal; p.causal_offset = causal_offset;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.status = device_status_word(device);
  if (Sq > ATT_BM)  // more than one query tile: the two-tile kernel
    return D == 128 ? launch_fwd2<128>(tq, tk, tv, p, device, stream)
                    : launch_fwd2<64>(tq, tk, tv, p, device, stream);
  return D == 128 ? launch_fwd<128>(tq, tk, tv, p, device, stream)
                  : launch_fwd<64>(tq, tk, tv, p, device, stream);
}
