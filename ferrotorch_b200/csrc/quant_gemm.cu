// GEMMs whose weight operand is expanded on the fly inside the tcgen05 main loop (sm_100a):
//
//   mode Q4_0   Y[M,N] = X[M,K] * dequant(Wq)[N,K]^T, GGUF Q4_0 weights (32-element blocks, fp16
//               scale + 16 nibble bytes, value = (q - 8) * d; element j = low nibble of byte j,
//               element j+16 = high nibble, the GGML file format's order.  The reference's decoder
//               emits the nibbles of byte j as elements 2j, 2j+1 instead, ferrotorch-serialize/src/
//               gguf.rs:543-577; data in that convention is re-packed on the host,
//               csrc/host/gguf.cpp ftg_repack_nibbles).  The
//               reference dequantises the whole tensor to f32 on the GPU, bounces it through the
//               host and stores bf16 (ferrotorch-llama/src/gpu_gguf.rs:14-27); it has no fused
//               dequant-GEMM.  Here the weights stay 4-bit in HBM (0.5625 bytes / element).
//   mode SP24   Y = X * W^T with W in 2:4 semi-structured form: per group of 4 consecutive K
//               elements two kept values (bf16) and two 2-bit positions (one metadata nibble per
//               group).  The reference calls cuSPARSELt (ferrotorch-gpu/src/cusparselt.rs:547-932);
//               this kernel keeps the compressed form in HBM (0.5625 bytes / element-slot) and
//               expands tiles in the producer, so memory-bound shapes gain the bandwidth while the
//               math runs as dense MMAs.
//
// Structure = the dense GEMM (gemm_tcgen05.cu) with the B-side TMA load replaced by eight
// "expander" warps in two groups that alternate k-blocks: a thread owns row r of the 128 x 64 B
// tile, reads its compressed bytes with plain loads (several of its k-blocks ahead, so that HBM
// latency is paid once per tile, not per k-block), expands to 64 bf16 in registers and writes
// one 128-byte row in the swizzled
// K-major layout the MMA descriptor expects (fence.proxy.async, then arrive on the stage's
// full barrier).  A comes by TMA.  All waits are bounded.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int QG_BM = 128, QG_BN = 128, QG_BK = 64;
constexpr int QG_THREADS = 512;   // TMA, MMA, TMEM, idle, 4 epilogue, 8 expander warps
constexpr int QG_A_BYTES = QG_BM * QG_BK * 2, QG_B_BYTES = QG_BN * QG_BK * 2;
constexpr int QG_STAGE = QG_A_BYTES + QG_B_BYTES;
constexpr int QG_STAGES = 5;
// ring of two slots of compressed weight bytes brought in by TMA: 128 rows x 128 bytes (main,
// 128-byte swizzle) + 128 rows x 16 bytes (scales / metadata); one slot covers QG_CK k-blocks
constexpr int QG_COMP_MAIN = QG_BN * 128, QG_COMP_AUX = QG_BN * 16;
constexpr int QG_COMP_SLOT = QG_COMP_MAIN + QG_COMP_AUX;
constexpr int QG_COMP_OFF = QG_STAGES * QG_STAGE;
constexpr int QG_BAR_OFF = QG_COMP_OFF + 2 * QG_COMP_SLOT;
constexpr int QG_SMEM = QG_BAR_OFF + 1024 + 256;

struct QgParams {
  int mode;  // 0 = Q4_0, 1 = SP24
  void* C; long long ldc; int out_f32;
  const void* bias;
  int M, N, K;
  // Q4_0: nibbles [N, K/2] u8, scales [N, K/32] fp16.  SP24: values [N, K/2] bf16, meta [N, K/8] u8
  const uint8_t* w0;
  const uint8_t* w1;
  int* status;
};

__device__ __forceinline__ void store_row_unit(uint32_t row_base, int r, int u, uint4 v) {
  const uint32_t addr = row_base + ((u ^ (r & 7)) << 4);
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Expand one 64-wide k-block of row r (compressed bytes in q0..q3 / aux0, aux1) into the 128-byte
// row of the swizzled K-major B tile at row_base.
template <int MODE>
__device__ __forceinline__ void expand_row(uint32_t row_base, int r, const uint4& q0, const uint4& q1, const uint4& q2,
                                           const uint4& q3, uint32_t aux0, uint32_t aux1) {
  if (MODE == 0) {
    const uint32_t nib[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
    for (int blk = 0; blk < 2; ++blk) {
      const float d = __half2float(__ushort_as_half(static_cast<unsigned short>(blk ? (aux0 >> 16) : (aux0 & 0xFFFF))));
#pragma unroll
      for (int hi = 0; hi < 2; ++hi) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          // 8 elements: nibbles (low or high) of bytes [half*8, half*8+8) of this block
          const uint32_t w0 = nib[blk * 4 + half * 2] >> (hi * 4), w1 = nib[blk * 4 + half * 2 + 1] >> (hi * 4);
          float f[8];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // 0x4B000000 | q is the float 2^23 + q: the nibble becomes a float without an I2F
            f[e] = (__uint_as_float(((w0 >> (8 * e)) & 0xFu) | 0x4B000000u) - 8388616.f) * d;
            f[4 + e] = (__uint_as_float(((w1 >> (8 * e)) & 0xFu) | 0x4B000000u) - 8388616.f) * d;
          }
          uint4 o;
          o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
          o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
          store_row_unit(row_base, r, blk * 4 + hi * 2 + half, o);
        }
      }
    }
  } else {
    // 16 groups of 4 slots; group g: two bf16 values (one word) at slots (m & 3), (m >> 2)
    const uint32_t vals[16] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w,
                               q2.x, q2.y, q2.z, q2.w, q3.x, q3.y, q3.z, q3.w};
#pragma unroll
    for (int u = 0; u < 8; ++u) {        // one 16-byte unit = 8 slots = 2 groups
      uint32_t outw[4];
#pragma unroll
      for (int gg = 0; gg < 2; ++gg) {
        const int g = u * 2 + gg;
        const uint32_t m4 = ((g < 8 ? aux0 : aux1) >> ((g & 7) * 4)) & 0xF;
        const uint32_t v_lo = vals[g] & 0xFFFFu, v_hi = vals[g] >> 16;
        const uint32_t p0 = m4 & 3u, p1 = m4 >> 2;
        // slot s of the group lives in half-word (s & 1) of word (s >> 1): build both words
        // with selects instead of indexing a register array by a run-time value
        outw[gg * 2] = (p0 == 0u ? v_lo : 0u) | (p0 == 1u ? v_lo << 16 : 0u) | (p1 == 1u ? v_hi << 16 : 0u);
        outw[gg * 2 + 1] = (p0 == 2u ? v_lo : 0u) | (p1 == 2u ? v_hi : 0u) | (p1 == 3u ? v_hi << 16 : 0u);
      }
      store_row_unit(row_base, r, u, make_uint4(outw[0], outw[1], outw[2], outw[3]));
    }
  }
}

// MODE: 0 = Q4_0, 1 = SP24.  TMA_W: the compressed weight bytes come through TMA into a small
// shared-memory ring in 128-byte row segments (four k-blocks of Q4_0, two of 2:4 at a time), which
// is what keeps HBM efficient -- a thread fetching 32 bytes of its own row per k-block opens a
// DRAM page per access.  Without TMA_W (strides not multiples of 16 bytes) the expander threads
// load their rows directly.
template <int MODE, bool TMA_W>
__global__ void __launch_bounds__(QG_THREADS, 1)
expand_gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmW0,
                           const __grid_constant__ CUtensorMap tmW1, const QgParams p) {
  constexpr int CK = MODE == 0 ? 4 : 2;   // k-blocks per compressed slot
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + QG_BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * QG_STAGES + 8);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem), bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (QG_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * QG_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * QG_STAGES + 2 + a); };
  auto cfull_bar = [&](int c) { return bar_base + 8u * (2 * QG_STAGES + 4 + c); };
  auto cempty_bar = [&](int c) { return bar_base + 8u * (2 * QG_STAGES + 6 + c); };
  const int m_blocks = (p.M + QG_BM - 1) / QG_BM, n_blocks = (p.N + QG_BN - 1) / QG_BN;
  const int num_tiles = m_blocks * n_blocks, k_blocks = (p.K + QG_BK - 1) / QG_BK;
  // m fastest: consecutive CTAs share the (expensive to expand) weight rows through L2
  auto coords = [&](int t, int& mb, int& nb) { mb = t % m_blocks; nb = t / m_blocks; };

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < QG_STAGES; ++s) { mbar_init(full_bar(s), 1 + 4); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    for (int c = 0; c < 2; ++c) { mbar_init(cfull_bar(c), 1); mbar_init(cempty_bar(c), 8); }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    if (TMA_W) { tma_prefetch_desc(&tmW0); tma_prefetch_desc(&tmW1); }
  }
  if (warp == 2) { tmem_alloc(smem_u32(tmem_slot), 2 * QG_BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb; coords(tile, mb, nb);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), QG_A_BYTES);
          tma_load_2d(smem_base + stage * QG_STAGE, &tmA, full_bar(stage), kb * QG_BK, mb * QG_BM);
          if (++stage == QG_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*abort_word) { const unsigned long long t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000); }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(QG_BM, QG_BN, 1, 0, 0);
      int stage = 0, acc = 0; uint32_t phase = 0, acc_phase = 0; bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_word, FT_ERR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * QG_BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_word, FT_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * QG_STAGE, sB = sA + QG_A_BYTES;
#pragma unroll
          for (int k = 0; k < QG_BK / 16; ++k)
            umma_f16_ss(d, make_smem_desc_sw128(sA + k * 32, 16, 1024), make_smem_desc_sw128(sB + k * 32, 16, 1024),
                        idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == QG_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp == 3) {
    // ---------------------------------------------------------------- compressed-weight producer
    if (TMA_W && lane == 0) {
      const int c_blocks = (k_blocks + CK - 1) / CK;
      long long cseq = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb; coords(tile, mb, nb);
        for (int cb = 0; cb < c_blocks; ++cb, ++cseq) {
          const int slot = static_cast<int>(cseq & 1);
          const uint32_t ph = static_cast<uint32_t>((cseq >> 1) & 1);
          if (!mbar_wait(cempty_bar(slot), ph ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t dst = smem_base + QG_COMP_OFF + slot * QG_COMP_SLOT;
          mbar_expect_tx(cfull_bar(slot), QG_COMP_SLOT);
          tma_load_2d(dst, &tmW0, cfull_bar(slot), cb * 128, nb * QG_BN);
          tma_load_2d(dst + QG_COMP_MAIN, &tmW1, cfull_bar(slot), cb * 16, nb * QG_BN);
        }
      }
      if (*abort_word) { const unsigned long long t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000); }
    }
  } else if (warp >= 8) {
    // ---------------------------------------------------------------- expander warps
    // Two groups of four warps; group g expands the k-blocks whose running number is g (mod 2),
    // thread r of a group owns row r of the 128 x 64 B tile.  The chain wait -> expand -> store ->
    // proxy fence -> arrive of one k-block therefore overlaps with the other group's k-block.
    const int grp = (warp - 8) >> 2;
    const int r = ((warp - 8) & 3) * 32 + lane;
    if (TMA_W) {
      // k-blocks of even / odd index within the tile go to group 0 / 1; every warp releases a
      // compressed slot once it has expanded its k-blocks of that slot
      const int c_blocks = (k_blocks + CK - 1) / CK;
      long long seq0 = 0, cseq = 0;
      bool ok = true;
      const uint32_t swz = static_cast<uint32_t>(r & 7);
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, seq0 += k_blocks) {
        for (int cb = 0; cb < c_blocks && ok; ++cb, ++cseq) {
          const int slot = static_cast<int>(cseq & 1);
          const uint32_t cph = static_cast<uint32_t>((cseq >> 1) & 1);
          if (!mbar_wait(cfull_bar(slot), cph, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t cmain = smem_base + QG_COMP_OFF + slot * QG_COMP_SLOT + r * 128;
          const uint32_t caux = smem_base + QG_COMP_OFF + slot * QG_COMP_SLOT + QG_COMP_MAIN + r * 16;
#pragma unroll
          for (int j = 0; j < CK; ++j) {
            const int kb = cb * CK + j;
            if (kb >= k_blocks || !ok) break;
            if ((kb & 1) != grp) continue;
            auto lds128 = [&](uint32_t chunk) {
              uint4 v;
              asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                           : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(cmain + ((chunk ^ swz) << 4)) : "memory");
              return v;
            };
            uint4 q0, q1, q2 = make_uint4(0, 0, 0, 0), q3 = q2;
            uint32_t aux0, aux1 = 0;
            if (MODE == 0) {
              q0 = lds128(2 * j);
              q1 = lds128(2 * j + 1);
              asm volatile("ld.shared.u32 %0, [%1];" : "=r"(aux0) : "r"(caux + j * 4) : "memory");
            } else {
              q0 = lds128(4 * j); q1 = lds128(4 * j + 1); q2 = lds128(4 * j + 2); q3 = lds128(4 * j + 3);
              asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(aux0), "=r"(aux1) : "r"(caux + j * 8) : "memory");
            }
            const long long seq = seq0 + kb;
            const int stage = static_cast<int>(seq % QG_STAGES);
            const uint32_t phase = static_cast<uint32_t>((seq / QG_STAGES) & 1);
            if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
            const uint32_t row_base = smem_base + stage * QG_STAGE + QG_A_BYTES + r * 128;
            expand_row<MODE>(row_base, r, q0, q1, q2, q3, aux0, aux1);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(full_bar(stage));
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(cempty_bar(slot));
        }
      }
    } else {
    // compressed bytes of one 64-wide k-block of this thread's row
    struct Comp { uint4 q0, q1, q2, q3; uint32_t aux0, aux1; };
    constexpr int PF = MODE == 0 ? 3 : 2;  // own k-blocks fetched ahead (every second k-block is this group's)
    long long seq0 = 0;                    // running number of the tile's first k-block
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, seq0 += k_blocks) {
      int mb, nb; coords(tile, mb, nb);
      const int n = nb * QG_BN + r;
      const bool row_ok = n < p.N;
      auto fetch = [&](int kb, Comp& c) {
        c.q0 = c.q1 = c.q2 = c.q3 = make_uint4(0, 0, 0, 0);
        c.aux0 = c.aux1 = 0;
        const int k0 = kb * QG_BK;
        if (!row_ok || kb >= k_blocks || k0 + QG_BK > p.K) return;  // K is a multiple of 64 (checked by the host)
        if (MODE == 0) {
          const uint8_t* nb_ptr = p.w0 + static_cast<long long>(n) * (p.K >> 1) + (k0 >> 1);
          c.q0 = __ldg(reinterpret_cast<const uint4*>(nb_ptr));
          c.q1 = __ldg(reinterpret_cast<const uint4*>(nb_ptr) + 1);
          c.aux0 = __ldg(reinterpret_cast<const uint32_t*>(p.w1 + (static_cast<long long>(n) * (p.K >> 5) + (k0 >> 5)) * 2));
        } else {
          const uint8_t* v_ptr = p.w0 + (static_cast<long long>(n) * (p.K >> 1) + (k0 >> 1)) * 2;
          c.q0 = __ldg(reinterpret_cast<const uint4*>(v_ptr));
          c.q1 = __ldg(reinterpret_cast<const uint4*>(v_ptr) + 1);
          c.q2 = __ldg(reinterpret_cast<const uint4*>(v_ptr) + 2);
          c.q3 = __ldg(reinterpret_cast<const uint4*>(v_ptr) + 3);
          const uint2 mt = __ldg(reinterpret_cast<const uint2*>(p.w1 + static_cast<long long>(n) * (p.K >> 3) + (k0 >> 3)));
          c.aux0 = mt.x; c.aux1 = mt.y;
        }
      };
      const int kb_first = static_cast<int>((grp - seq0) & 1);   // first k-block of this tile that is ours
      Comp buf[PF];
#pragma unroll
      for (int i = 0; i < PF; ++i) fetch(kb_first + 2 * i, buf[i]);
      for (int kb0 = kb_first; kb0 < k_blocks && ok; kb0 += 2 * PF) {
#pragma unroll
        for (int j = 0; j < PF; ++j) {
          const int kb = kb0 + 2 * j;
          if (kb >= k_blocks || !ok) break;
          const uint4 q0 = buf[j].q0, q1 = buf[j].q1, q2 = buf[j].q2, q3 = buf[j].q3;
          const uint32_t aux0 = buf[j].aux0, aux1 = buf[j].aux1;
          fetch(kb + 2 * PF, buf[j]);
          const long long seq = seq0 + kb;
          const int stage = static_cast<int>(seq % QG_STAGES);
          const uint32_t phase = static_cast<uint32_t>((seq / QG_STAGES) & 1);
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t row_base = smem_base + stage * QG_STAGE + QG_A_BYTES + r * 128;
          expand_row<MODE>(row_base, r, q0, q1, q2, q3, aux0, aux1);
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(full_bar(stage));
        }
      }
    }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- epilogue
    const int ew = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mb, nb; coords(tile, mb, nb);
      const int m0 = mb * QG_BM, n0 = nb * QG_BN;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int row = m0 + ew * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * QG_BN;
#pragma unroll 1
      for (int c = 0; c < QG_BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(t_row + c * 32, rr);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row >= p.M || col0 >= p.N) continue;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          if (col0 + g * 8 + 8 > p.N) continue;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            v[j] = __uint_as_float(rr[g * 8 + j]);
            if (p.bias) v[j] += __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col0 + g * 8 + j]);
          }
          if (p.out_f32) {
            float* o = static_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0 + g * 8;
            *reinterpret_cast<float4*>(o) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(o + 4) = make_float4(v[4], v[5], v[6], v[7]);
          } else {
            uint4 o;
            o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
            o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0 + g * 8) = o;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1; if (acc == 0) acc_phase ^= 1u;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 2 * QG_BN); }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status) atomicCAS(p.status, 0, *abort_word);
}

template <int MODE, bool TMA_W>
static int launch_expand_t(const CUtensorMap& tmA, const CUtensorMap& tmW0, const CUtensorMap& tmW1, const QgParams& p,
                           int device, int grid, cudaStream_t stream) {
  auto kern = expand_gemm_tcgen05_kernel<MODE, TMA_W>;
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, QG_SMEM));
    attr_set[device] = true;
  }
  kern<<<grid, QG_THREADS, QG_SMEM, stream>>>(tmA, tmW0, tmW1, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

static int launch_expand(const void* x, const QgParams& p0, long long ldx, int device, cudaStream_t stream) {
  QgParams p = p0;
  CUtensorMap tmA, tmW0, tmW1;
  int rc = make_tmap_2d(&tmA, x, 2, p.K, p.M, ldx * 2, QG_BK, QG_BM, 3);
  if (rc) return rc;
  // compressed operands as byte matrices: main rows of K/2 (Q4_0 nibbles) or K (2:4 values) bytes,
  // aux rows of K/16 (fp16 scales) or K/8 (metadata) bytes; TMA needs 16-byte strides and bases
  const long long main_row = p.mode == 0 ? (p.K >> 1) : p.K;
  const long long aux_row = p.mode == 0 ? (p.K >> 4) : (p.K >> 3);
  const bool tma_w = main_row % 16 == 0 && aux_row % 16 == 0 && (reinterpret_cast<uintptr_t>(p.w0) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(p.w1) & 15) == 0;
  if (tma_w) {
    rc = make_tmap_2d(&tmW0, p.w0, 1, main_row, p.N, main_row, 128, QG_BN, 3);
    if (rc) return rc;
    rc = make_tmap_2d(&tmW1, p.w1, 1, aux_row, p.N, aux_row, 16, QG_BN, 0);
    if (rc) return rc;
  } else {
    tmW0 = tmA;
    tmW1 = tmA;
  }
  p.status = device_status_word(device);
  const int tiles = ((p.M + QG_BM - 1) / QG_BM) * ((p.N + QG_BN - 1) / QG_BN);
  const int grid = tiles < sm_count(device) ? tiles : sm_count(device);
  if (p.mode == 0)
    return tma_w ? launch_expand_t<0, true>(tmA, tmW0, tmW1, p, device, grid, stream)
                 : launch_expand_t<0, false>(tmA, tmW0, tmW1, p, device, grid, stream);
  return tma_w ? launch_expand_t<1, true>(tmA, tmW0, tmW1, p, device, grid, stream)
               : launch_expand_t<1, false>(tmA, tmW0, tmW1, p, device, grid, stream);
}

}  // namespace ft

using namespace ft;

// y[M,N] = x[M,K] (bf16, row stride ldx) * dequant_q4_0(nibbles [N, K/2], scales fp16 [N, K/32])^T (+ bias).
FT_API int ft_q4_0_gemm(const void* x, const void* nibbles, const void* scales, void* y, const void* bias, int M,
                        int N, int K, long long ldx, long long ldy, int out_f32, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && nibbles && scales && y, "ft_q4_0_gemm: null pointer");
  FT_REQUIRE(M > 0 && N > 0 && K > 0 && K % 64 == 0 && N % 8 == 0 && ldx % 8 == 0 && ldy % (out_f32 ? 4 : 8) == 0,
             "ft_q4_0_gemm: K must be a multiple of 64, N of 8");
  FT_REQUIRE((reinterpret_cast<uintptr_t>(nibbles) & 15) == 0 && (reinterpret_cast<uintptr_t>(scales) & 3) == 0,
             "ft_q4_0_gemm: nibble plane must be 16-byte aligned");
  QgParams p{};
  p.mode = 0; p.C = y; p.ldc = ldy; p.out_f32 = out_f32; p.bias = bias; p.M = M; p.N = N; p.K = K;
  p.w0 = static_cast<const uint8_t*>(nibbles); p.w1 = static_cast<const uint8_t*>(scales);
  return launch_expand(x, p, ldx, device, stream);
}

// y[M,N] = x[M,K] * W^T with W 2:4-compressed: values bf16 [N, K/2], meta u8 [N, K/8] (one nibble
// per group of 4: bits 0-1 = slot of the first kept value, bits 2-3 = slot of the second).
FT_API int ft_sparse24_gemm(const void* x, const void* values, const void* meta, void* y, const void* bias, int M,
                            int N, int K, long long ldx, long long ldy, int out_f32, int device,
                            cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && values && meta && y, "ft_sparse24_gemm: null pointer");
  FT_REQUIRE(M > 0 && N > 0 && K > 0 && K % 64 == 0 && N % 8 == 0 && ldx % 8 == 0 && ldy % (out_f32 ? 4 : 8) == 0,
             "ft_sparse24_gemm: K must be a multiple of 64, N of 8");
  FT_REQUIRE((reinterpret_cast<uintptr_t>(values) & 15) == 0 && (reinterpret_cast<uintptr_t>(meta) & 7) == 0,
             "ft_sparse24_gemm: value plane must be 16-byte aligned, metadata 8-byte aligned");
  QgParams p{};
  p.mode = 1; p.C = y; p.ldc = ldy; p.out_f32 = out_f32; p.bias = bias; p.M = M; p.N = N; p.K = K;
  p.w0 = static_cast<const uint8_t*>(values); p.w1 = static_cast<const uint8_t*>(meta);
  return launch_expand(x, p, ldx, device, stream);
}
