// bf16 GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM),
// operands staged in shared memory by TMA through an mbarrier pipeline.
//
//   C[M,N] (+)= A[M,K] * B[N,K]^T (+ bias[N])
//
// Both operands may be stored K-major (row-major [rows, K], the nn.Linear layout)
// or MN-major (row-major [K, rows]); the four combinations cover the forward
// (X W^T), data-gradient (dY W) and weight-gradient (dY^T X) products of a linear
// layer without any transposed copy.  This replaces the cuBLAS GemmEx calls of the
// reference (ferrotorch-gpu/src/blas.rs:3186-3306, 2769-2886) and its separate
// bias launch (ferrotorch-core/src/grad_fns/linalg.rs:1643-1655).
//
// Two kernels share this file.  Problems with at least 256 rows and N >= 128 run on the
// CTA-pair kernel (tcgen05.mma.cta_group::2, 256 x BN tiles, TMA-store epilogue; described at
// gemm_bf16_pair_kernel).  Smaller problems run on the one-CTA kernel:
//
// Kernel structure (one persistent CTA per SM, 256 threads):
//   warp 0    TMA producer: one elected thread fills a STAGES-deep ring of
//             {A 128x64, B BNx64} bf16 tiles (128-byte swizzle)
//   warp 1    MMA issuer: one thread issues 4 x tcgen05.mma (128 x BN x 16) per
//             stage and commits the stage's "empty" barrier; after the last
//             k-block it commits the accumulator's "full" barrier
//   warp 2    allocates / frees tensor memory (2 accumulators of BN columns so the
//             epilogue of tile i overlaps the main loop of tile i+1)
//   warps 4-7 epilogue: tcgen05.ld -> fp32 registers -> (+C, +bias) -> bf16/fp32
//             -> global
// Every wait is bounded; a wait that runs out aborts the CTA cleanly and reports
// through the device status word.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 256;
constexpr int GEMM_GROUP_M = 16;

enum GemmFlags : int {
  GEMM_OUT_F32 = 1,     // C is fp32 (default bf16)
  GEMM_ACCUMULATE = 2,  // C += A B^T
  GEMM_BIAS = 4,        // + bias[N] (bf16)
  GEMM_BIAS_F32 = 8,    // bias is fp32
  GEMM_RELU = 16,       // activation fused in the epilogue (after bias)
  GEMM_GELU = 32,
  GEMM_SILU = 64,
  GEMM_EPI_DIRECT = 1 << 16,  // internal: per-lane read-modify-write epilogue
  GEMM_EPI_TRANSPOSED = 1 << 17,  // internal: the tile holds C^T; lane = column of C, register = row of C
};

template <int BN>
struct GemmCfg {
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (200 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  // stages + barriers (full, empty, tmem_full[2], tmem_empty[2]) + tmem ptr + abort + align slack
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

constexpr int GEMM_MAX_TAPS = 49;  // up to a 7 x 7 filter

struct GemmParams {
  void* C;
  const void* bias;
  int M, N, K;
  long long ldc;
  int flags;
  int* status;
  // Shifted-row GEMMs (convolutions over zero-padded, flattened NHWC activations; see
  // gemm_bf16_pair_kernel).  taps == 0: plain GEMM.
  int taps;                  // filter taps
  int cblocks;               // 64-channel k-blocks per tap (fprop: K = taps * cblocks * 64)
  int ksplit;                // filter gradient: pieces the pixel dimension is cut into
  int shift[GEMM_MAX_TAPS];  // row offset of tap t in the flattened padded activation
  // MODE 1 output: GEMM row p = (n * gHp + i) * gWp + j is written to row
  // (n * cHo + i - c_oh) * cWo + j - c_ow of C when (i - c_oh, j - c_ow) lies inside the
  // cHo x cWo window, and dropped otherwise (cHo == 0: rows are stored as they are).
  int gHp, gWp, cHo, cWo, c_oh, c_ow;
  // MODE 2 without accumulation: piece ks of the split contraction stores its tile at row
  // ks * split_rows + m (one slice of the workspace per piece; summed later in a fixed order).
  int split_rows;
};

__device__ __forceinline__ void tile_coords(int tile, int m_blocks, int n_blocks, int& mb, int& nb) {
  const int group_tiles = GEMM_GROUP_M * n_blocks;
  const int g = tile / group_tiles;
  const int first_m = g * GEMM_GROUP_M;
  const int gm = min(GEMM_GROUP_M, m_blocks - first_m);
  const int r = tile - g * group_tiles;
  mb = first_m + (r % gm);
  nb = r / gm;
}

__device__ __forceinline__ float apply_act(float v, int flags) {
  if (flags & GEMM_RELU) return fmaxf(v, 0.f);
  if (flags & GEMM_GELU) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  if (flags & GEMM_SILU) return v / (1.f + __expf(-v));
  return v;
}


// Epilogue that writes straight to global memory, one accumulator row per lane.  Used where the
// output needs a read-modify-write in fp32 before rounding (bf16 accumulate) or an activation
// after the accumulation.  `t_row` addresses this warp's 32 TMEM lanes at the tile's first
// column; `row` is this lane's global row, `n0` the tile's first column.
template <int BN>
__device__ __forceinline__ void epilogue_direct(const GemmParams& p, uint32_t t_row, int row, int n0) {
  const bool row_ok = row < p.M;
  const bool out_f32 = (p.flags & GEMM_OUT_F32) != 0;
  const bool accumulate = (p.flags & GEMM_ACCUMULATE) != 0;
  const bool has_bias = (p.flags & (GEMM_BIAS | GEMM_BIAS_F32)) != 0;
  const bool has_act = (p.flags & (GEMM_RELU | GEMM_GELU | GEMM_SILU)) != 0;
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(t_row + c * 32, r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    if (!row_ok || col0 >= p.N) continue;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (has_bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        if (col < p.N) {
          v[j] += (p.flags & GEMM_BIAS_F32)
                      ? static_cast<const float*>(p.bias)[col]
                      : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col]);
        }
      }
    }
    if (out_f32) {
      float* crow = static_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        if (col0 + g * 4 + 4 <= p.N) {
          float4 o = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
          if (accumulate) {
            const float4 old = *reinterpret_cast<const float4*>(crow + g * 4);
            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
          }
          if (has_act) {
            o.x = apply_act(o.x, p.flags); o.y = apply_act(o.y, p.flags);
            o.z = apply_act(o.z, p.flags); o.w = apply_act(o.w, p.flags);
          }
          *reinterpret_cast<float4*>(crow + g * 4) = o;
        }
      }
    } else {
      __nv_bfloat16* crow =
          static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (col0 + g * 8 + 8 <= p.N) {
          float* vv = v + g * 8;
          if (accumulate) {
            const uint4 old = *reinterpret_cast<const uint4*>(crow + g * 8);
            const float2 o0 = unpack_bf16x2(old.x), o1 = unpack_bf16x2(old.y),
                         o2 = unpack_bf16x2(old.z), o3 = unpack_bf16x2(old.w);
            vv[0] += o0.x; vv[1] += o0.y; vv[2] += o1.x; vv[3] += o1.y;
            vv[4] += o2.x; vv[5] += o2.y; vv[6] += o3.x; vv[7] += o3.y;
          }
          if (has_act) {
#pragma unroll
            for (int j = 0; j < 8; ++j) vv[j] = apply_act(vv[j], p.flags);
          }
          uint4 o;
          o.x = pack_bf16x2(vv[0], vv[1]);
          o.y = pack_bf16x2(vv[2], vv[3]);
          o.z = pack_bf16x2(vv[4], vv[5]);
          o.w = pack_bf16x2(vv[6], vv[7]);
          *reinterpret_cast<uint4*>(crow + g * 8) = o;
        }
      }
    }
  }
}


// MODE 1 epilogue with the crop folded in: one accumulator row per lane, written to its pixel's
// row of the unpadded NHWC output (rows of the padded border are dropped).  bias / activation as
// in the other epilogues; no accumulation.
template <int BN>
__device__ __forceinline__ void epilogue_crop(const GemmParams& p, uint32_t t_row, int row, int n0) {
  const bool out_f32 = (p.flags & GEMM_OUT_F32) != 0;
  const bool has_bias = (p.flags & (GEMM_BIAS | GEMM_BIAS_F32)) != 0;
  const bool has_act = (p.flags & (GEMM_RELU | GEMM_GELU | GEMM_SILU)) != 0;
  bool row_ok = row < p.M;
  long long dst_row = 0;
  {
    const int plane = p.gHp * p.gWp;
    const int n = row / plane;
    const int r = row - n * plane;
    const int i = r / p.gWp - p.c_oh, j = r - (r / p.gWp) * p.gWp - p.c_ow;
    row_ok = row_ok && i >= 0 && i < p.cHo && j >= 0 && j < p.cWo;
    dst_row = (static_cast<long long>(n) * p.cHo + i) * p.cWo + j;
  }
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(t_row + c * 32, r);
    tmem_ld_wait();
    const int col0 = n0 + c * 32;
    if (!row_ok || col0 >= p.N) continue;
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
    if (has_bias) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        if (col < p.N)
          v[j] += (p.flags & GEMM_BIAS_F32) ? static_cast<const float*>(p.bias)[col]
                                            : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col]);
      }
    }
    if (has_act) {
#pragma unroll
      for (int j = 0; j < 32; ++j) v[j] = apply_act(v[j], p.flags);
    }
    if (out_f32) {
      float* crow = static_cast<float*>(p.C) + dst_row * p.ldc + col0;
#pragma unroll
      for (int g = 0; g < 8; ++g)
        if (col0 + g * 4 + 4 <= p.N)
          *reinterpret_cast<float4*>(crow + g * 4) = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
    } else {
      __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.C) + dst_row * p.ldc + col0;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        if (col0 + g * 8 + 8 <= p.N) {
          uint4 o;
          o.x = pack_bf16x2(v[g * 8], v[g * 8 + 1]);
          o.y = pack_bf16x2(v[g * 8 + 2], v[g * 8 + 3]);
          o.z = pack_bf16x2(v[g * 8 + 4], v[g * 8 + 5]);
          o.w = pack_bf16x2(v[g * 8 + 6], v[g * 8 + 7]);
          *reinterpret_cast<uint4*>(crow + g * 8) = o;
        }
      }
    }
  }
}


// Epilogue for a tile that holds C^T (small-batch GEMMs are issued with the weight as the
// 128-row MMA operand): accumulator row = column n of C, accumulator column = row m of C.  For
// a fixed m the 32 lanes of a warp write 32 consecutive bf16 of row m: 64-byte segments.
// p.M / p.N are the extents of the *tile space* (rows of W, batch), p.ldc the row stride of C.
template <int BN>
__device__ __forceinline__ void epilogue_transposed(const GemmParams& p, uint32_t t_row, int n_idx, int m0) {
  const bool n_ok = n_idx < p.M;
  const bool has_bias = (p.flags & (GEMM_BIAS | GEMM_BIAS_F32)) != 0;
  const bool has_act = (p.flags & (GEMM_RELU | GEMM_GELU | GEMM_SILU)) != 0;
  float bias = 0.f;
  if (has_bias && n_ok)
    bias = (p.flags & GEMM_BIAS_F32) ? static_cast<const float*>(p.bias)[n_idx]
                                     : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[n_idx]);
#pragma unroll 1
  for (int c = 0; c < BN / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(t_row + c * 32, r);
    tmem_ld_wait();
    if (!n_ok) continue;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int m = m0 + c * 32 + j;
      if (m < p.N) {
        float v = __uint_as_float(r[j]) + bias;
        if (has_act) v = apply_act(v, p.flags);
        if (p.flags & GEMM_OUT_F32)
          static_cast<float*>(p.C)[static_cast<long long>(m) * p.ldc + n_idx] = v;
        else
          static_cast<__nv_bfloat16*>(p.C)[static_cast<long long>(m) * p.ldc + n_idx] = __float2bfloat16(v);
      }
    }
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA,
                         const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  const int m_blocks = (p.M + GEMM_BM - 1) / GEMM_BM;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_blocks = (p.K + GEMM_BK - 1) / GEMM_BK;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);  // one arrival per epilogue warp
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
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
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb;
        tile_coords(tile, m_blocks, n_blocks, mb, nb);
        const int m0 = mb * GEMM_BM, n0 = nb * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
          const int k0 = kb * GEMM_BK;
          if constexpr (!A_MN) {
            tma_load_2d(sA, &tmA, full_bar(stage), k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c)
              tma_load_2d(sA + c * (GEMM_BK * 128), &tmA, full_bar(stage), m0 + c * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d(sB, &tmB, full_bar(stage), k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * (GEMM_BK * 128), &tmB, full_bar(stage), n0 + c * 64, k0);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        // Drain: give the loads already issued a bounded time to land before the
        // CTA's shared memory is released.
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(GEMM_BM, BN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_word, FT_ERR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_word, FT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sA + k * 2048, GEMM_BK * 128, 1024)
                                        : make_smem_desc_sw128(sA + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sB + k * 2048, GEMM_BK * 128, 1024)
                                        : make_smem_desc_sw128(sB + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int ew = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mb, nb;
      tile_coords(tile, m_blocks, n_blocks, mb, nb);
      const int m0 = mb * GEMM_BM, n0 = nb * BN;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
      epilogue_direct<BN>(p, t_row, m0 + ew * 32 + lane, n0);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}


// ----------------------------------------------------------------------------- CTA-pair kernel
// The large-problem kernel.  Two CTAs of a thread-block cluster work on one 256 x BN output
// tile with tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own half
// (BN/2 rows) of B with plain TMA loads, so a k-block costs each SM 16 KB + BN*64 bytes of
// shared-memory fill instead of 16 KB + BN*128, and the tensor core of each SM reads half of B
// from its neighbour.  The even CTA of the pair (the leader) issues every MMA; its commits
// arrive on the "stage empty" and "accumulator full" barriers of both CTAs.  TMA completions of
// both CTAs are counted on the leader's "stage full" barrier, and the epilogue warps of both
// CTAs arrive on the leader's "accumulator empty" barrier.
//
// Epilogue: each of the four epilogue warps owns 32 accumulator rows.  It converts 128 bytes
// per row at a time (64 bf16 or 32 fp32 columns), writes them into a 128-byte-swizzled staging
// tile of its own in shared memory and hands the tile to a TMA store (or a TMA reduce-add for
// C += ...).  Two staging tiles per warp keep one store in flight while the next is filled; the
// stores clip at the M and N edges.
//
// MODE 1 and 2 turn the same pipeline into a convolution over activations stored zero-padded and
// flattened to [pixels, channels] (NHWC): in that layout the input pixel a filter tap reads
// for output pixel p is row p + shift[tap], a constant offset, so
//   MODE 1 (forward / input gradient): C[p, co] = sum_tap sum_ci A[p + shift[tap], ci] * W[co, tap, ci]
//          is a GEMM whose A tile of k-block (tap, 64 channels) is an ordinary 2-D TMA box at row
//          m0 + shift[tap] (rows before the first or past the last pixel read as zeros);
//   MODE 2 (filter gradient): dW[co, tap, ci] += sum_p dY[p, co] * X[p + shift[tap], ci], one
//          [Cout x Cin] GEMM per tap with the pixels as the (split) contraction dimension, both
//          operands MN-major, tiles added into an fp32 dW with the TMA reduce-add epilogue.
// Rows of the padded border hold zeros in the input of MODE 1 / in dY of MODE 2, and the caller
// drops the border rows of a MODE 1 output.
template <int BN>
struct PairCfg {
  static constexpr int BNH = BN / 2;
  static constexpr int A_BYTES = GEMM_BM * GEMM_BK * 2;
  static constexpr int B_BYTES = BNH * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_TILE_BYTES = 32 * 128;
  static constexpr int EPI_BYTES = 4 * 2 * EPI_TILE_BYTES;
  static constexpr int STAGES_RAW = (227 * 1024 - 2048 - EPI_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
};

constexpr int PAIR_GROUP_M = 8;  // 256-row blocks per rasterisation group

__device__ __forceinline__ void pair_tile_coords(int tile, int m_blocks, int n_blocks, int& mb, int& nb) {
  const int group_tiles = PAIR_GROUP_M * n_blocks;
  const int g = tile / group_tiles;
  const int first_m = g * PAIR_GROUP_M;
  const int gm = min(PAIR_GROUP_M, m_blocks - first_m);
  const int r = tile - g * group_tiles;
  mb = first_m + (r % gm);
  nb = r / gm;
}

// Work item of a CTA pair: output block, contraction range and (MODE 2) the filter tap.
struct PairTile {
  int mb, nb, kb_begin, kb_end, tap, ks;
};

template <int BN, int MODE>
__device__ __forceinline__ int pair_num_tiles(const GemmParams& p, int m_blocks, int n_blocks) {
  return MODE == 2 ? m_blocks * n_blocks * p.taps * p.ksplit : m_blocks * n_blocks;
}

template <int MODE>
__device__ __forceinline__ PairTile pair_tile(const GemmParams& p, int tile, int m_blocks, int n_blocks,
                                              int k_blocks) {
  PairTile t;
  if constexpr (MODE == 2) {
    // pixel range slowest: the tiles that run together read the same rows of dY and X
    const int mn = m_blocks * n_blocks;
    const int per_ks = mn * p.taps;
    const int ks = tile / per_ks;
    t.ks = ks;
    const int r = tile - ks * per_ks;
    t.tap = r / mn;
    const int q = r - t.tap * mn;
    t.mb = q % m_blocks;
    t.nb = q / m_blocks;
    const int per = (k_blocks + p.ksplit - 1) / p.ksplit;
    t.kb_begin = ks * per;
    t.kb_end = min(k_blocks, t.kb_begin + per);
  } else {
    pair_tile_coords(tile, m_blocks, n_blocks, t.mb, t.nb);
    t.kb_begin = 0;
    t.kb_end = k_blocks;
    t.tap = 0;
    t.ks = 0;
  }
  return t;
}

template <int BN, bool A_MN, bool B_MN, int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using Cfg = PairCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int BNH = Cfg::BNH;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi = smem + STAGES * Cfg::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + Cfg::EPI_BYTES);
  // bars[0..S) full (used in the leader), [S..2S) empty, [2S..2S+2) tmem_full,
  // [2S+2..2S+4) tmem_empty (used in the leader)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  const int m_blocks = (p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
  const int n_blocks = (p.N + BN - 1) / BN;
  const int k_blocks = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int num_tiles = pair_num_tiles<BN, MODE>(p, m_blocks, n_blocks);
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 8);  // four epilogue warps in each CTA of the pair
    }
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 2) {
    tmem_alloc_pair(smem_u32(tmem_slot), Cfg::TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers are initialised before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer (both CTAs)
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        const PairTile t = pair_tile<MODE>(p, tile, m_blocks, n_blocks, k_blocks);
        const int m0 = t.mb * 2 * GEMM_BM + static_cast<int>(rank) * GEMM_BM;
        const int n0 = t.nb * BN + static_cast<int>(rank) * BNH;
        for (int kb = t.kb_begin; kb < t.kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) {
            ok = false;
            break;
          }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
          // the leader's barrier counts the bytes of both CTAs
          if (leader) mbar_expect_tx(full_bar(stage), 2 * Cfg::STAGE_BYTES);
          const uint32_t fb = mapa_shared(full_bar(stage), 0);
          const int k0 = kb * GEMM_BK;
          if constexpr (MODE == 1) {
            // k-block = (tap, 64 channels): A rows shifted by the tap's offset in the padded image
            const int tap = kb / p.cblocks;
            tma_load_2d_pair(sA, &tmA, fb, (kb - tap * p.cblocks) * GEMM_BK, m0 + p.shift[tap]);
          } else if constexpr (!A_MN) {
            tma_load_2d_pair(sA, &tmA, fb, k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < GEMM_BM / 64; ++c)
              tma_load_2d_pair(sA + c * (GEMM_BK * 128), &tmA, fb, m0 + c * 64, k0);
          }
          if constexpr (!B_MN) {
            tma_load_2d_pair(sB, &tmB, fb, k0, n0);
          } else {
            // MODE 2: the pixels of X that tap t pairs with the pixels [k0, k0 + 64) of dY
            const int kx = MODE == 2 ? k0 + p.shift[t.tap] : k0;
#pragma unroll
            for (int c = 0; c < BNH / 64; ++c)
              tma_load_2d_pair(sB + c * (GEMM_BK * 128), &tmB, fb, n0 + c * 64, kx);
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(2 * GEMM_BM, BN, 1, A_MN ? 1 : 0, B_MN ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
        const PairTile t = pair_tile<MODE>(p, tile, m_blocks, n_blocks, k_blocks);
        if (!mbar_wait_cluster(tempty_bar(acc), acc_phase ^ 1u, abort_word, FT_ERR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = t.kb_begin; kb < t.kb_end; ++kb) {
          if (!mbar_wait_cluster(full_bar(stage), phase, abort_word, FT_ERR_TIMEOUT_MMA)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES;
          const uint32_t sB = sA + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            const uint64_t adesc = A_MN ? make_smem_desc_sw128(sA + k * 2048, GEMM_BK * 128, 1024)
                                        : make_smem_desc_sw128(sA + k * 32, 16, 1024);
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sB + k * 2048, GEMM_BK * 128, 1024)
                                        : make_smem_desc_sw128(sB + k * 32, 16, 1024);
            umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb > t.kb_begin || k > 0) ? 1u : 0u);
          }
          umma_commit_pair(empty_bar(stage), 3);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(tfull_bar(acc), 3);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue (both CTAs)
    const int ew = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool out_f32 = (p.flags & GEMM_OUT_F32) != 0;
    const bool accumulate = (p.flags & GEMM_ACCUMULATE) != 0;
    const bool has_bias = (p.flags & (GEMM_BIAS | GEMM_BIAS_F32)) != 0;
    const bool has_act = (p.flags & (GEMM_RELU | GEMM_GELU | GEMM_SILU)) != 0;
    const bool direct = (p.flags & GEMM_EPI_DIRECT) != 0;
    const uint32_t stage_tiles = smem_u32(epi) + static_cast<uint32_t>(ew) * 2u * Cfg::EPI_TILE_BYTES;
    int buf = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs) {
      const PairTile t = pair_tile<MODE>(p, tile, m_blocks, n_blocks, k_blocks);
      const int m0 = t.mb * 2 * GEMM_BM + static_cast<int>(rank) * GEMM_BM + ew * 32;
      const int n0 = t.nb * BN;
      const int c_off = MODE == 2 ? t.tap * p.N : 0;  // dW[co, tap, ci]: tap t starts at column t * Cin
      const int r_off = MODE == 2 ? t.ks * p.split_rows : 0;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) +
                             static_cast<uint32_t>(acc * BN);
      if (MODE == 1 && p.cHo > 0) {
        epilogue_crop<BN>(p, t_row, m0 + lane, n0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));
      } else if (p.flags & GEMM_EPI_TRANSPOSED) {
        epilogue_transposed<BN>(p, t_row, m0 + lane, n0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));
      } else if (direct) {
        epilogue_direct<BN>(p, t_row, m0 + lane, n0);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));
      } else {
        const int step_cols = out_f32 ? 32 : 64;
        const int steps = BN / step_cols;
#pragma unroll 1
        for (int c = 0; c < steps; ++c) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(t_row + c * step_cols, r0);
          if (!out_f32) {
            tmem_ld_32x32(t_row + c * step_cols + 32, r1);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r1[j] = 0u;
          }
          tmem_ld_wait();
          if (c == steps - 1) {
            // the accumulator is in registers: hand it back before the stores are issued
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty_bar(acc), 0));
          }
          const int col0 = n0 + c * step_cols;
          if (m0 >= p.M || col0 >= p.N) continue;  // warp-uniform: nothing of this piece is inside C
          if (has_bias) {
#pragma unroll
            for (int j = 0; j < 64; ++j) {
              const int col = col0 + j;
              if (j < step_cols && col < p.N) {
                const float b = (p.flags & GEMM_BIAS_F32)
                                    ? static_cast<const float*>(p.bias)[col]
                                    : __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col]);
                uint32_t& x = j < 32 ? r0[j & 31] : r1[j & 31];
                x = __float_as_uint(__uint_as_float(x) + b);
              }
            }
          }
          if (has_act) {
#pragma unroll
            for (int j = 0; j < 64; ++j)
              if (j < step_cols) {
                uint32_t& x = j < 32 ? r0[j & 31] : r1[j & 31];
                x = __float_as_uint(apply_act(__uint_as_float(x), p.flags));
              }
          }
          // the store issued two steps ago has finished reading this staging tile
          if (lane == 0) tma_store_wait_read<1>();
          __syncwarp();
          const uint32_t tile_s = stage_tiles + static_cast<uint32_t>(buf) * Cfg::EPI_TILE_BYTES;
          const uint32_t row_s = tile_s + static_cast<uint32_t>(lane) * 128u;
          const uint32_t sw = static_cast<uint32_t>(lane & 7);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint32_t x, y, z, w;
            if (out_f32) {
              x = r0[4 * j]; y = r0[4 * j + 1]; z = r0[4 * j + 2]; w = r0[4 * j + 3];
            } else {
              const uint32_t(&q)[32] = j < 4 ? r0 : r1;
              const int o = 8 * (j & 3);
              x = pack_bf16x2(__uint_as_float(q[o]), __uint_as_float(q[o + 1]));
              y = pack_bf16x2(__uint_as_float(q[o + 2]), __uint_as_float(q[o + 3]));
              z = pack_bf16x2(__uint_as_float(q[o + 4]), __uint_as_float(q[o + 5]));
              w = pack_bf16x2(__uint_as_float(q[o + 6]), __uint_as_float(q[o + 7]));
            }
            const uint32_t dst = row_s + ((static_cast<uint32_t>(j) ^ sw) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(x), "r"(y), "r"(z),
                         "r"(w)
                         : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (accumulate)
              tma_reduce_add_2d(&tmC, tile_s, c_off + col0, r_off + m0);
            else
              tma_store_2d(&tmC, tile_s, c_off + col0, r_off + m0);
            tma_store_commit();
          }
          buf ^= 1;
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    // shared memory must outlive the stores that read it
    if (lane == 0) tma_store_wait<0>();
    __syncwarp();
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA frees TMEM or exits while its peer can still reach it
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status != nullptr) atomicCAS(p.status, 0, *abort_word);
}

template <int BN, bool A_MN, bool B_MN, int MODE = 0>
static int launch_pair(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                       const GemmParams& p, int device, int max_ctas, cudaStream_t stream) {
  using Cfg = PairCfg<BN>;
  auto kern = gemm_bf16_pair_kernel<BN, A_MN, B_MN, MODE>;
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES));
    attr_set[device] = true;
  }
  const int m_blocks = (p.M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
  const int n_blocks = (p.N + BN - 1) / BN;
  int pairs = m_blocks * n_blocks * (MODE == 2 ? p.taps * p.ksplit : 1);
  int sms = sm_count(device);
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (pairs > sms / 2) pairs = sms / 2;
  if (pairs < 1) pairs = 1;
  kern<<<2 * pairs, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

template <int BN>
static int dispatch_pair(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                         const CUtensorMap& tmC, const GemmParams& p, int device, int max_ctas,
                         cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_pair<BN, false, false>(tmA, tmB, tmC, p, device, max_ctas, stream);
  if (!a_mn && b_mn) return launch_pair<BN, false, true>(tmA, tmB, tmC, p, device, max_ctas, stream);
  if (a_mn && !b_mn) return launch_pair<BN, true, false>(tmA, tmB, tmC, p, device, max_ctas, stream);
  return launch_pair<BN, true, true>(tmA, tmB, tmC, p, device, max_ctas, stream);
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmParams& p, int device,
                       int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  auto kern = gemm_bf16_tcgen05_kernel<BN, A_MN, B_MN>;
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::SMEM_BYTES));
    attr_set[device] = true;
  }
  const int m_blocks = (p.M + GEMM_BM - 1) / GEMM_BM;
  const int n_blocks = (p.N + BN - 1) / BN;
  int grid = m_blocks * n_blocks;
  int sms = sm_count(device);
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (grid > sms) grid = sms;
  kern<<<grid, GEMM_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

template <int BN>
static int dispatch_major(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                          const GemmParams& p, int device, int max_ctas, cudaStream_t stream) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false>(tmA, tmB, p, device, max_ctas, stream);
  if (!a_mn && b_mn) return launch_gemm<BN, false, true>(tmA, tmB, p, device, max_ctas, stream);
  if (a_mn && !b_mn) return launch_gemm<BN, true, false>(tmA, tmB, p, device, max_ctas, stream);
  return launch_gemm<BN, true, true>(tmA, tmB, p, device, max_ctas, stream);
}

}  // namespace ft

// C[M,N] (+)= A * B^T (+bias).  A is [M,K] (a_mn_major = 0, row stride lda) or stored
// transposed as [K,M] (a_mn_major = 1); B is [N,K] (b_mn_major = 0) or stored as
// [K,N] (b_mn_major = 1).  Strides are in elements.  bn = 0 picks the N tile
// automatically, a negative bn selects the one-CTA kernel with an N tile of -bn; max_ctas > 0 limits the persistent grid (used to leave SMs to a
// concurrent communication kernel).  Returns 0 or a negative error code
// (ft_last_error() has the text).
FT_API int ft_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K,
                        long long lda, long long ldb, long long ldc, int a_mn_major, int b_mn_major,
                        int flags, int bn, int max_ctas, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  using namespace ft;
  FT_REQUIRE(A && B && C, "ft_gemm_bf16: null operand");
  FT_REQUIRE(M > 0 && N > 0 && K > 0, "ft_gemm_bf16: empty problem %dx%dx%d", M, N, K);
  FT_REQUIRE(lda % 8 == 0 && ldb % 8 == 0, "ft_gemm_bf16: lda/ldb must be multiples of 8 elements");
  const bool out_f32 = flags & GEMM_OUT_F32;
  FT_REQUIRE(N % 8 == 0 && ldc % (out_f32 ? 4 : 8) == 0,
             "ft_gemm_bf16: N (%d) must be a multiple of 8 and ldc 16-byte aligned", N);
  FT_REQUIRE((reinterpret_cast<uintptr_t>(C) & 15) == 0, "ft_gemm_bf16: C must be 16-byte aligned");
  FT_REQUIRE(!(flags & (GEMM_BIAS | GEMM_BIAS_F32)) || bias, "ft_gemm_bf16: bias flag without bias");
  const bool force_single = bn < 0;
  if (force_single) bn = -bn;
  const bool has_act = (flags & (GEMM_RELU | GEMM_GELU | GEMM_SILU)) != 0;
  const bool accumulate = (flags & GEMM_ACCUMULATE) != 0;
  flags &= 0xFFFF;

  CUtensorMap tmA, tmB;
  int rc;
  GemmParams p;
  p.C = C; p.bias = bias; p.M = M; p.N = N; p.K = K; p.ldc = ldc; p.flags = flags;
  p.status = device_status_word(device);
  p.taps = 0; p.cblocks = 0; p.ksplit = 1;
  p.gHp = p.gWp = p.cHo = p.cWo = p.c_oh = p.c_ow = 0; p.split_rows = 0;

  // Problems with at least one full 256-row block and N >= 128 run on the CTA-pair kernel.
  if (!force_single && M >= 2 * GEMM_BM && N >= 128 && (bn == 0 || bn >= 128)) {
    const int pairs = (max_ctas > 0 && max_ctas < sm_count(device) ? max_ctas : sm_count(device)) / 2;
    const long long mb2 = (M + 2 * GEMM_BM - 1) / (2 * GEMM_BM);
    int pbn = bn ? bn : 256;
    if (bn == 0 && mb2 * ((N + 255) / 256) < pairs) pbn = 128;  // too few 256-wide tiles to fill the GPU
    if (N < 256) pbn = 128;
    // bf16 C += ... adds in fp32 before rounding once; an activation after the accumulation
    // also needs the old value in registers: both use the per-lane epilogue.
    if ((accumulate && !out_f32) || (accumulate && has_act)) p.flags |= GEMM_EPI_DIRECT;
    if (!a_mn_major)
      rc = make_tmap_2d(&tmA, A, 2, K, M, lda * 2, GEMM_BK, GEMM_BM, 3);
    else
      rc = make_tmap_2d(&tmA, A, 2, M, K, lda * 2, 64, GEMM_BK, 3);
    if (rc) return rc;
    if (!b_mn_major)
      rc = make_tmap_2d(&tmB, B, 2, K, N, ldb * 2, GEMM_BK, pbn / 2, 3);
    else
      rc = make_tmap_2d(&tmB, B, 2, N, K, ldb * 2, 64, GEMM_BK, 3);
    if (rc) return rc;
    CUtensorMap tmC;
    if (out_f32)
      rc = make_tmap_2d(&tmC, C, 4, N, M, ldc * 4, 32, 32, 3);
    else
      rc = make_tmap_2d(&tmC, C, 2, N, M, ldc * 2, 64, 32, 3);
    if (rc) return rc;
    if (pbn == 256) return dispatch_pair<256>(a_mn_major, b_mn_major, tmA, tmB, tmC, p, device, max_ctas, stream);
    return dispatch_pair<128>(a_mn_major, b_mn_major, tmA, tmB, tmC, p, device, max_ctas, stream);
  }

  if (bn == 0) {
    const int sms = sm_count(device);
    const long long mb = (M + GEMM_BM - 1) / GEMM_BM;
    bn = 256;
    while (bn > 32 && mb * ((N + bn - 1) / bn) < sms) bn >>= 1;
    if (N <= 32) bn = 32; else if (N <= 64 && bn > 64) bn = 64; else if (N <= 128 && bn > 128) bn = 128;
  }
  FT_REQUIRE(bn == 256 || bn == 128 || bn == 64 || bn == 32, "ft_gemm_bf16: bad N tile %d", bn);
  // an MN-major B tile is loaded in 64-element (128-byte swizzle) column chunks
  if (b_mn_major && bn < 64) bn = 64;

  if (!a_mn_major)
    rc = make_tmap_2d(&tmA, A, 2, K, M, lda * 2, GEMM_BK, GEMM_BM, 3);
  else
    rc = make_tmap_2d(&tmA, A, 2, M, K, lda * 2, 64, GEMM_BK, 3);
  if (rc) return rc;
  if (!b_mn_major)
    rc = make_tmap_2d(&tmB, B, 2, K, N, ldb * 2, GEMM_BK, bn, 3);
  else
    rc = make_tmap_2d(&tmB, B, 2, N, K, ldb * 2, 64, GEMM_BK, 3);
  if (rc) return rc;

  switch (bn) {
    case 256: return dispatch_major<256>(a_mn_major, b_mn_major, tmA, tmB, p, device, max_ctas, stream);
    case 128: return dispatch_major<128>(a_mn_major, b_mn_major, tmA, tmB, p, device, max_ctas, stream);
    case 64: return dispatch_major<64>(a_mn_major, b_mn_major, tmA, tmB, p, device, max_ctas, stream);
    default: return dispatch_major<32>(a_mn_major, b_mn_major, tmA, tmB, p, device, max_ctas, stream);
  }
}

// Convolution as a shifted-row GEMM (MODE 1 of the CTA-pair kernel).  xp: the input, zero-padded
// and flattened to [P, Cin] bf16 (P = images * padded height * padded width; row stride ldx
// elements), w: the filter as [Cout, taps * Cin] bf16 (OHWI order: tap-major, channel-minor),
// y: [P, Cout] bf16 (flags & 1: fp32) in the same padded pixel numbering -- rows that are padding
// hold values the caller drops.  shift[t]: row offset of tap t, e.g. (kh - pad_h) * Wp + (kw -
// pad_w) for a stride-1 filter.  xp has x_rows >= P rows (more when shifts reach into further
// planes of a stride-2 parity split).  bias / ReLU flags as in ft_gemm_bf16.  Cin % 64 == 0,
// Cout % 8 == 0.  crop (optional): {Hp, Wp, Ho, Wo, oh, ow} -- the GEMM rows form [images, Hp, Wp]
// grids and only the Ho x Wo window at (oh, ow) of each is written, densely, as [images, Ho, Wo,
// Cout]; y then has images * Ho * Wo rows.
FT_API int ft_conv_shift_gemm(const void* xp, const void* w, void* y, const void* bias, long long P,
                              long long x_rows, int Cin, int Cout, int taps, const int* shift, long long ldx,
                              long long ldy, int flags, const int* crop, int max_ctas, int device,
                              cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  using namespace ft;
  FT_REQUIRE(xp && w && y && shift, "ft_conv_shift_gemm: null pointer");
  FT_REQUIRE(P > 0 && P < (1ll << 31) - 65536 && Cin > 0 && Cin % 64 == 0 && Cout > 0 && Cout % 8 == 0,
             "ft_conv_shift_gemm: bad shape P=%lld Cin=%d Cout=%d", P, Cin, Cout);
  FT_REQUIRE(taps >= 1 && taps <= GEMM_MAX_TAPS, "ft_conv_shift_gemm: %d taps (1..%d)", taps, GEMM_MAX_TAPS);
  const bool out_f32 = flags & GEMM_OUT_F32;
  FT_REQUIRE(ldx % 8 == 0 && ldy % (out_f32 ? 4 : 8) == 0 && (reinterpret_cast<uintptr_t>(y) & 15) == 0,
             "ft_conv_shift_gemm: strides / output must be 16-byte aligned");
  FT_REQUIRE(!(flags & GEMM_ACCUMULATE), "ft_conv_shift_gemm: accumulation is not supported");
  FT_REQUIRE(!(flags & (GEMM_BIAS | GEMM_BIAS_F32)) || bias, "ft_conv_shift_gemm: bias flag without bias");
  GemmParams p;
  p.C = y; p.bias = bias; p.M = static_cast<int>(P); p.N = Cout; p.K = taps * Cin; p.ldc = ldy;
  p.flags = flags & 0xFFFF;
  p.status = device_status_word(device);
  p.taps = taps; p.cblocks = Cin / GEMM_BK; p.ksplit = 1;
  for (int t = 0; t < GEMM_MAX_TAPS; ++t) p.shift[t] = t < taps ? shift[t] : 0;
  p.gHp = p.gWp = p.cHo = p.cWo = p.c_oh = p.c_ow = 0; p.split_rows = 0;
  long long y_rows = P;
  if (crop) {
    p.gHp = crop[0]; p.gWp = crop[1]; p.cHo = crop[2]; p.cWo = crop[3]; p.c_oh = crop[4]; p.c_ow = crop[5];
    FT_REQUIRE(p.gHp > 0 && p.gWp > 0 && p.cHo > 0 && p.cWo > 0 && p.c_oh >= 0 && p.c_ow >= 0 &&
                   p.cHo + p.c_oh <= p.gHp && p.cWo + p.c_ow <= p.gWp && P % (static_cast<long long>(p.gHp) * p.gWp) == 0,
               "ft_conv_shift_gemm: the crop window does not fit the %d x %d grid", p.gHp, p.gWp);
    y_rows = P / (static_cast<long long>(p.gHp) * p.gWp) * p.cHo * p.cWo;
  }
  const int bn = Cout >= 256 ? 256 : (Cout > 64 ? 128 : 64);
  CUtensorMap tmA, tmB, tmC;
  FT_REQUIRE(x_rows >= P && x_rows < (1ll << 31), "ft_conv_shift_gemm: x_rows=%lld must be >= P=%lld", x_rows, P);
  int rc = make_tmap_2d(&tmA, xp, 2, Cin, x_rows, ldx * 2, GEMM_BK, GEMM_BM, 3);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, w, 2, static_cast<uint64_t>(taps) * Cin, Cout, static_cast<uint64_t>(taps) * Cin * 2,
                    GEMM_BK, bn / 2, 3);
  if (rc) return rc;
  rc = out_f32 ? make_tmap_2d(&tmC, y, 4, Cout, y_rows, ldy * 4, 32, 32, 3)
               : make_tmap_2d(&tmC, y, 2, Cout, y_rows, ldy * 2, 64, 32, 3);
  if (rc) return rc;
  if (bn == 256) return launch_pair<256, false, false, 1>(tmA, tmB, tmC, p, device, max_ctas, stream);
  if (bn == 128) return launch_pair<128, false, false, 1>(tmA, tmB, tmC, p, device, max_ctas, stream);
  return launch_pair<64, false, false, 1>(tmA, tmB, tmC, p, device, max_ctas, stream);
}

// Filter gradient of the same convolution (MODE 2): dw[Cout, taps * Cin] (fp32) +=
// sum_p dyp[p, co] * xp[p + shift[t], ci].  dyp: [P, Cout] bf16 with zeros in the padding rows,
// xp: [P, Cin] bf16.  The pixel dimension is cut into `ksplit` pieces (0 = chosen here) whose
// tiles are added into dw by the memory system, so the summation order, and with it the last
// bits of dw, can differ from run to run.  Cout % 64 == 0; Cin % 64 == 0 (Cin % 8 == 0 suffices
// for a single tap, i.e. a plain dY^T X product with the pixels as the split contraction).
FT_API int ft_conv_shift_wgrad(const void* dyp, const void* xp, float* dw, long long P, long long x_rows,
                               int Cin, int Cout, int taps, const int* shift, long long lddy, long long ldx,
                               int ksplit, int max_ctas, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  using namespace ft;
  FT_REQUIRE(dyp && xp && dw && shift, "ft_conv_shift_wgrad: null pointer");
  // with several taps, tap t's columns start at t * Cin and a 64-wide B chunk must not straddle them
  FT_REQUIRE(P > 0 && P < (1ll << 31) - 65536 && Cin > 0 && Cin % (taps > 1 ? 64 : 8) == 0 && Cout > 0 &&
                 Cout % 64 == 0,
             "ft_conv_shift_wgrad: bad shape P=%lld Cin=%d Cout=%d", P, Cin, Cout);
  FT_REQUIRE(taps >= 1 && taps <= GEMM_MAX_TAPS, "ft_conv_shift_wgrad: %d taps (1..%d)", taps, GEMM_MAX_TAPS);
  FT_REQUIRE(lddy % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(dw) & 15) == 0,
             "ft_conv_shift_wgrad: strides / output must be 16-byte aligned");
  GemmParams p;
  p.C = dw; p.bias = nullptr; p.M = Cout; p.N = Cin; p.K = static_cast<int>(P);
  p.ldc = static_cast<long long>(taps) * Cin;
  p.flags = GEMM_OUT_F32 | GEMM_ACCUMULATE;
  p.status = device_status_word(device);
  p.gHp = p.gWp = p.cHo = p.cWo = p.c_oh = p.c_ow = 0; p.split_rows = 0;
  p.taps = taps; p.cblocks = Cin / GEMM_BK;
  for (int t = 0; t < GEMM_MAX_TAPS; ++t) p.shift[t] = t < taps ? shift[t] : 0;
  const int bn = Cin >= 256 ? 256 : 128;
  const int k_blocks = static_cast<int>((P + GEMM_BK - 1) / GEMM_BK);
  if (ksplit <= 0) {
    const int pairs = (max_ctas > 0 && max_ctas < sm_count(device) ? max_ctas : sm_count(device)) / 2;
    const int mn = ((Cout + 255) / 256) * ((Cin + bn - 1) / bn) * taps;
    ksplit = (2 * pairs + mn - 1) / mn;          // about two tiles per CTA pair
    const int max_split = k_blocks / 8 > 0 ? k_blocks / 8 : 1;  // at least 8 k-blocks per tile
    if (ksplit > max_split) ksplit = max_split;
    if (ksplit < 1) ksplit = 1;
  }
  if (ksplit > k_blocks) ksplit = k_blocks;
  // no piece may be empty: an empty piece would add an unwritten accumulator into dw
  const int per = (k_blocks + ksplit - 1) / ksplit;
  p.ksplit = (k_blocks + per - 1) / per;
  CUtensorMap tmA, tmB, tmC;
  int rc = make_tmap_2d(&tmA, dyp, 2, Cout, P, lddy * 2, 64, GEMM_BK, 3);
  if (rc) return rc;
  FT_REQUIRE(x_rows >= P && x_rows < (1ll << 31), "ft_conv_shift_wgrad: x_rows=%lld must be >= P=%lld", x_rows, P);
  rc = make_tmap_2d(&tmB, xp, 2, Cin, x_rows, ldx * 2, 64, GEMM_BK, 3);
  if (rc) return rc;
  rc = make_tmap_2d(&tmC, dw, 4, static_cast<uint64_t>(taps) * Cin, Cout, static_cast<uint64_t>(taps) * Cin * 4,
                    32, 32, 3);
  if (rc) return rc;
  if (bn == 256) return launch_pair<256, true, true, 2>(tmA, tmB, tmC, p, device, max_ctas, stream);
  return launch_pair<128, true, true, 2>(tmA, tmB, tmC, p, device, max_ctas, stream);
}

namespace ft {

// ws holds the pieces of the split contraction: C^T as fp32 [ksplit][slice_rows >= N, ld_ws].  Write
// C[m, n] = sum_ks ws[ks][n, m] (+ bias[n]) (+ residual[m, n]) as bf16; the pieces are summed in
// index order, so the result does not depend on which CTA finished first.
__global__ void small_m_finalize_kernel(const float* __restrict__ ws, __nv_bfloat16* __restrict__ C,
                                        const __nv_bfloat16* __restrict__ residual, const void* __restrict__ bias,
                                        int bias_f32, int M, int N, int ld_ws, int ksplit, int slice_rows,
                                        long long ldc, long long ldr) {
  // block = 32 x 8 threads over a 32 (n) x 32 (m) patch, transposed through shared memory
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
  const long long slice = static_cast<long long>(slice_rows) * ld_ws;
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int n = n0 + i, m = m0 + threadIdx.x;
    float v = 0.f;
    if (n < N && m < ld_ws) {
      const float* src = ws + static_cast<long long>(n) * ld_ws + m;
      for (int ks = 0; ks < ksplit; ++ks) v += src[ks * slice];
    }
    tile[i][threadIdx.x] = v;
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += 8) {
    const int m = m0 + i, n = n0 + threadIdx.x;
    if (m < M && n < N) {
      float v = tile[threadIdx.x][i];
      if (bias) v += bias_f32 ? static_cast<const float*>(bias)[n] : __bfloat162float(static_cast<const __nv_bfloat16*>(bias)[n]);
      if (residual) v += __bfloat162float(residual[static_cast<long long>(m) * ldr + n]);
      C[static_cast<long long>(m) * ldc + n] = __float2bfloat16(v);
    }
  }
}

}  // namespace ft

constexpr int SMALL_M_MAX_SPLIT = 16;

// Floats of workspace ft_gemm_small_m may need for an [M, N] result (its contents do not matter).
FT_API long long ft_gemm_small_m_workspace(int M, int N) {
  const int mpad = M <= 64 ? 64 : 128;
  return static_cast<long long>((N + 255) / 256 * 256) * mpad * SMALL_M_MAX_SPLIT;
}

// C[M, N] = X[M, K] W[N, K]^T (+ bias[N]) (+ residual[M, N]) for a small batch M <= 128 (decode):
// the weight is the 128-row MMA operand, so every byte of W crosses the tensor core once with all
// 128 rows in use and the batch is only the (64- or 128-wide) N dimension of the instruction.
// When N / 256 tiles would leave most SMs idle, the contraction is split across CTA pairs; each
// piece stores its fp32 partial tile into its own slice of `workspace` and a second small kernel
// sums the slices in index order (deterministic) and writes C.  workspace:
// ft_gemm_small_m_workspace(M, N) floats, contents irrelevant (may be null when no split is
// needed; then residual must be null).
// All of X, W, C bf16; K-major operands; ldx, ldw, ldc, ldr in elements.
FT_API int ft_gemm_small_m(const void* X, const void* W, void* C, const void* bias, const void* residual,
                           float* workspace, int M, int N, int K, long long ldx, long long ldw, long long ldc,
                           long long ldr, int flags, int ksplit, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  using namespace ft;
  FT_REQUIRE(X && W && C, "ft_gemm_small_m: null operand");
  FT_REQUIRE(M > 0 && M <= 128 && N > 0 && K > 0, "ft_gemm_small_m: M=%d must be in 1..128 (N=%d K=%d)", M, N, K);
  FT_REQUIRE(ldx % 8 == 0 && ldw % 8 == 0 && N % 8 == 0, "ft_gemm_small_m: strides and N must be multiples of 8");
  FT_REQUIRE(!(flags & (GEMM_OUT_F32 | GEMM_ACCUMULATE)), "ft_gemm_small_m: bf16 output, no accumulation");
  FT_REQUIRE(!(flags & (GEMM_BIAS | GEMM_BIAS_F32)) || bias, "ft_gemm_small_m: bias flag without bias");
  const int bn = M <= 64 ? 64 : 128;
  const int sms = sm_count(device);
  const int pairs = sms / 2;
  const int tiles = (N + 255) / 256;
  const int k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  if (ksplit <= 0) {
    ksplit = 1;
    if (tiles < pairs && workspace) {
      // one wave: as many pieces per tile as there are CTA pairs to take them, each piece long
      // enough (>= 4 k-blocks) to be worth a pipeline fill
      ksplit = pairs / tiles;
      const int max_split = k_blocks / 4 > 0 ? k_blocks / 4 : 1;
      if (ksplit > max_split) ksplit = max_split;
      if (ksplit < 1) ksplit = 1;
    }
  }
  if (ksplit > SMALL_M_MAX_SPLIT) ksplit = SMALL_M_MAX_SPLIT;
  // the residual is added by the finalize pass, which only the split path has
  if (residual && ksplit == 1 && workspace && k_blocks >= 2) ksplit = 2;
  FT_REQUIRE(ksplit == 1 || workspace, "ft_gemm_small_m: a split contraction needs the workspace");
  FT_REQUIRE(ksplit > 1 || !residual, "ft_gemm_small_m: the residual is added by the split path only");
  GemmParams p;
  p.bias = bias; p.M = N; p.N = M; p.K = K;   // tile space: rows of W x batch
  p.status = device_status_word(device);
  p.taps = ksplit > 1 ? 1 : 0; p.cblocks = 0; p.ksplit = 1;
  for (int t = 0; t < GEMM_MAX_TAPS; ++t) p.shift[t] = 0;
  p.gHp = p.gWp = p.cHo = p.cWo = p.c_oh = p.c_ow = 0; p.split_rows = 0;
  CUtensorMap tmA, tmB, tmC;
  int rc = make_tmap_2d(&tmA, W, 2, K, N, ldw * 2, GEMM_BK, GEMM_BM, 3);
  if (rc) return rc;
  rc = make_tmap_2d(&tmB, X, 2, K, M, ldx * 2, GEMM_BK, bn / 2, 3);
  if (rc) return rc;
  if (ksplit == 1) {
    p.C = C; p.ldc = ldc;
    p.flags = (flags & 0xFFFF) | GEMM_EPI_TRANSPOSED;
    // the store map is not used by the transposed epilogue; point it at W so that it is valid
    rc = make_tmap_2d(&tmC, W, 2, K, N, ldw * 2, 64, 32, 3);
    if (rc) return rc;
    return bn == 64 ? launch_pair<64, false, false, 0>(tmA, tmB, tmC, p, device, 0, stream)
                    : launch_pair<128, false, false, 0>(tmA, tmB, tmC, p, device, 0, stream);
  }
  const int per = (k_blocks + ksplit - 1) / ksplit;
  p.ksplit = (k_blocks + per - 1) / per;
  p.C = workspace; p.ldc = bn;
  p.flags = GEMM_OUT_F32;
  // a slice is a whole number of 256-row tiles, so a tile that hangs over the end of W stays
  // inside its own slice
  p.split_rows = tiles * 256;
  rc = make_tmap_2d(&tmC, workspace, 4, bn, static_cast<uint64_t>(p.ksplit) * p.split_rows,
                    static_cast<uint64_t>(bn) * 4, 32, 32, 3);
  if (rc) return rc;
  rc = bn == 64 ? launch_pair<64, false, false, 2>(tmA, tmB, tmC, p, device, 0, stream)
                : launch_pair<128, false, false, 2>(tmA, tmB, tmC, p, device, 0, stream);
  if (rc) return rc;
  dim3 grid((N + 31) / 32, (M + 31) / 32), block(32, 8);
  small_m_finalize_kernel<<<grid, block, 0, stream>>>(workspace, static_cast<__nv_bfloat16*>(C),
                                                      static_cast<const __nv_bfloat16*>(residual), bias,
                                                      (flags & GEMM_BIAS_F32) ? 1 : 0, M, N, bn, p.ksplit,
                                                      p.split_rows, ldc, ldr);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}
