// Implicit-GEMM 2-D convolution forward on tcgen05 (sm_100a), NHWC bf16, fp32 accumulation:
//
//   y[n, ho, wo, co] = sum_{kh, kw, ci} x[n, ho*s - p + kh*d, wo*s - p + kw*d, ci] * w[co, kh, kw, ci]  (+ bias, ReLU)
//
// The reference lowers Conv2d to an explicit im2col buffer followed by an SGEMM
// (ferrotorch-gpu/src/conv.rs:520) and runs the backward pass on the host (ferrotorch-nn/src/
// conv.rs:1173).  Here the im2col matrix is never written: the GEMM is
//   D[M = N*Ho*Wo, Cout] = A[M, K = KH*KW*Cin] * W[Cout, K]^T
// and a 128 x 64 tile of A is one filter tap (kh, kw) and 64 consecutive input channels of 128
// output pixels, i.e. 128 rows of 128 contiguous bytes of x (or zeros in the padding).  Eight
// gather warps fetch those rows with plain 16-byte loads (two threads per row, several k-blocks
// ahead) and store them in the swizzled K-major layout the MMA descriptor expects, exactly as the
// expander warps of quant_gemm.cu do for compressed weights; the filter tile comes by TMA from
// the [Cout, K] matrix that an OHWI weight tensor already is.  Input-gradient of a stride-1
// convolution is the same kernel on dy with the filter flipped and its channel axes swapped
// (done on the host side of the binding).  All waits are bounded.
//
// Requirements: Cin % 64 == 0 (a k-block never straddles a tap), Cout % 8 == 0, 16-byte aligned x / w / y.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int CV_BM = 128, CV_BN = 128, CV_BK = 64;
constexpr int CV_THREADS = 512;   // warp 0 TMA (filter), 1 MMA, 2 TMEM, 3 idle, 4-7 epilogue, 8-15 gather
constexpr int CV_X_BYTES = CV_BM * CV_BK * 2, CV_W_BYTES = CV_BN * CV_BK * 2;
constexpr int CV_STAGE = CV_X_BYTES + CV_W_BYTES;
constexpr int CV_STAGES = 6;
constexpr int CV_BAR_OFF = CV_STAGES * CV_STAGE;
constexpr int CV_SMEM = CV_BAR_OFF + 1024 + 256;
constexpr int CV_PF = 2;          // k-blocks whose rows a gather thread holds in registers ahead of the store

struct ConvParams {
  const __nv_bfloat16* x;   // [N, H, W, Cin]
  __nv_bfloat16* y;         // [N, Ho, Wo, Cout]
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;   // optional [N, Ho, Wo, Cout], added before the activation
  int N, H, W, Cin, Cout, KH, KW, Ho, Wo;
  int stride, pad_h, pad_w, dil, relu;
  int M, K;                 // N*Ho*Wo, KH*KW*Cin
  int* status;
};

// Index arithmetic of the gather, shared by the kernel and by a host entry point that the CPU
// tests call: row m of the implicit matrix -> image n and the top-left input coordinate of its window.
__host__ __device__ __forceinline__ void conv_row_origin(const ConvParams& p, int m, int& n, int& hi0, int& wi0) {
  const int wo = m % p.Wo, ho = (m / p.Wo) % p.Ho;
  n = m / (p.Wo * p.Ho);
  hi0 = ho * p.stride - p.pad_h;
  wi0 = wo * p.stride - p.pad_w;
}

// Element offset into x of the 64 channels that k-block kb contributes to a row with the given
// origin, or -1 when the filter tap falls into the padding (the row is zero there).
__host__ __device__ __forceinline__ long long conv_tap_offset(const ConvParams& p, int n, int hi0, int wi0, int kb) {
  const int c_blocks = p.Cin / CV_BK;
  const int tap = kb / c_blocks, c0 = (kb - tap * c_blocks) * CV_BK;
  const int kh = tap / p.KW, kw = tap - kh * p.KW;
  const int hi = hi0 + kh * p.dil, wi = wi0 + kw * p.dil;
  if (hi < 0 || hi >= p.H || wi < 0 || wi >= p.W) return -1;
  return ((static_cast<long long>(n) * p.H + hi) * p.W + wi) * p.Cin + c0;
}

__global__ void __launch_bounds__(CV_THREADS, 1)
conv2d_fprop_tcgen05_kernel(const __grid_constant__ CUtensorMap tmW, const ConvParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + CV_BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * CV_STAGES + 4);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem), bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (CV_STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * CV_STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * CV_STAGES + 2 + a); };
  const int m_blocks = (p.M + CV_BM - 1) / CV_BM, n_blocks = (p.Cout + CV_BN - 1) / CV_BN;
  const int num_tiles = m_blocks * n_blocks, k_blocks = p.K / CV_BK;
  // n fastest: the CTAs that run together read the same pixels (through L2) against different
  // filter tiles; the whole filter is small enough to stay in L2 anyway
  auto coords = [&](int t, int& mb, int& nb) { nb = t % n_blocks; mb = t / n_blocks; };

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < CV_STAGES; ++s) { mbar_init(full_bar(s), 1 + 8); mbar_init(empty_bar(s), 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 4); }
    fence_mbar_init();
    tma_prefetch_desc(&tmW);
  }
  if (warp == 2) { tmem_alloc(smem_u32(tmem_slot), 2 * CV_BN); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ filter tiles by TMA
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int mb, nb; coords(tile, mb, nb);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          mbar_expect_tx(full_bar(stage), CV_W_BYTES);
          tma_load_2d(smem_base + stage * CV_STAGE + CV_X_BYTES, &tmW, full_bar(stage), kb * CV_BK, nb * CV_BN);
          if (++stage == CV_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*abort_word) { const unsigned long long t0 = globaltimer_ns(); while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000); }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_f16(CV_BM, CV_BN, 1, 0, 0);
      int stage = 0, acc = 0; uint32_t phase = 0, acc_phase = 0; bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_word, FT_ERR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * CV_BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_word, FT_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sX = smem_base + stage * CV_STAGE, sW = sX + CV_X_BYTES;
#pragma unroll
          for (int k = 0; k < CV_BK / 16; ++k)
            umma_f16_ss(d, make_smem_desc_sw128(sX + k * 32, 16, 1024), make_smem_desc_sw128(sW + k * 32, 16, 1024),
                        idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit(empty_bar(stage));
          if (++stage == CV_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        acc ^= 1; if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 8) {
    // ------------------------------------------------------------------ gather warps
    // thread g of 256: row r = g / 2 of the pixel tile, 64-byte half h = g % 2 of its 128-byte row
    const int g = threadIdx.x - 256;
    const int r = g >> 1, h = g & 1;
    struct Row { uint4 v[4]; };
    int stage = 0; uint32_t phase = 0; bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int mb, nb; coords(tile, mb, nb);
      const int m = mb * CV_BM + r;
      const bool row_ok = m < p.M;
      int n, hi0, wi0;
      conv_row_origin(p, row_ok ? m : 0, n, hi0, wi0);
      auto fetch = [&](int kb, Row& row) {
        row.v[0] = row.v[1] = row.v[2] = row.v[3] = make_uint4(0, 0, 0, 0);
        if (!row_ok || kb >= k_blocks) return;
        const long long off = conv_tap_offset(p, n, hi0, wi0, kb);
        if (off < 0) return;                                      // padding: the row stays zero
        const uint4* src = reinterpret_cast<const uint4*>(p.x + off + h * 32);
#pragma unroll
        for (int u = 0; u < 4; ++u) row.v[u] = __ldg(src + u);
      };
      Row buf[CV_PF];
#pragma unroll
      for (int i = 0; i < CV_PF; ++i) fetch(i, buf[i]);
      for (int kb0 = 0; kb0 < k_blocks && ok; kb0 += CV_PF) {
#pragma unroll
        for (int j = 0; j < CV_PF; ++j) {
          const int kb = kb0 + j;
          if (kb >= k_blocks || !ok) break;
          const Row cur = buf[j];
          fetch(kb + CV_PF, buf[j]);
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t row_base = smem_base + stage * CV_STAGE + r * 128;
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint32_t addr = row_base + (((h * 4 + u) ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(cur.v[u].x), "r"(cur.v[u].y),
                         "r"(cur.v[u].z), "r"(cur.v[u].w) : "memory");
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(full_bar(stage));
          if (++stage == CV_STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ epilogue
    const int ew = warp & 3;
    int acc = 0; uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int mb, nb; coords(tile, mb, nb);
      const int m0 = mb * CV_BM, n0 = nb * CV_BN;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) break;
      tc_fence_after();
      const int row = m0 + ew * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + acc * CV_BN;
#pragma unroll 1
      for (int c = 0; c < CV_BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(t_row + c * 32, rr);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row >= p.M || col0 >= p.Cout) continue;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (col0 + q * 8 + 8 > p.Cout) continue;
          const long long off = static_cast<long long>(row) * p.Cout + col0 + q * 8;
          float v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(rr[q * 8 + j]);
          if (p.bias) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] += __bfloat162float(p.bias[col0 + q * 8 + j]);
          }
          if (p.residual) {
            const uint4 rv = __ldg(reinterpret_cast<const uint4*>(p.residual + off));
            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[2 * j] += __uint_as_float(rw[j] << 16);
              v[2 * j + 1] += __uint_as_float(rw[j] & 0xFFFF0000u);
            }
          }
          if (p.relu) {
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = fmaxf(v[j], 0.f);
          }
          uint4 o;
          o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
          o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
          *reinterpret_cast<uint4*>(p.y + off) = o;
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
  if (warp == 2) { tc_fence_after(); tmem_dealloc(tmem_base, 2 * CV_BN); }
  if (threadIdx.x == 0 && *abort_word != 0 && p.status) atomicCAS(p.status, 0, *abort_word);
}

}  // namespace ft

using namespace ft;

// y = conv2d(x, w) (+ bias) (+ residual) (ReLU): x [N, H, W, Cin], w [Cout, KH, KW, Cin], y [N, Ho, Wo, Cout],
// all bf16 and densely packed; Ho = (H + 2*pad_h - dil*(KH-1) - 1) / stride + 1, likewise Wo.
FT_API int ft_conv2d_fprop_nhwc(const void* x, const void* w, const void* bias, const void* residual, void* y, int N,
                                int H, int W, int Cin, int Cout, int KH, int KW, int stride, int pad_h, int pad_w,
                                int dil, int relu, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && w && y, "ft_conv2d_fprop_nhwc: null pointer");
  FT_REQUIRE(N > 0 && H > 0 && W > 0 && KH > 0 && KW > 0 && stride > 0 && dil > 0 && pad_h >= 0 && pad_w >= 0,
             "ft_conv2d_fprop_nhwc: bad geometry");
  FT_REQUIRE(Cin > 0 && Cin % 64 == 0 && Cout > 0 && Cout % 8 == 0,
             "ft_conv2d_fprop_nhwc: Cin must be a multiple of 64, Cout of 8");
  FT_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(y) |
               reinterpret_cast<uintptr_t>(residual)) & 15) == 0,
             "ft_conv2d_fprop_nhwc: pointers must be 16-byte aligned");
  const long long eh = static_cast<long long>(H) + 2 * pad_h - static_cast<long long>(dil) * (KH - 1) - 1;
  const long long ew = static_cast<long long>(W) + 2 * pad_w - static_cast<long long>(dil) * (KW - 1) - 1;
  FT_REQUIRE(eh >= 0 && ew >= 0, "ft_conv2d_fprop_nhwc: the filter does not fit the padded input");
  const long long Ho = eh / stride + 1, Wo = ew / stride + 1;
  const long long M = static_cast<long long>(N) * Ho * Wo, K = static_cast<long long>(KH) * KW * Cin;
  FT_REQUIRE(M < (1ll << 31) - CV_BM && K < (1ll << 31), "ft_conv2d_fprop_nhwc: problem too large for 32-bit tile indices");
  ConvParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.N = N; p.H = H; p.W = W; p.Cin = Cin; p.Cout = Cout; p.KH = KH; p.KW = KW;
  p.Ho = static_cast<int>(Ho); p.Wo = static_cast<int>(Wo);
  p.stride = stride; p.pad_h = pad_h; p.pad_w = pad_w; p.dil = dil; p.relu = relu;
  p.M = static_cast<int>(M); p.K = static_cast<int>(K);
  CUtensorMap tmW;
  if (int rc = make_tmap_2d(&tmW, w, 2, static_cast<uint64_t>(K), static_cast<uint64_t>(Cout), static_cast<uint64_t>(K) * 2,
                            CV_BK, CV_BN, 3))
    return rc;
  p.status = device_status_word(device);
  const long long tiles = ((M + CV_BM - 1) / CV_BM) * ((Cout + CV_BN - 1) / CV_BN);
  const int grid = static_cast<int>(tiles < sm_count(device) ? tiles : sm_count(device));
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(conv2d_fprop_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CV_SMEM));
    attr_set[device] = true;
  }
  conv2d_fprop_tcgen05_kernel<<<grid, CV_THREADS, CV_SMEM, stream>>>(tmW, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}


// Host-side view of the kernel's gather indices: offsets[m * k_blocks + kb] = element offset into x
// (or -1 for padding) for every row m < M and k-block kb, computed by the functions the kernel calls.
FT_API int ft_conv2d_gather_offsets_host(long long* offsets, int N, int H, int W, int Cin, int KH, int KW, int stride,
                                         int pad_h, int pad_w, int dil) {
  FT_REQUIRE(offsets && N > 0 && H > 0 && W > 0 && Cin > 0 && Cin % 64 == 0 && KH > 0 && KW > 0 && stride > 0 && dil > 0,
             "ft_conv2d_gather_offsets_host: bad geometry");
  ConvParams p{};
  p.N = N; p.H = H; p.W = W; p.Cin = Cin; p.KH = KH; p.KW = KW; p.stride = stride; p.pad_h = pad_h; p.pad_w = pad_w; p.dil = dil;
  p.Ho = (H + 2 * pad_h - dil * (KH - 1) - 1) / stride + 1;
  p.Wo = (W + 2 * pad_w - dil * (KW - 1) - 1) / stride + 1;
  p.M = N * p.Ho * p.Wo;
  p.K = KH * KW * Cin;
  const int k_blocks = p.K / CV_BK;
  for (int m = 0; m < p.M; ++m) {
    int n, hi0, wi0;
    conv_row_origin(p, m, n, hi0, wi0);
    for (int kb = 0; kb < k_blocks; ++kb) offsets[static_cast<long long>(m) * k_blocks + kb] = conv_tap_offset(p, n, hi0, wi0, kb);
  }
  return FT_E_OK;
}
