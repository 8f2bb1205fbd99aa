// Layout kernels around the shifted-row convolution GEMMs (gemm_tcgen05.cu, MODE 1 / 2) for NHWC
// bf16 activations:
//   * embed: copy [N, H, W, C] into a zeroed [N, Hp, Wp, C] grid at offset (oh, ow), optionally
//     splitting the padded image into its four stride-2 parity planes (the layout in which a
//     stride-2 filter tap is again a constant row shift);
//   * crop:  the inverse for a GEMM output -- take [N, Ho, Wo, C] out of the padded grid;
//   * im2col for filters whose channel count is not a multiple of 64 (the 3-channel stem of a
//     ResNet): rows of [KH*KW*C] patches, zero-padded to a row length that TMA can address.
// The reference writes an im2col buffer for every convolution (ferrotorch-gpu/src/conv.rs:239-520);
// here only the stem does.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

// One thread per 16-byte vector (8 channels) of the destination grid.
// planes == 1: dst[n, i, j, :] = src[n, i - oh, j - ow, :] (zero outside).
// planes == 4: dst[(a, b), n, i, j, :] = padded[n, 2 i + a, 2 j + b, :], padded as above
//              (Hp, Wp are then the plane extents, i.e. half the padded image).
__global__ void conv_embed_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int N, int H, int W,
                                  int Cv, int Hp, int Wp, int oh, int ow, int planes) {
  const long long total = static_cast<long long>(planes) * N * Hp * Wp * Cv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % Cv);
    long long r = i / Cv;
    const int j = static_cast<int>(r % Wp); r /= Wp;
    const int ii = static_cast<int>(r % Hp); r /= Hp;
    const int n = static_cast<int>(r % N);
    const int pl = static_cast<int>(r / N);
    int hi, wi;
    if (planes == 4) {
      hi = 2 * ii + (pl >> 1) - oh;
      wi = 2 * j + (pl & 1) - ow;
    } else {
      hi = ii - oh;
      wi = j - ow;
    }
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (hi >= 0 && hi < H && wi >= 0 && wi < W)
      v = __ldg(src + ((static_cast<long long>(n) * H + hi) * W + wi) * Cv + c);
    dst[i] = v;
  }
}

// dst[n, i, j, :] = src[n, i + oh, j + ow, :] for a [N, Hp, Wp, C] source grid (bf16 or fp32,
// moved as 16-byte vectors).
__global__ void conv_crop_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int N, int Ho, int Wo,
                                 int Cv, int Hp, int Wp, int oh, int ow) {
  const long long total = static_cast<long long>(N) * Ho * Wo * Cv;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int c = static_cast<int>(i % Cv);
    long long r = i / Cv;
    const int j = static_cast<int>(r % Wo); r /= Wo;
    const int ii = static_cast<int>(r % Ho);
    const int n = static_cast<int>(r / Ho);
    dst[i] = __ldg(src + ((static_cast<long long>(n) * Hp + ii + oh) * Wp + j + ow) * Cv + c);
  }
}

// out[m, (kh * KW + kw) * C + c] = x[n, ho * s - ph + kh * d, wo * s - pw + kw * d, c]; columns
// [KH*KW*C, Kpad) are zero.  One thread per (row, tap).
__global__ void im2col_nhwc_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int N, int H,
                                   int W, int C, int KH, int KW, int stride, int ph, int pw, int dil, int Ho, int Wo,
                                   int Kpad) {
  const int taps = KH * KW;
  const long long total = static_cast<long long>(N) * Ho * Wo * (taps + 1);
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int tap = static_cast<int>(i % (taps + 1));
    const long long m = i / (taps + 1);
    __nv_bfloat16* row = out + m * Kpad;
    if (tap == taps) {  // the zero tail of the row
      for (int k = taps * C; k < Kpad; ++k) row[k] = __float2bfloat16(0.f);
      continue;
    }
    const int wo = static_cast<int>(m % Wo), ho = static_cast<int>((m / Wo) % Ho);
    const int n = static_cast<int>(m / (static_cast<long long>(Wo) * Ho));
    const int kh = tap / KW, kw = tap - kh * KW;
    const int hi = ho * stride - ph + kh * dil, wi = wo * stride - pw + kw * dil;
    const bool in = hi >= 0 && hi < H && wi >= 0 && wi < W;
    const __nv_bfloat16* src = x + ((static_cast<long long>(n) * H + hi) * W + wi) * C;
    if ((C & 3) == 0) {
      // 8-byte vectors: a pixel of C channels and its slot in the row are both 8-byte aligned
      const uint2* s2 = reinterpret_cast<const uint2*>(src);
      uint2* d2 = reinterpret_cast<uint2*>(row + tap * C);
      for (int c = 0; c < (C >> 2); ++c) d2[c] = in ? __ldg(s2 + c) : make_uint2(0u, 0u);
    } else {
      for (int c = 0; c < C; ++c) row[tap * C + c] = in ? src[c] : __float2bfloat16(0.f);
    }
  }
}

static inline int layout_grid(long long work, int device) {
  const long long blocks = (work + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 16;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace ft

using namespace ft;

// src [N, H, W, C] -> dst [planes, N, Hp, Wp, C] (planes 1 or 4), see conv_embed_kernel.
// elt_bytes: 2 (bf16) or 4 (fp32); C * elt_bytes must be a multiple of 16.
FT_API int ft_conv_embed(const void* src, void* dst, int N, int H, int W, int C, int Hp, int Wp, int oh, int ow,
                         int planes, int elt_bytes, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(src && dst, "ft_conv_embed: null pointer");
  FT_REQUIRE(N > 0 && H > 0 && W > 0 && C > 0 && Hp > 0 && Wp > 0 && (planes == 1 || planes == 4),
             "ft_conv_embed: bad geometry");
  FT_REQUIRE((elt_bytes == 2 || elt_bytes == 4) && (C * elt_bytes) % 16 == 0,
             "ft_conv_embed: a pixel (%d channels x %d bytes) must be a multiple of 16 bytes", C, elt_bytes);
  FT_REQUIRE(((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0,
             "ft_conv_embed: pointers must be 16-byte aligned");
  const int Cv = C * elt_bytes / 16;
  const long long total = static_cast<long long>(planes) * N * Hp * Wp * Cv;
  conv_embed_kernel<<<layout_grid(total, device), 256, 0, stream>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), N, H, W, Cv, Hp, Wp, oh, ow, planes);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// src [N, Hp, Wp, C] -> dst [N, Ho, Wo, C]: dst[n, i, j] = src[n, i + oh, j + ow].
FT_API int ft_conv_crop(const void* src, void* dst, int N, int Ho, int Wo, int C, int Hp, int Wp, int oh, int ow,
                        int elt_bytes, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(src && dst, "ft_conv_crop: null pointer");
  FT_REQUIRE(N > 0 && Ho > 0 && Wo > 0 && C > 0 && oh >= 0 && ow >= 0 && Ho + oh <= Hp && Wo + ow <= Wp,
             "ft_conv_crop: the window does not fit the source grid");
  FT_REQUIRE((elt_bytes == 2 || elt_bytes == 4) && (C * elt_bytes) % 16 == 0,
             "ft_conv_crop: a pixel (%d channels x %d bytes) must be a multiple of 16 bytes", C, elt_bytes);
  FT_REQUIRE(((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0,
             "ft_conv_crop: pointers must be 16-byte aligned");
  const int Cv = C * elt_bytes / 16;
  const long long total = static_cast<long long>(N) * Ho * Wo * Cv;
  conv_crop_kernel<<<layout_grid(total, device), 256, 0, stream>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), N, Ho, Wo, Cv, Hp, Wp, oh, ow);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// x [N, H, W, C] bf16 -> out [N*Ho*Wo, Kpad] bf16 patches (Kpad >= KH*KW*C, Kpad % 8 == 0).
FT_API int ft_im2col_nhwc(const void* x, void* out, int N, int H, int W, int C, int KH, int KW, int stride,
                          int ph, int pw, int dil, int Kpad, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && out, "ft_im2col_nhwc: null pointer");
  FT_REQUIRE(N > 0 && H > 0 && W > 0 && C > 0 && KH > 0 && KW > 0 && stride > 0 && dil > 0 && ph >= 0 && pw >= 0,
             "ft_im2col_nhwc: bad geometry");
  const int eh = H + 2 * ph - dil * (KH - 1) - 1, ew = W + 2 * pw - dil * (KW - 1) - 1;
  FT_REQUIRE(eh >= 0 && ew >= 0, "ft_im2col_nhwc: the filter does not fit the padded input");
  FT_REQUIRE(Kpad >= KH * KW * C && Kpad % 8 == 0, "ft_im2col_nhwc: Kpad=%d too small or not a multiple of 8", Kpad);
  const int Ho = eh / stride + 1, Wo = ew / stride + 1;
  const long long total = static_cast<long long>(N) * Ho * Wo * (KH * KW + 1);
  im2col_nhwc_kernel<<<layout_grid(total, device), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(out), N, H, W, C, KH, KW, stride, ph, pw,
      dil, Ho, Wo, Kpad);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}
