// Max pooling forward / backward for NHWC bf16 activations (the layout every convolution and batch
// norm of this framework runs in).  The reference has forward kernels only, on NCHW f32
// (ferrotorch-gpu/src/kernels.rs:11265 max pool, :11410 avg pool) and pools backward on the host.
//
// Forward: one thread per output pixel and group of 8 channels; each filter tap is one 16-byte load,
// the running maximum lives in registers, the winning tap index (kh * KW + kw, 255 = window entirely
// in the padding) is written beside the output so that backward needs neither the input nor a
// comparison.  Backward: one thread per *input* pixel and 8 channels gathers from the (at most
// ceil(K/stride)^2) windows that cover it and adds the gradient where the stored tap is its own --
// no atomics, deterministic.  Both are streaming kernels: the bound is HBM bandwidth.
//
// The window arithmetic lives in host/device functions; a host entry point runs the same functions
// on the CPU for the tests.
#include <cuda_bf16.h>
#include <math.h>

#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

struct PoolGeom {
  int N, H, W, C, KH, KW, Ho, Wo, stride, pad_h, pad_w;
};

// Input coordinate of tap (kh, kw) of output pixel (ho, wo); false when it lies in the padding.
__host__ __device__ __forceinline__ bool pool_tap(const PoolGeom& g, int ho, int wo, int kh, int kw, int& hi, int& wi) {
  hi = ho * g.stride - g.pad_h + kh;
  wi = wo * g.stride - g.pad_w + kw;
  return hi >= 0 && hi < g.H && wi >= 0 && wi < g.W;
}

// Range [lo, hi_excl) of output positions along one axis whose window covers input position i.
__host__ __device__ __forceinline__ void pool_cover(int i, int k, int stride, int pad, int n_out, int& lo, int& hi_excl) {
  const int a = i + pad - k + 1;                 // smallest o * stride that still reaches i
  lo = a <= 0 ? 0 : (a + stride - 1) / stride;
  hi_excl = (i + pad) / stride + 1;
  if (hi_excl > n_out) hi_excl = n_out;
}

__device__ __forceinline__ void unpack8(const uint4& v, float* f) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[2 * j] = __uint_as_float(w[j] << 16);
    f[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
  }
}

__global__ void __launch_bounds__(256)
maxpool_fwd_nhwc_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, uint8_t* __restrict__ arg,
                        const PoolGeom g) {
  const int c8 = g.C / 8;
  const long long total = static_cast<long long>(g.N) * g.Ho * g.Wo * c8;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total; t += step) {
    const int cg = static_cast<int>(t % c8);
    const long long pix = t / c8;
    const int wo = static_cast<int>(pix % g.Wo), ho = static_cast<int>((pix / g.Wo) % g.Ho), n = static_cast<int>(pix / (static_cast<long long>(g.Wo) * g.Ho));
    float best[8];
    uint32_t tap[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { best[j] = -INFINITY; tap[j] = 255u; }
    for (int kh = 0; kh < g.KH; ++kh)
      for (int kw = 0; kw < g.KW; ++kw) {
        int hi, wi;
        if (!pool_tap(g, ho, wo, kh, kw, hi, wi)) continue;
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + ((static_cast<long long>(n) * g.H + hi) * g.W + wi) * g.C) + cg);
        float f[8];
        unpack8(v, f);
        const uint32_t id = static_cast<uint32_t>(kh * g.KW + kw);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (f[j] > best[j] || tap[j] == 255u || f[j] != f[j]) { best[j] = f[j]; tap[j] = id; }   // first maximum wins; NaN propagates
      }
    uint4 o;
    o.x = pack_bf16x2(best[0], best[1]); o.y = pack_bf16x2(best[2], best[3]);
    o.z = pack_bf16x2(best[4], best[5]); o.w = pack_bf16x2(best[6], best[7]);
    reinterpret_cast<uint4*>(y + pix * g.C)[cg] = o;
    uint2 a;
    a.x = tap[0] | (tap[1] << 8) | (tap[2] << 16) | (tap[3] << 24);
    a.y = tap[4] | (tap[5] << 8) | (tap[6] << 16) | (tap[7] << 24);
    reinterpret_cast<uint2*>(arg + pix * g.C)[cg] = a;
  }
}

__global__ void __launch_bounds__(256)
maxpool_bwd_nhwc_kernel(const __nv_bfloat16* __restrict__ gy, const uint8_t* __restrict__ arg, __nv_bfloat16* __restrict__ gx,
                        const PoolGeom g) {
  const int c8 = g.C / 8;
  const long long total = static_cast<long long>(g.N) * g.H * g.W * c8;
  const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < total; t += step) {
    const int cg = static_cast<int>(t % c8);
    const long long pix = t / c8;
    const int wi = static_cast<int>(pix % g.W), hi = static_cast<int>((pix / g.W) % g.H), n = static_cast<int>(pix / (static_cast<long long>(g.W) * g.H));
    int ho0, ho1, wo0, wo1;
    pool_cover(hi, g.KH, g.stride, g.pad_h, g.Ho, ho0, ho1);
    pool_cover(wi, g.KW, g.stride, g.pad_w, g.Wo, wo0, wo1);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int ho = ho0; ho < ho1; ++ho)
      for (int wo = wo0; wo < wo1; ++wo) {
        const uint32_t mine = static_cast<uint32_t>((hi - ho * g.stride + g.pad_h) * g.KW + (wi - wo * g.stride + g.pad_w));
        const long long opix = (static_cast<long long>(n) * g.Ho + ho) * g.Wo + wo;
        const uint2 a = __ldg(reinterpret_cast<const uint2*>(arg + opix * g.C) + cg);
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(gy + opix * g.C) + cg);
        float f[8];
        unpack8(v, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const uint32_t tj = ((j < 4 ? a.x : a.y) >> (8 * (j & 3))) & 0xFFu;
          if (tj == mine) acc[j] += f[j];
        }
      }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(gx + pix * g.C)[cg] = o;
  }
}

static int make_geom(PoolGeom& g, int N, int H, int W, int C, int KH, int KW, int stride, int pad_h, int pad_w) {
  FT_REQUIRE(N > 0 && H > 0 && W > 0 && C > 0 && KH > 0 && KW > 0 && stride > 0 && pad_h >= 0 && pad_w >= 0 &&
                 2 * pad_h <= KH && 2 * pad_w <= KW && KH * KW < 255,
             "max pool: bad geometry (padding at most half the window, fewer than 255 taps)");
  FT_REQUIRE(H + 2 * pad_h >= KH && W + 2 * pad_w >= KW, "max pool: the window does not fit the padded input");
  g = PoolGeom{N, H, W, C, KH, KW, (H + 2 * pad_h - KH) / stride + 1, (W + 2 * pad_w - KW) / stride + 1, stride, pad_h, pad_w};
  return FT_E_OK;
}

}  // namespace ft

using namespace ft;

// y [N, Ho, Wo, C] bf16 and arg [N, Ho, Wo, C] u8 (winning tap) from x [N, H, W, C] bf16; C % 8 == 0.
FT_API int ft_maxpool2d_fwd_nhwc(const void* x, void* y, void* arg, int N, int H, int W, int C, int KH, int KW, int stride,
                                 int pad_h, int pad_w, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && y && arg && C % 8 == 0, "ft_maxpool2d_fwd_nhwc: null pointer or C not a multiple of 8");
  FT_REQUIRE(((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) == 0 && (reinterpret_cast<uintptr_t>(arg) & 7) == 0,
             "ft_maxpool2d_fwd_nhwc: x / y must be 16-byte aligned, arg 8-byte aligned");
  PoolGeom g;
  if (int rc = make_geom(g, N, H, W, C, KH, KW, stride, pad_h, pad_w)) return rc;
  const long long total = static_cast<long long>(N) * g.Ho * g.Wo * (C / 8);
  long long grid = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 16;
  maxpool_fwd_nhwc_kernel<<<static_cast<int>(grid < cap ? grid : cap), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), static_cast<uint8_t*>(arg), g);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// gx [N, H, W, C] bf16 from gy and arg of the forward call.
FT_API int ft_maxpool2d_bwd_nhwc(const void* gy, const void* arg, void* gx, int N, int H, int W, int C, int KH, int KW,
                                 int stride, int pad_h, int pad_w, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(gy && arg && gx && C % 8 == 0, "ft_maxpool2d_bwd_nhwc: null pointer or C not a multiple of 8");
  FT_REQUIRE(((reinterpret_cast<uintptr_t>(gy) | reinterpret_cast<uintptr_t>(gx)) & 15) == 0 && (reinterpret_cast<uintptr_t>(arg) & 7) == 0,
             "ft_maxpool2d_bwd_nhwc: gy / gx must be 16-byte aligned, arg 8-byte aligned");
  PoolGeom g;
  if (int rc = make_geom(g, N, H, W, C, KH, KW, stride, pad_h, pad_w)) return rc;
  const long long total = static_cast<long long>(N) * H * W * (C / 8);
  long long grid = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 16;
  maxpool_bwd_nhwc_kernel<<<static_cast<int>(grid < cap ? grid : cap), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gy), static_cast<const uint8_t*>(arg), static_cast<__nv_bfloat16*>(gx), g);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// The same forward and backward on the host in fp32 with the kernels' window functions (NHWC floats):
// what the CPU tests compare with torch's max_pool2d and its gradient.
FT_API int ft_maxpool2d_host(const float* x, float* y, unsigned char* arg, const float* gy, float* gx, int N, int H, int W,
                             int C, int KH, int KW, int stride, int pad_h, int pad_w) {
  FT_REQUIRE(x && y && arg, "ft_maxpool2d_host: null pointer");
  PoolGeom g;
  if (int rc = make_geom(g, N, H, W, C, KH, KW, stride, pad_h, pad_w)) return rc;
  for (int n = 0; n < N; ++n)
    for (int ho = 0; ho < g.Ho; ++ho)
      for (int wo = 0; wo < g.Wo; ++wo)
        for (int c = 0; c < C; ++c) {
          float best = -INFINITY;
          unsigned tap = 255u;
          for (int kh = 0; kh < KH; ++kh)
            for (int kw = 0; kw < KW; ++kw) {
              int hi, wi;
              if (!pool_tap(g, ho, wo, kh, kw, hi, wi)) continue;
              const float f = x[((static_cast<long long>(n) * H + hi) * W + wi) * C + c];
              if (f > best || tap == 255u || f != f) { best = f; tap = static_cast<unsigned>(kh * KW + kw); }
            }
          const long long o = ((static_cast<long long>(n) * g.Ho + ho) * g.Wo + wo) * C + c;
          y[o] = best;
          arg[o] = static_cast<unsigned char>(tap);
        }
  if (!gy || !gx) return FT_E_OK;
  for (int n = 0; n < N; ++n)
    for (int hi = 0; hi < H; ++hi)
      for (int wi = 0; wi < W; ++wi) {
        int ho0, ho1, wo0, wo1;
        pool_cover(hi, KH, stride, pad_h, g.Ho, ho0, ho1);
        pool_cover(wi, KW, stride, pad_w, g.Wo, wo0, wo1);
        for (int c = 0; c < C; ++c) {
          float acc = 0.f;
          for (int ho = ho0; ho < ho1; ++ho)
            for (int wo = wo0; wo < wo1; ++wo) {
              const unsigned mine = static_cast<unsigned>((hi - ho * stride + pad_h) * KW + (wi - wo * stride + pad_w));
              const long long o = ((static_cast<long long>(n) * g.Ho + ho) * g.Wo + wo) * C + c;
              if (arg[o] == mine) acc += gy[o];
            }
          gx[((static_cast<long long>(n) * H + hi) * W + wi) * C + c] = acc;
        }
      }
  return FT_E_OK;
}
