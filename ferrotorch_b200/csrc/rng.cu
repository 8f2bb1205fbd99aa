// Device-side Philox-4x32-10: raw words, uniform, normal and dropout, on the same stream layout as
// the host generator (csrc/host/philox.cpp, utils/philox.py): counter value c (64 bit, in the low
// two counter words, the high two zero) under the 64-bit seed as key gives stream words
// 4c .. 4c+3.  Every kernel addresses the stream by (seed, first counter): element i of an output
// uses word i of the stream that starts there, so a result is reproducible from two integers and a
// dropout mask never has to be stored -- the backward pass regenerates it.
//
// The reference draws uniform / normal / dropout numbers on the device from the same generator
// (ferrotorch-gpu/src/rng.rs:830-1460; dropout mask kernel :830, uniform :998, normal :1460).
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

struct Philox4 {
  uint32_t w[4];
};

__host__ __device__ __forceinline__ Philox4 philox4x32_10(unsigned long long counter, unsigned long long key) {
  uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = 0xD2511F53ull * c0, p1 = 0xCD9E8D57ull * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0, n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1, n3 = static_cast<uint32_t>(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  Philox4 o;
  o.w[0] = c0; o.w[1] = c1; o.w[2] = c2; o.w[3] = c3;
  return o;
}

// [0, 1) on a 2^-24 grid, as the host generator's next_f32.
__host__ __device__ __forceinline__ float philox_u01(uint32_t w) {
  return static_cast<float>(w >> 8) * (1.0f / 16777216.0f);
}

enum RngKind : int { RNG_WORDS = 0, RNG_UNIFORM = 1, RNG_NORMAL = 2 };

// One thread per counter value = four consecutive outputs.  out_kind: 0 uint32 / fp32 (by kind),
// 1 bf16.  Uniform: lo + (hi - lo) * u.  Normal: Box-Muller over the word pairs (0, 1) and (2, 3)
// of a counter, r = sqrt(-2 ln u1), outputs mean + std * r * (cos, sin)(2 pi u2); a zero u1 (one
// draw in 2^24) is replaced by 2^-25 instead of being re-drawn, which would shift the stream.
__global__ void philox_fill_kernel(void* __restrict__ out, long long n, unsigned long long seed,
                                   unsigned long long counter, int kind, int out_bf16, float a, float b) {
  const long long groups = (n + 3) >> 2;
  for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const Philox4 r = philox4x32_10(counter + static_cast<unsigned long long>(g), seed);
    float v[4];
    if (kind == RNG_UNIFORM) {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = a + (b - a) * philox_u01(r.w[j]);
    } else if (kind == RNG_NORMAL) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float u1 = philox_u01(r.w[2 * h]);
        const float u2 = philox_u01(r.w[2 * h + 1]);
        if (u1 == 0.f) u1 = 1.0f / 33554432.0f;
        const float rad = sqrtf(-2.f * logf(u1));
        float sn, cs;
        sincosf(6.283185307179586f * u2, &sn, &cs);
        v[2 * h] = a + b * rad * cs;
        v[2 * h + 1] = a + b * rad * sn;
      }
    }
    const long long i0 = g << 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (i0 + j >= n) break;
      if (kind == RNG_WORDS)
        static_cast<uint32_t*>(out)[i0 + j] = r.w[j];
      else if (out_bf16)
        static_cast<__nv_bfloat16*>(out)[i0 + j] = __float2bfloat16(v[j]);
      else
        static_cast<float*>(out)[i0 + j] = v[j];
    }
  }
}

// y[i] = keep(i) ? x[i] * scale : 0 with keep(i) = u01(word i) >= p; bf16 (elt 0) or fp32 (elt 1).
// The same kernel applied to dy is the backward pass.
template <typename T>
__global__ void philox_dropout_kernel(const T* __restrict__ x, T* __restrict__ y, long long n, float p, float scale,
                                      unsigned long long seed, unsigned long long counter) {
  const long long groups = (n + 3) >> 2;
  for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const Philox4 r = philox4x32_10(counter + static_cast<unsigned long long>(g), seed);
    const long long i0 = g << 2;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (i0 + j >= n) break;
      const float xv = static_cast<float>(x[i0 + j]);
      y[i0 + j] = static_cast<T>(philox_u01(r.w[j]) >= p ? xv * scale : 0.f);
    }
  }
}

__global__ void swiglu_dropout_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y,
                                          long long rows, int F, long long ld_gu, float p, float scale,
                                          unsigned long long seed, unsigned long long counter) {
  const long long n = rows * F, groups = n >> 2;   // F % 4 == 0: a group never straddles a row
  for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const Philox4 r = philox4x32_10(counter + static_cast<unsigned long long>(g), seed);
    const long long i0 = g << 2;
    const long long row = i0 / F;
    const int f = static_cast<int>(i0 - row * F);
    const __nv_bfloat16* gp = gu + row * ld_gu + f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gv = __bfloat162float(gp[j]), uv = __bfloat162float(gp[F + j]);
      const float act = gv / (1.f + __expf(-gv)) * uv;
      y[i0 + j] = __float2bfloat16(philox_u01(r.w[j]) >= p ? act * scale : 0.f);
    }
  }
}

// d(gate|up) of the fused forward: the mask is regenerated, nothing but (seed, counter) was kept.
__global__ void swiglu_dropout_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gu,
                                          __nv_bfloat16* __restrict__ dgu, long long rows, int F, long long ld_gu,
                                          float p, float scale, unsigned long long seed, unsigned long long counter) {
  const long long n = rows * F, groups = n >> 2;
  for (long long g = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; g < groups;
       g += static_cast<long long>(gridDim.x) * blockDim.x) {
    const Philox4 r = philox4x32_10(counter + static_cast<unsigned long long>(g), seed);
    const long long i0 = g << 2;
    const long long row = i0 / F;
    const int f = static_cast<int>(i0 - row * F);
    const __nv_bfloat16* gp = gu + row * ld_gu + f;
    __nv_bfloat16* op = dgu + row * ld_gu + f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float d = philox_u01(r.w[j]) >= p ? __bfloat162float(dy[i0 + j]) * scale : 0.f;
      const float gv = __bfloat162float(gp[j]), uv = __bfloat162float(gp[F + j]);
      const float s = 1.f / (1.f + __expf(-gv));
      op[j] = __float2bfloat16(d * uv * s * (1.f + gv * (1.f - s)));
      op[F + j] = __float2bfloat16(d * gv * s);
    }
  }
}

static inline int rng_grid(long long groups, int device) {
  const long long blocks = (groups + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 16;
  return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace ft

using namespace ft;

// kind: 0 raw uint32 words, 1 uniform in [a, b), 2 normal(mean a, std b).  out: uint32 (kind 0),
// else fp32 or (out_bf16) bf16.  Uses ceil(n / 4) counter values starting at `counter`.
FT_API int ft_philox_fill(void* out, long long n, unsigned long long seed, unsigned long long counter, int kind,
                          int out_bf16, float a, float b, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(out && n >= 0 && kind >= 0 && kind <= 2, "ft_philox_fill: bad arguments");
  if (n == 0) return FT_E_OK;
  philox_fill_kernel<<<rng_grid((n + 3) >> 2, device), 256, 0, stream>>>(out, n, seed, counter, kind, out_bf16, a, b);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// y = dropout(x) with keep probability 1 - p and scale 1 / (1 - p); elt: 0 bf16, 1 fp32.  Calling it
// on the upstream gradient with the same (seed, counter) is the backward pass.
FT_API int ft_philox_dropout(const void* x, void* y, long long n, float p, unsigned long long seed,
                             unsigned long long counter, int elt, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && y && n >= 0 && p >= 0.f && p < 1.f && (elt == 0 || elt == 1), "ft_philox_dropout: bad arguments");
  if (n == 0) return FT_E_OK;
  const float scale = 1.f / (1.f - p);
  const int grid = rng_grid((n + 3) >> 2, device);
  if (elt == 0)
    philox_dropout_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x),
                                                                   static_cast<__nv_bfloat16*>(y), n, p, scale, seed, counter);
  else
    philox_dropout_kernel<float><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), static_cast<float*>(y), n, p,
                                                           scale, seed, counter);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// Fused SwiGLU + dropout.  gu: [rows, 2 F] bf16 (row stride ld_gu), y: [rows, F] bf16.  backward == 0:
// y = dropout(silu(gate) * up); backward != 0: `y` is the upstream gradient [rows, F] (read) and
// `dgu` [rows, 2 F] receives the gradient of gu.  F % 4 == 0.
FT_API int ft_swiglu_dropout(const void* gu, void* y, void* dgu, long long rows, int F, long long ld_gu, float p,
                             unsigned long long seed, unsigned long long counter, int backward, int device,
                             cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(gu && y && rows >= 0 && F > 0 && F % 4 == 0 && ld_gu >= 2ll * F && p >= 0.f && p < 1.f,
             "ft_swiglu_dropout: bad arguments");
  FT_REQUIRE(!backward || dgu, "ft_swiglu_dropout: backward needs dgu");
  if (rows == 0) return FT_E_OK;
  const float scale = 1.f / (1.f - p);
  const int grid = rng_grid(rows * F / 4, device);
  if (!backward)
    swiglu_dropout_fwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(gu),
                                                        static_cast<__nv_bfloat16*>(y), rows, F, ld_gu, p, scale, seed,
                                                        counter);
  else
    swiglu_dropout_bwd_kernel<<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(y),
                                                        static_cast<const __nv_bfloat16*>(gu),
                                                        static_cast<__nv_bfloat16*>(dgu), rows, F, ld_gu, p, scale, seed,
                                                        counter);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// The first n words of the stream at (seed, counter), computed on the host by the same function
// the kernels call (for CPU tests of the device code's arithmetic).
FT_API int ft_philox_words_host(uint32_t* out, long long n, unsigned long long seed, unsigned long long counter) {
  FT_REQUIRE(out && n >= 0, "ft_philox_words_host: bad arguments");
  for (long long g = 0; g * 4 < n; ++g) {
    const Philox4 r = philox4x32_10(counter + static_cast<unsigned long long>(g), seed);
    for (int j = 0; j < 4 && g * 4 + j < n; ++j) out[g * 4 + j] = r.w[j];
  }
  return FT_E_OK;
}
