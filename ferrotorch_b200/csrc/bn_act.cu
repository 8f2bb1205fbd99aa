// Batch normalisation for channels-last (NHWC) bf16 activations, fused with the residual add
// and the ReLU that follow it in a ResNet block, forward and backward (sm_100a).
//
// The reference runs BatchNorm2d as separate statistics / normalise kernels on NCHW f32
// (ferrotorch-gpu/src/group_norm.rs:697 forward, :1095 backward) and ReLU and the residual add as
// further elementwise launches.  Here the activation tensor [R = N*H*W, C] is read once for the
// statistics and once for  y = relu(x * scale[c] + shift[c] (+ residual)),  and the backward reads
// dy and x twice and writes dx once; the ReLU mask is recomputed from x (or taken from y when a
// residual was added), so no mask tensor is stored.
//
// All reductions are deterministic: per-block partial sums in a scratch buffer, combined in
// double precision and in a fixed order by a small finalize kernel, which also adds dgamma /
// dbeta straight into the trainer's gradient arena when there is one.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int BN_THREADS = 256;
constexpr int BN_MAX_C = 2048;      // 8 channels per thread, one row per BN_THREADS / (C / 8) threads
constexpr int BN_MAX_BLOCKS = 1024;

__device__ __forceinline__ void bn_unpack8(const uint4& u, float* f) {
  const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 bn_pack8(const float* f) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  return o;
}
__device__ __forceinline__ void bn_load8f(const float* p, float* f) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p) + 1);
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

// Column sums of two per-element quantities over the rows of a [R, C] tensor.
//   MODE 0 (forward):  q0 = x,   q1 = x * x          (4 rows per thread in flight)
//   MODE 1 (backward): q0 = dz,  q1 = dz * x         with dz = dy * mask (2 rows in flight);
//                      the finalize kernel turns them into dbeta and dgamma = invstd * (q1 - mean * q0)
// Thread layout: tc = C / 8 threads across the channels, BN_THREADS / tc rows per pass.
// partial: [gridDim.x, 2, C] floats.
template <int MODE>
__global__ void __launch_bounds__(BN_THREADS)
bn_colsum_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                 const __nv_bfloat16* __restrict__ y, const float* __restrict__ scale,
                 const float* __restrict__ shift, int relu, long long R, int C, float* __restrict__ partial) {
  constexpr int U = MODE == 0 ? 4 : 2;
  __shared__ float red[2][BN_THREADS][9];   // padded: 8 values per thread
  const int tc = C >> 3;
  const int rows_per_pass = BN_THREADS / tc;
  const int rg = threadIdx.x / tc, cv = threadIdx.x - rg * tc;
  const bool active = rg < rows_per_pass;
  const bool recompute_mask = MODE == 1 && relu && !y;
  float s0[8], s1[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s0[j] = s1[j] = 0.f;
  float sc[8], sh[8];
  if (recompute_mask && active) {
    bn_load8f(scale + cv * 8, sc);
    bn_load8f(shift + cv * 8, sh);
  }
  if (active) {
    const long long stride = static_cast<long long>(gridDim.x) * rows_per_pass;
    for (long long r0 = static_cast<long long>(blockIdx.x) * rows_per_pass + rg; r0 < R; r0 += U * stride) {
      uint4 xq[U], dq[U], yq[U];
      bool ok[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long long r = r0 + u * stride;
        ok[u] = r < R;
        const long long o = (ok[u] ? r : r0) * C + cv * 8;
        xq[u] = __ldcs(reinterpret_cast<const uint4*>(x + o));
        if (MODE == 1) {
          dq[u] = __ldcs(reinterpret_cast<const uint4*>(dy + o));
          if (relu && y) yq[u] = __ldcs(reinterpret_cast<const uint4*>(y + o));
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (!ok[u]) continue;
        float xv[8];
        bn_unpack8(xq[u], xv);
        if (MODE == 0) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            s0[j] += xv[j];
            s1[j] = __fmaf_rn(xv[j], xv[j], s1[j]);
          }
        } else {
          float dv[8], yv[8];
          bn_unpack8(dq[u], dv);
          if (relu && y) bn_unpack8(yq[u], yv);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            bool on = true;
            if (relu) on = y ? (yv[j] > 0.f) : (__fmaf_rn(xv[j], sc[j], sh[j]) > 0.f);
            const float dz = on ? dv[j] : 0.f;
            s0[j] += dz;
            s1[j] = __fmaf_rn(dz, xv[j], s1[j]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[0][threadIdx.x][j] = s0[j];
    red[1][threadIdx.x][j] = s1[j];
  }
  __syncthreads();
  // the first tc threads add up the row groups of their channel vector (fixed order)
  if (threadIdx.x < tc) {
    float a0[8], a1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a0[j] = a1[j] = 0.f;
    for (int g = 0; g < rows_per_pass; ++g) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        a0[j] += red[0][g * tc + threadIdx.x][j];
        a1[j] += red[1][g * tc + threadIdx.x][j];
      }
    }
    float* p0 = partial + (static_cast<size_t>(blockIdx.x) * 2) * C + threadIdx.x * 8;
    float* p1 = p0 + C;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      p0[j] = a0[j];
      p1[j] = a1[j];
    }
  }
}

// Sum the per-block partials of 32 channels: blockDim = (32 channels, BN_FIN_GROUPS); group g adds
// the partials b = g, g + G, ... in double, then the groups are combined in a fixed order.
// Returns the two totals to the threads with threadIdx.y == 0.
constexpr int BN_FIN_GROUPS = 32;
__device__ __forceinline__ void bn_reduce_partials(const float* __restrict__ partial, int blocks, int C, int c,
                                                   double& s, double& q) {
  __shared__ double red[2][BN_FIN_GROUPS][33];
  double a0 = 0.0, a1 = 0.0;
  if (c < C) {
    for (int b = threadIdx.y; b < blocks; b += BN_FIN_GROUPS) {
      a0 += partial[(static_cast<size_t>(b) * 2) * C + c];
      a1 += partial[(static_cast<size_t>(b) * 2 + 1) * C + c];
    }
  }
  red[0][threadIdx.y][threadIdx.x] = a0;
  red[1][threadIdx.y][threadIdx.x] = a1;
  __syncthreads();
  s = q = 0.0;
  if (threadIdx.y == 0) {
    for (int g = 0; g < BN_FIN_GROUPS; ++g) {
      s += red[0][g][threadIdx.x];
      q += red[1][g][threadIdx.x];
    }
  }
}

// Forward finalize.  Writes mean, invstd (kept for the backward), scale = gamma * invstd,
// shift = beta - mean * scale, and updates the running statistics (unbiased variance) when given.
__global__ void __launch_bounds__(32 * BN_FIN_GROUPS)
bn_fwd_finalize_kernel(const float* __restrict__ partial, int blocks, long long R, int C,
                       const void* gamma, const void* beta, int affine_f32, void* running_mean,
                       void* running_var, int running_f32, float momentum, float eps,
                       float* __restrict__ mean, float* __restrict__ invstd,
                       float* __restrict__ scale, float* __restrict__ shift) {
  const int c = blockIdx.x * 32 + threadIdx.x;
  double s, q;
  bn_reduce_partials(partial, blocks, C, c, s, q);
  if (threadIdx.y != 0 || c >= C) return;
  const double m = s / static_cast<double>(R);
  double var = q / static_cast<double>(R) - m * m;
  if (var < 0.0) var = 0.0;
  const float is = rsqrtf(static_cast<float>(var) + eps);
  const float g = gamma ? (affine_f32 ? static_cast<const float*>(gamma)[c]
                                      : __bfloat162float(static_cast<const __nv_bfloat16*>(gamma)[c])) : 1.f;
  const float bb = beta ? (affine_f32 ? static_cast<const float*>(beta)[c]
                                      : __bfloat162float(static_cast<const __nv_bfloat16*>(beta)[c])) : 0.f;
  mean[c] = static_cast<float>(m);
  invstd[c] = is;
  const float sc = g * is;
  scale[c] = sc;
  shift[c] = __fmaf_rn(-static_cast<float>(m), sc, bb);
  if (running_mean && running_var) {
    const float unbiased = static_cast<float>(R > 1 ? var * static_cast<double>(R) / static_cast<double>(R - 1) : var);
    if (running_f32) {
      float* rm = static_cast<float*>(running_mean);
      float* rv = static_cast<float*>(running_var);
      rm[c] = (1.f - momentum) * rm[c] + momentum * static_cast<float>(m);
      rv[c] = (1.f - momentum) * rv[c] + momentum * unbiased;
    } else {
      __nv_bfloat16* rm = static_cast<__nv_bfloat16*>(running_mean);
      __nv_bfloat16* rv = static_cast<__nv_bfloat16*>(running_var);
      rm[c] = __float2bfloat16((1.f - momentum) * __bfloat162float(rm[c]) + momentum * static_cast<float>(m));
      rv[c] = __float2bfloat16((1.f - momentum) * __bfloat162float(rv[c]) + momentum * unbiased);
    }
  }
}

// y = act(x * scale[c] + shift[c] (+ residual)), 8 channels per thread, two vectors in flight.
// When BN_THREADS is a multiple of tc = C / 8 (every power-of-two C up to 2048) a thread always
// meets the same 8 channels, so their scale / shift are loaded once instead of per vector.
__global__ void __launch_bounds__(BN_THREADS)
bn_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ residual,
                const float* __restrict__ scale, const float* __restrict__ shift, __nv_bfloat16* __restrict__ y,
                int relu, long long total_vec, int tc) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool fixed = (BN_THREADS % tc) == 0;
  float sc[8], sh[8];
  if (fixed) {
    const int cv = threadIdx.x % tc;
    bn_load8f(scale + cv * 8, sc);
    bn_load8f(shift + cv * 8, sh);
  }
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total_vec; i0 += 2 * stride) {
    const long long i1 = i0 + stride < total_vec ? i0 + stride : i0;
    const uint4 xa = __ldcs(reinterpret_cast<const uint4*>(x) + i0), xb = __ldcs(reinterpret_cast<const uint4*>(x) + i1);
    uint4 ra, rb;
    if (residual) {
      ra = __ldcs(reinterpret_cast<const uint4*>(residual) + i0);
      rb = __ldcs(reinterpret_cast<const uint4*>(residual) + i1);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (k == 1 && i1 == i0) break;
      const long long i = k == 0 ? i0 : i1;
      if (!fixed) {
        const int cv = static_cast<int>(i % tc);
        bn_load8f(scale + cv * 8, sc);
        bn_load8f(shift + cv * 8, sh);
      }
      float xv[8], o[8];
      bn_unpack8(k == 0 ? xa : xb, xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __fmaf_rn(xv[j], sc[j], sh[j]);
      if (residual) {
        float rv[8];
        bn_unpack8(k == 0 ? ra : rb, rv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += rv[j];
      }
      if (relu) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = fmaxf(o[j], 0.f);
      }
      reinterpret_cast<uint4*>(y)[i] = bn_pack8(o);
    }
  }
}

// Backward finalize: dgamma, dbeta and the per-channel coefficients of
//   dx = gamma * invstd * (dz - dbeta / R - xhat * dgamma / R) = A * dz + B * x + D
// with A = gamma * invstd, B = -A * invstd * dgamma / R, D = -A * dbeta / R - B * mean.
// grad_kind 0: dgamma / dbeta are stored as fp32; 1: added to bf16 accumulators; 2: added to
// fp32 accumulators (the gradient arena of the flat-parameter trainer).
__global__ void __launch_bounds__(32 * BN_FIN_GROUPS)
bn_bwd_finalize_kernel(const float* __restrict__ partial, int blocks, long long R, int C,
                       const float* __restrict__ mean, const float* __restrict__ invstd,
                       const float* __restrict__ scale, void* dgamma, void* dbeta, int grad_kind,
                       float* __restrict__ coef) {
  const int c = blockIdx.x * 32 + threadIdx.x;
  double db, q1;
  bn_reduce_partials(partial, blocks, C, c, db, q1);
  if (threadIdx.y != 0 || c >= C) return;
  const double dg = static_cast<double>(invstd[c]) * (q1 - static_cast<double>(mean[c]) * db);
  if (grad_kind == 1) {
    __nv_bfloat16* g = static_cast<__nv_bfloat16*>(dgamma);
    __nv_bfloat16* b = static_cast<__nv_bfloat16*>(dbeta);
    if (g) g[c] = __float2bfloat16(__bfloat162float(g[c]) + static_cast<float>(dg));
    if (b) b[c] = __float2bfloat16(__bfloat162float(b[c]) + static_cast<float>(db));
  } else if (grad_kind == 2) {
    if (dgamma) static_cast<float*>(dgamma)[c] += static_cast<float>(dg);
    if (dbeta) static_cast<float*>(dbeta)[c] += static_cast<float>(db);
  } else {
    if (dgamma) static_cast<float*>(dgamma)[c] = static_cast<float>(dg);
    if (dbeta) static_cast<float*>(dbeta)[c] = static_cast<float>(db);
  }
  const double A = scale[c];
  const double B = -A * static_cast<double>(invstd[c]) * dg / static_cast<double>(R);
  coef[c] = static_cast<float>(A);
  coef[C + c] = static_cast<float>(B);
  coef[2 * C + c] = static_cast<float>(-A * db / static_cast<double>(R) - B * static_cast<double>(mean[c]));
}

// dx = A * dz + B * x + D; with a residual branch dres = dz.  Per-channel values are loaded once
// per thread when BN_THREADS is a multiple of tc (see bn_apply_kernel).
__global__ void __launch_bounds__(BN_THREADS)
bn_bwd_apply_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                    const __nv_bfloat16* __restrict__ y, const float* __restrict__ scale,
                    const float* __restrict__ shift, const float* __restrict__ coef, int relu,
                    __nv_bfloat16* __restrict__ dx, __nv_bfloat16* __restrict__ dres, long long total_vec,
                    int tc, int C) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const bool fixed = (BN_THREADS % tc) == 0;
  const bool recompute_mask = relu && !y;
  float cA[8], cB[8], cD[8], sc[8], sh[8];
  auto load_coefs = [&](int cv) {
    bn_load8f(coef + cv * 8, cA);
    bn_load8f(coef + C + cv * 8, cB);
    bn_load8f(coef + 2 * C + cv * 8, cD);
    if (recompute_mask) {
      bn_load8f(scale + cv * 8, sc);
      bn_load8f(shift + cv * 8, sh);
    }
  };
  if (fixed) load_coefs(threadIdx.x % tc);
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total_vec; i0 += 2 * stride) {
    const long long i1 = i0 + stride < total_vec ? i0 + stride : i0;
    const uint4 xa = __ldcs(reinterpret_cast<const uint4*>(x) + i0), xb = __ldcs(reinterpret_cast<const uint4*>(x) + i1);
    const uint4 da = __ldcs(reinterpret_cast<const uint4*>(dy) + i0), db = __ldcs(reinterpret_cast<const uint4*>(dy) + i1);
    uint4 ya, yb;
    if (relu && y) {
      ya = __ldcs(reinterpret_cast<const uint4*>(y) + i0);
      yb = __ldcs(reinterpret_cast<const uint4*>(y) + i1);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (k == 1 && i1 == i0) break;
      const long long i = k == 0 ? i0 : i1;
      if (!fixed) load_coefs(static_cast<int>(i % tc));
      float xv[8], dv[8], yv[8], o[8], dz[8];
      bn_unpack8(k == 0 ? xa : xb, xv);
      bn_unpack8(k == 0 ? da : db, dv);
      if (relu && y) bn_unpack8(k == 0 ? ya : yb, yv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        bool on = true;
        if (relu) on = y ? (yv[j] > 0.f) : (__fmaf_rn(xv[j], sc[j], sh[j]) > 0.f);
        dz[j] = on ? dv[j] : 0.f;
        o[j] = __fmaf_rn(cA[j], dz[j], __fmaf_rn(cB[j], xv[j], cD[j]));
      }
      reinterpret_cast<uint4*>(dx)[i] = bn_pack8(o);
      if (dres) reinterpret_cast<uint4*>(dres)[i] = bn_pack8(dz);
    }
  }
}

static int bn_blocks(long long R, int C, int device) {
  const int rows_per_pass = BN_THREADS / (C >> 3);
  long long b = (R + 2LL * rows_per_pass - 1) / (2LL * rows_per_pass);
  long long cap = static_cast<long long>(sm_count(device)) * 4;
  if (cap > BN_MAX_BLOCKS) cap = BN_MAX_BLOCKS;
  if (b > cap) b = cap;
  return b < 1 ? 1 : static_cast<int>(b);
}
static int bn_elem_blocks(long long total_vec, int device) {
  long long b = (total_vec + 2LL * BN_THREADS - 1) / (2LL * BN_THREADS);
  const long long cap = static_cast<long long>(sm_count(device)) * 8;
  if (b > cap) b = cap;
  return b < 1 ? 1 : static_cast<int>(b);
}

}  // namespace ft

using namespace ft;

// Floats of scratch the forward / backward need for the per-block partial sums.
FT_API long long ft_bn_scratch_floats(int C) { return 2LL * BN_MAX_BLOCKS * C; }

// Training forward.  x, y (and residual): [R, C] bf16, C a multiple of 8, at most 2048.
// gamma / beta: [C] bf16 or fp32 (affine_f32) or null.  running_*: [C] bf16 or fp32 or null.
// stats: 4 * C floats out = mean | invstd | scale | shift (kept for the backward).
FT_API int ft_bn_act_fwd(const void* x, const void* residual, void* y, const void* gamma, const void* beta,
                         int affine_f32, void* running_mean, void* running_var, int running_f32, float momentum,
                         float eps, int relu, long long R, int C, float* stats, float* scratch, int device,
                         cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && y && stats && scratch, "ft_bn_act_fwd: null pointer");
  FT_REQUIRE(R > 0 && C >= 8 && C % 8 == 0 && C <= BN_MAX_C, "ft_bn_act_fwd: C must be a multiple of 8 in [8, 2048]");
  const int blocks = bn_blocks(R, C, device);
  bn_colsum_kernel<0><<<blocks, BN_THREADS, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), nullptr, nullptr,
                                                         nullptr, nullptr, 0, R, C, scratch);
  FT_CUDA_CHECK(cudaGetLastError());
  bn_fwd_finalize_kernel<<<(C + 31) / 32, dim3(32, BN_FIN_GROUPS), 0, stream>>>(scratch, blocks, R, C, gamma, beta, affine_f32,
                                                              running_mean, running_var, running_f32, momentum, eps,
                                                              stats, stats + C, stats + 2 * C, stats + 3 * C);
  FT_CUDA_CHECK(cudaGetLastError());
  const long long total_vec = R * (C >> 3);
  bn_apply_kernel<<<bn_elem_blocks(total_vec, device), BN_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual), stats + 2 * C, stats + 3 * C,
      static_cast<__nv_bfloat16*>(y), relu, total_vec, C >> 3);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch(3);
  return FT_E_OK;
}

// Inference / frozen statistics: y = act(x * scale + shift (+ residual)) with caller-made
// scale | shift (2 * C floats).
FT_API int ft_bn_act_apply(const void* x, const void* residual, void* y, const float* scale_shift, int relu,
                           long long R, int C, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && y && scale_shift, "ft_bn_act_apply: null pointer");
  FT_REQUIRE(R > 0 && C >= 8 && C % 8 == 0, "ft_bn_act_apply: C must be a multiple of 8");
  const long long total_vec = R * (C >> 3);
  bn_apply_kernel<<<bn_elem_blocks(total_vec, device), BN_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(residual), scale_shift, scale_shift + C,
      static_cast<__nv_bfloat16*>(y), relu, total_vec, C >> 3);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// Training backward.  y is the forward output, needed only when a residual was added before
// the ReLU (else pass null and the mask is recomputed from x).  dres (optional): gradient of the
// residual branch.  dgamma / dbeta (each optional): [C]; grad_kind 0 = fp32 store, 1 = bf16
// accumulate, 2 = fp32 accumulate.  coef: 3 * C floats of scratch.
FT_API int ft_bn_act_bwd(const void* x, const void* dy, const void* y, const float* stats, int relu, long long R,
                         int C, void* dx, void* dres, void* dgamma, void* dbeta, int grad_kind, float* coef,
                         float* scratch, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && dy && stats && dx && coef && scratch, "ft_bn_act_bwd: null pointer");
  FT_REQUIRE(grad_kind >= 0 && grad_kind <= 2, "ft_bn_act_bwd: bad grad_kind");
  FT_REQUIRE(R > 0 && C >= 8 && C % 8 == 0 && C <= BN_MAX_C, "ft_bn_act_bwd: C must be a multiple of 8 in [8, 2048]");
  const float *mean = stats, *invstd = stats + C, *scale = stats + 2 * C, *shift = stats + 3 * C;
  const int blocks = bn_blocks(R, C, device);
  bn_colsum_kernel<1><<<blocks, BN_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
      static_cast<const __nv_bfloat16*>(y), scale, shift, relu, R, C, scratch);
  FT_CUDA_CHECK(cudaGetLastError());
  bn_bwd_finalize_kernel<<<(C + 31) / 32, dim3(32, BN_FIN_GROUPS), 0, stream>>>(scratch, blocks, R, C, mean, invstd,
                                                                                  scale, dgamma, dbeta, grad_kind, coef);
  FT_CUDA_CHECK(cudaGetLastError());
  const long long total_vec = R * (C >> 3);
  bn_bwd_apply_kernel<<<bn_elem_blocks(total_vec, device), BN_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dy),
      static_cast<const __nv_bfloat16*>(y), scale, shift, coef, relu,
      static_cast<__nv_bfloat16*>(dx), static_cast<__nv_bfloat16*>(dres), total_vec, C >> 3, C);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch(3);
  return FT_E_OK;
}
