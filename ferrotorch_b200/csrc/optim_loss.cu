// Flat-buffer optimizer and loss kernels for sm_100a.
//
//   * multi-tensor AdamW / SGD over flat parameter arenas: one launch updates every
//     element of a parameter group (fp32 master weights + moments, bf16 gradients in,
//     bf16 working weights out).  The reference runs ~17 elementwise launches per
//     parameter per step (ferrotorch-optim/src/adamw.rs:239-384) or one fused launch
//     per parameter (adam.rs:545 -> ferrotorch-gpu/src/kernels.rs:15962).  Update
//     rule = decoupled decay p*(1-lr*wd) - lr*m_hat/(sqrt(v_hat)+eps)
//     (adamw.rs:296-334); SGD = sgd.rs:224-330 (wd folded into the gradient,
//     dampening, nesterov).
//   * global gradient L2 norm + clip coefficient kept on the device, so the clip
//     (ferrotorch-nn/src/utils.rs:148-240) costs no host synchronisation: the
//     optimizer kernel multiplies by *grad_scale.
//   * fused softmax cross-entropy forward+backward over bf16 logits, in place
//     (the reference computes CrossEntropyLoss on the host, ferrotorch-nn/src/loss.rs:195-305).
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

struct AdamWArgs {
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2;  // bc = 1 - beta^t
  int adam_l2;  // 1: classic Adam (decay folded into the gradient) instead of decoupled
};

__device__ __forceinline__ void load_grad4(const void* g, int grad_f32, long long i4, float* out) {
  if (grad_f32) {
    const float4 v = reinterpret_cast<const float4*>(g)[i4];
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else {
    const uint2 v = reinterpret_cast<const uint2*>(g)[i4];
    const float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
    out[0] = a.x; out[1] = a.y; out[2] = b.x; out[3] = b.y;
  }
}

// n % 4 == 0 (arenas are padded).  p_lp may be null (fp32-only training).
__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                  const void* __restrict__ grad, __nv_bfloat16* __restrict__ p_lp, long long n,
                  int grad_f32, const float* __restrict__ grad_scale, AdamWArgs a) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[4];
    load_grad4(grad, grad_f32, i, g);
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i];
    float4 v4 = reinterpret_cast<float4*>(v)[i];
    float p[4] = {p4.x, p4.y, p4.z, p4.w};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w};
    float vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = g[j] * gs;
      if (a.adam_l2) gj += a.weight_decay * p[j];
      else p[j] *= (1.f - a.lr * a.weight_decay);
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      const float mhat = mm[j] / a.bc1;
      const float vhat = vv[j] / a.bc2;
      p[j] -= a.lr * mhat / (sqrtf(vhat) + a.eps);
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    if (p_lp) {
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
      reinterpret_cast<uint2*>(p_lp)[i] = o;
    }
  }
}

// Eight elements per thread, all seven 16-byte loads issued before the first use, streaming
// (evict-first) cache hints: the optimizer state is touched once per step and never fits in L2.
__global__ void __launch_bounds__(256)
adamw_flat8_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                   const void* __restrict__ grad, __nv_bfloat16* __restrict__ p_lp, long long n,
                   int grad_f32, const float* __restrict__ grad_scale, AdamWArgs a) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long n8 = n >> 3;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n8;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[8];
    if (grad_f32) {
      const float4 g0 = __ldcs(reinterpret_cast<const float4*>(grad) + 2 * i);
      const float4 g1 = __ldcs(reinterpret_cast<const float4*>(grad) + 2 * i + 1);
      g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
    } else {
      const uint4 gb = __ldcs(reinterpret_cast<const uint4*>(grad) + i);
      const float2 a0 = unpack_bf16x2(gb.x), a1 = unpack_bf16x2(gb.y), a2 = unpack_bf16x2(gb.z), a3 = unpack_bf16x2(gb.w);
      g[0] = a0.x; g[1] = a0.y; g[2] = a1.x; g[3] = a1.y; g[4] = a2.x; g[5] = a2.y; g[6] = a3.x; g[7] = a3.y;
    }
    float4* pm = reinterpret_cast<float4*>(master) + 2 * i;
    float4* pmm = reinterpret_cast<float4*>(m) + 2 * i;
    float4* pv = reinterpret_cast<float4*>(v) + 2 * i;
    const float4 p0 = __ldcs(pm), p1 = __ldcs(pm + 1);
    const float4 m0 = __ldcs(pmm), m1 = __ldcs(pmm + 1);
    const float4 v0 = __ldcs(pv), v1 = __ldcs(pv + 1);
    float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    float mm[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float gj = g[j] * gs;
      if (a.adam_l2) gj += a.weight_decay * p[j];
      else p[j] *= (1.f - a.lr * a.weight_decay);
      mm[j] = a.beta1 * mm[j] + (1.f - a.beta1) * gj;
      vv[j] = a.beta2 * vv[j] + (1.f - a.beta2) * gj * gj;
      const float mhat = mm[j] / a.bc1;
      const float vhat = vv[j] / a.bc2;
      p[j] -= a.lr * mhat / (sqrtf(vhat) + a.eps);
    }
    __stcs(pm, make_float4(p[0], p[1], p[2], p[3]));
    __stcs(pm + 1, make_float4(p[4], p[5], p[6], p[7]));
    __stcs(pmm, make_float4(mm[0], mm[1], mm[2], mm[3]));
    __stcs(pmm + 1, make_float4(mm[4], mm[5], mm[6], mm[7]));
    __stcs(pv, make_float4(vv[0], vv[1], vv[2], vv[3]));
    __stcs(pv + 1, make_float4(vv[4], vv[5], vv[6], vv[7]));
    if (p_lp) {
      uint4 o;
      o.x = pack_bf16x2(p[0], p[1]); o.y = pack_bf16x2(p[2], p[3]);
      o.z = pack_bf16x2(p[4], p[5]); o.w = pack_bf16x2(p[6], p[7]);
      reinterpret_cast<uint4*>(p_lp)[i] = o;
    }
  }
}

struct SgdArgs {
  float lr, momentum, dampening, weight_decay;
  int nesterov, first_step;
};

__global__ void __launch_bounds__(256)
sgd_flat_kernel(float* __restrict__ master, float* __restrict__ mom, const void* __restrict__ grad,
                __nv_bfloat16* __restrict__ p_lp, long long n, int grad_f32,
                const float* __restrict__ grad_scale, SgdArgs a) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[4];
    load_grad4(grad, grad_f32, i, g);
    float4 p4 = reinterpret_cast<float4*>(master)[i];
    float p[4] = {p4.x, p4.y, p4.z, p4.w};
    float b[4] = {0.f, 0.f, 0.f, 0.f};
    if (mom && !a.first_step) {
      const float4 b4 = reinterpret_cast<float4*>(mom)[i];
      b[0] = b4.x; b[1] = b4.y; b[2] = b4.z; b[3] = b4.w;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float gj = g[j] * gs + a.weight_decay * p[j];
      if (mom) {
        b[j] = a.first_step ? gj : a.momentum * b[j] + (1.f - a.dampening) * gj;
        gj = a.nesterov ? gj + a.momentum * b[j] : b[j];
      }
      p[j] -= a.lr * gj;
    }
    reinterpret_cast<float4*>(master)[i] = make_float4(p[0], p[1], p[2], p[3]);
    if (mom) reinterpret_cast<float4*>(mom)[i] = make_float4(b[0], b[1], b[2], b[3]);
    if (p_lp) {
      uint2 o;
      o.x = pack_bf16x2(p[0], p[1]);
      o.y = pack_bf16x2(p[2], p[3]);
      reinterpret_cast<uint2*>(p_lp)[i] = o;
    }
  }
}

// ---------------------------------------------------------------- gradient norm
// partial[b] = sum of squares seen by block b (fixed grid => deterministic order).
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const void* __restrict__ grad, long long n, int grad_f32, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float g[4];
    load_grad4(grad, grad_f32, i, g);
    s += g[0] * g[0] + g[1] * g[1] + g[2] * g[2] + g[3] * g[3];
  }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) partial[blockIdx.x] = t;
  }
}
// out[0] = total norm, out[1] = clip coefficient min(1, max_norm / (norm + 1e-6)).
// extra_sumsq (optional) is added before the square root (e.g. norm^2 reduced from other ranks).
__global__ void norm_finalize_kernel(const float* __restrict__ partial, int n, const float* extra_sumsq,
                                     float max_norm, float* __restrict__ out) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) {
      if (extra_sumsq) t += *extra_sumsq;
      const float nrm = sqrtf(t);
      out[0] = nrm;
      out[1] = max_norm > 0.f ? fminf(1.f, max_norm / (nrm + 1e-6f)) : 1.f;
      out[2] = t;
    }
  }
}

// ---------------------------------------------------------------- cross entropy
// One block per row.  loss[row] = logsumexp(z) - z[target] (0 for ignored rows);
// logits are overwritten with d loss_sum / d z * grad_scale = (softmax - onehot) * grad_scale.
__global__ void __launch_bounds__(512)
cross_entropy_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ target,
                             float* __restrict__ loss, int rows, int V, long long ld, float grad_scale,
                             long long ignore_index, int write_grad) {
  __shared__ float red[32];
  const int nvec = V >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* z = logits + static_cast<size_t>(row) * ld;
    const long long tgt = target[row];
    const bool ignored = (tgt == ignore_index) || tgt < 0 || tgt >= V;
    // pass 1: online max / sum-exp
    float mx = -INFINITY, se = 0.f;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      const uint4 u = reinterpret_cast<const uint4*>(z)[v];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      const float nm = fmaxf(mx, lm);
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += __expf(f[j] - nm);
      se = se * __expf(mx - nm) + acc;
      mx = nm;
    }
    for (int i = (nvec << 3) + threadIdx.x; i < V; i += blockDim.x) {  // tail (V % 8)
      const float f = __bfloat162float(z[i]);
      const float nm = fmaxf(mx, f);
      se = se * __expf(mx - nm) + __expf(f - nm);
      mx = nm;
    }
    // block combine
    float gmx = warp_max(mx);
    {
      const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
      __syncthreads();
      if (l == 0) red[w] = gmx;
      __syncthreads();
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -INFINITY;
      if (w == 0) { t = warp_max(t); if (l == 0) red[0] = t; }
      __syncthreads();
      gmx = red[0];
    }
    float part = (mx == -INFINITY) ? 0.f : se * __expf(mx - gmx);
    part = warp_sum(part);
    {
      const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
      __syncthreads();
      if (l == 0) red[w] = part;
      __syncthreads();
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      if (w == 0) { t = warp_sum(t); if (l == 0) red[0] = t; }
      __syncthreads();
      part = red[0];
    }
    const float lse = gmx + logf(part);
    if (threadIdx.x == 0)
      loss[row] = ignored ? 0.f : lse - __bfloat162float(z[tgt]);
    __syncthreads();  // z[tgt] read before it is overwritten below
    if (!write_grad) continue;
    const float gsc = ignored ? 0.f : grad_scale;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 u = reinterpret_cast<const uint4*>(z)[v];
      float f[8];
      float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
      f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
      const int base = v << 3;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float pj = __expf(f[j] - lse);
        if (base + j == tgt) pj -= 1.f;
        f[j] = pj * gsc;
      }
      uint4 o;
      o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
      o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
      reinterpret_cast<uint4*>(z)[v] = o;
    }
    for (int i = (nvec << 3) + threadIdx.x; i < V; i += blockDim.x) {
      float pj = __expf(__bfloat162float(z[i]) - lse);
      if (i == tgt) pj -= 1.f;
      z[i] = __float2bfloat16(pj * gsc);
    }
    __syncthreads();
  }
}

}  // namespace ft

using namespace ft;

static int flat_grid(long long n, int device) {
  long long b = ((n >> 2) + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 8;
  if (b > cap) b = cap;
  return b < 1 ? 1 : static_cast<int>(b);
}

FT_API int ft_adamw_flat(float* master, float* m, float* v, const void* grad, void* p_lp, long long n,
                         int grad_f32, const float* grad_scale, float lr, float beta1, float beta2,
                         float eps, float weight_decay, int step, int adam_l2, int device,
                         cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(master && m && v && grad, "ft_adamw_flat: null pointer");
  FT_REQUIRE(n % 4 == 0 && step >= 1, "ft_adamw_flat: n must be a multiple of 4 and step >= 1");
  if (n == 0) return FT_E_OK;
  AdamWArgs a;
  a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay;
  a.bc1 = 1.f - powf(beta1, static_cast<float>(step));
  a.bc2 = 1.f - powf(beta2, static_cast<float>(step));
  a.adam_l2 = adam_l2;
  const uintptr_t align = reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(m) |
                          reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(grad) |
                          reinterpret_cast<uintptr_t>(p_lp);
  if (n % 8 == 0 && (align & 15) == 0)
    adamw_flat8_kernel<<<flat_grid(n >> 1, device), 256, 0, stream>>>(
        master, m, v, grad, static_cast<__nv_bfloat16*>(p_lp), n, grad_f32, grad_scale, a);
  else
    adamw_flat_kernel<<<flat_grid(n, device), 256, 0, stream>>>(
        master, m, v, grad, static_cast<__nv_bfloat16*>(p_lp), n, grad_f32, grad_scale, a);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

FT_API int ft_sgd_flat(float* master, float* mom, const void* grad, void* p_lp, long long n,
                       int grad_f32, const float* grad_scale, float lr, float momentum, float dampening,
                       float weight_decay, int nesterov, int first_step, int device,
                       cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(master && grad, "ft_sgd_flat: null pointer");
  FT_REQUIRE(n % 4 == 0, "ft_sgd_flat: n must be a multiple of 4");
  FT_REQUIRE(momentum == 0.f || mom, "ft_sgd_flat: momentum without buffer");
  if (n == 0) return FT_E_OK;
  SgdArgs a;
  a.lr = lr; a.momentum = momentum; a.dampening = dampening; a.weight_decay = weight_decay;
  a.nesterov = nesterov; a.first_step = first_step;
  sgd_flat_kernel<<<flat_grid(n, device), 256, 0, stream>>>(
      master, momentum != 0.f ? mom : nullptr, grad, static_cast<__nv_bfloat16*>(p_lp), n, grad_f32,
      grad_scale, a);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// Number of fp32 partial slots ft_grad_norm needs.
FT_API int ft_grad_norm_scratch(int device) { return sm_count(device) * 4; }

// out: 3 floats {norm, clip_coef, norm^2}; partial: ft_grad_norm_scratch() floats.
FT_API int ft_grad_norm(const void* grad, long long n, int grad_f32, float* partial,
                        const float* extra_sumsq, float max_norm, float* out, int device,
                        cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(grad && partial && out && n % 4 == 0, "ft_grad_norm: bad arguments");
  const int blocks = ft_grad_norm_scratch(device);
  sumsq_partial_kernel<<<blocks, 256, 0, stream>>>(grad, n, grad_f32, partial);
  FT_CUDA_CHECK(cudaGetLastError());
  norm_finalize_kernel<<<1, 256, 0, stream>>>(partial, blocks, extra_sumsq, max_norm, out);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch(2);
  return FT_E_OK;
}

FT_API int ft_cross_entropy(void* logits, const long long* target, float* loss, int rows, int V,
                            long long ld, float grad_scale, long long ignore_index, int write_grad,
                            int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(logits && target && loss, "ft_cross_entropy: null pointer");
  FT_REQUIRE(ld % 8 == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0,
             "ft_cross_entropy: rows must be 16-byte aligned");
  if (rows <= 0) return FT_E_OK;
  const int grid = rows < sm_count(device) * 4 ? rows : sm_count(device) * 4;
  cross_entropy_fwd_bwd_kernel<<<grid, 512, 0, stream>>>(static_cast<__nv_bfloat16*>(logits), target,
                                                         loss, rows, V, ld, grad_scale, ignore_index,
                                                         write_grad);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}
