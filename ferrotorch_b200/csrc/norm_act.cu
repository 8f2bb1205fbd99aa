// Memory-bound transformer kernels for sm_100a: RMSNorm (+ fused residual add)
// forward/backward, rotary embedding (both pair conventions) forward/backward,
// SwiGLU forward/backward, embedding gather / scatter-add.
//
// Semantics follow the reference: RMSNorm = x * rsqrt(mean(x^2) + eps) * w with fp32
// statistics (ferrotorch-gpu/src/bf16.rs:1340-1346, kernels.rs:10578, 10725); RoPE
// rotates the pair (d, d + D/2) ("half" / HF convention, bf16.rs:1850-1855) or
// (2d, 2d+1) (interleaved, ferrotorch-nn/src/transformer.rs:66-72) with the backward
// of transformer.rs:132-156; SwiGLU = silu(gate) * up (ferrotorch-llama/src/gpu.rs:696-703).
// Unlike the reference (one launch per op, 256-thread 1-D grids) every kernel moves
// 16-byte vectors, keeps the row in registers between the statistics pass and the
// scale pass, and fuses the neighbouring residual add / gate multiply.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 4;  // 4 vec * 8 elems * 256 thr = rows up to 8192 wide in registers

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}
__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) {
    t = warp_max(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ---------------------------------------------------------------- RMSNorm forward
// y = (x [+ delta]) * rstd * w ; if delta != null also writes res_out = x + delta.
// One block per row, grid-stride over rows. H % 8 == 0.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                   const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                   __nv_bfloat16* __restrict__ res_out, float* __restrict__ rstd_out, int rows, int H,
                   float eps) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * H);
    const uint4* dr = delta ? reinterpret_cast<const uint4*>(delta + static_cast<size_t>(row) * H) : nullptr;
    float vals[NORM_MAX_VEC][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        unpack8(xr[v], vals[i]);
        if (dr) {
          float d[8];
          unpack8(dr[v], d);
#pragma unroll
          for (int j = 0; j < 8; ++j) vals[i][j] += d[j];
          if (res_out) {
            // round the residual stream to bf16 once; the statistics use the rounded value
            uint4 packed = pack8(vals[i]);
            reinterpret_cast<uint4*>(res_out + static_cast<size_t>(row) * H)[v] = packed;
            unpack8(packed, vals[i]);
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += vals[i][j] * vals[i][j];
      }
    }
    const float tot = block_sum(ss, red);
    const float rstd = rsqrtf(tot / static_cast<float>(H) + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float wv[8], o[8];
        unpack8(reinterpret_cast<const uint4*>(w)[v], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = vals[i][j] * rstd * wv[j];
        reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * H)[v] = pack8(o);
      }
    }
  }
}

// ---------------------------------------------------------------- RMSNorm backward
// dx = rstd * (g - xhat * mean(g * xhat)) [+ dres], g = dy * w, xhat = x * rstd.
// dw partial sums: each block keeps its columns' sums in registers over the rows it
// owns and writes one fp32 row of the scratch [gridDim.x, H]; rmsnorm_dw_reduce sums it.
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   const __nv_bfloat16* __restrict__ dres, __nv_bfloat16* __restrict__ dx,
                   float* __restrict__ dw_partial, int rows, int H) {
  __shared__ float red[32];
  const int nvec = H >> 3;
  float dwacc[NORM_MAX_VEC][8];
#pragma unroll
  for (int i = 0; i < NORM_MAX_VEC; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;

  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t off = static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    float g[NORM_MAX_VEC][8], xh[NORM_MAX_VEC][8];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float dyv[8], wv[8];
        unpack8(reinterpret_cast<const uint4*>(dy + off)[v], dyv);
        unpack8(reinterpret_cast<const uint4*>(x + off)[v], xh[i]);
        unpack8(reinterpret_cast<const uint4*>(w)[v], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i][j] *= rstd;
          g[i][j] = dyv[j] * wv[j];
          dot += g[i][j] * xh[i][j];
          dwacc[i][j] += dyv[j] * xh[i][j];
        }
      }
    }
    const float mean_dot = block_sum(dot, red) / static_cast<float>(H);
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = rstd * (g[i][j] - xh[i][j] * mean_dot);
        if (dres) {
          float r[8];
          unpack8(reinterpret_cast<const uint4*>(dres + off)[v], r);
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] += r[j];
        }
        reinterpret_cast<uint4*>(dx + off)[v] = pack8(o);
      }
    }
  }
  if (dw_partial) {
    float* out = dw_partial + static_cast<size_t>(blockIdx.x) * H;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int v = threadIdx.x + i * NORM_THREADS;
      if (v < nvec) {
        reinterpret_cast<float4*>(out)[2 * v] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
        reinterpret_cast<float4*>(out)[2 * v + 1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      }
    }
  }
}

// dw[h] (+)= sum_b partial[b, h]; writes bf16 or fp32.  A block owns 32 columns (one 128-byte
// segment of every partial row); its 8 warps each walk every 8th row with four loads in flight and
// the 8 sub-sums are added in warp order, so the result does not depend on scheduling.
constexpr int DW_RED_COLS = 32, DW_RED_WARPS = 8;
__global__ void __launch_bounds__(DW_RED_COLS * DW_RED_WARPS)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, void* __restrict__ dw, int nblocks, int H,
                         int out_f32, int accumulate) {
  __shared__ float sub[DW_RED_WARPS][DW_RED_COLS];
  const int tx = threadIdx.x & (DW_RED_COLS - 1), ty = threadIdx.x / DW_RED_COLS;
  const int h = blockIdx.x * DW_RED_COLS + tx;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (h < H) {
    const float* col = partial + h;
    int b = ty;
    for (; b + 3 * DW_RED_WARPS < nblocks; b += 4 * DW_RED_WARPS) {
      s0 += col[static_cast<size_t>(b) * H];
      s1 += col[static_cast<size_t>(b + DW_RED_WARPS) * H];
      s2 += col[static_cast<size_t>(b + 2 * DW_RED_WARPS) * H];
      s3 += col[static_cast<size_t>(b + 3 * DW_RED_WARPS) * H];
    }
    for (; b < nblocks; b += DW_RED_WARPS) s0 += col[static_cast<size_t>(b) * H];
  }
  sub[ty][tx] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (ty != 0 || h >= H) return;
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < DW_RED_WARPS; ++k) s += sub[k][tx];
  if (out_f32) {
    float* o = static_cast<float*>(dw);
    o[h] = accumulate ? o[h] + s : s;
  } else {
    __nv_bfloat16* o = static_cast<__nv_bfloat16*>(dw);
    o[h] = __float2bfloat16(accumulate ? __bfloat162float(o[h]) + s : s);
  }
}

// ---------------------------------------------------------------- RoPE
// x: [T, n_heads_total, D] with row stride `ld` (elements) between tokens; rotates
// heads [0, n_rot_heads).  cos/sin: fp32 [max_pos, D/2].  pos: int32 [T] or null
// (then position = (t % seq_len) + pos_offset).  sign = +1 forward, -1 backward.
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos, int T,
                            int n_rot_heads, int D, long long ld, int seq_len, int pos_offset,
                            int interleaved, float sign) {
  const int half = D >> 1;
  const int pairs_per_tok = n_rot_heads * half;
  const long long total = static_cast<long long>(T) * (pairs_per_tok >> 1);  // 2 pairs / thread
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / (pairs_per_tok >> 1));
    const int r = static_cast<int>(i - static_cast<long long>(t) * (pairs_per_tok >> 1)) * 2;
    const int h = r / half, d = r - h * half;  // d even
    const int p = pos ? pos[t] : (t % seq_len) + pos_offset;
    const float2 c = *reinterpret_cast<const float2*>(cos_t + static_cast<size_t>(p) * half + d);
    float2 s = *reinterpret_cast<const float2*>(sin_t + static_cast<size_t>(p) * half + d);
    s.x *= sign; s.y *= sign;
    __nv_bfloat16* base = x + static_cast<size_t>(t) * ld + static_cast<size_t>(h) * D;
    if (!interleaved) {
      __nv_bfloat162* p1 = reinterpret_cast<__nv_bfloat162*>(base + d);
      __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(base + d + half);
      const float2 a = __bfloat1622float2(*p1), b = __bfloat1622float2(*p2);
      *p1 = __floats2bfloat162_rn(a.x * c.x - b.x * s.x, a.y * c.y - b.y * s.y);
      *p2 = __floats2bfloat162_rn(b.x * c.x + a.x * s.x, b.y * c.y + a.y * s.y);
    } else {
      uint2* pp = reinterpret_cast<uint2*>(base + 2 * d);
      uint2 u = *pp;
      const float2 e0 = unpack_bf16x2(u.x), e1 = unpack_bf16x2(u.y);  // (x0,x1), (x2,x3)
      u.x = pack_bf16x2(e0.x * c.x - e0.y * s.x, e0.y * c.x + e0.x * s.x);
      u.y = pack_bf16x2(e1.x * c.y - e1.y * s.y, e1.y * c.y + e1.x * s.y);
      *pp = u;
    }
  }
}

// Vector version: one thread rotates 8 pairs.  Half-rotation layout: 16 bytes from the first
// half of a head and the 16 bytes that pair with them in the second half; interleaved layout:
// 32 contiguous bytes.  cos/sin come as two float4 each.  Needs D % 16 == 0 and 16-byte
// aligned rows (checked by the launcher).
__global__ void rope_vec_kernel(__nv_bfloat16* __restrict__ x, const float* __restrict__ cos_t,
                                const float* __restrict__ sin_t, const int* __restrict__ pos, int T,
                                int n_rot_heads, int D, long long ld, int seq_len, int pos_offset,
                                int interleaved, float sign) {
  const int half = D >> 1;
  const int groups_per_head = half >> 3;                       // 8 pairs per group
  const int groups_per_tok = n_rot_heads * groups_per_head;
  const long long total = static_cast<long long>(T) * groups_per_tok;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int t = static_cast<int>(i / groups_per_tok);
    const int r = static_cast<int>(i - static_cast<long long>(t) * groups_per_tok);
    const int h = r / groups_per_head, d = (r - h * groups_per_head) << 3;   // first pair index
    const int p = pos ? pos[t] : (t % seq_len) + pos_offset;
    const float4* cp = reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(p) * half + d);
    const float4* sp = reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(p) * half + d);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x * sign, s0.y * sign, s0.z * sign, s0.w * sign,
                         s1.x * sign, s1.y * sign, s1.z * sign, s1.w * sign};
    __nv_bfloat16* base = x + static_cast<size_t>(t) * ld + static_cast<size_t>(h) * D;
    float a[8], b[8], oa[8], ob[8];
    if (!interleaved) {
      uint4* p1 = reinterpret_cast<uint4*>(base + d);
      uint4* p2 = reinterpret_cast<uint4*>(base + d + half);
      unpack8(*p1, a);
      unpack8(*p2, b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        oa[j] = a[j] * c[j] - b[j] * sn[j];
        ob[j] = b[j] * c[j] + a[j] * sn[j];
      }
      *p1 = pack8(oa);
      *p2 = pack8(ob);
    } else {
      uint4* pp = reinterpret_cast<uint4*>(base + 2 * d);
      unpack8(pp[0], a);      // pairs 0..3 as (even, odd)
      unpack8(pp[1], b);      // pairs 4..7
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        oa[2 * j] = a[2 * j] * c[j] - a[2 * j + 1] * sn[j];
        oa[2 * j + 1] = a[2 * j + 1] * c[j] + a[2 * j] * sn[j];
        ob[2 * j] = b[2 * j] * c[4 + j] - b[2 * j + 1] * sn[4 + j];
        ob[2 * j + 1] = b[2 * j + 1] * c[4 + j] + b[2 * j] * sn[4 + j];
      }
      pp[0] = pack8(oa);
      pp[1] = pack8(ob);
    }
  }
}

// ---------------------------------------------------------------- SwiGLU
// gu: [T, 2F] (gate = [:, :F], up = [:, F:]), out: [T, F].  act: 0 silu, 1 relu, 2 gelu(tanh).
__device__ __forceinline__ float act_fwd(float g, int act) {
  if (act == 0) return g / (1.f + __expf(-g));
  if (act == 1) return fmaxf(g, 0.f);
  const float k = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  return 0.5f * g * (1.f + tanhf(k));
}
__device__ __forceinline__ float act_bwd(float g, int act) {
  if (act == 0) {
    const float s = 1.f / (1.f + __expf(-g));
    return s * (1.f + g * (1.f - s));
  }
  if (act == 1) return g > 0.f ? 1.f : 0.f;
  const float k = 0.7978845608028654f * (g + 0.044715f * g * g * g);
  const float t = tanhf(k);
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * g * g);
}
// Two vectors per thread with all loads issued first and streaming (evict-first) hints on the
// inputs, which are read exactly once.
__global__ void swiglu_fwd2_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                   long long T, int F, long long ld_gu, int act) {
  const int fv = F >> 3;
  const long long total = T * fv;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total; i0 += 2 * stride) {
    const long long i1 = i0 + stride < total ? i0 + stride : i0;
    const long long t0 = i0 / fv, t1 = i1 / fv;
    const int v0 = static_cast<int>(i0 - t0 * fv), v1 = static_cast<int>(i1 - t1 * fv);
    const uint4* r0 = reinterpret_cast<const uint4*>(gu + t0 * ld_gu);
    const uint4* r1 = reinterpret_cast<const uint4*>(gu + t1 * ld_gu);
    const uint4 g0 = __ldcs(r0 + v0), u0 = __ldcs(r0 + fv + v0), g1 = __ldcs(r1 + v1), u1 = __ldcs(r1 + fv + v1);
    float g[8], u[8], o[8];
    unpack8(g0, g);
    unpack8(u0, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], act) * u[j];
    reinterpret_cast<uint4*>(out + t0 * F)[v0] = pack8(o);
    if (i1 != i0) {
      unpack8(g1, g);
      unpack8(u1, u);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], act) * u[j];
      reinterpret_cast<uint4*>(out + t1 * F)[v1] = pack8(o);
    }
  }
}
__global__ void swiglu_bwd2_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ gu,
                                   __nv_bfloat16* __restrict__ dgu, long long T, int F, long long ld_gu,
                                   int act) {
  const int fv = F >> 3;
  const long long total = T * fv;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < total; i0 += 2 * stride) {
    const long long i1 = i0 + stride < total ? i0 + stride : i0;
    const long long tt[2] = {i0 / fv, i1 / fv};
    const int vv[2] = {static_cast<int>(i0 - tt[0] * fv), static_cast<int>(i1 - tt[1] * fv)};
    uint4 gq[2], uq[2], dq[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint4* row = reinterpret_cast<const uint4*>(gu + tt[k] * ld_gu);
      gq[k] = __ldcs(row + vv[k]);
      uq[k] = __ldcs(row + fv + vv[k]);
      dq[k] = __ldcs(reinterpret_cast<const uint4*>(dy + tt[k] * F) + vv[k]);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (k == 1 && i1 == i0) break;
      float g[8], u[8], d[8], dg[8], du[8];
      unpack8(gq[k], g);
      unpack8(uq[k], u);
      unpack8(dq[k], d);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        dg[j] = d[j] * u[j] * act_bwd(g[j], act);
        du[j] = d[j] * act_fwd(g[j], act);
      }
      uint4* orow = reinterpret_cast<uint4*>(dgu + tt[k] * ld_gu);
      orow[vv[k]] = pack8(dg);
      orow[fv + vv[k]] = pack8(du);
    }
  }
}

// ---------------------------------------------------------------- embedding
__global__ void embedding_fwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ w,
                                     __nv_bfloat16* __restrict__ out, int T, int H, int vocab) {
  const int hv = H >> 3;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    long long id = ids[t];
    if (id < 0 || id >= vocab) id = 0;  // host validates; never read out of range
    const uint4* src = reinterpret_cast<const uint4*>(w + static_cast<size_t>(id) * H);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * H);
    for (int v = threadIdx.x; v < hv; v += blockDim.x) dst[v] = src[v];
  }
}
__global__ void embedding_bwd_kernel(const long long* __restrict__ ids, const __nv_bfloat16* __restrict__ dy,
                                     __nv_bfloat16* __restrict__ dw, int T, int H, int vocab) {
  const int h2 = H >> 1;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    const long long id = ids[t];
    if (id < 0 || id >= vocab) continue;
    const __nv_bfloat162* src = reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<size_t>(t) * H);
    __nv_bfloat162* dst = reinterpret_cast<__nv_bfloat162*>(dw + static_cast<size_t>(id) * H);
    for (int v = threadIdx.x; v < h2; v += blockDim.x) atomicAdd(dst + v, src[v]);
  }
}

static inline int blocks_for(long long work, int threads, int device, int per_sm = 8) {
  long long b = (work + threads - 1) / threads;
  const long long cap = static_cast<long long>(sm_count(device)) * per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return static_cast<int>(b);
}

}  // namespace ft

using namespace ft;

FT_API int ft_rmsnorm_fwd(const void* x, const void* delta, const void* w, void* y, void* res_out,
                          float* rstd, int rows, int H, float eps, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && w && y, "ft_rmsnorm_fwd: null pointer");
  FT_REQUIRE(H % 8 == 0 && H <= NORM_THREADS * NORM_MAX_VEC * 8, "ft_rmsnorm_fwd: H=%d unsupported", H);
  if (rows <= 0) return FT_E_OK;
  const int grid = rows < sm_count(device) * 8 ? rows : sm_count(device) * 8;
  rmsnorm_fwd_kernel<<<grid, NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(delta),
      static_cast<const __nv_bfloat16*>(w), static_cast<__nv_bfloat16*>(y),
      static_cast<__nv_bfloat16*>(res_out), rstd, rows, H, eps);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// Number of fp32 scratch rows ft_rmsnorm_bwd needs for `rows` (scratch = n * H floats).
FT_API int ft_rmsnorm_bwd_scratch_rows(int rows, int device) {
  const int cap = sm_count(device) * 2;
  return rows < cap ? (rows > 0 ? rows : 1) : cap;
}

// dw may be null (then scratch may be null too).  dw_flags: bit0 fp32 output, bit1 accumulate.
FT_API int ft_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd,
                          const void* dres, void* dx, void* dw, float* scratch, int rows, int H,
                          int dw_flags, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(dy && x && w && rstd && dx, "ft_rmsnorm_bwd: null pointer");
  FT_REQUIRE(H % 8 == 0 && H <= NORM_THREADS * NORM_MAX_VEC * 8, "ft_rmsnorm_bwd: H=%d unsupported", H);
  FT_REQUIRE(!dw || scratch, "ft_rmsnorm_bwd: dw requested without scratch");
  if (rows <= 0) return FT_E_OK;
  const int grid = ft_rmsnorm_bwd_scratch_rows(rows, device);
  rmsnorm_bwd_kernel<<<grid, NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),
      static_cast<__nv_bfloat16*>(dx), dw ? scratch : nullptr, rows, H);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  if (dw) {
    rmsnorm_dw_reduce_kernel<<<(H + DW_RED_COLS - 1) / DW_RED_COLS, DW_RED_COLS * DW_RED_WARPS, 0, stream>>>(scratch, dw, grid, H, dw_flags & 1,
                                                                  (dw_flags >> 1) & 1);
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  return FT_E_OK;
}

FT_API int ft_rope(void* x, const float* cos_t, const float* sin_t, const int* pos, int T,
                   int n_rot_heads, int D, long long ld, int seq_len, int pos_offset, int interleaved,
                   int backward, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(x && cos_t && sin_t, "ft_rope: null pointer");
  FT_REQUIRE(D % 4 == 0 && ld % 4 == 0, "ft_rope: head_dim and row stride must be multiples of 4");
  FT_REQUIRE(pos || seq_len > 0, "ft_rope: need positions or seq_len");
  if (T <= 0 || n_rot_heads <= 0) return FT_E_OK;
  const long long work = static_cast<long long>(T) * n_rot_heads * (D / 4);
  if (D % 16 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(cos_t) & 15) == 0 && (reinterpret_cast<uintptr_t>(sin_t) & 15) == 0)
    rope_vec_kernel<<<blocks_for(work / 4, 256, device), 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(x), cos_t, sin_t, pos, T, n_rot_heads, D, ld, seq_len, pos_offset,
        interleaved, backward ? -1.f : 1.f);
  else
    rope_kernel<<<blocks_for(work, 256, device), 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(x), cos_t, sin_t, pos, T, n_rot_heads, D, ld, seq_len, pos_offset,
        interleaved, backward ? -1.f : 1.f);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

FT_API int ft_swiglu_fwd(const void* gu, void* out, long long T, int F, long long ld_gu, int act,
                         int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(gu && out, "ft_swiglu_fwd: null pointer");
  FT_REQUIRE(F % 8 == 0 && ld_gu % 8 == 0, "ft_swiglu_fwd: F must be a multiple of 8");
  if (T <= 0) return FT_E_OK;
  swiglu_fwd2_kernel<<<blocks_for(T * (F / 8) / 2 + 1, 256, device), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(gu), static_cast<__nv_bfloat16*>(out), T, F, ld_gu, act);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

FT_API int ft_swiglu_bwd(const void* dy, const void* gu, void* dgu, long long T, int F, long long ld_gu,
                         int act, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(dy && gu && dgu, "ft_swiglu_bwd: null pointer");
  FT_REQUIRE(F % 8 == 0 && ld_gu % 8 == 0, "ft_swiglu_bwd: F must be a multiple of 8");
  if (T <= 0) return FT_E_OK;
  swiglu_bwd2_kernel<<<blocks_for(T * (F / 8) / 2 + 1, 256, device), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(gu),
      static_cast<__nv_bfloat16*>(dgu), T, F, ld_gu, act);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

FT_API int ft_embedding_fwd(const long long* ids, const void* w, void* out, int T, int H, int vocab,
                            int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(ids && w && out && H % 8 == 0, "ft_embedding_fwd: bad arguments");
  if (T <= 0) return FT_E_OK;
  const int grid = T < sm_count(device) * 16 ? T : sm_count(device) * 16;
  embedding_fwd_kernel<<<grid, 128, 0, stream>>>(ids, static_cast<const __nv_bfloat16*>(w),
                                                 static_cast<__nv_bfloat16*>(out), T, H, vocab);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

FT_API int ft_embedding_bwd(const long long* ids, const void* dy, void* dw, int T, int H, int vocab,
                            int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(ids && dy && dw && H % 2 == 0, "ft_embedding_bwd: bad arguments");
  if (T <= 0) return FT_E_OK;
  const int grid = T < sm_count(device) * 16 ? T : sm_count(device) * 16;
  embedding_bwd_kernel<<<grid, 128, 0, stream>>>(ids, static_cast<const __nv_bfloat16*>(dy),
                                                 static_cast<__nv_bfloat16*>(dw), T, H, vocab);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// ---------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate (declaration and contract: ft_noalloc.h).
// The partial sums of dw go to this fixed array instead of caller-provided scratch.  In host
// code the name below is only a handle for cudaGetSymbolAddress, never a device pointer.
#include "ft_noalloc.h"

static __device__ __align__(256) float g_rmsnorm_noalloc_scratch[FT_NOALLOC_RMSNORM_ROWS * FT_NOALLOC_RMSNORM_MAX_H];

FT_API int ft_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                  const void* dres, void* dx, void* dw, int rows, int H, int dw_flags,
                                  int device, cudaStream_t stream) {
  FT_REQUIRE(dy && x && w && rstd && dx, "ft_rmsnorm_bwd_noalloc: null pointer");
  FT_REQUIRE(device >= 0 && device < 64, "ft_rmsnorm_bwd_noalloc: bad device %d", device);
  FT_REQUIRE(H > 0 && H % 8 == 0, "ft_rmsnorm_bwd_noalloc: H=%d must be a positive multiple of 8", H);
  if (H > FT_NOALLOC_RMSNORM_MAX_H) {
    set_last_error("ft_rmsnorm_bwd_noalloc: H=%d exceeds the fixed scratch (max %d); use ft_rmsnorm_bwd "
                   "with caller-provided scratch", H, FT_NOALLOC_RMSNORM_MAX_H);
    return FT_E_TOO_LARGE;
  }
  // The kernels below launch on the calling thread's current device, and the scratch address
  // belongs to `device`: the two must be the same GPU.  (Checked, not switched: switching would
  // have to be undone on every error path, and a caller that cannot allocate usually also wants
  // no hidden device changes.)
  int cur = -1;
  FT_CUDA_CHECK(cudaGetDevice(&cur));
  FT_REQUIRE(cur == device, "ft_rmsnorm_bwd_noalloc: device %d must be the current device (current is %d)",
             device, cur);
  if (rows <= 0) return FT_E_OK;
  // Once per device, with that device current: resolve the device address of the array.  Two
  // threads that race here both store the same value, so the unsynchronised write is benign.
  static float* scratch_of[64] = {nullptr};
  if (!scratch_of[device]) {
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_rmsnorm_noalloc_scratch);
    if (e != cudaSuccess || !ptr) {
      set_last_error("ft_rmsnorm_bwd_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return FT_E_CUDA;
    }
    scratch_of[device] = ptr;
  }
  float* scratch = scratch_of[device];
  const int grid = rows < FT_NOALLOC_RMSNORM_ROWS ? rows : FT_NOALLOC_RMSNORM_ROWS;
  // every partial row [0, grid) x [0, H) is written by the first kernel before the second reads
  // it, so the previous call's contents never leak into the result
  rmsnorm_bwd_kernel<<<grid, NORM_THREADS, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(x),
      static_cast<const __nv_bfloat16*>(w), rstd, static_cast<const __nv_bfloat16*>(dres),
      static_cast<__nv_bfloat16*>(dx), dw ? scratch : nullptr, rows, H);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  if (dw) {
    rmsnorm_dw_reduce_kernel<<<(H + DW_RED_COLS - 1) / DW_RED_COLS, DW_RED_COLS * DW_RED_WARPS, 0, stream>>>(scratch, dw, grid, H, dw_flags & 1,
                                                                  (dw_flags >> 1) & 1);
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
  }
  return FT_E_OK;
}
