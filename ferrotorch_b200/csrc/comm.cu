// Collectives and fused compute+collective kernels over NVLink peer memory (sm_100a).
//
// Every rank passes the same table of peer pointers (symmetric buffers mapped into its
// address space).  The kernels move data with plain peer loads / stores issued from inside
// the kernel and synchronise through 32-bit flags in symmetric memory:
//     writer:  data stores ; __threadfence_system() ; st.release.sys flag = epoch
//     reader:  bounded spin on ld.acquire.sys flag ; then the data loads
// Epochs are monotonic, so flags never need resetting and the kernels can be replayed from a
// CUDA graph.  Every spin is bounded by wall-clock time; when the limit runs out the kernel
// writes FT_ERR_TIMEOUT_PEER to the status word and returns (the context stays usable).
//
//   ft_ddp_reduce_update   the data-parallel hot path: for one gradient bucket, each rank
//       pulls its 1/W slice of the bf16 gradients from all W ranks, sums them in fp32 in rank
//       order (every element is reduced by exactly one rank, so replicas stay bitwise
//       identical), applies the mean and the AdamW / SGD update to its fp32 master weights
//       and moments, and pushes the new bf16 weights into every rank's parameter arena.
//       This replaces "all-reduce the bucket, then run the optimizer on all of it on every
//       rank" (the reference: host-staged bucket all-reduce after backward,
//       ferrotorch-distributed/src/ddp.rs:265-311, then ~17 launches per parameter,
//       ferrotorch-optim/src/adamw.rs:239-384).
//   ft_allreduce_bf16 / f32  two-shot all-reduce (sum or mean) with the same structure
//       (reduce own slice, push the result to every rank); fixed rank order.
//   ft_allgather / ft_reduce_scatter_f32  pull-based all-gather, slice reduce.
//   ft_comm_wait           waits until every peer has raised a flag (step / bucket barrier).
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int COMM_MAX_RANKS = 8;
constexpr int COMM_THREADS = 512;

struct PeerTable {
  void* ptr[COMM_MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_cg_f4(const void* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// Wait until flags[i] has reached `epoch` for all i < n (epochs are compared modulo 2^32).
// One thread per flag spins; returns false for the whole block when the limit ran out.
__device__ __forceinline__ bool wait_flags(const uint32_t* flags, int n, uint32_t epoch,
                                           unsigned long long limit_ns, int* status) {
  __shared__ int s_fail;
  if (threadIdx.x == 0) s_fail = 0;
  __syncthreads();
  if (threadIdx.x < n) {
    const unsigned long long t0 = globaltimer_ns();
    uint32_t backoff = 32;
    while (static_cast<int32_t>(ld_acquire_sys(flags + threadIdx.x) - epoch) < 0) {
      // also give up at once when an earlier kernel already reported a lost peer
      if ((status && *reinterpret_cast<const volatile int*>(status) != 0) || globaltimer_ns() - t0 > limit_ns) {
        s_fail = 1;
        if (status) atomicCAS(status, 0, FT_ERR_TIMEOUT_PEER);
        break;
      }
      __nanosleep(backoff);
      if (backoff < 1024) backoff <<= 1;
    }
  }
  __syncthreads();
  return s_fail == 0;
}

// Flag layout per rank (uint32): [kind][slot][src_rank], kind 0 = ready, 1 = done.
__device__ __forceinline__ size_t flag_index(int kind, int slot, int src, int n_slots) {
  return (static_cast<size_t>(kind) * n_slots + slot) * COMM_MAX_RANKS + src;
}

struct UpdateArgs {
  int kind;  // 0 none (plain all-reduce), 1 AdamW, 2 Adam (L2), 3 SGD
  float lr, beta1, beta2, eps, weight_decay, bc1, bc2, momentum, dampening;
  int nesterov, first_step;
};

struct DdpArgs {
  PeerTable grads;    // symmetric gradient arenas (bf16 or fp32), one pointer per rank
  PeerTable params;   // symmetric parameter arenas (bf16); unused for kind 0 with out == grads
  PeerTable flags;    // symmetric flag arrays
  float* master;      // local fp32 state (full-size arrays, indexed by arena offset)
  float* m;
  float* v;
  unsigned int* block_counter;  // local, one per slot, zero between launches
  long long lo;       // first arena element of the bucket
  long long n;        // bucket length, multiple of 8 * world
  int rank, world, slot, n_slots;
  uint32_t epoch;
  float scale;        // applied to the summed gradient (1/world for a mean)
  int grad_f32;
  unsigned long long limit_ns;
  UpdateArgs u;
  int* status;
};

__device__ __forceinline__ void apply_update(const UpdateArgs& u, float g, float& p, float& m, float& v) {
  if (u.kind == 1 || u.kind == 2) {
    if (u.kind == 2) g += u.weight_decay * p; else p *= (1.f - u.lr * u.weight_decay);
    m = u.beta1 * m + (1.f - u.beta1) * g;
    v = u.beta2 * v + (1.f - u.beta2) * g * g;
    p -= u.lr * (m / u.bc1) / (sqrtf(v / u.bc2) + u.eps);
  } else {  // SGD
    g += u.weight_decay * p;
    if (u.momentum != 0.f) {
      m = u.first_step ? g : u.momentum * m + (1.f - u.dampening) * g;
      g = u.nesterov ? g + u.momentum * m : m;
    }
    p -= u.lr * g;
  }
}

// Launched as clusters of two CTAs (nothing in the kernel uses the cluster): the pair occupies one
// SM pair, so a GEMM that runs beside it on CTA-pair clusters loses whole pairs, never half of two.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(COMM_THREADS)
ddp_reduce_update_kernel(const DdpArgs a) {
  uint32_t* my_flags = static_cast<uint32_t*>(a.flags.ptr[a.rank]);
  // 1. tell every peer that this rank's gradients of the bucket are final (they were written by
  //    kernels earlier in stream order; the fence makes them visible system-wide first)
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(a.flags.ptr[threadIdx.x]) + flag_index(0, a.slot, a.rank, a.n_slots),
                   a.epoch);
  }
  // 2. wait for every peer's gradients
  //    A block whose wait ran out skips the work but still takes part in step 4, so that the
  //    per-slot block counter returns to zero and a later launch on this slot is not confused.
  const bool peers_ok =
      wait_flags(my_flags + flag_index(0, a.slot, 0, a.n_slots), a.world, a.epoch, a.limit_ns, a.status);

  // 3. reduce + update the slice this rank owns, push the new weights to every rank
  const long long slice = a.n / a.world;
  const long long base = a.lo + static_cast<long long>(a.rank) * slice;
  const long long nvec = peers_ok ? (slice >> 3) : 0;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long e = base + (i << 3);
    float g[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < COMM_MAX_RANKS; ++r) {
      if (r < a.world) {
        if (a.grad_f32) {
          const float* src = static_cast<const float*>(a.grads.ptr[r]) + e;
          const float4 x = ld_cg_f4(src), y = ld_cg_f4(src + 4);
          g[0] += x.x; g[1] += x.y; g[2] += x.z; g[3] += x.w;
          g[4] += y.x; g[5] += y.y; g[6] += y.z; g[7] += y.w;
        } else {
          const uint4 x = ld_cg_u4(static_cast<const __nv_bfloat16*>(a.grads.ptr[r]) + e);
          const float2 f0 = unpack_bf16x2(x.x), f1 = unpack_bf16x2(x.y), f2 = unpack_bf16x2(x.z),
                       f3 = unpack_bf16x2(x.w);
          g[0] += f0.x; g[1] += f0.y; g[2] += f1.x; g[3] += f1.y;
          g[4] += f2.x; g[5] += f2.y; g[6] += f3.x; g[7] += f3.y;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= a.scale;
    if (a.u.kind == 0) {
      // plain all-reduce: the reduced values go back into every rank's gradient arena
      if (a.grad_f32) {
        const float4 o0 = make_float4(g[0], g[1], g[2], g[3]), o1 = make_float4(g[4], g[5], g[6], g[7]);
#pragma unroll
        for (int r = 0; r < COMM_MAX_RANKS; ++r)
          if (r < a.world) {
            float* dst = static_cast<float*>(a.grads.ptr[r]) + e;
            *reinterpret_cast<float4*>(dst) = o0;
            *reinterpret_cast<float4*>(dst + 4) = o1;
          }
      } else {
        uint4 o;
        o.x = pack_bf16x2(g[0], g[1]); o.y = pack_bf16x2(g[2], g[3]);
        o.z = pack_bf16x2(g[4], g[5]); o.w = pack_bf16x2(g[6], g[7]);
#pragma unroll
        for (int r = 0; r < COMM_MAX_RANKS; ++r)
          if (r < a.world) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.grads.ptr[r]) + e) = o;
      }
      continue;
    }
    float4 p0 = *reinterpret_cast<const float4*>(a.master + e), p1 = *reinterpret_cast<const float4*>(a.master + e + 4);
    float p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
    float mm[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, vv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (a.m) {
      const float4 m0 = *reinterpret_cast<const float4*>(a.m + e), m1 = *reinterpret_cast<const float4*>(a.m + e + 4);
      mm[0] = m0.x; mm[1] = m0.y; mm[2] = m0.z; mm[3] = m0.w; mm[4] = m1.x; mm[5] = m1.y; mm[6] = m1.z; mm[7] = m1.w;
    }
    if (a.v) {
      const float4 v0 = *reinterpret_cast<const float4*>(a.v + e), v1 = *reinterpret_cast<const float4*>(a.v + e + 4);
      vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) apply_update(a.u, g[j], p[j], mm[j], vv[j]);
    *reinterpret_cast<float4*>(a.master + e) = make_float4(p[0], p[1], p[2], p[3]);
    *reinterpret_cast<float4*>(a.master + e + 4) = make_float4(p[4], p[5], p[6], p[7]);
    if (a.m) {
      *reinterpret_cast<float4*>(a.m + e) = make_float4(mm[0], mm[1], mm[2], mm[3]);
      *reinterpret_cast<float4*>(a.m + e + 4) = make_float4(mm[4], mm[5], mm[6], mm[7]);
    }
    if (a.v) {
      *reinterpret_cast<float4*>(a.v + e) = make_float4(vv[0], vv[1], vv[2], vv[3]);
      *reinterpret_cast<float4*>(a.v + e + 4) = make_float4(vv[4], vv[5], vv[6], vv[7]);
    }
    uint4 o;
    o.x = pack_bf16x2(p[0], p[1]); o.y = pack_bf16x2(p[2], p[3]);
    o.z = pack_bf16x2(p[4], p[5]); o.w = pack_bf16x2(p[6], p[7]);
#pragma unroll
    for (int r = 0; r < COMM_MAX_RANKS; ++r)
      if (r < a.world) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.params.ptr[r]) + e) = o;
  }

  // 4. the last block to finish raises this rank's "done" flag on every peer (not after a
  //    timed-out wait anywhere in the grid: the status word is set then)
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(a.block_counter + a.slot, 1u);
    s_last = (done == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) a.block_counter[a.slot] = 0u;
    const bool clean = peers_ok && !(a.status && *reinterpret_cast<const volatile int*>(a.status) != 0);
    if (clean && threadIdx.x < a.world) {
      __threadfence_system();
      st_release_sys(static_cast<uint32_t*>(a.flags.ptr[threadIdx.x]) + flag_index(1, a.slot, a.rank, a.n_slots),
                     a.epoch);
    }
  }
}

// Wait until every peer raised flag `kind` of slots [slot0, slot0 + n_wait) to `epoch`.
__global__ void comm_wait_kernel(const uint32_t* my_flags, int kind, int slot0, int n_wait, int n_slots,
                                 int world, uint32_t epoch, unsigned long long limit_ns, int* status) {
  for (int s = slot0 + blockIdx.x; s < slot0 + n_wait; s += gridDim.x)
    if (!wait_flags(my_flags + flag_index(kind, s, 0, n_slots), world, epoch, limit_ns, status)) return;
}

// Raise flag `kind` of `slot` on every peer (used by tests and as a barrier building block).
__global__ void comm_signal_kernel(PeerTable flags, int kind, int slot, int n_slots, int rank, int world,
                                   uint32_t epoch) {
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(flags.ptr[threadIdx.x]) + flag_index(kind, slot, rank, n_slots), epoch);
  }
}

// out[r * n + i] = peer_r[i]: pull-based all-gather of n*elem_bytes bytes from every rank.
// Peers must have raised the ready flag of `slot` (done by the caller with comm_signal).
__global__ void __launch_bounds__(COMM_THREADS)
allgather_pull_kernel(PeerTable src, uint8_t* out, long long bytes_per_rank, const uint32_t* my_flags, int slot,
                      int n_slots, int world, uint32_t epoch, unsigned long long limit_ns, int* status) {
  if (!wait_flags(my_flags + flag_index(0, slot, 0, n_slots), world, epoch, limit_ns, status)) return;
  const long long nvec = bytes_per_rank >> 4;
  for (int r = 0; r < world; ++r) {
    const uint8_t* s = static_cast<const uint8_t*>(src.ptr[r]);
    uint8_t* d = out + static_cast<long long>(r) * bytes_per_rank;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
      *reinterpret_cast<uint4*>(d + (i << 4)) = ld_cg_u4(s + (i << 4));
  }
}

// General pull exchange (all-gather, all-to-all, uneven all-to-all): from every rank r copy
// bytes[r] bytes at offset src_off[r] of r's symmetric send buffer to out + dst_off[r].
// Raises this rank's ready flag first (its own send buffer is final in stream order), waits for
// every peer's, pulls in rotated rank order, and the last block raises the done flag on every
// peer: "this rank no longer reads your send buffer".
struct ExchangeArgs {
  PeerTable src;
  uint8_t* out;
  long long src_off[COMM_MAX_RANKS], dst_off[COMM_MAX_RANKS], bytes[COMM_MAX_RANKS];
  PeerTable flags;
  unsigned int* block_counter;
  int rank, world, slot, n_slots;
  uint32_t epoch;
  unsigned long long limit_ns;
  int* status;
};

__global__ void __launch_bounds__(COMM_THREADS) exchange_pull_kernel(const ExchangeArgs a) {
  const uint32_t* my_flags = static_cast<const uint32_t*>(a.flags.ptr[a.rank]);
  if (blockIdx.x == 0 && threadIdx.x < a.world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(a.flags.ptr[threadIdx.x]) + flag_index(0, a.slot, a.rank, a.n_slots),
                   a.epoch);
  }
  // a block whose wait ran out copies nothing but still counts itself below, so the per-slot
  // block counter is back at zero for the next launch
  const bool peers_ok =
      wait_flags(my_flags + flag_index(0, a.slot, 0, a.n_slots), a.world, a.epoch, a.limit_ns, a.status);
  for (int k = 0; k < (peers_ok ? a.world : 0); ++k) {
    const int r = (a.rank + k) % a.world;
    const uint8_t* s = static_cast<const uint8_t*>(a.src.ptr[r]) + a.src_off[r];
    uint8_t* d = a.out + a.dst_off[r];
    const long long nvec = a.bytes[r] >> 4;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long i0 = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i0 < nvec; i0 += 4 * stride) {
      uint4 v[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const long long i = i0 + q * stride;
        v[q] = ld_cg_u4(s + ((i < nvec ? i : i0) << 4));
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const long long i = i0 + q * stride;
        if (i < nvec) *reinterpret_cast<uint4*>(d + (i << 4)) = v[q];
      }
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ unsigned int s_last;
  if (threadIdx.x == 0) {
    const unsigned int done = atomicAdd(a.block_counter + a.slot, 1u);
    s_last = (done == gridDim.x - 1) ? 1u : 0u;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) a.block_counter[a.slot] = 0u;
    const bool clean = peers_ok && !(a.status && *reinterpret_cast<const volatile int*>(a.status) != 0);
    if (clean && threadIdx.x < a.world) {
      __threadfence_system();
      st_release_sys(static_cast<uint32_t*>(a.flags.ptr[threadIdx.x]) + flag_index(1, a.slot, a.rank, a.n_slots),
                     a.epoch);
    }
  }
}

static int fill_table(PeerTable& t, void* const* ptrs, int world) {
  for (int i = 0; i < COMM_MAX_RANKS; ++i) t.ptr[i] = i < world ? ptrs[i] : nullptr;
  for (int i = 0; i < world; ++i)
    if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)) return FT_E_BAD_ARG;
  return FT_E_OK;
}

}  // namespace ft

using namespace ft;

// Number of uint32 flags a rank's symmetric flag array must hold for n_slots buckets.
FT_API long long ft_comm_flag_count(int n_slots) { return 2LL * n_slots * COMM_MAX_RANKS; }

// One gradient bucket: reduce (sum * scale) the arena range [lo, lo + n) across ranks and
// update / write back.  update_kind: 0 plain all-reduce into the gradient arenas, 1 AdamW,
// 2 Adam (L2 decay), 3 SGD.  n must be a multiple of 8 * world and lo of 8.  `blocks` limits
// the grid (0 = default) so the kernel can share the GPU with the backward pass.
FT_API int ft_ddp_reduce_update(void* const* grad_ptrs, void* const* param_ptrs, void* const* flag_ptrs,
                                float* master, float* m, float* v, unsigned int* block_counter,
                                long long lo, long long n, int rank, int world, int slot, int n_slots,
                                unsigned int epoch, float scale, int grad_f32, int update_kind, float lr,
                                float beta1, float beta2, float eps, float weight_decay, int step,
                                float momentum, float dampening, int nesterov, int blocks,
                                long long timeout_ms, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(world >= 1 && world <= COMM_MAX_RANKS && rank >= 0 && rank < world, "ft_ddp_reduce_update: bad rank/world");
  FT_REQUIRE(n > 0 && n % (8LL * world) == 0 && lo % 8 == 0, "ft_ddp_reduce_update: bucket [%lld, +%lld) not aligned to 8*world", lo, n);
  FT_REQUIRE(slot >= 0 && slot < n_slots && block_counter, "ft_ddp_reduce_update: bad slot");
  FT_REQUIRE(update_kind == 0 || master, "ft_ddp_reduce_update: update without master weights");
  DdpArgs a;
  FT_REQUIRE(fill_table(a.grads, grad_ptrs, world) == 0, "ft_ddp_reduce_update: bad gradient pointers");
  FT_REQUIRE(fill_table(a.flags, flag_ptrs, world) == 0, "ft_ddp_reduce_update: bad flag pointers");
  if (update_kind != 0) FT_REQUIRE(fill_table(a.params, param_ptrs, world) == 0, "ft_ddp_reduce_update: bad parameter pointers");
  else for (int i = 0; i < COMM_MAX_RANKS; ++i) a.params.ptr[i] = nullptr;
  a.master = master; a.m = m; a.v = v; a.block_counter = block_counter;
  a.lo = lo; a.n = n; a.rank = rank; a.world = world; a.slot = slot; a.n_slots = n_slots;
  a.epoch = epoch; a.scale = scale; a.grad_f32 = grad_f32;
  a.limit_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 20000) * 1000000ull;
  a.u.kind = update_kind; a.u.lr = lr; a.u.beta1 = beta1; a.u.beta2 = beta2; a.u.eps = eps;
  a.u.weight_decay = weight_decay;
  a.u.bc1 = 1.f - powf(beta1, static_cast<float>(step > 0 ? step : 1));
  a.u.bc2 = 1.f - powf(beta2, static_cast<float>(step > 0 ? step : 1));
  a.u.momentum = momentum; a.u.dampening = dampening; a.u.nesterov = nesterov; a.u.first_step = step <= 1;
  a.status = device_status_word(device);
  const long long nvec = (n / world) >> 3;
  long long grid = (nvec + COMM_THREADS - 1) / COMM_THREADS;
  const long long cap = blocks > 0 ? blocks : sm_count(device);
  if (grid > cap) grid = cap;
  grid = (grid + 1) / 2 * 2;  // clusters of two
  if (grid < 2) grid = 2;
  ddp_reduce_update_kernel<<<static_cast<unsigned>(grid), COMM_THREADS, 0, stream>>>(a);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

FT_API int ft_comm_wait(const void* my_flags, int kind, int slot0, int n_wait, int n_slots, int world,
                        unsigned int epoch, long long timeout_ms, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(my_flags && n_wait > 0 && slot0 >= 0 && slot0 + n_wait <= n_slots, "ft_comm_wait: bad arguments");
  const unsigned long long limit = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 20000) * 1000000ull;
  comm_wait_kernel<<<n_wait < 64 ? n_wait : 64, 32, 0, stream>>>(static_cast<const uint32_t*>(my_flags), kind, slot0,
                                                                 n_wait, n_slots, world, epoch, limit,
                                                                 device_status_word(device));
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

FT_API int ft_comm_signal(void* const* flag_ptrs, int kind, int slot, int n_slots, int rank, int world,
                          unsigned int epoch, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  PeerTable t;
  FT_REQUIRE(world >= 1 && world <= COMM_MAX_RANKS && fill_table(t, flag_ptrs, world) == 0, "ft_comm_signal: bad arguments");
  comm_signal_kernel<<<1, 32, 0, stream>>>(t, kind, slot, n_slots, rank, world, epoch);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// All-gather: out (local, world * bytes_per_rank bytes) <- every rank's symmetric src buffer.
// Signals readiness of the local src, waits for the peers, then pulls.
FT_API int ft_allgather(void* const* src_ptrs, void* out, long long bytes_per_rank, void* const* flag_ptrs,
                        int slot, int n_slots, int rank, int world, unsigned int epoch, long long timeout_ms,
                        int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  PeerTable src, flags;
  FT_REQUIRE(world >= 1 && world <= COMM_MAX_RANKS && fill_table(src, src_ptrs, world) == 0 &&
                 fill_table(flags, flag_ptrs, world) == 0 && out && bytes_per_rank % 16 == 0,
             "ft_allgather: bad arguments (buffers must be 16-byte aligned and sized)");
  comm_signal_kernel<<<1, 32, 0, stream>>>(flags, 0, slot, n_slots, rank, world, epoch);
  FT_CUDA_CHECK(cudaGetLastError());
  const unsigned long long limit = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 20000) * 1000000ull;
  long long grid = ((bytes_per_rank >> 4) + COMM_THREADS - 1) / COMM_THREADS;
  if (grid > sm_count(device)) grid = sm_count(device);
  if (grid < 1) grid = 1;
  allgather_pull_kernel<<<static_cast<unsigned>(grid), COMM_THREADS, 0, stream>>>(
      src, static_cast<uint8_t*>(out), bytes_per_rank, static_cast<const uint32_t*>(flag_ptrs[rank]), slot, n_slots,
      world, epoch, limit, device_status_word(device));
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch(2);
  return FT_E_OK;
}

// Pull exchange over symmetric send buffers (see exchange_pull_kernel).  src_off / dst_off /
// bytes: host arrays of `world` entries, all multiples of 16.  block_counter: n_slots zeroed
// uint32 words in local memory.  Before the send buffer is written again the caller waits for
// flag (kind 1, slot) == epoch of this call (ft_comm_wait).
FT_API int ft_peer_exchange(void* const* src_ptrs, void* out, const long long* src_off, const long long* dst_off,
                            const long long* bytes, void* const* flag_ptrs, unsigned int* block_counter,
                            int slot, int n_slots, int rank, int world, unsigned int epoch, int blocks,
                            long long timeout_ms, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  ExchangeArgs a;
  FT_REQUIRE(world >= 1 && world <= COMM_MAX_RANKS && rank >= 0 && rank < world && out && block_counter &&
                 fill_table(a.src, src_ptrs, world) == 0 && fill_table(a.flags, flag_ptrs, world) == 0,
             "ft_peer_exchange: bad arguments");
  FT_REQUIRE(slot >= 0 && slot < n_slots && (reinterpret_cast<uintptr_t>(out) & 15) == 0, "ft_peer_exchange: bad slot or unaligned output");
  long long most = 0;
  for (int r = 0; r < COMM_MAX_RANKS; ++r) {
    a.src_off[r] = r < world ? src_off[r] : 0;
    a.dst_off[r] = r < world ? dst_off[r] : 0;
    a.bytes[r] = r < world ? bytes[r] : 0;
    FT_REQUIRE(((a.src_off[r] | a.dst_off[r] | a.bytes[r]) & 15) == 0 && a.bytes[r] >= 0,
               "ft_peer_exchange: offsets and sizes must be multiples of 16 bytes");
    if (a.bytes[r] > most) most = a.bytes[r];
  }
  a.out = static_cast<uint8_t*>(out); a.block_counter = block_counter;
  a.rank = rank; a.world = world; a.slot = slot; a.n_slots = n_slots; a.epoch = epoch;
  a.limit_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 20000) * 1000000ull;
  a.status = device_status_word(device);
  long long grid = ((most >> 4) + 4LL * COMM_THREADS - 1) / (4LL * COMM_THREADS);
  const long long cap = blocks > 0 ? blocks : sm_count(device);
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  exchange_pull_kernel<<<static_cast<unsigned>(grid), COMM_THREADS, 0, stream>>>(a);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// ---------------------------------------------------------------------------------------------
// Device-resident epochs.  A kernel argument is frozen when a CUDA graph is captured, so the
// graph-replayable variants keep each slot's epoch in device memory: the signal kernel
// increments it and publishes the new value, the wait kernel compares against the current
// value.  All ranks run the same launch sequence, so their counters advance in lockstep.
namespace ft {
__global__ void comm_signal_dev_kernel(PeerTable flags, int kind, int slot, int n_slots, int rank, int world,
                                       uint32_t* epoch_dev) {
  __shared__ uint32_t s_epoch;
  if (threadIdx.x == 0) {
    s_epoch = *epoch_dev + 1u;
    *epoch_dev = s_epoch;
  }
  __syncthreads();
  if (threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(static_cast<uint32_t*>(flags.ptr[threadIdx.x]) + flag_index(kind, slot, rank, n_slots), s_epoch);
  }
}
__global__ void comm_wait_dev_kernel(const uint32_t* my_flags, int kind, int slot, int n_slots, int world,
                                     const uint32_t* epoch_dev, unsigned long long limit_ns, int* status) {
  const uint32_t epoch = *epoch_dev;
  if (epoch == 0u) return;  // slot never used
  wait_flags(my_flags + flag_index(kind, slot, 0, n_slots), world, epoch, limit_ns, status);
}
}  // namespace ft

// Raise flag (kind, slot) on every peer to ++(*epoch_dev).
FT_API int ft_comm_signal_dev(void* const* flag_ptrs, int kind, int slot, int n_slots, int rank, int world,
                              unsigned int* epoch_dev, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  PeerTable t;
  FT_REQUIRE(epoch_dev && world >= 1 && world <= COMM_MAX_RANKS && fill_table(t, flag_ptrs, world) == 0,
             "ft_comm_signal_dev: bad arguments");
  comm_signal_dev_kernel<<<1, 32, 0, stream>>>(t, kind, slot, n_slots, rank, world, epoch_dev);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

// Wait until every peer raised flag (kind, slot) to the current *epoch_dev (no-op while it is 0).
FT_API int ft_comm_wait_dev(const void* my_flags, int kind, int slot, int n_slots, int world,
                            const unsigned int* epoch_dev, long long timeout_ms, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(my_flags && epoch_dev && slot >= 0 && slot < n_slots, "ft_comm_wait_dev: bad arguments");
  const unsigned long long limit = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 20000) * 1000000ull;
  comm_wait_dev_kernel<<<1, 32, 0, stream>>>(static_cast<const uint32_t*>(my_flags), kind, slot, n_slots, world,
                                            epoch_dev, limit, device_status_word(device));
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}
