// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sm_100a).
//
// The reference has no tensor / sequence parallelism (design only,
// .design/phase-7-distributed.md:269-307); a Megatron-style block needs two fused ops:
//
//   ft_tp_ag_gemm   Y[M, N_loc] = allgather_rows(X)[M, K] * W_loc[N_loc, K]^T
//       (column-parallel: QKV, gate/up).  Activations are sequence-sharded: rank s owns rows
//       [s*Ms, (s+1)*Ms) of a symmetric buffer Xg[M, K] and has written them before the call.
//       Inside ONE kernel, four "copy" warps of every CTA pull the other ranks' rows from peer
//       memory into the local Xg (each remote row crosses NVLink exactly once, in units of 16
//       rows, in the order the GEMM consumes them) and publish per-128-row block counters; the
//       tcgen05 GEMM roles of the same persistent CTAs start with the rows this rank already
//       owns and their TMA producers wait (bounded) on the block counter of each later tile, so
//       the transfer overlaps the math tile by tile and every SM runs tensor-core work.
//   ft_tp_gemm_rs   Out[Ms, N] (+ residual) = reduce_scatter_rows(X_loc[M, K_loc] * W_loc[N, K_loc]^T)
//       (row-parallel: o_proj, down_proj).  The epilogue stages each 32x64 piece of the partial
//       product in shared memory and stores it as 128-byte row segments straight into the
//       staging buffer of the rank that owns the row (peer stores), tiles for other ranks first; per-owner counters raise a system-scope flag on the owner when a
//       source has delivered everything; the same kernel then sums the W staged partials in
//       rank order in fp32, adds the residual and writes the owner's rows.
//
// Loads from peer memory are plain ld.global / non-multicast; TMA only ever reads this GPU's
// own memory here.  Every wait (mbarrier, block counter, peer flag) is bounded and reports
// through the device status word.
#include "ft_host.h"
#include "ft_ptx.cuh"

namespace ft {

constexpr int TP_BM = 128;
constexpr int TP_BK = 64;
constexpr int TP_THREADS = 320;     // producer, MMA, 2 copy, 4 epilogue, 2 copy warps
constexpr int TP_MAX_RANKS = 8;
constexpr int TP_UNIT_ROWS = 16;    // most rows of one all-gather copy unit
constexpr int TP_EPI_ROW = 144;     // bytes per staged epilogue row (128 + 16 of padding)
constexpr int TP_EPI_BYTES = 4 * 32 * TP_EPI_ROW;

struct TpPeers {
  void* ptr[TP_MAX_RANKS];
};

template <int BN>
struct TpCfg {
  static constexpr int A_BYTES = TP_BM * TP_BK * 2;
  static constexpr int B_BYTES = BN * TP_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES_RAW = (200 * 1024) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
  static constexpr int TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES + 256;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256 + TP_EPI_BYTES;
};

struct TpParams {
  int mode;  // 0 = all-gather -> GEMM, 1 = GEMM -> reduce-scatter
  int M, N, K;
  int rank, world, rows_per_rank;
  // mode 0
  __nv_bfloat16* C; long long ldc;       // local output [M, N]
  const void* bias;                      // optional bf16 [N]
  TpPeers xg; long long ldx;             // symmetric gathered-activation buffers [M, K]
  uint32_t* blk_ready;                   // local counters, one per 128-row block, zero at entry
  int n_copy;                            // CTAs of a gather-only launch
  int unit_rows;                         // rows per copy unit (1..TP_UNIT_ROWS, power of two)
  // mode 1
  TpPeers stage;                         // symmetric staging [world, rows_per_rank, N] bf16
  __nv_bfloat16* out; long long ldo;     // local output rows [rows_per_rank, N]
  const __nv_bfloat16* residual; long long ldr;
  unsigned int* owner_counter;           // local [world], zero at entry
  // both
  unsigned int* done_counter;            // local, zero at entry
  TpPeers flags; int slot, n_slots; uint32_t epoch;
  uint32_t* epoch_dev;                   // optional device-resident epoch (CUDA-graph replay), see below
  unsigned long long limit_ns;
  int* status;
};

__device__ __forceinline__ void tp_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tp_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t tp_ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void tp_fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ size_t tp_flag_index(int kind, int slot, int src, int n_slots) {
  return (static_cast<size_t>(kind) * n_slots + slot) * TP_MAX_RANKS + src;
}
// Bounded spin of ONE thread until *p >= want (acquire at the given scope).
template <bool SYS>
__device__ __forceinline__ bool tp_spin_ge(const uint32_t* p, uint32_t want, unsigned long long limit_ns,
                                           volatile int* abort_word, const int* status = nullptr) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t backoff = 32;
  while (static_cast<int32_t>((SYS ? tp_ld_acquire_sys(p) : tp_ld_acquire_gpu(p)) - want) < 0) {
    if (*abort_word) return false;
    // fail fast once any kernel on this device has reported a lost peer: later waits would only
    // repeat the same time-out one after the other
    if ((status && *reinterpret_cast<const volatile int*>(status) != 0) || globaltimer_ns() - t0 > limit_ns) {
      *abort_word = FT_ERR_TIMEOUT_PEER;
      return false;
    }
    __nanosleep(backoff);
    if (backoff < 512) backoff <<= 1;
  }
  return true;
}

// number of copy units (at most TP_UNIT_ROWS rows of one remote rank) in 128-row block mb
__device__ __forceinline__ int remote_units(int mb, int rows_per_rank, int M, int rank, int unit_rows) {
  const int lo = mb * TP_BM, hi = min(M, lo + TP_BM);
  int n = 0;
  for (int s = lo / rows_per_rank; s <= (hi - 1) / rows_per_rank; ++s) {
    if (s == rank) continue;
    const int r0 = max(lo, s * rows_per_rank), r1 = min(hi, (s + 1) * rows_per_rank);
    n += (r1 - r0 + unit_rows - 1) / unit_rows;
  }
  return n;
}

// All-gather by pull, one warp's share: the units are numbered in the order the GEMM consumes
// the 128-row blocks (starting at first_block) and unit u belongs to worker u % n_workers.  Each
// lane keeps 8 independent 16-byte peer loads in flight.  After a unit has landed the warp
// publishes it on the block counter (generic stores -> fence -> async-proxy readers).
__device__ __forceinline__ void tp_copy_units(const TpParams& p, int worker, int n_workers, uint32_t epoch,
                                              int first_block, int m_blocks, volatile int* abort_word) {
  const int lane = threadIdx.x & 31;
  const uint32_t* my_flags = static_cast<const uint32_t*>(p.flags.ptr[p.rank]);
  __nv_bfloat16* dst_base = static_cast<__nv_bfloat16*>(p.xg.ptr[p.rank]);
  const int vec_per_row = p.K >> 3;
  const int rpr = p.rows_per_rank;
  uint32_t seen = 0;
  int u = 0;
  for (int bi = 0; bi < m_blocks; ++bi) {
    const int mb = (first_block + bi) % m_blocks;
    const int lo = mb * TP_BM, hi = min(p.M, lo + TP_BM);
    for (int s = lo / rpr; s <= (hi - 1) / rpr; ++s) {
      if (s == p.rank) continue;
      const int r0 = max(lo, s * rpr), r1 = min(hi, (s + 1) * rpr);
      for (int ru = r0; ru < r1; ru += p.unit_rows, ++u) {
        if (u % n_workers != worker) continue;
        if (!((seen >> s) & 1u)) {
          int ok = 1;
          if (lane == 0)
            ok = tp_spin_ge<true>(my_flags + tp_flag_index(0, p.slot, s, p.n_slots), epoch, p.limit_ns, abort_word,
                                  p.status) ? 1 : 0;
          ok = __shfl_sync(0xffffffffu, ok, 0);
          if (!ok) return;
          seen |= 1u << s;
        }
        const __nv_bfloat16* src_base = static_cast<const __nv_bfloat16*>(p.xg.ptr[s]);
        const int total = min(p.unit_rows, r1 - ru) * vec_per_row;
        for (int v0 = lane; v0 < total; v0 += 32 * 8) {
          uint4 val[8];
          long long off[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int v = v0 + q * 32;
            const int vv = v < total ? v : v0;
            off[q] = static_cast<long long>(ru + vv / vec_per_row) * p.ldx + ((vv % vec_per_row) << 3);
            asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(val[q].x), "=r"(val[q].y), "=r"(val[q].z), "=r"(val[q].w)
                         : "l"(src_base + off[q]) : "memory");
          }
#pragma unroll
          for (int q = 0; q < 8; ++q)
            if (v0 + q * 32 < total) *reinterpret_cast<uint4*>(dst_base + off[q]) = val[q];
        }
        __threadfence();
        tp_fence_proxy_async();  // the consumers read these rows through TMA (async proxy)
        __syncwarp();
        if (lane == 0) atomicAdd(p.blk_ready + mb, 1u);
      }
    }
  }
}

// Last step of every CTA (one thread): report an abort, and in the last CTA to finish reset the
// local counters for the next launch and tell every peer that this rank no longer reads their
// buffers (mode 0) / has consumed its staging buffer (mode 1).
__device__ __forceinline__ void tp_finish(const TpParams& p, uint32_t epoch, int m_blocks, volatile int* abort_word) {
  if (*abort_word != 0 && p.status) atomicCAS(p.status, 0, *abort_word);
  __threadfence();
  const unsigned int done = atomicAdd(p.done_counter, 1u);
  if (done == gridDim.x - 1) {
    *p.done_counter = 0u;
    if (p.epoch_dev && p.mode == 1) *p.epoch_dev = epoch;
    if (p.mode == 0)
      for (int mb = 0; mb < m_blocks; ++mb) p.blk_ready[mb] = 0u;
    __threadfence_system();
    for (int r = 0; r < p.world; ++r)
      tp_st_release_sys(static_cast<uint32_t*>(p.flags.ptr[r]) + tp_flag_index(1, p.slot, p.rank, p.n_slots), epoch);
  }
}

// B_MN: the B operand is stored [K, N] (N contiguous) instead of [N, K]; its tiles are loaded as
// 64-column chunks and read through an MN-major descriptor, so the backward GEMMs (dY * W) use
// the weight as it is stored.
template <int BN, bool B_MN>
__global__ void __launch_bounds__(TP_THREADS, 1)
tp_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const TpParams p) {
  // With a device-resident epoch the value is read here instead of from the (frozen) argument:
  // mode 0 uses the value its signal kernel just published, mode 1 uses current + 1 and the
  // last CTA publishes it at the end.
  const uint32_t epoch = p.epoch_dev ? *p.epoch_dev + (p.mode == 1 ? 1u : 0u) : p.epoch;
  using Cfg = TpCfg<BN>;
  constexpr int STAGES = Cfg::STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t bar_base = smem_u32(bars);
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

  const int m_blocks = (p.M + TP_BM - 1) / TP_BM;
  const int n_blocks = (p.N + BN - 1) / BN;
  const int num_tiles = m_blocks * n_blocks;
  const int k_blocks = (p.K + TP_BK - 1) / TP_BK;
  const int n_gemm = static_cast<int>(gridDim.x);
  const int cta = static_cast<int>(blockIdx.x);
  uint32_t* my_flags = static_cast<uint32_t*>(p.flags.ptr[p.rank]);
  // rotation so that the rows this rank already holds (mode 0) come first and the rows this rank
  // owns (mode 1) come last
  const int own_block = (p.rank * p.rows_per_rank) / TP_BM;
  const int own_end_block = min(m_blocks, ((p.rank + 1) * p.rows_per_rank + TP_BM - 1) / TP_BM);
  const int first_block = p.mode == 0 ? own_block : (own_end_block % m_blocks);
  auto tile_coords = [&](int tile, int& mb, int& nb) {
    mb = (first_block + tile / n_blocks) % m_blocks;
    nb = tile % n_blocks;
  };

  if (threadIdx.x == 0) {
    *abort_word = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
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

  if (warp == 2 || warp == 3 || warp >= 8) {
    // ------------------------------------------------------------ all-gather by pull
    if (p.mode == 0 && p.world > 1) {
      const int w4 = warp >= 8 ? warp - 6 : warp - 2;   // 0..3
      tp_copy_units(p, cta * 4 + w4, n_gemm * 4, epoch, first_block, m_blocks, abort_word);
    }
  } else if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += n_gemm) {
        int mb, nb;
        tile_coords(tile, mb, nb);
        if (p.mode == 0) {
          const int need = p.world > 1 ? remote_units(mb, p.rows_per_rank, p.M, p.rank, p.unit_rows) : 0;
          if (need > 0) {
            if (!tp_spin_ge<false>(p.blk_ready + mb, static_cast<uint32_t>(need), p.limit_ns, abort_word, p.status)) break;
            tp_fence_proxy_async();
          }
        }
        const int m0 = mb * TP_BM, n0 = nb * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_word, FT_ERR_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES, sB = sA + Cfg::A_BYTES;
          mbar_expect_tx(full_bar(stage), Cfg::STAGE_BYTES);
          tma_load_2d(sA, &tmA, full_bar(stage), kb * TP_BK, m0);
          if constexpr (!B_MN) {
            tma_load_2d(sB, &tmB, full_bar(stage), kb * TP_BK, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c)
              tma_load_2d(sB + c * (TP_BK * 128), &tmB, full_bar(stage), n0 + c * 64, kb * TP_BK);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
      if (*abort_word) {
        const unsigned long long t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 2000000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t tmem_base = *tmem_slot;
      constexpr uint32_t idesc = make_idesc_f16(TP_BM, BN, 1, 0, B_MN ? 1 : 0);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = cta; tile < num_tiles && ok; tile += n_gemm) {
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_word, FT_ERR_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_word, FT_ERR_TIMEOUT_MMA)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_base + stage * Cfg::STAGE_BYTES, sB = sA + Cfg::A_BYTES;
#pragma unroll
          for (int k = 0; k < TP_BK / 16; ++k) {
            const uint64_t bdesc = B_MN ? make_smem_desc_sw128(sB + k * 2048, TP_BK * 128, 1024)
                                        : make_smem_desc_sw128(sB + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, make_smem_desc_sw128(sA + k * 32, 16, 1024), bdesc, idesc,
                        (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 4 && warp < 8) {
    // ------------------------------------------------------------ epilogue
    const uint32_t tmem_base = *tmem_slot;
    const int ew = warp & 3;
    const uint32_t epi_base = smem_base + Cfg::EPI_OFFSET + ew * (32 * TP_EPI_ROW);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    if (p.mode == 1 && epoch > 1) {
      // the owners must have finished reducing the previous use of their staging buffers
      if (lane < p.world)
        ok = tp_spin_ge<true>(my_flags + tp_flag_index(1, p.slot, lane, p.n_slots), epoch - 1, p.limit_ns, abort_word, p.status);
      ok = __all_sync(0xffffffffu, ok);
    }
    for (int tile = cta; tile < num_tiles && ok; tile += n_gemm) {
      int mb, nb;
      tile_coords(tile, mb, nb);
      const int m0 = mb * TP_BM, n0 = nb * BN;
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_word, FT_ERR_TIMEOUT_EPILOGUE)) { ok = false; break; }
      tc_fence_after();
      const int row = m0 + ew * 32 + lane;
      const bool row_ok = row < p.M;
      __nv_bfloat16* drow = nullptr;
      if (row_ok) {
        if (p.mode == 0) {
          drow = p.C + static_cast<long long>(row) * p.ldc;
        } else {
          const int owner = row / p.rows_per_rank, rl = row - owner * p.rows_per_rank;
          drow = static_cast<__nv_bfloat16*>(p.stage.ptr[owner]) +
                 (static_cast<long long>(p.rank) * p.rows_per_rank + rl) * p.N;
        }
      }
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(ew * 32) << 16) + static_cast<uint32_t>(acc * BN);
      const unsigned long long drow_bits = reinterpret_cast<unsigned long long>(drow);  // 0 for rows past M
      const int seg = lane & 7, rsub = lane >> 3;
#pragma unroll 1
      for (int c2 = 0; c2 < BN / 64; ++c2) {
        // stage a 32-row x 64-column piece: each lane converts its own row ...
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32(t_row + (c2 * 2 + h) * 32, r);
          tmem_ld_wait();
          const int col0 = n0 + (c2 * 2 + h) * 32;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[g * 8 + j]);
            if (p.mode == 0 && p.bias && col0 + g * 8 + 8 <= p.N) {
              const uint4 bb = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.bias) + col0 + g * 8);
              const float2 b0 = unpack_bf16x2(bb.x), b1 = unpack_bf16x2(bb.y), b2 = unpack_bf16x2(bb.z), b3 = unpack_bf16x2(bb.w);
              v[0] += b0.x; v[1] += b0.y; v[2] += b1.x; v[3] += b1.y; v[4] += b2.x; v[5] += b2.y; v[6] += b3.x; v[7] += b3.y;
            }
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(epi_base + lane * TP_EPI_ROW + h * 64 + g * 16),
                         "r"(pack_bf16x2(v[0], v[1])), "r"(pack_bf16x2(v[2], v[3])), "r"(pack_bf16x2(v[4], v[5])),
                         "r"(pack_bf16x2(v[6], v[7])) : "memory");
          }
        }
        __syncwarp();
        // ... and the warp writes it out as 128-byte row segments (8 lanes per row, 4 rows per store)
        const int colx = n0 + c2 * 64 + seg * 8;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + rsub;
          uint4 o;
          asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                       : "r"(epi_base + rr * TP_EPI_ROW + seg * 16) : "memory");
          const unsigned long long dp = __shfl_sync(0xffffffffu, drow_bits, rr);
          if (dp != 0ull && colx + 8 <= p.N) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dp) + colx) = o;
        }
        __syncwarp();
      }
      tc_fence_before();
      if (p.mode == 1) {
        // account this warp's share of the tile towards every owner the tile overlaps; the last
        // contribution for an owner raises this source's flag on that owner
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int o0 = m0 / p.rows_per_rank, o1 = (min(p.M, m0 + TP_BM) - 1) / p.rows_per_rank;
          for (int o = o0; o <= o1; ++o) {
            const int blk0 = (o * p.rows_per_rank) / TP_BM;
            const int blk1 = (min(p.M, (o + 1) * p.rows_per_rank) - 1) / TP_BM;
            const unsigned int expected = static_cast<unsigned int>((blk1 - blk0 + 1) * n_blocks * 4);
            const unsigned int v = atomicAdd(p.owner_counter + o, 1u);
            if (v + 1 == expected) {
              p.owner_counter[o] = 0u;
              __threadfence_system();
              tp_st_release_sys(static_cast<uint32_t*>(p.flags.ptr[o]) + tp_flag_index(0, p.slot, p.rank, p.n_slots), epoch);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  if (p.mode == 1) {
    // ---------------------------------------------------------- reduce the staged partials
    // Every role of this CTA has run out of tiles (or aborted); all ten warps now sum this
    // rank's rows over the sources in rank order, four 16-byte vectors per thread in flight
    // from each source.
    __syncthreads();
    // a rank past the last row (M < (rank + 1) * rows_per_rank with nothing left for it) owns
    // nothing: no source will ever raise its flag, so it must not wait for one
    const int rows = min(p.rows_per_rank, p.M - p.rank * p.rows_per_rank);
    bool ok = (*abort_word == 0) && rows > 0;
    if (ok && lane < p.world)
      ok = tp_spin_ge<true>(my_flags + tp_flag_index(0, p.slot, lane, p.n_slots), epoch, p.limit_ns, abort_word, p.status);
    ok = __all_sync(0xffffffffu, ok);
    if (ok) {
      const __nv_bfloat16* st = static_cast<const __nv_bfloat16*>(p.stage.ptr[p.rank]);
      const int vec_per_row = p.N >> 3;
      const long long total = static_cast<long long>(rows > 0 ? rows : 0) * vec_per_row;
      const long long slot_stride = static_cast<long long>(p.rows_per_rank) * p.N;
      const long long stride = static_cast<long long>(n_gemm) * TP_THREADS;
      for (long long v0 = static_cast<long long>(cta) * TP_THREADS + threadIdx.x; v0 < total; v0 += 4 * stride) {
        float acc8[4][8];
        int rr[4], cc[4];
        bool valid[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const long long v = v0 + j * stride;
          valid[j] = v < total;
          const long long vv = valid[j] ? v : v0;
          rr[j] = static_cast<int>(vv / vec_per_row);
          cc[j] = static_cast<int>(vv % vec_per_row) << 3;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc8[j][e] = 0.f;
        }
        for (int s = 0; s < p.world; ++s) {
          uint4 x[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(x[j].x), "=r"(x[j].y), "=r"(x[j].z), "=r"(x[j].w)
                         : "l"(st + s * slot_stride + static_cast<long long>(rr[j]) * p.N + cc[j]) : "memory");
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f0 = unpack_bf16x2(x[j].x), f1 = unpack_bf16x2(x[j].y), f2 = unpack_bf16x2(x[j].z), f3 = unpack_bf16x2(x[j].w);
            acc8[j][0] += f0.x; acc8[j][1] += f0.y; acc8[j][2] += f1.x; acc8[j][3] += f1.y;
            acc8[j][4] += f2.x; acc8[j][5] += f2.y; acc8[j][6] += f3.x; acc8[j][7] += f3.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (!valid[j]) continue;
          if (p.residual) {
            const uint4 x = *reinterpret_cast<const uint4*>(p.residual + static_cast<long long>(rr[j]) * p.ldr + cc[j]);
            const float2 f0 = unpack_bf16x2(x.x), f1 = unpack_bf16x2(x.y), f2 = unpack_bf16x2(x.z), f3 = unpack_bf16x2(x.w);
            acc8[j][0] += f0.x; acc8[j][1] += f0.y; acc8[j][2] += f1.x; acc8[j][3] += f1.y;
            acc8[j][4] += f2.x; acc8[j][5] += f2.y; acc8[j][6] += f3.x; acc8[j][7] += f3.y;
          }
          uint4 o;
          o.x = pack_bf16x2(acc8[j][0], acc8[j][1]); o.y = pack_bf16x2(acc8[j][2], acc8[j][3]);
          o.z = pack_bf16x2(acc8[j][4], acc8[j][5]); o.w = pack_bf16x2(acc8[j][6], acc8[j][7]);
          *reinterpret_cast<uint4*>(p.out + static_cast<long long>(rr[j]) * p.ldo + cc[j]) = o;
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(*tmem_slot, Cfg::TMEM_COLS);
  }
  if (threadIdx.x == 0) tp_finish(p, epoch, m_blocks, abort_word);
}

// The all-gather alone (no GEMM consumer): every warp of a small grid is a copy worker.  Uses
// next to no shared memory, so it runs beside a GEMM kernel on the same SMs.
__global__ void __launch_bounds__(256) tp_gather_kernel(const TpParams p) {
  __shared__ int s_abort;
  const uint32_t epoch = p.epoch_dev ? *p.epoch_dev : p.epoch;
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  const int m_blocks = (p.M + TP_BM - 1) / TP_BM;
  const int own_block = (p.rank * p.rows_per_rank) / TP_BM;
  tp_copy_units(p, static_cast<int>(blockIdx.x) * 8 + static_cast<int>(threadIdx.x >> 5),
                static_cast<int>(gridDim.x) * 8, epoch, own_block, m_blocks, &s_abort);
  __syncthreads();
  if (threadIdx.x == 0) tp_finish(p, epoch, m_blocks, &s_abort);
}

template <int BN, bool B_MN>
static int launch_tp(const CUtensorMap& tmA, const CUtensorMap& tmB, const TpParams& p, int device, int ctas,
                     cudaStream_t stream) {
  using Cfg = TpCfg<BN>;
  auto kern = tp_gemm_kernel<BN, B_MN>;
  static bool attr_set[64] = {false};
  if (!attr_set[device]) {
    FT_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
    attr_set[device] = true;
  }
  kern<<<ctas, TP_THREADS, Cfg::SMEM_BYTES, stream>>>(tmA, tmB, p);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}

static int dispatch_tp(int bn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB, const TpParams& p,
                       int device, int ctas, cudaStream_t stream) {
  if (!b_mn) {
    switch (bn) {
      case 256: return launch_tp<256, false>(tmA, tmB, p, device, ctas, stream);
      case 128: return launch_tp<128, false>(tmA, tmB, p, device, ctas, stream);
      default: return launch_tp<64, false>(tmA, tmB, p, device, ctas, stream);
    }
  }
  switch (bn) {
    case 256: return launch_tp<256, true>(tmA, tmB, p, device, ctas, stream);
    case 128: return launch_tp<128, true>(tmA, tmB, p, device, ctas, stream);
    default: return launch_tp<64, true>(tmA, tmB, p, device, ctas, stream);
  }
}

static int pick_bn(int M, int N, int sms) {
  const long long mb = (M + TP_BM - 1) / TP_BM;
  int bn = 256;
  while (bn > 64 && mb * ((N + bn - 1) / bn) < sms) bn >>= 1;
  return bn;
}

static int fill_peers(TpPeers& t, void* const* ptrs, int world) {
  for (int i = 0; i < TP_MAX_RANKS; ++i) t.ptr[i] = (ptrs && i < world) ? ptrs[i] : nullptr;
  if (!ptrs) return FT_E_BAD_ARG;
  for (int i = 0; i < world; ++i)
    if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 15)) return FT_E_BAD_ARG;
  return FT_E_OK;
}

}  // namespace ft

using namespace ft;

// Scratch words (uint32) the TP kernels need locally: counters[0] = done counter,
// counters[1 .. 1+8) = owner counters, counters[16 ...) = per-128-row-block counters.
FT_API long long ft_tp_counter_words(int M) { return 16 + (M + TP_BM - 1) / TP_BM; }

// Y[M, N] = allgather_rows(Xg)[M, K] * B (+ bias), where B is W[N, K]^T (b_mn_major = 0, row
// stride ldw) or W stored as [K, N] (b_mn_major = 1).  xg_ptrs: every rank's symmetric [M, K]
// buffer (row stride ldx); this rank's rows [rank*rows_per_rank, ...) must already be in its own
// buffer and every rank must have raised flag (kind 0, slot) after writing them
// (ft_comm_signal / ft_comm_signal_dev).  counters: ft_tp_counter_words(M) zeroed uint32 words,
// reused across calls.  The kernel raises flag (kind 1, slot) on every peer when it no longer
// reads their buffers.  With w == NULL only the gather runs (copy CTAs alone): afterwards the
// local buffer holds all M rows.
FT_API int ft_tp_ag_gemm2(void* const* xg_ptrs, const void* w, void* y, const void* bias, int M, int N, int K,
                          long long ldx, long long ldw, long long ldy, int b_mn_major, int rank, int world,
                          int rows_per_rank, unsigned int* counters, void* const* flag_ptrs, int slot,
                          int n_slots, unsigned int epoch, unsigned int* epoch_dev, int n_copy,
                          long long timeout_ms, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  const bool gather_only = (w == nullptr);
  FT_REQUIRE(world >= 1 && world <= TP_MAX_RANKS && rank >= 0 && rank < world, "ft_tp_ag_gemm: bad rank/world");
  FT_REQUIRE(M > 0 && K > 0 && K % 8 == 0 && ldx % 8 == 0, "ft_tp_ag_gemm: K and ldx must be multiples of 8");
  FT_REQUIRE(gather_only || (N > 0 && N % 8 == 0 && ldw % 8 == 0 && ldy % 8 == 0 && y),
             "ft_tp_ag_gemm: N and strides must be multiples of 8");
  FT_REQUIRE(rows_per_rank > 0 && rows_per_rank * world >= M, "ft_tp_ag_gemm: rows_per_rank * world < M");
  FT_REQUIRE(counters, "ft_tp_ag_gemm: null pointer");
  if (gather_only && world == 1) return FT_E_OK;
  TpParams p{};
  FT_REQUIRE(fill_peers(p.xg, xg_ptrs, world) == 0 && fill_peers(p.flags, flag_ptrs, world) == 0,
             "ft_tp_ag_gemm: bad peer pointers");
  for (int i = 0; i < TP_MAX_RANKS; ++i) p.stage.ptr[i] = nullptr;
  const int sms = sm_count(device);
  if (n_copy <= 0) n_copy = 32;
  if (n_copy > sms) n_copy = sms;
  if (gather_only) N = 0;
  p.mode = 0; p.M = M; p.N = N; p.K = K; p.rank = rank; p.world = world; p.rows_per_rank = rows_per_rank;
  p.C = static_cast<__nv_bfloat16*>(y); p.ldc = ldy; p.bias = bias; p.ldx = ldx;
  p.blk_ready = counters + 16; p.n_copy = n_copy; p.done_counter = counters; p.owner_counter = counters + 1;
  p.slot = slot; p.n_slots = n_slots; p.epoch = epoch; p.epoch_dev = epoch_dev;
  p.limit_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 20000) * 1000000ull;
  p.status = device_status_word(device);
  // small problems (decode) get smaller copy units so that every copy warp has work
  auto pick_unit = [&](int workers) {
    const int remote_rows = M - (M < rows_per_rank ? M : rows_per_rank);
    int ur = TP_UNIT_ROWS;
    while (ur > 1 && remote_rows / ur < workers) ur >>= 1;
    return ur;
  };
  if (gather_only) {
    p.unit_rows = pick_unit(n_copy * 8);
    tp_gather_kernel<<<n_copy, 256, 0, stream>>>(p);
    FT_CUDA_CHECK(cudaGetLastError());
    count_launch();
    return FT_E_OK;
  }
  const int bn = pick_bn(M, N, sms);
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, xg_ptrs[rank], 2, K, M, ldx * 2, TP_BK, TP_BM, 3);
  if (rc) return rc;
  if (!b_mn_major)
    rc = make_tmap_2d(&tmB, w, 2, K, N, ldw * 2, TP_BK, bn, 3);
  else
    rc = make_tmap_2d(&tmB, w, 2, N, K, ldw * 2, 64, TP_BK, 3);
  if (rc) return rc;
  const int tiles = ((M + TP_BM - 1) / TP_BM) * ((N + bn - 1) / bn);
  const int ctas = tiles < sms ? tiles : sms;
  p.unit_rows = pick_unit(ctas * 4);
  return dispatch_tp(bn, b_mn_major != 0, tmA, tmB, p, device, ctas, stream);
}

FT_API int ft_tp_ag_gemm(void* const* xg_ptrs, const void* w, void* y, const void* bias, int M, int N, int K,
                         long long ldx, long long ldw, long long ldy, int rank, int world, int rows_per_rank,
                         unsigned int* counters, void* const* flag_ptrs, int slot, int n_slots,
                         unsigned int epoch, unsigned int* epoch_dev, int n_copy, long long timeout_ms,
                         int device, cudaStream_t stream) {
  FT_REQUIRE(w != nullptr, "ft_tp_ag_gemm: null weight");
  return ft_tp_ag_gemm2(xg_ptrs, w, y, bias, M, N, K, ldx, ldw, ldy, 0, rank, world, rows_per_rank, counters,
                        flag_ptrs, slot, n_slots, epoch, epoch_dev, n_copy, timeout_ms, device, stream);
}

// Out[rows_per_rank, N] (+ residual) = reduce_scatter_rows(X[M, K] * B) over ranks, B as in
// ft_tp_ag_gemm2.  stage_ptrs: every rank's symmetric staging buffer of
// world * rows_per_rank * N bf16.  out / residual are local [rows_per_rank, N] (row strides
// ldo / ldr).  max_ctas > 0 limits the grid (leaves SMs to a concurrent gather).
FT_API int ft_tp_gemm_rs2(const void* x, const void* w, void* const* stage_ptrs, void* out, const void* residual,
                          int M, int N, int K, long long ldx, long long ldw, long long ldo, long long ldr,
                          int b_mn_major, int max_ctas, int rank, int world, int rows_per_rank,
                          unsigned int* counters, void* const* flag_ptrs, int slot, int n_slots,
                          unsigned int epoch, unsigned int* epoch_dev, long long timeout_ms, int device,
                          cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(world >= 1 && world <= TP_MAX_RANKS && rank >= 0 && rank < world, "ft_tp_gemm_rs: bad rank/world");
  FT_REQUIRE(M > 0 && N > 0 && K > 0 && N % 8 == 0 && K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0 && ldo % 8 == 0 &&
                 ldr % 8 == 0,
             "ft_tp_gemm_rs: N, K and strides must be multiples of 8");
  FT_REQUIRE(rows_per_rank > 0 && rows_per_rank * world >= M, "ft_tp_gemm_rs: rows_per_rank * world < M");
  // a rank that owns no rows (M < rank * rows_per_rank, e.g. a decode batch smaller than the group)
  // passes an empty output: it still computes and sends its partial products
  FT_REQUIRE(counters && x && w && (out || M <= rank * rows_per_rank), "ft_tp_gemm_rs: null pointer");
  TpParams p{};
  FT_REQUIRE(fill_peers(p.stage, stage_ptrs, world) == 0 && fill_peers(p.flags, flag_ptrs, world) == 0,
             "ft_tp_gemm_rs: bad peer pointers");
  for (int i = 0; i < TP_MAX_RANKS; ++i) p.xg.ptr[i] = nullptr;
  int sms = sm_count(device);
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  p.mode = 1; p.M = M; p.N = N; p.K = K; p.rank = rank; p.world = world; p.rows_per_rank = rows_per_rank;
  p.out = static_cast<__nv_bfloat16*>(out); p.ldo = ldo;
  p.residual = static_cast<const __nv_bfloat16*>(residual); p.ldr = ldr;
  p.done_counter = counters; p.owner_counter = counters + 1; p.blk_ready = counters + 16; p.n_copy = 0;
  p.unit_rows = TP_UNIT_ROWS;
  p.slot = slot; p.n_slots = n_slots; p.epoch = epoch; p.epoch_dev = epoch_dev;
  p.limit_ns = static_cast<unsigned long long>(timeout_ms > 0 ? timeout_ms : 20000) * 1000000ull;
  p.status = device_status_word(device);
  const int bn = pick_bn(M, N, sms);
  CUtensorMap tmA, tmB;
  int rc = make_tmap_2d(&tmA, x, 2, K, M, ldx * 2, TP_BK, TP_BM, 3);
  if (rc) return rc;
  if (!b_mn_major)
    rc = make_tmap_2d(&tmB, w, 2, K, N, ldw * 2, TP_BK, bn, 3);
  else
    rc = make_tmap_2d(&tmB, w, 2, N, K, ldw * 2, 64, TP_BK, 3);
  if (rc) return rc;
  const int tiles = ((M + TP_BM - 1) / TP_BM) * ((N + bn - 1) / bn);
  const int ctas = tiles < sms ? tiles : sms;
  return dispatch_tp(bn, b_mn_major != 0, tmA, tmB, p, device, ctas, stream);
}

FT_API int ft_tp_gemm_rs(const void* x, const void* w, void* const* stage_ptrs, void* out, const void* residual,
                         int M, int N, int K, long long ldx, long long ldw, long long ldo, long long ldr,
                         int rank, int world, int rows_per_rank, unsigned int* counters,
                         void* const* flag_ptrs, int slot, int n_slots, unsigned int epoch,
                         unsigned int* epoch_dev, long long timeout_ms, int device, cudaStream_t stream) {
  return ft_tp_gemm_rs2(x, w, stage_ptrs, out, residual, M, N, K, ldx, ldw, ldo, ldr, 0, 0, rank, world,
                        rows_per_rank, counters, flag_ptrs, slot, n_slots, epoch, epoch_dev, timeout_ms, device,
                        stream);
}
