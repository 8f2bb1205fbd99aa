// Entry points that never allocate.  (This header has no counterpart in the reference; it
// exists for embedders of this library, see below.)
//
// Most launchers in this library take their scratch memory from the caller, and the Python
// front end gets it from PyTorch's caching allocator.  Some callers cannot do either: code
// that runs inside a memory-pool callback, an out-of-memory handler that must still be able
// to run a kernel, and real-time or embedded hosts whose memory budget is fixed at start-up.  For them, calling cudaMalloc / cudaFree (or
// any routine that might) is either an error or an unbounded stall.
//
// ft_rmsnorm_bwd_noalloc is the RMSNorm backward of ft_rmsnorm_bwd with its partial-sum
// scratch taken from a fixed array that is part of the library image:
//
//   * Limit: hidden size H <= FT_NOALLOC_RMSNORM_MAX_H (8192), H a multiple of 8.  Any number of
//     rows.  Larger H is rejected with an error (code FT_E_TOO_LARGE, text in ft_last_error()).
//   * Cost: FT_NOALLOC_RMSNORM_ROWS * FT_NOALLOC_RMSNORM_MAX_H floats = 4 MiB of device memory on
//     every GPU that loads the library, held until the process exits.
//   * `device` must be the calling thread's current CUDA device (cudaGetDevice() == device);
//     otherwise the call fails with FT_E_BAD_ARG and launches nothing.  The entry point never
//     switches devices itself.
//   * The first call on a device looks up the array's device address (once per device, with
//     that device current).  Make that first call outside any stream capture; later calls only
//     launch kernels.
//   * The array is shared by all calls and keeps whatever the previous call left in it.  This
//     entry point overwrites every element it later reads, so nothing has to be cleared, but
//     two calls whose kernels overlap on the GPU (different streams, no ordering between them)
//     race on it: order them with an event or use ft_rmsnorm_bwd with separate scratch.
//   * It calls no cudaMalloc, cudaFree or allocating library routine.  Inputs and outputs are
//     still the caller's: dy, x, dx are bf16 [rows, H]; w bf16 [H]; rstd fp32 [rows] from the
//     forward; dres optional bf16 [rows, H] added to dx; dw bf16 or fp32 [H]
//     (dw_flags bit 0: fp32, bit 1: accumulate into dw).
#pragma once
#include <cuda_runtime.h>

#define FT_NOALLOC_RMSNORM_MAX_H 8192
#define FT_NOALLOC_RMSNORM_ROWS 128

extern "C" int ft_rmsnorm_bwd_noalloc(const void* dy, const void* x, const void* w, const float* rstd,
                                      const void* dres, void* dx, void* dw, int rows, int H, int dw_flags,
                                      int device, cudaStream_t stream);
