// Host-side helpers shared by every translation unit of libft_kernels.so:
//   * launch accounting (ft_launch_count) so callers can report how many kernels of
//     this library ran inside a timed region;
//   * a per-device status word that kernels write error codes to (bounded waits);
//   * TMA tensor-map creation through the driver entry point, resolved at run time
//     so that the library also loads on a machine without libcuda.so (build hosts).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define FT_API extern "C" __attribute__((visibility("default")))

namespace ft {

// Host error codes returned by the extern "C" entry points (0 = success).
enum : int {
  FT_E_OK = 0,
  FT_E_BAD_ARG = -1,
  FT_E_CUDA = -2,
  FT_E_NO_DRIVER = -3,
  FT_E_TOO_LARGE = -4,
  FT_E_DEVICE_STATUS = -5,
};

void count_launch(int n = 1);
const char* set_last_error(const char* fmt, ...);

// Device status word (one int per device, zero-initialised, lives until exit).
// Kernels with bounded waits atomically store their error code here.
int* device_status_word(int device);

// Encode a 2-D tiled tensor map.  `inner`/`outer` are extents in elements,
// `row_stride_bytes` the stride of the outer dimension, box = {box_inner, box_outer}.
// swizzle: 0 none, 1 32B, 2 64B, 3 128B (CUtensorMapSwizzle numbering).
// dtype_bytes: 2 (bf16) or 4 (fp32) or 1 (u8).
int make_tmap_2d(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle,
                 bool is_bf16 = true);
int make_tmap_3d(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t stride1_bytes, uint64_t stride2_bytes, uint32_t b0, uint32_t b1,
                 uint32_t b2, int swizzle, bool is_bf16 = true);
int make_tmap_4d(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0,
                 uint32_t b1, uint32_t b2, uint32_t b3, int swizzle, bool is_bf16 = true);

int sm_count(int device);

// Make `device` current for this library's CUDA runtime on the calling thread (checked against
// cudaGetDevice on every call, never cached).  Needed because worker threads (e.g. an autograd engine thread) start with no
// CUDA context bound, and driver entry points such as the tensor-map encoder require one.
int ensure_device(int device);

#define FT_CUDA_CHECK(expr)                                                        \
  do {                                                                             \
    cudaError_t _e = (expr);                                                       \
    if (_e != cudaSuccess) {                                                       \
      ft::set_last_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                         __FILE__, __LINE__);                                      \
      return ft::FT_E_CUDA;                                                        \
    }                                                                              \
  } while (0)

#define FT_REQUIRE(cond, ...)                    \
  do {                                           \
    if (!(cond)) {                               \
      ft::set_last_error(__VA_ARGS__);           \
      return ft::FT_E_BAD_ARG;                   \
    }                                            \
  } while (0)

}  // namespace ft
