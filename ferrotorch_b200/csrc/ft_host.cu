// Implementation of the host-side helpers declared in ft_host.h.
#include "ft_host.h"

#include <cstdlib>

#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

namespace ft {

static std::atomic<long long> g_launches{0};
static thread_local char g_err[512] = {0};

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

const char* set_last_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return g_err;
}

static std::mutex g_mu;
static int* g_status[64] = {nullptr};
static int g_sms[64] = {0};

// The status words live in a file-scope device array, so no allocation is needed;
// each device that loads the library holds its own 256-byte copy.
__device__ int g_dev_status[64];

int* device_status_word(int device) {
  if (device < 0 || device >= 64) return nullptr;
  std::lock_guard<std::mutex> lk(g_mu);
  if (!g_status[device]) {
    int prev = 0;
    cudaGetDevice(&prev);
    if (prev != device) cudaSetDevice(device);
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_dev_status) == cudaSuccess) g_status[device] = static_cast<int*>(p);
    if (prev != device) cudaSetDevice(prev);
  }
  return g_status[device];
}

int ensure_device(int device) {
  // Ask the runtime every time: torch (or the caller) may have switched devices since the last
  // call, so a cached value could launch on the wrong GPU.  cudaGetDevice is a host-only query.
  int cur = -1;
  if (cudaGetDevice(&cur) == cudaSuccess && cur == device) {
    static thread_local unsigned long long bound = 0;  // devices whose context this thread has touched
    if (device >= 0 && device < 64 && !((bound >> device) & 1ull)) {
      cudaFree(0);  // binds the primary context to this thread (worker threads start without one)
      bound |= 1ull << device;
    }
    return FT_E_OK;
  }
  if (cudaSetDevice(device) != cudaSuccess) {
    set_last_error("cudaSetDevice(%d) failed", device);
    return FT_E_CUDA;
  }
  cudaFree(0);
  return FT_E_OK;
}

int sm_count(int device) {
  if (device < 0 || device >= 64) return 148;
  if (!g_sms[device]) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || v <= 0)
      v = 148;
    g_sms[device] = v;
  }
  return g_sms[device];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

static CUtensorMapDataType dt_of(int bytes, bool is_bf16) {
  if (bytes == 1) return CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (bytes == 2) return is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
}

static int encode(CUtensorMap* out, const void* base, int dtype_bytes, int rank, const cuuint64_t* dims,
                  const cuuint64_t* strides, const cuuint32_t* box, int swizzle, bool is_bf16) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_last_error("cuTensorMapEncodeTiled is not available (no CUDA driver)");
    return FT_E_NO_DRIVER;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    set_last_error("TMA base address %p is not 16-byte aligned", base);
    return FT_E_BAD_ARG;
  }
  for (int i = 0; i + 1 < rank; ++i)
    if (strides[i] % 16 != 0) {
      set_last_error("TMA stride %d (%llu bytes) is not a multiple of 16", i,
                     (unsigned long long)strides[i]);
      return FT_E_BAD_ARG;
    }
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  CUresult r = fn(out, dt_of(dtype_bytes, is_bf16), rank, const_cast<void*>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(swizzle),
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_last_error("cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return FT_E_CUDA;
  }
  return FT_E_OK;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t inner, uint64_t outer,
                 uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle,
                 bool is_bf16) {
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  return encode(out, base, dtype_bytes, 2, dims, strides, box, swizzle, is_bf16);
}
int make_tmap_3d(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t s1, uint64_t s2, uint32_t b0, uint32_t b1, uint32_t b2,
                 int swizzle, bool is_bf16) {
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {b0, b1, b2};
  return encode(out, base, dtype_bytes, 3, dims, strides, box, swizzle, is_bf16);
}
int make_tmap_4d(CUtensorMap* out, const void* base, int dtype_bytes, uint64_t d0, uint64_t d1,
                 uint64_t d2, uint64_t d3, uint64_t s1, uint64_t s2, uint64_t s3, uint32_t b0,
                 uint32_t b1, uint32_t b2, uint32_t b3, int swizzle, bool is_bf16) {
  cuuint64_t dims[4] = {d0, d1, d2, d3};
  cuuint64_t strides[3] = {s1, s2, s3};
  cuuint32_t box[4] = {b0, b1, b2, b3};
  return encode(out, base, dtype_bytes, 4, dims, strides, box, swizzle, is_bf16);
}

}  // namespace ft

// Number of kernels this library has launched since load (monotonic).
FT_API long long ft_launch_count() { return ft::g_launches.load(std::memory_order_relaxed); }

// Text of the last error raised on the calling thread.
FT_API const char* ft_last_error() { return ft::g_err; }

// Read and clear the device status word (synchronises the device). 0 = no kernel
// reported an error since the last call.
FT_API int ft_read_device_status(int device) {
  int* p = ft::device_status_word(device);
  if (!p) return 0;
  int v = 0;
  if (cudaMemcpy(&v, p, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return ft::FT_E_CUDA;
  if (v != 0) cudaMemset(p, 0, sizeof(int));
  return v;
}

FT_API int ft_abi_version() { return 1; }

// Kernels this library's JIT compiles at run time are launched through the driver API from
// Python; they report their launches here so ft_launch_count() covers them too.
FT_API void ft_count_external_launch(int n) { ft::count_launch(n); }
