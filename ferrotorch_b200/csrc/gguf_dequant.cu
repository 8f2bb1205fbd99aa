// GGML quantised blocks -> bf16 / fp32 on the device (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1).
//
// The reference dequantises on the GPU with one CubeCL kernel per format, then copies the f32
// result to the host and back as bf16 (ferrotorch-cubecl/src/quant.rs:348-850, ferrotorch-llama/
// src/gpu_gguf.rs:14-27).  Here the raw blocks are uploaded once (0.56 - 1.06 bytes per element) and
// expanded in place on the device to the dtype the model runs in; the arithmetic is the header
// shared with the host reader (gguf_blocks.h), so host and device agree bit for bit in fp32.
// Q4_0 matrices that feed a linear layer need not be expanded at all (quant_gemm.cu).
//
// One thread decodes the element pair (i, i + 16) of a block; 16 consecutive threads share a block.
#include <cuda_bf16.h>

#include "ft_host.h"
#include "gguf_blocks.h"

namespace ft {

__device__ __forceinline__ void store(float* p, float v) { *p = v; }
__device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <typename OUT>
__global__ void __launch_bounds__(256)
gguf_dequant_kernel(const uint8_t* __restrict__ blocks, OUT* __restrict__ out, long long n_blocks, unsigned type, int bb) {
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long t = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; t < n_blocks * 16; t += stride) {
    const long long b = t >> 4;
    const int i = static_cast<int>(t & 15);
    float lo, hi;
    gguf_decode_pair(type, blocks + b * bb, i, lo, hi);
    store(out + b * 32 + i, lo);
    store(out + b * 32 + i + 16, hi);
  }
}

}  // namespace ft

using namespace ft;

// out[n_blocks * 32] (bf16 when out_f32 == 0) = dequantised blocks of GGML type `type`.
FT_API int ft_gguf_dequantize(const void* blocks, void* out, long long n_blocks, int type, int out_f32, int device,
                              cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(blocks && out && n_blocks >= 0, "ft_gguf_dequantize: null pointer or negative count");
  const int bb = gguf_block_bytes(static_cast<unsigned>(type));
  FT_REQUIRE(bb > 0, "ft_gguf_dequantize: type must be Q4_0, Q4_1, Q5_0, Q5_1, Q8_0 or Q8_1");
  if (n_blocks == 0) return FT_E_OK;
  const long long threads = n_blocks * 16;
  long long grid = (threads + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 16;
  if (grid > cap) grid = cap;
  if (out_f32)
    gguf_dequant_kernel<float><<<static_cast<int>(grid), 256, 0, stream>>>(static_cast<const uint8_t*>(blocks),
                                                                            static_cast<float*>(out), n_blocks,
                                                                            static_cast<unsigned>(type), bb);
  else
    gguf_dequant_kernel<__nv_bfloat16><<<static_cast<int>(grid), 256, 0, stream>>>(
        static_cast<const uint8_t*>(blocks), static_cast<__nv_bfloat16*>(out), n_blocks, static_cast<unsigned>(type), bb);
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}
