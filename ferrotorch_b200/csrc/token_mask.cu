// Grammar-constrained decoding on the device: logits[b, v] = -inf where bit v of row b's packed
// mask is clear.  The mask travels as 32 ids per little-endian word (16 KB for a 128 k vocabulary)
// instead of a byte per id.  The reference applies its masks with a CubeCL kernel
// (ferrotorch-cubecl/src/quant.rs:1417 kernel_apply_token_mask); this is the sm_100a counterpart,
// a plain grid-stride kernel bound by the logits' memory traffic.
#include <cuda_bf16.h>

#include "ft_host.h"

namespace ft {

template <typename T>
__global__ void __launch_bounds__(256) apply_token_mask_kernel(T* __restrict__ logits, const uint32_t* __restrict__ mask,
                                                               long long rows, long long vocab, long long ld,
                                                               long long words_per_row, T neg_inf) {
  const long long total = rows * vocab;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / vocab, v = i - r * vocab;
    const uint32_t w = mask[r * words_per_row + (v >> 5)];
    if (!((w >> (v & 31)) & 1u)) logits[r * ld + v] = neg_inf;
  }
}

}  // namespace ft

using namespace ft;

// logits: [rows, vocab] bf16 (is_f32 = 0) or fp32, row stride ld elements; mask: int32/uint32
// [rows, ceil(vocab / 32)] (or one row shared by all when mask_rows == 1).  In place.
FT_API int ft_apply_token_mask(void* logits, const void* mask, long long rows, long long vocab, long long ld,
                               int mask_rows, int is_f32, int device, cudaStream_t stream) {
  if (int _rc = ft::ensure_device(device)) return _rc;
  FT_REQUIRE(logits && mask, "ft_apply_token_mask: null pointer");
  FT_REQUIRE(rows >= 0 && vocab > 0 && ld >= vocab && (mask_rows == 1 || mask_rows == rows),
             "ft_apply_token_mask: bad shape");
  if (rows == 0) return FT_E_OK;
  const long long words = (vocab + 31) / 32;
  const long long total = rows * vocab;
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count(device)) * 8;
  if (blocks > cap) blocks = cap;
  const long long stride = mask_rows == 1 ? 0 : words;
  if (is_f32)
    apply_token_mask_kernel<float><<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<float*>(logits), static_cast<const uint32_t*>(mask), rows, vocab, ld, stride, -INFINITY);
  else
    apply_token_mask_kernel<__nv_bfloat16><<<static_cast<int>(blocks), 256, 0, stream>>>(
        static_cast<__nv_bfloat16*>(logits), static_cast<const uint32_t*>(mask), rows, vocab, ld, stride,
        __float2bfloat16(-INFINITY));
  FT_CUDA_CHECK(cudaGetLastError());
  count_launch();
  return FT_E_OK;
}
