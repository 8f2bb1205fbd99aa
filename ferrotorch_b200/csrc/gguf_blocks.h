// Element decoding of GGML quantised blocks, shared by the host reader (csrc/host/gguf.cpp) and the
// device dequantiser (csrc/gguf_dequant.cu) so that both run literally the same arithmetic.
//
// A block holds 32 elements.  gguf_decode_pair(type, block, i, lo, hi) yields elements i and
// i + 16 (i in 0..15): for the nibble formats those are the low and the high nibble of byte i,
// for Q8_0 / Q8_1 simply bytes i and i + 16.  Layouts (ferrotorch-serialize/src/gguf.rs:543-700):
//   Q4_0 18 B: d f16, 16 nibble bytes            value = (q - 8) d
//   Q4_1 20 B: d f16, m f16, 16 nibble bytes     value = q d + m
//   Q5_0 22 B: d f16, qh u32, 16 nibble bytes    value = ((q | bit5) - 16) d
//   Q5_1 24 B: d f16, m f16, qh u32, 16 bytes    value = (q | bit5) d + m
//   Q8_0 34 B: d f16, 32 int8                    value = q d
//   Q8_1 36 B: d f16, s f16, 32 int8             value = q d
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define FT_HD __host__ __device__ __forceinline__
#else
#define FT_HD inline
#endif

FT_HD float gguf_half_bits_to_float(uint16_t h) {
  const uint32_t sign = static_cast<uint32_t>(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {                                   // subnormal: renormalise
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
      bits = sign | (static_cast<uint32_t>(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  union { uint32_t u; float f; } c;
  c.u = bits;
  return c.f;
}

FT_HD uint16_t gguf_rd16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
FT_HD uint32_t gguf_rd32(const uint8_t* p) {
  return static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) | (static_cast<uint32_t>(p[2]) << 16) |
         (static_cast<uint32_t>(p[3]) << 24);
}

// Bytes per block for a GGML type id, 0 when the type is not a 32-element quantised block.
FT_HD int gguf_block_bytes(unsigned type) {
  switch (type) {
    case 2: return 18;
    case 3: return 20;
    case 6: return 22;
    case 7: return 24;
    case 8: return 34;
    case 9: return 36;
    default: return 0;
  }
}

FT_HD void gguf_decode_pair(unsigned type, const uint8_t* p, int i, float& lo, float& hi) {
  const float d = gguf_half_bits_to_float(gguf_rd16(p));
  switch (type) {
    case 2:
      lo = static_cast<float>((p[2 + i] & 0xF) - 8) * d;
      hi = static_cast<float>((p[2 + i] >> 4) - 8) * d;
      break;
    case 3: {
      const float m = gguf_half_bits_to_float(gguf_rd16(p + 2));
      lo = static_cast<float>(p[4 + i] & 0xF) * d + m;
      hi = static_cast<float>(p[4 + i] >> 4) * d + m;
      break;
    }
    case 6: {
      const uint32_t qh = gguf_rd32(p + 2);
      const int h0 = static_cast<int>((qh >> i) << 4) & 0x10, h1 = static_cast<int>(qh >> (i + 12)) & 0x10;
      lo = static_cast<float>(((p[6 + i] & 0xF) | h0) - 16) * d;
      hi = static_cast<float>(((p[6 + i] >> 4) | h1) - 16) * d;
      break;
    }
    case 7: {
      const float m = gguf_half_bits_to_float(gguf_rd16(p + 2));
      const uint32_t qh = gguf_rd32(p + 4);
      const int h0 = static_cast<int>((qh >> i) << 4) & 0x10, h1 = static_cast<int>(qh >> (i + 12)) & 0x10;
      lo = static_cast<float>((p[8 + i] & 0xF) | h0) * d + m;
      hi = static_cast<float>((p[8 + i] >> 4) | h1) * d + m;
      break;
    }
    case 8:
      lo = static_cast<float>(static_cast<int8_t>(p[2 + i])) * d;
      hi = static_cast<float>(static_cast<int8_t>(p[2 + i + 16])) * d;
      break;
    case 9:
      lo = static_cast<float>(static_cast<int8_t>(p[4 + i])) * d;
      hi = static_cast<float>(static_cast<int8_t>(p[4 + i + 16])) * d;
      break;
    default:
      lo = hi = 0.f;
  }
}
