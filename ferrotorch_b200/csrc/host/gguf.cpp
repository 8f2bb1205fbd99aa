// GGUF v2/v3 reader: mmap the file, parse header / metadata / tensor table, dequantise the
// block formats the reference supports (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0, Q8_1, F16, BF16, F32 --
// ferrotorch-serialize/src/gguf.rs:56-927; block = 32 elements, Q4_0 = fp16 scale + 16 nibble
// bytes) and re-lay Q4_0 weights out for the fused dequant-GEMM kernel (separate scale and nibble
// planes, csrc/quant_gemm.cu).
//
// Element order inside a block.  The GGML file format (what llama.cpp writes) puts element j in
// the low nibble of byte j and element j + 16 in the high nibble, and bit j / bit j + 16 of the
// Q5 high-bit word belong to the same two elements; that is the default here, so real model
// files decode correctly.  The reference's decoders emit the two nibbles of byte j as the
// consecutive elements 2j and 2j + 1 and take high bits 2j and 2j + 1 (gguf.rs:543-577, 614-660;
// ferrotorch-cubecl/src/quant.rs:348).  `interleaved = 1` selects that order for callers that need
// bit-for-bit agreement with tensors the reference decoded.
#include "../gguf_blocks.h"
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <string>
#include <vector>

#define FTG_API extern "C" __attribute__((visibility("default")))

namespace {

struct TensorInfo {
  std::string name;
  uint32_t type = 0, n_dims = 0;
  uint64_t dims[4] = {1, 1, 1, 1};
  uint64_t offset = 0, nbytes = 0;
};

struct Gguf {
  int fd = -1;
  const uint8_t* base = nullptr;
  size_t size = 0, data_off = 0;
  uint32_t version = 0;
  std::vector<TensorInfo> tensors;
  std::string kv_json;
  std::string error;
};

struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;
  template <typename T>
  T get() {
    T v{};
    if (p + sizeof(T) > end) { ok = false; return v; }
    memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    uint64_t n = get<uint64_t>();
    if (!ok || p + n > end) { ok = false; return {}; }
    std::string s(reinterpret_cast<const char*>(p), n);
    p += n;
    return s;
  }
};

void json_escape(std::string& out, const std::string& s) {
  out += '"';
  for (char c : s) {
    if (c == '"' || c == '\\') { out += '\\'; out += c; }
    else if (c == '\n') out += "\\n";
    else if (static_cast<unsigned char>(c) < 0x20) out += ' ';
    else out += c;
  }
  out += '"';
}

bool value_json(Reader& r, uint32_t type, std::string& out, int depth = 0) {
  char buf[64];
  switch (type) {
    case 0: snprintf(buf, sizeof buf, "%u", r.get<uint8_t>()); out += buf; break;
    case 1: snprintf(buf, sizeof buf, "%d", r.get<int8_t>()); out += buf; break;
    case 2: snprintf(buf, sizeof buf, "%u", r.get<uint16_t>()); out += buf; break;
    case 3: snprintf(buf, sizeof buf, "%d", r.get<int16_t>()); out += buf; break;
    case 4: snprintf(buf, sizeof buf, "%u", r.get<uint32_t>()); out += buf; break;
    case 5: snprintf(buf, sizeof buf, "%d", r.get<int32_t>()); out += buf; break;
    case 6: snprintf(buf, sizeof buf, "%.9g", r.get<float>()); out += buf; break;
    case 7: out += r.get<uint8_t>() ? "true" : "false"; break;
    case 8: json_escape(out, r.str()); break;
    case 9: {
      if (depth > 2) return false;
      uint32_t et = r.get<uint32_t>();
      uint64_t n = r.get<uint64_t>();
      out += '[';
      for (uint64_t i = 0; i < n && r.ok; ++i) {
        if (i) out += ',';
        // long arrays (token tables) are parsed but only the first 16 entries are kept
        if (i < 16) { if (!value_json(r, et, out, depth + 1)) return false; }
        else { std::string skip; if (!value_json(r, et, skip, depth + 1)) return false; out.pop_back(); }
      }
      out += ']';
      break;
    }
    case 10: snprintf(buf, sizeof buf, "%llu", (unsigned long long)r.get<uint64_t>()); out += buf; break;
    case 11: snprintf(buf, sizeof buf, "%lld", (long long)r.get<int64_t>()); out += buf; break;
    case 12: snprintf(buf, sizeof buf, "%.17g", r.get<double>()); out += buf; break;
    default: return false;
  }
  return r.ok;
}

// bytes per block and elements per block of a ggml type; 0 = unsupported
bool type_layout(uint32_t t, uint32_t* blk_elems, uint32_t* blk_bytes) {
  switch (t) {
    case 0: *blk_elems = 1; *blk_bytes = 4; return true;    // F32
    case 1: *blk_elems = 1; *blk_bytes = 2; return true;    // F16
    case 30: *blk_elems = 1; *blk_bytes = 2; return true;   // BF16
    case 2: *blk_elems = 32; *blk_bytes = 18; return true;  // Q4_0
    case 3: *blk_elems = 32; *blk_bytes = 20; return true;  // Q4_1
    case 6: *blk_elems = 32; *blk_bytes = 22; return true;  // Q5_0
    case 7: *blk_elems = 32; *blk_bytes = 24; return true;  // Q5_1
    case 8: *blk_elems = 32; *blk_bytes = 34; return true;  // Q8_0
    case 9: *blk_elems = 32; *blk_bytes = 36; return true;  // Q8_1
    default: return false;
  }
}

float half_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
  if (exp == 0) {
    if (man == 0) bits = sign;
    else {
      exp = 127 - 15 + 1;
      while (!(man & 0x400)) { man <<= 1; --exp; }
      bits = sign | (exp << 23) | ((man & 0x3FF) << 13);
    }
  } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
  else bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
  float f;
  memcpy(&f, &bits, 4);
  return f;
}
inline uint16_t rd16(const uint8_t* p) { uint16_t v; memcpy(&v, p, 2); return v; }
inline uint32_t rd32(const uint8_t* p) { uint32_t v; memcpy(&v, p, 4); return v; }

}  // namespace

FTG_API void* ftg_open(const char* path) {
  Gguf* g = new Gguf();
  g->fd = open(path, O_RDONLY);
  struct stat st;
  if (g->fd < 0 || fstat(g->fd, &st) != 0) { g->error = "cannot open file"; return g; }
  g->size = static_cast<size_t>(st.st_size);
  void* m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
  if (m == MAP_FAILED) { g->error = "mmap failed"; return g; }
  g->base = static_cast<const uint8_t*>(m);
  Reader r{g->base, g->base + g->size};
  if (g->size < 24 || memcmp(g->base, "GGUF", 4) != 0) { g->error = "not a GGUF file"; return g; }
  r.p += 4;
  g->version = r.get<uint32_t>();
  if (g->version < 2 || g->version > 3) { g->error = "unsupported GGUF version"; return g; }
  const uint64_t n_tensors = r.get<uint64_t>(), n_kv = r.get<uint64_t>();
  uint64_t alignment = 32;
  g->kv_json = "{";
  for (uint64_t i = 0; i < n_kv && r.ok; ++i) {
    std::string key = r.str();
    uint32_t vt = r.get<uint32_t>();
    if (i) g->kv_json += ',';
    json_escape(g->kv_json, key);
    g->kv_json += ':';
    const uint8_t* before = r.p;
    if (!value_json(r, vt, g->kv_json)) { g->error = "bad metadata value for " + key; return g; }
    if (key == "general.alignment" && vt == 4) alignment = rd32(before);
  }
  g->kv_json += '}';
  for (uint64_t i = 0; i < n_tensors && r.ok; ++i) {
    TensorInfo t;
    t.name = r.str();
    t.n_dims = r.get<uint32_t>();
    if (t.n_dims > 4) { g->error = "tensor with more than 4 dims"; return g; }
    uint64_t numel = 1;
    for (uint32_t d = 0; d < t.n_dims; ++d) { t.dims[d] = r.get<uint64_t>(); numel *= t.dims[d]; }
    t.type = r.get<uint32_t>();
    t.offset = r.get<uint64_t>();
    uint32_t be = 0, bb = 0;
    if (type_layout(t.type, &be, &bb)) t.nbytes = numel / be * bb;
    g->tensors.push_back(t);
  }
  if (!r.ok) { g->error = "truncated header"; return g; }
  size_t off = static_cast<size_t>(r.p - g->base);
  g->data_off = (off + alignment - 1) / alignment * alignment;
  for (auto& t : g->tensors)
    if (g->data_off + t.offset + t.nbytes > g->size) { g->error = "tensor data out of range: " + t.name; return g; }
  return g;
}

FTG_API const char* ftg_error(void* h) { return static_cast<Gguf*>(h)->error.c_str(); }
FTG_API void ftg_close(void* h) {
  Gguf* g = static_cast<Gguf*>(h);
  if (g->base) munmap(const_cast<uint8_t*>(g->base), g->size);
  if (g->fd >= 0) close(g->fd);
  delete g;
}
FTG_API int ftg_version(void* h) { return static_cast<int>(static_cast<Gguf*>(h)->version); }
FTG_API long long ftg_n_tensors(void* h) { return static_cast<long long>(static_cast<Gguf*>(h)->tensors.size()); }
FTG_API const char* ftg_metadata_json(void* h) { return static_cast<Gguf*>(h)->kv_json.c_str(); }
FTG_API const char* ftg_tensor_name(void* h, long long i) { return static_cast<Gguf*>(h)->tensors[i].name.c_str(); }
// out[0]=type, out[1]=n_dims, out[2..5]=dims (innermost first, as stored), out[6]=nbytes
FTG_API void ftg_tensor_info(void* h, long long i, unsigned long long* out) {
  const TensorInfo& t = static_cast<Gguf*>(h)->tensors[i];
  out[0] = t.type; out[1] = t.n_dims;
  for (int d = 0; d < 4; ++d) out[2 + d] = t.dims[d];
  out[6] = t.nbytes;
}
FTG_API const void* ftg_tensor_data(void* h, long long i) {
  Gguf* g = static_cast<Gguf*>(h);
  return g->base + g->data_off + g->tensors[i].offset;
}

// Dequantise n elements (n % 32 == 0 for block types) of ggml type `type` to fp32.
FTG_API int ftg_dequantize(unsigned type, const void* src_, float* dst, long long n) {
  const uint8_t* src = static_cast<const uint8_t*>(src_);
  uint32_t be = 0, bb = 0;
  if (!type_layout(type, &be, &bb) || n % be) return -1;
  if (type == 0) { memcpy(dst, src, static_cast<size_t>(n) * 4); return 0; }
  if (type == 1) { for (long long i = 0; i < n; ++i) dst[i] = half_to_float(rd16(src + 2 * i)); return 0; }
  if (type == 30) {
    for (long long i = 0; i < n; ++i) { uint32_t b = static_cast<uint32_t>(rd16(src + 2 * i)) << 16; memcpy(dst + i, &b, 4); }
    return 0;
  }
  const long long nb = n / 32;
  for (long long b = 0; b < nb; ++b) {
    const uint8_t* p = src + b * bb;
    float* y = dst + b * 32;
    const float d = half_to_float(rd16(p));
    switch (type) {
      case 2:
        for (int i = 0; i < 16; ++i) { y[i] = ((p[2 + i] & 0xF) - 8) * d; y[i + 16] = ((p[2 + i] >> 4) - 8) * d; }
        break;
      case 3: {
        const float m = half_to_float(rd16(p + 2));
        for (int i = 0; i < 16; ++i) { y[i] = (p[4 + i] & 0xF) * d + m; y[i + 16] = (p[4 + i] >> 4) * d + m; }
        break;
      }
      case 6: {
        const uint32_t qh = rd32(p + 2);
        for (int i = 0; i < 16; ++i) {
          const int h0 = ((qh >> i) << 4) & 0x10, h1 = (qh >> (i + 12)) & 0x10;
          y[i] = (((p[6 + i] & 0xF) | h0) - 16) * d;
          y[i + 16] = (((p[6 + i] >> 4) | h1) - 16) * d;
        }
        break;
      }
      case 7: {
        const float m = half_to_float(rd16(p + 2));
        const uint32_t qh = rd32(p + 4);
        for (int i = 0; i < 16; ++i) {
          const int h0 = ((qh >> i) << 4) & 0x10, h1 = (qh >> (i + 12)) & 0x10;
          y[i] = ((p[8 + i] & 0xF) | h0) * d + m;
          y[i + 16] = ((p[8 + i] >> 4) | h1) * d + m;
        }
        break;
      }
      case 8:
        for (int i = 0; i < 32; ++i) y[i] = static_cast<int8_t>(p[2 + i]) * d;
        break;
      case 9:
        for (int i = 0; i < 32; ++i) y[i] = static_cast<int8_t>(p[4 + i]) * d;
        break;
    }
  }
  return 0;
}

// The quantised block types decoded pair by pair through the header the device kernel includes
// (csrc/gguf_dequant.cu): running this on the host checks the device arithmetic without a device.
FTG_API int ftg_dequantize_pairwise(unsigned type, const void* src_, float* dst, long long n) {
  const int bb = gguf_block_bytes(type);
  if (bb == 0 || n % 32) return -1;
  const uint8_t* src = static_cast<const uint8_t*>(src_);
  for (long long b = 0; b < n / 32; ++b)
    for (int i = 0; i < 16; ++i) gguf_decode_pair(type, src + b * bb, i, dst[b * 32 + i], dst[b * 32 + i + 16]);
  return 0;
}

// The same with the element order chosen by the caller (see the head of this file).
FTG_API int ftg_dequantize_ex(unsigned type, const void* src_, float* dst, long long n, int interleaved) {
  if (!interleaved || !(type == 2 || type == 3 || type == 6 || type == 7)) return ftg_dequantize(type, src_, dst, n);
  const uint8_t* src = static_cast<const uint8_t*>(src_);
  uint32_t be = 0, bb = 0;
  if (!type_layout(type, &be, &bb) || n % be) return -1;
  const long long nb = n / 32;
  for (long long b = 0; b < nb; ++b) {
    const uint8_t* p = src + b * bb;
    float* y = dst + b * 32;
    const float d = half_to_float(rd16(p));
    const float m = (type == 3 || type == 7) ? half_to_float(rd16(p + 2)) : 0.f;
    const uint8_t* q = p + (type == 2 ? 2 : type == 3 ? 4 : type == 6 ? 6 : 8);
    const uint32_t qh = type == 6 ? rd32(p + 2) : type == 7 ? rd32(p + 4) : 0u;
    for (int j = 0; j < 16; ++j) {
      int lo = q[j] & 0xF, hi = q[j] >> 4;
      if (type >= 6) { lo |= ((qh >> (2 * j)) & 1) << 4; hi |= ((qh >> (2 * j + 1)) & 1) << 4; }
      switch (type) {
        case 2: y[2 * j] = (lo - 8) * d; y[2 * j + 1] = (hi - 8) * d; break;
        case 3: case 7: y[2 * j] = lo * d + m; y[2 * j + 1] = hi * d + m; break;
        case 6: y[2 * j] = (lo - 16) * d; y[2 * j + 1] = (hi - 16) * d; break;
      }
    }
  }
  return 0;
}

// Rewrite the nibble bytes of Q4_0 / Q4_1 blocks in place from the interleaved element order to the
// file format's order (or back, `to_interleaved`), so data meant for one convention can be fed to
// code of the other: the dequant-GEMM kernel always reads the file format's order.
FTG_API int ftg_repack_nibbles(unsigned type, void* data_, long long n_blocks, int to_interleaved) {
  if (type != 2 && type != 3) return -1;
  uint8_t* data = static_cast<uint8_t*>(data_);
  const int bb = type == 2 ? 18 : 20, off = type == 2 ? 2 : 4;
  for (long long b = 0; b < n_blocks; ++b) {
    uint8_t* q = data + b * bb + off;
    uint8_t e[32], out[16];
    if (!to_interleaved) {
      for (int j = 0; j < 16; ++j) { e[2 * j] = q[j] & 0xF; e[2 * j + 1] = q[j] >> 4; }
      for (int j = 0; j < 16; ++j) out[j] = static_cast<uint8_t>(e[j] | (e[j + 16] << 4));
    } else {
      for (int j = 0; j < 16; ++j) { e[j] = q[j] & 0xF; e[j + 16] = q[j] >> 4; }
      for (int j = 0; j < 16; ++j) out[j] = static_cast<uint8_t>(e[2 * j] | (e[2 * j + 1] << 4));
    }
    memcpy(q, out, 16);
  }
  return 0;
}

// Q4_0 [rows, cols] (cols % 32 == 0) -> planes for the dequant-GEMM: scales fp16 [rows, cols/32]
// and nibbles u8 [rows, cols/2] where byte j of a 32-element block holds elements (j, j+16),
// exactly as in the file, so the kernel's unpack matches ftg_dequantize bit for bit.  (For the
// interleaved convention, run ftg_repack_nibbles over the planes' source first.)
FTG_API int ftg_split_q4_0(const void* src_, long long rows, long long cols, unsigned short* scales,
                           unsigned char* nibbles) {
  if (cols % 32) return -1;
  const uint8_t* src = static_cast<const uint8_t*>(src_);
  const long long bpr = cols / 32;
  for (long long r = 0; r < rows; ++r)
    for (long long b = 0; b < bpr; ++b) {
      const uint8_t* p = src + (r * bpr + b) * 18;
      scales[r * bpr + b] = rd16(p);
      memcpy(nibbles + (r * bpr + b) * 16, p + 2, 16);
    }
  return 0;
}
