// Philox-4x32-10 word stream on the host (ferrotorch-gpu/src/rng.rs:300-390 is the reference's
// scalar generator).  One 64-bit counter value gives four 32-bit words: counter in the low two
// counter words, the other two zero, the 64-bit seed as the key.  ftp_fill_words writes the n words
// that follow position (counter, offset) of the stream; utils/philox.py keeps the state.
#include <cmath>
#include <cstdint>
#include <thread>
#include <vector>

namespace {

inline void philox4x32_10(uint64_t counter, uint64_t key, uint32_t out[4]) {
  uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32), c2 = 0, c3 = 0;
  uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = 0xD2511F53ull * c0, p1 = 0xCD9E8D57ull * c2;
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1 ^ k0, n1 = static_cast<uint32_t>(p1);
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c3 ^ k1, n3 = static_cast<uint32_t>(p0);
    c0 = n0; c1 = n1; c2 = n2; c3 = n3;
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int ftp_fill_words(unsigned long long counter, unsigned long long key, int offset, long long n, uint32_t* out) {
  if (!out || n < 0 || offset < 0 || offset > 3) return -1;
  long long i = 0;
  uint32_t w[4];
  if (offset != 0 && n > 0) {                    // finish the partly used counter
    philox4x32_10(counter, key, w);
    for (int j = offset; j < 4 && i < n; ++j) out[i++] = w[j];
    ++counter;
  }
  for (; i + 4 <= n; i += 4, ++counter) philox4x32_10(counter, key, out + i);
  if (i < n) {
    philox4x32_10(counter, key, w);
    for (int j = 0; i < n; ++j) out[i++] = w[j];
  }
  return 0;
}

// ---------------------------------------------------------------------------------------------
// Threaded fills on the device kernels' stream layout: output element i of a call that starts at
// counter c is made from stream word 4 c + i (so a host tensor and a device tensor filled from the
// same (seed, counter) hold the same uniforms, and normals that agree to the rounding of log /
// sincos).  A counter-based generator needs no state hand-over between threads: thread t takes a
// contiguous range of counters.
//   kind 1: a + (b - a) * u,  u = (word >> 8) * 2^-24
//   kind 2: Box-Muller over the word pairs (0, 1) and (2, 3) of a counter: r = sqrt(-2 ln u1),
//           a + b * r * (cos, sin)(2 pi u2); u1 == 0 is replaced by 2^-25 (as the device kernel does).
namespace {

inline float u01(uint32_t w) { return static_cast<float>(w >> 8) * (1.0f / 16777216.0f); }

// Eight counters per trip in structure-of-arrays form: the rounds are plain 32 x 32 -> 64 bit
// multiplies and xors over arrays of eight, which the compiler turns into vector code (one clone per
// instruction set, picked when the library is loaded).
constexpr int LANES = 8;

#if defined(__x86_64__) && defined(__GNUC__) && !defined(__clang__)
__attribute__((target_clones("avx512f", "avx2", "default")))
#endif
void philox_lanes(uint64_t first_counter, uint64_t key, uint32_t w[4][LANES]) {
  uint32_t c0[LANES], c1[LANES], c2[LANES], c3[LANES];
  for (int l = 0; l < LANES; ++l) {
    const uint64_t c = first_counter + static_cast<uint64_t>(l);
    c0[l] = static_cast<uint32_t>(c); c1[l] = static_cast<uint32_t>(c >> 32); c2[l] = 0; c3[l] = 0;
  }
  uint32_t k0 = static_cast<uint32_t>(key), k1 = static_cast<uint32_t>(key >> 32);
  for (int r = 0; r < 10; ++r) {
    for (int l = 0; l < LANES; ++l) {
      const uint64_t p0 = 0xD2511F53ull * c0[l], p1 = 0xCD9E8D57ull * c2[l];
      const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c1[l] ^ k0, n2 = static_cast<uint32_t>(p0 >> 32) ^ c3[l] ^ k1;
      c0[l] = n0; c1[l] = static_cast<uint32_t>(p1); c2[l] = n2; c3[l] = static_cast<uint32_t>(p0);
    }
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  for (int l = 0; l < LANES; ++l) { w[0][l] = c0[l]; w[1][l] = c1[l]; w[2][l] = c2[l]; w[3][l] = c3[l]; }
}

inline void block_values(const uint32_t w[4], int kind, float a, float b, float v[4]) {
  if (kind == 1) {
    for (int j = 0; j < 4; ++j) v[j] = a + (b - a) * u01(w[j]);
    return;
  }
  for (int h = 0; h < 2; ++h) {
    float u1 = u01(w[2 * h]);
    const float u2 = u01(w[2 * h + 1]);
    if (u1 == 0.f) u1 = 1.0f / 33554432.0f;
    const float rad = std::sqrt(-2.f * std::log(u1));
    const float ang = 6.283185307179586f * u2;
    v[2 * h] = a + b * rad * std::cos(ang);
    v[2 * h + 1] = a + b * rad * std::sin(ang);
  }
}

void fill_range(uint64_t counter, uint64_t key, long long first_block, long long last_block, long long n, int kind, float a,
                float b, float* out) {
  uint32_t lanes[4][LANES], w[4];
  float v[4];
  long long blk = first_block;
  for (; blk + LANES <= last_block && 4 * (blk + LANES) <= n; blk += LANES) {       // whole groups, no ragged tail
    philox_lanes(counter + static_cast<uint64_t>(blk), key, lanes);
    float* o = out + 4 * blk;
    if (kind == 1) {
      const float scale = b - a;
      for (int l = 0; l < LANES; ++l)
        for (int j = 0; j < 4; ++j) o[4 * l + j] = a + scale * u01(lanes[j][l]);
    } else {
      for (int l = 0; l < LANES; ++l) {
        for (int j = 0; j < 4; ++j) w[j] = lanes[j][l];
        block_values(w, kind, a, b, o + 4 * l);
      }
    }
  }
  for (; blk < last_block; ++blk) {
    philox4x32_10(counter + static_cast<uint64_t>(blk), key, w);
    block_values(w, kind, a, b, v);
    const long long base = 4 * blk;
    const int m = static_cast<int>(n - base < 4 ? n - base : 4);
    for (int j = 0; j < m; ++j) out[base + j] = v[j];
  }
}

}  // namespace

extern "C" __attribute__((visibility("default")))
int ftp_fill_f32(unsigned long long counter, unsigned long long key, long long n, int kind, float a, float b, float* out,
                 int threads) {
  if (!out || n < 0 || (kind != 1 && kind != 2)) return -1;
  const long long blocks = (n + 3) / 4;
  if (threads < 1) threads = 1;
  const long long min_blocks_per_thread = 1 << 13;   // 32 K values: below that a thread costs more than it saves
  long long want = blocks / min_blocks_per_thread;
  if (want < 1) want = 1;
  if (threads > want) threads = static_cast<int>(want);
  if (threads == 1) {
    fill_range(counter, key, 0, blocks, n, kind, a, b, out);
    return 0;
  }
  std::vector<std::thread> pool;
  pool.reserve(threads);
  for (int t = 0; t < threads; ++t) {
    const long long lo = blocks * t / threads, hi = blocks * (t + 1) / threads;
    pool.emplace_back(fill_range, counter, key, lo, hi, n, kind, a, b, out);
  }
  for (auto& th : pool) th.join();
  return 0;
}
