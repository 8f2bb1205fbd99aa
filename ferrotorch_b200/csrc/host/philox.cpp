// Philox-4x32-10 word stream on the host (ferrotorch-gpu/src/rng.rs:300-390 is the reference's
// scalar generator).  One 64-bit counter value gives four 32-bit words: counter in the low two
// counter words, the other two zero, the 64-bit seed as the key.  ftp_fill_words writes the n words
// that follow position (counter, offset) of the stream; utils/philox.py keeps the state.
#include <cstdint>

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
