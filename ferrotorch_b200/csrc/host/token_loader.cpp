// Multi-threaded token-batch loader over a memory-mapped file of token ids.
//
// The reference's DataLoader runs dataset reads on rayon worker threads with a prefetch queue,
// optional pinned staging and a distributed sampler that gives rank r the permuted samples
// r, r + world, ... (ferrotorch-data/src/dataloader.rs:219-458, sampler.rs:74-182).  This is the
// part of that job a language-model run needs, done natively: the file (uint16 or uint32 ids,
// little endian) is mapped once; sample s is the window [s * seq_len, s * seq_len + seq_len + 1)
// (inputs plus next-token labels); each epoch has its own seeded permutation; worker threads
// assemble whole batches as int64 into a ring of buffers ahead of the consumer, which receives
// them strictly in order, so a run is reproducible whatever the thread timing.
//
// C ABI (all functions return 0 on success, negative on error unless stated otherwise):
//   ftd_open / ftd_close, ftd_num_samples, ftd_batches_per_epoch, ftd_next, ftd_last_error.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace {

thread_local std::string g_err;

struct SplitMix64 {
  uint64_t s;
  uint64_t next() {
    uint64_t z = (s += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
};

struct Slot {
  std::vector<int64_t> data;
  long long batch = -1;   // global batch number held, -1 = free
  bool ready = false;
};

struct Loader {
  int fd = -1;
  const uint8_t* map = nullptr;
  size_t map_bytes = 0;
  int dtype_bytes = 2;
  long long n_tokens = 0, n_samples = 0;
  int seq_len = 0, batch = 0, rank = 0, world = 1;
  bool shuffle = true;
  uint64_t seed = 0;

  long long batches_per_epoch = 0;
  std::vector<Slot> ring;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv_ready, cv_free;
  long long next_to_build = 0;   // next global batch number a worker may claim
  long long next_to_serve = 0;   // next global batch number the consumer takes
  long long epoch_base = 0;      // global batch number of the first batch of `epoch`
  long long epoch = 0;
  std::vector<long long> perm;   // this rank's samples of the current epoch, in order
  std::vector<long long> perm_next;  // and of the next one (workers run ahead across the boundary)
  bool stop = false;

  void make_perm(long long ep, std::vector<long long>& out) const {
    std::vector<long long> all(n_samples);
    for (long long i = 0; i < n_samples; ++i) all[i] = i;
    if (shuffle) {
      SplitMix64 rng{seed * 0x100000001B3ull + static_cast<uint64_t>(ep) + 1};
      for (long long i = n_samples - 1; i > 0; --i) {
        const long long j = static_cast<long long>(rng.next() % static_cast<uint64_t>(i + 1));
        std::swap(all[i], all[j]);
      }
    }
    out.clear();
    const long long per_rank = batches_per_epoch * batch;
    for (long long i = 0; i < per_rank; ++i) out.push_back(all[rank + i * world]);
  }

  // Sample numbers of a batch (call with the lock held: the consumer rotates the permutations).
  void samples_of(long long global_batch, std::vector<long long>& out) const {
    // which epoch does this batch belong to?  (only the current or the next one can be asked for)
    const bool next_epoch = global_batch >= epoch_base + batches_per_epoch;
    const std::vector<long long>& p = next_epoch ? perm_next : perm;
    const long long b = global_batch - epoch_base - (next_epoch ? batches_per_epoch : 0);
    out.assign(p.begin() + b * batch, p.begin() + (b + 1) * batch);
  }

  void fill(const std::vector<long long>& samples, std::vector<int64_t>& dst) const {
    const int w = seq_len + 1;
    for (int i = 0; i < batch; ++i) {
      const long long s = samples[i];
      const size_t off = static_cast<size_t>(s) * seq_len;
      int64_t* out = dst.data() + static_cast<size_t>(i) * w;
      if (dtype_bytes == 2) {
        const uint16_t* src = reinterpret_cast<const uint16_t*>(map) + off;
        for (int t = 0; t < w; ++t) out[t] = src[t];
      } else {
        const uint32_t* src = reinterpret_cast<const uint32_t*>(map) + off;
        for (int t = 0; t < w; ++t) out[t] = src[t];
      }
    }
  }

  void worker_loop() {
    std::vector<long long> samples;
    for (;;) {
      long long mine;
      Slot* slot;
      {
        std::unique_lock<std::mutex> lk(mu);
        for (;;) {
          if (stop) return;
          mine = next_to_build;
          slot = &ring[static_cast<size_t>(mine % static_cast<long long>(ring.size()))];
          // claim the batch when its slot is free and it lies in the current or the next epoch
          if (slot->batch == -1 && mine < epoch_base + 2 * batches_per_epoch &&
              mine < next_to_serve + static_cast<long long>(ring.size()))
            break;
          cv_free.wait(lk);
        }
        slot->batch = mine;
        slot->ready = false;
        ++next_to_build;
        samples_of(mine, samples);
      }
      fill(samples, slot->data);
      {
        std::lock_guard<std::mutex> lk(mu);
        slot->ready = true;
      }
      cv_ready.notify_all();
    }
  }
};

int fail(const char* msg) {
  g_err = msg;
  return -1;
}

}  // namespace

#define FTD_API __attribute__((visibility("default")))

extern "C" {

FTD_API const char* ftd_last_error() { return g_err.c_str(); }

// dtype_bytes: 2 or 4.  prefetch: batches built ahead (ring size), n_workers >= 1.
FTD_API void* ftd_open(const char* path, int dtype_bytes, int seq_len, int batch, int n_workers, int prefetch,
               unsigned long long seed, int shuffle, int rank, int world) {
  if ((dtype_bytes != 2 && dtype_bytes != 4) || seq_len <= 0 || batch <= 0 || n_workers <= 0 || prefetch <= 0 ||
      world <= 0 || rank < 0 || rank >= world) {
    fail("ftd_open: bad arguments");
    return nullptr;
  }
  auto* L = new Loader();
  L->fd = ::open(path, O_RDONLY);
  struct stat st;
  if (L->fd < 0 || fstat(L->fd, &st) != 0) {
    fail("ftd_open: cannot open the token file");
    delete L;
    return nullptr;
  }
  L->map_bytes = static_cast<size_t>(st.st_size);
  L->dtype_bytes = dtype_bytes;
  L->n_tokens = static_cast<long long>(L->map_bytes / dtype_bytes);
  L->seq_len = seq_len; L->batch = batch; L->rank = rank; L->world = world;
  L->shuffle = shuffle != 0; L->seed = seed;
  L->n_samples = L->n_tokens > 0 ? (L->n_tokens - 1) / seq_len : 0;
  L->batches_per_epoch = L->n_samples / (static_cast<long long>(batch) * world);   // drop_last
  if (L->batches_per_epoch <= 0) {
    ::close(L->fd);
    fail("ftd_open: the file holds less than one batch per rank");
    delete L;
    return nullptr;
  }
  void* m = mmap(nullptr, L->map_bytes, PROT_READ, MAP_PRIVATE, L->fd, 0);
  if (m == MAP_FAILED) {
    ::close(L->fd);
    fail("ftd_open: mmap failed");
    delete L;
    return nullptr;
  }
  L->map = static_cast<const uint8_t*>(m);
  madvise(m, L->map_bytes, MADV_RANDOM);
  L->ring.resize(static_cast<size_t>(prefetch));
  for (auto& s : L->ring) s.data.resize(static_cast<size_t>(batch) * (seq_len + 1));
  L->make_perm(0, L->perm);
  L->make_perm(1, L->perm_next);
  for (int i = 0; i < n_workers; ++i) L->workers.emplace_back([L] { L->worker_loop(); });
  return L;
}

FTD_API long long ftd_num_samples(void* h) { return h ? static_cast<Loader*>(h)->n_samples : -1; }
FTD_API long long ftd_batches_per_epoch(void* h) { return h ? static_cast<Loader*>(h)->batches_per_epoch : -1; }

// Copy the next batch ([batch, seq_len + 1] int64) into out.  Returns the epoch the batch belongs
// to (>= 0); batches of one epoch are followed directly by those of the next.
FTD_API long long ftd_next(void* h, long long* out) {
  if (!h || !out) return fail("ftd_next: null argument");
  auto* L = static_cast<Loader*>(h);
  std::unique_lock<std::mutex> lk(L->mu);
  if (L->next_to_serve == L->epoch_base + L->batches_per_epoch) {
    // the consumer crosses into the next epoch: rotate the permutations
    L->epoch_base += L->batches_per_epoch;
    ++L->epoch;
    L->perm.swap(L->perm_next);
    L->make_perm(L->epoch + 1, L->perm_next);
    L->cv_free.notify_all();
  }
  const long long want = L->next_to_serve;
  Slot& slot = L->ring[static_cast<size_t>(want % static_cast<long long>(L->ring.size()))];
  L->cv_ready.wait(lk, [&] { return slot.batch == want && slot.ready; });
  // the slot is ours until it is marked free: copy without holding the lock, so the workers can
  // keep claiming and filling other slots meanwhile
  lk.unlock();
  std::memcpy(out, slot.data.data(), slot.data.size() * sizeof(int64_t));
  lk.lock();
  slot.batch = -1;
  slot.ready = false;
  ++L->next_to_serve;
  const long long ep = L->epoch;
  lk.unlock();
  L->cv_free.notify_all();
  return ep;
}

FTD_API void ftd_close(void* h) {
  if (!h) return;
  auto* L = static_cast<Loader*>(h);
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->stop = true;
  }
  L->cv_free.notify_all();
  for (auto& t : L->workers) t.join();
  if (L->map) munmap(const_cast<uint8_t*>(L->map), L->map_bytes);
  if (L->fd >= 0) ::close(L->fd);
  delete L;
}

}  // extern "C"
