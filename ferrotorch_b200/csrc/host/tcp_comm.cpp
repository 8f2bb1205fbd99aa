// Host-side communication back-end for CPU ranks: TCP rendezvous, framed point-to-point
// messages with receive timeouts, and deterministic collectives on top.
//
// Behaviour follows the reference's CPU back-ends:
//   * rendezvous: rank 0 listens on MASTER_ADDR:MASTER_PORT, every other rank connects and
//     sends its rank as a little-endian u64 (ferrotorch-distributed/src/backend.rs:132-170);
//     connecting retries until a deadline (gloo_native/connect.rs:46-47);
//   * frames: 8-byte little-endian length + payload, a length mismatch is an error
//     (backend.rs:234-246, 280-286); receives take a timeout and fail with FTC_TIMEOUT
//     (backend.rs:295-370);
//   * all-reduce (star): ranks send to rank 0, which accumulates in rank order, divides for
//     a mean and sends the result back, so every rank ends bitwise identical
//     (collective.rs:105-134); broadcast, all-gather and barrier use the same star;
//   * ring all-reduce over a full mesh: reduce-scatter phase then all-gather phase with
//     chunk i = [i*N/W, (i+1)*N/W) (gloo_native/collectives.rs:98-160).
// The full mesh is built lazily: after the star exists, rank r listens on an ephemeral port,
// the ports are gathered at rank 0 and broadcast, and rank r connects to every rank below it.
#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <stdint.h>
#include <string.h>
#include <sys/socket.h>
#include <unistd.h>

#include <chrono>
#include <string>
#include <thread>
#include <vector>

#define FTC_API extern "C" __attribute__((visibility("default")))

enum {
  FTC_OK = 0,
  FTC_INVALID_RANK = -1,
  FTC_INVALID_WORLD = -2,
  FTC_SELF_SEND = -3,
  FTC_NO_CONNECTION = -4,
  FTC_SIZE_MISMATCH = -5,
  FTC_IO = -6,
  FTC_TIMEOUT = -7,
  FTC_UNSUPPORTED = -8,
};

namespace {

struct Comm {
  int rank = 0, world = 1;
  std::vector<int> star;   // rank 0: socket per peer; others: star[0] = socket to rank 0
  std::vector<int> mesh;   // full mesh sockets (lazy), mesh[rank] = -1
  int listen_fd = -1;
  long long timeout_ms = 60000;  // default collective timeout (collective.rs:35)
  std::string host;
};

using Clock = std::chrono::steady_clock;

int wait_fd(int fd, short ev, long long timeout_ms) {
  pollfd p{fd, ev, 0};
  int r = poll(&p, 1, timeout_ms < 0 ? -1 : static_cast<int>(timeout_ms));
  if (r == 0) return FTC_TIMEOUT;
  if (r < 0) return FTC_IO;
  return FTC_OK;
}

int write_all(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n > 0) {
    ssize_t k = ::send(fd, p, n, MSG_NOSIGNAL);
    if (k < 0) {
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) {
        if (wait_fd(fd, POLLOUT, 60000) != FTC_OK) return FTC_IO;
        continue;
      }
      return FTC_IO;
    }
    p += k;
    n -= static_cast<size_t>(k);
  }
  return FTC_OK;
}

int read_all(int fd, void* buf, size_t n, long long timeout_ms) {
  char* p = static_cast<char*>(buf);
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  while (n > 0) {
    long long left = timeout_ms < 0 ? -1
                                    : std::chrono::duration_cast<std::chrono::milliseconds>(deadline - Clock::now()).count();
    if (timeout_ms >= 0 && left <= 0) return FTC_TIMEOUT;
    int w = wait_fd(fd, POLLIN, left);
    if (w != FTC_OK) return w;
    ssize_t k = ::recv(fd, p, n, 0);
    if (k == 0) return FTC_NO_CONNECTION;  // peer closed
    if (k < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      return FTC_IO;
    }
    p += k;
    n -= static_cast<size_t>(k);
  }
  return FTC_OK;
}

int send_frame(int fd, const void* buf, uint64_t n) {
  uint64_t len = n;  // little-endian hosts only (x86-64 / aarch64)
  int rc = write_all(fd, &len, 8);
  if (rc) return rc;
  return n ? write_all(fd, buf, n) : FTC_OK;
}

int recv_frame(int fd, void* buf, uint64_t n, long long timeout_ms) {
  uint64_t len = 0;
  int rc = read_all(fd, &len, 8, timeout_ms);
  if (rc) return rc;
  if (len != n) {
    // drain nothing: the stream is now out of step, the caller must tear the group down
    return FTC_SIZE_MISMATCH;
  }
  return n ? read_all(fd, buf, n, timeout_ms) : FTC_OK;
}

void tune(int fd) {
  int one = 1;
  setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
  int sz = 4 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &sz, sizeof(sz));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
}

int listen_on(const char* host, int port, int* out_port) {
  int fd = socket(AF_INET, SOCK_STREAM, 0);
  if (fd < 0) return -1;
  int one = 1;
  setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(static_cast<uint16_t>(port));
  if (!host || !*host || inet_pton(AF_INET, host, &a.sin_addr) != 1) a.sin_addr.s_addr = htonl(INADDR_ANY);
  if (bind(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) < 0 || listen(fd, 64) < 0) {
    close(fd);
    return -1;
  }
  if (out_port) {
    socklen_t l = sizeof(a);
    getsockname(fd, reinterpret_cast<sockaddr*>(&a), &l);
    *out_port = ntohs(a.sin_port);
  }
  return fd;
}

int connect_to(const char* host, int port, long long timeout_ms) {
  auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
  while (true) {
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons(static_cast<uint16_t>(port));
    if (inet_pton(AF_INET, host, &a.sin_addr) != 1) {
      hostent* he = gethostbyname(host);
      if (!he) { close(fd); return -1; }
      memcpy(&a.sin_addr, he->h_addr_list[0], sizeof(a.sin_addr));
    }
    if (connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof(a)) == 0) {
      tune(fd);
      return fd;
    }
    close(fd);
    if (Clock::now() > deadline) return -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(50));
  }
}

int accept_one(int lfd, long long timeout_ms) {
  if (wait_fd(lfd, POLLIN, timeout_ms) != FTC_OK) return -1;
  int fd = accept(lfd, nullptr, nullptr);
  if (fd >= 0) tune(fd);
  return fd;
}

int star_fd(Comm* c, int peer) {
  if (c->rank == 0) return (peer > 0 && peer < c->world) ? c->star[peer] : -1;
  return peer == 0 ? c->star[0] : -1;
}

int pair_fd(Comm* c, int peer) {
  if (!c->mesh.empty() && peer >= 0 && peer < c->world && c->mesh[peer] >= 0) return c->mesh[peer];
  return star_fd(c, peer);
}

}  // namespace

// Create a group.  Returns a handle or null (see ftc_last_error_code).
static thread_local int g_last = 0;
FTC_API int ftc_last_error_code() { return g_last; }

FTC_API void* ftc_create(const char* master_addr, int master_port, int rank, int world, long long timeout_ms) {
  g_last = FTC_OK;
  if (world < 1) { g_last = FTC_INVALID_WORLD; return nullptr; }
  if (rank < 0 || rank >= world) { g_last = FTC_INVALID_RANK; return nullptr; }
  Comm* c = new Comm();
  c->rank = rank; c->world = world; c->host = master_addr ? master_addr : "127.0.0.1";
  if (timeout_ms > 0) c->timeout_ms = timeout_ms;
  if (world == 1) return c;
  if (rank == 0) {
    c->listen_fd = listen_on(c->host.c_str(), master_port, nullptr);
    if (c->listen_fd < 0) { g_last = FTC_IO; delete c; return nullptr; }
    c->star.assign(world, -1);
    for (int i = 1; i < world; ++i) {
      int fd = accept_one(c->listen_fd, c->timeout_ms);
      uint64_t r = 0;
      if (fd < 0 || read_all(fd, &r, 8, c->timeout_ms) != FTC_OK || r == 0 || r >= static_cast<uint64_t>(world) ||
          c->star[r] != -1) {
        g_last = fd < 0 ? FTC_TIMEOUT : FTC_INVALID_RANK;
        if (fd >= 0) close(fd);
        for (int f : c->star) if (f >= 0) close(f);
        close(c->listen_fd);
        delete c;
        return nullptr;
      }
      c->star[r] = fd;
    }
  } else {
    int fd = connect_to(c->host.c_str(), master_port, 30000);
    if (fd < 0) { g_last = FTC_NO_CONNECTION; delete c; return nullptr; }
    uint64_t r = static_cast<uint64_t>(rank);
    if (write_all(fd, &r, 8) != FTC_OK) { g_last = FTC_IO; close(fd); delete c; return nullptr; }
    c->star.assign(1, fd);
  }
  return c;
}

FTC_API void ftc_destroy(void* h) {
  Comm* c = static_cast<Comm*>(h);
  if (!c) return;
  for (int f : c->star) if (f >= 0) close(f);
  for (int f : c->mesh) if (f >= 0) close(f);
  if (c->listen_fd >= 0) close(c->listen_fd);
  delete c;
}

FTC_API int ftc_rank(void* h) { return static_cast<Comm*>(h)->rank; }
FTC_API int ftc_world(void* h) { return static_cast<Comm*>(h)->world; }
FTC_API void ftc_set_timeout(void* h, long long ms) { static_cast<Comm*>(h)->timeout_ms = ms; }

FTC_API int ftc_send(void* h, const void* buf, long long n, int dst) {
  Comm* c = static_cast<Comm*>(h);
  if (dst == c->rank) return FTC_SELF_SEND;
  if (dst < 0 || dst >= c->world) return FTC_INVALID_RANK;
  int fd = pair_fd(c, dst);
  if (fd < 0) return FTC_NO_CONNECTION;
  return send_frame(fd, buf, static_cast<uint64_t>(n));
}

FTC_API int ftc_recv(void* h, void* buf, long long n, int src, long long timeout_ms) {
  Comm* c = static_cast<Comm*>(h);
  if (src == c->rank) return FTC_SELF_SEND;
  if (src < 0 || src >= c->world) return FTC_INVALID_RANK;
  int fd = pair_fd(c, src);
  if (fd < 0) return FTC_NO_CONNECTION;
  return recv_frame(fd, buf, static_cast<uint64_t>(n), timeout_ms >= 0 ? timeout_ms : c->timeout_ms);
}

// barrier: gather one byte at rank 0, then scatter one byte (backend.rs:372-390)
FTC_API int ftc_barrier(void* h) {
  Comm* c = static_cast<Comm*>(h);
  if (c->world == 1) return FTC_OK;
  char b = 1;
  int rc;
  if (c->rank == 0) {
    for (int r = 1; r < c->world; ++r) if ((rc = recv_frame(c->star[r], &b, 1, c->timeout_ms))) return rc;
    for (int r = 1; r < c->world; ++r) if ((rc = send_frame(c->star[r], &b, 1))) return rc;
  } else {
    if ((rc = send_frame(c->star[0], &b, 1))) return rc;
    if ((rc = recv_frame(c->star[0], &b, 1, c->timeout_ms))) return rc;
  }
  return FTC_OK;
}

FTC_API int ftc_broadcast(void* h, void* buf, long long nbytes, int root) {
  Comm* c = static_cast<Comm*>(h);
  if (root < 0 || root >= c->world) return FTC_INVALID_RANK;
  if (c->world == 1) return FTC_OK;
  int rc;
  // through rank 0: root -> 0 -> everyone else
  if (root != 0) {
    if (c->rank == root) { if ((rc = send_frame(c->star[0], buf, nbytes))) return rc; }
    if (c->rank == 0) { if ((rc = recv_frame(c->star[root], buf, nbytes, c->timeout_ms))) return rc; }
  }
  if (c->rank == 0) {
    for (int r = 1; r < c->world; ++r)
      if (r != root && (rc = send_frame(c->star[r], buf, nbytes))) return rc;
  } else if (c->rank != root) {
    if ((rc = recv_frame(c->star[0], buf, nbytes, c->timeout_ms))) return rc;
  }
  return FTC_OK;
}

template <typename T>
static int allreduce_star(Comm* c, T* data, long long n, int mean) {
  if (c->world == 1) return FTC_OK;
  int rc;
  const uint64_t bytes = static_cast<uint64_t>(n) * sizeof(T);
  if (c->rank == 0) {
    std::vector<T> tmp(static_cast<size_t>(n));
    for (int r = 1; r < c->world; ++r) {  // accumulate in rank order
      if ((rc = recv_frame(c->star[r], tmp.data(), bytes, c->timeout_ms))) return rc;
      for (long long i = 0; i < n; ++i) data[i] += tmp[i];
    }
    if (mean) {
      const T w = static_cast<T>(c->world);
      for (long long i = 0; i < n; ++i) data[i] /= w;
    }
    for (int r = 1; r < c->world; ++r) if ((rc = send_frame(c->star[r], data, bytes))) return rc;
  } else {
    if ((rc = send_frame(c->star[0], data, bytes))) return rc;
    if ((rc = recv_frame(c->star[0], data, bytes, c->timeout_ms))) return rc;
  }
  return FTC_OK;
}

FTC_API int ftc_allreduce_f32(void* h, float* data, long long n, int mean) {
  return allreduce_star(static_cast<Comm*>(h), data, n, mean);
}
FTC_API int ftc_allreduce_f64(void* h, double* data, long long n, int mean) {
  return allreduce_star(static_cast<Comm*>(h), data, n, mean);
}

// all-gather: out[r*nbytes ...] = rank r's buffer (concat on dim 0, collective.rs:225-298)
FTC_API int ftc_allgather(void* h, const void* in, void* out, long long nbytes) {
  Comm* c = static_cast<Comm*>(h);
  char* o = static_cast<char*>(out);
  memcpy(o + static_cast<size_t>(c->rank) * nbytes, in, static_cast<size_t>(nbytes));
  if (c->world == 1) return FTC_OK;
  int rc;
  const uint64_t total = static_cast<uint64_t>(nbytes) * c->world;
  if (c->rank == 0) {
    for (int r = 1; r < c->world; ++r)
      if ((rc = recv_frame(c->star[r], o + static_cast<size_t>(r) * nbytes, nbytes, c->timeout_ms))) return rc;
    for (int r = 1; r < c->world; ++r) if ((rc = send_frame(c->star[r], o, total))) return rc;
  } else {
    if ((rc = send_frame(c->star[0], in, nbytes))) return rc;
    if ((rc = recv_frame(c->star[0], o, total, c->timeout_ms))) return rc;
  }
  return FTC_OK;
}

// Build the full mesh (needed by the ring and by peer-to-peer between non-zero ranks).
FTC_API int ftc_connect_mesh(void* h) {
  Comm* c = static_cast<Comm*>(h);
  if (!c->mesh.empty() || c->world == 1) return FTC_OK;
  int port = 0;
  int lfd = listen_on(nullptr, 0, &port);
  if (lfd < 0) return FTC_IO;
  std::vector<int> ports(static_cast<size_t>(c->world), 0);
  int rc = ftc_allgather(h, &port, ports.data(), sizeof(int));
  if (rc) { close(lfd); return rc; }
  c->mesh.assign(static_cast<size_t>(c->world), -1);
  // rank r connects to every lower rank and accepts from every higher rank
  for (int peer = 0; peer < c->rank; ++peer) {
    int fd = connect_to(c->host.c_str(), ports[peer], 30000);
    uint64_t me = static_cast<uint64_t>(c->rank);
    if (fd < 0 || write_all(fd, &me, 8) != FTC_OK) { close(lfd); return FTC_NO_CONNECTION; }
    c->mesh[peer] = fd;
  }
  for (int k = c->rank + 1; k < c->world; ++k) {
    int fd = accept_one(lfd, c->timeout_ms);
    uint64_t who = 0;
    if (fd < 0 || read_all(fd, &who, 8, c->timeout_ms) != FTC_OK || who >= static_cast<uint64_t>(c->world)) {
      close(lfd);
      return FTC_TIMEOUT;
    }
    c->mesh[who] = fd;
  }
  close(lfd);
  return ftc_barrier(h);
}

// Ring all-reduce (sum or mean) on f32: reduce-scatter lap then all-gather lap; the send runs
// on a helper thread so that neighbours never block each other (collectives.rs:208-226).
FTC_API int ftc_ring_allreduce_f32(void* h, float* data, long long n, int mean) {
  Comm* c = static_cast<Comm*>(h);
  const int W = c->world, r = c->rank;
  if (W == 1) return FTC_OK;
  int rc = ftc_connect_mesh(h);
  if (rc) return rc;
  const int right = (r + 1) % W, left = (r + W - 1) % W;
  auto lo = [&](int i) { return static_cast<long long>(i) * n / W; };
  auto len = [&](int i) { return lo(i + 1) - lo(i); };
  std::vector<float> tmp(static_cast<size_t>(n / W + 2));
  for (int phase = 0; phase < 2; ++phase) {
    for (int s = 0; s < W - 1; ++s) {
      const int send_chunk = phase == 0 ? (r - s + W) % W : (r + 1 - s + W) % W;
      const int recv_chunk = phase == 0 ? (r - s - 1 + 2 * W) % W : (r - s + W) % W;
      int send_rc = FTC_OK;
      std::thread t([&] { send_rc = send_frame(c->mesh[right], data + lo(send_chunk), len(send_chunk) * 4); });
      float* dst = phase == 0 ? tmp.data() : data + lo(recv_chunk);
      rc = recv_frame(c->mesh[left], dst, len(recv_chunk) * 4, c->timeout_ms);
      t.join();
      if (rc) return rc;
      if (send_rc) return send_rc;
      if (phase == 0) {
        float* d = data + lo(recv_chunk);
        for (long long i = 0; i < len(recv_chunk); ++i) d[i] += tmp[i];
      }
    }
    if (phase == 0 && mean) {
      const int own = (r + 1) % W;  // the chunk this rank holds fully reduced
      float* d = data + lo(own);
      for (long long i = 0; i < len(own); ++i) d[i] /= static_cast<float>(W);
    }
  }
  return FTC_OK;
}

// Broadcast down a binary tree laid over the mesh (gloo_native/collectives.rs:232-275): with
// v = (rank - root) mod W a rank's parent is (v - 1) / 2 and its children are 2v + 1 and 2v + 2,
// so the depth is ceil(log2 W) instead of the star's W - 1 sequential sends from rank 0.
FTC_API int ftc_tree_broadcast(void* h, void* buf, long long nbytes, int root) {
  Comm* c = static_cast<Comm*>(h);
  const int W = c->world;
  if (root < 0 || root >= W) return FTC_INVALID_RANK;
  if (W == 1) return FTC_OK;
  int rc = ftc_connect_mesh(h);
  if (rc) return rc;
  const int v = (c->rank - root + W) % W;
  auto real = [&](int tree_rank) { return (tree_rank + root) % W; };
  if (v != 0 && (rc = recv_frame(c->mesh[real((v - 1) / 2)], buf, nbytes, c->timeout_ms))) return rc;
  for (int child = 2 * v + 1; child <= 2 * v + 2 && child < W; ++child)
    if ((rc = send_frame(c->mesh[real(child)], buf, nbytes))) return rc;
  return FTC_OK;
}

// Barrier without a coordinator: a one-byte token travels the ring twice
// (gloo_native/collectives.rs:285-320).  The first lap proves that every rank has arrived, the
// second releases them; nobody leaves before everybody has entered.
FTC_API int ftc_ring_barrier(void* h) {
  Comm* c = static_cast<Comm*>(h);
  const int W = c->world, r = c->rank;
  if (W == 1) return FTC_OK;
  int rc = ftc_connect_mesh(h);
  if (rc) return rc;
  const int next = c->mesh[(r + 1) % W], prev = c->mesh[(r + W - 1) % W];
  char token = 1, got = 0;
  for (int lap = 0; lap < 2; ++lap) {
    if (r == 0) {
      if ((rc = send_frame(next, &token, 1))) return rc;
      if ((rc = recv_frame(prev, &got, 1, c->timeout_ms))) return rc;
    } else {
      if ((rc = recv_frame(prev, &got, 1, c->timeout_ms))) return rc;
      if ((rc = send_frame(next, &token, 1))) return rc;
    }
  }
  return FTC_OK;
}
