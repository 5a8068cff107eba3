// Host-side rendezvous / liveness runtime: the reference's TCP message framing
// ([type u8][len u32 LE][payload], rust-nn src/distributed.rs:268-370) and a small key-value store
// built on it (set / get-with-timeout / add / heartbeat), used for rendezvous, handle exchange and
// failure detection among ranks. Unlike the reference's accept loop (which spins without a timeout,
// src/distributed.rs:448-457) every blocking call here takes a deadline.
#include <arpa/inet.h>
#include <atomic>
#include <cerrno>
#include <chrono>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <map>
#include <mutex>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <string>
#include <sys/socket.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace {

enum MsgType : uint8_t { GradientChunk = 0, Barrier = 1, Heartbeat = 2, Shutdown = 3, Parameters = 4,
                         // store operations (values above the reference's five types)
                         StoreSet = 16, StoreGet = 17, StoreAdd = 18, StoreReply = 19, StoreMissing = 20 };

bool wait_fd(int fd, short ev, int timeout_ms) {
  struct pollfd p{fd, ev, 0};
  int r;
  do { r = poll(&p, 1, timeout_ms); } while (r < 0 && errno == EINTR);
  return r > 0 && (p.revents & ev);
}
bool send_all(int fd, const uint8_t* b, size_t n, int timeout_ms) {
  size_t done = 0;
  while (done < n) {
    if (!wait_fd(fd, POLLOUT, timeout_ms)) return false;
    ssize_t w = send(fd, b + done, n - done, MSG_NOSIGNAL);
    if (w <= 0) { if (errno == EINTR || errno == EAGAIN) continue; return false; }
    done += (size_t)w;
  }
  return true;
}
bool recv_all(int fd, uint8_t* b, size_t n, int timeout_ms) {
  size_t done = 0;
  while (done < n) {
    if (!wait_fd(fd, POLLIN, timeout_ms)) return false;
    ssize_t r = recv(fd, b + done, n - done, 0);
    if (r <= 0) { if (r < 0 && (errno == EINTR || errno == EAGAIN)) continue; return false; }
    done += (size_t)r;
  }
  return true;
}
bool send_frame(int fd, uint8_t type, const uint8_t* payload, uint32_t len, int timeout_ms) {
  uint8_t hdr[5]; hdr[0] = type; memcpy(hdr + 1, &len, 4);
  return send_all(fd, hdr, 5, timeout_ms) && (len == 0 || send_all(fd, payload, len, timeout_ms));
}
bool recv_frame(int fd, uint8_t& type, std::vector<uint8_t>& payload, int timeout_ms) {
  uint8_t hdr[5];
  if (!recv_all(fd, hdr, 5, timeout_ms)) return false;
  uint32_t len; memcpy(&len, hdr + 1, 4);
  if (len > (1u << 30)) return false;
  type = hdr[0]; payload.resize(len);
  return len == 0 || recv_all(fd, payload.data(), len, timeout_ms);
}

struct Server {
  int listen_fd = -1;
  int port = 0;
  std::atomic<bool> stop{false};
  std::thread acceptor;
  std::vector<std::thread> workers;
  std::mutex mu;
  std::condition_variable cv;
  std::map<std::string, std::vector<uint8_t>> kv;

  void serve(int fd) {
    while (!stop.load()) {
      uint8_t type; std::vector<uint8_t> pl;
      if (!wait_fd(fd, POLLIN, 200)) {
        // distinguish idle from closed
        char c; ssize_t r = recv(fd, &c, 1, MSG_PEEK | MSG_DONTWAIT);
        if (r == 0) break;
        continue;
      }
      if (!recv_frame(fd, type, pl, 5000)) break;
      if (type == Shutdown) break;
      // payload: u32 key_len | key | value / timeout
      if (pl.size() < 4) break;
      uint32_t kl; memcpy(&kl, pl.data(), 4);
      if (pl.size() < 4 + (size_t)kl) break;
      std::string key((const char*)pl.data() + 4, kl);
      const uint8_t* rest = pl.data() + 4 + kl; size_t rn = pl.size() - 4 - kl;
      if (type == StoreSet) {
        { std::lock_guard<std::mutex> g(mu); kv[key].assign(rest, rest + rn); }
        cv.notify_all();
        if (!send_frame(fd, StoreReply, nullptr, 0, 5000)) break;
      } else if (type == StoreGet) {
        int32_t to_ms = 0; if (rn >= 4) memcpy(&to_ms, rest, 4);
        std::vector<uint8_t> val; bool found = false;
        {
          std::unique_lock<std::mutex> lk(mu);
          found = cv.wait_for(lk, std::chrono::milliseconds(to_ms), [&] { return kv.count(key) > 0 || stop.load(); }) && kv.count(key);
          if (found) val = kv[key];
        }
        if (!send_frame(fd, found ? StoreReply : StoreMissing, val.data(), (uint32_t)val.size(), 5000)) break;
      } else if (type == StoreAdd) {
        int64_t delta = 0; if (rn >= 8) memcpy(&delta, rest, 8);
        int64_t cur = 0;
        {
          std::lock_guard<std::mutex> g(mu);
          auto& v = kv[key];
          if (v.size() == 8) memcpy(&cur, v.data(), 8);
          cur += delta; v.resize(8); memcpy(v.data(), &cur, 8);
        }
        cv.notify_all();
        if (!send_frame(fd, StoreReply, (const uint8_t*)&cur, 8, 5000)) break;
      } else break;
    }
    close(fd);
  }
};

}  // namespace

extern "C" {

// ---- message framing (byte-compatible with the reference)
long long b200_msg_serialize(int type, const unsigned char* payload, long long len, unsigned char* out, long long cap) {
  if (len < 0 || len > 0xFFFFFFFFLL || cap < 5 + len) return -1;
  out[0] = (uint8_t)type; uint32_t l = (uint32_t)len; memcpy(out + 1, &l, 4);
  if (len) memcpy(out + 5, payload, (size_t)len);
  return 5 + len;
}
// returns payload length (>= 0) and writes the type, or -1 for a truncated / invalid frame
long long b200_msg_deserialize(const unsigned char* data, long long len, int* type) {
  if (len < 5 || data[0] > 4) return -1;
  uint32_t l; memcpy(&l, data + 1, 4);
  if (len < 5 + (long long)l) return -1;
  *type = data[0];
  return l;
}

// ---- store server
void* b200_store_server_start(int port, int* bound_port) {
  Server* s = new Server();
  s->listen_fd = socket(AF_INET, SOCK_STREAM, 0);
  if (s->listen_fd < 0) { delete s; return nullptr; }
  int one = 1; setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof one);
  sockaddr_in a{}; a.sin_family = AF_INET; a.sin_addr.s_addr = htonl(INADDR_LOOPBACK); a.sin_port = htons((uint16_t)port);
  if (bind(s->listen_fd, (sockaddr*)&a, sizeof a) != 0 || listen(s->listen_fd, 64) != 0) { close(s->listen_fd); delete s; return nullptr; }
  socklen_t al = sizeof a; getsockname(s->listen_fd, (sockaddr*)&a, &al);
  s->port = ntohs(a.sin_port); if (bound_port) *bound_port = s->port;
  s->acceptor = std::thread([s] {
    while (!s->stop.load()) {
      if (!wait_fd(s->listen_fd, POLLIN, 100)) continue;
      int fd = accept(s->listen_fd, nullptr, nullptr);
      if (fd < 0) continue;
      int one = 1; setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one);
      std::lock_guard<std::mutex> g(s->mu);
      s->workers.emplace_back([s, fd] { s->serve(fd); });
    }
  });
  return s;
}
void b200_store_server_stop(void* h) {
  Server* s = (Server*)h; if (!s) return;
  s->stop.store(true); s->cv.notify_all();
  if (s->acceptor.joinable()) s->acceptor.join();
  std::vector<std::thread> ws; { std::lock_guard<std::mutex> g(s->mu); ws.swap(s->workers); }
  for (auto& t : ws) if (t.joinable()) t.join();
  close(s->listen_fd); delete s;
}

// ---- store client (one socket per client handle)
long long b200_store_connect(const char* host, int port, int timeout_ms) {
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (true) {
    int fd = socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return -1;
    sockaddr_in a{}; a.sin_family = AF_INET; a.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host, &a.sin_addr) != 1) { close(fd); return -1; }
    if (connect(fd, (sockaddr*)&a, sizeof a) == 0) { int one = 1; setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof one); return fd; }
    close(fd);
    if (std::chrono::steady_clock::now() >= deadline) return -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(20));
  }
}
void b200_store_close(long long fd) { if (fd >= 0) { send_frame((int)fd, Shutdown, nullptr, 0, 200); close((int)fd); } }

static std::vector<uint8_t> key_payload(const char* key, const uint8_t* extra, size_t n) {
  uint32_t kl = (uint32_t)strlen(key);
  std::vector<uint8_t> p(4 + kl + n);
  memcpy(p.data(), &kl, 4); memcpy(p.data() + 4, key, kl); if (n) memcpy(p.data() + 4 + kl, extra, n);
  return p;
}
int b200_store_set(long long fd, const char* key, const unsigned char* val, long long len, int timeout_ms) {
  auto p = key_payload(key, val, (size_t)len);
  if (!send_frame((int)fd, StoreSet, p.data(), (uint32_t)p.size(), timeout_ms)) return -1;
  uint8_t t; std::vector<uint8_t> r;
  return recv_frame((int)fd, t, r, timeout_ms) && t == StoreReply ? 0 : -1;
}
// returns value length, -2 when the key did not appear within wait_ms, -1 on a transport error
long long b200_store_get(long long fd, const char* key, unsigned char* out, long long cap, int wait_ms) {
  int32_t w = wait_ms;
  auto p = key_payload(key, (const uint8_t*)&w, 4);
  if (!send_frame((int)fd, StoreGet, p.data(), (uint32_t)p.size(), 5000)) return -1;
  uint8_t t; std::vector<uint8_t> r;
  if (!recv_frame((int)fd, t, r, wait_ms + 5000)) return -1;
  if (t == StoreMissing) return -2;
  if ((long long)r.size() > cap) return -1;
  if (!r.empty()) memcpy(out, r.data(), r.size());
  return (long long)r.size();
}
long long b200_store_add(long long fd, const char* key, long long delta, int timeout_ms) {
  int64_t d = delta;
  auto p = key_payload(key, (const uint8_t*)&d, 8);
  if (!send_frame((int)fd, StoreAdd, p.data(), (uint32_t)p.size(), timeout_ms)) return INT64_MIN;
  uint8_t t; std::vector<uint8_t> r;
  if (!recv_frame((int)fd, t, r, timeout_ms) || r.size() != 8) return INT64_MIN;
  int64_t v; memcpy(&v, r.data(), 8); return v;
}

}  // extern "C"
