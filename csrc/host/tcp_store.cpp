// TCP key-value store for rendezvous: C++ server + client.
//
// Wire format (crates/torsh-distributed/src/store/tcp.rs:38-76,99-200): every message is a 4-byte
// big-endian length (1 .. 100 MiB) followed by the bincode-standard encoding of
//   StoreMessage  { Set{key,value}, Get{key}, Wait{keys}, Delete{key}, NumKeys, Contains{key},
//                   SetWithExpiry{key,value,ttl_secs}, CompareAndSwap{key,expected:Option,value}, Add{key,i64} }
//   StoreResponse { Ok, Value(Option<bytes>), NumKeys(usize), Bool(bool), I64(i64), Error(String) }
// Expiry is checked lazily on access; Wait blocks on a condition variable until every key exists.
// The server runs one thread per connection (rendezvous traffic is a handful of small messages per rank).
#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdlib>
#include <map>
#include <mutex>
#include <thread>
#include <vector>

#include "bincode.h"
#include "host_api.h"

namespace tsh {

using Clock = std::chrono::steady_clock;
constexpr uint32_t MAX_MSG = 100u * 1024 * 1024;

static bool send_all(int fd, const void* p, size_t n) {
  const uint8_t* b = static_cast<const uint8_t*>(p);
  while (n) {
    ssize_t k = ::send(fd, b, n, MSG_NOSIGNAL);
    if (k <= 0) return false;
    b += k;
    n -= (size_t)k;
  }
  return true;
}
static bool recv_all(int fd, void* p, size_t n) {
  uint8_t* b = static_cast<uint8_t*>(p);
  while (n) {
    ssize_t k = ::recv(fd, b, n, 0);
    if (k <= 0) return false;
    b += k;
    n -= (size_t)k;
  }
  return true;
}
static bool send_frame(int fd, const std::vector<uint8_t>& body) {
  uint32_t be = htonl((uint32_t)body.size());
  return send_all(fd, &be, 4) && send_all(fd, body.data(), body.size());
}
static bool recv_frame(int fd, std::vector<uint8_t>& body) {
  uint32_t be;
  if (!recv_all(fd, &be, 4)) return false;
  uint32_t n = ntohl(be);
  if (n == 0 || n > MAX_MSG) return false;
  body.resize(n);
  return recv_all(fd, body.data(), n);
}

struct Entry {
  std::vector<uint8_t> value;
  bool has_expiry = false;
  Clock::time_point expiry;
};

struct Server {
  int listen_fd = -1;
  int port = 0;
  std::atomic<bool> stop{false};
  std::thread accept_thread;
  std::mutex mu;
  std::condition_variable cv;
  std::map<std::string, Entry> kv;
  std::vector<std::thread> workers;
  std::vector<int> client_fds;

  bool alive(const std::string& k) {  // caller holds mu
    auto it = kv.find(k);
    if (it == kv.end()) return false;
    if (it->second.has_expiry && Clock::now() >= it->second.expiry) {
      kv.erase(it);
      return false;
    }
    return true;
  }

  std::vector<uint8_t> handle(Reader& r) {
    Writer w;
    uint64_t op = r.varu();
    std::unique_lock<std::mutex> lk(mu);
    switch (op) {
      case 0: {  // Set
        std::string k = r.str();
        Entry e;
        e.value = r.bytes();
        kv[k] = std::move(e);
        cv.notify_all();
        w.varu(0);
        break;
      }
      case 1: {  // Get
        std::string k = r.str();
        w.varu(1);
        if (alive(k)) {
          w.u8(1);
          w.bytes(kv[k].value.data(), kv[k].value.size());
        } else {
          w.u8(0);
        }
        break;
      }
      case 2: {  // Wait
        uint64_t n = r.varu();
        std::vector<std::string> keys;
        for (uint64_t i = 0; i < n; ++i) keys.push_back(r.str());
        auto all = [&] {
          for (auto& k : keys)
            if (!alive(k)) return false;
          return true;
        };
        while (!all() && !stop.load()) cv.wait_for(lk, std::chrono::milliseconds(100));
        if (stop.load() && !all()) {
          w.varu(5);
          w.str("store is shutting down");
        } else {
          w.varu(0);
        }
        break;
      }
      case 3: {  // Delete
        kv.erase(r.str());
        w.varu(0);
        break;
      }
      case 4: {  // NumKeys
        for (auto it = kv.begin(); it != kv.end();) {
          if (it->second.has_expiry && Clock::now() >= it->second.expiry) it = kv.erase(it); else ++it;
        }
        w.varu(2);
        w.varu(kv.size());
        break;
      }
      case 5: {  // Contains
        w.varu(3);
        w.boolean(alive(r.str()));
        break;
      }
      case 6: {  // SetWithExpiry
        std::string k = r.str();
        Entry e;
        e.value = r.bytes();
        uint64_t ttl = r.varu();
        e.has_expiry = true;
        e.expiry = Clock::now() + std::chrono::seconds(ttl);
        kv[k] = std::move(e);
        cv.notify_all();
        w.varu(0);
        break;
      }
      case 7: {  // CompareAndSwap
        std::string k = r.str();
        bool has_expected = r.u8() == 1;
        std::vector<uint8_t> expected;
        if (has_expected) expected = r.bytes();
        std::vector<uint8_t> value = r.bytes();
        bool present = alive(k);
        bool match = has_expected ? (present && kv[k].value == expected) : !present;
        if (match) {
          Entry e;
          e.value = std::move(value);
          kv[k] = std::move(e);
          cv.notify_all();
        }
        w.varu(3);
        w.boolean(match);
        break;
      }
      case 8: {  // Add
        std::string k = r.str();
        int64_t delta = r.vari();
        int64_t cur = 0;
        if (alive(k)) {
          const auto& v = kv[k].value;
          if (v.size() == 8) memcpy(&cur, v.data(), 8);
          else { try { cur = std::stoll(std::string(v.begin(), v.end())); } catch (...) { cur = 0; } }
        }
        cur += delta;
        Entry e;
        e.value.resize(8);
        memcpy(e.value.data(), &cur, 8);
        kv[k] = std::move(e);
        cv.notify_all();
        w.varu(4);
        w.vari(cur);
        break;
      }
      default:
        w.varu(5);
        w.str("unknown store operation");
    }
    return w.buf;
  }

  void serve(int fd) {
    std::vector<uint8_t> body;
    while (!stop.load() && recv_frame(fd, body)) {
      std::vector<uint8_t> resp;
      try {
        Reader r(body.data(), body.size());
        resp = handle(r);
      } catch (const std::exception& e) {
        Writer w;
        w.varu(5);
        w.str(e.what());
        resp = w.buf;
      }
      if (!send_frame(fd, resp)) break;
    }
    ::close(fd);
  }

  void accept_loop() {
    while (!stop.load()) {
      pollfd p{listen_fd, POLLIN, 0};
      int r = ::poll(&p, 1, 100);
      if (r <= 0) continue;
      int fd = ::accept(listen_fd, nullptr, nullptr);
      if (fd < 0) continue;
      int one = 1;
      setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      std::lock_guard<std::mutex> lk(mu);
      client_fds.push_back(fd);
      workers.emplace_back([this, fd] { serve(fd); });
    }
  }
};

struct Client {
  int fd = -1;
  std::mutex mu;
  std::string host;
  int port = 0;
  int timeout_ms = 30000;

  bool connect_once() {
    fd = ::socket(AF_INET, SOCK_STREAM, 0);
    if (fd < 0) return false;
    sockaddr_in a{};
    a.sin_family = AF_INET;
    a.sin_port = htons((uint16_t)port);
    if (inet_pton(AF_INET, host.c_str(), &a.sin_addr) != 1) { ::close(fd); fd = -1; return false; }
    if (::connect(fd, (sockaddr*)&a, sizeof(a)) != 0) { ::close(fd); fd = -1; return false; }
    int one = 1;
    setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    return true;
  }
  bool connect_retry() {
    auto deadline = Clock::now() + std::chrono::milliseconds(timeout_ms);
    int backoff = 10;
    while (Clock::now() < deadline) {
      if (connect_once()) return true;
      std::this_thread::sleep_for(std::chrono::milliseconds(backoff));
      backoff = backoff * 2 > 500 ? 500 : backoff * 2;
    }
    return false;
  }
  void set_recv_timeout(int ms) {
    timeval tv{ms / 1000, (ms % 1000) * 1000};
    setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof(tv));
  }
  // Returns false on transport failure / timeout (connection is re-established for the next call).
  bool roundtrip(const std::vector<uint8_t>& req, std::vector<uint8_t>& resp, int wait_ms) {
    std::lock_guard<std::mutex> lk(mu);
    if (fd < 0 && !connect_retry()) { g_err = "store: cannot connect to " + host + ":" + std::to_string(port); return false; }
    set_recv_timeout(wait_ms > 0 ? wait_ms : timeout_ms);
    if (!send_frame(fd, req) || !recv_frame(fd, resp)) {
      ::close(fd);
      fd = -1;
      g_err = "store: request timed out or connection lost";
      return false;
    }
    return true;
  }
};

static int expect_ok(Reader& r) {
  uint64_t tag = r.varu();
  if (tag == 0) return 0;
  if (tag == 5) { g_err = "store error: " + r.str(); return -2; }
  g_err = "store: unexpected response variant";
  return -3;
}

}  // namespace tsh
using namespace tsh;

TSH_EXPORT void* tsh_store_server_start(const char* host, int port, int* bound_port) {
  Server* s = new Server();
  s->listen_fd = ::socket(AF_INET, SOCK_STREAM, 0);
  int one = 1;
  setsockopt(s->listen_fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)port);
  if (inet_pton(AF_INET, host, &a.sin_addr) != 1) a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  if (::bind(s->listen_fd, (sockaddr*)&a, sizeof(a)) != 0 || ::listen(s->listen_fd, 256) != 0) {
    g_err = "store: cannot bind/listen on " + std::string(host) + ":" + std::to_string(port);
    ::close(s->listen_fd);
    delete s;
    return nullptr;
  }
  socklen_t len = sizeof(a);
  getsockname(s->listen_fd, (sockaddr*)&a, &len);
  s->port = ntohs(a.sin_port);
  if (bound_port) *bound_port = s->port;
  s->accept_thread = std::thread([s] { s->accept_loop(); });
  return s;
}
TSH_EXPORT void tsh_store_server_stop(void* h) {
  Server* s = static_cast<Server*>(h);
  if (!s) return;
  s->stop.store(true);
  s->cv.notify_all();
  if (s->accept_thread.joinable()) s->accept_thread.join();
  {
    std::lock_guard<std::mutex> lk(s->mu);
    for (int fd : s->client_fds) ::shutdown(fd, SHUT_RDWR);
  }
  for (auto& t : s->workers)
    if (t.joinable()) t.join();
  ::close(s->listen_fd);
  delete s;
}
TSH_EXPORT void* tsh_store_client_connect(const char* host, int port, int timeout_ms) {
  Client* c = new Client();
  c->host = host;
  c->port = port;
  c->timeout_ms = timeout_ms > 0 ? timeout_ms : 30000;
  if (!c->connect_retry()) {
    g_err = "store: cannot connect to " + c->host + ":" + std::to_string(port);
    delete c;
    return nullptr;
  }
  return c;
}
TSH_EXPORT void tsh_store_client_close(void* h) {
  Client* c = static_cast<Client*>(h);
  if (!c) return;
  if (c->fd >= 0) ::close(c->fd);
  delete c;
}
TSH_EXPORT int tsh_store_set(void* h, const char* key, const uint8_t* val, uint64_t n, int64_t ttl_secs) {
  Writer w;
  if (ttl_secs >= 0) { w.varu(6); w.str(key); w.bytes(val, n); w.varu((uint64_t)ttl_secs); }
  else { w.varu(0); w.str(key); w.bytes(val, n); }
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, 0)) return -1;
  Reader r(resp.data(), resp.size());
  return expect_ok(r);
}
// returns 1 when found (*out malloc'd), 0 when absent, < 0 on error
TSH_EXPORT int tsh_store_get(void* h, const char* key, uint8_t** out, uint64_t* n) {
  Writer w;
  w.varu(1);
  w.str(key);
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, 0)) return -1;
  try {
    Reader r(resp.data(), resp.size());
    uint64_t tag = r.varu();
    if (tag == 5) { g_err = "store error: " + r.str(); return -2; }
    if (tag != 1) { g_err = "store: unexpected response variant"; return -3; }
    if (r.u8() == 0) return 0;
    std::vector<uint8_t> v = r.bytes();
    *out = static_cast<uint8_t*>(malloc(v.size() ? v.size() : 1));
    memcpy(*out, v.data(), v.size());
    *n = v.size();
    return 1;
  } catch (const std::exception& e) { g_err = e.what(); return -4; }
}
// returns 0 when all keys exist, -1 on timeout / transport error
TSH_EXPORT int tsh_store_wait(void* h, const char** keys, int nkeys, int timeout_ms) {
  Writer w;
  w.varu(2);
  w.varu((uint64_t)nkeys);
  for (int i = 0; i < nkeys; ++i) w.str(keys[i]);
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, timeout_ms)) return -1;
  Reader r(resp.data(), resp.size());
  return expect_ok(r);
}
TSH_EXPORT int tsh_store_delete(void* h, const char* key) {
  Writer w;
  w.varu(3);
  w.str(key);
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, 0)) return -1;
  Reader r(resp.data(), resp.size());
  return expect_ok(r);
}
TSH_EXPORT int64_t tsh_store_num_keys(void* h) {
  Writer w;
  w.varu(4);
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, 0)) return -1;
  Reader r(resp.data(), resp.size());
  if (r.varu() != 2) return -3;
  return (int64_t)r.varu();
}
TSH_EXPORT int tsh_store_contains(void* h, const char* key) {
  Writer w;
  w.varu(5);
  w.str(key);
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, 0)) return -1;
  Reader r(resp.data(), resp.size());
  if (r.varu() != 3) return -3;
  return r.boolean() ? 1 : 0;
}
// expected == nullptr means "only if absent". returns 1 swapped, 0 not swapped, < 0 error
TSH_EXPORT int tsh_store_cas(void* h, const char* key, const uint8_t* expected, uint64_t en, int has_expected,
                             const uint8_t* val, uint64_t n) {
  Writer w;
  w.varu(7);
  w.str(key);
  if (has_expected) { w.u8(1); w.bytes(expected, en); } else { w.u8(0); }
  w.bytes(val, n);
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, 0)) return -1;
  Reader r(resp.data(), resp.size());
  if (r.varu() != 3) return -3;
  return r.boolean() ? 1 : 0;
}
TSH_EXPORT int tsh_store_add(void* h, const char* key, int64_t delta, int64_t* result) {
  Writer w;
  w.varu(8);
  w.str(key);
  w.vari(delta);
  std::vector<uint8_t> resp;
  if (!static_cast<Client*>(h)->roundtrip(w.buf, resp, 0)) return -1;
  Reader r(resp.data(), resp.size());
  if (r.varu() != 4) return -3;
  *result = r.vari();
  return 0;
}
