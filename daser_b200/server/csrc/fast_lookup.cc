// Native read path of the control plane: a thread that answers `lookup_chunks {keys}` on a Unix
// socket of its own, without the Python interpreter.
//
// The reference serves every RPC from one asyncio loop (daser/server/ipc_server.py:113-164), and so
// does the Python server here: about 130 us per 8-key lookup and ~5k lookups/s in total, however
// many engines are attached.  The lookup by key is the RPC on the request path of a RAG engine
// (one per request: which of my chunks are stored, and where), it reads one small record per key
// and mutates nothing, so it is served here instead: an epoll loop, the same framing (4-byte
// big-endian length + msgpack map) and the same reply shape, a hash map under a reader/writer lock
// that the Python server updates when a chunk is committed, evicted or aborted.  Anything else a
// client sends on this socket is answered with an error frame and belongs on the main socket.
#include <arpa/inet.h>
#include <errno.h>
#include <fcntl.h>
#include <stdint.h>
#include <string.h>
#include <sys/epoll.h>
#include <sys/eventfd.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <mutex>
#include <shared_mutex>
#include <string>
#include <thread>
#include <unordered_map>
#include <vector>

#define DASER_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr size_t kMaxFrame = 16u << 20;  // a lookup by key is small; larger frames are refused

struct Rec {
  std::string model_id;
  int64_t start_slot, num_slots, token_count, pos_offset;
};

// ---- msgpack: just enough to read {"op": str, "keys": [str...], "model_id": str, ...} -------------
struct Reader {
  const uint8_t* p;
  const uint8_t* end;
  bool ok = true;
  bool need(size_t n) {
    if ((size_t)(end - p) < n) ok = false;
    return ok;
  }
  uint64_t be(int n) {
    uint64_t v = 0;
    if (!need((size_t)n)) return 0;
    for (int i = 0; i < n; ++i) v = (v << 8) | *p++;
    return v;
  }
  // str / bin header -> length, or -1 when the next object is something else (not consumed)
  int64_t str_len() {
    if (!need(1)) return -1;
    const uint8_t t = *p;
    if ((t & 0xE0) == 0xA0) { ++p; return t & 0x1F; }
    if (t == 0xD9 || t == 0xC4) { ++p; return (int64_t)be(1); }
    if (t == 0xDA || t == 0xC5) { ++p; return (int64_t)be(2); }
    if (t == 0xDB || t == 0xC6) { ++p; return (int64_t)be(4); }
    return -1;
  }
  bool read_str(std::string* out) {
    const int64_t n = str_len();
    if (n < 0 || !need((size_t)n)) { ok = false; return false; }
    out->assign((const char*)p, (size_t)n);
    p += n;
    return true;
  }
  int64_t array_len() {
    if (!need(1)) return -1;
    const uint8_t t = *p;
    if ((t & 0xF0) == 0x90) { ++p; return t & 0x0F; }
    if (t == 0xDC) { ++p; return (int64_t)be(2); }
    if (t == 0xDD) { ++p; return (int64_t)be(4); }
    return -1;
  }
  int64_t map_len() {
    if (!need(1)) return -1;
    const uint8_t t = *p;
    if ((t & 0xF0) == 0x80) { ++p; return t & 0x0F; }
    if (t == 0xDE) { ++p; return (int64_t)be(2); }
    if (t == 0xDF) { ++p; return (int64_t)be(4); }
    return -1;
  }
  void skip(int depth = 0) {  // any object
    if (depth > 32 || !need(1)) { ok = false; return; }
    const uint8_t t = *p;
    int64_t n;
    if (t <= 0x7F || t >= 0xE0 || t == 0xC0 || t == 0xC2 || t == 0xC3) { ++p; return; }
    if ((n = str_len()) >= 0) { if (need((size_t)n)) p += n; return; }
    if (!ok) return;
    if ((t & 0xF0) == 0x90 || t == 0xDC || t == 0xDD) {
      n = array_len();
      for (int64_t i = 0; i < n && ok; ++i) skip(depth + 1);
      return;
    }
    if ((t & 0xF0) == 0x80 || t == 0xDE || t == 0xDF) {
      n = map_len();
      for (int64_t i = 0; i < 2 * n && ok; ++i) skip(depth + 1);
      return;
    }
    ++p;
    switch (t) {
      case 0xCC: case 0xD0: if (need(1)) p += 1; return;
      case 0xCD: case 0xD1: if (need(2)) p += 2; return;
      case 0xCA: case 0xCE: case 0xD2: if (need(4)) p += 4; return;
      case 0xCB: case 0xCF: case 0xD3: if (need(8)) p += 8; return;
      case 0xD4: if (need(2)) p += 2; return;   // fixext 1
      case 0xD5: if (need(3)) p += 3; return;
      case 0xD6: if (need(5)) p += 5; return;
      case 0xD7: if (need(9)) p += 9; return;
      case 0xD8: if (need(17)) p += 17; return;
      case 0xC7: { const uint64_t m = be(1); if (need(m + 1)) p += m + 1; return; }
      case 0xC8: { const uint64_t m = be(2); if (need(m + 1)) p += m + 1; return; }
      case 0xC9: { const uint64_t m = be(4); if (need(m + 1)) p += m + 1; return; }
      default: ok = false;
    }
  }
};

struct Writer {
  std::string out;
  void u8(uint8_t v) { out.push_back((char)v); }
  void be(uint64_t v, int n) { for (int i = n - 1; i >= 0; --i) u8((uint8_t)(v >> (8 * i))); }
  void nil() { u8(0xC0); }
  void map(uint32_t n) { if (n < 16) u8(0x80 | n); else { u8(0xDE); be(n, 2); } }
  void array(uint32_t n) { if (n < 16) u8(0x90 | n); else if (n < 65536) { u8(0xDC); be(n, 2); } else { u8(0xDD); be(n, 4); } }
  void str(const char* s, size_t n) {
    if (n < 32) u8(0xA0 | (uint8_t)n); else if (n < 256) { u8(0xD9); be(n, 1); } else if (n < 65536) { u8(0xDA); be(n, 2); } else { u8(0xDB); be(n, 4); }
    out.append(s, n);
  }
  void str(const std::string& s) { str(s.data(), s.size()); }
  void lit(const char* s) { str(s, strlen(s)); }
  void i64(int64_t v) {
    if (v >= 0 && v < 128) u8((uint8_t)v);
    else if (v >= 0 && v <= 0xFFFFFFFFll) { u8(0xCE); be((uint64_t)v, 4); }
    else if (v >= 0) { u8(0xCF); be((uint64_t)v, 8); }
    else { u8(0xD3); be((uint64_t)v, 8); }
  }
};

struct Conn {
  int fd;
  std::string in;   // bytes received, not yet a whole frame
  std::string out;  // bytes of replies not yet written
};

}  // namespace

struct daser_fast {
  std::unordered_map<std::string, Rec> recs;
  std::shared_mutex mu;
  int64_t slot_size = 0;
  int listen_fd = -1, ep = -1, wake = -1;
  std::thread th;
  std::atomic<bool> stop{false};
  std::atomic<uint64_t> calls{0}, hits{0}, misses{0}, refused{0};
  std::string path;
  std::unordered_map<int, Conn> conns;

  void reply_error(Conn& c, const char* what) {
    Writer w;
    w.map(1);
    w.lit("error");
    w.lit(what);
    frame(c, w.out);
  }
  static void frame(Conn& c, const std::string& body) {
    const uint32_t n = htonl((uint32_t)body.size());
    c.out.append((const char*)&n, 4);
    c.out.append(body);
  }

  void handle(Conn& c, const uint8_t* body, size_t n) {
    calls.fetch_add(1, std::memory_order_relaxed);
    Reader r{body, body + n};
    const int64_t fields = r.map_len();
    if (fields < 0) return reply_error(c, "ProtocolError: request is not a map");
    std::string op, model = "default", key;
    std::vector<std::string> keys;
    bool have_keys = false, other_query = false;
    for (int64_t i = 0; i < fields && r.ok; ++i) {
      if (!r.read_str(&key)) break;
      if (key == "op") r.read_str(&op);
      else if (key == "model_id") r.read_str(&model);
      else if (key == "keys") {
        const int64_t m = r.array_len();
        if (m < 0 || m > r.end - r.p) { r.ok = false; break; }  // every key takes a byte at least
        have_keys = true;
        keys.resize((size_t)m);
        for (int64_t j = 0; j < m && r.ok; ++j) r.read_str(&keys[(size_t)j]);
      } else {
        if (key == "tokens" || key == "tokens_bin") other_query = true;
        r.skip();
      }
    }
    if (!r.ok) return reply_error(c, "ProtocolError: malformed request");
    if (op != "lookup_chunks" || !have_keys || other_query) {
      refused.fetch_add(1, std::memory_order_relaxed);
      return reply_error(c, "ProtocolError: only lookup_chunks by keys is served on the fast socket");
    }
    Writer w;
    w.map(1);
    w.lit("chunks");
    w.array((uint32_t)keys.size());
    uint64_t h = 0, m = 0;
    {
      std::shared_lock<std::shared_mutex> g(mu);
      for (const std::string& k : keys) {
        auto it = recs.find(k);
        if (it == recs.end() || it->second.model_id != model) { w.nil(); ++m; continue; }
        const Rec& rec = it->second;
        ++h;
        w.map(7);
        w.lit("chunk_key"); w.str(k);
        w.lit("start_slot"); w.i64(rec.start_slot);
        w.lit("num_slots"); w.i64(rec.num_slots);
        w.lit("token_count"); w.i64(rec.token_count);
        w.lit("pos_offset"); w.i64(rec.pos_offset);
        w.lit("model_id"); w.str(rec.model_id);
        w.lit("file_offset"); w.i64(rec.start_slot * slot_size);
      }
    }
    hits.fetch_add(h, std::memory_order_relaxed);
    misses.fetch_add(m, std::memory_order_relaxed);
    frame(c, w.out);
  }

  // returns false when the connection is to be closed
  bool on_readable(Conn& c) {
    char buf[65536];
    for (;;) {
      const ssize_t n = recv(c.fd, buf, sizeof buf, 0);
      if (n > 0) { c.in.append(buf, (size_t)n); continue; }
      if (n == 0) return false;
      if (errno == EAGAIN || errno == EWOULDBLOCK) break;
      if (errno == EINTR) continue;
      return false;
    }
    size_t off = 0;
    while (c.in.size() - off >= 4) {
      uint32_t len;
      memcpy(&len, c.in.data() + off, 4);
      len = ntohl(len);
      if (len > kMaxFrame) return false;
      if (c.in.size() - off - 4 < len) break;
      handle(c, (const uint8_t*)c.in.data() + off + 4, len);
      off += 4 + (size_t)len;
    }
    c.in.erase(0, off);
    return flush(c);
  }
  bool flush(Conn& c) {
    while (!c.out.empty()) {
      const ssize_t n = send(c.fd, c.out.data(), c.out.size(), MSG_NOSIGNAL);
      if (n > 0) { c.out.erase(0, (size_t)n); continue; }
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) break;
      return false;
    }
    epoll_event ev{};
    ev.events = EPOLLIN | (c.out.empty() ? 0u : (uint32_t)EPOLLOUT);
    ev.data.fd = c.fd;
    epoll_ctl(ep, EPOLL_CTL_MOD, c.fd, &ev);
    return true;
  }
  void drop(int fd) {
    epoll_ctl(ep, EPOLL_CTL_DEL, fd, nullptr);
    close(fd);
    conns.erase(fd);
  }

  void run() {
    epoll_event evs[64];
    while (!stop.load(std::memory_order_acquire)) {
      const int n = epoll_wait(ep, evs, 64, 500);
      if (n < 0 && errno != EINTR) break;
      for (int i = 0; i < n; ++i) {
        const int fd = evs[i].data.fd;
        if (fd == wake) continue;  // stop is re-read by the loop condition
        if (fd == listen_fd) {
          for (;;) {
            const int cfd = accept4(listen_fd, nullptr, nullptr, SOCK_NONBLOCK | SOCK_CLOEXEC);
            if (cfd < 0) break;
            epoll_event ev{};
            ev.events = EPOLLIN;
            ev.data.fd = cfd;
            if (epoll_ctl(ep, EPOLL_CTL_ADD, cfd, &ev) != 0) { close(cfd); continue; }
            conns[cfd] = Conn{cfd, {}, {}};
          }
          continue;
        }
        auto it = conns.find(fd);
        if (it == conns.end()) continue;
        bool keep = true;
        if (evs[i].events & (EPOLLHUP | EPOLLERR)) keep = false;
        if (keep && (evs[i].events & EPOLLIN)) keep = on_readable(it->second);
        if (keep && (evs[i].events & EPOLLOUT)) keep = flush(it->second);
        if (!keep) drop(fd);
      }
    }
    std::vector<int> open_fds;
    for (auto& kv : conns) open_fds.push_back(kv.first);
    for (int fd : open_fds) drop(fd);
  }
};

// Starts the thread; returns null when the socket cannot be bound.
DASER_API daser_fast* daser_fast_start(const char* socket_path, int64_t slot_size) {
  if (!socket_path || slot_size <= 0) return nullptr;
  sockaddr_un addr{};
  addr.sun_family = AF_UNIX;
  if (strlen(socket_path) >= sizeof(addr.sun_path)) return nullptr;
  strcpy(addr.sun_path, socket_path);
  const int fd = socket(AF_UNIX, SOCK_STREAM | SOCK_NONBLOCK | SOCK_CLOEXEC, 0);
  if (fd < 0) return nullptr;
  unlink(socket_path);  // a stale socket of an earlier run
  if (bind(fd, (sockaddr*)&addr, sizeof addr) != 0 || listen(fd, 256) != 0) {
    close(fd);
    return nullptr;
  }
  daser_fast* f = new daser_fast();
  f->slot_size = slot_size;
  f->path = socket_path;
  f->listen_fd = fd;
  f->ep = epoll_create1(EPOLL_CLOEXEC);
  f->wake = eventfd(0, EFD_NONBLOCK | EFD_CLOEXEC);
  epoll_event ev{};
  ev.events = EPOLLIN;
  ev.data.fd = fd;
  epoll_ctl(f->ep, EPOLL_CTL_ADD, fd, &ev);
  ev.data.fd = f->wake;
  epoll_ctl(f->ep, EPOLL_CTL_ADD, f->wake, &ev);
  f->th = std::thread([f] { f->run(); });
  return f;
}

DASER_API void daser_fast_stop(daser_fast* f) {
  if (!f) return;
  f->stop.store(true, std::memory_order_release);
  const uint64_t one = 1;
  if (write(f->wake, &one, 8) < 0) { /* the loop also wakes by its time limit */ }
  if (f->th.joinable()) f->th.join();
  close(f->listen_fd);
  close(f->wake);
  close(f->ep);
  unlink(f->path.c_str());
  delete f;
}

DASER_API int daser_fast_put(daser_fast* f, const char* key, const char* model_id, int64_t start_slot,
                             int64_t num_slots, int64_t token_count, int64_t pos_offset) {
  if (!f || !key || !model_id) return -1;
  std::unique_lock<std::shared_mutex> g(f->mu);
  f->recs[key] = Rec{model_id, start_slot, num_slots, token_count, pos_offset};
  return 0;
}

DASER_API int daser_fast_del(daser_fast* f, const char* key) {
  if (!f || !key) return -1;
  std::unique_lock<std::shared_mutex> g(f->mu);
  return (int)f->recs.erase(key);
}

DASER_API void daser_fast_clear(daser_fast* f) {
  if (!f) return;
  std::unique_lock<std::shared_mutex> g(f->mu);
  f->recs.clear();
}

// out[0..5) = records, calls, hits, misses, refused
DASER_API void daser_fast_stats(daser_fast* f, int64_t* out) {
  if (!f || !out) return;
  {
    std::shared_lock<std::shared_mutex> g(f->mu);
    out[0] = (int64_t)f->recs.size();
  }
  out[1] = (int64_t)f->calls.load();
  out[2] = (int64_t)f->hits.load();
  out[3] = (int64_t)f->misses.load();
  out[4] = (int64_t)f->refused.load();
}
