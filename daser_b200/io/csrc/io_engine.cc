// Implementation of the storage engine declared in io_engine.h.
#include "io_engine.h"

#include <dlfcn.h>
#include <errno.h>
#include <fcntl.h>
#include <linux/io_uring.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <sys/types.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <condition_variable>
#include <cstdio>
#include <deque>
#include <mutex>
#include <thread>
#include <unordered_map>
#include <vector>

namespace {

constexpr int64_t kPieceBytes = 2 << 20;
constexpr int64_t kDirectAlign = 4096;

struct Piece {
  int64_t ticket;
  bool write;
  bool device;
  char* buf;
  int64_t off;
  int64_t len;
};

struct TicketState {
  int pending = 0;
  int error = 0;
};

// ---- cuFile, loaded at run time -------------------------------------------------------------
struct CuFileApi {
  // Minimal mirror of cufile.h (types reduced to what is passed through).
  struct Error { int err; int cu_err; };
  struct Descr { int type; union { int fd; void* handle; } handle; const void* fs_ops; };
  void* lib = nullptr;
  Error (*driver_open)() = nullptr;
  Error (*driver_close)() = nullptr;
  Error (*handle_register)(void**, Descr*) = nullptr;
  void (*handle_deregister)(void*) = nullptr;
  ssize_t (*read)(void*, void*, size_t, off_t, off_t) = nullptr;
  ssize_t (*write)(void*, const void*, size_t, off_t, off_t) = nullptr;
  int (*cuda_set_device)(int) = nullptr;

  bool load() {
    lib = dlopen("libcufile.so.0", RTLD_NOW | RTLD_LOCAL);
    if (!lib) lib = dlopen("libcufile.so", RTLD_NOW | RTLD_LOCAL);
    if (!lib) return false;
    driver_open = (Error(*)())dlsym(lib, "cuFileDriverOpen");
    driver_close = (Error(*)())dlsym(lib, "cuFileDriverClose");
    handle_register = (Error(*)(void**, Descr*))dlsym(lib, "cuFileHandleRegister");
    handle_deregister = (void (*)(void*))dlsym(lib, "cuFileHandleDeregister");
    read = (ssize_t(*)(void*, void*, size_t, off_t, off_t))dlsym(lib, "cuFileRead");
    write = (ssize_t(*)(void*, const void*, size_t, off_t, off_t))dlsym(lib, "cuFileWrite");
    void* rt = dlopen("libcudart.so.12", RTLD_NOW | RTLD_GLOBAL);
    if (!rt) rt = dlopen("libcudart.so", RTLD_NOW | RTLD_GLOBAL);
    if (rt) cuda_set_device = (int (*)(int))dlsym(rt, "cudaSetDevice");
    return driver_open && handle_register && handle_deregister && read && write;
  }
};

// ---- raw io_uring ------------------------------------------------------------------------------
struct Uring {
  int fd = -1;
  unsigned entries = 0;
  void* sq_ring = MAP_FAILED;
  void* cq_ring = MAP_FAILED;
  size_t sq_ring_sz = 0, cq_ring_sz = 0, sqes_sz = 0;
  io_uring_sqe* sqes = (io_uring_sqe*)MAP_FAILED;
  unsigned *sq_head = nullptr, *sq_tail = nullptr, *sq_mask = nullptr, *sq_array = nullptr;
  unsigned *cq_head = nullptr, *cq_tail = nullptr, *cq_mask = nullptr;
  io_uring_cqe* cqes = nullptr;

  bool setup(unsigned want) {
    io_uring_params p;
    memset(&p, 0, sizeof(p));
    fd = (int)syscall(__NR_io_uring_setup, want, &p);
    if (fd < 0) return false;
    entries = p.sq_entries;
    sq_ring_sz = p.sq_off.array + p.sq_entries * sizeof(unsigned);
    cq_ring_sz = p.cq_off.cqes + p.cq_entries * sizeof(io_uring_cqe);
    sqes_sz = p.sq_entries * sizeof(io_uring_sqe);
    sq_ring = mmap(nullptr, sq_ring_sz, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_SQ_RING);
    cq_ring = mmap(nullptr, cq_ring_sz, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_CQ_RING);
    sqes = (io_uring_sqe*)mmap(nullptr, sqes_sz, PROT_READ | PROT_WRITE, MAP_SHARED | MAP_POPULATE, fd, IORING_OFF_SQES);
    if (sq_ring == MAP_FAILED || cq_ring == MAP_FAILED || sqes == (io_uring_sqe*)MAP_FAILED) {
      teardown();
      return false;
    }
    char* s = (char*)sq_ring;
    sq_head = (unsigned*)(s + p.sq_off.head);
    sq_tail = (unsigned*)(s + p.sq_off.tail);
    sq_mask = (unsigned*)(s + p.sq_off.ring_mask);
    sq_array = (unsigned*)(s + p.sq_off.array);
    char* c = (char*)cq_ring;
    cq_head = (unsigned*)(c + p.cq_off.head);
    cq_tail = (unsigned*)(c + p.cq_off.tail);
    cq_mask = (unsigned*)(c + p.cq_off.ring_mask);
    cqes = (io_uring_cqe*)(c + p.cq_off.cqes);
    return true;
  }

  // Pin and map `n` buffers once (IORING_REGISTER_BUFFERS): fixed reads / writes into them skip
  // the per-IO page lookup.  One registration per ring; returns 0 or -errno.
  int register_buffers(const iovec* iov, unsigned n) {
    const long r = syscall(__NR_io_uring_register, fd, IORING_REGISTER_BUFFERS, iov, n);
    return r < 0 ? -errno : 0;
  }

  void teardown() {
    if (sq_ring != MAP_FAILED) munmap(sq_ring, sq_ring_sz);
    if (cq_ring != MAP_FAILED) munmap(cq_ring, cq_ring_sz);
    if (sqes != (io_uring_sqe*)MAP_FAILED) munmap(sqes, sqes_sz);
    sq_ring = cq_ring = MAP_FAILED;
    sqes = (io_uring_sqe*)MAP_FAILED;
    if (fd >= 0) close(fd);
    fd = -1;
  }

  // Caller holds the submit lock and has checked that a slot is free.
  bool push(int opcode, int file_fd, void* buf, unsigned len, int64_t off, uint64_t user_data, int buf_index = -1) {
    const unsigned tail = *sq_tail;
    const unsigned idx = tail & *sq_mask;
    io_uring_sqe* e = &sqes[idx];
    memset(e, 0, sizeof(*e));
    e->opcode = (uint8_t)opcode;
    e->fd = file_fd;
    e->addr = (uint64_t)(uintptr_t)buf;
    e->len = len;
    e->off = (uint64_t)off;
    e->user_data = user_data;
    if (buf_index >= 0) e->buf_index = (uint16_t)buf_index;  // READ_FIXED / WRITE_FIXED
    sq_array[idx] = idx;
    __atomic_store_n(sq_tail, tail + 1, __ATOMIC_RELEASE);
    for (;;) {
      const long r = syscall(__NR_io_uring_enter, fd, 1, 0, 0, nullptr, 0);
      if (r >= 0) return true;
      if (errno == EINTR || errno == EAGAIN || errno == EBUSY) continue;
      return false;
    }
  }
};

}  // namespace

struct daser_io {
  int backend = DASER_IO_POSIX;
  int fd = -1;         // buffered
  int fd_direct = -1;  // O_DIRECT, -1 when the filesystem refuses it
  int device = -1;
  int64_t file_size = 0;

  std::mutex mu;
  std::condition_variable cv;
  std::unordered_map<int64_t, TicketState> tickets;
  int64_t next_ticket = 1;
  bool closing = false;

  // worker pool (POSIX and GDS)
  std::deque<Piece> queue;
  std::condition_variable queue_cv;
  std::vector<std::thread> workers;

  // io_uring
  Uring ring;
  std::mutex ring_mu;  // guards SQ, backlog and inflight
  std::deque<Piece*> backlog;
  unsigned inflight = 0;
  unsigned depth = 64;
  struct Region { uintptr_t base; size_t len; int index; };
  std::vector<Region> fixed;  // registered buffers (written once, before any IO that uses them)
  std::atomic<int64_t> st_fixed{0};
  std::condition_variable_any ring_idle_cv;  // signalled when inflight and backlog both reach zero
  std::thread reaper;

  // cuFile
  CuFileApi cf;
  void* cf_handle = nullptr;

  // fault injection
  std::atomic<int> inject_count{0};
  std::atomic<int> inject_errno{0};
  std::atomic<int64_t> inject_short{-1};

  std::atomic<int64_t> st_pieces{0}, st_read{0}, st_written{0}, st_resubmits{0}, st_direct{0};

  bool direct_ok(const Piece& p) const {
    return fd_direct >= 0 && !p.device && p.off % kDirectAlign == 0 && p.len % kDirectAlign == 0 &&
           ((uintptr_t)p.buf) % kDirectAlign == 0;
  }

  void finish(int64_t ticket, int error) {
    std::lock_guard<std::mutex> g(mu);
    auto it = tickets.find(ticket);
    if (it == tickets.end()) return;
    if (error && !it->second.error) it->second.error = error;
    if (--it->second.pending <= 0) cv.notify_all();
  }

  // Returns true and fills (err, cut) when a fault should be injected into this piece.
  bool take_injection(int* err, int64_t* cut) {
    int c = inject_count.load();
    while (c > 0) {
      if (inject_count.compare_exchange_weak(c, c - 1)) {
        *err = inject_errno.load();
        *cut = inject_short.load();
        return true;
      }
    }
    return false;
  }

  // ---- worker pool --------------------------------------------------------------------------
  void run_piece_sync(Piece p) {
    int64_t done = 0;
    while (done < p.len) {
      Piece rest = p;
      rest.buf += done;
      rest.off += done;
      rest.len -= done;
      int64_t want = rest.len;
      int inj_err = 0;
      int64_t inj_cut = -1;
      if (take_injection(&inj_err, &inj_cut)) {
        if (inj_err > 0) { finish(p.ticket, -inj_err); return; }
        if (inj_cut >= 0 && inj_cut < want) want = inj_cut > 0 ? inj_cut : 1;
      }
      ssize_t n;
      if (backend == DASER_IO_GDS && p.device) {
        n = p.write ? cf.write(cf_handle, rest.buf, (size_t)want, (off_t)rest.off, 0)
                    : cf.read(cf_handle, rest.buf, (size_t)want, (off_t)rest.off, 0);
        if (n < 0) { finish(p.ticket, n == -1 ? -errno : -EIO); return; }
      } else {
        const bool direct = want == rest.len && direct_ok(rest);
        const int f = direct ? fd_direct : fd;
        if (direct) st_direct++;
        n = p.write ? pwrite(f, rest.buf, (size_t)want, (off_t)rest.off)
                    : pread(f, rest.buf, (size_t)want, (off_t)rest.off);
        if (n < 0) {
          if (errno == EINTR) continue;
          finish(p.ticket, -errno);
          return;
        }
      }
      if (n == 0) { finish(p.ticket, -ENODATA); return; }  // read past the end of the file
      if (n < rest.len) st_resubmits++;
      done += n;
    }
    (p.write ? st_written : st_read) += p.len;
    finish(p.ticket, 0);
  }

  void worker_loop() {
    if (backend == DASER_IO_GDS && device >= 0 && cf.cuda_set_device) cf.cuda_set_device(device);
    for (;;) {
      Piece p;
      {
        std::unique_lock<std::mutex> g(mu);
        queue_cv.wait(g, [&] { return closing || !queue.empty(); });
        if (queue.empty()) return;
        p = queue.front();
        queue.pop_front();
      }
      run_piece_sync(p);
    }
  }

  // ---- io_uring -----------------------------------------------------------------------------------
  // ring_mu held.
  int fixed_index(const Piece& p) const {
    const uintptr_t a = (uintptr_t)p.buf;
    for (const Region& r : fixed)
      if (a >= r.base && a + (size_t)p.len <= r.base + r.len) return r.index;
    return -1;
  }

  void ring_submit_locked(Piece* p) {
    const bool direct = direct_ok(*p);
    if (direct) st_direct++;
    const unsigned len = (unsigned)p->len;
    const int bi = fixed_index(*p);
    if (bi >= 0) st_fixed++;
    const int op = bi >= 0 ? (p->write ? IORING_OP_WRITE_FIXED : IORING_OP_READ_FIXED)
                           : (p->write ? IORING_OP_WRITE : IORING_OP_READ);
    if (!ring.push(op, direct ? fd_direct : fd, p->buf, len, p->off, (uint64_t)(uintptr_t)p, bi)) {
      const int e = errno ? errno : EIO;
      finish(p->ticket, -e);
      delete p;
      return;
    }
    inflight++;
  }

  void ring_enqueue(Piece* p) {
    std::lock_guard<std::mutex> g(ring_mu);
    if (inflight < depth) ring_submit_locked(p);
    else backlog.push_back(p);
  }

  void reaper_loop() {
    for (;;) {
      unsigned head = *ring.cq_head;
      if (head == __atomic_load_n(ring.cq_tail, __ATOMIC_ACQUIRE)) {
        const long r = syscall(__NR_io_uring_enter, ring.fd, 0, 1, IORING_ENTER_GETEVENTS, nullptr, 0);
        if (r < 0 && errno != EINTR && errno != EAGAIN && errno != EBUSY) return;
        continue;
      }
      const io_uring_cqe cqe = ring.cqes[head & *ring.cq_mask];
      __atomic_store_n(ring.cq_head, head + 1, __ATOMIC_RELEASE);
      if (cqe.user_data == 0) return;  // shutdown sentinel
      Piece* p = (Piece*)(uintptr_t)cqe.user_data;
      int64_t res = cqe.res;
      int inj_err = 0;
      int64_t inj_cut = -1;
      if (res > 0 && take_injection(&inj_err, &inj_cut)) {
        if (inj_err > 0) res = -inj_err;
        else if (inj_cut >= 0 && inj_cut < res) res = inj_cut > 0 ? inj_cut : 1;
      }
      std::unique_lock<std::mutex> g(ring_mu);
      inflight--;
      if (res < 0 && (res == -EINTR || res == -EAGAIN)) {
        ring_submit_locked(p);  // transient: same piece again
      } else if (res < 0) {
        g.unlock();
        finish(p->ticket, (int)res);
        delete p;
        g.lock();
      } else if (res == 0) {
        g.unlock();
        finish(p->ticket, -ENODATA);
        delete p;
        g.lock();
      } else if (res < p->len) {
        st_resubmits++;
        (p->write ? st_written : st_read) += res;
        p->buf += res;
        p->off += res;
        p->len -= res;
        ring_submit_locked(p);  // remainder (falls back to the buffered fd if now unaligned)
      } else {
        (p->write ? st_written : st_read) += res;
        g.unlock();
        finish(p->ticket, 0);
        delete p;
        g.lock();
      }
      while (inflight < depth && !backlog.empty()) {
        Piece* q = backlog.front();
        backlog.pop_front();
        ring_submit_locked(q);
      }
      if (inflight == 0 && backlog.empty()) ring_idle_cv.notify_all();
    }
  }
};

static void set_err(char* err, int err_len, const char* msg, int e) {
  if (err && err_len > 0) snprintf(err, (size_t)err_len, "%s: %s", msg, e ? strerror(e) : "failed");
}

extern "C" {

daser_io* daser_io_open(const char* path, int backend, int want_device, int queue_depth, int nthreads, char* err,
                        int err_len, int* err_no) {
  if (err_no) *err_no = 0;
  const int fd = open(path, O_RDWR | O_CLOEXEC);
  if (fd < 0) {
    if (err_no) *err_no = errno;
    set_err(err, err_len, "open", errno);
    return nullptr;
  }
  daser_io* io = new daser_io();
  io->fd = fd;
  io->fd_direct = open(path, O_RDWR | O_CLOEXEC | O_DIRECT);
  io->device = want_device > 0 ? want_device - 1 : -1;
  struct stat st;
  if (fstat(fd, &st) == 0) io->file_size = st.st_size;
  if (queue_depth <= 0) queue_depth = 64;
  if (nthreads <= 0) nthreads = 4;
  io->depth = (unsigned)queue_depth;

  int chosen = 0;
  // AUTO only tries cuFile when the nvidia-fs kernel driver is loaded: without it
  // cuFileDriverOpen can stall for a long time probing for the driver before it gives up.
  const bool nvfs = access("/proc/driver/nvidia-fs/stats", R_OK) == 0;
  if ((backend == DASER_IO_AUTO && want_device > 0 && nvfs) || backend == DASER_IO_GDS) {
    if (io->cf.load()) {
      if (io->cf.cuda_set_device && io->device >= 0) io->cf.cuda_set_device(io->device);
      CuFileApi::Error e = io->cf.driver_open();
      if (e.err == 0) {
        CuFileApi::Descr d;
        memset(&d, 0, sizeof(d));
        d.type = 1;  // CU_FILE_HANDLE_TYPE_OPAQUE_FD
        d.handle.fd = io->fd_direct >= 0 ? io->fd_direct : io->fd;
        e = io->cf.handle_register(&io->cf_handle, &d);
        if (e.err == 0) chosen = DASER_IO_GDS;
      }
    }
    if (!chosen && backend == DASER_IO_GDS) {
      set_err(err, err_len, "cuFile (GDS) is not usable here", 0);
      if (err_no) *err_no = ENOTSUP;
      daser_io_close(io);
      return nullptr;
    }
  }
  if (!chosen && (backend == DASER_IO_AUTO || backend == DASER_IO_URING)) {
    if (io->ring.setup((unsigned)queue_depth)) {
      if (io->depth > io->ring.entries) io->depth = io->ring.entries;
      chosen = DASER_IO_URING;
    } else if (backend == DASER_IO_URING) {
      if (err_no) *err_no = errno;
      set_err(err, err_len, "io_uring_setup", errno);
      daser_io_close(io);
      return nullptr;
    }
  }
  if (!chosen) chosen = DASER_IO_POSIX;
  io->backend = chosen;
  if (chosen == DASER_IO_URING) {
    io->reaper = std::thread([io] { io->reaper_loop(); });
    // device pieces are not accepted by this backend; no worker pool needed
  } else {
    for (int i = 0; i < nthreads; ++i) io->workers.emplace_back([io] { io->worker_loop(); });
  }
  return io;
}

int daser_io_backend(const daser_io* io) { return io ? io->backend : -1; }

// Register host buffers with the ring (io_uring backend only; call once, before IO into them).
// Buffers larger than 1 GiB are registered as consecutive 1 GiB regions.  Returns the number
// of regions registered, 0 when the backend has no use for it, or -errno (the engine keeps
// working with plain reads and writes in that case).
int64_t daser_io_register_buffers(daser_io* io, void* const* bufs, const int64_t* lens, int n) {
  if (!io || n < 0 || (n && (!bufs || !lens))) return -EINVAL;
  if (io->backend != DASER_IO_URING) return 0;
  std::lock_guard<std::mutex> g(io->ring_mu);
  if (!io->fixed.empty()) return -EBUSY;
  const size_t kMax = (size_t)1 << 30;
  std::vector<iovec> iov;
  for (int i = 0; i < n; ++i) {
    if (!bufs[i] || lens[i] <= 0) return -EINVAL;
    for (size_t off = 0; off < (size_t)lens[i]; off += kMax) {
      iovec v;
      v.iov_base = (char*)bufs[i] + off;
      v.iov_len = (size_t)lens[i] - off < kMax ? (size_t)lens[i] - off : kMax;
      iov.push_back(v);
    }
  }
  if (iov.empty()) return 0;
  if (iov.size() > 1024) return -E2BIG;
  const int rc = io->ring.register_buffers(iov.data(), (unsigned)iov.size());
  if (rc != 0) return rc;
  for (size_t i = 0; i < iov.size(); ++i)
    io->fixed.push_back({(uintptr_t)iov[i].iov_base, iov[i].iov_len, (int)i});
  return (int64_t)iov.size();
}
int64_t daser_io_file_size(const daser_io* io) { return io ? io->file_size : -1; }

int64_t daser_io_submit_strided(daser_io* io, int is_write, void* buf, int device, int64_t file_offset,
                                int64_t nbytes, int count, int64_t stride) {
  if (!io || !buf || file_offset < 0 || nbytes <= 0 || count <= 0 || (count > 1 && stride < nbytes)) return -EINVAL;
  if (device && io->backend != DASER_IO_GDS) return -ENOTSUP;
  const int per_extent = (int)((nbytes + kPieceBytes - 1) / kPieceBytes);
  const int64_t npieces = (int64_t)per_extent * count;
  if (npieces > (1 << 24)) return -EINVAL;
  int64_t ticket;
  {
    std::lock_guard<std::mutex> g(io->mu);
    if (io->closing) return -ESHUTDOWN;
    ticket = io->next_ticket++;
    io->tickets[ticket].pending = (int)npieces;
  }
  io->st_pieces += npieces;
  for (int e = 0; e < count; ++e) {
    char* ebuf = (char*)buf + (int64_t)e * stride;
    const int64_t eoff = file_offset + (int64_t)e * stride;
    for (int i = 0; i < per_extent; ++i) {
      Piece p;
      p.ticket = ticket;
      p.write = is_write != 0;
      p.device = device != 0;
      p.buf = ebuf + (int64_t)i * kPieceBytes;
      p.off = eoff + (int64_t)i * kPieceBytes;
      p.len = nbytes - (int64_t)i * kPieceBytes < kPieceBytes ? nbytes - (int64_t)i * kPieceBytes : kPieceBytes;
      if (io->backend == DASER_IO_URING) {
        io->ring_enqueue(new Piece(p));
      } else {
        {
          std::lock_guard<std::mutex> g(io->mu);
          io->queue.push_back(p);
        }
        io->queue_cv.notify_one();
      }
    }
  }
  return ticket;
}

int64_t daser_io_submit(daser_io* io, int is_write, void* buf, int device, int64_t file_offset, int64_t nbytes) {
  return daser_io_submit_strided(io, is_write, buf, device, file_offset, nbytes, 1, 0);
}

int daser_io_wait(daser_io* io, int64_t ticket, int timeout_ms) {
  if (!io) return -EINVAL;
  std::unique_lock<std::mutex> g(io->mu);
  auto it = io->tickets.find(ticket);
  if (it == io->tickets.end()) return -ENOENT;
  auto ready = [&] { return io->tickets[ticket].pending <= 0; };
  if (timeout_ms < 0) {
    io->cv.wait(g, ready);
  } else if (!io->cv.wait_for(g, std::chrono::milliseconds(timeout_ms), ready)) {
    return DASER_IO_TIMEOUT;
  }
  const int e = io->tickets[ticket].error;
  io->tickets.erase(ticket);
  return e;
}

int daser_io_poll(daser_io* io, int64_t ticket) {
  if (!io) return -EINVAL;
  std::lock_guard<std::mutex> g(io->mu);
  auto it = io->tickets.find(ticket);
  if (it == io->tickets.end()) return -ENOENT;
  return it->second.pending <= 0 ? 1 : 0;
}

int daser_io_close(daser_io* io) {
  if (!io) return 0;
  {
    std::lock_guard<std::mutex> g(io->mu);
    io->closing = true;
  }
  io->queue_cv.notify_all();
  for (auto& t : io->workers) t.join();
  if (io->reaper.joinable()) {
    {
      // Every submitted piece completes before the sentinel goes in: the caller's buffers are
      // not written after this function returns, and no piece is left behind un-freed.
      std::unique_lock<std::mutex> g(io->ring_mu);
      io->ring_idle_cv.wait_for(g, std::chrono::seconds(30), [&] { return io->inflight == 0 && io->backlog.empty(); });
      io->ring.push(IORING_OP_NOP, -1, nullptr, 0, 0, 0);
    }
    io->reaper.join();
  }
  io->ring.teardown();
  if (io->cf_handle && io->cf.handle_deregister) io->cf.handle_deregister(io->cf_handle);
  if (io->fd_direct >= 0) close(io->fd_direct);
  if (io->fd >= 0) close(io->fd);
  delete io;
  return 0;
}

int daser_io_preallocate(const char* path, int64_t size) {
  const int fd = open(path, O_RDWR | O_CREAT | O_CLOEXEC, 0644);
  if (fd < 0) return -errno;
  int r = posix_fallocate(fd, 0, (off_t)size);
  if (r == EOPNOTSUPP || r == EINVAL) r = ftruncate(fd, (off_t)size) == 0 ? 0 : errno;
  close(fd);
  return -r;
}

void daser_io_inject(daser_io* io, int count, int err_no, int64_t short_bytes) {
  if (!io) return;
  io->inject_errno = err_no;
  io->inject_short = short_bytes;
  io->inject_count = count;
}

int64_t daser_io_fixed_pieces(const daser_io* io) { return io ? io->st_fixed.load() : 0; }

void daser_io_stats(const daser_io* io, int64_t out[5]) {
  out[0] = io->st_pieces;
  out[1] = io->st_read;
  out[2] = io->st_written;
  out[3] = io->st_resubmits;
  out[4] = io->st_direct;
}

}  // extern "C"
