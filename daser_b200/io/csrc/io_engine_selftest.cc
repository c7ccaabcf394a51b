// Stand-alone exerciser of the storage engine, meant to be built with
// -fsanitize=address,undefined (and, separately, -fsanitize=thread) and run by the tests:
// concurrent submitters on both host backends, short-IO resubmission, injected errors,
// shutdown with work in flight.  Exit code 0 = everything matched.
#include <errno.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <thread>
#include <vector>

#include "io_engine.h"

static int run_backend(const char* path, int backend) {
  char err[256];
  int err_no = 0;
  daser_io* io = daser_io_open(path, backend, 0, 32, 4, err, sizeof(err), &err_no);
  if (!io) {
    if (backend == DASER_IO_URING) {
      printf("io_uring unavailable (%s): skipped\n", err);
      return 0;
    }
    fprintf(stderr, "open failed: %s\n", err);
    return 1;
  }
  // half of the submitters work inside a registered region (fixed-buffer operations on io_uring)
  const int64_t region_bytes = (int64_t)2 * (3 << 20) * 2;
  void* region = nullptr;
  if (posix_memalign(&region, 4096, region_bytes)) return 1;
  {
    void* bufs[1] = {region};
    int64_t lens[1] = {region_bytes};
    const int64_t got = daser_io_register_buffers(io, bufs, lens, 1);
    if (backend == DASER_IO_URING && got < 0) printf("buffer registration refused (%lld): plain IO\n", (long long)got);
    if (backend != DASER_IO_URING && got != 0) { fprintf(stderr, "registration on a backend without it\n"); return 1; }
  }
  const int64_t chunk = 3 << 20;  // 3 MiB: two pieces, second one short of the piece size
  const int nthreads = 4, per_thread = 6;
  std::vector<std::thread> threads;
  std::vector<int> bad(nthreads, 0);
  for (int t = 0; t < nthreads; ++t) {
    threads.emplace_back([&, t] {
      void* wbuf = nullptr;
      void* rbuf = nullptr;
      const bool in_region = t < 2;  // two submitters share the registered region, two use their own memory
      if (in_region) {
        wbuf = (char*)region + (int64_t)t * 2 * chunk;
        rbuf = (char*)wbuf + chunk;
      } else if (posix_memalign(&wbuf, 4096, chunk) || posix_memalign(&rbuf, 4096, chunk)) { bad[t] = 1; return; }
      for (int i = 0; i < per_thread; ++i) {
        const int64_t off = ((int64_t)t * per_thread + i) * chunk;
        memset(wbuf, 1 + t * 16 + i, chunk);
        int64_t tk = daser_io_submit(io, 1, wbuf, 0, off, chunk);
        if (tk < 0 || daser_io_wait(io, tk, 30000) != 0) { bad[t] = 2; break; }
        memset(rbuf, 0, chunk);
        tk = daser_io_submit(io, 0, rbuf, 0, off, chunk);
        if (tk < 0 || daser_io_wait(io, tk, 30000) != 0) { bad[t] = 3; break; }
        if (memcmp(wbuf, rbuf, chunk) != 0) { bad[t] = 4; break; }
      }
      if (!in_region) {
        free(wbuf);
        free(rbuf);
      }
    });
  }
  for (auto& th : threads) th.join();
  for (int t = 0; t < nthreads; ++t)
    if (bad[t]) { fprintf(stderr, "thread %d failed at stage %d\n", t, bad[t]); daser_io_close(io); return 1; }
  // injected error, then a short completion that must be resubmitted
  void* buf = nullptr;
  if (posix_memalign(&buf, 4096, 1 << 20)) return 1;
  daser_io_inject(io, 1, EIO, -1);
  int64_t tk = daser_io_submit(io, 0, buf, 0, 0, 1 << 20);
  if (daser_io_wait(io, tk, 30000) != -EIO) { fprintf(stderr, "injected EIO not reported\n"); return 1; }
  daser_io_inject(io, 1, 0, 777);
  tk = daser_io_submit(io, 0, buf, 0, 0, 1 << 20);
  if (daser_io_wait(io, tk, 30000) != 0) { fprintf(stderr, "short read not recovered\n"); return 1; }
  int64_t st[5];
  daser_io_stats(io, st);
  if (st[3] < 1) { fprintf(stderr, "no resubmission counted\n"); return 1; }
  // close with a submission that nobody waits for
  daser_io_submit(io, 0, buf, 0, 0, 1 << 20);
  const int64_t fixed = daser_io_fixed_pieces(io);
  daser_io_close(io);
  free(buf);
  free(region);
  if (backend == DASER_IO_URING) printf("fixed-buffer pieces: %lld\n", (long long)fixed);
  return 0;
}

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  if (daser_io_preallocate(argv[1], (int64_t)80 << 20) != 0) return 1;
  int rc = run_backend(argv[1], DASER_IO_POSIX);
  if (rc == 0) rc = run_backend(argv[1], DASER_IO_URING);
  printf(rc == 0 ? "SELFTEST_OK\n" : "SELFTEST_FAIL\n");
  return rc;
}
