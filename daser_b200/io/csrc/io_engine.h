// Storage engine: asynchronous reads/writes between one pre-allocated store file and
// host or device memory.
//
// Replaces what the reference gets from kvikio (daser/connector/gds_transfer.py:29-127:
// CuFile.pread/pwrite futures, GDS when available, a POSIX thread pool with a CPU bounce
// buffer otherwise).  The reference's documentation also names an io_uring fallback that its
// code does not contain; this engine has one.
//
// Backends, chosen once at open and immutable afterwards:
//   GDS       cuFile (libcufile.so loaded at run time): NVMe <-> GPU memory DMA.
//   IO_URING  raw io_uring (io_uring_setup / io_uring_enter, no liburing), O_DIRECT when the
//             request is 4 KiB aligned, requests split into pieces for queue depth.
//   POSIX     pread/pwrite on a worker pool.
// IO_URING and POSIX move host memory only; the caller stages device data through pinned
// host buffers (daser_b200/connector/transfer.py does it on a dedicated copy stream).
//
// All functions are thread safe.  A submit returns a ticket; wait(ticket) returns 0, a
// negative errno, or DASER_IO_TIMEOUT.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DASER_IO_AUTO 0
#define DASER_IO_GDS 1
#define DASER_IO_URING 2
#define DASER_IO_POSIX 3

#define DASER_IO_TIMEOUT 1

#define DASER_IO_API __attribute__((visibility("default")))

typedef struct daser_io daser_io;

// Opens an existing file read/write.  Returns NULL and fills `err` on failure (a missing file
// reports ENOENT in *err_no).  `backend` = DASER_IO_AUTO tries GDS (only if `want_device`),
// then io_uring, then POSIX.
DASER_IO_API daser_io* daser_io_open(const char* path, int backend, int want_device, int queue_depth,
                                     int nthreads, char* err, int err_len, int* err_no);
DASER_IO_API int daser_io_backend(const daser_io* io);

/* Register host buffers with the io_uring ring so that IO into them uses READ_FIXED /
 * WRITE_FIXED (no per-IO page pinning).  Call once, before IO into the buffers; buffers above
 * 1 GiB are split.  Returns the number of regions, 0 on other backends, or -errno (plain IO
 * keeps working). */
DASER_IO_API int64_t daser_io_register_buffers(daser_io* io, void* const* bufs, const int64_t* lens, int n);
/* Pieces submitted as fixed-buffer operations so far. */
DASER_IO_API int64_t daser_io_fixed_pieces(const daser_io* io);
DASER_IO_API int64_t daser_io_file_size(const daser_io* io);

// `device` != 0: buf is a CUDA device pointer (GDS backend only).
// `count` extents of `nbytes` each under ONE ticket: extent i moves file bytes
// [file_offset + i * stride, + nbytes) to or from buf + i * stride (the same stride on both
// sides: a run of equally spaced slices of a larger image, e.g. some layers of every slot of a
// chunk).  Completes when every extent has; the first error wins.
DASER_IO_API int64_t daser_io_submit_strided(daser_io* io, int is_write, void* buf, int device, int64_t file_offset,
                                             int64_t nbytes, int count, int64_t stride);
DASER_IO_API int64_t daser_io_submit(daser_io* io, int is_write, void* buf, int device, int64_t file_offset,
                                     int64_t nbytes);
DASER_IO_API int daser_io_wait(daser_io* io, int64_t ticket, int timeout_ms);
// 1 if every piece of the ticket has completed, 0 if some are pending, -ENOENT for an unknown (or
// already waited-for) ticket.  Does not consume the ticket: daser_io_wait still reports its outcome.
DASER_IO_API int daser_io_poll(daser_io* io, int64_t ticket);
DASER_IO_API int daser_io_close(daser_io* io);

// Creates (or extends) a file of `size` bytes without writing zeros through user space.
DASER_IO_API int daser_io_preallocate(const char* path, int64_t size);

// Fault injection for tests (host side only): the next `count` pieces complete with -err_no
// (err_no > 0), or are cut short to `short_bytes` once (err_no == 0, short_bytes >= 0; the
// engine must then resubmit the remainder).
DASER_IO_API void daser_io_inject(daser_io* io, int count, int err_no, int64_t short_bytes);

// Counters: [0] pieces submitted, [1] bytes read, [2] bytes written, [3] resubmits after short IO,
// [4] direct-IO pieces.
DASER_IO_API void daser_io_stats(const daser_io* io, int64_t out[5]);

#ifdef __cplusplus
}
#endif
