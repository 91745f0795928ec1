// C ABI of the host runtime (libnoeira_b200_host.so).  Every function returns 0 / a non-negative count on success and a
// negative errno-style code on failure unless stated otherwise.  Handles are opaque pointers.
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- single-producer / single-consumer ring of variable-size messages (ring.cpp)
void* nbh_ring_create(size_t capacity_bytes);
void nbh_ring_destroy(void* ring);
int nbh_ring_push(void* ring, const void* data, uint32_t size);           // 0, or -EAGAIN when full
int64_t nbh_ring_pop(void* ring, void* out, uint32_t out_capacity);       // size, -EAGAIN when empty, -EMSGSIZE
size_t nbh_ring_used(void* ring);
// background worker that drains a ring into a file (append), used by the CSV / event loggers
void* nbh_filesink_start(void* ring, const char* path);
int nbh_filesink_stop(void* sink);                                        // drains, joins, closes; returns messages written

// ---- serial port, raw mode (serial.cpp)
int nbh_serial_open(const char* path, int baud);                          // fd or -errno
int nbh_serial_configure(int fd, int baud);                               // raw 8N1 on an already open fd (pty tests)
int64_t nbh_serial_write(int fd, const void* data, size_t n);
int64_t nbh_serial_read(int fd, void* out, size_t n, int timeout_ms);     // bytes read (0 on timeout)
int nbh_serial_flush(int fd);
int nbh_serial_close(int fd);

// ---- HTTP/1.1 client on POSIX sockets + gzip (http.cpp)
// One request; the body is returned decoded (chunked transfer and gzip content-encoding are undone).
// Returns the HTTP status (>= 100) or -errno.  *out_body is malloc'ed: release with nbh_free.
int nbh_http_request(const char* method, const char* url, const char* headers /* "K: V\r\n..." or NULL */,
                     const void* body, size_t body_len, int timeout_ms, void** out_body, size_t* out_len);
int64_t nbh_gzip_inflate(const void* src, size_t n, void** out, size_t* out_len);
void nbh_free(void* p);

// ---- 3-D convex hull (hull.cpp): triangles with outward normals, counter-clockwise seen from outside
// tri_out receives up to max_tris * 3 vertex indices; returns the triangle count, or -ERANGE / -EINVAL (degenerate input).
int nbh_convex_hull(const double* xyz, int n, int32_t* tri_out, int max_tris);

// ---- atomic chunked file IO (fileio.cpp)
int nbh_write_file_atomic(const char* path, const void* const* chunks, const size_t* sizes, int n_chunks);
int64_t nbh_read_file_range(const char* path, uint64_t offset, void* out, size_t n);
int nbh_sha256(const void* data, size_t n, uint8_t out32[32]);

// ---- prefetching record loader (loader.cpp): fixed-size records in one binary file, shuffled per epoch with a keyed
// bijection, `threads` readers fill `slots` batch buffers ahead of the consumer.
void* nbh_loader_create(const char* path, uint64_t header_bytes, uint64_t record_bytes, uint64_t n_records, uint32_t batch,
                        uint32_t slots, uint32_t threads, uint64_t seed, int shuffle, int drop_last);
int64_t nbh_loader_next(void* loader, void* dst, uint64_t* out_indices);  // records in the batch; 0 = epoch ended
int nbh_loader_reset(void* loader, uint64_t epoch);
void nbh_loader_destroy(void* loader);

#ifdef __cplusplus
}
#endif
