// Lock-free single-producer / single-consumer message ring and a file-sink worker thread.
// Counterpart of the reference's concurrency backbone (noeira/core/concurrent/ring.mojo:443 SpscRing,
// worker.mojo:218 BackgroundThread); here plain C++17 atomics and std::thread.
#include <atomic>
#include <cerrno>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "host_api.h"

namespace {

struct alignas(64) Ring {
  size_t cap;                                  // power of two
  uint8_t* buf;
  alignas(64) std::atomic<uint64_t> head{0};   // consumer position
  alignas(64) std::atomic<uint64_t> tail{0};   // producer position
};

inline void copy_in(Ring* r, uint64_t pos, const void* src, size_t n) {
  const size_t o = pos & (r->cap - 1), first = n < r->cap - o ? n : r->cap - o;
  memcpy(r->buf + o, src, first);
  if (n > first) memcpy(r->buf, (const uint8_t*)src + first, n - first);
}
inline void copy_out(Ring* r, uint64_t pos, void* dst, size_t n) {
  const size_t o = pos & (r->cap - 1), first = n < r->cap - o ? n : r->cap - o;
  memcpy(dst, r->buf + o, first);
  if (n > first) memcpy((uint8_t*)dst + first, r->buf, n - first);
}

struct FileSink {
  Ring* ring;
  FILE* f;
  std::thread th;
  std::atomic<bool> stop{false};
  int written = 0;
};

}  // namespace

extern "C" {

void* nbh_ring_create(size_t capacity_bytes) {
  size_t cap = 64;
  while (cap < capacity_bytes) cap <<= 1;
  Ring* r = new (std::nothrow) Ring();
  if (!r) return nullptr;
  r->cap = cap;
  r->buf = (uint8_t*)malloc(cap);
  if (!r->buf) { delete r; return nullptr; }
  return r;
}

void nbh_ring_destroy(void* ring) {
  Ring* r = (Ring*)ring;
  if (!r) return;
  free(r->buf);
  delete r;
}

int nbh_ring_push(void* ring, const void* data, uint32_t size) {
  Ring* r = (Ring*)ring;
  const uint64_t need = (uint64_t)size + 4;
  if (need > r->cap) return -EMSGSIZE;
  const uint64_t t = r->tail.load(std::memory_order_relaxed), h = r->head.load(std::memory_order_acquire);
  if (t - h + need > r->cap) return -EAGAIN;
  copy_in(r, t, &size, 4);
  copy_in(r, t + 4, data, size);
  r->tail.store(t + need, std::memory_order_release);
  return 0;
}

int64_t nbh_ring_pop(void* ring, void* out, uint32_t out_capacity) {
  Ring* r = (Ring*)ring;
  const uint64_t h = r->head.load(std::memory_order_relaxed), t = r->tail.load(std::memory_order_acquire);
  if (h == t) return -EAGAIN;
  uint32_t size;
  copy_out(r, h, &size, 4);
  if (size > out_capacity) return -EMSGSIZE;
  copy_out(r, h + 4, out, size);
  r->head.store(h + 4 + size, std::memory_order_release);
  return size;
}

size_t nbh_ring_used(void* ring) {
  Ring* r = (Ring*)ring;
  return (size_t)(r->tail.load(std::memory_order_acquire) - r->head.load(std::memory_order_acquire));
}

void* nbh_filesink_start(void* ring, const char* path) {
  FILE* f = fopen(path, "ab");
  if (!f) return nullptr;
  FileSink* s = new FileSink();
  s->ring = (Ring*)ring;
  s->f = f;
  s->th = std::thread([s]() {
    std::vector<uint8_t> msg(1 << 16);
    for (;;) {
      const int64_t n = nbh_ring_pop(s->ring, msg.data(), (uint32_t)msg.size());
      if (n >= 0) {
        fwrite(msg.data(), 1, (size_t)n, s->f);
        ++s->written;
        continue;
      }
      if (n == -EMSGSIZE) { msg.resize(msg.size() * 2); continue; }
      if (s->stop.load(std::memory_order_acquire)) break;   // empty and asked to stop
      fflush(s->f);
      std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
    fflush(s->f);
  });
  return s;
}

int nbh_filesink_stop(void* sink) {
  FileSink* s = (FileSink*)sink;
  s->stop.store(true, std::memory_order_release);
  s->th.join();
  fclose(s->f);
  const int w = s->written;
  delete s;
  return w;
}

}  // extern "C"
