// Prefetching record loader: reader threads fill batch slots ahead of the consumer from one binary file of fixed-size
// records; the per-epoch order is a keyed Feistel bijection of the record index (same family as the device-side
// minibatch shuffle), so any (seed, epoch) order is reproducible without storing a permutation.
// Counterpart of the reference's resident / sampled dataset feeders (noeira/data/sampler.mojo:97, data/resident.mojo:79)
// and its BackgroundThread workers.
#include <atomic>
#include <cerrno>
#include <condition_variable>
#include <cstdint>
#include <cstring>
#include <fcntl.h>
#include <mutex>
#include <thread>
#include <unistd.h>
#include <vector>

#include "host_api.h"

namespace {

inline uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}
// bijection on [0, n): 4-round Feistel on 2*hb bits with cycle walking
uint64_t permute(uint64_t i, uint64_t n, uint32_t key) {
  unsigned bits = 1;
  while ((1ull << bits) < n) ++bits;
  const unsigned hb = (bits + 1) / 2;
  const uint64_t mask = (1ull << hb) - 1;
  uint64_t x = i;
  do {
    uint64_t l = x >> hb, r = x & mask;
    for (uint32_t round = 0; round < 4; ++round) {
      const uint64_t f = mix32((uint32_t)r * 0x9E3779B1u + key + round * 0x85EBCA6Bu) & mask;
      const uint64_t nl = r, nr = l ^ f;
      l = nl; r = nr;
    }
    x = (l << hb) | r;
  } while (x >= n);
  return x;
}

struct Slot {
  std::vector<uint8_t> data;
  std::vector<uint64_t> idx;
  uint32_t count = 0;
  int64_t batch_no = -1;  // which batch of the epoch this slot holds
  bool ready = false;
};

struct Loader {
  int fd = -1;
  uint64_t header, rec, n, seed;
  uint32_t batch, nslots;
  bool shuffle, drop_last;
  uint64_t epoch = 0, n_batches = 0;
  std::vector<Slot> slots;
  std::vector<std::thread> threads;
  std::mutex mu;
  std::condition_variable cv_ready, cv_free, cv_idle;
  int inflight = 0;  // workers currently writing into a slot buffer (outside the lock)
  int64_t next_to_fill = 0, next_to_consume = 0;
  uint64_t generation = 0;
  bool stop = false;
  int error = 0;
};

void worker(Loader* L) {
  for (;;) {
    int64_t b;
    uint64_t gen, epoch;
    Slot* s;
    {
      std::unique_lock<std::mutex> lk(L->mu);
      for (;;) {
        if (L->stop) return;
        b = L->next_to_fill;
        if (b < (int64_t)L->n_batches && b < L->next_to_consume + (int64_t)L->nslots) break;
        L->cv_free.wait(lk);
      }
      ++L->next_to_fill;
      ++L->inflight;
      gen = L->generation;
      epoch = L->epoch;
      s = &L->slots[(size_t)b % L->nslots];
      s->ready = false;
    }
    const uint64_t first = (uint64_t)b * L->batch;
    const uint32_t cnt = (uint32_t)std::min<uint64_t>(L->batch, L->n - first);
    const uint32_t key = mix32((uint32_t)L->seed ^ mix32((uint32_t)epoch + 0x9E3779B9u));
    int err = 0;
    for (uint32_t k = 0; k < cnt && !err; ++k) {
      const uint64_t r = L->shuffle ? permute(first + k, L->n, key) : first + k;
      s->idx[k] = r;
      size_t done = 0;
      while (done < L->rec) {
        const ssize_t got = pread(L->fd, s->data.data() + (size_t)k * L->rec + done, L->rec - done,
                                  (off_t)(L->header + r * L->rec + done));
        if (got <= 0) { if (got < 0 && errno == EINTR) continue; err = got < 0 ? -errno : -EIO; break; }
        done += (size_t)got;
      }
    }
    {
      std::lock_guard<std::mutex> lk(L->mu);
      if (gen == L->generation) {     // a reset in between discards this batch
        s->count = cnt;
        s->batch_no = b;
        s->ready = true;
        if (err) L->error = err;
      }
      --L->inflight;
    }
    L->cv_ready.notify_all();
    L->cv_idle.notify_all();
  }
}

}  // namespace

extern "C" {

void* nbh_loader_create(const char* path, uint64_t header_bytes, uint64_t record_bytes, uint64_t n_records, uint32_t batch,
                        uint32_t slots, uint32_t threads, uint64_t seed, int shuffle, int drop_last) {
  if (!record_bytes || !n_records || !batch || !slots || !threads) return nullptr;
  Loader* L = new Loader();
  L->fd = open(path, O_RDONLY);
  if (L->fd < 0) { delete L; return nullptr; }
  L->header = header_bytes; L->rec = record_bytes; L->n = n_records; L->seed = seed;
  L->batch = batch; L->nslots = slots; L->shuffle = shuffle != 0; L->drop_last = drop_last != 0;
  L->n_batches = drop_last ? n_records / batch : (n_records + batch - 1) / batch;
  L->slots.resize(slots);
  for (auto& s : L->slots) { s.data.resize((size_t)batch * record_bytes); s.idx.resize(batch); }
  for (uint32_t t = 0; t < threads; ++t) L->threads.emplace_back(worker, L);
  return L;
}

int64_t nbh_loader_next(void* loader, void* dst, uint64_t* out_indices) {
  Loader* L = (Loader*)loader;
  std::unique_lock<std::mutex> lk(L->mu);
  if (L->next_to_consume >= (int64_t)L->n_batches) return 0;
  const int64_t b = L->next_to_consume;
  Slot* s = &L->slots[(size_t)b % L->nslots];
  L->cv_ready.wait(lk, [&] { return (s->ready && s->batch_no == b) || L->error; });
  if (L->error) return L->error;
  const uint32_t cnt = s->count;
  lk.unlock();
  memcpy(dst, s->data.data(), (size_t)cnt * L->rec);      // the slot is not refilled before next_to_consume moves
  if (out_indices) memcpy(out_indices, s->idx.data(), cnt * sizeof(uint64_t));
  lk.lock();
  s->ready = false;
  ++L->next_to_consume;
  lk.unlock();
  L->cv_free.notify_all();
  return cnt;
}

int nbh_loader_reset(void* loader, uint64_t epoch) {
  Loader* L = (Loader*)loader;
  {
    // A fill that is still running belongs to the old epoch and writes into its slot buffer without the lock.
    // Bump the generation first (so its result is discarded and no new fill of the old epoch starts: the
    // counters below park the workers), then wait until every such fill has left the buffers before the slots are
    // handed out again.
    std::unique_lock<std::mutex> lk(L->mu);
    ++L->generation;
    L->next_to_fill = (int64_t)L->n_batches;   // nothing new starts while draining
    L->cv_idle.wait(lk, [&] { return L->inflight == 0; });
    L->epoch = epoch;
    L->next_to_fill = 0;
    L->next_to_consume = 0;
    for (auto& s : L->slots) { s.ready = false; s.batch_no = -1; }
  }
  L->cv_free.notify_all();
  return 0;
}

void nbh_loader_destroy(void* loader) {
  Loader* L = (Loader*)loader;
  {
    std::lock_guard<std::mutex> lk(L->mu);
    L->stop = true;
  }
  L->cv_free.notify_all();
  for (auto& t : L->threads) t.join();
  close(L->fd);
  delete L;
}

}  // extern "C"
