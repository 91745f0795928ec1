// Device-resident replay buffer kernels: ring store of a batch of transitions, index generation (uniform,
// emphasising-recent-experience, prioritised through a sum tree) with device-side size / write offset, gather of the
// sampled transitions into contiguous minibatch tensors, priority updates.  No host round trip anywhere, so a
// captured off-policy update graph can include store + sample + gather.
// Reference: noeira/data/replay_gpu.mojo:54-330 (store, gather, uniform / ERE / PER indices, device size / offset).
#include "common.cuh"

namespace {
using namespace nb;

// meta[0] = write offset, meta[1] = current size, meta[2] = sample counter (rng stream position)
__global__ void replay_store_kernel(float* __restrict__ buf, int width, long long capacity, long long* __restrict__ meta,
                                    const float* __restrict__ rows, int n, int demo_prefix) {
  const long long off = meta[0];
  const long long ring = capacity - demo_prefix;        // the demo prefix is never overwritten
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n * width;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    long long dst = off + r;
    if (dst >= capacity) dst = demo_prefix + (dst - demo_prefix) % ring;
    buf[dst * width + c] = rows[i];
  }
}
__global__ void replay_advance_kernel(long long* meta, long long capacity, int n, int demo_prefix) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const long long ring = capacity - demo_prefix;
    long long off = meta[0] + n;
    if (off >= capacity) off = demo_prefix + (off - demo_prefix) % ring;
    meta[0] = off;
    meta[1] = min(meta[1] + (long long)n, capacity);
  }
}

// mode 0: uniform over [0, size); mode 1: ERE — uniform over the most recent c_k transitions, c_k = max(size·eta^(k·1000/K), cmin)
__global__ void replay_indices_kernel(long long* __restrict__ idx, int batch, const long long* __restrict__ meta,
                                      unsigned long long seed, int mode, float ere_frac, long long cmin,
                                      long long capacity, int demo_prefix) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch) return;
  const long long size = max(meta[1], 1LL);
  Philox ph(seed);
  uint32_t r[4];
  const unsigned long long ctr = (unsigned long long)meta[2];
  ph((uint32_t)i, 0u, (uint32_t)ctr, (uint32_t)(ctr >> 32), r);
  const double u = ((double)r[0] * 4294967296.0 + (double)r[1]) / 18446744073709551616.0;
  if (mode == 0) {
    idx[i] = min((long long)(u * (double)size), size - 1);
  } else {
    long long ck = max((long long)((double)size * (double)ere_frac), min(cmin, size));
    ck = min(ck, size);
    const long long back = min((long long)(u * (double)ck), ck - 1);   // 0 = newest
    long long pos = meta[0] - 1 - back;                                  // walk back from the write offset
    const long long ring = capacity - demo_prefix;
    if (size < capacity) { if (pos < 0) pos += size; }
    else if (pos < demo_prefix) pos += ring;
    idx[i] = pos;
  }
}

// ---- sum tree over `leaves` (power of two) priorities: tree[1] = total, children of n are 2n, 2n+1, leaves at [leaves, 2·leaves)
__global__ void per_set_kernel(float* __restrict__ tree, long long leaves, const long long* __restrict__ idx,
                               const float* __restrict__ prio, int n, float alpha, float eps) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if (!NB_IN_BOUNDS(idx[i] >= 0 && idx[i] < leaves, 612, idx[i])) continue;
    tree[leaves + idx[i]] = powf(fabsf(prio[i]) + eps, alpha);
  }
}
// After the leaves idx[0..n) changed, re-sum their ancestors one level per launch (level k = nodes (leaves+idx)>>k).
// Threads that share an ancestor write the same value, so the result is deterministic without atomics, and the
// work is n·log2(leaves) whatever the capacity.
__global__ void per_ancestors_kernel(float* __restrict__ tree, long long leaves, const long long* __restrict__ idx, int n,
                                     int level) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if (!NB_IN_BOUNDS(idx[i] >= 0 && idx[i] < leaves, 613, idx[i])) continue;
    const long long node = (leaves + idx[i]) >> level;
    tree[node] = tree[2 * node] + tree[2 * node + 1];
  }
}
// Full rebuild of one level (grid-stride: any capacity).
__global__ void per_rebuild_level_kernel(float* __restrict__ tree, long long first, long long count) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const long long n = first + i;
    tree[n] = tree[2 * n] + tree[2 * n + 1];
  }
}
// stratified prefix-sum descent; also returns the importance weight (N·P(i))^-beta normalised by its maximum bound
__global__ void per_sample_kernel(const float* __restrict__ tree, long long leaves, long long* __restrict__ idx,
                                  float* __restrict__ weight, int batch, const long long* __restrict__ meta,
                                  unsigned long long seed, float beta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= batch) return;
  const long long size = max(meta[1], 1LL);
  Philox ph(seed ^ 0x9E3779B97F4A7C15ull);
  uint32_t r[4];
  const unsigned long long ctr = (unsigned long long)meta[2];
  ph((uint32_t)i, 1u, (uint32_t)ctr, (uint32_t)(ctr >> 32), r);
  const float total = tree[1];
  const float seg = total / batch;
  float target = (i + u32_to_unit(r[0])) * seg;
  long long n = 1;
  while (n < leaves) {
    const float left = tree[2 * n];
    if (target <= left || tree[2 * n + 1] <= 0.f) n = 2 * n;
    else { target -= left; n = 2 * n + 1; }
  }
  long long leaf = min(n - leaves, size - 1);
  idx[i] = leaf;
  if (weight) {
    const float p = fmaxf(tree[leaves + leaf], 1e-12f) / fmaxf(total, 1e-12f);
    weight[i] = powf((float)size * p, -beta);
  }
}
__global__ void replay_bump_counter_kernel(long long* meta) {
  if (threadIdx.x == 0 && blockIdx.x == 0) meta[2] += 1;
}

__global__ void replay_gather_kernel(const float* __restrict__ buf, int width, const long long* __restrict__ idx,
                                     float* __restrict__ out, int batch, long long capacity) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)batch * width;
       i += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(i / width), c = (int)(i % width);
    if (!NB_IN_BOUNDS(idx[r] >= 0 && (capacity <= 0 || idx[r] < capacity), 611, idx[r])) continue;
    out[i] = buf[idx[r] * width + c];
  }
}
inline int blocks_for(long long n) { long long b = (n + 255) / 256; return (int)(b < 1 ? 1 : (b > 148 * 8 ? 148 * 8 : b)); }
}  // namespace

NB_BOUNDS_REGISTER(replay)

extern "C" {

int nb_replay_store(float* buf, int width, long long capacity, long long* meta, const float* rows, int n, int demo_prefix,
                    void* stream) {
  if (n <= 0 || width <= 0 || n > capacity - demo_prefix) return NB_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  replay_store_kernel<<<blocks_for((long long)n * width), 256, 0, s>>>(buf, width, capacity, meta, rows, n, demo_prefix);
  NB_LAUNCH_CHECK();
  replay_advance_kernel<<<1, 32, 0, s>>>(meta, capacity, n, demo_prefix);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_replay_indices(long long* idx, int batch, long long* meta, unsigned long long seed, int mode, float ere_frac,
                      long long cmin, long long capacity, int demo_prefix, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  replay_indices_kernel<<<blocks_for(batch), 256, 0, s>>>(idx, batch, meta, seed, mode, ere_frac, cmin, capacity, demo_prefix);
  NB_LAUNCH_CHECK();
  replay_bump_counter_kernel<<<1, 32, 0, s>>>(meta);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_per_update(float* tree, long long leaves, const long long* idx, const float* prio, int n, float alpha, float eps,
                  void* stream) {
  if (leaves <= 0 || (leaves & (leaves - 1))) return NB_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  per_set_kernel<<<blocks_for(n), 256, 0, s>>>(tree, leaves, idx, prio, n, alpha, eps);
  NB_LAUNCH_CHECK();
  int level = 1;
  for (long long count = leaves / 2; count >= 1; count /= 2, ++level) {
    per_ancestors_kernel<<<blocks_for(n), 256, 0, s>>>(tree, leaves, idx, n, level);
    NB_LAUNCH_CHECK();
  }
  return NB_OK;
}

// Recompute every inner node from the leaves (after loading a checkpointed priority array).
int nb_per_rebuild(float* tree, long long leaves, void* stream) {
  if (leaves <= 0 || (leaves & (leaves - 1))) return NB_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  for (long long count = leaves / 2; count >= 1; count /= 2) {
    per_rebuild_level_kernel<<<blocks_for(count), 256, 0, s>>>(tree, count, count);
    NB_LAUNCH_CHECK();
  }
  return NB_OK;
}

int nb_per_sample(const float* tree, long long leaves, long long* idx, float* weight, int batch, long long* meta,
                  unsigned long long seed, float beta, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  per_sample_kernel<<<blocks_for(batch), 256, 0, s>>>(tree, leaves, idx, weight, batch, meta, seed, beta);
  NB_LAUNCH_CHECK();
  replay_bump_counter_kernel<<<1, 32, 0, s>>>(meta);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// capacity: number of rows of `buf` (<= 0: unknown; only the bounds-checked build reads it)
int nb_replay_gather(const float* buf, int width, const long long* idx, float* out, int batch, long long capacity, void* stream) {
  replay_gather_kernel<<<blocks_for((long long)batch * width), 256, 0, (cudaStream_t)stream>>>(buf, width, idx, out, batch, capacity);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
