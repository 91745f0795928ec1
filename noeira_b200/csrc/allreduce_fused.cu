// Gradient all-reduce over NVLink peer memory, FUSED with scale / clip partials / Adam(W) / bf16
// recast / gradient zeroing — one kernel per bucket, no NCCL on this path.
//
// Every rank maps every peer's gradient arena (CUDA IPC) and a small signal pad.  Three algorithms,
// picked by the caller per bucket size:
//
//   one-shot   each rank loads the bucket from ALL peers (plain P2P loads, rank order 0..N-1 so every
//              replica computes bit-identical sums) and applies the update directly.  (N-1)·bytes in
//              per GPU, one flag round before and one after.  Best for small buckets.
//   two-shot   rank r reduces slice r from all peers and PUSHES the sum into every peer's `red`
//              buffer (reduce-scatter + all-gather through peer stores, 2(N-1)/N·bytes per GPU),
//              cross-GPU flag round, then every rank updates the whole bucket from its local `red`.
//   multimem   same structure as two-shot but the reduction is done by NVSwitch:
//              multimem.ld_reduce.add on the multicast address of slice r, multimem.st of the sum to
//              every peer (≈ bytes/N in and out per GPU).  Needs a multicast mapping of grd and red.
//
// Synchronisation: monotone u32 counters in each rank's signal pad, written with
// red.release.sys.add and polled with ld.acquire.sys; wait targets derive from device-resident bases,
// so a captured CUDA graph replays correctly.  Every wait is bounded: on a timeout the kernel writes
// NB_ST_PEER_TIMEOUT (+ which phase) into `status`, skips the data phase and returns.
// Grids are persistent (≤ one wave) because blocks of one kernel wait on one another.
//
// Reference path being replaced: MAX comm allreduce → _scale_copy_kernel → 3 clip kernels →
// _grouped_adam_kernel (noeira/nn/distributed/data_parallel.mojo:190-202,257-298;
// noeira/nn/optimizer/grad_clip.mojo:255-320; noeira/nn/optimizer/adam.mojo:91-128).
#include <string.h>

#include "common.cuh"
#include "optim_math.cuh"

namespace {
using namespace nb;

constexpr int MAX_RANKS = 8;
// signal pad slots (u32)
// counters [0..3] are monotone; [16+k] holds the value counter k had reached when the previous launch
// that used it finished ("base").  A launch waits for base + arrivals expected in this launch, and its
// last block publishes the new base — so launches with different grid sizes can share one pad.
constexpr int SIG_ARRIVE = 0, SIG_DONE = 1, SIG_PHASE = 2, SIG_GRID = 3, SIG_TICKET = 9, SIG_BASE = 16;

struct ARParams {
  float* grd[MAX_RANKS];          // every rank's gradient bucket (own pointer at [rank])
  float* red[MAX_RANKS];          // every rank's reduced-gradient scratch (two-shot / clip)
  unsigned int* sig[MAX_RANKS];   // every rank's signal pad
  float* grd_mc;                  // multicast address of grd (multimem variant) or null
  float* red_mc;                  // multicast address of red
  int world, rank;
  long long n4;                   // bucket length in float4
  unsigned int spin_limit;
};

struct AdamBufs {
  float *val, *m, *v;
  __nv_bfloat16* shadow;
  const unsigned char* row_flags;
  const float* hyper;
  float* partials;   // >= gridDim.x floats (clip)
  float* norm_out;   // optional
  float max_norm;    // <= 0: no clip
  int do_update;     // 0: plain all-reduce (sum lands in red[rank], scaled by hyper[GSCALE] if hyper)
  int zero_grad;
};

__device__ __forceinline__ float4 ld_peer4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer4(float* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 multimem_ld_reduce4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

// All blocks of all ranks meet: every block adds 1 to slot `slot` of every rank's pad, then waits
// until its own pad shows base + world·gridDim.x.  Returns false on timeout (block uniform).
__device__ __forceinline__ bool cross_barrier(const ARParams& p, int slot, unsigned int base, unsigned int* status,
                                              unsigned int where, bool* sh_ok) {
  __syncthreads();
  if (threadIdx.x < p.world) {
    __threadfence_system();
    red_release_sys_add(p.sig[threadIdx.x] + slot, 1u);
  }
  if (threadIdx.x == 0) {
    const unsigned int target = base + (unsigned int)p.world * gridDim.x;
    *sh_ok = wait_flag_ge(p.sig[p.rank] + slot, target, status, where, 0u, p.spin_limit);
  }
  __syncthreads();
  return *sh_ok;
}

// Blocks of THIS grid meet (co-resident persistent grid).  Counter is monotone across launches.
__device__ __forceinline__ bool grid_barrier(unsigned int* ctr, unsigned int base, unsigned int* status,
                                             unsigned int where, unsigned int limit, bool* sh_ok) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(ctr, 1u);
    const unsigned int target = base + gridDim.x;
    bool ok = false;
    for (unsigned int it = 0; it < limit; ++it) {
      if ((int)(ld_acquire_sys(ctr) - target) >= 0) { ok = true; break; }
      __nanosleep(20);
    }
    if (!ok) report(status, NB_ST_PEER_TIMEOUT, where, 0xFFFFu);
    *sh_ok = ok;
  }
  __syncthreads();
  return *sh_ok;
}

__device__ __forceinline__ void write_shadow4(__nv_bfloat16* shadow, long long i, float4 p) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
  uint2 pk;
  pk.x = *reinterpret_cast<uint32_t*>(&lo);
  pk.y = *reinterpret_cast<uint32_t*>(&hi);
  reinterpret_cast<uint2*>(shadow)[i] = pk;
}

__device__ __forceinline__ void update4(const AdamBufs& a, const AdamHyper& h, long long i, float4 g) {
  const unsigned char fl = a.row_flags ? a.row_flags[i >> 3] : (unsigned char)1;
  float4 pv = reinterpret_cast<float4*>(a.val)[i];
  if (!(fl & 2)) {
    float4 mm = reinterpret_cast<float4*>(a.m)[i];
    float4 vv = reinterpret_cast<float4*>(a.v)[i];
    adamw_update4(pv, g, mm, vv, h, (fl & 1) != 0);
    reinterpret_cast<float4*>(a.val)[i] = pv;
    reinterpret_cast<float4*>(a.m)[i] = mm;
    reinterpret_cast<float4*>(a.v)[i] = vv;
  }
  if (a.shadow) write_shadow4(a.shadow, i, pv);
}

// clip scale from ordered partials: every block computes the same value (deterministic).
__device__ __forceinline__ float clip_scale_from_partials(const AdamBufs& a, float base_scale, float* sh) {
  float s = 0.f;
  for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) s += a.partials[i];
  s = block_sum(s, sh);
  const float norm = sqrtf(s) * base_scale;
  if (a.norm_out && blockIdx.x == 0 && threadIdx.x == 0) a.norm_out[0] = norm;
  if (!isfinite(norm)) return 0.f;
  if (a.max_norm > 0.f && norm > a.max_norm) return base_scale * a.max_norm / (norm + 1e-6f);
  return base_scale;
}

// Last block of the grid publishes the new bases (mask: which counters this kernel used).
__device__ __forceinline__ void publish_bases(unsigned int* my, const unsigned int* bases, int world, unsigned int mask) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const unsigned int t = atomicAdd(my + SIG_TICKET, 1u);
    if (t == gridDim.x - 1) {
      my[SIG_TICKET] = 0u;
      for (int k = 0; k < 4; ++k)
        if (mask >> k & 1u) my[SIG_BASE + k] = bases[k] + (k == SIG_GRID ? 1u : (unsigned int)world) * gridDim.x;
      __threadfence();
    }
  }
}

// ------------------------------------------------------------------------------------------ one-shot
__global__ void __launch_bounds__(512)
ar_oneshot_kernel(ARParams p, AdamBufs a, unsigned int* status) {
  __shared__ bool sh_ok;
  __shared__ float sh[32];
  unsigned int* my = p.sig[p.rank];
  unsigned int bases[4];
  for (int k = 0; k < 4; ++k) bases[k] = ld_acquire_sys(my + SIG_BASE + k);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool ok = cross_barrier(p, SIG_ARRIVE, bases[SIG_ARRIVE], status, 10, &sh_ok);
  AdamHyper h;
  if (a.hyper) h = load_hyper(a.hyper);
  const bool clip = a.do_update && a.max_norm > 0.f;
  if (ok) {
    float ss = 0.f;
    for (long long i = i0; i < p.n4; i += stride) {
      float4 g = ld_peer4(p.grd[0] + 4 * i);
      for (int r = 1; r < p.world; ++r) {
        const float4 x = ld_peer4(p.grd[r] + 4 * i);
        g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
      }
      if (!a.do_update) {
        const float s = a.hyper ? h.gscale : 1.f;
        reinterpret_cast<float4*>(p.red[p.rank])[i] = make_float4(g.x * s, g.y * s, g.z * s, g.w * s);
      } else if (clip) {
        ss += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
        reinterpret_cast<float4*>(p.red[p.rank])[i] = g;
      } else {
        update4(a, h, i, g);
      }
    }
    if (clip) {
      ss = block_sum(ss, sh);
      if (threadIdx.x == 0) a.partials[blockIdx.x] = ss;
      ok = grid_barrier(my + SIG_GRID, bases[SIG_GRID], status, 11, p.spin_limit, &sh_ok);
      if (ok) {
        h.gscale = clip_scale_from_partials(a, h.gscale, sh);
        for (long long i = i0; i < p.n4; i += stride) update4(a, h, i, reinterpret_cast<float4*>(p.red[p.rank])[i]);
      }
    }
  }
  // everyone has finished READING my gradients before I clear them / the next backward writes them
  ok = cross_barrier(p, SIG_DONE, bases[SIG_DONE], status, 12, &sh_ok) && ok;
  if (ok && a.zero_grad) {
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long i = i0; i < p.n4; i += stride) reinterpret_cast<float4*>(p.grd[p.rank])[i] = z;
  }
  publish_bases(my, bases, p.world, (1u << SIG_ARRIVE) | (1u << SIG_DONE) | (clip ? (1u << SIG_GRID) : 0u));
}

// ------------------------------------------------------------------------------------------ two-shot / multimem
template <bool MULTIMEM>
__global__ void __launch_bounds__(512)
ar_twoshot_kernel(ARParams p, AdamBufs a, unsigned int* status) {
  __shared__ bool sh_ok;
  __shared__ float sh[32];
  unsigned int* my = p.sig[p.rank];
  unsigned int bases[4];
  for (int k = 0; k < 4; ++k) bases[k] = ld_acquire_sys(my + SIG_BASE + k);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool ok = cross_barrier(p, SIG_ARRIVE, bases[SIG_ARRIVE], status, 20, &sh_ok);
  AdamHyper h;
  if (a.hyper) h = load_hyper(a.hyper);
  const bool clip = a.do_update && a.max_norm > 0.f;
  // slice of this rank (in float4 units, 128-byte granules so stores stay aligned)
  const long long per = ((p.n4 + p.world - 1) / p.world + 7) / 8 * 8;
  const long long lo = min(p.n4, per * p.rank), hi = min(p.n4, per * (p.rank + 1));
  // plain all-reduce: the scale rides on the slice owner's sum, so no extra pass over the result is needed
  const float presc = (!a.do_update && a.hyper) ? h.gscale : 1.f;
  if (ok) {
    if (MULTIMEM) {
      for (long long i = lo + i0; i < hi; i += stride) {
        float4 g = multimem_ld_reduce4(p.grd_mc + 4 * i);
        if (presc != 1.f) { g.x *= presc; g.y *= presc; g.z *= presc; g.w *= presc; }
        multimem_st4(p.red_mc + 4 * i, g);
      }
    } else {
      // Loads from ALL peers are issued before the first sum (2 float4 per peer and thread = 16 independent loads in
      // flight per thread at N = 8): an NVLink round trip is microseconds, so the reduction is latency-bound unless
      // every link has requests outstanding all the time.  The sum itself stays in rank order (bit-identical replicas).
      constexpr int U = 2;
      for (long long i = lo + i0; i < hi; i += stride * U) {
        float4 x[MAX_RANKS][U];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) {
          if (r < p.world) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const long long k = i + u * stride;
              x[r][u] = k < hi ? ld_peer4(p.grd[r] + 4 * k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          float4 g = x[0][u];
#pragma unroll
          for (int r = 1; r < MAX_RANKS; ++r) {
            if (r < p.world) { g.x += x[r][u].x; g.y += x[r][u].y; g.z += x[r][u].z; g.w += x[r][u].w; }
          }
          const long long k = i + u * stride;
          if (k < hi) {
            if (presc != 1.f) { g.x *= presc; g.y *= presc; g.z *= presc; g.w *= presc; }
            for (int d = 0; d < p.world; ++d) {
              const int r = (p.rank + d) % p.world;   // ring order spreads the stores over the links
              st_peer4(p.red[r] + 4 * k, g);
            }
          }
        }
      }
    }
  }
  // all slices have landed in my `red`, and nobody reads my grd any more
  ok = cross_barrier(p, SIG_PHASE, bases[SIG_PHASE], status, 21, &sh_ok) && ok;
  if (ok) {
    const float4* red = reinterpret_cast<const float4*>(p.red[p.rank]);
    if (a.do_update) {
      if (clip) {
        float ss = 0.f;
        for (long long i = i0; i < p.n4; i += stride) {
          const float4 g = red[i];
          ss += g.x * g.x + g.y * g.y + g.z * g.z + g.w * g.w;
        }
        ss = block_sum(ss, sh);
        if (threadIdx.x == 0) a.partials[blockIdx.x] = ss;
        ok = grid_barrier(my + SIG_GRID, bases[SIG_GRID], status, 22, p.spin_limit, &sh_ok);
        if (ok) h.gscale = clip_scale_from_partials(a, h.gscale, sh);
      }
      if (ok)
        for (long long i = i0; i < p.n4; i += stride) update4(a, h, i, red[i]);
    }
    if (a.zero_grad) {
      const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      for (long long i = i0; i < p.n4; i += stride) reinterpret_cast<float4*>(p.grd[p.rank])[i] = z;
    }
  }
  // `red` of every peer may be overwritten by the next launch only after everyone consumed it
  ok = cross_barrier(p, SIG_DONE, bases[SIG_DONE], status, 23, &sh_ok) && ok;
  publish_bases(my, bases, p.world,
                (1u << SIG_ARRIVE) | (1u << SIG_DONE) | (1u << SIG_PHASE) | (clip ? (1u << SIG_GRID) : 0u));
}

// ------------------------------------------------------------------------------------------ ZeRO step
// Reduce-scatter fused with the shard's Adam(W) and all-gather fused with the bf16 recast, one kernel:
// rank r sums slice r of every peer's gradients (peer loads, rank order), updates ITS shard of the fp32 values with
// moments that exist only at shard size (m_shard / v_shard: Ψ/N floats each), and pushes the new values and their bf16
// shadow into every peer's arenas (peer stores).  Two flag rounds: all gradients are ready / every push has landed.
// Reference path: reduce_scatter → shard Adam → all_gather_rows as separate collectives
// (noeira/nn/distributed/zero.mojo:284-402).
struct ZeroBufs {
  float* val[MAX_RANKS];             // every rank's fp32 value arena
  __nv_bfloat16* shadow[MAX_RANKS];  // every rank's bf16 shadow arena (may be null)
  float *m_shard, *v_shard;          // this rank's moments: slice_len floats
  const unsigned char* row_flags;
  const float* hyper;
  int zero_grad;
};

__global__ void __launch_bounds__(512)
ar_zero_kernel(ARParams p, ZeroBufs z, unsigned int* status) {
  __shared__ bool sh_ok;
  unsigned int* my = p.sig[p.rank];
  unsigned int bases[4];
  for (int k = 0; k < 4; ++k) bases[k] = ld_acquire_sys(my + SIG_BASE + k);
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  bool ok = cross_barrier(p, SIG_ARRIVE, bases[SIG_ARRIVE], status, 40, &sh_ok);
  const AdamHyper h = load_hyper(z.hyper);
  const long long per = ((p.n4 + p.world - 1) / p.world + 7) / 8 * 8;
  const long long lo = min(p.n4, per * p.rank), hi = min(p.n4, per * (p.rank + 1));
  if (ok) {
    for (long long i = lo + i0; i < hi; i += stride) {
      float4 x[MAX_RANKS];
#pragma unroll
      for (int r = 0; r < MAX_RANKS; ++r)
        if (r < p.world) x[r] = ld_peer4(p.grd[r] + 4 * i);
      float4 g = x[0];
#pragma unroll
      for (int r = 1; r < MAX_RANKS; ++r)
        if (r < p.world) { g.x += x[r].x; g.y += x[r].y; g.z += x[r].z; g.w += x[r].w; }
      const unsigned char fl = z.row_flags ? z.row_flags[i >> 3] : (unsigned char)1;
      float4 pv = reinterpret_cast<const float4*>(z.val[p.rank])[i];
      if (!(fl & 2)) {
        const long long j = i - lo;
        float4 mm = reinterpret_cast<float4*>(z.m_shard)[j];
        float4 vv = reinterpret_cast<float4*>(z.v_shard)[j];
        adamw_update4(pv, g, mm, vv, h, (fl & 1) != 0);
        reinterpret_cast<float4*>(z.m_shard)[j] = mm;
        reinterpret_cast<float4*>(z.v_shard)[j] = vv;
      }
      __nv_bfloat162 b0 = __floats2bfloat162_rn(pv.x, pv.y), b1 = __floats2bfloat162_rn(pv.z, pv.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&b0);
      pk.y = *reinterpret_cast<uint32_t*>(&b1);
      for (int d = 0; d < p.world; ++d) {
        const int r = (p.rank + d) % p.world;
        st_peer4(z.val[r] + 4 * i, pv);
        if (z.shadow[r])
          asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(reinterpret_cast<uint2*>(z.shadow[r]) + i), "r"(pk.x), "r"(pk.y) : "memory");
      }
    }
  }
  // every shard has landed in my values, and nobody reads my gradients any more
  ok = cross_barrier(p, SIG_PHASE, bases[SIG_PHASE], status, 41, &sh_ok) && ok;
  if (ok && z.zero_grad) {
    const float4 zz = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long i = i0; i < p.n4; i += stride) reinterpret_cast<float4*>(p.grd[p.rank])[i] = zz;
  }
  publish_bases(my, bases, p.world, (1u << SIG_ARRIVE) | (1u << SIG_PHASE));
}

// ------------------------------------------------------------------------------------------ push (small buckets)
// Latency-optimal form for buckets of up to a few MB: ONE NVLink traversal and no cross-GPU barrier.
//   1. every block loads its 16 KB chunk of the local gradients and STORES it into a per-source inbox on every peer,
//      then publishes one flag per (source, block) on that peer (st.release.sys after a block barrier);
//   2. the block spins on ITS OWN local flags (one per peer) and sums the chunk in rank order 0..N-1 (own
//      contribution from registers), so every replica computes bit-identical sums;
//   3. Adam(W) + bf16 recast (or the plain scaled sum), and the local gradients are cleared at once: nobody reads
//      them remotely in this protocol.
// The inbox is double-buffered by the parity of a device-resident epoch, so "done" needs no round: a peer can only
// write parity e again in launch e+2, and its launch e+1 completed only after it saw this rank's flags of e+1,
// which this rank's launch e+1 sends after its launch e (all reads of parity e) has finished.
// Blocks never wait before they send, so any schedule of the grid makes progress: no co-residency requirement.
// Several optimizers' arenas ("segments") travel in one launch; the Adam step counters advance in the same kernel.
constexpr int PUSH_THREADS = 256, PUSH_U = 4, PUSH_MAX_SEG = 4, PUSH_MAX_BLOCKS = 1024;
constexpr int PUSH_CHUNK4 = PUSH_THREADS * PUSH_U;  // float4 per block

struct PushSeg {
  float* grd;            // local gradients of this segment
  float* out;            // plain all-reduce: where the (scaled) sum goes; null with an update
  float *val, *m, *v;
  __nv_bfloat16* shadow;
  const unsigned char* row_flags;
  float* hyper;          // device hyper block; its step counter advances here when `advance`
  long long n4;          // float4 count
  long long off4;        // offset of the segment inside an inbox plane (float4)
  int first_block;
  int advance, zero_grad;
};
struct PushParams {
  float* inbox[MAX_RANKS];         // every rank's inbox  [2][world][plane4] float4
  unsigned int* flags[MAX_RANKS];  // every rank's flags  [2][world][PUSH_MAX_BLOCKS]
  unsigned int* ctl;               // local: [0] epoch of the last finished launch, [1] ticket
  long long plane4;
  int world, rank, nseg;
  unsigned long long wait_ns;
  PushSeg seg[PUSH_MAX_SEG];
};

__global__ void __launch_bounds__(PUSH_THREADS)
ar_push_kernel(const __grid_constant__ PushParams p, unsigned int* status) {
  __shared__ int sh_ok;
  const unsigned int epoch = ld_acquire_sys(p.ctl) + 1u;
  const unsigned int par = epoch & 1u;
  int s = 0;
  while (s + 1 < p.nseg && (int)blockIdx.x >= p.seg[s + 1].first_block) ++s;
  const PushSeg& sg = p.seg[s];
  const long long base = (long long)((int)blockIdx.x - sg.first_block) * PUSH_CHUNK4 + threadIdx.x;
  float4 g[PUSH_U];
#pragma unroll
  for (int u = 0; u < PUSH_U; ++u) {
    const long long i = base + u * PUSH_THREADS;
    g[u] = i < sg.n4 ? reinterpret_cast<const float4*>(sg.grd)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  // ---- 1. push to every peer (ring order spreads the traffic over the links), then one flag per peer
  const long long plane = ((long long)par * p.world + p.rank) * p.plane4 + sg.off4;
  for (int d = 1; d < p.world; ++d) {
    float* dst = p.inbox[(p.rank + d) % p.world] + 4 * plane;
#pragma unroll
    for (int u = 0; u < PUSH_U; ++u) {
      const long long i = base + u * PUSH_THREADS;
      if (i < sg.n4) st_peer4(dst + 4 * i, g[u]);
    }
  }
  if (threadIdx.x == 0) sh_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < p.world - 1) {
    const int peer = (p.rank + 1 + threadIdx.x) % p.world;
    __threadfence_system();
    st_release_sys(p.flags[peer] + ((size_t)par * p.world + p.rank) * PUSH_MAX_BLOCKS + blockIdx.x, epoch);
  }
  // ---- 2. wait for this block's chunk from every peer (local polls)
  if ((int)threadIdx.x < p.world && (int)threadIdx.x != p.rank) {
    if (!wait_flag_ge_ns(p.flags[p.rank] + ((size_t)par * p.world + threadIdx.x) * PUSH_MAX_BLOCKS + blockIdx.x, epoch, status,
                         30, threadIdx.x, p.wait_ns))
      sh_ok = 0;
  }
  __syncthreads();
  const bool ok = sh_ok != 0;
  // ---- 3. rank-ordered sum, update, clear
  AdamHyper h;
  if (sg.hyper) {
    h = load_hyper(sg.hyper);
    if (sg.advance) { h.b1t *= h.beta1; h.b2t *= h.beta2; }
  }
  if (ok) {
    const float* mine = p.inbox[p.rank];
#pragma unroll
    for (int u = 0; u < PUSH_U; ++u) {
      const long long i = base + u * PUSH_THREADS;
      if (i >= sg.n4) continue;
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int r = 0; r < p.world; ++r) {
        const float4 x = r == p.rank ? g[u] : ld_peer4(mine + 4 * ((((long long)par * p.world + r) * p.plane4 + sg.off4) + i));
        acc.x += x.x; acc.y += x.y; acc.z += x.z; acc.w += x.w;
      }
      if (sg.val) {
        AdamBufs a;
        a.val = sg.val; a.m = sg.m; a.v = sg.v; a.shadow = sg.shadow; a.row_flags = sg.row_flags;
        update4(a, h, i, acc);
      } else if (sg.out) {
        const float sc = sg.hyper ? h.gscale : 1.f;
        reinterpret_cast<float4*>(sg.out)[i] = make_float4(acc.x * sc, acc.y * sc, acc.z * sc, acc.w * sc);
      }
      if (sg.zero_grad) reinterpret_cast<float4*>(sg.grd)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  // ---- 4. last block publishes the epoch and the advanced step counters
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(p.ctl + 1, 1u) == gridDim.x - 1) {
      p.ctl[1] = 0u;
      for (int k = 0; k < p.nseg; ++k) {
        float* hy = p.seg[k].hyper;
        if (hy && p.seg[k].advance) {
          hy[NB_H_T] += 1.f;
          hy[NB_H_B1T] *= hy[NB_H_BETA1];
          hy[NB_H_B2T] *= hy[NB_H_BETA2];
        }
      }
      __threadfence();
      st_release_sys(p.ctl, epoch);
    }
  }
}

// Waits on a flag that the caller controls: exercises the bounded-wait → status path without any
// fault (used by the failure-detection tests with a flag that nothing sets).
__global__ void wait_flag_probe_kernel(const unsigned int* flag, unsigned int target, unsigned int limit,
                                       unsigned int* status, unsigned int* result) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const bool ok = wait_flag_ge(flag, target, status, 99, 7u, limit);
    result[0] = ok ? 1u : 0u;
  }
}

int grid_for(long long n4, int threads) {
  long long b = (n4 + threads - 1) / threads;
  if (b < 1) b = 1;
  if (b > 148) b = 148;  // one co-resident wave: blocks wait on each other
  return (int)b;
}

}  // namespace

extern "C" {

// ---- CUDA IPC plumbing for the symmetric heap (set-up time only)
int nb_symm_alloc(void** out, long long bytes) {
  NB_CUDA(cudaMalloc(out, (size_t)bytes));
  NB_CUDA(cudaMemset(*out, 0, (size_t)bytes));
  return NB_OK;
}
int nb_symm_free(void* p) { return (int)cudaFree(p); }
int nb_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  NB_CUDA(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, sizeof(h));
  return NB_OK;
}
int nb_ipc_open_handle(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  NB_CUDA(cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess));
  return NB_OK;
}
int nb_ipc_close_handle(void* p) { return (int)cudaIpcCloseMemHandle(p); }
int nb_enable_peer_access(int peer_dev) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_dev, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); return NB_OK; }
  return (int)e;
}

// algo: 0 one-shot, 1 two-shot, 2 multimem.  Pointers arrays have `world` entries.
// val == NULL → plain all-reduce: the (optionally scaled) sum lands in red[rank].
int nb_allreduce_fused(int algo, int world, int rank, void* const* grd_ptrs, void* const* red_ptrs,
                       void* const* sig_ptrs, void* grd_mc, void* red_mc, long long n, float* val, float* m,
                       float* v, void* shadow, const unsigned char* row_flags, const float* hyper, float* partials,
                       float* norm_out, float max_norm, int zero_grad, unsigned int spin_limit, unsigned int* status,
                       void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return NB_ERR_BAD_ARG;
  if (n % 4) return NB_ERR_UNALIGNED;
  if (algo == 2 && (!grd_mc || !red_mc)) return NB_ERR_BAD_ARG;
  ARParams p;
  for (int r = 0; r < MAX_RANKS; ++r) {
    p.grd[r] = r < world ? (float*)grd_ptrs[r] : nullptr;
    p.red[r] = (r < world && red_ptrs) ? (float*)red_ptrs[r] : nullptr;
    p.sig[r] = r < world ? (unsigned int*)sig_ptrs[r] : nullptr;
  }
  p.grd_mc = (float*)grd_mc;
  p.red_mc = (float*)red_mc;
  p.world = world;
  p.rank = rank;
  p.n4 = n / 4;
  p.spin_limit = spin_limit ? spin_limit : (1u << 24);
  AdamBufs a;
  a.val = val; a.m = m; a.v = v;
  a.shadow = (__nv_bfloat16*)shadow;
  a.row_flags = row_flags;
  a.hyper = hyper;
  a.partials = partials;
  a.norm_out = norm_out;
  a.max_norm = max_norm;
  a.do_update = val != nullptr;
  a.zero_grad = zero_grad;
  if ((a.do_update && max_norm > 0.f && !partials) || ((algo != 0 || !a.do_update || max_norm > 0.f) && !red_ptrs))
    return NB_ERR_BAD_ARG;
  cudaStream_t s = (cudaStream_t)stream;
  const int threads = 512;
  if (algo == 0) {
    ar_oneshot_kernel<<<grid_for(p.n4, threads), threads, 0, s>>>(p, a, status);
  } else {
    const long long per = (p.n4 + world - 1) / world;
    // grid sized for the larger of the two phases but never beyond one wave
    const int grid = grid_for(p.n4 > per * 2 ? p.n4 / 2 : p.n4, threads);
    if (algo == 1) ar_twoshot_kernel<false><<<grid, threads, 0, s>>>(p, a, status);
    else ar_twoshot_kernel<true><<<grid, threads, 0, s>>>(p, a, status);
  }
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// Push all-reduce of up to PUSH_MAX_SEG arenas in one launch (see ar_push_kernel).  Per segment k: grd[k] (local,
// n[k] floats, multiple of 4), and either an update (val/m/v/shadow/row_flags/hyper; `advance` also steps the Adam
// counters t, β₁ᵗ, β₂ᵗ inside the kernel) or a plain sum into out[k] (scaled by hyper[GSCALE] when hyper[k] is given).
// inbox_ptrs / flag_ptrs: every rank's inbox (2·world·plane floats, plane = Σ n[k] rounded up to 1024-float chunks
// per segment) and flag block (2·world·1024 u32, zero-initialised); ctl: 4 local u32, zero-initialised.
int nb_push_blocks(long long n) { return (int)((n / 4 + PUSH_CHUNK4 - 1) / PUSH_CHUNK4); }
int nb_allreduce_push(int world, int rank, int nseg, void* const* inbox_ptrs, void* const* flag_ptrs, unsigned int* ctl,
                      float* const* grd, float* const* out, float* const* val, float* const* m, float* const* v,
                      void* const* shadow, const unsigned char* const* row_flags, float* const* hyper, const long long* n,
                      int advance, int zero_grad, unsigned int spin_limit, unsigned int* status, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || nseg < 1 || nseg > PUSH_MAX_SEG) return NB_ERR_BAD_ARG;
  PushParams p;
  memset(&p, 0, sizeof(p));
  for (int r = 0; r < world; ++r) {
    p.inbox[r] = (float*)inbox_ptrs[r];
    p.flags[r] = (unsigned int*)flag_ptrs[r];
  }
  p.ctl = ctl;
  p.world = world; p.rank = rank; p.nseg = nseg;
  p.wait_ns = 256ull * (spin_limit ? spin_limit : (1u << 24));
  int blocks = 0;
  long long off4 = 0;
  for (int k = 0; k < nseg; ++k) {
    if (n[k] <= 0 || n[k] % 4) return NB_ERR_UNALIGNED;
    PushSeg& sg = p.seg[k];
    sg.grd = grd[k];
    sg.out = out ? out[k] : nullptr;
    sg.val = val ? val[k] : nullptr;
    sg.m = m ? m[k] : nullptr;
    sg.v = v ? v[k] : nullptr;
    sg.shadow = shadow ? (__nv_bfloat16*)shadow[k] : nullptr;
    sg.row_flags = row_flags ? row_flags[k] : nullptr;
    sg.hyper = hyper ? hyper[k] : nullptr;
    sg.n4 = n[k] / 4;
    sg.off4 = off4;
    sg.first_block = blocks;
    sg.advance = advance && sg.val != nullptr;
    sg.zero_grad = zero_grad;
    if (sg.val && (!sg.m || !sg.v || !sg.hyper)) return NB_ERR_BAD_ARG;
    const int nb_ = nb_push_blocks(n[k]);
    blocks += nb_;
    off4 += (long long)nb_ * PUSH_CHUNK4;
  }
  if (blocks > PUSH_MAX_BLOCKS) return NB_ERR_TOO_LARGE;
  p.plane4 = off4;
  ar_push_kernel<<<blocks, PUSH_THREADS, 0, (cudaStream_t)stream>>>(p, status);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// ZeRO-1 step in one kernel (see ar_zero_kernel).  n: arena length in floats (multiple of 4); the slice of rank r is
// float4 range [per·r, per·(r+1)) with per = nb_zero_slice4(n, world); m_shard / v_shard hold 4·per floats.
long long nb_zero_slice4(long long n, int world) { return ((n / 4 + world - 1) / world + 7) / 8 * 8; }
int nb_zero_step_fused(int world, int rank, void* const* grd_ptrs, void* const* val_ptrs, void* const* shadow_ptrs,
                       void* const* sig_ptrs, long long n, float* m_shard, float* v_shard, const unsigned char* row_flags,
                       const float* hyper, int zero_grad, unsigned int spin_limit, unsigned int* status, void* stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || !hyper || !m_shard || !v_shard) return NB_ERR_BAD_ARG;
  if (n % 4) return NB_ERR_UNALIGNED;
  ARParams p;
  ZeroBufs z;
  for (int r = 0; r < MAX_RANKS; ++r) {
    p.grd[r] = r < world ? (float*)grd_ptrs[r] : nullptr;
    p.red[r] = nullptr;
    p.sig[r] = r < world ? (unsigned int*)sig_ptrs[r] : nullptr;
    z.val[r] = r < world ? (float*)val_ptrs[r] : nullptr;
    z.shadow[r] = (r < world && shadow_ptrs) ? (__nv_bfloat16*)shadow_ptrs[r] : nullptr;
  }
  p.grd_mc = p.red_mc = nullptr;
  p.world = world; p.rank = rank; p.n4 = n / 4;
  p.spin_limit = spin_limit ? spin_limit : (1u << 24);
  z.m_shard = m_shard; z.v_shard = v_shard; z.row_flags = row_flags; z.hyper = hyper; z.zero_grad = zero_grad;
  ar_zero_kernel<<<grid_for(p.n4 / world > 0 ? p.n4 / world : 1, 512), 512, 0, (cudaStream_t)stream>>>(p, z, status);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_wait_flag_probe(const unsigned int* flag, unsigned int target, unsigned int limit, unsigned int* status,
                       unsigned int* result, void* stream) {
  wait_flag_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flag, target, limit, status, result);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
