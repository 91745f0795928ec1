// Tensor-parallel GEMMs fused with their collective over NVLink peer memory (sequence-parallel Megatron
// layout: activations outside attention / FFN are sharded by token rows across the P ranks of a node).
//
//   all-gather → GEMM   Y[P·Ms, N] = concat_p(X_p)[P·Ms, K] · B        (column-parallel weight: each rank owns N columns)
//   GEMM → reduce-scatter   Y_r[Ms, N] = Σ_p ( A_p[P·Ms, K_p] · B_p )[rows of rank r]   (row-parallel weight)
//
// Both are ONE kernel per rank built around the tcgen05 main loop of gemm_tcgen05.cu (TMA → smem ring →
// tcgen05.mma into TMEM → epilogue warps), with the transfer overlapped tile by tile:
//
//   AG→GEMM   a few "fetch" CTAs pull the peers' row shards into a local staging buffer, 128-row block by block, in
//             ring order starting at the neighbour, and publish a per-block ready flag; the GEMM CTAs walk the
//             tiles in the same order (own rows first), their TMA producer waits on the flag of a row block before
//             loading it.  A remote row crosses NVLink exactly once, however many N tiles consume it.  The fetch
//             itself is a ring of untiled bulk copies (peer global → shared → local global, 32 KB each, five in
//             flight per CTA) issued by one thread, so a handful of CTAs keep megabytes of reads outstanding;
//             shards whose rows are not contiguous fall back to P2P vector loads.  No copy carries a multicast
//             qualifier, and the tensor-map loads of the GEMM only ever address local memory.
//   GEMM→RS   the epilogue converts each partial tile to bf16 in shared memory (128-byte swizzle) and ships it to
//             the OWNER rank's slot buffer slot[src][row, :] with two tensor-map TMA stores over NVLink, then
//             bumps the owner's per-row-block arrival counter (red.release.sys) once the store has completed;
//             tiles owned by other ranks are computed first.  When a CTA runs out of tiles it reduces local row
//             blocks whose P·tiles_n arrivals are complete — in rank order, so the sum is deterministic —
//             optionally adds a residual, and writes the bf16 result.
//
// Flags are monotone epochs in device memory (graph-replay safe); every wait is bounded by elapsed time (a peer may
// be late by a host-side hiccup) and reports NB_ST_PEER_TIMEOUT / NB_ST_MBAR_TIMEOUT through `status`.  The reference has no tensor parallelism
// (noeira/nn/distributed/strategy.mojo:1-33 lists DDP and ZeRO only); the baseline these kernels are measured
// against is NCCL all_gather_into_tensor / reduce_scatter_tensor around the unfused GEMM.
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "gemm_api.h"

namespace {
using namespace nb;

constexpr int BM = 128, BN = 128, BK = 64, UMMA_K = 16, STAGES = 5;
constexpr int NUM_THREADS = 192;
constexpr int MAX_RANKS = 8;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
// reduce-scatter epilogue staging: two buffers of one bf16 tile = 2 boxes of [128 rows x 64 columns], 128-byte swizzle
constexpr uint32_t EPI_BOX_BYTES = BM * 64 * 2, EPI_BUF_BYTES = 2 * EPI_BOX_BYTES, EPI_BYTES = 2 * EPI_BUF_BYTES;
// all-gather fetch ring (fetch CTAs reuse the dynamic shared memory of the GEMM pipeline)
constexpr int FETCH_SLOTS = 6;
constexpr uint32_t FETCH_CHUNK = 32768;
// control block (u32, local device memory, zero-initialised once):
//   [0] epoch of the last completed launch   [1] ticket   [2] arrive counter (peers add)   [3] done counter
//   [16 + i] per-row-block flag / arrival counter
constexpr int CTL_EPOCH = 0, CTL_TICKET = 1, CTL_ARRIVE = 2, CTL_DONE = 3, CTL_BLOCKS = 16;

struct TpParams {
  int M, N, K;          // GEMM extents on this rank (M = P·Ms for both kernels)
  int Ms;               // rows per rank shard
  int world, rank;
  int b_mn;             // B operand major
  int ldd;              // output pitch (elements)
  int tiles_m, tiles_n, num_kb;
  int n_fetch;          // AG: number of fetch CTAs
  int ldx;              // AG: pitch of the shard / staging rows (elements)
  int ld_slot;          // RS: pitch of a slot row (elements)
  int ld_res;           // RS: residual pitch
  const float* bias;
  int act;
  unsigned long long wait_ns;  // bound of every wait that depends on a peer; mbarrier waits get twice that
  const __nv_bfloat16* x_peer[MAX_RANKS];  // AG: every rank's shard [Ms, K]
  __nv_bfloat16* stage;                    // AG: local staging [P·Ms, K]
  __nv_bfloat16* slot_peer[MAX_RANKS];     // RS: every rank's slot buffer [P][Ms, N]
  unsigned int* ctl_peer[MAX_RANKS];       // control blocks
  __nv_bfloat16* D;                        // AG: [M, N] local output; RS: [Ms, N] reduced output
  const __nv_bfloat16* residual;           // RS: optional [Ms, N]
  unsigned int* status;
};
struct SlotMaps {
  CUtensorMap m[MAX_RANKS];  // RS: every rank's slot buffer [P·Ms, N] as seen from this process (box 64 x 128)
};

__device__ __forceinline__ float act_apply(int act, float v) {
  if (act == NB_ACT_RELU) return fmaxf(v, 0.f);
  if (act == NB_ACT_TANH) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(v));
    return y;
  }
  if (act == NB_ACT_SILU) return v / (1.f + __expf(-v));
  if (act == NB_ACT_GELU) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    return 0.5f * v * (1.f + t);
  }
  return v;
}

__device__ __forceinline__ uint4 ld_peer16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned int* p, unsigned int v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ bool wait_ge_gpu(const unsigned int* p, unsigned int target, unsigned int* status,
                                            unsigned int where, unsigned long long limit_ns) {
  if ((int)(ld_acquire_gpu(p) - target) >= 0) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    for (int i = 0; i < 64; ++i) {
      if ((int)(ld_acquire_gpu(p) - target) >= 0) return true;
      __nanosleep(40);
    }
    if (globaltimer_ns() - t0 > limit_ns) break;
  }
  report(status, NB_ST_PEER_TIMEOUT, where, target);
  return false;
}

// Row blocks in ring order: own rank first, then rank+1, ... ; `first_remote` rotates so that OTHER ranks'
// blocks come first (reduce-scatter).  Returns the global row-block index of position `pos`.
__device__ __forceinline__ int ordered_block(const TpParams& p, int pos, int blocks_per_rank, bool remote_first) {
  const int rr = pos / blocks_per_rank, within = pos - rr * blocks_per_rank;
  const int owner = (p.rank + rr + (remote_first ? 1 : 0)) % p.world;
  return owner * blocks_per_rank + within;
}

// ------------------------------------------------------------------------------------------ shared main loop
struct Pipe {
  uint8_t* smem;
  uint8_t* epi;  // reduce-scatter staging (EPI_BYTES, 1024-byte aligned)
  uint64_t *full_bar, *empty_bar, *tfull_bar, *tempty_bar;
  uint32_t* tmem_slot;
  volatile uint32_t* abort_flag;
  unsigned long long mbar_ns;
};

__device__ __forceinline__ Pipe carve_pipe(uint8_t* smem_raw, unsigned long long wait_ns) {
  Pipe q;
  q.smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  q.epi = q.smem + STAGES * STAGE_BYTES;
  q.mbar_ns = 2ull * wait_ns;
  q.full_bar = reinterpret_cast<uint64_t*>(q.smem + STAGES * STAGE_BYTES + EPI_BYTES);
  q.empty_bar = q.full_bar + STAGES;
  q.tfull_bar = q.empty_bar + STAGES;
  q.tempty_bar = q.tfull_bar + 2;
  q.tmem_slot = reinterpret_cast<uint32_t*>(q.tempty_bar + 2);
  q.abort_flag = q.tmem_slot + 1;
  return q;
}

__device__ __forceinline__ void issue_tile_mma(const Pipe& q, uint32_t d_tmem, uint32_t idesc, int b_mn, int num_kb,
                                               int& stage, uint32_t& phase, unsigned int* status, bool& ok) {
  for (int kb = 0; kb < num_kb; ++kb) {
    if (*q.abort_flag || !mbar_wait_ns(&q.full_bar[stage], phase, status, 403, q.mbar_ns)) { ok = false; *q.abort_flag = 1; return; }
    tc_fence_after();
    const uint32_t sa = smem_u32(q.smem + stage * STAGE_BYTES), sb = sa + A_BYTES;
#pragma unroll
    for (int k = 0; k < BK / UMMA_K; ++k) {
      const uint64_t adesc = make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024, 2);
      const uint64_t bdesc = b_mn ? make_smem_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024, 2)
                                  : make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024, 2);
      umma_f16(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
    }
    umma_commit(&q.empty_bar[stage]);
    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
  }
}

__device__ __forceinline__ void load_b_tile(const Pipe& q, const CUtensorMap* tmB, int b_mn, int stage, int kb, int nb_) {
  uint8_t* sb = q.smem + stage * STAGE_BYTES + A_BYTES;
  if (!b_mn) {
    tma_load_2d(sb, tmB, &q.full_bar[stage], kb * BK, nb_ * BN);
  } else {
#pragma unroll
    for (int h = 0; h < BN / 64; ++h) tma_load_2d(sb + h * (64 * BK * 2), tmB, &q.full_bar[stage], nb_ * BN + h * 64, kb * BK);
  }
}

__device__ __forceinline__ void pipe_setup(const Pipe& q, int warp) {
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&q.full_bar[s], 1);
      mbar_init(&q.empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&q.tfull_bar[a], 1);
      mbar_init(&q.tempty_bar[a], 4);
    }
    *q.abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(q.tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

// Last CTA of the grid publishes the epoch.
__device__ __forceinline__ void finish_epoch(unsigned int* ctl, unsigned int epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctl + CTL_TICKET, 1u) == gridDim.x - 1) {
      ctl[CTL_TICKET] = 0u;
      __threadfence();
      st_release_gpu(ctl + CTL_EPOCH, epoch);
    }
  }
}

// ------------------------------------------------------------------------------------------ AG → GEMM
__global__ void __launch_bounds__(NUM_THREADS, 1)
tp_ag_gemm_kernel(const __grid_constant__ CUtensorMap tmOwn, const __grid_constant__ CUtensorMap tmStage,
                  const __grid_constant__ CUtensorMap tmB, const TpParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  unsigned int* ctl = p.ctl_peer[p.rank];
  const unsigned int epoch = ld_acquire_gpu(ctl + CTL_EPOCH) + 1u;
  const int bpr = p.Ms / BM;  // row blocks per rank
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if ((int)blockIdx.x < p.n_fetch) {
    // ---------------------------------------------------------------- fetch CTAs
    __shared__ bool sh_ok;
    // everyone's shard is complete once every rank has entered this launch
    if (threadIdx.x == 0) {
      bool ok = true;
      if (blockIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < p.world; ++r) red_release_sys_add(p.ctl_peer[r] + CTL_ARRIVE, 1u);
      }
      ok = wait_flag_ge_ns(ctl + CTL_ARRIVE, epoch * (unsigned int)p.world, p.status, 410, 0u, p.wait_ns);
      asm volatile("fence.proxy.async.global;" ::: "memory");  // the bulk copies below read what the peers' kernels wrote
      sh_ok = ok;
    }
    __syncthreads();
    bool ok = sh_ok;
    const int row_vecs = p.K / 8;  // 16-byte vectors per row
    const int remote_blocks = (p.world - 1) * bpr;
    if (p.ldx == p.K) {
      // Rows are contiguous: a row block is one byte range.  One thread runs a ring of bulk copies
      // peer → shared → local; the other threads of the CTA have nothing to do.
      if (threadIdx.x == 0 && ok) {
        uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
        uint64_t* fbar = reinterpret_cast<uint64_t*>(ring + (size_t)FETCH_SLOTS * FETCH_CHUNK);
        for (int i = 0; i < FETCH_SLOTS; ++i) mbar_init(&fbar[i], 1);
        fence_barrier_init();
        const uint32_t block_bytes = (uint32_t)BM * (uint32_t)p.K * 2u;
        const uint32_t cpb = (block_bytes + FETCH_CHUNK - 1) / FETCH_CHUNK;  // chunks per row block
        int my_blocks = 0;
        for (int pos = blockIdx.x; pos < remote_blocks; pos += p.n_fetch) ++my_blocks;
        const uint32_t total = (uint32_t)my_blocks * cpb;
        uint32_t issued = 0;
        for (uint32_t done = 0; done < total && ok; ++done) {
          // keep FETCH_SLOTS - 1 loads in flight ahead of the chunk being stored
          while (issued < total && issued < done + FETCH_SLOTS - 1 + (done == 0 ? 1 : 0)) {
            const uint32_t bi = issued / cpb, ci = issued - bi * cpb;
            const int gb = ordered_block(p, blockIdx.x + (int)bi * p.n_fetch, bpr, true);
            const int owner = gb / bpr, lb = gb - owner * bpr;
            const uint32_t off = ci * FETCH_CHUNK;
            const uint32_t bytes = min(FETCH_CHUNK, block_bytes - off);
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.x_peer[owner]) + (size_t)lb * block_bytes + off;
            const uint32_t slot = issued % FETCH_SLOTS;
            mbar_expect_tx(&fbar[slot], bytes);
            bulk_load(ring + (size_t)slot * FETCH_CHUNK, src, bytes, &fbar[slot]);
            ++issued;
          }
          const uint32_t bi = done / cpb, ci = done - bi * cpb;
          const int gb = ordered_block(p, blockIdx.x + (int)bi * p.n_fetch, bpr, true);
          const uint32_t off = ci * FETCH_CHUNK;
          const uint32_t bytes = min(FETCH_CHUNK, block_bytes - off);
          const uint32_t slot = done % FETCH_SLOTS;
          if (!mbar_wait_ns(&fbar[slot], (done / FETCH_SLOTS) & 1u, p.status, 412, 2ull * p.wait_ns)) { ok = false; break; }
          bulk_store(reinterpret_cast<uint8_t*>(p.stage) + (size_t)gb * block_bytes + off, ring + (size_t)slot * FETCH_CHUNK, bytes);
          tma_store_commit();
          if (ci == cpb - 1) {
            // the whole row block has been written locally: make it visible, then publish its flag
            tma_store_wait_all();
            asm volatile("fence.proxy.async.global;" ::: "memory");
            __threadfence();
            st_release_gpu(ctl + CTL_BLOCKS + gb, epoch);
          } else {
            tma_store_wait_read();  // the slot may be refilled once the store has read it
          }
        }
        tma_store_wait_all();
        sh_ok = ok;
      }
      __syncthreads();
      ok = sh_ok;
    } else {
      for (int pos = blockIdx.x; pos < remote_blocks && ok; pos += p.n_fetch) {
        const int gb = ordered_block(p, pos, bpr, true);  // remote ranks in ring order
        const int owner = gb / bpr, lb = gb - owner * bpr;
        const __nv_bfloat16* src = p.x_peer[owner] + (size_t)lb * BM * p.ldx;
        __nv_bfloat16* dst = p.stage + (size_t)gb * BM * p.ldx;
        const int total = BM * row_vecs;
        for (int i0 = threadIdx.x; i0 < total; i0 += NUM_THREADS * 8) {
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * NUM_THREADS;
            if (i < total) {
              const int rr = i / row_vecs, cv = i - rr * row_vecs;
              v[u] = ld_peer16(src + (size_t)rr * p.ldx + cv * 8);
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int i = i0 + u * NUM_THREADS;
            if (i < total) {
              const int rr = i / row_vecs, cv = i - rr * row_vecs;
              *reinterpret_cast<uint4*>(dst + (size_t)rr * p.ldx + cv * 8) = v[u];
            }
          }
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) st_release_gpu(ctl + CTL_BLOCKS + gb, epoch);
      }
    }
    // nobody may overwrite a shard while a peer still reads it: wait until every rank has fetched everything
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      for (int r = 0; r < p.world; ++r) red_release_sys_add(p.ctl_peer[r] + CTL_DONE, 1u);
      wait_flag_ge_ns(ctl + CTL_DONE, epoch * (unsigned int)(p.world * p.n_fetch), p.status, 411, 0u, p.wait_ns);
    }
    finish_epoch(ctl, epoch);
    return;
  }

  // ------------------------------------------------------------------ GEMM CTAs
  Pipe q = carve_pipe(smem_raw, p.wait_ns);
  pipe_setup(q, warp);
  const uint32_t tmem_base = *q.tmem_slot;
  const int ncta = gridDim.x - p.n_fetch, cta = blockIdx.x - p.n_fetch;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        const int pos = t / p.tiles_n, nb_ = t - pos * p.tiles_n;
        const int gb = ordered_block(p, pos, bpr, false);  // own rows first
        const int owner = gb / bpr;
        const bool own = owner == p.rank;
        if (!own) {
          if (!wait_ge_gpu(ctl + CTL_BLOCKS + gb, epoch, p.status, 420, p.wait_ns)) { ok = false; *q.abort_flag = 1; break; }
          asm volatile("fence.proxy.async.global;" ::: "memory");  // staged rows were written through the generic proxy
        }
        const int row0 = own ? (gb - owner * bpr) * BM : gb * BM;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (*q.abort_flag || !mbar_wait_ns(&q.empty_bar[stage], phase ^ 1u, p.status, 401, q.mbar_ns)) { ok = false; *q.abort_flag = 1; break; }
          mbar_expect_tx(&q.full_bar[stage], STAGE_BYTES);
          tma_load_2d(q.smem + stage * STAGE_BYTES, own ? &tmOwn : &tmStage, &q.full_bar[stage], kb * BK, row0);
          load_b_tile(q, &tmB, p.b_mn, stage, kb, nb_);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc(1u, BM, BN, 0u, (uint32_t)p.b_mn);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        if (*q.abort_flag || !mbar_wait_ns(&q.tempty_bar[acc], acc_phase ^ 1u, p.status, 402, q.mbar_ns)) { ok = false; *q.abort_flag = 1; break; }
        tc_fence_after();
        issue_tile_mma(q, tmem_base + acc * BN, idesc, p.b_mn, p.num_kb, stage, phase, p.status, ok);
        if (!ok) break;
        umma_commit(&q.tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int t = cta; t < num_tiles && ok; t += ncta) {
      const int pos = t / p.tiles_n, nb_ = t - pos * p.tiles_n;
      const int gb = ordered_block(p, pos, bpr, false);
      if (*q.abort_flag || !mbar_wait_ns(&q.tfull_bar[acc], acc_phase, p.status, 404, q.mbar_ns)) { ok = false; *q.abort_flag = 1; break; }
      tc_fence_after();
      const int row = gb * BM + quarter * 32 + lane;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32b_x32(taddr0 + c0, r);
        tmem_ld_wait();
        const int col0 = nb_ * BN + c0;
        if (row < p.M && col0 < p.N) {
          __nv_bfloat16* o = p.D + (size_t)row * p.ldd + col0;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              v[u] = __uint_as_float(r[j + u]);
              if (p.bias && col0 + j + u < p.N) v[u] += p.bias[col0 + j + u];
              if (p.act) v[u] = act_apply(p.act, v[u]);
            }
            if (col0 + j + 8 <= p.N) {
              uint4 pk;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(v[0], v[1]), h1 = __floats2bfloat162_rn(v[2], v[3]),
                             h2 = __floats2bfloat162_rn(v[4], v[5]), h3 = __floats2bfloat162_rn(v[6], v[7]);
              pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
              pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
              *reinterpret_cast<uint4*>(o + j) = pk;
            } else {
              for (int u = 0; u < 8; ++u)
                if (col0 + j + u < p.N) o[j + u] = __float2bfloat16(v[u]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q.tempty_bar[acc]);
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  finish_epoch(ctl, epoch);
}

// Sum of the `world` slot copies of one 128 x 128 output tile of this rank (+ residual) → bf16 D.  W = upper bound of the
// world size, U = vectors per thread and batch: W·U 16-byte loads are in flight per thread.
template <int W, int U>
__device__ __forceinline__ void rs_reduce_tile(const TpParams& p, int lb, int nb_, int t128) {
  const __nv_bfloat16* mine = p.slot_peer[p.rank];
  const int c0 = nb_ * BN;
  const int tv = min(BN, p.N - c0) >> 3;   // 16-byte vectors per row of this tile
  const int total = BM * tv;
  for (int i0 = t128; i0 < total; i0 += 128 * U) {
    uint4 sv[U][W];
    uint4 rv[U];
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int i = i0 + k * 128;
      if (i < total) {
        const int rr = i / tv, cv = i - rr * tv;
        const int lrow = lb * BM + rr;
#pragma unroll
        for (int r = 0; r < W; ++r)
          if (r < p.world) sv[k][r] = ld_peer16(mine + ((size_t)r * p.Ms + lrow) * p.ld_slot + c0 + cv * 8);
        if (p.residual) rv[k] = *reinterpret_cast<const uint4*>(p.residual + (size_t)lrow * p.ld_res + c0 + cv * 8);
      }
    }
#pragma unroll
    for (int k = 0; k < U; ++k) {
      const int i = i0 + k * 128;
      if (i < total) {
        const int rr = i / tv, cv = i - rr * tv;
        const int lrow = lb * BM + rr;
        float a[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = 0.f;
        if (p.residual) {
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&rv[k]);
#pragma unroll
          for (int e = 0; e < 4; ++e) { a[2 * e] = __low2float(h[e]); a[2 * e + 1] = __high2float(h[e]); }
        }
#pragma unroll
        for (int r = 0; r < W; ++r) {
          if (r < p.world) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&sv[k][r]);
#pragma unroll
            for (int e = 0; e < 4; ++e) { a[2 * e] += __low2float(h[e]); a[2 * e + 1] += __high2float(h[e]); }
          }
        }
        uint4 pk;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(a[0], a[1]), h1 = __floats2bfloat162_rn(a[2], a[3]),
                       h2 = __floats2bfloat162_rn(a[4], a[5]), h3 = __floats2bfloat162_rn(a[6], a[7]);
        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(p.D + (size_t)lrow * p.ldd + c0 + cv * 8) = pk;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ GEMM → RS
__global__ void __launch_bounds__(NUM_THREADS, 1)
tp_gemm_rs_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                  const __grid_constant__ SlotMaps slots, const TpParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  unsigned int* ctl = p.ctl_peer[p.rank];
  const unsigned int epoch = ld_acquire_gpu(ctl + CTL_EPOCH) + 1u;
  const int bpr = p.Ms / BM;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  Pipe q = carve_pipe(smem_raw, p.wait_ns);
  pipe_setup(q, warp);
  const uint32_t tmem_base = *q.tmem_slot;
  const int ncta = gridDim.x, cta = blockIdx.x;
  const int num_tiles = p.tiles_m * p.tiles_n;
  // entering launch `epoch` tells every peer that this rank has finished reading its slots of launch epoch-1
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < p.world; ++r) red_release_sys_add(p.ctl_peer[r] + CTL_ARRIVE, 1u);
  }

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        const int pos = t / p.tiles_n, nb_ = t - pos * p.tiles_n;
        const int gb = ordered_block(p, pos, bpr, true);  // other ranks' rows first
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (*q.abort_flag || !mbar_wait_ns(&q.empty_bar[stage], phase ^ 1u, p.status, 501, q.mbar_ns)) { ok = false; *q.abort_flag = 1; break; }
          mbar_expect_tx(&q.full_bar[stage], STAGE_BYTES);
          tma_load_2d(q.smem + stage * STAGE_BYTES, &tmA, &q.full_bar[stage], kb * BK, gb * BM);
          load_b_tile(q, &tmB, p.b_mn, stage, kb, nb_);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc(1u, BM, BN, 0u, (uint32_t)p.b_mn);
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int t = cta; t < num_tiles && ok; t += ncta) {
        if (*q.abort_flag || !mbar_wait_ns(&q.tempty_bar[acc], acc_phase ^ 1u, p.status, 502, q.mbar_ns)) { ok = false; *q.abort_flag = 1; break; }
        tc_fence_after();
        issue_tile_mma(q, tmem_base + acc * BN, idesc, p.b_mn, p.num_kb, stage, phase, p.status, ok);
        if (!ok) break;
        umma_commit(&q.tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    // peers must have finished consuming the previous launch before their slots are overwritten
    if (warp == 2 && lane == 0)
      if (!wait_flag_ge_ns(ctl + CTL_ARRIVE, epoch * (unsigned int)p.world, p.status, 510, 0u, p.wait_ns)) *q.abort_flag = 1;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    // Every epilogue thread executes every named barrier below, whatever happened before it (a thread that
    // left early would strand the others), so failures only switch the work off.
    // One thread (`issuer`) owns the TMA stores of this CTA, so their bulk async-groups complete in tile order.
    const bool issuer = warp == 2 && lane == 0;
    int it = 0;
    int pend[3] = {-1, -1, -1};  // (owner << 20 | row block) of the tiles whose stores are in flight, oldest first
    auto signal_block = [&](int packed) {
      asm volatile("fence.proxy.async.global;" ::: "memory");
      __threadfence_system();
      red_release_sys_add(p.ctl_peer[packed >> 20] + CTL_BLOCKS + (packed & 0xFFFFF), 1u);
    };
    for (int t = cta; t < num_tiles; t += ncta, ++it) {
      const int pos = t / p.tiles_n, nb_ = t - pos * p.tiles_n;
      const int gb = ordered_block(p, pos, bpr, true);
      const int owner = gb / bpr, lb = gb - owner * bpr;
      uint8_t* buf = q.epi + (size_t)(it & 1) * EPI_BUF_BYTES;
      if (ok && (*q.abort_flag || !mbar_wait_ns(&q.tfull_bar[acc], acc_phase, p.status, 504, q.mbar_ns))) { ok = false; *q.abort_flag = 1; }
      if (ok) {
        tc_fence_after();
        const int row = quarter * 32 + lane;  // row inside the tile
        const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(taddr0 + c0, r);
          tmem_ld_wait();
          // 32 columns = 4 chunks of 16 bytes inside the 64-column box `c0 / 64`; chunk c of row r sits at c ^ (r & 7)
          uint8_t* box = buf + (size_t)(c0 >> 6) * EPI_BOX_BYTES + (size_t)row * 128;
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1])),
                           h1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])),
                           h2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5])),
                           h3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
            const int chunk = ((c0 & 63) + j) >> 3;
            *reinterpret_cast<uint4*>(box + (size_t)((chunk ^ (row & 7)) << 4)) = pk;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&q.tempty_bar[acc]);
        fence_proxy_async();  // the TMA store reads these shared-memory writes
      }
      // the buffer of the NEXT tile is the one the previous tile's store reads: that read must be over before
      // anyone passes this barrier
      if (issuer) tma_store_wait_read();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (issuer) {
        if (ok) {
          const int y = p.rank * p.Ms + lb * BM;  // row of the tile inside the owner's [P·Ms, N] slot buffer
          tma_store_2d(&slots.m[owner], buf, nb_ * BN, y);
          if (nb_ * BN + 64 < p.N) tma_store_2d(&slots.m[owner], buf + EPI_BOX_BYTES, nb_ * BN + 64, y);
        }
        tma_store_commit();
        // Exactly one bulk group per tile.  Once at most the three newest are pending, the store of tile it-3 has
        // completed → one arrival on its owner's row-block counter.  Four stores in flight hide the NVLink round trip.
        tma_store_wait_all_but<3>();
        if (pend[0] >= 0) signal_block(pend[0]);
        pend[0] = pend[1]; pend[1] = pend[2];
        pend[2] = ok ? ((owner << 20) | lb) : -1;
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (issuer) {
      tma_store_wait_all();
#pragma unroll
      for (int i = 0; i < 3; ++i)
        if (pend[i] >= 0) signal_block(pend[i]);
    }
    // ---- tail: reduce the local row blocks in rank order (deterministic), add the residual, write bf16.  Work unit =
    // one 128 x 128 tile so that every CTA has some; all slot loads of a batch are issued before the first add.
    const unsigned int need = epoch * (unsigned int)(p.world * p.tiles_n);
    const int t128 = (warp - 2) * 32 + lane;  // 0..127
    for (int u = cta; u < bpr * p.tiles_n; u += ncta) {
      const int lb = u / p.tiles_n, nb_ = u - lb * p.tiles_n;
      if (warp == 2 && lane == 0 && !*q.abort_flag)
        if (!wait_flag_ge_ns(ctl + CTL_BLOCKS + lb, need, p.status, 520, (unsigned)lb, p.wait_ns)) *q.abort_flag = 1;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*q.abort_flag) continue;
      if (p.world <= 2) rs_reduce_tile<2, 4>(p, lb, nb_, t128);
      else if (p.world <= 4) rs_reduce_tile<4, 2>(p, lb, nb_, t128);
      else rs_reduce_tile<8, 1>(p, lb, nb_, t128);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
  finish_epoch(ctl, epoch);
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}
int make_tmap(CUtensorMap* tm, const void* base, long long inner, long long outer, long long ld, int box_inner,
              int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return NB_ERR_NO_DRIVER_SYMBOL;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return NB_ERR_UNALIGNED;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NB_OK : NB_ERR_TENSORMAP;
}
int sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}
constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + EPI_BYTES + 1024 + 256;
static_assert(SMEM_BYTES <= 232448, "shared memory budget of one CTA");
static_assert((size_t)FETCH_SLOTS * FETCH_CHUNK + 64 <= (size_t)STAGES * STAGE_BYTES + EPI_BYTES, "fetch ring fits the GEMM pipeline area");

int fill_common(TpParams& p, int world, int rank, int Ms, int N, int K, int b_mn, unsigned int spin_limit,
                void* const* ctl_ptrs, unsigned int* status) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world) return NB_ERR_BAD_ARG;
  if (Ms <= 0 || Ms % BM != 0) return NB_ERR_BAD_ARG;  // shards are whole 128-row blocks
  if (CTL_BLOCKS + world * (Ms / BM) > 4096) return NB_ERR_TOO_LARGE;
  p.world = world; p.rank = rank; p.Ms = Ms; p.M = Ms * world; p.N = N; p.K = K; p.b_mn = b_mn;
  p.tiles_m = p.M / BM; p.tiles_n = ceil_div(N, BN); p.num_kb = ceil_div(K, BK);
  // `spin_limit` counts units of 256 ns (the default 1 << 24 is about 4.3 s)
  p.wait_ns = 256ull * (spin_limit ? spin_limit : (1u << 24));
  p.status = status;
  for (int r = 0; r < MAX_RANKS; ++r) {
    p.ctl_peer[r] = r < world ? (unsigned int*)ctl_ptrs[r] : nullptr;
    p.x_peer[r] = nullptr;
    p.slot_peer[r] = nullptr;
  }
  p.bias = nullptr; p.act = 0; p.residual = nullptr; p.stage = nullptr; p.n_fetch = 0;
  p.ldx = p.ld_slot = p.ld_res = 0;
  return NB_OK;
}
}  // namespace

extern "C" {

// Number of u32 words a control block needs (allocate zeroed, in the symmetric heap).
int nb_tp_ctl_words() { return 4096; }

// Y[P·Ms, N] = act(concat_p(X_p) · B + bias).  x_ptrs[p]: rank p's shard [Ms, K] (pitch ldx) in THIS process'
// address space; stage: local [P·Ms, K] (pitch ldx; the own block is never written); B: [N,K] (b_mn=0, pitch ldb)
// or [K,N] (b_mn=1).  After the call `stage` holds every REMOTE shard (own rows stay in x_ptrs[rank]).
int nb_tp_ag_gemm(int world, int rank, void* const* x_ptrs, void* stage, void* const* ctl_ptrs, const void* B, void* D,
                  int Ms, int N, int K, int ldx, int ldb, int ldd, int b_mn, const float* bias, int act, int n_fetch,
                  unsigned int spin_limit, unsigned int* status, void* stream) {
  TpParams p;
  int rc = fill_common(p, world, rank, Ms, N, K, b_mn, spin_limit, ctl_ptrs, status);
  if (rc) return rc;
  if (K % 8 || ldx % 8) return NB_ERR_UNALIGNED;
  for (int r = 0; r < world; ++r) p.x_peer[r] = (const __nv_bfloat16*)x_ptrs[r];
  p.stage = (__nv_bfloat16*)stage;
  p.ldx = ldx; p.ldd = ldd; p.D = (__nv_bfloat16*)D; p.bias = bias; p.act = act;
  p.n_fetch = world > 1 ? (n_fetch > 0 ? n_fetch : 24) : 0;
  CUtensorMap tmOwn, tmStage, tmB;
  rc = make_tmap(&tmOwn, x_ptrs[rank], K, Ms, ldx, BK, BM);
  if (rc) return rc;
  rc = make_tmap(&tmStage, stage, K, (long long)Ms * world, ldx, BK, BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap(&tmB, B, N, K, ldb, 64, BK) : make_tmap(&tmB, B, K, N, ldb, BK, BN);
  if (rc) return rc;
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(tp_ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    configured = true;
  }
  // one co-resident wave: fetch CTAs and GEMM CTAs wait on one another
  const int tiles = p.tiles_m * p.tiles_n;
  int gemm_ctas = sm_count() - p.n_fetch;
  if (gemm_ctas > tiles) gemm_ctas = tiles;
  tp_ag_gemm_kernel<<<p.n_fetch + gemm_ctas, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tmOwn, tmStage, tmB, p);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// out[Ms, N] = residual + Σ_p (A_p · B_p)[rows of this rank].  A: local [P·Ms, K] (pitch lda); slot_ptrs[p]: rank p's
// slot buffer [P][Ms, N] (pitch ld_slot) in this process' address space.
int nb_tp_gemm_rs(int world, int rank, const void* A, const void* B, void* const* slot_ptrs, void* const* ctl_ptrs,
                  void* out, const void* residual, int Ms, int N, int K, int lda, int ldb, int ld_slot, int ldd,
                  int ld_res, int b_mn, unsigned int spin_limit, unsigned int* status, void* stream) {
  TpParams p;
  int rc = fill_common(p, world, rank, Ms, N, K, b_mn, spin_limit, ctl_ptrs, status);
  if (rc) return rc;
  if (N % 8 || ld_slot % 8 || ldd % 8 || (residual && ld_res % 8)) return NB_ERR_UNALIGNED;
  for (int r = 0; r < world; ++r) p.slot_peer[r] = (__nv_bfloat16*)slot_ptrs[r];
  p.ld_slot = ld_slot; p.ldd = ldd; p.ld_res = ld_res;
  p.D = (__nv_bfloat16*)out; p.residual = (const __nv_bfloat16*)residual;
  CUtensorMap tmA, tmB;
  rc = make_tmap(&tmA, A, K, (long long)Ms * world, lda, BK, BM);
  if (rc) return rc;
  rc = b_mn ? make_tmap(&tmB, B, N, K, ldb, 64, BK) : make_tmap(&tmB, B, K, N, ldb, BK, BN);
  if (rc) return rc;
  SlotMaps slots;
  memset(&slots, 0, sizeof(slots));
  for (int r = 0; r < world; ++r) {
    rc = make_tmap(&slots.m[r], slot_ptrs[r], N, (long long)Ms * world, ld_slot, 64, BM);
    if (rc) return rc;
  }
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(tp_gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
    configured = true;
  }
  const int tiles = p.tiles_m * p.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  tp_gemm_rs_kernel<<<grid, NUM_THREADS, SMEM_BYTES, (cudaStream_t)stream>>>(tmA, tmB, slots, p);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
