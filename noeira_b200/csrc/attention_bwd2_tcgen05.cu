// Flash attention backward, second generation: the same two deterministic kernels (dQ per query tile, dK / dV per key
// tile; no atomics) as attention_bwd_tcgen05.cu, rebuilt so that the tensor core is never left waiting for a load or
// for the exponentials:
//
//   * P and dS never pass through shared memory: they are written back to TENSOR MEMORY as packed bf16 and consumed
//     from there as the A operand of the following GEMM (tcgen05.mma with a TMEM A operand).  That frees 32 - 64 KB of
//     shared memory per CTA, which buys a second stage for the streamed tiles at head_dim 128 — the first-generation
//     kernels exposed one full TMA round trip per block there.
//   * dQ kernel: tensor memory S | dP | dS | dQ.  The softmax threads copy S_j and dP_j into registers and release both
//     accumulators at once, so S_{j+1} = Q K_{j+1}ᵀ and dP_{j+1} = dO V_{j+1}ᵀ run on the tensor core while the threads
//     compute dS_j = P ⊙ (dP − Δ) · scale; dQ += dS_j K_j follows from tensor memory.
//   * dK / dV kernel: works on the TRANSPOSED score tile, Sᵀ = K Qᵀ and dPᵀ = V dOᵀ (rows = keys, columns = queries),
//     because Pᵀ and dSᵀ are then exactly the A operands of dV += Pᵀ dO and dK += dSᵀ Q.  The per-query statistics
//     (log-sum-exp, Δ) become per-COLUMN values, staged in shared memory once per query tile.  The work of a block
//     is split in two phases so that every phase overlaps two GEMMs:  P from Sᵀ  ‖ dK_{i-1}, dPᵀ_i   and
//     dS from dPᵀ ‖ dV_i, Sᵀ_{i+1}.
// Masks, GQA, bounded waits and outputs as in the first generation.
// Reference kernels: noeira/nn/primitives/flash_attention_mma.mojo:375-521 (dq / dkdv split, mma.sync).
#include "attention_common.cuh"

namespace {
using namespace nb;
using namespace nbattn;

// 64 fp32 values of one TMEM row → registers (issued together, one wait)
__device__ __forceinline__ void ld64(uint32_t addr, float (&v)[64]) {
  tmem_ld_32x32b_x32_nowait(addr, reinterpret_cast<uint32_t*>(v));
  tmem_ld_32x32b_x32_nowait(addr + 32, reinterpret_cast<uint32_t*>(v) + 32);
}
// 64 values as 32 packed bf16x2 words → 32 TMEM columns
__device__ __forceinline__ void st32(uint32_t addr, const uint32_t (&w)[32]) { tmem_st_32x32b_x32(addr, w); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// TMEM accumulator row (NC fp32) → bf16 → global
template <int NC>
__device__ __forceinline__ void store_row(uint32_t taddr, __nv_bfloat16* dst) {
#pragma unroll
  for (int c = 0; c < NC; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(taddr + c, r);
    tmem_ld_wait();
    if (dst) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 pk;
        pk.x = pack_bf16(__uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        pk.y = pack_bf16(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        pk.z = pack_bf16(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
        pk.w = pack_bf16(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
        *reinterpret_cast<uint4*>(dst + c + i) = pk;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ dQ
template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_bwd2_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const FaParams p) {
  constexpr int NSUB = HD / 64;
  constexpr int ST = (HD == 64) ? 4 : 2;      // K / V ring depth
  constexpr uint32_t T_BYTES = 128 * HD * 2;  // one [128 x HD] bf16 tile
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DS_COL = 256, DQ_COL = 384;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aQ = smem_u32(smem), adO = aQ + T_BYTES, aK = adO + T_BYTES, aV = aK + ST * T_BYTES, aB = aV + ST * T_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * T_BYTES + 2 * ST * T_BYTES);
  // barrier indices
  constexpr int Q_FULL = 0, KV_FULL = 1, KV_EMPTY = 1 + ST, SDP_FULL = 1 + 2 * ST, SDP_EMPTY = 2 + 2 * ST, DS_FULL = 3 + 2 * ST,
                DS_EMPTY = 4 + 2 * ST, DQ_FULL = 5 + 2 * ST, NBARS = 6 + 2 * ST;
  auto bar = [&](int i) { return aB + 8u * (uint32_t)i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // masked shapes: longest query tiles first
  const int nqt = ceil_div(p.Sq, BQ);
  int qt, hb;
  if (p.mask_mode == NB_MASK_NONE) {
    qt = blockIdx.x % nqt;
    hb = blockIdx.x / nqt;
  } else {
    const int nhb = p.Hq * p.B;
    qt = nqt - 1 - blockIdx.x / nhb;
    hb = blockIdx.x % nhb;
  }
  const int q0 = qt * BQ, h = hb % p.Hq, b = hb / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  const int klim = kv_limit(p, q0);
  const int nkb = klim < 0 ? 0 : klim / BKV + 1;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NBARS; ++i) {
      const bool eight = (i == SDP_EMPTY || i == DS_FULL);
      mbar_init(&bars[i], eight ? 8 : 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
    prefetch_tensormap(&tmdO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one() && nkb > 0) {
      mbar_expect_tx_a(bar(Q_FULL), 2 * T_BYTES);
#pragma unroll
      for (int s = 0; s < NSUB; ++s) {
        tma_load_4d_a(aQ + s * (BQ * 128), &tmQ, bar(Q_FULL), s * 64, h, q0, b);
        tma_load_4d_a(adO + s * (BQ * 128), &tmdO, bar(Q_FULL), s * 64, h, q0, b);
      }
      for (int j = 0; j < nkb; ++j) {
        const int st = j % ST;
        const uint32_t ph = (uint32_t)(j / ST) & 1u;
        if (*abort_flag || !mbar_wait_a(bar(KV_EMPTY + st), ph ^ 1u, p.status, 401)) { *abort_flag = 1; break; }
        mbar_expect_tx_a(bar(KV_FULL + st), 2 * T_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
          tma_load_4d_a(aK + st * T_BYTES + s * (BKV * 128), &tmK, bar(KV_FULL + st), s * 64, hkv, j * BKV, b);
          tma_load_4d_a(aV + st * T_BYTES + s * (BKV * 128), &tmV, bar(KV_FULL + st), s * 64, hkv, j * BKV, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nkb > 0) {
      const uint32_t idesc_s = make_idesc(1u, BQ, BKV, 0u, 0u);  // S, dP: K-major x K-major
      const uint32_t idesc_q = make_idesc(1u, BQ, HD, 0u, 1u);   // dQ = dS K: dS from tensor memory, K tile read MN-major
      bool ok = mbar_wait_a(bar(Q_FULL), 0u, p.status, 410);
      auto issue_sdp = [&](int j) -> bool {
        const int st = j % ST;
        if (*abort_flag || !mbar_wait_a(bar(KV_FULL + st), (uint32_t)(j / ST) & 1u, p.status, 411)) return false;
        if (j > 0 && !mbar_wait_a(bar(SDP_EMPTY), (uint32_t)(j - 1) & 1u, p.status, 412)) return false;
        tc_fence_after();
        const uint64_t qd = make_smem_desc(aQ, 16, 1024, 2), od = make_smem_desc(adO, 16, 1024, 2);
        const uint64_t kd = make_smem_desc(aK + st * T_BYTES, 16, 1024, 2), vd = make_smem_desc(aV + st * T_BYTES, 16, 1024, 2);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = ((k / 4) * (128 * 128) + (k % 4) * 32) >> 4;
          umma_f16(tmem_base + S_COL, qd + off, kd + off, idesc_s, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = ((k / 4) * (128 * 128) + (k % 4) * 32) >> 4;
          umma_f16(tmem_base + DP_COL, od + off, vd + off, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit_a(bar(SDP_FULL));
        return true;
      };
      if (ok) ok = issue_sdp(0);
      for (int j = 0; j < nkb && ok; ++j) {
        if (j + 1 < nkb && !issue_sdp(j + 1)) { ok = false; break; }
        const int st = j % ST;
        if (*abort_flag || !mbar_wait_a(bar(DS_FULL), (uint32_t)j & 1u, p.status, 413)) { ok = false; break; }
        tc_fence_after();
        const uint64_t kd = make_smem_desc(aK + st * T_BYTES, BKV * 128, 1024, 2);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k)   // dS: 16 keys = 8 packed columns per k-step; K: 16 key-rows of 128 B per k-step
          umma_f16_ts(tmem_base + DQ_COL, tmem_base + DS_COL + k * 8, kd + ((k * 16 * 128) >> 4), idesc_q, (j | k) != 0 ? 1u : 0u);
        umma_commit_a(bar(DS_EMPTY));
        umma_commit_a(bar(KV_EMPTY + st));
      }
      if (ok) umma_commit_a(bar(DQ_FULL));
      if (!ok) *abort_flag = 1;
    }
  } else {
    // two threads per query row: key columns [64·half, 64·half + 64) of every block
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t ridx = ((size_t)b * p.Hq + h) * p.Sq + min(q, p.Sq - 1);
    const float lse_row = p.lse[ridx], delta_row = p.delta[ridx];
    const bool dead = !(lse_row > -INFINITY) || q >= p.Sq;
    const unsigned char* kvalid = p.key_valid ? p.key_valid + (size_t)b * p.Sk : nullptr;
    const float* bias_row = (p.bias && q < p.Sq) ? p.bias + (size_t)q * p.Sk : nullptr;
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      const int k0 = j * BKV + half * 64;
      if (!__all_sync(0xffffffffu, !*abort_flag && mbar_wait_a(bar(SDP_FULL), (uint32_t)j & 1u, p.status, 420))) { ok = false; break; }
      tc_fence_after();
      float s[64], dp[64];
      ld64(lane_addr + S_COL + half * 64, s);
      ld64(lane_addr + DP_COL + half * 64, dp);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_a(bar(SDP_EMPTY));   // both accumulators are in registers: the next S / dP may start
      const int lim = dead ? 0 : row_limit(p, q, j * BKV) - half * 64;   // allowed leading columns of my half
      uint32_t w[32];
      if (lim >= 64 && !kvalid && !bias_row) {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          const float p0 = exp2_fast(fmaf(s[i], p.scale_log2, -lse_row)), p1 = exp2_fast(fmaf(s[i + 1], p.scale_log2, -lse_row));
          w[i >> 1] = pack_bf16(p0 * (dp[i] - delta_row) * p.scale, p1 * (dp[i + 1] - delta_row) * p.scale);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 64; i += 2) {
          float pv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            float sc = s[i + u] * p.scale_log2;
            bool a = (i + u) < lim;
            if (kvalid || bias_row) {
              const int k = min(k0 + i + u, p.Sk - 1);
              if (kvalid) a = a && (kvalid[k] != 0);
              if (bias_row) sc += bias_row[k] * 1.4426950408889634f;
            }
            pv[u] = a ? exp2_fast(sc - lse_row) : 0.f;
          }
          w[i >> 1] = pack_bf16(pv[0] * (dp[i] - delta_row) * p.scale, pv[1] * (dp[i + 1] - delta_row) * p.scale);
        }
      }
      // dS_{j-1} must have been consumed by dQ += dS_{j-1} K_{j-1}
      if (j > 0 && !__all_sync(0xffffffffu, mbar_wait_a(bar(DS_EMPTY), (uint32_t)(j - 1) & 1u, p.status, 421))) { ok = false; break; }
      tc_fence_after();
      st32(lane_addr + DS_COL + half * 32, w);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_a(bar(DS_FULL));
    }
    if (ok && nkb > 0) ok = __all_sync(0xffffffffu, mbar_wait_a(bar(DQ_FULL), 0u, p.status, 422));
    if (!ok) *abort_flag = 1;
    if (ok) {
      tc_fence_after();
      constexpr int HC = HD / 2;
      __nv_bfloat16* dst = (q < p.Sq) ? p.dQ + ((size_t)b * p.Sq + q) * p.ld_dq + (size_t)h * HD + half * HC : nullptr;
      if (nkb > 0) {
        store_row<HC>(lane_addr + DQ_COL + half * HC, dst);
      } else if (dst) {
        for (int c = 0; c < HC; c += 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0, 0, 0, 0);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------ dK, dV (transposed tiles)
// first query index that may attend key k
__device__ __forceinline__ int q_first_of_key(const FaParams& p, int k) {
  if (p.mask_mode == NB_MASK_CAUSAL) return max(0, k - p.causal_off);
  if (p.mask_mode == NB_MASK_BLOCK_CAUSAL) return (k / p.frame) * p.frame;
  return 0;
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_bwd2_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const FaParams p) {
  constexpr int NSUB = HD / 64;
  constexpr int ST = (HD == 64) ? 4 : 2;      // Q / dO ring depth
  constexpr uint32_t T_BYTES = 128 * HD * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 384;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t aK = smem_u32(smem), aV = aK + T_BYTES, aQ = aV + T_BYTES, adO = aQ + ST * T_BYTES, aB = adO + ST * T_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 2 * T_BYTES + 2 * ST * T_BYTES);
  constexpr int KV_FULL = 0, Q_FULL = 1, Q_EMPTY = 1 + ST, S_FULL = 1 + 2 * ST, DP_FULL = 2 + 2 * ST, P_FULL = 3 + 2 * ST,
                DS_FULL = 4 + 2 * ST, ACC_FULL = 5 + 2 * ST, NBARS = 6 + 2 * ST;
  auto bar = [&](int i) { return aB + 8u * (uint32_t)i; };
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NBARS);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* stat = reinterpret_cast<float*>(tmem_slot + 4);   // [2 buffers][lse 128 | delta 128]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * BKV, hkv = blockIdx.y, b = blockIdx.z;
  const int rep = p.Hq / p.Hkv;
  const int qb0 = q_first_of_key(p, k0) / BQ;       // first query tile any key of this tile can be seen from
  const int nqb = ceil_div(p.Sq, BQ);
  const int per_head = max(nqb - qb0, 0);
  const int total = per_head * rep;  // iterations: (g, i) with i = qb0 + it % per_head, g = it / per_head

  if (threadIdx.x == 0) {
    for (int i = 0; i < NBARS; ++i) mbar_init(&bars[i], (i == P_FULL || i == DS_FULL) ? 8 : 1);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
    prefetch_tensormap(&tmdO);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one() && total > 0) {
      mbar_expect_tx_a(bar(KV_FULL), 2 * T_BYTES);
#pragma unroll
      for (int s = 0; s < NSUB; ++s) {
        tma_load_4d_a(aK + s * (BKV * 128), &tmK, bar(KV_FULL), s * 64, hkv, k0, b);
        tma_load_4d_a(aV + s * (BKV * 128), &tmV, bar(KV_FULL), s * 64, hkv, k0, b);
      }
      for (int it = 0; it < total; ++it) {
        const int st = it % ST;
        const uint32_t ph = (uint32_t)(it / ST) & 1u;
        const int hq = hkv * rep + it / per_head, qi = (qb0 + it % per_head) * BQ;
        if (*abort_flag || !mbar_wait_a(bar(Q_EMPTY + st), ph ^ 1u, p.status, 501)) { *abort_flag = 1; break; }
        mbar_expect_tx_a(bar(Q_FULL + st), 2 * T_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
          tma_load_4d_a(aQ + st * T_BYTES + s * (BQ * 128), &tmQ, bar(Q_FULL + st), s * 64, hq, qi, b);
          tma_load_4d_a(adO + st * T_BYTES + s * (BQ * 128), &tmdO, bar(Q_FULL + st), s * 64, hq, qi, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one() && total > 0) {
      const uint32_t idesc_s = make_idesc(1u, BKV, BQ, 0u, 0u);  // Sᵀ = K Qᵀ, dPᵀ = V dOᵀ: K-major x K-major
      const uint32_t idesc_t = make_idesc(1u, BKV, HD, 0u, 1u);  // dV = Pᵀ dO, dK = dSᵀ Q: A from tensor memory, B MN-major
      bool ok = mbar_wait_a(bar(KV_FULL), 0u, p.status, 510);
      const uint64_t kd = make_smem_desc(aK, 16, 1024, 2), vd = make_smem_desc(aV, 16, 1024, 2);
      auto issue_st = [&](int it) -> bool {     // Sᵀ(it)
        const int st = it % ST;
        if (*abort_flag || !mbar_wait_a(bar(Q_FULL + st), (uint32_t)(it / ST) & 1u, p.status, 511)) return false;
        tc_fence_after();
        const uint64_t qd = make_smem_desc(aQ + st * T_BYTES, 16, 1024, 2);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = ((k / 4) * (128 * 128) + (k % 4) * 32) >> 4;
          umma_f16(tmem_base + S_COL, kd + off, qd + off, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit_a(bar(S_FULL));
        return true;
      };
      auto issue_dpt = [&](int it) {            // dPᵀ(it); Q_FULL of this stage was already waited for by Sᵀ(it)
        const int st = it % ST;
        const uint64_t od = make_smem_desc(adO + st * T_BYTES, 16, 1024, 2);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = ((k / 4) * (128 * 128) + (k % 4) * 32) >> 4;
          umma_f16(tmem_base + DP_COL, vd + off, od + off, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit_a(bar(DP_FULL));
      };
      // A operand in tensor memory: queries [0,64) of the block at columns [0,32), queries [64,128) at [64,96)
      auto a_col = [](int k) { return (uint32_t)((k >> 2) * 64 + (k & 3) * 8); };
      if (ok) ok = issue_st(0);
      if (ok) issue_dpt(0);
      for (int it = 0; it < total && ok; ++it) {
        const int st = it % ST;
        if (*abort_flag || !mbar_wait_a(bar(P_FULL), (uint32_t)it & 1u, p.status, 512)) { ok = false; break; }
        tc_fence_after();
        {
          const uint64_t od = make_smem_desc(adO + st * T_BYTES, BQ * 128, 1024, 2);   // dO read MN-major: 16 query rows per k-step
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k)
            umma_f16_ts(tmem_base + DV_COL, tmem_base + S_COL + a_col(k), od + ((k * 16 * 128) >> 4), idesc_t, (it | k) != 0 ? 1u : 0u);
        }
        if (it + 1 < total && !issue_st(it + 1)) { ok = false; break; }    // the Sᵀ columns are free once dV has read Pᵀ
        if (!mbar_wait_a(bar(DS_FULL), (uint32_t)it & 1u, p.status, 513)) { ok = false; break; }
        tc_fence_after();
        {
          const uint64_t qd = make_smem_desc(aQ + st * T_BYTES, BQ * 128, 1024, 2);
#pragma unroll
          for (int k = 0; k < BQ / 16; ++k)
            umma_f16_ts(tmem_base + DK_COL, tmem_base + DP_COL + a_col(k), qd + ((k * 16 * 128) >> 4), idesc_t, (it | k) != 0 ? 1u : 0u);
        }
        umma_commit_a(bar(Q_EMPTY + st));
        if (it + 1 < total) issue_dpt(it + 1);                                // the dPᵀ columns are free once dK has read dSᵀ
      }
      if (ok) umma_commit_a(bar(ACC_FULL));
      if (!ok) *abort_flag = 1;
    }
  } else {
    // two threads per KEY row: query columns [64·half, 64·half + 64) of every block
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int tid = (warp - 2) * 32 + lane;          // 0..255 among the softmax threads
    const int k = k0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool row_ok = k < p.Sk && (!p.key_valid || p.key_valid[(size_t)b * p.Sk + k] != 0);
    const int qf = q_first_of_key(p, min(k, p.Sk - 1));   // queries before qf do not see this key
    bool ok = true;
    // Every softmax thread executes the named barrier of EVERY iteration, whatever happened before (a warp that left
    // early would strand the others at it); a failed wait only switches the remaining work off.
    for (int it = 0; it < total; ++it) {
      const int hq = hkv * rep + it / per_head, qi = (qb0 + it % per_head) * BQ;
      // per-query statistics of this tile → shared memory (lse: threads 0..127, Δ: threads 128..255)
      float* sb = stat + (it & 1) * 256;
      {
        const int qq = qi + (tid & 127);
        const size_t ridx = ((size_t)b * p.Hq + hq) * p.Sq + min(qq, p.Sq - 1);
        float v;
        if (tid < 128) {
          v = p.lse[ridx];
          if (!(v > -INFINITY) || qq >= p.Sq) v = INFINITY;   // dead query row or past the end: P = 2^(-inf) = 0
        } else {
          v = p.delta[ridx];
        }
        sb[tid] = v;
      }
      asm volatile("bar.sync 1, 256;" ::: "memory");
      if (!ok) continue;
      const float* lse_s = sb + half * 64;
      const float* del_s = sb + 128 + half * 64;
      const int c0 = qi + half * 64;                     // query index of my column 0
      const int cfirst = max(qf - c0, 0);                // my columns below cfirst are masked
      const float* bias_col = p.bias ? p.bias + (size_t)c0 * p.Sk + min(k, p.Sk - 1) : nullptr;   // + c · Sk per column
      // ---- phase A: Pᵀ from Sᵀ
      if (!__all_sync(0xffffffffu, !*abort_flag && mbar_wait_a(bar(S_FULL), (uint32_t)it & 1u, p.status, 520))) { ok = false; *abort_flag = 1; continue; }
      tc_fence_after();
      uint32_t pw[32];
      {
        float s[64];
        ld64(lane_addr + S_COL + half * 64, s);
        tmem_ld_wait();
        if (row_ok && cfirst == 0 && !bias_col) {
#pragma unroll
          for (int c = 0; c < 64; c += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(lse_s + c);
            pw[c >> 1] = pack_bf16(exp2_fast(fmaf(s[c], p.scale_log2, -l4.x)), exp2_fast(fmaf(s[c + 1], p.scale_log2, -l4.y)));
            pw[(c >> 1) + 1] = pack_bf16(exp2_fast(fmaf(s[c + 2], p.scale_log2, -l4.z)), exp2_fast(fmaf(s[c + 3], p.scale_log2, -l4.w)));
          }
        } else {
#pragma unroll
          for (int c = 0; c < 64; c += 2) {
            float pv[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              float sc = s[c + u] * p.scale_log2;
              const bool a = row_ok && (c + u) >= cfirst;
              if (bias_col && c0 + c + u < p.Sq) sc += bias_col[(size_t)(c + u) * p.Sk] * 1.4426950408889634f;
              pv[u] = a ? exp2_fast(sc - lse_s[c + u]) : 0.f;
            }
            pw[c >> 1] = pack_bf16(pv[0], pv[1]);
          }
        }
      }
      st32(lane_addr + S_COL + half * 64, pw);   // Pᵀ over the first half of my own Sᵀ columns
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_a(bar(P_FULL));
      // ---- phase B: dSᵀ = Pᵀ ⊙ (dPᵀ − Δ) · scale
      if (!__all_sync(0xffffffffu, mbar_wait_a(bar(DP_FULL), (uint32_t)it & 1u, p.status, 521))) { ok = false; *abort_flag = 1; continue; }
      tc_fence_after();
      {
        float dp[64];
        ld64(lane_addr + DP_COL + half * 64, dp);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 64; c += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(del_s + c);
          const __nv_bfloat162 h0 = *reinterpret_cast<const __nv_bfloat162*>(&pw[c >> 1]);
          const __nv_bfloat162 h1 = *reinterpret_cast<const __nv_bfloat162*>(&pw[(c >> 1) + 1]);
          pw[c >> 1] = pack_bf16(__low2float(h0) * (dp[c] - d4.x) * p.scale, __high2float(h0) * (dp[c + 1] - d4.y) * p.scale);
          pw[(c >> 1) + 1] = pack_bf16(__low2float(h1) * (dp[c + 2] - d4.z) * p.scale, __high2float(h1) * (dp[c + 3] - d4.w) * p.scale);
        }
      }
      st32(lane_addr + DP_COL + half * 64, pw);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_a(bar(DS_FULL));
    }
    if (ok && total > 0) ok = __all_sync(0xffffffffu, mbar_wait_a(bar(ACC_FULL), 0u, p.status, 522));
    if (!ok) *abort_flag = 1;
    if (ok) {
      tc_fence_after();
      constexpr int HC = HD / 2;
      __nv_bfloat16* dv = (k < p.Sk) ? p.dV + ((size_t)b * p.Sk + k) * p.ld_dv + (size_t)hkv * HD + half * HC : nullptr;
      __nv_bfloat16* dk = (k < p.Sk) ? p.dK + ((size_t)b * p.Sk + k) * p.ld_dk + (size_t)hkv * HD + half * HC : nullptr;
      if (total > 0) {
        store_row<HC>(lane_addr + DV_COL + half * HC, dv);
        store_row<HC>(lane_addr + DK_COL + half * HC, dk);
      } else if (dv) {
        for (int c = 0; c < HC; c += 8) {
          *reinterpret_cast<uint4*>(dv + c) = make_uint4(0, 0, 0, 0);
          *reinterpret_cast<uint4*>(dk + c) = make_uint4(0, 0, 0, 0);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int HD>
int launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo, const FaParams& p,
           cudaStream_t s) {
  constexpr int ST = (HD == 64) ? 4 : 2;
  constexpr size_t T = 128 * HD * 2;
  constexpr size_t smem = 2 * T + 2 * ST * T + 1024 /*align*/ + 256 /*barriers*/ + 2048 /*statistics*/;
  static_assert(smem <= 232448, "shared memory budget of one CTA");
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(fa_bwd2_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    NB_CUDA(cudaFuncSetAttribute(fa_bwd2_dkdv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  fa_bwd2_dq_kernel<HD><<<dim3(ceil_div(p.Sq, BQ) * p.Hq * p.B), FA_THREADS, smem, s>>>(tq, tk, tv, tdo, p);
  NB_LAUNCH_CHECK();
  fa_bwd2_dkdv_kernel<HD><<<dim3(ceil_div(p.Sk, BKV), p.Hkv, p.B), FA_THREADS, smem, s>>>(tq, tk, tv, tdo, p);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // namespace

namespace nbattn {
int launch_bwd_gen2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                    const FaParams& p, int HD, cudaStream_t s) {
  if (HD == 64) return launch<64>(tq, tk, tv, tdo, p, s);
  return launch<128>(tq, tk, tv, tdo, p, s);
}
}  // namespace nbattn
