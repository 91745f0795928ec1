// Flash attention backward on tcgen05 — deterministic, two kernels (no atomics), like the reference's
// dq / dkdv split (noeira/nn/primitives/flash_attention_mma.mojo:375,521; "deterministic (no atomics)"
// flash_attention.mojo:12-15), re-derived for TMEM accumulators:
//
//   delta      Δ[b,h,q] = Σ_d dO·O                                     (SIMT, one warp per row)
//   dq kernel  CTA = 128-query tile of one (b,h); loops over key tiles:
//                S = Q Kᵀ, dP = dO Vᵀ (TMEM) → threads (row = query): P = 2^(S·c − LSE), dS = P⊙(dP − Δ)·scale
//                → bf16 dS tile in swizzled smem → dQ += dS K   (accumulates in TMEM over all key tiles)
//   dkdv       CTA = 128-key tile of one (b, kv-head); loops over the q-heads of the group and query tiles:
//                same S, dP, P, dS; P and dS tiles go to smem and are consumed TRANSPOSED through MN-major
//                operand descriptors:  dV += Pᵀ dO,  dK += dSᵀ Q   (both accumulate in TMEM)
// The K tile serves as K-major B operand of S = Q Kᵀ and, unchanged in shared memory, as MN-major B operand
// of dQ += dS K; likewise Q / dO in the dkdv kernel.  Masks, GQA and bounded waits as in the forward.
#include "attention_common.cuh"

namespace {
using namespace nb;
using namespace nbattn;

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// one warp per (b, q, h) row: Δ = Σ_d dO·O
__global__ void __launch_bounds__(256)
fa_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO, float* __restrict__ delta,
                int B, int Sq, int Hq, int HD, long long o_ss, long long do_ss) {
  const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= (long long)B * Sq * Hq) return;
  const int h = (int)(row % Hq);
  const long long bq = row / Hq;
  const int q = (int)(bq % Sq);
  const int b = (int)(bq / Sq);
  const __nv_bfloat16* o = O + ((long long)b * Sq + q) * o_ss + (long long)h * HD;
  const __nv_bfloat16* d = dO + ((long long)b * Sq + q) * do_ss + (long long)h * HD;
  float acc = 0.f;
  for (int i = lane * 2; i < HD; i += 64) {
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(o + i);
    const __nv_bfloat162 c = *reinterpret_cast<const __nv_bfloat162*>(d + i);
    acc += __low2float(a) * __low2float(c) + __high2float(a) * __high2float(c);
  }
  acc = warp_sum(acc);
  if (lane == 0) delta[((long long)b * Hq + h) * Sq + q] = acc;
}

// Two threads per query row (column halves) turn one S / dP tile pair into bf16 P and dS tiles in swizzled
// shared memory.  sP may be null (dq kernel needs dS only).
__device__ __forceinline__ void softmax_bwd_tile(const FaParams& p, uint32_t s_addr, uint32_t dp_addr, int q, int k0,
                                                 int row, int half, float lse_row, float delta_row,
                                                 const unsigned char* kvalid, const float* bias_row, uint8_t* sP,
                                                 uint8_t* sdS) {
  const bool dead = !(lse_row > -INFINITY) || q >= p.Sq;
  const int lim = dead ? 0 : row_limit(p, q, k0) - half * 64;
  const bool fast = (lim >= 64) && !kvalid && !bias_row;
  const int roff = half * (BQ * 128) + (row >> 3) * 1024 + (row & 7) * 128;
#pragma unroll 1
  for (int c = 0; c < 64; c += 32) {
    uint32_t rs[32], rd[32];
    tmem_ld_32x32b_x32_nowait(s_addr + half * 64 + c, rs);
    tmem_ld_32x32b_x32_nowait(dp_addr + half * 64 + c, rd);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; i += 8) {
      uint32_t pp[4], pd[4];
#pragma unroll
      for (int w2 = 0; w2 < 4; ++w2) {
        float pv[2], dv[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int e = i + 2 * w2 + u;
          float pr;
          if (fast) {
            pr = exp2_fast(fmaf(__uint_as_float(rs[e]), p.scale_log2, -lse_row));
          } else {
            float sc = __uint_as_float(rs[e]) * p.scale_log2;
            bool a = (c + e) < lim;
            if (kvalid || bias_row) {
              const int k = min(k0 + half * 64 + c + e, p.Sk - 1);
              if (kvalid) a = a && (kvalid[k] != 0);
              if (bias_row) sc += bias_row[k] * 1.4426950408889634f;
            }
            pr = a ? exp2_fast(sc - lse_row) : 0.f;
          }
          pv[u] = pr;
          dv[u] = pr * (__uint_as_float(rd[e]) - delta_row) * p.scale;
        }
        __nv_bfloat162 hp = __floats2bfloat162_rn(pv[0], pv[1]), hd = __floats2bfloat162_rn(dv[0], dv[1]);
        pp[w2] = *reinterpret_cast<uint32_t*>(&hp);
        pd[w2] = *reinterpret_cast<uint32_t*>(&hd);
      }
      const int off = roff + ((((c + i) >> 3) ^ (row & 7)) << 4);
      if (sP) *reinterpret_cast<uint4*>(sP + off) = make_uint4(pp[0], pp[1], pp[2], pp[3]);
      *reinterpret_cast<uint4*>(sdS + off) = make_uint4(pd[0], pd[1], pd[2], pd[3]);
    }
  }
}

// TMEM accumulator row (HD fp32) → bf16 → global
template <int NC>
__device__ __forceinline__ void store_row_bf16(uint32_t taddr, __nv_bfloat16* dst) {
#pragma unroll
  for (int c = 0; c < NC; c += 32) {
    uint32_t r[32];
    tmem_ld_32x32b_x32(taddr + c, r);
    tmem_ld_wait();
    if (dst) {
#pragma unroll
      for (int i = 0; i < 32; i += 8) {
        uint4 pk;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                       h1 = __floats2bfloat162_rn(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                       h2 = __floats2bfloat162_rn(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                       h3 = __floats2bfloat162_rn(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
        pk.x = *reinterpret_cast<uint32_t*>(&h0);
        pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2);
        pk.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(dst + c + i) = pk;
      }
    }
  }
}

// ------------------------------------------------------------------------------------------ dQ
template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, const FaParams p) {
  constexpr int NSUB = HD / 64;
  constexpr int STAGES = (HD == 64) ? 2 : 1;
  constexpr uint32_t T_BYTES = 128 * HD * 2;  // one [128 x HD] bf16 tile
  constexpr uint32_t DS_BYTES = BQ * BKV * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DQ_COL = 256;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + T_BYTES;
  uint8_t* sK = sdO + T_BYTES;             // STAGES
  uint8_t* sV = sK + STAGES * T_BYTES;     // STAGES
  uint8_t* sdS = sV + STAGES * T_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + DS_BYTES);
  uint64_t* q_full = bars;          // Q and dO
  uint64_t* kv_full = bars + 1;     // [2]
  uint64_t* kv_empty = bars + 3;    // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* sdp_empty = bars + 6;
  uint64_t* ds_full = bars + 7;
  uint64_t* ds_empty = bars + 8;
  uint64_t* dq_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (p.Hq / p.Hkv);
  const int klim = kv_limit(p, q0);
  const int nkb = klim < 0 ? 0 : klim / BKV + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_empty, 8);
    mbar_init(ds_full, 8);
    mbar_init(ds_empty, 1);
    mbar_init(dq_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
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
    if (elect_one()) {
      mbar_expect_tx(q_full, 2 * T_BYTES);
#pragma unroll
      for (int s = 0; s < NSUB; ++s) {
        tma_load_4d(sQ + s * (BQ * 128), &tmQ, q_full, s * 64, h, q0, b);
        tma_load_4d(sdO + s * (BQ * 128), &tmdO, q_full, s * 64, h, q0, b);
      }
      for (int j = 0; j < nkb; ++j) {
        const int st = j % STAGES;
        const uint32_t ph = (uint32_t)(j / STAGES) & 1u;
        if (*abort_flag || !mbar_wait(&kv_empty[st], ph ^ 1u, p.status, 201)) { *abort_flag = 1; break; }
        mbar_expect_tx(&kv_full[st], 2 * T_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
          tma_load_4d(sK + st * T_BYTES + s * (BKV * 128), &tmK, &kv_full[st], s * 64, hkv, j * BKV, b);
          tma_load_4d(sV + st * T_BYTES + s * (BKV * 128), &tmV, &kv_full[st], s * 64, hkv, j * BKV, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(1u, BQ, BKV, 0u, 0u);  // S, dP: K-major x K-major
      const uint32_t idesc_q = make_idesc(1u, BQ, HD, 0u, 1u);   // dQ = dS K: K tile read MN-major
      bool ok = mbar_wait(q_full, 0u, p.status, 210);
      auto issue_dq = [&](int j) -> bool {
        const int st = j % STAGES;
        if (*abort_flag || !mbar_wait(ds_full, (uint32_t)j & 1u, p.status, 211)) return false;
        tc_fence_after();
        const uint32_t da = smem_u32(sdS), kb = smem_u32(sK + st * T_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          const uint64_t adesc = make_smem_desc(da + (k / 4) * (BQ * 128) + (k % 4) * 32, 16, 1024, 2);
          const uint64_t bdesc = make_smem_desc(kb + k * (16 * 128), BKV * 128, 1024, 2);
          umma_f16(tmem_base + DQ_COL, adesc, bdesc, idesc_q, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(ds_empty);
        umma_commit(&kv_empty[st]);
        return true;
      };
      for (int j = 0; j < nkb && ok; ++j) {
        if (j > 0 && !issue_dq(j - 1)) { ok = false; break; }
        const int st = j % STAGES;
        const uint32_t ph = (uint32_t)(j / STAGES) & 1u;
        if (*abort_flag || !mbar_wait(&kv_full[st], ph, p.status, 212)) { ok = false; break; }
        if (!mbar_wait(sdp_empty, ((uint32_t)j & 1u) ^ 1u, p.status, 213)) { ok = false; break; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), oa = smem_u32(sdO), kb = smem_u32(sK + st * T_BYTES),
                       vb = smem_u32(sV + st * T_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k / 4) * (128 * 128) + (k % 4) * 32;
          umma_f16(tmem_base + S_COL, make_smem_desc(qa + off, 16, 1024, 2), make_smem_desc(kb + off, 16, 1024, 2),
                   idesc_s, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k / 4) * (128 * 128) + (k % 4) * 32;
          umma_f16(tmem_base + DP_COL, make_smem_desc(oa + off, 16, 1024, 2), make_smem_desc(vb + off, 16, 1024, 2),
                   idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
      }
      if (ok && nkb > 0 && !issue_dq(nkb - 1)) ok = false;
      if (ok) umma_commit(dq_full);
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t ridx = ((size_t)b * p.Hq + h) * p.Sq + min(q, p.Sq - 1);
    const float lse_row = p.lse[ridx], delta_row = p.delta[ridx];
    const unsigned char* kvalid = p.key_valid ? p.key_valid + (size_t)b * p.Sk : nullptr;
    const float* bias_row = (p.bias && q < p.Sq) ? p.bias + (size_t)q * p.Sk : nullptr;
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      if (*abort_flag || !mbar_wait(sdp_full, (uint32_t)j & 1u, p.status, 220)) { ok = false; break; }
      if (!mbar_wait(ds_empty, ((uint32_t)j & 1u) ^ 1u, p.status, 221)) { ok = false; break; }
      tc_fence_after();
      softmax_bwd_tile(p, lane_addr + S_COL, lane_addr + DP_COL, q, j * BKV, row, half, lse_row, delta_row, kvalid,
                       bias_row, nullptr, sdS);
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(sdp_empty);
        mbar_arrive(ds_full);
      }
    }
    if (ok && nkb > 0) ok = mbar_wait(dq_full, 0u, p.status, 222);
    if (!ok) *abort_flag = 1;
    if (ok) {
      tc_fence_after();
      constexpr int HC = HD / 2;
      __nv_bfloat16* dst = (q < p.Sq) ? p.dQ + ((size_t)b * p.Sq + q) * p.ld_dq + (size_t)h * HD + half * HC : nullptr;
      if (nkb > 0) {
        store_row_bf16<HC>(lane_addr + DQ_COL + half * HC, dst);
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

// ------------------------------------------------------------------------------------------ dK, dV
// first query index that may attend key tile [k0, k0+BKV)
__device__ __forceinline__ int q_first(const FaParams& p, int k0) {
  if (p.mask_mode == NB_MASK_CAUSAL) return max(0, k0 - p.causal_off);
  if (p.mask_mode == NB_MASK_BLOCK_CAUSAL) return (k0 / p.frame) * p.frame;
  return 0;
}

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                   const FaParams p) {
  constexpr int NSUB = HD / 64;
  constexpr int STAGES = (HD == 64) ? 2 : 1;
  constexpr uint32_t T_BYTES = 128 * HD * 2;
  constexpr uint32_t PS_BYTES = BQ * BKV * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + HD;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + T_BYTES;
  uint8_t* sQ = sV + T_BYTES;               // STAGES
  uint8_t* sdO = sQ + STAGES * T_BYTES;     // STAGES
  uint8_t* sP = sdO + STAGES * T_BYTES;
  uint8_t* sdS = sP + PS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + PS_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;     // [2]  Q_i and dO_i
  uint64_t* q_empty = bars + 3;    // [2]
  uint64_t* sdp_full = bars + 5;
  uint64_t* sdp_empty = bars + 6;
  uint64_t* pds_full = bars + 7;
  uint64_t* pds_empty = bars + 8;
  uint64_t* acc_full = bars + 9;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k0 = blockIdx.x * BKV, hkv = blockIdx.y, b = blockIdx.z;
  const int rep = p.Hq / p.Hkv;
  const int qb0 = q_first(p, k0) / BQ;
  const int nqb = ceil_div(p.Sq, BQ);
  const int per_head = max(nqb - qb0, 0);
  const int total = per_head * rep;  // iterations: (g, i) with i = qb0 + it % per_head, g = it / per_head

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(sdp_empty, 8);
    mbar_init(pds_full, 8);
    mbar_init(pds_empty, 1);
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
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
    if (elect_one()) {
      mbar_expect_tx(kv_full, 2 * T_BYTES);
#pragma unroll
      for (int s = 0; s < NSUB; ++s) {
        tma_load_4d(sK + s * (BKV * 128), &tmK, kv_full, s * 64, hkv, k0, b);
        tma_load_4d(sV + s * (BKV * 128), &tmV, kv_full, s * 64, hkv, k0, b);
      }
      for (int it = 0; it < total; ++it) {
        const int st = it % STAGES;
        const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
        const int hq = hkv * rep + it / per_head, qi = (qb0 + it % per_head) * BQ;
        if (*abort_flag || !mbar_wait(&q_empty[st], ph ^ 1u, p.status, 301)) { *abort_flag = 1; break; }
        mbar_expect_tx(&q_full[st], 2 * T_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
          tma_load_4d(sQ + st * T_BYTES + s * (BQ * 128), &tmQ, &q_full[st], s * 64, hq, qi, b);
          tma_load_4d(sdO + st * T_BYTES + s * (BQ * 128), &tmdO, &q_full[st], s * 64, hq, qi, b);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(1u, BQ, BKV, 0u, 0u);
      const uint32_t idesc_t = make_idesc(1u, BKV, HD, 1u, 1u);  // dV = Pᵀ dO, dK = dSᵀ Q: both MN-major
      bool ok = mbar_wait(kv_full, 0u, p.status, 310);
      auto issue_acc = [&](int it) -> bool {
        const int st = it % STAGES;
        if (*abort_flag || !mbar_wait(pds_full, (uint32_t)it & 1u, p.status, 311)) return false;
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), da = smem_u32(sdS), qa = smem_u32(sQ + st * T_BYTES),
                       oa = smem_u32(sdO + st * T_BYTES);
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {
          // contraction over queries: 16 query-rows of 128 B per step; 64-wide MN chunks are 16 KB apart
          const uint32_t off = k * (16 * 128);
          umma_f16(tmem_base + DV_COL, make_smem_desc(pa + off, BQ * 128, 1024, 2),
                   make_smem_desc(oa + off, BQ * 128, 1024, 2), idesc_t, (it | k) != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < BQ / 16; ++k) {
          const uint32_t off = k * (16 * 128);
          umma_f16(tmem_base + DK_COL, make_smem_desc(da + off, BQ * 128, 1024, 2),
                   make_smem_desc(qa + off, BQ * 128, 1024, 2), idesc_t, (it | k) != 0 ? 1u : 0u);
        }
        umma_commit(pds_empty);
        umma_commit(&q_empty[st]);
        return true;
      };
      for (int it = 0; it < total && ok; ++it) {
        if (it > 0 && !issue_acc(it - 1)) { ok = false; break; }
        const int st = it % STAGES;
        const uint32_t ph = (uint32_t)(it / STAGES) & 1u;
        if (*abort_flag || !mbar_wait(&q_full[st], ph, p.status, 312)) { ok = false; break; }
        if (!mbar_wait(sdp_empty, ((uint32_t)it & 1u) ^ 1u, p.status, 313)) { ok = false; break; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * T_BYTES), oa = smem_u32(sdO + st * T_BYTES), kb = smem_u32(sK),
                       vb = smem_u32(sV);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k / 4) * (128 * 128) + (k % 4) * 32;
          umma_f16(tmem_base + S_COL, make_smem_desc(qa + off, 16, 1024, 2), make_smem_desc(kb + off, 16, 1024, 2),
                   idesc_s, k != 0 ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = (k / 4) * (128 * 128) + (k % 4) * 32;
          umma_f16(tmem_base + DP_COL, make_smem_desc(oa + off, 16, 1024, 2), make_smem_desc(vb + off, 16, 1024, 2),
                   idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(sdp_full);
      }
      if (ok && total > 0 && !issue_acc(total - 1)) ok = false;
      if (ok) umma_commit(acc_full);
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const unsigned char* kvalid = p.key_valid ? p.key_valid + (size_t)b * p.Sk : nullptr;
    bool ok = true;
    for (int it = 0; it < total && ok; ++it) {
      const int hq = hkv * rep + it / per_head, qi = (qb0 + it % per_head) * BQ;
      const int q = qi + row;
      const size_t ridx = ((size_t)b * p.Hq + hq) * p.Sq + min(q, p.Sq - 1);
      const float lse_row = p.lse[ridx], delta_row = p.delta[ridx];
      const float* bias_row = (p.bias && q < p.Sq) ? p.bias + (size_t)q * p.Sk : nullptr;
      if (*abort_flag || !mbar_wait(sdp_full, (uint32_t)it & 1u, p.status, 320)) { ok = false; break; }
      if (!mbar_wait(pds_empty, ((uint32_t)it & 1u) ^ 1u, p.status, 321)) { ok = false; break; }
      tc_fence_after();
      softmax_bwd_tile(p, lane_addr + S_COL, lane_addr + DP_COL, q, k0, row, half, lse_row, delta_row, kvalid, bias_row,
                       sP, sdS);
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(sdp_empty);
        mbar_arrive(pds_full);
      }
    }
    if (ok && total > 0) ok = mbar_wait(acc_full, 0u, p.status, 322);
    if (!ok) *abort_flag = 1;
    if (ok) {
      tc_fence_after();
      // accumulator rows are KEYS here (M = BKV)
      constexpr int HC = HD / 2;
      const int k = k0 + row;
      __nv_bfloat16* dv = (k < p.Sk) ? p.dV + ((size_t)b * p.Sk + k) * p.ld_dv + (size_t)hkv * HD + half * HC : nullptr;
      __nv_bfloat16* dk = (k < p.Sk) ? p.dK + ((size_t)b * p.Sk + k) * p.ld_dk + (size_t)hkv * HD + half * HC : nullptr;
      if (total > 0) {
        store_row_bf16<HC>(lane_addr + DV_COL + half * HC, dv);
        store_row_bf16<HC>(lane_addr + DK_COL + half * HC, dk);
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
int launch_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
               const FaParams& p, cudaStream_t s) {
  constexpr int STAGES = (HD == 64) ? 2 : 1;
  constexpr size_t T = 128 * HD * 2;
  constexpr size_t smem_dq = 2 * T + 2 * STAGES * T + (size_t)BQ * BKV * 2 + 1024 + 256;
  constexpr size_t smem_kv = 2 * T + 2 * STAGES * T + 2 * (size_t)BQ * BKV * 2 + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(fa_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_dq));
    NB_CUDA(cudaFuncSetAttribute(fa_bwd_dkdv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
    configured = true;
  }
  fa_bwd_dq_kernel<HD><<<dim3(ceil_div(p.Sq, BQ), p.Hq, p.B), FA_THREADS, smem_dq, s>>>(tq, tk, tv, tdo, p);
  NB_LAUNCH_CHECK();
  fa_bwd_dkdv_kernel<HD><<<dim3(ceil_div(p.Sk, BKV), p.Hkv, p.B), FA_THREADS, smem_kv, s>>>(tq, tk, tv, tdo, p);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int g_bwd_mode = 0;  // 0 = second-generation kernels, 1 = first generation (kept for comparison)

}  // namespace

extern "C" {

// Selects the backward kernels; returns the previous setting.
int nb_flash_attn_bwd_mode(int mode) {
  const int old = g_bwd_mode;
  if (mode >= 0 && mode <= 1) g_bwd_mode = mode;
  return old;
}

// Strides in elements (batch, token, head); HD stride 1 everywhere.  delta: scratch [B,Hq,Sq] fp32 supplied by the
// caller.  dQ/dK/dV are written (not accumulated) as [B,S,H,HD] with token pitches dq_ss / dk_ss / dv_ss.
int nb_flash_attn_bwd(const void* Q, const void* K, const void* V, const void* O, const void* dO, const float* lse,
                      float* delta, void* dQ, void* dK, void* dV, int B, int Hq, int Hkv, int Sq, int Sk, int HD,
                      long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss, long long k_sh,
                      long long v_sb, long long v_ss, long long v_sh, long long o_ss, long long do_sb, long long do_ss,
                      long long do_sh, long long dq_ss, long long dk_ss, long long dv_ss, float scale, int mask_mode,
                      int frame, int causal_off, const unsigned char* key_valid, const float* bias,
                      unsigned int* status, void* stream) {
  if (HD != 64 && HD != 128) return NB_ERR_BAD_ARG;
  if (Hkv <= 0 || Hq % Hkv != 0 || B <= 0 || Sq <= 0 || Sk <= 0) return NB_ERR_BAD_ARG;
  if (mask_mode == NB_MASK_BLOCK_CAUSAL && frame <= 0) return NB_ERR_BAD_ARG;
  if (((dq_ss | dk_ss | dv_ss) * 2) % 16 != 0) return NB_ERR_UNALIGNED;
  cudaStream_t s = (cudaStream_t)stream;
  const long long rows = (long long)B * Sq * Hq;
  fa_delta_kernel<<<(unsigned)ceil_div_ll(rows, 8), 256, 0, s>>>((const __nv_bfloat16*)O, (const __nv_bfloat16*)dO, delta,
                                                                 B, Sq, Hq, HD, o_ss, do_ss);
  NB_LAUNCH_CHECK();
  CUtensorMap tq, tk, tv, tdo;
  int rc = make_tmap_bshd(&tq, Q, B, Sq, Hq, HD, q_sb, q_ss, q_sh, BQ);
  if (rc) return rc;
  rc = make_tmap_bshd(&tk, K, B, Sk, Hkv, HD, k_sb, k_ss, k_sh, BKV);
  if (rc) return rc;
  rc = make_tmap_bshd(&tv, V, B, Sk, Hkv, HD, v_sb, v_ss, v_sh, BKV);
  if (rc) return rc;
  rc = make_tmap_bshd(&tdo, dO, B, Sq, Hq, HD, do_sb, do_ss, do_sh, BQ);
  if (rc) return rc;
  FaParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk;
  p.mask_mode = mask_mode; p.frame = frame; p.causal_off = causal_off;
  p.ld_o = (int)o_ss;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.scale = scale;
  p.key_valid = key_valid; p.bias = bias;
  p.O = nullptr; p.lse = const_cast<float*>(lse); p.status = status;
  p.delta = delta;
  p.dQ = (__nv_bfloat16*)dQ; p.dK = (__nv_bfloat16*)dK; p.dV = (__nv_bfloat16*)dV;
  p.ld_dq = (int)dq_ss; p.ld_dk = (int)dk_ss; p.ld_dv = (int)dv_ss;
  if (g_bwd_mode == 0) return launch_bwd_gen2(tq, tk, tv, tdo, p, HD, s);
  if (HD == 64) return launch_bwd<64>(tq, tk, tv, tdo, p, s);
  return launch_bwd<128>(tq, tk, tv, tdo, p, s);
}

}  // extern "C"
