// Flash attention forward, two query tiles per CTA ("ping-pong"): O = softmax(scale · Q Kᵀ + mask) V.
//
// One CTA owns 256 consecutive queries of one (batch, head) as two 128-row tiles.  The per-block chain of one tile
// (S = Q Kᵀ on the tensor core → row softmax on the CUDA cores → O += P V on the tensor core) is latency-serial;
// with two tiles the tensor core multiplies for one tile while the other tile's softmax runs, and both tiles share
// every K / V tile that TMA brings in (half the shared-memory fill traffic per query).
//
//   warp 0      TMA producer: Q0, Q1 once, then a ring of K tiles and a ring of V tiles (128 keys each)
//   warp 1      MMA issuer.  Steady state per key block j:   [P0_j ready] O0 += P0_j V_j ; S0_{j+1} = Q0 K_{j+1}ᵀ
//                                                             [P1_j ready] O1 += P1_j V_j ; S1_{j+1} = Q1 K_{j+1}ᵀ
//               P_t(j) is published in two halves (64 keys each): the first four k-steps of P V start while the
//               softmax still computes the second half.
//   warps 2,3   idle (they complete the first warpgroup, which gives its registers away with setmaxnreg)
//   warps 4..7  softmax of tile 0, warps 8..11 softmax of tile 1: thread = query row (TMEM lane), 128 scores in
//               registers (setmaxnreg raises these two warpgroups to 208 registers), one row maximum / sum without
//               any cross-thread traffic; packed fp32 arithmetic (fma / add on register pairs) and a three-input
//               maximum keep the instruction count near 3.5 per score.  Blocks that no row of the tile has masked
//               run a loop without any mask arithmetic; diagonal blocks (index masks) select -inf first and then
//               share that code; key-validity / bias calls take a general loop.
// Tensor memory (512 columns): S0 | S1 | O0 | O1.  The probabilities P_t are written back as packed bf16 INTO the first
// 64 columns of S_t with tcgen05.st and consumed from there as the A operand of the second GEMM, so P never passes
// through shared memory and needs no proxy fence.  MMAs of one thread execute in issue order, so S_t(j+1) — issued
// directly after P_t(j) V_j — cannot overwrite P_t(j) early, and the commit that publishes S_t(j+1) also covers
// P_t(j) V_j: a softmax thread that sees S_t(j+1) may rescale O_t.  O_t stays in tensor memory and is rescaled lazily
// (only when a row maximum grows by more than 2^8).  CTAs of masked shapes are launched longest first.
// Masks, GQA, Q_LEN ≠ KV_LEN, outputs: as in the one-tile kernel (attention_tcgen05.cu).
// Reference kernels: noeira/nn/primitives/flash_attention_mma.mojo:227-521 (mma.sync, 64-query CTAs).
#include <type_traits>

#include "attention_common.cuh"


namespace {
using namespace nb;
using namespace nbattn;

// P = 2^(s * mult - m) of half a row (scores [64·HALF, 64·HALF + 64) of 128), written as packed bf16 into tensor-memory
// columns [s_addr + 32·HALF, +32); returns the sum of that half.  Arguments and the running sum are formed as packed
// fp32 pairs (one FMA-pipe instruction per two scores).  All exponentials run on the special-function unit: moving a
// share of them to a polynomial on the FMA pipe was measured (1/8, 1/4 and 1/2 of the elements, packed and scalar
// forms) and lost to the extra instructions and registers it costs a thread that already holds 128 scores.
template <int HALF>
__device__ __forceinline__ float exp_store(const float (&s)[128], float mult, float m_use, uint32_t s_addr) {
  uint64_t lsum2 = pack2(0.f, 0.f);
  const uint64_t mult2 = pack2(mult, mult), negm2 = pack2(-m_use, -m_use);
#pragma unroll
  for (int c = HALF * 4; c < HALF * 4 + 4; ++c) {
    uint32_t pk[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      uint64_t x2 = fma2(pack2(s[c * 16 + 2 * u], s[c * 16 + 2 * u + 1]), mult2, negm2);
      float e0, e1;
      unpack2(x2, e0, e1);
      e0 = exp2_fast(e0);
      e1 = exp2_fast(e1);
      x2 = pack2(e0, e1);
      lsum2 = add2(lsum2, x2);
      __nv_bfloat162 hv = __floats2bfloat162_rn(e0, e1);
      pk[u] = *reinterpret_cast<uint32_t*>(&hv);
    }
    // 16 keys → 8 packed columns
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(s_addr + c * 8),
                 "r"(pk[0]), "r"(pk[1]), "r"(pk[2]), "r"(pk[3]), "r"(pk[4]), "r"(pk[5]), "r"(pk[6]), "r"(pk[7])
                 : "memory");
  }
  float l0, l1;
  unpack2(lsum2, l0, l1);
  return l0 + l1;
}

constexpr int FA2_THREADS = 384;  // three warpgroups: {TMA, MMA, 2 idle}, softmax tile 0, softmax tile 1
// Register budget: the CTA is launched with 384 x 168 registers and setmaxnreg only moves registers inside that
// allocation (an increase BLOCKS until the CTA's pool has them), so 128 x 88 + 256 x 208 must not exceed 384 x 168.
static_assert(128 * 88 + 256 * 208 <= FA2_THREADS * 168, "setmaxnreg budget");

template <int HD>
__global__ void __launch_bounds__(FA2_THREADS, 1)
fa_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
               const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  constexpr int NSUB = HD / 64;                 // 64-wide swizzle atoms per row
  constexpr int KS = (HD == 64) ? 4 : 2;        // K ring and V ring depth
  constexpr uint32_t Q_BYTES = BQ * HD * 2;
  constexpr uint32_t KV_BYTES = BKV * HD * 2;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr float RESCALE_THRESHOLD = 8.f;      // log2 units: exponentials stay below 2^8 between rescales

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                      // 2 tiles
  uint8_t* sK = sQ + 2 * Q_BYTES;          // KS stages
  uint8_t* sV = sK + KS * KV_BYTES;        // KS stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KS * KV_BYTES);
  uint64_t* q_full = bars;                 // [2]
  uint64_t* k_full = bars + 2;             // [KS]
  uint64_t* k_empty = k_full + KS;
  uint64_t* v_full = k_empty + KS;
  uint64_t* v_empty = v_full + KS;
  uint64_t* s_full = v_empty + KS;         // [2] S_t(j) complete (and every MMA issued before it)
  uint64_t* p_full = s_full + 2;           // [2] P_t(j) stored in tensor memory, O_t rescaled
  uint64_t* o_done = p_full + 2;           // [2] last P V of tile t retired
  uint64_t* p_lo = o_done + 2;             // [2] first 64 keys of P_t(j) stored
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(p_lo + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 1-D grid.  Index masks make the work of a CTA grow with its query position, so those launch the LAST query
  // super-tiles of every (head, batch) first (longest first: the short ones fill the tail of the last wave);
  // without a mask consecutive CTAs walk the queries of one (head, batch) and share its K / V in L2.
  const int nqs = ceil_div(p.Sq, 2 * BQ);
  int qs, hb;
  if (p.mask_mode == NB_MASK_NONE) {
    qs = blockIdx.x % nqs;
    hb = blockIdx.x / nqs;
  } else {
    const int nhb = p.Hq * p.B;
    qs = nqs - 1 - blockIdx.x / nhb;
    hb = blockIdx.x % nhb;
  }
  const int q0 = qs * (2 * BQ), h = hb % p.Hq, b = hb / p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);
  int nkb[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qt = q0 + t * BQ;
    const int klim = qt < p.Sq ? kv_limit(p, qt) : -1;
    nkb[t] = klim < 0 ? 0 : klim / BKV + 1;
  }
  const int nmax = max(nkb[0], nkb[1]);

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_done[i], 1);
      mbar_init(&p_lo[i], 4);
    }
    for (int i = 0; i < KS; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // 32-bit shared-memory addresses: one base per array, everything else is base + constant
  const uint32_t aQ = smem_u32(sQ), aK = aQ + 2 * Q_BYTES, aV = aK + KS * KV_BYTES, aB = aV + KS * KV_BYTES;
  auto q_full_a = [&](int i) { return aB + 8u * (uint32_t)i; };
  auto k_full_a = [&](int i) { return aB + 8u * (uint32_t)(2 + i); };
  auto k_empty_a = [&](int i) { return aB + 8u * (uint32_t)(2 + KS + i); };
  auto v_full_a = [&](int i) { return aB + 8u * (uint32_t)(2 + 2 * KS + i); };
  auto v_empty_a = [&](int i) { return aB + 8u * (uint32_t)(2 + 3 * KS + i); };
  auto s_full_a = [&](int i) { return aB + 8u * (uint32_t)(2 + 4 * KS + i); };
  auto p_full_a = [&](int i) { return aB + 8u * (uint32_t)(4 + 4 * KS + i); };
  auto o_done_a = [&](int i) { return aB + 8u * (uint32_t)(6 + 4 * KS + i); };
  auto p_lo_a = [&](int i) { return aB + 8u * (uint32_t)(8 + 4 * KS + i); };

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    if (elect_one()) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        if (nkb[t] == 0) continue;
        mbar_expect_tx_a(q_full_a(t), Q_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d_a(aQ + t * Q_BYTES + s * (BQ * 128), &tmQ, q_full_a(t), s * 64, h, q0 + t * BQ, b);
      }
      for (int j = 0; j < nmax; ++j) {
        const int st = j % KS;
        const uint32_t ph = (uint32_t)(j / KS) & 1u;
        if (*abort_flag || !mbar_wait_a(k_empty_a(st), ph ^ 1u, p.status, 201)) { *abort_flag = 1; break; }
        mbar_expect_tx_a(k_full_a(st), KV_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d_a(aK + st * KV_BYTES + s * (BKV * 128), &tmK, k_full_a(st), s * 64, hkv, j * BKV, b);
        if (*abort_flag || !mbar_wait_a(v_empty_a(st), ph ^ 1u, p.status, 202)) { *abort_flag = 1; break; }
        mbar_expect_tx_a(v_full_a(st), KV_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d_a(aV + st * KV_BYTES + s * (BKV * 128), &tmV, v_full_a(st), s * 64, hkv, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(1u, BQ, BKV, 0u, 0u);  // S = Q Kᵀ : both K-major
      const uint32_t idesc_o = make_idesc(1u, BQ, HD, 0u, 1u);   // O += P V : P from tensor memory, V MN-major
      bool ok = true;
      // S_t(j) = Q_t K_jᵀ; K_j is first used by the lowest active tile and released after the highest
      auto issue_s = [&](int t, int j) -> bool {
        const int st = j % KS;
        const bool first = (t == 0) || !(j < nkb[0]);
        const bool last = (t == 1) || !(j < nkb[1]);
        if (j == 0 && !mbar_wait_a(q_full_a(t), 0u, p.status, 210)) return false;
        if (first && !mbar_wait_a(k_full_a(st), (uint32_t)(j / KS) & 1u, p.status, 211)) return false;
        tc_fence_after();
        // descriptors of the k-steps differ from the first one only in the start-address field (bytes >> 4)
        const uint64_t adesc0 = make_smem_desc(aQ + t * Q_BYTES, 16, 1024, 2);
        const uint64_t bdesc0 = make_smem_desc(aK + st * KV_BYTES, 16, 1024, 2);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t off = ((k / 4) * (BQ * 128) + (k % 4) * 32) >> 4;
          umma_f16(tmem_base + t * 128, adesc0 + off, bdesc0 + off, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit_a(s_full_a(t));
        if (last) umma_commit_a(k_empty_a(st));
        return true;
      };
      auto issue_pv = [&](int t, int j) -> bool {
        const int st = j % KS;
        const bool first = (t == 0) || !(j < nkb[0]);
        const bool last = (t == 1) || !(j < nkb[1]);
        if (*abort_flag || !mbar_wait_a(p_lo_a(t), (uint32_t)j & 1u, p.status, 214)) return false;
        if (first && !mbar_wait_a(v_full_a(st), (uint32_t)(j / KS) & 1u, p.status, 213)) return false;
        tc_fence_after();
        const uint64_t bdesc0 = make_smem_desc(aV + st * KV_BYTES, BKV * 128, 1024, 2);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // the second half of the keys waits for the second half of P
          if (k == BKV / 32) {
            if (!mbar_wait_a(p_full_a(t), (uint32_t)j & 1u, p.status, 212)) return false;
            tc_fence_after();
          }
          // P: 16 keys = 8 packed columns per k-step; V: 16 key-rows of 128 B per k-step, 64-column chunks 16 KB apart
          umma_f16_ts(tmem_base + 256 + t * 128, tmem_base + t * 128 + k * 8, bdesc0 + ((k * 16 * 128) >> 4), idesc_o,
                      (j | k) != 0 ? 1u : 0u);
        }
        if (last) umma_commit_a(v_empty_a(st));
        if (j == nkb[t] - 1) umma_commit_a(o_done_a(t));
        return true;
      };
      for (int t = 0; t < 2 && ok; ++t)
        if (nkb[t] > 0) ok = issue_s(t, 0);
      for (int j = 0; j < nmax && ok; ++j) {
        for (int t = 0; t < 2 && ok; ++t) {
          if (j >= nkb[t]) continue;
          ok = issue_pv(t, j);
          if (ok && j + 1 < nkb[t]) ok = issue_s(t, j + 1);
        }
      }
      if (!ok) *abort_flag = 1;
    }
  } else if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  } else {
    // ---------------------------------------------------------------- softmax / epilogue: one thread per query row
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int t = (warp - 4) >> 2;
    const int quarter = warp & 3;          // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;
    const int q = q0 + t * BQ + row;
    const int n = nkb[t];
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t s_addr = lane_addr + t * 128, o_addr = lane_addr + 256 + t * 128;
    float m_ref = -INFINITY, l = 0.f;      // m_ref: the (possibly stale) maximum the exponentials are taken against
    const unsigned char* kvalid = p.key_valid ? p.key_valid + (size_t)b * p.Sk : nullptr;
    const float* bias_row = (p.bias && q < p.Sq) ? p.bias + (size_t)q * p.Sk : nullptr;
    bool ok = true;
    // One key block of this row.  MODE 0: no score of the block is masked for any row of the tile (the hot loop: no
    // mask arithmetic at all); MODE 1: index masks only, a prefix of the block is allowed (diagonal blocks); MODE 2: key
    // validity and / or an additive bias (every block of such a call).
    auto block = [&](int j, auto mode_tag) -> bool {
      constexpr int MODE = decltype(mode_tag)::value;
      const int k0 = j * BKV;
      if (!__all_sync(0xffffffffu, !*abort_flag && mbar_wait_a(s_full_a(t), (uint32_t)j & 1u, p.status, 220))) return false;
      tc_fence_after();
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld_32x32b_x32_nowait(s_addr + c * 32, reinterpret_cast<uint32_t*>(s) + c * 32);
      float mult = p.scale_log2;                     // exp argument = s * mult − m (MODE 2 pre-scales, mult = 1)
      float mx;
      tmem_ld_wait();
      if (MODE <= 1) {
        if (MODE == 1) {
          const int lim = row_limit(p, q, k0);       // allowed leading columns of this block
#pragma unroll
          for (int i = 0; i < 128; ++i) s[i] = i < lim ? s[i] : -INFINITY;
        }
        float m0 = s[0], m1 = s[1], m2 = s[2], m3 = s[3];
#pragma unroll
        for (int i = 4; i < 124; i += 8) {   // three-input maximum: 64 instructions for 128 scores
          m0 = max3(m0, s[i], s[i + 1]);
          m1 = max3(m1, s[i + 2], s[i + 3]);
          m2 = max3(m2, s[i + 4], s[i + 5]);
          m3 = max3(m3, s[i + 6], s[i + 7]);
        }
        m0 = max3(m0, s[124], s[125]);
        m1 = max3(m1, s[126], s[127]);
        mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * mult;   // -inf stays -inf (the scale is positive)
      } else {
        const int lim = row_limit(p, q, k0);
        mult = 1.f;
        mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          float v = s[i] * p.scale_log2;
          bool a = i < lim;
          const int k = min(k0 + i, p.Sk - 1);
          if (kvalid) a = a && (kvalid[k] != 0);
          if (bias_row) v += bias_row[k] * 1.4426950408889634f;
          v = a ? v : -INFINITY;
          s[i] = v;
          mx = fmaxf(mx, v);
        }
      }
      // lazy rescale: keep the old reference unless the maximum grew by more than the threshold
      float alpha = 1.f;
      const bool grow = mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx > -INFINITY);
      if (grow) {
        alpha = exp2_fast(m_ref - mx);  // m_ref = -inf → 0
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // S_t(j) was committed after P_t(j-1) V_{j-1}, so O_t holds blocks < j
#pragma unroll
        for (int c = 0; c < HD; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(o_addr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x32(o_addr + c, r);
        }
      }
      // The first 64 keys of P are published on their own so that the tensor core starts P V half a softmax earlier.
      float lblk = exp_store<0>(s, mult, m_use, s_addr);
      {
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_a(p_lo_a(t));
      }
      lblk += exp_store<1>(s, mult, m_use, s_addr);
      l = l * alpha + lblk;
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_a(p_full_a(t));
      return true;
    };
    // blocks [0, nfull) are unmasked for every row of the tile: all keys exist and the tile's FIRST query may see them
    int nfull = 0;
    if (!kvalid && !p.bias) {
      const int qf = min(q0 + t * BQ, p.Sq - 1);
      int last = p.Sk - 1;
      if (p.mask_mode == NB_MASK_CAUSAL) last = min(last, qf + p.causal_off);
      else if (p.mask_mode == NB_MASK_BLOCK_CAUSAL) last = min(last, (qf / p.frame + 1) * p.frame - 1);
      nfull = max(0, min(n, (last + 1) / BKV));
    }
    int j = 0;
#pragma unroll 1
    for (; j < nfull && ok; ++j) ok = block(j, std::integral_constant<int, 0>{});
    if (!kvalid && !p.bias) {
#pragma unroll 1
      for (; j < n && ok; ++j) ok = block(j, std::integral_constant<int, 1>{});
    } else {
#pragma unroll 1
      for (; j < n && ok; ++j) ok = block(j, std::integral_constant<int, 2>{});
    }
    if (ok && n > 0) ok = __all_sync(0xffffffffu, mbar_wait_a(o_done_a(t), 0u, p.status, 222));
    if (!ok) *abort_flag = 1;
    if (ok && q0 + t * BQ < p.Sq) {
      tc_fence_after();
      const float inv = (m_ref > -INFINITY && l > 0.f) ? 1.f / l : 0.f;   // no allowed key at all → zeros
      __nv_bfloat16* orow = p.O + ((size_t)b * p.Sq + min(q, p.Sq - 1)) * p.ld_o + (size_t)h * HD;
#pragma unroll
      for (int c = 0; c < HD; c += 32) {
        uint32_t r[32];
        if (n > 0) {
          tmem_ld_32x32b_x32(o_addr + c, r);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0u;
        }
        if (q < p.Sq) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 pk;
            __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv),
                           h1 = __floats2bfloat162_rn(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv),
                           h2 = __floats2bfloat162_rn(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv),
                           h3 = __floats2bfloat162_rn(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            pk.x = *reinterpret_cast<uint32_t*>(&h0);
            pk.y = *reinterpret_cast<uint32_t*>(&h1);
            pk.z = *reinterpret_cast<uint32_t*>(&h2);
            pk.w = *reinterpret_cast<uint32_t*>(&h3);
            *reinterpret_cast<uint4*>(orow + c + i) = pk;
          }
        }
      }
      if (p.lse && q < p.Sq) p.lse[((size_t)b * p.Hq + h) * p.Sq + q] = (m_ref > -INFINITY && l > 0.f) ? m_ref + log2f(l) : -INFINITY;
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
int launch_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, cudaStream_t s) {
  constexpr int KS = (HD == 64) ? 4 : 2;
  constexpr size_t smem = 2 * (size_t)BQ * HD * 2 + 2 * KS * (size_t)BKV * HD * 2 + 1024 + 512;
  static_assert(smem <= 232448, "shared memory budget");
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(fa_fwd2_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid(ceil_div(p.Sq, 2 * BQ) * p.Hq * p.B);
  fa_fwd2_kernel<HD><<<grid, FA2_THREADS, smem, s>>>(tq, tk, tv, p);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // namespace

namespace nbattn {
int launch_fwd_two_tile(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, int HD,
                        cudaStream_t s) {
  if (HD == 64) return launch_fwd2<64>(tq, tk, tv, p, s);
  return launch_fwd2<128>(tq, tk, tv, p, s);
}
}  // namespace nbattn
