// Flash attention forward on tcgen05: O = softmax(scale · Q Kᵀ + mask) V, never materialising S×S.
//
// One CTA owns a 128-query tile of one (batch, head).  Warp roles (192 threads):
//   warp 0      TMA producer: Q once, then a 2-stage ring of K and of V tiles (128 keys each)
//   warp 1      MMA issuer:  S_j = Q K_jᵀ  (128×128, accumulator in TMEM, double buffered) and
//               O_j = P_j V_j (128×HD, TMEM); S_{j+1} is issued before P_j is consumed so the tensor
//               core works on the next scores while the softmax warps work on the current ones
//   warps 2..5  softmax: thread t owns query row t (TMEM lane t) — the row maximum, the exponentials and
//               the running sum need no cross-thread traffic.  P_j is written as bf16 straight into the
//               128-byte-swizzled K-major shared-memory layout the tensor core reads as the A operand of
//               the second GEMM; the output accumulator lives in registers and is rescaled there
//               (O ← O·α + O_j), so TMEM is only ever written by the tensor core.
// Masks (evaluated from indices, no S×S tensor): none, causal (k ≤ q + off), block-causal with frame size F
// ((k / F) ≤ (q / F): full attention inside a frame, causal across frames), per-batch key validity
// (key padding, 1 = attend), optional additive fp32 bias [Sq, Sk] (static masks).  Fully masked KV tiles are
// skipped.  GQA: kv head = q head / (Hq / Hkv).  Q_LEN ≠ KV_LEN supported.
// Outputs: O bf16 [B, Sq, Hq, HD] and the row log-sum-exp in base 2 (of the scaled scores) for the backward.
//
// Reference kernels: mma.sync.m16n8k16 flash attention, grid (⌈S/64⌉, B·H), 4 warps
// (noeira/nn/primitives/flash_attention_mma.mojo:227-521, launcher flash_attention.mojo:602-698) and the
// masked / cross / block variants (cross_attention.mojo:97-550, deep_agents/smolvla/block_attention.mojo).
#include "attention_common.cuh"

namespace {
using namespace nb;
using namespace nbattn;

template <int HD>
__global__ void __launch_bounds__(FA_THREADS, 1)
fa_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
              const __grid_constant__ CUtensorMap tmV, const FaParams p) {
  constexpr int NSUB = HD / 64;                 // 64-wide swizzle atoms per row
  constexpr uint32_t Q_BYTES = BQ * HD * 2;
  constexpr uint32_t KV_BYTES = BKV * HD * 2;
  constexpr uint32_t P_BYTES = BQ * BKV * 2;
  // P ring: with two buffers the softmax of block j+1 (exponentials, packing) runs while the tensor core still
  // multiplies P_j V_j; at HD = 128 shared memory only has room for one.
  constexpr int PS = (HD == 64) ? 2 : 1;
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t S_COL = 0, O_COL = 128;    // S: 128 columns, O: HD columns
  constexpr float RESCALE_THRESHOLD = 8.f;      // log2 units: exponentials stay below 2^8 between rescales

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Q_BYTES;             // 2 stages
  uint8_t* sV = sK + 2 * KV_BYTES;        // 2 stages
  uint8_t* sP = sV + 2 * KV_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + PS * P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;    // [2]
  uint64_t* k_empty = bars + 3;   // [2]
  uint64_t* v_full = bars + 5;    // [2]
  uint64_t* v_empty = bars + 7;   // [2]
  uint64_t* s_full = bars + 9;
  uint64_t* s_empty = bars + 10;
  uint64_t* p_full = bars + 11;   // [2] P_j in smem and O rescaled → the PV GEMM may run        (ring index j % PS)
  uint64_t* pv_done = bars + 13;  // [2] PV_j retired: P buffer free, O holds blocks 0..j        (ring index j % PS)
  uint64_t* x_bar = bars + 15;    // the two threads of a row exchange their partial maxima / sums
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  float* sh_x = reinterpret_cast<float*>(tmem_slot + 4);  // [2 buffers][2 halves][128 rows]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * BQ, h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (p.Hq / p.Hkv);
  const int klim = kv_limit(p, q0);
  const int nkb = klim < 0 ? 0 : klim / BKV + 1;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_empty, 8);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&p_full[i], 8);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(x_bar, 8);        // one arrival per softmax warp (256 per-thread arrivals serialise on the barrier word)
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

  if (warp == 0) {
    // ---------------------------------------------------------------- producer
    if (elect_one()) {
      mbar_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int s = 0; s < NSUB; ++s) tma_load_4d(sQ + s * (BQ * 128), &tmQ, q_full, s * 64, h, q0, b);
      for (int j = 0; j < nkb; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (*abort_flag || !mbar_wait(&k_empty[st], ph ^ 1u, p.status, 101)) { *abort_flag = 1; break; }
        mbar_expect_tx(&k_full[st], KV_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d(sK + st * KV_BYTES + s * (BKV * 128), &tmK, &k_full[st], s * 64, hkv, j * BKV, b);
        if (*abort_flag || !mbar_wait(&v_empty[st], ph ^ 1u, p.status, 102)) { *abort_flag = 1; break; }
        mbar_expect_tx(&v_full[st], KV_BYTES);
#pragma unroll
        for (int s = 0; s < NSUB; ++s)
          tma_load_4d(sV + st * KV_BYTES + s * (BKV * 128), &tmV, &v_full[st], s * 64, hkv, j * BKV, b);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc(1u, BQ, BKV, 0u, 0u);  // S = Q Kᵀ : both K-major
      const uint32_t idesc_o = make_idesc(1u, BQ, HD, 0u, 1u);   // O += P V : V is MN-major
      bool ok = mbar_wait(q_full, 0u, p.status, 110);
      if (!ok) *abort_flag = 1;
      auto issue_pv = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        const int ps = j % PS;
        if (*abort_flag || !mbar_wait(&p_full[ps], (uint32_t)(j / PS) & 1u, p.status, 111)) return false;
        if (!mbar_wait(&v_full[st], ph, p.status, 112)) return false;
        tc_fence_after();
        const uint32_t pa = smem_u32(sP + ps * P_BYTES), vb = smem_u32(sV + st * KV_BYTES);
#pragma unroll
        for (int k = 0; k < BKV / 16; ++k) {
          // P: two 64-key sub-tiles of 16 KB; V: 16 key-rows of 128 B per k-step, 64-column chunks 16 KB apart
          const uint64_t adesc = make_smem_desc(pa + (k / 4) * (BQ * 128) + (k % 4) * 32, 16, 1024, 2);
          const uint64_t bdesc = make_smem_desc(vb + k * (16 * 128), BKV * 128, 1024, 2);
          umma_f16(tmem_base + O_COL, adesc, bdesc, idesc_o, (j | k) != 0 ? 1u : 0u);
        }
        umma_commit(&pv_done[ps]);
        umma_commit(&v_empty[st]);
        return true;
      };
      for (int j = 0; j < nkb && ok; ++j) {
        const int st = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (*abort_flag || !mbar_wait(&k_full[st], ph, p.status, 114)) { ok = false; break; }
        if (!mbar_wait(s_empty, ((uint32_t)j & 1u) ^ 1u, p.status, 115)) { ok = false; break; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), kb = smem_u32(sK + st * KV_BYTES);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint64_t adesc = make_smem_desc(qa + (k / 4) * (BQ * 128) + (k % 4) * 32, 16, 1024, 2);
          const uint64_t bdesc = make_smem_desc(kb + (k / 4) * (BKV * 128) + (k % 4) * 32, 16, 1024, 2);
          umma_f16(tmem_base + S_COL, adesc, bdesc, idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(s_full);
        umma_commit(&k_empty[st]);
        if (j > 0 && !issue_pv(j - 1)) { ok = false; break; }
      }
      if (ok && nkb > 0 && !issue_pv(nkb - 1)) ok = false;
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ---------------------------------------------------------------- softmax / epilogue
    // two threads per query row: warps 2..5 take key columns [0,64) of the tile, warps 6..9 columns [64,128)
    constexpr int HC = HD / 2;  // output columns per thread
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;
    const int q = q0 + row;
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    float m_ref = -INFINITY, l = 0.f;  // m_ref: the (possibly stale) maximum the exponentials are taken against
    const unsigned char* kvalid = p.key_valid ? p.key_valid + (size_t)b * p.Sk : nullptr;
    const float* bias_row = (p.bias && q < p.Sq) ? p.bias + (size_t)q * p.Sk : nullptr;
    uint8_t* prow0 = sP + half * (BQ * 128) + (row >> 3) * 1024 + (row & 7) * 128;
    bool ok = true;
    for (int j = 0; j < nkb && ok; ++j) {
      const int k0 = j * BKV;
      if (!__all_sync(0xffffffffu, !*abort_flag && mbar_wait(s_full, (uint32_t)j & 1u, p.status, 120))) { ok = false; break; }
      tc_fence_after();
      // my 64 scores → registers with ONE wait, then hand the S buffer back to the tensor core
      float s[64];
      tmem_ld_32x32b_x32_nowait(lane_addr + S_COL + half * 64, reinterpret_cast<uint32_t*>(s));
      tmem_ld_32x32b_x32_nowait(lane_addr + S_COL + half * 64 + 32, reinterpret_cast<uint32_t*>(s) + 32);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_empty);
      const int lim = row_limit(p, q, k0) - half * 64;  // allowed leading columns of my half
      const bool fast = (lim >= 64) && !kvalid && !bias_row;
      float mult = p.scale_log2;  // exp argument = s * mult − m   (slow path pre-scales and uses mult = 1)
      float mx = -INFINITY;
      if (fast) {
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, s[i]);
        mx *= mult;
      } else {
        mult = 1.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float v = s[i] * p.scale_log2;
          bool a = i < lim;
          if (kvalid || bias_row) {
            const int k = min(k0 + half * 64 + i, p.Sk - 1);
            if (kvalid) a = a && (kvalid[k] != 0);
            if (bias_row) v += bias_row[k] * 1.4426950408889634f;
          }
          v = a ? v : -INFINITY;
          s[i] = v;
          mx = fmaxf(mx, v);
        }
      }
      // row maximum = max over the two halves
      float* xb = sh_x + (j & 1) * 256;
      xb[half * 128 + row] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(x_bar);
      if (!__all_sync(0xffffffffu, mbar_wait(x_bar, (uint32_t)j & 1u, p.status, 123))) { ok = false; break; }
      mx = fmaxf(mx, xb[(half ^ 1) * 128 + row]);
      // lazy rescale: keep the old reference unless the maximum grew by more than the threshold
      float alpha = 1.f;
      const bool grow = mx > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && mx > -INFINITY);
      if (grow) {
        alpha = exp2_fast(m_ref - mx);  // m_ref = -inf → 0
        m_ref = mx;
      }
      const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
      // the P buffer of this block is free once PV_{j-PS} has retired
      uint8_t* prow = prow0 + (j % PS) * P_BYTES;
      if (!__all_sync(0xffffffffu, mbar_wait(&pv_done[j % PS], ((uint32_t)(j / PS) & 1u) ^ 1u, p.status, 121))) { ok = false; break; }
      tc_fence_after();
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O holds blocks < j only after PV_{j-1} has retired (with one buffer that is the wait above)
        if (PS > 1 && !__all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) % PS], (uint32_t)((j - 1) / PS) & 1u, p.status, 125))) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < HC; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(lane_addr + O_COL + half * HC + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32b_x32(lane_addr + O_COL + half * HC + c, r);
        }
        tmem_st_wait();
      }
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          __nv_bfloat162 hv = __floats2bfloat162_rn(exp2_fast(fmaf(s[c + 2 * u], mult, -m_use)),
                                                    exp2_fast(fmaf(s[c + 2 * u + 1], mult, -m_use)));
          // the sum uses the ROUNDED probabilities so that l matches what the tensor core multiplies
          lsum += __low2float(hv) + __high2float(hv);
          pk[u] = *reinterpret_cast<uint32_t*>(&hv);
        }
        // 16-byte chunk index inside the 64-wide sub-tile is XOR-swizzled with (row & 7)
        *reinterpret_cast<uint4*>(prow + (((c >> 3) ^ (row & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l = l * alpha + lsum;
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[j % PS]);
    }
    // row sum = sum over the two halves
    if (ok) {
      float* xb = sh_x + (nkb & 1) * 256;
      xb[half * 128 + row] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(x_bar);
      ok = __all_sync(0xffffffffu, mbar_wait(x_bar, (uint32_t)nkb & 1u, p.status, 124));
      if (ok) l += xb[(half ^ 1) * 128 + row];
    }
    if (ok && nkb > 0) ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(nkb - 1) % PS], (uint32_t)((nkb - 1) / PS) & 1u, p.status, 122));
    if (!ok) *abort_flag = 1;
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.O + ((size_t)b * p.Sq + min(q, p.Sq - 1)) * p.ld_o + (size_t)h * HD + half * HC;
#pragma unroll
      for (int c = 0; c < HC; c += 32) {
        uint32_t r[32];
        if (nkb > 0) {
          tmem_ld_32x32b_x32(lane_addr + O_COL + half * HC + c, r);
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
      if (p.lse && q < p.Sq && half == 0)
        p.lse[((size_t)b * p.Hq + h) * p.Sq + q] = (l > 0.f) ? m_ref + log2f(l) : -INFINITY;
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
int launch_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p,
               cudaStream_t s) {
  constexpr size_t smem = (size_t)BQ * HD * 2 + 4 * (size_t)BKV * HD * 2 + (HD == 64 ? 2 : 1) * (size_t)BQ * BKV * 2 + 1024 + 256 + 2048;
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(fa_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  dim3 grid(ceil_div(p.Sq, BQ), p.Hq, p.B);
  fa_fwd_kernel<HD><<<grid, FA_THREADS, smem, s>>>(tq, tk, tv, p);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // namespace

static int g_fwd_mode = 0;  // 0 = choose by problem size, 1 = one query tile per CTA, 2 = two query tiles per CTA

extern "C" {

// Selects the forward kernel (tests and benchmarks compare the two forms); returns the previous setting.
int nb_flash_attn_fwd_mode(int mode) {
  const int old = g_fwd_mode;
  if (mode >= 0 && mode <= 2) g_fwd_mode = mode;
  return old;
}

// Q [B,Sq,Hq,HD], K/V [B,Sk,Hkv,HD] bf16, element strides given per tensor as (batch, token, head);
// the innermost (HD) stride is 1.  O is written with the same batch/token/head strides as described by
// (o_sb, o_ss) and head stride HD.
int nb_flash_attn_fwd(const void* Q, const void* K, const void* V, void* O, float* lse, int B, int Hq, int Hkv, int Sq,
                      int Sk, int HD, long long q_sb, long long q_ss, long long q_sh, long long k_sb, long long k_ss,
                      long long k_sh, long long v_sb, long long v_ss, long long v_sh, long long o_ss, float scale,
                      int mask_mode, int frame, int causal_off, const unsigned char* key_valid, const float* bias,
                      unsigned int* status, void* stream) {
  if (HD != 64 && HD != 128) return NB_ERR_BAD_ARG;
  if (Hkv <= 0 || Hq % Hkv != 0 || B <= 0 || Sq <= 0 || Sk <= 0) return NB_ERR_BAD_ARG;
  if (mask_mode == NB_MASK_BLOCK_CAUSAL && frame <= 0) return NB_ERR_BAD_ARG;
  if ((o_ss * 2) % 16 != 0 || (reinterpret_cast<uintptr_t>(O) & 15)) return NB_ERR_UNALIGNED;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_bshd(&tq, Q, B, Sq, Hq, HD, q_sb, q_ss, q_sh, BQ);
  if (rc) return rc;
  rc = make_tmap_bshd(&tk, K, B, Sk, Hkv, HD, k_sb, k_ss, k_sh, BKV);
  if (rc) return rc;
  rc = make_tmap_bshd(&tv, V, B, Sk, Hkv, HD, v_sb, v_ss, v_sh, BKV);
  if (rc) return rc;
  FaParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk;
  p.mask_mode = mask_mode; p.frame = frame; p.causal_off = causal_off;
  p.ld_o = (int)o_ss;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.key_valid = key_valid; p.bias = bias;
  p.O = (__nv_bfloat16*)O; p.lse = lse; p.status = status;
  cudaStream_t s = (cudaStream_t)stream;
  // two tiles per CTA pay once every SM has a CTA of 256 queries; small problems keep the finer grid
  const bool two = g_fwd_mode == 2 || (g_fwd_mode == 0 && Sq > BQ && (long long)ceil_div(Sq, 2 * BQ) * Hq * B >= 148);
  if (two) return launch_fwd_two_tile(tq, tk, tv, p, HD, s);
  if (HD == 64) return launch_fwd<64>(tq, tk, tv, p, s);
  return launch_fwd<128>(tq, tk, tv, p, s);
}

}  // extern "C"
