// bf16 GEMM on the 5th generation tensor cores: D = epilogue(A · B), fp32 accumulation in TMEM.
//
//   * operands are fetched by TMA (128-byte swizzle, no multicast) into a multi-stage shared
//     memory ring; one elected thread issues tcgen05.mma (M=128, N=BN, K=16) four times per
//     64-wide k-block; tcgen05.commit releases the stage / publishes the accumulator;
//   * persistent CTAs (one per SM) walk the tile list; two TMEM accumulators let the epilogue
//     of tile i overlap the main loop of tile i+1;
//   * warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
//     warps 2..5 = epilogue (TMEM quarter = warp_id % 4);
//   * both operands may be K-major ([rows, K] row-major) or MN-major ([K, rows] row-major), so
//     forward (x·W, W stored [IN, OUT]), dgrad (dy·Wᵀ) and wgrad (xᵀ·dy) all run from the
//     natural layouts without a transpose pass;
//   * epilogue: +bias[n], activation, or multiplication by the activation derivative taken from
//     a saved tensor (dgrad of tanh / relu / gelu / silu), optional accumulate into fp32 output
//     (dW += …), bf16 or fp32 store;
//   * every mbarrier wait is bounded; on a timeout the CTA records it in `status`, all roles
//     drain, TMEM is released and the kernel returns.
//
// Counterpart in the reference: library GEMMs only (cuBLAS / cuBLASLt epilogues / MAX matmul;
// noeira/nn/primitives/linear.mojo:1295-1387, noeira/nn/core/cublaslt_gemm.mojo:66-73).
#include <cuda.h>

#include "common.cuh"
#include "gemm_api.h"

namespace {

using namespace nb;

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;  // operand majors
  int tf32;        // 1: operands are fp32 read as TF32 (kind::tf32, 8 k per instruction, 32 elements per 128-byte row)
  int ldd;         // output row pitch (elements)
  int ld_aux;      // aux row pitch (elements, bf16)
  int out_f32, accumulate, act, dact;
  int tiles_m, tiles_n, num_kb;
  int splits, kb_per_split;  // split-K: work item = (tile, split); partial tiles meet in `ws`
  float alpha;
  float* ws;                 // splits>1: fp32 partial tiles, [tile][split][BM*BN]
  unsigned int* tile_ctr;    // splits>1: one arrival counter per tile (zero between launches)
  void* D;
  const float* bias;
  const __nv_bfloat16* aux;
  unsigned int* status;
  // implicit-GEMM convolution (conv != 0): A is never materialised; the producer reads activation patches of the NHWC
  // input through a 4-D tensor map (c, w, h, b), one box of conv_bw output pixels x 64 channels per TMA
  // conv == 2: weight gradient.  A = patches^T is MN-major: the SAME shared-memory image as the forward's A tile (rows =
  // pixels, 128 bytes of channels), now read with the pixels as the reduction dimension; B = dy, MN-major
  int conv, conv_c, conv_ow, conv_oh, conv_kw, conv_pad, conv_bw, conv_taps, conv_b;
};

__device__ __forceinline__ void tma_load_4d_g(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// MUFU tanh: one instruction, max relative error 2^-11 — below bf16 resolution of the stored result.
__device__ __forceinline__ float tanh_fast(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The activation code is selected ONCE per 16-column chunk and the taken case is a short straight run: the
// epilogue executes few instructions per tile, so its speed is set by instruction fetch, i.e. by code size.
__device__ __forceinline__ void act_apply16(int act, float (&v)[16]) {
  switch (act) {
    case NB_ACT_RELU:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = fmaxf(v[j], 0.f);
      break;
    case NB_ACT_TANH:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = tanh_fast(v[j]);
      break;
    case NB_ACT_GELU:
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const float x = v[j];
        v[j] = 0.5f * x * (1.f + tanh_fast(0.7978845608028654f * (x + 0.044715f * x * x * x)));
      }
      break;
    case NB_ACT_SILU:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = v[j] / (1.f + __expf(-v[j]));
      break;
    case NB_ACT_SIGMOID:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = 1.f / (1.f + __expf(-v[j]));
      break;
    default: break;
  }
}
// derivative factor from the SAVED tensor: tanh/relu/sigmoid save the output y, gelu/silu save the input x
__device__ __forceinline__ float dact_apply(int dact, float s) {
  switch (dact) {
    case NB_ACT_RELU: return s > 0.f ? 1.f : 0.f;
    case NB_ACT_TANH: return 1.f - s * s;
    case NB_ACT_SIGMOID: return s * (1.f - s);
    case NB_ACT_GELU: {
      const float c = 0.7978845608028654f;
      const float u = c * (s + 0.044715f * s * s * s);
      const float t = tanh_fast(u);
      return 0.5f * (1.f + t) + 0.5f * s * (1.f - t * t) * c * (1.f + 3.f * 0.044715f * s * s);
    }
    case NB_ACT_SILU: {
      const float sg = 1.f / (1.f + __expf(-s));
      return sg * (1.f + s * (1.f - sg));
    }
    default: return 1.f;
  }
}
__device__ __forceinline__ void dact_apply16(int dact, float (&v)[16], const float (&sv)[16]) {
  switch (dact) {
    case NB_ACT_RELU:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = sv[j] > 0.f ? v[j] : 0.f;
      break;
    case NB_ACT_TANH:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] *= 1.f - sv[j] * sv[j];
      break;
    case NB_ACT_SIGMOID:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] *= sv[j] * (1.f - sv[j]);
      break;
    case NB_ACT_GELU:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] *= dact_apply(NB_ACT_GELU, sv[j]);
      break;
    case NB_ACT_SILU:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] *= dact_apply(NB_ACT_SILU, sv[j]);
      break;
    case NB_AUX_ADD:
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] += sv[j];
      break;
    default: break;
  }
}

// Epilogue for 16 consecutive columns of one output row, in two phases so that the global loads it needs (the saved
// activation for a fused derivative, the old output when accumulating) can be issued one chunk ahead of their use:
// a chunk costs a DRAM / L2 round trip otherwise, which made narrow-K GEMMs epilogue-bound.
struct EpiPrefetch {
  uint4 aux[2];   // 16 bf16 of the saved tensor
  float4 old[4];  // 16 fp32 of the previous output (accumulate)
};

__device__ __forceinline__ void epilogue_prefetch16(const GemmParams& p, int row, int col0, bool active, EpiPrefetch& pf) {
  if (!active || col0 + 16 > p.N) return;
  if (p.dact && (p.ld_aux % 8 == 0)) {
    const __nv_bfloat16* ax = p.aux + (size_t)row * p.ld_aux + col0;
    pf.aux[0] = __ldg(reinterpret_cast<const uint4*>(ax));
    pf.aux[1] = __ldg(reinterpret_cast<const uint4*>(ax + 8));
  }
  if (p.out_f32 && p.accumulate && (p.ldd % 4 == 0)) {
    const float* o = reinterpret_cast<const float*>(p.D) + (size_t)row * p.ldd + col0;
#pragma unroll
    for (int j = 0; j < 4; ++j) pf.old[j] = *reinterpret_cast<const float4*>(o + 4 * j);
  }
}

__device__ __forceinline__ void epilogue_store16(const GemmParams& p, int row, int col0, float (&v)[16],
                                                 const EpiPrefetch& pf) {
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] *= p.alpha;
  const bool full = (col0 + 16 <= p.N);
  if (p.bias) {
    if (full && (col0 % 4 == 0)) {
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + col0 + j));
        v[j] += bv.x; v[j + 1] += bv.y; v[j + 2] += bv.z; v[j + 3] += bv.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (col0 + j < p.N) v[j] += p.bias[col0 + j];
    }
  }
  if (p.act) act_apply16(p.act, v);
  if (p.dact) {
    float sv[16];
    if (full && (p.ld_aux % 8 == 0)) {
      const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&pf.aux[0]);
      const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&pf.aux[1]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sv[2 * j] = __low2float(h0[j]);
        sv[2 * j + 1] = __high2float(h0[j]);
        sv[8 + 2 * j] = __low2float(h1[j]);
        sv[8 + 2 * j + 1] = __high2float(h1[j]);
      }
    } else {
      const __nv_bfloat16* ax = p.aux + (size_t)row * p.ld_aux + col0;
#pragma unroll
      for (int j = 0; j < 16; ++j) sv[j] = (col0 + j < p.N) ? __bfloat162float(ax[j]) : 0.f;
    }
    dact_apply16(p.dact, v, sv);
  }
  if (p.out_f32) {
    float* o = reinterpret_cast<float*>(p.D) + (size_t)row * p.ldd + col0;
    if (full && (p.ldd % 4 == 0)) {
#pragma unroll
      for (int j = 0; j < 16; j += 4) {
        float4 x = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
        if (p.accumulate) {
          const float4 y = pf.old[j >> 2];
          x.x += y.x; x.y += y.y; x.z += y.z; x.w += y.w;
        }
        *reinterpret_cast<float4*>(o + j) = x;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (col0 + j < p.N) o[j] = p.accumulate ? o[j] + v[j] : v[j];
    }
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(p.D) + (size_t)row * p.ldd + col0;
    if (full && (p.ldd % 8 == 0)) {
#pragma unroll
      for (int j = 0; j < 16; j += 8) {
        uint4 pk;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(v[j], v[j + 1]), h1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]),
                       h2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), h3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
        pk.x = *reinterpret_cast<uint32_t*>(&h0);
        pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2);
        pk.w = *reinterpret_cast<uint32_t*>(&h3);
        *reinterpret_cast<uint4*>(o + j) = pk;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (col0 + j < p.N) o[j] = __float2bfloat16(v[j]);
    }
  }
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& mb, int& nb_) {
  constexpr int GM = 8;
  const int per_group = GM * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GM;
  const int gsz = min(tiles_m - first_m, GM);
  const int in_group = tile - group * per_group;
  mb = first_m + in_group % gsz;
  nb_ = in_group / gsz;
}

template <int BN, int STAGES>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;
  constexpr uint32_t B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* ticket_slot = tmem_slot + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_items = p.tiles_m * p.tiles_n * p.splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
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
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      // a k-block is one 128-byte swizzle row of K: 64 bf16 or 32 fp32 elements; an MN-major operand arrives in chunks of
      // that many MN elements, each chunk bk rows of 128 bytes
      const int bk = p.tf32 ? BK / 2 : BK, chunk = bk;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int mb, nb_;
        const int tile = item / p.splits, split = item - tile * p.splits;
        tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb_);
        const int kb0 = split * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (*abort_flag || !mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, 1)) { ok = false; *abort_flag = 1; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          mbar_expect_tx(&full_bar[stage], STAGE_BYTES);
          if (p.conv == 2) {
            // rows of the tile = 2 chunks of 64 channels of one filter tap each; k-block kb = 64 output pixels as runs of
            // bw consecutive pixels of one output row.  A chunk past the last tap and pixels past the last image read the
            // zero fill (image index out of range), so the byte count of the stage stays the same.
            const int bw = p.conv_bw, per_img = p.conv_oh * p.conv_ow;
            for (int h = 0; h < BM / 64; ++h) {
              const int kpos = mb * BM + h * 64, tap = kpos / p.conv_c, c0 = kpos - tap * p.conv_c;
              const int kh = tap / p.conv_kw, kw = tap - kh * p.conv_kw;
              for (int i = 0; i < BK / bw; ++i) {
                const int m0 = kb * BK + i * bw;
                int bimg = m0 / per_img;
                const int rem = m0 - bimg * per_img;
                const int oh = rem / p.conv_ow, ow0 = rem - oh * p.conv_ow;
                if (tap >= p.conv_taps) bimg = p.conv_b;
                tma_load_4d_g(sa + h * (64 * BK * 2) + i * bw * 128, &tmA, &full_bar[stage], c0, ow0 - p.conv_pad + kw,
                              oh - p.conv_pad + kh, bimg);
              }
            }
          } else if (p.conv) {
            // k-block kb = 64 channels [c0, c0+64) of filter tap (kh, kw); the 128 output pixels of the tile are
            // 128 / bw runs of bw consecutive pixels of one output row (bw divides OW and 128), stride 1:
            // input pixel = output pixel + tap − pad; coordinates outside the image read the zero fill
            const int kpos = kb * BK, tap = kpos / p.conv_c, c0 = kpos - tap * p.conv_c;
            const int kh = tap / p.conv_kw, kw = tap - kh * p.conv_kw;
            const int bw = p.conv_bw, per_img = p.conv_oh * p.conv_ow;
            for (int i = 0; i < BM / bw; ++i) {
              const int m0 = mb * BM + i * bw;
              const int bimg = m0 / per_img, rem = m0 - bimg * per_img;
              const int oh = rem / p.conv_ow, ow0 = rem - oh * p.conv_ow;
              tma_load_4d_g(sa + i * bw * 128, &tmA, &full_bar[stage], c0, ow0 - p.conv_pad + kw, oh - p.conv_pad + kh, bimg);
            }
          } else if (!p.a_mn) {
            tma_load_2d(sa, &tmA, &full_bar[stage], kb * bk, mb * BM);
          } else {
            for (int h = 0; h < BM / chunk; ++h)
              tma_load_2d(sa + h * (bk * 128), &tmA, &full_bar[stage], mb * BM + h * chunk, kb * bk);
          }
          if (!p.b_mn) {
            tma_load_2d(sb, &tmB, &full_bar[stage], kb * bk, nb_ * BN);
          } else {
            for (int h = 0; h < (BN + chunk - 1) / chunk; ++h)
              tma_load_2d(sb + h * (bk * 128), &tmB, &full_bar[stage], nb_ * BN + h * chunk, kb * bk);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc(p.tf32 ? 2u : 1u, BM, BN, (uint32_t)p.a_mn, (uint32_t)p.b_mn);
      // one instruction consumes 32 bytes of K: 16 bf16 or 8 tf32.  K-major: 32 bytes further inside the swizzle row;
      // MN-major: that many k-rows of 128 bytes further, chunks of MN one k-block of rows apart
      // an MN-major TF32 operand is in the 32-byte-atom form of the 128-byte swizzle (descriptor layout 1): its pattern
      // repeats every 4 k-rows, so the stride between row groups is 512 bytes instead of 1024
      const uint32_t kadv_mn = p.tf32 ? 8u * 128u : 16u * 128u, lbo_mn = p.tf32 ? 32u * 128u : 64u * 128u;
      const uint32_t sbo_mn = p.tf32 ? 512u : 1024u, lay_mn = p.tf32 ? 1u : 2u;
      const bool tf32 = p.tf32 != 0;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        if (*abort_flag || !mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, p.status, 2)) { ok = false; *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        const int split = item % p.splits;
        const int kb0 = split * p.kb_per_split, kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (*abort_flag || !mbar_wait(&full_bar[stage], phase, p.status, 3)) { ok = false; *abort_flag = 1; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: advance 32 bytes inside the 128B swizzle row; MN-major: 16 k-rows of 128 B
            const uint64_t adesc = p.a_mn ? make_smem_desc(sa + k * kadv_mn, lbo_mn, sbo_mn, lay_mn)
                                          : make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024, 2);
            const uint64_t bdesc = p.b_mn ? make_smem_desc(sb + k * kadv_mn, lbo_mn, sbo_mn, lay_mn)
                                          : make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024, 2);
            if (tf32) umma_tf32(d_tmem, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
            else umma_f16(d_tmem, adesc, bdesc, idesc, ((kb - kb0) | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
      int mb, nb_;
      const int tile = item / p.splits;
      tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb_);
      if (*abort_flag || !mbar_wait(&tfull_bar[acc], acc_phase, p.status, 4)) { ok = false; *abort_flag = 1; break; }
      tc_fence_after();
      const int row_in_tile = quarter * 32 + lane;
      const int row = mb * BM + row_in_tile;
      const bool row_ok = row < p.M;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN);
      if (p.splits == 1) {
        // rolled on purpose (one copy of the chunk body in the instruction cache); the chunk's global loads
        // (saved activation, old output) are issued one chunk ahead of their use
        EpiPrefetch pf;
        epilogue_prefetch16(p, row, nb_ * BN, row_ok, pf);
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr0 + (uint32_t)c0, r);
          const EpiPrefetch cur = pf;
          if (c0 + 16 < BN) epilogue_prefetch16(p, row, nb_ * BN + c0 + 16, row_ok, pf);
          tmem_ld_wait();
          const int col0 = nb_ * BN + c0;
          if (row_ok && col0 < p.N) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
            epilogue_store16(p, row, col0, v, cur);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      } else {
        // split-K: park the fp32 partial tile; splitk_reduce_kernel sums the splits in index order afterwards
        float* wtile = p.ws + (size_t)item * (BM * BN) + (size_t)row_in_tile * BN;
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          uint32_t r[16];
          tmem_ld_32x32b_x16(taddr0 + (uint32_t)c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; j += 4)
            *reinterpret_cast<uint4*>(wtile + c0 + j) = make_uint4(r[j], r[j + 1], r[j + 2], r[j + 3]);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------------------------------ two-CTA tiles
// The same GEMM with cta_group::2: a cluster of two CTAs (two SMs) owns one 256 x 256 output tile.  Each CTA stages 128
// rows of A and 128 of the 256 B columns; ONE thread of the leader CTA issues tcgen05.mma.cta_group::2 (M = 256,
// N = 256), which reads both CTAs' shared memory and writes rows [0,128) of the tile into the leader's tensor memory
// and rows [128,256) into the peer's.  Per SM that is half the B bytes of a 128 x 256 one-CTA tile for the same
// FLOPs, i.e. 64 instead of 96 shared-memory bytes per tensor-core clock.
//   * both CTAs' TMA loads complete on the LEADER's full barrier (cp.async.bulk.tensor with cta_group::2 may signal a
//     barrier of the peer; no multicast is used); the leader arms it with the bytes of both;
//   * tcgen05.commit with a two-CTA mask frees the stage / publishes the accumulator in both CTAs;
//   * the peer's epilogue warps release the accumulator on the leader's barrier (remote arrive).
constexpr int BN2 = 256;       // tile columns (both CTAs together)
constexpr int STAGES2 = 6;     // 6 x (16 KB A + 16 KB B) per CTA

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t mapa_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load whose completion bytes go to a barrier given as a shared::cluster address (possibly the peer CTA's)
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const void* tmap, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                              uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far have retired
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"((unsigned short)3)
               : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmParams p) {
  constexpr uint32_t A_BYTES = BM * BK * 2;            // this CTA's 128 rows of A
  constexpr uint32_t B_BYTES = (BN2 / 2) * BK * 2;     // this CTA's 128 of the 256 B columns
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 512;                  // two accumulators of 256 columns

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES2 * STAGE_BYTES);   // used in the leader only
  uint64_t* empty_bar = full_bar + STAGES2;
  uint64_t* tfull_bar = empty_bar + STAGES2;
  uint64_t* tempty_bar = tfull_bar + 2;                                             // used in the leader only
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();           // 0 = leader
  const int cluster_id = blockIdx.x >> 1, num_clusters = gridDim.x >> 1;
  const int num_tiles = p.tiles_m * p.tiles_n;       // tiles of 256 x 256

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES2; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 8);   // four epilogue warps in each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        int mb, nb_;
        tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb_);
        const int m0 = mb * (2 * BM) + (int)rank * BM;          // this CTA's rows of A
        const int n0 = nb_ * BN2 + (int)rank * (BN2 / 2);       // this CTA's columns of B
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (*abort_flag || !mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, 21)) { ok = false; *abort_flag = 1; break; }
          uint8_t* sa = smem + stage * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          const uint32_t fb = mapa_rank(smem_u32(&full_bar[stage]), 0);
          if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * STAGE_BYTES);
          if (!p.a_mn) {
            tma_load_2d_pair(sa, &tmA, fb, kb * BK, m0);
          } else {
#pragma unroll
            for (int h = 0; h < BM / 64; ++h) tma_load_2d_pair(sa + h * (64 * BK * 2), &tmA, fb, m0 + h * 64, kb * BK);
          }
          if (!p.b_mn) {
            tma_load_2d_pair(sb, &tmB, fb, kb * BK, n0);
          } else {
#pragma unroll
            for (int h = 0; h < BN2 / 128; ++h) tma_load_2d_pair(sb + h * (64 * BK * 2), &tmB, fb, n0 + h * 64, kb * BK);
          }
          if (++stage == STAGES2) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc(1u, 2 * BM, BN2, (uint32_t)p.a_mn, (uint32_t)p.b_mn);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
        if (*abort_flag || !mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, p.status, 22)) { ok = false; *abort_flag = 1; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN2);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (*abort_flag || !mbar_wait(&full_bar[stage], phase, p.status, 23)) { ok = false; *abort_flag = 1; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = p.a_mn ? make_smem_desc(sa + k * (UMMA_K * 128), 64 * BK * 2, 1024, 2)
                                          : make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024, 2);
            const uint64_t bdesc = p.b_mn ? make_smem_desc(sb + k * (UMMA_K * 128), 64 * BK * 2, 1024, 2)
                                          : make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024, 2);
            umma_f16_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);
          if (++stage == STAGES2) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[acc]);
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5 of both CTAs)
    const int quarter = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = cluster_id; tile < num_tiles && ok; tile += num_clusters) {
      int mb, nb_;
      tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb_);
      if (*abort_flag || !mbar_wait(&tfull_bar[acc], acc_phase, p.status, 24)) { ok = false; *abort_flag = 1; break; }
      tc_fence_after();
      const int row = mb * (2 * BM) + (int)rank * BM + quarter * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr0 = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * BN2);
      EpiPrefetch pf;
      epilogue_prefetch16(p, row, nb_ * BN2, row_ok, pf);
#pragma unroll 1
      for (int c0 = 0; c0 < BN2; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(taddr0 + (uint32_t)c0, r);
        const EpiPrefetch cur = pf;
        if (c0 + 16 < BN2) epilogue_prefetch16(p, row, nb_ * BN2 + c0 + 16, row_ok, pf);
        tmem_ld_wait();
        const int col0 = nb_ * BN2 + c0;
        if (row_ok && col0 < p.N) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
          epilogue_store16(p, row, col0, v, cur);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_rank(smem_u32(&tempty_bar[acc]), 0));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves (or frees tensor memory) while the other may still read or signal it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// Second phase of a split-K GEMM: one thread per (row, 16-column chunk) of the output sums that chunk over the
// splits in index order (deterministic) and runs the epilogue.  A separate launch, not a "last CTA reduces" tail:
// the serial tail cost 20 us for 18 splits, and a tail that waits for sibling CTAs could deadlock against a
// second split-K kernel running on another stream.
__global__ void __launch_bounds__(128)
splitk_reduce_kernel(const GemmParams p, int BN) {
  const int chunks = BN / 16;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)p.tiles_m * p.tiles_n * BM * chunks;
  if (idx >= total) return;
  const int c = (int)(idx % chunks);
  const int row_in_tile = (int)((idx / chunks) % BM);
  const int tile = (int)(idx / ((long long)chunks * BM));
  int mb, nb_;
  tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb_);
  const int row = mb * BM + row_in_tile, col0 = nb_ * BN + c * 16;
  if (row >= p.M || col0 >= p.N) return;
  EpiPrefetch pf;
  epilogue_prefetch16(p, row, col0, true, pf);
  const size_t tile_elems = (size_t)BM * BN;
  const float* src = p.ws + (size_t)tile * p.splits * tile_elems + (size_t)row_in_tile * BN + c * 16;
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = 0.f;
  int sp = 0;
  for (; sp + 8 <= p.splits; sp += 8) {
    float4 x[8][4];
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int j = 0; j < 4; ++j) x[u][j] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + u) * tile_elems) + j);
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[4 * j] += x[u][j].x; v[4 * j + 1] += x[u][j].y; v[4 * j + 2] += x[u][j].z; v[4 * j + 3] += x[u][j].w;
      }
  }
  for (; sp < p.splits; ++sp) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * tile_elems) + j);
      v[4 * j] += x.x; v[4 * j + 1] += x.y; v[4 * j + 2] += x.z; v[4 * j + 3] += x.w;
    }
  }
  epilogue_store16(p, row, col0, v, pf);
}

// The weight-gradient case (fp32 output, plain or accumulating, no bias / activation): one thread per FOUR output
// columns, so a 256 x 256 gradient has 16 k threads in flight instead of 4 k and every split's load of a warp is one
// contiguous 512-byte run.  Splits are still added in index order.
__global__ void __launch_bounds__(256)
splitk_reduce_f32_kernel(const GemmParams p, int BN) {
  const int quads = BN / 4;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long total = (long long)p.tiles_m * p.tiles_n * BM * quads;
  if (idx >= total) return;
  const int c = (int)(idx % quads);
  const int row_in_tile = (int)((idx / quads) % BM);
  const int tile = (int)(idx / ((long long)quads * BM));
  int mb, nb_;
  tile_coords(tile, p.tiles_m, p.tiles_n, mb, nb_);
  const int row = mb * BM + row_in_tile, col0 = nb_ * BN + c * 4;
  if (row >= p.M || col0 >= p.N) return;
  const size_t tile_elems = (size_t)BM * BN;
  const float* src = p.ws + (size_t)tile * p.splits * tile_elems + (size_t)row_in_tile * BN + c * 4;
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  int sp = 0;
  for (; sp + 8 <= p.splits; sp += 8) {
    float4 x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) x[u] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + u) * tile_elems));
#pragma unroll
    for (int u = 0; u < 8; ++u) { v.x += x[u].x; v.y += x[u].y; v.z += x[u].z; v.w += x[u].w; }
  }
  for (; sp < p.splits; ++sp) {
    const float4 x = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * tile_elems));
    v.x += x.x; v.y += x.y; v.z += x.z; v.w += x.w;
  }
  v.x *= p.alpha; v.y *= p.alpha; v.z *= p.alpha; v.w *= p.alpha;
  float* o = reinterpret_cast<float*>(p.D) + (size_t)row * p.ldd + col0;
  if (col0 + 4 <= p.N && (p.ldd % 4 == 0)) {
    if (p.accumulate) {
      const float4 y = *reinterpret_cast<const float4*>(o);
      v.x += y.x; v.y += y.y; v.z += y.z; v.w += y.w;
    }
    *reinterpret_cast<float4*>(o) = v;
  } else {
    const float e[4] = {v.x, v.y, v.z, v.w};
    for (int j = 0; j < 4; ++j)
      if (col0 + j < p.N) o[j] = p.accumulate ? o[j] + e[j] : e[j];
  }
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

// 2-D bf16 tensor map: inner extent `inner` (contiguous), outer extent `outer`, row pitch `ld` elements.
// `mn_major` matters for 32-bit elements only: an MN-major TF32 operand has to use the 128-byte swizzle with 32-byte
// atoms (two-bit XOR of the 32-byte chunk index with the row index modulo 4); every other operand uses the 16-byte-atom form
int make_tmap_elt(CUtensorMap* tm, const void* base, long long inner, long long outer, long long ld, int box_inner,
                  int box_outer, int elt_bytes, int mn_major = 0) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return NB_ERR_NO_DRIVER_SYMBOL;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * elt_bytes) & 15)) return NB_ERR_UNALIGNED;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * elt_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  // fp32 operands are loaded as TFLOAT32: the copy rounds them to the 10-bit mantissa the tensor core reads
  CUresult r = enc(tm, elt_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   (elt_bytes == 4 && mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NB_OK : NB_ERR_TENSORMAP;
}
int make_tmap_bf16(CUtensorMap* tm, const void* base, long long inner, long long outer, long long ld, int box_inner,
                   int box_outer) {
  return make_tmap_elt(tm, base, inner, outer, ld, box_inner, box_outer, 2);
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

template <int BN, int STAGES>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, long long ws_bytes, int ws_tiles_cap,
           cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 /*align*/ + 256 /*barriers*/;
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  p.tiles_m = ceil_div(p.M, BM);
  p.tiles_n = ceil_div(p.N, BN);
  p.num_kb = ceil_div(p.K, p.tf32 ? BK / 2 : BK);
  const int tiles = p.tiles_m * p.tiles_n;
  // split-K when the tile count leaves most SMs idle and K is deep: each split keeps >= 4 k-blocks
  int splits = 1;
  if (p.ws && p.tile_ctr && tiles * 2 <= sm_count() && p.num_kb >= 8 && tiles <= ws_tiles_cap) {
    splits = sm_count() / tiles;
    if (splits > p.num_kb / 4) splits = p.num_kb / 4;
    const long long cap = ws_bytes / ((long long)tiles * BM * BN * 4);
    if (splits > cap) splits = (int)cap;
    if (splits < 1) splits = 1;
  }
  p.kb_per_split = ceil_div(p.num_kb, splits);
  p.splits = ceil_div(p.num_kb, p.kb_per_split);
  const int items = tiles * p.splits;
  const int grid = items < sm_count() ? items : sm_count();
  gemm_bf16_kernel<BN, STAGES><<<grid, NUM_THREADS, smem, stream>>>(tmA, tmB, p);
  NB_LAUNCH_CHECK();
  if (p.splits > 1) {
    if (p.out_f32 && !p.bias && !p.act && !p.dact) {
      const long long threads = (long long)tiles * BM * (BN / 4);
      splitk_reduce_f32_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(p, BN);
    } else {
      const long long threads = (long long)tiles * BM * (BN / 16);
      splitk_reduce_kernel<<<(unsigned)((threads + 127) / 128), 128, 0, stream>>>(p, BN);
    }
    NB_LAUNCH_CHECK();
  }
  return NB_OK;
}

int launch_two_cta(const CUtensorMap& tmA, const CUtensorMap& tmB, GemmParams& p, cudaStream_t stream) {
  constexpr size_t smem = (size_t)STAGES2 * (BM * BK * 2 + (BN2 / 2) * BK * 2) + 1024 /*align*/ + 256 /*barriers*/;
  static_assert(smem <= 232448, "shared memory budget of one CTA");
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(gemm2_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  p.tiles_m = ceil_div(p.M, 2 * BM);
  p.tiles_n = ceil_div(p.N, BN2);
  p.num_kb = ceil_div(p.K, BK);
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  const int tiles = p.tiles_m * p.tiles_n;
  const int clusters = tiles < sm_count() / 2 ? tiles : sm_count() / 2;
  gemm2_bf16_kernel<<<2 * clusters, NUM_THREADS, smem, stream>>>(tmA, tmB, p);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int g_two_cta_mode = 0;  // 0 = by problem size, 1 = never, 2 = whenever the shape allows it

}  // namespace

extern "C" {

// Selects between one-CTA tiles and two-CTA (cta_group::2) 256 x 256 tiles; returns the previous setting.
int nb_gemm_two_cta_mode(int mode) {
  const int old = g_two_cta_mode;
  if (mode >= 0 && mode <= 2) g_two_cta_mode = mode;
  return old;
}

// D[M,N] = epi(alpha * A·B).  A: a_mn=0 → [M,K] row-major (lda = pitch of a row of K), a_mn=1 → [K,M]
// row-major (lda = pitch of a row of M).  B: b_mn=0 → [N,K] row-major, b_mn=1 → [K,N] row-major.
// Pitches in elements; every pitch*2 bytes and every base must be 16-byte aligned (TMA).
static int gemm_any(int tf32, const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd, int a_mn,
                    int b_mn, int out_f32, int accumulate, float alpha, const float* bias, int act, const void* aux,
                    int ld_aux, int dact, unsigned int* status, int bn_hint, void* workspace, long long workspace_bytes,
                    void* stream) {
  if (M <= 0 || N <= 0 || K <= 0) return NB_ERR_BAD_ARG;
  const int elt = tf32 ? 4 : 2, bk = 128 / elt;   // elements per 128-byte row = k-block depth = MN-major chunk width
  if (accumulate && !out_f32) return NB_ERR_BAD_ARG;
  if (dact && !aux) return NB_ERR_BAD_ARG;
  int BN = bn_hint;
  if (BN == 0) {
    // widest tile that still gives every SM work; MN-major B needs whole 64-column boxes
    BN = 128;
    const long long t128 = (long long)ceil_div(M, BM) * ceil_div(N, 128);
    if (N <= 64 || t128 < sm_count()) BN = 64;
    if (N >= 256 && (long long)ceil_div(M, BM) * ceil_div(N, 256) >= 2LL * sm_count()) BN = 256;
    if (!b_mn) {
      if (N <= 16) BN = 16;
      else if (N <= 32) BN = 32;
    }
  }
  if (b_mn && BN < bk) BN = bk;
  // two-CTA tiles once the 256 x 256 tiles keep about two thirds of the SM pairs busy (measured: 2048 x 2048 x 16384,
  // 64 tiles on 74 pairs, runs 1.74x faster this way than as split-K one-CTA tiles)
  bool two_cta = false;
  if (!tf32 && bn_hint == 0 && g_two_cta_mode != 1 && M >= 256 && N >= 256 && K >= 128) {
    const long long t2 = (long long)ceil_div(M, 2 * BM) * ceil_div(N, BN2);
    two_cta = g_two_cta_mode == 2 || t2 * 3 >= (long long)sm_count();
  }
  if (two_cta) BN = BN2 / 2;   // the B box of one CTA
  CUtensorMap tmA, tmB;
  int rc;
  if (!a_mn) rc = make_tmap_elt(&tmA, A, K, M, lda, bk, BM, elt);
  else rc = make_tmap_elt(&tmA, A, M, K, lda, bk, bk, elt, 1);
  if (rc) return rc;
  if (!b_mn) rc = make_tmap_elt(&tmB, B, K, N, ldb, bk, BN, elt);
  else rc = make_tmap_elt(&tmB, B, N, K, ldb, bk, bk, elt, 1);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.a_mn = a_mn; p.b_mn = b_mn; p.tf32 = tf32;
  p.ldd = ldd; p.ld_aux = ld_aux;
  p.out_f32 = out_f32; p.accumulate = accumulate; p.act = act; p.dact = dact;
  p.alpha = alpha;
  p.D = D; p.bias = bias; p.aux = (const __nv_bfloat16*)aux; p.status = status;
  p.conv = 0;
  // workspace layout: [NB_GEMM_WS_COUNTERS u32 tile counters (zero at rest)] [fp32 partial tiles]
  long long ws_bytes = 0;
  p.ws = nullptr;
  p.tile_ctr = nullptr;
  if (workspace && workspace_bytes > NB_GEMM_WS_COUNTERS * 4 + (1 << 20)) {
    p.tile_ctr = (unsigned int*)workspace;
    p.ws = (float*)((char*)workspace + NB_GEMM_WS_COUNTERS * 4);
    ws_bytes = workspace_bytes - NB_GEMM_WS_COUNTERS * 4;
  }
  cudaStream_t s = (cudaStream_t)stream;
  if (two_cta) return launch_two_cta(tmA, tmB, p, s);
  switch (BN) {
    case 256: return launch<256, 4>(tmA, tmB, p, ws_bytes, NB_GEMM_WS_COUNTERS, s);
    case 128: return launch<128, 6>(tmA, tmB, p, ws_bytes, NB_GEMM_WS_COUNTERS, s);
    case 64: return launch<64, 8>(tmA, tmB, p, ws_bytes, NB_GEMM_WS_COUNTERS, s);
    case 32: return launch<32, 8>(tmA, tmB, p, ws_bytes, NB_GEMM_WS_COUNTERS, s);
    case 16: return launch<16, 8>(tmA, tmB, p, ws_bytes, NB_GEMM_WS_COUNTERS, s);
    default: return NB_ERR_BAD_ARG;
  }
}

int nb_gemm_bf16(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd, int a_mn,
                 int b_mn, int out_f32, int accumulate, float alpha, const float* bias, int act, const void* aux,
                 int ld_aux, int dact, unsigned int* status, int bn_hint, void* workspace, long long workspace_bytes,
                 void* stream) {
  return gemm_any(0, A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, accumulate, alpha, bias, act, aux, ld_aux, dact,
                  status, bn_hint, workspace, workspace_bytes, stream);
}
// The same contraction on fp32 operands read as TF32 (10-bit mantissa, fp32 accumulation): `kind::tf32`, one-CTA tiles.
// Pitches in fp32 elements (multiples of 4); `aux` stays a bf16 tensor.
int nb_gemm_tf32(const void* A, const void* B, void* D, int M, int N, int K, int lda, int ldb, int ldd, int a_mn,
                 int b_mn, int out_f32, int accumulate, float alpha, const float* bias, int act, const void* aux,
                 int ld_aux, int dact, unsigned int* status, int bn_hint, void* workspace, long long workspace_bytes,
                 void* stream) {
  return gemm_any(1, A, B, D, M, N, K, lda, ldb, ldd, a_mn, b_mn, out_f32, accumulate, alpha, bias, act, aux, ld_aux, dact,
                  status, bn_hint, workspace, workspace_bytes, stream);
}

// Implicit-GEMM convolution forward, stride 1: y[B·OH·OW, OC] = epi(patches(x) · W), x NHWC bf16 [B, H, W, C] with
// C % 64 == 0, W in GEMM layout [KH·KW·C, OC] (row pitch ldw).  OW must have a power-of-two factor bw >= 8 (the run
// length of one TMA box).  Output spatial size: OH = H + 2·pad − KH + 1, OW likewise.
int nb_conv_implicit_fwd(const void* x, const void* Wt, void* y, int B, int H, int Wd, int C, int OC, int KH, int KW, int pad,
                         int ldw, int ldy, const float* bias, int act, const void* residual, int ld_res,
                         unsigned int* status, void* stream) {
  const int OH = H + 2 * pad - KH + 1, OW = Wd + 2 * pad - KW + 1;
  if (B <= 0 || OH <= 0 || OW <= 0 || C % 64 || OC <= 0) return NB_ERR_BAD_ARG;
  int bw = 1;
  while (bw < 128 && OW % (bw * 2) == 0) bw *= 2;
  if (bw < 8) return NB_ERR_BAD_ARG;   // every box then starts on a 1024-byte swizzle atom of the A tile
  EncodeTiledFn enc = get_encode();
  if (!enc) return NB_ERR_NO_DRIVER_SYMBOL;
  if (reinterpret_cast<uintptr_t>(x) & 15) return NB_ERR_UNALIGNED;
  CUtensorMap tmA, tmB;
  {
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Wd, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)Wd * C * 2, (cuuint64_t)H * Wd * C * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)bw, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return NB_ERR_TENSORMAP;
  }
  const int M = B * OH * OW, K = KH * KW * C;
  int BN = 128;
  if (OC <= 64 || (long long)ceil_div(M, BM) * ceil_div(OC, 128) < sm_count()) BN = 64;
  int rc = make_tmap_bf16(&tmB, Wt, OC, K, ldw, 64, BK);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = OC; p.K = K;
  p.a_mn = 0; p.b_mn = 1; p.tf32 = 0;
  p.ldd = ldy; p.ld_aux = ld_res;
  p.out_f32 = 0; p.accumulate = 0; p.act = act; p.dact = residual ? NB_AUX_ADD : 0;
  p.alpha = 1.f;
  p.D = y; p.bias = bias; p.aux = (const __nv_bfloat16*)residual; p.status = status;
  p.ws = nullptr; p.tile_ctr = nullptr;
  p.conv = 1; p.conv_c = C; p.conv_ow = OW; p.conv_oh = OH; p.conv_kw = KW; p.conv_pad = pad; p.conv_bw = bw;
  p.conv_taps = KH * KW; p.conv_b = B;
  cudaStream_t s = (cudaStream_t)stream;
  if (BN == 128) return launch<128, 6>(tmA, tmB, p, 0, 0, s);
  return launch<64, 8>(tmA, tmB, p, 0, 0, s);
}


// Implicit-GEMM weight gradient of a stride-1 convolution: dW[KH·KW·C, OC] (+)= patches(x)^T · dy without the patch
// matrix.  x NHWC bf16 [B, H, W, C], C % 64 == 0; dy bf16 [B·OH·OW, OC] (row pitch ld_dy); dW fp32 (row pitch ld_dw), the
// result is ADDED to it.  OW needs a power-of-two factor bw in [8, 64].  Split-K over the pixels through `workspace`.
int nb_conv_implicit_wgrad(const void* x, const void* dy, float* dW, int B, int H, int Wd, int C, int OC, int KH, int KW, int pad,
                           int ld_dy, int ld_dw, unsigned int* status, void* workspace, long long workspace_bytes, void* stream) {
  const int OH = H + 2 * pad - KH + 1, OW = Wd + 2 * pad - KW + 1;
  if (B <= 0 || OH <= 0 || OW <= 0 || C % 64 || OC <= 0) return NB_ERR_BAD_ARG;
  int bw = 1;
  while (bw < 64 && OW % (bw * 2) == 0) bw *= 2;
  if (bw < 8) return NB_ERR_BAD_ARG;
  EncodeTiledFn enc = get_encode();
  if (!enc) return NB_ERR_NO_DRIVER_SYMBOL;
  if (reinterpret_cast<uintptr_t>(x) & 15) return NB_ERR_UNALIGNED;
  CUtensorMap tmA, tmB;
  {
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Wd, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t strides[3] = {(cuuint64_t)C * 2, (cuuint64_t)Wd * C * 2, (cuuint64_t)H * Wd * C * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)bw, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
      return NB_ERR_TENSORMAP;
  }
  const int Mpix = B * OH * OW, Kc = KH * KW * C;
  int BN = 128;
  if (OC <= 64 || (long long)ceil_div(Kc, BM) * ceil_div(OC, 128) * 2 < sm_count()) BN = 64;
  int rc = make_tmap_bf16(&tmB, dy, OC, Mpix, ld_dy, 64, BK);
  if (rc) return rc;
  GemmParams p;
  p.M = Kc; p.N = OC; p.K = Mpix;
  p.a_mn = 1; p.b_mn = 1; p.tf32 = 0;
  p.ldd = ld_dw; p.ld_aux = 0;
  p.out_f32 = 1; p.accumulate = 1; p.act = 0; p.dact = 0;
  p.alpha = 1.f;
  p.D = dW; p.bias = nullptr; p.aux = nullptr; p.status = status;
  p.ws = nullptr; p.tile_ctr = nullptr;
  long long ws_bytes = 0;
  if (workspace && workspace_bytes > NB_GEMM_WS_COUNTERS * 4 + (1 << 20)) {
    p.tile_ctr = (unsigned int*)workspace;
    p.ws = (float*)((char*)workspace + NB_GEMM_WS_COUNTERS * 4);
    ws_bytes = workspace_bytes - NB_GEMM_WS_COUNTERS * 4;
  }
  p.conv = 2; p.conv_c = C; p.conv_ow = OW; p.conv_oh = OH; p.conv_kw = KW; p.conv_pad = pad; p.conv_bw = bw;
  p.conv_taps = KH * KW; p.conv_b = B;
  cudaStream_t s = (cudaStream_t)stream;
  if (BN == 128) return launch<128, 6>(tmA, tmB, p, ws_bytes, NB_GEMM_WS_COUNTERS, s);
  return launch<64, 8>(tmA, tmB, p, ws_bytes, NB_GEMM_WS_COUNTERS, s);
}

}  // extern "C"
