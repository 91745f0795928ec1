// Fused forward of a three-layer MLP  out = (act(act(X W1 + b1) W2 + b2)) W3 + b3  with hidden width 256:
// one CTA per 128 rows keeps the hidden activations on chip — TMEM accumulators, bf16 A-operand tile in shared
// memory — so the actor / critic forward of the RL trainers is ONE launch instead of three GEMM launches whose
// run time is launch latency and pipeline fill (13 us each for 16384 x 256 x 256).  The hidden activations are
// optionally written to global memory (bf16) for the backward pass.
//   warp 0      TMA: X tile and W1, then W2 in four 64-row k-blocks through a 2-stage ring
//   warp 1      MMA issuer: layer 1 (K <= 64), layer 2 (K = 256, N = 256), layer 3 (K = 256, N = 16)
//   warps 2..9  epilogue: two warps per TMEM lane quarter, each takes half of the 256 columns of its 32 rows; bias +
//               activation, bf16 tile for the next layer in the 128-byte-swizzled K-major layout, final fp32 output;
//               also stage W3ᵀ into shared memory at start
// Weights are [IN, OUT] row-major bf16 (the framework's Linear layout): W1, W2 are MN-major B operands, W3 (narrow,
// OUT <= 16) is transposed into a K-major tile by the epilogue threads.
// Reference counterpart: none as one kernel (the reference issues cuBLAS GEMMs + bias / activation kernels per layer,
// noeira/nn/primitives/linear.mojo:1295-1387); the captured actor step it optimises is noeira_max/README.md's
// "MLP actor inference 17-256-256-6: 21.5 us eager / 12.7 captured".
#include <cuda.h>
#include <string.h>

#include "common.cuh"
#include "gemm_api.h"

namespace {
using namespace nb;

constexpr int HID = 256;
constexpr int ROWS = 128;
constexpr int N3P = 16;
constexpr int MLP_THREADS = 320;   // warp 0 TMA, warp 1 MMA, warps 2..9 epilogue (two warps per TMEM lane quarter)
constexpr int EPI_THREADS = 256;

struct MlpParams {
  int M, k0, n3;            // rows, input width (<= 64), real output width (<= 16)
  int ld_w3, ld_out, ld_h;  // pitches in elements
  int act;                  // NB_ACT_TANH or NB_ACT_RELU
  const __nv_bfloat16* w3;  // [HID, ld_w3]
  const float *b1, *b2, *b3;
  float* out;               // [M, ld_out] fp32
  __nv_bfloat16 *h1, *h2;   // optional [M, ld_h] saves
  unsigned int* status;
};

__device__ __forceinline__ float act1(int act, float v) {
  if (act == NB_ACT_TANH) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(v));
    return y;
  }
  return fmaxf(v, 0.f);
}

struct MlpMaps {
  CUtensorMap x, w1, w2;
};
struct MlpGroup {
  MlpMaps maps[2];
  MlpParams prm[2];
};

// blockIdx.y selects the network: the actor and the critic of an RL update run in ONE launch.
__global__ void __launch_bounds__(MLP_THREADS, 1)
mlp3_fwd_kernel(const __grid_constant__ MlpGroup grp) {
  const MlpParams& p = grp.prm[blockIdx.y];
  const CUtensorMap& tmX = grp.maps[blockIdx.y].x;
  const CUtensorMap& tmW1 = grp.maps[blockIdx.y].w1;
  const CUtensorMap& tmW2 = grp.maps[blockIdx.y].w2;
  if ((int)blockIdx.x * ROWS >= p.M) return;
  constexpr uint32_t X_BYTES = ROWS * 64 * 2;        // 16 KB
  constexpr uint32_t W1_BYTES = 64 * HID * 2;        // 32 KB (64 k-rows x 256)
  constexpr uint32_t W2_STAGE = 64 * HID * 2;        // 32 KB per k-block
  constexpr uint32_t H_BYTES = ROWS * HID * 2;       // 64 KB, four k-blocks of 16 KB
  constexpr uint32_t W3_BYTES = N3P * HID * 2;       // 8 KB, four k-blocks of 2 KB
  constexpr uint32_t TMEM_COLS = 512;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sX = smem;
  uint8_t* sW1 = sX + X_BYTES;
  uint8_t* sW2 = sW1 + W1_BYTES;            // 2 stages
  uint8_t* sH = sW2 + 2 * W2_STAGE;
  uint8_t* sW3 = sH + H_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sW3 + W3_BYTES);
  uint64_t* x_full = bars;
  uint64_t* w2_full = bars + 1;    // [2]
  uint64_t* w2_empty = bars + 3;   // [2]
  uint64_t* acc_full = bars + 5;   // [3]
  uint64_t* h_ready = bars + 8;    // [2]
  uint64_t* w3_ready = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * ROWS;

  if (threadIdx.x == 0) {
    mbar_init(x_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&w2_full[i], 1);
      mbar_init(&w2_empty[i], 1);
      mbar_init(&h_ready[i], 8);
    }
    for (int i = 0; i < 3; ++i) mbar_init(&acc_full[i], 1);
    mbar_init(w3_ready, 8);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmX);
    prefetch_tensormap(&tmW1);
    prefetch_tensormap(&tmW2);
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
      mbar_expect_tx(x_full, X_BYTES + W1_BYTES);
      tma_load_2d(sX, &tmX, x_full, 0, row0);                                   // box {64 k, 128 rows}, zero fill past k0 / M
      for (int h = 0; h < HID / 64; ++h) tma_load_2d(sW1 + h * 8192, &tmW1, x_full, h * 64, 0);   // boxes {64 n, 64 k}
      for (int kb = 0; kb < HID / 64; ++kb) {
        const int st = kb & 1;
        if (*abort_flag || !mbar_wait(&w2_empty[st], ((uint32_t)(kb >> 1) & 1u) ^ 1u, p.status, 301)) { *abort_flag = 1; break; }
        mbar_expect_tx(&w2_full[st], W2_STAGE);
        for (int h = 0; h < HID / 64; ++h) tma_load_2d(sW2 + st * W2_STAGE + h * 8192, &tmW2, &w2_full[st], h * 64, kb * 64);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc_h = make_idesc(1u, ROWS, HID, 0u, 1u);   // A K-major, B (weights) MN-major, N = 256
      const uint32_t idesc_o = make_idesc(1u, ROWS, N3P, 0u, 0u);   // W3ᵀ staged K-major, N = 16
      bool ok = mbar_wait(x_full, 0u, p.status, 310);
      if (ok) {
        tc_fence_after();
        const uint32_t xa = smem_u32(sX), wb = smem_u32(sW1);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_base, make_smem_desc(xa + k * 32, 16, 1024, 2), make_smem_desc(wb + k * (16 * 128), 8192, 1024, 2),
                   idesc_h, k != 0 ? 1u : 0u);
        umma_commit(&acc_full[0]);
      }
      if (ok) ok = mbar_wait(&h_ready[0], 0u, p.status, 311);
      for (int kb = 0; kb < HID / 64 && ok; ++kb) {
        const int st = kb & 1;
        if (!mbar_wait(&w2_full[st], (uint32_t)(kb >> 1) & 1u, p.status, 312)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ha = smem_u32(sH + kb * 16384), wb = smem_u32(sW2 + st * W2_STAGE);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_base + 256, make_smem_desc(ha + k * 32, 16, 1024, 2),
                   make_smem_desc(wb + k * (16 * 128), 8192, 1024, 2), idesc_h, (kb | k) != 0 ? 1u : 0u);
        umma_commit(&w2_empty[st]);
      }
      if (ok) umma_commit(&acc_full[1]);
      if (ok) ok = mbar_wait(&h_ready[1], 0u, p.status, 313) && mbar_wait(w3_ready, 0u, p.status, 314);
      if (ok) {
        tc_fence_after();
        for (int kb = 0; kb < HID / 64; ++kb) {
          const uint32_t ha = smem_u32(sH + kb * 16384), wb = smem_u32(sW3 + kb * 2048);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16(tmem_base, make_smem_desc(ha + k * 32, 16, 1024, 2), make_smem_desc(wb + k * 32, 16, 1024, 2), idesc_o,
                     (kb | k) != 0 ? 1u : 0u);
        }
        umma_commit(&acc_full[2]);
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;             // which 128 columns of the 256 this warp handles
    const int r = quarter * 32 + lane;            // row of the tile = TMEM lane
    const int row = row0 + r;
    const int t = (warp - 2) * 32 + lane;         // 0..255 for cooperative loads
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    // ---- stage W3ᵀ: element (n, k) of the K-major [16 x 256] tile
    for (int e = t; e < N3P * HID; e += EPI_THREADS) {
      const int k = e / N3P, n = e - k * N3P;
      const __nv_bfloat16 v = (n < p.n3) ? p.w3[(size_t)k * p.ld_w3 + n] : __float2bfloat16(0.f);
      const int kb = k >> 6, kk = k & 63;
      uint8_t* dst = sW3 + kb * 2048 + (n >> 3) * 1024 + (n & 7) * 128 + ((((kk >> 3) ^ (n & 7))) << 4) + (kk & 7) * 2;
      *reinterpret_cast<__nv_bfloat16*>(dst) = v;
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(w3_ready);
    bool ok = true;
    uint8_t* hrow = sH + (r >> 3) * 1024 + (r & 7) * 128;
    for (int layer = 0; layer < 2 && ok; ++layer) {
      if (!__all_sync(0xffffffffu, !*abort_flag && mbar_wait(&acc_full[layer], 0u, p.status, 320 + layer))) { ok = false; break; }
      tc_fence_after();
      const float* bias = layer == 0 ? p.b1 : p.b2;
      __nv_bfloat16* hsave = layer == 0 ? p.h1 : p.h2;
      const uint32_t acc = lane_addr + (uint32_t)(layer * 256 + half * 128);
      // 32 columns per step, two register sets in ping-pong: the next step's TMEM load is in flight while this one is
      // converted and stored.  Written out as four steps (no loop-carried register copy may sit before a wait).
      auto process = [&](const uint32_t (&cur)[32], int s4) {
        const int c0 = half * 128 + s4 * 32;
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          const float4 bv = bias ? __ldg(reinterpret_cast<const float4*>(bias + c0 + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
          __nv_bfloat162 a = __floats2bfloat162_rn(act1(p.act, __uint_as_float(cur[j]) + bv.x),
                                                   act1(p.act, __uint_as_float(cur[j + 1]) + bv.y));
          __nv_bfloat162 b = __floats2bfloat162_rn(act1(p.act, __uint_as_float(cur[j + 2]) + bv.z),
                                                   act1(p.act, __uint_as_float(cur[j + 3]) + bv.w));
          pk[j / 2] = *reinterpret_cast<uint32_t*>(&a);
          pk[j / 2 + 1] = *reinterpret_cast<uint32_t*>(&b);
        }
        // k-block of the next layer's A tile = c0 / 64; 16-byte chunk index inside the 128-byte row is XOR-swizzled
        const int kb = c0 >> 6, ch = (c0 & 63) >> 3;
        uint8_t* base = hrow + kb * 16384;
#pragma unroll
        for (int q = 0; q < 4; ++q)
          *reinterpret_cast<uint4*>(base + (((ch + q) ^ (r & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        if (hsave && row < p.M) {
          uint4* g = reinterpret_cast<uint4*>(hsave + (size_t)row * p.ld_h + c0);
#pragma unroll
          for (int q = 0; q < 4; ++q) g[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      };
      uint32_t ra[32], rb[32];
      tmem_ld_32x32b_x32_nowait(acc, ra);
      tmem_ld_wait();
      tmem_ld_32x32b_x32_nowait(acc + 32u, rb);
      process(ra, 0);
      tmem_ld_wait();
      tmem_ld_32x32b_x32_nowait(acc + 64u, ra);
      process(rb, 1);
      tmem_ld_wait();
      tmem_ld_32x32b_x32_nowait(acc + 96u, rb);
      process(ra, 2);
      tmem_ld_wait();
      process(rb, 3);
      tc_fence_before();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&h_ready[layer]);
    }
    if (ok && !__all_sync(0xffffffffu, !*abort_flag && mbar_wait(&acc_full[2], 0u, p.status, 322))) ok = false;
    if (ok && half == 0) {
      tc_fence_after();
      uint32_t rr[16];
      tmem_ld_32x32b_x16(lane_addr, rr);
      tmem_ld_wait();
      if (row < p.M) {
        for (int j = 0; j < p.n3; ++j) p.out[(size_t)row * p.ld_out + j] = __uint_as_float(rr[j]) + (p.b3 ? p.b3[j] : 0.f);
      }
    }
    if (!ok) *abort_flag = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}
int tmap2d(CUtensorMap* tm, const void* base, long long inner, long long outer, long long ld, int box_inner, int box_outer) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return NB_ERR_NO_DRIVER_SYMBOL;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((ld * 2) & 15)) return NB_ERR_UNALIGNED;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  return enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS ? NB_OK : NB_ERR_TENSORMAP;
}

// ------------------------------------------------------------------------------------------ backward (data gradients)
// G2 = (dY W3ᵀ) ⊙ f'(h2),  G1 = (G2 W2ᵀ) ⊙ f'(h1)  for one 128-row tile per CTA, both chained on chip: the first
// product has K = 16 (one tcgen05.mma), its result is multiplied by the activation derivative taken from the saved
// h2, written out in bf16 (the weight-gradient GEMMs read it) and kept in shared memory as the A operand of the second
// product.  G1 and G2 are the gradients with respect to the layers' PRE-activations, i.e. exactly the operands of
// dW1 = Xᵀ G1, dW2 = h1ᵀ G2, dW3 = h2ᵀ dY and of the bias column sums.  The first layer's input gradient is not needed.
// The bias gradients ride along: every CTA sums the columns of its dY, G2 and G1 tiles out of shared memory and
// writes the three partial rows; a small second kernel adds the partials in CTA order (deterministic).
//   warp 0      TMA: W2 as a K-major B operand (box 64 k x 256 n per k-block), 2-stage ring
//   warp 1      MMA issuer
//   warps 2..9  stage dY and W3 (zero padded to K = 64) into swizzled tiles; epilogues (two warps per TMEM lane
//               quarter, half of the columns each); column sums
struct MlpBwdParams {
  int M, n3;
  int ld_dy, ld_w3, ld_h, ld_g;
  int act;
  const __nv_bfloat16 *dy, *w3, *h1, *h2;
  __nv_bfloat16 *g1, *g2;
  float* bias_part;   // optional [gridDim.x][3][256]: this CTA's column sums of g1, g2, dy (bias gradients, unreduced)
  unsigned int* status;
};
struct MlpBwdGroup {
  CUtensorMap w2[2];
  MlpBwdParams prm[2];
};

// Sum of column `col` over the 128 rows of a [128 x 256] bf16 tile in the swizzled K-major layout (four k-blocks of
// 16 KB; row r of a k-block at (r>>3)·1024 + (r&7)·128, 16-byte chunk c at position c ^ (r&7)).
__device__ __forceinline__ float tile_colsum(const uint8_t* tile, int col) {
  const uint8_t* kb = tile + (col >> 6) * 16384;
  const int ch = (col & 63) >> 3, within = (col & 7) * 2;
  float acc = 0.f;
#pragma unroll 8
  for (int r = 0; r < ROWS; ++r)
    acc += __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(kb + (r >> 3) * 1024 + (r & 7) * 128 + ((ch ^ (r & 7)) << 4) + within));
  return acc;
}

__device__ __forceinline__ float dact1(int act, float h) { return act == NB_ACT_TANH ? 1.f - h * h : (h > 0.f ? 1.f : 0.f); }

__global__ void __launch_bounds__(MLP_THREADS, 1)
mlp3_bwd_kernel(const __grid_constant__ MlpBwdGroup grp) {
  const MlpBwdParams& p = grp.prm[blockIdx.y];
  const CUtensorMap& tmW2 = grp.w2[blockIdx.y];
  if ((int)blockIdx.x * ROWS >= p.M) return;
  constexpr uint32_t DY_BYTES = ROWS * 64 * 2;       // 16 KB: A tile [128 x 64] K-major, columns >= n3 zero
  constexpr uint32_t W3_BYTES = HID * 64 * 2;        // 32 KB: B tile [256 n x 64 k] K-major, columns >= n3 zero
  constexpr uint32_t W2_STAGE = HID * 64 * 2;        // 32 KB per k-block: [256 n x 64 k] K-major
  constexpr uint32_t G_BYTES = ROWS * HID * 2;       // 64 KB: G2 as the next A operand, four k-blocks of 16 KB
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sDY = smem;
  uint8_t* sW3 = sDY + DY_BYTES;
  uint8_t* sW2 = sW3 + W3_BYTES;            // 2 stages
  uint8_t* sG = sW2 + 2 * W2_STAGE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sG + G_BYTES);
  uint64_t* w2_full = bars;        // [2]
  uint64_t* w2_empty = bars + 2;   // [2]
  uint64_t* acc_full = bars + 4;   // [2]
  uint64_t* staged = bars + 6;     // dY and W3 tiles written (4 warps)
  uint64_t* g_ready = bars + 7;    // G2 tile written (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * ROWS;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&w2_full[i], 1);
      mbar_init(&w2_empty[i], 1);
      mbar_init(&acc_full[i], 1);
    }
    mbar_init(staged, 8);
    mbar_init(g_ready, 8);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tensormap(&tmW2);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      for (int kb = 0; kb < HID / 64; ++kb) {
        const int st = kb & 1;
        if (*abort_flag || !mbar_wait(&w2_empty[st], ((uint32_t)(kb >> 1) & 1u) ^ 1u, p.status, 331)) { *abort_flag = 1; break; }
        mbar_expect_tx(&w2_full[st], W2_STAGE);
        // B(n, k) of G2 W2ᵀ is W2[n, k]: row n of the [IN, OUT] matrix, 64 consecutive columns
        tma_load_2d(sW2 + st * W2_STAGE, &tmW2, &w2_full[st], kb * 64, 0);
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc(1u, ROWS, HID, 0u, 0u);   // both operands K-major, N = 256
      bool ok = mbar_wait(staged, 0u, p.status, 340);
      if (ok) {
        tc_fence_after();
        umma_f16(tmem_base, make_smem_desc(smem_u32(sDY), 16, 1024, 2), make_smem_desc(smem_u32(sW3), 16, 1024, 2), idesc, 0u);
        umma_commit(&acc_full[0]);
        ok = mbar_wait(g_ready, 0u, p.status, 341);
      }
      for (int kb = 0; kb < HID / 64 && ok; ++kb) {
        const int st = kb & 1;
        if (!mbar_wait(&w2_full[st], (uint32_t)(kb >> 1) & 1u, p.status, 342)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ga = smem_u32(sG + kb * 16384), wb = smem_u32(sW2 + st * W2_STAGE);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16(tmem_base + 256, make_smem_desc(ga + k * 32, 16, 1024, 2), make_smem_desc(wb + k * 32, 16, 1024, 2), idesc,
                   (kb | k) != 0 ? 1u : 0u);
        umma_commit(&w2_empty[st]);
      }
      if (ok) umma_commit(&acc_full[1]);
      if (!ok) *abort_flag = 1;
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;             // which 128 columns of the 256 this warp handles
    const int r = quarter * 32 + lane;            // row of the tile = TMEM lane
    const int row = row0 + r;
    const int t = (warp - 2) * 32 + lane;         // 0..255
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
    // ---- stage dY (threads 0..127: one row each) and W3 (one row of the 256 each)
    if (t < ROWS) {
      const int rr = t, grow_ = row0 + rr;
      uint4 c[2] = {zero4, zero4};
      if (grow_ < p.M) {
        const __nv_bfloat16* src = p.dy + (size_t)grow_ * p.ld_dy;
        __nv_bfloat16 v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = j < p.n3 ? src[j] : __float2bfloat16(0.f);
        c[0] = *reinterpret_cast<uint4*>(&v[0]);
        c[1] = *reinterpret_cast<uint4*>(&v[8]);
      }
      uint8_t* dst = sDY + (rr >> 3) * 1024 + (rr & 7) * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(dst + ((ch ^ (rr & 7)) << 4)) = ch < 2 ? c[ch] : zero4;
    }
    {
      const int n = t;
      const __nv_bfloat16* src = p.w3 + (size_t)n * p.ld_w3;
      __nv_bfloat16 v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = j < p.n3 ? src[j] : __float2bfloat16(0.f);
      uint8_t* dst = sW3 + (n >> 3) * 1024 + (n & 7) * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch)
        *reinterpret_cast<uint4*>(dst + ((ch ^ (n & 7)) << 4)) = ch < 2 ? *reinterpret_cast<uint4*>(&v[ch * 8]) : zero4;
    }
    fence_proxy_async();
    __syncwarp();
    if (lane == 0) mbar_arrive(staged);
    float* part = p.bias_part ? p.bias_part + (size_t)blockIdx.x * 3 * HID : nullptr;
    if (part) {
      asm volatile("bar.sync 1, 256;" ::: "memory");   // every row of the dY tile is in shared memory
      if (t < N3P) part[2 * HID + t] = tile_colsum(sDY, t);
    }
    bool ok = true;
    uint8_t* grow = sG + (r >> 3) * 1024 + (r & 7) * 128;
    for (int layer = 0; layer < 2 && ok; ++layer) {
      if (!__all_sync(0xffffffffu, !*abort_flag && mbar_wait(&acc_full[layer], 0u, p.status, 350 + layer))) { ok = false; break; }
      tc_fence_after();
      const __nv_bfloat16* hsrc = (layer == 0 ? p.h2 : p.h1) + (size_t)row * p.ld_h;
      __nv_bfloat16* gdst = (layer == 0 ? p.g2 : p.g1) + (size_t)row * p.ld_g;
      const uint32_t acc = lane_addr + (uint32_t)(layer * 256 + half * 128);
      auto process = [&](const uint32_t (&cur)[32], const uint4 (&hv)[4], int s4) {
        const int c0 = half * 128 + s4 * 32;
        const __nv_bfloat162* hp = reinterpret_cast<const __nv_bfloat162*>(hv);
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float h0 = __low2float(hp[j]), h1 = __high2float(hp[j]);
          __nv_bfloat162 g = __floats2bfloat162_rn(__uint_as_float(cur[2 * j]) * dact1(p.act, h0),
                                                   __uint_as_float(cur[2 * j + 1]) * dact1(p.act, h1));
          pk[j] = *reinterpret_cast<uint32_t*>(&g);
        }
        if (layer == 0 || part) {
          // layer 0: G2 is the A operand of the second product.  layer 1: that product has completed (acc_full[1]),
          // so the same tile holds G1 for the column sums.
          const int kb = c0 >> 6, ch = (c0 & 63) >> 3;
          uint8_t* base = grow + kb * 16384;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(base + (((ch + q) ^ (r & 7)) << 4)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
        if (row < p.M) {
          uint4* g = reinterpret_cast<uint4*>(gdst + c0);
#pragma unroll
          for (int q = 0; q < 4; ++q) g[q] = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
        }
      };
      auto load_h = [&](uint4 (&hv)[4], int s4) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
          hv[q] = row < p.M ? __ldg(reinterpret_cast<const uint4*>(hsrc + half * 128 + s4 * 32 + 8 * q)) : zero4;
      };
      // two register sets in ping-pong, written out as four steps (no loop-carried register copy before a wait)
      uint32_t ra[32], rb[32];
      uint4 ha[4], hb[4];
      tmem_ld_32x32b_x32_nowait(acc, ra);
      load_h(ha, 0);
      tmem_ld_wait();
      tmem_ld_32x32b_x32_nowait(acc + 32u, rb);
      load_h(hb, 1);
      process(ra, ha, 0);
      tmem_ld_wait();
      tmem_ld_32x32b_x32_nowait(acc + 64u, ra);
      load_h(ha, 2);
      process(rb, hb, 1);
      tmem_ld_wait();
      tmem_ld_32x32b_x32_nowait(acc + 96u, rb);
      load_h(hb, 3);
      process(ra, ha, 2);
      tmem_ld_wait();
      process(rb, hb, 3);
      if (layer == 0) {
        tc_fence_before();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(g_ready);
      }
      if (part) {
        asm volatile("bar.sync 1, 256;" ::: "memory");   // the whole tile is written
        part[(layer == 0 ? HID : 0) + t] = tile_colsum(sG, t);       // [0] g1, [1] g2, [2] dy
        if (layer == 0) asm volatile("bar.sync 1, 256;" ::: "memory");   // sums read before layer 1 overwrites the tile
      }
    }
    if (!ok) *abort_flag = 1;
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// Bias gradients: db1 += Σ_cta part[cta][0], db2 += Σ part[cta][1], db3 += Σ part[cta][2][:n3], in CTA order.
struct BiasFinishNet {
  const float* part;
  float *db1, *db2, *db3;
  int ctas, n3;
};
struct BiasFinishGroup {
  BiasFinishNet net[2];
};
__global__ void __launch_bounds__(4 * HID)
mlp3_bias_finish_kernel(const BiasFinishGroup g) {
  // 4 x 256 threads: thread (q, col) sums CTAs q, q+4, ...; the four partial sums are added in the order q = 0..3
  __shared__ float sh[4][HID];
  const BiasFinishNet& n = g.net[blockIdx.y];
  const int layer = blockIdx.x, col = threadIdx.x & (HID - 1), q = threadIdx.x >> 8;
  if (n.part == nullptr) return;
  float* dst = layer == 0 ? n.db1 : (layer == 1 ? n.db2 : n.db3);
  if (dst == nullptr) return;
  float acc = 0.f;
  if (layer != 2 || col < n.n3)
    for (int c = q; c < n.ctas; c += 4) acc += n.part[((size_t)c * 3 + layer) * HID + col];
  sh[q][col] = acc;
  __syncthreads();
  if (q == 0 && (layer != 2 || col < n.n3)) dst[col] += ((sh[0][col] + sh[1][col]) + sh[2][col]) + sh[3][col];
}

}  // namespace

// One network of a grouped launch (mirrored by a ctypes.Structure in noeira_b200/ops/mlp.py — keep the field order).
struct NbMlpNet {
  const void *x, *w1, *w2, *w3;      // x [M, k0] bf16; W1 [k0, 256], W2 [256, 256], W3 [256, n3] bf16 row-major
  const float *b1, *b2, *b3;         // fp32 biases (b3 may be null)
  float* out;                        // forward: fp32 [M, ld_out]
  void *h1, *h2;                     // forward: optional saves / backward: saved activations, bf16 [M, ld_h]
  const void* dy;                    // backward: bf16 [M, ld_dy], n3 columns used
  void *g1, *g2;                     // backward: bf16 [M, ld_g] gradients of the pre-activations of layers 1 and 2
  float* bias_part;                  // backward: optional fp32 scratch [ceil(M/128)][3][256] for the bias gradients
  float *db1, *db2, *db3;            // backward: fp32 bias gradients (accumulated into) when bias_part is given
  int ldx, ldw1, ldw2, ldw3, ld_out, ld_h, ld_dy, ld_g;
  int M, k0, n3, act;
};

namespace {
using namespace nb;
constexpr size_t FWD_SMEM = 16384 + 32768 + 2 * 32768 + 65536 + 8192 + 1024 + 256;
constexpr size_t BWD_SMEM = 16384 + 32768 + 2 * 32768 + 65536 + 1024 + 256;

int check_net(const NbMlpNet& n) {
  if (n.M <= 0 || n.k0 <= 0 || n.k0 > 64 || n.n3 <= 0 || n.n3 > N3P) return NB_ERR_BAD_ARG;
  if (n.act != NB_ACT_TANH && n.act != NB_ACT_RELU) return NB_ERR_BAD_ARG;
  if ((n.h1 || n.h2) && (n.ld_h % 8 || ((uintptr_t)n.h1 & 15) || ((uintptr_t)n.h2 & 15))) return NB_ERR_UNALIGNED;
  return NB_OK;
}
}  // namespace

extern "C" {

// Forward of `nets` (1 or 2) three-layer MLPs in one launch; act: NB_ACT_TANH / NB_ACT_RELU.
int nb_mlp3_fwd_group(const NbMlpNet* net, int nets, unsigned int* status, void* stream) {
  if (nets < 1 || nets > 2) return NB_ERR_BAD_ARG;
  MlpGroup g;
  memset(&g, 0, sizeof(g));
  int max_m = 0;
  for (int i = 0; i < nets; ++i) {
    const NbMlpNet& n = net[i];
    int rc = check_net(n);
    if (rc) return rc;
    rc = tmap2d(&g.maps[i].x, n.x, n.k0, n.M, n.ldx, 64, ROWS);
    if (rc) return rc;
    rc = tmap2d(&g.maps[i].w1, n.w1, HID, n.k0, n.ldw1, 64, 64);
    if (rc) return rc;
    rc = tmap2d(&g.maps[i].w2, n.w2, HID, HID, n.ldw2, 64, 64);
    if (rc) return rc;
    MlpParams& p = g.prm[i];
    p.M = n.M; p.k0 = n.k0; p.n3 = n.n3;
    p.ld_w3 = n.ldw3; p.ld_out = n.ld_out; p.ld_h = n.ld_h;
    p.act = n.act;
    p.w3 = (const __nv_bfloat16*)n.w3;
    p.b1 = n.b1; p.b2 = n.b2; p.b3 = n.b3;
    p.out = n.out;
    p.h1 = (__nv_bfloat16*)n.h1; p.h2 = (__nv_bfloat16*)n.h2;
    p.status = status;
    max_m = n.M > max_m ? n.M : max_m;
  }
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(mlp3_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)FWD_SMEM));
    configured = true;
  }
  mlp3_fwd_kernel<<<dim3(ceil_div(max_m, ROWS), nets), MLP_THREADS, FWD_SMEM, (cudaStream_t)stream>>>(g);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// Data-gradient chain of `nets` (1 or 2) three-layer MLPs in one launch: g2 = (dy W3ᵀ) ⊙ f'(h2), g1 = (g2 W2ᵀ) ⊙ f'(h1).
int nb_mlp3_bwd_group(const NbMlpNet* net, int nets, unsigned int* status, void* stream) {
  if (nets < 1 || nets > 2) return NB_ERR_BAD_ARG;
  MlpBwdGroup g;
  memset(&g, 0, sizeof(g));
  int max_m = 0;
  for (int i = 0; i < nets; ++i) {
    const NbMlpNet& n = net[i];
    int rc = check_net(n);
    if (rc) return rc;
    if (!n.dy || !n.h1 || !n.h2 || !n.g1 || !n.g2) return NB_ERR_BAD_ARG;
    if (n.ld_g % 8 || ((uintptr_t)n.g1 & 15) || ((uintptr_t)n.g2 & 15) || n.ldw3 < n.n3 || n.ld_dy < n.n3) return NB_ERR_UNALIGNED;
    rc = tmap2d(&g.w2[i], n.w2, HID, HID, n.ldw2, 64, HID);
    if (rc) return rc;
    MlpBwdParams& p = g.prm[i];
    p.M = n.M; p.n3 = n.n3;
    p.ld_dy = n.ld_dy; p.ld_w3 = n.ldw3; p.ld_h = n.ld_h; p.ld_g = n.ld_g;
    p.act = n.act;
    p.dy = (const __nv_bfloat16*)n.dy; p.w3 = (const __nv_bfloat16*)n.w3;
    p.h1 = (const __nv_bfloat16*)n.h1; p.h2 = (const __nv_bfloat16*)n.h2;
    p.g1 = (__nv_bfloat16*)n.g1; p.g2 = (__nv_bfloat16*)n.g2;
    p.bias_part = n.bias_part;
    p.status = status;
    max_m = n.M > max_m ? n.M : max_m;
  }
  static bool configured = false;
  if (!configured) {
    NB_CUDA(cudaFuncSetAttribute(mlp3_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)BWD_SMEM));
    configured = true;
  }
  mlp3_bwd_kernel<<<dim3(ceil_div(max_m, ROWS), nets), MLP_THREADS, BWD_SMEM, (cudaStream_t)stream>>>(g);
  NB_LAUNCH_CHECK();
  BiasFinishGroup f;
  memset(&f, 0, sizeof(f));
  bool any = false;
  for (int i = 0; i < nets; ++i) {
    const NbMlpNet& n = net[i];
    if (!n.bias_part) continue;
    any = true;
    f.net[i].part = n.bias_part; f.net[i].db1 = n.db1; f.net[i].db2 = n.db2; f.net[i].db3 = n.db3;
    f.net[i].ctas = ceil_div(n.M, ROWS); f.net[i].n3 = n.n3;
  }
  if (any) {
    mlp3_bias_finish_kernel<<<dim3(3, nets), 4 * HID, 0, (cudaStream_t)stream>>>(f);
    NB_LAUNCH_CHECK();
  }
  return NB_OK;
}

// Single-network forward (see nb_mlp3_fwd_group).
int nb_mlp3_fwd(const void* x, int ldx, const void* w1, int ldw1, const void* w2, int ldw2, const void* w3, int ldw3,
                const float* b1, const float* b2, const float* b3, float* out, int ld_out, void* h1, void* h2, int ld_h, int M,
                int k0, int n3, int act, unsigned int* status, void* stream) {
  NbMlpNet n;
  memset(&n, 0, sizeof(n));
  n.x = x; n.w1 = w1; n.w2 = w2; n.w3 = w3; n.b1 = b1; n.b2 = b2; n.b3 = b3; n.out = out; n.h1 = h1; n.h2 = h2;
  n.ldx = ldx; n.ldw1 = ldw1; n.ldw2 = ldw2; n.ldw3 = ldw3; n.ld_out = ld_out; n.ld_h = ld_h;
  n.M = M; n.k0 = k0; n.n3 = n3; n.act = act;
  return nb_mlp3_fwd_group(&n, 1, status, stream);
}

}  // extern "C"
