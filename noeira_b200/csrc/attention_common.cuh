// Shared pieces of the tcgen05 attention kernels (forward and backward): tile sizes, parameter block,
// mask predicates, 4-D TMA load, tensor-map construction for [B, S, H, HD] tensors.
#pragma once
#include <cuda.h>

#include "attention_api.h"
#include "common.cuh"

namespace nbattn {
using namespace nb;

constexpr int BQ = 128;   // queries per CTA
constexpr int BKV = 128;  // keys per step
constexpr int FA_THREADS = 320;  // warp 0 TMA, warp 1 MMA, warps 2..9 softmax (two threads per query row)

struct FaParams {
  int B, Hq, Hkv, Sq, Sk;
  int mask_mode, frame, causal_off;
  int ld_o;  // elements between consecutive tokens of O
  float scale_log2;
  const unsigned char* key_valid;  // [B, Sk] or null
  const float* bias;               // [Sq, Sk] additive (natural units) or null
  __nv_bfloat16* O;
  float* lse;  // [B, Hq, Sq]
  unsigned int* status;
  // backward only
  const float* delta;      // [B, Hq, Sq]  rowsum(dO ⊙ O)
  __nv_bfloat16* dQ;       // [B, Sq, Hq, HD], token pitch ld_dq
  __nv_bfloat16* dK;       // [B, Sk, Hkv, HD], token pitch ld_dk
  __nv_bfloat16* dV;
  int ld_dq, ld_dk, ld_dv;
  float scale;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const void* tmap, uint64_t* bar, int x, int y, int z,
                                            int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z),
      "r"(w)
      : "memory");
}

// ---- the same primitives on 32-bit shared-memory addresses.  A role that owns dozens of barriers keeps ONE base
// address in a register and forms the others by adding constants (rematerialised for free), instead of a hoisted
// 64-bit pointer + conversion per barrier; that is what lets the TMA and MMA threads run in a small register budget.
__device__ __forceinline__ bool mbar_try_wait_a(uint32_t addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P1;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P1, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P1;\n"
      "}\n"
      : "=r"(ok)
      : "r"(addr), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_a(uint32_t addr, uint32_t parity, unsigned int* status, unsigned int where) {
  for (uint32_t it = 0; it < NB_SPIN_LIMIT; ++it)
    if (mbar_try_wait_a(addr, parity)) return true;
  report(status, NB_ST_MBAR_TIMEOUT, where, parity);
  return false;
}
__device__ __forceinline__ void mbar_expect_tx_a(uint32_t addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_a(uint32_t addr) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void umma_commit_a(uint32_t addr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ void tma_load_4d_a(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- packed fp32 pairs (two lanes of the FMA pipe per instruction)
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// last key index (inclusive) any query of [q0, q0+BQ) may attend, given the mask mode
__device__ __forceinline__ int kv_limit(const FaParams& p, int q0) {
  const int qmax = min(q0 + BQ, p.Sq) - 1;
  if (p.mask_mode == NB_MASK_CAUSAL) return min(p.Sk - 1, qmax + p.causal_off);
  if (p.mask_mode == NB_MASK_BLOCK_CAUSAL) return min(p.Sk - 1, (qmax / p.frame + 1) * p.frame - 1);
  return p.Sk - 1;
}
// Index masks allow a PREFIX of every key tile: number of leading columns of tile [k0, k0+BKV) that
// query q may attend (0..BKV).
__device__ __forceinline__ int row_limit(const FaParams& p, int q, int k0) {
  int last = p.Sk - 1;
  if (p.mask_mode == NB_MASK_CAUSAL) last = min(last, q + p.causal_off);
  else if (p.mask_mode == NB_MASK_BLOCK_CAUSAL) last = min(last, (q / p.frame + 1) * p.frame - 1);
  return max(0, min(BKV, last - k0 + 1));
}
// the same for a window of `width` keys starting at k0
__device__ __forceinline__ int row_limit_w(const FaParams& p, int q, int k0, int width) {
  int last = p.Sk - 1;
  if (p.mask_mode == NB_MASK_CAUSAL) last = min(last, q + p.causal_off);
  else if (p.mask_mode == NB_MASK_BLOCK_CAUSAL) last = min(last, (q / p.frame + 1) * p.frame - 1);
  return max(0, min(width, last - k0 + 1));
}
__device__ __forceinline__ bool allowed(const FaParams& p, int q, int k) {
  if (k >= p.Sk) return false;
  if (p.mask_mode == NB_MASK_CAUSAL) return k <= q + p.causal_off;
  if (p.mask_mode == NB_MASK_BLOCK_CAUSAL) return (k / p.frame) <= (q / p.frame);
  return true;
}

// ------------------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiledFn get_encode() {
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

// [B, S, H, HD] bf16 with element strides (sb, ss, sh, 1): 4-D map (hd, h, s, b), box (64, 1, rows, 1).
inline int make_tmap_bshd(CUtensorMap* tm, const void* base, int B, int S, int H, int HD, long long sb, long long ss,
                   long long sh, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return NB_ERR_NO_DRIVER_SYMBOL;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || ((sb * 2) & 15) || ((ss * 2) & 15) || ((sh * 2) & 15))
    return NB_ERR_UNALIGNED;
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)H, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)sh * 2, (cuuint64_t)ss * 2, (cuuint64_t)sb * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? NB_OK : NB_ERR_TENSORMAP;
}

// forward with two query tiles per CTA (attention_fwd2_tcgen05.cu)
int launch_fwd_two_tile(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FaParams& p, int HD,
                        cudaStream_t s);// backward, second generation (attention_bwd2_tcgen05.cu)
int launch_bwd_gen2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const CUtensorMap& tdo,
                    const FaParams& p, int HD, cudaStream_t s);

}  // namespace nbattn
