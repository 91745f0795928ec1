// LayerNorm / RMSNorm forward and backward: bf16 activations, fp32 statistics, one warp per row,
// 16-byte vector accesses, one pass over x in the forward (values cached in registers for D ≤ 2048).
// Parameter gradients are deterministic two-stage column reductions (slab partials, ordered finish).
// Reference: block-per-row register-cached kernels, LN_TPB = 128 (noeira/nn/primitives/layer_norm.mojo:60,151;
// rms_norm.mojo:46,120,184).
#include "common.cuh"

namespace {
using namespace nb;

constexpr int MAXV = 8;  // 8 vectors x 8 elements x 32 lanes = 2048 columns cached in registers

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    f[2 * k] = __low2float(h[k]);
    f[2 * k + 1] = __high2float(h[k]);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162 h0 = __floats2bfloat162_rn(f[0], f[1]), h1 = __floats2bfloat162_rn(f[2], f[3]),
                 h2 = __floats2bfloat162_rn(f[4], f[5]), h3 = __floats2bfloat162_rn(f[6], f[7]);
  v.x = *reinterpret_cast<uint32_t*>(&h0);
  v.y = *reinterpret_cast<uint32_t*>(&h1);
  v.z = *reinterpret_cast<uint32_t*>(&h2);
  v.w = *reinterpret_cast<uint32_t*>(&h3);
  return v;
}

// y = (x - mean) * rstd * gamma + beta   (RMS: mean = 0, no beta).  stats[row] = (mean, rstd).
// NV = 16-byte vectors cached per lane (the row is read once when D <= NV * 256).  The cache holds the packed
// bf16 words, so D = 768 needs 12 registers and five 256-thread blocks fit on an SM: the kernel is bound by
// bytes in flight per SM, i.e. by occupancy.
template <bool RMS, int NV>
__global__ void __launch_bounds__(256)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const float* __restrict__ gamma,
                const float* __restrict__ beta, __nv_bfloat16* __restrict__ y, int ldy, float2* __restrict__ stats,
                int M, int D, float eps) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  const int nvec = D / 8;
  uint4 c[NV];
  float s = 0.f, ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int v = lane + k * 32;
    if (v < nvec) c[k] = *reinterpret_cast<const uint4*>(xr + v * 8);
  }
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int v = lane + k * 32;
    if (v < nvec) {
      float t[8];
      unpack8(c[k], t);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s += t[i];
        ss += t[i] * t[i];
      }
    }
  }
  for (int v = lane + NV * 32; v < nvec; v += 32) {  // columns beyond the register cache
    float t[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + v * 8), t);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      s += t[i];
      ss += t[i] * t[i];
    }
  }
  s = warp_sum(s);
  ss = warp_sum(ss);
  const float mean = RMS ? 0.f : s / D;
  const float var = RMS ? ss / D : fmaxf(ss / D - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  if (lane == 0 && stats) stats[row] = make_float2(mean, rstd);
  __nv_bfloat16* yr = y + (size_t)row * ldy;
  auto emit = [&](int v, const uint4& packed) {
    float t[8], o[8], g[8], bt[8];
    unpack8(packed, t);
    if (gamma) {
      const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + v * 8)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + v * 8) + 1);
      g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) g[i] = 1.f;
    }
    if (!RMS && beta) {
      const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + v * 8)), b1 = __ldg(reinterpret_cast<const float4*>(beta + v * 8) + 1);
      bt[0] = b0.x; bt[1] = b0.y; bt[2] = b0.z; bt[3] = b0.w; bt[4] = b1.x; bt[5] = b1.y; bt[6] = b1.z; bt[7] = b1.w;
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) bt[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (t[i] - mean) * rstd * g[i] + bt[i];
    *reinterpret_cast<uint4*>(yr + v * 8) = pack8(o);
  };
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int v = lane + k * 32;
    if (v < nvec) emit(v, c[k]);
  }
  for (int v = lane + NV * 32; v < nvec; v += 32) emit(v, *reinterpret_cast<const uint4*>(xr + v * 8));
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)),  g = dy * gamma   (RMS: no mean(g) term)
template <bool RMS>
__global__ void __launch_bounds__(256)
norm_bwd_dx_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ dy, int lddy,
                   const float* __restrict__ gamma, const float2* __restrict__ stats, __nv_bfloat16* __restrict__ dx,
                   int lddx, int M, int D, int accumulate) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= M) return;
  const __nv_bfloat16* xr = x + (size_t)row * ldx;
  const __nv_bfloat16* dr = dy + (size_t)row * lddy;
  const float2 st = stats[row];
  const int nvec = D / 8;
  float s1 = 0.f, s2 = 0.f;
  for (int v = lane; v < nvec; v += 32) {
    float a[8], g[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + v * 8), a);
    unpack8(*reinterpret_cast<const uint4*>(dr + v * 8), g);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gg = g[i] * (gamma ? gamma[v * 8 + i] : 1.f);
      s1 += gg;
      s2 += gg * (a[i] - st.x) * st.y;
    }
  }
  s1 = warp_sum(s1) / D;
  s2 = warp_sum(s2) / D;
  if (RMS) s1 = 0.f;
  __nv_bfloat16* or_ = dx + (size_t)row * lddx;
  for (int v = lane; v < nvec; v += 32) {
    float a[8], g[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(xr + v * 8), a);
    unpack8(*reinterpret_cast<const uint4*>(dr + v * 8), g);
    if (accumulate) unpack8(*reinterpret_cast<const uint4*>(or_ + v * 8), o);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float gg = g[i] * (gamma ? gamma[v * 8 + i] : 1.f);
      const float xh = (a[i] - st.x) * st.y;
      const float d = st.y * (gg - s1 - xh * s2);
      o[i] = accumulate ? o[i] + d : d;
    }
    *reinterpret_cast<uint4*>(or_ + v * 8) = pack8(o);
  }
}

// stage 1 of dgamma = Σ_rows dy·xhat and dbeta = Σ_rows dy: block (bx, by) owns 256 columns x a row slab
__global__ void __launch_bounds__(256)
norm_bwd_params_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ dy, int lddy,
                       const float2* __restrict__ stats, float* __restrict__ pg, float* __restrict__ pb, int M, int D,
                       int rows_per_block) {
  __shared__ float shg[8][256 + 8], shb[8][256 + 8];
  const int cg = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + cg * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
  float ag[8], ab[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) ag[k] = ab[k] = 0.f;
  if (col < D) {
    for (int r = r0 + rg; r < r1; r += 8) {
      float a[8], g[8];
      unpack8(__ldg(reinterpret_cast<const uint4*>(x + (size_t)r * ldx + col)), a);
      unpack8(__ldg(reinterpret_cast<const uint4*>(dy + (size_t)r * lddy + col)), g);
      const float2 st = stats[r];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        ag[k] += g[k] * (a[k] - st.x) * st.y;
        ab[k] += g[k];
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    shg[rg][cg * 8 + k] = ag[k];
    shb[rg][cg * 8 + k] = ab[k];
  }
  __syncthreads();
  float sg = 0.f, sb = 0.f;
#pragma unroll
  for (int g = 0; g < 8; ++g) {
    sg += shg[g][threadIdx.x];
    sb += shb[g][threadIdx.x];
  }
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < D) {
    pg[(size_t)blockIdx.y * D + c] = sg;
    if (pb) pb[(size_t)blockIdx.y * D + c] = sb;
  }
}

__global__ void norm_bwd_params_finish_kernel(const float* __restrict__ pg, const float* __restrict__ pb, int D,
                                              int split, float* __restrict__ dgamma, float* __restrict__ dbeta) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float sg = 0.f, sb = 0.f;
  for (int k = 0; k < split; ++k) {
    sg += pg[(size_t)k * D + c];
    if (pb) sb += pb[(size_t)k * D + c];
  }
  if (dgamma) dgamma[c] += sg;
  if (dbeta && pb) dbeta[c] += sb;
}

}  // namespace

extern "C" {

int nb_norm_split(int M) {
  int s = M / 64;
  return s < 1 ? 1 : (s > 128 ? 128 : s);
}

// rms != 0 → RMSNorm.  stats: M float2 (mean, rstd) kept for the backward.
int nb_norm_fwd(const void* x, int ldx, const float* gamma, const float* beta, void* y, int ldy, void* stats, int M,
                int D, float eps, int rms, void* stream) {
  if (D % 8 || ldx % 8 || ldy % 8) return NB_ERR_UNALIGNED;
  dim3 grid(ceil_div(M, 8));
  cudaStream_t st = (cudaStream_t)stream;
  const int need = ceil_div(D, 256);
#define NB_NORM_FWD(R, NVV)                                                                                        \
  norm_fwd_kernel<R, NVV><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, ldx, gamma, beta, (__nv_bfloat16*)y, ldy, \
                                                (float2*)stats, M, D, eps)
  if (rms) {
    if (need <= 1) NB_NORM_FWD(true, 1);
    else if (need <= 2) NB_NORM_FWD(true, 2);
    else if (need <= 4) NB_NORM_FWD(true, 4);
    else NB_NORM_FWD(true, 8);
  } else {
    if (need <= 1) NB_NORM_FWD(false, 1);
    else if (need <= 2) NB_NORM_FWD(false, 2);
    else if (need <= 4) NB_NORM_FWD(false, 4);
    else NB_NORM_FWD(false, 8);
  }
#undef NB_NORM_FWD
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// dgamma / dbeta are ACCUMULATED (+=) into fp32; partials: 2 * nb_norm_split(M) * D floats of scratch.
int nb_norm_bwd(const void* x, int ldx, const void* dy, int lddy, const float* gamma, const void* stats, void* dx,
                int lddx, float* dgamma, float* dbeta, float* partials, int M, int D, int rms, int accumulate_dx,
                void* stream) {
  if (D % 8 || ldx % 8 || lddy % 8 || lddx % 8) return NB_ERR_UNALIGNED;
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(ceil_div(M, 8));
  if (dx) {
    if (rms)
      norm_bwd_dx_kernel<true><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)dy, lddy, gamma,
                                                   (const float2*)stats, (__nv_bfloat16*)dx, lddx, M, D, accumulate_dx);
    else
      norm_bwd_dx_kernel<false><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)dy, lddy,
                                                    gamma, (const float2*)stats, (__nv_bfloat16*)dx, lddx, M, D,
                                                    accumulate_dx);
    NB_LAUNCH_CHECK();
  }
  if (dgamma) {
    const int split = nb_norm_split(M);
    const int rows = ceil_div(M, split);
    float* pg = partials;
    float* pb = (rms || !dbeta) ? nullptr : partials + (size_t)split * D;
    norm_bwd_params_kernel<<<dim3(ceil_div(D, 256), ceil_div(M, rows)), 256, 0, s>>>(
        (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)dy, lddy, (const float2*)stats, pg, pb, M, D, rows);
    NB_LAUNCH_CHECK();
    norm_bwd_params_finish_kernel<<<ceil_div(D, 128), 128, 0, s>>>(pg, pb, D, ceil_div(M, rows), dgamma, dbeta);
    NB_LAUNCH_CHECK();
  }
  return NB_OK;
}

}  // extern "C"
