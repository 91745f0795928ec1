// Small SIMT kernels around the tensor-core ops: bias gradients (column sums), standalone
// activation forward/backward, residual adds, casts, gathers.  All vectorised for 16-byte accesses
// where the pitch allows; bf16 I/O with fp32 math.
// Reference counterparts: noeira/nn/primitives/elementwise.mojo, bias_add.mojo, ops/*.mojo
// (1 thread per element, TPB 128 — noeira/nn/constants.mojo:30-31).
#include <mutex>

#include "common.cuh"
#include "gemm_api.h"
#include "noalloc_api.h"

namespace {
using namespace nb;

__device__ __forceinline__ float act_f(int act, float v) {
  switch (act) {
    case NB_ACT_RELU: return fmaxf(v, 0.f);
    case NB_ACT_TANH: return tanhf(v);
    case NB_ACT_GELU: {
      const float c = 0.7978845608028654f;
      return 0.5f * v * (1.f + tanhf(c * (v + 0.044715f * v * v * v)));
    }
    case NB_ACT_SILU: return v / (1.f + __expf(-v));
    case NB_ACT_SIGMOID: return 1.f / (1.f + __expf(-v));
    default: return v;
  }
}
__device__ __forceinline__ float dact_f(int act, float s) {
  switch (act) {
    case NB_ACT_RELU: return s > 0.f ? 1.f : 0.f;
    case NB_ACT_TANH: return 1.f - s * s;
    case NB_ACT_SIGMOID: return s * (1.f - s);
    case NB_ACT_GELU: {
      const float c = 0.7978845608028654f;
      const float u = c * (s + 0.044715f * s * s * s);
      const float t = tanhf(u);
      return 0.5f * (1.f + t) + 0.5f * s * (1.f - t * t) * c * (1.f + 3.f * 0.044715f * s * s);
    }
    case NB_ACT_SILU: {
      const float sg = 1.f / (1.f + __expf(-s));
      return sg * (1.f + s * (1.f - sg));
    }
    default: return 1.f;
  }
}

// Column sums (bias gradients): out[n] (+)= Σ_m x[m, n], deterministic.
// Stage 1, grid (ceil(N/64), SPLIT): block (bx, by) reduces rows [by·rows, (by+1)·rows) of 64 columns
// into partials[by][n].  Stage 2 adds the SPLIT partials of a column in index order.
__global__ void __launch_bounds__(256)
colsum_bf16_kernel(const __nv_bfloat16* __restrict__ x, int M, int N, int ld, float* __restrict__ partials,
                   int rows_per_block) {
  __shared__ float sh[8][64];
  const int cp = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + cp * 2;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
  float a0 = 0.f, a1 = 0.f;
  if (col < N) {
    const bool two = (col + 1 < N);
    for (int r = r0 + rg; r < r1; r += 8) {
      const __nv_bfloat16* p = x + (size_t)r * ld + col;
      if (two && ((ld & 1) == 0)) {
        const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(p);
        a0 += __low2float(v);
        a1 += __high2float(v);
      } else {
        a0 += __bfloat162float(p[0]);
        if (two) a1 += __bfloat162float(p[1]);
      }
    }
  }
  sh[rg][cp * 2] = a0;
  sh[rg][cp * 2 + 1] = a1;
  __syncthreads();
  if (threadIdx.x < 64) {
    float s = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) s += sh[g][threadIdx.x];
    const int c = blockIdx.x * 64 + threadIdx.x;
    if (c < N) partials[(size_t)blockIdx.y * N + c] = s;
  }
}

// Vector variant (N % 8 == 0, 16-byte aligned rows): a thread owns 8 columns (one 16-byte load per row),
// 32 column groups x 8 row lanes per block, grid (ceil(N/256), SPLIT).
__global__ void __launch_bounds__(256)
colsum_bf16_vec_kernel(const __nv_bfloat16* __restrict__ x, int M, int N, int ld, float* __restrict__ partials,
                       int rows_per_block) {
  __shared__ float sh[8][256 + 8];
  const int cg = threadIdx.x & 31, rg = threadIdx.x >> 5;
  const int col = blockIdx.x * 256 + cg * 8;
  const int r0 = blockIdx.y * rows_per_block, r1 = min(M, r0 + rows_per_block);
  float acc[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) acc[k] = 0.f;
  if (col < N) {
#pragma unroll 4
    for (int r = r0 + rg; r < r1; r += 8) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(x + (size_t)r * ld + col));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        acc[2 * k] += __low2float(h[k]);
        acc[2 * k + 1] += __high2float(h[k]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) sh[rg][cg * 8 + k] = acc[k];
  __syncthreads();
  float s = 0.f;
#pragma unroll
  for (int g = 0; g < 8; ++g) s += sh[g][threadIdx.x];
  const int c = blockIdx.x * 256 + threadIdx.x;
  if (c < N) partials[(size_t)blockIdx.y * N + c] = s;
}

__global__ void colsum_finish_kernel(const float* __restrict__ partials, int N, int split, float* __restrict__ out,
                                     int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= N) return;
  float s = 0.f;
  for (int k = 0; k < split; ++k) s += partials[(size_t)k * N + c];
  out[c] = accumulate ? out[c] + s : s;
}

__global__ void __launch_bounds__(256)
act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long n, int act) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    y[i] = __float2bfloat16(act_f(act, __bfloat162float(x[i])));
}

// dx = dy ⊙ f'(saved)
__global__ void __launch_bounds__(256)
act_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ saved,
               __nv_bfloat16* __restrict__ dx, long long n, int act) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dx[i] = __float2bfloat16(__bfloat162float(dy[i]) * dact_f(act, __bfloat162float(saved[i])));
}

// y = a + b (bf16), 8 elements per thread
__global__ void __launch_bounds__(256)
add_bf16_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, long long n8) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    uint4 va = reinterpret_cast<const uint4*>(a)[i], vb = reinterpret_cast<const uint4*>(b)[i], vo;
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&va);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&vb);
    __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&vo);
#pragma unroll
    for (int k = 0; k < 4; ++k) po[k] = __hadd2(pa[k], pb[k]);
    reinterpret_cast<uint4*>(y)[i] = vo;
  }
}

// SwiGLU: h[m, j] = silu(g[m, j]) * u[m, j] with gu = [gate | up] of width 2H (pitch ld).
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, int ld, __nv_bfloat16* __restrict__ h, int ldh, int M,
                  int H) {
  const long long total = (long long)M * (H / 2);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int m = (int)(i / (H / 2)), j = (int)(i % (H / 2)) * 2;
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)m * ld + j);
    const __nv_bfloat162 u = *reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)m * ld + H + j);
    const float g0 = __low2float(g), g1 = __high2float(g);
    const float r0 = g0 / (1.f + __expf(-g0)) * __low2float(u), r1 = g1 / (1.f + __expf(-g1)) * __high2float(u);
    *reinterpret_cast<__nv_bfloat162*>(h + (size_t)m * ldh + j) = __floats2bfloat162_rn(r0, r1);
  }
}
// backward: dgu = [dh * u * silu'(g) | dh * silu(g)]
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, int ld, const __nv_bfloat16* __restrict__ dh, int ldh,
                  __nv_bfloat16* __restrict__ dgu, int M, int H) {
  const long long total = (long long)M * (H / 2);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int m = (int)(i / (H / 2)), j = (int)(i % (H / 2)) * 2;
    const __nv_bfloat162 g = *reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)m * ld + j);
    const __nv_bfloat162 u = *reinterpret_cast<const __nv_bfloat162*>(gu + (size_t)m * ld + H + j);
    const __nv_bfloat162 d = *reinterpret_cast<const __nv_bfloat162*>(dh + (size_t)m * ldh + j);
    float gg[2] = {__low2float(g), __high2float(g)}, uu[2] = {__low2float(u), __high2float(u)},
          dd[2] = {__low2float(d), __high2float(d)}, dg[2], du[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const float sg = 1.f / (1.f + __expf(-gg[k]));
      const float si = gg[k] * sg;
      dg[k] = dd[k] * uu[k] * sg * (1.f + gg[k] * (1.f - sg));
      du[k] = dd[k] * si;
    }
    *reinterpret_cast<__nv_bfloat162*>(dgu + (size_t)m * ld + j) = __floats2bfloat162_rn(dg[0], dg[1]);
    *reinterpret_cast<__nv_bfloat162*>(dgu + (size_t)m * ld + H + j) = __floats2bfloat162_rn(du[0], du[1]);
  }
}

// fp32 [M, N] (pitch lds) → bf16 [M, N] (pitch ldd)
__global__ void __launch_bounds__(256)
cast_rows_kernel(const float* __restrict__ s, int lds, __nv_bfloat16* __restrict__ d, int ldd, int M, int N) {
  const long long total = (long long)M * N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int m = (int)(i / N), n = (int)(i % N);
    d[(size_t)m * ldd + n] = __float2bfloat16(s[(size_t)m * lds + n]);
  }
}

// Scratch of the allocation-free column sum (see noalloc_api.h).  In host code this name is only a
// handle for cudaGetSymbolAddress — it is NOT a device address and must never be passed to a kernel.
static __device__ __align__(256) float g_colsum_noalloc_scratch[NB_COLSUM_NOALLOC_SCRATCH_FLOATS];

constexpr int NB_MAX_DEVICES = 64;
std::mutex g_noalloc_mutex;
float* g_noalloc_scratch_ptr[NB_MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the CURRENT device, resolved once per device.
int noalloc_scratch(float** out) {
  int dev = -1;
  NB_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= NB_MAX_DEVICES) return NB_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_scratch_ptr[dev] == nullptr) {
    float* ptr = nullptr;
    NB_CUDA(cudaGetSymbolAddress((void**)&ptr, g_colsum_noalloc_scratch));
    if (ptr == nullptr) return NB_ERR_BAD_ARG;
    g_noalloc_scratch_ptr[dev] = ptr;
  }
  *out = g_noalloc_scratch_ptr[dev];
  return NB_OK;
}

inline int grid1d(long long n) {
  long long b = (n + 255) / 256;
  const long long cap = 148LL * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}
}  // namespace

// Counter-hash dropout: keep(i) = philox(seed; i / 4, step)[i % 4] >= p·2^32.  `step` is read from device memory,
// so a captured graph draws fresh masks at every replay once the owner advances the counter between steps.
// Eight elements per thread; the keep bits are stored (one byte per element) for the backward pass.
__global__ void __launch_bounds__(256)
dropout_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, unsigned char* __restrict__ keep,
                   long long n, unsigned long long seed, const unsigned long long* __restrict__ step, float p,
                   float scale) {
  const unsigned long long st = step ? step[0] : 0ull;
  const uint32_t thresh = (uint32_t)fminf(p * 4294967296.0f, 4294967295.0f);
  Philox ph(seed);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g * 8 < n; g += stride) {
    uint32_t ra[4], rb[4];
    ph((uint32_t)(2 * g), (uint32_t)((2 * g) >> 32), (uint32_t)st, (uint32_t)(st >> 32), ra);
    ph((uint32_t)(2 * g + 1), (uint32_t)((2 * g + 1) >> 32), (uint32_t)st, (uint32_t)(st >> 32), rb);
    const long long i0 = g * 8;
    if (i0 + 8 <= n) {
      const uint4 in = *reinterpret_cast<const uint4*>(x + i0);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&in);
      uint4 out;
      __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&out);
      unsigned long long kb = 0ull;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t r0 = j < 2 ? ra[2 * j] : rb[2 * j - 4], r1 = j < 2 ? ra[2 * j + 1] : rb[2 * j - 3];
        const bool k0 = r0 >= thresh, k1 = r1 >= thresh;
        o[j] = __floats2bfloat162_rn(k0 ? __low2float(h[j]) * scale : 0.f, k1 ? __high2float(h[j]) * scale : 0.f);
        kb |= (unsigned long long)(k0 ? 1u : 0u) << (16 * j);
        kb |= (unsigned long long)(k1 ? 1u : 0u) << (16 * j + 8);
      }
      *reinterpret_cast<uint4*>(y + i0) = out;
      *reinterpret_cast<unsigned long long*>(keep + i0) = kb;
    } else {
      for (int j = 0; j < 8 && i0 + j < n; ++j) {
        const uint32_t r = j < 4 ? ra[j] : rb[j - 4];
        const bool k = r >= thresh;
        y[i0 + j] = __float2bfloat16(k ? __bfloat162float(x[i0 + j]) * scale : 0.f);
        keep[i0 + j] = k ? 1 : 0;
      }
    }
  }
}

__global__ void __launch_bounds__(256)
dropout_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const unsigned char* __restrict__ keep,
                   __nv_bfloat16* __restrict__ dx, long long n, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    dx[i] = __float2bfloat16(keep[i] ? __bfloat162float(dy[i]) * scale : 0.f);
}

__global__ void u64_add_kernel(unsigned long long* c, unsigned long long inc) {
  if (threadIdx.x == 0 && blockIdx.x == 0) c[0] += inc;
}

extern "C" {

// Split factor used for a column sum over M rows (the caller sizes `partials` as split·N floats).
int nb_colsum_split(int M) {
  int split = M / 64;
  if (split < 1) split = 1;
  if (split > 256) split = 256;
  return split;
}

// partials: nb_colsum_split(M)·N floats of scratch.
int nb_colsum_bf16(const void* x, int M, int N, int ld, float* out, int accumulate, float* partials, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  const int split = nb_colsum_split(M);
  const int rows = ceil_div(M, split);
  if (N % 8 == 0 && ld % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    dim3 grid(ceil_div(N, 256), split);
    colsum_bf16_vec_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, M, N, ld, partials, rows);
  } else {
    dim3 grid(ceil_div(N, 64), split);
    colsum_bf16_kernel<<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, M, N, ld, partials, rows);
  }
  NB_LAUNCH_CHECK();
  colsum_finish_kernel<<<ceil_div(N, 128), 128, 0, s>>>(partials, N, split, out, accumulate);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// Column sum whose scratch lives in the library image; full contract in noalloc_api.h.
int nb_colsum_bf16_noalloc(const void* x, int M, int N, int ld, float* out, int accumulate, void* stream) {
  if (M <= 0 || N <= 0 || ld < N) return NB_ERR_BAD_ARG;
  const int split = nb_colsum_split(M);
  if ((long long)split * N > (long long)NB_COLSUM_NOALLOC_SCRATCH_FLOATS) return NB_ERR_TOO_LARGE;
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != NB_OK) return rc;
  return nb_colsum_bf16(x, M, N, ld, out, accumulate, scratch, stream);
}

int nb_act_fwd(const void* x, void* y, long long n, int act, void* stream) {
  act_fwd_kernel<<<grid1d(n), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, n, act);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_act_bwd(const void* dy, const void* saved, void* dx, long long n, int act, void* stream) {
  act_bwd_kernel<<<grid1d(n), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)saved,
                                                             (__nv_bfloat16*)dx, n, act);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_add_bf16(const void* a, const void* b, void* y, long long n, void* stream) {
  if (n % 8) return NB_ERR_UNALIGNED;
  add_bf16_kernel<<<grid1d(n / 8), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                 (__nv_bfloat16*)y, n / 8);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_swiglu_fwd(const void* gu, int ld, void* h, int ldh, int M, int H, void* stream) {
  if (H % 2 || ld % 2 || ldh % 2) return NB_ERR_UNALIGNED;
  swiglu_fwd_kernel<<<grid1d((long long)M * H / 2), 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, ld,
                                                                                 (__nv_bfloat16*)h, ldh, M, H);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_swiglu_bwd(const void* gu, int ld, const void* dh, int ldh, void* dgu, int M, int H, void* stream) {
  if (H % 2 || ld % 2 || ldh % 2) return NB_ERR_UNALIGNED;
  swiglu_bwd_kernel<<<grid1d((long long)M * H / 2), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)gu, ld, (const __nv_bfloat16*)dh, ldh, (__nv_bfloat16*)dgu, M, H);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_cast_rows(const float* s, int lds, void* d, int ldd, int M, int N, void* stream) {
  cast_rows_kernel<<<grid1d((long long)M * N), 256, 0, (cudaStream_t)stream>>>(s, lds, (__nv_bfloat16*)d, ldd, M, N);
  NB_LAUNCH_CHECK();
  return NB_OK;
}


// y = dropout(x) with keep probability 1 − p and scale 1 / (1 − p); x, y 16-byte aligned when n >= 8.
int nb_dropout_fwd(const void* x, void* y, unsigned char* keep, long long n, unsigned long long seed,
                   const unsigned long long* step, float p, void* stream) {
  if (n <= 0) return NB_OK;
  if (p < 0.f || p >= 1.f) return NB_ERR_BAD_ARG;
  if ((((uintptr_t)x | (uintptr_t)y) & 15) || ((uintptr_t)keep & 7)) return NB_ERR_UNALIGNED;
  const long long groups = (n + 7) / 8;
  long long blocks = (groups + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dropout_fwd_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, keep, n,
                                                                   seed, step, p, 1.f / (1.f - p));
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_dropout_bwd(const void* dy, const unsigned char* keep, void* dx, long long n, float p, void* stream) {
  if (n <= 0) return NB_OK;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dropout_bwd_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dy, keep, (__nv_bfloat16*)dx, n,
                                                                   1.f / (1.f - p));
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_u64_add(unsigned long long* counter, unsigned long long inc, void* stream) {
  u64_add_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(counter, inc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
}  // extern "C"
