// RoPE, embedding gather / scatter-add, and fused loss forward+gradient kernels (MSE, masked L1, KL to a
// standard normal, softmax cross-entropy).  Losses accumulate into device-resident fp32 accumulators so the
// hot loop never copies to the host (noeira/deep_agents/training/device_mean_accum.mojo:157); gradients
// are written in bf16 for the backward GEMMs.
// Reference: noeira/nn/primitives/rope.mojo:84,114; embedding.mojo:54-406; noeira/nn/loss/*.mojo.
#include "common.cuh"

namespace {
using namespace nb;

// x [B, S, H, D] (strides sb, ss, sh, 1), rotate-half pairing (i, i + D/2), angle = (pos0 + s) * theta^(-2i/D).
// dir = +1 forward, -1 backward (the transpose of a rotation is the opposite rotation).  In place.
__global__ void __launch_bounds__(256)
rope_kernel(__nv_bfloat16* __restrict__ x, int B, int S, int H, int D, long long sb, long long ss, long long sh,
            float log2_theta, int pos0, float dir) {
  const int half = D / 2;
  const long long total = (long long)B * S * H * half;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int d = (int)(i % half);
    long long r = i / half;
    const int h = (int)(r % H);
    r /= H;
    const int s = (int)(r % S);
    const int b = (int)(r / S);
    const float inv_freq = exp2f(-(2.f * d / D) * log2_theta);
    float sn, cs;
    sincosf((float)(pos0 + s) * inv_freq, &sn, &cs);
    sn *= dir;
    __nv_bfloat16* p = x + b * sb + s * ss + h * sh;
    const float x1 = __bfloat162float(p[d]), x2 = __bfloat162float(p[d + half]);
    p[d] = __float2bfloat16(x1 * cs - x2 * sn);
    p[d + half] = __float2bfloat16(x2 * cs + x1 * sn);
  }
}

// out[t, :] = table[idx[t], :] * scale
__global__ void __launch_bounds__(256)
embedding_fwd_kernel(const __nv_bfloat16* __restrict__ table, int ldt, const long long* __restrict__ idx,
                     __nv_bfloat16* __restrict__ out, int ldo, int T, int D, float scale, int vocab) {
  const int nvec = D / 8;
  const long long total = (long long)T * nvec;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int t = (int)(i / nvec), v = (int)(i % nvec);
    if (!NB_IN_BOUNDS(idx[t] >= 0 && (vocab <= 0 || idx[t] < vocab), 601, idx[t])) continue;
    uint4 w = *reinterpret_cast<const uint4*>(table + (size_t)idx[t] * ldt + v * 8);
    if (scale != 1.f) {
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
      for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(__low2float(h[k]) * scale, __high2float(h[k]) * scale);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * ldo + v * 8) = w;
  }
}
// dtable[idx[t], :] += dy[t, :] * scale   (fp32 atomics: order, hence the last bit, is not reproducible)
__global__ void __launch_bounds__(256)
embedding_bwd_kernel(float* __restrict__ dtable, int ldt, const long long* __restrict__ idx,
                     const __nv_bfloat16* __restrict__ dy, int ldy, int T, int D, float scale, int vocab) {
  const long long total = (long long)T * D;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int t = (int)(i / D), d = (int)(i % D);
    if (!NB_IN_BOUNDS(idx[t] >= 0 && (vocab <= 0 || idx[t] < vocab), 602, idx[t])) continue;
    atomicAdd(dtable + (size_t)idx[t] * ldt + d, __bfloat162float(dy[(size_t)t * ldy + d]) * scale);
  }
}

// Σ w·(pred − target)² over [M, N] (first n_real columns only); dpred = 2·w·(pred − target)·gscale.
// `rowmask` (optional, [M]) zeroes whole rows.  One partial per block, ordered finish by the caller's finish.
template <typename TP>
__global__ void __launch_bounds__(256)
mse_kernel(const TP* __restrict__ pred, int ldp, const float* __restrict__ target, int ldt,
           const float* __restrict__ rowmask, __nv_bfloat16* __restrict__ dpred, int ldd, float* __restrict__ partials,
           int M, int N, int n_real, float gscale, int l1) {
  __shared__ float sh[32];
  const long long total = (long long)M * N;
  const long long stride = (long long)gridDim.x * blockDim.x;
  float acc = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int m = (int)(i / N), n = (int)(i % N);
    float g = 0.f;
    if (n < n_real && (!rowmask || rowmask[m] != 0.f)) {
      const float d = (float)pred[(size_t)m * ldp + n] - target[(size_t)m * ldt + n];
      if (l1) {
        acc += fabsf(d);
        g = (d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f)) * gscale;
      } else {
        acc += d * d;
        g = 2.f * d * gscale;
      }
    }
    if (dpred) dpred[(size_t)m * ldd + n] = __float2bfloat16(g);
  }
  acc = block_sum(acc, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

__global__ void finish_sum_kernel(const float* __restrict__ partials, int n, float scale, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
  s = block_sum(s, sh);
  if (threadIdx.x == 0) out[0] += s * scale;
}

// KL(N(mu, exp(logvar)) || N(0,1)) summed over latent, mean over batch; info = [mu | logvar] fp32 [B, 2L].
// dinfo (bf16 [B, 2L]) = weight/B * (mu, 0.5 (exp(logvar) − 1)).
__global__ void kl_stdnormal_kernel(const float* __restrict__ info, int ld, __nv_bfloat16* __restrict__ dinfo, int ldd,
                                    float* __restrict__ partials, int B, int L, float weight) {
  __shared__ float sh[32];
  float acc = 0.f;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < B * L; i += gridDim.x * blockDim.x) {
    const int b = i / L, j = i % L;
    const float mu = info[(size_t)b * ld + j], lv = info[(size_t)b * ld + L + j];
    const float ev = __expf(lv);
    acc += -0.5f * (1.f + lv - mu * mu - ev);
    if (dinfo) {
      dinfo[(size_t)b * ldd + j] = __float2bfloat16(weight / B * mu);
      dinfo[(size_t)b * ldd + L + j] = __float2bfloat16(weight / B * 0.5f * (ev - 1.f));
    }
  }
  acc = block_sum(acc, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = acc;
}

// Softmax cross-entropy, one block per row: loss_row = lse − logit[target]; dlogits = (softmax − onehot)·gscale
// written IN PLACE over the bf16 logits.  ignore_index rows contribute nothing.
__global__ void __launch_bounds__(256)
cross_entropy_kernel(__nv_bfloat16* __restrict__ logits, int ld, const long long* __restrict__ target, int V,
                     float* __restrict__ row_loss, float gscale, long long ignore_index, int write_grad) {
  __shared__ float sh[32];
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (size_t)row * ld;
  long long tg = target[row];
  if (!NB_IN_BOUNDS(tg == ignore_index || (tg >= 0 && tg < V), 603, tg)) tg = ignore_index;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < V; i += blockDim.x) mx = fmaxf(mx, __bfloat162float(lr[i]));
  mx = block_max(mx, sh);
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(__bfloat162float(lr[i]) - mx);
  s = block_sum(s, sh);
  const float lse = mx + logf(s);
  const bool live = tg != ignore_index && tg >= 0 && tg < V;
  if (threadIdx.x == 0) row_loss[row] = live ? lse - __bfloat162float(lr[tg]) : 0.f;
  if (write_grad) {
    __syncthreads();
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      float g = 0.f;
      if (live) g = (__expf(__bfloat162float(lr[i]) - lse) - (i == tg ? 1.f : 0.f)) * gscale;
      lr[i] = __float2bfloat16(g);
    }
  }
}

// Sinusoidal embedding of a scalar per row: out[b, :] = [sin(t·w_i) | cos(t·w_i)], periods geometric in
// [min_period, max_period] (flow-matching time embedding).
__global__ void sincos_embed_kernel(const float* __restrict__ t, __nv_bfloat16* __restrict__ out, int ld, int B, int D,
                                    float min_period, float max_period) {
  const int half = D / 2;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < B * half; i += gridDim.x * blockDim.x) {
    const int b = i / half, j = i % half;
    const float frac = half > 1 ? (float)j / (half - 1) : 0.f;
    const float period = min_period * powf(max_period / min_period, frac);
    const float a = t[b] * 6.283185307179586f / period;
    float sn, cs;
    sincosf(a, &sn, &cs);
    out[(size_t)b * ld + j] = __float2bfloat16(sn);
    out[(size_t)b * ld + half + j] = __float2bfloat16(cs);
  }
}

inline int g1(long long n) {
  long long b = (n + 255) / 256;
  return (int)(b < 1 ? 1 : (b > 1184 ? 1184 : b));
}
}  // namespace

NB_BOUNDS_REGISTER(misc_ops)

extern "C" {

int nb_rope(void* x, int B, int S, int H, int D, long long sb, long long ss, long long sh, float theta, int pos0,
            int backward, void* stream) {
  if (D % 2) return NB_ERR_BAD_ARG;
  rope_kernel<<<g1((long long)B * S * H * (D / 2)), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)x, B, S, H, D, sb, ss, sh, log2f(theta), pos0, backward ? -1.f : 1.f);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// vocab: number of table rows (<= 0: unknown; only the bounds-checked build reads it)
int nb_embedding_fwd(const void* table, int ldt, const long long* idx, void* out, int ldo, int T, int D, float scale,
                     int vocab, void* stream) {
  if (D % 8 || ldt % 8 || ldo % 8) return NB_ERR_UNALIGNED;
  embedding_fwd_kernel<<<g1((long long)T * D / 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)table, ldt, idx, (__nv_bfloat16*)out, ldo, T, D, scale, vocab);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_embedding_bwd(float* dtable, int ldt, const long long* idx, const void* dy, int ldy, int T, int D, float scale,
                     int vocab, void* stream) {
  embedding_bwd_kernel<<<g1((long long)T * D), 256, 0, (cudaStream_t)stream>>>(dtable, ldt, idx,
                                                                              (const __nv_bfloat16*)dy, ldy, T, D, scale, vocab);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// loss_acc[0] += loss_scale · Σ …;  partials: >= 1184 floats.
int nb_mse_loss(const void* pred, int ldp, const float* target, int ldt, const float* rowmask, void* dpred, int ldd,
                float* partials, float* loss_acc, int M, int N, int n_real, float gscale, float loss_scale, int l1,
                int pred_f32, void* stream) {
  const int grid = g1((long long)M * N);
  cudaStream_t s = (cudaStream_t)stream;
  if (pred_f32)
    mse_kernel<float><<<grid, 256, 0, s>>>((const float*)pred, ldp, target, ldt, rowmask, (__nv_bfloat16*)dpred, ldd,
                                           partials, M, N, n_real, gscale, l1);
  else
    mse_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)pred, ldp, target, ldt, rowmask,
                                                   (__nv_bfloat16*)dpred, ldd, partials, M, N, n_real, gscale, l1);
  NB_LAUNCH_CHECK();
  finish_sum_kernel<<<1, 256, 0, s>>>(partials, grid, loss_scale, loss_acc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_kl_stdnormal(const float* info, int ld, void* dinfo, int ldd, float* partials, float* loss_acc, int B, int L,
                    float weight, void* stream) {
  const int grid = g1((long long)B * L);
  cudaStream_t s = (cudaStream_t)stream;
  kl_stdnormal_kernel<<<grid, 256, 0, s>>>(info, ld, (__nv_bfloat16*)dinfo, ldd, partials, B, L, weight);
  NB_LAUNCH_CHECK();
  finish_sum_kernel<<<1, 256, 0, s>>>(partials, grid, weight / B, loss_acc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// row_loss: M floats of scratch; loss_acc[0] += loss_scale · Σ row_loss
int nb_cross_entropy(void* logits, int ld, const long long* target, int M, int V, float* row_loss, float* loss_acc,
                     float gscale, float loss_scale, long long ignore_index, int write_grad, void* stream) {
  cudaStream_t s = (cudaStream_t)stream;
  cross_entropy_kernel<<<M, 256, 0, s>>>((__nv_bfloat16*)logits, ld, target, V, row_loss, gscale, ignore_index,
                                         write_grad);
  NB_LAUNCH_CHECK();
  finish_sum_kernel<<<1, 256, 0, s>>>(row_loss, M, loss_scale, loss_acc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_sincos_embed(const float* t, void* out, int ld, int B, int D, float min_period, float max_period,
                    void* stream) {
  sincos_embed_kernel<<<g1((long long)B * D / 2), 256, 0, (cudaStream_t)stream>>>(t, (__nv_bfloat16*)out, ld, B, D,
                                                                                min_period, max_period);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"

// ------------------------------------------------------------------------------------------ Q4_0 weights
// Block of 32 values along a ROW of the [IN, OUT] weight: one fp16 scale d and 16 bytes of 4-bit codes q in [0, 15];
// byte j of a block holds element j (low nibble) and element j + 16 (high nibble); value = (q − 8)·d.
// (Same block format as noeira/nn/quant/q4_0.mojo.)  Output: bf16 [rows, ld] — the tcgen05 GEMM then reads it.
namespace {
__global__ void __launch_bounds__(256)
q4_0_dequant_kernel(const unsigned char* __restrict__ codes, const __half* __restrict__ scales, __nv_bfloat16* __restrict__ out,
                    int rows, int cols, int ld) {
  const int blocks_per_row = cols / 32;
  const long long total = (long long)rows * blocks_per_row;
  for (long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x; b < total; b += (long long)gridDim.x * blockDim.x) {
    const int r = (int)(b / blocks_per_row), cb = (int)(b % blocks_per_row);
    const float d = __half2float(scales[b]);
    const uint4 q = *reinterpret_cast<const uint4*>(codes + b * 16);
    const unsigned char* qb = reinterpret_cast<const unsigned char*>(&q);
    __nv_bfloat16* o = out + (size_t)r * ld + cb * 32;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      o[j] = __float2bfloat16(((int)(qb[j] & 15) - 8) * d);
      o[j + 16] = __float2bfloat16(((int)(qb[j] >> 4) - 8) * d);
    }
  }
}
}  // namespace

extern "C" int nb_q4_0_dequant(const unsigned char* codes, const void* scales, void* out, int rows, int cols, int ld,
                               void* stream) {
  if (cols % 32 || ((uintptr_t)codes & 15)) return NB_ERR_UNALIGNED;
  const long long total = (long long)rows * (cols / 32);
  long long blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  q4_0_dequant_kernel<<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(codes, (const __half*)scales, (__nv_bfloat16*)out, rows,
                                                                    cols, ld);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
