// Flat-arena optimizer kernels (single GPU part; the multi-GPU fused reduce+update lives in
// allreduce_fused.cu and reuses `adamw_update4` from optim_math.cuh).
//
// The arena is the storage model of the framework: all trainable parameters of a trainer live in
// ONE contiguous fp32 buffer `val`, with `grd`, `m`, `v` of identical shape and an optional bf16
// shadow used as the tensor-core operand.  Parameters start on 128-byte boundaries (32 floats),
// so per-parameter attributes are stored per 32-float row in `row_flags`
// (bit 0: weight decay applies, bit 1: frozen — no update).
// Reference semantics: noeira/nn/optimizer/adam.mojo:75-128 (device resident beta powers, one
// grouped kernel), noeira/nn/optimizer/grad_clip.mojo:255-320 (sumsq → finalize → scale, a
// non-finite norm zeroes the step), noeira/nn/optimizer/param_arena.mojo:250 (Polyak).
#include "common.cuh"
#include "optim_math.cuh"

namespace {

// hyper layout (device floats): see optim_math.cuh

__global__ void adam_advance_kernel(float* __restrict__ hyper) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    hyper[NB_H_T] += 1.0f;
    hyper[NB_H_B1T] *= hyper[NB_H_BETA1];
    hyper[NB_H_B2T] *= hyper[NB_H_BETA2];
  }
}

__global__ void __launch_bounds__(256)
arena_adamw_kernel(float* __restrict__ val, const float* __restrict__ grd, float* __restrict__ m,
                   float* __restrict__ v, __nv_bfloat16* __restrict__ shadow,
                   const unsigned char* __restrict__ row_flags, long long n4, const float* __restrict__ hyper,
                   int zero_grad, float* __restrict__ grd_mut) {
  const nb::AdamHyper h = nb::load_hyper(hyper);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const unsigned char fl = row_flags ? row_flags[i >> 3] : (unsigned char)1;
    float4 p = reinterpret_cast<float4*>(val)[i];
    if (!(fl & 2)) {
      float4 g = reinterpret_cast<const float4*>(grd)[i];
      float4 mm = reinterpret_cast<float4*>(m)[i];
      float4 vv = reinterpret_cast<float4*>(v)[i];
      nb::adamw_update4(p, g, mm, vv, h, (fl & 1) != 0);
      reinterpret_cast<float4*>(val)[i] = p;
      reinterpret_cast<float4*>(m)[i] = mm;
      reinterpret_cast<float4*>(v)[i] = vv;
    }
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[i] = pk;
    }
    if (zero_grad) reinterpret_cast<float4*>(grd_mut)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Several arenas (optimizers) in ONE launch, the step counters t, β₁ᵗ, β₂ᵗ advanced in the same kernel: every block
// derives the advanced powers from the values it reads at entry, the last block (ticket) writes them back.  Four
// launches (advance + update per optimizer) of an actor-critic update become one.
constexpr int MULTI_MAX = 4, MULTI_U = 2, MULTI_CHUNK4 = 256 * MULTI_U;   // small chunks: arenas of a few 100 KB still fill the GPU
struct MultiSeg {
  float *val, *grd, *m, *v;
  __nv_bfloat16* shadow;
  const unsigned char* row_flags;
  float* hyper;
  long long n4;
  int first_block;
};
struct MultiArgs {
  MultiSeg seg[MULTI_MAX];
  int nseg, zero_grad;
  unsigned int* ticket;
};
__global__ void __launch_bounds__(256)
arena_adamw_multi_kernel(const __grid_constant__ MultiArgs a) {
  int s = 0;
  while (s + 1 < a.nseg && (int)blockIdx.x >= a.seg[s + 1].first_block) ++s;
  const MultiSeg& sg = a.seg[s];
  nb::AdamHyper h = nb::load_hyper(sg.hyper);
  h.b1t *= h.beta1;
  h.b2t *= h.beta2;
  const long long base = (long long)((int)blockIdx.x - sg.first_block) * MULTI_CHUNK4;
#pragma unroll
  for (int u = 0; u < MULTI_U; ++u) {
    const long long i = base + u * 256 + threadIdx.x;
    if (i >= sg.n4) break;
    const unsigned char fl = sg.row_flags ? sg.row_flags[i >> 3] : (unsigned char)1;
    float4 p = reinterpret_cast<float4*>(sg.val)[i];
    if (!(fl & 2)) {
      float4 g = reinterpret_cast<const float4*>(sg.grd)[i];
      float4 mm = reinterpret_cast<float4*>(sg.m)[i];
      float4 vv = reinterpret_cast<float4*>(sg.v)[i];
      nb::adamw_update4(p, g, mm, vv, h, (fl & 1) != 0);
      reinterpret_cast<float4*>(sg.val)[i] = p;
      reinterpret_cast<float4*>(sg.m)[i] = mm;
      reinterpret_cast<float4*>(sg.v)[i] = vv;
    }
    if (sg.shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(sg.shadow)[i] = pk;
    }
    if (a.zero_grad) reinterpret_cast<float4*>(sg.grd)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(a.ticket, 1u) == gridDim.x - 1) {
      *a.ticket = 0u;
      for (int k = 0; k < a.nseg; ++k) {
        float* hy = a.seg[k].hyper;
        hy[NB_H_T] += 1.f;
        hy[NB_H_B1T] *= hy[NB_H_BETA1];
        hy[NB_H_B2T] *= hy[NB_H_BETA2];
      }
    }
  }
}

__global__ void __launch_bounds__(256)
arena_sgd_kernel(float* __restrict__ val, const float* __restrict__ grd, float* __restrict__ mom,
                 __nv_bfloat16* __restrict__ shadow, const unsigned char* __restrict__ row_flags, long long n4,
                 const float* __restrict__ hyper, float momentum, int nesterov) {
  const float lr = hyper[NB_H_LR], wd = hyper[NB_H_WD], gs = hyper[NB_H_GSCALE];
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const unsigned char fl = row_flags ? row_flags[i >> 3] : (unsigned char)1;
    float4 p = reinterpret_cast<float4*>(val)[i];
    if (!(fl & 2)) {
      float4 g = reinterpret_cast<const float4*>(grd)[i];
      float pe[4] = {p.x, p.y, p.z, p.w}, ge[4] = {g.x, g.y, g.z, g.w}, me[4] = {0, 0, 0, 0};
      if (mom) {
        float4 mm = reinterpret_cast<float4*>(mom)[i];
        me[0] = mm.x; me[1] = mm.y; me[2] = mm.z; me[3] = mm.w;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        float gk = ge[k] * gs + ((fl & 1) ? wd * pe[k] : 0.f);
        if (mom) {
          me[k] = momentum * me[k] + gk;
          gk = nesterov ? gk + momentum * me[k] : me[k];
        }
        pe[k] -= lr * gk;
      }
      p = make_float4(pe[0], pe[1], pe[2], pe[3]);
      reinterpret_cast<float4*>(val)[i] = p;
      if (mom) reinterpret_cast<float4*>(mom)[i] = make_float4(me[0], me[1], me[2], me[3]);
    }
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[i] = pk;
    }
  }
}

// LaProp-style update with adaptive gradient clipping per 32-float row group, used by the
// Dreamer-family trainers (noeira/nn/optimizer/dreamer_opt.mojo:179): g is normalised by
// sqrt(v) BEFORE entering the momentum.
__global__ void __launch_bounds__(256)
arena_laprop_kernel(float* __restrict__ val, const float* __restrict__ grd, float* __restrict__ m,
                    float* __restrict__ v, __nv_bfloat16* __restrict__ shadow,
                    const unsigned char* __restrict__ row_flags, long long n4, const float* __restrict__ hyper) {
  const nb::AdamHyper h = nb::load_hyper(hyper);
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const unsigned char fl = row_flags ? row_flags[i >> 3] : (unsigned char)1;
    float4 p = reinterpret_cast<float4*>(val)[i];
    if (!(fl & 2)) {
      float4 g = reinterpret_cast<const float4*>(grd)[i];
      float4 mm = reinterpret_cast<float4*>(m)[i];
      float4 vv = reinterpret_cast<float4*>(v)[i];
      float pe[4] = {p.x, p.y, p.z, p.w}, ge[4] = {g.x, g.y, g.z, g.w};
      float me[4] = {mm.x, mm.y, mm.z, mm.w}, ve[4] = {vv.x, vv.y, vv.z, vv.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float gk = ge[k] * h.gscale;
        ve[k] = h.beta2 * ve[k] + (1.f - h.beta2) * gk * gk;
        const float denom = sqrtf(ve[k] / (1.f - h.b2t)) + h.eps;
        me[k] = h.beta1 * me[k] + (1.f - h.beta1) * (gk / denom);
        const float upd = me[k] / (1.f - h.b1t);
        pe[k] -= h.lr * (upd + ((fl & 1) ? h.wd * pe[k] : 0.f));
      }
      p = make_float4(pe[0], pe[1], pe[2], pe[3]);
      reinterpret_cast<float4*>(val)[i] = p;
      reinterpret_cast<float4*>(m)[i] = make_float4(me[0], me[1], me[2], me[3]);
      reinterpret_cast<float4*>(v)[i] = make_float4(ve[0], ve[1], ve[2], ve[3]);
    }
    if (shadow) {
      __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&lo);
      pk.y = *reinterpret_cast<uint32_t*>(&hi);
      reinterpret_cast<uint2*>(shadow)[i] = pk;
    }
  }
}

// Σ g² — deterministic two level reduction: each block writes one partial, the last block
// (elected with a ticket) sums the partials in index order.
__global__ void __launch_bounds__(256)
arena_sumsq_kernel(const float* __restrict__ g, long long n4, float* __restrict__ partials,
                   unsigned int* __restrict__ ticket, float* __restrict__ out) {
  __shared__ float sh[32];
  __shared__ bool last;
  float acc = 0.f;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 x = reinterpret_cast<const float4*>(g)[i];
    acc += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
  }
  acc = nb::block_sum(acc, sh);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = acc;
    __threadfence();
    unsigned int t = atomicAdd(ticket, 1u);
    last = (t == gridDim.x - 1);
  }
  __syncthreads();
  if (last) {
    __threadfence();
    float s = 0.f;
    for (int i = threadIdx.x; i < (int)gridDim.x; i += blockDim.x) s += partials[i];
    s = nb::block_sum(s, sh);
    if (threadIdx.x == 0) {
      out[0] = s;
      *ticket = 0u;
    }
  }
}

// hyper[GSCALE] = base_scale * min(1, max_norm / (sqrt(sumsq)*base_scale + 1e-6)); non-finite → 0.
__global__ void clip_finalize_kernel(const float* __restrict__ sumsq, float max_norm, float base_scale,
                                     float* __restrict__ hyper, float* __restrict__ norm_out) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    float norm = sqrtf(sumsq[0]) * base_scale;
    float s = base_scale;
    if (!isfinite(norm)) s = 0.f;
    else if (max_norm > 0.f && norm > max_norm) s = base_scale * max_norm / (norm + 1e-6f);
    hyper[NB_H_GSCALE] = s;
    if (norm_out) norm_out[0] = norm;
  }
}

__global__ void __launch_bounds__(256)
polyak_kernel(float* __restrict__ target, const float* __restrict__ online, long long n4, float tau) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 t = reinterpret_cast<float4*>(target)[i];
    const float4 o = reinterpret_cast<const float4*>(online)[i];
    t.x += tau * (o.x - t.x);
    t.y += tau * (o.y - t.y);
    t.z += tau * (o.z - t.z);
    t.w += tau * (o.w - t.w);
    reinterpret_cast<float4*>(target)[i] = t;
  }
}

__global__ void __launch_bounds__(256)
cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n4, float scale) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 p = reinterpret_cast<const float4*>(src)[i];
    __nv_bfloat162 lo = __floats2bfloat162_rn(p.x * scale, p.y * scale),
                   hi = __floats2bfloat162_rn(p.z * scale, p.w * scale);
    uint2 pk;
    pk.x = *reinterpret_cast<uint32_t*>(&lo);
    pk.y = *reinterpret_cast<uint32_t*>(&hi);
    reinterpret_cast<uint2*>(dst)[i] = pk;
  }
}

__global__ void __launch_bounds__(256) fill_kernel(float* __restrict__ dst, long long n4, float v) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float4 f = make_float4(v, v, v, v);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride)
    reinterpret_cast<float4*>(dst)[i] = f;
}

// Scalar Adam on a single device resident value (SAC temperature):
// state = [log_alpha, m, v, b1t, b2t, alpha]; grad = -(mean_logp + target_entropy) (d/dlogα of
// -logα·(logπ + H)).  noeira/nn/optimizer/scalar_adam.mojo:73.
__global__ void scalar_adam_alpha_kernel(float* __restrict__ st, const float* __restrict__ mean_logp,
                                         float target_entropy, float lr, float b1, float b2, float eps) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    const float g = -(mean_logp[0] + target_entropy);
    st[3] *= b1;
    st[4] *= b2;
    st[1] = b1 * st[1] + (1.f - b1) * g;
    st[2] = b2 * st[2] + (1.f - b2) * g * g;
    const float mh = st[1] / (1.f - st[3]), vh = st[2] / (1.f - st[4]);
    st[0] -= lr * mh / (sqrtf(vh) + eps);
    st[5] = expf(st[0]);
  }
}

inline int grid_for(long long n4) {
  long long b = (n4 + 255) / 256;
  const long long cap = 148LL * 8;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

}  // namespace

extern "C" {

int nb_adam_advance(float* hyper, void* stream) {
  adam_advance_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(hyper);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// Adam(W) step of up to 4 arenas in one launch, step counters included (see arena_adamw_multi_kernel).  `ticket`: one
// zero-initialised u32 owned by the caller.
int nb_arena_adamw_multi(int nseg, float* const* val, float* const* grd, float* const* m, float* const* v,
                         void* const* shadow, const unsigned char* const* row_flags, float* const* hyper,
                         const long long* n, int zero_grad, unsigned int* ticket, void* stream) {
  if (nseg < 1 || nseg > MULTI_MAX || !ticket) return NB_ERR_BAD_ARG;
  MultiArgs a;
  a.nseg = nseg; a.zero_grad = zero_grad; a.ticket = ticket;
  int blocks = 0;
  for (int k = 0; k < nseg; ++k) {
    if (n[k] <= 0 || n[k] % 4) return NB_ERR_UNALIGNED;
    MultiSeg& s = a.seg[k];
    s.val = val[k]; s.grd = grd[k]; s.m = m[k]; s.v = v[k];
    s.shadow = shadow ? (__nv_bfloat16*)shadow[k] : nullptr;
    s.row_flags = row_flags ? row_flags[k] : nullptr;
    s.hyper = hyper[k];
    s.n4 = n[k] / 4;
    s.first_block = blocks;
    blocks += (int)((s.n4 + MULTI_CHUNK4 - 1) / MULTI_CHUNK4);
  }
  arena_adamw_multi_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(a);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_arena_adamw(float* val, float* grd, float* m, float* v, void* shadow_bf16,
                   const unsigned char* row_flags, long long n, const float* hyper, int zero_grad,
                   void* stream) {
  if (n % 4 != 0) return NB_ERR_UNALIGNED;
  const long long n4 = n / 4;
  if (n4 == 0) return NB_OK;
  arena_adamw_kernel<<<grid_for(n4), 256, 0, (cudaStream_t)stream>>>(
      val, grd, m, v, (__nv_bfloat16*)shadow_bf16, row_flags, n4, hyper, zero_grad, grd);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_arena_sgd(float* val, const float* grd, float* mom, void* shadow_bf16, const unsigned char* row_flags,
                 long long n, const float* hyper, float momentum, int nesterov, void* stream) {
  if (n % 4 != 0) return NB_ERR_UNALIGNED;
  const long long n4 = n / 4;
  if (n4 == 0) return NB_OK;
  arena_sgd_kernel<<<grid_for(n4), 256, 0, (cudaStream_t)stream>>>(val, grd, mom, (__nv_bfloat16*)shadow_bf16,
                                                                 row_flags, n4, hyper, momentum, nesterov);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_arena_laprop(float* val, const float* grd, float* m, float* v, void* shadow_bf16,
                    const unsigned char* row_flags, long long n, const float* hyper, void* stream) {
  if (n % 4 != 0) return NB_ERR_UNALIGNED;
  const long long n4 = n / 4;
  if (n4 == 0) return NB_OK;
  arena_laprop_kernel<<<grid_for(n4), 256, 0, (cudaStream_t)stream>>>(val, grd, m, v, (__nv_bfloat16*)shadow_bf16,
                                                                    row_flags, n4, hyper);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// scratch: >= 1184 floats of partials followed by one uint ticket (zero initialised once).
int nb_arena_sumsq(const float* g, long long n, float* partials, unsigned int* ticket, float* out,
                   void* stream) {
  if (n % 4 != 0) return NB_ERR_UNALIGNED;
  const long long n4 = n / 4;
  arena_sumsq_kernel<<<grid_for(n4 > 0 ? n4 : 1), 256, 0, (cudaStream_t)stream>>>(g, n4, partials, ticket, out);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_clip_finalize(const float* sumsq, float max_norm, float base_scale, float* hyper, float* norm_out,
                     void* stream) {
  clip_finalize_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(sumsq, max_norm, base_scale, hyper, norm_out);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_polyak(float* target, const float* online, long long n, float tau, void* stream) {
  if (n % 4 != 0) return NB_ERR_UNALIGNED;
  if (n == 0) return NB_OK;
  polyak_kernel<<<grid_for(n / 4), 256, 0, (cudaStream_t)stream>>>(target, online, n / 4, tau);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_cast_bf16(const float* src, void* dst, long long n, float scale, void* stream) {
  if (n % 4 != 0) return NB_ERR_UNALIGNED;
  if (n == 0) return NB_OK;
  cast_bf16_kernel<<<grid_for(n / 4), 256, 0, (cudaStream_t)stream>>>(src, (__nv_bfloat16*)dst, n / 4, scale);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_fill_f32(float* dst, long long n, float v, void* stream) {
  if (n % 4 != 0) return NB_ERR_UNALIGNED;
  if (n == 0) return NB_OK;
  fill_kernel<<<grid_for(n / 4), 256, 0, (cudaStream_t)stream>>>(dst, n / 4, v);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_scalar_adam_alpha(float* state, const float* mean_logp, float target_entropy, float lr, float b1,
                         float b2, float eps, void* stream) {
  scalar_adam_alpha_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(state, mean_logp, target_entropy, lr, b1, b2,
                                                                eps);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_set_device(int dev) { return (int)cudaSetDevice(dev); }

}  // extern "C"
