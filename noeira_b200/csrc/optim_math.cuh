// AdamW arithmetic shared by the single-GPU arena kernel and the fused all-reduce+update kernels.
#pragma once
#include "common.cuh"

// Device-resident hyper-parameter block (floats).  It lives on the device so a captured CUDA
// graph sees new learning rates / step counts on replay without re-capture.
#define NB_H_LR 0
#define NB_H_BETA1 1
#define NB_H_BETA2 2
#define NB_H_EPS 3
#define NB_H_WD 4
#define NB_H_T 5       // step count (float)
#define NB_H_B1T 6     // beta1^t
#define NB_H_B2T 7     // beta2^t
#define NB_H_GSCALE 8  // gradient pre-scale: 1/world * clip scale
#define NB_H_SIZE 16

namespace nb {

struct AdamHyper {
  float lr, beta1, beta2, eps, wd, b1t, b2t, gscale;
};

__device__ __forceinline__ AdamHyper load_hyper(const float* __restrict__ h) {
  AdamHyper a;
  a.lr = h[NB_H_LR];
  a.beta1 = h[NB_H_BETA1];
  a.beta2 = h[NB_H_BETA2];
  a.eps = h[NB_H_EPS];
  a.wd = h[NB_H_WD];
  a.b1t = h[NB_H_B1T];
  a.b2t = h[NB_H_B2T];
  a.gscale = h[NB_H_GSCALE];
  return a;
}

// Decoupled weight decay (AdamW): p -= lr * (m̂ / (sqrt(v̂) + eps) + wd * p).
__device__ __forceinline__ void adamw_update1(float& p, float g, float& m, float& v, const AdamHyper& h,
                                              bool decay) {
  g *= h.gscale;
  m = h.beta1 * m + (1.f - h.beta1) * g;
  v = h.beta2 * v + (1.f - h.beta2) * g * g;
  const float mh = m / (1.f - h.b1t);
  const float vh = v / (1.f - h.b2t);
  float upd = mh / (sqrtf(vh) + h.eps);
  if (decay) upd += h.wd * p;
  p -= h.lr * upd;
}

__device__ __forceinline__ void adamw_update4(float4& p, const float4& g, float4& m, float4& v,
                                              const AdamHyper& h, bool decay) {
  adamw_update1(p.x, g.x, m.x, v.x, h, decay);
  adamw_update1(p.y, g.y, m.y, v.y, h, decay);
  adamw_update1(p.z, g.z, m.z, v.z, h, decay);
  adamw_update1(p.w, g.w, m.w, v.w, h, decay);
}

}  // namespace nb
