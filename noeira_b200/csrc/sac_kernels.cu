// SAC / TD3 device glue: everything between the actor and critic GEMMs of one update, so that a captured update is
// GEMMs + these kernels + the arena optimizers with no framework elementwise launches in between.
//
//   sac_sample      [μ | ln σ] (fp32 rows) + standard-normal noise → squashed action a = c·tanh(μ + σ z), log-probability
//                   with the tanh correction, the tensors the backward needs (y = tanh u, σ z, clamp mask), and the critic
//                   input row [s | a | 0-pad] in bf16
//   sac_pack_sa     [s | a | 0-pad] in bf16 for replayed (s, a)
//   sac_target      y = r + γ (1 − d) (min(Q1', Q2') − α logπ')                (α read from device memory)
//   sac_critic_grad dQ_i = 2 (Q_i − y) / B as bf16 rows, Σ (Q_i − y)² per block
//   sac_actor_qgrad picks the smaller critic per sample: dQ1 = −[Q1 ≤ Q2] / B, dQ2 = −[Q1 > Q2] / B, block sums of
//                   α logπ − min Q, logπ and Q1
//   sac_dist_bwd    dL/da (columns [obs, obs + act) of the two critics' input gradients) and dL/dlogπ = α / B through the
//                   squashed Gaussian → gradient of [μ | ln σ] as bf16 rows
//   td3_target      y = r + γ (1 − d) min(Q1', Q2')
//   sum_partials    deterministic second pass of every block reduction
// Math: noeira/deep_agents/sac (squashed Gaussian act / loss kernels, trainer.mojo:604-703), ln σ clamped to [−5, 2],
// log(c (1 − y²) + 1e-6) correction.
#include "common.cuh"

namespace {
using namespace nb;

constexpr float LOG_2PI = 1.8378770664093453f;
constexpr float LS_MIN = -5.f, LS_MAX = 2.f;

__global__ void sac_pack_sa_kernel(const float* __restrict__ s, int ld_s, const float* __restrict__ a, int ld_a,
                                   __nv_bfloat16* __restrict__ out, int ld_o, int B, int O, int A) {
  const int i = blockIdx.x;
  for (int j = threadIdx.x; j < ld_o; j += blockDim.x) {
    float v = 0.f;
    if (j < O) v = s[(size_t)i * ld_s + j];
    else if (j < O + A) v = a[(size_t)i * ld_a + j - O];
    out[(size_t)i * ld_o + j] = __float2bfloat16(v);
  }
}

// one thread per sample; A is small (action dimensions)
__global__ void sac_sample_kernel(const float* __restrict__ packed, int ld_p, const float* __restrict__ z,
                                  const float* __restrict__ s, int ld_s, float* __restrict__ act, float* __restrict__ logp,
                                  float* __restrict__ y_out, float* __restrict__ sdz_out, unsigned char* __restrict__ free_out,
                                  __nv_bfloat16* __restrict__ sa, int ld_sa, int B, int O, int A, float c) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  float lp = 0.f;
  for (int j = 0; j < A; ++j) {
    const float mu = packed[(size_t)i * ld_p + j], lr = packed[(size_t)i * ld_p + A + j];
    const float ls = fminf(fmaxf(lr, LS_MIN), LS_MAX);
    const float sd = expf(ls), zz = z[(size_t)i * A + j];
    const float y = tanhf(mu + sd * zz);
    lp += -0.5f * zz * zz - ls - 0.5f * LOG_2PI - logf(c * (1.f - y * y) + 1e-6f);
    act[(size_t)i * A + j] = c * y;
    if (y_out) {
      y_out[(size_t)i * A + j] = y;
      sdz_out[(size_t)i * A + j] = sd * zz;
      free_out[(size_t)i * A + j] = (lr > LS_MIN && lr < LS_MAX) ? 1 : 0;
    }
    if (sa) sa[(size_t)i * ld_sa + O + j] = __float2bfloat16(c * y);
  }
  logp[i] = lp;
  if (sa) {
    for (int j = 0; j < O; ++j) sa[(size_t)i * ld_sa + j] = __float2bfloat16(s[(size_t)i * ld_s + j]);
    for (int j = O + A; j < ld_sa; ++j) sa[(size_t)i * ld_sa + j] = __float2bfloat16(0.f);
  }
}

__global__ void sac_target_kernel(const float* __restrict__ q1, int ld1, const float* __restrict__ q2, int ld2,
                                  const float* __restrict__ logp, const float* __restrict__ r, const float* __restrict__ d,
                                  const float* __restrict__ alpha, float gamma, float* __restrict__ y, int B) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const float q = fminf(q1[(size_t)i * ld1], q2[(size_t)i * ld2]);
  const float ent = logp ? alpha[0] * logp[i] : 0.f;
  y[i] = r[i] + gamma * (1.f - d[i]) * (q - ent);
}

__global__ void __launch_bounds__(256)
sac_critic_grad_kernel(const float* __restrict__ q1, int ld1, const float* __restrict__ q2, int ld2,
                       const float* __restrict__ y, __nv_bfloat16* __restrict__ dq1, __nv_bfloat16* __restrict__ dq2,
                       int ld_dq, float* __restrict__ partials, int B) {
  __shared__ float sh[32];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  float l = 0.f;
  if (i < B) {
    const float e1 = q1[(size_t)i * ld1] - y[i], e2 = q2[(size_t)i * ld2] - y[i];
    l = e1 * e1 + e2 * e2;
    const float g = 2.f / (float)B;
    for (int j = 0; j < ld_dq; ++j) {
      dq1[(size_t)i * ld_dq + j] = __float2bfloat16(j == 0 ? g * e1 : 0.f);
      dq2[(size_t)i * ld_dq + j] = __float2bfloat16(j == 0 ? g * e2 : 0.f);
    }
  }
  const float s = block_sum(l, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// partials layout: [3][nblocks]: Σ (α logπ − min Q), Σ logπ, Σ Q1
__global__ void __launch_bounds__(256)
sac_actor_qgrad_kernel(const float* __restrict__ q1, int ld1, const float* __restrict__ q2, int ld2,
                       const float* __restrict__ logp, const float* __restrict__ alpha, __nv_bfloat16* __restrict__ dq1,
                       __nv_bfloat16* __restrict__ dq2, int ld_dq, float* __restrict__ partials, int nblocks, int B) {
  __shared__ float sh[32];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  float l = 0.f, lp = 0.f, qq = 0.f;
  if (i < B) {
    const float a = q1[(size_t)i * ld1], b = q2[(size_t)i * ld2];
    const bool use1 = a <= b;
    lp = logp[i];
    qq = a;
    l = alpha[0] * lp - fminf(a, b);
    const float g = -1.f / (float)B;
    for (int j = 0; j < ld_dq; ++j) {
      dq1[(size_t)i * ld_dq + j] = __float2bfloat16(j == 0 && use1 ? g : 0.f);
      dq2[(size_t)i * ld_dq + j] = __float2bfloat16(j == 0 && !use1 ? g : 0.f);
    }
  }
  const float s0 = block_sum(l, sh), s1 = block_sum(lp, sh), s2 = block_sum(qq, sh);
  if (threadIdx.x == 0) {
    partials[blockIdx.x] = s0;
    partials[nblocks + blockIdx.x] = s1;
    partials[2 * nblocks + blockIdx.x] = s2;
  }
}

__global__ void sac_dist_bwd_kernel(const __nv_bfloat16* __restrict__ d1, int ld1, const __nv_bfloat16* __restrict__ d2,
                                    int ld2, const float* __restrict__ y, const float* __restrict__ sdz,
                                    const unsigned char* __restrict__ free_, const float* __restrict__ alpha,
                                    __nv_bfloat16* __restrict__ dpacked, int ld_dp, int B, int O, int A, float c) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  const float dlogp = alpha[0] / (float)B;
  for (int j = 0; j < A; ++j) {
    const float da = __bfloat162float(d1[(size_t)i * ld1 + O + j]) + __bfloat162float(d2[(size_t)i * ld2 + O + j]);
    const float yy = y[(size_t)i * A + j];
    const float one = 1.f - yy * yy;
    const float gu = 2.f * c * yy * one / (c * one + 1e-6f);       // d logπ / du
    const float du = da * c * one + dlogp * gu;
    const float dls = free_[(size_t)i * A + j] ? du * sdz[(size_t)i * A + j] - dlogp : 0.f;
    dpacked[(size_t)i * ld_dp + j] = __float2bfloat16(du);
    dpacked[(size_t)i * ld_dp + A + j] = __float2bfloat16(dls);
  }
  for (int j = 2 * A; j < ld_dp; ++j) dpacked[(size_t)i * ld_dp + j] = __float2bfloat16(0.f);
}

// TD3 / DDPG: critic input row [s | clamp(c·a + clamp(σ z, ±nc), ±c) | 0] from the actor's bf16 output (tanh applied);
// z == nullptr: no smoothing noise (the actor pass)
__global__ void td3_pack_kernel(const float* __restrict__ s, int ld_s, const __nv_bfloat16* __restrict__ a, int ld_a,
                                const float* __restrict__ z, float sigma, float noise_clip, float c,
                                __nv_bfloat16* __restrict__ out, int ld_o, int B, int O, int A) {
  const int i = blockIdx.x;
  for (int j = threadIdx.x; j < ld_o; j += blockDim.x) {
    float v = 0.f;
    if (j < O) v = s[(size_t)i * ld_s + j];
    else if (j < O + A) {
      const int k = j - O;
      v = c * __bfloat162float(a[(size_t)i * ld_a + k]);
      if (z) v = fminf(fmaxf(v + fminf(fmaxf(sigma * z[(size_t)i * A + k], -noise_clip), noise_clip), -c), c);
    }
    out[(size_t)i * ld_o + j] = __float2bfloat16(v);
  }
}
// dL/d(actor output) = c · dQ/da from the critic's input gradient (columns [O, O + A)), as bf16 rows
__global__ void td3_actor_grad_kernel(const __nv_bfloat16* __restrict__ dsa, int ld, __nv_bfloat16* __restrict__ out, int ld_o,
                                      int B, int O, int A, float c) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= B) return;
  for (int j = 0; j < ld_o; ++j)
    out[(size_t)i * ld_o + j] = __float2bfloat16(j < A ? c * __bfloat162float(dsa[(size_t)i * ld + O + j]) : 0.f);
}
__global__ void __launch_bounds__(256)
column_partials_kernel(const float* __restrict__ x, int ld, float* __restrict__ partials, int B) {
  __shared__ float sh[32];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const float s = block_sum(i < B ? x[(size_t)i * ld] : 0.f, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

// out[k] = scale · Σ partials[k][0..n)
__global__ void sac_sum_partials_kernel(const float* __restrict__ partials, int n, int groups, float scale,
                                        float* __restrict__ out) {
  __shared__ float sh[32];
  for (int g = 0; g < groups; ++g) {
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[(size_t)g * n + i];
    s = block_sum(s, sh);
    if (threadIdx.x == 0) out[g] = s * scale;
    __syncthreads();
  }
}

}  // namespace

extern "C" {

int nb_sac_pack_sa(const float* s, int ld_s, const float* a, int ld_a, void* out, int ld_o, int B, int O, int A, void* stream) {
  if (B <= 0 || O + A > ld_o) return NB_ERR_BAD_ARG;
  sac_pack_sa_kernel<<<B, 64, 0, (cudaStream_t)stream>>>(s, ld_s, a, ld_a, (__nv_bfloat16*)out, ld_o, B, O, A);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_sac_sample(const float* packed, int ld_p, const float* z, const float* s, int ld_s, float* act, float* logp,
                  float* y_out, float* sdz_out, unsigned char* free_out, void* sa, int ld_sa, int B, int O, int A, float c,
                  void* stream) {
  if (B <= 0 || (sa && O + A > ld_sa)) return NB_ERR_BAD_ARG;
  sac_sample_kernel<<<ceil_div(B, 128), 128, 0, (cudaStream_t)stream>>>(packed, ld_p, z, s, ld_s, act, logp, y_out, sdz_out,
                                                                       free_out, (__nv_bfloat16*)sa, ld_sa, B, O, A, c);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// logp == nullptr gives the TD3 / DDPG target (no entropy term)
int nb_sac_target(const float* q1, int ld1, const float* q2, int ld2, const float* logp, const float* r, const float* d,
                  const float* alpha, float gamma, float* y, int B, void* stream) {
  sac_target_kernel<<<ceil_div(B, 256), 256, 0, (cudaStream_t)stream>>>(q1, ld1, q2, ld2, logp, r, d, alpha, gamma, y, B);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// loss_out[0] = mean (Q1 − y)² + mean (Q2 − y)²; partials needs ceil(B / 256) floats
int nb_sac_critic_grad(const float* q1, int ld1, const float* q2, int ld2, const float* y, void* dq1, void* dq2, int ld_dq,
                       float* partials, float* loss_out, int B, void* stream) {
  const int nb_ = ceil_div(B, 256);
  cudaStream_t st = (cudaStream_t)stream;
  sac_critic_grad_kernel<<<nb_, 256, 0, st>>>(q1, ld1, q2, ld2, y, (__nv_bfloat16*)dq1, (__nv_bfloat16*)dq2, ld_dq, partials, B);
  NB_LAUNCH_CHECK();
  sac_sum_partials_kernel<<<1, 256, 0, st>>>(partials, nb_, 1, 1.f / (float)B, loss_out);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// stats_out[0..3) = mean (α logπ − min Q), mean logπ, mean Q1; partials needs 3 · ceil(B / 256) floats
int nb_sac_actor_qgrad(const float* q1, int ld1, const float* q2, int ld2, const float* logp, const float* alpha, void* dq1,
                       void* dq2, int ld_dq, float* partials, float* stats_out, int B, void* stream) {
  const int nb_ = ceil_div(B, 256);
  cudaStream_t st = (cudaStream_t)stream;
  sac_actor_qgrad_kernel<<<nb_, 256, 0, st>>>(q1, ld1, q2, ld2, logp, alpha, (__nv_bfloat16*)dq1, (__nv_bfloat16*)dq2, ld_dq,
                                              partials, nb_, B);
  NB_LAUNCH_CHECK();
  sac_sum_partials_kernel<<<1, 256, 0, st>>>(partials, nb_, 3, 1.f / (float)B, stats_out);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_sac_dist_bwd(const void* d1, int ld1, const void* d2, int ld2, const float* y, const float* sdz,
                    const unsigned char* free_, const float* alpha, void* dpacked, int ld_dp, int B, int O, int A, float c,
                    void* stream) {
  if (2 * A > ld_dp) return NB_ERR_BAD_ARG;
  sac_dist_bwd_kernel<<<ceil_div(B, 128), 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)d1, ld1, (const __nv_bfloat16*)d2,
                                                                         ld2, y, sdz, free_, alpha, (__nv_bfloat16*)dpacked,
                                                                         ld_dp, B, O, A, c);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_td3_pack(const float* s, int ld_s, const void* a, int ld_a, const float* z, float sigma, float noise_clip, float c,
                void* out, int ld_o, int B, int O, int A, void* stream) {
  if (B <= 0 || O + A > ld_o) return NB_ERR_BAD_ARG;
  td3_pack_kernel<<<B, 64, 0, (cudaStream_t)stream>>>(s, ld_s, (const __nv_bfloat16*)a, ld_a, z, sigma, noise_clip, c,
                                                     (__nv_bfloat16*)out, ld_o, B, O, A);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_td3_actor_grad(const void* dsa, int ld, void* out, int ld_o, int B, int O, int A, float c, void* stream) {
  td3_actor_grad_kernel<<<ceil_div(B, 128), 128, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)dsa, ld, (__nv_bfloat16*)out, ld_o,
                                                                           B, O, A, c);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// out[0] = scale · Σ_i x[i · ld]   (mean of a column with scale = ±1 / B); partials needs ceil(B / 256) floats
int nb_column_sum(const float* x, int ld, float* partials, float* out, float scale, int B, void* stream) {
  const int nb_ = ceil_div(B, 256);
  cudaStream_t st = (cudaStream_t)stream;
  column_partials_kernel<<<nb_, 256, 0, st>>>(x, ld, partials, B);
  NB_LAUNCH_CHECK();
  sac_sum_partials_kernel<<<1, 256, 0, st>>>(partials, nb_, 1, scale, out);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
