// PPO device glue: action sampling, GAE, minibatch gather with a keyed bijective shuffle,
// clipped-surrogate objective (forward + gradient) and value loss.  Everything needed between the
// policy GEMMs stays on the device with device-resident counters, so one captured minibatch step
// is replayed N_EPOCHS·N_MINIBATCHES times and one captured rollout step T times.
//
// Math follows noeira/deep_agents/ppo (act_step.mojo:74-152, gae_step.mojo:60-116,
// minibatch_gather_step.mojo:53-111, objective.mojo:14-103):
//   sample = μ + σ z, env action = clamp(sample, ±scale), stored action = unclamped sample,
//   logp = Σ_j −½(log 2π + 2 lnσ_j + ((a−μ)/(σ+1e-6))²), ln σ clamped to [−5, 2];
//   GAE with truncation bootstrap from the episode's own pre-reset state;
//   per-minibatch advantage normalisation (population std, +1e-8);
//   loss = −min(r·A, clip(r, 1±ε)·A) − c_ent·Σ_j ½(log 2πe + 2 lnσ_j), r = exp(clamp(Δlogp, ±20)),
//   per-element gradient clip ±10, seed 1/MB.
// The shuffle differs by design: instead of a host Fisher–Yates uploaded once per rollout, every
// index is computed on the fly by a keyed Feistel permutation with cycle walking (O(1) state,
// capture safe, identical on every replay position given the device counters).
#include "common.cuh"

namespace {
using namespace nb;

constexpr float LOG_2PI = 1.8378770664093453f;
constexpr float LS_MIN = -5.f, LS_MAX = 2.f;

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}
// Bijection on [0, n) : 4-round Feistel over 2·hb bits + cycle walking.
__device__ __forceinline__ uint32_t feistel_perm(uint32_t i, uint32_t n, uint32_t hb, uint32_t key) {
  const uint32_t mask = (1u << hb) - 1u;
  uint32_t x = i;
  do {
    uint32_t l = x >> hb, r = x & mask;
#pragma unroll
    for (int rd = 0; rd < 4; ++rd) {
      const uint32_t f = mix32(r ^ (key + 0x9E3779B9u * (rd + 1))) & mask;
      const uint32_t nl = r;
      r = l ^ f;
      l = nl;
    }
    x = (l << hb) | r;
  } while (x >= n);
  return x;
}

// ------------------------------------------------------------------------------------------
// counters: [0] minibatch index within the update (0 .. E*K-1), [1] rollout index, [2] rng counter
__global__ void ppo_sample_kernel(const float* __restrict__ mu, int ld_mu, const float* __restrict__ log_std,
                                  const float* __restrict__ value, int ld_v, float* __restrict__ sample, int ld_s,
                                  float* __restrict__ env_action, int ld_a, float* __restrict__ logp,
                                  float* __restrict__ val_out, int n_envs, int act_dim, float action_scale,
                                  unsigned long long seed, const unsigned long long* __restrict__ counters,
                                  int ctr_offset, int deterministic) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_envs) return;
  const unsigned long long ctr = counters[2] + (unsigned long long)ctr_offset;
  Philox ph(seed);
  float lp = 0.f;
  for (int j0 = 0; j0 < act_dim; j0 += 4) {
    uint32_t rnd[4];
    ph((uint32_t)e, (uint32_t)j0, (uint32_t)ctr, (uint32_t)(ctr >> 32) ^ 0xA5A5A5A5u, rnd);
    float z[4];
    box_muller(rnd[0], rnd[1], z[0], z[1]);
    box_muller(rnd[2], rnd[3], z[2], z[3]);
    for (int k = 0; k < 4 && j0 + k < act_dim; ++k) {
      const int j = j0 + k;
      const float ls = fminf(fmaxf(log_std[j], LS_MIN), LS_MAX);
      const float sd = __expf(ls);
      const float m = mu[(size_t)e * ld_mu + j];
      const float a = deterministic ? m : m + sd * z[k];
      const float d = (a - m) / (sd + 1e-6f);
      lp += -0.5f * (LOG_2PI + 2.f * ls + d * d);
      sample[(size_t)e * ld_s + j] = a;
      env_action[(size_t)e * ld_a + j] = fminf(fmaxf(a, -action_scale), action_scale);
    }
  }
  logp[e] = lp;
  if (value) val_out[e] = value[(size_t)e * ld_v];
}

__global__ void ppo_counters_kernel(unsigned long long* __restrict__ counters, int which, int reset, int inc) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    if (reset) counters[which] = 0ull; else counters[which] += (unsigned long long)inc;
  }
}

// One thread per env, reverse scan over the T-major rollout.
__global__ void ppo_gae_kernel(const float* __restrict__ rew, const float* __restrict__ done,
                               const float* __restrict__ term, const float* __restrict__ val, int ld_v,
                               const float* __restrict__ vnext, int ld_vn, float* __restrict__ adv,
                               float* __restrict__ ret, int T, int n_envs, float gamma, float lam) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_envs) return;
  float gae = 0.f;
  for (int t = T - 1; t >= 0; --t) {
    const size_t i = (size_t)t * n_envs + e;
    const float d = done[i];
    float nv;
    if (d != 0.f || t == T - 1) nv = (1.f - term[i]) * vnext[i * ld_vn];
    else nv = val[(i + n_envs) * ld_v];
    const float v = val[i * ld_v];
    const float delta = rew[i] + gamma * nv - v;
    gae = delta + gamma * lam * (1.f - d) * gae;
    adv[i] = gae;
    ret[i] = gae + v;
  }
}

// Gather minibatch `mb = counters[0]` : rows idx = perm_epoch(k·MB + i).  obs rows are obs_words
// 16-byte words wide.  Each block also writes partial Σadv, Σadv² for the normalisation.
__global__ void __launch_bounds__(256)
ppo_gather_kernel(const uint4* __restrict__ obs_pool, int obs_words, const float* __restrict__ act_pool, int ld_act,
                  const float* __restrict__ logp_pool, const float* __restrict__ adv_pool,
                  const float* __restrict__ ret_pool, uint4* __restrict__ obs_mb, float* __restrict__ act_mb,
                  float* __restrict__ logp_mb, float* __restrict__ adv_mb, float* __restrict__ ret_mb,
                  float* __restrict__ partials, int pool, int mb_size, int n_mb, unsigned int hb,
                  unsigned long long seed, const unsigned long long* __restrict__ counters) {
  __shared__ float sh[32];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned long long c = counters[0];
  const uint32_t epoch = (uint32_t)(c / (unsigned long long)n_mb), k = (uint32_t)(c % (unsigned long long)n_mb);
  const uint32_t key = mix32((uint32_t)seed ^ mix32(epoch + 0x632BE5ABu * (uint32_t)(counters[1] + 1ull)));
  float a = 0.f;
  if (i < mb_size) {
    uint32_t src = feistel_perm(k * (uint32_t)mb_size + (uint32_t)i, (uint32_t)pool, hb, key);
    if (!NB_IN_BOUNDS(src < (uint32_t)pool, 621, src)) src = 0;
    for (int w = 0; w < obs_words; ++w) obs_mb[(size_t)i * obs_words + w] = obs_pool[(size_t)src * obs_words + w];
    for (int j = 0; j < ld_act; ++j) act_mb[(size_t)i * ld_act + j] = act_pool[(size_t)src * ld_act + j];
    logp_mb[i] = logp_pool[src];
    a = adv_pool[src];
    adv_mb[i] = a;
    ret_mb[i] = ret_pool[src];
  }
  const float s1 = block_sum(a, sh);
  const float s2 = block_sum(a * a, sh);
  if (threadIdx.x == 0) {
    partials[blockIdx.x * 2] = s1;
    partials[blockIdx.x * 2 + 1] = s2;
  }
}

// stats[0] = mean, stats[1] = 1/(std + 1e-8) from the ordered partials.
__global__ void ppo_adv_stats_kernel(const float* __restrict__ partials, int nblocks, int mb_size,
                                     float* __restrict__ stats) {
  __shared__ float sh[32];
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < nblocks; i += blockDim.x) {
    s1 += partials[i * 2];
    s2 += partials[i * 2 + 1];
  }
  s1 = block_sum(s1, sh);
  s2 = block_sum(s2, sh);
  if (threadIdx.x == 0) {
    const float mean = s1 / mb_size;
    const float var = fmaxf(s2 / mb_size - mean * mean, 0.f);
    stats[0] = mean;
    stats[1] = 1.f / (sqrtf(var) + 1e-8f);
  }
}

// Clipped surrogate: forward value + gradient wrt μ (bf16 rows for the backward GEMM) and ln σ.
// metrics (device accumulators, fp32): [0] Σ policy loss, [1] Σ approx-KL, [2] Σ clip fraction,
// [3] Σ entropy, [4] sample count.
__global__ void __launch_bounds__(256)
ppo_objective_kernel(const float* __restrict__ mu, int ld_mu, const float* __restrict__ log_std,
                     const float* __restrict__ act, int ld_act, const float* __restrict__ old_logp,
                     const float* __restrict__ adv, const float* __restrict__ stats,
                     __nv_bfloat16* __restrict__ dmu, int ld_dmu, float* __restrict__ dls_partials,
                     float* __restrict__ metric_partials, int mb_size, int act_dim, float clip_eps, float c_ent,
                     float grad_scale) {
  __shared__ float sh[32];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const bool on = i < mb_size;
  float loss = 0.f, kl = 0.f, cf = 0.f, dL_dlp = 0.f;
  float lp = 0.f;
  if (on) {
    for (int j = 0; j < act_dim; ++j) {
      const float ls = fminf(fmaxf(log_std[j], LS_MIN), LS_MAX);
      const float sd = __expf(ls) + 1e-6f;
      const float d = (act[(size_t)i * ld_act + j] - mu[(size_t)i * ld_mu + j]) / sd;
      lp += -0.5f * (LOG_2PI + 2.f * ls + d * d);
    }
    const float A = (adv[i] - stats[0]) * stats[1];
    const float diff = fminf(fmaxf(lp - old_logp[i], -20.f), 20.f);
    const float ratio = __expf(diff);
    const float unclipped = ratio * A;
    const float clipped = fminf(fmaxf(ratio, 1.f - clip_eps), 1.f + clip_eps) * A;
    loss = -fminf(unclipped, clipped);
    // gradient flows through the unclipped branch only when it is the active minimum and diff not saturated
    const bool active = (unclipped <= clipped) && (fabsf(lp - old_logp[i]) < 20.f);
    dL_dlp = active ? -ratio * A : 0.f;
    kl = (ratio - 1.f) - diff;
    cf = (fabsf(ratio - 1.f) > clip_eps) ? 1.f : 0.f;
  }
  float ent = 0.f;
  for (int j = 0; j < act_dim; ++j) {
    const float raw = log_std[j];
    const float ls = fminf(fmaxf(raw, LS_MIN), LS_MAX);
    const bool ls_free = raw > LS_MIN && raw < LS_MAX;
    ent += 0.5f * (LOG_2PI + 1.f) + ls;
    float gmu = 0.f, gls = 0.f;
    if (on) {
      const float sd = __expf(ls) + 1e-6f;
      const float d = (act[(size_t)i * ld_act + j] - mu[(size_t)i * ld_mu + j]) / sd;
      // d logp / d mu = d / sd ; d logp / d ls = d² · (σ/(σ+1e-6)) − 1 ≈ d² − 1
      gmu = dL_dlp * d / sd;
      gls = ls_free ? (dL_dlp * (d * d * ((sd - 1e-6f) / sd) - 1.f) - c_ent) : 0.f;
      gmu = fminf(fmaxf(gmu, -10.f), 10.f) * grad_scale;
      gls = fminf(fmaxf(gls, -10.f), 10.f) * grad_scale;
      dmu[(size_t)i * ld_dmu + j] = __float2bfloat16(gmu);
    }
    const float s = block_sum(gls, sh);
    if (threadIdx.x == 0) dls_partials[blockIdx.x * act_dim + j] = s;
  }
  if (on) {
    for (int j = act_dim; j < ld_dmu; ++j) dmu[(size_t)i * ld_dmu + j] = __float2bfloat16(0.f);
    loss -= c_ent * ent;
  }
  const float s0 = block_sum(on ? loss : 0.f, sh), s1 = block_sum(kl, sh), s2 = block_sum(cf, sh);
  if (threadIdx.x == 0) {
    metric_partials[blockIdx.x * 4 + 0] = s0;
    metric_partials[blockIdx.x * 4 + 1] = s1;
    metric_partials[blockIdx.x * 4 + 2] = s2;
    metric_partials[blockIdx.x * 4 + 3] = ent;
  }
}

// Ordered reduction of the per-block partials: ln σ gradient (added into the parameter gradient)
// and metrics (added into the device accumulators).
__global__ void ppo_objective_finalize_kernel(const float* __restrict__ dls_partials,
                                              const float* __restrict__ metric_partials, int nblocks, int act_dim,
                                              int mb_size, float* __restrict__ dls, float* __restrict__ metrics) {
  const int t = threadIdx.x;
  if (t < act_dim) {
    float s = 0.f;
    for (int b = 0; b < nblocks; ++b) s += dls_partials[b * act_dim + t];
    dls[t] += s;
  }
  if (t >= 32 && t < 35) {
    const int k = t - 32;
    float s = 0.f;
    for (int b = 0; b < nblocks; ++b) s += metric_partials[b * 4 + k];
    metrics[k] += s;
  }
  if (t == 35) {
    metrics[3] += metric_partials[3] * mb_size;
    metrics[4] += (float)mb_size;
  }
}

// Value loss: L = mean (v − ret)², dv = 2 (v − ret) / MB → bf16 [MB, ld_dv] (column 0).
__global__ void __launch_bounds__(256)
ppo_value_loss_kernel(const float* __restrict__ v, int ld_v, const float* __restrict__ ret,
                      __nv_bfloat16* __restrict__ dv, int ld_dv, float* __restrict__ partials, int mb_size,
                      float grad_scale) {
  __shared__ float sh[32];
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  float l = 0.f;
  if (i < mb_size) {
    const float d = v[(size_t)i * ld_v] - ret[i];
    l = d * d;
    dv[(size_t)i * ld_dv] = __float2bfloat16(2.f * d * grad_scale);
    for (int j = 1; j < ld_dv; ++j) dv[(size_t)i * ld_dv + j] = __float2bfloat16(0.f);
  }
  const float s = block_sum(l, sh);
  if (threadIdx.x == 0) partials[blockIdx.x] = s;
}

__global__ void sum_partials_kernel(const float* __restrict__ partials, int n, float* __restrict__ out) {
  __shared__ float sh[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partials[i];
  s = block_sum(s, sh);
  if (threadIdx.x == 0) out[0] += s;
}

}  // namespace

NB_BOUNDS_REGISTER(ppo_kernels)

extern "C" {

int nb_ppo_sample(const float* mu, int ld_mu, const float* log_std, const float* value, int ld_v, float* sample,
                  int ld_s, float* env_action, int ld_a, float* logp, float* val_out, int n_envs, int act_dim,
                  float action_scale, unsigned long long seed, const unsigned long long* counters, int ctr_offset,
                  int deterministic, void* stream) {
  ppo_sample_kernel<<<ceil_div(n_envs, 128), 128, 0, (cudaStream_t)stream>>>(
      mu, ld_mu, log_std, value, ld_v, sample, ld_s, env_action, ld_a, logp, val_out, n_envs, act_dim, action_scale,
      seed, counters, ctr_offset, deterministic);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_ppo_counter_add(unsigned long long* counters, int which, int inc, void* stream) {
  ppo_counters_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(counters, which, 0, inc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_ppo_counter(unsigned long long* counters, int which, int reset, void* stream) {
  ppo_counters_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(counters, which, reset, 1);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_ppo_gae(const float* rew, const float* done, const float* term, const float* val, int ld_v, const float* vnext,
               int ld_vn, float* adv, float* ret, int T, int n_envs, float gamma, float lam, void* stream) {
  ppo_gae_kernel<<<ceil_div(n_envs, 128), 128, 0, (cudaStream_t)stream>>>(rew, done, term, val, ld_v, vnext, ld_vn, adv, ret,
                                                                        T, n_envs, gamma, lam);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// partials: >= 2*ceil(mb/256) floats; stats: 2 floats.
int nb_ppo_gather(const void* obs_pool, int obs_row_bytes, const float* act_pool, int ld_act, const float* logp_pool,
                  const float* adv_pool, const float* ret_pool, void* obs_mb, float* act_mb, float* logp_mb,
                  float* adv_mb, float* ret_mb, float* partials, float* stats, int pool, int mb_size, int n_mb,
                  unsigned long long seed, const unsigned long long* counters, void* stream) {
  if (obs_row_bytes % 16) return NB_ERR_UNALIGNED;
  if (pool < 2) return NB_ERR_BAD_ARG;
  unsigned int bits = 1;
  while ((1ull << bits) < (unsigned long long)pool) ++bits;
  const unsigned int hb = (bits + 1) / 2;
  const int nblocks = ceil_div(mb_size, 256);
  cudaStream_t s = (cudaStream_t)stream;
  ppo_gather_kernel<<<nblocks, 256, 0, s>>>((const uint4*)obs_pool, obs_row_bytes / 16, act_pool, ld_act, logp_pool,
                                           adv_pool, ret_pool, (uint4*)obs_mb, act_mb, logp_mb, adv_mb, ret_mb,
                                           partials, pool, mb_size, n_mb, hb, seed, counters);
  NB_LAUNCH_CHECK();
  ppo_adv_stats_kernel<<<1, 256, 0, s>>>(partials, nblocks, mb_size, stats);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// dls_partials: ceil(mb/256)*act_dim floats; metric_partials: ceil(mb/256)*4 floats.
int nb_ppo_objective(const float* mu, int ld_mu, const float* log_std, const float* act, int ld_act,
                     const float* old_logp, const float* adv, const float* stats, void* dmu, int ld_dmu,
                     float* dls_partials, float* metric_partials, float* dls, float* metrics, int mb_size,
                     int act_dim, float clip_eps, float c_ent, float grad_scale, void* stream) {
  if (act_dim > 32) return NB_ERR_TOO_LARGE;
  const int nblocks = ceil_div(mb_size, 256);
  cudaStream_t s = (cudaStream_t)stream;
  ppo_objective_kernel<<<nblocks, 256, 0, s>>>(mu, ld_mu, log_std, act, ld_act, old_logp, adv, stats,
                                              (__nv_bfloat16*)dmu, ld_dmu, dls_partials, metric_partials, mb_size,
                                              act_dim, clip_eps, c_ent, grad_scale);
  NB_LAUNCH_CHECK();
  ppo_objective_finalize_kernel<<<1, 64, 0, s>>>(dls_partials, metric_partials, nblocks, act_dim, mb_size, dls,
                                                 metrics);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_ppo_value_loss(const float* v, int ld_v, const float* ret, void* dv, int ld_dv, float* partials,
                      float* loss_acc, int mb_size, float grad_scale, void* stream) {
  const int nblocks = ceil_div(mb_size, 256);
  cudaStream_t s = (cudaStream_t)stream;
  ppo_value_loss_kernel<<<nblocks, 256, 0, s>>>(v, ld_v, ret, (__nv_bfloat16*)dv, ld_dv, partials, mb_size,
                                               grad_scale);
  NB_LAUNCH_CHECK();
  sum_partials_kernel<<<1, 256, 0, s>>>(partials, nblocks, loss_acc);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
