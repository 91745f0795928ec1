// Batched BipedalWalker: one thread per environment runs the shared 2-D rigid-body core (physics2d.h, compiled here with
// five bodies / four joints / a 64-knot terrain) and the environment rules (bipedal_walker_core.h); state lives in a device
// array of WalkerState.  Step + reward + selective reset in one launch; observations as fp32 and as a zero-padded bf16
// mirror for the policy GEMM.
// Reference: noeira/envs/bipedal_walker/ (step / reset kernels), noeira/physics2d/.
#include <cuda_bf16.h>

#include "common.cuh"
#include "bipedal_walker_core.h"

namespace {
using namespace nbbw;

__global__ void __launch_bounds__(128)
bipedal_reset_kernel(WalkerState* st, int n, unsigned int seed, float* obs, __nv_bfloat16* obs_bf16, int obs_pad) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  WalkerState s = st[e];
  s.episode = 0u;
  reset(s, seed, (unsigned)e);
  float o[OBS_DIM];
  observe(s, false, false, o);
  st[e] = s;
  for (int i = 0; i < OBS_DIM; ++i) {
    if (obs) obs[(size_t)e * OBS_DIM + i] = o[i];
    if (obs_bf16) obs_bf16[(size_t)e * obs_pad + i] = __float2bfloat16(o[i]);
  }
}

__global__ void __launch_bounds__(128)
bipedal_step_kernel(WalkerState* st, int n, unsigned int seed, const float* __restrict__ action, int act_ld, float* reward,
                  float* done, float* terminated, float* obs, __nv_bfloat16* obs_bf16, float* next_obs,
                  __nv_bfloat16* next_obs_bf16, int obs_pad, float* finished_return, float* ep_stats, int do_reset) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  WalkerState s = st[e];
  float a[ACT_DIM];
  for (int i = 0; i < ACT_DIM; ++i) a[i] = action[(size_t)e * act_ld + i];
  float o[OBS_DIM];
  bool term, trunc;
  const float r = env_step(s, a, seed, (unsigned)e, o, term, trunc);
  const bool fin = term || trunc;
  reward[e] = r;
  done[e] = fin ? 1.f : 0.f;
  terminated[e] = term ? 1.f : 0.f;
  for (int i = 0; i < OBS_DIM; ++i) {
    if (next_obs) next_obs[(size_t)e * OBS_DIM + i] = o[i];
    if (next_obs_bf16) next_obs_bf16[(size_t)e * obs_pad + i] = __float2bfloat16(o[i]);
  }
  if (finished_return) finished_return[e] = fin ? s.ep_return : __int_as_float(0x7fc00000);
  if (ep_stats) {
    if (fin) {
      atomicAdd(ep_stats + 0, s.ep_return);
      atomicAdd(ep_stats + 1, 1.0f);
      atomicAdd(ep_stats + 3, (float)s.steps);
    }
    atomicAdd(ep_stats + 2, r);
  }
  if (fin && do_reset) {
    reset(s, seed, (unsigned)e);
    observe(s, false, false, o);
  }
  for (int i = 0; i < OBS_DIM; ++i) {
    if (obs) obs[(size_t)e * OBS_DIM + i] = o[i];
    if (obs_bf16) obs_bf16[(size_t)e * obs_pad + i] = __float2bfloat16(o[i]);
  }
  st[e] = s;
}

}  // namespace

extern "C" {

int nb_bipedal_state_bytes() { return (int)sizeof(nbbw::WalkerState); }

int nb_bipedal_reset(void* state, int n, unsigned int seed, float* obs, void* obs_bf16, int obs_pad, void* stream) {
  if (n <= 0) return NB_ERR_BAD_ARG;
  bipedal_reset_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>((WalkerState*)state, n, seed, obs, (__nv_bfloat16*)obs_bf16,
                                                                       obs_pad);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_bipedal_step(void* state, int n, unsigned int seed, const float* action, int act_ld, float* reward, float* done,
                  float* terminated, float* obs, void* obs_bf16, float* next_obs, void* next_obs_bf16, int obs_pad,
                  float* finished_return, float* ep_stats, int do_reset, void* stream) {
  if (n <= 0 || act_ld < 4) return NB_ERR_BAD_ARG;
  bipedal_step_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
      (WalkerState*)state, n, seed, action, act_ld, reward, done, terminated, obs, (__nv_bfloat16*)obs_bf16, next_obs,
      (__nv_bfloat16*)next_obs_bf16, obs_pad, finished_return, ep_stats, do_reset);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
