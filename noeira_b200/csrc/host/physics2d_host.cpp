// CPU build of the 2-D rigid-body core and of LunarLander: the oracle of the GPU tests and the CPU path of the
// environment (same source as the CUDA kernels: csrc/physics2d.h, csrc/lunar_lander_core.h).
#include <cstring>

#include "../lunar_lander_core.h"
#include "host_api.h"

extern "C" {

int nbh_lunar_state_bytes() { return (int)sizeof(nbll::LanderState); }

void nbh_lunar_reset(void* state, int n, unsigned int seed, float* obs) {
  auto* st = static_cast<nbll::LanderState*>(state);
  for (int e = 0; e < n; ++e) {
    st[e].episode = 0u;
    nbll::reset(st[e], seed, (unsigned)e);
    nbll::observe(st[e], false, false, obs + (size_t)e * nbll::OBS_DIM);
  }
}

// next_obs: the pre-reset observation; obs: post-reset.  finished_return may be null.
void nbh_lunar_step(void* state, int n, unsigned int seed, const float* action, int act_ld, float* reward, float* done,
                    float* terminated, float* obs, float* next_obs, float* finished_return, int do_reset) {
  auto* st = static_cast<nbll::LanderState*>(state);
  for (int e = 0; e < n; ++e) {
    float o[nbll::OBS_DIM];
    bool term, trunc;
    const float r = nbll::env_step(st[e], action + (size_t)e * act_ld, seed, (unsigned)e, o, term, trunc);
    const bool fin = term || trunc;
    reward[e] = r;
    done[e] = fin ? 1.f : 0.f;
    terminated[e] = term ? 1.f : 0.f;
    if (next_obs) std::memcpy(next_obs + (size_t)e * nbll::OBS_DIM, o, sizeof(o));
    if (finished_return) finished_return[e] = fin ? st[e].ep_return : NAN;
    if (fin && do_reset) {
      nbll::reset(st[e], seed, (unsigned)e);
      nbll::observe(st[e], false, false, o);
    }
    std::memcpy(obs + (size_t)e * nbll::OBS_DIM, o, sizeof(o));
  }
}

}  // extern "C"
