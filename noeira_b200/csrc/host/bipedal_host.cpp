// CPU build of BipedalWalker on the 2-D rigid-body core: the oracle of the GPU tests and the CPU path of the
// environment (same source as the CUDA kernels: csrc/physics2d.h, csrc/bipedal_walker_core.h).
#include <cstring>

#include "../bipedal_walker_core.h"
#include "host_api.h"

extern "C" {

int nbh_bipedal_state_bytes() { return (int)sizeof(nbbw::WalkerState); }

void nbh_bipedal_reset(void* state, int n, unsigned int seed, float* obs) {
  auto* st = static_cast<nbbw::WalkerState*>(state);
  for (int e = 0; e < n; ++e) {
    st[e].episode = 0u;
    nbbw::reset(st[e], seed, (unsigned)e);
    nbbw::observe(st[e], false, false, obs + (size_t)e * nbbw::OBS_DIM);
  }
}

// next_obs: the pre-reset observation; obs: post-reset.  finished_return may be null.
void nbh_bipedal_step(void* state, int n, unsigned int seed, const float* action, int act_ld, float* reward, float* done,
                    float* terminated, float* obs, float* next_obs, float* finished_return, int do_reset) {
  auto* st = static_cast<nbbw::WalkerState*>(state);
  for (int e = 0; e < n; ++e) {
    float o[nbbw::OBS_DIM];
    bool term, trunc;
    const float r = nbbw::env_step(st[e], action + (size_t)e * act_ld, seed, (unsigned)e, o, term, trunc);
    const bool fin = term || trunc;
    reward[e] = r;
    done[e] = fin ? 1.f : 0.f;
    terminated[e] = term ? 1.f : 0.f;
    if (next_obs) std::memcpy(next_obs + (size_t)e * nbbw::OBS_DIM, o, sizeof(o));
    if (finished_return) finished_return[e] = fin ? st[e].ep_return : NAN;
    if (fin && do_reset) {
      nbbw::reset(st[e], seed, (unsigned)e);
      nbbw::observe(st[e], false, false, o);
    }
    std::memcpy(obs + (size_t)e * nbbw::OBS_DIM, o, sizeof(o));
  }
}

}  // extern "C"
