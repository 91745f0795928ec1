// LunarLander (continuous actions) on the 2-D rigid-body core: lander hull + two legs on revolute joints with limits and
// spring-like motors, random height-field terrain with a flat helipad, main and side engines applied as impulses with
// dispersion noise, the Gymnasium observation / shaping reward / termination rules.  Host/device source shared by the
// CUDA kernel (one thread per environment) and the CPU oracle.
// Reference: noeira/envs/lunar_lander/{constants,lunar_lander,action,helpers}.mojo.
#pragma once
#include "physics2d.h"

namespace nbll {
using namespace nb2d;

constexpr float SCALE = 30.0f, FPS = 50.0f;
constexpr float VIEWPORT_W = 600.0f, VIEWPORT_H = 400.0f;
constexpr float W_UNITS = VIEWPORT_W / SCALE, H_UNITS = VIEWPORT_H / SCALE;
constexpr float HELIPAD_Y = H_UNITS / 4.0f;
constexpr float MAIN_ENGINE_POWER = 13.0f, SIDE_ENGINE_POWER = 0.6f;
constexpr float INITIAL_RANDOM = 1000.0f;
constexpr float LEG_AWAY = 20.0f, LEG_DOWN = 18.0f, LEG_W = 2.0f, LEG_H = 8.0f, LEG_SPRING_TORQUE = 40.0f;
constexpr float SIDE_ENGINE_HEIGHT = 14.0f, SIDE_ENGINE_AWAY = 12.0f;
constexpr float LANDER_MASS = 4.816667f, LANDER_INERTIA = 0.783881f, LEG_MASS = 0.071111f, LEG_INERTIA = 0.001791f;
constexpr int CHUNKS = 11;
constexpr int OBS_DIM = 8, ACT_DIM = 2;
constexpr int MAX_STEPS = 1000;

// persistent per-environment state (everything else is rebuilt each step)
struct LanderState {
  float pose[3][6];        // lander, left leg, right leg: x, y, angle, vx, vy, omega
  float height[CHUNKS];
  float prev_shaping;
  float sleep_time;
  float ep_return;
  int steps;
  int has_shaping;
  unsigned int episode;    // counter part of the random stream
  // solver warm start (accumulated impulses of the previous step)
  float jwarm[2][5];
  int cwarm_vert[3][CONTACTS_PER_BODY];
  float cwarm_imp[3][CONTACTS_PER_BODY][2];
};

// counter-based uniform in [0, 1): the same numbers on the GPU and on the host
NB2D_HD float uniform01(unsigned int seed, unsigned int env, unsigned int episode, unsigned int step, unsigned int k) {
  unsigned int x = seed * 0x9E3779B9u ^ (env + 0x7F4A7C15u) * 0x85EBCA6Bu ^ (episode + 1u) * 0xC2B2AE35u ^ (step + 1u) * 0x27D4EB2Fu ^
                   (k + 1u) * 0x165667B1u;
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return (float)(x >> 8) * (1.0f / 16777216.0f);
}

NB2D_HD void build_world(const LanderState& s, World& w) {
  w.nbody = 3; w.njoint = 2; w.ncontact = 0;
  w.gx = 0.f; w.gy = -10.0f; w.dt = 1.0f / FPS;
  w.vel_iters = 180; w.pos_iters = 8;   // a 68:1 mass ratio (hull on legs): Gauss-Seidel needs this many sweeps even warm-started
  w.baumgarte = 0.2f; w.slop = 0.005f; w.max_correction = 0.2f;
  w.sleep_time = s.sleep_time;
  const float lx[6] = {-14.f, -17.f, -17.f, 17.f, 17.f, 14.f}, ly[6] = {17.f, 0.f, -10.f, -10.f, 0.f, 17.f};
  for (int i = 0; i < 3; ++i) {
    Body& b = w.body[i];
    b.x = s.pose[i][0]; b.y = s.pose[i][1]; b.a = s.pose[i][2];
    b.vx = s.pose[i][3]; b.vy = s.pose[i][4]; b.w = s.pose[i][5];
    b.fx = b.fy = b.tq = 0.f;
    b.friction = i == 0 ? 0.1f : 0.2f;
    if (i == 0) {
      b.inv_m = 1.0f / LANDER_MASS; b.inv_i = 1.0f / LANDER_INERTIA;
      b.nvert = 6;
      for (int v = 0; v < 6; ++v) { b.px[v] = lx[v] / SCALE; b.py[v] = ly[v] / SCALE; }
    } else {
      b.inv_m = 1.0f / LEG_MASS; b.inv_i = 1.0f / LEG_INERTIA;
      b.nvert = 4;
      const float hw = LEG_W / SCALE, hh = LEG_H / SCALE;
      b.px[0] = -hw; b.py[0] = -hh; b.px[1] = hw; b.py[1] = -hh; b.px[2] = hw; b.py[2] = hh; b.px[3] = -hw; b.py[3] = hh;
    }
  }
  for (int k = 0; k < 2; ++k) {
    const float sgn = k == 0 ? -1.f : 1.f;
    Revolute& j = w.joint[k];
    j.a = 0; j.b = 1 + k;
    j.ax = 0.f; j.ay = 0.f;
    j.bx = sgn * LEG_AWAY / SCALE; j.by = LEG_DOWN / SCALE;
    j.ref = 0.f;
    j.enable_motor = 1; j.enable_limit = 1;
    j.max_torque = LEG_SPRING_TORQUE;
    j.motor_speed = 0.3f * sgn;
    if (k == 0) { j.lower = 0.9f - 0.5f; j.upper = 0.9f; }
    else { j.lower = -0.9f; j.upper = -0.9f + 0.5f; }
  }
  clear_warm_start(w);
  for (int j = 0; j < 2; ++j)
    for (int k = 0; k < 5; ++k) w.jwarm[j][k] = s.jwarm[j][k];
  for (int b = 0; b < 3; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      w.cwarm_vert[b][k] = s.cwarm_vert[b][k];
      w.cwarm_imp[b][k][0] = s.cwarm_imp[b][k][0];
      w.cwarm_imp[b][k][1] = s.cwarm_imp[b][k][1];
    }
  w.terrain.n = CHUNKS;
  w.terrain.x0 = 0.f;
  w.terrain.dx = W_UNITS / (float)(CHUNKS - 1);
  for (int i = 0; i < CHUNKS; ++i) w.terrain.h[i] = s.height[i];
}

NB2D_HD void save_world(const World& w, LanderState& s) {
  for (int i = 0; i < 3; ++i) {
    const Body& b = w.body[i];
    s.pose[i][0] = b.x; s.pose[i][1] = b.y; s.pose[i][2] = b.a;
    s.pose[i][3] = b.vx; s.pose[i][4] = b.vy; s.pose[i][5] = b.w;
  }
  s.sleep_time = w.sleep_time;
  for (int j = 0; j < 2; ++j)
    for (int k = 0; k < 5; ++k) s.jwarm[j][k] = w.jwarm[j][k];
  for (int b = 0; b < 3; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      s.cwarm_vert[b][k] = w.cwarm_vert[b][k];
      s.cwarm_imp[b][k][0] = w.cwarm_imp[b][k][0];
      s.cwarm_imp[b][k][1] = w.cwarm_imp[b][k][1];
    }
}

NB2D_HD void observe(const LanderState& s, bool leg0, bool leg1, float* obs) {
  const float x = s.pose[0][0], y = s.pose[0][1];
  obs[0] = (x - W_UNITS / 2.0f) / (W_UNITS / 2.0f);
  obs[1] = (y - (HELIPAD_Y + LEG_DOWN / SCALE)) / (H_UNITS / 2.0f);
  obs[2] = s.pose[0][3] * (W_UNITS / 2.0f) / FPS;
  obs[3] = s.pose[0][4] * (H_UNITS / 2.0f) / FPS;
  obs[4] = s.pose[0][2];
  obs[5] = 20.0f * s.pose[0][5] / FPS;
  obs[6] = leg0 ? 1.f : 0.f;
  obs[7] = leg1 ? 1.f : 0.f;
}

NB2D_HD void reset(LanderState& s, unsigned int seed, unsigned int env) {
  s.episode += 1u;
  // terrain: random heights, smoothed, flat helipad on the five middle knots
  float raw[CHUNKS + 1];
  for (int i = 0; i <= CHUNKS; ++i) raw[i] = uniform01(seed, env, s.episode, 0u, 100u + i) * (H_UNITS / 2.0f);
  for (int k = -2; k <= 2; ++k) raw[CHUNKS / 2 + k] = HELIPAD_Y;
  for (int i = 0; i < CHUNKS; ++i) {
    const float a = raw[i > 0 ? i - 1 : CHUNKS], b = raw[i], c = raw[i + 1];
    s.height[i] = 0.33f * (a + b + c);
  }
  for (int k = -1; k <= 1; ++k) s.height[CHUNKS / 2 + k] = HELIPAD_Y;
  const float x0 = W_UNITS / 2.0f, y0 = H_UNITS;
  for (int i = 0; i < 3; ++i)
    for (int k = 0; k < 6; ++k) s.pose[i][k] = 0.f;
  s.pose[0][0] = x0; s.pose[0][1] = y0;
  for (int k = 0; k < 2; ++k) {
    const float sgn = k == 0 ? -1.f : 1.f;
    // leg centre such that its anchor coincides with the lander centre at the initial leg angle
    const float ang = sgn * 0.05f;
    const float bx = sgn * LEG_AWAY / SCALE, by = LEG_DOWN / SCALE;
    const float c = cosf(ang), sn = sinf(ang);
    s.pose[1 + k][0] = x0 - (c * bx - sn * by);
    s.pose[1 + k][1] = y0 - (sn * bx + c * by);
    s.pose[1 + k][2] = ang;
  }
  // initial random push on the hull: a force applied for one step
  const float fx = (2.0f * uniform01(seed, env, s.episode, 0u, 1u) - 1.0f) * INITIAL_RANDOM;
  const float fy = (2.0f * uniform01(seed, env, s.episode, 0u, 2u) - 1.0f) * INITIAL_RANDOM;
  s.pose[0][3] = fx / LANDER_MASS / FPS;
  s.pose[0][4] = fy / LANDER_MASS / FPS;
  s.prev_shaping = 0.f; s.has_shaping = 0;
  s.sleep_time = 0.f; s.ep_return = 0.f; s.steps = 0;
  for (int j = 0; j < 2; ++j)
    for (int k = 0; k < 5; ++k) s.jwarm[j][k] = 0.f;
  for (int b = 0; b < 3; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      s.cwarm_vert[b][k] = -1;
      s.cwarm_imp[b][k][0] = s.cwarm_imp[b][k][1] = 0.f;
    }
}

// One environment step.  action: [main throttle, lateral throttle] in [-1, 1].  Returns the reward; sets terminated /
// truncated and writes the (pre-reset) observation.
NB2D_HD float env_step(LanderState& s, const float* action, unsigned int seed, unsigned int env, float* obs, bool& terminated,
                       bool& truncated) {
  World w;
  build_world(s, w);
  Body& L = w.body[0];
  const float a0 = clampf(action[0], -1.f, 1.f), a1 = clampf(action[1], -1.f, 1.f);
  const float tipx = sinf(L.a), tipy = cosf(L.a);
  const float sidex = -tipy, sidey = tipx;
  const float d0 = (2.0f * uniform01(seed, env, s.episode, (unsigned)s.steps + 1u, 3u) - 1.0f) / SCALE;
  const float d1 = (2.0f * uniform01(seed, env, s.episode, (unsigned)s.steps + 1u, 4u) - 1.0f) / SCALE;
  float m_power = 0.f, s_power = 0.f;
  if (a0 > 0.f) {
    m_power = (clampf(a0, 0.f, 1.f) + 1.0f) * 0.5f;
    const float ox = tipx * (4.0f / SCALE + 2.0f * d0) + sidex * d1;
    const float oy = -tipy * (4.0f / SCALE + 2.0f * d0) - sidey * d1;
    apply_impulse_at(L, -ox * MAIN_ENGINE_POWER * m_power, -oy * MAIN_ENGINE_POWER * m_power, L.x + ox, L.y + oy);
  }
  if (fabsf(a1) > 0.5f) {
    const float dir = a1 > 0.f ? 1.f : -1.f;
    s_power = clampf(fabsf(a1), 0.5f, 1.0f);
    const float ox = tipx * d0 + sidex * (3.0f * d1 + dir * SIDE_ENGINE_AWAY / SCALE);
    const float oy = -tipy * d0 - sidey * (3.0f * d1 + dir * SIDE_ENGINE_AWAY / SCALE);
    apply_impulse_at(L, -ox * SIDE_ENGINE_POWER * s_power, -oy * SIDE_ENGINE_POWER * s_power,
                     L.x + ox - tipx * 17.0f / SCALE, L.y + oy + tipy * SIDE_ENGINE_HEIGHT / SCALE);
  }
  step(w);
  bool hull = false, leg0 = false, leg1 = false;
  for (int c = 0; c < w.ncontact; ++c) {
    if (w.contact[c].body == 0) hull = true;
    if (w.contact[c].body == 1) leg0 = true;
    if (w.contact[c].body == 2) leg1 = true;
  }
  save_world(w, s);
  s.steps += 1;
  observe(s, leg0, leg1, obs);
  const float shaping = -100.0f * sqrtf(obs[0] * obs[0] + obs[1] * obs[1]) - 100.0f * sqrtf(obs[2] * obs[2] + obs[3] * obs[3]) -
                        100.0f * fabsf(obs[4]) + 10.0f * obs[6] + 10.0f * obs[7];
  float reward = s.has_shaping ? shaping - s.prev_shaping : 0.f;
  s.prev_shaping = shaping;
  s.has_shaping = 1;
  reward -= m_power * 0.30f;
  reward -= s_power * 0.03f;
  terminated = false;
  if (hull || fabsf(obs[0]) >= 1.0f) {
    terminated = true;
    reward = -100.0f;
  } else if (s.sleep_time >= 0.5f) {       // at rest: landed
    terminated = true;
    reward = 100.0f;
  }
  truncated = !terminated && s.steps >= MAX_STEPS;
  s.ep_return += reward;
  return reward;
}

}  // namespace nbll
