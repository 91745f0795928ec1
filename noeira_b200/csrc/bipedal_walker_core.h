// BipedalWalker on the 2-D rigid-body core: hull + two legs of two segments each on motorised revolute joints with limits,
// rolling random terrain (a smoothed random walk of knot heights), 10 lidar rays against the terrain, the Gymnasium
// observation (24) / shaping reward / termination rules.  Host/device source shared by the CUDA kernel (one thread per
// environment) and the CPU oracle.
// Reference: noeira/envs/bipedal_walker/ (constants, step, lidar), noeira/physics2d/.
#pragma once
#define NB2D_NS nb2d_bw
#define NB2D_MAX_BODIES 5
#define NB2D_MAX_JOINTS 4
#define NB2D_MAX_TERRAIN 64
#include "physics2d.h"

namespace nbbw {
using namespace nb2d_bw;

constexpr float SCALE = 30.0f, FPS = 50.0f;
constexpr float VIEWPORT_W = 600.0f, VIEWPORT_H = 400.0f;
constexpr float MOTORS_TORQUE = 80.0f, SPEED_HIP = 4.0f, SPEED_KNEE = 6.0f;
constexpr float LIDAR_RANGE = 160.0f / SCALE;
constexpr float INITIAL_RANDOM = 5.0f;
constexpr float LEG_DOWN = -8.0f / SCALE, LEG_W = 8.0f / SCALE, LEG_H = 34.0f / SCALE;
constexpr float TERRAIN_STEP = 14.0f / SCALE, TERRAIN_HEIGHT = VIEWPORT_H / SCALE / 4.0f;
constexpr int TERRAIN_LENGTH = 200, TERRAIN_GRASS = 10, TERRAIN_STARTPAD = 20;
constexpr float KNOT_DX = 3.0f * TERRAIN_STEP;       // one height knot per three reference terrain steps
constexpr float FRICTION = 2.5f;
// polygon mass properties at the reference densities (hull 5, legs 1), vertices re-centred on the centre of mass
constexpr float HULL_MASS = 5.4222222f, HULL_INERTIA = 1.9993952f, HULL_CX = -0.02003643f, HULL_CY = -0.00564663f;
constexpr float UPPER_MASS = 0.30222222f, UPPER_INERTIA = 0.03413992f;
constexpr float LOWER_MASS = 0.24177778f, LOWER_INERTIA = 0.02679614f;
constexpr int OBS_DIM = 24, ACT_DIM = 4, N_LIDAR = 10;
constexpr int MAX_STEPS = 1600;

struct WalkerState {
  float pose[5][6];        // hull, upper 1, lower 1, upper 2, lower 2: x, y, angle, vx, vy, omega
  float height[MAX_TERRAIN];
  float prev_shaping;
  float ep_return;
  int steps;
  int has_shaping;
  unsigned int episode;
  float jwarm[4][5];
  int cwarm_vert[5][CONTACTS_PER_BODY];
  float cwarm_imp[5][CONTACTS_PER_BODY][2];
};

NB2D_HD float uniform01(unsigned int seed, unsigned int env, unsigned int episode, unsigned int step, unsigned int k) {
  unsigned int x = seed * 0x9E3779B9u ^ (env + 0x7F4A7C15u) * 0x85EBCA6Bu ^ (episode + 1u) * 0xC2B2AE35u ^ (step + 1u) * 0x27D4EB2Fu ^
                   (k + 1u) * 0x165667B1u;
  x ^= x >> 16; x *= 0x7FEB352Du; x ^= x >> 15; x *= 0x846CA68Bu; x ^= x >> 16;
  return (float)(x >> 8) * (1.0f / 16777216.0f);
}

NB2D_HD void build_world(const WalkerState& s, const float* action, World& w) {
  w.nbody = 5; w.njoint = 4; w.ncontact = 0;
  w.gx = 0.f; w.gy = -10.0f; w.dt = 1.0f / FPS;
  w.vel_iters = 90; w.pos_iters = 8;
  w.baumgarte = 0.2f; w.slop = 0.005f; w.max_correction = 0.2f;
  w.sleep_time = 0.f;
  const float hx[5] = {-30.f, -30.f, 34.f, 34.f, 6.f}, hy[5] = {9.f, -8.f, -8.f, 1.f, 9.f};      // counter-clockwise
  for (int i = 0; i < 5; ++i) {
    Body& b = w.body[i];
    b.x = s.pose[i][0]; b.y = s.pose[i][1]; b.a = s.pose[i][2];
    b.vx = s.pose[i][3]; b.vy = s.pose[i][4]; b.w = s.pose[i][5];
    b.fx = b.fy = b.tq = 0.f;
    b.friction = FRICTION;
    if (i == 0) {
      b.inv_m = 1.0f / HULL_MASS; b.inv_i = 1.0f / HULL_INERTIA;
      b.nvert = 5;
      for (int v = 0; v < 5; ++v) { b.px[v] = hx[v] / SCALE - HULL_CX; b.py[v] = hy[v] / SCALE - HULL_CY; }
    } else {
      const bool lower = (i % 2) == 0;
      b.inv_m = 1.0f / (lower ? LOWER_MASS : UPPER_MASS); b.inv_i = 1.0f / (lower ? LOWER_INERTIA : UPPER_INERTIA);
      b.nvert = 4;
      const float hw = (lower ? 0.8f : 1.0f) * LEG_W / 2.0f, hh = LEG_H / 2.0f;
      b.px[0] = -hw; b.py[0] = -hh; b.px[1] = hw; b.py[1] = -hh; b.px[2] = hw; b.py[2] = hh; b.px[3] = -hw; b.py[3] = hh;
    }
  }
  for (int k = 0; k < 4; ++k) {
    Revolute& j = w.joint[k];
    const bool knee = (k % 2) == 1;
    const int leg = k / 2;
    if (!knee) {            // hip: hull → upper leg
      j.a = 0; j.b = 1 + 2 * leg;
      j.ax = 0.f - HULL_CX; j.ay = LEG_DOWN - HULL_CY;
      j.bx = 0.f; j.by = LEG_H / 2.0f;
      j.lower = -0.8f; j.upper = 1.1f;
    } else {                // knee: upper → lower leg
      j.a = 1 + 2 * leg; j.b = 2 + 2 * leg;
      j.ax = 0.f; j.ay = -LEG_H / 2.0f;
      j.bx = 0.f; j.by = LEG_H / 2.0f;
      j.lower = -1.6f; j.upper = -0.1f;
    }
    j.ref = 0.f;
    j.enable_motor = 1; j.enable_limit = 1;
    const float a = action ? clampf(action[k], -1.f, 1.f) : 0.f;
    j.motor_speed = (knee ? SPEED_KNEE : SPEED_HIP) * (a > 0.f ? 1.f : (a < 0.f ? -1.f : 0.f));
    j.max_torque = MOTORS_TORQUE * fabsf(a);
  }
  clear_warm_start(w);
  for (int j = 0; j < 4; ++j)
    for (int k = 0; k < 5; ++k) w.jwarm[j][k] = s.jwarm[j][k];
  for (int b = 0; b < 5; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      w.cwarm_vert[b][k] = s.cwarm_vert[b][k];
      w.cwarm_imp[b][k][0] = s.cwarm_imp[b][k][0];
      w.cwarm_imp[b][k][1] = s.cwarm_imp[b][k][1];
    }
  w.terrain.n = MAX_TERRAIN;
  w.terrain.x0 = 0.f;
  w.terrain.dx = KNOT_DX;
  for (int i = 0; i < MAX_TERRAIN; ++i) w.terrain.h[i] = s.height[i];
}

NB2D_HD void save_world(const World& w, WalkerState& s) {
  for (int i = 0; i < 5; ++i) {
    const Body& b = w.body[i];
    s.pose[i][0] = b.x; s.pose[i][1] = b.y; s.pose[i][2] = b.a;
    s.pose[i][3] = b.vx; s.pose[i][4] = b.vy; s.pose[i][5] = b.w;
  }
  for (int j = 0; j < 4; ++j)
    for (int k = 0; k < 5; ++k) s.jwarm[j][k] = w.jwarm[j][k];
  for (int b = 0; b < 5; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      s.cwarm_vert[b][k] = w.cwarm_vert[b][k];
      s.cwarm_imp[b][k][0] = w.cwarm_imp[b][k][0];
      s.cwarm_imp[b][k][1] = w.cwarm_imp[b][k][1];
    }
}

NB2D_HD float terrain_height(const WalkerState& s, float x) {
  float u = x / KNOT_DX;
  int i = (int)floorf(u);
  i = i < 0 ? 0 : (i > MAX_TERRAIN - 2 ? MAX_TERRAIN - 2 : i);
  const float f = u - (float)i;
  return s.height[i] + (s.height[i + 1] - s.height[i]) * f;
}

// fraction of the ray (x, y) + t (dx, dy), t in [0, 1], before it goes below the terrain (1 = no hit): 32 marching steps,
// the crossing refined linearly between the last point above and the first below
NB2D_HD float lidar_fraction(const WalkerState& s, float x, float y, float dx, float dy) {
  float prev_t = 0.f, prev_g = y - terrain_height(s, x);
  if (prev_g <= 0.f) return 0.f;
  for (int k = 1; k <= 32; ++k) {
    const float t = (float)k / 32.0f;
    const float g = (y + t * dy) - terrain_height(s, x + t * dx);
    if (g <= 0.f) return prev_t + (t - prev_t) * prev_g / (prev_g - g);
    prev_t = t; prev_g = g;
  }
  return 1.0f;
}

NB2D_HD void observe(const WalkerState& s, bool leg1, bool leg2, float* obs) {
  const float* H = s.pose[0];
  obs[0] = H[2];
  obs[1] = 2.0f * H[5] / FPS;
  obs[2] = 0.3f * H[3] * (VIEWPORT_W / SCALE) / FPS;
  obs[3] = 0.3f * H[4] * (VIEWPORT_H / SCALE) / FPS;
  for (int leg = 0; leg < 2; ++leg) {
    const float* U = s.pose[1 + 2 * leg];
    const float* L = s.pose[2 + 2 * leg];
    float* o = obs + 4 + 5 * leg;
    o[0] = U[2] - H[2];                    // hip angle
    o[1] = (U[5] - H[5]) / SPEED_HIP;
    o[2] = L[2] - U[2] + 1.0f;             // knee angle + 1
    o[3] = (L[5] - U[5]) / SPEED_KNEE;
    o[4] = (leg == 0 ? leg1 : leg2) ? 1.f : 0.f;
  }
  // the hull's body origin (where the lidar sits) from its centre of mass
  const float c = cosf(H[2]), sn = sinf(H[2]);
  const float ox = H[0] - (c * HULL_CX - sn * HULL_CY), oy = H[1] - (sn * HULL_CX + c * HULL_CY);
  for (int i = 0; i < N_LIDAR; ++i) {
    const float ang = 1.5f * (float)i / 10.0f;
    obs[14 + i] = lidar_fraction(s, ox, oy, sinf(ang) * LIDAR_RANGE, -cosf(ang) * LIDAR_RANGE);
  }
}

NB2D_HD void reset(WalkerState& s, unsigned int seed, unsigned int env) {
  s.episode += 1u;
  // terrain: the reference's velocity random walk, one knot per three terrain steps, flat start pad
  float y = TERRAIN_HEIGHT, vel = 0.f;
  int knot = 0;
  for (int i = 0; i < TERRAIN_LENGTH && knot < MAX_TERRAIN; ++i) {
    vel = 0.8f * vel + 0.01f * (TERRAIN_HEIGHT > y ? 1.f : (TERRAIN_HEIGHT < y ? -1.f : 0.f));
    if (i > TERRAIN_STARTPAD) vel += (2.0f * uniform01(seed, env, s.episode, 0u, 100u + i) - 1.0f) / SCALE;
    y += vel;
    if (i % 3 == 0) s.height[knot++] = i <= TERRAIN_STARTPAD ? TERRAIN_HEIGHT : y;
  }
  for (; knot < MAX_TERRAIN; ++knot) s.height[knot] = y;
  // feet just above the start pad (hip below the hull origin by -LEG_DOWN, two leg segments)
  const float x0 = TERRAIN_STEP * TERRAIN_STARTPAD / 2.0f, y0 = TERRAIN_HEIGHT + 2.0f * LEG_H - LEG_DOWN + 0.02f;
  for (int i = 0; i < 5; ++i)
    for (int k = 0; k < 6; ++k) s.pose[i][k] = 0.f;
  s.pose[0][0] = x0 + HULL_CX; s.pose[0][1] = y0 + HULL_CY;
  for (int leg = 0; leg < 2; ++leg) {
    const float ang = (leg == 0 ? -1.f : 1.f) * 0.05f;
    // the upper leg hangs from the hip anchor, the lower leg from the knee, both at the initial angle
    const float hipx = x0, hipy = y0 + LEG_DOWN;
    const float c = cosf(ang), sn = sinf(ang);
    float* U = s.pose[1 + 2 * leg];
    float* L = s.pose[2 + 2 * leg];
    U[0] = hipx - (-sn * (LEG_H / 2.0f)); U[1] = hipy - (c * (LEG_H / 2.0f)); U[2] = ang;
    const float kx = U[0] + (-sn * (-LEG_H / 2.0f)), ky = U[1] + (c * (-LEG_H / 2.0f));
    L[0] = kx - (-sn * (LEG_H / 2.0f)); L[1] = ky - (c * (LEG_H / 2.0f)); L[2] = ang;
  }
  const float fx = (2.0f * uniform01(seed, env, s.episode, 0u, 1u) - 1.0f) * INITIAL_RANDOM;
  s.pose[0][3] = fx / HULL_MASS / FPS;
  s.prev_shaping = 0.f; s.has_shaping = 0;
  s.ep_return = 0.f; s.steps = 0;
  for (int j = 0; j < 4; ++j)
    for (int k = 0; k < 5; ++k) s.jwarm[j][k] = 0.f;
  for (int b = 0; b < 5; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      s.cwarm_vert[b][k] = -1;
      s.cwarm_imp[b][k][0] = s.cwarm_imp[b][k][1] = 0.f;
    }
}

// One environment step.  action: hip 1, knee 1, hip 2, knee 2 in [-1, 1] (sign = motor direction, magnitude = torque
// fraction).  Returns the reward; sets terminated / truncated and writes the (pre-reset) observation.
NB2D_HD float env_step(WalkerState& s, const float* action, unsigned int seed, unsigned int env, float* obs, bool& terminated,
                       bool& truncated) {
  World w;
  build_world(s, action, w);
  step(w);
  bool hull = false, leg1 = false, leg2 = false;
  for (int c = 0; c < w.ncontact; ++c) {
    if (w.contact[c].body == 0) hull = true;
    if (w.contact[c].body == 2) leg1 = true;
    if (w.contact[c].body == 4) leg2 = true;
  }
  save_world(w, s);
  s.steps += 1;
  observe(s, leg1, leg2, obs);
  const float px = s.pose[0][0] - HULL_CX;
  const float shaping = 130.0f * px / SCALE - 5.0f * fabsf(obs[0]);
  float reward = s.has_shaping ? shaping - s.prev_shaping : 0.f;
  s.prev_shaping = shaping;
  s.has_shaping = 1;
  for (int k = 0; k < 4; ++k) reward -= 0.00035f * MOTORS_TORQUE * clampf(fabsf(action[k]), 0.f, 1.f);
  terminated = false;
  if (hull || px < 0.f) {
    terminated = true;
    reward = -100.0f;
  } else if (px > (float)(TERRAIN_LENGTH - TERRAIN_GRASS) * TERRAIN_STEP) {
    terminated = true;
  }
  truncated = !terminated && s.steps >= MAX_STEPS;
  s.ep_return += reward;
  (void)seed; (void)env;
  return reward;
}

}  // namespace nbbw
