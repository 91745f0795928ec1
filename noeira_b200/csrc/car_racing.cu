// Top-down car racing: one fused step kernel (tile test + tire model + rigid hull, one warp per lane of the batch) and the
// ego-centric grey-scale camera (one CTA per lane: cull the track to the view, then to blocks of 8 x 8 pixels, one warp each).
// The tire model is the slip model of Gymnasium's car_dynamics.py on a single rigid hull, as the reference's
// noeira/physics2d/car/ does (wheel_friction.mojo, car_dynamics.mojo); the image palette (grass 0.3, road 0.7, car 1.0)
// follows noeira/envs/car_racing/car_racing_pixel.mojo.
#include "common.cuh"

namespace {

struct CarParams {
  float dt, engine_power, brake_force, wheel_moment, wheel_radius, friction_limit, friction_coef, grass_friction;
  float steer_limit, steer_speed, steer_gain, hull_mass, hull_inertia, half_width, playfield, tile_reward, lap_fraction;
  float wheel_x[4], wheel_y[4];
};

constexpr int CAR_HDR = 16;   // x y angle vx vy omega | joint_fl joint_fr | wheel omega x4 | track id | visited | gas | spare

__device__ __forceinline__ float seg_dist2(float qx, float qy, float ax, float ay, float bx, float by) {
  const float ex = bx - ax, ey = by - ay, px = qx - ax, py = qy - ay;
  const float l2 = ex * ex + ey * ey;
  float t = l2 > 0.f ? (px * ex + py * ey) / l2 : 0.f;
  t = fminf(fmaxf(t, 0.f), 1.f);
  const float dx = px - t * ex, dy = py - t * ey;
  return dx * dx + dy * dy;
}

struct CarStepOut {      // valid in lane 0
  float hdr[CAR_HDR];
  float reward;
  int term;
};

// One warp advances one lane of the batch: the lanes share the tiles (surface under each wheel, visit flags written to
// ``o_flags``), lane 0 integrates the tire model and the hull.  ``s`` is the state row, ``a`` its action (steer, gas, brake).
__device__ __forceinline__ void car_step_warp(const float* __restrict__ s, const float* __restrict__ a, const float* __restrict__ tr,
                                              int T, float* __restrict__ o_flags, const CarParams& P, int lane, CarStepOut& R) {
  const float x = s[0], y = s[1], ang = s[2], vx = s[3], vy = s[4], om = s[5];
  float joint[4] = {s[6], s[7], 0.f, 0.f}, womega[4] = {s[8], s[9], s[10], s[11]};
  float gas_state = s[14];
  const float ca = cosf(ang), sa = sinf(ang);
  float wx[4], wy[4], rx[4], ry[4];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    rx[w] = ca * P.wheel_x[w] - sa * P.wheel_y[w];
    ry[w] = sa * P.wheel_x[w] + ca * P.wheel_y[w];
    wx[w] = x + rx[w];
    wy[w] = y + ry[w];
  }
  // tiles under the wheels: friction surface, visit flags, reward
  const float w2 = P.half_width * P.half_width;
  float dmin[4] = {3.4e38f, 3.4e38f, 3.4e38f, 3.4e38f};
  int fresh = 0;
  for (int j = lane; j < T; j += 32) {
    const int j1 = j + 1 == T ? 0 : j + 1;
    const float ax = tr[2 * j], ay = tr[2 * j + 1], bx = tr[2 * j1], by = tr[2 * j1 + 1];
    bool hit = false;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float d = seg_dist2(wx[w], wy[w], ax, ay, bx, by);
      dmin[w] = fminf(dmin[w], d);
      hit |= d <= w2;
    }
    const float was = s[CAR_HDR + j];
    if (hit && was == 0.f) ++fresh;
    o_flags[j] = (hit || was != 0.f) ? 1.f : 0.f;
  }
#pragma unroll
  for (int sft = 16; sft; sft >>= 1) {
    fresh += __shfl_xor_sync(0xffffffffu, fresh, sft);
#pragma unroll
    for (int w = 0; w < 4; ++w) dmin[w] = fminf(dmin[w], __shfl_xor_sync(0xffffffffu, dmin[w], sft));
  }
  if (lane) return;
  const float steer = fminf(fmaxf(a[0], -1.f), 1.f), gas = fminf(fmaxf(a[1], 0.f), 1.f), brake = fminf(fmaxf(a[2], 0.f), 1.f);
  gas_state += fminf(gas - gas_state, 0.1f);
  float fx = 0.f, fy = 0.f, tq = 0.f;
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    if (w < 2) {   // steering servo
      const float diff = -steer * P.steer_limit - joint[w];
      const float rate = copysignf(fminf(P.steer_gain * fabsf(diff), P.steer_speed), diff);
      const float stepv = rate * P.dt;
      joint[w] += fabsf(stepv) > fabsf(diff) ? diff : stepv;
    } else {       // engine on the rear axle
      womega[w] += P.dt * P.engine_power * gas_state / P.wheel_moment / (fabsf(womega[w]) + 5.f);
    }
    if (brake >= 0.9f) womega[w] = 0.f;
    else if (brake > 0.f) {
      const float val = fminf(P.brake_force * brake, fabsf(womega[w]));
      womega[w] -= copysignf(val, womega[w]);
    }
    const float wa = ang + joint[w], cw = cosf(wa), sw = sinf(wa);
    const float fdx = -sw, fdy = cw, sdx = cw, sdy = sw;
    const float pvx = vx - om * ry[w], pvy = vy + om * rx[w];
    const float vf = fdx * pvx + fdy * pvy, vs = sdx * pvx + sdy * pvy;
    float ff = (-vf + womega[w] * P.wheel_radius) * P.friction_coef, pf = -vs * P.friction_coef;
    const float lim = P.friction_limit * (dmin[w] <= w2 ? 1.f : P.grass_friction);
    const float mag = sqrtf(ff * ff + pf * pf);
    if (mag > lim) { ff *= lim / mag; pf *= lim / mag; }
    womega[w] -= P.dt * ff * P.wheel_radius / P.wheel_moment;
    const float gx = pf * sdx + ff * fdx, gy = pf * sdy + ff * fdy;
    fx += gx; fy += gy; tq += rx[w] * gy - ry[w] * gx;
  }
  const float vx2 = vx + P.dt * fx / P.hull_mass, vy2 = vy + P.dt * fy / P.hull_mass, om2 = om + P.dt * tq / P.hull_inertia;
  const float x2 = x + P.dt * vx2, y2 = y + P.dt * vy2;
  const float visited = s[13] + (float)fresh;
  const bool out = fabsf(x2) > P.playfield || fabsf(y2) > P.playfield;
  const bool lap = visited >= P.lap_fraction * (float)T;
  float* o = R.hdr;
  o[0] = x2; o[1] = y2; o[2] = ang + P.dt * om2; o[3] = vx2; o[4] = vy2; o[5] = om2;
  o[6] = joint[0]; o[7] = joint[1];
  o[8] = womega[0]; o[9] = womega[1]; o[10] = womega[2]; o[11] = womega[3];
  o[12] = s[12]; o[13] = visited; o[14] = gas_state; o[15] = s[15];
  R.reward = out ? -100.f : -0.1f + P.tile_reward * (float)fresh;
  R.term = (out || lap) ? 1 : 0;
}

// state [N, CAR_HDR + T] -> next [N, CAR_HDR + T]; action [N, lda] (steer, gas, brake); track [K, T, 2]
__global__ void car_step_kernel(const float* __restrict__ state, const float* __restrict__ action, int lda,
                                const float* __restrict__ track, int T, float* __restrict__ next, float* __restrict__ reward,
                                float* __restrict__ term, int N, CarParams P) {
  const int env = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (env >= N) return;
  const int S = CAR_HDR + T;
  const float* s = state + (size_t)env * S;
  float* o = next + (size_t)env * S;
  CarStepOut R;
  car_step_warp(s, action + (size_t)env * lda, track + (size_t)((int)s[12]) * T * 2, T, o + CAR_HDR, P, lane, R);
  if (lane) return;
#pragma unroll
  for (int i = 0; i < CAR_HDR; ++i) o[i] = R.hdr[i];
  reward[env] = R.reward;
  term[env] = R.term ? 1.f : 0.f;
}

struct CarEnvIO {
  const float* state; float* state_out; float* pre_out;          // [N, CAR_HDR + T]: current, after reset, before reset
  const float* action; int lda;
  const float* track; int T, K;
  const float* start_pose;                                        // [K, 3] x, y, heading at tile 0
  int* steps; float* ep_return; int* episodes;                    // [N]
  float* reward; float* done; float* term; float* finished_return; float* ep_stats;
  float* obs; float* next_obs;                                    // [N, obs_dim] fp32 (may be null)
  __nv_bfloat16* obs_bf16; __nv_bfloat16* next_obs_bf16; int ld_bf16;   // (may be null)
  int N, obs_dim, lookahead, stride, max_steps, do_reset;
  unsigned seed;
};

__device__ __forceinline__ void car_write_obs(const float* h, const float* tr, int T, int near, int lookahead, int stride,
                                              float* o32, __nv_bfloat16* o16, int lane) {
  // 13 values from the header and the speed, then look-ahead points in the car frame (x right, y forward)
  const float sa = sinf(h[2]), ca = cosf(h[2]);
  for (int i = lane; i < 13 + 2 * lookahead; i += 32) {
    float v;
    if (i < 12) v = h[i];
    else if (i == 12) v = sqrtf(h[3] * h[3] + h[4] * h[4]);
    else {
      const int l = (i - 13) >> 1;
      const int idx = (near + (1 + l) * stride) % T;
      const float rx = tr[2 * idx] - h[0], ry = tr[2 * idx + 1] - h[1];
      v = ((i - 13) & 1) ? (-sa * rx + ca * ry) : (ca * rx + sa * ry);
    }
    if (o32) o32[i] = v;
    if (o16) o16[i] = __float2bfloat16(v);
  }
}

// The whole environment step for one lane of the batch per warp: dynamics, reward, time limit, episode statistics,
// the observation of the successor, the reset (a new track from a counter hash, the start pose of that track, cleared visit
// flags) and the observation after it.  ``state_out`` may be ``state`` itself: every read of the old row precedes the
// warp-wide exchange of lane 0's results, every write of the new row follows it.
__global__ void car_env_step_kernel(CarEnvIO io, CarParams P) {
  const int env = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (env >= io.N) return;
  const int T = io.T, S = CAR_HDR + T;
  const float* s = io.state + (size_t)env * S;
  float* pre = io.pre_out + (size_t)env * S;
  float* post = io.state_out + (size_t)env * S;
  const float* tr = io.track + (size_t)((int)s[12]) * T * 2;
  CarStepOut R;
  car_step_warp(s, io.action + (size_t)env * io.lda, tr, T, pre + CAR_HDR, P, lane, R);
  float h[CAR_HDR];
#pragma unroll
  for (int i = 0; i < CAR_HDR; ++i) h[i] = __shfl_sync(0xffffffffu, R.hdr[i], 0);
  const int term = __shfl_sync(0xffffffffu, R.term, 0);
  const float reward = __shfl_sync(0xffffffffu, R.reward, 0);
  const int steps = io.steps[env] + 1;
  const int done = term || steps >= io.max_steps;
  // nearest tile to the hull (for the look-ahead points)
  int near = 0;
  if (io.lookahead > 0) {
    float best = 3.4e38f;
    for (int j = lane; j < T; j += 32) {
      const float dx = tr[2 * j] - h[0], dy = tr[2 * j + 1] - h[1], d = dx * dx + dy * dy;
      if (d < best) { best = d; near = j; }
    }
#pragma unroll
    for (int sft = 16; sft; sft >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, sft);
      const int on = __shfl_xor_sync(0xffffffffu, near, sft);
      if (ob < best || (ob == best && on < near)) { best = ob; near = on; }
    }
  }
  __syncwarp();                                   // the visit flags of ``pre`` are read back below
  if (lane < CAR_HDR) pre[lane] = h[lane];
  car_write_obs(h, tr, T, near, io.lookahead, io.stride, io.next_obs ? io.next_obs + (size_t)env * io.obs_dim : nullptr,
                io.next_obs_bf16 ? io.next_obs_bf16 + (size_t)env * io.ld_bf16 : nullptr, lane);
  const bool reset = done && io.do_reset;
  const float ret = io.ep_return[env] + reward;
  if (lane == 0) {
    io.reward[env] = reward;
    io.term[env] = term ? 1.f : 0.f;
    io.done[env] = done ? 1.f : 0.f;
    if (io.ep_stats) {
      atomicAdd(io.ep_stats + 2, reward);
      atomicAdd(io.ep_stats + 3, 1.f);
      if (reset) { atomicAdd(io.ep_stats + 0, ret); atomicAdd(io.ep_stats + 1, 1.f); }
    }
    if (reset && io.finished_return) io.finished_return[env] = ret;
    io.ep_return[env] = reset ? 0.f : ret;
    io.steps[env] = reset ? 0 : steps;
  }
  if (!reset) {
    for (int j = lane; j < S; j += 32) post[j] = j < CAR_HDR ? h[j] : pre[j];
    car_write_obs(h, tr, T, near, io.lookahead, io.stride, io.obs ? io.obs + (size_t)env * io.obs_dim : nullptr,
                  io.obs_bf16 ? io.obs_bf16 + (size_t)env * io.ld_bf16 : nullptr, lane);
    return;
  }
  int ep = 0;
  if (lane == 0) { ep = io.episodes[env] + 1; io.episodes[env] = ep; }
  ep = __shfl_sync(0xffffffffu, ep, 0);
  unsigned z = io.seed * 0x9E3779B9u + (unsigned)env * 0x85EBCA6Bu + (unsigned)ep * 0xC2B2AE35u;    // a counter hash
  z ^= z >> 16; z *= 0x7FEB352Du; z ^= z >> 15; z *= 0x846CA68Bu; z ^= z >> 16;
  const int tid = (int)(z % (unsigned)io.K);
  float g[CAR_HDR];
#pragma unroll
  for (int i = 0; i < CAR_HDR; ++i) g[i] = 0.f;
  g[0] = io.start_pose[3 * tid]; g[1] = io.start_pose[3 * tid + 1]; g[2] = io.start_pose[3 * tid + 2];
  g[12] = (float)tid;
  for (int j = lane; j < S; j += 32) post[j] = j < CAR_HDR ? g[j] : 0.f;
  car_write_obs(g, io.track + (size_t)tid * T * 2, T, 0, io.lookahead, io.stride,
                io.obs ? io.obs + (size_t)env * io.obs_dim : nullptr,
                io.obs_bf16 ? io.obs_bf16 + (size_t)env * io.ld_bf16 : nullptr, lane);
}

// pose = the state rows (x, y, angle first, track id at 12); image [N, res, res], the car at (res/2, cy) heading up
template <typename Pix>
__global__ void car_render_kernel(const float* __restrict__ state, int S, const float* __restrict__ track, int T,
                                  Pix* __restrict__ img, int res, float px_per_unit, float cy, float half_width,
                                  float car_hw, float car_hl) {
  extern __shared__ float seg[];   // culled segments: ax ay bx by
  __shared__ int nseg;
  const int env = blockIdx.x;
  const float* s = state + (size_t)env * S;
  const float x = s[0], y = s[1], ang = s[2];
  const float* tr = track + (size_t)((int)s[12]) * T * 2;
  if (threadIdx.x == 0) nseg = 0;
  __syncthreads();
  const float ca = cosf(ang), sa = sinf(ang);
  // the view is a square of res / px_per_unit world units; its circumscribed circle about the view centre
  const float span = (float)res / px_per_unit;
  const float vcy = (cy - 0.5f * (float)res) / px_per_unit;        // view centre ahead of the car by this much
  const float ccx = x + (-sa) * vcy, ccy = y + ca * vcy;
  const float R = 0.7072f * span + half_width;
  for (int j = threadIdx.x; j < T; j += blockDim.x) {
    const int j1 = j + 1 == T ? 0 : j + 1;
    const float ax = tr[2 * j], ay = tr[2 * j + 1], bx = tr[2 * j1], by = tr[2 * j1 + 1];
    if (seg_dist2(ccx, ccy, ax, ay, bx, by) <= R * R) {
      const int k = atomicAdd(&nseg, 1);
      seg[4 * k] = ax; seg[4 * k + 1] = ay; seg[4 * k + 2] = bx; seg[4 * k + 3] = by;
    }
  }
  __syncthreads();
  const int n = nseg;
  const float w2 = half_width * half_width;
  // second level of culling: the image in blocks of 8 x 8 pixels, one warp per block.  The lanes test the view's segments
  // against the block's circumscribed circle (grown by the road's half width) and compact the survivors into the warp's
  // list; most blocks of grass keep none, blocks of road two or three, so a pixel tests a handful of segments.
  int* mine = reinterpret_cast<int*>(seg + 4 * T) + (threadIdx.x >> 5) * T;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int nb = (res + 7) >> 3;
  const float rb = 5.657f / px_per_unit + half_width;                  // half diagonal of 8 pixels, in world units
  for (int b = warp; b < nb * nb; b += nwarp) {
    const int by = b / nb, bx = b - by * nb;
    const float clx = ((float)(bx * 8 + 4) - 0.5f * (float)res) / px_per_unit, cly = (cy - (float)(by * 8 + 4)) / px_per_unit;
    const float bcx = x + ca * clx - sa * cly, bcy = y + sa * clx + ca * cly;
    int m = 0;
    for (int k0 = 0; k0 < n; k0 += 32) {
      const int k = k0 + lane;
      const bool hit = k < n && seg_dist2(bcx, bcy, seg[4 * k], seg[4 * k + 1], seg[4 * k + 2], seg[4 * k + 3]) <= rb * rb;
      const unsigned bal = __ballot_sync(0xffffffffu, hit);
      if (hit) mine[m + __popc(bal & ((1u << lane) - 1u))] = k;
      m += __popc(bal);
    }
    __syncwarp();
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int p = lane + 32 * half;
      const int i = by * 8 + (p >> 3), j = bx * 8 + (p & 7);
      if (i < res && j < res) {
        const float lx = ((float)j + 0.5f - 0.5f * (float)res) / px_per_unit, ly = (cy - ((float)i + 0.5f)) / px_per_unit;
        float v = 0.3f;
        if (fabsf(lx) <= car_hw && fabsf(ly) <= car_hl) v = 1.0f;
        else {
          const float qx = x + ca * lx - sa * ly, qy = y + sa * lx + ca * ly;
          for (int q = 0; q < m; ++q) {
            const int k = mine[q];
            if (seg_dist2(qx, qy, seg[4 * k], seg[4 * k + 1], seg[4 * k + 2], seg[4 * k + 3]) <= w2) { v = 0.7f; break; }
          }
        }
        img[(size_t)env * res * res + (size_t)i * res + j] = sizeof(Pix) == 1 ? (Pix)(v * 255.f + 0.5f) : (Pix)v;
      }
    }
    __syncwarp();
  }
}

}  // namespace

extern "C" {

// params: 17 scalars in the order of CarParams followed by wheel_x[4], wheel_y[4] (25 floats, host memory)
int nb_car_step(const float* state, const float* action, int lda, const float* track, int T, float* next, float* reward,
                float* term, int N, const float* params, void* stream) {
  if (N <= 0 || T <= 0 || lda < 3) return NB_ERR_BAD_ARG;
  CarParams P;
  float* dst = &P.dt;
  for (int i = 0; i < 17; ++i) dst[i] = params[i];
  for (int w = 0; w < 4; ++w) { P.wheel_x[w] = params[17 + w]; P.wheel_y[w] = params[21 + w]; }
  const int tpb = 128;
  car_step_kernel<<<(N * 32 + tpb - 1) / tpb, tpb, 0, (cudaStream_t)stream>>>(state, action, lda, track, T, next, reward, term, N, P);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_car_env_step(const void* state, void* state_out, void* pre_out, const void* action, int lda, const void* track, int T, int K,
                    const void* start_pose, void* steps, void* ep_return, void* episodes, void* reward, void* done, void* term,
                    void* finished_return, void* ep_stats, void* obs, void* next_obs, void* obs_bf16, void* next_obs_bf16,
                    int ld_bf16, int N, int obs_dim, int lookahead, int stride, int max_steps, int do_reset, unsigned seed,
                    const float* params, void* stream) {
  if (N <= 0 || T <= 0 || K <= 0 || lda < 3 || obs_dim != 13 + 2 * lookahead || state == pre_out || state_out == pre_out)
    return NB_ERR_BAD_ARG;
  CarParams P;
  float* dst = &P.dt;
  for (int i = 0; i < 17; ++i) dst[i] = params[i];
  for (int w = 0; w < 4; ++w) { P.wheel_x[w] = params[17 + w]; P.wheel_y[w] = params[21 + w]; }
  CarEnvIO io;
  io.state = (const float*)state; io.state_out = (float*)state_out; io.pre_out = (float*)pre_out;
  io.action = (const float*)action; io.lda = lda; io.track = (const float*)track; io.T = T; io.K = K;
  io.start_pose = (const float*)start_pose; io.steps = (int*)steps; io.ep_return = (float*)ep_return; io.episodes = (int*)episodes;
  io.reward = (float*)reward; io.done = (float*)done; io.term = (float*)term; io.finished_return = (float*)finished_return;
  io.ep_stats = (float*)ep_stats; io.obs = (float*)obs; io.next_obs = (float*)next_obs;
  io.obs_bf16 = (__nv_bfloat16*)obs_bf16; io.next_obs_bf16 = (__nv_bfloat16*)next_obs_bf16; io.ld_bf16 = ld_bf16;
  io.N = N; io.obs_dim = obs_dim; io.lookahead = lookahead; io.stride = stride; io.max_steps = max_steps; io.do_reset = do_reset;
  io.seed = seed;
  const int tpb = 128;
  car_env_step_kernel<<<(N * 32 + tpb - 1) / tpb, tpb, 0, (cudaStream_t)stream>>>(io, P);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

// img: fp32 values 0.3 / 0.7 / 1.0, or with ``u8`` bytes 77 / 179 / 255
int nb_car_render(const float* state, int S, const float* track, int T, void* img, int N, int res, float px_per_unit,
                  float cy, float half_width, float car_hw, float car_hl, int u8, void* stream) {
  if (N <= 0 || T <= 0 || res <= 0 || (size_t)T * 48 > 48 * 1024) return NB_ERR_BAD_ARG;
  const size_t smem = (size_t)T * 16 + 8 * (size_t)T * 4;
  if (u8)
    car_render_kernel<unsigned char><<<N, 256, smem, (cudaStream_t)stream>>>(state, S, track, T, (unsigned char*)img, res, px_per_unit,
                                                                            cy, half_width, car_hw, car_hl);
  else
    car_render_kernel<float><<<N, 256, smem, (cudaStream_t)stream>>>(state, S, track, T, (float*)img, res, px_per_unit, cy, half_width,
                                                                    car_hw, car_hl);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
