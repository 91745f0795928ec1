// Goal-predicate tape evaluated per environment: success bit and shaping distance of a task goal, where the reward runs.
// One thread per environment walks the postfix tape (at most 32 terms) with a value stack in registers.  The op codes
// and the semantics of every test mirror tasks/predicates.py::evaluate, which is the oracle of the GPU test.
// Reference: noeira/tasks/predicates.mojo (tape layout), noeira/tasks/gpu_eval.mojo (device evaluation).
#include "common.cuh"

namespace {
using namespace nb;

enum { OP_IN = 0, OP_ON = 1, OP_NEAR = 2, OP_ABOVE = 3, OP_UPRIGHT = 4, OP_AT_REGION = 6, OP_AND = 9, OP_OR = 10, OP_NOT = 11,
       OP_JOINT = 12, OP_ON_BODY = 13 };
constexpr int MAX_TERMS = 32;
constexpr float ON_BAND = 0.03f, ON_BODY_BELOW = 0.01f;

__global__ void __launch_bounds__(128)
goal_eval_kernel(const float* __restrict__ pos, const float* __restrict__ quat, const float* __restrict__ site,
                 const float* __restrict__ rect, const float* __restrict__ geom, const float* __restrict__ qpos, int N, int S,
                 int R, int nq, const int* __restrict__ op, const int* __restrict__ ta, const int* __restrict__ tb,
                 const float* __restrict__ prm, int nterms, unsigned char* __restrict__ ok, float* __restrict__ dist) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= N) return;
  const float* P = pos + (size_t)e * S * 3;
  const float* Q = quat + (size_t)e * S * 4;
  const float* St = site + (size_t)e * R * 3;
  bool sv[MAX_TERMS];
  float dv[MAX_TERMS];
  int sp = 0;
  for (int i = 0; i < nterms; ++i) {
    const int o = op[i], a = ta[i], b = tb[i];
    const float pr = prm[i];
    bool s = false;
    float d = 0.f;
    if (o == OP_AND || o == OP_OR) {
      s = sv[sp - 1];
      d = dv[sp - 1];
      for (int k = 1; k < a; ++k) {
        const bool s2 = sv[sp - 1 - k];
        const float d2 = dv[sp - 1 - k];
        s = (o == OP_AND) ? (s && s2) : (s || s2);
        d = (o == OP_AND) ? d + d2 : fminf(d, d2);
      }
      sp -= a;
    } else if (o == OP_NOT) {
      const bool s1 = sv[--sp];
      s = !s1;
      d = s1 ? 1.f : 0.f;
    } else if (o == OP_IN || o == OP_AT_REGION || o == OP_ON) {
      const float dx = P[a * 3] - St[b * 3], dy = P[a * 3 + 1] - St[b * 3 + 1], dz = P[a * 3 + 2] - St[b * 3 + 2];
      const float* r = rect + b * 5;
      const float ox = fmaxf(r[0] - dx, 0.f) + fmaxf(dx - r[2], 0.f);
      const float oy = fmaxf(r[1] - dy, 0.f) + fmaxf(dy - r[3], 0.f);
      float oz;
      if (o == OP_ON) {
        const float h = dz + geom[a * 3];
        oz = fmaxf(-h, 0.f) + fmaxf(h - pr, 0.f);
      } else {
        oz = fmaxf(fabsf(dz) - r[4], 0.f);
      }
      d = ox + oy + oz;
      s = d <= 0.f;
    } else if (o == OP_ON_BODY) {
      const float dx = P[a * 3] - P[b * 3], dy = P[a * 3 + 1] - P[b * 3 + 1], dz = P[a * 3 + 2] - P[b * 3 + 2];
      const float dxy = fmaxf(sqrtf(dx * dx + dy * dy) - pr, 0.f);
      const float h = dz + geom[a * 3] - geom[b * 3 + 1];
      d = dxy + fmaxf(-ON_BODY_BELOW - h, 0.f) + fmaxf(h - ON_BAND, 0.f);
      s = d <= 0.f;
    } else if (o == OP_NEAR) {
      const float dx = P[a * 3] - P[b * 3], dy = P[a * 3 + 1] - P[b * 3 + 1], dz = P[a * 3 + 2] - P[b * 3 + 2];
      d = fmaxf(sqrtf(dx * dx + dy * dy + dz * dz) - pr, 0.f);
      s = d <= 0.f;
    } else if (o == OP_ABOVE) {
      const float g = P[a * 3 + 2] - P[b * 3 + 2] - pr;
      s = g > 0.f;
      d = fmaxf(-g, 0.f);
    } else if (o == OP_UPRIGHT) {
      const float qx = Q[a * 4 + 1], qy = Q[a * 4 + 2];
      const float zz = 1.f - 2.f * (qx * qx + qy * qy);
      s = zz >= pr;
      d = fmaxf(pr - zz, 0.f);
    } else if (o == OP_JOINT) {
      const float v = qpos[(size_t)e * nq + a];
      if (b == 0) { s = v < pr; d = fmaxf(v - pr, 0.f); }
      else if (b == 1) { s = v <= pr; d = fmaxf(v - pr, 0.f); }
      else if (b == 2) { s = v > pr; d = fmaxf(pr - v, 0.f); }
      else { s = v >= pr; d = fmaxf(pr - v, 0.f); }
    }
    sv[sp] = s;
    dv[sp] = d;
    ++sp;
  }
  ok[e] = (sp == 1 && sv[0]) ? 1 : 0;
  dist[e] = sp == 1 ? dv[0] : 0.f;
}

}  // namespace

extern "C" int nb_goal_eval(const float* pos, const float* quat, const float* site, const float* rect, const float* geom,
                            const float* qpos, int N, int S, int R, int nq, const int* op, const int* a, const int* b,
                            const float* prm, int nterms, unsigned char* ok, float* dist, void* stream) {
  if (N <= 0 || nterms <= 0 || nterms > MAX_TERMS) return NB_ERR_BAD_ARG;
  goal_eval_kernel<<<(N + 127) / 128, 128, 0, (cudaStream_t)stream>>>(pos, quat, site, rect, geom, qpos, N, S, R, nq, op, a, b,
                                                                     prm, nterms, ok, dist);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
