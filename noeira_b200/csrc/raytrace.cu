// Ray-traced cameras for batched worlds: one thread per (world, camera, pixel); primary ray against every geom of
// the world (plane / sphere / capsule / box), Lambert + ambient shading with one directional light, hard shadows
// from a second ray, checkerboard ground, sky gradient.  Output uint8 RGB [W, cam, H, Wpx, 3] and fp32 depth.
// Reference: noeira/physics3d/raytrace/batch.mojo (one thread per (world, pixel)), render.mojo, appearance.mojo;
// host oracle host_render.mojo.  The same math runs on the CPU in physics/raytrace.py (the oracle of the tests).
#include "common.cuh"

namespace {

struct RtGeom {      // 24 floats per geom in the table
  float type;        // 0 plane (z = 0 of its frame), 1 sphere, 2 capsule (axis = local z), 3 box
  float body;        // body index, -1 = world frame
  float pos[3];      // local position in the body frame
  float rot[9];      // local rotation (row-major)
  float size[3];     // sphere: r; capsule: r, half length; box: half extents
  float rgba[4];
  float pad[3];
};
static_assert(sizeof(RtGeom) == 24 * 4, "geom record");

struct Hit { float t; float n[3]; int geom; };

__device__ __forceinline__ void mat_vec(const float* m, const float* v, float* o) {
  o[0] = m[0] * v[0] + m[1] * v[1] + m[2] * v[2];
  o[1] = m[3] * v[0] + m[4] * v[1] + m[5] * v[2];
  o[2] = m[6] * v[0] + m[7] * v[1] + m[8] * v[2];
}
__device__ __forceinline__ void matT_vec(const float* m, const float* v, float* o) {
  o[0] = m[0] * v[0] + m[3] * v[1] + m[6] * v[2];
  o[1] = m[1] * v[0] + m[4] * v[1] + m[7] * v[2];
  o[2] = m[2] * v[0] + m[5] * v[1] + m[8] * v[2];
}
__device__ __forceinline__ float dot3(const float* a, const float* b) { return a[0] * b[0] + a[1] * b[1] + a[2] * b[2]; }

// ray (o, d) in the geom's local frame; returns t > tmin of the nearest hit or -1; n = local normal
__device__ float hit_local(int type, const float* size, const float* o, const float* d, float tmin, float* n) {
  if (type == 0) {
    if (fabsf(d[2]) < 1e-9f) return -1.f;
    const float t = -o[2] / d[2];
    if (t <= tmin) return -1.f;
    n[0] = 0.f; n[1] = 0.f; n[2] = 1.f;
    return t;
  }
  if (type == 1) {
    const float b = dot3(o, d), c = dot3(o, o) - size[0] * size[0], disc = b * b - c;
    if (disc < 0.f) return -1.f;
    const float s = sqrtf(disc);
    float t = -b - s;
    if (t <= tmin) t = -b + s;
    if (t <= tmin) return -1.f;
    const float inv = 1.f / size[0];
    for (int k = 0; k < 3; ++k) n[k] = (o[k] + t * d[k]) * inv;
    return t;
  }
  if (type == 2) {
    const float r = size[0], h = size[1];
    float best = -1.f;
    // infinite cylinder around z
    const float a = d[0] * d[0] + d[1] * d[1], b = o[0] * d[0] + o[1] * d[1], c = o[0] * o[0] + o[1] * o[1] - r * r;
    if (a > 1e-12f) {
      const float disc = b * b - a * c;
      if (disc >= 0.f) {
        const float s = sqrtf(disc);
        for (int sgn = -1; sgn <= 1; sgn += 2) {
          const float t = (-b + sgn * s) / a;
          const float z = o[2] + t * d[2];
          if (t > tmin && fabsf(z) <= h && (best < 0.f || t < best)) {
            best = t;
            n[0] = (o[0] + t * d[0]) / r; n[1] = (o[1] + t * d[1]) / r; n[2] = 0.f;
          }
        }
      }
    }
    for (int cap = -1; cap <= 1; cap += 2) {   // end spheres
      const float oc[3] = {o[0], o[1], o[2] - cap * h};
      const float bb = dot3(oc, d), cc = dot3(oc, oc) - r * r, disc = bb * bb - cc;
      if (disc < 0.f) continue;
      const float s = sqrtf(disc);
      for (int sgn = -1; sgn <= 1; sgn += 2) {
        const float t = -bb + sgn * s;
        const float z = oc[2] + t * d[2];
        if (t > tmin && z * cap >= 0.f && (best < 0.f || t < best)) {
          best = t;
          for (int k = 0; k < 3; ++k) n[k] = (oc[k] + t * d[k]) / r;
        }
      }
    }
    return best;
  }
  // box: slabs
  float t0 = -1e30f, t1 = 1e30f;
  int ax0 = 0, ax1 = 0;
  float s0 = 0.f, s1 = 0.f;
  for (int k = 0; k < 3; ++k) {
    if (fabsf(d[k]) < 1e-12f) {
      if (fabsf(o[k]) > size[k]) return -1.f;
      continue;
    }
    float ta = (-size[k] - o[k]) / d[k], tb = (size[k] - o[k]) / d[k];
    float sa = -1.f, sb = 1.f;
    if (ta > tb) { float tmp = ta; ta = tb; tb = tmp; sa = 1.f; sb = -1.f; }
    if (ta > t0) { t0 = ta; ax0 = k; s0 = sa; }
    if (tb < t1) { t1 = tb; ax1 = k; s1 = sb; }
  }
  if (t0 > t1) return -1.f;
  n[0] = n[1] = n[2] = 0.f;
  if (t0 > tmin) { n[ax0] = s0; return t0; }
  if (t1 > tmin) { n[ax1] = s1; return t1; }
  return -1.f;
}

// nearest hit of a world-space ray against all geoms of one world
__device__ Hit trace(const RtGeom* __restrict__ geoms, int n_geoms, const float* __restrict__ xpos,
                     const float* __restrict__ xmat, const float* o, const float* d, float tmin, float tmax) {
  Hit best;
  best.t = tmax; best.geom = -1;
  best.n[0] = best.n[1] = 0.f; best.n[2] = 1.f;
  for (int g = 0; g < n_geoms; ++g) {
    const RtGeom& G = geoms[g];
    float R[9], p[3];
    const int body = (int)G.body;
    if (body >= 0) {
      const float* bm = xmat + body * 9;
      const float* bp = xpos + body * 3;
      // world rotation = body · local; world position = body_pos + body · local_pos
      for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) R[i * 3 + j] = bm[i * 3] * G.rot[j] + bm[i * 3 + 1] * G.rot[3 + j] + bm[i * 3 + 2] * G.rot[6 + j];
      float lp[3];
      mat_vec(bm, G.pos, lp);
      for (int k = 0; k < 3; ++k) p[k] = bp[k] + lp[k];
    } else {
      for (int k = 0; k < 9; ++k) R[k] = G.rot[k];
      for (int k = 0; k < 3; ++k) p[k] = G.pos[k];
    }
    float rel[3] = {o[0] - p[0], o[1] - p[1], o[2] - p[2]}, ol[3], dl[3], nl[3];
    matT_vec(R, rel, ol);
    matT_vec(R, d, dl);
    const float t = hit_local((int)G.type, G.size, ol, dl, tmin, nl);
    if (t > 0.f && t < best.t) {
      best.t = t;
      best.geom = g;
      mat_vec(R, nl, best.n);
    }
  }
  return best;
}

// cams: per camera 16 floats: pos[3], rot[9] (columns right, up, back), fovy (rad), track body (or -1), pad[2]
__global__ void __launch_bounds__(128)
raytrace_kernel(const RtGeom* __restrict__ geoms, int n_geoms, const float* __restrict__ xpos,
                const float* __restrict__ xmat, int n_body, const float* __restrict__ cams, int n_cam, int H, int W,
                const float* __restrict__ light /* dir[3] (towards the light), ambient, diffuse, shadows */,
                unsigned char* __restrict__ rgb, float* __restrict__ depth, int n_worlds) {
  const long long total = (long long)n_worlds * n_cam * H * W;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int px = (int)(i % W);
    long long r = i / W;
    const int py = (int)(r % H); r /= H;
    const int cam = (int)(r % n_cam);
    const int w = (int)(r / n_cam);
    const float* C = cams + cam * 16;
    const float* wp = xpos + (size_t)w * n_body * 3;
    const float* wm = xmat + (size_t)w * n_body * 9;
    float o[3] = {C[0], C[1], C[2]};
    const int track = (int)C[13];
    if (track >= 0)
      for (int k = 0; k < 3; ++k) o[k] += wp[track * 3 + k];
    const float th = tanf(0.5f * C[12]);
    const float u = (2.f * (px + 0.5f) / W - 1.f) * th * ((float)W / H), v = (1.f - 2.f * (py + 0.5f) / H) * th;
    // camera looks along -back
    float d[3];
    for (int k = 0; k < 3; ++k) d[k] = u * C[3 + k * 3] + v * C[3 + k * 3 + 1] - C[3 + k * 3 + 2];
    const float inv = rsqrtf(dot3(d, d));
    for (int k = 0; k < 3; ++k) d[k] *= inv;
    const Hit h = trace(geoms, n_geoms, wp, wm, o, d, 1e-4f, 1e30f);
    float col[3];
    float dep = 0.f;
    if (h.geom < 0) {
      const float s = 0.5f * (d[2] + 1.f);
      col[0] = 0.55f + 0.25f * (1.f - s); col[1] = 0.70f + 0.15f * (1.f - s); col[2] = 0.95f;
    } else {
      dep = h.t;
      const RtGeom& G = geoms[h.geom];
      float base[3] = {G.rgba[0], G.rgba[1], G.rgba[2]};
      float hp[3];
      for (int k = 0; k < 3; ++k) hp[k] = o[k] + h.t * d[k];
      if ((int)G.type == 0) {      // checkerboard on planes, 0.5 m squares
        const int cx = (int)floorf(hp[0] * 2.f), cy = (int)floorf(hp[1] * 2.f);
        const float f = ((cx + cy) & 1) ? 1.f : 0.6f;
        for (int k = 0; k < 3; ++k) base[k] *= f;
      }
      float nn[3] = {h.n[0], h.n[1], h.n[2]};
      if (dot3(nn, d) > 0.f) for (int k = 0; k < 3; ++k) nn[k] = -nn[k];
      float diff = fmaxf(dot3(nn, light), 0.f);
      if (light[5] != 0.f && diff > 0.f) {
        float so[3];
        for (int k = 0; k < 3; ++k) so[k] = hp[k] + 1e-3f * nn[k];
        const Hit sh = trace(geoms, n_geoms, wp, wm, so, light, 1e-4f, 1e30f);
        if (sh.geom >= 0) diff = 0.f;
      }
      const float lum = light[3] + light[4] * diff;
      for (int k = 0; k < 3; ++k) col[k] = fminf(base[k] * lum, 1.f);
    }
    for (int k = 0; k < 3; ++k) rgb[i * 3 + k] = (unsigned char)(col[k] * 255.f + 0.5f);
    if (depth) depth[i] = dep;
  }
}

}  // namespace

extern "C" int nb_raytrace(const float* geoms, int n_geoms, const float* xpos, const float* xmat, int n_body, const float* cams,
                           int n_cam, int H, int W, const float* light, unsigned char* rgb, float* depth, int n_worlds,
                           void* stream) {
  if (n_geoms <= 0 || n_cam <= 0 || H <= 0 || W <= 0 || n_worlds <= 0) return NB_ERR_BAD_ARG;
  const long long total = (long long)n_worlds * n_cam * H * W;
  long long blocks = (total + 127) / 128;
  if (blocks > 148LL * 64) blocks = 148LL * 64;
  raytrace_kernel<<<(int)blocks, 128, 0, (cudaStream_t)stream>>>((const RtGeom*)geoms, n_geoms, xpos, xmat, n_body, cams, n_cam,
                                                                H, W, light, rgb, depth, n_worlds);
  NB_LAUNCH_CHECK();
  return NB_OK;
}
