// 2-D rigid-body core: bodies, revolute joints (limit + motor), convex-polygon-vs-terrain contacts and a sequential
// impulse solver, written once as plain host/device functions.  The CUDA environments (lunar_lander.cu) run it with
// one thread per environment and the world in registers / local memory; the host library compiles the SAME source
// (csrc/host/physics2d_host.cpp) as the CPU oracle of the GPU tests.
//
//   step:  integrate velocities (gravity, applied forces) → prepare joints and contacts → velocity iterations
//          (joint motors, joint limits, joint point constraints, contact friction, contact normals; accumulated
//          impulses are clamped) → integrate positions → position iterations (Baumgarte correction of contact
//          penetration, joint drift and limit violation) → sleep clock.
// The terrain is a height field over evenly spaced x knots (the reference's "edge terrain"); a contact is a polygon
// vertex below its terrain segment, at most two (the deepest) per body.
// Reference: noeira/physics2d/ (impulse solver solvers/, joints/revolute, collision/edge terrain, island sleep).
#pragma once
#include <math.h>

#ifdef __CUDACC__
#define NB2D_HD __host__ __device__ __forceinline__
#else
#define NB2D_HD inline
#endif

// The capacities are compile-time constants of the including translation unit: an environment with more bodies defines
// NB2D_MAX_BODIES / NB2D_MAX_JOINTS / NB2D_MAX_TERRAIN and its own namespace name NB2D_NS before the include, so that two
// environments with different capacities can live in one library.
#ifndef NB2D_NS
#define NB2D_NS nb2d
#endif
#ifndef NB2D_MAX_BODIES
#define NB2D_MAX_BODIES 4
#endif
#ifndef NB2D_MAX_JOINTS
#define NB2D_MAX_JOINTS 3
#endif
#ifndef NB2D_MAX_TERRAIN
#define NB2D_MAX_TERRAIN 16
#endif

namespace NB2D_NS {

constexpr int MAX_BODIES = NB2D_MAX_BODIES;
constexpr int MAX_JOINTS = NB2D_MAX_JOINTS;
constexpr int MAX_VERTS = 6;
constexpr int CONTACTS_PER_BODY = 2;
constexpr int MAX_CONTACTS = MAX_BODIES * CONTACTS_PER_BODY;
constexpr int MAX_TERRAIN = NB2D_MAX_TERRAIN;

struct Body {
  float x, y, a;          // pose (centre of mass, angle)
  float vx, vy, w;        // velocity
  float inv_m, inv_i;     // 0 for a static body
  float fx, fy, tq;       // force / torque accumulated for the next step (cleared by it)
  int nvert;              // convex polygon in the body frame
  float px[MAX_VERTS], py[MAX_VERTS];
  float friction;
};

struct Revolute {
  int a, b;
  float ax, ay, bx, by;   // anchors in the frames of a and b
  float ref;              // reference angle: joint angle = angle_b - angle_a - ref
  float lower, upper;
  float motor_speed, max_torque;
  int enable_limit, enable_motor;
  // solver state
  float rax, ray, rbx, rby, k11, k12, k22, motor_mass;
  float imp_x, imp_y, imp_motor, imp_lower, imp_upper;
};

struct Contact {
  int body, vert;
  float nx, ny;           // terrain normal (pointing out of the ground)
  float rx, ry;           // contact point relative to the body centre
  float pen;              // penetration depth (> 0 inside)
  float mass_n, mass_t;
  float imp_n, imp_t;
};

struct Terrain {
  int n;                  // knots
  float x0, dx;           // knot i at x0 + i dx
  float h[MAX_TERRAIN];
};

struct World {
  int nbody, njoint, ncontact;
  Body body[MAX_BODIES];
  Revolute joint[MAX_JOINTS];
  Contact contact[MAX_CONTACTS];
  Terrain terrain;
  float gx, gy, dt;
  int vel_iters, pos_iters;
  float baumgarte, slop, max_correction;
  float sleep_time;       // seconds every body has been below the sleep tolerances
  // warm start: the accumulated impulses of the previous step, re-applied before the iterations.  With a heavy hull
  // resting on light legs Gauss-Seidel loses only a few percent of its error per sweep; started from the previous
  // solution ten sweeps hold what hundreds of cold sweeps do not.
  float jwarm[MAX_JOINTS][5];                          // imp_x, imp_y, motor, lower, upper
  int cwarm_vert[MAX_BODIES][CONTACTS_PER_BODY];       // vertex of the stored contact, -1 = none
  float cwarm_imp[MAX_BODIES][CONTACTS_PER_BODY][2];   // normal, tangent
};

NB2D_HD void clear_warm_start(World& w) {
  for (int j = 0; j < MAX_JOINTS; ++j)
    for (int k = 0; k < 5; ++k) w.jwarm[j][k] = 0.f;
  for (int b = 0; b < MAX_BODIES; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      w.cwarm_vert[b][k] = -1;
      w.cwarm_imp[b][k][0] = w.cwarm_imp[b][k][1] = 0.f;
    }
}

NB2D_HD float cross2(float ax, float ay, float bx, float by) { return ax * by - ay * bx; }
NB2D_HD float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }

NB2D_HD void body_point(const Body& b, float lx, float ly, float& wx, float& wy) {
  const float c = cosf(b.a), s = sinf(b.a);
  wx = b.x + c * lx - s * ly;
  wy = b.y + s * lx + c * ly;
}
NB2D_HD void apply_impulse(Body& b, float jx, float jy, float rx, float ry) {
  b.vx += b.inv_m * jx;
  b.vy += b.inv_m * jy;
  b.w += b.inv_i * cross2(rx, ry, jx, jy);
}
// impulse at a WORLD point (engines)
NB2D_HD void apply_impulse_at(Body& b, float jx, float jy, float px, float py) { apply_impulse(b, jx, jy, px - b.x, py - b.y); }

// terrain height and outward normal under x
NB2D_HD void terrain_at(const Terrain& t, float x, float& h, float& nx, float& ny) {
  float u = (x - t.x0) / t.dx;
  int i = (int)floorf(u);
  i = i < 0 ? 0 : (i > t.n - 2 ? t.n - 2 : i);
  const float f = u - (float)i;
  const float h0 = t.h[i], h1 = t.h[i + 1];
  h = h0 + (h1 - h0) * f;
  // segment direction (dx, h1-h0); normal = (-(h1-h0), dx) normalised
  const float ex = t.dx, ey = h1 - h0;
  const float inv = 1.0f / sqrtf(ex * ex + ey * ey);
  nx = -ey * inv;
  ny = ex * inv;
}

NB2D_HD void detect_contacts(World& w) {
  w.ncontact = 0;
  for (int bi = 0; bi < w.nbody; ++bi) {
    const Body& b = w.body[bi];
    if (b.inv_m == 0.f) continue;
    // the two deepest vertices of this body
    int best[CONTACTS_PER_BODY] = {-1, -1};
    float depth[CONTACTS_PER_BODY] = {0.f, 0.f};
    float cnx[CONTACTS_PER_BODY], cny[CONTACTS_PER_BODY], crx[CONTACTS_PER_BODY], cry[CONTACTS_PER_BODY];
    const float c = cosf(b.a), s = sinf(b.a);
    for (int v = 0; v < b.nvert; ++v) {
      const float rx = c * b.px[v] - s * b.py[v], ry = s * b.px[v] + c * b.py[v];
      const float wx = b.x + rx, wy = b.y + ry;
      float h, nx, ny;
      terrain_at(w.terrain, wx, h, nx, ny);
      const float pen = (h - wy) * ny;      // distance below the segment, along its normal
      if (pen <= 0.f) continue;
      int slot = -1;
      if (best[0] < 0 || pen > depth[0]) {
        best[1] = best[0]; depth[1] = depth[0]; cnx[1] = cnx[0]; cny[1] = cny[0]; crx[1] = crx[0]; cry[1] = cry[0];
        slot = 0;
      } else if (best[1] < 0 || pen > depth[1]) {
        slot = 1;
      }
      if (slot >= 0) { best[slot] = v; depth[slot] = pen; cnx[slot] = nx; cny[slot] = ny; crx[slot] = rx; cry[slot] = ry; }
    }
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) {
      if (best[k] < 0) continue;
      Contact& ct = w.contact[w.ncontact++];
      ct.body = bi; ct.vert = best[k];
      ct.nx = cnx[k]; ct.ny = cny[k]; ct.rx = crx[k]; ct.ry = cry[k];
      ct.pen = depth[k];
      const float rn = cross2(ct.rx, ct.ry, ct.nx, ct.ny);
      const float rt = cross2(ct.rx, ct.ry, ct.ny, -ct.nx);
      ct.mass_n = 1.0f / (b.inv_m + b.inv_i * rn * rn);
      ct.mass_t = 1.0f / (b.inv_m + b.inv_i * rt * rt);
      ct.imp_n = ct.imp_t = 0.f;
    }
  }
}

NB2D_HD void prepare_joint(const World& w, Revolute& j) {
  const Body& A = w.body[j.a];
  const Body& B = w.body[j.b];
  const float ca = cosf(A.a), sa = sinf(A.a), cb = cosf(B.a), sb = sinf(B.a);
  j.rax = ca * j.ax - sa * j.ay; j.ray = sa * j.ax + ca * j.ay;
  j.rbx = cb * j.bx - sb * j.by; j.rby = sb * j.bx + cb * j.by;
  const float mA = A.inv_m, mB = B.inv_m, iA = A.inv_i, iB = B.inv_i;
  j.k11 = mA + mB + iA * j.ray * j.ray + iB * j.rby * j.rby;
  j.k12 = -iA * j.rax * j.ray - iB * j.rbx * j.rby;
  j.k22 = mA + mB + iA * j.rax * j.rax + iB * j.rbx * j.rbx;
  const float im = iA + iB;
  j.motor_mass = im > 0.f ? 1.0f / im : 0.f;
  j.imp_x = j.imp_y = j.imp_motor = j.imp_lower = j.imp_upper = 0.f;
}

NB2D_HD void solve_joint_velocity(World& w, Revolute& j) {
  Body& A = w.body[j.a];
  Body& B = w.body[j.b];
  const float iA = A.inv_i, iB = B.inv_i;
  if (j.enable_motor) {
    const float cdot = B.w - A.w - j.motor_speed;
    float imp = -j.motor_mass * cdot;
    const float old = j.imp_motor, mx = w.dt * j.max_torque;
    j.imp_motor = clampf(old + imp, -mx, mx);
    imp = j.imp_motor - old;
    A.w -= iA * imp;
    B.w += iB * imp;
  }
  if (j.enable_limit) {
    const float angle = B.a - A.a - j.ref;
    {  // lower
      const float c = angle - j.lower;
      const float cdot = B.w - A.w;
      float imp = -j.motor_mass * (cdot + fmaxf(c, 0.f) / w.dt);
      const float nw = fmaxf(j.imp_lower + imp, 0.f);
      imp = nw - j.imp_lower;
      j.imp_lower = nw;
      A.w -= iA * imp;
      B.w += iB * imp;
    }
    {  // upper
      const float c = j.upper - angle;
      const float cdot = A.w - B.w;
      float imp = -j.motor_mass * (cdot + fmaxf(c, 0.f) / w.dt);
      const float nw = fmaxf(j.imp_upper + imp, 0.f);
      imp = nw - j.imp_upper;
      j.imp_upper = nw;
      A.w += iA * imp;
      B.w -= iB * imp;
    }
  }
  // point constraint
  const float cdx = B.vx - B.w * j.rby - A.vx + A.w * j.ray;
  const float cdy = B.vy + B.w * j.rbx - A.vy - A.w * j.rax;
  const float det = j.k11 * j.k22 - j.k12 * j.k12;
  const float inv = det != 0.f ? 1.0f / det : 0.f;
  const float ix = -inv * (j.k22 * cdx - j.k12 * cdy);
  const float iy = -inv * (j.k11 * cdy - j.k12 * cdx);
  j.imp_x += ix;
  j.imp_y += iy;
  apply_impulse(A, -ix, -iy, j.rax, j.ray);
  apply_impulse(B, ix, iy, j.rbx, j.rby);
}

NB2D_HD void solve_contact_velocity(World& w, Contact& c) {
  Body& b = w.body[c.body];
  const float tx = c.ny, ty = -c.nx;
  {  // friction
    const float vx = b.vx - b.w * c.ry, vy = b.vy + b.w * c.rx;
    float imp = -c.mass_t * (vx * tx + vy * ty);
    const float mx = b.friction * c.imp_n;
    const float nw = clampf(c.imp_t + imp, -mx, mx);
    imp = nw - c.imp_t;
    c.imp_t = nw;
    apply_impulse(b, imp * tx, imp * ty, c.rx, c.ry);
  }
  {  // normal (no restitution)
    const float vx = b.vx - b.w * c.ry, vy = b.vy + b.w * c.rx;
    float imp = -c.mass_n * (vx * c.nx + vy * c.ny);
    const float nw = fmaxf(c.imp_n + imp, 0.f);
    imp = nw - c.imp_n;
    c.imp_n = nw;
    apply_impulse(b, imp * c.nx, imp * c.ny, c.rx, c.ry);
  }
}

NB2D_HD void solve_positions(World& w) {
  // contacts: re-evaluate the penetration of the stored vertex at the current pose
  for (int i = 0; i < w.ncontact; ++i) {
    Contact& c = w.contact[i];
    Body& b = w.body[c.body];
    const float cs = cosf(b.a), sn = sinf(b.a);
    const float rx = cs * b.px[c.vert] - sn * b.py[c.vert], ry = sn * b.px[c.vert] + cs * b.py[c.vert];
    float h, nx, ny;
    terrain_at(w.terrain, b.x + rx, h, nx, ny);
    const float sep = -(h - (b.y + ry)) * ny;
    const float C = clampf(w.baumgarte * (sep + w.slop), -w.max_correction, 0.f);
    const float rn = cross2(rx, ry, nx, ny);
    const float k = b.inv_m + b.inv_i * rn * rn;
    const float imp = k > 0.f ? -C / k : 0.f;
    b.x += b.inv_m * imp * nx;
    b.y += b.inv_m * imp * ny;
    b.a += b.inv_i * rn * imp;
  }
  for (int ji = 0; ji < w.njoint; ++ji) {
    Revolute& j = w.joint[ji];
    Body& A = w.body[j.a];
    Body& B = w.body[j.b];
    const float iA = A.inv_i, iB = B.inv_i;
    if (j.enable_limit) {
      const float angle = B.a - A.a - j.ref;
      float C = 0.f;
      if (angle < j.lower) C = clampf(angle - j.lower + 0.0349f, -0.1396f, 0.f);        // angular slop 2°, max correction 8°
      else if (angle > j.upper) C = clampf(angle - j.upper - 0.0349f, 0.f, 0.1396f);
      const float imp = -j.motor_mass * C;
      A.a -= iA * imp;
      B.a += iB * imp;
    }
    const float ca = cosf(A.a), sa = sinf(A.a), cb = cosf(B.a), sb = sinf(B.a);
    const float rax = ca * j.ax - sa * j.ay, ray = sa * j.ax + ca * j.ay;
    const float rbx = cb * j.bx - sb * j.by, rby = sb * j.bx + cb * j.by;
    const float cx = B.x + rbx - A.x - rax, cy = B.y + rby - A.y - ray;
    const float mA = A.inv_m, mB = B.inv_m;
    const float k11 = mA + mB + iA * ray * ray + iB * rby * rby;
    const float k12 = -iA * rax * ray - iB * rbx * rby;
    const float k22 = mA + mB + iA * rax * rax + iB * rbx * rbx;
    const float det = k11 * k22 - k12 * k12;
    const float inv = det != 0.f ? 1.0f / det : 0.f;
    const float ix = -inv * (k22 * cx - k12 * cy);
    const float iy = -inv * (k11 * cy - k12 * cx);
    A.x -= mA * ix; A.y -= mA * iy; A.a -= iA * cross2(rax, ray, ix, iy);
    B.x += mB * ix; B.y += mB * iy; B.a += iB * cross2(rbx, rby, ix, iy);
  }
}

NB2D_HD void step(World& w) {
  const float dt = w.dt;
  for (int i = 0; i < w.nbody; ++i) {
    Body& b = w.body[i];
    if (b.inv_m == 0.f) continue;
    b.vx += dt * (w.gx + b.inv_m * b.fx);
    b.vy += dt * (w.gy + b.inv_m * b.fy);
    b.w += dt * b.inv_i * b.tq;
    b.fx = b.fy = b.tq = 0.f;
  }
  detect_contacts(w);
  for (int j = 0; j < w.njoint; ++j) prepare_joint(w, w.joint[j]);
  // ---- warm start
  for (int ji = 0; ji < w.njoint; ++ji) {
    Revolute& j = w.joint[ji];
    j.imp_x = w.jwarm[ji][0]; j.imp_y = w.jwarm[ji][1];
    j.imp_motor = j.enable_motor ? w.jwarm[ji][2] : 0.f;
    j.imp_lower = j.enable_limit ? w.jwarm[ji][3] : 0.f;
    j.imp_upper = j.enable_limit ? w.jwarm[ji][4] : 0.f;
    Body& A = w.body[j.a];
    Body& B = w.body[j.b];
    const float axial = j.imp_motor + j.imp_lower - j.imp_upper;
    apply_impulse(A, -j.imp_x, -j.imp_y, j.rax, j.ray);
    A.w -= A.inv_i * axial;
    apply_impulse(B, j.imp_x, j.imp_y, j.rbx, j.rby);
    B.w += B.inv_i * axial;
  }
  for (int ci = 0; ci < w.ncontact; ++ci) {
    Contact& c = w.contact[ci];
    for (int k = 0; k < CONTACTS_PER_BODY; ++k)
      if (w.cwarm_vert[c.body][k] == c.vert) {
        c.imp_n = w.cwarm_imp[c.body][k][0];
        c.imp_t = w.cwarm_imp[c.body][k][1];
      }
    Body& b = w.body[c.body];
    apply_impulse(b, c.imp_n * c.nx + c.imp_t * c.ny, c.imp_n * c.ny - c.imp_t * c.nx, c.rx, c.ry);
  }
  for (int it = 0; it < w.vel_iters; ++it) {
    for (int j = 0; j < w.njoint; ++j) solve_joint_velocity(w, w.joint[j]);
    for (int c = 0; c < w.ncontact; ++c) solve_contact_velocity(w, w.contact[c]);
  }
  for (int i = 0; i < w.nbody; ++i) {
    Body& b = w.body[i];
    b.x += dt * b.vx;
    b.y += dt * b.vy;
    b.a += dt * b.w;
  }
  // ---- keep the solution for the next step
  for (int ji = 0; ji < w.njoint; ++ji) {
    const Revolute& j = w.joint[ji];
    w.jwarm[ji][0] = j.imp_x; w.jwarm[ji][1] = j.imp_y; w.jwarm[ji][2] = j.imp_motor;
    w.jwarm[ji][3] = j.imp_lower; w.jwarm[ji][4] = j.imp_upper;
  }
  for (int b = 0; b < MAX_BODIES; ++b)
    for (int k = 0; k < CONTACTS_PER_BODY; ++k) w.cwarm_vert[b][k] = -1;
  {
    int used[MAX_BODIES];
    for (int b = 0; b < MAX_BODIES; ++b) used[b] = 0;
    for (int ci = 0; ci < w.ncontact; ++ci) {
      const Contact& c = w.contact[ci];
      const int k = used[c.body]++;
      if (k < CONTACTS_PER_BODY) {
        w.cwarm_vert[c.body][k] = c.vert;
        w.cwarm_imp[c.body][k][0] = c.imp_n;
        w.cwarm_imp[c.body][k][1] = c.imp_t;
      }
    }
  }
  for (int it = 0; it < w.pos_iters; ++it) solve_positions(w);
  // sleep clock (linear 0.01 m/s, angular 2°/s, as the island sleep of the reference)
  bool slow = true;
  for (int i = 0; i < w.nbody; ++i) {
    const Body& b = w.body[i];
    if (b.inv_m == 0.f) continue;
    if (b.vx * b.vx + b.vy * b.vy > 1e-4f || fabsf(b.w) > 0.0349f) slow = false;
  }
  w.sleep_time = slow ? w.sleep_time + dt : 0.f;
}

}  // namespace NB2D_NS
