// Fused batched rigid-body step for generalized-coordinate tree models (hinge / slide joints).
//
// One WARP owns one environment for the whole control step: all `frame_skip` substeps, reward,
// observation extraction and the selective reset run inside a single launch, with per-env
// scratch in shared memory and the (batch-shared) model staged once per block.  The reference
// runs the same pipeline as 15–20 launches per substep with one thread per env
// (noeira/physics3d/integrator/euler.mojo:831-1360, stage order :1-22); on B200 the 4096-env
// batch then fills 32 warps of a 148-SM part.  Here 4096 envs are 4096 warps (all co-resident),
// and inside a warp the lanes take whichever axis is parallel at that stage:
//
//   stage                          lanes own        math
//   FK (level synchronous)         bodies           pose = parent ∘ (pos,quat) ∘ joints
//   motion axes S, inertias        dofs / bodies    spatial vectors about c = xpos[body 0]
//   velocities + RNE forces        bodies           a_b = a0 + Σ (V_cum × S_d) q̇_d ; f = I a + V ×* I V
//   bias, composite inertia, CRBA  dofs / bodies    M_ij = S_j · (Ic_body(i) S_i)
//   Cholesky of M + arm + dt·D     trailing matrix  in place
//   constraint rows                rows             J row by mask walk, B = M̂⁻¹Jᵀ by two triangular solves
//   projected Gauss-Seidel         dofs             a_r = J_r·qacc (shuffle reduce), qacc += B_r Δλ
//   integrate                      dofs             semi-implicit Euler
//
// Contacts are "contact spheres" (a body-fixed point + radius) against the ground plane: a
// capsule contributes its two end spheres (noeira/physics3d/collision/collision_primitives.mojo:375-463
// tests the lower end only; both ends give the capsule a stable resting manifold).  Constraints
// are soft, at acceleration level, with MuJoCo's solref/solimp parameterisation
// (noeira/physics3d/constraints/contact_solve.mojo:1295-2536): aref = -b v - k·imp·dist,
// R = (1-imp)/imp · A_rr, unilateral normal/limit rows, box-bounded friction rows |λ_t| ≤ μ λ_n,
// warm-started from the previous substep through fixed per-slot storage.
// Joint damping is integrated implicitly by factoring M̂ = M + diag(armature + dt·damping) once
// and using it for both the smooth solve and the constraint response (the reference re-factors in
// its finalize stage, euler.mojo:404-552).
#include <type_traits>

#include "common.cuh"
#include "physics_params.h"

namespace {

using namespace nb;

struct V3 {
  float x, y, z;
};
__device__ __forceinline__ V3 v3(float x, float y, float z) { return V3{x, y, z}; }
__device__ __forceinline__ V3 operator+(V3 a, V3 b) { return v3(a.x + b.x, a.y + b.y, a.z + b.z); }
__device__ __forceinline__ V3 operator-(V3 a, V3 b) { return v3(a.x - b.x, a.y - b.y, a.z - b.z); }
__device__ __forceinline__ V3 operator*(float s, V3 a) { return v3(s * a.x, s * a.y, s * a.z); }
__device__ __forceinline__ float dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
__device__ __forceinline__ V3 cross(V3 a, V3 b) {
  return v3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}
__device__ __forceinline__ V3 ld3(const float* p) { return v3(p[0], p[1], p[2]); }
__device__ __forceinline__ void st3(float* p, V3 a) {
  p[0] = a.x;
  p[1] = a.y;
  p[2] = a.z;
}

struct Q4 {
  float w, x, y, z;
};
__device__ __forceinline__ Q4 qmul(Q4 a, Q4 b) {
  return Q4{a.w * b.w - a.x * b.x - a.y * b.y - a.z * b.z, a.w * b.x + a.x * b.w + a.y * b.z - a.z * b.y,
            a.w * b.y - a.x * b.z + a.y * b.w + a.z * b.x, a.w * b.z + a.x * b.y - a.y * b.x + a.z * b.w};
}
__device__ __forceinline__ V3 qrot(Q4 q, V3 v) {
  // v + 2 w (u × v) + 2 u × (u × v)
  V3 u = v3(q.x, q.y, q.z);
  V3 t = 2.f * cross(u, v);
  return v + q.w * t + cross(u, t);
}
__device__ __forceinline__ void qmat(Q4 q, float* m) {
  const float xx = q.x * q.x, yy = q.y * q.y, zz = q.z * q.z, xy = q.x * q.y, xz = q.x * q.z, yz = q.y * q.z,
              wx = q.w * q.x, wy = q.w * q.y, wz = q.w * q.z;
  m[0] = 1.f - 2.f * (yy + zz);
  m[1] = 2.f * (xy - wz);
  m[2] = 2.f * (xz + wy);
  m[3] = 2.f * (xy + wz);
  m[4] = 1.f - 2.f * (xx + zz);
  m[5] = 2.f * (yz - wx);
  m[6] = 2.f * (xz - wy);
  m[7] = 2.f * (yz + wx);
  m[8] = 1.f - 2.f * (xx + yy);
}

// Spatial inertia about the reference point, world axes: [Ixx Iyy Izz Ixy Ixz Iyz | m·h | m].
// y = I * [w; v]  → angular n = Iref w + mh × v ; linear f = m v + w × mh
__device__ __forceinline__ void inertia_mul(const float* I, V3 w, V3 v, V3& n, V3& f) {
  V3 mh = v3(I[6], I[7], I[8]);
  n = v3(I[0] * w.x + I[3] * w.y + I[4] * w.z, I[3] * w.x + I[1] * w.y + I[5] * w.z,
         I[4] * w.x + I[5] * w.y + I[2] * w.z) +
      cross(mh, v);
  f = I[9] * v + cross(w, mh);
}

__device__ __forceinline__ float impedance(const PhysParams& P, float pen) {
  float x = pen / P.solimp_width;
  x = fminf(fmaxf(x, 0.f), 1.f);
  float y;
  if (P.solimp_pow == 2.f) {  // the default exponent: no transcendental
    y = (x <= P.solimp_mid) ? x * x / P.solimp_mid : 1.f - (1.f - x) * (1.f - x) / (1.f - P.solimp_mid);
  } else if (x <= P.solimp_mid) {
    y = powf(x, P.solimp_pow) / powf(P.solimp_mid, P.solimp_pow - 1.f);
  } else {
    y = 1.f - powf(1.f - x, P.solimp_pow) / powf(1.f - P.solimp_mid, P.solimp_pow - 1.f);
  }
  float imp = P.solimp_d0 + y * (P.solimp_dmax - P.solimp_d0);
  return fminf(fmaxf(imp, 1e-4f), 0.9999f);
}

// Row kinds
#define ROW_LIMIT 0
#define ROW_NORMAL 1
#define ROW_TANGENT 2

struct WarpScratch {
  float *xpos, *xmat, *xquat, *S, *I, *Ic, *V, *F, *M, *vec, *J, *B, *row, *A;
  int* rowi;
};

// Layout of one warp's scratch.  The Delassus matrix A (symmetric, packed lower triangle: 528 words for 32 rows) is
// built after the inertias, velocities, forces and body quaternions have been consumed, so it overlays them; the
// scratch of a 9-dof chain is then 7 KB and 28 warps (environments) fit one SM.
__device__ __forceinline__ WarpScratch carve(float* base, const PhysParams& P) {
  WarpScratch w;
  const int nb_ = P.nbody, nv = P.nv, nvp = P.nvp, rmax = P.rmax;
  float* p = base;
  w.xpos = p; p += nb_ * 3;
  w.xmat = p; p += nb_ * 9;
  w.S = p; p += nv * 6;
  w.M = p; p += nv * nvp;
  w.vec = p; p += 4 * 32;
  w.J = p; p += rmax * nvp;
  w.B = p; p += rmax * nvp;
  w.row = p; p += rmax * 4;
  w.rowi = reinterpret_cast<int*>(p); p += rmax * 4;  // rmax * 4 ints
  w.A = p;  // packed 32 x 32 lower triangle (dual PGS, rmax <= 32); shares its space with the five arrays below
  w.xquat = p; p += nb_ * 4;
  w.I = p; p += nb_ * 10;
  w.Ic = p; p += nb_ * 10;
  w.V = p; p += nb_ * 6;
  w.F = p; p += nb_ * 6;
  return w;
}

struct ModelView {
  const int *body_parent, *body_depth, *body_dofadr, *body_dofnum, *body_dofmask, *body_ancmask, *dof_body,
      *dof_type, *lim_dof, *cs_body, *act_dof;
  const float *body_pos, *body_quat, *body_ipos, *body_inertia6, *body_mass, *dof_axis, *dof_pos, *dof_armature,
      *dof_damping, *dof_stiffness, *dof_springref, *lim_lo, *lim_hi, *cs_local, *cs_radius, *cs_mu, *act_gear,
      *act_lo, *act_hi, *qpos0, *reset_noise;
};

__device__ __forceinline__ ModelView view(const int* im, const float* fm, const PhysParams& P) {
  ModelView m;
  const int nb_ = P.nbody, nv = P.nv;
  const int* i = im;
  m.body_parent = i; i += nb_;
  m.body_depth = i; i += nb_;
  m.body_dofadr = i; i += nb_;
  m.body_dofnum = i; i += nb_;
  m.body_dofmask = i; i += nb_;
  m.body_ancmask = i; i += nb_;
  m.dof_body = i; i += nv;
  m.dof_type = i; i += nv;
  m.lim_dof = i; i += P.nlimit;
  m.cs_body = i; i += P.ncs;
  m.act_dof = i; i += P.nu;
  const float* f = fm;
  m.body_pos = f; f += nb_ * 3;
  m.body_quat = f; f += nb_ * 4;
  m.body_ipos = f; f += nb_ * 3;
  m.body_inertia6 = f; f += nb_ * 6;
  m.body_mass = f; f += nb_;
  m.dof_axis = f; f += nv * 3;
  m.dof_pos = f; f += nv * 3;
  m.dof_armature = f; f += nv;
  m.dof_damping = f; f += nv;
  m.dof_stiffness = f; f += nv;
  m.dof_springref = f; f += nv;
  m.lim_lo = f; f += P.nlimit;
  m.lim_hi = f; f += P.nlimit;
  m.cs_local = f; f += P.ncs * 3;
  m.cs_radius = f; f += P.ncs;
  m.cs_mu = f; f += P.ncs;
  m.act_gear = f; f += P.nu;
  m.act_lo = f; f += P.nu;
  m.act_hi = f; f += P.nu;
  m.qpos0 = f; f += nv;
  m.reset_noise = f; f += 2;
  return m;
}

// ------------------------------------------------------------------------------------------
// Forward kinematics by pointer jumping.  Lane b owns body b (at most 32 bodies).
//   1. every lane composes its body's LOCAL transform (frame offset ∘ joints) relative to the parent frame — no
//      dependence on other bodies; per dof it records the joint axis and anchor in the parent frame;
//   2. ⌈log2(depth + 1)⌉ rounds of T[b] ← T[anc[b]] ∘ T[b], anc[b] ← anc[anc[b]] through warp shuffles turn the local
//      transforms into world transforms (a 7-link chain needs 3 rounds with all lanes busy instead of 7 levels with
//      one lane busy each);
//   3. lane d maps dof d's axis and anchor through its body's parent's world transform.
// On exit xpos / xquat / xmat are the body frames and S[d] holds (axis_w, anchor_w) per dof (converted to motion axes
// later).
__device__ __forceinline__ void forward_kinematics(const PhysParams& P, const ModelView& m, WarpScratch& w,
                                                   const float* qpos_sh, int lane) {
  const bool has_body = lane < P.nbody;
  const int b = has_body ? lane : 0;
  V3 pos = v3(0.f, 0.f, 0.f);
  Q4 q = Q4{1.f, 0.f, 0.f, 0.f};
  int anc = -1;
  if (has_body) {
    anc = m.body_parent[b];
    pos = ld3(m.body_pos + b * 3);
    q = Q4{m.body_quat[b * 4], m.body_quat[b * 4 + 1], m.body_quat[b * 4 + 2], m.body_quat[b * 4 + 3]};
    const int d0 = m.body_dofadr[b], dn = m.body_dofnum[b];
    for (int k = 0; k < dn; ++k) {
      const int d = d0 + k;
      const V3 al = ld3(m.dof_axis + d * 3);
      const V3 axis_p = qrot(q, al);                 // joint axis in the parent frame
      const float qd = qpos_sh[d] - m.qpos0[d];
      if (m.dof_type[d] == NB_JOINT_HINGE) {
        const V3 dp = ld3(m.dof_pos + d * 3);
        const V3 anchor = pos + qrot(q, dp);
        float sn, cs;
        {
          float hf = 0.5f * qd;
          hf -= 6.283185307179586f * rintf(hf * 0.15915494309189535f);
          __sincosf(hf, &sn, &cs);
        }
        q = qmul(q, Q4{cs, sn * al.x, sn * al.y, sn * al.z});
        pos = anchor - qrot(q, dp);
        st3(w.S + d * 6, axis_p);
        st3(w.S + d * 6 + 3, anchor);
      } else {
        pos = pos + qd * axis_p;
        st3(w.S + d * 6, axis_p);
        st3(w.S + d * 6 + 3, pos);
      }
    }
  }
  // parent's WORLD transform of every body is needed in step 3: remember the parent lane before the jumps change anc
  const int par = anc;
  for (int round = 0; round < 5; ++round) {
    if (__all_sync(0xffffffffu, anc < 0)) break;
    const int src = anc < 0 ? lane : anc;
    const float apx = __shfl_sync(0xffffffffu, pos.x, src), apy = __shfl_sync(0xffffffffu, pos.y, src),
                apz = __shfl_sync(0xffffffffu, pos.z, src);
    const float aqw = __shfl_sync(0xffffffffu, q.w, src), aqx = __shfl_sync(0xffffffffu, q.x, src),
                aqy = __shfl_sync(0xffffffffu, q.y, src), aqz = __shfl_sync(0xffffffffu, q.z, src);
    const int aanc = __shfl_sync(0xffffffffu, anc, src);
    if (anc >= 0) {
      const Q4 aq = Q4{aqw, aqx, aqy, aqz};
      pos = v3(apx, apy, apz) + qrot(aq, pos);
      q = qmul(aq, q);
      anc = aanc;
    }
  }
  if (has_body) {
    const float inv = rsqrtf(q.w * q.w + q.x * q.x + q.y * q.y + q.z * q.z);
    q = Q4{q.w * inv, q.x * inv, q.y * inv, q.z * inv};
    st3(w.xpos + b * 3, pos);
    w.xquat[b * 4] = q.w;
    w.xquat[b * 4 + 1] = q.x;
    w.xquat[b * 4 + 2] = q.y;
    w.xquat[b * 4 + 3] = q.z;
    qmat(q, w.xmat + b * 9);
  }
  __syncwarp();
  (void)par;
  // step 3: dof axes / anchors from the parent frame of their body to the world
  if (lane < P.nv) {
    const int d = lane;
    const int pb = m.body_parent[m.dof_body[d]];
    if (pb >= 0) {
      const V3 pp = ld3(w.xpos + pb * 3);
      const Q4 pq = Q4{w.xquat[pb * 4], w.xquat[pb * 4 + 1], w.xquat[pb * 4 + 2], w.xquat[pb * 4 + 3]};
      const V3 ax = qrot(pq, ld3(w.S + d * 6));
      const V3 an = pp + qrot(pq, ld3(w.S + d * 6 + 3));
      st3(w.S + d * 6, ax);
      st3(w.S + d * 6 + 3, an);
    }
  }
  __syncwarp();
}

// Stage timers of the diagnostic (bounds-checked) build: with a debug buffer, environment 0 adds the clocks each stage
// of its first substep took to dbg[PHYS_TIMER_BASE + stage].  The normal build compiles them away.
#define PHYS_TIMER_BASE 240
#if defined(NB_BOUNDS) && NB_BOUNDS
#define PHYS_STAGE_BEGIN() long long tstage_ = clock64()
#define PHYS_STAGE(i)                                             \
  do {                                                            \
    if (dbg && lane == 0) {                                       \
      const long long t_ = clock64();                             \
      dbg[PHYS_TIMER_BASE + (i)] += (float)(t_ - tstage_);        \
      tstage_ = t_;                                               \
    }                                                             \
  } while (0)
#else
#define PHYS_STAGE_BEGIN() do {} while (0)
#define PHYS_STAGE(i) do {} while (0)
#endif

// One dynamics substep for the env owned by this warp.  qpos/qvel/ctrl live in registers of
// lane d (< nv); everything else in the warp's shared scratch.
__device__ __forceinline__ void substep(const PhysParams& P, const ModelView& m, WarpScratch& w, float& qpos,
                                        float& qvel, float tau_act, float* warm, int lane, float* dbg) {
  const int nv = P.nv, nvp = P.nvp, nbody = P.nbody;
  float* qpos_sh = w.vec;        // [32]
  float* qvel_sh = w.vec + 32;   // [32]
  float* qacc_sh = w.vec + 64;   // [32] smooth acceleration
  float* tau_sh = w.vec + 96;    // [32]
  qpos_sh[lane] = qpos;
  qvel_sh[lane] = qvel;
  __syncwarp();
  PHYS_STAGE_BEGIN();

  forward_kinematics(P, m, w, qpos_sh, lane);
  const V3 c = ld3(w.xpos);  // reference point: origin of body 0
  PHYS_STAGE(0);

  // ---- motion axes about c (lane = dof) and body inertias about c (lane = body)
  if (lane < nv) {
    const V3 ax = ld3(w.S + lane * 6);
    if (m.dof_type[lane] == NB_JOINT_HINGE) {
      const V3 r = ld3(w.S + lane * 6 + 3) - c;
      st3(w.S + lane * 6 + 3, cross(r, ax));
    } else {
      st3(w.S + lane * 6, v3(0.f, 0.f, 0.f));
      st3(w.S + lane * 6 + 3, ax);
    }
  }
  if (lane < nbody) {
    const float* R = w.xmat + lane * 9;
    const float* Ib = m.body_inertia6 + lane * 6;  // body frame: xx yy zz xy xz yz
    // A = R * Ib (3x3), Iw = A * R^T
    const float b00 = Ib[0], b11 = Ib[1], b22 = Ib[2], b01 = Ib[3], b02 = Ib[4], b12 = Ib[5];
    float A[9];
#pragma unroll
    for (int r = 0; r < 3; ++r) {
      A[r * 3 + 0] = R[r * 3] * b00 + R[r * 3 + 1] * b01 + R[r * 3 + 2] * b02;
      A[r * 3 + 1] = R[r * 3] * b01 + R[r * 3 + 1] * b11 + R[r * 3 + 2] * b12;
      A[r * 3 + 2] = R[r * 3] * b02 + R[r * 3 + 1] * b12 + R[r * 3 + 2] * b22;
    }
    float Iw[6];
    Iw[0] = A[0] * R[0] + A[1] * R[1] + A[2] * R[2];
    Iw[1] = A[3] * R[3] + A[4] * R[4] + A[5] * R[5];
    Iw[2] = A[6] * R[6] + A[7] * R[7] + A[8] * R[8];
    Iw[3] = A[0] * R[3] + A[1] * R[4] + A[2] * R[5];
    Iw[4] = A[0] * R[6] + A[1] * R[7] + A[2] * R[8];
    Iw[5] = A[3] * R[6] + A[4] * R[7] + A[5] * R[8];
    const float mass = m.body_mass[lane];
    const V3 ip = ld3(m.body_ipos + lane * 3);
    const V3 h = ld3(w.xpos + lane * 3) + v3(R[0] * ip.x + R[1] * ip.y + R[2] * ip.z,
                                             R[3] * ip.x + R[4] * ip.y + R[5] * ip.z,
                                             R[6] * ip.x + R[7] * ip.y + R[8] * ip.z) - c;
    const float hh = dot(h, h);
    float* I = w.I + lane * 10;
    I[0] = Iw[0] + mass * (hh - h.x * h.x);
    I[1] = Iw[1] + mass * (hh - h.y * h.y);
    I[2] = Iw[2] + mass * (hh - h.z * h.z);
    I[3] = Iw[3] - mass * h.x * h.y;
    I[4] = Iw[4] - mass * h.x * h.z;
    I[5] = Iw[5] - mass * h.y * h.z;
    I[6] = mass * h.x;
    I[7] = mass * h.y;
    I[8] = mass * h.z;
    I[9] = mass;
  }
  __syncwarp();

  PHYS_STAGE(1);
  // ---- body velocity, bias acceleration and the resulting spatial force (lane = body)
  if (lane < nbody) {
    V3 vw = v3(0, 0, 0), vv = v3(0, 0, 0);            // cumulative spatial velocity
    V3 aw = v3(0, 0, 0), av = v3(-P.gx, -P.gy, -P.gz);  // gravity as base acceleration
    unsigned mask = (unsigned)m.body_dofmask[lane];
    while (mask) {
      const int d = __ffs(mask) - 1;
      mask &= mask - 1;
      const V3 sw = ld3(w.S + d * 6), sv = ld3(w.S + d * 6 + 3);
      const float qd = qvel_sh[d];
      // crm(V_cum) S_d * qd
      aw = aw + qd * cross(vw, sw);
      av = av + qd * (cross(vw, sv) + cross(vv, sw));
      vw = vw + qd * sw;
      vv = vv + qd * sv;
    }
    st3(w.V + lane * 6, vw);
    st3(w.V + lane * 6 + 3, vv);
    V3 n1, f1, n2, f2;
    inertia_mul(w.I + lane * 10, aw, av, n1, f1);
    inertia_mul(w.I + lane * 10, vw, vv, n2, f2);
    // crf(V) [n2; f2] = [w × n2 + v × f2 ; w × f2]
    st3(w.F + lane * 6, n1 + cross(vw, n2) + cross(vv, f2));
    st3(w.F + lane * 6 + 3, f1 + cross(vw, f2));
  }
  __syncwarp();

  PHYS_STAGE(2);
  // ---- composite inertias (lane = body): Ic_b = Σ_{b' : b ∈ anc(b')} I_b'
  if (lane < nbody) {
    float acc[10];
#pragma unroll
    for (int k = 0; k < 10; ++k) acc[k] = 0.f;
    for (int b2 = lane; b2 < nbody; ++b2) {
      if ((unsigned)m.body_ancmask[b2] >> lane & 1u) {
#pragma unroll
        for (int k = 0; k < 10; ++k) acc[k] += w.I[b2 * 10 + k];
      }
    }
#pragma unroll
    for (int k = 0; k < 10; ++k) w.Ic[lane * 10 + k] = acc[k];
  }
  PHYS_STAGE(3);
  // ---- bias force per dof (lane = dof): S_d · Σ_{b in subtree(body(d))} f_b
  float bias = 0.f;
  if (lane < nv) {
    V3 fn = v3(0, 0, 0), ff = v3(0, 0, 0);
    for (int b2 = m.dof_body[lane]; b2 < nbody; ++b2) {
      if ((unsigned)m.body_dofmask[b2] >> lane & 1u) {
        fn = fn + ld3(w.F + b2 * 6);
        ff = ff + ld3(w.F + b2 * 6 + 3);
      }
    }
    bias = dot(ld3(w.S + lane * 6), fn) + dot(ld3(w.S + lane * 6 + 3), ff);
  }
  __syncwarp();

  PHYS_STAGE(4);
  // ---- CRBA (lane = dof i): M[i][j] = S_j · (Ic_body(i) S_i) for ancestor dofs j <= i
  if (lane < nv) {
    const int i = lane, bi = m.dof_body[i];
    V3 n, f;
    inertia_mul(w.Ic + bi * 10, ld3(w.S + i * 6), ld3(w.S + i * 6 + 3), n, f);
    const unsigned mask = (unsigned)m.body_dofmask[bi];
    for (int j = 0; j <= i; ++j) {
      float v = 0.f;
      if (mask >> j & 1u) v = dot(ld3(w.S + j * 6), n) + dot(ld3(w.S + j * 6 + 3), f);
      if (j == i) v += m.dof_armature[i] + P.dt * m.dof_damping[i];
      w.M[i * nvp + j] = v;
      w.M[j * nvp + i] = v;
    }
    tau_sh[lane] = tau_act - bias - m.dof_damping[lane] * qvel - m.dof_stiffness[lane] * (qpos - m.dof_springref[lane]);
  }
  __syncwarp();
  if (dbg && lane < nv) {
    for (int j = 0; j < nv; ++j) dbg[lane * nv + j] = w.M[lane * nvp + j];
    dbg[nv * nv + lane] = bias;
  }
  __syncwarp();

  PHYS_STAGE(5);
  // ---- in-place Cholesky M̂ = L Lᵀ (lower).  Column k: lane r > k scales, then trailing update.
  auto cholesky_stage = [&](auto nv_tag) {
    constexpr int NV = decltype(nv_tag)::value;
    if constexpr (NV > 0) {
      // lane r keeps row r of the matrix in registers; the column of the current pivot travels by shuffles, so the
      // factorisation needs neither shared-memory round trips nor warp barriers between its NV dependent columns
      float Lr[NV];
      const int rr = lane < NV ? lane : NV - 1;
#pragma unroll
      for (int j = 0; j < NV; ++j) Lr[j] = w.M[rr * nvp + j];
#pragma unroll
      for (int k = 0; k < NV; ++k) {
        const float dkk = __shfl_sync(0xffffffffu, Lr[k], k);
        const float inv = rsqrtf(fmaxf(dkk, 1e-10f));
        const float lrk = Lr[k] * inv;                 // L[r][k] for r > k
        if (lane == k) Lr[k] = inv;                    // the diagonal keeps 1/L_kk
        else if (lane > k) Lr[k] = lrk;
#pragma unroll
        for (int cc = 0; cc < NV; ++cc) {
          if (cc > k) {
            const float lck = __shfl_sync(0xffffffffu, lrk, cc);
            if (lane >= cc) Lr[cc] -= lrk * lck;
          }
        }
      }
#pragma unroll
      for (int j = 0; j < NV; ++j)
        if (lane < NV && j <= lane) w.M[lane * nvp + j] = Lr[j];
      __syncwarp();
    } else {
      for (int k = 0; k < nv; ++k) {
        float dkk = w.M[k * nvp + k];
        const float inv = rsqrtf(fmaxf(dkk, 1e-10f));
        __syncwarp();
        if (lane == k) w.M[k * nvp + k] = inv;  // the diagonal keeps 1/L_kk
        if (lane > k && lane < nv) w.M[lane * nvp + k] *= inv;
        __syncwarp();
        // trailing: element (r, c) for k < c <= r < nv; lanes stride over the flattened lower triangle rows
        if (lane > k && lane < nv) {
          const float lrk = w.M[lane * nvp + k];
          for (int cc = k + 1; cc <= lane; ++cc) w.M[lane * nvp + cc] -= lrk * w.M[cc * nvp + k];
        }
        __syncwarp();
      }
    }
  };
  if (nv == 9) cholesky_stage(std::integral_constant<int, 9>{});
  else cholesky_stage(std::integral_constant<int, 0>{});

  PHYS_STAGE(6);
  // ---- constraint detection.  Slots: [0, nlimit) joint limits, [nlimit, nlimit+ncs) contact spheres.
  // Rows are allocated by ballot compaction: first all unilateral rows (limit / normal), then two
  // tangent rows per contact while space remains.
  const int nslot = P.nlimit + P.ncs;
  int nrow = 0;
  const V3 pn = v3(P.plane_nx, P.plane_ny, P.plane_nz);
  for (int s0 = 0; s0 < nslot; s0 += 32) {
    const int s = s0 + lane;
    bool active = false;
    float dist = 0.f, sgn = 1.f;
    if (s < P.nlimit) {
      const int d = m.lim_dof[s];
      const float q = qpos_sh[d];
      const float dlo = q - m.lim_lo[s], dhi = m.lim_hi[s] - q;
      if (dlo < dhi) { dist = dlo; sgn = 1.f; } else { dist = dhi; sgn = -1.f; }
      active = dist < P.margin;
    } else if (s < nslot) {
      const int cs = s - P.nlimit, b = m.cs_body[cs];
      const float* R = w.xmat + b * 9;
      const V3 l = ld3(m.cs_local + cs * 3);
      const V3 p = ld3(w.xpos + b * 3) + v3(R[0] * l.x + R[1] * l.y + R[2] * l.z, R[3] * l.x + R[4] * l.y + R[5] * l.z,
                                           R[6] * l.x + R[7] * l.y + R[8] * l.z);
      dist = dot(pn, p) - P.plane_off - m.cs_radius[cs];
      active = dist < P.margin;
    }
    const unsigned bal = __ballot_sync(0xffffffffu, active);
    const int my = nrow + __popc(bal & ((1u << lane) - 1u));
    if (active && my < P.rmax) {
      w.rowi[my * 4 + 0] = (s < P.nlimit) ? ROW_LIMIT : ROW_NORMAL;
      w.rowi[my * 4 + 1] = s;
      w.rowi[my * 4 + 2] = -1;
      w.row[my * 4 + 0] = dist;
      w.row[my * 4 + 1] = sgn;
    }
    nrow = min(P.rmax, nrow + __popc(bal));
    if (!active && s < nslot) {  // inactive slots forget their multipliers
      if (s < P.nlimit) warm[s] = 0.f;
      else { const int o = P.nlimit + (s - P.nlimit) * 3; warm[o] = 0.f; warm[o + 1] = 0.f; warm[o + 2] = 0.f; }
    }
  }
  __syncwarp();
  const int nuni = nrow;
  if (P.friction_rows) {
    for (int r0 = 0; r0 < nuni; r0 += 32) {
      const int r = r0 + lane;
      const bool isn = (r < nuni) && w.rowi[r * 4] == ROW_NORMAL;
      const unsigned bal = __ballot_sync(0xffffffffu, isn);
      const int nd = P.friction_rows;  // 1: planar model (only t1 can move), 2: t1 and t2
      const int my = nrow + nd * __popc(bal & ((1u << lane) - 1u));
      if (isn && my + nd - 1 < P.rmax) {  // written for a prefix of the contacts only
        for (int t = 0; t < nd; ++t) {
          w.rowi[(my + t) * 4 + 0] = ROW_TANGENT + t;
          w.rowi[(my + t) * 4 + 1] = w.rowi[r * 4 + 1];
          w.rowi[(my + t) * 4 + 2] = r;
          w.row[(my + t) * 4 + 0] = 0.f;
          w.row[(my + t) * 4 + 1] = 1.f;
        }
      }
      const int fit = max(0, (P.rmax - nrow) / nd);
      nrow += nd * min(fit, __popc(bal));
    }
  }
  __syncwarp();

  // tangent frame of the plane
  V3 t1 = v3(1.f, 0.f, 0.f) - pn.x * pn;
  {
    const float l2 = dot(t1, t1);
    if (l2 < 1e-6f) t1 = v3(0.f, 1.f, 0.f) - pn.y * pn;
    t1 = rsqrtf(dot(t1, t1)) * t1;
  }
  const V3 t2 = cross(pn, t1);

  PHYS_STAGE(7);
  // ---- per row (lane = row): Jacobian row, B = M̂⁻¹ Jᵀ, diag, aref, R.  Row `nrow` (virtual)
  // is the smooth solve qacc = M̂⁻¹ tau, handled by the same triangular solves.
  const float k_s = 1.f / (P.solimp_dmax * P.solimp_dmax * P.solref_tc * P.solref_tc * P.solref_dr * P.solref_dr);
  const float b_s = 2.f / (P.solimp_dmax * P.solref_tc);
  // The solves of a row are a dependency chain; with the dof count known at compile time the loops unroll, the row's
  // J and B live in registers (instead of going through shared memory and back between dependent steps) and the loads
  // of the factor are hoisted ahead of the chain.  NV = 0 is the generic path with run-time loops.
  auto rows_stage = [&](auto nv_tag) {
    constexpr int NV = decltype(nv_tag)::value;
    if constexpr (NV > 0) {
      for (int r0 = 0; r0 <= nrow; r0 += 32) {
        const int r = r0 + lane;
        if (r <= nrow) {
          const bool smooth = (r == nrow);
          float Jl[NV], Bl[NV];
          int kind = 0, slot = 0;
          if (smooth) {
#pragma unroll
            for (int j = 0; j < NV; ++j) Jl[j] = tau_sh[j];
          } else {
            kind = w.rowi[r * 4];
            slot = w.rowi[r * 4 + 1];
            if (kind == ROW_LIMIT) {
              const int d = m.lim_dof[slot];
              const float sgn = w.row[r * 4 + 1];
#pragma unroll
              for (int j = 0; j < NV; ++j) Jl[j] = (j == d) ? sgn : 0.f;
            } else {
              const int cs = slot - P.nlimit, b = m.cs_body[cs];
              const float* R = w.xmat + b * 9;
              const V3 l = ld3(m.cs_local + cs * 3);
              const V3 p = ld3(w.xpos + b * 3) + v3(R[0] * l.x + R[1] * l.y + R[2] * l.z, R[3] * l.x + R[4] * l.y + R[5] * l.z,
                                                   R[6] * l.x + R[7] * l.y + R[8] * l.z);
              const float dist = dot(pn, p) - P.plane_off - m.cs_radius[cs];
              const V3 pc = p - (m.cs_radius[cs] + 0.5f * dist) * pn - c;  // contact point relative to c
              const V3 dir = (kind == ROW_NORMAL) ? pn : (kind == ROW_TANGENT ? t1 : t2);
              const unsigned mask = (unsigned)m.body_dofmask[b];
#pragma unroll
              for (int j = 0; j < NV; ++j) {
                float v = 0.f;
                if (mask >> j & 1u) {
                  const V3 sw = ld3(w.S + j * 6), sv = ld3(w.S + j * 6 + 3);
                  v = dot(dir, sv + cross(sw, pc));
                }
                Jl[j] = v;
              }
            }
          }
          // forward solve L y = J, then back solve Lᵀ x = y
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            float acc = Jl[i];
#pragma unroll
            for (int j = 0; j < i; ++j) acc -= w.M[i * nvp + j] * Bl[j];
            Bl[i] = acc * w.M[i * nvp + i];
          }
#pragma unroll
          for (int i = NV - 1; i >= 0; --i) {
            float acc = Bl[i];
#pragma unroll
            for (int j = i + 1; j < NV; ++j) acc -= w.M[j * nvp + i] * Bl[j];
            Bl[i] = acc * w.M[i * nvp + i];
          }
          float* Br = smooth ? qacc_sh : (w.B + r * nvp);
#pragma unroll
          for (int j = 0; j < NV; ++j) Br[j] = Bl[j];
          if (!smooth) {
            float* Jr = w.J + r * nvp;
            float diag = 0.f, vel = 0.f;
#pragma unroll
            for (int j = 0; j < NV; ++j) {
              Jr[j] = Jl[j];
              diag += Jl[j] * Bl[j];
              vel += Jl[j] * qvel_sh[j];
            }
            diag = fmaxf(diag, 1e-10f);
            const float dist = w.row[r * 4 + 0];
            const float imp = impedance(P, fabsf(dist));
            float aref, Rr;
            if (kind == ROW_LIMIT || kind == ROW_NORMAL) {
              aref = -b_s * vel - k_s * imp * dist;
              Rr = (1.f - imp) / imp * diag;
            } else {
              aref = -b_s * vel;
              const float impf = P.solimp_dmax;
              Rr = (1.f - impf) / impf * diag * P.friction_reg;
            }
            int ws;
            if (kind == ROW_LIMIT) ws = slot;
            else ws = P.nlimit + (slot - P.nlimit) * 3 + (kind == ROW_NORMAL ? 0 : (kind == ROW_TANGENT ? 1 : 2));
            w.row[r * 4 + 0] = aref;
            w.row[r * 4 + 1] = Rr;
            w.row[r * 4 + 2] = 1.f / (diag + Rr);
            w.row[r * 4 + 3] = warm[ws];
            w.rowi[r * 4 + 3] = ws;
          }
        }
      }
    } else {
      for (int r0 = 0; r0 <= nrow; r0 += 32) {
        const int r = r0 + lane;
        if (r <= nrow) {
          const bool smooth = (r == nrow);
          float* Jr = smooth ? tau_sh : (w.J + r * nvp);
          float* Br = smooth ? qacc_sh : (w.B + r * nvp);
          int kind = 0, slot = 0;
          if (!smooth) {
            kind = w.rowi[r * 4];
            slot = w.rowi[r * 4 + 1];
            if (kind == ROW_LIMIT) {
              const int d = m.lim_dof[slot];
              const float sgn = w.row[r * 4 + 1];
              for (int j = 0; j < nv; ++j) Jr[j] = (j == d) ? sgn : 0.f;
            } else {
              const int cs = slot - P.nlimit, b = m.cs_body[cs];
              const float* R = w.xmat + b * 9;
              const V3 l = ld3(m.cs_local + cs * 3);
              const V3 p = ld3(w.xpos + b * 3) + v3(R[0] * l.x + R[1] * l.y + R[2] * l.z, R[3] * l.x + R[4] * l.y + R[5] * l.z,
                                                   R[6] * l.x + R[7] * l.y + R[8] * l.z);
              const float dist = dot(pn, p) - P.plane_off - m.cs_radius[cs];
              const V3 pc = p - (m.cs_radius[cs] + 0.5f * dist) * pn - c;  // contact point relative to c
              const V3 dir = (kind == ROW_NORMAL) ? pn : (kind == ROW_TANGENT ? t1 : t2);
              const unsigned mask = (unsigned)m.body_dofmask[b];
              for (int j = 0; j < nv; ++j) {
                float v = 0.f;
                if (mask >> j & 1u) {
                  const V3 sw = ld3(w.S + j * 6), sv = ld3(w.S + j * 6 + 3);
                  v = dot(dir, sv + cross(sw, pc));
                }
                Jr[j] = v;
              }
            }
          }
          // forward solve L y = J, then back solve Lᵀ x = y
          for (int i = 0; i < nv; ++i) {
            float acc = Jr[i];
            for (int j = 0; j < i; ++j) acc -= w.M[i * nvp + j] * Br[j];
            Br[i] = acc * w.M[i * nvp + i];
          }
          for (int i = nv - 1; i >= 0; --i) {
            float acc = Br[i];
            for (int j = i + 1; j < nv; ++j) acc -= w.M[j * nvp + i] * Br[j];
            Br[i] = acc * w.M[i * nvp + i];
          }
          if (!smooth) {
            float diag = 0.f, vel = 0.f;
            for (int j = 0; j < nv; ++j) {
              diag += Jr[j] * Br[j];
              vel += Jr[j] * qvel_sh[j];
            }
            diag = fmaxf(diag, 1e-10f);
            const float dist = w.row[r * 4 + 0];
            const float imp = impedance(P, fabsf(dist));
            float aref, Rr;
            if (kind == ROW_LIMIT || kind == ROW_NORMAL) {
              aref = -b_s * vel - k_s * imp * dist;
              Rr = (1.f - imp) / imp * diag;
            } else {
              aref = -b_s * vel;
              const float impf = P.solimp_dmax;
              Rr = (1.f - impf) / impf * diag * P.friction_reg;
            }
            // warm start slot index
            int ws;
            if (kind == ROW_LIMIT) ws = slot;
            else ws = P.nlimit + (slot - P.nlimit) * 3 + (kind == ROW_NORMAL ? 0 : (kind == ROW_TANGENT ? 1 : 2));
            w.row[r * 4 + 0] = aref;
            w.row[r * 4 + 1] = Rr;
            w.row[r * 4 + 2] = 1.f / (diag + Rr);
            w.row[r * 4 + 3] = warm[ws];
            w.rowi[r * 4 + 3] = ws;
          }
        }
      }
    }
  };
  if (nv == 9) rows_stage(std::integral_constant<int, 9>{});
  else rows_stage(std::integral_constant<int, 0>{});
  __syncwarp();
  if (dbg) {
    if (lane < nv) { dbg[nv * nv + nv + lane] = qacc_sh[lane]; }
    if (lane == 0) dbg[nv * nv + 3 * nv] = (float)nrow;
  }

  PHYS_STAGE(8);
  // ---- projected Gauss-Seidel.  Dual form, lane = row: each lane keeps c_r = J_r·qacc − aref_r (without
  // the R_r λ_r term) in a register; when row s moves by Δλ every lane adds A_rs·Δλ with
  // A = J M̂⁻¹ Jᵀ, so a row update costs two shuffles instead of a cross-lane dot product.  The iterates
  // are those of the primal sweep (qacc += B_s Δλ) in exact arithmetic.
  float qacc;
  if (P.rmax <= 32) {
    const int r = lane;
    const bool on = r < nrow;
    float c = 0.f, lam = 0.f, k1 = 0.f, invd = 0.f, mu = 0.f;
    int parent = 0;
    // A[r][s] = A[s][r] lives at tri(max) + min with tri(k) = k(k+1)/2; the triangular numbers are a permutation
    // modulo 32, so a sweep column is read without bank conflicts.  Lane r writes its own row's lower part only
    // (one writer per element: deterministic).
    const int tri_r = r * (r + 1) / 2;
    if (on) {
      float acc = 0.f;
      for (int j = 0; j < nv; ++j) acc += w.J[r * nvp + j] * qacc_sh[j];
      c = acc - w.row[r * 4 + 0];
      invd = w.row[r * 4 + 2];
      k1 = 1.f - w.row[r * 4 + 1] * invd;  // λ_new = λ·k1 − c·invd
      lam = w.row[r * 4 + 3];
      parent = max(w.rowi[r * 4 + 2], 0);
      if (w.rowi[r * 4] >= ROW_TANGENT) mu = m.cs_mu[w.rowi[r * 4 + 1] - P.nlimit];
    }
    __syncwarp();  // every lane has read what it needs from the arrays that A overlays (none are read below)
    if (on) {
      if (nv == 9) {   // dof count known: the row of J stays in registers, the dot products unroll
        float Jl[9];
#pragma unroll
        for (int j = 0; j < 9; ++j) Jl[j] = w.J[r * nvp + j];
        for (int s2 = 0; s2 <= r; ++s2) {
          const float* Bs = w.B + s2 * nvp;
          float a0 = 0.f, a1 = 0.f, a2 = 0.f;
#pragma unroll
          for (int j = 0; j < 9; j += 3) {
            a0 += Jl[j] * Bs[j];
            a1 += Jl[j + 1] * Bs[j + 1];
            a2 += Jl[j + 2] * Bs[j + 2];
          }
          w.A[tri_r + s2] = a0 + a1 + a2;
        }
      } else {
        for (int s2 = 0; s2 <= r; ++s2) {
          float a = 0.f;
          for (int j = 0; j < nv; ++j) a += w.J[r * nvp + j] * w.B[s2 * nvp + j];
          w.A[tri_r + s2] = a;
        }
      }
    }
    __syncwarp();
#define NB_A_AT(s2, tri_s) (on ? w.A[(s2) <= r ? tri_r + (s2) : (tri_s) + r] : 0.f)
    for (int s2 = 0, ts = 0; s2 < nrow; ts += ++s2) {  // warm start
      const float ls = __shfl_sync(0xffffffffu, lam, s2);
      c += NB_A_AT(s2, ts) * ls;
    }
    for (int it = 0; it < P.pgs_iters; ++it) {
      // unilateral rows [0, nuni): limits and contact normals
      int ts = 0;
      for (int s2 = 0; s2 < nuni; ts += ++s2) {
        const float a_rs = NB_A_AT(s2, ts);
        const float ln = fmaxf(lam * k1 - c * invd, 0.f);
        const float dl = __shfl_sync(0xffffffffu, ln - lam, s2);
        if (lane == s2) lam = ln;
        c += a_rs * dl;
      }
      // friction rows [nuni, nrow): box bounds from the parent normal multiplier
      for (int s2 = nuni; s2 < nrow; ts += ++s2) {
        const float a_rs = NB_A_AT(s2, ts);
        const float bound = mu * __shfl_sync(0xffffffffu, lam, parent);
        const float ln = fminf(fmaxf(lam * k1 - c * invd, -bound), bound);
        const float dl = __shfl_sync(0xffffffffu, ln - lam, s2);
        if (lane == s2) lam = ln;
        c += a_rs * dl;
      }
    }
#undef NB_A_AT
    if (on) w.row[r * 4 + 3] = lam;
    qacc = (lane < nv) ? qacc_sh[lane] : 0.f;
    for (int s2 = 0; s2 < nrow; ++s2) {
      const float ls = __shfl_sync(0xffffffffu, lam, s2);
      if (lane < nv) qacc += w.B[s2 * nvp + lane] * ls;
    }
    __syncwarp();
  } else {
    // primal sweep for models that need more than 32 rows (lane = dof)
    qacc = (lane < nv) ? qacc_sh[lane] : 0.f;
    for (int r = 0; r < nrow; ++r) {
      const float lam = w.row[r * 4 + 3];
      if (lam != 0.f && lane < nv) qacc += w.B[r * nvp + lane] * lam;
    }
    for (int it = 0; it < P.pgs_iters; ++it) {
      for (int r = 0; r < nrow; ++r) {
        float part = (lane < nv) ? w.J[r * nvp + lane] * qacc : 0.f;
        part = warp_sum(part);
        const float lam = w.row[r * 4 + 3];
        const float res = part - w.row[r * 4 + 0] + w.row[r * 4 + 1] * lam;
        float ln = lam - res * w.row[r * 4 + 2];
        const int kind = w.rowi[r * 4];
        if (kind <= ROW_NORMAL) {
          ln = fmaxf(ln, 0.f);
        } else {
          const int pr = w.rowi[r * 4 + 2];
          const float bound = m.cs_mu[w.rowi[r * 4 + 1] - P.nlimit] * w.row[pr * 4 + 3];
          ln = fminf(fmaxf(ln, -bound), bound);
        }
        const float dl = ln - lam;
        if (lane == 0) w.row[r * 4 + 3] = ln;
        if (lane < nv) qacc += w.B[r * nvp + lane] * dl;
        __syncwarp();
      }
    }
  }
  PHYS_STAGE(9);
  // store multipliers for the next substep
  for (int r = lane; r < nrow; r += 32) warm[w.rowi[r * 4 + 3]] = w.row[r * 4 + 3];
  if (dbg && lane < nv) dbg[nv * nv + 2 * nv + lane] = qacc;

  PHYS_STAGE(10);
  // ---- semi-implicit Euler
  if (lane < nv) {
    if (!isfinite(qacc)) qacc = 0.f;
    qvel += P.dt * qacc;
    qvel = fminf(fmaxf(qvel, -P.max_vel), P.max_vel);
    qpos += P.dt * qvel;
  }
  __syncwarp();
}

// ------------------------------------------------------------------------------------------
// WARPS environments per block, MINB blocks per SM: <7, 4> keeps 28 environments resident per SM (4096 on 148 SMs
// in one wave) at 72 registers per thread; <8, 2> is the general form for models with a larger scratch.
template <int WARPS, int MINB>
__global__ void __launch_bounds__(WARPS * 32, MINB)
phys_env_step_kernel(PhysParams P, const int* __restrict__ imodel, const float* __restrict__ fmodel,
                     float* __restrict__ qpos_g, float* __restrict__ qvel_g, float* __restrict__ warm_g,
                     int* __restrict__ step_count, float* __restrict__ ep_return, const float* __restrict__ action,
                     int action_stride, float* __restrict__ obs_f32, __nv_bfloat16* __restrict__ obs_bf16,
                     int obs_bf16_stride, float* __restrict__ next_obs_f32, __nv_bfloat16* __restrict__ next_obs_bf16,
                     float* __restrict__ reward, float* __restrict__ done, float* __restrict__ terminated,
                     float* __restrict__ finished_return, const unsigned long long* __restrict__ rng_counter,
                     unsigned long long seed, int n_envs, int do_reset, float* __restrict__ ep_stats,
                     float* __restrict__ dbg) {
  extern __shared__ __align__(16) float smem[];
  // stage the model
  int* im_sh = reinterpret_cast<int*>(smem);
  float* fm_sh = smem + P.imodel_words;
  for (int i = threadIdx.x; i < P.imodel_words; i += blockDim.x) im_sh[i] = imodel[i];
  for (int i = threadIdx.x; i < P.fmodel_words; i += blockDim.x) fm_sh[i] = fmodel[i];
  __syncthreads();
  const ModelView m = view(im_sh, fm_sh, P);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int env = blockIdx.x * (int)(blockDim.x >> 5) + warp;
  if (env >= n_envs) return;
  float* base = smem + P.imodel_words + P.fmodel_words + warp * P.warp_words;
  WarpScratch w = carve(base, P);
  const int nv = P.nv;
  const int nwarm = P.nlimit + 3 * P.ncs;
  float* warm = base + P.warp_words - P.warm_words;  // tail of the warp scratch
  for (int i = lane; i < nwarm; i += 32) warm[i] = warm_g[(size_t)env * nwarm + i];

  float qpos = 0.f, qvel = 0.f, tau_act = 0.f;
  if (lane < nv) {
    qpos = qpos_g[(size_t)env * nv + lane];
    qvel = qvel_g[(size_t)env * nv + lane];
  }
  // actuator forces: tau[dof] = gear * clamp(ctrl)
  float ctrl_cost = 0.f;
  for (int a = 0; a < P.nu; ++a) {
    float u = action[(size_t)env * action_stride + a];
    if (!isfinite(u)) u = 0.f;
    u = fminf(fmaxf(u, m.act_lo[a]), m.act_hi[a]);
    ctrl_cost += u * u;
    if (m.act_dof[a] == lane) tau_act += m.act_gear[a] * u;
  }
  const float x_before = __shfl_sync(0xffffffffu, qpos, P.forward_dof);
  __syncwarp();

  for (int s = 0; s < P.frame_skip; ++s) {
    substep(P, m, w, qpos, qvel, tau_act, warm, lane, (dbg && env == 0 && s == 0) ? dbg : nullptr);
  }

  const float x_after = __shfl_sync(0xffffffffu, qpos, P.forward_dof);
  const float fwd = (x_after - x_before) / (P.dt * P.frame_skip);
  float rew = P.w_forward * fwd - P.w_ctrl * ctrl_cost + P.w_alive;
  // divergence guard: a non-finite state or a velocity pinned at the clamp ends the episode with zero
  // reward (the reference ends a lane whose obs/reward goes non-finite, docs algorithms/ppo.mdx:231-232)
  const bool bad = __any_sync(0xffffffffu, !isfinite(qpos) || !isfinite(qvel) || fabsf(qvel) >= P.max_vel);
  bool term = bad;
  if (P.term_dof >= 0) {
    const float a = __shfl_sync(0xffffffffu, qpos, P.term_dof);
    term = term || (a < P.term_lo) || (a > P.term_hi);
  }
  if (bad) rew = 0.f;
  int steps = step_count[env] + 1;
  const bool trunc = steps >= P.max_steps;
  const bool dn = term || trunc;

  // pre-reset observation (bootstrap state): obs = qpos[skip:] ‖ qvel
  const int nobs = (nv - P.obs_qpos_skip) + nv;
  {
    const float qp = bad ? 0.f : qpos, qv = bad ? 0.f : fminf(fmaxf(qvel, -P.obs_clip), P.obs_clip);
    if (lane < nv) {
      if (lane >= P.obs_qpos_skip) {
        const int o = lane - P.obs_qpos_skip;
        if (next_obs_f32) next_obs_f32[(size_t)env * nobs + o] = qp;
        if (next_obs_bf16) next_obs_bf16[(size_t)env * obs_bf16_stride + o] = __float2bfloat16(qp);
      }
      const int o = nv - P.obs_qpos_skip + lane;
      if (next_obs_f32) next_obs_f32[(size_t)env * nobs + o] = qv;
      if (next_obs_bf16) next_obs_bf16[(size_t)env * obs_bf16_stride + o] = __float2bfloat16(qv);
    }
  }
  float ret = ep_return[env] + rew;
  if (lane == 0) {
    reward[env] = rew;
    done[env] = dn ? 1.f : 0.f;
    terminated[env] = term ? 1.f : 0.f;
    if (finished_return) finished_return[env] = dn ? ret : NAN;
    if (ep_stats) {  // [0] Σ finished returns, [1] finished episodes, [2] Σ reward, [3] Σ episode length
      if (dn) {
        atomicAdd(ep_stats + 0, ret);
        atomicAdd(ep_stats + 1, 1.f);
        atomicAdd(ep_stats + 3, (float)steps);
      }
      atomicAdd(ep_stats + 2, rew);
    }
  }
  if (dn && do_reset) {
    // selective reset: qpos0 + U(-noise, noise), qvel = U(-noise, noise); counter based RNG
    const unsigned long long ctr = rng_counter ? rng_counter[0] : 0ull;
    Philox ph(seed);
    uint32_t rnd[4];
    ph((uint32_t)env, (uint32_t)lane, (uint32_t)ctr, (uint32_t)(ctr >> 32), rnd);
    const float npos = m.reset_noise[0], nvel = m.reset_noise[1];
    if (lane < nv) {
      qpos = m.qpos0[lane] + npos * (2.f * u32_to_unit(rnd[0]) - 1.f);
      qvel = nvel * (2.f * u32_to_unit(rnd[1]) - 1.f);
    }
    for (int i = lane; i < nwarm; i += 32) warm[i] = 0.f;
    steps = 0;
    ret = 0.f;
  }
  if (lane == 0) {
    step_count[env] = steps;
    ep_return[env] = ret;
  }
  if (lane < nv) {
    qpos_g[(size_t)env * nv + lane] = qpos;
    qvel_g[(size_t)env * nv + lane] = qvel;
    const float qv = fminf(fmaxf(qvel, -P.obs_clip), P.obs_clip);
    if (lane >= P.obs_qpos_skip) {
      const int o = lane - P.obs_qpos_skip;
      if (obs_f32) obs_f32[(size_t)env * nobs + o] = qpos;
      if (obs_bf16) obs_bf16[(size_t)env * obs_bf16_stride + o] = __float2bfloat16(qpos);
    }
    const int o = nv - P.obs_qpos_skip + lane;
    if (obs_f32) obs_f32[(size_t)env * nobs + o] = qv;
    if (obs_bf16) obs_bf16[(size_t)env * obs_bf16_stride + o] = __float2bfloat16(qv);
  }
  for (int i = lane; i < nwarm; i += 32) warm_g[(size_t)env * nwarm + i] = warm[i];
}

// Reset every env (or only those with mask != 0) and write the observation.
__global__ void phys_env_reset_kernel(PhysParams P, const float* __restrict__ fmodel, float* __restrict__ qpos_g,
                                      float* __restrict__ qvel_g, float* __restrict__ warm_g,
                                      int* __restrict__ step_count, float* __restrict__ ep_return,
                                      const float* __restrict__ mask, float* __restrict__ obs_f32,
                                      __nv_bfloat16* __restrict__ obs_bf16, int obs_bf16_stride,
                                      unsigned long long seed, unsigned long long counter, int n_envs) {
  const int env = blockIdx.x * blockDim.x + threadIdx.x;
  if (env >= n_envs) return;
  if (mask && mask[env] == 0.f) return;
  const ModelView m = view(nullptr, fmodel, P);
  const int nv = P.nv, nobs = (nv - P.obs_qpos_skip) + nv;
  Philox ph(seed);
  const float npos = m.reset_noise[0], nvel = m.reset_noise[1];
  for (int d = 0; d < nv; ++d) {
    uint32_t rnd[4];
    ph((uint32_t)env, (uint32_t)d, (uint32_t)counter, (uint32_t)(counter >> 32) ^ 0x5bd1e995u, rnd);
    const float q = m.qpos0[d] + npos * (2.f * u32_to_unit(rnd[0]) - 1.f);
    const float v = nvel * (2.f * u32_to_unit(rnd[1]) - 1.f);
    qpos_g[(size_t)env * nv + d] = q;
    qvel_g[(size_t)env * nv + d] = v;
    if (d >= P.obs_qpos_skip) {
      const int o = d - P.obs_qpos_skip;
      if (obs_f32) obs_f32[(size_t)env * nobs + o] = q;
      if (obs_bf16) obs_bf16[(size_t)env * obs_bf16_stride + o] = __float2bfloat16(q);
    }
    const int o = nv - P.obs_qpos_skip + d;
    if (obs_f32) obs_f32[(size_t)env * nobs + o] = v;
    if (obs_bf16) obs_bf16[(size_t)env * obs_bf16_stride + o] = __float2bfloat16(v);
  }
  const int nwarm = P.nlimit + 3 * P.ncs;
  for (int i = 0; i < nwarm; ++i) warm_g[(size_t)env * nwarm + i] = 0.f;
  step_count[env] = 0;
  ep_return[env] = 0.f;
}

// Body poses for rendering / sensors: xpos [N, nbody, 3], xmat [N, nbody, 9].
__global__ void __launch_bounds__(NB_PHYS_WARPS * 32)
phys_fk_kernel(PhysParams P, const int* __restrict__ imodel, const float* __restrict__ fmodel,
               const float* __restrict__ qpos_g, float* __restrict__ xpos_out, float* __restrict__ xmat_out,
               int n_envs) {
  extern __shared__ __align__(16) float smem[];
  int* im_sh = reinterpret_cast<int*>(smem);
  float* fm_sh = smem + P.imodel_words;
  for (int i = threadIdx.x; i < P.imodel_words; i += blockDim.x) im_sh[i] = imodel[i];
  for (int i = threadIdx.x; i < P.fmodel_words; i += blockDim.x) fm_sh[i] = fmodel[i];
  __syncthreads();
  const ModelView m = view(im_sh, fm_sh, P);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int env = blockIdx.x * (int)(blockDim.x >> 5) + warp;
  if (env >= n_envs) return;
  float* base = smem + P.imodel_words + P.fmodel_words + warp * P.warp_words;
  WarpScratch w = carve(base, P);
  w.vec[lane] = (lane < P.nv) ? qpos_g[(size_t)env * P.nv + lane] : 0.f;
  __syncwarp();
  forward_kinematics(P, m, w, w.vec, lane);
  for (int i = lane; i < P.nbody * 3; i += 32) xpos_out[(size_t)env * P.nbody * 3 + i] = w.xpos[i];
  for (int i = lane; i < P.nbody * 9; i += 32) xmat_out[(size_t)env * P.nbody * 9 + i] = w.xmat[i];
}

}  // namespace

extern "C" {

static int phys_smem_bytes(const PhysParams* P, int warps) {
  return (int)sizeof(float) * (P->imodel_words + P->fmodel_words + warps * P->warp_words);
}
// Warps (= environments) per block.  When four blocks of 7 warps fit one SM (small models: the packed constraint
// scratch of a 9-dof chain is 7 KB per environment) 28 environments are resident per SM and a 4096-environment batch
// is a single wave on 148 SMs; otherwise 8 warps per block, or fewer for models whose scratch needs it.
static bool phys_dense(const PhysParams* P) { return 4 * (phys_smem_bytes(P, 7) + 1024) <= 227 * 1024; }
static int phys_pick_warps(const PhysParams* P) {
  if (phys_dense(P)) return 7;
  for (int wpb = NB_PHYS_WARPS; wpb >= 1; --wpb)
    if (phys_smem_bytes(P, wpb) + 1024 <= 227 * 1024) return wpb;
  return 1;
}
int nb_phys_smem_bytes(const PhysParams* P) { return phys_smem_bytes(P, phys_pick_warps(P)); }
int nb_phys_warps_per_block(const PhysParams* P) { return phys_pick_warps(P); }

int nb_phys_env_step(const PhysParams* P, const int* imodel, const float* fmodel, float* qpos, float* qvel,
                     float* warm, int* step_count, float* ep_return, const float* action, int action_stride,
                     float* obs_f32, void* obs_bf16, int obs_bf16_stride, float* next_obs_f32, void* next_obs_bf16,
                     float* reward, float* done, float* terminated, float* finished_return,
                     const unsigned long long* rng_counter, unsigned long long seed, int n_envs, int do_reset,
                     float* ep_stats, float* dbg, void* stream) {
  if (P->nv > 32 || P->nbody > 32 || P->nv < 1) return NB_ERR_TOO_LARGE;
  const int smem = nb_phys_smem_bytes(P);
  if (smem > 227 * 1024) return NB_ERR_TOO_LARGE;
  const int wpb = phys_pick_warps(P);
  const int grid = nb::ceil_div(n_envs, wpb);
  if (phys_dense(P)) {
    static int configured = 0;
    if (configured < smem) {
      NB_CUDA(cudaFuncSetAttribute(phys_env_step_kernel<7, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
      NB_CUDA(cudaFuncSetAttribute(phys_env_step_kernel<7, 4>, cudaFuncAttributePreferredSharedMemoryCarveout, 100));
      configured = smem;
    }
    phys_env_step_kernel<7, 4><<<grid, wpb * 32, smem, (cudaStream_t)stream>>>(
        *P, imodel, fmodel, qpos, qvel, warm, step_count, ep_return, action, action_stride, obs_f32,
        (__nv_bfloat16*)obs_bf16, obs_bf16_stride, next_obs_f32, (__nv_bfloat16*)next_obs_bf16, reward, done,
        terminated, finished_return, rng_counter, seed, n_envs, do_reset, ep_stats, dbg);
    NB_LAUNCH_CHECK();
    return NB_OK;
  }
  static int configured = 0;
  if (configured < smem) {
    NB_CUDA(cudaFuncSetAttribute(phys_env_step_kernel<NB_PHYS_WARPS, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = smem;
  }
  phys_env_step_kernel<NB_PHYS_WARPS, 2><<<grid, wpb * 32, smem, (cudaStream_t)stream>>>(
      *P, imodel, fmodel, qpos, qvel, warm, step_count, ep_return, action, action_stride, obs_f32,
      (__nv_bfloat16*)obs_bf16, obs_bf16_stride, next_obs_f32, (__nv_bfloat16*)next_obs_bf16, reward, done,
      terminated, finished_return, rng_counter, seed, n_envs, do_reset, ep_stats, dbg);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_phys_env_reset(const PhysParams* P, const float* fmodel, float* qpos, float* qvel, float* warm,
                      int* step_count, float* ep_return, const float* mask, float* obs_f32, void* obs_bf16,
                      int obs_bf16_stride, unsigned long long seed, unsigned long long counter, int n_envs,
                      void* stream) {
  phys_env_reset_kernel<<<nb::ceil_div(n_envs, 128), 128, 0, (cudaStream_t)stream>>>(
      *P, fmodel, qpos, qvel, warm, step_count, ep_return, mask, obs_f32, (__nv_bfloat16*)obs_bf16,
      obs_bf16_stride, seed, counter, n_envs);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

int nb_phys_fk(const PhysParams* P, const int* imodel, const float* fmodel, const float* qpos, float* xpos,
               float* xmat, int n_envs, void* stream) {
  const int smem = nb_phys_smem_bytes(P);
  if (smem > 227 * 1024) return NB_ERR_TOO_LARGE;
  static int configured = 0;
  if (configured < smem) {
    NB_CUDA(cudaFuncSetAttribute(phys_fk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    configured = smem;
  }
  const int wpb = phys_pick_warps(P);
  phys_fk_kernel<<<nb::ceil_div(n_envs, wpb), wpb * 32, smem, (cudaStream_t)stream>>>(
      *P, imodel, fmodel, qpos, xpos, xmat, n_envs);
  NB_LAUNCH_CHECK();
  return NB_OK;
}

}  // extern "C"
