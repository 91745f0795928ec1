// Parameter block of the fused physics step (passed by value to the kernel, mirrored by a
// ctypes.Structure in noeira_b200/physics/engine.py — keep the field order identical).
#pragma once

#define NB_PHYS_WARPS 8
#define NB_JOINT_SLIDE 0
#define NB_JOINT_HINGE 1

struct PhysParams {
  // sizes
  int nbody, nv, nvp, nlimit, ncs, nu, maxdepth, rmax;
  int imodel_words, fmodel_words, warp_words, warm_words;
  int frame_skip, pgs_iters, friction_rows, max_steps;
  int forward_dof, term_dof, obs_qpos_skip, pad0;
  // dynamics
  float dt, gx, gy, gz;
  float solref_tc, solref_dr, solimp_d0, solimp_dmax, solimp_width, solimp_mid, solimp_pow, margin;
  float plane_nx, plane_ny, plane_nz, plane_off;
  float friction_reg, max_vel, obs_clip, pad1;
  // task
  float w_forward, w_ctrl, w_alive, term_lo, term_hi, pad2, pad3, pad4;
};
