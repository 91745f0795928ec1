"""General batched rigid-body dynamics as a tensor program: every joint type, geom pairs, three integrators, two solvers.

The fused CUDA step (``csrc/physics_step.cu``) covers hinge / slide trees with sphere-vs-plane contacts at full speed; this
module is the general engine beside it.  State and algorithms follow the generalized-coordinate formulation of the
reference's 3-D engine (noeira/physics3d/: model / data, kinematics, CRBA + RNE, collision, constraint solvers,
integrators, sensors), batched over environments as plain tensor operations (any device, float64 by default):

  joints        free (7 position numbers, 6 velocities: world-frame linear + body-frame angular), ball (quaternion, body-frame
                angular velocity), hinge, slide; several joints per body; armature, damping, springs, limits on 1-dof joints
  kinematics    body frames, per-dof world motion axes and anchors, body / point Jacobians, frame velocities
  dynamics      mass matrix M = Σ m JvᵀJv + Jwᵀ I Jw (+ armature), bias force from the time derivative of the Jacobians
                (Coriolis / centrifugal / gyroscopic) and gravity, passive forces, motors
  collision     plane vs sphere / capsule / box, sphere–sphere, sphere–capsule, capsule–capsule (closest points of segments),
                sphere–box (closest point of the box), box–box (corner-in-box contacts both ways)
  constraints   soft constraints with reference acceleration −b·v − k·r and impedance-regularised diagonal; contact normal +
                two friction rows (box friction |f_t| ≤ μ f_n), joint limits; solvers: projected Gauss-Seidel, projected conjugate
                gradients, and an active-set Newton method on the dual (batched linear solves on the free set)
  integrators   semi-implicit Euler, Euler with implicit joint damping, 4th-order Runge-Kutta on the manifold
  sensors       joint position / velocity, frame position / orientation / linear / angular velocity, accelerometer, gyro,
                touch (contact normal force per body), actuator force, subtree centre of mass, energies
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .model import Body, Geom, Joint, Options, capsule_mass_inertia, sphere_mass_inertia

SLIDE, HINGE, FREE, BALL = 0, 1, 2, 3


# ------------------------------------------------------------------------------------------ small algebra (batched)
def quat_mul(a, b):
    aw, ax, ay, az = a.unbind(-1)
    bw, bx, by, bz = b.unbind(-1)
    return torch.stack([aw * bw - ax * bx - ay * by - az * bz, aw * bx + ax * bw + ay * bz - az * by,
                        aw * by - ax * bz + ay * bw + az * bx, aw * bz + ax * by - ay * bx + az * bw], -1)


def quat_to_mat(q):
    w, x, y, z = q.unbind(-1)
    return torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y),
                        2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x),
                        2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)], -1).reshape(*q.shape[:-1], 3, 3)


def quat_integrate(q, w_local, dt):
    """q ⊗ exp(½ ω dt) for a body-frame angular velocity."""
    ang = w_local.norm(dim=-1, keepdim=True) * dt
    axis = w_local / w_local.norm(dim=-1, keepdim=True).clamp(min=1e-30)
    dq = torch.cat([torch.cos(0.5 * ang), torch.sin(0.5 * ang) * axis], -1)
    out = quat_mul(q, dq)
    return out / out.norm(dim=-1, keepdim=True)


def axis_angle_mat(axis, angle):
    """Rodrigues rotation for a constant unit ``axis [3]`` and batched ``angle [B]``."""
    K = torch.zeros(3, 3, dtype=angle.dtype, device=angle.device)
    K[0, 1], K[0, 2], K[1, 0], K[1, 2], K[2, 0], K[2, 1] = -axis[2], axis[1], axis[2], -axis[0], -axis[1], axis[0]
    s, c = torch.sin(angle)[:, None, None], torch.cos(angle)[:, None, None]
    return torch.eye(3, dtype=angle.dtype, device=angle.device) + s * K + (1 - c) * (K @ K)


def box_mass_inertia(half, density):
    x, y, z = (2 * h for h in half)
    m = density * x * y * z
    return m, [m * (y * y + z * z) / 12, m * (x * x + z * z) / 12, m * (x * x + y * y) / 12]


# ------------------------------------------------------------------------------------------ model
@dataclass
class Motor:
    joint: str
    gear: float = 1.0
    ctrlrange: Tuple[float, float] = (-1.0, 1.0)


@dataclass
class Tendon:
    """Fixed tendon: length L = Σ coef_j · q_j over 1-dof joints, with a spring (``stiffness`` about ``springlength``), a
    damper and an optional length range enforced as a constraint."""
    coefs: Dict[str, float]
    stiffness: float = 0.0
    springlength: float = 0.0
    damping: float = 0.0
    range: Optional[Tuple[float, float]] = None


@dataclass
class _Dof:
    body: int
    jtype: int
    k: int                  # index inside a free (0..5) / ball (0..2) joint, 0 otherwise
    qadr: int
    joint: int


class GeneralModel:
    """Flattened description of a tree of bodies.  ``bodies[i].parent`` is an index into the list or −1 (world); a free joint
    is only allowed on a child of the world.  Inertia: ``Body.mass / inertia / ipos`` (principal axes = body axes) or summed
    from the geoms (each about its own centre, axis-aligned approximation for rotated capsules)."""

    def __init__(self, bodies: Sequence[Body], motors: Sequence[Motor] = (), opt: Options = None, dtype=torch.float64,
                 device="cpu", collide_pairs: Optional[Sequence[Tuple[int, int]]] = None, plane: bool = True,
                 tendons: Sequence[Tendon] = (), hfield=None, broadphase: bool = False):
        self.opt = opt or Options()
        self.hfield, self.broadphase = hfield, broadphase            # a narrowphase.HeightField fixed in the world; SAP pruning
        self.dtype, self.device = dtype, torch.device(device)
        t = lambda x: torch.as_tensor(x, dtype=dtype, device=self.device)
        self.nb = len(bodies)
        self.parent = [b.parent for b in bodies]
        self.pos = [t(b.pos) for b in bodies]
        self.quat = [t(b.quat) for b in bodies]
        self.names = [b.name for b in bodies]
        self.joints: List[Tuple[int, Joint]] = []
        self.dofs: List[_Dof] = []
        self.body_joints: List[List[int]] = []
        nq = 0
        q0 = []
        for bi, b in enumerate(bodies):
            ids = []
            for j in b.joints:
                ji = len(self.joints)
                self.joints.append((bi, j))
                ids.append(ji)
                if j.type == FREE:
                    assert b.parent < 0, "a free joint connects to the world"
                    self.dofs += [_Dof(bi, FREE, k, nq, ji) for k in range(6)]
                    q0 += [*b.pos, *b.quat]
                    nq += 7
                elif j.type == BALL:
                    self.dofs += [_Dof(bi, BALL, k, nq, ji) for k in range(3)]
                    q0 += [1.0, 0.0, 0.0, 0.0]
                    nq += 4
                else:
                    self.dofs.append(_Dof(bi, j.type, 0, nq, ji))
                    q0.append(j.qpos0)
                    nq += 1
            self.body_joints.append(ids)
        self.nq, self.nv = nq, len(self.dofs)
        self.qpos0 = t(q0)
        self.joint_qadr, self.joint_dadr = {}, {}
        for d, dof in enumerate(self.dofs):
            self.joint_dadr.setdefault(dof.joint, d)
            self.joint_qadr.setdefault(dof.joint, dof.qadr)
        self.joint_by_name = {j.name: i for i, (_, j) in enumerate(self.joints) if j.name}
        # inertial properties
        mass, inertia, ipos = [], [], []
        for b in bodies:
            if b.mass is not None:
                mass.append(float(b.mass)), inertia.append(list(b.inertia)), ipos.append(list(b.ipos or (0, 0, 0)))
                continue
            m_tot, first, parts = 0.0, [0.0, 0.0, 0.0], []
            for g in b.geoms:
                if g.type == "sphere":
                    m, I = sphere_mass_inertia(g.size[0], g.density)
                elif g.type == "capsule":
                    m, I = capsule_mass_inertia(g.size[0], g.size[1], g.density)
                    R = quat_to_mat(t(g.quat))
                    I = torch.diagonal(R @ torch.diag(t(I)) @ R.T).tolist()
                elif g.type == "mesh":
                    from .narrowphase import mesh_mass_inertia
                    m, I, c = mesh_mass_inertia(g.vertices, g.density)            # in the geom's axes (taken as the body's)
                    parts.append((m, list(I), [a + b for a, b in zip(g.pos, c)]))
                    m_tot += m
                    first = [f + m * (a + b) for f, a, b in zip(first, g.pos, c)]
                    continue
                else:
                    m, I = box_mass_inertia(g.size, g.density)
                parts.append((m, list(I), list(g.pos)))
                m_tot += m
                first = [f + m * p for f, p in zip(first, g.pos)]
            com = [f / max(m_tot, 1e-30) for f in first]
            I_tot = [0.0, 0.0, 0.0]
            for m, I, p in parts:
                d = [p[i] - com[i] for i in range(3)]
                I_tot = [I_tot[0] + I[0] + m * (d[1] ** 2 + d[2] ** 2), I_tot[1] + I[1] + m * (d[0] ** 2 + d[2] ** 2),
                         I_tot[2] + I[2] + m * (d[0] ** 2 + d[1] ** 2)]
            mass.append(m_tot), inertia.append(I_tot), ipos.append(com)
        self.mass, self.inertia, self.ipos = t(mass), t(inertia), t(ipos)
        # ancestry: anc[b, d] = dof d moves body b
        anc = torch.zeros(self.nb, self.nv, dtype=torch.bool)
        for b in range(self.nb):
            a = b
            while a >= 0:
                for d, dof in enumerate(self.dofs):
                    if dof.body == a:
                        anc[b, d] = True
                a = self.parent[a]
        self.anc = anc.to(self.device)
        self.is_rot = torch.tensor([(d.jtype == HINGE) or (d.jtype == BALL) or (d.jtype == FREE and d.k >= 3) for d in self.dofs],
                                   device=self.device)
        one = lambda f: t([f(self.joints[d.joint][1]) if d.jtype in (HINGE, SLIDE) else 0.0 for d in self.dofs])
        self.armature, self.damping = one(lambda j: j.armature), one(lambda j: j.damping)
        self.stiffness, self.springref = one(lambda j: j.stiffness), one(lambda j: j.springref)
        self.limits = [(d, self.joints[dof.joint][1].range) for d, dof in enumerate(self.dofs)
                       if dof.jtype in (HINGE, SLIDE) and self.joints[dof.joint][1].range is not None]
        self.motors = list(motors)
        self.motor_dof = [self.joint_dadr[self.joint_by_name[m.joint]] for m in self.motors]
        self.gravity = t(self.opt.gravity)
        # fixed tendons: one coefficient row over the dofs each
        self.tendons = list(tendons)
        self.tendon_coef = torch.zeros(len(self.tendons), self.nv, dtype=dtype, device=self.device)
        for ti, td in enumerate(self.tendons):
            for jn, cf in td.coefs.items():
                d = self.joint_dadr[self.joint_by_name[jn]]
                assert self.dofs[d].jtype in (HINGE, SLIDE), "fixed tendons run over hinge / slide joints"
                self.tendon_coef[ti, d] = cf
        self.tendon_k = t([td.stiffness for td in self.tendons])
        self.tendon_l0 = t([td.springlength for td in self.tendons])
        self.tendon_d = t([td.damping for td in self.tendons])
        # collision geoms and pairs
        self.geoms = [(bi, g) for bi, b in enumerate(bodies) for g in b.geoms if g.contact]
        self.plane = plane
        if collide_pairs is None:
            collide_pairs = [(i, j) for i in range(len(self.geoms)) for j in range(i + 1, len(self.geoms))
                             if self.geoms[i][0] != self.geoms[j][0] and self.parent[self.geoms[i][0]] != self.geoms[j][0]
                             and self.parent[self.geoms[j][0]] != self.geoms[i][0]]
        self.pairs = list(collide_pairs)

    def t(self, x):
        return torch.as_tensor(x, dtype=self.dtype, device=self.device)

    def init_state(self, n: int):
        return self.qpos0.expand(n, -1).clone(), torch.zeros(n, self.nv, dtype=self.dtype, device=self.device)


# ------------------------------------------------------------------------------------------ kinematics
@dataclass
class Kin:
    xpos: torch.Tensor       # [B, nb, 3] body frame origins
    xmat: torch.Tensor       # [B, nb, 3, 3]
    com: torch.Tensor        # [B, nb, 3]
    axis: torch.Tensor       # [B, nv, 3] world motion axis per dof
    anchor: torch.Tensor     # [B, nv, 3]
    w_body: torch.Tensor     # [B, nb, 3] angular velocity
    v_com: torch.Tensor      # [B, nb, 3]
    w_frame: torch.Tensor    # [B, nv, 3] angular velocity of the frame the dof axis is fixed in
    v_anchor: torch.Tensor   # [B, nv, 3]


def kinematics(m: GeneralModel, qpos, qvel) -> Kin:
    B, dt_ = qpos.shape[0], qpos.dtype
    z3 = lambda: torch.zeros(B, 3, dtype=dt_, device=qpos.device)
    eye = torch.eye(3, dtype=dt_, device=qpos.device)
    xpos, xmat, wb, vo = [None] * m.nb, [None] * m.nb, [None] * m.nb, [None] * m.nb
    axis, anchor = [None] * m.nv, [None] * m.nv
    w_frame, v_anchor = [None] * m.nv, [None] * m.nv
    for b in range(m.nb):
        p = m.parent[b]
        if p < 0:
            pR, pp, w, v = eye.expand(B, 3, 3), z3(), z3(), z3()
        else:
            pR, pp, w, v = xmat[p], xpos[p], wb[p], vo[p]
        pos = pp + (pR @ m.pos[b])
        v = v + torch.linalg.cross(w, pos - pp)                       # velocity of the new origin, still rigid with the parent
        R = pR @ quat_to_mat(m.quat[b])
        for ji in m.body_joints[b]:
            j = m.joints[ji][1]
            d0, qa = m.joint_dadr[ji], m.joint_qadr[ji]
            if j.type == FREE:
                pos, R = qpos[:, qa:qa + 3], quat_to_mat(qpos[:, qa + 3:qa + 7])
                v = qvel[:, d0:d0 + 3]
                w = (R @ qvel[:, d0 + 3:d0 + 6, None])[..., 0]
                for k in range(3):
                    axis[d0 + k], anchor[d0 + k] = eye[k].expand(B, 3), pos
                    w_frame[d0 + k], v_anchor[d0 + k] = z3(), v
                    axis[d0 + 3 + k], anchor[d0 + 3 + k] = R[:, :, k], pos
                    w_frame[d0 + 3 + k], v_anchor[d0 + 3 + k] = w, v
            elif j.type == BALL:
                jp = m.t(j.pos)
                anc = pos + R @ jp
                va = v + torch.linalg.cross(w, anc - pos)
                R = R @ quat_to_mat(qpos[:, qa:qa + 4])
                w = w + (R @ qvel[:, d0:d0 + 3, None])[..., 0]
                pos = anc - R @ jp
                v = va + torch.linalg.cross(w, pos - anc)
                for k in range(3):
                    axis[d0 + k], anchor[d0 + k], w_frame[d0 + k], v_anchor[d0 + k] = R[:, :, k], anc, w, va
            elif j.type == HINGE:
                ax_l, jp = m.t(j.axis) / m.t(j.axis).norm(), m.t(j.pos)
                aw = R @ ax_l
                anc = pos + R @ jp
                va = v + torch.linalg.cross(w, anc - pos)
                axis[d0], anchor[d0], w_frame[d0], v_anchor[d0] = aw, anc, w, va
                R = R @ axis_angle_mat(ax_l, qpos[:, qa] - j.qpos0)
                w = w + aw * qvel[:, d0:d0 + 1]
                pos = anc - R @ jp
                v = va + torch.linalg.cross(w, pos - anc)
            else:
                aw = R @ (m.t(j.axis) / m.t(j.axis).norm())
                s = (qpos[:, qa] - j.qpos0)[:, None]
                axis[d0], anchor[d0], w_frame[d0], v_anchor[d0] = aw, pos, w, v
                v = v + torch.linalg.cross(w, aw * s) + aw * qvel[:, d0:d0 + 1]
                pos = pos + aw * s
        xpos[b], xmat[b], wb[b], vo[b] = pos, R, w, v
    xpos, xmat, wb, vo = torch.stack(xpos, 1), torch.stack(xmat, 1), torch.stack(wb, 1), torch.stack(vo, 1)
    com = xpos + (xmat @ m.ipos[None, :, :, None])[..., 0]
    st = lambda xs: torch.stack(xs, 1) if xs else torch.zeros(B, 0, 3, dtype=dt_, device=qpos.device)
    return Kin(xpos, xmat, com, st(axis), st(anchor), wb, vo + torch.linalg.cross(wb, com - xpos), st(w_frame), st(v_anchor))


def point_jacobian(m: GeneralModel, k: Kin, body: int, point):
    """Linear-velocity Jacobian ``[B, 3, nv]`` of a world ``point [B, 3]`` moving with ``body``."""
    r = point[:, None] - k.anchor
    col = torch.where(m.is_rot[None, :, None], torch.linalg.cross(k.axis, r), k.axis)
    return (col * m.anc[body][None, :, None]).transpose(1, 2)


def body_jacobians(m: GeneralModel, k: Kin):
    """(Jv ``[B, nb, 3, nv]`` of the centres of mass, Jw ``[B, nb, 3, nv]``)."""
    r = k.com[:, :, None] - k.anchor[:, None]                                    # [B, nb, nv, 3]
    rot = m.is_rot[None, None, :, None]
    ax = k.axis[:, None].expand_as(r)
    mask = m.anc[None, :, :, None]
    Jv = torch.where(rot, torch.linalg.cross(ax, r), ax) * mask
    Jw = torch.where(rot, ax, torch.zeros_like(ax)) * mask
    return Jv.transpose(2, 3), Jw.transpose(2, 3)


def world_inertia(m: GeneralModel, k: Kin):
    return k.xmat @ torch.diag_embed(m.inertia)[None] @ k.xmat.transpose(-1, -2)


def mass_matrix(m: GeneralModel, k: Kin, Jv=None, Jw=None):
    if Jv is None:
        Jv, Jw = body_jacobians(m, k)
    M = (m.mass[None, :, None, None] * (Jv.transpose(-1, -2) @ Jv)).sum(1) + (Jw.transpose(-1, -2) @ world_inertia(m, k) @ Jw).sum(1)
    return M + torch.diag_embed(m.armature)[None]


def bias_force(m: GeneralModel, k: Kin, qvel, Jv=None, Jw=None):
    """c(q, v) with M q̈ + c = τ: Coriolis / centrifugal / gyroscopic terms from the time derivative of the Jacobians, and gravity."""
    if Jv is None:
        Jv, Jw = body_jacobians(m, k)
    daxis = torch.linalg.cross(k.w_frame, k.axis)                                                    # [B, nv, 3]
    r = k.com[:, :, None] - k.anchor[:, None]                                                         # [B, nb, nv, 3]
    dr = k.v_com[:, :, None] - k.v_anchor[:, None]
    rot = m.is_rot[None, None, :, None]
    da = daxis[:, None].expand_as(r)
    ax = k.axis[:, None].expand_as(r)
    dcol_v = torch.where(rot, torch.linalg.cross(da, r) + torch.linalg.cross(ax, dr), da)
    dcol_w = torch.where(rot, da, torch.zeros_like(da))
    wgt = (m.anc[None].to(qvel.dtype) * qvel[:, None])[..., None]                                     # [B, nb, nv, 1]
    a_bias, al_bias = (dcol_v * wgt).sum(2), (dcol_w * wgt).sum(2)                                     # [B, nb, 3]
    Iw = world_inertia(m, k)
    f = m.mass[None, :, None] * (a_bias - m.gravity)
    tau = (Iw @ al_bias[..., None])[..., 0] + torch.linalg.cross(k.w_body, (Iw @ k.w_body[..., None])[..., 0])
    return (Jv.transpose(-1, -2) @ f[..., None]).sum(1)[..., 0] + (Jw.transpose(-1, -2) @ tau[..., None]).sum(1)[..., 0]


def point_bias_acceleration(m: GeneralModel, k: Kin, qvel, body: int, point, vpoint):
    """J̇ v of a point moving with ``body`` (``vpoint`` = its velocity): the acceleration it has at q̈ = 0."""
    daxis = torch.linalg.cross(k.w_frame, k.axis)
    r, dr = point[:, None] - k.anchor, vpoint[:, None] - k.v_anchor
    dcol = torch.where(m.is_rot[None, :, None], torch.linalg.cross(daxis, r) + torch.linalg.cross(k.axis, dr), daxis)
    return (dcol * (m.anc[body][None].to(qvel.dtype) * qvel)[..., None]).sum(1)


def _scalar_q(m: GeneralModel, qpos):
    """Joint coordinate per dof for the 1-dof joints (zero elsewhere)."""
    out = torch.zeros(qpos.shape[0], m.nv, dtype=qpos.dtype, device=qpos.device)
    for d, dof in enumerate(m.dofs):
        if dof.jtype in (HINGE, SLIDE):
            out[:, d] = qpos[:, dof.qadr]
    return out


def tendon_length(m: GeneralModel, qpos):
    return _scalar_q(m, qpos) @ m.tendon_coef.T                                   # [B, nt]


def passive_force(m: GeneralModel, qpos, qvel, with_damping=True):
    f = -m.stiffness * (_scalar_q(m, qpos) - m.springref)
    if m.tendons:
        ft = -m.tendon_k * (tendon_length(m, qpos) - m.tendon_l0)
        if with_damping:
            ft = ft - m.tendon_d * (qvel @ m.tendon_coef.T)
        f = f + ft @ m.tendon_coef
    return f - m.damping * qvel if with_damping else f


def integrate_pos(m: GeneralModel, qpos, qvel, dt):
    q = qpos.clone()
    done = set()
    for d, dof in enumerate(m.dofs):
        if dof.jtype in (HINGE, SLIDE):
            q[:, dof.qadr] = qpos[:, dof.qadr] + dt * qvel[:, d]
        elif dof.joint not in done:
            done.add(dof.joint)
            if dof.jtype == FREE:
                q[:, dof.qadr:dof.qadr + 3] = qpos[:, dof.qadr:dof.qadr + 3] + dt * qvel[:, d:d + 3]
                q[:, dof.qadr + 3:dof.qadr + 7] = quat_integrate(qpos[:, dof.qadr + 3:dof.qadr + 7], qvel[:, d + 3:d + 6], dt)
            else:
                q[:, dof.qadr:dof.qadr + 4] = quat_integrate(qpos[:, dof.qadr:dof.qadr + 4], qvel[:, d:d + 3], dt)
    return q


def energy(m: GeneralModel, qpos, qvel):
    k = kinematics(m, qpos, qvel)
    M = mass_matrix(m, k)
    T = 0.5 * (qvel[:, None] @ M @ qvel[:, :, None])[:, 0, 0]
    U = -(m.mass[None, :, None] * k.com * m.gravity).sum((1, 2)) + 0.5 * (m.stiffness * (_scalar_q(m, qpos) - m.springref) ** 2).sum(1)
    if m.tendons:
        U = U + 0.5 * (m.tendon_k * (tendon_length(m, qpos) - m.tendon_l0) ** 2).sum(1)
    return T, U


# ------------------------------------------------------------------------------------------ collision
def closest_segment_points(p1, d1, p2, d2):
    """Closest points of the segments p1 + s·d1 and p2 + t·d2 (s, t ∈ [0, 1]), batched ``[B, 3]``."""
    r = p1 - p2
    a, e, f = (d1 * d1).sum(-1), (d2 * d2).sum(-1), (d2 * r).sum(-1)
    b, c = (d1 * d2).sum(-1), (d1 * r).sum(-1)
    den = a * e - b * b
    s = torch.where(den > 1e-12, ((b * f - c * e) / den.clamp(min=1e-12)).clamp(0, 1), torch.zeros_like(den))
    t = ((b * s + f) / e.clamp(min=1e-12))
    s = torch.where(t < 0, (-c / a.clamp(min=1e-12)).clamp(0, 1), torch.where(t > 1, ((b - c) / a.clamp(min=1e-12)).clamp(0, 1), s))
    t = t.clamp(0, 1)
    return p1 + s[:, None] * d1, p2 + t[:, None] * d2


@dataclass
class Contacts:
    point: torch.Tensor      # [B, nc, 3]
    normal: torch.Tensor     # [B, nc, 3] from the first body (or the world) towards the second
    depth: torch.Tensor      # [B, nc] penetration (positive = overlapping)
    body1: List[int]         # −1 = world
    body2: List[int]
    mu: torch.Tensor         # [nc]


def _geom_frame(m, k, gi):
    b, g = m.geoms[gi]
    c = k.xpos[:, b] + (k.xmat[:, b] @ m.t(g.pos))
    R = k.xmat[:, b] @ quat_to_mat(m.t(g.quat))
    return b, g, c, R


def _spheres_of(m, k, gi):
    """A sphere or the axis segment of a capsule as (start, direction, radius)."""
    b, g, c, R = _geom_frame(m, k, gi)
    if g.type == "sphere":
        return b, c, torch.zeros_like(c), g.size[0]
    ax = R[:, :, 2] * g.size[1]
    return b, c - ax, 2 * ax, g.size[0]


def collide(m: GeneralModel, k: Kin) -> Contacts:
    pts, nrm, dep, b1, b2, mu = [], [], [], [], [], []
    n_pl = m.t(m.opt.plane_normal)

    def add(p, n, d, a, b, fr):
        pts.append(p), nrm.append(n), dep.append(d), b1.append(a), b2.append(b), mu.append(fr)

    if m.plane:
        for gi in range(len(m.geoms)):
            b, g, c, R = _geom_frame(m, k, gi)
            if g.type == "mesh":
                for vtx in g.vertices:
                    p = c + R @ m.t(vtx)
                    d = g.size[0] + m.opt.plane_offset - (p * n_pl).sum(-1)
                    add(p - n_pl * (g.size[0] - 0.5 * d)[:, None], n_pl.expand_as(p), d, -1, b, g.friction)
                continue
            if g.type == "box":
                h = m.t(g.size)
                for sx in (-1, 1):
                    for sy in (-1, 1):
                        for sz in (-1, 1):
                            p = c + R @ (h * m.t([sx, sy, sz]))
                            d = m.opt.plane_offset - (p * n_pl).sum(-1)
                            add(p + n_pl * (0.5 * d)[:, None], n_pl.expand_as(p), d, -1, b, g.friction)
                continue
            ends = [c] if g.type == "sphere" else [c - R[:, :, 2] * g.size[1], c + R[:, :, 2] * g.size[1]]
            for e in ends:
                d = g.size[0] - ((e * n_pl).sum(-1) - m.opt.plane_offset)
                add(e - n_pl * (g.size[0] - 0.5 * d)[:, None], n_pl.expand_as(e), d, -1, b, g.friction)
    if m.hfield is not None:
        for gi in range(len(m.geoms)):
            b, g, c, R = _geom_frame(m, k, gi)
            fr = math.sqrt(g.friction * m.hfield.friction)
            for centre, radius in _support_points(m, g, c, R):
                p, n, d = m.hfield.contact(centre, radius)
                add(p, n, d, -1, b, fr)
    pairs = m.pairs
    if m.broadphase and len(m.geoms) >= 2:
        from .narrowphase import sap_overlaps
        lo, hi = _geom_aabbs(m, k)
        keep = sap_overlaps(lo, hi, pairs)
        pairs = [pr for pr, kp in zip(pairs, keep) if kp]
    for gi, gj in pairs:
        ta, tb = m.geoms[gi][1].type, m.geoms[gj][1].type
        fr = math.sqrt(m.geoms[gi][1].friction * m.geoms[gj][1].friction)
        if ta == "mesh" or tb == "mesh":
            for p, n, d in _convex_pair(m, k, gi, gj):
                add(p, n, d, m.geoms[gi][0], m.geoms[gj][0], fr)
            continue
        if ta == "box" or tb == "box":
            if ta == "box" and tb == "box":
                # vertex-face contacts both ways (8 + 8 slots): a corner of one box inside the other is pushed out through
                # the nearest face of the box that contains it; one more slot holds the edge-edge contact of the separating-axis
                # test (active only when an edge-cross axis is the axis of least overlap)
                for g_in, g_box in ((gi, gj), (gj, gi)):
                    b_in, gin, c_in, R_in = _geom_frame(m, k, g_in)
                    b_bx, gbx, c_bx, R_bx = _geom_frame(m, k, g_box)
                    h_in, h_bx = m.t(gin.size), m.t(gbx.size)
                    for sx in (-1, 1):
                        for sy in (-1, 1):
                            for sz in (-1, 1):
                                p = c_in + R_in @ (h_in * m.t([sx, sy, sz]))
                                n, d = _point_in_box(p, c_bx, R_bx, h_bx)
                                add(p + n * (0.5 * d)[:, None], n, d, b_bx, b_in, fr)
                p, n, d = _box_box_edge_contact(*_geom_frame(m, k, gi)[2:], m.t(m.geoms[gi][1].size),
                                                *_geom_frame(m, k, gj)[2:], m.t(m.geoms[gj][1].size))
                add(p, n, d, m.geoms[gi][0], m.geoms[gj][0], fr)
            else:
                g_s, g_b = (gi, gj) if tb == "box" else (gj, gi)
                b_s, gs, c_s, R_s = _geom_frame(m, k, g_s)
                b_b, gb, c_b, R_b = _geom_frame(m, k, g_b)
                h = m.t(gb.size)
                if gs.type == "sphere":
                    centres = [c_s]
                else:
                    # capsule: the point of its axis nearest to the box (alternating projections between the segment and
                    # the box, both convex) and the two ends, each as a sphere against the box
                    ax = R_s[:, :, 2] * gs.size[1]
                    centres = [_segment_point_nearest_box(c_s - ax, 2 * ax, c_b, R_b, h), c_s - ax, c_s + ax]
                for cc in centres:
                    p, n, d = _sphere_box(cc, gs.size[0], c_b, R_b, h)
                    add(p, n, d, b_b, b_s, fr)
            continue
        ba, pa, da, ra = _spheres_of(m, k, gi)
        bb, pb, db, rb = _spheres_of(m, k, gj)
        ca, cb = closest_segment_points(pa, da, pb, db)
        diff = cb - ca
        dist = diff.norm(dim=-1)
        n = diff / dist.clamp(min=1e-12)[:, None]
        d = ra + rb - dist
        add(ca + n * (ra - 0.5 * d)[:, None], n, d, ba, bb, math.sqrt(m.geoms[gi][1].friction * m.geoms[gj][1].friction))
    if not pts:
        B = k.xpos.shape[0]
        z = torch.zeros(B, 0, 3, dtype=k.xpos.dtype, device=k.xpos.device)
        return Contacts(z, z, z[..., 0], [], [], m.t([]))
    return Contacts(torch.stack(pts, 1), torch.stack(nrm, 1), torch.stack(dep, 1), b1, b2, m.t(mu))


def _support_points(m, g, c, R):
    """The shape as spheres for point-wise tests (terrain): (centres [B, 3], radius) per sphere, capsule end, box corner or
    mesh vertex."""
    if g.type == "sphere":
        return [(c, g.size[0])]
    if g.type == "capsule":
        ax = R[:, :, 2] * g.size[1]
        return [(c - ax, g.size[0]), (c + ax, g.size[0])]
    if g.type == "box":
        h = m.t(g.size)
        return [(c + R @ (h * m.t([sx, sy, sz])), 0.0) for sx in (-1, 1) for sy in (-1, 1) for sz in (-1, 1)]
    return [(c + R @ m.t(v), g.size[0]) for v in g.vertices]


def _core(m, g, c, R):
    """(vertices [B, n, 3] of the convex core, inflation radius) of a geom for the GJK / EPA pair test."""
    pts = _support_points(m, g, c, R)
    return torch.stack([p for p, _ in pts], 1), float(pts[0][1])


def _geom_aabbs(m, k):
    lo, hi = [], []
    for gi in range(len(m.geoms)):
        _, g, c, R = _geom_frame(m, k, gi)
        v, r = _core(m, g, c, R)
        lo.append(v.amin(1) - r - m.opt.margin), hi.append(v.amax(1) + r + m.opt.margin)
    return torch.stack(lo, 1), torch.stack(hi, 1)


_MANIFOLD_SLOTS = 5


def _convex_pair(m, k, gi, gj):
    """Contacts of a pair that involves a convex mesh: GJK / EPA on the host, lane by lane, into a fixed number of slots
    (unused slots carry depth −1)."""
    from .narrowphase import contact_manifold
    _, ga, ca, Ra = _geom_frame(m, k, gi)
    _, gb, cb, Rb = _geom_frame(m, k, gj)
    va, ra = _core(m, ga, ca, Ra)
    vb, rb = _core(m, gb, cb, Rb)
    B = va.shape[0]
    P = torch.zeros(B, _MANIFOLD_SLOTS, 3, dtype=va.dtype)
    Nn = torch.zeros(B, _MANIFOLD_SLOTS, 3, dtype=va.dtype)
    Nn[:, :, 2] = 1.0
    D = -torch.ones(B, _MANIFOLD_SLOTS, dtype=va.dtype)
    va_n, vb_n, cb_n = va.detach().cpu().numpy(), vb.detach().cpu().numpy(), cb.detach().cpu().numpy()
    for e in range(B):
        for s_, (p, n, d) in enumerate(contact_manifold(va_n[e], vb_n[e], ra, rb, cb_n[e], margin=m.opt.margin)[:_MANIFOLD_SLOTS]):
            P[e, s_], Nn[e, s_], D[e, s_] = torch.as_tensor(p), torch.as_tensor(n), float(d)
    dev = va.device
    return [(P[:, s_].to(dev), Nn[:, s_].to(dev), D[:, s_].to(dev)) for s_ in range(_MANIFOLD_SLOTS)]


def _sphere_box(c_s, radius, c_b, R_b, h):
    """Contact (point, normal from the box to the sphere, depth) of a sphere against a box."""
    loc = (R_b.transpose(1, 2) @ (c_s - c_b)[:, :, None])[..., 0]
    near = c_b + (R_b @ torch.maximum(torch.minimum(loc, h), -h)[:, :, None])[..., 0]      # closest point of the box
    diff = c_s - near
    dist = diff.norm(dim=-1)
    inside = dist < 1e-9
    n_in, d_in = _point_in_box(c_s, c_b, R_b, h)                                       # centre inside the box
    n = torch.where(inside[:, None], n_in, diff / dist.clamp(min=1e-12)[:, None])
    d = torch.where(inside, d_in + radius, radius - dist)
    return c_s - n * (radius - 0.5 * d)[:, None], n, d


def _segment_point_nearest_box(p0, dvec, c_b, R_b, h, iters: int = 12):
    """The point of the segment p0 + t·dvec (t ∈ [0, 1]) nearest to a box, by alternating projections."""
    l2 = (dvec * dvec).sum(-1).clamp(min=1e-18)
    t = torch.full_like(l2, 0.5)
    for _ in range(iters):
        q = p0 + t[:, None] * dvec
        loc = (R_b.transpose(1, 2) @ (q - c_b)[:, :, None])[..., 0]
        on_box = c_b + (R_b @ torch.maximum(torch.minimum(loc, h), -h)[:, :, None])[..., 0]
        t = (((on_box - p0) * dvec).sum(-1) / l2).clamp(0, 1)
    return p0 + t[:, None] * dvec


def _box_box_edge_contact(c_a, R_a, h_a, c_b, R_b, h_b):
    """Separating-axis test of two boxes over the 6 face axes and the 9 edge-cross axes.  Returns one contact (point,
    normal from A to B, depth) that is active (depth > 0) only where the boxes overlap AND the axis of least overlap is an
    edge-cross axis: the closest points of the two supporting edges.  Face-axis cases are left to the vertex-face contacts."""
    B = c_a.shape[0]
    t = c_b - c_a
    best_d = torch.full((B,), float("inf"), dtype=c_a.dtype, device=c_a.device)
    face_d = best_d.clone()
    best_n = torch.zeros(B, 3, dtype=c_a.dtype, device=c_a.device)
    best_ij = torch.zeros(B, 2, dtype=torch.long, device=c_a.device)
    separated = torch.zeros(B, dtype=torch.bool, device=c_a.device)

    def overlap(axis):
        ra = ((R_a.transpose(1, 2) @ axis[:, :, None])[..., 0].abs() * h_a).sum(-1)
        rb = ((R_b.transpose(1, 2) @ axis[:, :, None])[..., 0].abs() * h_b).sum(-1)
        return ra + rb - (t * axis).sum(-1).abs()
    for R in (R_a, R_b):
        for i in range(3):
            ov = overlap(R[:, :, i])
            separated |= ov <= 0
            face_d = torch.minimum(face_d, ov)
    for i in range(3):
        for j in range(3):
            cr = torch.linalg.cross(R_a[:, :, i], R_b[:, :, j])
            ln = cr.norm(dim=-1)
            ok = ln > 1e-6                                       # parallel edges: the face axes cover it
            axis = cr / ln.clamp(min=1e-12)[:, None]
            ov = torch.where(ok, overlap(axis), torch.full_like(ln, float("inf")))
            separated |= ov <= 0
            better = ov < best_d
            best_d = torch.where(better, ov, best_d)
            sgn = torch.where((t * axis).sum(-1) < 0, -1.0, 1.0)
            best_n = torch.where(better[:, None], axis * sgn[:, None], best_n)
            best_ij = torch.where(better[:, None], torch.tensor([i, j], device=c_a.device)[None].expand(B, 2), best_ij)
    # a small bias towards face contacts keeps resting boxes on their vertex-face contacts
    use = (~separated) & (best_d < 0.95 * face_d - 1e-9)
    # the supporting edges: from each centre go to the extreme along ±n on the two axes that are not the edge's own
    def edge(c, R, h, idx, direction):
        pt = c.clone()
        for kx in range(3):
            sg = torch.sign((R[:, :, kx] * direction).sum(-1))
            sg = torch.where(sg == 0, torch.ones_like(sg), sg)
            pt = pt + torch.where(idx == kx, torch.zeros_like(sg), sg * h[kx])[:, None] * R[:, :, kx]
        d = R.gather(2, idx[:, None, None].expand(-1, 3, 1))[..., 0] * h[idx][:, None]
        return pt - d, 2 * d
    pa, da = edge(c_a, R_a, h_a, best_ij[:, 0], best_n)
    pb, db = edge(c_b, R_b, h_b, best_ij[:, 1], -best_n)
    qa, qb = closest_segment_points(pa, da, pb, db)
    depth = torch.where(use, best_d, -torch.ones_like(best_d))
    return 0.5 * (qa + qb), best_n, depth


def _point_in_box(p, c, R, h):
    """(outward normal of the nearest face, depth below it) of a point relative to a box; depth <= 0 outside."""
    loc = (R.transpose(1, 2) @ (p - c)[:, :, None])[..., 0]
    room = h - loc.abs()                                        # distance to the face pair of every axis
    inside = (room > 0).all(-1)
    ax = room.argmin(-1)
    sgn = torch.sign(loc.gather(1, ax[:, None]))[:, 0]
    sgn = torch.where(sgn == 0, torch.ones_like(sgn), sgn)
    n = R.gather(2, ax[:, None, None].expand(-1, 3, 1))[..., 0] * sgn[:, None]
    depth = torch.where(inside, room.min(-1).values, -torch.ones_like(sgn))
    return n, depth


def _tangents(n):
    ref = torch.where((n[..., 0:1].abs() < 0.9), torch.tensor([1.0, 0, 0], dtype=n.dtype, device=n.device),
                      torch.tensor([0.0, 1.0, 0], dtype=n.dtype, device=n.device))
    t1 = torch.linalg.cross(n, ref.expand_as(n))
    t1 = t1 / t1.norm(dim=-1, keepdim=True)
    return t1, torch.linalg.cross(n, t1)


# ------------------------------------------------------------------------------------------ constraints
def _impedance(opt, pen):
    d0, dmax, width, mid, power = opt.solimp
    x = (pen / width).clamp(0, 1)
    y = torch.where(x <= mid, x ** power / mid ** (power - 1), 1 - (1 - x) ** power / (1 - mid) ** (power - 1))
    return (d0 + y * (dmax - d0)).clamp(1e-4, 0.9999)


@dataclass
class Rows:
    J: torch.Tensor          # [B, nr, nv]
    aref: torch.Tensor       # [B, nr]
    d: torch.Tensor          # [B, nr] impedance
    active: torch.Tensor     # [B, nr] bool
    kind: List[int]          # 0 unilateral (limit / contact normal), 1 friction
    parent_row: List[int]    # friction rows: index of their normal row
    mu: torch.Tensor         # [nr]
    body: List[int]          # body that feels the force (touch sensor), −1 for limits


def constraint_rows(m: GeneralModel, k: Kin, qpos, qvel, con: Contacts) -> Rows:
    B, opt = qpos.shape[0], m.opt
    tc, dr = opt.solref
    dmax = opt.solimp[1]
    kk, bb = 1.0 / (dmax * dmax * tc * tc * dr * dr), 2.0 / (dmax * tc)
    J, r, kind, par, mu, body, vel_only = [], [], [], [], [], [], []
    zero = torch.zeros(B, dtype=qpos.dtype, device=qpos.device)
    for d, (lo, hi) in m.limits:
        q = qpos[:, m.dofs[d].qadr]
        for sgn, dist in ((1.0, q - lo), (-1.0, hi - q)):
            e = torch.zeros(B, m.nv, dtype=qpos.dtype, device=qpos.device)
            e[:, d] = sgn
            J.append(e), r.append(dist), kind.append(0), par.append(-1), mu.append(0.0), body.append(-1)
    if m.tendons:
        L = tendon_length(m, qpos)
        for ti, td in enumerate(m.tendons):
            if td.range is None:
                continue
            for sgn, dist in ((1.0, L[:, ti] - td.range[0]), (-1.0, td.range[1] - L[:, ti])):
                J.append((sgn * m.tendon_coef[ti])[None].expand(B, -1)), r.append(dist), kind.append(0), par.append(-1)
                mu.append(0.0), body.append(-1)
    nc = con.depth.shape[1]
    normal_row = []
    for c in range(nc):
        Jp = point_jacobian(m, k, con.body2[c], con.point[:, c])
        if con.body1[c] >= 0:
            Jp = Jp - point_jacobian(m, k, con.body1[c], con.point[:, c])
        normal_row.append(len(J))
        J.append((con.normal[:, c, None] @ Jp)[:, 0]), r.append(-con.depth[:, c]), kind.append(0), par.append(-1)
        mu.append(0.0), body.append(con.body2[c])
        con_J = Jp
        if opt.friction_rows:
            t1, t2 = _tangents(con.normal[:, c])
            for tt in (t1, t2):
                J.append((tt[:, None] @ con_J)[:, 0]), r.append(zero), kind.append(1), par.append(normal_row[-1])
                mu.append(float(con.mu[c])), body.append(con.body2[c])
    if not J:
        e = torch.zeros(B, 0, dtype=qpos.dtype, device=qpos.device)
        return Rows(torch.zeros(B, 0, m.nv, dtype=qpos.dtype, device=qpos.device), e, e, e.bool(), [], [], m.t([]), [])
    J, r = torch.stack(J, 1), torch.stack(r, 1)
    kind_t = torch.tensor(kind, device=qpos.device)
    vel = (J @ qvel[:, :, None])[..., 0]
    aref = torch.where(kind_t[None] == 0, -bb * vel - kk * r, -bb * vel)
    active = r < opt.margin
    for i, p in enumerate(par):
        if p >= 0:
            active[:, i] = active[:, p]
    dimp = _impedance(opt, (-r).clamp(min=0))
    for i, p in enumerate(par):
        if p >= 0:
            dimp[:, i] = dimp[:, p]
    return Rows(J, aref, dimp, active, kind, par, m.t(mu), body)


def _disc_qp(Q, c, radius, newton_iters: int = 12):
    """argmin ½ xᵀQx + cᵀx over ‖x‖ ≤ radius for batched symmetric positive 2 × 2 ``Q``: the unconstrained minimiser when it
    lies inside, else (Q + λI)⁻¹(−c) with λ > 0 from Newton's iteration on the secular equation ‖x(λ)‖ = radius."""
    w, V = torch.linalg.eigh(Q)                                                    # [B, 2], [B, 2, 2]
    g = -(V.transpose(1, 2) @ c[:, :, None])[..., 0]                              # −c in the eigenbasis
    w = w.clamp(min=1e-12)
    y0 = g / w
    inside = y0.norm(dim=1) <= radius
    lam = torch.zeros_like(radius)
    r = radius.clamp(min=1e-30)
    for _ in range(newton_iters):
        den = w + lam[:, None]
        nrm = (g / den).norm(dim=1).clamp(min=1e-30)
        # φ(λ) = 1/‖x‖ − 1/r is nearly linear in λ: Newton on it converges from λ = 0 without safeguards
        dn = -((g * g) / den ** 3).sum(1) / nrm
        lam = (lam - (1 / nrm - 1 / r) / (-dn / nrm ** 2)).clamp(min=0)
    y = torch.where(inside[:, None], y0, g / (w + lam[:, None]))
    y = torch.where((radius <= 0)[:, None], torch.zeros_like(y), y)
    return (V @ y[:, :, None])[..., 0]


def constraint_islands(M, rows: Rows, eps: float = 1e-12) -> List[List[int]]:
    """Connected components of the constraint rows: two rows are coupled when J M⁻¹ Jᵀ links them in any lane of the batch
    (they touch the same kinematic chain).  Friction rows stay with their normal row.  Rows that are inactive in every lane
    come out as singletons."""
    nr = rows.aref.shape[1]
    if nr == 0:
        return []
    A = rows.J @ torch.linalg.solve(M, rows.J.transpose(1, 2))
    act = rows.active.to(A.dtype)
    link = ((A * act[:, :, None] * act[:, None, :]).abs() > eps).any(0).cpu()
    root = list(range(nr))

    def find(i):
        while root[i] != i:
            root[i] = root[root[i]]
            i = root[i]
        return i
    for i in range(nr):
        if rows.parent_row[i] >= 0:
            root[find(i)] = find(rows.parent_row[i])
        for j in torch.nonzero(link[i]).flatten().tolist():
            root[find(i)] = find(j)
    groups: Dict[int, List[int]] = {}
    for i in range(nr):
        groups.setdefault(find(i), []).append(i)
    return sorted(groups.values())


def solve_constraints(m: GeneralModel, M, qacc0, rows: Rows, solver="pgs", iters=50, cone: str = "pyramidal", noslip_iters: int = 0,
                      islands: bool = False):
    """Forces ``f [B, nr]`` of the soft-constraint problem (A + R) f + J q̈₀ − a_ref = 0 with f ≥ 0 on unilateral rows and
    |f| ≤ μ f_normal on friction rows.  Returns (f, q̈).

    ``cone="elliptic"`` (PGS only) bounds the NORM of the two tangential forces of a contact by μ f_normal (a circular cone)
    instead of each of them (the box that circumscribes it): the pair is updated as a block, the exact minimiser of the
    two-variable quadratic over the disc (``_disc_qp``).
    ``islands=True`` splits the rows into their connected components first (``constraint_islands``).
    ``noslip_iters`` more PGS sweeps over the friction rows alone, with their regularisation R removed, take out the slow
    creep that the soft friction rows allow under a sustained tangential load."""
    B, nr = rows.aref.shape
    if nr == 0:
        return rows.aref, qacc0
    if islands:
        # every island is its own problem (the coupling matrix is block diagonal over them): smaller dense solves for the
        # Newton method, shorter sweeps for PGS
        f = torch.zeros_like(rows.aref)
        for isl in constraint_islands(M, rows):
            local = {g: l for l, g in enumerate(isl)}
            sub = Rows(rows.J[:, isl], rows.aref[:, isl], rows.d[:, isl], rows.active[:, isl], [rows.kind[i] for i in isl],
                       [local.get(rows.parent_row[i], -1) for i in isl], rows.mu[isl], [rows.body[i] for i in isl])
            f[:, isl] = solve_constraints(m, M, qacc0, sub, solver, iters, cone, noslip_iters)[0]
        return f, qacc0 + (torch.linalg.solve(M, rows.J.transpose(1, 2)) @ f[:, :, None])[..., 0]
    Minv_Jt = torch.linalg.solve(M, rows.J.transpose(1, 2))                     # [B, nv, nr]
    A = rows.J @ Minv_Jt
    act = rows.active.to(A.dtype)
    diag = torch.diagonal(A, dim1=1, dim2=2)
    R = (1 - rows.d) / rows.d * diag.clamp(min=1e-10)
    A = A * act[:, :, None] * act[:, None, :] + torch.diag_embed(R + (1 - act))          # inactive rows: identity, zero force
    b = ((rows.J @ qacc0[:, :, None])[..., 0] - rows.aref) * act
    f = torch.zeros(B, nr, dtype=A.dtype, device=A.device)
    kind, par, mu = rows.kind, rows.parent_row, rows.mu

    def project(f):
        lo = torch.zeros_like(f)
        hi = torch.full_like(f, float("inf"))
        for i in range(nr):
            if kind[i] == 1:
                lim = mu[i] * f[:, par[i]].clamp(min=0)
                lo[:, i], hi[:, i] = -lim, lim
        return lo, hi

    if solver == "pgs":
        dA = torch.diagonal(A, dim1=1, dim2=2)
        pair_first = {i for i in range(nr - 1) if kind[i] == 1 and kind[i + 1] == 1 and par[i] == par[i + 1]
                      and (i == 0 or not (kind[i - 1] == 1 and par[i - 1] == par[i]))}
        for _ in range(iters):
            skip = -1
            for i in range(nr):
                if i == skip:
                    continue
                if cone == "elliptic" and i in pair_first:
                    # the two tangential forces of a contact as one block: the quadratic restricted to them, minimised
                    # over the disc of radius μ f_normal (a two-variable QCQP, solved in the block's eigenbasis)
                    j = i + 1
                    idx = [i, j]
                    Att = A[:, idx][:, :, idx]                                           # [B, 2, 2]
                    c = (A[:, idx] * f[:, None, :]).sum(-1) + b[:, idx] - (Att @ f[:, idx, None])[..., 0]
                    f = f.clone()
                    f[:, idx] = _disc_qp(Att, c, mu[i] * f[:, par[i]].clamp(min=0))
                    skip = j
                    continue
                res = (A[:, i] * f).sum(-1) + b[:, i]
                fi = f[:, i] - res / dA[:, i]
                if kind[i] == 0:
                    fi = fi.clamp(min=0)
                else:
                    lim = mu[i] * f[:, par[i]].clamp(min=0)
                    fi = torch.maximum(torch.minimum(fi, lim), -lim)
                f = f.clone()
                f[:, i] = fi
    elif solver == "newton":
        eye = torch.eye(nr, dtype=A.dtype, device=A.device)[None]
        for _ in range(iters):
            lo, hi = project(f)
            g = (A @ f[:, :, None])[..., 0] + b
            # free set: strictly inside the bounds, or on a bound with the gradient pointing inwards
            free = ~(((f <= lo) & (g > 0)) | ((f >= hi) & (g < 0)))
            fm = free.to(A.dtype)
            Af = A * fm[:, :, None] * fm[:, None, :] + eye * (1 - fm)[:, :, None]
            fixed = torch.where(free, torch.zeros_like(f), torch.maximum(torch.minimum(f, hi), lo))
            rhs = -(b + (A @ fixed[:, :, None])[..., 0]) * fm
            sol = torch.linalg.solve(Af, rhs[:, :, None])[..., 0]
            new = torch.where(free, sol, fixed)
            lo, hi = project(new)
            new = torch.maximum(torch.minimum(new, hi), lo)
            if float((new - f).abs().max()) < 1e-12:
                f = new
                break
            f = new
    elif solver == "cg":
        # projected conjugate gradients on the dual.  Outer rounds fix the friction bounds at μ times the current normal
        # forces, which leaves a plain box-constrained quadratic; inside, Polak-Ribière directions on the free set, steps
        # clipped to the box, and a restart of the direction whenever a step was clipped
        outer = 6
        inner = max(iters // outer, 4)
        for _ in range(outer):
            lo, hi = project(f)
            f = torch.maximum(torch.minimum(f, hi), lo)
            p = torch.zeros_like(f)
            r_prev = torch.zeros_like(f)
            restart = torch.ones(B, dtype=torch.bool, device=A.device)
            for _ in range(inner):
                g = (A @ f[:, :, None])[..., 0] + b
                free = ~(((f <= lo) & (g > 0)) | ((f >= hi) & (g < 0)))
                r = -g * free
                rr_prev = (r_prev * r_prev).sum(1)
                beta = ((r * (r - r_prev)).sum(1) / rr_prev.clamp(min=1e-30)).clamp(min=0)
                beta = torch.where(restart | (rr_prev <= 0), torch.zeros_like(beta), beta)
                p = (r + beta[:, None] * p) * free
                Ap = (A @ p[:, :, None])[..., 0]
                denom = (p * Ap).sum(1)
                alpha = torch.where(denom > 1e-30, (r * p).sum(1) / denom.clamp(min=1e-30), torch.zeros_like(denom))
                step = f + alpha[:, None] * p
                new = torch.maximum(torch.minimum(step, hi), lo)
                restart = (new != step).any(1)
                r_prev = r
                done = float((new - f).abs().max()) < 1e-13
                f = new
                if done:
                    break
        lo, hi = project(f)
        f = torch.maximum(torch.minimum(f, hi), lo)
    else:
        raise ValueError(solver)
    if noslip_iters > 0:
        fr_rows = [i for i in range(nr) if kind[i] == 1]
        dA0 = torch.diagonal(A, dim1=1, dim2=2) - R * act                          # friction rows without their softness
        for _ in range(noslip_iters):
            for i in fr_rows:
                res = (A[:, i] * f).sum(-1) - R[:, i] * act[:, i] * f[:, i] + b[:, i]
                fi = f[:, i] - res / dA0[:, i].clamp(min=1e-12)
                lim = mu[i] * f[:, par[i]].clamp(min=0)
                f = f.clone()
                f[:, i] = torch.maximum(torch.minimum(fi, lim), -lim)
                if cone == "elliptic" and i > 0 and kind[i - 1] == 1 and par[i - 1] == par[i]:
                    nrm = (f[:, i - 1] ** 2 + f[:, i] ** 2).sqrt()
                    sc = torch.where(nrm > lim, lim / nrm.clamp(min=1e-30), torch.ones_like(nrm))
                    f[:, i - 1], f[:, i] = f[:, i - 1] * sc, f[:, i] * sc
    f = f * act
    return f, qacc0 + (Minv_Jt @ f[:, :, None])[..., 0]


# ------------------------------------------------------------------------------------------ stepping
class GeneralSim:
    def __init__(self, model: GeneralModel, n: int, integrator: str = "euler", solver: str = "newton", solver_iters: int = 20,
                 cone: str = "pyramidal", noslip_iters: int = 0, islands: bool = False):
        self.cone, self.noslip_iters, self.islands = cone, noslip_iters, islands
        if cone == "elliptic" and solver != "pgs":
            raise ValueError("the elliptic cone is a projection of the PGS solver")
        self.m, self.n, self.integrator, self.solver, self.solver_iters = model, n, integrator, solver, solver_iters
        self.qpos, self.qvel = model.init_state(n)
        self.ctrl = torch.zeros(n, len(model.motors), dtype=model.dtype, device=model.device)
        self.qfrc_applied = torch.zeros(n, model.nv, dtype=model.dtype, device=model.device)      # external generalized force
        self.last: Dict[str, torch.Tensor] = {}

    def _applied(self):
        m = self.m
        tau = self.qfrc_applied.clone()
        self._act_force = torch.zeros_like(self.ctrl)
        for i, (mot, d) in enumerate(zip(m.motors, m.motor_dof)):
            self._act_force[:, i] = mot.gear * self.ctrl[:, i].clamp(*mot.ctrlrange)
            tau[:, d] += self._act_force[:, i]
        return tau

    def forward(self, qpos, qvel, implicit_damping=False, dt=0.0):
        """Constrained forward dynamics → q̈ (and the by-products the sensors read)."""
        m = self.m
        k = kinematics(m, qpos, qvel)
        Jv, Jw = body_jacobians(m, k)
        M = mass_matrix(m, k, Jv, Jw)
        c = bias_force(m, k, qvel, Jv, Jw)
        tau = self._applied() + passive_force(m, qpos, qvel) - c
        Mh = M + dt * torch.diag_embed(m.damping)[None] if implicit_damping else M
        qacc0 = torch.linalg.solve(Mh, tau[:, :, None])[..., 0]
        con = collide(m, k)
        rows = constraint_rows(m, k, qpos, qvel, con)
        f, qacc = solve_constraints(m, Mh, qacc0, rows, self.solver, self.solver_iters, self.cone, self.noslip_iters, self.islands)
        self.last = dict(kin=k, M=M, qacc=qacc, rows=rows, force=f, contacts=con, qvel=qvel)
        return qacc

    def step(self, ctrl=None):
        m, dt = self.m, self.m.opt.timestep
        if ctrl is not None:
            self.ctrl = ctrl.to(m.dtype)
        q, v = self.qpos, self.qvel
        if self.integrator in ("euler", "implicit"):
            a = self.forward(q, v, implicit_damping=self.integrator == "implicit", dt=dt)
            v = v + dt * a
            q = integrate_pos(m, q, v, dt)
        elif self.integrator == "rk4":
            k1v, k1a = v, self.forward(q, v)
            q2, v2 = integrate_pos(m, q, k1v, dt / 2), v + dt / 2 * k1a
            k2v, k2a = v2, self.forward(q2, v2)
            q3, v3 = integrate_pos(m, q, k2v, dt / 2), v + dt / 2 * k2a
            k3v, k3a = v3, self.forward(q3, v3)
            q4, v4 = integrate_pos(m, q, k3v, dt), v + dt * k3a
            k4v, k4a = v4, self.forward(q4, v4)
            q = integrate_pos(m, q, (k1v + 2 * k2v + 2 * k3v + k4v) / 6, dt)
            v = v + dt / 6 * (k1a + 2 * k2a + 2 * k3a + k4a)
        else:
            raise ValueError(self.integrator)
        self.qpos, self.qvel = q, v
        return q, v

    # ---- sensors (state of the LAST forward call, i.e. the beginning of the last step for Euler)
    def sensors(self, body: int = 0) -> Dict[str, torch.Tensor]:
        m = self.m
        if not self.last:
            self.forward(self.qpos, self.qvel)
        k, rows, f, qacc = self.last["kin"], self.last["rows"], self.last["force"], self.last["qacc"]
        R = k.xmat[:, body]
        Jp = point_jacobian(m, k, body, k.xpos[:, body])
        v_origin = k.v_com[:, body] - torch.linalg.cross(k.w_body[:, body], k.com[:, body] - k.xpos[:, body])
        qv = self.last["qvel"]
        lin_acc = (Jp @ qacc[:, :, None])[..., 0] + point_bias_acceleration(m, k, qv, body, k.xpos[:, body], v_origin)   # J q̈ + J̇ v
        touch = torch.zeros(self.n, dtype=m.dtype, device=m.device)
        for i, b in enumerate(rows.body):
            if b == body and rows.kind[i] == 0:
                touch = touch + f[:, i]
        sub = [b for b in range(m.nb) if self._in_subtree(b, body)]
        msub = m.mass[sub]
        return dict(
            jointpos=self.qpos.clone(), jointvel=self.qvel.clone(),
            framepos=k.xpos[:, body], framexmat=R,
            framelinvel=v_origin,
            frameangvel=k.w_body[:, body],
            gyro=(R.transpose(1, 2) @ k.w_body[:, body, :, None])[..., 0],
            accelerometer=(R.transpose(1, 2) @ (lin_acc - m.gravity)[:, :, None])[..., 0],
            touch=touch, actuatorfrc=self._act_force.clone(),
            subtreecom=(k.com[:, sub] * msub[None, :, None]).sum(1) / msub.sum(),
        )

    def _in_subtree(self, b, root):
        while b >= 0:
            if b == root:
                return True
            b = self.m.parent[b]
        return False


def osc_torque(m: GeneralModel, qpos, qvel, body: int, point_local, x_des, kp: float = 100.0, kd: Optional[float] = None,
               null_damping: float = 1.0, max_accel: float = 200.0):
    """Operational-space controller for a point fixed on ``body``: generalized forces that give the point the task-space
    acceleration kp (x_des − x) − kd ẋ through the task-space inertia Λ = (J M⁻¹ Jᵀ)⁻¹, compensate the bias force
    (gravity, Coriolis) and damp the motion in the null space of the task.  Returns ``(tau [B, nv], x [B, 3])``."""
    kd = 2.0 * math.sqrt(kp) if kd is None else kd
    k = kinematics(m, qpos, qvel)
    Jv, Jw = body_jacobians(m, k)
    M = mass_matrix(m, k, Jv, Jw)
    c = bias_force(m, k, qvel, Jv, Jw)
    x = k.xpos[:, body] + (k.xmat[:, body] @ m.t(point_local))
    J = point_jacobian(m, k, body, x)                                             # [B, 3, nv]
    xd = (J @ qvel[:, :, None])[..., 0]
    v_body_pt = xd
    jdqd = point_bias_acceleration(m, k, qvel, body, x, v_body_pt)
    Minv_Jt = torch.linalg.solve(M, J.transpose(1, 2))                            # [B, nv, 3]
    lam_inv = J @ Minv_Jt + 1e-6 * torch.eye(3, dtype=qpos.dtype, device=qpos.device)
    acc = (kp * (m.t(x_des) - x) - kd * xd)
    n = acc.norm(dim=-1, keepdim=True)
    acc = acc * torch.clamp(max_accel / n.clamp(min=1e-9), max=1.0)
    F = torch.linalg.solve(lam_inv, (acc - jdqd)[:, :, None])                     # Λ (ẍ* − J̇ q̇)
    tau = (J.transpose(1, 2) @ F)[..., 0] + c
    # null-space damping: (I − Jᵀ J̄ᵀ)(−k M q̇), J̄ = M⁻¹ Jᵀ Λ
    Jbar_T = torch.linalg.solve(lam_inv, Minv_Jt.transpose(1, 2))                 # Λ J M⁻¹  [B, 3, nv]
    t0 = -null_damping * (M @ qvel[:, :, None])[..., 0]
    tau = tau + t0 - (J.transpose(1, 2) @ (Jbar_T @ t0[:, :, None]))[..., 0]
    return tau, x
