"""Float64 NumPy oracle of the fused physics step.

The dynamics part is derived differently from the kernel so that agreement means something:
the kernel uses spatial-vector CRBA + recursive Newton-Euler about a moving reference point; the
oracle builds the mass matrix from per-body COM Jacobians, M = Σ m JvᵀJv + Jwᵀ I Jw, and the bias
force from the Lagrangian, c = Ṁ q̇ − ½ ∂(q̇ᵀ M q̇)/∂q + ∂U/∂q, with central finite differences
in double precision.  The constraint part (row order, soft-constraint parameters, projected
Gauss-Seidel sweeps, warm start) restates the kernel's algorithm one env at a time.
"""
from __future__ import annotations

import numpy as np

from .model import HINGE, RigidModel

ROW_LIMIT, ROW_NORMAL, ROW_T1, ROW_T2 = 0, 1, 2, 3


def _axis_angle_mat(axis, angle):
    a = axis / np.linalg.norm(axis)
    K = np.array([[0, -a[2], a[1]], [a[2], 0, -a[0]], [-a[1], a[0], 0]])
    return np.eye(3) + np.sin(angle) * K + (1 - np.cos(angle)) * (K @ K)


def _quat_mat(q):
    from .model import quat_to_mat
    return quat_to_mat(q)


def fk(m: RigidModel, qpos):
    """Body frames (xpos [nb,3], xmat [nb,3,3]) and per-dof world axis / anchor."""
    nb = m.nbody
    xpos = np.zeros((nb, 3))
    xmat = np.zeros((nb, 3, 3))
    axis_w = np.zeros((m.nv, 3))
    anchor_w = np.zeros((m.nv, 3))
    for b in range(nb):
        p = m.body_parent[b]
        pp, pR = (np.zeros(3), np.eye(3)) if p < 0 else (xpos[p], xmat[p])
        pos = pp + pR @ m.body_pos[b]
        R = pR @ _quat_mat(m.body_quat[b])
        for k in range(m.body_dofnum[b]):
            d = m.body_dofadr[b] + k
            q = qpos[d] - m.qpos0[d]
            aw = R @ m.dof_axis[d]
            axis_w[d] = aw
            if m.dof_type[d] == HINGE:
                anc = pos + R @ m.dof_pos[d]
                anchor_w[d] = anc
                R = R @ _axis_angle_mat(m.dof_axis[d], q)
                pos = anc - R @ m.dof_pos[d]
            else:
                pos = pos + q * aw
                anchor_w[d] = pos
        xpos[b], xmat[b] = pos, R
    return xpos, xmat, axis_w, anchor_w


def _is_anc(m, b, d):
    return bool((int(m.body_dofmask[b]) >> d) & 1)


def point_jacobian(m, axis_w, anchor_w, b, p):
    """3 x nv translational Jacobian of world point p fixed on body b, and 3 x nv rotational."""
    Jv = np.zeros((3, m.nv))
    Jw = np.zeros((3, m.nv))
    for d in range(m.nv):
        if not _is_anc(m, b, d):
            continue
        if m.dof_type[d] == HINGE:
            Jw[:, d] = axis_w[d]
            Jv[:, d] = np.cross(axis_w[d], p - anchor_w[d])
        else:
            Jv[:, d] = axis_w[d]
    return Jv, Jw


def mass_matrix(m: RigidModel, qpos):
    xpos, xmat, aw, an = fk(m, qpos)
    M = np.zeros((m.nv, m.nv))
    for b in range(m.nbody):
        R = xmat[b]
        com = xpos[b] + R @ m.body_ipos[b]
        i6 = m.body_inertia6[b]
        Ib = np.array([[i6[0], i6[3], i6[4]], [i6[3], i6[1], i6[5]], [i6[4], i6[5], i6[2]]])
        Iw = R @ Ib @ R.T
        Jv, Jw = point_jacobian(m, aw, an, b, com)
        M += m.body_mass[b] * Jv.T @ Jv + Jw.T @ Iw @ Jw
    return M


def potential(m: RigidModel, qpos):
    xpos, xmat, _, _ = fk(m, qpos)
    g = np.asarray(m.opt.gravity, np.float64)
    U = 0.0
    for b in range(m.nbody):
        com = xpos[b] + xmat[b] @ m.body_ipos[b]
        U -= m.body_mass[b] * np.dot(g, com)
    return U


def bias_force(m: RigidModel, qpos, qvel, eps=1e-6):
    """Coriolis/centrifugal + gravity generalized force via the Lagrangian."""
    nv = m.nv
    dM = np.zeros((nv, nv, nv))
    dU = np.zeros(nv)
    for k in range(nv):
        e = np.zeros(nv)
        e[k] = eps
        dM[k] = (mass_matrix(m, qpos + e) - mass_matrix(m, qpos - e)) / (2 * eps)
        dU[k] = (potential(m, qpos + e) - potential(m, qpos - e)) / (2 * eps)
    Mdot = np.einsum("kij,k->ij", dM, qvel)
    c = Mdot @ qvel - 0.5 * np.einsum("kij,i,j->k", dM, qvel, qvel)
    return c + dU


def impedance(opt, pen):
    d0, dmax, width, mid, power = opt.solimp
    x = min(max(pen / width, 0.0), 1.0)
    if x <= mid:
        y = x ** power / mid ** (power - 1)
    else:
        y = 1 - (1 - x) ** power / (1 - mid) ** (power - 1)
    return min(max(d0 + y * (dmax - d0), 1e-4), 0.9999)


def substep(m: RigidModel, qpos, qvel, tau_act, warm, debug=None):
    """One substep for ONE env; returns (qpos, qvel). `warm` [nlimit + 3 ncs] is updated in place."""
    o = m.opt
    dt = o.timestep
    nv = m.nv
    xpos, xmat, aw, an = fk(m, qpos)
    M = mass_matrix(m, qpos)
    bias = bias_force(m, qpos, qvel)
    Mh = M + np.diag(m.dof_armature + dt * m.dof_damping)
    tau = tau_act - bias - m.dof_damping * qvel - m.dof_stiffness * (qpos - m.dof_springref)
    Mh_inv = np.linalg.inv(Mh)
    qacc_s = Mh_inv @ tau
    pn = np.asarray(o.plane_normal, np.float64)
    # detection
    rows = []  # (kind, slot, parent, dist, sgn)
    for s in range(m.nlimit):
        q = qpos[m.lim_dof[s]]
        dlo, dhi = q - m.lim_lo[s], m.lim_hi[s] - q
        dist, sgn = (dlo, 1.0) if dlo < dhi else (dhi, -1.0)
        if dist < o.margin:
            rows.append([ROW_LIMIT, s, -1, dist, sgn])
        else:
            warm[s] = 0.0
    pts = {}
    for cs in range(m.ncs):
        b = m.cs_body[cs]
        p = xpos[b] + xmat[b] @ m.cs_local[cs]
        dist = np.dot(pn, p) - o.plane_offset - m.cs_radius[cs]
        pts[cs] = (p, dist)
        if dist < o.margin:
            rows.append([ROW_NORMAL, m.nlimit + cs, -1, dist, 1.0])
        else:
            warm[m.nlimit + 3 * cs: m.nlimit + 3 * cs + 3] = 0.0
    rows = rows[: o.rmax]
    nuni = len(rows)
    if o.friction_rows:
        nd = 1 if m.planar else 2
        for r in range(nuni):
            if rows[r][0] == ROW_NORMAL and len(rows) + nd - 1 < o.rmax:
                rows.append([ROW_T1, rows[r][1], r, 0.0, 1.0])
                if nd == 2:
                    rows.append([ROW_T2, rows[r][1], r, 0.0, 1.0])
    t1 = np.array([1.0, 0, 0]) - pn[0] * pn
    if np.dot(t1, t1) < 1e-6:
        t1 = np.array([0, 1.0, 0]) - pn[1] * pn
    t1 /= np.linalg.norm(t1)
    t2 = np.cross(pn, t1)
    tc, dr = o.solref
    dmax = o.solimp[1]
    k_s = 1.0 / (dmax * dmax * tc * tc * dr * dr)
    b_s = 2.0 / (dmax * tc)
    nr = len(rows)
    J = np.zeros((nr, nv))
    aref = np.zeros(nr)
    Rr = np.zeros(nr)
    lam = np.zeros(nr)
    ws = np.zeros(nr, np.int64)
    mu = np.zeros(nr)
    for r, (kind, slot, parent, dist, sgn) in enumerate(rows):
        if kind == ROW_LIMIT:
            J[r, m.lim_dof[slot]] = sgn
            ws[r] = slot
        else:
            cs = slot - m.nlimit
            p, d = pts[cs]
            pc = p - (m.cs_radius[cs] + 0.5 * d) * pn
            Jv, _ = point_jacobian(m, aw, an, m.cs_body[cs], pc)
            dirv = pn if kind == ROW_NORMAL else (t1 if kind == ROW_T1 else t2)
            J[r] = dirv @ Jv
            ws[r] = m.nlimit + 3 * cs + (0 if kind == ROW_NORMAL else (1 if kind == ROW_T1 else 2))
            mu[r] = m.cs_mu[cs]
    B = J @ Mh_inv  # rows: M̂⁻¹ Jᵀ
    for r, (kind, slot, parent, dist, sgn) in enumerate(rows):
        diag = max(float(J[r] @ B[r]), 1e-10)
        vel = float(J[r] @ qvel)
        imp = impedance(o, abs(dist))
        if kind <= ROW_NORMAL:
            aref[r] = -b_s * vel - k_s * imp * dist
            Rr[r] = (1 - imp) / imp * diag
        else:
            aref[r] = -b_s * vel
            Rr[r] = (1 - dmax) / dmax * diag * o.friction_reg
        rows[r].append(1.0 / (diag + Rr[r]))
        lam[r] = warm[ws[r]]
    qacc = qacc_s.copy()
    for r in range(nr):
        qacc += B[r] * lam[r]
    for _ in range(o.pgs_iters):
        for r in range(nr):
            res = J[r] @ qacc - aref[r] + Rr[r] * lam[r]
            ln = lam[r] - res * rows[r][5]
            if rows[r][0] <= ROW_NORMAL:
                ln = max(ln, 0.0)
            else:
                bound = mu[r] * lam[rows[r][2]]
                ln = min(max(ln, -bound), bound)
            qacc += B[r] * (ln - lam[r])
            lam[r] = ln
    for r in range(nr):
        warm[ws[r]] = lam[r]
    if debug is not None:
        debug.update(M=M + np.diag(m.dof_armature + dt * m.dof_damping), bias=bias, qacc_smooth=qacc_s, qacc=qacc,
                     nrow=nr, J=J, lam=lam.copy())
    qvel = np.clip(qvel + dt * qacc, -o.max_vel, o.max_vel)
    qpos = qpos + dt * qvel
    return qpos, qvel


def env_step(m: RigidModel, qpos, qvel, action, warm, frame_skip=5, debug=None):
    """Control step for one env: clamp ctrl, apply gear, integrate `frame_skip` substeps."""
    u = np.clip(np.asarray(action, np.float64), m.act_lo, m.act_hi)
    tau = np.zeros(m.nv)
    for a in range(m.nu):
        tau[m.act_dof[a]] += m.act_gear[a] * u[a]
    for s in range(frame_skip):
        qpos, qvel = substep(m, qpos, qvel, tau, warm, debug if s == 0 else None)
    return qpos, qvel
