"""Rigid-body model description (batch-shared) and builders.

The model is a kinematic tree of bodies; every degree of freedom is a hinge or a slide joint
(nq == nv).  State is batched, the model is not ("batches STATE, not MODEL",
noeira/physics3d/gpu/constants.mojo:162-171).  Geometry that can touch the ground plane is
reduced at build time to *contact spheres* (body-fixed centre + radius): a capsule gives its two
end spheres, a sphere gives one.

Builders:
    planar_chain(...)   the 7-capsule planar chain of the PPO benchmark configuration
    half_cheetah()      HalfCheetah-class planar runner (noeira/envs/half_cheetah/assets/half_cheetah.xml)
    hopper(), pendulum_cart()  smaller trees used by tests / examples
    from_mjcf(xml)      MJCF subset parser (physics/mjcf.py)
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np

SLIDE, HINGE = 0, 1


def quat_from_axis_angle(axis, angle):
    axis = np.asarray(axis, np.float64)
    axis = axis / (np.linalg.norm(axis) + 1e-30)
    s = np.sin(0.5 * angle)
    return np.array([np.cos(0.5 * angle), *(s * axis)])


def quat_mul(a, b):
    aw, ax, ay, az = a
    bw, bx, by, bz = b
    return np.array([aw * bw - ax * bx - ay * by - az * bz, aw * bx + ax * bw + ay * bz - az * by,
                     aw * by - ax * bz + ay * bw + az * bx, aw * bz + ax * by - ay * bx + az * bw])


def quat_to_mat(q):
    w, x, y, z = q
    return np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - w * z), 2 * (x * z + w * y)],
                     [2 * (x * y + w * z), 1 - 2 * (x * x + z * z), 2 * (y * z - w * x)],
                     [2 * (x * z - w * y), 2 * (y * z + w * x), 1 - 2 * (x * x + y * y)]])


def quat_z_to(vec):
    """Quaternion rotating +z onto `vec`."""
    v = np.asarray(vec, np.float64)
    v = v / np.linalg.norm(v)
    z = np.array([0.0, 0.0, 1.0])
    c = float(np.dot(z, v))
    if c > 1 - 1e-12:
        return np.array([1.0, 0, 0, 0])
    if c < -1 + 1e-12:
        return np.array([0.0, 1.0, 0, 0])
    axis = np.cross(z, v)
    return quat_from_axis_angle(axis, np.arccos(c))


def capsule_mass_inertia(radius, half_length, density):
    """Mass and principal inertia (about the centre, axis = z) of a solid capsule."""
    r, h = radius, 2.0 * half_length
    m_cyl = density * np.pi * r * r * h
    m_sph = density * 4.0 / 3.0 * np.pi * r ** 3
    izz = 0.5 * m_cyl * r * r + 0.4 * m_sph * r * r
    # hemisphere caps: parallel-axis from the cylinder ends
    ixx = m_cyl * (h * h / 12.0 + r * r / 4.0) + m_sph * (0.4 * r * r + 0.375 * r * h + 0.25 * h * h)
    return m_cyl + m_sph, np.array([ixx, ixx, izz])


def sphere_mass_inertia(radius, density):
    m = density * 4.0 / 3.0 * np.pi * radius ** 3
    i = 0.4 * m * radius * radius
    return m, np.array([i, i, i])


@dataclass
class Joint:
    type: int
    axis: Sequence[float]
    pos: Sequence[float] = (0.0, 0.0, 0.0)
    range: Optional[Sequence[float]] = None
    armature: float = 0.0
    damping: float = 0.0
    stiffness: float = 0.0
    springref: float = 0.0
    qpos0: float = 0.0
    name: str = ""


@dataclass
class Geom:
    type: str  # "capsule" | "sphere"
    size: Sequence[float]  # capsule: (radius, half_length); sphere: (radius,)
    pos: Sequence[float] = (0.0, 0.0, 0.0)
    quat: Sequence[float] = (1.0, 0.0, 0.0, 0.0)  # capsule axis = local z
    friction: float = 1.0
    density: float = 1000.0
    rgba: Sequence[float] = (0.7, 0.7, 0.7, 1.0)
    contact: bool = True
    vertices: Optional[Sequence[Sequence[float]]] = None  # type "mesh": points whose convex hull is the shape; size = (margin,)


@dataclass
class Body:
    parent: int
    pos: Sequence[float]
    quat: Sequence[float] = (1.0, 0.0, 0.0, 0.0)
    joints: List[Joint] = field(default_factory=list)
    geoms: List[Geom] = field(default_factory=list)
    name: str = ""
    mass: Optional[float] = None  # explicit inertial overrides geoms
    inertia: Optional[Sequence[float]] = None
    ipos: Optional[Sequence[float]] = None


@dataclass
class Actuator:
    joint: str
    gear: float
    ctrlrange: Sequence[float] = (-1.0, 1.0)


@dataclass
class Options:
    timestep: float = 0.01
    gravity: Sequence[float] = (0.0, 0.0, -9.81)
    solref: Sequence[float] = (0.02, 1.0)
    solimp: Sequence[float] = (0.9, 0.95, 0.001, 0.5, 2.0)
    margin: float = 0.0
    pgs_iters: int = 8
    friction_rows: bool = True
    friction_reg: float = 1.0
    plane_normal: Sequence[float] = (0.0, 0.0, 1.0)
    plane_offset: float = 0.0
    max_vel: float = 100.0
    rmax: int = 32


class RigidModel:
    """Flattened arrays consumed by the CUDA kernel and by the NumPy oracle."""

    def __init__(self, bodies: List[Body], actuators: List[Actuator], opt: Options = None, total_mass: float = None):
        self.opt = opt or Options()
        self.bodies = bodies
        nb = len(bodies)
        if nb > 32:
            raise ValueError("at most 32 bodies per tree")
        self.nbody = nb
        self.body_parent = np.array([b.parent for b in bodies], np.int32)
        for i, p in enumerate(self.body_parent):
            if p >= i:
                raise ValueError("bodies must be topologically ordered (parent < child)")
        self.body_depth = np.zeros(nb, np.int32)
        for i in range(nb):
            self.body_depth[i] = 0 if self.body_parent[i] < 0 else self.body_depth[self.body_parent[i]] + 1
        self.body_pos = np.array([b.pos for b in bodies], np.float64).reshape(nb, 3)
        self.body_quat = np.array([b.quat for b in bodies], np.float64).reshape(nb, 4)
        # dofs
        dof_type, dof_axis, dof_pos, dof_body, arm, damp, stiff, sref, qpos0, names = [], [], [], [], [], [], [], [], [], []
        lim_dof, lim_lo, lim_hi = [], [], []
        self.body_dofadr = np.zeros(nb, np.int32)
        self.body_dofnum = np.zeros(nb, np.int32)
        for i, b in enumerate(bodies):
            self.body_dofadr[i] = len(dof_type)
            self.body_dofnum[i] = len(b.joints)
            for j in b.joints:
                ax = np.asarray(j.axis, np.float64)
                ax = ax / np.linalg.norm(ax)
                if j.range is not None:
                    lim_dof.append(len(dof_type))
                    lim_lo.append(float(j.range[0]))
                    lim_hi.append(float(j.range[1]))
                dof_type.append(j.type)
                dof_axis.append(ax)
                dof_pos.append(np.asarray(j.pos, np.float64))
                dof_body.append(i)
                arm.append(j.armature)
                damp.append(j.damping)
                stiff.append(j.stiffness)
                sref.append(j.springref)
                qpos0.append(j.qpos0)
                names.append(j.name or f"dof{len(names)}")
        nv = len(dof_type)
        if nv > 32 or nv < 1:
            raise ValueError("1..32 degrees of freedom supported")
        self.nv = nv
        self.dof_names = names
        self.dof_type = np.array(dof_type, np.int32)
        self.dof_axis = np.array(dof_axis, np.float64).reshape(nv, 3)
        self.dof_pos = np.array(dof_pos, np.float64).reshape(nv, 3)
        self.dof_body = np.array(dof_body, np.int32)
        self.dof_armature = np.array(arm, np.float64)
        self.dof_damping = np.array(damp, np.float64)
        self.dof_stiffness = np.array(stiff, np.float64)
        self.dof_springref = np.array(sref, np.float64)
        self.qpos0 = np.array(qpos0, np.float64)
        self.lim_dof = np.array(lim_dof, np.int32)
        self.lim_lo = np.array(lim_lo, np.float64)
        self.lim_hi = np.array(lim_hi, np.float64)
        self.nlimit = len(lim_dof)
        # ancestor masks
        self.body_ancmask = np.zeros(nb, np.uint32)
        self.body_dofmask = np.zeros(nb, np.uint32)
        for i in range(nb):
            am = np.uint32(1) << np.uint32(i)
            dm = np.uint32(0)
            for k in range(self.body_dofnum[i]):
                dm |= np.uint32(1) << np.uint32(self.body_dofadr[i] + k)
            p = self.body_parent[i]
            if p >= 0:
                am |= self.body_ancmask[p]
                dm |= self.body_dofmask[p]
            self.body_ancmask[i] = am
            self.body_dofmask[i] = dm
        # inertial properties from geoms
        self.body_mass = np.zeros(nb)
        self.body_ipos = np.zeros((nb, 3))
        self.body_inertia6 = np.zeros((nb, 6))  # xx yy zz xy xz yz about the COM, body axes
        cs_body, cs_local, cs_radius, cs_mu = [], [], [], []
        self.geoms = []  # (body, type, pos, quat, size, rgba) for rendering
        for i, b in enumerate(bodies):
            if b.mass is not None:
                self.body_mass[i] = b.mass
                self.body_ipos[i] = np.zeros(3) if b.ipos is None else b.ipos
                d = np.asarray(b.inertia if b.inertia is not None else (1e-3,) * 3, np.float64)
                self.body_inertia6[i, :3] = d
            else:
                ms, cs, Is = [], [], []
                for g in b.geoms:
                    R = quat_to_mat(np.asarray(g.quat, np.float64))
                    if g.type == "capsule":
                        m, d = capsule_mass_inertia(g.size[0], g.size[1], g.density)
                    elif g.type == "sphere":
                        m, d = sphere_mass_inertia(g.size[0], g.density)
                    else:
                        raise ValueError(g.type)
                    ms.append(m)
                    cs.append(np.asarray(g.pos, np.float64))
                    Is.append(R @ np.diag(d) @ R.T)
                M = float(np.sum(ms)) if ms else 0.0
                if M <= 0:
                    raise ValueError(f"body {i} has no mass")
                com = sum(m * c for m, c in zip(ms, cs)) / M
                I = np.zeros((3, 3))
                for m, c, Ig in zip(ms, cs, Is):
                    r = c - com
                    I += Ig + m * (np.dot(r, r) * np.eye(3) - np.outer(r, r))
                self.body_mass[i] = M
                self.body_ipos[i] = com
                self.body_inertia6[i] = [I[0, 0], I[1, 1], I[2, 2], I[0, 1], I[0, 2], I[1, 2]]
            for g in b.geoms:
                self.geoms.append((i, g.type, np.asarray(g.pos, np.float64), np.asarray(g.quat, np.float64),
                                   tuple(g.size), tuple(g.rgba)))
                if not g.contact:
                    continue
                R = quat_to_mat(np.asarray(g.quat, np.float64))
                if g.type == "capsule":
                    for sgn in (-1.0, 1.0):
                        cs_body.append(i)
                        cs_local.append(np.asarray(g.pos) + sgn * g.size[1] * R[:, 2])
                        cs_radius.append(g.size[0])
                        cs_mu.append(g.friction)
                else:
                    cs_body.append(i)
                    cs_local.append(np.asarray(g.pos, np.float64))
                    cs_radius.append(g.size[0])
                    cs_mu.append(g.friction)
        if total_mass is not None:
            s = total_mass / self.body_mass.sum()
            self.body_mass *= s
            self.body_inertia6 *= s
        self.ncs = len(cs_body)
        self.cs_body = np.array(cs_body, np.int32)
        self.cs_local = np.array(cs_local, np.float64).reshape(self.ncs, 3)
        self.cs_radius = np.array(cs_radius, np.float64)
        self.cs_mu = np.array(cs_mu, np.float64)
        # actuators
        self.nu = len(actuators)
        self.act_dof = np.array([names.index(a.joint) for a in actuators], np.int32)
        self.act_gear = np.array([a.gear for a in actuators], np.float64)
        self.act_lo = np.array([a.ctrlrange[0] for a in actuators], np.float64)
        self.act_hi = np.array([a.ctrlrange[1] for a in actuators], np.float64)
        self.maxdepth = int(self.body_depth.max())
        # planar mechanism in the x-z plane: every hinge about ±y, every slide inside the plane, bodies not
        # rotated out of it → the y tangent of a ground contact can never move and gets no friction row
        ey = np.array([0.0, 1.0, 0.0])
        self.planar = bool(
            all((abs(abs(a @ ey) - 1) < 1e-9) if t == HINGE else (abs(a @ ey) < 1e-9)
                for a, t in zip(self.dof_axis, self.dof_type))
            and all(abs(q[1]) < 1e-9 and abs(q[3]) < 1e-9 for q in self.body_quat)
            and abs(np.asarray(self.opt.plane_normal) @ ey) < 1e-9)

    # -------------------------------------------------------------- packing for the kernel
    def pack(self, reset_noise=(0.1, 0.1)):
        i32 = np.concatenate([
            self.body_parent, self.body_depth, self.body_dofadr, self.body_dofnum,
            self.body_dofmask.view(np.int32), self.body_ancmask.view(np.int32), self.dof_body, self.dof_type,
            self.lim_dof, self.cs_body, self.act_dof]).astype(np.int32)
        f32 = np.concatenate([
            self.body_pos.ravel(), self.body_quat.ravel(), self.body_ipos.ravel(), self.body_inertia6.ravel(),
            self.body_mass, self.dof_axis.ravel(), self.dof_pos.ravel(), self.dof_armature, self.dof_damping,
            self.dof_stiffness, self.dof_springref, self.lim_lo, self.lim_hi, self.cs_local.ravel(),
            self.cs_radius, self.cs_mu, self.act_gear, self.act_lo, self.act_hi, self.qpos0,
            np.asarray(reset_noise, np.float64)]).astype(np.float32)
        return i32, f32


# ------------------------------------------------------------------------------------------ builders

def planar_chain(seed: int = 0, n_links: int = 7, radius: float = 0.046, length_range=(0.2, 0.3),
                 density: float = 1000.0, gear: float = 120.0, joint_range=(-1.0, 1.0), friction: float = 0.4,
                 armature: float = 0.1, damping: float = 4.0, z0: float = 0.5, opt: Options = None) -> RigidModel:
    """Planar chain: root slide-x, slide-z, hinge-y, then ``n_links-1`` hinge-y joints between capsule
    links laid along +x.  Link lengths are U(length_range) drawn from ``seed``.  nq = nv = n_links + 2."""
    rng = np.random.RandomState(seed)
    lengths = rng.uniform(length_range[0], length_range[1], size=n_links)
    qx = quat_z_to([1.0, 0.0, 0.0])
    bodies: List[Body] = []
    acts: List[Actuator] = []
    for i in range(n_links):
        hl = 0.5 * lengths[i]
        geom = Geom("capsule", (radius, hl), pos=(hl, 0.0, 0.0), quat=tuple(qx), friction=friction, density=density,
                    rgba=(0.2 + 0.1 * i, 0.5, 0.9 - 0.1 * i, 1.0))
        if i == 0:
            joints = [Joint(SLIDE, (1, 0, 0), name="rootx", qpos0=0.0),
                      Joint(SLIDE, (0, 0, 1), name="rootz", qpos0=0.0),
                      Joint(HINGE, (0, 1, 0), name="rooty")]
            bodies.append(Body(-1, (0.0, 0.0, z0), joints=joints, geoms=[geom], name="link0"))
        else:
            j = Joint(HINGE, (0, 1, 0), range=joint_range, armature=armature, damping=damping, name=f"hinge{i}")
            bodies.append(Body(i - 1, (lengths[i - 1], 0.0, 0.0), joints=[j], geoms=[geom], name=f"link{i}"))
            acts.append(Actuator(f"hinge{i}", gear))
    return RigidModel(bodies, acts, opt or Options())


def half_cheetah(opt: Options = None) -> RigidModel:
    """HalfCheetah-class planar runner: torso with slide-x / slide-z / hinge-y root, back and front
    legs of three hinged capsules each (stiffness, damping, gear and ranges as in
    noeira/envs/half_cheetah/assets/half_cheetah.xml:3-61), total mass 14."""
    r = 0.046
    fr = 0.4

    def cap(frm, to):
        frm, to = np.asarray(frm, float), np.asarray(to, float)
        c = 0.5 * (frm + to)
        hl = 0.5 * np.linalg.norm(to - frm)
        return Geom("capsule", (r, hl), pos=tuple(c), quat=tuple(quat_z_to(to - frm)), friction=fr)

    def hinge(name, rng, stiff, damp, pos=(0, 0, 0)):
        return Joint(HINGE, (0, 1, 0), pos=pos, range=rng, armature=0.1, damping=damp, stiffness=stiff, name=name)

    bodies = [
        Body(-1, (0, 0, 0.7), joints=[Joint(SLIDE, (1, 0, 0), name="rootx", armature=0.0),
                                      Joint(SLIDE, (0, 0, 1), name="rootz", armature=0.0),
                                      Joint(HINGE, (0, 1, 0), name="rooty", armature=0.0)],
             geoms=[cap((-0.5, 0, 0), (0.5, 0, 0)), cap((0.5, 0, 0), (0.7, 0, 0.14))], name="torso"),
        Body(0, (-0.5, 0, 0), joints=[hinge("bthigh", (-0.52, 1.05), 240, 6)], geoms=[cap((0, 0, 0), (0.16, 0, -0.25))], name="bthigh"),
        Body(1, (0.16, 0, -0.25), joints=[hinge("bshin", (-0.785, 0.785), 180, 4.5)], geoms=[cap((0, 0, 0), (-0.28, 0, -0.14))], name="bshin"),
        Body(2, (-0.28, 0, -0.14), joints=[hinge("bfoot", (-0.4, 0.785), 120, 3)], geoms=[cap((0, 0, 0), (0.13, 0, -0.18))], name="bfoot"),
        Body(0, (0.5, 0, 0), joints=[hinge("fthigh", (-1.0, 0.7), 180, 4.5)], geoms=[cap((0, 0, 0), (-0.14, 0, -0.24))], name="fthigh"),
        Body(4, (-0.14, 0, -0.24), joints=[hinge("fshin", (-1.2, 0.87), 120, 3)], geoms=[cap((0, 0, 0), (0.13, 0, -0.18))], name="fshin"),
        Body(5, (0.13, 0, -0.18), joints=[hinge("ffoot", (-0.5, 0.5), 60, 1.5)], geoms=[cap((0, 0, 0), (0.09, 0, -0.14))], name="ffoot"),
    ]
    gears = dict(bthigh=120, bshin=90, bfoot=60, fthigh=120, fshin=60, ffoot=30)
    acts = [Actuator(k, v) for k, v in gears.items()]
    o = opt or Options(solimp=(0.0, 0.8, 0.01, 0.5, 2.0))
    return RigidModel(bodies, acts, o, total_mass=14.0)


def hopper(opt: Options = None) -> RigidModel:
    """Hopper-class planar monoped: torso, thigh, leg, foot (3 actuated hinges)."""
    def cap(frm, to, rad, fr=0.9):
        frm, to = np.asarray(frm, float), np.asarray(to, float)
        return Geom("capsule", (rad, 0.5 * np.linalg.norm(to - frm)), pos=tuple(0.5 * (frm + to)),
                    quat=tuple(quat_z_to(to - frm)), friction=fr)

    bodies = [
        Body(-1, (0, 0, 1.25), joints=[Joint(SLIDE, (1, 0, 0), name="rootx"), Joint(SLIDE, (0, 0, 1), name="rootz"),
                                       Joint(HINGE, (0, 1, 0), name="rooty")],
             geoms=[cap((0, 0, 0.2), (0, 0, -0.2), 0.05)], name="torso"),
        Body(0, (0, 0, -0.2), joints=[Joint(HINGE, (0, -1, 0), range=(-2.6, 0.0), armature=1.0, damping=1.0, name="thigh")],
             geoms=[cap((0, 0, 0), (0, 0, -0.45), 0.05)], name="thigh"),
        Body(1, (0, 0, -0.45), joints=[Joint(HINGE, (0, -1, 0), range=(-2.6, 0.0), armature=1.0, damping=1.0, name="leg")],
             geoms=[cap((0, 0, 0), (0, 0, -0.5), 0.04)], name="leg"),
        Body(2, (0, 0, -0.5), joints=[Joint(HINGE, (0, -1, 0), range=(-0.785, 0.785), armature=1.0, damping=1.0, name="foot")],
             geoms=[cap((-0.13, 0, 0), (0.26, 0, 0), 0.06, fr=2.0)], name="foot"),
    ]
    acts = [Actuator("thigh", 200), Actuator("leg", 200), Actuator("foot", 200)]
    return RigidModel(bodies, acts, opt or Options(timestep=0.002))


def pendulum_cart(opt: Options = None) -> RigidModel:
    """Cart (slide-x) with a free-swinging pole (hinge-y); no ground contact geoms."""
    bodies = [
        Body(-1, (0, 0, 1.0), joints=[Joint(SLIDE, (1, 0, 0), name="slider", damping=0.0)],
             geoms=[Geom("sphere", (0.1,), contact=False)], name="cart"),
        Body(0, (0, 0, 0), joints=[Joint(HINGE, (0, 1, 0), name="hinge")],
             geoms=[Geom("capsule", (0.045, 0.3), pos=(0, 0, 0.3), contact=False)], name="pole"),
    ]
    return RigidModel(bodies, [Actuator("slider", 100.0)], opt or Options())


def walker2d(opt: Options = None) -> RigidModel:
    """Walker2d-class planar biped: torso and two legs of thigh / leg / foot (6 actuated hinges, 9 degrees of freedom)."""
    def cap(frm, to, rad, fr=0.9):
        frm, to = np.asarray(frm, float), np.asarray(to, float)
        return Geom("capsule", (rad, 0.5 * np.linalg.norm(to - frm)), pos=tuple(0.5 * (frm + to)),
                    quat=tuple(quat_z_to(to - frm)), friction=fr)

    def leg(side, foot_friction):
        j = lambda n, rng: Joint(HINGE, (0, -1, 0), range=rng, armature=0.01, damping=0.1, name=f"{n}_{side}")
        return [("thigh", 0, (0, 0, -0.2), j("thigh", (-2.6, 0.0)), cap((0, 0, 0), (0, 0, -0.45), 0.05)),
                ("leg", 1, (0, 0, -0.45), j("leg", (-2.6, 0.0)), cap((0, 0, 0), (0, 0, -0.5), 0.04)),
                ("foot", 2, (0, 0, -0.5), j("foot", (-0.785, 0.785)), cap((0, 0, 0), (0.2, 0, 0), 0.06, fr=foot_friction))]

    bodies = [Body(-1, (0, 0, 1.25), joints=[Joint(SLIDE, (1, 0, 0), name="rootx"), Joint(SLIDE, (0, 0, 1), name="rootz"),
                                             Joint(HINGE, (0, 1, 0), name="rooty")],
                   geoms=[cap((0, 0, 0.2), (0, 0, -0.2), 0.05)], name="torso")]
    for side, fr in (("right", 0.9), ("left", 1.9)):
        base = len(bodies)
        for name, up, pos, joint, geom in leg(side, fr):
            parent = 0 if up == 0 else base + up - 1
            bodies.append(Body(parent, pos, joints=[joint], geoms=[geom], name=f"{name}_{side}"))
    acts = [Actuator(f"{n}_{s}", g) for s in ("right", "left") for n, g in (("thigh", 100), ("leg", 100), ("foot", 20))]
    return RigidModel(bodies, acts, opt or Options(timestep=0.002))


def inverted_double_pendulum(opt: Options = None) -> RigidModel:
    """Cart on a rail with two poles in series (slide + two hinges); the cart force is the only actuator."""
    bodies = [
        Body(-1, (0, 0, 0.0), joints=[Joint(SLIDE, (1, 0, 0), range=(-1.0, 1.0), damping=0.05, name="slider")],
             geoms=[Geom("sphere", (0.1,), contact=False)], name="cart"),
        Body(0, (0, 0, 0), joints=[Joint(HINGE, (0, 1, 0), damping=0.05, name="hinge")],
             geoms=[Geom("capsule", (0.045, 0.3), pos=(0, 0, 0.3), contact=False)], name="pole"),
        Body(1, (0, 0, 0.6), joints=[Joint(HINGE, (0, 1, 0), damping=0.05, name="hinge2")],
             geoms=[Geom("capsule", (0.045, 0.3), pos=(0, 0, 0.3), contact=False)], name="pole2"),
    ]
    return RigidModel(bodies, [Actuator("slider", 500.0)], opt or Options(timestep=0.01))


def reacher(opt: Options = None) -> RigidModel:
    """Two-link planar arm in the horizontal plane (gravity off): two actuated hinges about z."""
    o = opt or Options(timestep=0.01, gravity=(0.0, 0.0, 0.0))
    bodies = [
        Body(-1, (0, 0, 0.01), joints=[Joint(HINGE, (0, 0, 1), damping=1.0, armature=1.0, name="joint0")],
             geoms=[Geom("capsule", (0.01, 0.05), pos=(0.05, 0, 0), quat=tuple(quat_z_to((1, 0, 0))), contact=False)], name="link0"),
        Body(0, (0.1, 0, 0), joints=[Joint(HINGE, (0, 0, 1), range=(-3.0, 3.0), damping=1.0, armature=1.0, name="joint1")],
             geoms=[Geom("capsule", (0.01, 0.05), pos=(0.05, 0, 0), quat=tuple(quat_z_to((1, 0, 0))), contact=False)], name="link1"),
    ]
    return RigidModel(bodies, [Actuator("joint0", 200.0), Actuator("joint1", 200.0)], o)
