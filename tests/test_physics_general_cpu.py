"""General rigid-body engine: agreement with the hinge / slide oracle, conservation laws for free and ball joints,
collision geometry, resting / sliding / colliding contacts with both solvers, joint limits, integrators, sensors."""
import math

import numpy as np
import pytest
import torch

from noeira_b200.physics import general as G
from noeira_b200.physics.model import Body, Geom, Joint, Options


def _free_box(opt=None, half=(0.2, 0.1, 0.05), z=1.0, plane=False, friction=1.0):
    b = Body(parent=-1, pos=(0, 0, z), joints=[Joint(G.FREE, (0, 0, 1), name="root")],
             geoms=[Geom("box", half, friction=friction)])
    return G.GeneralModel([b], opt=opt or Options(timestep=0.002), plane=plane)


def test_mass_matrix_and_bias_match_the_hinge_slide_oracle():
    from noeira_b200.physics import oracle
    from noeira_b200.physics.model import planar_chain
    rm = planar_chain(seed=2)
    gm = G.GeneralModel(rm.bodies, opt=rm.opt, plane=False)
    assert gm.nv == rm.nv
    rng = np.random.default_rng(0)
    q = rm.qpos0 + rng.normal(0, 0.4, rm.nv)
    v = rng.normal(0, 1.0, rm.nv)
    k = G.kinematics(gm, torch.tensor(q)[None], torch.tensor(v)[None])
    M = G.mass_matrix(gm, k)[0].numpy()
    c = G.bias_force(gm, k, torch.tensor(v)[None])[0].numpy()
    Mo = oracle.mass_matrix(rm, q)
    co = oracle.bias_force(rm, q, v)
    Mo = Mo + np.diag(rm.dof_armature) if np.abs(np.diag(M) - np.diag(Mo)).max() > 1e-9 else Mo
    assert np.abs(M - Mo).max() < 1e-8 * max(1.0, np.abs(Mo).max())
    assert np.abs(c - co).max() < 2e-5 * max(1.0, np.abs(co).max())          # the oracle differentiates numerically


def test_kinetic_energy_from_body_velocities_equals_quadratic_form():
    """½ vᵀ M v (Jacobians) against Σ ½ m |v_com|² + ½ ωᵀ I ω (the recursive velocity pass): two code paths."""
    bodies = [Body(-1, (0, 0, 1), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("box", (0.2, 0.1, 0.05))]),
              Body(0, (0.3, 0, 0), joints=[Joint(G.BALL, (0, 0, 1), pos=(-0.1, 0, 0))], geoms=[Geom("capsule", (0.04, 0.15), pos=(0.1, 0, 0))]),
              Body(1, (0.3, 0, 0), quat=(0.9238795, 0, 0.3826834, 0), joints=[Joint(G.HINGE, (0, 1, 0), pos=(0, 0.02, 0)), Joint(G.SLIDE, (1, 0, 0))],
                   geoms=[Geom("sphere", (0.07,), pos=(0.05, 0, 0.02))])]
    m = G.GeneralModel(bodies, plane=False)
    assert (m.nq, m.nv) == (7 + 4 + 2, 6 + 3 + 2)
    g = torch.Generator().manual_seed(0)
    q, v = m.init_state(3)
    q[:, 3:7] = torch.nn.functional.normalize(torch.randn(3, 4, generator=g, dtype=torch.float64), dim=-1)
    q[:, 7:11] = torch.nn.functional.normalize(torch.randn(3, 4, generator=g, dtype=torch.float64), dim=-1)
    q[:, 11:] = torch.randn(3, 2, generator=g, dtype=torch.float64) * 0.3
    v = torch.randn(3, m.nv, generator=g, dtype=torch.float64)
    k = G.kinematics(m, q, v)
    M = G.mass_matrix(m, k)
    T1 = 0.5 * (v[:, None] @ M @ v[:, :, None])[:, 0, 0]
    Iw = G.world_inertia(m, k)
    T2 = (0.5 * m.mass[None] * (k.v_com ** 2).sum(-1)).sum(1) + 0.5 * (k.w_body[:, :, None] @ Iw @ k.w_body[..., None])[..., 0, 0].sum(1)
    assert torch.allclose(T1, T2, rtol=1e-10)
    # velocities from the Jacobians equal the recursive ones
    Jv, Jw = G.body_jacobians(m, k)
    assert torch.allclose((Jv @ v[:, None, :, None])[..., 0], k.v_com, atol=1e-10)
    assert torch.allclose((Jw @ v[:, None, :, None])[..., 0], k.w_body, atol=1e-10)


@pytest.mark.parametrize("integrator,tol,etol", [("rk4", 5e-4, 1e-5), ("euler", 0.1, 0.05)])
def test_conservation_laws_of_a_free_chain(integrator, tol, etol):
    """No gravity: linear and angular momentum and the energy of a tumbling free body with a ball-jointed and a hinged link.
    (The errors shrink with the step: second order for Runge-Kutta with averaged body-frame rates, first order for Euler.)"""
    opt = Options(timestep=0.002, gravity=(0, 0, 0))
    bodies = [Body(-1, (0, 0, 0), joints=[Joint(G.FREE, (0, 0, 1))], mass=2.0, inertia=(0.02, 0.05, 0.04)),
              Body(0, (0.3, 0, 0), joints=[Joint(G.BALL, (0, 0, 1))], mass=1.0, inertia=(0.01, 0.02, 0.015), ipos=(0.1, 0.05, 0)),
              Body(1, (0.2, 0.1, 0), joints=[Joint(G.HINGE, (0, 0.6, 0.8))], mass=0.5, inertia=(0.004, 0.006, 0.005), ipos=(0, 0.1, 0.05))]
    m = G.GeneralModel(bodies, opt=opt, plane=False)
    sim = G.GeneralSim(m, 2, integrator=integrator)
    g = torch.Generator().manual_seed(1)
    sim.qvel = torch.randn(2, m.nv, generator=g, dtype=torch.float64) * torch.tensor([0.3] * 3 + [2.0] * 7)

    def momenta():
        k = G.kinematics(m, sim.qpos, sim.qvel)
        P = (m.mass[None, :, None] * k.v_com).sum(1)
        Iw = G.world_inertia(m, k)
        L = (torch.linalg.cross(k.com, m.mass[None, :, None] * k.v_com) + (Iw @ k.w_body[..., None])[..., 0]).sum(1)
        T, U = G.energy(m, sim.qpos, sim.qvel)
        return P, L, T + U

    P0, L0, E0 = momenta()
    for _ in range(300):
        sim.step()
    P1, L1, E1 = momenta()
    assert torch.allclose(P0, P1, atol=tol) and torch.allclose(L0, L1, atol=tol)
    assert ((E1 - E0).abs() / E0 < etol).all()


def test_spherical_pendulum_energy_and_hinge_period():
    opt = Options(timestep=0.002)
    ball = G.GeneralModel([Body(-1, (0, 0, 2), joints=[Joint(G.BALL, (0, 0, 1))], mass=1.0, inertia=(0.01, 0.01, 0.01), ipos=(0, 0, -0.5))],
                          opt=opt, plane=False)
    sim = G.GeneralSim(ball, 1, integrator="rk4")
    sim.qvel = torch.tensor([[1.5, -0.7, 0.9]], dtype=torch.float64)
    E0 = sum(G.energy(ball, sim.qpos, sim.qvel))
    for _ in range(500):
        sim.step()
    E1 = sum(G.energy(ball, sim.qpos, sim.qvel))
    assert abs(float(E1 - E0)) < 1e-6 * abs(float(E0))
    # point-mass hinge pendulum, small angle: period 2π sqrt(l / g)
    L = 0.8
    hinge = G.GeneralModel([Body(-1, (0, 0, 2), joints=[Joint(G.HINGE, (0, 1, 0))], mass=1.0, inertia=(1e-9, 1e-9, 1e-9), ipos=(0, 0, -L))],
                           opt=opt, plane=False)
    sim = G.GeneralSim(hinge, 1, integrator="rk4")
    sim.qpos[:, 0] = 0.02
    prev, crossings = float(sim.qpos[0, 0]), []
    for i in range(2200):
        sim.step()
        cur = float(sim.qpos[0, 0])
        if prev > 0 >= cur:
            crossings.append(i * opt.timestep + opt.timestep * prev / (prev - cur))
        prev = cur
    period = crossings[1] - crossings[0]
    assert abs(period - 2 * math.pi * math.sqrt(L / 9.81)) < 2e-3


def test_segment_distance_against_dense_sampling():
    g = torch.Generator().manual_seed(0)
    p1, d1, p2, d2 = (torch.randn(64, 3, generator=g, dtype=torch.float64) for _ in range(4))
    d2[:8] = d1[:8] * 0.7                                           # parallel segments
    d1[8:12] = 0                                                    # a point against a segment
    c1, c2 = G.closest_segment_points(p1, d1, p2, d2)
    s = torch.linspace(0, 1, 201, dtype=torch.float64)
    a = p1[:, None, None] + s[None, :, None, None] * d1[:, None, None]
    b = p2[:, None, None] + s[None, None, :, None] * d2[:, None, None]
    brute = (a - b).norm(dim=-1).reshape(64, -1).min(1).values
    got = (c1 - c2).norm(dim=-1)
    assert (got <= brute + 1e-9).all() and (brute - got < 2e-2).all()


@pytest.mark.parametrize("solver", ["pgs", "newton", "cg"])
def test_resting_box_sliding_friction_and_touch(solver):
    opt = Options(timestep=0.002, solref=(0.01, 1.0))
    m = _free_box(opt, z=0.05, plane=True, friction=0.5)
    sim = G.GeneralSim(m, 2, integrator="euler", solver=solver, solver_iters={"pgs": 60, "newton": 20, "cg": 60}[solver])
    sim.qvel[1, 0] = 2.0                                            # env 1 slides along x
    xs = []
    for i in range(400):
        sim.step()
        xs.append(float(sim.qvel[1, 0]))
    mass = float(m.mass[0])
    s = sim.sensors(0)
    assert abs(float(sim.qpos[0, 2]) - 0.05) < 2e-3 and float(sim.qvel[0].abs().max()) < 1e-3      # at rest on its face
    assert abs(float(s["touch"][0]) - mass * 9.81) < 0.02 * mass * 9.81                             # the plane carries the weight
    assert abs(float(s["accelerometer"][0, 2]) - 9.81) < 0.2                                        # proper acceleration at rest
    # Coulomb friction: deceleration μ g until it stops (box friction on two axes bounds it by μ g √2)
    t_stop = next(i for i, v in enumerate(xs) if v < 1e-3) * opt.timestep
    assert 2.0 / (0.5 * 9.81 * 1.45) < t_stop < 2.0 / (0.5 * 9.81) * 1.1, t_stop
    assert abs(float(sim.qvel[1, 0])) < 1e-3 and float(sim.qpos[1, 0]) > 0.25


def test_solvers_agree_on_the_contact_forces():
    opt = Options(timestep=0.002)
    bodies = [Body(-1, (0, 0, 0.1), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("capsule", (0.1, 0.3), quat=(0.70710678, 0, 0.70710678, 0))]),
              Body(-1, (0.05, 0.02, 0.28), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("sphere", (0.1,))])]
    m = G.GeneralModel(bodies, opt=opt, plane=True)
    assert len(m.pairs) == 1
    q, v = m.init_state(1)
    v[0, 8] = -0.3
    out = {}
    for solver, it in (("pgs", 400), ("newton", 30), ("cg", 200)):
        sim = G.GeneralSim(m, 1, solver=solver, solver_iters=it)
        sim.forward(q, v)
        out[solver] = (sim.last["force"].clone(), sim.last["qacc"].clone())
    assert out["newton"][0].max() > 1.0
    assert torch.allclose(out["pgs"][0], out["newton"][0], atol=2e-3 * float(out["newton"][0].abs().max()))
    assert torch.allclose(out["pgs"][1], out["newton"][1], atol=1e-2)
    assert torch.allclose(out["cg"][0], out["newton"][0], atol=2e-3 * float(out["newton"][0].abs().max()))


def test_sphere_sphere_collision_conserves_momentum_and_separates():
    opt = Options(timestep=0.001, gravity=(0, 0, 0), solref=(0.005, 0.3))
    mk = lambda x: Body(-1, (x, 0, 0), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("sphere", (0.1,), friction=0.0)])
    m = G.GeneralModel([mk(-0.3), mk(0.3)], opt=opt, plane=False)
    sim = G.GeneralSim(m, 1)
    sim.qvel[0, 0], sim.qvel[0, 6] = 1.0, -0.5
    p0 = float(sim.qvel[0, 0] + sim.qvel[0, 6])
    for _ in range(800):
        sim.step()
    assert abs(float(sim.qvel[0, 0] + sim.qvel[0, 6]) - p0) < 1e-9          # equal masses: Σ v conserved
    assert float(sim.qvel[0, 0]) < float(sim.qvel[0, 6])                       # they separated
    assert float(sim.qpos[0, 7] - sim.qpos[0, 0]) > 0.2 - 1e-3


def test_joint_limit_and_implicit_damping():
    opt = Options(timestep=0.002)
    j = Joint(G.HINGE, (0, 1, 0), range=(-0.5, 0.5), damping=0.0, name="h")
    m = G.GeneralModel([Body(-1, (0, 0, 1), joints=[j], mass=1.0, inertia=(0.01, 0.01, 0.01), ipos=(0.3, 0, 0))], opt=opt, plane=False)
    sim = G.GeneralSim(m, 1)
    lo = 0.0
    for _ in range(1500):
        sim.step()
        lo = max(lo, float(sim.qpos[0, 0]))
    assert 0.5 < lo < 0.56 and abs(float(sim.qpos[0, 0]) - 0.5) < 0.03       # gravity pushes it into the upper stop and it stays there
    # stiff damping: explicit Euler diverges at this step size, the implicit form decays
    jd = Joint(G.HINGE, (0, 1, 0), damping=40.0, name="h")
    md = G.GeneralModel([Body(-1, (0, 0, 1), joints=[jd], mass=1.0, inertia=(0.01, 0.01, 0.01))], opt=Options(timestep=0.002, gravity=(0, 0, 0)), plane=False)
    res = {}
    for integ in ("euler", "implicit"):
        s2 = G.GeneralSim(md, 1, integrator=integ)
        s2.qvel[0, 0] = 1.0
        for _ in range(50):
            s2.step()
        res[integ] = abs(float(s2.qvel[0, 0]))
    assert res["implicit"] < 1e-3 and res["euler"] > 1e3


def test_motor_and_sensors_on_a_spinning_body():
    opt = Options(timestep=0.002, gravity=(0, 0, 0))
    j = Joint(G.HINGE, (0, 0, 1), name="spin")
    m = G.GeneralModel([Body(-1, (0, 0, 0), joints=[j], mass=1.0, inertia=(0.1, 0.1, 0.2))], motors=[G.Motor("spin", gear=2.0)], opt=opt, plane=False)
    sim = G.GeneralSim(m, 1, integrator="rk4")
    for _ in range(100):
        sim.step(torch.tensor([[0.5]]))
    w = 2.0 * 0.5 / 0.2 * 0.2                                                 # τ / I · t
    s = sim.sensors(0)
    assert abs(float(sim.qvel[0, 0]) - w) < 1e-9 and abs(float(s["gyro"][0, 2]) - w) < 0.02
    assert float(s["actuatorfrc"][0, 0]) == 1.0 and s["jointpos"].shape == (1, 1)


def test_mjcf_with_free_and_ball_joints_and_boxes():
    from noeira_b200.physics.mjcf import MjcfError, from_mjcf
    xml = """<mujoco><compiler angle="radian"/><option timestep="0.002"/>
      <worldbody><geom type="plane" pos="0 0 0" size="5 5 0.1"/>
        <body name="base" pos="0 0 0.3"><freejoint name="root"/><geom type="box" size="0.2 0.1 0.05"/>
          <body name="arm" pos="0.2 0 0.05"><joint type="ball" name="shoulder"/><geom type="capsule" fromto="0 0 0 0.3 0 0" size="0.03"/>
            <body name="hand" pos="0.3 0 0"><joint type="hinge" axis="0 1 0" range="-1 1" name="wrist"/><geom type="sphere" size="0.04"/></body>
          </body></body></worldbody>
      <actuator><motor joint="wrist" gear="3"/></actuator></mujoco>"""
    m = from_mjcf(xml, general=True)
    assert (m.nb, m.nq, m.nv) == (3, 12, 10) and len(m.motors) == 1 and m.limits[0][0] == 9
    with pytest.raises(MjcfError):
        from_mjcf(xml)
    sim = G.GeneralSim(m, 2, solver="newton")
    for _ in range(300):
        sim.step(torch.tensor([[0.3], [-0.3]]))
    assert torch.isfinite(sim.qpos).all() and float(sim.qpos[:, 2].min()) > 0.03           # the box landed on the plane and stayed
    assert abs(float(sim.qpos[0, 3:7].norm()) - 1) < 1e-9


def test_box_on_box_and_sphere_on_box_rest():
    opt = Options(timestep=0.002, solref=(0.01, 1.0))
    base = Body(-1, (0, 0, 0.1), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("box", (0.3, 0.3, 0.1), density=2000.0)])
    top = Body(-1, (0.05, -0.03, 0.27), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("box", (0.1, 0.1, 0.07))])
    ball = Body(-1, (-0.15, 0.1, 0.285), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("sphere", (0.08,))])
    m = G.GeneralModel([base, top, ball], opt=opt, plane=True)
    assert len(m.pairs) == 3
    sim = G.GeneralSim(m, 1, solver="newton", solver_iters=30)
    for _ in range(500):
        sim.step()
    q = sim.qpos[0]
    assert float(sim.qvel.abs().max()) < 5e-3                                       # everything came to rest
    assert abs(float(q[2]) - 0.1) < 3e-3                                            # the base on the plane
    assert abs(float(q[7 + 2]) - 0.27) < 4e-3                                       # the small box on the base (0.2 + 0.07)
    assert abs(float(q[14 + 2]) - 0.28) < 4e-3                                      # the ball on the base (0.2 + 0.08)
    assert abs(float(q[7]) - 0.05) < 2e-3 and abs(float(q[14]) + 0.15) < 2e-3       # friction keeps them in place
    # the base feels its own weight plus the two riders from the plane
    s = sim.sensors(0)
    assert abs(float(s["touch"][0]) - float(m.mass.sum()) * 9.81) < 0.03 * float(m.mass.sum()) * 9.81
    # geometry helper: a point inside / outside a rotated box
    R = G.quat_to_mat(torch.tensor([[0.9238795, 0.0, 0.0, 0.3826834]], dtype=torch.float64))
    n, d = G._point_in_box(torch.tensor([[0.0, 0.0, 0.09]], dtype=torch.float64), torch.zeros(1, 3, dtype=torch.float64), R,
                           torch.tensor([0.3, 0.2, 0.1], dtype=torch.float64))
    assert torch.allclose(n, torch.tensor([[0.0, 0.0, 1.0]], dtype=torch.float64)) and abs(float(d) - 0.01) < 1e-9
    _, d2 = G._point_in_box(torch.tensor([[0.0, 0.0, 0.2]], dtype=torch.float64), torch.zeros(1, 3, dtype=torch.float64), R,
                            torch.tensor([0.3, 0.2, 0.1], dtype=torch.float64))
    assert float(d2) < 0


def test_operational_space_controller_reaches_a_target_against_gravity():
    opt = Options(timestep=0.002)
    link = lambda parent, pos, name: Body(parent, pos, joints=[Joint(G.HINGE, (0, 1, 0), name=name)], mass=1.0, inertia=(0.01, 0.01, 0.01),
                                          ipos=(0.15, 0, 0))
    bodies = [link(-1, (0, 0, 1.0), "j0"), link(0, (0.3, 0, 0), "j1"), link(1, (0.3, 0, 0), "j2")]
    bodies[0].joints.insert(0, Joint(G.HINGE, (0, 0, 1), name="yaw"))            # 4 dofs for a 3-D point task: one redundant
    m = G.GeneralModel(bodies, opt=opt, plane=False)
    sim = G.GeneralSim(m, 2, integrator="euler")
    sim.qpos[:, 1:] = torch.tensor([0.3, -0.6, 0.4], dtype=torch.float64)
    targets = torch.tensor([[0.45, 0.25, 1.2], [0.3, -0.3, 0.7]], dtype=torch.float64)
    for _ in range(2000):
        tau, x = G.osc_torque(m, sim.qpos, sim.qvel, body=2, point_local=(0.3, 0, 0), x_des=targets, kp=150.0, null_damping=8.0)
        sim.qfrc_applied = tau
        sim.step()
    _, x = G.osc_torque(m, sim.qpos, sim.qvel, 2, (0.3, 0, 0), targets)
    assert float((x - targets).norm(dim=-1).max()) < 5e-3, x
    assert float(sim.qvel.abs().max()) < 2e-2                                    # and it holds still there (null space damped)


def test_fixed_tendon_spring_limit_and_energy():
    opt = Options(timestep=0.001, gravity=(0, 0, 0))
    mk = lambda x, n: Body(-1, (x, 0, 0), joints=[Joint(G.SLIDE, (0, 0, 1), name=n)], mass=1.0, inertia=(0.01, 0.01, 0.01))
    td = G.Tendon({"a": 1.0, "b": -1.0}, stiffness=50.0, springlength=0.0)      # pulls the two sliders to equal heights
    m = G.GeneralModel([mk(0, "a"), mk(1, "b")], opt=opt, plane=False, tendons=[td])
    sim = G.GeneralSim(m, 1, integrator="rk4")
    sim.qpos[0, 0] = 0.2
    E0 = sum(G.energy(m, sim.qpos, sim.qvel))
    mid = []
    for _ in range(700):
        sim.step()
        mid.append(float(sim.qpos[0, 0] + sim.qpos[0, 1]))
    E1 = sum(G.energy(m, sim.qpos, sim.qvel))
    assert abs(float(E1 - E0)) < 1e-8 and max(abs(v - 0.2) for v in mid) < 1e-9       # energy and the common mode are conserved
    # relative coordinate oscillates at sqrt(2k/m): period 2π / 10
    assert abs(float(G.tendon_length(m, sim.qpos)[0, 0]) - 0.2 * __import__("math").cos(10.0 * 0.7)) < 2e-4
    # a length range acts as a stop
    td2 = G.Tendon({"a": 1.0, "b": -1.0}, range=(-0.05, 0.05))
    m2 = G.GeneralModel([mk(0, "a"), mk(1, "b")], opt=Options(timestep=0.002, gravity=(0, 0, 0)), plane=False, tendons=[td2])
    s2 = G.GeneralSim(m2, 1)
    s2.qvel[0, 0] = 0.5
    worst = 0.0
    for _ in range(400):
        s2.step()
        worst = max(worst, float(G.tendon_length(m2, s2.qpos)[0, 0]))
    # the stop absorbs most of the relative motion (a soft, critically damped constraint), momentum is shared
    assert 0.05 <= worst < 0.06 and abs(float(s2.qvel[0, 0] - s2.qvel[0, 1])) < 0.1
    assert abs(float(s2.qvel[0, 0] + s2.qvel[0, 1]) - 0.5) < 1e-9


def test_capsule_on_box_and_crossed_boxes_edge_contact():
    opt = Options(timestep=0.002, solref=(0.01, 1.0))
    base = Body(-1, (0, 0, 0.1), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("box", (0.4, 0.4, 0.1), density=3000.0)])
    # a capsule lying along x on top of the box: axis point + both ends carry it, so it neither sinks nor tips
    cap = Body(-1, (0.05, 0.0, 0.262), joints=[Joint(G.FREE, (0, 0, 1))],
               geoms=[Geom("capsule", (0.06, 0.2), quat=(0.70710678, 0, 0.70710678, 0))])
    m = G.GeneralModel([base, cap], opt=opt, plane=True)
    sim = G.GeneralSim(m, 1, solver="newton", solver_iters=30)
    for _ in range(500):
        sim.step()
    assert float(sim.qvel.abs().max()) < 5e-3
    assert abs(float(sim.qpos[0, 7 + 2]) - 0.26) < 4e-3                             # box top 0.2 + radius 0.06
    zaxis = G.quat_to_mat(sim.qpos[:, 10:14])[0, :, 2]
    assert float(zaxis[2]) > 0.9995                                                 # the body did not tip (its capsule stays level)
    # geometry: the nearest point of a segment to a box, against dense sampling
    g = torch.Generator().manual_seed(0)
    p0 = torch.randn(64, 3, generator=g, dtype=torch.float64)
    dv = torch.randn(64, 3, generator=g, dtype=torch.float64)
    cb = 0.3 * torch.randn(64, 3, generator=g, dtype=torch.float64)
    q = torch.randn(64, 4, generator=g, dtype=torch.float64)
    Rb = G.quat_to_mat(q / q.norm(dim=1, keepdim=True))
    h = torch.tensor([0.3, 0.2, 0.1], dtype=torch.float64)

    def dist_to_box(pts):
        loc = (Rb.transpose(1, 2)[:, None] @ (pts - cb[:, None])[..., None])[..., 0]
        return (loc - torch.maximum(torch.minimum(loc, h), -h)).norm(dim=-1)
    near = G._segment_point_nearest_box(p0, dv, cb, Rb, h, iters=40)
    ts = torch.linspace(0, 1, 2001, dtype=torch.float64)
    dense = dist_to_box(p0[:, None] + ts[None, :, None] * dv[:, None]).min(1).values
    assert (dist_to_box(near[:, None])[:, 0] - dense).abs().max() < 2e-3

    # two boxes crossed at 45° and tilted so that an EDGE of the upper one lies across an EDGE of the lower one
    c_a, c_b = torch.zeros(1, 3, dtype=torch.float64), torch.tensor([[0.0, 0.0, 0.27]], dtype=torch.float64)
    R_a = G.axis_angle_mat(torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64), torch.tensor([math.pi / 4], dtype=torch.float64))
    R_b = G.axis_angle_mat(torch.tensor([0.0, 1.0, 0.0], dtype=torch.float64), torch.tensor([math.pi / 4], dtype=torch.float64))
    ha = hb = torch.tensor([0.5, 0.1, 0.1], dtype=torch.float64)
    # lower box: long axis x, its upper edge along x at height 0.1·√2; upper box: long axis... rotate so its long axis is y
    R_b = G.axis_angle_mat(torch.tensor([0.0, 0.0, 1.0], dtype=torch.float64), torch.tensor([math.pi / 2], dtype=torch.float64)) @ \
        G.axis_angle_mat(torch.tensor([1.0, 0.0, 0.0], dtype=torch.float64), torch.tensor([math.pi / 4], dtype=torch.float64))
    p, n, d = G._box_box_edge_contact(c_a, R_a, ha, c_b, R_b, hb)
    want = 2 * 0.1 * math.sqrt(2) - 0.27                                            # the two ridge edges overlap by this much
    assert abs(float(d) - want) < 1e-9 and torch.allclose(n, torch.tensor([[0.0, 0.0, 1.0]], dtype=torch.float64), atol=1e-9)
    assert torch.allclose(p, torch.tensor([[0.0, 0.0, 0.135]], dtype=torch.float64), atol=1e-9)
    # no corner of either box is inside the other: the vertex-face test alone finds nothing here
    for (ci, Ri, hi, cj, Rj, hj) in ((c_a, R_a, ha, c_b, R_b, hb), (c_b, R_b, hb, c_a, R_a, ha)):
        for sx in (-1, 1):
            for sy in (-1, 1):
                for sz in (-1, 1):
                    corner = ci + (Ri @ (hi * torch.tensor([sx, sy, sz], dtype=torch.float64)))
                    assert float(G._point_in_box(corner, cj, Rj, hj)[1]) < 0
    # separated, and face-to-face stacks, give no edge contact
    assert float(G._box_box_edge_contact(c_a, R_a, ha, c_b + 0.1, R_b, hb)[2]) < 0
    eye = torch.eye(3, dtype=torch.float64)[None]
    assert float(G._box_box_edge_contact(c_a, eye, ha, torch.tensor([[0.0, 0.0, 0.19]], dtype=torch.float64), eye, hb)[2]) < 0
    # dynamics: the crossed upper box comes to rest on the ridge of the lower one (held fixed as a heavy body on the plane)
    low = Body(-1, (0, 0, 0.1 * math.sqrt(2)), quat=(math.cos(math.pi / 8), math.sin(math.pi / 8), 0, 0), joints=[],
               geoms=[Geom("box", (0.5, 0.1, 0.1))])
    qz, qx = (math.cos(math.pi / 4), 0, 0, math.sin(math.pi / 4)), (math.cos(math.pi / 8), math.sin(math.pi / 8), 0, 0)
    quat = tuple(float(v) for v in G.quat_mul(torch.tensor([qz], dtype=torch.float64), torch.tensor([qx], dtype=torch.float64))[0])
    up = Body(-1, (0, 0, 0.1 * math.sqrt(2) + 0.28), quat=quat, joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("box", (0.5, 0.1, 0.1))])
    m2 = G.GeneralModel([low, up], opt=opt, plane=False)
    sim2 = G.GeneralSim(m2, 1, solver="newton", solver_iters=30)
    for _ in range(150):
        sim2.step()
    z = float(sim2.qpos[0, 2])
    assert 0.1 * math.sqrt(2) + 0.27 < z < 0.1 * math.sqrt(2) + 0.285 and abs(float(sim2.qvel[0, 2])) < 0.05    # caught by the edge contact


def test_disc_qp_against_a_polar_grid():
    g = torch.Generator().manual_seed(0)
    M = torch.randn(32, 2, 2, generator=g, dtype=torch.float64)
    Q = M @ M.transpose(1, 2) + 0.1 * torch.eye(2, dtype=torch.float64)
    c = torch.randn(32, 2, generator=g, dtype=torch.float64) * 3
    r = torch.rand(32, generator=g, dtype=torch.float64) * 1.5
    r[0] = 0.0
    x = G._disc_qp(Q, c, r)
    obj = lambda v: 0.5 * (v[:, None] @ Q @ v[:, :, None])[:, 0, 0] + (c * v).sum(1)
    assert (x.norm(dim=1) <= r + 1e-9).all() and float(x[0].abs().max()) == 0.0
    th = torch.linspace(0, 2 * math.pi, 361, dtype=torch.float64)
    best = torch.full((32,), float("inf"), dtype=torch.float64)
    for k in torch.linspace(0, 1, 101, dtype=torch.float64):
        cand = torch.stack([torch.cos(th), torch.sin(th)], 1)[None] * (k * r)[:, None, None]      # [32, 361, 2]
        val = 0.5 * ((cand @ Q) * cand).sum(-1) + (cand * c[:, None]).sum(-1)
        best = torch.minimum(best, val.min(1).values)
    assert (obj(x) <= best + 1e-9).all() and (obj(x) >= best - 1e-2).all()
    inside = torch.linalg.solve(Q, -c[:, :, None])[..., 0]
    free = inside.norm(dim=1) <= r
    assert free.any() and torch.allclose(x[free], inside[free], atol=1e-10)


def test_elliptic_cone_is_isotropic_and_noslip_removes_creep():
    opt = Options(timestep=0.002, solref=(0.01, 1.0))
    # slide the same box along a tangent axis and along the diagonal between the two: the circular cone decelerates both at
    # μ g, the pyramid's diagonal gets up to √2 μ g
    stop = {}
    for cone in ("pyramidal", "elliptic"):
        m = _free_box(opt, z=0.05, plane=True, friction=0.5)
        sim = G.GeneralSim(m, 2, integrator="euler", solver="pgs", solver_iters=25, cone=cone)
        sim.qvel[0, 0] = 2.0
        sim.qvel[1, 0] = sim.qvel[1, 1] = 2.0 / math.sqrt(2)
        t = [None, None]
        for i in range(250):
            sim.step()
            sp = sim.qvel[:, :2].norm(dim=1)
            for e in range(2):
                if t[e] is None and float(sp[e]) < 1e-3:
                    t[e] = i * opt.timestep
        stop[cone] = t
    ideal = 2.0 / (0.5 * 9.81)
    assert all(abs(v - ideal) < 0.04 * ideal for v in stop["elliptic"]), stop        # the block solve is isotropic
    assert abs(stop["elliptic"][0] - stop["elliptic"][1]) < 0.01 * ideal
    assert min(stop["pyramidal"]) < 0.85 * ideal                                    # the box bound brakes one of them harder
    with pytest.raises(ValueError):
        G.GeneralSim(m, 1, solver="newton", cone="elliptic")
    # a box on a slope below the friction angle creeps with soft friction rows and holds with the no-slip sweeps
    slope = math.radians(15.0)
    drift = {}
    for ns in (0, 10):
        o2 = Options(timestep=0.002, solref=(0.02, 1.0), gravity=(9.81 * math.sin(slope), 0.0, -9.81 * math.cos(slope)))
        m = _free_box(o2, z=0.05, plane=True, friction=0.8)
        sim = G.GeneralSim(m, 1, solver="pgs", solver_iters=20, noslip_iters=ns)
        for _ in range(150):
            sim.step()
        drift[ns] = abs(float(sim.qpos[0, 0]))
    assert drift[10] < 0.2 * drift[0] and drift[10] < 1e-3, drift


def test_constraint_islands_split_independent_bodies_and_give_the_same_forces():
    opt = Options(timestep=0.002, solref=(0.01, 1.0))
    bodies = [Body(-1, (0, 0, 0.049), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("box", (0.2, 0.1, 0.05))]),
              Body(-1, (3.0, 0, 0.099), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("sphere", (0.1,))]),
              Body(-1, (3.0, 0, 0.29), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("sphere", (0.1,))])]      # stacked on the second
    m = G.GeneralModel(bodies, opt=opt, plane=True)
    qpos, qvel = m.init_state(2)
    qvel[1, 0] = 0.5
    k = G.kinematics(m, qpos, qvel)
    con = G.collide(m, k)
    rows = G.constraint_rows(m, k, qpos, qvel, con)
    M = G.mass_matrix(m, k)
    isl = G.constraint_islands(M, rows)
    active = [i for i in range(rows.aref.shape[1]) if bool(rows.active[:, i].any())]
    big = [g for g in isl if len(g) > 1 and any(i in active for i in g)]
    bodies_of = [{rows.body[i] for i in g if i in active} for g in big]
    assert any(b == {0} for b in bodies_of) and any({1, 2} <= b for b in bodies_of)      # the box alone; the two balls together
    assert not any(0 in b and (1 in b or 2 in b) for b in bodies_of)
    qacc0 = torch.linalg.solve(M, (-G.bias_force(m, k, qvel))[:, :, None])[..., 0]
    for solver, iters in (("newton", 30), ("pgs", 200)):
        f1, a1 = G.solve_constraints(m, M, qacc0, rows, solver, iters)
        f2, a2 = G.solve_constraints(m, M, qacc0, rows, solver, iters, islands=True)
        assert (f1 - f2).abs().max() < 1e-6 * max(1.0, float(f1.abs().max())) and (a1 - a2).abs().max() < 1e-6
    sim = G.GeneralSim(m, 1, solver="newton", solver_iters=20, islands=True)
    for _ in range(100):
        sim.step()
    assert abs(float(sim.qpos[0, 2]) - 0.05) < 2e-3 and abs(float(sim.qpos[0, 14 + 2]) - 0.3) < 6e-3
