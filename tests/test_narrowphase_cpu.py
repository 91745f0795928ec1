"""GJK / EPA against closed forms and brute force, mesh mass properties, terrain, sweep and prune, and the engine with
convex meshes, a height field and the broad phase."""
import math

import numpy as np
import torch

from noeira_b200.physics import general as G
from noeira_b200.physics.model import Body, Geom, Joint, Options
from noeira_b200.physics.narrowphase import HeightField, contact_manifold, gjk_epa, mesh_mass_inertia, sap_overlaps

CUBE = np.array([[sx, sy, sz] for sx in (-1, 1) for sy in (-1, 1) for sz in (-1, 1)], float)


def _rot(rng):
    q = rng.normal(size=4)
    q /= np.linalg.norm(q)
    return G.quat_to_mat(torch.tensor(q[None])).numpy()[0]


def test_gjk_distance_matches_closed_forms_and_sampling():
    # sphere-sphere and capsule-capsule through point and segment cores
    d, n, pa, pb = gjk_epa(np.zeros((1, 3)), np.array([[3.0, 0, 0]]), 1.0, 0.5)
    assert abs(d - 1.5) < 1e-12 and np.allclose(n, [1, 0, 0]) and np.allclose(pa, [1, 0, 0]) and np.allclose(pb, [2.5, 0, 0])
    d, n, _, _ = gjk_epa(np.array([[-1.0, 0, 0], [1, 0, 0]]), np.array([[0, -1.0, 0.7], [0, 1, 0.7]]), 0.2, 0.1)
    assert abs(d - 0.4) < 1e-12 and np.allclose(n, [0, 0, 1])
    # random boxes: against a dense search over the second box's surface points for the distance to the first
    rng = np.random.default_rng(0)
    for _ in range(20):
        ha, hb = rng.uniform(0.2, 0.6, 3), rng.uniform(0.2, 0.6, 3)
        Ra, Rb = _rot(rng), _rot(rng)
        cb = rng.normal(size=3) * 1.2
        cb *= max(1.0, 2.2 / np.linalg.norm(cb))             # beyond the sum of the half diagonals: surely separated
        va, vb = (CUBE * ha) @ Ra.T, (CUBE * hb) @ Rb.T + cb
        d, n, pa, pb = gjk_epa(va, vb)
        assert d > 0 and abs(np.linalg.norm(pb - pa) - d) < 1e-9 and np.allclose((pb - pa) / d, n, atol=1e-7)
        # the witness points lie on the boxes, and no vertex of either box crosses the separating slab
        for pt, R, h, c in ((pa, Ra, ha, np.zeros(3)), (pb, Rb, hb, cb)):
            assert (np.abs((pt - c) @ R) <= h + 1e-8).all()
        assert ((va - pa) @ n).max() < 1e-8 and ((vb - pb) @ n).min() > -1e-8


def test_epa_depth_of_overlapping_boxes_and_mesh_against_sphere():
    va = CUBE * 0.5
    for shift, want_n, want_d in (((0.8, 0.1, 0.05), (1, 0, 0), 0.2), ((0.1, -0.7, 0.0), (0, -1, 0), 0.3), ((0, 0.1, 0.9), (0, 0, 1), 0.1)):
        d, n, pa, pb = gjk_epa(va, CUBE * 0.5 + np.array(shift))
        assert abs(d + want_d) < 1e-8 and np.allclose(n, want_n, atol=1e-7), (shift, d, n)
        assert abs((pa - pb) @ n - want_d) < 1e-8
    # rotated overlap: the depth is the least translation that separates (checked by separating and re-testing)
    rng = np.random.default_rng(1)
    for _ in range(10):
        Rb = _rot(rng)
        vb = (CUBE * rng.uniform(0.3, 0.6, 3)) @ Rb.T + rng.normal(size=3) * 0.25
        d, n, _, _ = gjk_epa(va, vb)
        assert d < 0
        assert gjk_epa(va, vb + n * (-d + 1e-6))[0] > 0 and gjk_epa(va, vb + n * (-d - 1e-3))[0] < 0
    # a sphere sunk into a tetrahedron's face
    tet = np.array([[0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1]], float)
    d, n, _, _ = gjk_epa(tet, np.array([[0.25, 0.25, -0.1]]), 0.0, 0.3)
    assert abs(d + 0.2) < 1e-9 and np.allclose(n, [0, 0, -1])


def test_manifold_of_stacked_boxes_has_a_supporting_polygon():
    cons = contact_manifold(CUBE * 0.5, CUBE * np.array([0.3, 0.3, 0.2]) + np.array([0.0, 0, 0.69]), margin=1e-3)
    assert len(cons) >= 4 and all(abs(c[2] - 0.01) < 2e-2 for c in cons) and all(np.allclose(c[1], [0, 0, 1], atol=1e-6) for c in cons)
    pts = np.array([c[0] for c in cons])
    assert np.ptp(pts[:, 0]) > 0.4 and np.ptp(pts[:, 1]) > 0.4                     # spread over the small box's footprint


def test_mesh_mass_properties():
    m, I, c = mesh_mass_inertia(CUBE * np.array([0.2, 0.1, 0.05]) + np.array([1.0, 2.0, 3.0]), 1000.0)
    mb, Ib = G.box_mass_inertia((0.2, 0.1, 0.05), 1000.0)
    assert abs(m - mb) < 1e-9 and np.allclose(I, Ib, rtol=1e-9) and np.allclose(c, [1, 2, 3])
    tet = np.array([[0, 0, 0], [1, 0, 0], [0, 1, 0], [0, 0, 1]], float)
    m, I, c = mesh_mass_inertia(tet, 6.0)
    assert abs(m - 1.0) < 1e-12 and np.allclose(c, [0.25, 0.25, 0.25]) and np.allclose(I, [3 / 40] * 3)


def test_height_field_and_sweep_and_prune():
    xs = np.linspace(-2, 2, 41)
    hf = HeightField(0.3 * xs[None, :] + 0.0 * xs[:, None], 2.0, 2.0)             # a ramp of slope 0.3 along x
    h, n = hf.sample(torch.tensor([0.5, -1.0], dtype=torch.float64), torch.tensor([0.3, 0.0], dtype=torch.float64))
    assert torch.allclose(h, torch.tensor([0.15, -0.3], dtype=torch.float64), atol=1e-12)
    want = torch.tensor([-0.3, 0.0, 1.0], dtype=torch.float64) / math.sqrt(1.09)
    assert torch.allclose(n, want.expand(2, 3), atol=1e-12)
    p, nn, d = hf.contact(torch.tensor([[0.0, 0.0, 0.1]], dtype=torch.float64), 0.2)
    assert abs(float(d) - (0.2 - 0.1 / math.sqrt(1.09))) < 1e-12                    # exact distance to the plane of the ramp
    g = torch.Generator().manual_seed(0)
    lo = torch.rand(3, 24, 3, generator=g, dtype=torch.float64) * 10
    hi = lo + torch.rand(3, 24, 3, generator=g, dtype=torch.float64) * 1.5
    pairs = [(i, j) for i in range(24) for j in range(i + 1, 24)]
    brute = [bool(((lo[:, i] <= hi[:, j]) & (lo[:, j] <= hi[:, i])).all(-1).any()) for i, j in pairs]
    assert sap_overlaps(lo, hi, pairs) == brute and 0 < sum(brute) < len(pairs) // 3


def test_engine_with_a_convex_mesh_on_terrain_and_on_a_box():
    opt = Options(timestep=0.002, solref=(0.01, 1.0))
    # an octahedron-like gem dropped on a box that lies on the plane; the broad phase prunes nothing it should keep
    gem = [[0.12, 0, 0], [-0.12, 0, 0], [0, 0.12, 0], [0, -0.12, 0], [0.08, 0.08, 0.1], [-0.08, 0.08, 0.1], [0.08, -0.08, 0.1],
           [-0.08, -0.08, 0.1], [0.08, 0.08, -0.1], [-0.08, 0.08, -0.1], [0.08, -0.08, -0.1], [-0.08, -0.08, -0.1]]
    base = Body(-1, (0, 0, 0.1), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("box", (0.4, 0.4, 0.1), density=3000.0)])
    rock = Body(-1, (0.05, 0.02, 0.32), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("mesh", (0.0,), vertices=gem)])
    far = Body(-1, (5.0, 5.0, 0.2), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("sphere", (0.2,))])
    m = G.GeneralModel([base, rock, far], opt=opt, plane=True, broadphase=True)
    sim = G.GeneralSim(m, 2, solver="newton", solver_iters=30)
    for _ in range(300):
        sim.step()
    assert float(sim.qvel.abs().max()) < 2e-2
    assert abs(float(sim.qpos[0, 7 + 2]) - 0.3) < 5e-3                              # flat facets: rests 0.1 above the box top
    assert abs(float(sim.qpos[0, 14 + 2]) - 0.2) < 3e-3
    # a ball rolls down a ramp of terrain: it accelerates along −x at (5/7) g sin θ cos θ (rolling without slipping)
    xs = np.linspace(-4, 4, 81)
    hf = HeightField(0.2 * xs[None, :] + 0.0 * xs[:, None], 4.0, 4.0)
    ball = Body(-1, (1.0, 0, 0.2 + 0.1 * math.sqrt(1.04) + 1e-3), joints=[Joint(G.FREE, (0, 0, 1))], geoms=[Geom("sphere", (0.1,))])
    m2 = G.GeneralModel([ball], opt=opt, plane=False, hfield=hf)
    sim2 = G.GeneralSim(m2, 1, solver="newton", solver_iters=30)
    for _ in range(250):
        sim2.step()
    th = math.atan(0.2)
    want_vx = -(5.0 / 7.0) * 9.81 * math.sin(th) * math.cos(th) * 0.5
    assert abs(float(sim2.qvel[0, 0]) - want_vx) < 0.06 * abs(want_vx), (float(sim2.qvel[0, 0]), want_vx)
    h_now, _ = hf.sample(sim2.qpos[:, 0], sim2.qpos[:, 1])
    assert abs(float(sim2.qpos[0, 2] - h_now) - 0.1 * math.sqrt(1.04)) < 3e-3       # still on the surface
