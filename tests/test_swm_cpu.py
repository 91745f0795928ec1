"""Sheaf world model: O(d) algebra, Procrustes by polar iteration, holonomy classes of the Möbius ring and its orientable
twin from noisy observation pairs, the sheaf Laplacian's spectrum, Dirichlet inference, confidences and the planner."""
import math

import torch

from noeira_b200.experimental.swm import (DT, MobiusRing, PlaceGraph, cayley, dirichlet_energy, expm_skew, fit_ring,
                                          gnc_confidence, householder, plan_double_cover, polar_orthogonal, procrustes,
                                          sheaf_inference, sheaf_laplacian, skew_from_vector, transported_fraction)


def test_orthogonal_group_maps():
    g = torch.Generator().manual_seed(0)
    for d in (2, 3, 5):
        a = skew_from_vector(torch.randn(d * (d - 1) // 2, generator=g, dtype=DT), d)
        eye = torch.eye(d, dtype=DT)
        for q in (cayley(a), expm_skew(a)):
            assert (q @ q.T - eye).abs().max() < 1e-12 and abs(float(torch.linalg.det(q)) - 1) < 1e-12
        h = householder(torch.randn(d, generator=g, dtype=DT))
        assert (h @ h - eye).abs().max() < 1e-12 and abs(float(torch.linalg.det(h)) + 1) < 1e-12
        # the cocycle loss is blind to reflections: ‖H − I‖² = 4 for every one of them
        assert abs(float((h - eye).pow(2).sum()) - 4.0) < 1e-12


def test_procrustes_matches_the_svd_solution_and_keeps_reflections():
    g = torch.Generator().manual_seed(1)
    for d, reflect in ((2, False), (3, True), (4, True)):
        r_true = expm_skew(skew_from_vector(torch.randn(d * (d - 1) // 2, generator=g, dtype=DT), d))
        if reflect:
            r_true = householder(torch.randn(d, generator=g, dtype=DT)) @ r_true
        x = torch.randn(200, d, generator=g, dtype=DT)
        y = x @ r_true.T + 0.01 * torch.randn(200, d, generator=g, dtype=DT)
        r, res = procrustes(x, y)
        u, _, vt = torch.linalg.svd(y.T @ x)
        assert (r - u @ vt).abs().max() < 1e-12                                # the polar factor IS U Vᵀ
        assert (r - r_true).abs().max() < 5e-3 and res < 0.03
        assert float(torch.linalg.det(r)) * float(torch.linalg.det(r_true)) > 0
    m = torch.randn(4, 4, generator=g, dtype=DT)
    q = polar_orthogonal(m)
    assert (q @ q.T - torch.eye(4, dtype=DT)).abs().max() < 1e-12


def test_holonomy_reads_the_twist_in_every_seed_and_never_invents_one():
    for seed in range(12):
        for d in (2, 3):
            for twist in (True, False):
                world = MobiusRing(n=10, d=d, twist=twist, noise=0.02, seed=seed)
                graph = fit_ring(world, samples=30)
                cycles = graph.fundamental_cycles()
                assert len(cycles) == 1 and cycles[0][0] == cycles[0][-1] and len(cycles[0]) == 11
                c = graph.classify_cycle(cycles[0])
                assert c["det"] == (-1.0 if twist else 1.0), (seed, d, twist)
                assert c["residual"] < 10 * 0.02 * 3                            # every edge is locally consistent
    # the frame channel is transported, the texture channel is not
    world = MobiusRing(n=10, d=2, twist=True, noise=0.02, seed=3)
    a, b = world.sample_edge(4, 200)
    assert transported_fraction(a, b, (0, 1)) > 0.98 and transported_fraction(a, b, (2, 3)) < 0.1


def test_sheaf_laplacian_spectrum_of_the_ring():
    n = 16
    for twist, want in ((True, 2 * (1 - math.cos(math.pi / n))), (False, 0.0)):
        g = PlaceGraph(n, 1)
        for i in range(n):
            g.add_edge(i, (i + 1) % n, torch.tensor([[-1.0 if (twist and i == n - 1) else 1.0]], dtype=DT))
        lam = torch.linalg.eigvalsh(sheaf_laplacian(g))
        assert abs(float(lam[0]) - want) < 1e-12                                 # no global section on the twisted ring
    # the quadratic form of L is the Dirichlet energy
    world = MobiusRing(n=6, d=3, seed=0)
    graph = fit_ring(world, 20)
    x = torch.randn(6, 3, dtype=DT)
    assert abs(float(x.reshape(-1) @ sheaf_laplacian(graph) @ x.reshape(-1)) - float(dirichlet_energy(graph, x))) < 1e-10


def test_inference_extends_observations_along_the_transports():
    world = MobiusRing(n=8, d=2, twist=False, noise=0.0, seed=2)
    graph = fit_ring(world, 10)
    lm = torch.tensor([0.7, -0.2], dtype=DT)
    truth = torch.stack([world.frames[i] @ lm for i in range(8)])
    exact = sheaf_inference(graph, {0: truth[0]})
    assert (exact - truth).abs().max() < 1e-9 and float(dirichlet_energy(graph, exact)) < 1e-16
    slow = sheaf_inference(graph, {0: truth[0], 4: truth[4]}, iters=400)
    assert (slow - truth).abs().max() < 1e-3
    # on the twisted ring no section fits: the energy stays positive and spreads over the edges
    mob = fit_ring(MobiusRing(n=8, d=2, twist=True, noise=0.0, seed=2), 10)
    sec = sheaf_inference(mob, {0: truth[0]})
    assert float(dirichlet_energy(mob, sec)) > 1e-3


def test_confidences_and_the_double_cover_planner():
    w = gnc_confidence([0.01, 0.1, 1.0], c=0.1)
    assert w[0] > 0.95 and abs(w[1] - 0.25) < 1e-12 and w[2] < 0.001
    mob = fit_ring(MobiusRing(n=8, d=2, twist=True, noise=0.01, seed=1), 20)
    same = plan_double_cover(mob, 0, 3, goal_parity=0)
    flipped = plan_double_cover(mob, 0, 3, goal_parity=1)
    assert same == [0, 1, 2, 3] and flipped == [0, 7, 6, 5, 4, 3]           # the long way round crosses the seam
    lap = plan_double_cover(mob, 0, 0, goal_parity=1)
    assert lap is not None and len(lap) == 9                                   # one full lap returns mirrored
    ring = fit_ring(MobiusRing(n=8, d=2, twist=False, noise=0.01, seed=1), 20)
    assert plan_double_cover(ring, 0, 3, goal_parity=1) is None                 # an orientable world cannot flip
