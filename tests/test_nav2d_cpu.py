"""Grid navigation: batched distance fields agree with A*, paths avoid obstacles and corners, shortcutting keeps visibility."""
import math

import torch


def test_distance_field_matches_astar_and_paths_are_valid():
    from noeira_b200.planners.nav2d import astar, descend, distance_field, shortcut
    g = torch.Generator().manual_seed(0)
    B, H, W = 4, 18, 24
    occ = torch.rand(B, H, W, generator=g) < 0.25
    occ[:, 0, 0] = False
    occ[:, H - 1, W - 1] = False
    occ[3] = False
    occ[3, 3:15, 12] = True                                            # one wall with a gap at the top and bottom
    goals = torch.tensor([[H - 1, W - 1]] * B)
    field = distance_field(occ, goals)
    assert field.shape == (B, H, W) and (field[occ] == float("inf")).all() and (field[:, H - 1, W - 1] == 0).all()
    for b in range(B):
        path, cost = astar(occ[b], (0, 0), (H - 1, W - 1))
        f0 = float(field[b, 0, 0])
        if not path:
            assert math.isinf(f0)
            continue
        assert abs(cost - f0) < 1e-4                                      # value iteration is exact on the same move set
        p2 = descend(field[b], (0, 0), occ[b])
        assert p2[0] == (0, 0) and p2[-1] == (H - 1, W - 1)
        length = sum(math.hypot(a[0] - c[0], a[1] - c[1]) for a, c in zip(p2, p2[1:]))
        assert abs(length - cost) < 1e-4 and not any(bool(occ[b, r, c]) for r, c in p2)
        for (r0, c0), (r1, c1) in zip(p2, p2[1:]):                        # no corner cutting
            if r0 != r1 and c0 != c1:
                assert not bool(occ[b, r1, c0]) and not bool(occ[b, r0, c1])
        s = shortcut(occ[b], path)
        assert s[0] == path[0] and s[-1] == path[-1] and len(s) <= len(path)
    wall_path, _ = astar(occ[3], (8, 2), (8, 22))
    short = shortcut(occ[3], wall_path)
    assert 3 <= len(short) <= 5 and all(not bool(occ[3, r, c]) for r, c in short)    # around the wall with a few way-points
    blocked = torch.zeros(1, 5, 5, dtype=torch.bool)
    blocked[0, 2, :] = True
    assert math.isinf(float(distance_field(blocked, torch.tensor([[4, 4]]))[0, 0, 0])) and astar(blocked[0], (0, 0), (4, 4))[0] == []
