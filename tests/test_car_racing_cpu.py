"""Car racing on CPU: track geometry, tire-model behaviour, rewards, the camera and the scripted driver."""
import math

import numpy as np
import torch

from noeira_b200.envs.car_racing import (CarRacingDiscreteEnv, CarRacingEnv, CarRacingPixelEnv, make_track, scripted_driver)


def test_track_is_a_closed_loop_of_even_tiles():
    tr = make_track(np.random.default_rng(0), tiles=256)
    seg = np.linalg.norm(np.roll(tr, -1, 0) - tr, axis=1)
    assert tr.shape == (256, 2) and seg.max() < 1.6 * seg.min()           # equal arc length up to chord error
    ang = np.unwrap(np.arctan2(tr[:, 1], tr[:, 0]))
    assert abs(ang[-1] - ang[0]) > 1.7 * math.pi                           # once around the origin
    assert np.abs(tr).max() < 2000 / 6


def test_gas_accelerates_along_the_heading_and_steering_turns_the_right_way():
    env = CarRacingEnv(4, seed=1)
    env.reset_batch()
    s0 = env.state.clone()
    fwd0, side0 = env._frames(s0)
    a = torch.tensor([[0.0, 1.0, 0.0], [1.0, 1.0, 0.0], [-1.0, 1.0, 0.0], [0.0, 0.0, 0.0]])
    for _ in range(60):
        env.step_batch(a, auto_reset=False)
    s = env.state
    d = s[:, 0:2] - s0[:, 0:2]
    along, across = (d * fwd0).sum(1), (d * side0).sum(1)
    assert along[0] > 5.0 and abs(across[0]) < 0.2 * along[0]              # straight ahead
    assert across[1] > 1.0 and across[2] < -1.0                             # +steer = right, −steer = left
    assert s[1, 2] < s0[1, 2] and s[2, 2] > s0[2, 2]                        # right turn = clockwise
    assert d[3].abs().max() < 1e-4                                         # no input, no motion
    # braking stops the car
    for _ in range(80):
        env.step_batch(torch.tensor([[0.0, 0.0, 1.0]]).expand(4, 3), auto_reset=False)
    assert torch.linalg.vector_norm(env.state[:, 3:5], dim=1).max() < 0.5


def test_grass_has_less_grip_than_road():
    env = CarRacingEnv(2, seed=2)
    env.reset_batch()
    s = env.state.clone()
    fwd, side = env._frames(s)
    s[:, 3:5] = side * 12.0                                                 # sliding sideways at 12 m/s
    s[1, 0:2] = torch.tensor([330.0, 330.0])                                # far from any track: grass
    s2, _, _ = env._dynamics_tensor(s, torch.zeros(2, 3))
    lost = 12.0 - (s2[:, 3:5] * side).sum(1)
    assert lost[0] > 0 and abs(lost[1] / lost[0] - 0.6) < 0.02


def test_reward_counts_each_tile_once_and_leaving_the_field_ends_the_episode():
    env = CarRacingEnv(1, seed=3, tiles=128)
    env.reset_batch()
    total, tiles_seen = 0.0, 0
    for _ in range(200):
        _, r, done, _ = env.step_batch(scripted_driver(env), auto_reset=False)
        total += float(r)
    visited = int(env.state[0, 13])
    assert visited > 5 and abs(total - (-0.1 * 200 + visited * 1000.0 / 128)) < 1e-2
    assert int(env.state[0, 16:].sum()) == visited
    s = env.state.clone()
    s[0, 0] = env.params["playfield"] + 1.0
    _, r, term = env._dynamics_tensor(s, torch.zeros(1, 3))
    assert float(r) == -100.0 and bool(term)


def test_scripted_driver_completes_most_of_a_lap():
    env = CarRacingEnv(8, seed=4, n_tracks=4)
    env.reset_batch()
    best = torch.zeros(8)
    for _ in range(1000):
        _, _, done, _ = env.step_batch(scripted_driver(env, target_speed=50.0), auto_reset=False)
        best = torch.maximum(best, env.visited_fraction())
    assert best.min() > 0.9, best          # every lane all but completes its lap


def test_camera_shows_road_ahead_and_the_car():
    env = CarRacingEnv(3, seed=5, lookahead=4)
    obs = env.reset_batch()
    assert obs.shape == (3, 13 + 8)
    assert (obs[:, 14::2] > 0).all()                                        # look-ahead points lie ahead of the car
    img = env.render(64)
    assert img.shape == (3, 64, 64) and set(torch.unique(img).tolist()) <= {0.30000001192092896, 0.699999988079071, 1.0}
    assert (img[:, 48, 32] == 1.0).all()                                    # the car
    assert (img[:, 36:44, 32] == 0.7).all()                                 # road straight ahead of it
    assert (img == 0.3).float().mean() > 0.2                                # grass beside the road


def test_pixel_and_discrete_variants():
    env = CarRacingPixelEnv(2, seed=6, res=48)
    obs = env.reset_batch()
    assert obs.shape == (2, 4, 48, 48) and torch.equal(obs[:, 0], obs[:, 3])
    first = obs[:, 3].clone()
    for _ in range(30):
        obs, r, done, term = env.step_batch(torch.tensor([3, 3]))
    assert torch.equal(env.next_obs, obs)                                   # nothing finished: successor frames = new frames
    assert not torch.equal(obs[:, 3], first)
    denv = CarRacingDiscreteEnv(2, seed=6)
    denv.reset_batch()
    o, r, d, t = denv.step_batch(torch.tensor([3, 4]))
    assert o.shape == (2, 13) and denv.n_actions == 5
