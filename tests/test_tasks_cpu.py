"""Task layer: documents, goal language, placement sampling, the family environment and a short SAC family run."""
import math

import pytest
import torch

FAMILY = """schema_version=1
name=tabletop
base=scene.xml
horizon=60
control_freq=20
slot=brick:free:assets/brick.xml
slot=cube:free:assets/cube.xml
slot=box:free:assets/box.xml
slot=table:static:assets/table.xml:0.0,0.0,0.0
region=table_top:site:table:-0.2,-0.2,0.2,0.2:0.12
region=left_half:site:table:-0.2,-0.2,0.0,0.2:0.12
region=box_inside:box:box:-0.04,-0.04,0.04,0.04:0.05
"""

PICK = """schema_version=1
name=brick_in_box
family=tabletop
language=put the brick in the box
active=brick
active=box
active=table
init=brick@left_half:yaw:sep=0.08
init=box@table_top
goal=In(brick, box_inside)
"""

STACK = """schema_version=1
name=stack
family=tabletop
language=stack the cube on the brick
active=brick
active=cube
active=table
init=brick@table_top
init=cube@table_top:sep=0.1
goal=And(On(cube, brick), Not(Near(gripper, cube, 0.05)))
"""


def _family():
    from noeira_b200.tasks import parse_family
    f = parse_family(FAMILY)
    f.slots[f.slot_index("brick")].set_geom(-0.015, 0.015, 0.02)
    f.slots[f.slot_index("cube")].set_geom(-0.02, 0.02, 0.025)
    f.slots[f.slot_index("box")].set_geom(-0.01, 0.03, 0.06)
    f.slots[f.slot_index("table")].set_geom(0.0, 0.0, 0.3)
    return f


def test_documents_round_trip_and_refuse_unknown_keys():
    from noeira_b200.tasks import parse_family, parse_task, validate_task_against_family
    f = parse_family(FAMILY)
    assert parse_family(f.to_text()).to_text() == f.to_text()
    t = parse_task(PICK)
    assert parse_task(t.to_text()).to_text() == t.to_text()
    assert t.inits[0].yaw and t.inits[0].sep_mm == 80 and not t.inits[1].yaw
    validate_task_against_family(t, f)
    with pytest.raises(ValueError, match="unknown key"):
        parse_task(PICK + "gaol=In(brick, box_inside)\n")
    with pytest.raises(ValueError, match="static slot"):
        parse_family(FAMILY.replace("slot=table:static:assets/table.xml:0.0,0.0,0.0", "slot=table:static:assets/table.xml"))
    with pytest.raises(ValueError, match="must not carry a pose"):
        parse_family(FAMILY.replace("slot=brick:free:assets/brick.xml", "slot=brick:free:assets/brick.xml:0,0,0"))
    with pytest.raises(ValueError, match="has no init"):
        validate_task_against_family(parse_task(PICK.replace("init=box@table_top\n", "")), f)
    with pytest.raises(ValueError, match="missing goal"):
        parse_task(PICK.replace("goal=In(brick, box_inside)\n", ""))


def test_goal_language_parse_bind_evaluate():
    from noeira_b200.tasks import GoalState, bind_goal, evaluate, family_tables, parse_goal, require_evaluable
    from noeira_b200.tasks.predicates import OP_AND, OP_IN, OP_NOT, OP_ON_BODY, OP_UPRIGHT
    f = _family()
    g = parse_goal("And(In(brick, box_inside), Not(Upright(cube, 0.95)), On(cube, brick))")
    assert g.describe() == "And(In(brick, box_inside), Not(Upright(cube, 0.95)), On(cube, brick))"
    bg = bind_goal(g, f)
    assert bg.op == [OP_IN, OP_UPRIGHT, OP_NOT, OP_ON_BODY, OP_AND] and bg.a[-1] == 3
    with pytest.raises(ValueError, match="unknown predicate"):
        parse_goal("Inside(brick, box)")
    with pytest.raises(KeyError):
        bind_goal(parse_goal("In(brick, nowhere)"), f)
    with pytest.raises(ValueError, match="contact"):
        require_evaluable(bind_goal(parse_goal("Touching(brick, cube)"), f))
    rect, geom = family_tables(f, "cpu")
    S = len(f.slots)
    pos = torch.zeros(2, S, 3)
    quat = torch.zeros(2, S, 4); quat[..., 0] = 1
    bi, ci, xi = f.slot_index("brick"), f.slot_index("cube"), f.slot_index("box")
    pos[:, xi] = torch.tensor([0.1, 0.1, 0.01])
    site = torch.zeros(2, len(f.regions), 3)
    site[:, f.region_index("box_inside")] = pos[:, xi] + torch.tensor([0, 0, 0.03])
    pos[0, bi] = torch.tensor([0.11, 0.09, 0.03])     # env 0: brick in the box
    pos[1, bi] = torch.tensor([-0.1, 0.0, 0.025])     # env 1: brick away
    pos[:, ci] = pos[:, bi] + torch.tensor([0.0, 0.0, 0.045])   # cube resting on the brick
    tilt = math.radians(40)
    quat[:, ci] = torch.tensor([math.cos(tilt / 2), math.sin(tilt / 2), 0, 0])
    ok, dist = evaluate(bg, GoalState(pos, quat, site, rect, geom))
    assert ok.tolist() == [True, False]
    assert dist[0].item() == 0.0 and dist[1].item() > 0.1


def test_sampler_separation_stack_and_table():
    from noeira_b200.tasks import InitTable, parse_task, sample_placements
    f = _family()
    sites = {r.name: torch.tensor([0.0, 0.0, 0.0]) for r in f.regions}
    t = parse_task(PICK)
    pl = sample_placements(t, f, sites, 512, torch.Generator().manual_seed(0))
    assert bool(pl.ok.all())
    bi, xi = f.slot_index("brick"), f.slot_index("box")
    d = torch.linalg.vector_norm(pl.pos[:, bi, :2] - pl.pos[:, xi, :2], dim=-1)
    assert d.min().item() >= 0.08 - 1e-6                       # sep = max(r_i + r_j = 0.08, sep 0.08)
    assert pl.pos[:, bi, 0].max().item() <= 0.0 + 1e-6         # left half
    assert abs(pl.pos[0, bi, 2].item() - (0.0 + 0.01 + 0.015)) < 1e-6
    assert pl.quat[:, bi, 3].abs().max().item() > 0.5 and pl.quat[:, xi, 3].abs().max().item() == 0.0
    st = parse_task(STACK.replace("init=cube@table_top:sep=0.1", "init=cube@brick"))
    ps = sample_placements(st, f, sites, 8)
    ci = f.slot_index("cube")
    assert torch.allclose(ps.pos[:, ci, :2], ps.pos[:, bi, :2])
    assert abs((ps.pos[0, ci, 2] - ps.pos[0, bi, 2]).item() - (0.015 + 0.01 + 0.02)) < 1e-6
    tab = InitTable(t, f, sites, k=256)
    p, q = tab.draw(32)
    assert p.shape == (32, len(f.slots), 3) and len(tab) + tab.rejected == 256


def test_family_env_scripted_pick_and_place_succeeds():
    from noeira_b200.tasks import parse_task
    from noeira_b200.tasks.family import TabletopFamilyEnv
    f = _family()
    env = TabletopFamilyEnv(f, [parse_task(PICK), parse_task(STACK)], 8, device="cpu", seed=3)
    env.reset_batch()
    fam = env.family
    bi, xi, gi = fam.slot_index("brick"), fam.slot_index("box"), fam.slot_index("gripper")
    lanes = (env.lane_task == 0).nonzero().squeeze(-1)
    total = torch.zeros(env.n_envs)
    succeeded = torch.zeros(env.n_envs, dtype=torch.bool)
    for step in range(59):
        g = env.pos[:, gi]
        holding = env.holding >= 0
        target = torch.where(holding[:, None], env.pos[:, xi] + torch.tensor([0.0, 0.0, 0.08]), env.pos[:, bi])
        delta = ((target - g) / env.move_step).clamp(-1, 1)
        at = torch.linalg.vector_norm(target - g, dim=-1) < 0.01
        grip = torch.where(holding & at, -torch.ones(8), torch.ones(8))     # close to take, open above the box
        env.step_batch(torch.cat([delta, grip[:, None]], dim=1))
        total += env.reward
        succeeded |= env.terminated.bool()
    assert bool(succeeded[lanes].all()), env.success_rates()
    assert env.success_rates()["brick_in_box"] == 1.0
    assert total[lanes].min().item() > 3.0          # shaping + bonus outweigh the step cost
    assert env.obs.shape == (8, env.obs_dim) and torch.isfinite(env.obs).all()


def test_sac_family_driver_runs():
    from noeira_b200.tasks import parse_task
    from noeira_b200.tasks.family import sac_family_driver
    f = _family()
    trainer, env, log, rates = sac_family_driver(f, [parse_task(PICK), parse_task(STACK)], n_envs=16, total_env_steps=16 * 40,
                                                 hidden=64)
    assert set(rates) == {"brick_in_box", "stack"}
    assert float(env.episode_count.sum()) >= 0
