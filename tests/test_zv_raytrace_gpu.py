"""Ray-traced camera kernel against the NumPy restatement of the same math, on poses produced by the physics engine."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_raytrace_kernel_matches_oracle():
    from noeira_b200.envs import PlanarChainEnv
    from noeira_b200.physics.model import Body, Geom, Joint, RigidModel
    from noeira_b200.physics.raytrace import BatchedCameraRenderer, Camera, render_reference
    env = PlanarChainEnv(4, seed=3)
    env.reset_batch()
    a = torch.rand(4, env.act_dim, device="cuda") * 2 - 1
    for _ in range(15):
        env.step_batch(a)
    xpos, xmat = env.engine.body_poses()
    cams = [Camera((0.3, -2.5, 0.9), (0.3, 0.0, 0.4)), Camera((0.0, -1.8, 0.6), track_body=0, fovy_deg=60)]
    r = BatchedCameraRenderer(env.engine.model, cams, 40, 56)
    # add a box and a sphere in the world frame so that every primitive is covered
    extra = np.zeros((2, 24), np.float32)
    extra[0, 0], extra[0, 1], extra[0, 2:5], extra[0, 14:17], extra[0, 17:21] = 3, -1, (1.2, 0.4, 0.3), (0.2, 0.3, 0.3), (0.8, 0.3, 0.2, 1)
    extra[0, 5:14] = np.eye(3).reshape(-1)
    extra[1, 0], extra[1, 1], extra[1, 2:5], extra[1, 14], extra[1, 17:21] = 1, -1, (-0.6, 0.3, 0.35), 0.35, (0.2, 0.3, 0.9, 1)
    extra[1, 5:14] = np.eye(3).reshape(-1)
    r.geoms_np = np.concatenate([r.geoms_np, extra])
    r.geoms = torch.from_numpy(r.geoms_np).cuda()
    rgb, depth = r.render(xpos, xmat)
    torch.cuda.synchronize()
    ref_rgb, ref_depth = render_reference(r.geoms_np, xpos.cpu().numpy(), xmat.cpu().numpy(), r.cams_np, 40, 56, r.light_np)
    got, gd = rgb.cpu().numpy().astype(np.int32), depth.cpu().numpy()
    bad = (np.abs(got - ref_rgb.astype(np.int32)).max(-1) > 3).mean()
    assert bad < 0.01, bad                                # silhouette / shadow edges may flip by rounding
    both = (gd > 0) & (ref_depth > 0)
    assert (both.mean() > 0.3) and np.abs(gd[both] - ref_depth[both]).max() < 0.05 or np.percentile(np.abs(gd[both] - ref_depth[both]), 99) < 1e-3
    assert ((gd > 0) != (ref_depth > 0)).mean() < 0.005
