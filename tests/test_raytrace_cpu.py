import numpy as np
import torch


def test_reference_renderer_geometry():
    from noeira_b200.physics.model import planar_chain
    from noeira_b200.physics.raytrace import BatchedCameraRenderer, Camera
    m = planar_chain(seed=0)
    r = BatchedCameraRenderer(m, [Camera((0.5, -3.0, 1.0), (0.5, 0.0, 0.4))], 48, 64, device="cpu")
    nb = m.nbody
    xpos = torch.zeros(1, nb, 3)
    xpos[0, :, 0] = torch.arange(nb) * 0.25
    xpos[0, :, 2] = 0.5
    xmat = torch.eye(3).reshape(1, 1, 9).repeat(1, nb, 1)
    rgb, depth = r.render(xpos, xmat)
    assert rgb.shape == (1, 1, 48, 64, 3) and depth.shape == (1, 1, 48, 64)
    assert (depth[0, 0, :8] == 0).all()                 # sky at the top
    assert (depth[0, 0, -4:] > 0).all()                 # ground at the bottom
    mid = depth[0, 0, 20:34, 20:44]
    assert mid[mid > 0].min() < 3.2                      # the chain is nearer than the ground behind it
    assert len(np.unique(rgb.reshape(-1, 3), axis=0)) > 20
