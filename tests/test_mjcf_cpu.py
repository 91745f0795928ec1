import numpy as np
import pytest

XML = """
<mujoco model="hop">
  <compiler angle="degree"/>
  <option timestep="0.005" gravity="0 0 -9.81"/>
  <default>
    <joint damping="1.5" armature="0.05"/>
    <geom friction="0.8" rgba="0.2 0.4 0.9 1"/>
    <default class="leg"><joint range="-60 30" damping="2.5"/><geom size="0.04"/></default>
  </default>
  <worldbody>
    <geom type="plane" pos="0 0 0" size="10 10 1"/>
    <body name="torso" pos="0 0 1.2">
      <joint name="rootx" type="slide" axis="1 0 0" damping="0"/>
      <joint name="rootz" type="slide" axis="0 0 1" damping="0"/>
      <joint name="rooty" type="hinge" axis="0 1 0" damping="0"/>
      <geom type="capsule" fromto="0 0 -0.2 0 0 0.2" size="0.05"/>
      <body name="thigh" pos="0 0 -0.2" childclass="leg">
        <joint name="hip" type="hinge" axis="0 1 0"/>
        <geom type="capsule" fromto="0 0 0 0 0 -0.45"/>
        <body name="foot" pos="0 0 -0.45">
          <joint name="ankle" type="hinge" axis="0 1 0" range="-45 45"/>
          <geom type="sphere" size="0.06" pos="0.05 0 0"/>
        </body>
      </body>
    </body>
  </worldbody>
  <actuator><motor joint="hip" gear="100"/><motor joint="ankle" gear="40" ctrlrange="-0.5 0.5"/></actuator>
</mujoco>
"""


def test_mjcf_subset_parses_defaults_and_tree():
    from noeira_b200.physics.mjcf import MjcfError, from_mjcf
    m = from_mjcf(XML)
    assert m.nbody == 3 and list(m.body_parent) == [-1, 0, 1]
    assert m.opt.timestep == 0.005
    names = [j.name for b in m.bodies for j in b.joints]
    assert names == ["rootx", "rootz", "rooty", "hip", "ankle"]
    hip, ankle = m.bodies[1].joints[0], m.bodies[2].joints[0]
    assert hip.damping == 2.5 and hip.armature == 0.05                       # class "leg" over the main defaults
    assert np.allclose(hip.range, np.deg2rad([-60, 30])) and np.allclose(ankle.range, np.deg2rad([-45, 45]))
    assert m.bodies[0].joints[0].damping == 0.0
    thigh = m.bodies[1].geoms[0]
    assert thigh.type == "capsule" and abs(thigh.size[0] - 0.04) < 1e-12 and abs(thigh.size[1] - 0.225) < 1e-12
    assert thigh.friction == 0.8 and thigh.rgba[2] == 0.9
    assert list(m.act_gear) == [100.0, 40.0] and m.act_lo[1] == -0.5
    with pytest.raises(MjcfError):
        from_mjcf(XML.replace('type="sphere"', 'type="mesh"'))
    with pytest.raises(MjcfError):
        from_mjcf(XML.replace('<joint name="hip" type="hinge"', '<joint name="hip" type="ball"'))


def test_mjcf_model_matches_hand_built(tmp_path):
    """The parsed model and the same tree built by hand give identical packed tables and oracle dynamics."""
    from noeira_b200.physics.mjcf import from_mjcf
    from noeira_b200.physics.model import HINGE, SLIDE, Actuator, Body, Geom, Joint, Options, RigidModel, quat_z_to
    (tmp_path / "leg.xml").write_text('<mujocoinclude><body name="leg" pos="0.3 0 0"><joint name="knee" type="hinge" axis="0 1 0" '
                                      'range="-1 1"/><geom type="capsule" fromto="0 0 0 0 0 -0.3" size="0.03"/></body></mujocoinclude>')
    (tmp_path / "m.xml").write_text('<mujoco><compiler angle="radian"/><worldbody><geom type="plane"/><body name="cart" pos="0 0 0.5">'
                                    '<joint name="x" type="slide" axis="1 0 0"/><geom type="sphere" size="0.1"/><include file="leg.xml"/>'
                                    '</body></worldbody><actuator><motor joint="knee" gear="5"/></actuator></mujoco>')
    a = from_mjcf(str(tmp_path / "m.xml"))
    b = RigidModel([Body(-1, (0, 0, 0.5), joints=[Joint(SLIDE, (1, 0, 0), name="x")], geoms=[Geom("sphere", (0.1,))], name="cart"),
                    Body(0, (0.3, 0, 0), joints=[Joint(HINGE, (0, 1, 0), range=(-1, 1), name="knee")],
                         geoms=[Geom("capsule", (0.03, 0.15), pos=(0, 0, -0.15), quat=tuple(quat_z_to((0, 0, -0.3))))], name="leg")],
                   [Actuator("knee", 5.0)], Options())
    (ia, fa), (ib, fb) = a.pack(), b.pack()
    assert (ia == ib).all() and np.allclose(fa, fb, atol=1e-7)


def test_inline_mesh_and_height_field_assets_in_the_general_engine():
    import torch
    from noeira_b200.physics import general as G
    from noeira_b200.physics.mjcf import MjcfError, from_mjcf
    xml = """<mujoco><option timestep="0.002"/>
      <asset>
        <mesh name="wedge" vertex="0 0 0  0.2 0 0  0 0.2 0  0.2 0.2 0  0 0 0.1  0 0.2 0.1" scale="1 1 2"/>
        <hfield name="ramp" nrow="2" ncol="3" size="2 1 0.4 0.1" elevation="0 0.5 1  0 0.5 1"/>
      </asset>
      <worldbody>
        <geom type="hfield" hfield="ramp" friction="0.9"/>
        <body name="rock" pos="0 0 1"><freejoint/><geom type="mesh" mesh="wedge" density="500"/></body>
        <body name="ball" pos="-1 0 0.5"><freejoint/><geom type="sphere" size="0.1"/></body>
      </worldbody></mujoco>"""
    m = from_mjcf(xml, general=True)
    g = m.geoms[0][1]
    assert g.type == "mesh" and len(g.vertices) == 6 and max(v[2] for v in g.vertices) == 0.2        # scaled
    assert abs(float(m.mass[0]) - 500 * 0.5 * 0.2 * 0.2 * 0.2) < 1e-9                                  # a triangular prism
    assert m.hfield is not None and not m.plane and m.hfield.friction == 0.9
    h, n = m.hfield.sample(torch.tensor([-2.0, 0.0, 2.0], dtype=torch.float64), torch.zeros(3, dtype=torch.float64))
    assert torch.allclose(h, torch.tensor([0.0, 0.2, 0.4], dtype=torch.float64))
    sim = G.GeneralSim(m, 1, solver="newton", solver_iters=20)
    for _ in range(200):
        sim.step()
    hb, _ = m.hfield.sample(sim.qpos[:, 7], sim.qpos[:, 8])
    assert 0.09 < float(sim.qpos[0, 9] - hb) < 0.12                                                    # the ball sits on the ramp
    assert float(sim.qpos[0, 7]) < -1.0                                                                # and rolled downhill
    with pytest.raises(MjcfError):
        from_mjcf(xml.replace('vertex="0 0 0  0.2 0 0  0 0.2 0  0.2 0.2 0  0 0 0.1  0 0.2 0.1"', 'file="wedge.stl"'), general=True)
