"""LeRobot v3 layout: export → import round trip (parquet + packed mp4 per camera) into the trajectory store."""
import json
import os

import numpy as np
import pytest


def _episodes(n=3, cams=("front", "wrist")):
    rng = np.random.default_rng(0)
    eps = []
    for e in range(n):
        T = 5 + 2 * e
        ep = {"observation.state": rng.normal(size=(T, 6)).astype(np.float32), "action": rng.normal(size=(T, 6)).astype(np.float32)}
        for ci, c in enumerate(cams):
            f = np.zeros((T, 48, 64, 3), np.uint8)
            for t in range(T):
                f[t, :, :, 0] = 40 * e + 8 * t           # flat colour encodes (episode, frame): survives the codec
                f[t, :, :, 1] = 100 + 50 * ci
                f[t, :, :, 2] = 30
            ep[f"observation.images.{c}"] = f
        eps.append(ep)
    return eps


def test_export_import_round_trip(tmp_path):
    pytest.importorskip("cv2")
    from noeira_b200.data.datasets import TrajectoryStore
    from noeira_b200.data.lerobot import import_lerobot_v3, write_lerobot_v3
    eps = _episodes()
    root = str(tmp_path / "ds")
    write_lerobot_v3(root, eps, fps=20.0, cameras=("front", "wrist"))
    info = json.load(open(os.path.join(root, "meta", "info.json")))
    assert info["codebase_version"] == "v3.0" and info["total_frames"] == sum(len(e["action"]) for e in eps)
    out = str(tmp_path / "store")
    s = import_lerobot_v3(root, out, height=24, width=32)
    assert s["episodes"] == 3 and s["frames"] == info["total_frames"] and len(s["cameras"]) == 2
    st = TrajectoryStore(out + ".traj")
    assert st.lengths == [5, 7, 9]
    for e in range(3):
        got = st.episode(e)
        assert np.allclose(got["state"], eps[e]["observation.state"]) and np.allclose(got["action"], eps[e]["action"])
    img = np.load(out + ".images.npy", mmap_mode="r")
    assert img.shape == (21, 2, 24, 32, 3)
    # every frame landed on its own row: the red channel encodes (episode, frame), the green one the camera
    row = 0
    for e in range(3):
        for t in range(len(eps[e]["action"])):
            assert abs(int(img[row, 0, 10, 10, 0]) - (40 * e + 8 * t)) <= 6, (e, t, img[row, 0, 10, 10])
            assert abs(int(img[row, 0, 10, 10, 1]) - 100) <= 8 and abs(int(img[row, 1, 10, 10, 1]) - 150) <= 8
            row += 1
    norm = json.load(open(out + ".norm.json"))
    allact = np.concatenate([e["action"] for e in eps])
    assert np.allclose(norm["action"]["mean"], allact.mean(0), atol=1e-5)
    assert min(norm["state"]["std"]) >= 1e-2
    # skipping an episode keeps the rest aligned
    s2 = import_lerobot_v3(root, str(tmp_path / "store2"), height=24, width=32, skip_episodes=[1])
    img2 = np.load(str(tmp_path / "store2") + ".images.npy", mmap_mode="r")
    assert s2["episodes"] == 2 and abs(int(img2[5, 0, 5, 5, 0]) - 80) <= 6      # first frame of episode 2


def test_out_of_order_video_layout_is_refused(tmp_path):
    pytest.importorskip("cv2")
    import pyarrow.parquet as pq
    from noeira_b200.data.lerobot import import_lerobot_v3, write_lerobot_v3
    root = str(tmp_path / "ds")
    write_lerobot_v3(root, _episodes(cams=("front",)), fps=20.0, cameras=("front",))
    p = os.path.join(root, "meta", "episodes", "chunk-000", "file-000.parquet")
    t = pq.read_table(p).to_pydict()
    k = "videos/observation.images.front/from_timestamp"
    t[k][1], t[k][2] = t[k][2], t[k][1]
    import pyarrow as pa
    pq.write_table(pa.table(t), p)
    with pytest.raises(ValueError, match="dataset order"):
        import_lerobot_v3(root, str(tmp_path / "o"), height=24, width=32)
