"""Vision: camera reader thread on a scripted source, ChArUco calibration on rendered views, rigid fits, PIL-exact resize."""
import time

import numpy as np
import pytest

cv2 = pytest.importorskip("cv2")


class _Scripted:
    def __init__(self, n, delay=0.002):
        self.n, self.i, self.delay = n, 0, delay

    def read(self):
        time.sleep(self.delay)
        if self.i >= self.n:
            return False, None
        self.i += 1
        return True, np.full((4, 6, 3), self.i % 256, np.uint8)


def test_camera_reader_latest_frame_semantics():
    from noeira_b200.vision import CameraReader, parse_camera_specs
    assert parse_camera_specs("0, /dev/video2,clip.mp4") == ["0", "/dev/video2", "clip.mp4"]
    with pytest.raises(ValueError):
        parse_camera_specs("1,1")
    r = CameraReader(_Scripted(60), depth=2).start()
    time.sleep(0.08)
    f = r.take_latest()
    assert f is not None and f.shape == (4, 6, 3) and int(f[0, 0, 0]) > 5          # the newest, not the first
    assert r.take_latest() is None or True
    got = [r.take_blocking(500) for _ in range(3)]
    assert all(g is not None for g in got) and int(got[2][0, 0, 0]) > int(got[0][0, 0, 0])
    time.sleep(0.3)
    r.stop()
    assert r.eof and r.frames == 60 and r.dropped > 0 and r.delivered >= 4


def _render(board, K, rvec, tvec, size=(640, 480)):
    img = board.generateImage((700, 500), marginSize=0)
    bw, bh = 7 * 0.04, 5 * 0.04
    obj = np.array([[0, 0, 0], [bw, 0, 0], [bw, bh, 0], [0, bh, 0]], np.float32)
    px, _ = cv2.projectPoints(obj, rvec, tvec, K, None)
    H = cv2.getPerspectiveTransform(np.array([[0, 0], [700, 0], [700, 500], [0, 500]], np.float32), px.reshape(4, 2).astype(np.float32))
    return cv2.warpPerspective(img, H, size, borderValue=255)


def test_charuco_calibration_recovers_intrinsics(tmp_path):
    from noeira_b200.vision import calibrate_charuco, make_charuco_board, read_calib, write_calib
    from noeira_b200.vision.calib import board_pose
    board = make_charuco_board()
    K = np.array([[600.0, 0, 320], [0, 600.0, 240], [0, 0, 1]])
    rng = np.random.default_rng(0)
    views = []
    for _ in range(8):
        rvec = rng.uniform(-0.35, 0.35, 3)
        tvec = np.array([rng.uniform(-0.18, -0.10), rng.uniform(-0.14, -0.06), rng.uniform(0.45, 0.7)])
        views.append(_render(board, K, rvec, tvec))
    c = calibrate_charuco(views, board)
    assert c.n_views >= 5 and c.rms_px < 1.0
    assert abs(c.fx - 600) < 25 and abs(c.fy - 600) < 25 and abs(c.cx - 320) < 25 and abs(c.cy - 240) < 25
    p = str(tmp_path / "cal" / "cam.json")
    write_calib(p, c)
    d = read_calib(p)
    assert d == c
    with pytest.raises(ValueError):
        d.require_size(1280, 720)
    pose = board_pose(views[0], board, d)
    assert pose is not None and 0.4 < pose[1][2] < 0.75


def test_rigid_fit_and_offset():
    from noeira_b200.vision import fit_rigid, fit_rigid_with_offset
    rng = np.random.default_rng(1)
    R, _ = np.linalg.qr(rng.normal(size=(3, 3)))
    R *= np.sign(np.linalg.det(R))
    t = np.array([0.3, -0.1, 0.5])
    a = rng.uniform(-0.2, 0.2, (12, 3))
    b = a @ R.T + t + rng.normal(scale=2e-4, size=(12, 3))
    f = fit_rigid(a, b)
    assert np.allclose(f.R, R, atol=5e-3) and np.allclose(f.t, t, atol=2e-3) and f.rms_mm < 1.0
    with pytest.raises(ValueError):
        fit_rigid(np.c_[a[:, :2], np.zeros(12)], b)                     # coplanar: degenerate
    o = np.array([0.01, -0.02, 0.05])
    tool_R = np.stack([np.linalg.qr(rng.normal(size=(3, 3)))[0] for _ in range(12)])
    tool_R *= np.sign(np.linalg.det(tool_R))[:, None, None]
    tool_t = rng.uniform(-0.2, 0.2, (12, 3))
    base = np.einsum("nij,j->ni", tool_R, o) + tool_t
    cam = (base - t) @ R                                                # camera coordinates of those base points
    f2, o2 = fit_rigid_with_offset(cam, tool_R, tool_t)
    assert np.allclose(o2, o, atol=1e-3) and f2.rms_mm < 0.5


def test_pil_bilinear_is_bit_exact():
    from PIL import Image
    from noeira_b200.vision import camera_frame_to_chw_rgb, pil_bilinear_u8, resize_pad
    rng = np.random.default_rng(2)
    img = rng.integers(0, 256, (48, 64, 3), dtype=np.uint8)
    for oh, ow in ((24, 32), (30, 50), (96, 100), (48, 20)):
        want = np.asarray(Image.fromarray(img).resize((ow, oh), Image.BILINEAR))
        got = pil_bilinear_u8(img, oh, ow)
        assert np.array_equal(got, want), (oh, ow, np.abs(got.astype(int) - want.astype(int)).max())
    chw = camera_frame_to_chw_rgb(img, 24, 32)
    assert chw.shape == (3, 24, 32) and np.array_equal(chw[0], pil_bilinear_u8(img[:, :, 2], 24, 32))
    padded = resize_pad(img, 64, 64)
    assert padded.shape == (64, 64, 3) and padded[48:].max() == 0 and padded[:48].max() > 0
