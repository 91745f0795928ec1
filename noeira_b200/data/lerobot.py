"""LeRobot v3.0 datasets: import into the trajectory store, and export.

    meta/info.json                        features, fps, total_{episodes,frames}
    meta/episodes/chunk-*/file-*.parquet  per-episode index (dataset_from_index / dataset_to_index) + per-camera video map
    data/chunk-*/file-*.parquet           action / observation.state / timestamp / frame_index / episode_index / index
    videos/<key>/chunk-*/file-*.mp4       MANY episodes concatenated per file

``import_lerobot_v3(root, out)`` writes ``<out>.traj`` (state + action, float32, the trajectory container of
data/datasets.py), ``<out>.images.npy`` (uint8 ``[frames, cameras, H, W, 3]``, memory-mapped while written, frames
resized with the PIL-exact bilinear filter) and ``<out>.norm.json`` (mean / std of state and action, std floored at
1e-2 as ACT does).  Per camera ONE sequential decoder is advanced in lock step with the episode loop, so peak memory is
one frame per camera.  That relies on episodes sitting in their video files in dataset order, which is a property of the
writer, not of the format — it is CHECKED: an episode that would need the decoder to go backwards raises.
``write_lerobot_v3`` produces the same layout from episodes in memory (tests, recorded demonstrations).
Reference: noeira/data/lerobot.mojo:1-80, noeira/data/lerobot_write.mojo, noeira/io/parquet.
"""
from __future__ import annotations

import glob
import json
import os
from typing import Dict, List, Optional, Sequence

import numpy as np

from ..io.video import VideoDecoder, VideoEncoder
from .datasets import TrajectoryWriter

STD_FLOOR = 1e-2


def _pa():
    import pyarrow as pa
    import pyarrow.parquet as pq
    return pa, pq


def _read_tables(pattern: str):
    _, pq = _pa()
    files = sorted(glob.glob(pattern))
    if not files:
        raise FileNotFoundError(f"no parquet file matches {pattern}")
    return [pq.read_table(f) for f in files]


def write_lerobot_v3(root: str, episodes: Sequence[Dict[str, np.ndarray]], fps: float = 30.0, cameras: Sequence[str] = (),
                     robot_type: str = "so101", task: str = "demo") -> None:
    """``episodes``: dicts with ``observation.state [T, S]``, ``action [T, A]`` and, per camera key ``k`` of ``cameras``,
    ``observation.images.k`` uint8 ``[T, H, W, 3]``.  All episodes go into one data file and one video file per camera."""
    pa, pq = _pa()
    os.makedirs(os.path.join(root, "meta", "episodes", "chunk-000"), exist_ok=True)
    os.makedirs(os.path.join(root, "data", "chunk-000"), exist_ok=True)
    rows = {k: [] for k in ("observation.state", "action", "timestamp", "frame_index", "episode_index", "index", "task_index")}
    ep_rows = {"episode_index": [], "length": [], "dataset_from_index": [], "dataset_to_index": [], "tasks": []}
    encoders, vid_pos = {}, {}
    for cam in cameras:
        key = f"observation.images.{cam}"
        os.makedirs(os.path.join(root, "videos", key, "chunk-000"), exist_ok=True)
        h, w = episodes[0][key].shape[1:3]
        encoders[key] = VideoEncoder(os.path.join(root, "videos", key, "chunk-000", "file-000.mp4"), w, h, fps)
        vid_pos[key] = 0
        for c in ("chunk_index", "file_index", "from_timestamp", "to_timestamp"):
            ep_rows[f"videos/{key}/{c}"] = []
    n = 0
    for ei, ep in enumerate(episodes):
        T = len(ep["action"])
        rows["observation.state"] += [np.asarray(r, np.float32) for r in ep["observation.state"]]
        rows["action"] += [np.asarray(r, np.float32) for r in ep["action"]]
        rows["timestamp"] += [np.float32(t / fps) for t in range(T)]
        rows["frame_index"] += list(range(T))
        rows["episode_index"] += [ei] * T
        rows["index"] += list(range(n, n + T))
        rows["task_index"] += [0] * T
        ep_rows["episode_index"].append(ei); ep_rows["length"].append(T)
        ep_rows["dataset_from_index"].append(n); ep_rows["dataset_to_index"].append(n + T); ep_rows["tasks"].append([task])
        for key, enc in encoders.items():
            for f in ep[key]:
                enc.write(np.asarray(f, np.uint8))
            ep_rows[f"videos/{key}/chunk_index"].append(0); ep_rows[f"videos/{key}/file_index"].append(0)
            ep_rows[f"videos/{key}/from_timestamp"].append(vid_pos[key] / fps)
            vid_pos[key] += T
            ep_rows[f"videos/{key}/to_timestamp"].append(vid_pos[key] / fps)
        n += T
    for enc in encoders.values():
        enc.close()
    S, A = len(rows["observation.state"][0]), len(rows["action"][0])
    table = pa.table({
        "observation.state": pa.array([r.tolist() for r in rows["observation.state"]], pa.list_(pa.float32(), S)),
        "action": pa.array([r.tolist() for r in rows["action"]], pa.list_(pa.float32(), A)),
        "timestamp": pa.array(rows["timestamp"], pa.float32()), "frame_index": pa.array(rows["frame_index"], pa.int64()),
        "episode_index": pa.array(rows["episode_index"], pa.int64()), "index": pa.array(rows["index"], pa.int64()),
        "task_index": pa.array(rows["task_index"], pa.int64())})
    pq.write_table(table, os.path.join(root, "data", "chunk-000", "file-000.parquet"), compression="snappy")
    pq.write_table(pa.table(ep_rows), os.path.join(root, "meta", "episodes", "chunk-000", "file-000.parquet"))
    feats = {"observation.state": {"dtype": "float32", "shape": [S]}, "action": {"dtype": "float32", "shape": [A]}}
    for cam in cameras:
        key = f"observation.images.{cam}"
        h, w = episodes[0][key].shape[1:3]
        feats[key] = {"dtype": "video", "shape": [h, w, 3], "names": ["height", "width", "channels"]}
    info = {"codebase_version": "v3.0", "robot_type": robot_type, "fps": fps, "total_episodes": len(episodes), "total_frames": n,
            "total_tasks": 1, "features": feats,
            "data_path": "data/chunk-{chunk_index:03d}/file-{file_index:03d}.parquet",
            "video_path": "videos/{video_key}/chunk-{chunk_index:03d}/file-{file_index:03d}.mp4"}
    with open(os.path.join(root, "meta", "info.json"), "w") as f:
        json.dump(info, f, indent=1)


def import_lerobot_v3(root: str, out_path: str, height: int = 240, width: int = 320, cameras: Optional[Sequence[str]] = None,
                      skip_episodes: Sequence[int] = ()) -> Dict[str, object]:
    """Returns a summary dict; writes ``out_path + {.traj, .images.npy, .norm.json}``."""
    from ..vision.preprocess import pil_bilinear_u8
    with open(os.path.join(root, "meta", "info.json")) as f:
        info = json.load(f)
    if not str(info.get("codebase_version", "")).startswith("v3"):
        raise ValueError(f"{root}: codebase_version {info.get('codebase_version')!r} is not a v3 dataset")
    fps = float(info["fps"])
    cam_keys = [k for k, v in info["features"].items() if v.get("dtype") == "video"]
    if cameras is not None:
        cam_keys = [f"observation.images.{c}" if not c.startswith("observation.") else c for c in cameras]
    import pyarrow as pa
    eps = pa.concat_tables(_read_tables(os.path.join(root, "meta", "episodes", "chunk-*", "file-*.parquet"))).to_pydict()
    data = pa.concat_tables(_read_tables(os.path.join(root, "data", "chunk-*", "file-*.parquet")))
    state = np.asarray(data.column("observation.state").to_pylist(), np.float32)
    action = np.asarray(data.column("action").to_pylist(), np.float32)
    order = np.argsort(np.asarray(eps["episode_index"]))
    skip = set(int(s) for s in skip_episodes)
    kept = [int(i) for i in order if int(eps["episode_index"][i]) not in skip]
    n_frames = sum(int(eps["dataset_to_index"][i]) - int(eps["dataset_from_index"][i]) for i in kept)
    # the decoders only move forward: every camera's episodes must sit in (file, first frame) order
    for key in cam_keys:
        last = (-1, -1)
        for i in kept:
            cur = (int(eps[f"videos/{key}/chunk_index"][i]) * 100000 + int(eps[f"videos/{key}/file_index"][i]),
                   int(round(float(eps[f"videos/{key}/from_timestamp"][i]) * fps)))
            if cur < last:
                raise ValueError(f"{root}: episodes of camera {key} are not stored in dataset order "
                                 f"(episode {eps['episode_index'][i]} starts at {cur}, after {last})")
            last = cur
    writer = TrajectoryWriter(out_path + ".traj", {"state": state.shape[1], "action": action.shape[1]},
                              meta={"source": "lerobot_v3", "fps": fps, "cameras": cam_keys, "height": height, "width": width})
    images = None
    if cam_keys:
        images = np.lib.format.open_memmap(out_path + ".images.npy", mode="w+", dtype=np.uint8,
                                           shape=(n_frames, len(cam_keys), height, width, 3))
    decoders: Dict[str, tuple] = {}
    row = 0
    for i in kept:
        lo, hi = int(eps["dataset_from_index"][i]), int(eps["dataset_to_index"][i])
        writer.add_episode(state=state[lo:hi], action=action[lo:hi])
        for ci, key in enumerate(cam_keys):
            chunk, fidx = int(eps[f"videos/{key}/chunk_index"][i]), int(eps[f"videos/{key}/file_index"][i])
            path = os.path.join(root, "videos", key, f"chunk-{chunk:03d}", f"file-{fidx:03d}.mp4")
            cur = decoders.get(key)
            if cur is None or cur[0] != path:
                if cur is not None:
                    cur[1].close()
                cur = (path, VideoDecoder(path))
                decoders[key] = cur
            dec = cur[1]
            dec.skip_to(int(round(float(eps[f"videos/{key}/from_timestamp"][i]) * fps)))
            for t in range(hi - lo):
                images[row + t, ci] = pil_bilinear_u8(dec.read(), height, width)
        row += hi - lo
    for _, dec in decoders.values():
        dec.close()
    writer.close()
    if images is not None:
        images.flush()
    rows = np.concatenate([np.arange(int(eps["dataset_from_index"][i]), int(eps["dataset_to_index"][i])) for i in kept])
    norm = {name: {"mean": arr[rows].mean(0).tolist(), "std": np.maximum(arr[rows].std(0), STD_FLOOR).tolist()}
            for name, arr in (("state", state), ("action", action))}
    with open(out_path + ".norm.json", "w") as f:
        json.dump(norm, f)
    return {"episodes": len(kept), "frames": n_frames, "cameras": cam_keys, "fps": fps}
