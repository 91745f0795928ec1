"""HDF5 reader / writer (classic layout): round trips, chunked + shuffled + deflated data, partial reads, many links,
attributes, structural checks of the bytes the writer produces, error reporting."""
import struct

import numpy as np
import pytest


def _episode(rng, T=37):
    return {"action": rng.normal(size=(T, 14)).astype(np.float32),
            "observations": {"qpos": rng.normal(size=(T, 14)), "qvel": rng.normal(size=(T, 14)).astype(np.float32),
                             "images": {"top": rng.integers(0, 255, size=(T, 12, 16, 3), dtype=np.uint8),
                                        "wrist": rng.integers(0, 255, size=(T, 12, 16, 3), dtype=np.uint8)}},
            "steps": np.arange(T, dtype=np.int64), "scalar": np.float32(3.5)}


@pytest.mark.parametrize("compression", [None, "gzip"])
def test_round_trip_nested_groups(tmp_path, compression):
    from noeira_b200.io.hdf5 import H5Dataset, H5File, H5Group, read_hdf5, write_hdf5
    rng = np.random.default_rng(0)
    ep = _episode(rng)
    path = str(tmp_path / "episode_0.hdf5")
    write_hdf5(path, ep, compression=compression, chunk_rows=8,
               attrs={"": {"sim": True, "robot": "aloha"}, "observations/qpos": {"unit": "rad", "scale": np.float64(2.0)}})
    with H5File(path) as f:
        assert f.keys() == ["action", "observations", "scalar", "steps"] and "observations" in f
        assert f.attrs == {"sim": 1, "robot": "aloha"}
        obs = f["observations"]
        assert isinstance(obs, H5Group) and obs.keys() == ["images", "qpos", "qvel"]
        qpos = f["observations/qpos"]
        assert isinstance(qpos, H5Dataset) and qpos.shape == (37, 14) and qpos.dtype == np.float64
        assert qpos.attrs["unit"] == "rad" and qpos.attrs["scale"] == 2.0
        assert np.array_equal(qpos[...], ep["observations"]["qpos"])
        top = f["observations/images/top"]
        assert top.dtype == np.uint8 and np.array_equal(top.read(), ep["observations"]["images"]["top"])
        # partial reads touch only the chunks they need and agree with slicing
        assert np.array_equal(top[5:19], ep["observations"]["images"]["top"][5:19])
        assert np.array_equal(top[36], ep["observations"]["images"]["top"][36]) and len(top) == 37
        assert np.array_equal(f["steps"][-3:], np.arange(34, 37))
        assert float(f["scalar"].read().item()) == 3.5
        if compression:
            assert [fid for fid, _ in top.filters] == [2, 1]              # shuffle, then deflate
        paths = [p for p, _ in f.visit()]
        assert paths == ["action", "observations/images/top", "observations/images/wrist", "observations/qpos", "observations/qvel",
                         "scalar", "steps"]
    flat = read_hdf5(path)
    assert np.array_equal(flat["action"], ep["action"]) and flat["observations/qvel"].dtype == np.float32


def test_compression_shrinks_and_many_links(tmp_path):
    from noeira_b200.io.hdf5 import H5File, write_hdf5
    big = {"zeros": np.zeros((600, 64), np.float32), "ramp": np.arange(600 * 8, dtype=np.int32).reshape(600, 8)}
    a, b = str(tmp_path / "a.h5"), str(tmp_path / "b.h5")
    write_hdf5(a, big)
    write_hdf5(b, big, compression="gzip")
    import os
    assert os.path.getsize(b) < 0.2 * os.path.getsize(a)
    with H5File(b) as f:
        assert np.array_equal(f["ramp"].read(), big["ramp"]) and not f["zeros"].read().any()
    # a group with more links than one symbol node holds (8): several nodes under one B-tree node, names stay sorted
    many = {f"demo_{i}": np.full((3,), i, np.int16) for i in range(40)}
    c = str(tmp_path / "c.h5")
    write_hdf5(c, {"data": many})
    with H5File(c) as f:
        g = f["data"]
        assert len(g.keys()) == 40 and all(int(g[f"demo_{i}"].read()[0]) == i for i in range(40))
        with pytest.raises(KeyError):
            f["data/demo_99"]


def test_written_bytes_follow_the_format(tmp_path):
    """Field-by-field check of the superblock, the root header's symbol-table message, the heap and a symbol node."""
    from noeira_b200.io.hdf5 import write_hdf5
    path = str(tmp_path / "s.h5")
    write_hdf5(path, {"x": np.arange(6, dtype=np.float32).reshape(2, 3)})
    raw = open(path, "rb").read()
    assert raw[:8] == b"\x89HDF\r\n\x1a\n" and raw[8] == 0 and raw[13] == 8 and raw[14] == 8
    leaf_k, internal_k = struct.unpack_from("<HH", raw, 16)
    assert (leaf_k, internal_k) == (4, 16)
    base, free, eof, drv = struct.unpack_from("<QQQQ", raw, 24)
    assert base == 0 and free == drv == 0xFFFFFFFFFFFFFFFF and eof == len(raw)
    name_off, hdr, cache, _ = struct.unpack_from("<QQII", raw, 56)
    btree, heap = struct.unpack_from("<QQ", raw, 80)
    assert cache == 1 and hdr % 8 == 0
    ver, _, nmsg, refs, hsize = struct.unpack_from("<BBHII", raw, hdr)
    assert ver == 1 and refs == 1 and nmsg == 1 and hsize == 24
    mtype, msize = struct.unpack_from("<HH", raw, hdr + 16)
    assert mtype == 0x11 and msize == 16 and struct.unpack_from("<QQ", raw, hdr + 24) == (btree, heap)
    assert raw[heap: heap + 4] == b"HEAP" and raw[btree: btree + 4] == b"TREE" and raw[btree + 4] == 0
    seg = struct.unpack_from("<Q", raw, heap + 24)[0]
    assert raw[seg + 8: seg + 10] == b"x\0"
    snod = struct.unpack_from("<Q", raw, btree + 32)[0]
    assert raw[snod: snod + 4] == b"SNOD" and struct.unpack_from("<H", raw, snod + 6)[0] == 1
    obj = struct.unpack_from("<Q", raw, snod + 16)[0]
    types = []
    p = obj + 16
    for _ in range(struct.unpack_from("<H", raw, obj + 2)[0]):
        t, sz = struct.unpack_from("<HH", raw, p)
        types.append(t)
        if t == 0x3:                                      # IEEE little-endian float32: class 1, 32 bits, bias 127
            cls, _, sign, _, size = struct.unpack_from("<BBBBI", raw, p + 8)
            assert cls == 0x11 and sign == 31 and size == 4 and struct.unpack_from("<I", raw, p + 8 + 16)[0] == 127
        if t == 0x8:
            v, c, addr, nbytes = struct.unpack_from("<BBQQ", raw, p + 8)
            assert (v, c, nbytes) == (3, 1, 24) and np.array_equal(np.frombuffer(raw, np.float32, 6, addr), np.arange(6))
        p += 8 + sz
    assert types == [0x1, 0x3, 0x5, 0x8]


def test_rejects_other_files(tmp_path):
    from noeira_b200.io.hdf5 import H5Error, H5File
    p = tmp_path / "not.h5"
    p.write_bytes(b"PK\x03\x04" + b"\0" * 600)
    with pytest.raises(H5Error):
        H5File(str(p))


def test_aloha_episode_files_feed_the_act_dataset(tmp_path):
    import torch
    from noeira_b200.data.act_dataset import ACTDataset, load_aloha_episode, save_aloha_episode, synthetic_episodes
    eps = synthetic_episodes(3, 40, cams=2, height=12, width=16, joints=6, seed=1)
    paths = []
    for i, e in enumerate(eps):
        p = str(tmp_path / f"episode_{i}.hdf5")
        save_aloha_episode(p, e, cameras=["top", "wrist"])
        paths.append(p)
    back = [load_aloha_episode(p) for p in paths]
    assert back[0]["cameras"] == ["top", "wrist"] and back[0]["attrs"] == {"sim": 0}
    for a, b in zip(eps, back):
        assert torch.equal(a["images"], b["images"]) and torch.allclose(a["qpos"], b["qpos"]) and torch.allclose(a["action"], b["action"])
    ds = ACTDataset(back, chunk=8)
    q, img, act, valid = ds.sample(5)
    assert img.shape == (5, 2, 3, 12, 16) and act.shape == (5, 8, 6) and valid.shape == (5, 10)


def test_variable_length_strings_round_trip(tmp_path):
    import struct
    from noeira_b200.io.hdf5 import H5File, write_hdf5
    words = np.array(["pick up the red block", "", "naïve café ☕", "x" * 3000], dtype=object)
    grid = np.array([["a", "bb"], ["ccc", "dddd"]], dtype=object)
    path = str(tmp_path / "text.h5")
    write_hdf5(path, {"task": {"instruction": words, "grid": grid, "fixed": np.array([b"ab", b"cd"])}, "n": np.arange(3)},
               attrs={"task/instruction": {"langs": np.array(["en", "français"], dtype=object), "kind": "text"}})
    with H5File(path) as f:
        ds = f["task/instruction"]
        got = ds.read()
        assert got.dtype == object and list(got) == list(words)
        assert list(ds.read(1, 3)) == list(words[1:3]) and ds[2] == words[2]
        assert f["task/grid"].read().tolist() == grid.tolist()
        assert list(ds.attrs["langs"]) == ["en", "français"] and ds.attrs["kind"] == "text"
        assert f["task/fixed"].read().tolist() == [b"ab", b"cd"] and f["n"].read().tolist() == [0, 1, 2]
    raw = open(path, "rb").read()
    at = raw.index(b"GCOL")
    ver, size = struct.unpack_from("<B3xQ", raw, at + 4)
    assert ver == 1 and size >= 4096 and size % 8 == 0 and at % 8 == 0
    oid, ref, _, osize = struct.unpack_from("<HHIQ", raw, at + 16)
    assert (oid, ref, osize) == (1, 1, len(words[0])) and raw[at + 32: at + 32 + osize] == words[0].encode()
