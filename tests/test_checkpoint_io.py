"""Weights checkpoint I/O in the reference's positional safetensors format (crates/pm-train/src/checkpoint.rs:25-97).
The format code is host-only, so these tests need no GPU; the `safetensors` Python package (same on-disk format as
the Rust crate the reference uses) is the independent reader / writer."""
import json
import struct

import numpy as np
import pytest

sf = pytest.importorskip("safetensors.numpy")


@pytest.fixture(scope="module")
def pm():
    import __graft_entry__ as ge
    ge.build()
    import pm_b200
    return pm_b200


def _arrays():
    rng = np.random.default_rng(7)
    shapes = [(11, 8), (8, 20), (6, 1, 4), (6,), (2,), (2,), (2,), (4,), (4, 8)]
    return shapes, [rng.standard_normal(s).astype(np.float32) for s in shapes]


def test_written_file_is_read_by_the_safetensors_package(pm, tmp_path):
    shapes, arrs = _arrays()
    path = tmp_path / "w.safetensors"
    pm.save_checkpoint_f32(path, arrs)
    got = sf.load_file(str(path))
    assert sorted(got) == [f"p_{i:04d}" for i in range(len(arrs))]
    for i, a in enumerate(arrs):
        assert got[f"p_{i:04d}"].dtype == np.float32 and got[f"p_{i:04d}"].shape == a.shape
        assert np.array_equal(got[f"p_{i:04d}"], a)
    raw = path.read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    assert hlen % 8 == 0                                   # header padded like the reference's serializer
    hdr = json.loads(raw[8:8 + hlen])
    assert hdr["p_0002"] == {"dtype": "F32", "shape": [6, 1, 4], "data_offsets": hdr["p_0002"]["data_offsets"]}
    assert len(raw) == 8 + hlen + sum(a.nbytes for a in arrs)


def test_file_of_the_safetensors_package_is_read_back(pm, tmp_path):
    shapes, arrs = _arrays()
    path = tmp_path / "r.safetensors"
    sf.save_file({f"p_{i:04d}": a for i, a in enumerate(arrs)}, str(path), metadata={"step": "12", "note": "a \"quoted\" {brace}"})
    got = pm.load_checkpoint_f32(path, shapes)
    for a, b in zip(arrs, got):
        assert np.array_equal(a, b)


def test_round_trip_with_empty_and_scalar_like_tensors(pm, tmp_path):
    arrs = [np.zeros((0, 3), np.float32), np.array([1.5], np.float32), np.arange(6, dtype=np.float32).reshape(1, 2, 3)]
    path = tmp_path / "e.safetensors"
    pm.save_checkpoint_f32(path, arrs)
    got = pm.load_checkpoint_f32(path, [a.shape for a in arrs])
    for a, b in zip(arrs, got):
        assert a.shape == b.shape and np.array_equal(a, b)


def test_load_rejects_count_shape_and_dtype_mismatch(pm, tmp_path):
    shapes, arrs = _arrays()
    path = tmp_path / "m.safetensors"
    pm.save_checkpoint_f32(path, arrs)
    with pytest.raises(pm.PmbError, match="tensors, model has"):           # checkpoint.rs:66-71
        pm.load_checkpoint_f32(path, shapes[:-1])
    bad = list(shapes); bad[1] = (20, 8)
    with pytest.raises(pm.PmbError, match="shape mismatch"):               # checkpoint.rs:84-89
        pm.load_checkpoint_f32(path, bad)
    p16 = tmp_path / "h.safetensors"
    sf.save_file({f"p_{i:04d}": a.astype(np.float16) for i, a in enumerate(arrs)}, str(p16))
    with pytest.raises(pm.PmbError, match="expected F32"):                 # checkpoint.rs:78-83
        pm.load_checkpoint_f32(p16, shapes)
    with pytest.raises(pm.PmbError, match="cannot open"):
        pm.load_checkpoint_f32(tmp_path / "missing.safetensors", shapes)
    trunc = tmp_path / "t.safetensors"
    trunc.write_bytes(path.read_bytes()[:-10])
    with pytest.raises(pm.PmbError, match="file ends inside"):
        pm.load_checkpoint_f32(trunc, shapes)
