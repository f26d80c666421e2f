"""The checkpoint container: round trips, the stated layout, and damaged files. CPU only."""

import hashlib
import json

import numpy as np
import pytest

from flint_b200.checkpoint import CheckpointError, read_checkpoint, write_checkpoint


def sample():
    rng = np.random.default_rng(1)
    return {
        "param/wte.weight": rng.standard_normal((37, 12)).astype(np.float32),
        "param/ln_f.bias": rng.standard_normal(12).astype(np.float32),
        "m/ln_f.bias": np.zeros(12, dtype=np.float32),
        "steps": np.array([3, 1, 4], dtype=np.int64),
        "empty": np.zeros((0, 5), dtype=np.float32),
    }


def test_round_trip_and_layout(tmp_path):
    path = tmp_path / "step.ckpt"
    meta = {"step_count": 7, "loss_scale": 32768.0, "data": {"shard": "shard_001.bin", "position": 4096}}
    sha = write_checkpoint(path, meta, sample())
    raw = path.read_bytes()
    assert raw[:8] == b"FLINTCKP" and int.from_bytes(raw[8:12], "little") == 1
    length = int.from_bytes(raw[12:16], "little")
    record = json.loads(raw[16:16 + length])
    assert record["meta"] == meta
    assert raw[-32:] == hashlib.sha256(raw[:-32]).digest() and sha == raw[-32:].hex()
    assert not list(tmp_path.glob("*.tmp"))
    got_meta, arrays = read_checkpoint(path, verify=True)
    assert got_meta == meta and list(arrays) == list(sample())
    for name, want in sample().items():
        assert arrays[name].dtype == want.dtype and arrays[name].shape == want.shape
        assert np.array_equal(arrays[name], want)
        assert arrays[name].flags.writeable is False
        entry = next(e for e in record["arrays"] if e["name"] == name)
        assert entry["offset"] % 64 == 0
        assert raw[entry["offset"]:entry["offset"] + entry["nbytes"]] == want.tobytes()


def test_no_arrays_and_large_records(tmp_path):
    write_checkpoint(tmp_path / "a.ckpt", {"x": 1}, {})
    assert read_checkpoint(tmp_path / "a.ckpt", verify=True) == ({"x": 1}, {})
    many = {f"t{i}": np.full(i % 7, i, dtype=np.float32) for i in range(300)}
    write_checkpoint(tmp_path / "b.ckpt", {"note": "x" * 1000}, many)
    _, arrays = read_checkpoint(tmp_path / "b.ckpt", verify=True)
    assert all(np.array_equal(arrays[k], v) for k, v in many.items())


def test_damage_is_detected(tmp_path):
    path = tmp_path / "step.ckpt"
    write_checkpoint(path, {"step": 1}, sample())
    good = path.read_bytes()

    def check(data, verify=True):
        path.write_bytes(data)
        with pytest.raises(CheckpointError):
            read_checkpoint(path, verify=verify)

    check(b"X" + good[1:])                       # magic
    check(good[:8] + b"\x02" + good[9:])         # version
    check(good[:-1], verify=False)               # truncated
    check(good + b"\0", verify=False)            # extra byte
    check(good[:10], verify=False)               # shorter than the prefix
    flipped = bytearray(good)
    flipped[len(good) // 2] ^= 1
    check(bytes(flipped))                        # a flipped payload bit
    path.write_bytes(bytes(flipped))
    read_checkpoint(path, verify=False)          # ... which only the checksum can see


def test_a_failed_write_keeps_the_old_checkpoint(tmp_path, monkeypatch):
    import flint_b200.checkpoint as module

    path = tmp_path / "step.ckpt"
    write_checkpoint(path, {"step": 1}, sample())
    before = path.read_bytes()

    def explode(*_):
        raise OSError("disk full")
    monkeypatch.setattr(module.os, "fsync", explode)
    with pytest.raises(OSError):
        write_checkpoint(path, {"step": 2}, sample())
    assert path.read_bytes() == before and not list(tmp_path.glob("*.tmp"))
