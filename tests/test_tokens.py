"""Token files (the reference's FLINTTOK format, scripts/fineweb.py:27-37) and the batch
stream over them: the byte layout the reference's tests state (tests/test_fineweb.py:160-218),
its rejection cases, and the rank/step walk of TokenBatches. CPU only."""

import hashlib

import numpy as np
import pytest

from flint_b200 import tokens as tk


def test_file_bytes_are_the_stated_layout(tmp_path):
    path = tmp_path / "tokens.bin"
    values = np.array([50256, 0, 1, 65535, 12345], dtype=np.uint16)
    sha = tk.write_token_file(path, values)
    raw = path.read_bytes()
    assert raw[:8] == b"FLINTTOK"
    assert raw[8:12] == (1).to_bytes(4, "little") and raw[12:16] == (1).to_bytes(4, "little")
    assert raw[16:24] == (5).to_bytes(8, "little") and raw[24:64] == bytes(40)
    assert raw[64:] == values.astype("<u2").tobytes() and len(raw) == 64 + 2 * 5
    assert sha == hashlib.sha256(raw).hexdigest()
    loaded = tk.read_token_file(path)
    assert loaded.dtype == np.dtype("<u2") and np.array_equal(loaded, values)
    assert loaded.flags.writeable is False
    assert not list(tmp_path.glob("*.tmp"))


def test_wider_integers_are_narrowed_only_when_they_fit(tmp_path):
    tk.write_token_file(tmp_path / "a.bin", np.array([1, 50256], dtype=np.int64))
    assert tk.read_token_file(tmp_path / "a.bin").tolist() == [1, 50256]
    for bad in ([70000], [-1]):
        with pytest.raises(ValueError):
            tk.write_token_file(tmp_path / "b.bin", np.array(bad, dtype=np.int64))
        assert not (tmp_path / "b.bin").exists() and not list(tmp_path.glob("*.tmp"))


def test_an_empty_file_is_just_the_header(tmp_path):
    tk.write_token_file(tmp_path / "empty.bin", np.empty(0, dtype=np.uint16))
    assert (tmp_path / "empty.bin").stat().st_size == 64
    assert len(tk.read_token_file(tmp_path / "empty.bin")) == 0


def _set(index, value):
    def change(raw):
        raw[index] = value
        return raw
    return change


DAMAGE = {
    "magic": _set(0, ord("X")),
    "version": _set(8, 2),
    "tokenizer id": _set(12, 7),
    "reserved bytes": _set(40, 1),
    "count too big": _set(16, 9),
    "count too small": _set(16, 2),
    "truncated": lambda raw: raw[:-1],
    "extra byte": lambda raw: raw + b"\0",
    "shorter than the header": lambda raw: raw[:30],
}


@pytest.mark.parametrize("case", sorted(DAMAGE))
def test_damaged_files_are_rejected(tmp_path, case):
    path = tmp_path / "tokens.bin"
    tk.write_token_file(path, np.arange(5, dtype=np.uint16))
    path.write_bytes(bytes(DAMAGE[case](bytearray(path.read_bytes()))))
    with pytest.raises(tk.TokenFileError):
        tk.read_token_file(path)


def test_a_failed_write_leaves_no_file(tmp_path, monkeypatch):
    def explode(*_):
        raise OSError("disk full")
    monkeypatch.setattr(tk.os, "fsync", explode)
    with pytest.raises(OSError):
        tk.write_token_file(tmp_path / "tokens.bin", np.arange(5, dtype=np.uint16))
    assert not list(tmp_path.iterdir())


# ---- the batch stream ----------------------------------------------------------------------------


def shards(tmp_path, sizes, vocab=50257, seed=0):
    rng = np.random.default_rng(seed)
    paths, streams = [], []
    for i, size in enumerate(sizes):
        values = rng.integers(0, vocab, size=size, dtype=np.uint16)
        path = tmp_path / f"shard_{i:03d}.bin"
        tk.write_token_file(path, values)
        paths.append(path)
        streams.append(values)
    return paths, streams


def test_ranks_tile_the_stream_and_targets_are_the_next_tokens(tmp_path):
    paths, (stream,) = shards(tmp_path, [2 * 3 * 8 * 4 + 1])
    world, sequences, length = 3, 2, 8
    loaders = [tk.TokenBatches(paths, sequences, length, rank, world) for rank in range(world)]
    per_rank = sequences * length
    for step in range(4):
        for rank, loader in enumerate(loaders):
            tokens, targets = loader.next_batch()
            begin = (step * world + rank) * per_rank
            assert tokens.dtype == np.uint16 and tokens.shape == (sequences, length)
            assert np.array_equal(tokens.reshape(-1), stream[begin:begin + per_rank])
            assert np.array_equal(targets.reshape(-1), stream[begin + 1:begin + per_rank + 1])
    assert loaders[0].steps_per_epoch() == 4 and loaders[0].epoch == 0
    loaders[0].next_batch()
    assert loaders[0].epoch == 1 and loaders[0].position == loaders[0].per_step


def test_a_shard_is_left_when_it_cannot_feed_every_rank(tmp_path):
    # 40 tokens per step (+1): the first shard gives 2 steps (its last 19 tokens are skipped),
    # the second is too small to use, the third gives 1.
    paths, streams = shards(tmp_path, [100, 30, 41])
    loader = tk.TokenBatches(paths, 2, 10, rank=1, world=2)
    assert loader.usable == [0, 2] and loader.steps_per_epoch() == 3
    seen = [loader.next_batch()[0].reshape(-1).copy() for _ in range(4)]
    assert np.array_equal(seen[0], streams[0][20:40])
    assert np.array_equal(seen[1], streams[0][60:80])
    assert np.array_equal(seen[2], streams[2][20:40])
    assert np.array_equal(seen[3], streams[0][20:40]) and loader.epoch == 1


def test_the_position_round_trips_through_state(tmp_path):
    paths, _ = shards(tmp_path, [500, 300])
    a = tk.TokenBatches(paths, 2, 16, rank=0, world=2)
    for _ in range(9):
        a.next_batch()
    saved = a.state()
    b = tk.TokenBatches(paths, 2, 16, rank=0, world=2)
    b.restore(saved)
    for _ in range(12):
        left, right = a.next_batch(), b.next_batch()
        assert np.array_equal(left[0], right[0]) and np.array_equal(left[1], right[1])
    assert a.state() == b.state()
    with pytest.raises(ValueError):
        tk.TokenBatches(paths, 2, 16, rank=0, world=4).restore(saved)


def test_batches_land_in_the_callers_buffers_and_tokens_are_range_checked(tmp_path):
    paths, (stream,) = shards(tmp_path, [200], vocab=100)
    loader = tk.TokenBatches(paths, 2, 8, vocab=100)
    tokens = np.zeros((2, 8), dtype=np.uint16)
    targets = np.zeros((2, 8), dtype=np.uint16)
    out = loader.next_batch(tokens, targets)
    assert out[0] is tokens and np.array_equal(tokens.reshape(-1), stream[:16])
    with pytest.raises(ValueError):
        loader.next_batch(np.zeros((8, 2), dtype=np.uint16), targets)
    with pytest.raises(tk.TokenFileError):
        tk.TokenBatches(paths, 2, 8, vocab=50).next_batch()
    with pytest.raises(tk.TokenFileError):
        tk.TokenBatches(paths, 2, 200)
