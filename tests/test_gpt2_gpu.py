"""The GPT-2 assembly and the trainer against the FP32 oracle, on a B200.

Tolerances are the ones the task states for this path: training loss within 1e-2 of
the FP32 oracle on the same seeded inputs, gradient cosine similarity >= 0.999, for
weights that are FP16-representable (tests/test_gpt2.py:194-208 in the reference).
"""

import ctypes

import numpy as np
import pytest
import torch

import flint_b200
import flint_oracle as oracle
from flint_b200.trainer import Trainer, TrainerConfig

pytestmark = pytest.mark.gpu
DEV = "cuda"

SMALL = dict(n_layer=2, n_head=2, n_embd=128, block_size=64, vocab_size=200, padded_vocab_size=208)
SEQUENCES, LENGTH = 3, 64


def model_config(cfg, sequences, length, backward):
    return flint_b200.Gpt2Config(cfg["n_layer"], cfg["n_head"], cfg["n_embd"], cfg["block_size"],
                                 cfg["vocab_size"], cfg["padded_vocab_size"], sequences, length, 0,
                                 int(backward))


def u16(t):
    return torch.from_numpy(t.numpy().astype(np.uint16).view(np.int16)).to(DEV)


def cosine(a, b):
    return torch.nn.functional.cosine_similarity(a.double().flatten(), b.double().flatten(), dim=0)


@pytest.fixture(scope="module")
def case():
    params = oracle.gpt2_round_to_half(oracle.gpt2_init(SMALL, seed=1234))
    g = torch.Generator().manual_seed(5)
    for name in params:  # non-trivial biases and LayerNorm parameters
        if name.endswith(".bias"):
            params[name] = (torch.randn(params[name].shape, generator=g) * 0.01).half().float()
    idx, targets = oracle.synthetic_tokens(SEQUENCES, LENGTH, SMALL["vocab_size"], seed=7)
    loss, grads = oracle.gpt2_loss_and_gradients(SMALL, params, idx, targets)
    return params, idx, targets, loss, grads


@pytest.mark.parametrize("flash", [None, True])
def test_forward_and_backward_match_the_oracle(flint, case, flash):
    params, idx, targets, want_loss, want_grads = case
    rows = SEQUENCES * LENGTH
    with flint_b200.Gpt2(flint, model_config(SMALL, SEQUENCES, LENGTH, True), flash) as model:
        assert [p[0] for p in model.parameters()] == list(params)
        model.load({k: v.to(DEV) for k, v in params.items()})
        scale = 1024.0 / rows
        model.forward(u16(idx.flatten()), u16(targets.flatten()), scale)
        model.backward(u16(idx.flatten()), False)
        loss = model.mean_loss()
        assert not flint.kernel_fault()
        assert abs(loss - want_loss) <= 1e-2
        for name, address, rows_, cols in model.gradients():
            got = model.read(address, (rows_, cols), torch.float32).cpu() / 1024.0
            want = want_grads[name].reshape(rows_, cols)
            assert cosine(got, want) >= 0.999, name
            assert torch.allclose(got, want, rtol=0.05, atol=2e-3 * want.abs().max().item()), name
        # Accumulating a second pass doubles every gradient (up to FP32 rounding).
        first = {n: model.read(a, (r, c), torch.float32) for n, a, r, c in model.gradients()}
        model.forward(u16(idx.flatten()), u16(targets.flatten()), scale)
        model.backward(u16(idx.flatten()), True)
        for name, address, rows_, cols in model.gradients():
            got = model.read(address, (rows_, cols), torch.float32)
            assert torch.allclose(got, 2 * first[name], rtol=1e-3, atol=1e-6), name


def test_bytes_is_the_sum_of_the_documented_buffers(flint):
    cfg = model_config(oracle.GPT2, 8, 1024, False)
    size = ctypes.c_size_t()
    flint.check(flint.lib.flint_gpt2_bytes(ctypes.byref(cfg), ctypes.byref(size)))
    up = lambda b: -(-b // 256) * 256
    w, rows, heads, t, v, layers = 768, 8192, 12, 1024, 50304, 12
    params = [v * w, 1024 * w] + layers * [w, w, 3 * w * w, 3 * w, w * w, w, w, w, 4 * w * w,
                                           4 * w, 4 * w * w, w] + [w, w]
    total = sum(up(4 * p) for p in params)
    total += up(2 * v * w) + layers * sum(up(2 * n) for n in (3 * w * w, w * w, 4 * w * w, 4 * w * w))
    matrix = 8 * heads * t * t * 2
    total += 2 * up(rows * w * 4) + up(rows * w * 2) + 2 * up(rows * 4) + up(rows * 3 * w * 2)
    total += 3 * up(rows * w * 2) + 2 * up(matrix) + 2 * up(rows * w * 2) + 2 * up(rows * 4 * w * 2)
    total += 2 * up(rows * v * 2) + up(rows * 4)
    assert size.value == total


def test_config_errors(flint):
    bad = model_config(SMALL, SEQUENCES, 60, False)  # length not a multiple of 8
    handle = ctypes.c_void_p(1)
    status = flint.lib.flint_gpt2_create(ctypes.byref(bad), ctypes.byref(handle))
    assert status == flint_b200.ERROR_INVALID_ARGUMENT and handle.value is None
    assert "length (60) must be a multiple of 8" in flint.last_error()
    with flint_b200.Gpt2(flint, model_config(SMALL, SEQUENCES, LENGTH, False)) as model:
        with pytest.raises(flint_b200.FlintError, match="created without backward"):
            model.backward(torch.zeros(SEQUENCES * LENGTH, dtype=torch.int16, device=DEV))


def test_trainer_steps_follow_the_oracle(flint, case):
    params, idx, targets, _, _ = case
    config = TrainerConfig(layers=2, heads=2, width=128, block_size=64, vocab=200, padded_vocab=208,
                           sequences=SEQUENCES, length=LENGTH, loss_scale=1024.0)
    trainer = Trainer(flint, config, state=params)
    ref = {k: v.clone() for k, v in params.items()}
    moments = {k: (torch.zeros_like(v), torch.zeros_like(v)) for k, v in ref.items()}
    try:
        for step in range(1, 4):
            want_loss, grads = oracle.gpt2_loss_and_gradients(SMALL, ref, idx, targets)
            for name, p in ref.items():
                wd = oracle.WEIGHT_DECAY if oracle.decayed(name, p.shape) else 0.0
                oracle.adamw_step(p, *moments[name], grads[name], step, weight_decay=wd)
            trainer.step(u16(idx.flatten()), u16(targets.flatten()))
            loss = trainer.finish_step()
            assert not flint.kernel_fault()
            assert abs(loss - want_loss) <= 1e-2
        assert trainer.skipped == 0
        # Adam's first steps move every weight by about lr whatever its gradient's size, so
        # compare the updates' directions. The key bias's gradient is zero in exact
        # arithmetic (softmax ignores a shift of all scores), so its update is rounding
        # noise: biases are only checked as part of the whole model's update.
        all_moved, all_expected = [], []
        for name, address, rows_, cols in trainer.model.parameters():
            got = trainer.model.read(address, (rows_, cols), torch.float32).cpu()
            want = ref[name].reshape(rows_, cols)
            moved = got - params[name].reshape(rows_, cols)
            expected = want - params[name].reshape(rows_, cols)
            all_moved.append(moved.flatten())
            all_expected.append(expected.flatten())
            if rows_ > 1:
                assert cosine(moved, expected) >= 0.98, name
        assert cosine(torch.cat(all_moved), torch.cat(all_expected)) >= 0.99
    finally:
        trainer.close()


def test_trainer_skips_a_step_with_nonfinite_gradients(flint, case):
    params, idx, targets, _, _ = case
    config = TrainerConfig(layers=2, heads=2, width=128, block_size=64, vocab=200, padded_vocab=208,
                           sequences=SEQUENCES, length=LENGTH, loss_scale=2.0 ** 40)
    trainer = Trainer(flint, config, state=params)
    try:
        before = {n: trainer.model.read(a, (r, c), torch.float32) for n, a, r, c in
                  trainer.model.parameters()}
        trainer.step(u16(idx.flatten()), u16(targets.flatten()))
        trainer.finish_step()
        assert trainer.skipped == 1 and trainer.scaler.scale == 2.0 ** 39
        for n, a, r, c in trainer.model.parameters():
            assert torch.equal(trainer.model.read(a, (r, c), torch.float32), before[n]), n
    finally:
        trainer.close()


def test_a_resumed_run_repeats_the_uninterrupted_one_bit_for_bit(flint, case, tmp_path):
    """Token files feed the trainer; a checkpoint taken after two steps (weights, moments,
    loss scale, counters, the stream's position) restored into a fresh trainer gives the
    same losses and the same final weights as the run that never stopped."""
    from flint_b200.tokens import TokenBatches, write_token_file

    params = case[0]
    rng = np.random.default_rng(11)
    paths = []
    for i, size in enumerate((SEQUENCES * LENGTH * 3 + 1, SEQUENCES * LENGTH * 2 + 40)):
        paths.append(tmp_path / f"shard_{i:03d}.bin")
        write_token_file(paths[-1], rng.integers(0, SMALL["vocab_size"], size=size, dtype=np.uint16))
    config = TrainerConfig(layers=2, heads=2, width=128, block_size=64, vocab=200, padded_vocab=208,
                           sequences=SEQUENCES, length=LENGTH, loss_scale=1024.0, growth_interval=3)

    def run(trainer, batches, steps):
        losses = []
        for _ in range(steps):
            tokens, targets = batches.next_batch()
            trainer.step(torch.from_numpy(tokens.view(np.int16)).to(DEV).flatten(),
                         torch.from_numpy(targets.view(np.int16)).to(DEV).flatten())
            losses.append(trainer.finish_step())
        return losses

    def weights(trainer):
        return {n: trainer.model.read(a, (r, c), torch.float32).cpu()
                for n, a, r, c in trainer.model.parameters()}

    first = Trainer(flint, config, state=params)
    try:
        batches = TokenBatches(paths, SEQUENCES, LENGTH, vocab=SMALL["vocab_size"])
        run(first, batches, 2)
        first.save(tmp_path / "step2.ckpt", data_state=batches.state())
        want_losses = run(first, batches, 4)  # crosses into the second shard and a scale growth
        want = weights(first)
        want_scale, want_steps = first.scaler.scale, first.step_count
    finally:
        first.close()

    second = Trainer(flint, config, state={k: torch.zeros_like(v) for k, v in params.items()})
    try:
        batches = TokenBatches(paths, SEQUENCES, LENGTH, vocab=SMALL["vocab_size"])
        batches.restore(second.restore(tmp_path / "step2.ckpt"))
        assert second.step_count == 2
        assert run(second, batches, 4) == want_losses
        assert second.scaler.scale == want_scale and second.step_count == want_steps
        got = weights(second)
        for name in want:
            assert torch.equal(got[name], want[name]), name
    finally:
        second.close()
    assert not flint.kernel_fault()


def test_the_training_driver_resumes_from_its_checkpoint(tmp_path, capsys):
    """`python -m flint_b200.train` in process: four steps in one go, and two + two through
    a checkpoint file, log the same losses."""
    from flint_b200 import train
    from flint_b200.tokens import write_token_file

    rng = np.random.default_rng(3)
    shard = tmp_path / "shard_001.bin"
    write_token_file(shard, rng.integers(0, 200, size=2 * 64 * 5 + 1, dtype=np.uint16))
    common = ["--tokens", str(shard), "--sequences", "2", "--length", "64", "--layers", "2",
              "--heads", "2", "--width", "128", "--block-size", "64", "--vocab", "200",
              "--padded-vocab", "208", "--loss-scale", "1024"]
    whole = train.main(common + ["--steps", "4"])
    ckpt = str(tmp_path / "run.ckpt")
    head = train.main(common + ["--steps", "2", "--checkpoint", ckpt])
    tail = train.main(common + ["--steps", "2", "--resume", ckpt])
    assert len(whole) == 4 and head + tail == whole
    assert all(np.isfinite(whole))
    lines = [line for line in capsys.readouterr().out.splitlines() if line.startswith("{")]
    assert len(lines) == 8 and '"step": 4' in lines[3] and '"step": 4' in lines[7]


def test_accumulated_micro_batches_equal_one_large_batch(flint, case):
    """Two micro-batches accumulated into one optimizer step (the reference's train_step over
    a list of batches, scripts/gpt2_torch.py:178-192) against the same six sequences as one
    batch: the same mean loss, and weight updates that agree to rounding."""
    params = case[0]
    idx, targets = oracle.synthetic_tokens(2 * SEQUENCES, LENGTH, SMALL["vocab_size"], seed=21)
    shape = dict(layers=2, heads=2, width=128, block_size=64, vocab=200, padded_vocab=208,
                 length=LENGTH, loss_scale=1024.0)

    def updated(trainer):
        return torch.cat([trainer.model.read(a, (r, c), torch.float32).cpu().flatten()
                          for _, a, r, c in trainer.model.parameters()])

    whole = Trainer(flint, TrainerConfig(sequences=2 * SEQUENCES, **shape), state=params)
    try:
        start = torch.cat([params[name].flatten() for name, *_ in whole.model.parameters()])
        whole.step(u16(idx.flatten()), u16(targets.flatten()))
        want_loss = whole.finish_step()
        want = updated(whole)
    finally:
        whole.close()
    parts = Trainer(flint, TrainerConfig(sequences=SEQUENCES, **shape), state=params)
    try:
        parts.step_batches([(u16(idx[:SEQUENCES].flatten()), u16(targets[:SEQUENCES].flatten())),
                            (u16(idx[SEQUENCES:].flatten()), u16(targets[SEQUENCES:].flatten()))])
        loss = parts.finish_step()
        got = updated(parts)
        assert parts.step_count == 1 and parts.skipped == 0
    finally:
        parts.close()
    assert abs(loss - want_loss) <= 1e-5
    assert cosine(got - start, want - start) >= 0.999
    assert not flint.kernel_fault()


def test_trainer_on_the_reference_layout_with_a_width_that_leaves_gaps_in_the_arena(flint):
    """Width 72: 72 * 4 bytes is not a multiple of the arena's 256-byte rounding, so there
    are gaps between the gradient tensors that backward never writes. The trainer checks and
    reduces the arena as one array; the gaps start as zeros, so no step is skipped."""
    cfg = dict(n_layer=2, n_head=3, n_embd=72, block_size=64, vocab_size=200, padded_vocab_size=208)
    params = oracle.gpt2_round_to_half(oracle.gpt2_init(cfg, seed=1234))
    idx, targets = oracle.synthetic_tokens(2, 64, 200, seed=8)
    want_loss, _ = oracle.gpt2_loss_and_gradients(cfg, params, idx, targets)
    config = TrainerConfig(layers=2, heads=3, width=72, block_size=64, vocab=200, padded_vocab=208,
                           sequences=2, length=64, loss_scale=1024.0, flash_attention=False)
    trainer = Trainer(flint, config, state=params)
    try:
        for _ in range(2):
            trainer.step(u16(idx.flatten()), u16(targets.flatten()))
            loss = trainer.finish_step()
        assert trainer.skipped == 0 and trainer.scaler.scale == 1024.0
        assert np.isfinite(loss)
    finally:
        trainer.close()
    trainer = Trainer(flint, config, state=params)
    try:
        trainer.step(u16(idx.flatten()), u16(targets.flatten()))
        assert abs(trainer.finish_step() - want_loss) <= 1e-2
        assert trainer.skipped == 0
    finally:
        trainer.close()
