"""The optimizer kernels element by element, through the C ABI on a B200.

flint_b200_adamw, flint_b200_adamw_run and flint_b200_check_gradients against the oracle's
AdamW (torch.optim.AdamW's update as the reference configures it,
scripts/gpt2_torch.py:150-175) and its gradient clipping (:187-188). The oracle runs in
float64; the kernels compute in FP32, so every value must agree to FP32 rounding: relative
1e-6 on weights and moments, and 1e-4 on the step itself (the weight's change, which is what
a wrong bias correction or a misplaced epsilon would alter by per cent). The FP16 compute
copy must be the updated weight rounded once, bit for bit.
"""

import math

import numpy as np
import pytest
import torch

import flint_b200
import flint_oracle as oracle
from flint_b200.trainer import Trainer, TrainerConfig

pytestmark = pytest.mark.gpu
DEV = "cuda"
HYPER = dict(lr=6e-4, beta1=0.9, beta2=0.95, eps=1e-8)


def oracle_steps(p, grads, weight_decay, grad_scale=1.0, first_step=1):
    """float64 AdamW over a list of gradients; returns the (p, m, v) after each step."""
    p = p.double().clone()
    m, v = torch.zeros_like(p), torch.zeros_like(p)
    out = []
    for i, g in enumerate(grads):
        oracle.adamw_step(p, m, v, g.double() * grad_scale, first_step + i, lr=HYPER["lr"],
                          betas=(HYPER["beta1"], HYPER["beta2"]), eps=HYPER["eps"],
                          weight_decay=weight_decay)
        out.append((p.clone(), m.clone(), v.clone()))
    return out


def assert_close(got, want, rtol, what, operands=None):
    """|got - want| <= rtol * max(|want|, |operands|): where a result is the small difference
    of larger operands (a weight crossing zero, a moment changing sign) FP32's error is
    relative to those operands, not to the result."""
    got, want = got.double().cpu(), want.double()
    size = want.abs() if operands is None else torch.maximum(want.abs(), operands.double().abs())
    worst = ((got - want).abs() - rtol * size - 1e-30).max().item()
    assert worst <= 0, (what, worst)


@pytest.mark.parametrize("count", [1, 3, 4, 5, 1023, 8192 * 3 + 2])
@pytest.mark.parametrize("weight_decay", [0.0, 0.1])
def test_adamw_follows_the_oracle_element_by_element(flint, count, weight_decay):
    g = torch.Generator().manual_seed(count)
    start = torch.randn(count, generator=g) * 0.02
    # Each element has its own gradient magnitude, from 1e-6 to 10 (the same in every step, so
    # that FP32's error in a moment is relative to that element's own scale), and some
    # gradients are exactly zero (v stays small: the epsilon decides).
    magnitude = 10.0 ** torch.randint(-6, 2, (count,), generator=g).float()
    grads = [torch.randn(count, generator=g) * magnitude for _ in range(3)]
    grads[1][::7] = 0.0
    grad_scale = 1.0 / 1024.0
    p = start.to(DEV)
    m, v = torch.zeros(count, device=DEV), torch.zeros(count, device=DEV)
    half = torch.zeros(count + 8, dtype=torch.half, device=DEV)
    want = oracle_steps(start, grads, weight_decay, grad_scale)
    previous = start.double()
    for step, grad in enumerate(grads, start=1):
        flint.adamw(p, m, v, grad.to(DEV), half, count, HYPER["lr"], HYPER["beta1"], HYPER["beta2"],
                    HYPER["eps"], weight_decay, grad_scale, step)
        torch.cuda.synchronize()
        wp, wm, wv = want[step - 1]
        assert_close(p, wp, 1e-6, f"p at step {step}", torch.full_like(wp, HYPER["lr"]).maximum(previous.abs()))
        assert_close(m, wm, 1e-6, f"m at step {step}", magnitude * grad_scale)
        assert_close(v, wv, 1e-6, f"v at step {step}", (magnitude * grad_scale) ** 2)
        moved, expected = p.double().cpu() - previous, wp - previous
        assert ((moved - expected).abs() <= 1e-4 * expected.abs() + 1e-8).all(), step
        assert torch.equal(half[:count].view(torch.int16), p.half().view(torch.int16))
        assert not half[count:].any()
        previous = p.double().cpu()


def test_adamw_skip_flag_and_null_half_copy(flint):
    count = 1000
    g = torch.Generator().manual_seed(1)
    p = torch.randn(count, generator=g).to(DEV)
    m, v = torch.rand(count, generator=g).to(DEV), torch.rand(count, generator=g).to(DEV)
    grad = torch.randn(count, generator=g).to(DEV)
    before = (p.clone(), m.clone(), v.clone())
    skip = torch.ones(1, dtype=torch.int32, device=DEV)
    flint.adamw(p, m, v, grad, None, count, 6e-4, 0.9, 0.95, 1e-8, 0.1, 1.0, 1, skip)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip((p, m, v), before))
    skip.zero_()
    flint.adamw(p, m, v, grad, None, count, 6e-4, 0.9, 0.95, 1e-8, 0.1, 1.0, 1, skip)
    torch.cuda.synchronize()
    assert not torch.equal(p, before[0])
    with pytest.raises(flint_b200.FlintError, match="step .0. must be at least 1"):
        flint.adamw(p, m, v, grad, None, count, 6e-4, 0.9, 0.95, 1e-8, 0.1, 1.0, 0)


def test_adamw_run_updates_every_tensor_of_a_plan_with_its_own_decay(flint):
    """Tensors of ragged sizes (crossing the 8,192-value work items), two decay groups, FP16
    copies on some: three steps equal the oracle's, and a raised skip flag changes nothing."""
    g = torch.Generator().manual_seed(2)
    sizes = [(8192 * 2 + 4, 0.1, True), (768, 0.0, False), (5, 0.0, False), (8192, 0.1, True),
             (12, 0.1, False)]
    starts = [torch.randn(n, generator=g) * 0.02 for n, _, _ in sizes]
    ps = [s.to(DEV) for s in starts]
    ms = [torch.zeros(n, device=DEV) for n, _, _ in sizes]
    vs = [torch.zeros(n, device=DEV) for n, _, _ in sizes]
    gs = [torch.zeros(n, device=DEV) for n, _, _ in sizes]
    hs = [torch.zeros(n, dtype=torch.half, device=DEV) if h else None for n, _, h in sizes]
    plan, items = flint.adamw_plan([(p.data_ptr(), m.data_ptr(), v.data_ptr(), gr.data_ptr(),
                                     h.data_ptr() if h is not None else None, n, wd)
                                    for p, m, v, gr, h, (n, wd, _) in zip(ps, ms, vs, gs, hs, sizes)])
    assert items == sum(-(-n // 8192) for n, _, _ in sizes)
    grads = [[torch.randn(n, generator=g) for n, _, _ in sizes] for _ in range(3)]
    skip = torch.zeros(1, dtype=torch.int32, device=DEV)
    for step in (1, 2, 3):
        for gr, new in zip(gs, grads[step - 1]):
            gr.copy_(new)
        flint.adamw_run(plan, items, HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"], 0.5,
                        step, skip)
    torch.cuda.synchronize()
    for i, (n, wd, has_half) in enumerate(sizes):
        wp, wm, wv = oracle_steps(starts[i], [grads[s][i] for s in range(3)], wd, 0.5)[-1]
        assert_close(ps[i], wp, 1e-6, f"tensor {i} p", starts[i].abs().clamp_min(3 * HYPER["lr"]))
        assert_close(ms[i], wm, 1e-6, f"tensor {i} m", torch.stack([grads[s][i] for s in range(3)]).abs().amax(0))
        assert_close(vs[i], wv, 1e-6, f"tensor {i} v")
        if has_half:
            assert torch.equal(hs[i].view(torch.int16), ps[i].half().view(torch.int16))
    before = [p.clone() for p in ps]
    skip.fill_(1)
    flint.adamw_run(plan, items, HYPER["lr"], HYPER["beta1"], HYPER["beta2"], HYPER["eps"], 0.5, 4, skip)
    torch.cuda.synchronize()
    assert all(torch.equal(a, b) for a, b in zip(ps, before))


@pytest.mark.parametrize("count", [1, 5, 4096, 1_000_003])
def test_check_gradients_flags_nonfinite_values_and_sums_squares(flint, count):
    g = torch.Generator().manual_seed(count)
    grad = (torch.randn(count, generator=g) * 3).to(DEV)
    found = torch.zeros(1, dtype=torch.int32, device=DEV)
    total = torch.full((1,), 2.5, dtype=torch.float64, device=DEV)   # the call adds to it
    scale = 1.0 / 64.0
    flint.check_gradients(grad, count, scale, found, total)
    torch.cuda.synchronize()
    assert found.item() == 0
    want = 2.5 + float((grad.double().cpu() * scale).pow(2).sum())
    assert total.item() == pytest.approx(want, rel=1e-5)
    # The flag is only ever raised, so several calls can share it; a null sum is allowed.
    for position, bad in ((0, float("inf")), (count - 1, float("nan")), (count // 2, float("-inf"))):
        poisoned = grad.clone()
        poisoned[position] = bad
        found.zero_()
        flint.check_gradients(poisoned, count, scale, found, None)
        flint.check_gradients(grad, count, scale, found, None)
        torch.cuda.synchronize()
        assert found.item() == 1, (position, bad)


SMALL = dict(n_layer=2, n_head=2, n_embd=128, block_size=64, vocab_size=200, padded_vocab_size=208)


def u16(t):
    return torch.from_numpy(t.numpy().astype(np.uint16).view(np.int16)).to(DEV)


@pytest.mark.parametrize("max_grad_norm", [0.0, 1.0], ids=["no-clip", "clip-1.0"])
def test_trainer_steps_equal_the_oracle_train_step_weight_by_weight(flint, max_grad_norm):
    """Three optimizer steps of the trainer against the oracle's train_step (the reference's
    scripts/gpt2_torch.py:178-192: unscale, clip_grad_norm_(1.0), AdamW), compared weight by
    weight. Adam normalises each gradient by its own magnitude, so the comparison is made where
    it is well conditioned: on parameters whose oracle gradient is well above the FP16
    forward/backward noise the update must agree to a few per cent element-wise; for all
    parameters the update's direction must agree (cosine >= 0.99 per tensor with two or more
    dimensions) and its size must not exceed Adam's bound lr * (1 + small) per element."""
    g = torch.Generator().manual_seed(5)
    params = oracle.gpt2_round_to_half(oracle.gpt2_init(SMALL, seed=1234))
    for name in params:
        if name.endswith(".bias"):
            params[name] = (torch.randn(params[name].shape, generator=g) * 0.01).half().float()
    sequences, length = 3, 64
    config = TrainerConfig(layers=2, heads=2, width=128, block_size=64, vocab=200, padded_vocab=208,
                           sequences=sequences, length=length, loss_scale=1024.0,
                           max_grad_norm=max_grad_norm)
    trainer = Trainer(flint, config, state=params)
    ref = {k: v.clone() for k, v in params.items()}
    moments = {k: (torch.zeros_like(v), torch.zeros_like(v)) for k, v in ref.items()}
    try:
        norms = []
        for step in (1, 2, 3):
            idx, targets = oracle.synthetic_tokens(sequences, length, SMALL["vocab_size"], seed=30 + step)
            before = {k: v.clone() for k, v in ref.items()}
            want_loss, skipped, norm = oracle.train_step(SMALL, ref, moments, [(idx, targets)], step,
                                                         loss_scale=1024.0, max_grad_norm=max_grad_norm)
            norms.append(norm)
            assert not skipped
            trainer.step(u16(idx.flatten()), u16(targets.flatten()))
            loss = trainer.finish_step()
            assert abs(loss - want_loss) <= 1e-2
            if step > 1:
                continue
            # After the first step Adam's update is -lr * g / (|g| + eps'): its sign pattern.
            _, grads = oracle.gpt2_loss_and_gradients(SMALL, before, idx, targets)
            for name, address, rows, cols in trainer.model.parameters():
                got = trainer.model.read(address, (rows, cols), torch.float32).cpu()
                moved = got - before[name].reshape(rows, cols)
                expected = ref[name].reshape(rows, cols) - before[name].reshape(rows, cols)
                gradient = grads[name].reshape(rows, cols)
                strong = gradient.abs() > 0.05 * gradient.abs().max()
                assert strong.any()
                assert torch.allclose(moved[strong], expected[strong], rtol=0.05, atol=1e-6), name
                assert moved.abs().max().item() <= config.lr * 1.01 + 0.2 * config.lr * before[name].abs().max().item()
        assert trainer.skipped == 0 and trainer.step_count == 3
        if max_grad_norm:
            assert min(norms) > 1.2 * max_grad_norm          # every step was clipped
        all_moved, all_expected = [], []
        for name, address, rows, cols in trainer.model.parameters():
            got = trainer.model.read(address, (rows, cols), torch.float32).cpu()
            moved = got - params[name].reshape(rows, cols)
            expected = ref[name].reshape(rows, cols) - params[name].reshape(rows, cols)
            all_moved.append(moved.flatten())
            all_expected.append(expected.flatten())
            if rows > 1:
                cos = torch.nn.functional.cosine_similarity(moved.flatten().double(),
                                                            expected.flatten().double(), dim=0).item()
                assert cos >= 0.98, (name, cos)
        cos = torch.nn.functional.cosine_similarity(torch.cat(all_moved).double(),
                                                    torch.cat(all_expected).double(), dim=0).item()
        assert cos >= 0.99
        assert not flint.kernel_fault()
    finally:
        trainer.close()


def test_trainer_clip_coefficient_uses_the_norm_of_the_unscaled_gradients(flint):
    """The clip path in isolation: gradients written by hand into the model's arena (times the
    loss scale, as backward leaves them), the trainer's check + clip + AdamW run on them twice,
    against oracle.clip_coefficient and oracle.adamw_step element by element. Adam's first
    step does not depend on the gradient's scale, so the second one, whose moments mix two
    differently clipped gradients, is the one that pins the coefficient."""
    config = TrainerConfig(layers=2, heads=2, width=128, block_size=64, vocab=200, padded_vocab=208,
                           sequences=2, length=64, loss_scale=256.0, max_grad_norm=1.0)
    params = oracle.gpt2_round_to_half(oracle.gpt2_init(SMALL, seed=1234))
    trainer = Trainer(flint, config, state=params)
    try:
        g = torch.Generator().manual_seed(9)
        want = {k: v.double().flatten().clone() for k, v in params.items()}
        moments = {k: (torch.zeros_like(v), torch.zeros_like(v)) for k, v in want.items()}
        for step, sigma in ((1, 0.05), (2, 0.004), (3, 1e-4)):
            grads = {}
            trainer.gradients.zero_()
            for name, _, rows, cols, first in trainer.layout:
                grads[name] = torch.randn(rows * cols, generator=g) * sigma
                trainer.gradients[first:first + rows * cols] = (grads[name] * 256.0).to(DEV)
            previous = {name: trainer.model.read(address, (rows * cols,), torch.float32).cpu().double()
                        for name, address, rows, cols in trainer.model.parameters()}
            trainer.apply_update()
            torch.cuda.synchronize()
            assert trainer.found.item() == 0
            coefficient, norm = oracle.clip_coefficient(grads.values(), 1.0)
            assert math.sqrt(trainer.norm_squared.item()) == pytest.approx(norm, rel=1e-5)
            # Clipped hard, clipped a little, not clipped at all.
            assert (coefficient < 0.2, coefficient < 1.0) == {1: (True, True), 2: (False, True),
                                                              3: (False, False)}[step], coefficient
            for name, address, rows, cols in trainer.model.parameters():
                wd = oracle.WEIGHT_DECAY if oracle.decayed(name, params[name].shape) else 0.0
                before = want[name].clone()
                oracle.adamw_step(want[name], *moments[name], grads[name].double() * coefficient, step,
                                  weight_decay=wd)
                got = trainer.model.read(address, (rows * cols,), torch.float32).cpu().double()
                moved, expected = got - previous[name], want[name] - before
                # FP32 rounds the new weight to 2^-24 of itself (LayerNorm gains are near 1).
                rounding = 2.0 ** -23 * previous[name].abs().clamp_min(0.05)
                assert ((moved - expected).abs() <= 2e-4 * expected.abs() + rounding).all(), (step, name)
    finally:
        trainer.close()
