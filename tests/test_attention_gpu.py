"""Fused causal attention (extension) against the float64 oracle, on a B200.

Oracle: softmax(scale * Q K^T + causal mask) V and its autograd gradients in float64
(oracle.attention), the same chain the reference's tests/test_softmax_backward.py:1429-1440
uses for its unfused kernels. Tolerance: relative Frobenius error <= 2e-3 forward (the
GEMM bound) and <= 5e-3 for the gradients (P and dS round to FP16 before their GEMMs).
"""

import numpy as np
import pytest
import torch

import flint_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def rel_error(got, want):
    got = got.double().cpu()
    want = torch.as_tensor(np.asarray(want)).double()
    return ((got - want).norm() / want.norm().clamp_min(1e-300)).item()


# The last two cases give the backward kernels more items than a B200 has SMs (39 x 8 = 312 and
# 101 x 3 = 303 items for 148 persistent CTAs): two full rounds and a short third one.
@pytest.mark.parametrize("batches, length", [(4, 128), (3, 256), (2, 1024), (5, 40), (2, 136),
                                             (1, 8), (7, 520), (39, 1024), (101, 328)])
def test_attention_forward_and_backward(flint, batches, length):
    g = torch.Generator().manual_seed(length)
    q, k, v, d_o = (torch.randn(batches, length, 64, generator=g).half() for _ in range(4))
    scale = 0.125
    o = torch.full((batches, length, 64), 7.0, dtype=torch.half, device=DEV)
    lse = torch.zeros(batches, length, device=DEV)
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, d_o))
    flint.attention_forward(o, lse, qd, kd, vd, batches, length, 64, scale)
    dq, dk, dv = (torch.full((batches, length, 64), 7.0, dtype=torch.half, device=DEV)
                  for _ in range(3))
    delta = torch.zeros(batches, length, device=DEV)
    flint.attention_backward(dq, dk, dv, dod, o, lse, delta, qd, kd, vd, batches, length, 64,
                             scale)
    torch.cuda.synchronize()
    assert not flint.kernel_fault()
    want_o, want_lse, want_dq, want_dk, want_dv = oracle.attention(q, k, v, scale, d_o)
    assert rel_error(o, want_o) <= 2e-3
    assert np.allclose(lse.cpu().numpy(), want_lse, rtol=1e-4, atol=1e-4)
    assert rel_error(dq, want_dq) <= 5e-3
    assert rel_error(dk, want_dk) <= 5e-3
    assert rel_error(dv, want_dv) <= 5e-3


def test_attention_is_deterministic_and_row_zero_copies_v(flint):
    batches, length = 12, 1024
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(batches, length, 64, generator=g).half().to(DEV) for _ in range(3))
    outs = []
    for fill in (1.0, -3.0):
        o = torch.full((batches, length, 64), fill, dtype=torch.half, device=DEV)
        lse = torch.zeros(batches, length, device=DEV)
        flint.attention_forward(o, lse, q, k, v, batches, length, 64, 0.125)
        outs.append(o)
    torch.cuda.synchronize()
    assert torch.equal(outs[0].view(torch.int16), outs[1].view(torch.int16))
    assert torch.equal(outs[0][:, 0].view(torch.int16), v[:, 0].view(torch.int16))


def test_attention_backward_is_deterministic_over_many_items(flint):
    """Persistent CTAs take several items each; every output element still comes from one
    CTA in a fixed order, so two runs agree bit for bit."""
    batches, length = 60, 1024
    g = torch.Generator().manual_seed(5)
    q, k, v, d_o = (torch.randn(batches, length, 64, generator=g).half().to(DEV) for _ in range(4))
    o = torch.zeros(batches, length, 64, dtype=torch.half, device=DEV)
    lse = torch.zeros(batches, length, device=DEV)
    flint.attention_forward(o, lse, q, k, v, batches, length, 64, 0.125)
    runs = []
    for fill in (2.0, -5.0):
        grads = [torch.full((batches, length, 64), fill, dtype=torch.half, device=DEV)
                 for _ in range(3)]
        delta = torch.full((batches, length), fill, device=DEV)
        flint.attention_backward(*grads, d_o, o, lse, delta, q, k, v, batches, length, 64, 0.125)
        runs.append(grads)
    torch.cuda.synchronize()
    assert not flint.kernel_fault()
    for a, b in zip(*runs):
        assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_mma_clock_probe(flint):
    """The diagnostic behind `kernel_bench --group mma`: sane numbers and argument checks."""
    import ctypes

    from flint_b200.binding import FlintError
    from flint_b200.kernel_bench import mma_rates

    rates = {r["case"]: r for r in mma_rates(flint, 128)}
    assert len(rates) == 4
    for r in rates.values():
        # No MMA can beat the tensor work of its shape; none should take ten times as long.
        assert r["tensor_clocks_each"] * 0.9 <= r["complete_clocks_each"] <= r["tensor_clocks_each"] * 10
        assert r["issue_clocks_each"] <= r["complete_clocks_each"]
    clocks = ctypes.c_longlong()
    for n, count in ((96, 16), (64, 0), (64, 5000)):
        with pytest.raises(FlintError):
            flint.check(flint.lib.flint_b200_mma_clocks(n, 0, count, ctypes.byref(clocks),
                                                        ctypes.byref(clocks), None))
    assert not flint.kernel_fault()


def test_attention_does_not_depend_on_cache_state(flint):
    """The kernels' roles meet only through mbarriers, so a result must not depend on how
    long a load takes. Each trial first pushes Q, K, V out of the L2 with a 512 MB write
    (loads then arrive late and out of step with the tensor pipe) and fills the outputs
    with a different value; every trial must give the first trial's bits, and the first
    trial must match torch's attention. 192 (sequence, head) pairs are the training step's
    count and give every persistent CTA several items in a row."""
    batches, length = 192, 1024
    g = torch.Generator(device=DEV).manual_seed(11)
    q, k, v, d_o = (torch.randn(batches, length, 64, generator=g, device=DEV).half()
                    for _ in range(4))
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=DEV)
    first = None
    for trial in range(10):
        fill = float(trial + 1)
        o = torch.full((batches, length, 64), fill, dtype=torch.half, device=DEV)
        lse = torch.full((batches, length), fill, device=DEV)
        grads = [torch.full((batches, length, 64), fill, dtype=torch.half, device=DEV)
                 for _ in range(3)]
        delta = torch.full((batches, length), fill, device=DEV)
        flush.fill_(trial)
        flint.attention_forward(o, lse, q, k, v, batches, length, 64, 0.125)
        flush.fill_(trial + 100)
        flint.attention_backward(*grads, d_o, o, lse, delta, q, k, v, batches, length, 64, 0.125)
        torch.cuda.synchronize()
        assert not flint.kernel_fault()
        got = [o, lse, *grads]
        if first is None:
            first = got
            leaves = [t.clone().requires_grad_(True) for t in (q, k, v)]
            want = torch.nn.functional.scaled_dot_product_attention(*leaves, is_causal=True,
                                                                    scale=0.125)
            want_grads = torch.autograd.grad(want, leaves, d_o)
            for mine, theirs in zip([o, *grads], [want, *want_grads]):
                error = (mine.float() - theirs.float()).norm() / theirs.float().norm()
                assert error.item() <= 2e-3
            continue
        for what, a, b in zip(("o", "lse", "dq", "dk", "dv"), first, got):
            assert torch.equal(a.view(torch.int32 if a.dtype == torch.float32 else torch.int16),
                               b.view(torch.int32 if b.dtype == torch.float32 else torch.int16)), \
                f"{what} differs in trial {trial}"


@pytest.mark.parametrize("case", ["at_a", "at_b", "at_c"])
def test_attention_matches_the_golden_vectors(flint, golden, case):
    """Known answers made by the reference's float64 attention chain
    (tests/golden/make_golden.py: float_references)."""
    g = golden("float_references")
    q, k, v, d_o = (torch.from_numpy(g[case + n]).to(DEV) for n in ("_q", "_k", "_v", "_do"))
    batches, length, _ = q.shape
    o = torch.zeros_like(q)
    lse = torch.zeros(batches, length, device=DEV)
    flint.attention_forward(o, lse, q, k, v, batches, length, 64, 0.125)
    dq, dk, dv = (torch.zeros_like(q) for _ in range(3))
    delta = torch.zeros(batches, length, device=DEV)
    flint.attention_backward(dq, dk, dv, d_o, o, lse, delta, q, k, v, batches, length, 64, 0.125)
    torch.cuda.synchronize()
    assert not flint.kernel_fault()
    assert rel_error(o, g[case + "_o"]) <= 2e-3
    assert rel_error(dq, g[case + "_dq"]) <= 5e-3
    assert rel_error(dk, g[case + "_dk"]) <= 5e-3
    assert rel_error(dv, g[case + "_dv"]) <= 5e-3
