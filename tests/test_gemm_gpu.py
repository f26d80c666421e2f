"""Parity of the tensor-core GEMMs with the oracle, through the C ABI on a B200.

Tolerance: relative Frobenius error <= 2e-3 against the float64 product of the same FP16
inputs (FP16 outputs), <= 1e-4 for TN's FP32 output; plus the bit identities the
reference pins between variants (tests/test_gemm*.py): batched == plain per batch,
bias of -0 == plain, dGELU at pre = +inf == NN, accumulate == old + plain, run-to-run
determinism, integer-exact products, NaN/inf placement and the argument errors' texts.
"""

import numpy as np
import pytest
import torch

import flint_b200
import flint_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
GPT2_ROWS = 8192


def rel_error(got, want):
    got = got.double().cpu()
    want = torch.as_tensor(np.asarray(want)).double()
    return ((got - want).norm() / want.norm().clamp_min(1e-300)).item()


def inputs(shape_x, shape_w, seed, sigma_w=0.02):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(*shape_x, generator=g).half()
    w = (torch.randn(*shape_w, generator=g) * sigma_w).half()
    return x, w


def no_fault(flint):
    torch.cuda.synchronize()
    assert not flint.kernel_fault()


NT_SHAPES = [(GPT2_ROWS, 2304, 768), (GPT2_ROWS, 768, 768), (GPT2_ROWS, 3072, 768),
             (GPT2_ROWS, 768, 3072), (512, 50304, 768),
             (1, 1, 8), (100, 50, 72), (129, 257, 8), (300, 333, 1000), (128, 64, 64)]


@pytest.mark.parametrize("m, n, k", NT_SHAPES)
def test_gemm_nt(flint, m, n, k):
    x, w = inputs((m, k), (n, k), m + n + k)
    guard = 64
    y = torch.full((m * n + 2 * guard,), 7.0, dtype=torch.half, device=DEV)
    flint.gemm_nt(y.data_ptr() + 2 * guard, x.to(DEV), w.to(DEV), m, n, k)
    no_fault(flint)
    assert rel_error(y[guard:guard + m * n].view(m, n), oracle.gemm_nt(x, w)) <= 2e-3
    assert bool((y[:guard] == 7).all()) and bool((y[guard + m * n:] == 7).all())


@pytest.mark.parametrize("m, n, k", [(GPT2_ROWS, 768, 2304), (GPT2_ROWS, 768, 768),
                                     (GPT2_ROWS, 768, 3072), (GPT2_ROWS, 3072, 768),
                                     (512, 768, 50304), (100, 56, 72), (1, 8, 8), (130, 264, 40)])
def test_gemm_nn(flint, m, n, k):
    x, w = inputs((m, k), (k, n), m + n + k)
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    flint.gemm_nn(y, x.to(DEV), w.to(DEV), m, n, k)
    no_fault(flint)
    assert rel_error(y, oracle.gemm_nn(x, w)) <= 2e-3


@pytest.mark.parametrize("m, n, k", [(2304, 768, GPT2_ROWS), (768, 768, GPT2_ROWS),
                                     (3072, 768, GPT2_ROWS), (768, 3072, GPT2_ROWS),
                                     (50304, 768, 1024), (8, 8, 1), (104, 56, 77),
                                     (8, 8, 16384), (136, 120, 3000), (296, 200, 2049)])
def test_gemm_tn_writes_and_accumulates(flint, m, n, k):
    g = torch.Generator().manual_seed(m + n + k)
    x = torch.randn(k, m, generator=g).half()
    w = torch.randn(k, n, generator=g).half()
    nbytes = flint.gemm_tn_workspace(m, n, k)
    assert nbytes % (m * n * 4) == 0 and nbytes // (m * n * 4) <= 16
    ws = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)
    xd, wd = x.to(DEV), w.to(DEV)
    y = torch.full((m, n), 3.0, device=DEV)
    flint.gemm_tn(y, xd, wd, m, n, k, False, ws)
    again = torch.full((m, n), -5.0, device=DEV)
    flint.gemm_tn(again, xd, wd, m, n, k, False, ws)
    old = torch.randn(m, n, generator=g).to(DEV)
    acc = old.clone()
    flint.gemm_tn(acc, xd, wd, m, n, k, True, ws)
    no_fault(flint)
    assert rel_error(y, oracle.gemm_tn(x, w)) <= 1e-4
    assert torch.equal(y, again)                      # deterministic
    assert torch.equal(acc, old + y)                  # one FP32 add


def test_gemm_tn_workspace_rules(flint):
    # k below 2,048 never splits; shapes whose tiles already fill the GPU need none.
    for shape in [(8, 8, 1), (8, 8, 1000), (136, 120, 1023), (8, 8, 1024), (50304, 768, 1024),
                  (50304, 768, 65536), (4096, 4096, 65536), (2304, 768, 1024)]:
        assert flint.gemm_tn_workspace(*shape) == 0, shape
    for shape in [(8, 8, 16384), (136, 120, 3000), (296, 200, 2049), (1032, 8, 4096),
                  (2056, 16, 8192)]:
        assert flint.gemm_tn_workspace(*shape) > 0, shape
    with pytest.raises(flint_b200.FlintError, match=r"needs \d+ bytes of workspace, given 0"):
        x = torch.zeros(16384, 8, dtype=torch.half, device=DEV)
        y = torch.zeros(8, 8, device=DEV)
        flint.gemm_tn(y, x, x, 8, 8, 16384, False, None)


@pytest.mark.parametrize("m, n, k", [(GPT2_ROWS, 2304, 768), (GPT2_ROWS, 768, 3072), (100, 50, 72)])
def test_gemm_nt_bias(flint, m, n, k):
    x, w = inputs((m, k), (n, k), 1 + m)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(2)) * 0.5
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    flint.gemm_nt_bias(y, x.to(DEV), w.to(DEV), bias.to(DEV), m, n, k)
    plain = torch.zeros_like(y)
    flint.gemm_nt(plain, x.to(DEV), w.to(DEV), m, n, k)
    minus_zero = torch.zeros_like(y)
    flint.gemm_nt_bias(minus_zero, x.to(DEV), w.to(DEV), torch.full((n,), -0.0, device=DEV), m, n, k)
    no_fault(flint)
    assert rel_error(y, oracle.gemm_nt(x, w, bias)) <= 2e-3
    assert torch.equal(minus_zero.view(torch.int16), plain.view(torch.int16))


@pytest.mark.parametrize("m, n, k", [(GPT2_ROWS, 3072, 768), (100, 50, 72)])
def test_gemm_nt_bias_gelu(flint, m, n, k):
    x, w = inputs((m, k), (n, k), 3 + m, sigma_w=0.05)
    bias = torch.randn(n, generator=torch.Generator().manual_seed(4)) * 0.5
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    pre = torch.zeros_like(y)
    flint.gemm_nt_bias_gelu(y, pre, x.to(DEV), w.to(DEV), bias.to(DEV), m, n, k)
    no_fault(flint)
    want_pre, want_y = oracle.gemm_nt_bias_gelu(x, w, bias)
    assert rel_error(pre, want_pre) <= 2e-3
    assert rel_error(y, want_y) <= 2e-3
    # GELU is applied to the unrounded sum: y is within one FP16 ulp of gelu(exact s).
    ulp = np.spacing(np.abs(want_y.numpy()).astype(np.float16)).astype(np.float64)
    close = np.abs(y.double().cpu().numpy() - want_y.numpy()) <= 2 * ulp + 1e-3 * np.abs(want_y.numpy())
    assert close.mean() > 0.999


@pytest.mark.parametrize("m, n, k", [(GPT2_ROWS, 3072, 768), (100, 56, 72)])
def test_gemm_nn_dgelu(flint, m, n, k):
    x, w = inputs((m, k), (k, n), 5 + m, sigma_w=0.05)
    pre = (torch.randn(m, n, generator=torch.Generator().manual_seed(6)) * 2).half()
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    flint.gemm_nn_dgelu(y, x.to(DEV), w.to(DEV), pre.to(DEV), m, n, k)
    at_inf = torch.zeros_like(y)
    flint.gemm_nn_dgelu(at_inf, x.to(DEV), w.to(DEV),
                        torch.full((m, n), float("inf"), dtype=torch.half, device=DEV), m, n, k)
    plain = torch.zeros_like(y)
    flint.gemm_nn(plain, x.to(DEV), w.to(DEV), m, n, k)
    no_fault(flint)
    assert rel_error(y, oracle.gemm_nn_dgelu(x, w, pre)) <= 2e-3
    assert torch.equal(at_inf.view(torch.int16), plain.view(torch.int16))


@pytest.mark.parametrize("m, n, k", [(GPT2_ROWS, 768, 768), (GPT2_ROWS, 768, 3072), (100, 50, 72),
                                     (33, 6, 8)])
def test_gemm_nt_bias_residual(flint, m, n, k):
    x, w = inputs((m, k), (n, k), 7 + m)
    g = torch.Generator().manual_seed(8)
    bias = torch.randn(n, generator=g) * 0.5
    residual = torch.randn(m, n, generator=g).half().float()
    y = torch.zeros(m, n, device=DEV)
    flint.gemm_nt_bias_residual(y, x.to(DEV), w.to(DEV), bias.to(DEV), residual.to(DEV), m, n, k)
    no_fault(flint)
    want = residual.double() + oracle.gemm_nt(x, w, bias)
    assert rel_error(y, want) <= 1e-5


def test_batched_gemms_equal_the_plain_ones_per_batch(flint):
    batches, t, d = 6, 264, 64
    g = torch.Generator().manual_seed(9)
    q = torch.randn(batches, t, d, generator=g).half().to(DEV)
    k = torch.randn(batches, t, d, generator=g).half().to(DEV)
    p = torch.rand(batches, t, t, generator=g).half().to(DEV)
    s = torch.zeros(batches, t, t, dtype=torch.half, device=DEV)
    flint.gemm_nt_batched(s, q, k, batches, t, t, d, 1.0)
    o = torch.zeros(batches, t, d, dtype=torch.half, device=DEV)
    flint.gemm_nn_batched(o, p, k, batches, t, d, t)
    dv = torch.zeros(batches, t, d, dtype=torch.half, device=DEV)
    flint.gemm_tn_batched(dv, p, q, batches, t, d, t)
    for j in range(batches):
        one = torch.zeros(t, t, dtype=torch.half, device=DEV)
        flint.gemm_nt(one, q[j], k[j], t, t, d)
        assert torch.equal(one.view(torch.int16), s[j].view(torch.int16))
        one = torch.zeros(t, d, dtype=torch.half, device=DEV)
        flint.gemm_nn(one, p[j], k[j], t, d, t)
        assert torch.equal(one.view(torch.int16), o[j].view(torch.int16))
        full = torch.zeros(t, d, device=DEV)
        flint.gemm_tn(full, p[j], q[j], t, d, t, False, None)
        assert torch.equal(full.half().view(torch.int16), dv[j].view(torch.int16))
    no_fault(flint)
    scaled = torch.zeros_like(s)
    flint.gemm_nt_batched(scaled, q, k, batches, t, t, d, 0.125)
    assert rel_error(scaled, oracle.gemm_nt(q.cpu(), k.cpu()) * 0.125) <= 2e-3


def test_attention_shaped_batched_gemms_at_gpt2_size(flint):
    batches, t, d = 96, 1024, 64
    g = torch.Generator().manual_seed(10)
    q = torch.randn(batches, t, d, generator=g).half()
    k = torch.randn(batches, t, d, generator=g).half()
    s = torch.zeros(batches, t, t, dtype=torch.half, device=DEV)
    flint.gemm_nt_batched(s, q.to(DEV), k.to(DEV), batches, t, t, d, 0.125)
    no_fault(flint)
    for j in (0, 41, 95):
        assert rel_error(s[j], oracle.gemm_nt(q[j], k[j]) * 0.125) <= 2e-3


def test_integer_products_are_exact_and_nonfinite_values_propagate(flint):
    m, n, k = 64, 72, 65536
    x = torch.ones(m, k, dtype=torch.half, device=DEV)
    w = torch.zeros(n, k, dtype=torch.half, device=DEV)
    w[:, :2048] = 1.0
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    flint.gemm_nt(y, x, w, m, n, k)
    torch.cuda.synchronize()
    assert bool((y == 2048).all())
    x[3, 5] = float("nan")
    x[7, 9] = float("inf")
    flint.gemm_nt(y, x, w, m, n, k)
    torch.cuda.synchronize()
    assert bool(torch.isnan(y[3]).all()) and bool(torch.isinf(y[7]).all())
    assert bool((y[[0, 1, 2, 4, 5, 6]] == 2048).all())
    big = torch.full((8, 8), 300.0, dtype=torch.half, device=DEV)
    out = torch.zeros(8, 8, dtype=torch.half, device=DEV)
    flint.gemm_nt(out, big, big, 8, 8, 8)
    torch.cuda.synchronize()
    assert bool(torch.isinf(out).all())  # 720,000 overflows FP16


def test_argument_errors_name_the_problem(flint):
    a = torch.zeros(64, 64, dtype=torch.half, device=DEV)
    b = torch.zeros(64, 64, dtype=torch.half, device=DEV)
    c = torch.zeros(64, 64, dtype=torch.half, device=DEV)
    cases = [
        (lambda: flint.gemm_nt(c, a, b, 8, 8, 12), "k (12) must be a positive multiple of 8"),
        (lambda: flint.gemm_nn(c, a, b, 8, 12, 8), "n (12) must be a multiple of 8"),
        (lambda: flint.gemm_nt(c, a, b, 8, 8, 1 << 17), "too large"),
        (lambda: flint.gemm_nt(None, a, b, 8, 8, 8), "y is null"),
        (lambda: flint.gemm_nt(c.data_ptr() + 2, a, b, 8, 8, 8), "y is not 16-byte aligned"),
        (lambda: flint.gemm_nt(a, a, b, 8, 8, 8), "y and x overlap"),
        (lambda: flint.gemm_nt(b, a, b, 8, 8, 8), "y and w overlap"),
        (lambda: flint.gemm_nt_bias(c, a, b, None, 8, 8, 8), "bias is null"),
        (lambda: flint.gemm_nt_bias_residual(c, a, b, a, a, 8, 7, 8), "n (7) must be even"),
        (lambda: flint.gemm_tn(c, a, b, 12, 8, 8), "m (12) must be a multiple of 8"),
        (lambda: flint.gemm_tn(c, a, b, 8, 8, 0), "k must be positive"),
        (lambda: flint.gemm_nt_batched(c, a, b, 1, 8, 8, 8, float("inf")), "must be finite"),
        (lambda: flint.gemm_nt_batched(c, a, b, 70000, 8, 8, 8, 1.0), "batches (70000) can be up to 65535"),
        (lambda: flint.gemm_nn_batched(c, a, b, 1, 2048, 8, 8), "m (2048) can be up to 1024"),
    ]
    for call, text in cases:
        with pytest.raises(flint_b200.FlintError) as error:
            call()
        assert text in str(error.value) and text in flint.last_error()
        assert error.value.status == flint_b200.ERROR_INVALID_ARGUMENT
    # Zero-sized problems succeed even with null pointers.
    flint.gemm_nt(None, None, None, 0, 8, 8)
    flint.gemm_tn(None, None, None, 8, 0, 8)
    flint.gemm_nn_batched(None, None, None, 0, 8, 8, 8)
