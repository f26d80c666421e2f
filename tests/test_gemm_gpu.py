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


# ---- the logits shapes of the GPT-2 sweep at full size ----------------------------------------
# 8192 x 50304 x 768 and its two gradients. The float64 product of the whole matrix would take
# minutes on the host, so sampled rows / columns are compared (every tile column of the output
# is crossed by a sampled row and every tile row by a sampled column) and the rest is covered by
# a checksum identity: the sum over an output row equals x_row . (sum of w's rows).

VOCAB_COLUMNS = 50304


def sample(count, size, seed):
    g = torch.Generator().manual_seed(seed)
    picked = torch.randperm(size, generator=g)[:count]
    edge = torch.tensor([0, size - 1, size // 2])
    return torch.unique(torch.cat([picked, edge]))


def test_gemm_nt_at_the_full_logits_shape(flint):
    m, n, k = GPT2_ROWS, VOCAB_COLUMNS, 768
    x, w = inputs((m, k), (n, k), 50)
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    flint.gemm_nt(y, x.to(DEV), w.to(DEV), m, n, k)
    no_fault(flint)
    rows = sample(48, m, 1)
    assert rel_error(y[rows.to(DEV)], oracle.gemm_nt(x[rows], w)) <= 2e-3
    cols = sample(48, n, 2)
    assert rel_error(y[:, cols.to(DEV)], oracle.gemm_nt(x, w[cols])) <= 2e-3
    # Every element takes part: row sums against x . sum(w) in float64.
    want = x.double() @ w.double().sum(0)
    got = y.double().sum(1).cpu()
    scale = (x.double().abs() @ w.double().abs().sum(0))
    assert ((got - want).abs() <= 2e-3 * scale).all()


def test_gemm_nn_at_the_full_logits_gradient_shape(flint):
    m, n, k = GPT2_ROWS, 768, VOCAB_COLUMNS
    g = torch.Generator().manual_seed(51)
    x = (torch.randn(m, k, generator=g) * 0.05).half()
    w = (torch.randn(k, n, generator=g) * 0.02).half()
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    flint.gemm_nn(y, x.to(DEV), w.to(DEV), m, n, k)
    no_fault(flint)
    rows = sample(48, m, 3)
    assert rel_error(y[rows.to(DEV)], oracle.gemm_nn(x[rows], w)) <= 2e-3
    cols = sample(24, n, 4)
    assert rel_error(y[:, cols.to(DEV)], oracle.gemm_nn(x, w[:, cols])) <= 2e-3


def test_gemm_tn_at_the_full_tied_weight_gradient_shape(flint):
    m, n, k = VOCAB_COLUMNS, 768, GPT2_ROWS
    g = torch.Generator().manual_seed(52)
    x = (torch.randn(k, m, generator=g) * 0.05).half()
    w = torch.randn(k, n, generator=g).half()
    ws = torch.empty(max(flint.gemm_tn_workspace(m, n, k), 16), dtype=torch.uint8, device=DEV)
    xd, wd = x.to(DEV), w.to(DEV)
    y = torch.full((m, n), 3.0, device=DEV)
    flint.gemm_tn(y, xd, wd, m, n, k, False, ws)
    old = torch.randn(m, n, generator=g).to(DEV)
    acc = old.clone()
    flint.gemm_tn(acc, xd, wd, m, n, k, True, ws)
    no_fault(flint)
    rows = sample(48, m, 5)
    assert rel_error(y[rows.to(DEV)], oracle.gemm_tn(x[:, rows], w)) <= 1e-4
    cols = sample(16, n, 6)
    assert rel_error(y[:, cols.to(DEV)], oracle.gemm_tn(x, w[:, cols])) <= 1e-4
    assert torch.equal(acc, old + y)


# ---- the GELU and its derivative, point by point -------------------------------------------------
# With x = 0 every sum is exactly the bias, so y must be GELU(bias) rounded once to FP16; with
# a one-hot x and w every sum is exactly dh, so y must be dh * GELU'(pre) rounded once. The
# bounds are the reference's (tests/test_gemm_bias_gelu.py:255-306, tests/test_gemm_dgelu.py:377-406):
# within one FP16 ulp everywhere, and the correctly rounded value wherever the exact result is
# farther from a rounding boundary than the FP32 evaluation's error model.


def gelu_sweep():
    g = torch.Generator().manual_seed(7)
    grid = torch.linspace(-12.0, 12.0, 32768, dtype=torch.float64)
    random = torch.rand(16384, generator=g, dtype=torch.float64) * 24 - 12
    extremes = []
    for magnitude in (1e-40, 1e-30, 2.0 ** -25, 6e-8, 1e-5, 65504.0, 65519.0, 65520.0, 65536.0, 1e5,
                      1e6, 1e30, 3.4028234e38, 20.0, 30.0, 100.0, 1000.0, 1e4, 65000.0):
        extremes += [magnitude, -magnitude]
    extremes.append(0.0)
    return torch.cat([grid, random, torch.tensor(extremes, dtype=torch.float64)]).float()


def test_gelu_is_the_correctly_rounded_function_of_the_unrounded_sum(flint):
    bias = gelu_sweep()
    n = bias.numel()
    m, k = 2, 8
    x = torch.zeros(m, k, dtype=torch.half, device=DEV)
    w = torch.ones(n, k, dtype=torch.half, device=DEV)
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    pre = torch.zeros_like(y)
    flint.gemm_nt_bias_gelu(y, pre, x, w, bias.to(DEV), m, n, k)
    no_fault(flint)
    y, pre = y.cpu(), pre.cpu()
    assert torch.equal(pre.view(torch.int16), bias.half().expand(m, n).contiguous().view(torch.int16))
    assert torch.equal(y[0].view(torch.int16), y[1].view(torch.int16))
    exact64 = oracle.gelu_tanh(bias.double())
    exact = oracle.round_to_half(exact64)
    distance = (oracle.half_ordered(y[0]) - oracle.half_ordered(exact)).abs()
    assert distance.max().item() <= 1, bias[distance.argmax()].item()
    safe = oracle.half_rounding_margin(exact64) > 2.0 ** -21 * (2 + oracle.gelu_exponent(bias).abs())
    assert safe.sum() > 0.95 * n
    wrong = safe & (oracle.half_ordered(y[0]) != oracle.half_ordered(exact))
    assert not wrong.any(), (int(wrong.sum()), bias[wrong][0].item())
    # GELU of the FP32 sum, not of the sum rounded to FP16 first.
    from_pre = oracle.round_to_half(oracle.gelu_tanh(bias.half().double()))
    differs = safe & (oracle.half_ordered(from_pre) != oracle.half_ordered(exact))
    assert differs.sum() > 1000
    assert (oracle.half_ordered(y[0])[differs] != oracle.half_ordered(from_pre)[differs]).all()


def test_gelu_derivative_is_within_one_ulp_and_correctly_rounded_where_that_is_defined(flint):
    all_bits = torch.arange(-32768, 32768, dtype=torch.int32).to(torch.int16)
    values = all_bits.view(torch.float16)
    s = values[torch.isfinite(values)]
    n = s.numel()
    assert n == 63488
    sweep_dh = [1.0, 1000.0, 2.0 ** -10, -1.0, -3.0, float(np.float16(0.1))]
    m, k = len(sweep_dh), 8
    x = torch.zeros(m, k, dtype=torch.half)
    x[:, 0] = torch.tensor(sweep_dh).half()
    w = torch.zeros(k, n, dtype=torch.half)
    w[0] = 1
    y = torch.zeros(m, n, dtype=torch.half, device=DEV)
    flint.gemm_nn_dgelu(y, x.to(DEV), w.to(DEV), s[None, :].expand(m, n).contiguous().to(DEV), m, n, k)
    no_fault(flint)
    y = y.cpu()
    g, a = oracle.gelu_tanh_derivative(s)           # a is the forward form's exponent (-2c(...))
    dh = x[:, 0].double()[:, None]
    v = dh * g[None, :]
    exact = oracle.round_to_half(v)
    root, window, root_e = -0.7525, 0.25, 1e-7       # the derivative's zero: absolute bound there
    near_root = ((s.double() - root).abs() < window)[None, :].expand(m, n)
    distance = (oracle.half_ordered(y) - oracle.half_ordered(exact)).abs()
    close = (y.double() - v).abs() <= dh.abs() * root_e
    wrong = (distance > 1) & ~(near_root & close)
    assert not wrong.any(), int(wrong.sum())
    relative = 2.0 ** -21 * (2 + a.clamp(min=0))
    absolute = torch.where(near_root[0], root_e / g.abs(), torch.zeros_like(g))
    safe = oracle.half_rounding_margin(v) > (relative + absolute)[None, :]
    assert safe.sum() > 0.95 * safe.numel()
    wrong = safe & (oracle.half_ordered(y) != oracle.half_ordered(exact))
    assert not wrong.any(), int(wrong.sum())
