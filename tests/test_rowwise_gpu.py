"""Parity of the bandwidth-bound kernels with the oracle, through the C ABI on a B200.

Bit-exact where the reference pins the arithmetic (bias gradient, LayerNorm backward,
softmax backward, embedding forward/backward, convert, copy, heads), within 1 FP16
ulp / the reference's stated tolerances elsewhere. Modelled on the reference's
tests/test_bias_gradient.py, test_layernorm*.py, test_softmax*.py, test_cross_entropy.py,
test_embedding*.py, test_convert.py, test_copy.py and test_heads.py.
"""

import numpy as np
import pytest
import torch

import flint_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bits(t):
    """Bit pattern of a float tensor with NaNs canonicalised (payloads are not promised)."""
    t = t.detach().cpu()
    view = {2: torch.int16, 4: torch.int32}[t.element_size()]
    canonical = torch.where(torch.isnan(t), torch.full_like(t, float("nan")), t)
    return canonical.view(view)


def same_bits(a, b):
    return torch.equal(bits(a), bits(torch.as_tensor(np.asarray(b)) if not torch.is_tensor(b) else b))


def crafted(rng, shape, spread=6):
    base = rng.standard_normal(shape)
    return np.clip(base * np.exp2(rng.integers(-spread, spread + 1, shape)), -60000, 60000)


def workspace(nbytes):
    return torch.empty(max(nbytes, 16), dtype=torch.uint8, device=DEV)


def tokens16(values):
    """uint16 bit patterns in an int16 tensor."""
    a = np.asarray(values).astype(np.uint16)
    return torch.from_numpy(a.view(np.int16)).to(DEV)


# ---- copy / convert / heads / embedding forward ---------------------------------------------


@pytest.mark.parametrize("nbytes", [1, 15, 16, 17, 4099, 1 << 20, (16 << 20) + 5])
@pytest.mark.parametrize("offsets", [(0, 0), (1, 1), (3, 5), (16, 0), (0, 8)])
def test_copy_is_bitwise_for_any_size_and_alignment(flint, nbytes, offsets):
    so, do = offsets
    src = torch.randint(0, 256, (nbytes + 64,), dtype=torch.uint8, device=DEV)
    dst = torch.full((nbytes + 64,), 0xA5, dtype=torch.uint8, device=DEV)
    flint.copy(dst.data_ptr() + do, src.data_ptr() + so, nbytes)
    torch.cuda.synchronize()
    assert torch.equal(dst[do:do + nbytes], src[so:so + nbytes])
    assert bool((dst[:do] == 0xA5).all()) and bool((dst[do + nbytes:] == 0xA5).all())


def test_copy_rejects_overlap_and_null(flint):
    import flint_b200

    a = torch.zeros(64, dtype=torch.uint8, device=DEV)
    with pytest.raises(flint_b200.FlintError, match="dst and src overlap"):
        flint.copy(a.data_ptr() + 8, a.data_ptr(), 16)
    with pytest.raises(flint_b200.FlintError, match="dst is null"):
        flint.copy(None, a, 16)
    flint.copy(None, None, 0)  # zero bytes succeeds with null pointers


@pytest.mark.parametrize("count", [1, 7, 8, 9, 1023, 768 * 8192 + 3])
def test_convert_rounds_to_nearest_even(flint, count):
    g = torch.Generator(device="cpu").manual_seed(count)
    x = (torch.randn(count, generator=g) * 300).to(DEV)
    special = torch.tensor([65504.0, 65520.0, 65519.99, 1e-8, -0.0, float("inf"), float("nan"),
                            2.0 ** -24, 2.0 ** -25, 3 * 2.0 ** -25, 2049.0, 2051.0], device=DEV)
    x[: min(count, len(special))] = special[:count]
    y = torch.full((count + 8,), 7.0, dtype=torch.half, device=DEV)
    flint.fp32_to_fp16(y, x, count)
    torch.cuda.synchronize()
    assert same_bits(y[:count], x.half())
    assert bool((y[count:] == 7).all())


@pytest.mark.parametrize("shape", [(8, 1024, 12, 64, 3), (3, 40, 5, 24, 2), (2, 7, 1, 8, 1)])
def test_heads_split_and_merge_move_bits(flint, shape):
    batches, length, heads, hw, parts = shape
    row_width = parts * heads * hw
    x = torch.randn(batches * length, row_width, device=DEV).half()
    x.view(torch.int16)[0, :4] = torch.tensor([0x7E01, -1, -32768, 0x0001], dtype=torch.int16)
    rebuilt = torch.zeros_like(x)
    for j in range(parts):
        y = torch.zeros(batches, heads, length, hw, dtype=torch.half, device=DEV)
        flint.heads_split(y, x, batches, length, heads, hw, row_width, j * heads * hw)
        want = x[:, j * heads * hw:(j + 1) * heads * hw].view(batches, length, heads, hw)
        assert torch.equal(y.view(torch.int16), want.permute(0, 2, 1, 3).contiguous().view(torch.int16))
        flint.heads_merge(rebuilt, y, batches, length, heads, hw, row_width, j * heads * hw)
    torch.cuda.synchronize()
    assert torch.equal(rebuilt.view(torch.int16), x.view(torch.int16))


def test_embedding_forward_is_one_fp32_add(flint):
    seqs, length, vocab, width = 8, 1024, 50304, 768
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, vocab, (seqs * length,), generator=g)
    tok[:3] = torch.tensor([0, vocab - 1, 40000])  # tokens above 2^15 read as unsigned
    wte = (torch.randn(vocab, width, generator=g) * 0.02).to(DEV)
    wpe = (torch.randn(length, width, generator=g) * 0.02).to(DEV)
    x = torch.zeros(seqs * length, width, device=DEV)
    flint.embedding_forward(x, tokens16(tok.numpy()), wte, wpe, seqs, length, vocab, width)
    torch.cuda.synchronize()
    want = oracle.embedding_forward(tok.numpy(), wte.cpu().numpy(), wpe.cpu().numpy(), length)
    assert same_bits(x, want)


# ---- bias gradient ---------------------------------------------------------------------------


@pytest.mark.parametrize("case", ["bg_a", "bg_b", "bg_c", "bg_d"])
def test_bias_gradient_matches_the_golden_vectors(flint, golden, case):
    g = golden("bias_gradient")
    dy = torch.from_numpy(g[case + "_dy"]).to(DEV)
    rows, cols = dy.shape
    nbytes = flint.bias_gradient_workspace(rows, cols)
    assert nbytes == -(-rows // 256) * cols * 8
    ws = workspace(nbytes)
    out = torch.full((cols,), 3.0, device=DEV)
    flint.bias_gradient(out, dy, rows, cols, False, ws)
    torch.cuda.synchronize()
    assert same_bits(out, g[case + "_total"])
    # The workspace holds each chunk's sums then errors, as two FP32 rows.
    chunks = -(-rows // 256)
    held = ws[:nbytes].view(torch.float32).view(chunks, 2, cols).cpu()
    assert same_bits(held[:, 0], g[case + "_partial_s"])
    acc = torch.from_numpy(g[case + "_old"]).to(DEV)
    flint.bias_gradient(acc, dy, rows, cols, True, ws)
    torch.cuda.synchronize()
    assert same_bits(acc, g[case + "_accumulated"])


@pytest.mark.parametrize("shape", [(8192, 768), (8192, 2304), (16384, 3072), (1, 8), (257, 264)])
def test_bias_gradient_matches_the_oracle_bit_for_bit(flint, shape):
    rows, cols = shape
    rng = np.random.default_rng(rows * 31 + cols)
    dy = crafted(rng, shape).astype(np.float16)
    ws = workspace(flint.bias_gradient_workspace(rows, cols))
    out = torch.zeros(cols, device=DEV)
    flint.bias_gradient(out, torch.from_numpy(dy).to(DEV), rows, cols, False, ws)
    torch.cuda.synchronize()
    assert same_bits(out, oracle.bias_gradient(dy))


# ---- LayerNorm -------------------------------------------------------------------------------


def ulps32(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    spacing = np.spacing(np.abs(b).astype(np.float32)).astype(np.float64)
    return np.abs(a - b) / spacing


@pytest.mark.parametrize("shape", [(8192, 768), (5, 8), (33, 100), (7, 257), (3, 2048), (9, 1536)])
def test_layernorm_forward_statistics_and_output(flint, shape):
    rows, cols = shape
    rng = np.random.default_rng(cols)
    x = rng.standard_normal(shape).astype(np.float32)
    x[0, : min(4, cols)] += 3000.0  # an outlier channel
    gamma = (1 + 0.02 * rng.standard_normal(cols)).astype(np.float32)
    beta = (0.02 * rng.standard_normal(cols)).astype(np.float32)
    y = torch.zeros(rows, cols, dtype=torch.half, device=DEV)
    mean = torch.zeros(rows, device=DEV)
    rstd = torch.zeros(rows, device=DEV)
    flint.layernorm_forward(y, mean, rstd, torch.from_numpy(x).to(DEV),
                            torch.from_numpy(gamma).to(DEV), torch.from_numpy(beta).to(DEV), rows,
                            cols, 1e-5)
    torch.cuda.synchronize()
    want_y, want_mean, want_rstd = oracle.layernorm_forward(x, gamma, beta)
    # The reference's bounds: mean within 1.5 FP32 ulps, rstd within 3 (tests/test_layernorm.py:289-318).
    assert ulps32(mean.cpu().numpy(), want_mean).max() <= 1.5
    assert ulps32(rstd.cpu().numpy(), want_rstd).max() <= 3.0
    # y within 1 FP16 ulp of the exact value.
    got = y.cpu().numpy().astype(np.float64)
    ulp16 = np.spacing(np.abs(want_y).astype(np.float16)).astype(np.float64)
    assert (np.abs(got - want_y) <= ulp16 + 1e-7).all()


@pytest.mark.parametrize("case", ["ln_a", "ln_b", "ln_c"])
def test_layernorm_backward_matches_the_golden_vectors(flint, golden, case):
    g = golden("layernorm_backward")
    t = {k: torch.from_numpy(g[case + "_" + k]).to(DEV) for k in ("dy", "x", "mean", "rstd", "gamma")}
    rows, cols = t["x"].shape
    ws = workspace(flint.layernorm_backward_workspace(rows, cols))
    dx = torch.zeros(rows, cols, device=DEV)
    dgamma = torch.zeros(cols, device=DEV)
    dbeta = torch.zeros(cols, device=DEV)
    flint.layernorm_backward(dx, dgamma, dbeta, t["dy"], t["x"], t["mean"], t["rstd"], t["gamma"],
                             rows, cols, False, False, ws)
    torch.cuda.synchronize()
    assert same_bits(dx, g[case + "_dx"])
    assert same_bits(dgamma, g[case + "_dgamma"])
    assert same_bits(dbeta, g[case + "_dbeta"])
    chunks = -(-rows // 256)
    held = ws[: chunks * cols * 8].view(torch.float32).view(chunks, 2, cols).cpu()
    assert same_bits(held[:, 0], g[case + "_dgamma_partial_s"])
    assert same_bits(held[:, 1], g[case + "_dgamma_partial_e"])
    if case + "_old" in g:
        acc = torch.from_numpy(g[case + "_old"]).to(DEV)
        flint.layernorm_backward(acc, dgamma, dbeta, t["dy"], t["x"], t["mean"], t["rstd"],
                                 t["gamma"], rows, cols, True, False, ws)
        torch.cuda.synchronize()
        assert same_bits(acc, g[case + "_dx_accumulated"])


@pytest.mark.parametrize("shape", [(8192, 768), (1000, 1536), (17, 2048), (3, 8)])
def test_layernorm_backward_matches_the_oracle_bit_for_bit(flint, shape):
    rows, cols = shape
    rng = np.random.default_rng(rows + cols)
    x = crafted(rng, shape, 3).astype(np.float32)
    dy = crafted(rng, shape, 3).astype(np.float16)
    gamma = (1 + 0.02 * rng.standard_normal(cols)).astype(np.float32)
    mean = x.astype(np.float64).mean(1).astype(np.float32)
    rstd = (1 / np.sqrt(x.astype(np.float64).var(1) + 1e-5)).astype(np.float32)
    ws = workspace(flint.layernorm_backward_workspace(rows, cols))
    dx = torch.zeros(rows, cols, device=DEV)
    dgamma = torch.ones(cols, device=DEV)
    dbeta = torch.ones(cols, device=DEV)
    to = lambda a: torch.from_numpy(a).to(DEV)
    flint.layernorm_backward(dx, dgamma, dbeta, to(dy), to(x), to(mean), to(rstd), to(gamma), rows,
                             cols, False, True, ws)
    torch.cuda.synchronize()
    want = oracle.layernorm_backward(dy, x, mean, rstd, gamma, old_dgamma=np.ones(cols, np.float32),
                                     old_dbeta=np.ones(cols, np.float32))
    assert same_bits(dx, want[0])
    assert same_bits(dgamma, want[1])
    assert same_bits(dbeta, want[2])


# ---- causal softmax ---------------------------------------------------------------------------


@pytest.mark.parametrize("shape", [(96, 1024), (3, 8), (5, 264), (2, 512), (2, 1000)])
def test_causal_softmax_forward_is_within_one_ulp(flint, shape):
    batches, length = shape
    g = torch.Generator().manual_seed(length)
    s = torch.randn(batches, length, length, generator=g).half()
    noisy = s.clone()
    mask = torch.tril(torch.ones(length, length, dtype=torch.bool))
    noisy.masked_fill_(~mask, float("nan"))  # masked inputs are ignored even when NaN
    p = torch.full((batches, length, length), 7.0, dtype=torch.half, device=DEV)
    flint.causal_softmax_forward(p, noisy.to(DEV), batches, length)
    torch.cuda.synchronize()
    want = oracle.causal_softmax_forward(s.numpy())
    got = p.cpu().numpy().astype(np.float64)
    ulp16 = np.spacing(np.abs(want).astype(np.float16)).astype(np.float64)
    assert (np.abs(got - want) <= ulp16).all()
    assert (got[:, ~mask.numpy()] == 0).all()
    assert (got[:, 0, 0] == 1.0).all()  # row 0 sees one score


@pytest.mark.parametrize("case", ["sb_a", "sb_b", "sb_c"])
def test_causal_softmax_backward_matches_the_golden_vectors(flint, golden, case):
    g = golden("softmax_backward")
    p = torch.from_numpy(g[case + "_p"]).to(DEV)
    dp = torch.from_numpy(g[case + "_dp"]).to(DEV)
    batches, length, _ = p.shape
    ds = torch.full_like(p, 5.0)
    flint.causal_softmax_backward(ds, p, dp, batches, length, 0.125)
    in_place = dp.clone()
    flint.causal_softmax_backward(in_place, p, in_place, batches, length, 0.125)
    torch.cuda.synchronize()
    assert same_bits(ds, g[case + "_ds"])
    assert same_bits(in_place, g[case + "_ds"])


def test_causal_softmax_backward_matches_the_oracle_at_full_size(flint):
    batches, length = 12, 1024
    g = torch.Generator().manual_seed(5)
    mask = torch.tril(torch.ones(length, length, dtype=torch.bool))
    s = torch.randn(batches, length, length, generator=g)
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1).half()
    dp = (torch.randn(batches, length, length, generator=g) * 0.5).half()
    ds = torch.zeros(batches, length, length, dtype=torch.half, device=DEV)
    flint.causal_softmax_backward(ds, p.to(DEV), dp.to(DEV), batches, length, 0.125)
    torch.cuda.synchronize()
    assert same_bits(ds, oracle.causal_softmax_backward(p.numpy(), dp.numpy(), 0.125))


# ---- softmax + cross-entropy ----------------------------------------------------------------------


# The last two shapes give every persistent CTA several rows (unevenly), the first of them at
# GPT-2's width.
@pytest.mark.parametrize("shape", [(64, 50257, 50304), (5, 8, 8), (9, 1000, 1024),
                                   (3, 65536, 65536), (4, 3, 16), (700, 50257, 50304),
                                   (1500, 1003, 1008)])
def test_cross_entropy_loss_and_gradient(flint, shape):
    rows, vocab, cols = shape
    g = torch.Generator().manual_seed(rows)
    logits = (torch.randn(rows, cols, generator=g) * 2).half()
    logits[:, vocab:] = float("nan")  # padded columns are ignored
    targets = torch.randint(0, vocab, (rows,), generator=g)
    scale = 65536.0 / rows
    dl = torch.full((rows, cols), 9.0, dtype=torch.half, device=DEV)
    loss = torch.zeros(rows, device=DEV)
    flint.softmax_cross_entropy(dl, loss, logits.to(DEV), tokens16(targets.numpy()), scale, rows,
                                vocab, cols)
    torch.cuda.synchronize()
    want_loss, want_grad = oracle.softmax_cross_entropy(logits.numpy(), targets.numpy(), scale, vocab)
    assert np.allclose(loss.cpu().numpy(), want_loss, rtol=2e-6, atol=2e-6)
    got = dl.cpu().numpy().astype(np.float64)
    ulp16 = np.spacing(np.abs(want_grad).astype(np.float16)).astype(np.float64)
    assert (np.abs(got - want_grad) <= ulp16).all()
    assert (got[:, vocab:] == 0).all()
    # The target's gradient is indexed exactly: it is the only negative entry of its row.
    negative = got < 0
    assert (negative.sum(1) <= 1).all()
    rows_with_negative = negative.any(1)
    assert (negative.argmax(1)[rows_with_negative] == targets.numpy()[rows_with_negative]).all()


def test_cross_entropy_of_a_dominant_target_is_zero(flint):
    rows, vocab, cols = 2, 50257, 50304
    logits = torch.zeros(rows, cols, dtype=torch.half)
    targets = torch.tensor([7, 50256])
    logits[0, 7] = 60.0
    logits[1, 50256] = 60.0
    dl = torch.zeros(rows, cols, dtype=torch.half, device=DEV)
    loss = torch.ones(rows, device=DEV)
    flint.softmax_cross_entropy(dl, loss, logits.to(DEV), tokens16(targets.numpy()), 1.0, rows,
                                vocab, cols)
    torch.cuda.synchronize()
    assert loss.cpu().tolist() == [0.0, 0.0]


# ---- embedding backward --------------------------------------------------------------------------


@pytest.mark.parametrize("case", ["eb_a", "eb_b", "eb_c"])
def test_embedding_backward_matches_the_golden_vectors(flint, golden, case):
    g = golden("embedding_backward")
    seqs, length, vocab, width = (int(v) for v in g[case + "_shape"])
    dx = torch.from_numpy(g[case + "_dx"]).to(DEV)
    tok = tokens16(g[case + "_tokens"])
    ws = workspace(flint.embedding_backward_workspace(seqs, length, vocab, width))
    dwte = torch.full((vocab, width), 5.0, device=DEV)
    dwpe = torch.full((length + 2, width), 5.0, device=DEV)
    flint.embedding_backward(dwte, dwpe, dx, tok, seqs, length, vocab, width, False, False, ws)
    torch.cuda.synchronize()
    assert same_bits(dwte, g[case + "_dwte"])
    assert same_bits(dwpe[:length], g[case + "_dwpe"])
    assert bool((dwpe[length:] == 5).all())  # rows past length are untouched
    acc_wte = torch.from_numpy(g[case + "_old_wte"]).to(DEV)
    acc_wpe = torch.from_numpy(g[case + "_old_wpe"]).to(DEV)
    flint.embedding_backward(acc_wte, acc_wpe, dx, tok, seqs, length, vocab, width, True, True, ws)
    torch.cuda.synchronize()
    assert same_bits(acc_wte, g[case + "_dwte_accumulated"])
    assert same_bits(acc_wpe, g[case + "_dwpe_accumulated"])


def test_embedding_backward_matches_the_oracle_at_gpt2_size(flint):
    seqs, length, vocab, width = 8, 1024, 50304, 768
    rng = np.random.default_rng(11)
    tokens = rng.integers(0, 50257, seqs * length).astype(np.uint16)
    tokens[::97] = 198  # a token repeated many times
    dx = crafted(rng, (seqs * length, width), 3).astype(np.float32)
    ws = workspace(flint.embedding_backward_workspace(seqs, length, vocab, width))
    dwte = torch.full((vocab, width), 5.0, device=DEV)
    dwpe = torch.zeros(length, width, device=DEV)
    flint.embedding_backward(dwte, dwpe, torch.from_numpy(dx).to(DEV), tokens16(tokens), seqs,
                             length, vocab, width, False, False, ws)
    torch.cuda.synchronize()
    want_wte, want_wpe, *_ = oracle.embedding_backward(dx, tokens, seqs, length, vocab)
    assert same_bits(dwte, want_wte)
    assert same_bits(dwpe, want_wpe)


def test_cross_entropy_with_extreme_and_non_finite_logits(flint):
    """The exponential's clamp and NaN handling: logits spanning FP16's range, -inf entries
    (probability 0), and rows with +inf or NaN (every output of such a row is NaN, as in the
    float64 reference)."""
    rows, vocab, cols = 6, 1003, 1008
    g = torch.Generator().manual_seed(3)
    logits = (torch.randn(rows, cols, generator=g) * 3).half()
    logits[0, :50] = -65504.0           # far below the row maximum
    logits[0, 60] = 65504.0
    logits[1] = -65504.0                # a very negative maximum
    logits[1, 7] = -65000.0
    logits[2, 100:200] = float("-inf")
    logits[3, 5] = float("inf")
    logits[4, 9] = float("nan")
    targets = torch.tensor([60, 7, 3, 1, 2, 500])
    scale = 4.0
    dl = torch.full((rows, cols), 9.0, dtype=torch.half, device=DEV)
    loss = torch.zeros(rows, device=DEV)
    flint.softmax_cross_entropy(dl, loss, logits.to(DEV), tokens16(targets.numpy()), scale, rows,
                                vocab, cols)
    torch.cuda.synchronize()
    got = dl.cpu().numpy().astype(np.float64)
    got_loss = loss.cpu().numpy()
    finite_rows = [0, 1, 2, 5]
    x = logits.numpy().astype(np.float64)[:, :vocab]
    for r in finite_rows:
        m = x[r].max()
        e = np.exp(x[r] - m)
        p = e / e.sum()
        want = p * scale
        want[targets[r]] = (p[targets[r]] - 1.0) * scale
        ulp16 = np.spacing(np.abs(want).astype(np.float16)).astype(np.float64)
        assert (np.abs(got[r, :vocab] - want) <= ulp16 + 2.0 ** -23 * scale).all(), r
        want_loss = np.log(e.sum()) - (x[r, targets[r]] - m)
        assert abs(got_loss[r] - want_loss) <= 4e-6 * max(1.0, abs(want_loss)), r
        assert (got[r, vocab:] == 0).all()
    assert (got[2, 100:200] == 0).all()
    for r in (3, 4):
        assert np.isnan(got[r, :vocab]).all(), r
        assert np.isnan(got_loss[r]), r


# ---- known answers from the reference's float64 references (tests/golden/float_references.npz) ----


def ulp16_of(want):
    return np.spacing(np.abs(np.asarray(want)).astype(np.float16)).astype(np.float64)


@pytest.mark.parametrize("case", ["ln_a", "ln_b", "ln_c"])
def test_layernorm_forward_matches_the_golden_vectors(flint, golden, case):
    g = golden("float_references")
    x, gamma, beta = (torch.from_numpy(g[case + k]).to(DEV) for k in ("_x", "_gamma", "_beta"))
    rows, cols = x.shape
    y = torch.zeros(rows, cols, dtype=torch.half, device=DEV)
    mean, rstd = torch.zeros(rows, device=DEV), torch.zeros(rows, device=DEV)
    flint.layernorm_forward(y, mean, rstd, x, gamma, beta, rows, cols, 1e-5)
    torch.cuda.synchronize()
    assert ulps32(mean.cpu().numpy(), g[case + "_mean"]).max() <= 1.5
    assert ulps32(rstd.cpu().numpy(), g[case + "_rstd"]).max() <= 3.0
    want = g[case + "_y"]
    assert (np.abs(y.cpu().numpy().astype(np.float64) - want) <= ulp16_of(want) + 1e-7).all()
    if case == "ln_a":  # the constant row: mean exact, y exactly beta rounded
        assert mean[2].item() == 4.25
        assert same_bits(y[2], beta.half())


@pytest.mark.parametrize("case", ["sm_a", "sm_b", "sm_c"])
def test_causal_softmax_forward_matches_the_golden_vectors(flint, golden, case):
    g = golden("float_references")
    s = torch.from_numpy(g[case + "_s"]).to(DEV)
    batches, length, _ = s.shape
    p = torch.full_like(s, 7.0)
    flint.causal_softmax_forward(p, s, batches, length)
    torch.cuda.synchronize()
    want = g[case + "_p"]
    assert (np.abs(p.cpu().numpy().astype(np.float64) - want) <= ulp16_of(want)).all()


@pytest.mark.parametrize("case", ["ce_a", "ce_b", "ce_c"])
def test_cross_entropy_matches_the_golden_vectors(flint, golden, case):
    g = golden("float_references")
    logits = torch.from_numpy(g[case + "_logits"]).to(DEV)
    targets = g[case + "_targets"]
    vocab = int(g[case + "_vocab"])
    rows, cols = logits.shape
    dl = torch.full((rows, cols), 9.0, dtype=torch.half, device=DEV)
    loss = torch.zeros(rows, device=DEV)
    flint.softmax_cross_entropy(dl, loss, logits, tokens16(targets), 0.75, rows, vocab, cols)
    torch.cuda.synchronize()
    assert np.allclose(loss.cpu().numpy(), g[case + "_loss"], rtol=2e-6, atol=2e-6)
    got = dl.cpu().numpy().astype(np.float64)
    want = g[case + "_grad"]
    assert (np.abs(got[:, :vocab] - want) <= ulp16_of(want)).all()
    assert (got[:, vocab:] == 0).all()
    assert (got[np.arange(rows), targets] < 0).all() and ((got < 0).sum(1) == 1).all()


def test_embedding_forward_matches_the_golden_vectors(flint, golden):
    g = golden("float_references")
    seqs, length, vocab, width = (int(v) for v in g["emb_shape"])
    x = torch.zeros(seqs * length, width, device=DEV)
    flint.embedding_forward(x, tokens16(g["emb_ids"]), torch.from_numpy(g["emb_wte"]).to(DEV),
                            torch.from_numpy(g["emb_wpe"]).to(DEV), seqs, length, vocab, width)
    torch.cuda.synchronize()
    assert same_bits(x, g["emb_x"])


# ---- what embedding backward leaves in its workspace ------------------------------------------


def embedding_workspace_parts(ws, sequences, length, vocab, width):
    """(sorted tokens, sorted rows, offsets, position partial sums, position partial errors)
    read from the workspace. Its layout is part of the interface: the position-table partial
    sums first (the bias gradient's workspace for dx viewed as sequences x (length * width)),
    then, each 16-byte aligned, the sorted tokens (uint16), their rows (uint32) and
    offsets[vocab + 1] (uint32) (src/kernels/embedding_backward.cuh:31-79 in the reference)."""
    up = lambda b: -(-b // 16) * 16
    rows = sequences * length
    chunks = -(-sequences // 256)
    cols = length * width
    raw = ws.cpu().numpy()
    partials = raw[: chunks * cols * 8].view(np.float32).reshape(chunks, 2, cols)
    at = up(chunks * cols * 8)
    tokens = raw[at:at + rows * 2].view(np.uint16)
    at += up(rows * 2)
    sorted_rows = raw[at:at + rows * 4].view(np.uint32)
    at += up(rows * 4)
    offsets = raw[at:at + (vocab + 1) * 4].view(np.uint32)
    return tokens, sorted_rows, offsets, partials[:, 0], partials[:, 1]


@pytest.mark.parametrize("case", ["eb_a", "eb_b", "eb_c"])
def test_embedding_backward_workspace_holds_the_sorted_tokens_rows_and_offsets(flint, golden, case):
    g = golden("embedding_backward")
    seqs, length, vocab, width = (int(v) for v in g[case + "_shape"])
    ws = workspace(flint.embedding_backward_workspace(seqs, length, vocab, width))
    ws.fill_(0xA5)
    dwte = torch.zeros(vocab, width, device=DEV)
    dwpe = torch.zeros(length, width, device=DEV)
    flint.embedding_backward(dwte, dwpe, torch.from_numpy(g[case + "_dx"]).to(DEV),
                             tokens16(g[case + "_tokens"]), seqs, length, vocab, width, False, False, ws)
    torch.cuda.synchronize()
    tokens, rows, offsets, _, _ = embedding_workspace_parts(ws, seqs, length, vocab, width)
    assert np.array_equal(tokens, g[case + "_sorted_tokens"].astype(np.uint16))
    assert np.array_equal(rows, g[case + "_sorted_rows"].astype(np.uint32))
    assert np.array_equal(offsets, g[case + "_offsets"].astype(np.uint32))


def test_embedding_backward_workspace_at_gpt2_size_matches_the_oracle(flint):
    seqs, length, vocab, width = 8, 1024, 50304, 768
    rng = np.random.default_rng(12)
    tokens = rng.integers(0, 50257, seqs * length).astype(np.uint16)
    tokens[::5] = 50256  # a token above 2^15 repeated many times
    dx = crafted(rng, (seqs * length, width), 3).astype(np.float32)
    ws = workspace(flint.embedding_backward_workspace(seqs, length, vocab, width))
    dwte = torch.zeros(vocab, width, device=DEV)
    dwpe = torch.zeros(length, width, device=DEV)
    flint.embedding_backward(dwte, dwpe, torch.from_numpy(dx).to(DEV), tokens16(tokens), seqs,
                             length, vocab, width, False, False, ws)
    torch.cuda.synchronize()
    _, _, want_tokens, want_rows, want_offsets = oracle.embedding_backward(dx, tokens, seqs, length, vocab)
    got_tokens, got_rows, got_offsets, sums, errors = embedding_workspace_parts(ws, seqs, length, vocab, width)
    assert np.array_equal(got_tokens, want_tokens.astype(np.uint16))
    assert np.array_equal(got_rows, want_rows.astype(np.uint32))
    assert np.array_equal(got_offsets, want_offsets.astype(np.uint32))
    # The position table's partial sums are the column-sum scheme's over [sequences, length * width].
    want_s, want_e, _ = oracle._column_sums(dx.reshape(seqs, length * width))
    assert same_bits(torch.from_numpy(sums.copy()), want_s)
    assert same_bits(torch.from_numpy(errors.copy()), want_e)
