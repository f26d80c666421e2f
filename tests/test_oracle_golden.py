"""Pins oracle/flint_oracle.py against the fixtures the reference's own emulations,
float references and PyTorch model produced (tests/golden/make_golden.py). CPU only."""

import numpy as np
import pytest
import torch

import flint_oracle as oracle


def same_bits(a, b):
    a, b = np.asarray(a), np.asarray(b)
    assert a.dtype == b.dtype and a.shape == b.shape
    width = {2: np.uint16, 4: np.uint32}[a.dtype.itemsize]
    # NaN payloads are not promised; compare NaN positions and every other bit pattern.
    nan = np.isnan(a)
    assert np.array_equal(nan, np.isnan(b))
    return np.array_equal(a.view(width)[~nan], b.view(width)[~nan])


@pytest.mark.parametrize("case", ["bg_a", "bg_b", "bg_c", "bg_d"])
def test_bias_gradient_matches_reference_emulation(golden, case):
    g = golden("bias_gradient")
    total, ps, pe = oracle.bias_gradient(g[case + "_dy"], with_partials=True)
    assert same_bits(total, g[case + "_total"])
    finite = np.isfinite(g[case + "_partial_s"])
    assert same_bits(ps, g[case + "_partial_s"])
    assert same_bits(np.where(finite, pe, 0), np.where(finite, g[case + "_partial_e"], 0))
    assert same_bits(oracle.bias_gradient(g[case + "_dy"], old=g[case + "_old"]),
                     g[case + "_accumulated"])


@pytest.mark.parametrize("case", ["ln_a", "ln_b", "ln_c"])
def test_layernorm_backward_matches_reference_emulation(golden, case):
    g = golden("layernorm_backward")
    args = [g[case + k] for k in ("_dy", "_x", "_mean", "_rstd", "_gamma")]
    dx, dgamma, dbeta, ps, pe = oracle.layernorm_backward(*args, with_partials=True)
    assert same_bits(dx, g[case + "_dx"])
    assert same_bits(dgamma, g[case + "_dgamma"])
    assert same_bits(dbeta, g[case + "_dbeta"])
    assert same_bits(ps, g[case + "_dgamma_partial_s"])
    assert same_bits(pe, g[case + "_dgamma_partial_e"])
    if case + "_old" in g:
        dx2, _, _ = oracle.layernorm_backward(*args, old_dx=g[case + "_old"])
        assert same_bits(dx2, g[case + "_dx_accumulated"])


@pytest.mark.parametrize("case", ["sb_a", "sb_b", "sb_c"])
def test_softmax_backward_matches_reference_emulation(golden, case):
    g = golden("softmax_backward")
    assert same_bits(oracle.causal_softmax_backward(g[case + "_p"], g[case + "_dp"], 0.125),
                     g[case + "_ds"])


@pytest.mark.parametrize("case", ["eb_a", "eb_b", "eb_c"])
def test_embedding_backward_matches_reference_emulation(golden, case):
    g = golden("embedding_backward")
    seqs, length, vocab, _ = (int(v) for v in g[case + "_shape"])
    dwte, dwpe, st, sr, off = oracle.embedding_backward(g[case + "_dx"], g[case + "_tokens"], seqs,
                                                        length, vocab)
    assert same_bits(dwte, g[case + "_dwte"])
    assert same_bits(dwpe, g[case + "_dwpe"])
    assert np.array_equal(st, g[case + "_sorted_tokens"].astype(np.int64))
    assert np.array_equal(sr, g[case + "_sorted_rows"].astype(np.int64))
    assert np.array_equal(off, g[case + "_offsets"].astype(np.int64))
    dwte2, dwpe2, *_ = oracle.embedding_backward(g[case + "_dx"], g[case + "_tokens"], seqs, length,
                                                 vocab, g[case + "_old_wte"], g[case + "_old_wpe"])
    assert same_bits(dwte2, g[case + "_dwte_accumulated"])
    assert same_bits(dwpe2, g[case + "_dwpe_accumulated"])


def test_gemm_references_match_the_gate(golden):
    g = golden("gemm_reference")
    close = lambda a, b: np.allclose(np.asarray(a), b, rtol=1e-12, atol=1e-12)
    assert close(oracle.gemm_nt(g["x"], g["w"]), g["nt"])
    assert close(oracle.gemm_nt(g["x"], g["w"], g["bias"]), g["nt_bias"])
    assert close(oracle.gemm_nt_bias_gelu(g["x"], g["w"], g["bias"])[1], g["nt_bias_gelu"])
    assert close(oracle.gemm_nn(g["x"], g["wn"]), g["nn"])
    assert close(oracle.gemm_nn_dgelu(g["x"], g["wn"], g["pre"]), g["nn_dgelu"])
    assert close(oracle.gemm_tn(g["xt"], g["wn"]), g["tn"])


SMALL = dict(n_layer=2, n_head=2, n_embd=64, block_size=32, vocab_size=200, padded_vocab_size=208)


def test_gpt2_init_matches_the_reference_model(golden):
    g = golden("gpt2_torch")
    params = oracle.gpt2_init(SMALL, seed=1234)
    assert list(params) == [str(n) for n in g["names"]]
    for name, p in params.items():
        assert p.double().sum().item() == pytest.approx(g["param_sum/" + name].item(), abs=1e-9)
        assert p.double().abs().sum().item() == pytest.approx(g["param_abs/" + name].item(),
                                                              abs=1e-9)
    tiny = oracle.gpt2_init(oracle.TINY, seed=1234)
    for name, p in tiny.items():
        assert p.double().sum().item() == pytest.approx(g["tiny_sum/" + name].item(), abs=1e-9)


def test_gpt2_loss_gradients_and_adamw_match_the_reference_model(golden):
    g = golden("gpt2_torch")
    params = oracle.gpt2_init(SMALL, seed=1234)
    idx, targets = torch.from_numpy(g["idx"]), torch.from_numpy(g["targets"])
    loss, grads = oracle.gpt2_loss_and_gradients(SMALL, params, idx, targets)
    assert loss == pytest.approx(g["loss"].item(), rel=1e-5)
    for name, grad in grads.items():
        want = torch.from_numpy(g["grad/" + name])
        assert torch.allclose(grad, want, rtol=1e-3, atol=1e-6), name
        cos = torch.nn.functional.cosine_similarity(grad.flatten().double(),
                                                    want.flatten().double(), dim=0)
        assert cos > 0.99999, name
    # One AdamW step from zero moments with the reference's gradients.
    for name, p in params.items():
        grad = torch.from_numpy(g["grad/" + name])
        m, v = torch.zeros_like(p), torch.zeros_like(p)
        wd = oracle.WEIGHT_DECAY if oracle.decayed(name, p.shape) else 0.0
        oracle.adamw_step(p, m, v, grad, 1, weight_decay=wd)
        assert torch.allclose(p, torch.from_numpy(g["stepped/" + name]), rtol=1e-5, atol=1e-7), name


# ---- float64 references and the optimizer (float_references.npz, optimizer.npz) --------------

def close64(a, b, tol=1e-12):
    return np.allclose(np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64), rtol=tol,
                       atol=tol)


@pytest.mark.parametrize("case", ["ln_a", "ln_b", "ln_c"])
def test_layernorm_forward_matches_the_reference_float64(golden, case):
    g = golden("float_references")
    y, mean, rstd = oracle.layernorm_forward(g[case + "_x"], g[case + "_gamma"], g[case + "_beta"],
                                             float(np.float32(1e-5)))
    assert close64(mean, g[case + "_mean"]) and close64(rstd, g[case + "_rstd"], 1e-11)
    assert close64(y, g[case + "_y"], 1e-10)


@pytest.mark.parametrize("case", ["sm_a", "sm_b", "sm_c"])
def test_causal_softmax_forward_matches_the_reference_float64(golden, case):
    g = golden("float_references")
    assert close64(oracle.causal_softmax_forward(g[case + "_s"]), g[case + "_p"])


@pytest.mark.parametrize("case", ["ce_a", "ce_b", "ce_c"])
def test_cross_entropy_matches_the_reference_float64(golden, case):
    g = golden("float_references")
    vocab = int(g[case + "_vocab"])
    loss, grad = oracle.softmax_cross_entropy(g[case + "_logits"], g[case + "_targets"], 0.75, vocab)
    assert close64(loss, g[case + "_loss"])
    assert close64(grad[:, :vocab], g[case + "_grad"]) and not grad[:, vocab:].any()
    rows = np.arange(len(loss))
    assert close64(np.exp(-loss), g[case + "_p_target"])
    assert (grad[rows, g[case + "_targets"]] < 0).all()


def test_embedding_forward_matches_the_reference(golden):
    g = golden("float_references")
    _, length, _, _ = (int(v) for v in g["emb_shape"])
    got = oracle.embedding_forward(g["emb_ids"], g["emb_wte"], g["emb_wpe"], length)
    assert same_bits(got, g["emb_x"])


@pytest.mark.parametrize("case", ["at_a", "at_b", "at_c"])
def test_attention_matches_the_reference_float64(golden, case):
    g = golden("float_references")
    o, lse, dq, dk, dv = oracle.attention(g[case + "_q"], g[case + "_k"], g[case + "_v"], 0.125,
                                          g[case + "_do"])
    assert close64(o, g[case + "_o"], 1e-10)
    assert close64(dq, g[case + "_dq"], 1e-10) and close64(dk, g[case + "_dk"], 1e-10)
    assert close64(dv, g[case + "_dv"], 1e-10)
    # The log-sum-exp against the scores' own definition.
    s = np.einsum("bqd,bkd->bqk", g[case + "_q"].astype(np.float64),
                  g[case + "_k"].astype(np.float64)) * 0.125
    t = s.shape[1]
    s = np.where(np.tril(np.ones((t, t), dtype=bool)), s, -np.inf)
    assert close64(lse, np.log(np.exp(s - s.max(-1, keepdims=True)).sum(-1)) + s.max(-1), 1e-10)


def test_gelu_helpers_match_the_reference_closed_forms(golden):
    g = golden("float_references")
    s = torch.from_numpy(g["gelu_s"])
    assert close64(oracle.gelu_tanh(s), g["gelu_y"], 1e-14)
    assert close64(oracle.gelu_exponent(s), g["gelu_exponent"], 1e-14)
    margin = oracle.half_rounding_margin(oracle.gelu_tanh(s)).numpy()
    finite = np.isfinite(g["gelu_margin"])
    assert np.array_equal(finite, np.isfinite(margin))
    assert close64(margin[finite], g["gelu_margin"][finite], 1e-9)
    assert np.array_equal(oracle.half_ordered(s.half().numpy()).numpy(), g["gelu_ordered"])
    derivative, exponent = oracle.gelu_tanh_derivative(s)
    assert close64(derivative, g["dgelu_g"], 1e-13)
    assert close64(-exponent, g["dgelu_a"], 1e-14)     # the reference names -a
    assert same_bits(oracle.round_to_half(derivative * 3.0).numpy(), g["dgelu_rounded"])


def test_three_clipped_adamw_steps_match_the_reference_optimizer(golden):
    """oracle.clip_coefficient + oracle.adamw_step against torch.optim.AdamW and
    clip_grad_norm_ as the reference configures them, on the reference's own gradients."""
    g = golden("optimizer")
    names = [str(n) for n in g["names"]]
    params = {n: torch.from_numpy(g["start/" + n].copy()) for n in names}
    moments = {n: (torch.zeros_like(p), torch.zeros_like(p)) for n, p in params.items()}
    for step in (1, 2, 3):
        grads = {n: torch.from_numpy(g[f"grad/{step}/" + n]) for n in names}
        coefficient, norm = oracle.clip_coefficient(grads.values())
        assert norm == pytest.approx(float(g[f"norm/{step}"]), rel=1e-5) and coefficient < 0.02
        for n, p in params.items():
            wd = oracle.WEIGHT_DECAY if oracle.decayed(n, p.shape) else 0.0
            oracle.adamw_step(p, *moments[n], grads[n] * coefficient, step, weight_decay=wd)
            want = torch.from_numpy(g[f"param/{step}/" + n])
            assert torch.allclose(p, want, rtol=2e-6, atol=1e-8), (step, n)
