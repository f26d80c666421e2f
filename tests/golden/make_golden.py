"""Generates tests/golden/*.npz from the reference checkout.

Run once, in a container where the reference repository is checked out:

    python tests/golden/make_golden.py /path/to/reference [fixture ...]

(with no fixture names every file is rewritten; `float_references` and `optimizer` name the
two files float_references() and optimizer_steps() write).

It imports the reference's own test helpers (the bit-exact numpy emulations
of its kernels and its float references) and its PyTorch GPT-2 model, runs
them on seeded inputs, and stores inputs and outputs as small fixtures. The
fixtures pin oracle/flint_oracle.py (tests/test_oracle_golden.py) and serve
as known-answer vectors for the CUDA kernels (the `golden` cases of tests/test_*_gpu.py).
Nothing else reads the reference, and no test needs it at run time.
"""

import contextlib
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


@contextlib.contextmanager
def cuda_factories_on_cpu():
    """Some of the reference's float64 helpers build their masks and index vectors with
    device="cuda". This container has no GPU, so while they run the torch factory functions
    they use are redirected to the CPU; the float64 arithmetic itself is untouched."""
    names = ("ones", "zeros", "arange", "empty", "full", "tensor")
    saved = {n: getattr(torch, n) for n in names}

    def redirect(fn):
        def call(*args, **kwargs):
            if str(kwargs.get("device", "")).startswith("cuda"):
                kwargs["device"] = "cpu"
            return fn(*args, **kwargs)
        return call

    for n in names:
        setattr(torch, n, redirect(saved[n]))
    try:
        yield
    finally:
        for n in names:
            setattr(torch, n, saved[n])


def crafted(rng, shape, spread=6):
    """N(0,1) * 2^U{-spread..spread}: sums that round differently in different orders."""
    base = rng.standard_normal(shape)
    scale = np.exp2(rng.integers(-spread, spread + 1, shape))
    return np.clip(base * scale, -60000, 60000)


def float_references() -> None:
    """Known answers from the reference's float64 references for the kernels whose tests
    bound an error instead of pinning bits: LayerNorm forward (tests/test_layernorm.py:126-135),
    causal softmax (tests/test_softmax.py:106-111), cross-entropy
    (tests/test_cross_entropy.py:220-231), embedding (tests/test_embedding.py:94-99), causal
    attention forward and gradients (tests/test_softmax.py:1058-1066,
    tests/test_softmax_backward.py:1429-1440), and the GELU and its derivative in closed form
    (tests/test_gemm_bias_gelu.py:193-227, tests/test_gemm_dgelu.py:262-298)."""
    import test_cross_entropy as ce
    import test_embedding as emb
    import test_gemm_bias_gelu as gelu
    import test_gemm_dgelu as dgelu
    import test_layernorm as ln
    import test_softmax as sm
    import test_softmax_backward as sb

    rng = np.random.default_rng(20260102)
    out = {}
    with cuda_factories_on_cpu():
        for name, (rows, cols) in {"ln_a": (5, 8), "ln_b": (37, 768), "ln_c": (9, 1027)}.items():
            x = torch.from_numpy((rng.standard_normal((rows, cols)) * 3 + 1).astype(np.float32))
            if name == "ln_a":
                x[2] = 4.25                                     # a constant row
            gamma = torch.from_numpy((1 + 0.02 * rng.standard_normal(cols)).astype(np.float32))
            beta = torch.from_numpy((0.1 * rng.standard_normal(cols)).astype(np.float32))
            y, mean, rstd = ln.reference_layernorm(x, gamma, beta, 1e-5)
            out[name + "_x"], out[name + "_gamma"], out[name + "_beta"] = x.numpy(), gamma.numpy(), beta.numpy()
            out[name + "_y"], out[name + "_mean"], out[name + "_rstd"] = y.numpy(), mean.numpy(), rstd.numpy()

        for name, (batches, t) in {"sm_a": (2, 8), "sm_b": (2, 136), "sm_c": (1, 264)}.items():
            s = torch.from_numpy((rng.standard_normal((batches, t, t)) * (8 if name == "sm_b" else 1))
                                 .astype(np.float16))
            out[name + "_s"] = s.numpy()
            out[name + "_p"] = sm.reference(s, torch.float64).numpy()

        for name, (rows, cols, vocab) in {"ce_a": (4, 8, 5), "ce_b": (33, 1000, 937),
                                          "ce_c": (2, 50304, 50257)}.items():
            logits = torch.from_numpy((rng.standard_normal((rows, cols)) * 2).astype(np.float16))
            if name == "ce_b":
                logits[:, vocab:] = 30.0                        # padding that must not be read
            targets = torch.from_numpy(rng.integers(0, vocab, rows).astype(np.int64))
            loss, grad, p_target = ce.reference(logits, targets, 0.75, vocab)
            out[name + "_logits"], out[name + "_targets"] = logits.numpy(), targets.numpy()
            out[name + "_vocab"] = np.array(vocab)
            out[name + "_loss"], out[name + "_grad"] = loss.numpy(), grad.numpy()
            out[name + "_p_target"] = p_target.numpy()

        seqs, length, vocab, width = 3, 16, 70, 24
        ids = torch.from_numpy(rng.integers(0, vocab, seqs * length).astype(np.int64))
        wte = torch.from_numpy(rng.standard_normal((vocab, width)).astype(np.float32))
        wpe = torch.from_numpy(rng.standard_normal((length + 4, width)).astype(np.float32))
        out["emb_ids"], out["emb_wte"], out["emb_wpe"] = ids.numpy(), wte.numpy(), wpe.numpy()
        out["emb_shape"] = np.array([seqs, length, vocab, width])
        out["emb_x"] = emb.reference_embedding(ids, wte, wpe, seqs, length).reshape(-1, width).numpy()

        for name, (batches, t) in {"at_a": (2, 64), "at_b": (2, 200), "at_c": (1, 520)}.items():
            q, k, v, d_o = (torch.from_numpy(rng.standard_normal((batches, t, 64)).astype(np.float16))
                            for _ in range(4))
            out[name + "_q"], out[name + "_k"], out[name + "_v"] = q.numpy(), k.numpy(), v.numpy()
            out[name + "_do"] = d_o.numpy()
            out[name + "_o"] = sm.pytorch_attention(q, k, v, torch.float64).numpy()
            dq, dk = sb.reference_gradients(q, k, v, d_o)
            out[name + "_dq"], out[name + "_dk"] = dq.numpy(), dk.numpy()
            vd = v.double().requires_grad_()
            sm.pytorch_attention(q.double(), k.double(), vd).backward(d_o.double())
            out[name + "_dv"] = vd.grad.numpy()

    s = torch.cat([torch.linspace(-12.0, 12.0, 4001, dtype=torch.float64),
                   torch.tensor([1e-30, -1e-30, 65504.0, -65504.0, 100.0, -100.0, 1e6, -1e6],
                                dtype=torch.float64)])
    out["gelu_s"] = s.numpy()
    out["gelu_y"] = gelu.gelu64(s).numpy()
    out["gelu_exponent"] = gelu.gelu_exponent(s).numpy()
    out["gelu_margin"] = gelu.rounding_margin(gelu.gelu64(s)).numpy()
    out["gelu_ordered"] = gelu.ordered(s.half()).numpy()
    g, a = dgelu.dgelu64(s)
    out["dgelu_g"], out["dgelu_a"] = g.numpy(), a.numpy()
    out["dgelu_rounded"] = dgelu.rounded_to_fp16(g * 3.0).numpy()
    np.savez_compressed(HERE / "float_references.npz", **out)


def optimizer_steps() -> None:
    """Three steps of the reference's optimizer set-up (scripts/gpt2_torch.py:150-175: AdamW,
    lr 6e-4, betas 0.9/0.95, eps 1e-8, weight decay 0.1 on parameters of two or more
    dimensions) with its gradient clipping (:187-188) on a small model: every parameter after
    each step, and the clip's total norm."""
    import gpt2_torch

    out = {}
    cfg = gpt2_torch.GPTConfig(n_layer=2, n_head=2, n_embd=32, block_size=16, vocab_size=100,
                               padded_vocab_size=104)
    model = gpt2_torch.build_model(cfg, seed=1234)
    params = [p for p in model.parameters()]
    opt = gpt2_torch.configure_optimizer(model)
    gen = torch.Generator().manual_seed(123)
    out["names"] = np.array([n for n, _ in model.named_parameters()])
    for name, p in model.named_parameters():
        out["start/" + name] = p.detach().numpy().copy()
    for step in (1, 2, 3):
        ids = torch.randint(0, cfg.vocab_size, (3 * 16 + 1,), generator=gen)
        idx, targets = ids[:-1].view(3, 16), ids[1:].view(3, 16)
        out[f"idx/{step}"], out[f"targets/{step}"] = idx.numpy(), targets.numpy()
        loss = model(idx, targets)
        # Large enough for the clip to bite on every step.
        (loss * 40.0).backward()
        for name, p in model.named_parameters():
            out[f"grad/{step}/" + name] = p.grad.numpy().copy()
        norm = torch.nn.utils.clip_grad_norm_(params, gpt2_torch.MAX_GRAD_NORM)
        out[f"norm/{step}"] = np.array(norm.item())
        opt.step()
        opt.zero_grad(set_to_none=True)
        for name, p in model.named_parameters():
            out[f"param/{step}/" + name] = p.detach().numpy().copy()
    np.savez_compressed(HERE / "optimizer.npz", **out)


def main(reference_root: str, only=()) -> None:
    root = Path(reference_root)
    sys.path.insert(0, str(root / "tests"))
    sys.path.insert(0, str(root / "scripts"))
    if not only or "float_references" in only:
        float_references()
    if not only or "optimizer" in only:
        optimizer_steps()
    if only:
        print("wrote", sorted(only))
        return
    import gate
    import gpt2_torch
    import test_bias_gradient as bg
    import test_embedding_backward as eb
    import test_layernorm_backward as lb
    import test_softmax_backward as sb

    rng = np.random.default_rng(20260101)
    out = {}

    # Bias gradient: ragged chunk counts, a column with inf, accumulate.
    for name, (rows, cols) in {"bg_a": (1, 8), "bg_b": (300, 24), "bg_c": (8453, 16),
                               "bg_d": (33 * 256 + 5, 8)}.items():
        dy = crafted(rng, (rows, cols)).astype(np.float16)
        if name == "bg_b":
            dy[17, 3] = np.inf
            dy[5, 4] = np.nan
        old = rng.standard_normal(cols).astype(np.float32)
        total, ps, pe = bg.emulate(dy, with_partials=True)
        out[name + "_dy"] = dy
        out[name + "_old"] = old
        out[name + "_total"] = total
        out[name + "_partial_s"] = ps
        out[name + "_partial_e"] = pe
        out[name + "_accumulated"] = bg.emulate(dy, old=old)
    np.savez_compressed(HERE / "bias_gradient.npz", **out)

    # LayerNorm backward.
    out = {}
    for name, (rows, cols) in {"ln_a": (3, 8), "ln_b": (300, 104), "ln_c": (260, 768)}.items():
        x = (crafted(rng, (rows, cols), 3)).astype(np.float32)
        dy = crafted(rng, (rows, cols), 3).astype(np.float16)
        gamma = (1 + 0.02 * rng.standard_normal(cols)).astype(np.float32)
        x64 = x.astype(np.float64)
        mean = x64.mean(1).astype(np.float32)
        rstd = (1 / np.sqrt(x64.var(1) + 1e-5)).astype(np.float32)
        old = rng.standard_normal((rows, cols)).astype(np.float32)
        out[name + "_x"], out[name + "_dy"], out[name + "_gamma"] = x, dy, gamma
        out[name + "_mean"], out[name + "_rstd"] = mean, rstd
        out[name + "_dx"] = lb.emulate_dx(dy, x, mean, rstd, gamma)
        if name != "ln_c":  # keep the fixture small
            out[name + "_old"] = old
            out[name + "_dx_accumulated"] = lb.emulate_dx(dy, x, mean, rstd, gamma, old=old)
        dgamma, ps, pe = lb.emulate_dgamma(dy, x, mean, rstd, with_partials=True)
        out[name + "_dgamma"], out[name + "_dgamma_partial_s"] = dgamma, ps
        out[name + "_dgamma_partial_e"] = pe
        out[name + "_dbeta"] = bg.emulate(dy)
    np.savez_compressed(HERE / "layernorm_backward.npz", **out)

    # Causal softmax backward.
    out = {}
    for name, (batches, t) in {"sb_a": (2, 8), "sb_b": (3, 72), "sb_c": (1, 328)}.items():
        s = torch.from_numpy(rng.standard_normal((batches, t, t)) * 3)
        mask = torch.tril(torch.ones(t, t, dtype=torch.bool))
        p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1).to(torch.float16).numpy()
        p = np.where(mask.numpy(), p, rng.standard_normal((batches, t, t)).astype(np.float16))
        dp = crafted(rng, (batches, t, t), 3).astype(np.float16)
        out[name + "_p"], out[name + "_dp"] = p, dp
        out[name + "_ds"] = sb.emulate(p, dp, 0.125)
    np.savez_compressed(HERE / "softmax_backward.npz", **out)

    # Embedding backward.
    out = {}
    for name, (seqs, length, vocab, width) in {"eb_a": (3, 8, 10, 8), "eb_b": (5, 40, 300, 16),
                                               "eb_c": (260, 8, 4, 8)}.items():
        rows = seqs * length
        tokens = rng.integers(0, vocab, rows).astype(np.uint16)
        if name == "eb_b":
            tokens[::3] = 7
        dx = crafted(rng, (rows, width), 4).astype(np.float32)
        old_wte = rng.standard_normal((vocab, width)).astype(np.float32)
        old_wpe = rng.standard_normal((length, width)).astype(np.float32)
        e = eb.emulate_all(dx, tokens, seqs, length, vocab)
        ea = eb.emulate_all(dx, tokens, seqs, length, vocab, old_wte, old_wpe)
        out[name + "_dx"], out[name + "_tokens"] = dx, tokens
        out[name + "_shape"] = np.array([seqs, length, vocab, width])
        out[name + "_old_wte"], out[name + "_old_wpe"] = old_wte, old_wpe
        out[name + "_dwte"], out[name + "_dwpe"] = e[0], e[1]
        out[name + "_sorted_tokens"], out[name + "_sorted_rows"] = e[2], e[3]
        out[name + "_offsets"] = e[4]
        out[name + "_dwte_accumulated"], out[name + "_dwpe_accumulated"] = ea[0], ea[1]
    np.savez_compressed(HERE / "embedding_backward.npz", **out)

    # GEMM float references (gate.py) on small shapes.
    out = {}
    g = torch.Generator().manual_seed(7)
    m, n, k = 72, 56, 40
    x = torch.randn(m, k, generator=g).half()
    w = (torch.randn(n, k, generator=g) * 0.05).half()
    wn = (torch.randn(k, n, generator=g) * 0.05).half()
    xt = torch.randn(k, m, generator=g).half()
    bias = torch.randn(n, generator=g)
    pre = torch.randn(m, n, generator=g).half()
    out.update(x=x.numpy(), w=w.numpy(), wn=wn.numpy(), xt=xt.numpy(), bias=bias.numpy(),
               pre=pre.numpy())
    out["nt"] = gate.reference(x, w).numpy()
    out["nt_bias"] = gate.reference_bias(x, w, bias).numpy()
    out["nt_bias_gelu"] = gate.reference_bias_gelu(x, w, bias).numpy()
    out["nn"] = gate.reference_nn(x, wn).numpy()
    out["nn_dgelu"] = gate.reference_dgelu(x, wn, pre).numpy()
    out["tn"] = gate.reference_tn(xt, wn).numpy()
    np.savez_compressed(HERE / "gemm_reference.npz", **out)

    # The PyTorch model: init checksums, loss and gradients of a small configuration, and one
    # AdamW step, all FP32 on the CPU.
    out = {}
    cfg = gpt2_torch.GPTConfig(n_layer=2, n_head=2, n_embd=64, block_size=32, vocab_size=200,
                               padded_vocab_size=208)
    model = gpt2_torch.build_model(cfg, seed=1234)
    gen = torch.Generator().manual_seed(99)
    ids = torch.randint(0, cfg.vocab_size, (2 * 32 + 1,), generator=gen)
    idx, targets = ids[:-1].view(2, 32), ids[1:].view(2, 32)
    loss = model(idx, targets)
    loss.backward()
    out["idx"], out["targets"] = idx.numpy(), targets.numpy()
    out["loss"] = np.array(loss.item())
    for name, p in model.named_parameters():
        out["param_sum/" + name] = np.array(p.detach().double().sum().item())
        out["param_abs/" + name] = np.array(p.detach().double().abs().sum().item())
        out["grad/" + name] = p.grad.numpy().copy()
    optimizer = gpt2_torch.configure_optimizer(model)
    optimizer.step()
    for name, p in model.named_parameters():
        out["stepped/" + name] = p.detach().numpy().copy()
    tiny = gpt2_torch.build_model(gpt2_torch.TINY_CONFIG, seed=1234)
    for name, p in tiny.named_parameters():
        out["tiny_sum/" + name] = np.array(p.detach().double().sum().item())
    out["names"] = np.array([n for n, _ in model.named_parameters()])
    np.savez_compressed(HERE / "gpt2_torch.npz", **out)
    print("wrote", sorted(p.name for p in HERE.glob("*.npz")))


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference [fixture ...]")
    main(sys.argv[1], tuple(sys.argv[2:]))
