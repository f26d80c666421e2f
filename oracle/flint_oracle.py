"""CPU oracle for the GPT-2 training-step kernels. TEST INFRASTRUCTURE ONLY.

This module restates, in numpy float32 / torch CPU arithmetic, what the
reference library (bayareahomelander/Flint) computes on the path this
repository accelerates. Only tests/, __graft_entry__.smoke() and bench.py's
CPU-baseline legs may import it, and only as the checker or as the timed CPU
baseline: the product (flint_b200/) never does.

Parity status: PINNED. tests/test_oracle_golden.py checks every function here
against tests/golden/*.npz, which tests/golden/make_golden.py generated in a
container that had the reference checked out, by calling the reference's own
bit-exact emulations (tests/test_bias_gradient.py, test_layernorm_backward.py,
test_softmax_backward.py, test_embedding_backward.py), its float references
(tests/gate.py and the float64 references inside test_layernorm.py,
test_softmax.py, test_cross_entropy.py, test_embedding.py,
test_gemm_bias_gelu.py, test_gemm_dgelu.py and the attention chain of
test_softmax_backward.py) and its PyTorch model and optimizer
(scripts/gpt2_torch.py).

Each function cites the reference file:line whose arithmetic it follows.
"""

import math

import numpy as np
import torch

F32 = np.float32
CHUNK_ROWS = 256  # rows per first-pass chunk of a column sum
LANE_ROWS = 8     # interleaved row streams inside a chunk
BUTTERFLY = (16, 8, 4, 2, 1)


# ---------------------------------------------------------------------------------------
# Compensated FP32 arithmetic (src/kernels/bias_gradient.cu:55-69, :127-129)
# ---------------------------------------------------------------------------------------

def two_sum_add(s, e, v):
    """(s, e) <- (s, e) + v with Knuth's TwoSum; every operation rounds to float32."""
    t = s + v
    vp = t - s
    err = (s - (t - vp)) + (v - vp)
    return t, e + err


def merge(a, b):
    """a <- a merged with b: errors added first, b's sum through TwoSum, errors added back."""
    errs = a[1] + b[1]
    s, e = two_sum_add(a[0], np.zeros_like(a[1]), b[0])
    return s, e + errs


def value(s, e):
    """sum + error, or the sum itself when it is not finite."""
    with np.errstate(all="ignore"):
        return np.where(np.isfinite(s), s + e, s).astype(F32)


def _column_sums(values, product_errors=None):
    """The two-pass column sum of an FP32 matrix [rows, cols].

    Pass 1 (bias_gradient.cu:82-119): per 256-row chunk, row stream y adds rows
    y, y+8, ... in order; stream 0 then merges streams 1..7 in order. Pass 2
    (:141-178): lane l merges chunks l, l+32, ...; a butterfly (xor 16, 8, 4, 2, 1)
    merges the lanes. product_errors (same shape), when given, holds each value's
    own exact rounding error, added to the error term before the value
    (layernorm_backward.cu:67-71).

    Returns (partial sums [chunks, cols], partial errors [chunks, cols], total [cols]).
    """
    values = np.ascontiguousarray(values, dtype=F32)
    rows, cols = values.shape
    chunks = -(-rows // CHUNK_ROWS)
    padded = chunks * CHUNK_ROWS
    with np.errstate(all="ignore"):
        s = np.zeros((chunks, LANE_ROWS, cols), dtype=F32)
        e = np.zeros_like(s)
        steps = CHUNK_ROWS // LANE_ROWS
        row_index = np.arange(padded).reshape(chunks, steps, LANE_ROWS)
        for i in range(steps):
            idx = row_index[:, i, :]                    # [chunks, 8]
            valid = (idx < rows)[..., None]             # rows past the end are never visited
            safe = np.minimum(idx, rows - 1)
            v = values[safe]                            # [chunks, 8, cols]
            if product_errors is not None:
                e_in = e + product_errors[safe]
            else:
                e_in = e
            ns, ne = two_sum_add(s, e_in, v)
            s = np.where(valid, ns, s)
            e = np.where(valid, ne, e)
        ps, pe = s[:, 0], e[:, 0]
        for y in range(1, LANE_ROWS):
            ps, pe = merge((ps, pe), (s[:, y], e[:, y]))
        # Pass 2.
        ls = np.zeros((32, cols), dtype=F32)
        le = np.zeros((32, cols), dtype=F32)
        for first in range(0, chunks, 32):
            n = min(32, chunks - first)
            ms, me = merge((ls[:n], le[:n]), (ps[first:first + n], pe[first:first + n]))
            ls[:n], le[:n] = ms, me
        lanes = np.arange(32)
        for off in BUTTERFLY:
            ls, le = merge((ls, le), (ls[lanes ^ off], le[lanes ^ off]))
        total = value(ls[0], le[0])
    return ps.astype(F32), pe.astype(F32), total


def _accumulate(total, old):
    return total if old is None else (np.asarray(old, dtype=F32) + total).astype(F32)


# ---------------------------------------------------------------------------------------
# flint_bias_gradient (src/kernels/bias_gradient.cu; emulation in tests/test_bias_gradient.py:165-403)
# ---------------------------------------------------------------------------------------

def bias_gradient(dy, old=None, with_partials=False):
    """dbias (float32 [cols]) for dy (float16 [rows, cols]); old + total with one add."""
    dy = np.asarray(dy)
    assert dy.dtype == np.float16 and dy.ndim == 2
    ps, pe, total = _column_sums(dy.astype(F32))
    with np.errstate(all="ignore"):
        total = _accumulate(total, old)
    return (total, ps, pe) if with_partials else total


# ---------------------------------------------------------------------------------------
# flint_layernorm_forward (src/kernels/layernorm.cu:105-155; FP64 reference in
# tests/test_layernorm.py:126-135)
# ---------------------------------------------------------------------------------------

def layernorm_forward(x, gamma, beta, eps=1e-5):
    """(y float64, mean float64, rstd float64) of the exact LayerNorm of float32 x."""
    x = torch.as_tensor(np.asarray(x), dtype=torch.float64)
    mean = x.mean(1)
    var = x.var(1, unbiased=False)
    rstd = 1.0 / torch.sqrt(var + eps)
    g = torch.as_tensor(np.asarray(gamma), dtype=torch.float64)
    b = torch.as_tensor(np.asarray(beta), dtype=torch.float64)
    y = (x - mean[:, None]) * rstd[:, None] * g + b
    return y.numpy(), mean.numpy(), rstd.numpy()


# ---------------------------------------------------------------------------------------
# flint_layernorm_backward (src/kernels/layernorm_backward.cu:119-233; emulation in
# tests/test_layernorm_backward.py:148-372)
# ---------------------------------------------------------------------------------------

def _xhat(x, mean, rstd):
    """(x - mean) * rstd with two roundings (layernorm_backward.cu:92-94)."""
    return ((x - mean[:, None]).astype(F32) * rstd[:, None]).astype(F32)


def layernorm_backward(dy, x, mean, rstd, gamma, old_dx=None, old_dgamma=None, old_dbeta=None,
                       with_partials=False):
    """(dx [rows, cols], dgamma [cols], dbeta [cols]) as float32, bit for bit.

    dx: lane l of a warp owns the 8-column pieces l, l+32, ... and adds g = dy*gamma
    and g*xhat over them in order with plain FP32 adds; a butterfly adds the lanes;
    dx = rstd * ((g - mean(g)) - xhat * mean(g*xhat)) (layernorm_backward.cu:138-169).
    dgamma: the column sum of dy*xhat with each product's rounding error
    (:185-233); dbeta: the column sum of dy.
    """
    dy = np.asarray(dy)
    assert dy.dtype == np.float16
    x = np.asarray(x, dtype=F32)
    mean = np.asarray(mean, dtype=F32)
    rstd = np.asarray(rstd, dtype=F32)
    gamma = np.asarray(gamma, dtype=F32)
    rows, cols = x.shape
    d = dy.astype(F32)
    with np.errstate(all="ignore"):
        xh = _xhat(x, mean, rstd)
        g = (d * gamma[None, :]).astype(F32)
        gx = (g * xh).astype(F32)
        pieces = cols // 8
        g_sum = np.zeros((rows, 32), dtype=F32)
        gx_sum = np.zeros((rows, 32), dtype=F32)
        lanes = np.arange(32)
        for k in range(-(-pieces // 32)):
            piece = lanes + 32 * k
            valid = piece < pieces
            safe = np.minimum(piece, pieces - 1)
            for j in range(8):
                col = safe * 8 + j
                g_sum = np.where(valid[None, :], g_sum + g[:, col], g_sum)
                gx_sum = np.where(valid[None, :], gx_sum + gx[:, col], gx_sum)
        for off in BUTTERFLY:
            g_sum = g_sum + g_sum[:, lanes ^ off]
            gx_sum = gx_sum + gx_sum[:, lanes ^ off]
        n = F32(cols)
        g_mean = (g_sum[:, 0] / n).astype(F32)
        gx_mean = (gx_sum[:, 0] / n).astype(F32)
        inner = ((g - g_mean[:, None]).astype(F32) - (xh * gx_mean[:, None]).astype(F32)).astype(F32)
        dx = (rstd[:, None] * inner).astype(F32)
        if old_dx is not None:
            dx = (np.asarray(old_dx, dtype=F32) + dx).astype(F32)

        # dgamma: products and their exact errors (float64 holds fp16 * fp32 exactly).
        prod = (d * xh).astype(F32)
        err = (d.astype(np.float64) * xh.astype(np.float64) - prod.astype(np.float64)).astype(F32)
        gs, ge, dgamma = _column_sums(prod, err)
        dgamma = _accumulate(dgamma, old_dgamma)
        dbeta = _accumulate(_column_sums(d)[2], old_dbeta)
    if with_partials:
        return dx, dgamma, dbeta, gs, ge
    return dx, dgamma, dbeta


# ---------------------------------------------------------------------------------------
# flint_causal_softmax_forward / _backward (src/kernels/softmax.cu:68-122,
# src/kernels/softmax_backward.cu:111-154; emulation in tests/test_softmax_backward.py:120-233)
# ---------------------------------------------------------------------------------------

def causal_softmax_forward(s):
    """float64 probabilities [batches, T, T] of float16 scores; zero above the diagonal."""
    s = torch.as_tensor(np.asarray(s)).to(torch.float64)
    t = s.shape[-1]
    mask = torch.tril(torch.ones(t, t, dtype=torch.bool))
    p = torch.softmax(s.masked_fill(~mask, float("-inf")), -1)
    return p.masked_fill(~mask, 0.0).numpy()


def causal_softmax_backward(p, dp, scale):
    """ds (float16 [batches, T, T]) bit for bit: lane l owns the visible 8-column
    chunks l, l+32, ...; v = p*dp is exact; TwoSum; butterfly merge; the error is
    dropped when the sum is not finite; out = (p * ((dp - s) - e)) * scale."""
    p = np.asarray(p)
    dp = np.asarray(dp)
    assert p.dtype == np.float16 and dp.dtype == np.float16
    batches, t_len, _ = p.shape
    pf = p.astype(F32).reshape(-1, t_len)
    df = dp.astype(F32).reshape(-1, t_len)
    rows = pf.shape[0]
    t = (np.arange(rows) % t_len)
    lanes = np.arange(32)
    scale = F32(scale)
    with np.errstate(all="ignore"):
        s = np.zeros((rows, 32), dtype=F32)
        e = np.zeros((rows, 32), dtype=F32)
        for k in range(-(-(t_len // 8) // 32)):
            chunk = lanes + 32 * k
            for j in range(8):
                col = chunk * 8 + j                                   # [32]
                valid = col[None, :] <= t[:, None]                    # [rows, 32]
                safe = np.minimum(col, t_len - 1)
                v = (pf[:, safe] * df[:, safe]).astype(F32)
                ns, ne = two_sum_add(s, e, v)
                s = np.where(valid, ns, s)
                e = np.where(valid, ne, e)
        for off in BUTTERFLY:
            s, e = merge((s, e), (s[:, lanes ^ off], e[:, lanes ^ off]))
        ds_sum = s[:, 0]
        ds_err = np.where(np.isfinite(ds_sum), e[:, 0], F32(0))
        diff = ((df - ds_sum[:, None]).astype(F32) - ds_err[:, None]).astype(F32)
        out = ((pf * diff).astype(F32) * scale).astype(F32)
        cols = np.arange(t_len)
        out = np.where(cols[None, :] <= t[:, None], out, F32(0))
    return out.astype(np.float16).reshape(batches, t_len, t_len)


# ---------------------------------------------------------------------------------------
# flint_softmax_cross_entropy (src/kernels/cross_entropy.cu:106-172; FP64 reference in
# tests/test_cross_entropy.py:220-231)
# ---------------------------------------------------------------------------------------

def softmax_cross_entropy(logits, targets, scale, vocab):
    """(row_loss float64 [rows], dlogits float64 [rows, cols]) of float16 logits."""
    lg = torch.as_tensor(np.asarray(logits)).to(torch.float64)
    tg = torch.as_tensor(np.asarray(targets).astype(np.int64))
    rows, cols = lg.shape
    visible = lg[:, :vocab]
    loss = torch.nn.functional.cross_entropy(visible, tg, reduction="none")
    grad = torch.softmax(visible, -1)
    grad[torch.arange(rows), tg] -= 1.0
    out = torch.zeros(rows, cols, dtype=torch.float64)
    out[:, :vocab] = grad * scale
    return loss.numpy(), out.numpy()


# ---------------------------------------------------------------------------------------
# flint_embedding_forward / _backward (src/kernels/embedding.cu:22-47,
# src/kernels/embedding_backward.cu:241-345; emulation in tests/test_embedding_backward.py:227-340)
# ---------------------------------------------------------------------------------------

def embedding_forward(tokens, wte, wpe, length):
    """x[r] = wte[tokens[r]] + wpe[r % length], one float32 add."""
    tokens = np.asarray(tokens).astype(np.int64)
    wte = np.asarray(wte, dtype=F32)
    wpe = np.asarray(wpe, dtype=F32)
    pos = np.arange(len(tokens)) % length
    return (wte[tokens] + wpe[pos]).astype(F32)


def embedding_backward(dx, tokens, sequences, length, vocab, old_dwte=None, old_dwpe=None):
    """(dwte [vocab, width], dwpe [length, width], sorted_tokens, sorted_rows, offsets).

    dwte[v]: TwoSum over token v's rows in ascending row order starting from +0,
    value = sum + error; untouched rows are +0 (or left alone when accumulating).
    dwpe: the column sum of dx viewed as [sequences, length*width]."""
    dx = np.asarray(dx, dtype=F32)
    tokens = np.asarray(tokens).astype(np.int64)
    rows, width = dx.shape
    order = np.argsort(tokens, kind="stable")
    sorted_tokens = tokens[order]
    offsets = np.searchsorted(sorted_tokens, np.arange(vocab + 1), side="left")
    counts = offsets[1:] - offsets[:-1]
    with np.errstate(all="ignore"):
        s = np.zeros((vocab, width), dtype=F32)
        e = np.zeros((vocab, width), dtype=F32)
        for rank in range(int(counts.max()) if vocab else 0):
            live = np.nonzero(counts > rank)[0]
            src = order[offsets[live] + rank]
            ns, ne = two_sum_add(s[live], e[live], dx[src])
            s[live], e[live] = ns, ne
        sums = value(s, e)
        touched = counts > 0
        if old_dwte is None:
            dwte = np.where(touched[:, None], sums, F32(0)).astype(F32)
        else:
            old = np.asarray(old_dwte, dtype=F32)
            dwte = np.where(touched[:, None], (old + sums).astype(F32), old)
        old_flat = None if old_dwpe is None else np.asarray(old_dwpe, dtype=F32).reshape(-1)
        dwpe = _accumulate(_column_sums(dx.reshape(sequences, length * width))[2], old_flat)
    return dwte, dwpe.reshape(length, width), sorted_tokens, order, offsets


# ---------------------------------------------------------------------------------------
# GEMM references (tests/gate.py:143-203): float64 products of the up-cast FP16 inputs
# ---------------------------------------------------------------------------------------

def _t64(a):
    return torch.as_tensor(np.asarray(a)).to(torch.float64)


def gelu_tanh(s):
    return torch.nn.functional.gelu(s, approximate="tanh")


def gelu_tanh_grad(pre):
    pre = pre.clone().requires_grad_(True)
    gelu_tanh(pre).sum().backward()
    return pre.grad


def gelu_exponent(s):
    """a in gelu(s) = s / (1 + exp(a)): -2 sqrt(2/pi) (s + 0.044715 s^3), float64
    (tests/test_gemm_bias_gelu.py:199-203)."""
    s = _t64(s)
    return -2.0 * math.sqrt(2.0 / math.pi) * s * (1.0 + 0.044715 * s * s)


def gelu_tanh_derivative(s):
    """(g, a): the derivative of the tanh GELU in closed form, float64, and its exponent a.
    With sigma = 1 / (1 + exp(a)): g = sigma + s sigma (1 - sigma) (-da/ds)
    (tests/test_gemm_dgelu.py:262-280). Limits 0 and 1 at -inf and +inf."""
    s = _t64(s)
    a = gelu_exponent(s)
    sigma = torch.sigmoid(-a)
    slope = 2.0 * math.sqrt(2.0 / math.pi) * (1.0 + 3 * 0.044715 * s * s)
    second = s * sigma * (1.0 - sigma) * slope
    second = torch.where(torch.isfinite(second), second, torch.zeros_like(second))
    return sigma + second, a


def half_ordered(h):
    """FP16 values as integers that rise with the value (both zeros are 0), so that
    neighbouring values differ by 1 (tests/test_gemm_bias_gelu.py:206-210)."""
    b = torch.as_tensor(np.asarray(h)).view(torch.int16).to(torch.int32)
    return torch.where(b < 0, -(b & 0x7FFF), b)


def half_rounding_margin(v):
    """How far each float64 value is from the nearest boundary between two FP16 roundings,
    as a fraction of the value; infinite for 0 and for values that overflow whatever their
    error (tests/test_gemm_bias_gelu.py:213-227)."""
    v = _t64(v)
    a = v.abs()
    exponent = torch.frexp(a)[1].double()
    ulp = torch.where(a < 2.0 ** -14, torch.full_like(a, 2.0 ** -24), torch.exp2(exponent - 11))
    fraction = (a / ulp) % 1.0
    margin = (fraction - 0.5).abs() * ulp / a
    margin = torch.where(a == 0, torch.full_like(a, math.inf), margin)
    return torch.where(a >= 65536, torch.full_like(a, math.inf), margin)


def round_to_half(v):
    """float64 -> FP16 with one rounding to nearest even. numpy converts directly; torch's
    double -> half goes through float and rounds twice (tests/test_gemm_dgelu.py:283-288)."""
    with np.errstate(over="ignore"):
        return torch.from_numpy(_t64(v).numpy().astype(np.float16))


def gemm_nt(x, w, bias=None):
    y = _t64(x) @ _t64(w).transpose(-1, -2)
    return y if bias is None else y + _t64(bias)


def gemm_nn(x, w):
    return _t64(x) @ _t64(w)


def gemm_tn(x, w):
    return _t64(x).transpose(-1, -2) @ _t64(w)


def gemm_nt_bias_gelu(x, w, bias):
    """(pre, y) in float64."""
    s = gemm_nt(x, w, bias)
    return s, gelu_tanh(s)


def gemm_nn_dgelu(x, w, pre):
    return gemm_nn(x, w) * gelu_tanh_grad(_t64(pre))


# ---------------------------------------------------------------------------------------
# Attention (scripts/gpt2_torch.py:52-60; FP64 chain in tests/test_softmax_backward.py:1429-1440)
# ---------------------------------------------------------------------------------------

def attention(q, k, v, scale, d_o=None):
    """Causal attention of [batches, T, d] float16 inputs in float64. Returns (o, lse) or,
    with d_o, (o, lse, dq, dk, dv)."""
    q, k, v = (_t64(a).requires_grad_(d_o is not None) for a in (q, k, v))
    t = q.shape[1]
    mask = torch.tril(torch.ones(t, t, dtype=torch.bool))
    s = (q @ k.transpose(1, 2)) * scale
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.softmax(s, -1) @ v
    if d_o is None:
        return o.numpy(), lse.numpy()
    o.backward(_t64(d_o))
    return (o.detach().numpy(), lse.detach().numpy(), q.grad.numpy(), k.grad.numpy(),
            v.grad.numpy())


# ---------------------------------------------------------------------------------------
# GPT-2 (scripts/gpt2_torch.py:21-192), functional FP32 restatement
# ---------------------------------------------------------------------------------------

INIT_STD = 0.02
LEARNING_RATE = 6e-4
BETAS = (0.9, 0.95)
EPSILON = 1e-8
WEIGHT_DECAY = 0.1
MAX_GRAD_NORM = 1.0

GPT2 = dict(n_layer=12, n_head=12, n_embd=768, block_size=1024, vocab_size=50257,
            padded_vocab_size=50304)
TINY = dict(n_layer=2, n_head=2, n_embd=128, block_size=64, vocab_size=50257,
            padded_vocab_size=50304)


def gpt2_parameter_shapes(cfg):
    """(name, shape) in torch's named_parameters order (gpt2_torch.py:86-93)."""
    w = cfg["n_embd"]
    out = [("wte.weight", (cfg["padded_vocab_size"], w)), ("wpe.weight", (cfg["block_size"], w))]
    for i in range(cfg["n_layer"]):
        p = f"blocks.{i}."
        out += [
            (p + "ln_1.weight", (w,)), (p + "ln_1.bias", (w,)),
            (p + "attn.c_attn.weight", (3 * w, w)), (p + "attn.c_attn.bias", (3 * w,)),
            (p + "attn.c_proj.weight", (w, w)), (p + "attn.c_proj.bias", (w,)),
            (p + "ln_2.weight", (w,)), (p + "ln_2.bias", (w,)),
            (p + "mlp.c_fc.weight", (4 * w, w)), (p + "mlp.c_fc.bias", (4 * w,)),
            (p + "mlp.c_proj.weight", (w, 4 * w)), (p + "mlp.c_proj.bias", (w,)),
        ]
    return out + [("ln_f.weight", (w,)), ("ln_f.bias", (w,))]


def gpt2_init(cfg, seed=1234):
    """The spec's init from a CPU generator (gpt2_torch.py:95-116): N(0, 0.02) for
    embeddings and Linear weights in module order, the residual projections scaled by
    1/sqrt(2 n_layer), zero biases, LayerNorm (1, 0), padded wte rows zero."""
    gen = torch.Generator("cpu").manual_seed(seed)
    residual_std = INIT_STD / math.sqrt(2 * cfg["n_layer"])
    params = {}
    for name, shape in gpt2_parameter_shapes(cfg):
        t = torch.empty(shape, dtype=torch.float32)
        if name.endswith(".bias"):
            t.zero_()
        elif ".ln_" in name or name.startswith("ln_f"):
            t.fill_(1.0)
        else:
            std = residual_std if name.endswith("c_proj.weight") else INIT_STD
            t.normal_(0.0, std, generator=gen)
        params[name] = t
    params["wte.weight"][cfg["vocab_size"]:].zero_()
    return params


def gpt2_round_to_half(params):
    """Every parameter rounded to an FP16-representable FP32 (tests/test_gpt2.py:194-208)."""
    return {k: v.half().float() for k, v in params.items()}


def _gpt2_hidden(cfg, p, idx):
    """The final LayerNorm's output [batch, length, width] of the model on idx [batch, length]
    (int64), with explicit causal-softmax attention; differentiable in the parameters."""
    batch, length = idx.shape
    w, h = cfg["n_embd"], cfg["n_head"]
    hw = w // h
    x = p["wte.weight"][idx] + p["wpe.weight"][:length]
    mask = torch.tril(torch.ones(length, length, dtype=torch.bool))
    for i in range(cfg["n_layer"]):
        b = f"blocks.{i}."
        y = torch.nn.functional.layer_norm(x, (w,), p[b + "ln_1.weight"], p[b + "ln_1.bias"], 1e-5)
        qkv = torch.nn.functional.linear(y, p[b + "attn.c_attn.weight"], p[b + "attn.c_attn.bias"])
        q, k, v = (t.view(batch, length, h, hw).transpose(1, 2) for t in qkv.split(w, dim=2))
        s = (q @ k.transpose(-1, -2)) * (1.0 / math.sqrt(hw))
        a = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ v
        a = a.transpose(1, 2).reshape(batch, length, w)
        x = x + torch.nn.functional.linear(a, p[b + "attn.c_proj.weight"], p[b + "attn.c_proj.bias"])
        y = torch.nn.functional.layer_norm(x, (w,), p[b + "ln_2.weight"], p[b + "ln_2.bias"], 1e-5)
        y = gelu_tanh(torch.nn.functional.linear(y, p[b + "mlp.c_fc.weight"], p[b + "mlp.c_fc.bias"]))
        x = x + torch.nn.functional.linear(y, p[b + "mlp.c_proj.weight"], p[b + "mlp.c_proj.bias"])
    return torch.nn.functional.layer_norm(x, (w,), p["ln_f.weight"], p["ln_f.bias"], 1e-5)


def gpt2_logits(cfg, params, idx, dtype=torch.float32):
    """Logits [batch * length, vocab_size] (padded columns dropped) of the model on idx
    [batch, length] (int64); differentiable in params."""
    p = {k: v.to(dtype) for k, v in params.items()} if dtype != torch.float32 else params
    x = _gpt2_hidden(cfg, p, idx)
    return torch.nn.functional.linear(x.reshape(-1, cfg["n_embd"]), p["wte.weight"])[:, :cfg["vocab_size"]]


def gpt2_loss(cfg, params, idx, targets, dtype=torch.float32):
    """Mean cross-entropy of the model on idx/targets [batch, length] (int64)."""
    logits = gpt2_logits(cfg, params, idx, dtype)
    return torch.nn.functional.cross_entropy(logits, targets.reshape(-1))


def gpt2_loss_and_gradients(cfg, params, idx, targets, dtype=torch.float32, with_logits=False):
    """(loss, {name: gradient}) by autograd on the CPU; with_logits adds the detached
    logits [rows, vocab_size] as a third value."""
    leaves = {k: v.detach().clone().to(dtype).requires_grad_(True) for k, v in params.items()}
    logits = gpt2_logits(cfg, leaves, idx)
    loss = torch.nn.functional.cross_entropy(logits, targets.reshape(-1))
    loss.backward()
    grads = {k: v.grad for k, v in leaves.items()}
    if with_logits:
        return loss.item(), grads, logits.detach()
    return loss.item(), grads


def clip_coefficient(grads, max_norm=MAX_GRAD_NORM):
    """(coefficient, total norm) of torch.nn.utils.clip_grad_norm_ over an iterable of
    gradients: min(1, max_norm / (norm + 1e-6)) (scripts/gpt2_torch.py:187-188)."""
    total = math.sqrt(sum(float(g.double().pow(2).sum()) for g in grads))
    return min(1.0, max_norm / (total + 1e-6)), total


def train_step(cfg, params, moments, batches, step, loss_scale=1.0, max_grad_norm=MAX_GRAD_NORM):
    """One optimizer step of scripts/gpt2_torch.py:178-192 on the CPU, in place: the
    micro-batches' gradients of loss / len(batches) accumulated, unscaled, clipped to
    max_grad_norm (0 or None: no clipping), then AdamW with the reference's two parameter
    groups. A non-finite gradient skips the update. Returns (mean loss, skipped, norm)."""
    total, loss_sum = None, 0.0
    for idx, targets in batches:
        loss, grads = gpt2_loss_and_gradients(cfg, params, idx, targets)
        loss_sum += loss
        scaled = {k: g * (loss_scale / len(batches)) for k, g in grads.items()}
        total = scaled if total is None else {k: total[k] + scaled[k] for k in total}
    grads = {k: g / loss_scale for k, g in total.items()}
    if not all(bool(torch.isfinite(g).all()) for g in grads.values()):
        return loss_sum / len(batches), True, math.inf
    coefficient, norm = clip_coefficient(grads.values(), max_grad_norm) if max_grad_norm else (1.0, 0.0)
    for name, p in params.items():
        wd = WEIGHT_DECAY if decayed(name, p.shape) else 0.0
        adamw_step(p, *moments[name], grads[name] * coefficient, step, weight_decay=wd)
    return loss_sum / len(batches), False, norm


def adamw_step(param, m, v, grad, step, lr=LEARNING_RATE, betas=BETAS, eps=EPSILON,
               weight_decay=WEIGHT_DECAY):
    """torch.optim.AdamW's update, in place, in float64 arithmetic rounded to the inputs'
    dtype at the end of each line (gpt2_torch.py:161-175 configures it)."""
    b1, b2 = betas
    m.mul_(b1).add_(grad, alpha=1 - b1)
    v.mul_(b2).addcmul_(grad, grad, value=1 - b2)
    m_hat = m / (1 - b1 ** step)
    v_hat = v / (1 - b2 ** step)
    param.mul_(1 - lr * weight_decay)
    param.sub_(lr * m_hat / (v_hat.sqrt() + eps))


def decayed(name, shape):
    """Weight decay applies to parameters with 2 or more dimensions (gpt2_torch.py:150-158)."""
    return len(shape) >= 2


def synthetic_tokens(sequences, length, vocab, seed):
    """Seeded uniform ids in [0, vocab): (idx, targets) with targets = ids shifted by one
    (tests/test_gpt2.py:219-241)."""
    gen = torch.Generator("cpu").manual_seed(seed)
    ids = torch.randint(0, vocab, (sequences * length + 1,), generator=gen)
    return ids[:-1].view(sequences, length), ids[1:].view(sequences, length)


# ---------------------------------------------------------------------------------------
# Decoding (the reference's inference milestone, README.md:148, has no code; the model is
# scripts/gpt2_torch.py's, so the logits of a position must be the full model's logits there)
# ---------------------------------------------------------------------------------------

def int8_rows(w):
    """Per-row symmetric int8 quantisation as the decoder applies it to the FP16 weights:
    scale = max|w[n, :]| / 127 (1 for an all-zero row) computed in float32, q = round-half-even
    (w / scale) clamped to [-127, 127]. Returns (q int8, scale float32, q * scale float32)."""
    w = torch.as_tensor(np.asarray(w)).to(torch.float16).float()
    top = w.abs().amax(1)
    scale = torch.where(top > 0, top / 127.0, torch.ones_like(top))
    inverse = (1.0 / scale)[:, None]
    q = torch.clamp(torch.round(w * inverse), -127, 127).to(torch.int8)
    return q, scale, q.float() * scale[:, None]


def decoder_weights(params, int8=False):
    """The weights a decoder computes with: every matrix rounded to FP16 (its compute copy),
    and with int8 replaced by its int8 approximation; the FP32 tables, biases and LayerNorm
    parameters as they are. The embedding lookup reads the FP32 table; the output layer the
    matrix copy."""
    out = {}
    for name, p in params.items():
        if p.dim() == 2 and name != "wpe.weight":
            half = p.half().float()
            out[name] = int8_rows(half)[2] if int8 else half
        else:
            out[name] = p
    return out


def gpt2_decode_logits(cfg, params, tokens, int8=False):
    """Logits [batch, length, vocab_size] of every position for tokens [batch, length], from
    the model with the decoder's weights (the token table stays FP32 for the lookup)."""
    weights = decoder_weights(params, int8)
    lookup = dict(weights)
    lookup["wte.weight"] = params["wte.weight"]
    batch, length = tokens.shape
    w = cfg["n_embd"]
    # gpt2_logits with two tables: the FP32 one for the embedding, the matrix copy for the head.
    hidden = _gpt2_hidden(cfg, lookup, tokens)
    logits = torch.nn.functional.linear(hidden.reshape(-1, w), weights["wte.weight"])
    return logits[:, :cfg["vocab_size"]].view(batch, length, -1)
