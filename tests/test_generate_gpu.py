"""Decoding with a KV cache (extension) against the oracle's full-sequence model, on a B200.

The reference has no decoder (README.md:148 lists it as a later milestone); its model is
scripts/gpt2_torch.py's, so the logits the decoder leaves after a position must be the
model's logits at that position of the whole sequence. The oracle runs the FP32 model with
the weights the decoder computes with (matrices rounded to FP16, or their per-row int8
approximation), so the bound is the kernels' own error: relative L2 <= 5e-3 on a position's
logits (FP16 activations under FP32 accumulation, as for the training forward pass).
"""

import numpy as np
import pytest
import torch

import flint_b200
import flint_oracle as oracle
from flint_b200.generate import Generator

pytestmark = pytest.mark.gpu
DEV = "cuda"
SMALL = dict(n_layer=2, n_head=2, n_embd=128, block_size=64, vocab_size=200, padded_vocab_size=208)


def u16(t):
    return torch.from_numpy(t.numpy().astype(np.uint16).view(np.int16)).to(DEV)


def rel_l2(got, want):
    return ((got.double() - want.double()).norm() / want.double().norm().clamp_min(1e-300)).item()


def weights(cfg, seed=1234):
    params = oracle.gpt2_init(cfg, seed=seed)
    g = torch.Generator().manual_seed(seed + 1)
    for name, p in params.items():                      # nothing trivially 0 or 1
        if name.endswith(".bias") and "ln_" not in name:
            params[name] = torch.randn(p.shape, generator=g) * 0.02
        elif "ln_" in name:
            params[name] = p + torch.randn(p.shape, generator=g) * 0.05
    return params


def model_for(flint, cfg, params):
    config = flint_b200.Gpt2Config(cfg["n_layer"], cfg["n_head"], cfg["n_embd"], cfg["block_size"],
                                   cfg["vocab_size"], cfg["padded_vocab_size"], 1, 8, 0, 0)
    model = flint_b200.Gpt2(flint, config, True)
    model.load({k: v.to(DEV) for k, v in params.items()})
    return model


@pytest.mark.parametrize("int8", [False, True], ids=["fp16", "int8"])
@pytest.mark.parametrize("sequences", [3, 12])
def test_prefill_and_teacher_forced_steps_match_the_full_model(flint, sequences, int8):
    """A prompt of 16 tokens, then 12 given tokens one at a time: the logits after each
    position against the oracle's logits of the whole 28-token sequence. 12 sequences take
    the tensor-core path for the layers and two groups through the output layer."""
    params = weights(SMALL)
    prompt, steps = 16, 12
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, SMALL["vocab_size"], (sequences, prompt + steps), generator=g)
    want = oracle.gpt2_decode_logits(SMALL, params, tokens, int8=int8)
    model = model_for(flint, SMALL, params)
    try:
        with Generator(flint, model, sequences, 64, int8) as gen:
            gen.prefill(u16(tokens[:, :prompt]))
            assert gen.position() == prompt
            assert rel_l2(gen.logits().cpu(), want[:, prompt - 1]) <= 5e-3
            for t in range(prompt, prompt + steps):
                chosen = gen.step(u16(tokens[:, t])).cpu().to(torch.int64) & 0xFFFF
                got = gen.logits().cpu()
                assert rel_l2(got, want[:, t]) <= 5e-3, t
                assert torch.equal(chosen, got.argmax(1)), t          # greedy = argmax of its logits
                assert int(chosen.max()) < SMALL["vocab_size"]
            assert gen.position() == prompt + steps
    finally:
        model.close()
    assert not flint.kernel_fault()


@pytest.mark.parametrize("int8", [False, True], ids=["fp16", "int8"])
def test_captured_steps_equal_plain_steps_bit_for_bit(flint, int8):
    params = weights(SMALL)
    g = torch.Generator().manual_seed(4)
    prompt = torch.randint(0, SMALL["vocab_size"], (4, 8), generator=g)
    model = model_for(flint, SMALL, params)
    try:
        runs = []
        for graph in (False, True):
            with Generator(flint, model, 4, 64, int8) as gen:
                chosen = gen.generate(u16(prompt), 20, graph=graph)
                runs.append((chosen, gen.logits().cpu()))
        assert torch.equal(runs[0][0], runs[1][0])
        assert torch.equal(runs[0][1], runs[1][1])
    finally:
        model.close()
    assert not flint.kernel_fault()


def test_gpt2_124m_decode_matches_the_full_model(flint):
    """GPT-2 124M, two sequences, a 64-token prompt and eight greedy steps: each step's logits
    against the oracle's on the sequence generated so far."""
    cfg = oracle.GPT2
    params = weights(cfg)
    g = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg["vocab_size"], (2, 64), generator=g)
    model = model_for(flint, cfg, params)
    try:
        with Generator(flint, model, 2, 128, False) as gen:
            chosen = gen.generate(u16(prompt), 9, graph=True)
            last = gen.logits().cpu()
        sequence = torch.cat([prompt, chosen[:, :8]], 1)             # 72 tokens
        want = oracle.gpt2_decode_logits(cfg, params, sequence)
        assert rel_l2(last, want[:, -1]) <= 5e-3
        # Each greedy choice is the oracle's, wherever the oracle's top two are not a near tie.
        for t in range(8):
            top = want[:, 63 + t].topk(2, dim=1)
            clear = (top.values[:, 0] - top.values[:, 1]) > 2e-2
            assert torch.equal(chosen[clear, t], top.indices[clear, 0]), t
    finally:
        model.close()
    assert not flint.kernel_fault()


def test_int8_copies_follow_the_stated_quantisation(flint):
    """The decoder's int8 path against the oracle's model with q * scale weights passes the
    same bound as FP16 (above); here the quantisation itself: weights that are already an
    int8 grid (up to their FP16 rounding) lose next to nothing when quantised again, so the
    int8 decoder follows the FP16 one far more closely than it would on arbitrary weights
    (about 2e-2 at these shapes)."""
    params = weights(SMALL)
    for name, p in params.items():
        if p.dim() == 2 and name != "wpe.weight":
            q, scale, approx = oracle.int8_rows(p)
            params[name] = approx.half().float() if name != "wte.weight" else p
    g = torch.Generator().manual_seed(7)
    tokens = torch.randint(0, SMALL["vocab_size"], (2, 16), generator=g)
    model = model_for(flint, SMALL, params)
    try:
        outs = []
        for int8 in (False, True):
            with Generator(flint, model, 2, 64, int8) as gen:
                gen.prefill(u16(tokens[:, :8]))
                for t in range(8, 16):
                    gen.step(u16(tokens[:, t]))
                outs.append(gen.logits().cpu())
        assert rel_l2(outs[1], outs[0]) <= 1e-2
    finally:
        model.close()


def test_generator_argument_errors(flint):
    params = weights(SMALL)
    model = model_for(flint, SMALL, params)
    try:
        import ctypes

        handle = ctypes.c_void_p(1)
        status = flint.lib.flint_b200_generator_create(model.handle, 0, 64, 0, ctypes.byref(handle))
        assert status == flint_b200.ERROR_INVALID_ARGUMENT and handle.value is None
        assert "sequences (0) must be from 1 to 64" in flint.last_error()
        status = flint.lib.flint_b200_generator_create(model.handle, 2, 60, 0, ctypes.byref(handle))
        assert status == flint_b200.ERROR_INVALID_ARGUMENT
        assert "max_length (60) must be a multiple of 8" in flint.last_error()
        with Generator(flint, model, 2, 16, False) as gen:
            with pytest.raises(flint_b200.FlintError, match="length .12. must be a multiple of 8"):
                gen.prefill(torch.zeros(2, 12, dtype=torch.int16, device=DEV))
            gen.prefill(torch.zeros(2, 16, dtype=torch.int16, device=DEV))
            with pytest.raises(flint_b200.FlintError, match="the cache is full"):
                gen.step(torch.zeros(2, dtype=torch.int16, device=DEV))
    finally:
        model.close()
