"""GPT-2 124M (12 layers, width 768, 12 heads, context 1024, vocabulary 50257 in 50304
columns) through flint_gpt2_forward / flint_gpt2_backward against the FP32 oracle, on a B200.

This is the configuration the benchmark times, at the shapes its kernels see: the
256 x 256 pair tiles of the GEMMs, the 50,304-column cross-entropy rows, twelve heads read
from the packed qkv rows by the fused attention kernels. Both model variants are checked: the
reference's layout (materialised scores) and the one built on fused attention. The bounds
are the task's: loss within 1e-2 of the FP32 oracle on the same seeded inputs, cosine
similarity >= 0.999 for every one of the 148 parameter gradients, and the target's entry of
dlogits at exactly the target's index. The reference gates the same quantities in
tests/test_gpt2.py:504-507 (logits, loss, dlogits, dlogits away from the targets) and
tests/test_gpt2_backward.py:285-317 (every parameter's gradient).

The default case runs 2 x 1024 tokens (the CPU oracle takes a few seconds); the `full_size`
case runs the whole 8 x 1024 batch of the single-step configuration.
"""

import numpy as np
import pytest
import torch

import flint_b200
import flint_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"
CFG = oracle.GPT2
LENGTH = 1024
LOSS_SCALE = 65536.0


def u16(t):
    return torch.from_numpy(t.numpy().astype(np.uint16).view(np.int16)).to(DEV)


def cosine(a, b):
    return torch.nn.functional.cosine_similarity(a.double().flatten(), b.double().flatten(), dim=0).item()


def rel_l2(got, want):
    return ((got.double() - want.double()).norm() / want.double().norm().clamp_min(1e-300)).item()


def weights(seed=1234):
    """The spec's initialisation rounded to FP16-representable FP32, with the reference's
    "mixed" perturbation so that no bias or LayerNorm parameter is trivially 0 or 1
    (tests/test_gpt2.py:194-208)."""
    params = oracle.gpt2_round_to_half(oracle.gpt2_init(CFG, seed=seed))
    g = torch.Generator().manual_seed(seed + 1)
    for name, p in params.items():
        if name.endswith(".bias") and "ln_" not in name:
            params[name] = (torch.randn(p.shape, generator=g) * 0.01).half().float()
        elif "ln_" in name:
            params[name] = (p + torch.randn(p.shape, generator=g) * 0.05).half().float()
    return params


class Case:
    def __init__(self, sequences, seed):
        self.sequences = sequences
        self.rows = sequences * LENGTH
        self.params = weights()
        self.idx, self.targets = oracle.synthetic_tokens(sequences, LENGTH, CFG["vocab_size"], seed=seed)
        # Two sequences at a time keep the oracle's saved T x T attention matrices to a few GB
        # of host memory; the chunks have equal sizes, so the batch's mean loss and its
        # gradient are the chunks' means.
        losses, logits, self.grads = [], [], None
        for first in range(0, sequences, 2):
            part = slice(first, first + 2)
            loss, grads, lg = oracle.gpt2_loss_and_gradients(CFG, self.params, self.idx[part],
                                                             self.targets[part], with_logits=True)
            losses.append(loss)
            logits.append(lg)
            if self.grads is None:
                self.grads = {k: g.double() for k, g in grads.items()}
            else:
                for k, g in grads.items():
                    self.grads[k] += g.double()
        chunks = len(losses)
        self.loss = sum(losses) / chunks
        self.logits = torch.cat(logits)
        self.grads = {k: (g / chunks).float() for k, g in self.grads.items()}


@pytest.fixture(scope="module")
def two_sequences():
    return Case(2, seed=11)


def run_and_check(flint, case, flash):
    config = flint_b200.Gpt2Config(CFG["n_layer"], CFG["n_head"], CFG["n_embd"], CFG["block_size"],
                                   CFG["vocab_size"], CFG["padded_vocab_size"], case.sequences, LENGTH,
                                   0, 1)
    vocab, padded, rows = CFG["vocab_size"], CFG["padded_vocab_size"], case.rows
    scale = LOSS_SCALE / rows
    targets = case.targets.flatten()
    with flint_b200.Gpt2(flint, config, flash) as model:
        names = [p[0] for p in model.parameters()]
        assert names == list(case.params) and len(names) == 148
        model.load({k: v.to(DEV) for k, v in case.params.items()})
        model.forward(u16(case.idx.flatten()), u16(targets), scale)
        model.backward(u16(case.idx.flatten()), False)
        loss = model.mean_loss()
        assert not flint.kernel_fault()

        # Loss and logits.
        assert abs(loss - case.loss) <= 1e-2, (loss, case.loss)
        logits_at, dlogits_at, row_loss_at = model.outputs()
        logits = model.read(logits_at, (rows, padded), torch.float16).cpu()
        assert rel_l2(logits[:, :vocab], case.logits) <= 2e-3
        assert not logits[:, vocab:].any()                      # padded wte rows are zero
        top1 = (logits[:, :vocab].float().argmax(1) == case.logits.argmax(1)).float().mean().item()
        assert top1 >= 0.95
        row_loss = model.read(row_loss_at, (rows,), torch.float32).cpu().double()
        want_rows = torch.nn.functional.cross_entropy(case.logits.double(), targets, reduction="none")
        assert (row_loss - want_rows).abs().max().item() <= 2e-2
        assert abs(row_loss.mean().item() - loss) <= 1e-6

        # dlogits: the target's entry sits at exactly the target's index (the only negative
        # entry of its row), padded columns are +0, and the whole matches scale * (p - onehot).
        dlogits = model.read(dlogits_at, (rows, padded), torch.float16).cpu()
        assert not dlogits[:, vocab:].view(torch.int16).any()
        negative = dlogits < 0
        assert bool((negative.sum(1) == 1).all())
        assert torch.equal(negative.float().argmax(1), targets)
        want = torch.softmax(case.logits.double(), 1) * scale
        want[torch.arange(rows), targets] -= scale
        assert rel_l2(dlogits[:, :vocab], want) <= 5e-3
        off_target = dlogits[:, :vocab].double().clone()
        off_target[torch.arange(rows), targets] = 0
        want[torch.arange(rows), targets] = 0
        assert rel_l2(off_target, want) <= 1e-2                 # the rest of each row, on its own
        del logits, dlogits, want, off_target

        # Every parameter's gradient.
        worst = (2.0, None)
        for name, address, rows_, cols in model.gradients():
            got = model.read(address, (rows_, cols), torch.float32).cpu() / LOSS_SCALE
            want = case.grads[name].reshape(rows_, cols)
            assert bool(torch.isfinite(got).all()), name
            c = cosine(got, want)
            worst = min(worst, (c, name))
            assert c >= 0.999, (name, c)
            assert rel_l2(got, want) <= 5e-2, (name, rel_l2(got, want))
        print(f"GPT-2 124M {case.sequences}x{LENGTH} flash={flash}: loss {loss:.5f} (oracle "
              f"{case.loss:.5f}), worst gradient cosine {worst[0]:.6f} at {worst[1]}")


@pytest.mark.parametrize("flash", [None, True], ids=["reference-layout", "fused-attention"])
def test_gpt2_124m_forward_and_backward_match_the_oracle(flint, two_sequences, flash):
    run_and_check(flint, two_sequences, flash)


@pytest.mark.parametrize("flash", [None, True], ids=["reference-layout", "fused-attention"])
def test_gpt2_124m_gradients_do_not_depend_on_cache_state(flint, flash):
    """Every kernel of the step hands work between its warps through mbarriers and between
    kernels through stream order (with programmatic dependent launch), so no result may depend
    on how long a load takes: forward + backward of 4 x 1024 tokens run four times, twice with
    the L2 flushed before the pass and twice warm, must leave bit-identical logits gradients
    and parameter gradients (one arena read compares all 148)."""
    sequences = 4
    config = flint_b200.Gpt2Config(CFG["n_layer"], CFG["n_head"], CFG["n_embd"], CFG["block_size"],
                                   CFG["vocab_size"], CFG["padded_vocab_size"], sequences, LENGTH,
                                   0, 1)
    rows = sequences * LENGTH
    idx, targets = oracle.synthetic_tokens(sequences, LENGTH, CFG["vocab_size"], seed=21)
    tokens, wanted = u16(idx.flatten()), u16(targets.flatten())
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=DEV)
    with flint_b200.Gpt2(flint, config, flash) as model:
        model.load({k: v.to(DEV) for k, v in weights().items()})
        grads = list(model.gradients())
        first_address = min(address for _, address, _, _ in grads)
        floats = (max(address + 4 * r * c for _, address, r, c in grads) - first_address) // 4
        _, dlogits_at, _ = model.outputs()
        first = None
        for trial in range(4):
            if trial % 2 == 0:
                flush.fill_(trial)
            model.forward(tokens, wanted, LOSS_SCALE / rows)
            model.backward(tokens, False)
            torch.cuda.synchronize()
            assert not flint.kernel_fault()
            got = (model.read(first_address, (floats,), torch.float32).clone(),
                   model.read(dlogits_at, (rows, CFG["padded_vocab_size"]), torch.float16).clone())
            if first is None:
                first = got
                continue
            assert torch.equal(first[0].view(torch.int32), got[0].view(torch.int32)), trial
            assert torch.equal(first[1].view(torch.int16), got[1].view(torch.int16)), trial


@pytest.mark.full_size
@pytest.mark.parametrize("flash", [None, True], ids=["reference-layout", "fused-attention"])
def test_gpt2_124m_single_step_configuration_at_8x1024(flint, flash, full_batch):
    run_and_check(flint, full_batch, flash)


@pytest.fixture(scope="module")
def full_batch():
    return Case(8, seed=12)
