"""Greedy decoding with a KV cache over the C ABI (``flint_b200_generator_*``).

The reference lists inference (KV cache, decode attention, int8 weights) as a later
milestone (``README.md:148``) and has no code for it; the model is the one its PyTorch
script defines (``scripts/gpt2_torch.py:52-131``), so a position's logits must be the full
model's logits there. ``Generator`` wraps the C entry points; ``python -m
flint_b200.generate`` measures decode throughput:

    python -m flint_b200.generate --sequences 8 --prompt 512 --tokens 256 [--int8] [--no-graph]

and prints one JSON object: tokens/s over all sequences, microseconds per step, the bytes a
step must read (weights once, the cache once) and the fraction of the measured HBM
bandwidth that this is.
"""

import argparse
import ctypes
import json
from pathlib import Path

import torch

from .binding import Flint, Gpt2, Gpt2Config, stream_handle


class Generator:
    """A decoder for `model`'s weights: `sequences` sequences of up to `max_length` tokens."""

    def __init__(self, flint: Flint, model: Gpt2, sequences: int, max_length: int, int8=False):
        self.flint = flint
        self.sequences = sequences
        self.max_length = max_length
        handle = ctypes.c_void_p()
        flint.check(flint.lib.flint_b200_generator_create(model.handle, sequences, max_length,
                                                          int(bool(int8)), ctypes.byref(handle)))
        self.handle = handle.value
        self.padded_vocab = model.config.padded_vocab
        self.vocab = model.config.vocab
        # One buffer carries the tokens in and the greedy choices out: a step reads it in its
        # first kernel and writes it in its last, so the choices feed the next step as they are.
        self.tokens = torch.zeros(sequences, dtype=torch.int16, device="cuda")

    def close(self) -> None:
        if self.handle is not None:
            self.flint.lib.flint_b200_generator_destroy(self.handle)
            self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()

    def refresh(self, stream=None) -> None:
        self.flint.check(self.flint.lib.flint_b200_generator_refresh(self.handle, stream_handle(stream)))

    def prefill(self, tokens, stream=None) -> None:
        """tokens: uint16 bit patterns in an int16 device tensor [sequences, length]."""
        length = tokens.shape[1]
        self.flint.check(self.flint.lib.flint_b200_generator_prefill(
            self.handle, tokens.data_ptr(), length, stream_handle(stream)))

    def step(self, tokens=None, graph=False, stream=None):
        """Appends one token per sequence (int16 device tensor [sequences]; default: what the
        last step chose) and returns the device tensor `self.tokens`, which then holds each
        sequence's next greedy token."""
        if tokens is not None:
            self.tokens.copy_(tokens)
        self.flint.check(self.flint.lib.flint_b200_generator_step(
            self.handle, self.tokens.data_ptr(), self.tokens.data_ptr(), int(bool(graph)),
            stream_handle(stream)))
        return self.tokens

    def position(self) -> int:
        position = ctypes.c_size_t()
        self.flint.check(self.flint.lib.flint_b200_generator_logits(self.handle, None, ctypes.byref(position)))
        return position.value

    def logits(self) -> torch.Tensor:
        """FP32 [sequences, vocab] logits of the last position processed (a copy)."""
        from .trainer import device_tensor

        address = ctypes.c_void_p()
        self.flint.check(self.flint.lib.flint_b200_generator_logits(self.handle, ctypes.byref(address), None))
        torch.cuda.synchronize()
        view = device_tensor(address.value, self.sequences * self.padded_vocab)
        return view.view(self.sequences, self.padded_vocab)[:, :self.vocab].clone()

    def bytes_per_step(self):
        weights, cache = ctypes.c_size_t(), ctypes.c_size_t()
        self.flint.check(self.flint.lib.flint_b200_generator_bytes_per_step(
            self.handle, ctypes.byref(weights), ctypes.byref(cache)))
        return weights.value, cache.value

    def generate(self, prompt, count: int, graph=True):
        """Greedy continuation: prompt int16 [sequences, length] (length a multiple of 8),
        returns an int64 CPU tensor [sequences, count] of the tokens chosen."""
        self.prefill(prompt)
        first = self.logits().argmax(1).to(torch.int16).cuda()
        out = [first.cpu()]
        self.tokens.copy_(first)
        for i in range(count - 1):
            # The first step runs uncaptured so that every kernel is configured before a capture.
            out.append(self.step(graph=graph and i > 0).cpu())
        return torch.stack(out, 1).to(torch.int64) & 0xFFFF


def measure(flint: Flint, sequences: int, prompt: int, tokens: int, int8: bool, graph: bool) -> dict:
    """Decode throughput on GPT-2 124M with random-init weights and a seeded random prompt."""
    from .trainer import TrainerConfig, initial_weights

    config = Gpt2Config(12, 12, 768, 1024, 50257, 50304, 1, 8, 0, 0)
    hbm = 6538.6
    peaks = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    if peaks.is_file():
        hbm = json.loads(peaks.read_text()).get("hbm_gbs", hbm)
    with Gpt2(flint, config, True) as model:
        model.load({k: v.cuda() for k, v in initial_weights(TrainerConfig(), 1234).items()})
        with Generator(flint, model, sequences, 1024, int8) as g:
            gen = torch.Generator().manual_seed(5)
            ids = torch.randint(0, 50257, (sequences, prompt), generator=gen).to(torch.int16).cuda()
            g.prefill(ids)
            g.step(g.logits().argmax(1).to(torch.int16).cuda())          # configures every kernel
            for _ in range(3):
                g.step(graph=graph)
            weights0, cache0 = g.bytes_per_step()
            torch.cuda.synchronize()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(tokens):
                g.step(graph=graph)
            stop.record()
            torch.cuda.synchronize()
            weights1, cache1 = g.bytes_per_step()
            ms = start.elapsed_time(stop)
            if flint.kernel_fault():
                raise RuntimeError("a kernel gave up on a bounded wait")
    step_us = ms * 1e3 / tokens
    step_bytes = weights0 + (cache0 + cache1) / 2
    return {"metric": "GPT-2 124M greedy decode tokens/s", "sequences": sequences, "prompt": prompt,
            "tokens_per_sequence": tokens, "weights": "int8 (per-row scales)" if int8 else "fp16",
            "cuda_graph": graph, "tokens_per_second": round(sequences * tokens / (ms / 1e3), 1),
            "us_per_step": round(step_us, 2), "weight_bytes_per_step": weights0,
            "cache_bytes_per_step": int((cache0 + cache1) / 2),
            "hbm_gbs": round(step_bytes / step_us / 1e3, 1), "hbm_peak_gbs": hbm,
            "frac_of_measured_hbm": round(step_bytes / step_us / 1e3 / hbm, 4)}


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--sequences", type=int, default=8)
    parser.add_argument("--prompt", type=int, default=512, help="prompt tokens (a multiple of 8)")
    parser.add_argument("--tokens", type=int, default=256, help="decode steps to time")
    parser.add_argument("--int8", action="store_true")
    parser.add_argument("--no-graph", action="store_true")
    args = parser.parse_args(argv)
    print(json.dumps(measure(Flint(), args.sequences, args.prompt, args.tokens, args.int8,
                             not args.no_graph)), flush=True)


if __name__ == "__main__":
    main()
