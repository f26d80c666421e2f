"""Per-kernel timings at GPT-2 124M training shapes, through the C ABI.

The reference ships a C++ harness for the same purpose (``bench/gemm_bench.cpp``,
``bench/copy_bench.cpp``: one kernel, one shape, CUDA events). This is its Python
counterpart over ``flint_b200.Flint``:

    python -m flint_b200.kernel_bench --group gemm            # timing table
    python -m flint_b200.kernel_bench --group all --rows 4096 --once

Timing mode rotates over enough operand sets to exceed the 126 MB L2 and times 24
back-to-back calls between two CUDA events on the launch stream (GEMMs, attention), or
flushes L2 before every call (the bandwidth kernels). ``--once`` makes one call per kernel
and prints nothing but a completion line: the form to run under a profiler, with ``--rows``
reduced so that a capture stays small.
"""

import argparse

import torch

from .binding import Flint

DEV = "cuda"
WIDTH = 768
VOCAB, PADDED_VOCAB = 50257, 50304
L2_BYTES = 126e6


class Runner:
    def __init__(self, flint: Flint, once: bool):
        self.flint = flint
        self.once = once
        self.flush = None if once else torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def sets(self, bytes_per_set: float) -> int:
        return 1 if self.once else max(2, min(8, int(3 * L2_BYTES // bytes_per_set) + 1))

    def rotating(self, name, fn, sets, work, unit):
        """fn(i) on operand set i; `work` per call in flops or bytes."""
        if self.once:
            fn(0)
            torch.cuda.synchronize()
            print(f"{name}: done", flush=True)
            return
        for i in range(3):
            fn(i % sets)
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        calls = 24
        start.record()
        for i in range(calls):
            fn(i % sets)
        stop.record()
        torch.cuda.synchronize()
        self.report(name, start.elapsed_time(stop) / calls, work, unit)

    def flushed(self, name, fn, work, unit):
        """L2 flushed before each call; the median of 8 single-call timings."""
        if self.once:
            fn()
            torch.cuda.synchronize()
            print(f"{name}: done", flush=True)
            return
        times = []
        for _ in range(10):
            self.flush.zero_()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            fn()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        self.report(name, sorted(times[2:])[4], work, unit)

    @staticmethod
    def report(name, ms, work, unit):
        rate = work / ms / 1e9 if unit == "TFLOP/s" else work / ms / 1e6
        print(f"{name:36s} {ms * 1e3:9.1f} us {rate:9.1f} {unit}", flush=True)


def half(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).half()


def group_gemm(r: Runner, rows: int):
    f, w, w4 = r.flint, WIDTH, 4 * WIDTH
    n = r.sets(rows * w4 * 2 * 2)
    x = [half(rows, w) for _ in range(n)]
    x4 = [half(rows, w4) for _ in range(n)]
    x3 = [half(rows, 3 * w) for _ in range(n)]
    residual = [torch.randn(rows, w, device=DEV) for _ in range(n)]
    fc = [half(w4, w, scale=0.02) for _ in range(n)]
    pj = [half(w, w4, scale=0.02) for _ in range(n)]
    aw = [half(3 * w, w, scale=0.02) for _ in range(n)]
    pw = [half(w, w, scale=0.02) for _ in range(n)]
    b4, b1, b3 = (torch.randn(c, device=DEV) for c in (w4, w, 3 * w))
    y4 = [half(rows, w4) for _ in range(n)]
    pre = [half(rows, w4) for _ in range(n)]
    yf = [torch.empty(rows, w, device=DEV) for _ in range(n)]
    y1 = [half(rows, w) for _ in range(n)]
    grad = [torch.zeros(w4, w, device=DEV) for _ in range(n)]
    ws_bytes = max(16, f.gemm_tn_workspace(w4, w, rows))
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    fl = lambda m, nn, k: 2.0 * m * nn * k  # noqa: E731
    T = "TFLOP/s"
    r.rotating("gemm_nt 3072x768", lambda i: f.gemm_nt(y4[i], x[i], fc[i], rows, w4, w), n, fl(rows, w4, w), T)
    r.rotating("gemm_nt_bias 2304x768", lambda i: f.gemm_nt_bias(x3[i], x[i], aw[i], b3, rows, 3 * w, w), n,
               fl(rows, 3 * w, w), T)
    r.rotating("gemm_nt_bias_gelu 3072x768",
               lambda i: f.gemm_nt_bias_gelu(y4[i], pre[i], x[i], fc[i], b4, rows, w4, w), n, fl(rows, w4, w), T)
    r.rotating("gemm_nt_bias_residual 768x768",
               lambda i: f.gemm_nt_bias_residual(yf[i], x[i], pw[i], b1, residual[i], rows, w, w), n,
               fl(rows, w, w), T)
    r.rotating("gemm_nt_bias_residual 768x3072",
               lambda i: f.gemm_nt_bias_residual(yf[i], x4[i], pj[i], b1, residual[i], rows, w, w4), n,
               fl(rows, w, w4), T)
    r.rotating("gemm_nn_dgelu 3072<-768", lambda i: f.gemm_nn_dgelu(y4[i], x[i], pj[i], pre[i], rows, w4, w), n,
               fl(rows, w4, w), T)
    r.rotating("gemm_nn 768<-3072", lambda i: f.gemm_nn(y1[i], x4[i], fc[i], rows, w, w4), n, fl(rows, w, w4), T)
    r.rotating("gemm_nn 768<-768", lambda i: f.gemm_nn(y1[i], x[i], pw[i], rows, w, w), n, fl(rows, w, w), T)
    r.rotating("gemm_nn 768<-2304", lambda i: f.gemm_nn(y1[i], x3[i], aw[i], rows, w, 3 * w), n,
               fl(rows, w, 3 * w), T)
    r.rotating("gemm_tn 3072x768 (k = rows)",
               lambda i: f.gemm_tn(grad[i], x4[i], x[i], w4, w, rows, True, ws, ws_bytes), n, fl(w4, w, rows), T)


def group_attention(r: Runner, rows: int):
    f = r.flint
    length, heads = 1024, 12
    batches = max(1, rows // length) * heads
    q, k, v, d_o = (half(batches, length, 64) for _ in range(4))
    o = torch.zeros_like(q)
    dq, dk, dv = (torch.zeros_like(q) for _ in range(3))
    lse = torch.zeros(batches, length, device=DEV)
    delta = torch.zeros(batches, length, device=DEV)
    flops = 4.0 * length * length * 64 * batches / 2
    r.rotating(f"attention_forward {batches}x{length}",
               lambda i: f.attention_forward(o, lse, q, k, v, batches, length, 64, 0.125), 1, flops, "TFLOP/s")
    r.rotating(f"attention_backward {batches}x{length}",
               lambda i: f.attention_backward(dq, dk, dv, d_o, o, lse, delta, q, k, v, batches, length, 64, 0.125),
               1, 2.5 * flops, "TFLOP/s")


def group_rowwise(r: Runner, rows: int):
    f, w = r.flint, WIDTH
    logits = half(rows, PADDED_VOCAB, scale=2.0)
    dlogits = torch.empty_like(logits)
    targets = torch.randint(0, VOCAB, (rows,), device=DEV).to(torch.int16)
    loss = torch.empty(rows, device=DEV)
    r.flushed("softmax_cross_entropy",
              lambda: f.softmax_cross_entropy(dlogits, loss, logits, targets, 4.0, rows, VOCAB, PADDED_VOCAB),
              rows * PADDED_VOCAB * 4.0, "GB/s")
    del logits, dlogits
    x = torch.randn(rows, w, device=DEV)
    gain, shift = torch.randn(w, device=DEV), torch.randn(w, device=DEV)
    y = torch.empty(rows, w, dtype=torch.half, device=DEV)
    mean, rstd = torch.empty(rows, device=DEV), torch.empty(rows, device=DEV)
    r.flushed("layernorm_forward 768", lambda: f.layernorm_forward(y, mean, rstd, x, gain, shift, rows, w, 1e-5),
              rows * w * 6.0, "GB/s")
    yh = torch.empty(rows * w, dtype=torch.half, device=DEV)
    r.flushed("fp32_to_fp16", lambda: f.fp32_to_fp16(yh, x, rows * w), rows * w * 6.0, "GB/s")


def group_reductions(r: Runner, rows: int):
    f, w = r.flint, WIDTH
    for cols in (w, 3 * w, 4 * w):
        dy = half(rows, cols)
        db = torch.empty(cols, device=DEV)
        ws_bytes = f.bias_gradient_workspace(rows, cols)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
        r.flushed(f"bias_gradient {cols}",
                  lambda: f.bias_gradient(db, dy, rows, cols, False, ws, ws_bytes), rows * cols * 2.0, "GB/s")
    x = torch.randn(rows, w, device=DEV)
    dy = half(rows, w)
    gain = torch.randn(w, device=DEV)
    mean, rstd = torch.randn(rows, device=DEV), torch.rand(rows, device=DEV) + 0.5
    dx, dgain, dshift = torch.empty(rows, w, device=DEV), torch.empty(w, device=DEV), torch.empty(w, device=DEV)
    ws_bytes = f.layernorm_backward_workspace(rows, w)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    r.flushed("layernorm_backward 768",
              lambda: f.layernorm_backward(dx, dgain, dshift, dy, x, mean, rstd, gain, rows, w, False, False,
                                           ws, ws_bytes), rows * w * 10.0, "GB/s")


GROUPS = {"gemm": group_gemm, "attention": group_attention, "rowwise": group_rowwise,
          "reductions": group_reductions}


def main():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--group", default="all", choices=["all"] + list(GROUPS))
    parser.add_argument("--rows", type=int, default=16384, help="token rows (16 x 1024 in the bench)")
    parser.add_argument("--once", action="store_true", help="one call per kernel, no timing")
    args = parser.parse_args()
    flint = Flint()
    runner = Runner(flint, args.once)
    for name, group in GROUPS.items():
        if args.group in ("all", name):
            group(runner, args.rows)
    if flint.kernel_fault():
        raise SystemExit("a kernel gave up on a bounded wait")


if __name__ == "__main__":
    main()
