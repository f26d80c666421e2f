"""Per-kernel benchmark at GPT-2 124M shapes, through the C ABI, beside cuBLAS/cuBLASLt.

The reference publishes its results with a C++ harness (``bench/gemm_bench.cpp:558-859``,
``bench/harness.cpp:158-311``, ``bench/report.cpp:372-560``): every kernel against its
cuBLAS / cuBLASLt counterpart, operand sets rotated past four times the L2 size,
interleaved rounds, the median with its range, an output check and clocks logged. This
module is that protocol over ``flint_b200.Flint``:

    python -m flint_b200.kernel_bench                         # every case, JSON lines + table
    python -m flint_b200.kernel_bench --group gemm --quick    # a subset, short samples
    python -m flint_b200.kernel_bench --group all --rows 2048 --once   # one call each, no timing

Cases (8,192 token rows = 8 x 1,024 unless ``--rows`` says otherwise):
  gemm       the 15 unfused GEMMs: forward NT, input-gradient NN, weight-gradient TN
             accumulating into FP32, FP16 entries N(0,1) * 0.02
  epilogue   the 8 fused-epilogue GEMMs: bias (qkv, projection, MLP up, MLP down), bias+GELU,
             GELU backward, bias+residual (two shapes)
  batched    the attention-shaped batched GEMMs of 96 heads
  attention  fused causal attention forward and backward, 96 heads x 1,024 x 64
  rowwise    LayerNorm forward/backward, causal softmax forward/backward, cross-entropy,
             embedding forward/backward, bias gradient, FP32->FP16, copy

The baseline arm is cuBLAS / cuBLASLt reached through torch, which is plumbing here, not
product: ``torch.mm`` / ``torch.addmm`` (``cublasGemmEx`` / ``cublasLtMatmul``, FP16 in, FP32
accumulate, reduced-precision reduction off), ``torch.addmm`` with a 1-D bias (the cuBLASLt
BIAS epilogue), ``torch._addmm_activation`` (GELU epilogue), cuDNN/flash attention through
``scaled_dot_product_attention``, and ATen's own kernels for the row-wise ops where one op
does the same job. Where torch exposes no single-call counterpart (the DGELU epilogue, the
FP32 bias+residual epilogue) the baseline is the shortest torch sequence and says so.

Each case prints one JSON object: microseconds per call (median over rounds, min, max),
TFLOP/s or GB/s from the algorithmic work, the fraction of the nominal peak (2,250 TFLOP/s
dense FP16; 8,000 GB/s) and of the peak measured on this pool (MEASURED_PEAKS.json: cuBLAS
burst, copy bandwidth), the baseline's figures, flint's speed relative to the baseline, the
median SM clock sampled while the case ran, whether the two arms' outputs agree, and for the
bandwidth-bound kernels the time a plain copy of the same number of bytes takes (kernels of
10 us are bound by launch and ramp-up: a 33 MB copy reaches about 0.6 of the peak itself).
``--once`` makes one call per kernel and prints nothing but a completion line: the form to
run under a profiler, with ``--rows`` reduced so that a capture stays small.
"""

import argparse
import ctypes
import json
import statistics
import sys
import threading
import time
from pathlib import Path

import torch

from .binding import Flint

DEV = "cuda"
WIDTH = 768
VOCAB, PADDED_VOCAB = 50257, 50304
HEADS, HEAD_WIDTH, LENGTH = 12, 64, 1024
NOMINAL_TFLOPS = 2250.0       # B200 dense FP16/BF16
NOMINAL_GBS = 8000.0          # HBM3e, "about 8 TB/s"
ROOT = Path(__file__).resolve().parent.parent


def measured_peaks():
    """(burst TFLOP/s, GB/s, source) for kernels timed in isolation."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return data.get("bf16_tflops", 1694.8), data.get("hbm_gbs", 6538.6), "measured"
    return 1590.0, 6650.0, "fallback"


class Clocks:
    """Samples the SM clock (NVML, every 10 ms) while a case runs. Reading only."""

    def __init__(self, index: int = 0):
        self.handle = None
        self.samples = []
        self.reasons = 0
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
        except Exception:  # no NVML: cases simply carry no clock
            self.handle = None
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        n = self.nvml
        while not self._stop.is_set():
            try:
                self.samples.append(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                self.reasons |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        self.samples, self.reasons = [], 0
        if self.handle is not None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *_):
        if self._thread is not None:
            self._stop.set()
            self._thread.join(timeout=2)
            self._thread = None

    def summary(self):
        if not self.samples:
            return None, []
        names = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                 0x40: "hw_thermal_slowdown"}
        return statistics.median(self.samples), [v for k, v in names.items() if self.reasons & k]


class Case:
    """One kernel at one shape: `flint(i)` and optionally `baseline(i)` run it on operand
    set i; `work` is the algorithmic FLOPs or bytes per call; `check()` returns the relative
    L2 distance between the two arms' outputs on set 0 (or None)."""

    def __init__(self, group, name, unit, work, sets, flint, baseline=None, baseline_name=None,
                 check=None, note=None, **shape):
        self.group, self.name, self.unit, self.work, self.sets = group, name, unit, work, sets
        self.flint, self.baseline, self.baseline_name = flint, baseline, baseline_name
        self.check, self.note, self.shape = check, note, shape


class Protocol:
    def __init__(self, quick: bool):
        self.warmup_s = 0.15 if quick else 1.0
        self.sample_ms = 25.0 if quick else 100.0
        self.rounds = 3 if quick else 10
        self.quick = quick


def time_calls(fn, sets, calls, first=0):
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(calls):
        fn((first + i) % sets)
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / calls


def warm(fn, sets, seconds):
    """Runs fn for about `seconds` and returns a first estimate of ms per call."""
    fn(0)
    torch.cuda.synchronize()
    estimate = max(time_calls(fn, sets, 3), 1e-3)
    calls = int(min(max(seconds * 1e3 / estimate, 3), 20000))
    return time_calls(fn, sets, calls)


# A call through ctypes (or through torch's dispatcher) costs the host about 8 us, more than the
# shortest kernels here run: below this estimate per call an arm is timed by replaying a CUDA
# graph of its calls, which takes the host out of the measurement (both arms, or neither).
GRAPH_BELOW_MS = 0.05


class Replay:
    """`fn` over all rotation sets, repeated until one graph holds about half a millisecond."""

    def __init__(self, fn, sets: int, estimate_ms: float):
        passes = max(1, int(0.5 / max(estimate_ms * sets, 1e-4)))
        self.calls = passes * sets
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(sets):
                fn(i)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            for _ in range(passes):
                for i in range(sets):
                    fn(i)
        self.graph.replay()
        torch.cuda.synchronize()

    def time(self, sample_ms: float, estimate_ms: float) -> float:
        replays = int(max(2, sample_ms / max(estimate_ms * self.calls, 1e-4)))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(replays):
            self.graph.replay()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) / (replays * self.calls)


def run_case(case: Case, protocol: Protocol, clocks: Clocks, peaks, copy_reference=None) -> dict:
    arms = {"flint": case.flint}
    if case.baseline is not None:
        arms["baseline"] = case.baseline
    estimate, failed = {}, {}
    for arm, fn in list(arms.items()):
        try:
            estimate[arm] = warm(fn, case.sets, protocol.warmup_s)
        except Exception as error:  # a baseline torch cannot run is reported, not fatal
            if arm == "flint":
                raise
            failed[arm] = f"{type(error).__name__}: {str(error).splitlines()[0][:160]}"
            del arms[arm]
    replays = {}
    if min(estimate[arm] for arm in arms) < GRAPH_BELOW_MS:
        try:
            replays = {arm: Replay(fn, case.sets, estimate[arm]) for arm, fn in arms.items()}
            for arm, replay in replays.items():
                estimate[arm] = replay.time(5.0, estimate[arm])
        except Exception:  # an arm that cannot be captured: both are timed from the stream
            replays = {}
            torch.cuda.synchronize()
    samples = {arm: [] for arm in arms}
    with clocks:
        for round_index in range(protocol.rounds):
            order = list(arms) if round_index % 2 == 0 else list(reversed(arms))
            for arm in order:
                if replays:
                    samples[arm].append(replays[arm].time(protocol.sample_ms, estimate[arm]))
                    continue
                calls = int(max(3, protocol.sample_ms / estimate[arm]))
                samples[arm].append(time_calls(arms[arm], case.sets, calls, first=round_index))
    sm_mhz, reasons = clocks.summary()
    tensor_peak, hbm_peak, source = peaks
    nominal, measured = (NOMINAL_TFLOPS, tensor_peak) if case.unit == "TFLOP/s" else (NOMINAL_GBS, hbm_peak)

    def side(ms_list):
        ms = statistics.median(ms_list)
        rate = case.work / ms / 1e9 if case.unit == "TFLOP/s" else case.work / ms / 1e6
        return {"us": round(ms * 1e3, 2), "us_min": round(min(ms_list) * 1e3, 2),
                "us_max": round(max(ms_list) * 1e3, 2), "rate": round(rate, 1),
                "frac_nominal": round(rate / nominal, 4), "frac_measured": round(rate / measured, 4)}

    out = {"group": case.group, "case": case.name, **case.shape, "unit": case.unit,
           "work_per_call": case.work, "rotation_sets": case.sets, "rounds": protocol.rounds,
           "sample_ms": protocol.sample_ms, "flint": side(samples["flint"]),
           "nominal_peak": nominal, "measured_peak": measured, "peak_source": source,
           "baseline_name": case.baseline_name, "baseline": None, "flint_over_baseline": None,
           "sm_mhz_median": sm_mhz, "clock_reasons": reasons,
           "timing": "cuda graph replay" if replays else "stream launches"}
    if "baseline" in samples:
        out["baseline"] = side(samples["baseline"])
        ratios = [b / f for f, b in zip(samples["flint"], samples["baseline"])]
        out["flint_over_baseline"] = {"median": round(statistics.median(ratios), 4),
                                      "min": round(min(ratios), 4), "max": round(max(ratios), 4)}
    if case.unit == "GB/s" and copy_reference is not None:
        # What a plain copy moving the same number of bytes achieves at this size: small kernels
        # are bound by launch and ramp-up, not by the memory system, and this shows by how much.
        copy_us = copy_reference(case.work)
        out["copy_same_bytes_us"] = round(copy_us, 2)
        out["flint_over_copy"] = round(copy_us / out["flint"]["us"], 4)
    if failed:
        out["baseline_error"] = failed.get("baseline")
    if case.note:
        out["note"] = case.note
    if case.check is not None and "baseline" in arms:
        try:
            out["outputs_rel_l2"] = case.check()
        except Exception as error:
            out["outputs_rel_l2"] = f"{type(error).__name__}: {str(error).splitlines()[0][:120]}"
    return out


class CopyReference:
    """Times flint_copy moving `bytes_moved` bytes (half read, half written) over rotating
    buffers larger than four times the L2, with the protocol's sample length; cached per size."""

    def __init__(self, flint: Flint, protocol: Protocol):
        self.flint, self.protocol, self.cache = flint, protocol, {}

    def __call__(self, bytes_moved: float) -> float:
        size = max(16, int(bytes_moved / 2) // 16 * 16)
        if size not in self.cache:
            sets = rotation_sets(2.0 * size, False)
            src = [torch.empty(size, dtype=torch.uint8, device=DEV) for _ in range(sets)]
            dst = [torch.empty(size, dtype=torch.uint8, device=DEV) for _ in range(sets)]
            fn = lambda i: self.flint.copy(dst[i], src[i], size)  # noqa: E731
            estimate = warm(fn, sets, min(self.protocol.warmup_s, 0.2))
            if estimate < GRAPH_BELOW_MS:
                replay = Replay(fn, sets, estimate)
                estimate = replay.time(5.0, estimate)
                samples = [replay.time(self.protocol.sample_ms, estimate)
                           for _ in range(self.protocol.rounds)]
            else:
                samples = [time_calls(fn, sets, int(max(3, self.protocol.sample_ms / estimate)), first=r)
                           for r in range(self.protocol.rounds)]
            self.cache[size] = statistics.median(samples) * 1e3
            del src, dst
        return self.cache[size]


# ---- operand helpers ---------------------------------------------------------------------------


def rotation_sets(bytes_per_set: float, once: bool) -> int:
    """floor(4 * L2 / bytes) + 1 operand sets (the reference's rule), capped so that the
    whole rotation stays under 6 GB."""
    if once:
        return 1
    l2 = torch.cuda.get_device_properties(0).L2_cache_size
    sets = int(4 * l2 // bytes_per_set) + 1
    return int(max(2, min(sets, 6e9 // bytes_per_set, 64)))


def half(*shape, scale=1.0, gen=None):
    return (torch.randn(*shape, device=DEV, generator=gen) * scale).half()


def rel_l2(a, b):
    a, b = a.double(), b.double()
    return round(((a - b).norm() / b.norm().clamp_min(1e-300)).item(), 7)


def flop(m, n, k):
    return 2.0 * m * n * k


# ---- groups --------------------------------------------------------------------------------------


def gemm_cases(f: Flint, rows: int, once: bool, sigma_x: float):
    w, v = WIDTH, PADDED_VOCAB
    gen = torch.Generator(device=DEV).manual_seed(0x5EED0001)
    cases = []
    nt = [(rows, 3 * w, w), (rows, w, w), (rows, 4 * w, w), (rows, w, 4 * w), (rows, v, w)]
    nn = [(rows, w, 3 * w), (rows, w, w), (rows, w, 4 * w), (rows, 4 * w, w), (rows, w, v)]
    tn = [(3 * w, w, rows), (w, w, rows), (4 * w, w, rows), (w, 4 * w, rows), (v, w, rows)]

    for m, n, k in nt:
        sets = rotation_sets((m * k + n * k + m * n) * 2, once)
        x = [half(m, k, scale=sigma_x, gen=gen) for _ in range(sets)]
        wt = [half(n, k, scale=0.02, gen=gen) for _ in range(sets)]
        y = [torch.empty(m, n, dtype=torch.half, device=DEV) for _ in range(sets)]
        yb = torch.empty(m, n, dtype=torch.half, device=DEV)
        cases.append(Case(
            "gemm", f"nt {m}x{n}x{k}", "TFLOP/s", flop(m, n, k), sets,
            lambda i, x=x, wt=wt, y=y, m=m, n=n, k=k: f.gemm_nt(y[i], x[i], wt[i], m, n, k),
            lambda i, x=x, wt=wt, yb=yb: torch.mm(x[i], wt[i].t(), out=yb), "cuBLAS (torch.mm)",
            lambda x=x, wt=wt, y=y, yb=yb, m=m, n=n, k=k: (
                f.gemm_nt(y[0], x[0], wt[0], m, n, k), torch.mm(x[0], wt[0].t(), out=yb),
                rel_l2(y[0], yb))[2],
            layout="NT", epilogue=None, m=m, n=n, k=k))
    for m, n, k in nn:
        sets = rotation_sets((m * k + n * k + m * n) * 2, once)
        x = [half(m, k, scale=sigma_x, gen=gen) for _ in range(sets)]
        wn = [half(k, n, scale=0.02, gen=gen) for _ in range(sets)]
        y = [torch.empty(m, n, dtype=torch.half, device=DEV) for _ in range(sets)]
        yb = torch.empty(m, n, dtype=torch.half, device=DEV)
        cases.append(Case(
            "gemm", f"nn {m}x{n}x{k}", "TFLOP/s", flop(m, n, k), sets,
            lambda i, x=x, wn=wn, y=y, m=m, n=n, k=k: f.gemm_nn(y[i], x[i], wn[i], m, n, k),
            lambda i, x=x, wn=wn, yb=yb: torch.mm(x[i], wn[i], out=yb), "cuBLAS (torch.mm)",
            lambda x=x, wn=wn, y=y, yb=yb, m=m, n=n, k=k: (
                f.gemm_nn(y[0], x[0], wn[0], m, n, k), torch.mm(x[0], wn[0], out=yb),
                rel_l2(y[0], yb))[2],
            layout="NN", epilogue=None, m=m, n=n, k=k))
    for m, n, k in tn:
        sets = rotation_sets((k * m + k * n) * 2 + m * n * 8, once)
        xt = [half(k, m, scale=sigma_x, gen=gen) for _ in range(sets)]
        wn = [half(k, n, scale=0.02, gen=gen) for _ in range(sets)]
        y = [torch.randn(m, n, device=DEV, generator=gen) for _ in range(sets)]
        yb = [t.clone() for t in y]
        nbytes = max(16, f.gemm_tn_workspace(m, n, k))
        ws = torch.empty(nbytes, dtype=torch.uint8, device=DEV)

        def check(xt=xt, wn=wn, m=m, n=n, k=k, ws=ws, nbytes=nbytes):
            a = torch.zeros(m, n, device=DEV)
            b = torch.zeros(m, n, device=DEV)
            f.gemm_tn(a, xt[0], wn[0], m, n, k, True, ws, nbytes)
            torch.addmm(b, xt[0].t(), wn[0], out_dtype=torch.float32, out=b)
            return rel_l2(a, b)

        cases.append(Case(
            "gemm", f"tn {m}x{n}x{k} (+= FP32)", "TFLOP/s", flop(m, n, k), sets,
            lambda i, xt=xt, wn=wn, y=y, m=m, n=n, k=k, ws=ws, nbytes=nbytes:
                f.gemm_tn(y[i], xt[i], wn[i], m, n, k, True, ws, nbytes),
            lambda i, xt=xt, wn=wn, yb=yb:
                torch.addmm(yb[i], xt[i].t(), wn[i], out_dtype=torch.float32, out=yb[i]),
            "cuBLAS (torch.addmm, FP32 C, beta 1)", check,
            layout="TN", epilogue="accumulate", m=m, n=n, k=k))
    return cases


def gelu_case(f: Flint, rows: int, once: bool, gen):
    """MLP up + bias + tanh-GELU (flint also writes the pre-activation)."""
    m, n, k = rows, 4 * WIDTH, WIDTH
    sets = rotation_sets((m * k + n * k + 2 * m * n) * 2, once)
    x = [half(m, k, gen=gen) for _ in range(sets)]
    wt = [half(n, k, scale=0.02, gen=gen) for _ in range(sets)]
    y = [torch.empty(m, n, dtype=torch.half, device=DEV) for _ in range(sets)]
    pre = [torch.empty(m, n, dtype=torch.half, device=DEV) for _ in range(sets)]
    bias = torch.randn(n, device=DEV, generator=gen) * 0.02
    bias16 = bias.half()
    return Case(
        "epilogue", f"nt+bias+gelu {m}x{n}x{k}", "TFLOP/s", flop(m, n, k), sets,
        lambda i: f.gemm_nt_bias_gelu(y[i], pre[i], x[i], wt[i], bias, m, n, k),
        lambda i: torch._addmm_activation(bias16, x[i], wt[i].t(), use_gelu=True),
        "cuBLASLt GELU_BIAS epilogue (torch._addmm_activation; no pre-activation output)",
        lambda: (f.gemm_nt_bias_gelu(y[0], pre[0], x[0], wt[0], bias, m, n, k),
                 rel_l2(y[0], torch._addmm_activation(bias16, x[0], wt[0].t(), use_gelu=True)))[1],
        note="flint writes two outputs (GELU and the saved pre-activation), the baseline one",
        layout="NT", epilogue="bias+gelu", m=m, n=n, k=k)


def dgelu_case(f: Flint, rows: int, once: bool, gen):
    """MLP-down input gradient + GELU backward from the saved pre-activation."""
    m, n, k = rows, 4 * WIDTH, WIDTH
    sets = rotation_sets((m * k + n * k + 2 * m * n) * 2, once)
    dy = [half(m, k, gen=gen) for _ in range(sets)]
    wn = [half(k, n, scale=0.02, gen=gen) for _ in range(sets)]
    saved = [half(m, n, scale=2.0, gen=gen) for _ in range(sets)]
    dh = [torch.empty(m, n, dtype=torch.half, device=DEV) for _ in range(sets)]
    tmp = torch.empty(m, n, dtype=torch.half, device=DEV)

    def baseline(i):
        torch.mm(dy[i], wn[i], out=tmp)
        return torch.ops.aten.gelu_backward(tmp, saved[i], approximate="tanh")

    return Case(
        "epilogue", f"nn+dgelu {m}x{n}x{k}", "TFLOP/s", flop(m, n, k), sets,
        lambda i: f.gemm_nn_dgelu(dh[i], dy[i], wn[i], saved[i], m, n, k), baseline,
        "cuBLAS GEMM + ATen gelu_backward (torch exposes no DGELU epilogue): two kernels",
        lambda: (f.gemm_nn_dgelu(dh[0], dy[0], wn[0], saved[0], m, n, k), rel_l2(dh[0], baseline(0)))[1],
        layout="NN", epilogue="dgelu", m=m, n=n, k=k)


def epilogue_cases(f: Flint, rows: int, once: bool):
    w, w4 = WIDTH, 4 * WIDTH
    gen = torch.Generator(device=DEV).manual_seed(0x5EED0002)
    cases = []
    # bias only: qkv, attention projection, MLP up, MLP down
    for label, (m, n, k) in {"qkv": (rows, 3 * w, w), "projection": (rows, w, w),
                             "mlp up": (rows, w4, w), "mlp down": (rows, w, w4)}.items():
        sets = rotation_sets((m * k + n * k + m * n) * 2, once)
        x = [half(m, k, gen=gen) for _ in range(sets)]
        wt = [half(n, k, scale=0.02, gen=gen) for _ in range(sets)]
        y = [torch.empty(m, n, dtype=torch.half, device=DEV) for _ in range(sets)]
        yb = torch.empty(m, n, dtype=torch.half, device=DEV)
        bias = torch.randn(n, device=DEV, generator=gen) * 0.02
        bias16 = bias.half()
        cases.append(Case(
            "epilogue", f"nt+bias {label} {m}x{n}x{k}", "TFLOP/s", flop(m, n, k), sets,
            lambda i, x=x, wt=wt, y=y, bias=bias, m=m, n=n, k=k:
                f.gemm_nt_bias(y[i], x[i], wt[i], bias, m, n, k),
            lambda i, x=x, wt=wt, yb=yb, bias16=bias16: torch.addmm(bias16, x[i], wt[i].t(), out=yb),
            "cuBLASLt BIAS epilogue (torch.addmm, FP16 bias)",
            lambda x=x, wt=wt, y=y, yb=yb, bias=bias, bias16=bias16, m=m, n=n, k=k: (
                f.gemm_nt_bias(y[0], x[0], wt[0], bias, m, n, k),
                torch.addmm(bias16, x[0], wt[0].t(), out=yb), rel_l2(y[0], yb))[2],
            layout="NT", epilogue="bias", m=m, n=n, k=k))

    cases.append(gelu_case(f, rows, once, gen))
    cases.append(dgelu_case(f, rows, once, gen))

    # bias + FP32 residual, FP32 out: attention projection and MLP down
    for label, (m, n, k) in {"projection": (rows, w, w), "mlp down": (rows, w, w4)}.items():
        sets = rotation_sets((m * k + n * k) * 2 + 2 * m * n * 4, once)
        x = [half(m, k, gen=gen) for _ in range(sets)]
        wt = [half(n, k, scale=0.02, gen=gen) for _ in range(sets)]
        residual = [torch.randn(m, n, device=DEV, generator=gen).half().float() for _ in range(sets)]
        y = [torch.empty(m, n, device=DEV) for _ in range(sets)]
        yb = torch.empty(m, n, device=DEV)
        bias = torch.randn(n, device=DEV, generator=gen) * 0.02

        def residual_baseline(i, x=x, wt=wt, residual=residual, yb=yb, bias=bias):
            torch.addmm(residual[i], x[i], wt[i].t(), out_dtype=torch.float32, out=yb)
            return yb.add_(bias)

        cases.append(Case(
            "epilogue", f"nt+bias+residual {label} {m}x{n}x{k}", "TFLOP/s", flop(m, n, k), sets,
            lambda i, x=x, wt=wt, y=y, residual=residual, bias=bias, m=m, n=n, k=k:
                f.gemm_nt_bias_residual(y[i], x[i], wt[i], bias, residual[i], m, n, k),
            residual_baseline,
            "cuBLAS (torch.addmm, FP32 C = residual, beta 1) + bias add: two kernels",
            lambda x=x, wt=wt, y=y, residual=residual, bias=bias, m=m, n=n, k=k, rb=residual_baseline: (
                f.gemm_nt_bias_residual(y[0], x[0], wt[0], bias, residual[0], m, n, k),
                rel_l2(y[0], rb(0)))[1],
            layout="NT", epilogue="bias+residual (FP32)", m=m, n=n, k=k))
    return cases


def batched_cases(f: Flint, rows: int, once: bool):
    batches = max(1, rows // LENGTH) * HEADS
    t, d = LENGTH, HEAD_WIDTH
    gen = torch.Generator(device=DEV).manual_seed(0x5EED0003)
    q, k_, v = (half(batches, t, d, gen=gen) for _ in range(3))
    p = half(batches, t, t, scale=0.03, gen=gen)
    s = torch.empty(batches, t, t, dtype=torch.half, device=DEV)
    sb = torch.empty_like(s)
    o = torch.empty(batches, t, d, dtype=torch.half, device=DEV)
    ob = torch.empty_like(o)
    cases = [
        Case("batched", f"nt batched {batches} x {t}x{t}x{d} (S = QK^T / 8)", "TFLOP/s",
             batches * flop(t, t, d), 1,
             lambda i: f.gemm_nt_batched(s, q, k_, batches, t, t, d, 0.125),
             lambda i: torch.baddbmm(sb, q, k_.transpose(1, 2), beta=0, alpha=0.125, out=sb),
             "cuBLAS strided batched (torch.baddbmm)",
             lambda: (f.gemm_nt_batched(s, q, k_, batches, t, t, d, 0.125),
                      torch.baddbmm(sb, q, k_.transpose(1, 2), beta=0, alpha=0.125, out=sb),
                      rel_l2(s, sb))[2],
             layout="NT", epilogue="scale", batches=batches, m=t, n=t, k=d),
        Case("batched", f"nn batched {batches} x {t}x{d}x{t} (O = PV)", "TFLOP/s",
             batches * flop(t, d, t), 1,
             lambda i: f.gemm_nn_batched(o, p, v, batches, t, d, t),
             lambda i: torch.bmm(p, v, out=ob), "cuBLAS strided batched (torch.bmm)",
             lambda: (f.gemm_nn_batched(o, p, v, batches, t, d, t), torch.bmm(p, v, out=ob),
                      rel_l2(o, ob))[2],
             layout="NN", epilogue=None, batches=batches, m=t, n=d, k=t),
        Case("batched", f"tn batched {batches} x {t}x{d}x{t} (dV = P^T dO)", "TFLOP/s",
             batches * flop(t, d, t), 1,
             lambda i: f.gemm_tn_batched(o, p, q, batches, t, d, t),
             lambda i: torch.bmm(p.transpose(1, 2), q, out=ob), "cuBLAS strided batched (torch.bmm)",
             lambda: (f.gemm_tn_batched(o, p, q, batches, t, d, t),
                      torch.bmm(p.transpose(1, 2), q, out=ob), rel_l2(o, ob))[2],
             layout="TN", epilogue=None, batches=batches, m=t, n=d, k=t),
    ]
    return cases


def attention_cases(f: Flint, rows: int, once: bool):
    batches = max(1, rows // LENGTH) * HEADS
    t, d = LENGTH, HEAD_WIDTH
    gen = torch.Generator(device=DEV).manual_seed(0x5EED0004)
    q, k_, v, d_o = (half(batches, t, d, gen=gen) for _ in range(4))
    o = torch.zeros_like(q)
    dq, dk, dv = (torch.zeros_like(q) for _ in range(3))
    lse = torch.zeros(batches, t, device=DEV)
    delta = torch.zeros(batches, t, device=DEV)
    flops = 4.0 * t * t * d * batches / 2
    sdpa = torch.nn.functional.scaled_dot_product_attention
    q4, k4, v4 = (a.view(batches // HEADS, HEADS, t, d) for a in (q, k_, v))
    leaves = [a.detach().clone().requires_grad_(True) for a in (q4, k4, v4)]
    state = {}

    def baseline_backward(i):
        if "out" not in state:
            state["out"] = sdpa(*leaves, is_causal=True, scale=0.125)
        return torch.autograd.grad(state["out"], leaves, d_o.view_as(q4), retain_graph=True)

    def check_backward():
        f.attention_forward(o, lse, q, k_, v, batches, t, d, 0.125)
        f.attention_backward(dq, dk, dv, d_o, o, lse, delta, q, k_, v, batches, t, d, 0.125)
        want = baseline_backward(0)
        return max(rel_l2(dq, want[0].reshape_as(dq)), rel_l2(dk, want[1].reshape_as(dk)),
                   rel_l2(dv, want[2].reshape_as(dv)))

    f.attention_forward(o, lse, q, k_, v, batches, t, d, 0.125)
    return [
        Case("attention", f"attention forward {batches} x {t} x {d}", "TFLOP/s", flops, 1,
             lambda i: f.attention_forward(o, lse, q, k_, v, batches, t, d, 0.125),
             lambda i: sdpa(q4, k4, v4, is_causal=True, scale=0.125),
             "torch scaled_dot_product_attention (fused library kernel)",
             lambda: (f.attention_forward(o, lse, q, k_, v, batches, t, d, 0.125),
                      rel_l2(o, sdpa(q4, k4, v4, is_causal=True, scale=0.125).reshape_as(o)))[1],
             batches=batches, length=t, head_width=d),
        Case("attention", f"attention backward {batches} x {t} x {d}", "TFLOP/s", 2.5 * flops, 1,
             lambda i: f.attention_backward(dq, dk, dv, d_o, o, lse, delta, q, k_, v, batches, t, d, 0.125),
             baseline_backward, "torch scaled_dot_product_attention backward (autograd.grad)",
             check_backward, batches=batches, length=t, head_width=d),
    ]


def rowwise_cases(f: Flint, rows: int, once: bool):
    w = WIDTH
    gen = torch.Generator(device=DEV).manual_seed(0x5EED0005)
    cases = []
    G = "GB/s"

    # LayerNorm forward: FP32 rows in, FP16 rows + mean + rstd out.
    sets = rotation_sets(rows * w * 6, once)
    x = [torch.randn(rows, w, device=DEV, generator=gen).half().float() for _ in range(sets)]
    gain = 1 + 0.02 * torch.randn(w, device=DEV, generator=gen)
    shift = torch.zeros(w, device=DEV)
    y = [torch.empty(rows, w, dtype=torch.half, device=DEV) for _ in range(sets)]
    mean, rstd = torch.empty(rows, device=DEV), torch.empty(rows, device=DEV)
    cases.append(Case("rowwise", f"layernorm forward {rows}x{w}", G, rows * w * 6.0 + rows * 8.0, sets,
                      lambda i: f.layernorm_forward(y[i], mean, rstd, x[i], gain, shift, rows, w, 1e-5),
                      lambda i: torch.native_layer_norm(x[i], [w], gain, shift, 1e-5),
                      "ATen native_layer_norm (FP32 out: 8 B per element)", rows=rows, cols=w))

    # LayerNorm backward.
    dy = [half(rows, w, gen=gen) for _ in range(sets)]
    dx = [torch.empty(rows, w, device=DEV) for _ in range(sets)]
    dgain, dshift = torch.empty(w, device=DEV), torch.empty(w, device=DEV)
    f.layernorm_forward(y[0], mean, rstd, x[0], gain, shift, rows, w, 1e-5)
    nbytes = f.layernorm_backward_workspace(rows, w)
    ws = torch.empty(max(16, nbytes), dtype=torch.uint8, device=DEV)
    dy32 = dy[0].float()
    cases.append(Case("rowwise", f"layernorm backward {rows}x{w}", G, rows * w * 10.0, sets,
                      lambda i: f.layernorm_backward(dx[i], dgain, dshift, dy[i], x[i], mean, rstd, gain,
                                                     rows, w, False, False, ws, nbytes),
                      lambda i: torch.ops.aten.native_layer_norm_backward(
                          dy32, x[i], [w], mean.view(rows, 1), rstd.view(rows, 1), gain, shift,
                          [True, True, True]),
                      "ATen native_layer_norm_backward (FP32 dy: 12 B per element)", rows=rows, cols=w))

    # Causal softmax forward / backward over [batches, T, T].
    batches = max(1, rows // LENGTH) * HEADS
    t = LENGTH
    matrix = batches * t * t
    visible = batches * t * (t + 1) // 2
    sets = rotation_sets(matrix * 4, once)
    s = [half(batches, t, t, gen=gen) for _ in range(sets)]
    p = [torch.empty(batches, t, t, dtype=torch.half, device=DEV) for _ in range(sets)]
    cases.append(Case("rowwise", f"causal softmax forward {batches}x{t}x{t}", G,
                      visible * 2.0 + matrix * 2.0, sets,
                      lambda i: f.causal_softmax_forward(p[i], s[i], batches, t),
                      lambda i: torch.softmax(s[i], -1),
                      "ATen softmax over full rows (no mask: reads all of s)", batches=batches, length=t))
    f.causal_softmax_forward(p[0], s[0], batches, t)
    dp = [half(batches, t, t, gen=gen) for _ in range(sets)]
    ds = [torch.empty(batches, t, t, dtype=torch.half, device=DEV) for _ in range(sets)]
    cases.append(Case("rowwise", f"causal softmax backward {batches}x{t}x{t}", G,
                      visible * 4.0 + matrix * 2.0, sets,
                      lambda i: f.causal_softmax_backward(ds[i], p[0], dp[i], batches, t, 0.125),
                      lambda i: torch.ops.aten._softmax_backward_data(dp[i], p[0], -1, torch.half),
                      "ATen _softmax_backward_data over full rows", batches=batches, length=t))

    # Fused softmax + cross-entropy.
    sets = rotation_sets(rows * PADDED_VOCAB * 4.0, once)
    logits = [half(rows, PADDED_VOCAB, scale=2.0, gen=gen) for _ in range(sets)]
    dlogits = [torch.empty(rows, PADDED_VOCAB, dtype=torch.half, device=DEV) for _ in range(sets)]
    targets = torch.randint(0, VOCAB, (rows,), device=DEV, generator=gen)
    targets16 = targets.to(torch.int16)
    loss = torch.empty(rows, device=DEV)
    cases.append(Case("rowwise", f"softmax cross-entropy {rows}x{PADDED_VOCAB}", G,
                      rows * VOCAB * 2.0 + rows * PADDED_VOCAB * 2.0 + rows * 6.0, sets,
                      lambda i: f.softmax_cross_entropy(dlogits[i], loss, logits[i], targets16,
                                                        65536.0 / rows, rows, VOCAB, PADDED_VOCAB),
                      rows=rows, cols=PADDED_VOCAB, vocab=VOCAB))

    # Embedding forward / backward.
    sequences = max(1, rows // LENGTH)
    wte = torch.randn(PADDED_VOCAB, w, device=DEV, generator=gen) * 0.02
    wpe = torch.randn(LENGTH, w, device=DEV, generator=gen) * 0.02
    tokens = torch.randint(0, VOCAB, (rows,), device=DEV, generator=gen)
    tokens16 = tokens.to(torch.int16)
    sets = rotation_sets(rows * w * 8.0, once)
    xe = [torch.empty(rows, w, device=DEV) for _ in range(sets)]
    positions = torch.arange(rows, device=DEV) % LENGTH
    cases.append(Case("rowwise", f"embedding forward {rows}x{w}", G,
                      rows * w * 8.0 + LENGTH * w * 4.0, sets,
                      lambda i: f.embedding_forward(xe[i], tokens16, wte, wpe, sequences, LENGTH,
                                                    PADDED_VOCAB, w),
                      lambda i: torch.embedding(wte, tokens).add_(torch.embedding(wpe, positions)),
                      "ATen embedding x 2 + add: three kernels", rows=rows, width=w))
    dxe = [torch.randn(rows, w, device=DEV, generator=gen) for _ in range(sets)]
    dwte = torch.zeros(PADDED_VOCAB, w, device=DEV)
    dwpe = torch.zeros(LENGTH, w, device=DEV)
    nbytes_e = f.embedding_backward_workspace(sequences, LENGTH, PADDED_VOCAB, w)
    wse = torch.empty(max(16, nbytes_e), dtype=torch.uint8, device=DEV)
    cases.append(Case("rowwise", f"embedding backward {rows}x{w} (write mode)", G,
                      rows * w * 4.0 + PADDED_VOCAB * w * 4.0 + LENGTH * w * 4.0, sets,
                      lambda i: f.embedding_backward(dwte, dwpe, dxe[i], tokens16, sequences, LENGTH,
                                                     PADDED_VOCAB, w, False, False, wse, nbytes_e),
                      lambda i: torch.ops.aten.embedding_dense_backward(dxe[i], tokens, PADDED_VOCAB, -1, False),
                      "ATen embedding_dense_backward (token table only, atomics)", rows=rows, width=w))

    # Bias gradient (column sums of FP16 rows).
    for cols in (w, 3 * w, 4 * w):
        sets = rotation_sets(rows * cols * 2.0, once)
        g = [half(rows, cols, gen=gen) for _ in range(sets)]
        db = torch.empty(cols, device=DEV)
        nb = f.bias_gradient_workspace(rows, cols)
        wsb = torch.empty(max(16, nb), dtype=torch.uint8, device=DEV)
        cases.append(Case("rowwise", f"bias gradient {rows}x{cols}", G, rows * cols * 2.0, sets,
                          lambda i, g=g, db=db, cols=cols, wsb=wsb, nb=nb:
                              f.bias_gradient(db, g[i], rows, cols, False, wsb, nb),
                          lambda i, g=g: torch.sum(g[i], 0, dtype=torch.float32),
                          "ATen sum over rows (FP32 accumulate)", rows=rows, cols=cols))

    # FP32 -> FP16 and copy.
    count = rows * w
    sets = rotation_sets(count * 6.0, once)
    src = [torch.randn(count, device=DEV, generator=gen) for _ in range(sets)]
    dst = [torch.empty(count, dtype=torch.half, device=DEV) for _ in range(sets)]
    cases.append(Case("rowwise", f"fp32 -> fp16 {count}", G, count * 6.0, sets,
                      lambda i: f.fp32_to_fp16(dst[i], src[i], count),
                      lambda i: dst[i].copy_(src[i]), "ATen copy_ (dtype cast)", count=count))
    for mib in (1, 16, 256):
        nbytes_c = mib << 20
        sets = rotation_sets(nbytes_c * 2.0, once)
        a = [torch.empty(nbytes_c, dtype=torch.uint8, device=DEV).random_(generator=gen) for _ in range(sets)]
        b = [torch.empty(nbytes_c, dtype=torch.uint8, device=DEV) for _ in range(sets)]
        cases.append(Case("rowwise", f"copy {mib} MiB", G, nbytes_c * 2.0, sets,
                          lambda i, a=a, b=b, n=nbytes_c: f.copy(b[i], a[i], n),
                          lambda i, a=a, b=b: b[i].copy_(a[i]), "cudaMemcpyAsync (torch copy_)",
                          bytes=nbytes_c))
    return cases


GROUPS = {"gemm": gemm_cases, "epilogue": epilogue_cases, "batched": batched_cases,
          "attention": attention_cases, "rowwise": rowwise_cases}


# ---- CPU timings of the same operations (the reference's PyTorch path on the host cores) ----------


def cpu_timings(rows: int, budget_s: float = 60.0):
    """torch FP32 CPU timings of the operations behind the kernels, at the same shapes, one to
    three calls each (a reported baseline, not a target)."""
    import os

    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()
    torch.set_num_threads(threads)
    w, w4 = WIDTH, 4 * WIDTH
    out = []
    begin = time.perf_counter()

    def timed(name, fn, work, unit):
        if time.perf_counter() - begin > budget_s:
            return
        fn()
        t0 = time.perf_counter()
        fn()
        seconds = time.perf_counter() - t0
        rate = work / seconds / (1e12 if unit == "TFLOP/s" else 1e9)
        out.append({"group": "cpu", "case": name, "us": round(seconds * 1e6, 1), "rate": round(rate, 4),
                    "unit": unit, "threads": threads})

    x = torch.randn(rows, w)
    for n, k in ((3 * w, w), (w, w), (w4, w), (w, w4)):
        a, b = torch.randn(rows, k), torch.randn(n, k)
        timed(f"matmul nt {rows}x{n}x{k} (FP32)", lambda a=a, b=b: a @ b.t(), flop(rows, n, k), "TFLOP/s")
    gain, shift = torch.ones(w), torch.zeros(w)
    timed(f"layer_norm {rows}x{w}", lambda: torch.nn.functional.layer_norm(x, (w,), gain, shift), rows * w * 8.0,
          "GB/s")
    s = torch.randn(HEADS, LENGTH, LENGTH)
    timed(f"softmax {HEADS}x{LENGTH}x{LENGTH}", lambda: torch.softmax(s, -1), HEADS * LENGTH * LENGTH * 8.0,
          "GB/s")
    logits = torch.randn(min(rows, 1024), VOCAB)
    targets = torch.randint(0, VOCAB, (logits.shape[0],))
    timed(f"cross_entropy {logits.shape[0]}x{VOCAB}",
          lambda: torch.nn.functional.cross_entropy(logits, targets), logits.numel() * 4.0, "GB/s")
    table = torch.randn(PADDED_VOCAB, w)
    ids = torch.randint(0, VOCAB, (rows,))
    timed(f"embedding {rows}x{w}", lambda: torch.embedding(table, ids), rows * w * 8.0, "GB/s")
    return out


def table(results) -> str:
    lines = ["| case | flint us | rate | of nominal | of measured | baseline us | flint / baseline | "
             "same-bytes copy us | SM MHz |",
             "| --- | ---: | ---: | ---: | ---: | ---: | ---: | ---: | ---: |"]
    for r in results:
        if r.get("group") == "cpu":
            lines.append(f"| CPU: {r['case']} | {r['us']} | {r['rate']} {r['unit']} | | | | | | |")
            continue
        fl, base, ratio = r["flint"], r["baseline"], r["flint_over_baseline"]
        lines.append(
            f"| {r['case']} | {fl['us']} | {fl['rate']} {r['unit']} | {fl['frac_nominal']:.3f} | "
            f"{fl['frac_measured']:.3f} | {base['us'] if base else '-'} | "
            f"{ratio['median'] if ratio else '-'} | {r.get('copy_same_bytes_us', '-')} | "
            f"{r['sm_mhz_median'] or '-'} |")
    return "\n".join(lines)


def run(flint: Flint, groups, rows: int, quick: bool, once: bool = False, sigma_x: float = 0.02,
        emit=None) -> list:
    """Runs the named groups; returns the list of result objects (and hands each to emit)."""
    torch.backends.cuda.matmul.allow_fp16_reduced_precision_reduction = False
    protocol = Protocol(quick)
    clocks = Clocks(torch.cuda.current_device())
    peaks = measured_peaks()
    copy_reference = None if once else CopyReference(flint, protocol)
    results = []
    for name in groups:
        builder = GROUPS[name]
        cases = builder(flint, rows, once, sigma_x) if name == "gemm" else builder(flint, rows, once)
        for case in cases:
            if once:
                case.flint(0)
                torch.cuda.synchronize()
                print(f"{case.name}: done", flush=True)
                continue
            result = run_case(case, protocol, clocks, peaks, copy_reference)
            results.append(result)
            if emit is not None:
                emit(result)
        del cases
        torch.cuda.empty_cache()
    if flint.kernel_fault():
        raise RuntimeError("a kernel gave up on a bounded wait")
    return results


def mma_rates(flint: Flint, count: int = 256) -> list:
    """Clocks per small tcgen05.mma (M 128, K 16) on an idle SM, by operand source and N: what
    bounds attention with head width 64, whose MMAs are all of these shapes."""
    results = []
    for n in (64, 128):
        for a_in_tmem in (0, 1):
            issue, complete = ctypes.c_longlong(), ctypes.c_longlong()
            for _ in range(3):
                flint.check(flint.lib.flint_b200_mma_clocks(n, a_in_tmem, count, ctypes.byref(issue),
                                                            ctypes.byref(complete), None))
            results.append({"group": "mma", "case": f"M 128, N {n}, K 16, A from "
                            f"{'tensor' if a_in_tmem else 'shared'} memory", "count": count,
                            "issue_clocks_each": round(issue.value / count, 1),
                            "complete_clocks_each": round(complete.value / count, 1),
                            "tensor_clocks_each": n // 2})
    return results


def mma_table(results) -> str:
    lines = ["| MMA | clocks until accepted, each | clocks until complete, each | tensor work, clocks |",
             "| --- | ---: | ---: | ---: |"]
    for r in results:
        lines.append(f"| {r['case']} | {r['issue_clocks_each']} | {r['complete_clocks_each']} | "
                     f"{r['tensor_clocks_each']} |")
    return "\n".join(lines)


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--group", default="all", choices=["all", "mma"] + list(GROUPS))
    parser.add_argument("--rows", type=int, default=8192, help="token rows (8 x 1024)")
    parser.add_argument("--quick", action="store_true", help="3 rounds of 25 ms samples instead of 10 x 100 ms")
    parser.add_argument("--once", action="store_true", help="one call per kernel, no timing")
    parser.add_argument("--reference-inputs", action="store_true",
                        help="GEMM activations N(0,1) as in the reference's own bench (default N(0,1) * 0.02)")
    parser.add_argument("--cpu", action="store_true", help="also time the torch CPU operations")
    parser.add_argument("--out", help="write the JSON lines and the table to this file too")
    args = parser.parse_args(argv)
    flint = Flint()
    if args.group == "mma":
        results = mma_rates(flint)
        text = "\n".join(json.dumps(r) for r in results) + "\n\n" + mma_table(results)
        print(text, flush=True)
        if args.out:
            Path(args.out).write_text(text + "\n")
        return
    groups = list(GROUPS) if args.group == "all" else [args.group]
    lines = []

    def emit(result):
        line = json.dumps(result)
        lines.append(line)
        print(line, flush=True)

    results = run(flint, groups, args.rows, args.quick, args.once,
                  1.0 if args.reference_inputs else 0.02, emit)
    if args.cpu and not args.once:
        for r in cpu_timings(args.rows):
            results.append(r)
            emit(r)
    if results:
        text = table(results)
        print(text, flush=True)
        if args.out:
            Path(args.out).write_text("\n".join(lines) + "\n\n" + text + "\n")


if __name__ == "__main__":
    main(sys.argv[1:])
