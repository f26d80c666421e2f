"""GPT-2 124M training throughput on N B200s of one node (tokens/s).

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...                      (the CPU arm)

Workload: the data-parallel training configuration: GPT-2 124M (12 layers, width 768,
12 heads, vocabulary 50257 padded to 50304, context 1024), a micro-batch of 16 x 1024 tokens
per GPU of seeded uniform token ids, forward + backward with fused attention, FP32 gradient
all-reduce over NCCL overlapped with backward, AdamW and dynamic loss scaling; FP16 operands
with FP32 accumulation. One step processes 16,384 tokens per GPU (weak scaling).

The JSON line's `value` is timed with the batches already in HBM; `e2e` is the same step
through Trainer.step()/finish_step() with the tokens copied from pinned host memory and the
loss read back every step. `roofline` describes the dominant kernel, the tensor-core GEMM:
all of one step's GEMM launches are replayed on the launch stream between CUDA events and
their algorithmic FLOPs (2 m n k each) divided by the measured time; `roofline.per_kernel`
(one GPU only) is the per-kernel sweep of flint_b200.kernel_bench in its short form: every
GEMM shape, fused epilogue, attention and row-wise kernel beside its cuBLAS / cuBLASLt / ATen
counterpart, with fractions of the nominal and measured peaks. `cpu_baseline` and
`--impl reference` time the CPU oracle (a port of the reference's PyTorch FP32 model) on all
the host cores, each step a bounded sample of 1 x 1024 tokens of the same workload.
"""

import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "GPT-2 124M train tokens/s"
SEQUENCES, LENGTH = 16, 1024
WORKLOAD = ("GPT-2 124M data-parallel training step: 16x1024 tokens per GPU, forward + backward "
            "(fused attention) + FP32 gradient all-reduce + AdamW + dynamic loss scaling")
FLOPS_PER_TOKEN = 855_383_040  # 6 N + 12 L d T with N = 123,689,472 (wpe excluded)


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return data.get("bf16_tflops_sustained", 1418.9), data.get("hbm_gbs", 6538.6), "measured"
    return 1400.0, 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                fields = [f.strip() for f in out.stdout.strip().split(",")]
                if len(fields) >= 6:
                    self.samples.append(float(fields[0]))
                    self.max_mhz = float(fields[1])
                    for name, value in zip(names, fields[2:6]):
                        if value.lower().startswith("active"):
                            self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *_):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons)}


def step_gemms(rows: int):
    """(entry point, m, n, k) of every GEMM launch of one training step, in the model's order
    (flint_b200/csrc/gpt2.cu, forward_block / backward_block and the head)."""
    w, v, layers = 768, 50304, 12
    forward = [("nt_bias", rows, 3 * w, w), ("nt_bias_residual", rows, w, w),
               ("nt_bias_gelu", rows, 4 * w, w), ("nt_bias_residual", rows, w, 4 * w)]
    backward = [("tn", w, 4 * w, rows), ("nn_dgelu", rows, 4 * w, w), ("tn", 4 * w, w, rows),
                ("nn", rows, w, 4 * w), ("tn", w, w, rows), ("nn", rows, w, w),
                ("tn", 3 * w, w, rows), ("nn", rows, w, 3 * w)]
    return layers * (forward + backward) + [("nt", rows, v, w), ("tn", v, w, rows),
                                            ("nn", rows, w, v)]


def gemm_traffic():
    """(DRAM bytes read + written per GEMM call, commit it was captured on) from the committed
    ncu summary of the replay below, or (None, None). The summary carries one line of the form
    `roofline.traffic: <bytes> bytes per GEMM call, captured on commit <sha>`."""
    path = ROOT / "profiles" / "gemm_step_replay_gpt2_124m.md"
    if path.is_file():
        found = re.search(r"roofline\.traffic:\s*([0-9.eE+]+) bytes per GEMM call, captured on commit (\w+)",
                          path.read_text())
        if found:
            return float(found.group(1)), found.group(2)
    return None, None


def gemm_roofline(flint, torch, rows: int, reps: int = 3):
    """Replays one step's GEMM launches, with the epilogues the model uses, between CUDA
    events on the launch stream. The buffers are fixed, so consecutive calls find the 25 MB
    activations and the weights of the call before in the 126 MB L2, as they do inside the
    real step: the per-shape numbers with operands rotated past the L2 are in `per_kernel`."""
    dev = "cuda"
    shapes = step_gemms(rows)
    a = torch.randn(rows * 50304, device=dev).half()      # big enough for every operand
    b = (torch.randn(50304 * 768, device=dev) * 0.02).half()
    y = torch.empty(rows * 50304, device=dev, dtype=torch.float16)
    pre = torch.randn(rows * 3072, device=dev).half()
    residual = torch.randn(rows * 768, device=dev)
    y32 = torch.zeros(50304 * 768, device=dev)
    bias = torch.randn(3072, device=dev)
    workspace = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def replay():
        for kind, m, n, k in shapes:
            if kind == "nt":
                flint.gemm_nt(y, a, b, m, n, k)
            elif kind == "nt_bias":
                flint.gemm_nt_bias(y, a, b, bias, m, n, k)
            elif kind == "nt_bias_gelu":
                flint.gemm_nt_bias_gelu(y, pre, a, b, bias, m, n, k)
            elif kind == "nt_bias_residual":
                flint.gemm_nt_bias_residual(y32, a, b, bias, residual, m, n, k)
            elif kind == "nn":
                flint.gemm_nn(y, a, b, m, n, k)
            elif kind == "nn_dgelu":
                flint.gemm_nn_dgelu(y, a, b, pre, m, n, k)
            else:
                flint.gemm_tn(y32, a, b, m, n, k, True, workspace)

    replay()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        replay()
    stop.record()
    torch.cuda.synchronize()
    seconds = start.elapsed_time(stop) / 1e3 / reps
    flops = sum(2.0 * m * n * k for _, m, n, k in shapes)
    peak, _, source = peaks()
    achieved = flops / seconds / 1e12
    return {"bound": "tensor",
            "kernel": "fb_gemm_pair / fb_gemm_tc / fb_gemm_tn_reduce (all 147 GEMM calls of one "
                      "step, with their epilogues)",
            "achieved": round(achieved, 1), "peak": peak, "unit": "TFLOP/s",
            "frac": round(achieved / peak, 4), "peak_source": source + " (sustained bf16 GEMM)",
            "launches_per_step": len(shapes), "avg_launch_us": round(seconds / len(shapes) * 1e6, 2),
            "operands": "fixed buffers (L2-warm between consecutive calls, as in the step)",
            "traffic": gemm_traffic()[0], "traffic_captured_on": gemm_traffic()[1]}


def host_cores() -> int:
    """Cores this process may run on (the launcher's OMP_NUM_THREADS=1 does not count)."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class CpuStep:
    """The CPU oracle's training step (FP32 forward, backward and AdamW of GPT-2 124M) on a
    bounded sample of the workload: 1 x 1024 tokens per step, on every host core."""

    SEQUENCES, LENGTH = 1, 1024

    def __init__(self):
        import torch

        sys.path.insert(0, str(ROOT / "oracle"))
        import flint_oracle as oracle

        # torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the baseline is
        # the reference's PyTorch path on all the cores the process may use.
        self.cores = host_cores()
        torch.set_num_threads(self.cores)
        self.oracle = oracle
        self.params = oracle.gpt2_init(oracle.GPT2, seed=1234)
        self.moments = {k: (torch.zeros_like(v), torch.zeros_like(v)) for k, v in self.params.items()}
        self.batch = oracle.synthetic_tokens(self.SEQUENCES, self.LENGTH, oracle.GPT2["vocab_size"], seed=1)
        self.step = 0

    def run(self, steps: int) -> float:
        """Runs `steps` optimizer steps; returns the seconds they took."""
        begin = time.perf_counter()
        for _ in range(steps):
            self.step += 1
            self.oracle.train_step(self.oracle.GPT2, self.params, self.moments, [self.batch], self.step,
                                   max_grad_norm=0.0)
        return time.perf_counter() - begin

    def sample(self, warmup: int, steps: int) -> str:
        return (f"{steps} steps of {self.SEQUENCES}x{self.LENGTH} tokens each (GPT-2 124M FP32 forward + "
                f"backward + AdamW, torch CPU, {self.cores} threads) after {warmup} warm-up steps; the "
                f"GPU arm's step is 16x1024 tokens per GPU")


def static_config(world: int) -> dict:
    """What both arms measure; identical in the two JSON lines."""
    return {"workload": WORKLOAD, "tokens_per_gpu_per_step": SEQUENCES * LENGTH,
            "parallelism": f"dp{world}",
            "l2": "each step streams several GB of activations and weights, far more than the "
                  "126 MB L2, so no flush is needed between steps"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = CpuStep()
    cpu.run(args.warmup)
    seconds = cpu.run(args.steps)
    tokens = CpuStep.SEQUENCES * CpuStep.LENGTH * args.steps
    value = tokens / seconds
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(seconds / args.steps * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": static_config(args.gpus),
        "cpu_baseline": {"value": round(value, 2), "unit": "tokens/s", "cores": cpu.cores,
                         "kind": "port", "sample": cpu.sample(args.warmup, args.steps)},
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def per_kernel_summary(flint):
    """The per-kernel sweep in its short form (3 rounds of 25 ms samples per arm), condensed
    to one small object per case."""
    from flint_b200 import kernel_bench

    results = kernel_bench.run(flint, list(kernel_bench.GROUPS), 8192, quick=True)
    out = []
    for r in results:
        base, ratio = r["baseline"], r["flint_over_baseline"]
        out.append({"case": r["case"], "us": r["flint"]["us"], "rate": r["flint"]["rate"],
                    "unit": r["unit"], "frac_nominal": r["flint"]["frac_nominal"],
                    "frac_measured": r["flint"]["frac_measured"],
                    "baseline_us": base["us"] if base else None,
                    "flint_over_baseline": ratio["median"] if ratio else None,
                    "copy_same_bytes_us": r.get("copy_same_bytes_us"),
                    "timing": r.get("timing"),
                    "sm_mhz": r["sm_mhz_median"]})
    return {"protocol": "operands rotated past 4x L2, 3 interleaved rounds of 25 ms samples per arm "
                        "(python -m flint_b200.kernel_bench runs 10 rounds of 100 ms); baseline = "
                        "cuBLAS / cuBLASLt / ATen through torch",
            "nominal_peaks": {"TFLOP/s": kernel_bench.NOMINAL_TFLOPS, "GB/s": kernel_bench.NOMINAL_GBS},
            "measured_peaks": dict(zip(("TFLOP/s", "GB/s"), kernel_bench.measured_peaks()[:2])),
            "cases": out}


class Watchdog:
    """Ends the process when a phase of the bench takes far longer than it can (a collective that
    never completes, say): a bench that hangs costs its caller the whole time limit and every
    other rank with it. `phase` names what is running and how long it may take."""

    def __init__(self):
        import threading

        self.deadline, self.name = None, ""
        self.lock = threading.Lock()
        threading.Thread(target=self._watch, daemon=True).start()

    def phase(self, name: str, seconds: float) -> None:
        with self.lock:
            self.name, self.deadline = name, time.monotonic() + seconds

    def done(self) -> None:
        with self.lock:
            self.deadline = None

    def _watch(self) -> None:
        while True:
            time.sleep(1.0)
            with self.lock:
                late = self.deadline is not None and time.monotonic() > self.deadline
                name = self.name
            if late:
                print(f"bench.py: '{name}' exceeded its time limit; giving up", file=sys.stderr,
                      flush=True)
                os._exit(3)


def run_flint(args):
    import numpy as np
    import torch
    import torch.distributed as dist

    import flint_b200
    from flint_b200.trainer import Trainer, TrainerConfig

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    watchdog = Watchdog()
    watchdog.phase("process group, model and NCCL communicator set-up", 240)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # The process group only carries rank 0's NCCL id, barriers and the max over ranks
        # (host-side, gloo); the gradient collectives are the training library's own NCCL calls.
        dist.init_process_group("gloo")
        group = dist.group.WORLD

    flint = flint_b200.Flint()
    # Four or more ranks: the optimizer state is sharded (reduce-scatter, AdamW on 1/world,
    # all-gather under the next forward pass); two ranks keep replicas, which measured 0.8%
    # faster there. FLINT_B200_SHARD=0/1 overrides.
    shard = os.environ.get("FLINT_B200_SHARD", "1" if world >= 4 else "0") != "0"
    config = TrainerConfig(sequences=SEQUENCES, length=LENGTH, shard_optimizer=shard,
                           overlap_update=os.environ.get("FLINT_B200_OVERLAP_UPDATE", "1") != "0")
    trainer = Trainer(flint, config, group=group, seed=1234)
    rows = SEQUENCES * LENGTH

    # Seeded uniform ids, a different stream per rank; targets are the ids shifted by one.
    pool = 4
    gen = torch.Generator().manual_seed(1000 + rank)
    host_batches = []
    for _ in range(pool):
        ids = torch.randint(0, config.vocab, (rows + 1,), generator=gen)
        tokens = torch.from_numpy(ids[:-1].numpy().astype(np.uint16).view(np.int16)).pin_memory()
        targets = torch.from_numpy(ids[1:].numpy().astype(np.uint16).view(np.int16)).pin_memory()
        host_batches.append((tokens, targets))
    device_batches = [(t.cuda(), y.cuda()) for t, y in host_batches]
    staging = (torch.empty(rows, dtype=torch.int16, device="cuda"),
               torch.empty(rows, dtype=torch.int16, device="cuda"))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- device-resident inputs ------------------------------------------------------
    watchdog.phase("warm-up and timed steps", 120 + 2.0 * (args.warmup + 2 * args.steps))
    for i in range(args.warmup):
        trainer.step(*device_batches[i % pool])
        trainer.finish_step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = flint.launch_count()
    with ClockSampler(local) as clocks:
        start.record()
        for i in range(args.steps):
            trainer.step(*device_batches[i % pool])
            trainer.finish_step()
        stop.record()
        barrier()
    launches = flint.launch_count() - launches_before
    ms = max_over_ranks(start.elapsed_time(stop))
    tokens_per_second = world * rows * args.steps / (ms / 1e3)
    last_loss = trainer.model.mean_loss()

    # ---- end to end: pinned host tokens in, loss out, every step -----------------------
    barrier()
    start.record()
    for i in range(args.steps):
        tokens, targets = host_batches[i % pool]
        staging[0].copy_(tokens, non_blocking=True)
        staging[1].copy_(targets, non_blocking=True)
        trainer.step(*staging)
        trainer.finish_step()
    stop.record()
    barrier()
    e2e_ms = max_over_ranks(start.elapsed_time(stop))
    e2e = world * rows * args.steps / (e2e_ms / 1e3)

    if flint.kernel_fault():
        raise RuntimeError("a tensor-core kernel gave up on a barrier wait during the bench")

    # The rest runs on rank 0 alone and on the host's clock: no limit that a slow box could hit.
    watchdog.done()
    roofline = gemm_roofline(flint, torch, rows) if rank == 0 else None
    run_facts = {"loss_scale": trainer.scaler.scale, "skipped_steps": trainer.skipped,
                 "last_loss": round(last_loss, 4)}
    trainer.close()
    trainer = None
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_per_kernel:
        roofline["per_kernel"] = per_kernel_summary(flint)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        step = CpuStep()
        step.run(2)
        steps = 12
        seconds = step.run(steps)
        value = CpuStep.SEQUENCES * CpuStep.LENGTH * steps / seconds
        cpu = {"value": round(value, 2), "unit": "tokens/s", "cores": step.cores, "kind": "port",
               "sample": step.sample(2, steps)}
    if rank == 0:
        peak, _, _ = peaks()
        run_facts["model_tflops"] = round(tokens_per_second * FLOPS_PER_TOKEN / 1e12, 1)
        run_facts["mfu_of_sustained_peak"] = round(
            tokens_per_second * FLOPS_PER_TOKEN / 1e12 / (peak * world), 4)
        line = {
            "metric": METRIC, "value": round(tokens_per_second, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
            "data": "synthetic",
            "config": static_config(world),
            "run": run_facts,
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * rows,
                    "d2h_bytes_per_step": 4 * rows + 4},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if trainer is not None:
        trainer.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=20)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", default="flint", choices=["flint", "reference"])
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-per-kernel", action="store_true",
                        help="skip the per-kernel sweep beside cuBLAS (roofline.per_kernel)")
    parser.add_argument("--gemm-replay", action="store_true",
                        help="only replay one step's GEMM calls once after a warm-up replay and "
                             "print the roofline object (the command profiled for its DRAM traffic)")
    args = parser.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.gemm_replay:
        import torch

        import flint_b200
        torch.cuda.set_device(0)
        print(json.dumps(gemm_roofline(flint_b200.Flint(), torch, SEQUENCES * LENGTH, reps=1)),
              flush=True)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_flint(args)


if __name__ == "__main__":
    main()
