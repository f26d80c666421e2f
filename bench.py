"""GPT-2 124M training throughput on N B200s of one node (tokens/s).

    python bench.py --gpus N --steps K --warmup W            (N = 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...                      (the CPU arm)

Workload: BASELINE's data-parallel training configuration: GPT-2 124M (12 layers, width 768,
12 heads, vocabulary 50257 padded to 50304, context 1024), a micro-batch of 16 x 1024 tokens
per GPU of seeded uniform token ids, forward + backward with fused attention, FP32 gradient
all-reduce over NCCL overlapped with backward, AdamW and dynamic loss scaling; FP16 operands
with FP32 accumulation. One step processes 16,384 tokens per GPU (weak scaling).

The JSON line's `value` is timed with the batches already in HBM; `e2e` is the same step
through Trainer.step()/finish_step() with the tokens copied from pinned host memory and the
loss read back every step. `roofline` describes the dominant kernel, the tensor-core GEMM:
all of one step's GEMM launches are replayed on the launch stream between CUDA events and
their algorithmic FLOPs (2 m n k each) divided by the measured time. `cpu_baseline` times
the CPU oracle (a port of the reference's PyTorch FP32 model) on the host cores.
"""

import argparse
import json
import os
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


# DRAM bytes (read + write) per GEMM call, averaged over the 147 calls of one step's replay
# below: `dram__bytes_read.sum + dram__bytes_write.sum` summed over the replay's kernels in the
# ncu capture summarised in profiles/gemm_step_replay_gpt2_124m.md.
GEMM_TRAFFIC_BYTES_PER_LAUNCH = 167.1e6


def gemm_roofline(flint, torch, rows: int, reps: int = 3):
    """Replays one step's GEMM launches, with the epilogues the model uses, between CUDA
    events on the launch stream."""
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
            "traffic": GEMM_TRAFFIC_BYTES_PER_LAUNCH}


def cpu_step_tokens_per_second(budget_seconds: float, threads=None):
    """The CPU oracle's training step (FP32 forward, backward and AdamW of GPT-2 124M) on
    1 x 1024 tokens per step, repeated while the budget lasts. Returns (tokens/s, cores, sample)."""
    import torch

    sys.path.insert(0, str(ROOT / "oracle"))
    import flint_oracle as oracle

    if threads:
        torch.set_num_threads(threads)
    cores = torch.get_num_threads()
    cfg = oracle.GPT2
    params = oracle.gpt2_init(cfg, seed=1234)
    moments = {k: (torch.zeros_like(v), torch.zeros_like(v)) for k, v in params.items()}
    sequences, length = 1, 1024
    idx, targets = oracle.synthetic_tokens(sequences, length, cfg["vocab_size"], seed=1)

    def one(step):
        _, grads = oracle.gpt2_loss_and_gradients(cfg, params, idx, targets)
        for name, p in params.items():
            wd = oracle.WEIGHT_DECAY if oracle.decayed(name, p.shape) else 0.0
            oracle.adamw_step(p, *moments[name], grads[name], step, weight_decay=wd)

    one(1)  # warm-up
    done, begin = 0, time.perf_counter()
    while done < 8 and (done == 0 or time.perf_counter() - begin < budget_seconds):
        one(done + 2)
        done += 1
    seconds = time.perf_counter() - begin
    sample = (f"{done} steps of {sequences}x{length} tokens (GPT-2 124M FP32 forward+backward+AdamW, "
              f"torch CPU, {cores} threads) after 1 warm-up")
    return sequences * length * done / seconds, cores, sample, seconds / done


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    value, cores, sample, step_seconds = cpu_step_tokens_per_second(
        budget_seconds=max(10.0, 4.0 * args.steps))
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 2), "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(step_seconds * 1e3, 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "note": "CPU oracle port of the reference's PyTorch "
                   "model; each step is a bounded sample of 1x1024 tokens"},
        "cpu_baseline": {"value": round(value, 2), "unit": "tokens/s", "cores": cores,
                         "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 2), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


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
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD

    flint = flint_b200.Flint()
    config = TrainerConfig(sequences=SEQUENCES, length=LENGTH,
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
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    # ---- device-resident inputs ------------------------------------------------------
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

    roofline = gemm_roofline(flint, torch, rows) if rank == 0 else None
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        value, cores, sample, _ = cpu_step_tokens_per_second(budget_seconds=15.0)
        cpu = {"value": round(value, 2), "unit": "tokens/s", "cores": cores, "kind": "port",
               "sample": sample}
    if rank == 0:
        peak, _, _ = peaks()
        line = {
            "metric": METRIC, "value": round(tokens_per_second, 1), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 3), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp16 (fp32 accumulate)",
            "data": "synthetic",
            "config": {"workload": WORKLOAD, "tokens_per_gpu_per_step": rows,
                       "parallelism": f"dp{world}",
                       "l2": "each step streams several GB of activations and weights, far "
                             "more than the 126 MB L2, so no flush is needed between steps",
                       "loss_scale": trainer.scaler.scale, "skipped_steps": trainer.skipped,
                       "last_loss": round(last_loss, 4),
                       "model_tflops": round(tokens_per_second * FLOPS_PER_TOKEN / 1e12, 1),
                       "mfu_of_sustained_peak": round(
                           tokens_per_second * FLOPS_PER_TOKEN / 1e12 / (peak * world), 4)},
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * rows,
                    "d2h_bytes_per_step": 4 * rows + 4},
            "gpu_launches": launches,
            "clocks": clocks.summary(),
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
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
