"""Host-side logic of the data-parallel trainer, on the CPU: the loss-scaling policy, the
initialisation, the bucket order, and (with two gloo ranks) that per-rank cross-entropy
scaling plus a plain sum all-reduce yields the gradient of the global mean loss."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import flint_oracle as oracle
from flint_b200 import trainer

SMALL = dict(n_layer=1, n_head=2, n_embd=32, block_size=16, vocab_size=50, padded_vocab_size=56)


def test_loss_scaler_follows_gradscaler_policy():
    scaler = trainer.LossScaler(65536.0, growth_interval=3)
    scaler.update(True)
    assert scaler.scale == 32768.0 and scaler.good_steps == 0
    for _ in range(2):
        scaler.update(False)
    assert scaler.scale == 32768.0
    scaler.update(False)
    assert scaler.scale == 65536.0 and scaler.good_steps == 0
    scaler.update(False)
    scaler.update(True)
    assert scaler.scale == 32768.0 and scaler.good_steps == 0


def test_initial_weights_are_the_oracle_initialisation():
    config = trainer.TrainerConfig(layers=2, heads=2, width=64, block_size=32, vocab=200,
                                   padded_vocab=208)
    cfg = dict(n_layer=2, n_head=2, n_embd=64, block_size=32, vocab_size=200,
               padded_vocab_size=208)
    mine = trainer.initial_weights(config, seed=1234)
    want = oracle.gpt2_init(cfg, seed=1234)
    assert list(mine) == list(want)
    for name in want:
        assert torch.equal(mine[name], want[name]), name


def test_bucket_order_and_scale():
    assert trainer.bucket_order(3) == ["ln_f", "blocks.2", "blocks.1", "blocks.0", "embeddings"]
    assert trainer.cross_entropy_scale(65536.0, 16384, 8) == 65536.0 / (16384 * 8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        params = oracle.gpt2_init(SMALL, seed=1)
        sequences, length = 2, 16
        idx, targets = oracle.synthetic_tokens(sequences * world, length, SMALL["vocab_size"], 9)
        mine = slice(rank * sequences, (rank + 1) * sequences)
        loss_scale = 1024.0
        rows = sequences * length
        scale = trainer.cross_entropy_scale(loss_scale, rows, world)
        # The fused cross-entropy's gradient is that of scale * sum(row_loss) = scale * rows * mean.
        _, grads = oracle.gpt2_loss_and_gradients(SMALL, params, idx[mine], targets[mine])
        flat = torch.cat([g.flatten() for g in grads.values()]) * (scale * rows)
        dist.all_reduce(flat, op=dist.ReduceOp.SUM)
        _, full = oracle.gpt2_loss_and_gradients(SMALL, params, idx, targets)
        want = torch.cat([g.flatten() for g in full.values()]) * loss_scale
        results[rank] = bool(torch.allclose(flat, want, rtol=1e-4, atol=1e-6))
    finally:
        dist.destroy_process_group()


@pytest.mark.timeout(120)
def test_two_ranks_sum_to_the_global_mean_gradient():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank_main, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_bench_watchdog_ends_a_phase_that_never_finishes():
    """bench.py's watchdog: a phase past its limit ends the process with status 3 and a
    message naming the phase; a phase that was closed in time does not."""
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    late = subprocess.run(
        [sys.executable, "-c",
         "import bench, time; w = bench.Watchdog(); w.phase('stuck collective', 0.5); time.sleep(10)"],
        cwd=root, capture_output=True, text=True, timeout=60)
    assert late.returncode == 3
    assert "stuck collective" in late.stderr
    fine = subprocess.run(
        [sys.executable, "-c",
         "import bench, time; w = bench.Watchdog(); w.phase('quick', 0.5); w.done(); "
         "time.sleep(2.5); print('finished')"],
        cwd=root, capture_output=True, text=True, timeout=60)
    assert fine.returncode == 0 and "finished" in fine.stdout
