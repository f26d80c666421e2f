"""One rank of the data-parallel trainer checks (launched by test_trainer_multi_gpu.py).

Run under torch.distributed.run with one process per GPU over NCCL. Every rank runs the
same sequence of small training jobs and asserts on its own results; a failed assertion
ends the process with a non-zero status, which fails the launching test.

  1. the update pipelined under the last all-reduce (overlap_update), the plain order and
     the sharded optimizer (reduce-scatter, AdamW on 1/world of every bucket, all-gather)
     give the same weights and AdamW moments (bit for bit on two ranks), and all ranks hold
     the same bits;
  2. the job over `world` ranks matches one rank stepping on the concatenated batch: the
     same mean loss, the same update direction;
  3. a non-finite value in ONE rank's embedding gradient (written by a plain fill from the
     host between the backward pass and the all-reduce) makes EVERY rank skip that step,
     halve its loss scale and leave weights and moments untouched, in all three modes;
  4. a checkpoint saved by a sharded trainer and restored into a fresh one continues bit for
     bit.
"""

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "oracle"))

import flint_b200  # noqa: E402
import flint_oracle as oracle  # noqa: E402
from flint_b200.trainer import Trainer, TrainerConfig, device_tensor  # noqa: E402

MODES = {"pipelined": dict(overlap_update=True), "plain": dict(overlap_update=False),
         "sharded": dict(shard_optimizer=True)}
SMALL = dict(n_layer=2, n_head=2, n_embd=128, block_size=64, vocab_size=200, padded_vocab_size=208)
PER_RANK, LENGTH, STEPS = 2, 64, 3


def u16(t):
    return torch.from_numpy(t.numpy().astype(np.uint16).view(np.int16)).cuda()


def config(sequences, **extra):
    return TrainerConfig(layers=2, heads=2, width=128, block_size=64, vocab=200, padded_vocab=208,
                         sequences=sequences, length=LENGTH, loss_scale=1024.0, **extra)


def state_of(trainer):
    torch.cuda.synchronize()
    weights = torch.cat([device_tensor(a, r * c).clone() for _, a, r, c in trainer.model.parameters()])
    return weights.cpu(), trainer.m.cpu().clone(), trainer.v.cpu().clone()


def poison(trainer, steps, rank=1):
    """Writes +inf into this rank's first embedding gradient right before the last bucket's
    collective of the steps listed (1-based), on `rank` only: a plain fill enqueued on the
    step's stream from the trainer's bucket hook."""

    def hook(bucket, address, nbytes):
        last = bucket == trainer.config.layers + 1
        if last and dist.get_rank() == rank and (trainer.step_count + 1) in steps:
            device_tensor(address, 1).fill_(float("inf"))

    trainer.set_bucket_hook(hook)


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    group = dist.group.WORLD
    flint = flint_b200.Flint()
    params = oracle.gpt2_round_to_half(oracle.gpt2_init(SMALL, seed=1234))
    batches = [oracle.synthetic_tokens(world * PER_RANK, LENGTH, SMALL["vocab_size"], seed=40 + s)
               for s in range(STEPS)]
    mine = slice(rank * PER_RANK, (rank + 1) * PER_RANK)

    def train(trainer, whole_batch=False):
        losses = []
        for idx, targets in batches:
            if not whole_batch:
                idx, targets = idx[mine], targets[mine]
            trainer.step(u16(idx.flatten()), u16(targets.flatten()))
            losses.append(trainer.finish_step())
        return losses

    # 1. the three ways to run the update agree, on and across ranks: replicated with the
    # update pipelined under the last all-reduce, replicated in plain order, and sharded.
    results = {}
    for name, mode in MODES.items():
        trainer = Trainer(flint, config(PER_RANK, **mode), state=params, group=group)
        try:
            losses = train(trainer)
            assert trainer.skipped == 0 and trainer.step_count == STEPS
            trainer.synchronize()
            ranges = trainer.ranges()
            if name == "sharded":
                assert len(ranges) == SMALL["n_layer"] + 2 and not any(r[3] for r in ranges)
                assert trainer.m.numel() == sum(r[1] for r in ranges)
                assert sum(r[1] for r in ranges) * world <= trainer.gradient_count
            else:
                assert ranges == [(0, trainer.gradient_count, 0, True)]
            weights = torch.cat([device_tensor(a, r * c).clone() for _, a, r, c in trainer.model.parameters()]).cpu()
            m, v = trainer._arena_moments()
            results[name] = (losses, weights, m.clone(), v.clone())
        finally:
            trainer.close()
    for a, b in zip(results["pipelined"][1:], results["plain"][1:]):
        assert torch.equal(a, b), "pipelined and plain updates differ"
    assert results["pipelined"][0] == results["plain"][0]
    assert results["sharded"][0] == results["plain"][0]
    for a, b in zip(results["sharded"][1:], results["plain"][1:]):
        # Two ranks: a + b in either order is the same FP32 sum, so even the bits agree.
        if world == 2:
            assert torch.equal(a, b), "sharded and replicated updates differ"
        else:
            assert torch.allclose(a, b, rtol=1e-4, atol=1e-7)
    for name in MODES:
        for tensor in results[name][1:]:
            reference = tensor.cuda()
            dist.broadcast(reference, 0)
            assert torch.equal(reference.cpu(), tensor), f"{name}: ranks hold different bits"

    # 2. against one rank on the concatenated batch.
    single = Trainer(flint, config(world * PER_RANK), state=params)
    try:
        single_losses = train(single, whole_batch=True)
        single_weights, _, _ = state_of(single)
    finally:
        single.close()
    mean_losses = torch.tensor(results["plain"][0], dtype=torch.float64, device="cuda")
    dist.all_reduce(mean_losses)
    mean_losses = (mean_losses / world).cpu().tolist()
    assert max(abs(a - b) for a, b in zip(mean_losses, single_losses)) <= 1e-5, (mean_losses, single_losses)
    start = torch.cat([params[name].flatten() for name, _ in oracle.gpt2_parameter_shapes(SMALL)])
    moved, expected = results["sharded"][1] - start, single_weights - start
    cosine = torch.nn.functional.cosine_similarity(moved.double(), expected.double(), dim=0).item()
    assert cosine >= 0.999, cosine

    # 3. a non-finite gradient on one rank: every rank skips, halves the scale, changes nothing.
    for name, mode in MODES.items():
        trainer = Trainer(flint, config(PER_RANK, **mode), state=params, group=group)
        poison(trainer, (2,))
        try:
            idx, targets = batches[0]
            trainer.step(u16(idx[mine].flatten()), u16(targets[mine].flatten()))
            trainer.finish_step()
            before = state_of(trainer)
            assert trainer.skipped == 0 and trainer.scaler.scale == 1024.0
            idx, targets = batches[1]
            trainer.step(u16(idx[mine].flatten()), u16(targets[mine].flatten()))
            trainer.finish_step()
            assert trainer.skipped == 1 and trainer.scaler.scale == 512.0, (rank, name, trainer.skipped)
            after = state_of(trainer)
            for a, b in zip(before, after):
                assert torch.equal(a, b), "a skipped step changed the state"
            idx, targets = batches[2]
            trainer.step(u16(idx[mine].flatten()), u16(targets[mine].flatten()))
            loss = trainer.finish_step()
            assert trainer.skipped == 1 and np.isfinite(loss)
            assert not torch.equal(state_of(trainer)[0], after[0])
        finally:
            trainer.close()

    # 4. a checkpoint written by a sharded trainer (its moments gathered over the ranks)
    # restored into a fresh sharded trainer: the next step repeats the uninterrupted run's.
    import tempfile

    first = Trainer(flint, config(PER_RANK, shard_optimizer=True), state=params, group=group)
    second = Trainer(flint, config(PER_RANK, shard_optimizer=True),
                     state={k: torch.zeros_like(v) for k, v in params.items()}, group=group)
    try:
        for idx, targets in batches[:2]:
            first.step(u16(idx[mine].flatten()), u16(targets[mine].flatten()))
            first.finish_step()
        with tempfile.TemporaryDirectory() as folder:
            path = os.path.join(folder, f"sharded.rank{rank}.ckpt")
            first.save(path)
            second.restore(path)
        assert second.step_count == 2 and second.scaler.scale == first.scaler.scale
        idx, targets = batches[2]
        losses = []
        for trainer in (first, second):
            trainer.step(u16(idx[mine].flatten()), u16(targets[mine].flatten()))
            losses.append(trainer.finish_step())
        assert losses[0] == losses[1]
        for a, b in zip(state_of(first), state_of(second)):
            assert torch.equal(a, b), "the restored trainer's step differs"
    finally:
        first.close()
        second.close()

    assert not flint.kernel_fault()
    dist.barrier()
    if rank == 0:
        print(f"trainer ranks ok: world {world}, cosine against one rank {cosine:.6f}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
