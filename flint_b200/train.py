"""Trains GPT-2 from Flint token files, one process per GPU.

    python -m flint_b200.train --tokens shard_001.bin shard_002.bin --steps 100 \\
        --checkpoint run.ckpt --every 50
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m flint_b200.train --tokens shard_*.bin --resume run.ckpt --steps 100

The reference's roadmap names this run (GPT-2 124M on FineWeb-Edu token shards,
``README.md:147``; shards as ``scripts/fineweb.py`` cuts them); its pieces here are
``TokenBatches`` (which rank reads which tokens), ``Trainer`` (the step) and the
checkpoint container. Each step's tokens and targets go through pinned host buffers to
the device on the compute stream; rank 0 prints one JSON line per logged step and writes
the checkpoints (every rank holds the same state).
"""

import argparse
import json
import os
import time

import numpy as np
import torch

from .binding import Flint
from .tokens import TokenBatches
from .trainer import Trainer, TrainerConfig


def parse(argv=None):
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("--tokens", nargs="+", required=True, help="token files, in training order")
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--sequences", type=int, default=16, help="sequences per GPU per step")
    p.add_argument("--length", type=int, default=1024)
    p.add_argument("--accumulate", type=int, default=1,
                   help="micro-batches per optimizer step (gradient accumulation)")
    p.add_argument("--layers", type=int, default=12)
    p.add_argument("--heads", type=int, default=12)
    p.add_argument("--width", type=int, default=768)
    p.add_argument("--block-size", type=int, default=1024)
    p.add_argument("--vocab", type=int, default=50257)
    p.add_argument("--padded-vocab", type=int, default=50304)
    p.add_argument("--lr", type=float, default=6e-4)
    p.add_argument("--loss-scale", type=float, default=65536.0)
    p.add_argument("--seed", type=int, default=1234)
    p.add_argument("--resume", help="checkpoint to continue from")
    p.add_argument("--checkpoint", help="where to write checkpoints")
    p.add_argument("--every", type=int, default=0, help="checkpoint every N steps (and at the end)")
    p.add_argument("--log-every", type=int, default=1)
    return p.parse_args(argv)


def main(argv=None) -> list:
    """Runs the job; returns the losses rank 0 logged (for tests)."""
    args = parse(argv)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    group = None
    if world > 1:
        import torch.distributed as dist

        if not dist.is_initialized():
            dist.init_process_group("gloo")  # carries the NCCL id only; see flint_train.h
        group = dist.group.WORLD

    config = TrainerConfig(layers=args.layers, heads=args.heads, width=args.width,
                           block_size=args.block_size, vocab=args.vocab,
                           padded_vocab=args.padded_vocab, sequences=args.sequences,
                           length=args.length, lr=args.lr, loss_scale=args.loss_scale)
    trainer = Trainer(Flint(), config, group=group, seed=args.seed)
    batches = TokenBatches(args.tokens, args.sequences, args.length, rank, world, vocab=args.vocab)
    if args.resume:
        saved = trainer.restore(args.resume)
        if saved is not None:
            batches.restore(saved)

    # One pinned host pair and one device pair per micro-batch of a step.
    shape = (args.sequences, args.length)
    micro = max(1, args.accumulate)
    host = [[torch.empty(shape, dtype=torch.int16).pin_memory() for _ in range(2)] for _ in range(micro)]
    views = [[h.numpy().view(np.uint16) for h in pair] for pair in host]
    device = [[torch.empty(shape, dtype=torch.int16, device="cuda") for _ in range(2)]
              for _ in range(micro)]
    losses = []
    tokens_per_step = args.sequences * args.length * world * micro

    def checkpoint():
        if args.checkpoint and rank == 0:
            trainer.save(args.checkpoint, data_state=batches.state())

    try:
        for index in range(args.steps):
            begin = time.perf_counter()
            for m in range(micro):
                batches.next_batch(views[m][0], views[m][1])
                device[m][0].copy_(host[m][0], non_blocking=True)
                device[m][1].copy_(host[m][1], non_blocking=True)
            trainer.step_batches([(pair[0].flatten(), pair[1].flatten()) for pair in device])
            loss = trainer.finish_step()  # waits for the step: the pinned buffers are free again
            seconds = time.perf_counter() - begin
            if rank == 0 and (index + 1) % max(1, args.log_every) == 0:
                losses.append(loss)
                print(json.dumps({"step": trainer.step_count, "loss": round(loss, 6),
                                  "loss_scale": trainer.scaler.scale, "skipped": trainer.skipped,
                                  "epoch": batches.epoch, "ms": round(seconds * 1e3, 3),
                                  "tokens_per_s": round(tokens_per_step / seconds, 1)}), flush=True)
            if args.every and (index + 1) % args.every == 0:
                checkpoint()
        checkpoint()
    finally:
        trainer.close()
    return losses


if __name__ == "__main__":
    main()
