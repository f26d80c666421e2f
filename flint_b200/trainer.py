"""Data-parallel GPT-2 training from Python: a thin caller of libflint_train.so.

The reference has no trainer in C++ (its README lists the optimizer, loss
scaling and multi-GPU as planned); what a step must do is fixed by its PyTorch
oracle, ``scripts/gpt2_torch.py:161-192``: forward and backward in FP16 with
FP32 accumulation and a dynamic loss scale, AdamW (lr 6e-4, betas 0.9/0.95,
eps 1e-8, weight decay 0.1 on parameters with two or more dimensions), and a
step that is skipped, with the scale halved, when a gradient is not finite.

The step itself lives in C++ behind ``include/flint/flint_train.h``
(``flint_b200/csrc/train.cpp``): streams, events, the per-bucket NCCL collectives
(all-reduce, or reduce-scatter + all-gather around a sharded AdamW), the loss-scale
policy and the optimizer launches. This module holds what is left for the host
language: the configuration, the initial weights, checkpoints, and zero-copy torch
views of the trainer's device arrays for tests and tools. torch supplies device
buffers, the current stream and (with any backend) the process group that carries
rank 0's NCCL id to the other ranks; it runs no kernel of the step.
"""

import math
from dataclasses import asdict, dataclass

import numpy as np
import torch

from .binding import Flint, Gpt2, Gpt2Config
from .checkpoint import CheckpointError, read_checkpoint, write_checkpoint


@dataclass
class TrainerConfig:
    layers: int = 12
    heads: int = 12
    width: int = 768
    block_size: int = 1024
    vocab: int = 50257
    padded_vocab: int = 50304
    sequences: int = 16          # per rank
    length: int = 1024
    lr: float = 6e-4
    beta1: float = 0.9
    beta2: float = 0.95
    eps: float = 1e-8
    weight_decay: float = 0.1
    loss_scale: float = 65536.0  # GradScaler's initial scale
    growth_interval: int = 2000
    max_grad_norm: float = 0.0   # 0 disables clipping
    flash_attention: bool = True
    overlap_update: bool = True  # replicated ranks > 1: update most of the model under the last all-reduce
    shard_optimizer: bool = False  # ranks > 1: reduce-scatter, per-rank AdamW on 1/world, all-gather


class _DeviceView:
    """Zero-copy torch view of raw device memory (the CUDA array interface)."""

    def __init__(self, address: int, count: int, typestr: str = "<f4"):
        self.__cuda_array_interface__ = {
            "shape": (count,), "typestr": typestr, "data": (address, False), "version": 2,
        }


def device_tensor(address: int, count: int, typestr: str = "<f4") -> torch.Tensor:
    return torch.as_tensor(_DeviceView(address, count, typestr), device="cuda")


def initial_weights(config: TrainerConfig, seed: int = 1234) -> dict:
    """GPT-2's initialisation from a CPU generator, in named_parameters order: N(0, 0.02)
    for the embeddings and linear weights, the residual projections scaled by
    1/sqrt(2 layers), zero biases, LayerNorm gain 1, padded wte rows zero."""
    gen = torch.Generator("cpu").manual_seed(seed)
    w = config.width
    std = 0.02
    residual = std / math.sqrt(2 * config.layers)
    state = {}

    def normal(name, shape, sigma):
        state[name] = torch.empty(shape).normal_(0.0, sigma, generator=gen)

    normal("wte.weight", (config.padded_vocab, w), std)
    normal("wpe.weight", (config.block_size, w), std)
    for i in range(config.layers):
        p = f"blocks.{i}."
        state[p + "ln_1.weight"] = torch.ones(w)
        state[p + "ln_1.bias"] = torch.zeros(w)
        normal(p + "attn.c_attn.weight", (3 * w, w), std)
        state[p + "attn.c_attn.bias"] = torch.zeros(3 * w)
        normal(p + "attn.c_proj.weight", (w, w), residual)
        state[p + "attn.c_proj.bias"] = torch.zeros(w)
        state[p + "ln_2.weight"] = torch.ones(w)
        state[p + "ln_2.bias"] = torch.zeros(w)
        normal(p + "mlp.c_fc.weight", (4 * w, w), std)
        state[p + "mlp.c_fc.bias"] = torch.zeros(4 * w)
        normal(p + "mlp.c_proj.weight", (w, 4 * w), residual)
        state[p + "mlp.c_proj.bias"] = torch.zeros(w)
    state["ln_f.weight"] = torch.ones(w)
    state["ln_f.bias"] = torch.zeros(w)
    state["wte.weight"][config.vocab:].zero_()
    return state


class LossScaler:
    """torch.cuda.amp.GradScaler's policy on the host: halve on a non-finite step,
    double after growth_interval consecutive good steps."""

    def __init__(self, scale: float, growth_interval: int):
        self.scale = float(scale)
        self.growth_interval = growth_interval
        self.good_steps = 0

    def update(self, found_nonfinite: bool) -> None:
        if found_nonfinite:
            self.scale *= 0.5
            self.good_steps = 0
            return
        self.good_steps += 1
        if self.good_steps >= self.growth_interval:
            self.scale *= 2.0
            self.good_steps = 0


def cross_entropy_scale(loss_scale: float, rows_per_rank: int, world: int) -> float:
    """The scale each rank hands to the fused cross-entropy so that the plain sum of the
    ranks' gradients is loss_scale times the gradient of the global mean loss."""
    return loss_scale / (rows_per_rank * world)


def bucket_order(layers: int) -> list:
    """Names of the gradient buckets in the order the backward pass completes them."""
    return ["ln_f"] + [f"blocks.{i}" for i in reversed(range(layers))] + ["embeddings"]


class _Scaler:
    """The trainer's dynamic loss scale as the C library holds it (GradScaler's policy)."""

    def __init__(self, trainer):
        self._trainer = trainer

    @property
    def scale(self) -> float:
        return self._trainer.status().loss_scale

    @scale.setter
    def scale(self, value: float) -> None:
        self._trainer.set_status(loss_scale=float(value))

    @property
    def good_steps(self) -> int:
        return self._trainer.status().good_steps

    @good_steps.setter
    def good_steps(self, value: int) -> None:
        self._trainer.set_status(good_steps=int(value))


class Trainer:
    """One rank of a data-parallel GPT-2 training job: a thin caller of libflint_train.so
    (``include/flint/flint_train.h``), which owns the model, the optimizer state, the
    collective stream and, for more than one rank, the NCCL communicator. `group` is a
    torch.distributed process group of any backend, or None for a single GPU; it is used
    for one thing only, handing rank 0's NCCL id to the other ranks."""

    def __init__(self, flint: Flint, config: TrainerConfig, state: dict = None, group=None,
                 seed: int = 1234):
        import ctypes

        from .binding import BUCKET_HOOK, TrainerConfigC

        self.flint = flint
        self.config = config
        self.group = group
        self.world, self.rank = 1, 0
        if group is not None:
            import torch.distributed as dist

            self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.lib = flint.train
        self.stream = torch.cuda.current_stream()
        self.rows = config.sequences * config.length

        nccl_id = None
        if self.world > 1:
            import torch.distributed as dist

            holder = [None]
            if self.rank == 0:
                buffer = ctypes.create_string_buffer(128)
                flint.check_train(self.lib.flint_train_nccl_id(buffer))
                holder[0] = buffer.raw
            dist.broadcast_object_list(holder, src=dist.get_global_rank(group, 0), group=group)
            nccl_id = ctypes.create_string_buffer(holder[0], 128)
        c = TrainerConfigC()
        c.model = Gpt2Config(config.layers, config.heads, config.width, config.block_size,
                             config.vocab, config.padded_vocab, config.sequences, config.length, 0, 1)
        c.flash_attention = int(config.flash_attention)
        c.lr, c.beta1, c.beta2, c.eps = config.lr, config.beta1, config.beta2, config.eps
        c.weight_decay = config.weight_decay
        c.loss_scale, c.growth_interval = config.loss_scale, config.growth_interval
        c.max_grad_norm = config.max_grad_norm
        c.world, c.rank = self.world, self.rank
        c.shard_optimizer = int(config.shard_optimizer)
        c.overlap_update = int(config.overlap_update)
        handle = ctypes.c_void_p()
        flint.check_train(self.lib.flint_trainer_create(ctypes.byref(c), nccl_id, ctypes.byref(handle)))
        self.handle = handle.value
        model = ctypes.c_void_p()
        flint.check_train(self.lib.flint_trainer_model(self.handle, ctypes.byref(model)))
        self.model = Gpt2(flint, c.model, borrowed=model.value)

        state = state if state is not None else initial_weights(config, seed)
        self.model.load({k: v.cuda() for k, v in state.items()})

        self.parameters = self.model.parameters()
        gradients = self.model.gradients()
        arena, arena_bytes = self.model.gradient_arena()
        self.gradient_address = arena
        self.gradient_count = arena_bytes // 4
        self.gradients = device_tensor(arena, self.gradient_count)
        # (name, master address, rows, cols, first float in the gradient arena)
        self.layout = [(name, address, rows, cols, (grad - arena) // 4)
                       for (name, address, rows, cols), (_, grad, _, _) in zip(self.parameters, gradients)]
        m, v, count = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_size_t()
        flint.check_train(self.lib.flint_trainer_moments(self.handle, ctypes.byref(m), ctypes.byref(v),
                                                         ctypes.byref(count)))
        # AdamW's moments. A replicated trainer's arrays share the gradient arena's layout; a
        # sharded one's hold this rank's ranges back to back (see ranges()).
        self.m = device_tensor(m.value, count.value)
        self.v = device_tensor(v.value, count.value)
        found, norm = ctypes.c_void_p(), ctypes.c_void_p()
        flint.check_train(self.lib.flint_trainer_flags(self.handle, ctypes.byref(found), ctypes.byref(norm)))
        self.found = device_tensor(found.value, 1, "<i4")
        self.norm_squared = device_tensor(norm.value, 1, "<f8")
        self.scaler = _Scaler(self)
        self._hook = None
        self._hook_type = BUCKET_HOOK
        torch.cuda.synchronize()

    def close(self) -> None:
        if self.handle is not None:
            self.lib.flint_trainer_destroy(self.handle)
            self.handle = None
            self.model.handle = None

    # -- state ----------------------------------------------------------------------------

    def status(self):
        from .binding import TrainerStatus
        import ctypes

        status = TrainerStatus()
        self.flint.check_train(self.lib.flint_trainer_get_status(self.handle, ctypes.byref(status)))
        return status

    def set_status(self, **changes) -> None:
        import ctypes

        status = self.status()
        for key, value in changes.items():
            setattr(status, key, value)
        self.flint.check_train(self.lib.flint_trainer_set_status(self.handle, ctypes.byref(status)))

    @property
    def step_count(self) -> int:
        return self.status().step_count

    @property
    def skipped(self) -> int:
        return self.status().skipped

    def ranges(self) -> list:
        """(first, count, storage, shared) of each range of the gradient arena this rank's
        optimizer owns: the moments of arena floats [first, first + count) are
        m[storage:storage + count]; shared ranges are held by every rank alike."""
        from .binding import TrainerRange
        import ctypes

        out = []
        for i in range(self.lib.flint_trainer_shard_count(self.handle)):
            r = TrainerRange()
            self.flint.check_train(self.lib.flint_trainer_shard(self.handle, i, ctypes.byref(r)))
            out.append((r.first, r.count, r.storage, bool(r.shared)))
        return out

    def synchronize(self) -> None:
        """Waits for the step and for the collective stream (a sharded trainer's weights may
        still be arriving when finish_step returns)."""
        self.flint.check_train(self.lib.flint_trainer_synchronize(self.handle, self.stream.cuda_stream))

    def set_bucket_hook(self, hook) -> None:
        """hook(bucket, address, nbytes), or None: called on the launching thread for each
        gradient bucket of a step's last micro-batch before its collective is enqueued (ranks
        > 1); it may enqueue work on the current stream."""
        if hook is None:
            self._hook = None
            self.flint.check_train(self.lib.flint_trainer_set_bucket_hook(self.handle, self._hook_type(0), None))
            return
        self._hook = self._hook_type(lambda _user, bucket, address, nbytes, _stream: hook(bucket, address, nbytes))
        self.flint.check_train(self.lib.flint_trainer_set_bucket_hook(self.handle, self._hook, None))

    # -- one optimizer step ---------------------------------------------------------------

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        """Enqueues forward, backward (with overlapped collectives), the gradient check and
        the AdamW update for one micro-batch of uint16 tokens/targets on this rank."""
        self.step_batches([(tokens, targets)])

    def step_batches(self, batches) -> None:
        """One optimizer step over several micro-batches, a list of (tokens, targets), as the
        reference's ``train_step`` takes them (``scripts/gpt2_torch.py:178-192``): each
        micro-batch's loss is divided by their number and the gradients accumulate in place.
        With more than one rank only the last micro-batch's backward starts the collectives,
        on the accumulated gradients."""
        import ctypes

        count = len(batches)
        if count == 0:
            raise ValueError("a step needs at least one micro-batch")
        tokens = (ctypes.c_void_p * count)(*[t.data_ptr() for t, _ in batches])
        targets = (ctypes.c_void_p * count)(*[y.data_ptr() for _, y in batches])
        self.flint.check_train(self.lib.flint_trainer_step(self.handle, tokens, targets, count,
                                                           self.stream.cuda_stream))

    def apply_update(self) -> None:
        """The optimizer's half of a step on whatever the gradient arena holds (gradients
        times the loss scale): the non-finite check, the optional clip of the unscaled
        gradients' global norm (``scripts/gpt2_torch.py:186-188``) and one AdamW launch that
        also writes the FP16 compute copies. Single rank only."""
        self.flint.check_train(self.lib.flint_trainer_update(self.handle, self.stream.cuda_stream))

    def finish_step(self) -> float:
        """Waits for the step, updates the loss scale from the non-finite flag and returns
        this rank's mean loss over the step's micro-batches (a device-to-host read)."""
        import ctypes

        loss, skipped = ctypes.c_double(), ctypes.c_int()
        self.flint.check_train(self.lib.flint_trainer_finish(
            self.handle, self.stream.cuda_stream, ctypes.cast(ctypes.byref(loss), ctypes.c_void_p),
            ctypes.cast(ctypes.byref(skipped), ctypes.c_void_p)))
        return loss.value

    # -- checkpoints ----------------------------------------------------------------------

    MODEL_KEYS = ("layers", "heads", "width", "block_size", "vocab", "padded_vocab")

    def _arena_moments(self):
        """(m, v) as CPU tensors in the gradient arena's layout. A sharded trainer's ranks
        each hold a slice of every bucket: the slices are put in place and summed over the
        ranks (disjoint, so the sum is the union; ranges every rank holds come from rank 0)."""
        ranges = self.ranges()
        if self.world == 1 or all(shared for _, _, _, shared in ranges):
            full_m, full_v = torch.zeros(self.gradient_count), torch.zeros(self.gradient_count)
            m, v = self.m.cpu(), self.v.cpu()
            for first, count, storage, _ in ranges:
                full_m[first:first + count] = m[storage:storage + count]
                full_v[first:first + count] = v[storage:storage + count]
            return full_m, full_v
        import torch.distributed as dist

        out = []
        for moment in (self.m.cpu(), self.v.cpu()):
            full = torch.zeros(self.gradient_count)
            for first, count, storage, shared in ranges:
                if not shared or self.rank == 0:
                    full[first:first + count] = moment[storage:storage + count]
            device = full.cuda() if dist.get_backend(self.group) == "nccl" else full
            dist.all_reduce(device, group=self.group)
            out.append(device.cpu())
        return out

    def save(self, path, data_state: dict = None) -> str:
        """Writes the FP32 master weights (under PyTorch's parameter names), both AdamW
        moments, the loss scaler and the step counters to path, with data_state (for
        instance TokenBatches.state()) alongside. The file does not depend on how the
        optimizer state was spread over ranks: a sharded trainer gathers its moments first
        (a collective: every rank must call save; rank 0's file is complete). Returns the
        file's sha256."""
        self.synchronize()
        m_full, v_full = self._arena_moments()
        arrays = {}
        for name, address, rows, cols, first in self.layout:
            count = rows * cols
            shape = (cols,) if rows == 1 else (rows, cols)
            arrays["param/" + name] = device_tensor(address, count).cpu().numpy().reshape(shape)
            arrays["m/" + name] = m_full[first:first + count].numpy().reshape(shape)
            arrays["v/" + name] = v_full[first:first + count].numpy().reshape(shape)
        meta = {
            "kind": "flint-b200 trainer",
            "config": asdict(self.config),
            "step_count": self.step_count,
            "skipped": self.skipped,
            "loss_scale": self.scaler.scale,
            "good_steps": self.scaler.good_steps,
            "data": data_state,
        }
        return write_checkpoint(path, meta, arrays)

    def restore(self, path, verify: bool = True):
        """Loads a checkpoint written by save() into this trainer (same model shape, any
        number of ranks) and returns the data_state stored with it. Each rank takes the
        moments of the ranges it owns; the FP16 compute copies are refreshed from the
        restored masters."""
        meta, arrays = read_checkpoint(path, verify=verify)
        if meta.get("kind") != "flint-b200 trainer":
            raise CheckpointError("not a trainer checkpoint")
        mine = asdict(self.config)
        for key in self.MODEL_KEYS:
            if meta["config"].get(key) != mine[key]:
                raise CheckpointError(
                    f"checkpoint's {key} is {meta['config'].get(key)}, this trainer's {mine[key]}")
        state = {}
        m_full = torch.zeros(self.gradient_count)
        v_full = torch.zeros(self.gradient_count)
        for name, _, rows, cols, first in self.layout:
            count = rows * cols
            for prefix in ("param/", "m/", "v/"):
                if prefix + name not in arrays or arrays[prefix + name].size != count:
                    raise CheckpointError(f"checkpoint lacks {prefix}{name} with {count} values")
            state[name] = torch.from_numpy(np.array(arrays["param/" + name], dtype=np.float32)).cuda()
            m_full[first:first + count] = torch.from_numpy(
                np.array(arrays["m/" + name], dtype=np.float32).reshape(-1))
            v_full[first:first + count] = torch.from_numpy(
                np.array(arrays["v/" + name], dtype=np.float32).reshape(-1))
        for first, count, storage, _ in self.ranges():
            self.m[storage:storage + count].copy_(m_full[first:first + count])
            self.v[storage:storage + count].copy_(v_full[first:first + count])
        self.model.load(state)
        self.set_status(step_count=int(meta["step_count"]), skipped=int(meta["skipped"]),
                        loss_scale=float(meta["loss_scale"]), good_steps=int(meta["good_steps"]))
        torch.cuda.synchronize()
        return meta.get("data")
