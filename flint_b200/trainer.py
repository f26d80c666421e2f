"""Data-parallel GPT-2 training step over the C ABI (one process per GPU).

The reference has no trainer in C++ (its README lists the optimizer, loss
scaling and multi-GPU as planned); what a step must do is fixed by its PyTorch
oracle, ``scripts/gpt2_torch.py:161-192``: forward and backward in FP16 with
FP32 accumulation and a dynamic loss scale, AdamW (lr 6e-4, betas 0.9/0.95,
eps 1e-8, weight decay 0.1 on parameters with two or more dimensions), and a
step that is skipped, with the scale halved, when a gradient is not finite.

Here every kernel is the library's: ``flint_gpt2_forward`` /
``flint_b200_gpt2_backward_buckets`` on a model built on the fused attention
kernels, ``flint_b200_check_gradients`` and one multi-tensor
``flint_b200_adamw_run`` that also refreshes the FP16 weight copies. With more
than one rank the FP32 gradients are summed by NCCL all-reduce over
NVLink/NVSwitch, one contiguous bucket per transformer block, started from the
backward pass's bucket callback on a second stream so the transfers overlap the
remaining backward kernels. Each rank scales its loss by
``loss_scale / (rows_per_rank * world)``, so the plain sum is the gradient of
the global mean loss and every rank takes the same skip decision.
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
    overlap_update: bool = True  # ranks > 1: update most of the model under the last all-reduce


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


class Trainer:
    """One rank of a data-parallel GPT-2 training job. `group` is a torch.distributed
    process group (NCCL) or None for a single GPU."""

    def __init__(self, flint: Flint, config: TrainerConfig, state: dict = None, group=None,
                 seed: int = 1234):
        self.flint = flint
        self.config = config
        self.group = group
        self.world = 1
        if group is not None:
            import torch.distributed as dist

            self.world = dist.get_world_size(group)
        model_config = Gpt2Config(config.layers, config.heads, config.width, config.block_size,
                                  config.vocab, config.padded_vocab, config.sequences,
                                  config.length, 0, 1)
        self.model = Gpt2(flint, model_config, flash_attention=config.flash_attention)
        self.rows = config.sequences * config.length
        self.stream = torch.cuda.current_stream()
        self.comm_stream = torch.cuda.Stream() if self.world > 1 else None

        state = state if state is not None else initial_weights(config, seed)
        self.model.load({k: v.cuda() for k, v in state.items()})

        self.parameters = self.model.parameters()
        gradients = self.model.gradients()
        arena, arena_bytes = self.model.gradient_arena()
        self.gradient_address = arena
        self.gradient_count = arena_bytes // 4
        self.gradients = device_tensor(arena, self.gradient_count)
        # Moments share the gradient arena's layout: one allocation each.
        self.m = torch.zeros(self.gradient_count, device="cuda")
        self.v = torch.zeros(self.gradient_count, device="cuda")
        half = self._half_copies()
        tensors = []
        # (name, master address, rows, cols, first float in the gradient/moment arenas)
        self.layout = [(name, address, rows, cols, (grad - arena) // 4)
                       for (name, address, rows, cols), (_, grad, _, _) in zip(self.parameters, gradients)]
        for (name, address, rows, cols), (_, grad, _, _) in zip(self.parameters, gradients):
            offset = grad - arena
            decay = config.weight_decay if rows > 1 else 0.0
            tensors.append((address, self.m.data_ptr() + offset, self.v.data_ptr() + offset, grad,
                            half.get(name), rows * cols, decay))
        self.plan, self.plan_items = flint.adamw_plan(tensors)
        # With more than one rank the update is pipelined with the last all-reduce (see
        # step()): one plan for the embeddings (the last bucket, the first two tensors of
        # the arena) and one for everything else.
        self.body_offset = (gradients[2][1] - arena) // 4  # first float after wte and wpe
        self.split_plans = None
        if self.world > 1:
            self.split_plans = (flint.adamw_plan(tensors[:2]), flint.adamw_plan(tensors[2:]))
        self.found = torch.zeros(1, dtype=torch.int32, device="cuda")
        self.norm_squared = torch.zeros(1, dtype=torch.float64, device="cuda")
        self._row_loss = device_tensor(self.model.outputs()[2], self.rows)
        self._loss_sum = torch.zeros((), dtype=torch.float64, device="cuda")
        self._micro_batches = 1
        self.scaler = LossScaler(config.loss_scale, config.growth_interval)
        self.step_count = 0
        self.skipped = 0
        self._events = []
        torch.cuda.synchronize()

    def _half_copies(self) -> dict:
        """{parameter name: address of its FP16 compute copy}. The copies follow the
        gradients in the model's arena in a fixed order: wte, then each block's four
        matrices; their addresses come from the model's layout."""
        import ctypes

        out = {}
        lib = self.flint.lib
        if hasattr(lib, "flint_b200_gpt2_compute_copy"):
            for index, (name, _, _, _) in enumerate(self.parameters):
                address = ctypes.c_void_p()
                self.flint.check(lib.flint_b200_gpt2_compute_copy(self.model.handle, index,
                                                                  ctypes.byref(address)))
                if address.value:
                    out[name] = address.value
        return out

    def close(self) -> None:
        self.model.close()

    # -- one optimizer step ---------------------------------------------------------------

    def _pipelined(self) -> bool:
        """Whether the update overlaps the last all-reduce: more than one rank, and no
        gradient clipping (the clip coefficient needs the norm of all reduced gradients)."""
        return self.world > 1 and self.config.overlap_update and self.config.max_grad_norm <= 0

    def _on_bucket(self, bucket: int, address: int, nbytes: int) -> None:
        import torch.distributed as dist

        last = bucket == self.config.layers + 1  # ln_f, the blocks, then the embeddings
        view = device_tensor(address, nbytes // 4)
        if last and self._pipelined():
            # This rank's embedding gradients are checked before they are summed: a
            # non-finite value on any rank makes the sum non-finite, so the maximum of the
            # ranks' flags (a four-byte all-reduce, ahead of the big one) is the flag the
            # summed gradients would raise.
            self.flint.check_gradients(view, nbytes // 4, 1.0 / self.scaler.scale, self.found,
                                       None)
        ready = torch.cuda.Event()
        ready.record(self.stream)
        self.comm_stream.wait_event(ready)
        with torch.cuda.stream(self.comm_stream):
            if last and self._pipelined():
                dist.all_reduce(self.found, op=dist.ReduceOp.MAX, group=self.group)
                self._flag_ready = torch.cuda.Event()
                self._flag_ready.record(self.comm_stream)
            dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group)

    def step(self, tokens: torch.Tensor, targets: torch.Tensor) -> None:
        """Enqueues forward, backward (with overlapped all-reduce), the gradient check and
        the AdamW update for one micro-batch of uint16 tokens/targets on this rank."""
        self.step_batches([(tokens, targets)])

    def step_batches(self, batches) -> None:
        """One optimizer step over several micro-batches, a list of (tokens, targets), as the
        reference's ``train_step`` takes them (``scripts/gpt2_torch.py:178-192``): each
        micro-batch's loss is divided by their number and the gradients accumulate in place
        (``flint_gpt2_backward`` with accumulate set from the second one on). With more
        than one rank only the last micro-batch's backward starts the all-reduces, on the
        accumulated gradients."""
        c = self.config
        count = len(batches)
        if count == 0:
            raise ValueError("a step needs at least one micro-batch")
        scale = cross_entropy_scale(self.scaler.scale, self.rows, self.world) / count
        inverse = 1.0 / self.scaler.scale
        pipelined = self._pipelined()
        self._micro_batches = count
        if count > 1:
            self._loss_sum.zero_()
        if pipelined:
            self.found.zero_()
        for index, (tokens, targets) in enumerate(batches):
            self.model.forward(tokens, targets, scale)
            if count > 1:
                self._loss_sum += self._row_loss.sum(dtype=torch.float64)
            reduce_now = self.world > 1 and index + 1 == count
            self.model.backward(tokens, index > 0,
                                callback=self._on_bucket if reduce_now else None)
        if pipelined:
            # Every bucket but the last is summed while backward runs; the last one (the
            # embeddings, a third of the bytes) would otherwise be waited for with nothing
            # to do. Its non-finite flag is settled early (see _on_bucket), so the rest of
            # the model is checked and updated while that all-reduce is in flight.
            done = torch.cuda.Event()
            done.record(self.comm_stream)
            self.stream.wait_event(self._flag_ready)
            body = self.gradients[self.body_offset:]
            self.flint.check_gradients(body, body.numel(), inverse, self.found, None)
            self.step_count += 1
            (embed_plan, embed_items), (body_plan, body_items) = self.split_plans
            step = self.step_count - self.skipped
            self.flint.adamw_run(body_plan, body_items, c.lr, c.beta1, c.beta2, c.eps, inverse, step,
                                 self.found)
            self.stream.wait_event(done)
            self.flint.adamw_run(embed_plan, embed_items, c.lr, c.beta1, c.beta2, c.eps, inverse,
                                 step, self.found)
            return
        if self.world > 1:
            done = torch.cuda.Event()
            done.record(self.comm_stream)
            self.stream.wait_event(done)
        self.apply_update()

    def apply_update(self) -> None:
        """The optimizer's half of a step on whatever the gradient arena holds (gradients
        times the loss scale, already summed over the ranks): the non-finite check, the
        optional clip of the unscaled gradients' global norm
        (``scripts/gpt2_torch.py:186-188``: ``unscale_`` then ``clip_grad_norm_``) and one
        AdamW launch that also writes the FP16 compute copies. A non-finite gradient leaves
        weights and moments untouched (the kernels read the flag on the device)."""
        c = self.config
        inverse = 1.0 / self.scaler.scale
        self.found.zero_()
        clip = c.max_grad_norm > 0
        if clip:
            self.norm_squared.zero_()
        self.flint.check_gradients(self.gradients, self.gradient_count, inverse, self.found,
                                   self.norm_squared if clip else None)
        grad_scale = inverse
        if clip:
            # The clip coefficient needs the norm on the host; clipping is off by default.
            norm = math.sqrt(self.norm_squared.item())
            if math.isfinite(norm) and norm > c.max_grad_norm:
                grad_scale *= c.max_grad_norm / (norm + 1e-6)
        self.step_count += 1
        self.flint.adamw_run(self.plan, self.plan_items, c.lr, c.beta1, c.beta2, c.eps, grad_scale,
                             self.step_count - self.skipped, self.found)

    def finish_step(self) -> float:
        """Waits for the step, updates the loss scale from the non-finite flag and returns
        this rank's mean loss over the step's micro-batches (a device-to-host read)."""
        if self._micro_batches > 1:
            loss = self._loss_sum.item() / (self.rows * self._micro_batches)
        else:
            loss = self.model.mean_loss()
        found = bool(self.found.item())
        if found:
            self.skipped += 1
        self.scaler.update(found)
        return loss

    # -- checkpoints ----------------------------------------------------------------------

    MODEL_KEYS = ("layers", "heads", "width", "block_size", "vocab", "padded_vocab")

    def save(self, path, data_state: dict = None) -> str:
        """Writes the FP32 master weights (under PyTorch's parameter names), both AdamW
        moments, the loss scaler and the step counters to path, with data_state (for
        instance TokenBatches.state()) alongside. Every rank holds the same state, so one
        rank writing is enough. Returns the file's sha256."""
        torch.cuda.synchronize()
        arrays = {}
        for name, address, rows, cols, first in self.layout:
            count = rows * cols
            shape = (cols,) if rows == 1 else (rows, cols)
            arrays["param/" + name] = device_tensor(address, count).cpu().numpy().reshape(shape)
            arrays["m/" + name] = self.m[first:first + count].cpu().numpy().reshape(shape)
            arrays["v/" + name] = self.v[first:first + count].cpu().numpy().reshape(shape)
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
        """Loads a checkpoint written by save() into this trainer (same model shape) and
        returns the data_state stored with it. The FP16 compute copies are refreshed from
        the restored masters."""
        meta, arrays = read_checkpoint(path, verify=verify)
        if meta.get("kind") != "flint-b200 trainer":
            raise CheckpointError("not a trainer checkpoint")
        mine = asdict(self.config)
        for key in self.MODEL_KEYS:
            if meta["config"].get(key) != mine[key]:
                raise CheckpointError(
                    f"checkpoint's {key} is {meta['config'].get(key)}, this trainer's {mine[key]}")
        state = {}
        for name, _, rows, cols, first in self.layout:
            count = rows * cols
            for prefix in ("param/", "m/", "v/"):
                if prefix + name not in arrays or arrays[prefix + name].size != count:
                    raise CheckpointError(f"checkpoint lacks {prefix}{name} with {count} values")
            state[name] = torch.from_numpy(np.array(arrays["param/" + name], dtype=np.float32)).cuda()
            self.m[first:first + count].copy_(
                torch.from_numpy(np.array(arrays["m/" + name], dtype=np.float32).reshape(-1)))
            self.v[first:first + count].copy_(
                torch.from_numpy(np.array(arrays["v/" + name], dtype=np.float32).reshape(-1)))
        self.model.load(state)
        self.step_count = int(meta["step_count"])
        self.skipped = int(meta["skipped"])
        self.scaler.scale = float(meta["loss_scale"])
        self.scaler.good_steps = int(meta["good_steps"])
        torch.cuda.synchronize()
        return meta.get("data")
