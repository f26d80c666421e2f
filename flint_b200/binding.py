"""ctypes binding of libflint.so, generated from the C headers.

The reference's tests reach the library through ``tests/flint_lib.py``: a
``Flint`` object whose methods take torch tensors (or raw addresses, or None)
for pointers and a torch stream (or handle, or None) for the stream, and raise
``FlintError`` with ``flint_last_error()`` on a non-zero status. This module
offers the same names and behaviour, but derives every ctypes signature by
parsing ``include/flint/flint.h`` and ``include/flint/flint_b200.h`` instead of
listing them by hand, so a declaration and its binding cannot drift apart.

The library is the CUDA product: there is no fallback. Loading fails loudly
when ``libflint.so`` has not been built.
"""

import ctypes
import os
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "flint" / "flint.h"
EXTENSION_HEADER = ROOT / "include" / "flint" / "flint_b200.h"
TRAIN_HEADER = ROOT / "include" / "flint" / "flint_train.h"
LIBRARY_NAME = "libflint.so"
TRAIN_LIBRARY_NAME = "libflint_train.so"

OK = 0
ERROR_INVALID_ARGUMENT = 1
ERROR_CUDA = 2


class Gpt2Config(ctypes.Structure):
    """flint_gpt2_config."""

    _fields_ = [
        ("layers", ctypes.c_size_t),
        ("heads", ctypes.c_size_t),
        ("width", ctypes.c_size_t),
        ("block_size", ctypes.c_size_t),
        ("vocab", ctypes.c_size_t),
        ("padded_vocab", ctypes.c_size_t),
        ("sequences", ctypes.c_size_t),
        ("length", ctypes.c_size_t),
        ("separate_buffers", ctypes.c_int),
        ("backward", ctypes.c_int),
    ]


class Gpt2ParameterInfo(ctypes.Structure):
    """flint_gpt2_parameter_info."""

    _fields_ = [
        ("name", ctypes.c_char_p),
        ("data", ctypes.c_void_p),
        ("rows", ctypes.c_size_t),
        ("cols", ctypes.c_size_t),
    ]


class AdamwTensor(ctypes.Structure):
    """flint_b200_adamw_tensor."""

    _fields_ = [
        ("param", ctypes.c_void_p),
        ("m", ctypes.c_void_p),
        ("v", ctypes.c_void_p),
        ("grad", ctypes.c_void_p),
        ("half_copy", ctypes.c_void_p),
        ("count", ctypes.c_size_t),
        ("weight_decay", ctypes.c_float),
    ]


class TrainerConfigC(ctypes.Structure):
    """flint_trainer_config."""

    _fields_ = [
        ("model", Gpt2Config),
        ("flash_attention", ctypes.c_int),
        ("lr", ctypes.c_float),
        ("beta1", ctypes.c_float),
        ("beta2", ctypes.c_float),
        ("eps", ctypes.c_float),
        ("weight_decay", ctypes.c_float),
        ("loss_scale", ctypes.c_float),
        ("growth_interval", ctypes.c_int),
        ("max_grad_norm", ctypes.c_float),
        ("world", ctypes.c_int),
        ("rank", ctypes.c_int),
        ("shard_optimizer", ctypes.c_int),
        ("overlap_update", ctypes.c_int),
    ]


class TrainerStatus(ctypes.Structure):
    """flint_trainer_status."""

    _fields_ = [
        ("loss_scale", ctypes.c_float),
        ("good_steps", ctypes.c_int),
        ("step_count", ctypes.c_longlong),
        ("skipped", ctypes.c_longlong),
        ("grad_norm", ctypes.c_double),
    ]


class TrainerRange(ctypes.Structure):
    """flint_trainer_range."""

    _fields_ = [("first", ctypes.c_size_t), ("count", ctypes.c_size_t), ("storage", ctypes.c_size_t),
                ("shared", ctypes.c_int)]


BUCKET_HOOK = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_size_t,
                               ctypes.c_void_p)
BUCKET_CALLBACK = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                   ctypes.c_size_t)
STAGE_CALLBACK = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_int)

_C_TYPES = {
    "void": None,
    "int": ctypes.c_int,
    "flint_status": ctypes.c_int,
    "float": ctypes.c_float,
    "size_t": ctypes.c_size_t,
    "const char*": ctypes.c_char_p,
    "void*": ctypes.c_void_p,
    "const void*": ctypes.c_void_p,
    "flint_stream": ctypes.c_void_p,
    "flint_gpt2*": ctypes.c_void_p,
    "const flint_gpt2*": ctypes.c_void_p,
    "int*": ctypes.c_void_p,
    "const int*": ctypes.c_void_p,
    "double*": ctypes.c_void_p,
    "unsigned long long*": ctypes.POINTER(ctypes.c_ulonglong),
    "long long*": ctypes.POINTER(ctypes.c_longlong),
    "size_t*": ctypes.POINTER(ctypes.c_size_t),
    "void**": ctypes.POINTER(ctypes.c_void_p),
    "const void**": ctypes.POINTER(ctypes.c_void_p),
    "flint_gpt2**": ctypes.POINTER(ctypes.c_void_p),
    "const flint_gpt2_config*": ctypes.POINTER(Gpt2Config),
    "flint_gpt2_parameter_info*": ctypes.POINTER(Gpt2ParameterInfo),
    "flint_b200_bucket_callback": BUCKET_CALLBACK,
    "flint_b200_stage_callback": STAGE_CALLBACK,
    "const flint_b200_adamw_tensor*": ctypes.POINTER(AdamwTensor),
    "float*": ctypes.POINTER(ctypes.c_float),
    "int**": ctypes.POINTER(ctypes.c_void_p),
    "double**": ctypes.POINTER(ctypes.c_void_p),
    "const void* const*": ctypes.POINTER(ctypes.c_void_p),
    "flint_b200_generator*": ctypes.c_void_p,
    "const flint_b200_generator*": ctypes.c_void_p,
    "flint_b200_generator**": ctypes.POINTER(ctypes.c_void_p),
    "flint_trainer*": ctypes.c_void_p,
    "const flint_trainer*": ctypes.c_void_p,
    "flint_trainer**": ctypes.POINTER(ctypes.c_void_p),
    "const flint_trainer_config*": ctypes.POINTER(TrainerConfigC),
    "flint_trainer_status*": ctypes.POINTER(TrainerStatus),
    "const flint_trainer_status*": ctypes.POINTER(TrainerStatus),
    "flint_trainer_range*": ctypes.POINTER(TrainerRange),
    "flint_trainer_bucket_hook": BUCKET_HOOK,
}

_DECLARATION = re.compile(r"FLINT_API\s+([^;(]*?)\b(flint_\w+)\s*\(([^;]*?)\)\s*;", re.S)


def _normalise(c_type: str) -> str:
    c_type = re.sub(r"\s+", " ", c_type.strip())
    return re.sub(r"\s*\*", "*", c_type)


def parse_header(path: Path) -> dict:
    """{function: (return type, [(parameter type, parameter name), ...])} as C strings."""
    text = re.sub(r"/\*.*?\*/", "", path.read_text(), flags=re.S)
    out = {}
    for ret, name, params in _DECLARATION.findall(text):
        parsed = []
        params = params.strip()
        if params and params != "void":
            for piece in params.split(","):
                match = re.match(r"(.*?)(\w+)$", piece.strip(), re.S)
                parsed.append((_normalise(match.group(1)), match.group(2)))
        out[name] = (_normalise(ret), parsed)
    return out


def declared_functions() -> dict:
    """Every function of both headers."""
    functions = parse_header(HEADER)
    functions.update(parse_header(EXTENSION_HEADER))
    return functions


SIGNATURES = parse_header(HEADER)
EXTENSION_SIGNATURES = parse_header(EXTENSION_HEADER)
TRAIN_SIGNATURES = parse_header(TRAIN_HEADER)


class FlintError(RuntimeError):
    """A call returned a status other than OK."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def pointer(value):
    """A device address from a torch tensor, an int, or None (null)."""
    if value is None or isinstance(value, int):
        return value
    return value.data_ptr()


def stream_handle(stream):
    """A cudaStream_t value from a torch stream, an int handle, or None (torch's current)."""
    if stream is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def library_path() -> Path:
    override = os.environ.get("FLINT_LIB")
    if override:
        return Path(override)
    return ROOT / "flint_b200" / "lib" / LIBRARY_NAME


def _nbytes(tensor) -> int:
    if tensor is None or isinstance(tensor, int):
        return 0
    return tensor.numel() * tensor.element_size()


def _bind(lib, functions: dict) -> None:
    for name, (ret, params) in functions.items():
        function = getattr(lib, name)  # AttributeError if a declared symbol is missing
        function.restype = _C_TYPES[ret]
        function.argtypes = [_C_TYPES[c_type] for c_type, _ in params]


class Flint:
    """The loaded library. Methods mirror the C functions without the flint_ prefix."""

    def __init__(self, path=None):
        self.path = Path(path) if path else library_path()
        if not self.path.is_file():
            raise FileNotFoundError(
                f"{self.path} not found: build it with `python -c 'import __graft_entry__ as g; "
                "g.build()'` (or `make -C flint_b200/csrc`); there is no fallback implementation"
            )
        self.lib = ctypes.CDLL(str(self.path), mode=ctypes.RTLD_GLOBAL)
        self.functions = declared_functions()
        _bind(self.lib, self.functions)
        self._train = None

    @property
    def train(self):
        """libflint_train.so (the training step behind a C ABI), loaded on first use from
        beside libflint.so. It is a client of libflint.so and opens NCCL itself at run time."""
        if self._train is None:
            path = self.path.with_name(TRAIN_LIBRARY_NAME)
            if not path.is_file():
                raise FileNotFoundError(f"{path} not found: build it with `make -C flint_b200/csrc`")
            lib = ctypes.CDLL(str(path))
            _bind(lib, TRAIN_SIGNATURES)
            self._train = lib
        return self._train

    def check_train(self, status: int) -> None:
        if status != OK:
            detail = self.train.flint_train_last_error().decode()
            message = f"{self.status_string(status)} (status {status})"
            raise FlintError(status, f"{message}: {detail}" if detail else message)

    # -- plumbing ---------------------------------------------------------------------

    def version(self) -> str:
        return self.lib.flint_version().decode()

    def status_string(self, status: int) -> str:
        return self.lib.flint_status_string(status).decode()

    def last_error(self) -> str:
        return self.lib.flint_last_error().decode()

    def check(self, status: int) -> None:
        if status != OK:
            message = f"{self.status_string(status)} (status {status})"
            detail = self.last_error()
            raise FlintError(status, f"{message}: {detail}" if detail else message)

    def call(self, name: str, *args, stream=None):
        """Calls a status-returning function: tensors become addresses, bools ints, and
        the stream argument (always last in the C signature) is filled in."""
        _, params = self.functions[name]
        converted = []
        values = list(args)
        for c_type, param in params:
            if c_type == "flint_stream":
                converted.append(stream_handle(stream))
                continue
            value = values.pop(0)
            if _C_TYPES[c_type] is ctypes.c_void_p:
                value = pointer(value)
            elif c_type == "int":
                value = int(value)
            converted.append(value)
        if values:
            raise TypeError(f"{name}: {len(values)} arguments too many")
        self.check(getattr(self.lib, name)(*converted))

    def _size_query(self, name: str, *dims) -> int:
        size = ctypes.c_size_t()
        self.check(getattr(self.lib, name)(*dims, ctypes.byref(size)))
        return size.value

    # -- data movement ----------------------------------------------------------------

    def copy(self, dst, src, nbytes: int, stream=None) -> None:
        self.call("flint_copy", dst, src, nbytes, stream=stream)

    def fp32_to_fp16(self, y, x, count: int, stream=None) -> None:
        self.call("flint_fp32_to_fp16", y, x, count, stream=stream)

    def heads_split(self, y, x, batches, length, heads, head_width, row_width, first=0,
                    stream=None) -> None:
        self.call("flint_heads_split", y, x, batches, length, heads, head_width, row_width, first,
                  stream=stream)

    def heads_merge(self, y, x, batches, length, heads, head_width, row_width, first=0,
                    stream=None) -> None:
        self.call("flint_heads_merge", y, x, batches, length, heads, head_width, row_width, first,
                  stream=stream)

    def embedding_forward(self, x, tokens, wte, wpe, sequences, length, vocab, width,
                          stream=None) -> None:
        self.call("flint_embedding_forward", x, tokens, wte, wpe, sequences, length, vocab, width,
                  stream=stream)

    # -- GEMMs ------------------------------------------------------------------------

    def gemm_nt(self, y, x, w, m, n, k, stream=None) -> None:
        self.call("flint_gemm_nt", y, x, w, m, n, k, stream=stream)

    def gemm_nt_bias(self, y, x, w, bias, m, n, k, stream=None) -> None:
        self.call("flint_gemm_nt_bias", y, x, w, bias, m, n, k, stream=stream)

    def gemm_nt_bias_gelu(self, y, pre, x, w, bias, m, n, k, stream=None) -> None:
        self.call("flint_gemm_nt_bias_gelu", y, pre, x, w, bias, m, n, k, stream=stream)

    def gemm_nt_bias_residual(self, y, x, w, bias, residual, m, n, k, stream=None) -> None:
        self.call("flint_gemm_nt_bias_residual", y, x, w, bias, residual, m, n, k, stream=stream)

    def gemm_nn(self, y, x, w, m, n, k, stream=None) -> None:
        self.call("flint_gemm_nn", y, x, w, m, n, k, stream=stream)

    def gemm_nn_dgelu(self, y, x, w, pre, m, n, k, stream=None) -> None:
        self.call("flint_gemm_nn_dgelu", y, x, w, pre, m, n, k, stream=stream)

    def gemm_tn_workspace(self, m, n, k) -> int:
        return self._size_query("flint_gemm_tn_workspace", m, n, k)

    def gemm_tn(self, y, x, w, m, n, k, accumulate=False, workspace=None, workspace_bytes=None,
                stream=None) -> None:
        if workspace_bytes is None:
            workspace_bytes = _nbytes(workspace)
        self.call("flint_gemm_tn", y, x, w, m, n, k, bool(accumulate), workspace, workspace_bytes,
                  stream=stream)

    def gemm_nt_batched(self, y, x, w, batches, m, n, k, scale=1.0, stream=None) -> None:
        self.call("flint_gemm_nt_batched", y, x, w, batches, m, n, k, scale, stream=stream)

    def gemm_nn_batched(self, y, x, w, batches, m, n, k, stream=None) -> None:
        self.call("flint_gemm_nn_batched", y, x, w, batches, m, n, k, stream=stream)

    def gemm_tn_batched(self, y, x, w, batches, m, n, k, stream=None) -> None:
        self.call("flint_gemm_tn_batched", y, x, w, batches, m, n, k, stream=stream)

    # -- reductions and row-wise kernels --------------------------------------------------

    def bias_gradient_workspace(self, rows, cols) -> int:
        return self._size_query("flint_bias_gradient_workspace", rows, cols)

    def bias_gradient(self, dbias, dy, rows, cols, accumulate=False, workspace=None,
                      workspace_bytes=None, stream=None) -> None:
        if workspace_bytes is None:
            workspace_bytes = _nbytes(workspace)
        self.call("flint_bias_gradient", dbias, dy, rows, cols, bool(accumulate), workspace,
                  workspace_bytes, stream=stream)

    def bias_gradient_static(self, dbias, dy, rows, cols, accumulate=False, stream=None) -> None:
        """bias_gradient without a caller workspace (built-in 4 MiB scratch, no allocation)."""
        self.call("flint_b200_bias_gradient_static", dbias, dy, rows, cols, bool(accumulate),
                  stream=stream)

    def layernorm_forward(self, y, mean, rstd, x, gamma, beta, rows, cols, eps=1e-5,
                          stream=None) -> None:
        self.call("flint_layernorm_forward", y, mean, rstd, x, gamma, beta, rows, cols, eps,
                  stream=stream)

    def layernorm_backward_workspace(self, rows, cols) -> int:
        return self._size_query("flint_layernorm_backward_workspace", rows, cols)

    def layernorm_backward(self, dx, dgamma, dbeta, dy, x, mean, rstd, gamma, rows, cols,
                           accumulate_dx=False, accumulate_params=False, workspace=None,
                           workspace_bytes=None, stream=None) -> None:
        if workspace_bytes is None:
            workspace_bytes = _nbytes(workspace)
        self.call("flint_layernorm_backward", dx, dgamma, dbeta, dy, x, mean, rstd, gamma, rows,
                  cols, bool(accumulate_dx), bool(accumulate_params), workspace, workspace_bytes,
                  stream=stream)

    def embedding_backward_workspace(self, sequences, length, vocab, width) -> int:
        return self._size_query("flint_embedding_backward_workspace", sequences, length, vocab,
                                width)

    def embedding_backward(self, dwte, dwpe, dx, tokens, sequences, length, vocab, width,
                           accumulate_wte=False, accumulate_wpe=False, workspace=None,
                           workspace_bytes=None, stream=None) -> None:
        if workspace_bytes is None:
            workspace_bytes = _nbytes(workspace)
        self.call("flint_embedding_backward", dwte, dwpe, dx, tokens, sequences, length, vocab,
                  width, bool(accumulate_wte), bool(accumulate_wpe), workspace, workspace_bytes,
                  stream=stream)

    def causal_softmax_forward(self, p, s, batches, length, stream=None) -> None:
        self.call("flint_causal_softmax_forward", p, s, batches, length, stream=stream)

    def causal_softmax_backward(self, ds, p, dp, batches, length, scale=0.125,
                                stream=None) -> None:
        self.call("flint_causal_softmax_backward", ds, p, dp, batches, length, scale,
                  stream=stream)

    def softmax_cross_entropy(self, dlogits, row_loss, logits, targets, scale, rows, vocab, cols,
                              stream=None) -> None:
        self.call("flint_softmax_cross_entropy", dlogits, row_loss, logits, targets, scale, rows,
                  vocab, cols, stream=stream)

    # -- extensions -----------------------------------------------------------------------

    def kernel_fault(self) -> bool:
        """True if a tensor-core kernel gave up on a barrier wait since the last call."""
        raised = ctypes.c_int(0)
        self.check(self.lib.flint_b200_kernel_fault(ctypes.addressof(raised)))
        return raised.value != 0

    def launch_count(self) -> int:
        """Kernels launched by the library in this process so far."""
        count = ctypes.c_ulonglong(0)
        self.check(self.lib.flint_b200_launch_count(ctypes.byref(count)))
        return count.value

    def attention_forward(self, o, lse, q, k, v, batches, length, head_width, scale,
                          stream=None) -> None:
        self.call("flint_b200_attention_forward", o, lse, q, k, v, batches, length, head_width,
                  scale, stream=stream)

    def attention_backward(self, dq, dk, dv, d_o, o, lse, delta, q, k, v, batches, length,
                           head_width, scale, stream=None) -> None:
        self.call("flint_b200_attention_backward", dq, dk, dv, d_o, o, lse, delta, q, k, v,
                  batches, length, head_width, scale, stream=stream)

    def adamw(self, param, m, v, grad, half_copy, count, lr, beta1, beta2, eps, weight_decay,
              grad_scale, step, skip=None, stream=None) -> None:
        self.call("flint_b200_adamw", param, m, v, grad, half_copy, count, lr, beta1, beta2, eps,
                  weight_decay, grad_scale, step, skip, stream=stream)

    def adamw_plan(self, tensors, stream=None):
        """A device-resident plan for adamw_run from (param, m, v, grad, half_copy, count,
        weight_decay) tuples of addresses. Returns (plan tensor, items)."""
        import torch

        array = (AdamwTensor * len(tensors))(*[AdamwTensor(*t) for t in tensors])
        nbytes, items = ctypes.c_size_t(), ctypes.c_size_t()
        self.check(self.lib.flint_b200_adamw_plan_bytes(array, len(tensors), ctypes.byref(nbytes)))
        self.check(self.lib.flint_b200_adamw_plan_items(array, len(tensors), ctypes.byref(items)))
        plan = torch.empty(nbytes.value + 16, dtype=torch.uint8, device="cuda")
        self.check(self.lib.flint_b200_adamw_plan(plan.data_ptr(), nbytes.value, array,
                                                  len(tensors), stream_handle(stream)))
        return plan, items.value

    def adamw_run(self, plan, items, lr, beta1, beta2, eps, grad_scale, step, skip=None,
                  stream=None) -> None:
        self.call("flint_b200_adamw_run", plan, items, lr, beta1, beta2, eps, grad_scale, step,
                  skip, stream=stream)

    def check_gradients(self, grad, count, scale, found_nonfinite, sum_squares=None,
                        stream=None) -> None:
        self.call("flint_b200_check_gradients", grad, count, scale, found_nonfinite, sum_squares,
                  stream=stream)


class Gpt2:
    """A flint_gpt2 model; freed by close() or on leaving a with block. Addresses of its
    weights, gradients and outputs are device addresses as ints."""

    def __init__(self, flint: Flint, config: Gpt2Config, flash_attention=None, borrowed=None):
        self.flint = flint
        self.config = config
        self.owned = borrowed is None
        if borrowed is not None:  # a model that something else (a trainer) owns and frees
            self.handle = borrowed
            return
        handle = ctypes.c_void_p()
        if flash_attention is None:
            status = flint.lib.flint_gpt2_create(ctypes.byref(config), ctypes.byref(handle))
        else:
            status = flint.lib.flint_b200_gpt2_create(ctypes.byref(config),
                                                      int(bool(flash_attention)),
                                                      ctypes.byref(handle))
        flint.check(status)
        self.handle = handle.value

    def close(self) -> None:
        if self.handle is not None and self.owned:
            self.flint.lib.flint_gpt2_destroy(self.handle)
        self.handle = None

    def __enter__(self):
        return self

    def __exit__(self, *_):
        self.close()

    def parameters(self) -> list:
        return self._infos(self.flint.lib.flint_gpt2_parameter)

    def gradients(self) -> list:
        return self._infos(self.flint.lib.flint_gpt2_gradient)

    def _infos(self, function) -> list:
        out = []
        for i in range(self.flint.lib.flint_gpt2_parameter_count(self.handle)):
            info = Gpt2ParameterInfo()
            self.flint.check(function(self.handle, i, ctypes.byref(info)))
            out.append((info.name.decode(), info.data, info.rows, info.cols))
        return out

    def load(self, state, stream=None) -> None:
        """Copies state[name] (FP32 device tensors) into the master weights and syncs."""
        import torch

        for name, address, rows, cols in self.parameters():
            tensor = state[name].contiguous()
            if tensor.dtype != torch.float32 or tensor.numel() != rows * cols:
                raise ValueError(f"{name}: {tensor.dtype} {tuple(tensor.shape)}, "
                                 f"expected FP32 {rows} x {cols}")
            self.flint.copy(address, tensor, rows * cols * 4, stream)
        self.sync_weights(stream)

    def sync_weights(self, stream=None) -> None:
        self.flint.check(
            self.flint.lib.flint_gpt2_sync_weights(self.handle, stream_handle(stream)))

    def forward(self, tokens, targets, scale: float, stream=None) -> None:
        self.flint.check(self.flint.lib.flint_gpt2_forward(
            self.handle, pointer(tokens), pointer(targets), scale, stream_handle(stream)))

    def backward(self, tokens, accumulate=False, stream=None, callback=None) -> None:
        """callback(bucket, address, nbytes), if given, runs as each gradient bucket's
        producers have been enqueued (see flint_b200_gpt2_backward_buckets)."""
        if callback is None:
            self.flint.check(self.flint.lib.flint_gpt2_backward(
                self.handle, pointer(tokens), int(accumulate), stream_handle(stream)))
            return
        raised = []

        def trampoline(_user, bucket, address, nbytes):
            try:
                callback(bucket, address, nbytes)
            except BaseException as error:  # never unwind through C
                raised.append(error)

        hook = BUCKET_CALLBACK(trampoline)
        status = self.flint.lib.flint_b200_gpt2_backward_buckets(
            self.handle, pointer(tokens), int(accumulate), stream_handle(stream), hook, None)
        if raised:
            raise raised[0]
        self.flint.check(status)

    def gradient_arena(self) -> tuple:
        base, size = ctypes.c_void_p(), ctypes.c_size_t()
        self.flint.check(self.flint.lib.flint_b200_gpt2_gradient_arena(
            self.handle, ctypes.byref(base), ctypes.byref(size)))
        return base.value, size.value

    def outputs(self) -> tuple:
        logits, dlogits, row_loss = ctypes.c_void_p(), ctypes.c_void_p(), ctypes.c_void_p()
        self.flint.check(self.flint.lib.flint_gpt2_outputs(
            self.handle, ctypes.byref(logits), ctypes.byref(dlogits), ctypes.byref(row_loss)))
        return logits.value, dlogits.value, row_loss.value

    def mean_loss(self, stream=None) -> float:
        loss = ctypes.c_double()
        self.flint.check(self.flint.lib.flint_gpt2_mean_loss(
            self.handle, stream_handle(stream), ctypes.addressof(loss)))
        return loss.value

    def read(self, address: int, shape, dtype, first_element: int = 0, stream=None):
        """A device tensor holding a copy of the memory at address."""
        import torch

        out = torch.empty(shape, dtype=dtype, device="cuda")
        size = torch.empty((), dtype=dtype).element_size()
        self.flint.copy(out, address + first_element * size, out.numel() * size, stream)
        torch.cuda.synchronize()
        return out
