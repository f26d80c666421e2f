"""The C ABI's GPU-free surface: exports, version, status strings, argument validation
that happens before any CUDA call, workspace formulas and the forward-only memory plan.
Runs on the CPU (no compute calls)."""

import ctypes
import re
import shutil
import subprocess

import pytest

import flint_b200
from flint_b200 import binding

REFERENCE_ABI = """
flint_version flint_status_string flint_last_error flint_copy flint_gemm_nt flint_gemm_nt_bias
flint_gemm_nt_bias_gelu flint_gemm_nt_bias_residual flint_gemm_nn flint_gemm_nn_dgelu
flint_gemm_tn flint_gemm_tn_workspace flint_bias_gradient flint_bias_gradient_workspace
flint_gemm_nt_batched flint_gemm_nn_batched flint_gemm_tn_batched flint_layernorm_forward
flint_layernorm_backward flint_layernorm_backward_workspace flint_embedding_forward
flint_embedding_backward flint_embedding_backward_workspace flint_fp32_to_fp16
flint_heads_split flint_heads_merge flint_causal_softmax_forward
flint_causal_softmax_backward flint_softmax_cross_entropy flint_gpt2_bytes flint_gpt2_create
flint_gpt2_destroy flint_gpt2_parameter_count flint_gpt2_parameter flint_gpt2_sync_weights
flint_gpt2_forward flint_gpt2_backward flint_gpt2_gradient flint_gpt2_outputs
flint_gpt2_mean_loss
""".split()


def test_header_declares_exactly_the_reference_abi():
    assert len(REFERENCE_ABI) == 40
    assert sorted(binding.SIGNATURES) == sorted(REFERENCE_ABI)


def test_library_exports_every_declared_function(flint):
    for name in list(binding.SIGNATURES) + list(binding.EXTENSION_SIGNATURES):
        assert hasattr(flint.lib, name), name


def test_status_codes_match_header():
    header = binding.HEADER.read_text()
    codes = dict(re.findall(r"\bFLINT_(OK|ERROR_\w+)\s*=\s*(\d+)", header))
    assert {n: getattr(flint_b200, n) for n in codes} == {n: int(v) for n, v in codes.items()}


def test_version_and_status_strings(flint):
    assert re.fullmatch(r"\d+\.\d+\.\d+", flint.version())
    assert [flint.status_string(s) for s in (0, 1, 2, -1, 3, 2**31 - 1)] == [
        "ok", "invalid argument", "CUDA error", "unknown status", "unknown status",
        "unknown status"]
    with pytest.raises(flint_b200.FlintError, match=r"^CUDA error \(status 2\)") as error:
        flint.check(flint_b200.ERROR_CUDA)
    assert error.value.status == flint_b200.ERROR_CUDA


def test_library_links_no_cuda_libraries(flint):
    readelf = shutil.which("readelf")
    if readelf is None:
        pytest.skip("readelf not installed")
    out = subprocess.run([readelf, "-d", str(flint.path)], capture_output=True, text=True).stdout
    needed = re.findall(r"\(NEEDED\)\s+Shared library: \[(.+?)\]", out)
    assert needed
    assert not [n for n in needed if re.search(r"cublas|cudnn|nvidia-ml|nvml|cudart|nccl", n, re.I)]
    assert not re.search(rb"cublas|cudnn|nvml", flint.path.read_bytes(), re.I)


def raises(flint, text, call):
    with pytest.raises(flint_b200.FlintError) as error:
        call()
    assert text in str(error.value)
    assert text in flint.last_error()
    assert error.value.status == flint_b200.ERROR_INVALID_ARGUMENT


def test_validation_runs_before_any_cuda_call(flint):
    s = 0  # the null stream; nothing reaches the GPU
    raises(flint, "flint_copy: dst is null", lambda: flint.copy(None, 16, 16, stream=s))
    raises(flint, "flint_copy: src is null", lambda: flint.copy(16, None, 16, stream=s))
    raises(flint, "dst and src overlap", lambda: flint.copy(32, 16, 32, stream=s))
    flint.copy(None, None, 0, stream=s)
    raises(flint, "k (7) must be a positive multiple of 8",
           lambda: flint.gemm_nt(16, 16, 16, 8, 8, 7, stream=s))
    raises(flint, "y is not 16-byte aligned",
           lambda: flint.gemm_nt(1 << 20 | 2, 2 << 20, 3 << 20, 8, 8, 8, stream=s))
    raises(flint, "m and n can be up to 8388480, and k up to 65536",
           lambda: flint.gemm_nn(1 << 20, 2 << 20, 3 << 20, 8388481, 8, 8, stream=s))
    raises(flint, "y and x overlap", lambda: flint.gemm_nt(1 << 20, 1 << 20, 3 << 20, 8, 8, 8,
                                                           stream=s))
    raises(flint, "cols (12) must be a multiple of 8 up to 16776960",
           lambda: flint.bias_gradient_workspace(8, 12))
    raises(flint, "rows (0) must be from 1 to 549755813632",
           lambda: flint.bias_gradient_workspace(0, 0))
    raises(flint, "cols (0) must be a multiple of 8 from 8 to 16776960",
           lambda: flint.layernorm_backward_workspace(8, 0))
    raises(flint, "eps (-1) must be finite and non-negative",
           lambda: flint.layernorm_forward(16, 32, 48, 64, 80, 96, 1, 8, -1.0, stream=s))
    raises(flint, "length (12) must be a multiple of 8 up to 1024",
           lambda: flint.causal_softmax_forward(16, 32, 1, 12, stream=s))
    raises(flint, "vocab (9) must be from 1 to cols (8)",
           lambda: flint.softmax_cross_entropy(16, 32, 48, 64, 1.0, 1, 9, 8, stream=s))
    raises(flint, "scale (inf) must be finite",
           lambda: flint.causal_softmax_backward(16, 32, 48, 1, 8, float("inf"), stream=s))
    raises(flint, "heads of 64 columns from column 8 run past row_width (128)",
           lambda: flint.heads_split(16, 32, 1, 8, 2, 64, 128, 8, stream=s))
    raises(flint, "count", lambda: flint.fp32_to_fp16(16, 32, 2**63, stream=s))
    raises(flint, "flint_b200_bias_gradient_static: dbias is null",
           lambda: flint.bias_gradient_static(None, 32, 8, 8, False, stream=s))
    raises(flint, "built-in scratch holds 4194304",
           lambda: flint.bias_gradient_static(16, 32, 65536, 4096, False, stream=s))
    raises(flint, "needs 64 bytes of workspace, given 0",
           lambda: flint.bias_gradient(1 << 20, 2 << 20, 8, 8, False, None, 0, stream=s))
    # Zero-sized calls succeed with null pointers.
    flint.gemm_nt(None, None, None, 0, 8, 8, stream=s)
    flint.layernorm_forward(None, None, None, None, None, None, 0, 8, 1e-5, stream=s)
    flint.causal_softmax_forward(None, None, 0, 8, stream=s)


def test_workspace_formulas(flint):
    assert flint.bias_gradient_workspace(8192, 768) == 32 * 768 * 8
    assert flint.bias_gradient_workspace(257, 8) == 2 * 8 * 8
    assert flint.layernorm_backward_workspace(8192, 768) == flint.bias_gradient_workspace(8192, 768)
    align = lambda b: -(-b // 16) * 16
    seqs, length, vocab, width = 8, 1024, 50304, 768
    rows = seqs * length
    want = (align(flint.bias_gradient_workspace(seqs, length * width)) + 2 * align(rows * 2)
            + 2 * align(rows * 4) + align((vocab + 1) * 4) + align(-(-rows // 2048) * 256 * 4))
    assert flint.embedding_backward_workspace(seqs, length, vocab, width) == want


def test_forward_only_memory_plan_needs_no_gpu(flint):
    cfg = flint_b200.Gpt2Config(2, 2, 128, 64, 200, 208, 3, 64, 0, 0)
    size = ctypes.c_size_t()
    flint.check(flint.lib.flint_gpt2_bytes(ctypes.byref(cfg), ctypes.byref(size)))
    up = lambda b: -(-b // 256) * 256
    w, rows, hb, t, v = 128, 192, 6, 64, 208
    params = [v * w, 64 * w] + 2 * [w, w, 3 * w * w, 3 * w, w * w, w, w, w, 4 * w * w, 4 * w,
                                    4 * w * w, w] + [w, w]
    total = sum(up(4 * p) for p in params)
    total += up(2 * v * w) + 2 * sum(up(2 * n) for n in (3 * w * w, w * w, 4 * w * w, 4 * w * w))
    total += 2 * up(rows * w * 4) + up(rows * w * 2) + 2 * up(rows * 4) + up(rows * 3 * w * 2)
    total += 3 * up(rows * w * 2) + 2 * up(hb * t * t * 2) + 2 * up(rows * w * 2)
    total += 2 * up(rows * 4 * w * 2) + 2 * up(rows * v * 2) + up(rows * 4)
    assert size.value == total
    bad = flint_b200.Gpt2Config(0, 2, 128, 64, 200, 208, 3, 64, 0, 0)
    status = flint.lib.flint_gpt2_bytes(ctypes.byref(bad), ctypes.byref(size))
    assert status == flint_b200.ERROR_INVALID_ARGUMENT
    assert "layers (0) must be from 1 to 1024" in flint.last_error()
    assert flint.lib.flint_gpt2_parameter_count(None) == 0


def test_the_kernel_bench_module_lists_its_groups():
    """python -m flint_b200.kernel_bench is the per-kernel counterpart of the reference's C++
    bench harness; importing it needs no GPU."""
    from flint_b200 import kernel_bench

    assert set(kernel_bench.GROUPS) == {"gemm", "epilogue", "batched", "attention", "rowwise"}
    assert kernel_bench.measured_peaks()[0] > 1000 and kernel_bench.NOMINAL_TFLOPS == 2250.0


# ---- libflint_train.so (the training step behind a C ABI) -----------------------------------------


def test_training_library_exports_its_header_and_links_no_nccl(flint):
    lib = flint.train
    assert len(binding.TRAIN_SIGNATURES) == 18
    for name in binding.TRAIN_SIGNATURES:
        assert hasattr(lib, name), name
    path = flint.path.with_name(binding.TRAIN_LIBRARY_NAME)
    readelf = shutil.which("readelf")
    if readelf is not None:
        out = subprocess.run([readelf, "-d", str(path)], capture_output=True, text=True).stdout
        needed = re.findall(r"\(NEEDED\)\s+Shared library: \[(.+?)\]", out)
        assert "libflint.so" in needed
        # NCCL is opened with dlopen at run time, and only for more than one rank.
        assert not [n for n in needed if re.search(r"nccl|cublas|cudnn|cudart|torch", n, re.I)]


def test_loss_scale_policy_is_gradscalers(flint):
    from flint_b200.trainer import LossScaler

    lib = flint.train
    python = LossScaler(65536.0, growth_interval=3)
    scale, good = 65536.0, 0
    for found in [0, 0, 1, 0, 0, 0, 0, 1, 1, 0, 0, 0]:
        next_scale, next_good = ctypes.c_float(), ctypes.c_int()
        status = lib.flint_train_scale_policy(scale, good, 3, found, ctypes.byref(next_scale),
                                              ctypes.cast(ctypes.byref(next_good), ctypes.c_void_p))
        assert status == flint_b200.OK
        scale, good = next_scale.value, next_good.value
        python.update(bool(found))
        assert (scale, good) == (python.scale, python.good_steps)
    assert scale == 32768.0 and good == 0  # 2^16: /2, x2, /2, /2, x2


def test_trainer_configuration_is_validated_before_any_cuda_call(flint):
    lib = flint.train

    def create(**changes):
        c = binding.TrainerConfigC()
        c.model = flint_b200.Gpt2Config(2, 2, 128, 64, 200, 208, 2, 64, 0, 1)
        c.flash_attention, c.lr, c.beta1, c.beta2, c.eps = 1, 6e-4, 0.9, 0.95, 1e-8
        c.weight_decay, c.loss_scale, c.growth_interval, c.max_grad_norm = 0.1, 65536.0, 2000, 0.0
        c.world, c.rank = 1, 0
        for key, value in changes.items():
            setattr(c, key, value)
        handle = ctypes.c_void_p(1)
        status = lib.flint_trainer_create(ctypes.byref(c), None, ctypes.byref(handle))
        return status, handle.value, lib.flint_train_last_error().decode()

    for changes, text in [(dict(world=0), "rank (0) must be from 0 to world (0) - 1"),
                          (dict(world=2, rank=2), "rank (2) must be from 0 to world (2) - 1"),
                          (dict(beta1=1.0), "betas in [0, 1)"),
                          (dict(loss_scale=0.0), "loss_scale (0) must be positive"),
                          (dict(growth_interval=0), "growth_interval (0) must be at least 1"),
                          (dict(max_grad_norm=-1.0), "max_grad_norm (-1) must be finite")]:
        status, handle, message = create(**changes)
        assert status == flint_b200.ERROR_INVALID_ARGUMENT and handle is None, changes
        assert text in message, (changes, message)
    assert lib.flint_trainer_step(None, None, None, 1, None) == flint_b200.ERROR_INVALID_ARGUMENT
    assert "must not be null" in lib.flint_train_last_error().decode()
