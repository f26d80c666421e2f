"""flint_b200_bias_gradient_static: the bias gradient for hosts that may not allocate.

Some callers cannot give the library a workspace because they are not allowed to
allocate device memory while running (an embedded plug-in whose host owns the memory
budget, or a loop that cannot take cudaMalloc's device-wide synchronisation). This
entry point keeps its partial sums in an array built into the library. The test calls
it through the C ABI twice in a row, with different shapes so the second call finds the
first one's leftovers in the shared array, and requires the same bits as
flint_bias_gradient, and as the CPU oracle's emulation of the pinned order, each time. The file sorts last so a run that stops at the first
failure has already exercised every other test.
"""

import numpy as np
import pytest
import torch

import flint_b200
import flint_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda"


def crafted(seed, rows, cols):
    rng = np.random.default_rng(seed)
    base = rng.standard_normal((rows, cols)) * np.exp2(rng.integers(-6, 7, (rows, cols)))
    return torch.from_numpy(np.clip(base, -60000, 60000).astype(np.float16)).to(DEV)


def test_static_scratch_matches_the_workspace_version_on_consecutive_calls(flint):
    for call, (rows, cols) in enumerate([(16384, 3072), (1000, 768)]):
        dy = crafted(call, rows, cols)
        workspace = torch.empty(flint.bias_gradient_workspace(rows, cols), dtype=torch.uint8,
                                device=DEV)
        want = torch.full((cols,), 3.0, device=DEV)
        flint.bias_gradient(want, dy, rows, cols, False, workspace)
        got = torch.full((cols,), -7.0, device=DEV)
        flint.bias_gradient_static(got, dy, rows, cols, False)
        torch.cuda.synchronize()
        assert torch.equal(got.view(torch.int32), want.view(torch.int32))
        from_oracle = torch.from_numpy(oracle.bias_gradient(dy.cpu().numpy()))
        assert torch.equal(got.cpu().view(torch.int32), from_oracle.view(torch.int32))
        # Accumulating adds the same sums to what is there, with one FP32 add each.
        old = torch.arange(cols, dtype=torch.float32, device=DEV)
        acc_want = old.clone()
        acc_got = old.clone()
        flint.bias_gradient(acc_want, dy, rows, cols, True, workspace)
        flint.bias_gradient_static(acc_got, dy, rows, cols, True)
        torch.cuda.synchronize()
        assert torch.equal(acc_got.view(torch.int32), acc_want.view(torch.int32))


def test_static_scratch_rejects_shapes_beyond_its_size(flint):
    rows, cols = 65536, 4096  # 256 chunks x 4096 cols x 8 bytes = 8 MiB
    dy = torch.zeros(8, dtype=torch.half, device=DEV)
    out = torch.zeros(cols, device=DEV)
    with pytest.raises(flint_b200.FlintError, match="built-in scratch holds 4194304") as error:
        flint.bias_gradient_static(out, dy, rows, cols, False)
    assert error.value.status == flint_b200.ERROR_INVALID_ARGUMENT
    flint.bias_gradient_static(None, None, 1, 0, False)  # zero columns: nothing to do


def test_static_scratch_names_a_bad_pointer_like_every_other_entry_point(flint):
    dy = torch.zeros(64, 8, dtype=torch.half, device=DEV)
    out = torch.zeros(8, device=DEV)
    with pytest.raises(flint_b200.FlintError, match="dbias is null") as error:
        flint.bias_gradient_static(None, dy, 64, 8, False)
    assert error.value.status == flint_b200.ERROR_INVALID_ARGUMENT
    with pytest.raises(flint_b200.FlintError, match="dy is not 16-byte aligned"):
        flint.bias_gradient_static(out, dy.data_ptr() + 2, 32, 8, False)
