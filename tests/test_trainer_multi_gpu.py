"""The data-parallel trainer on two or more GPUs of one box, over NCCL.

Launches tests/trainer_ranks.py with one process per GPU (torch.distributed.run on
127.0.0.1) and requires every rank to exit 0; the checks themselves are listed in that
file's docstring. NVLink multicast is switched off for NCCL (NCCL_NVLS_ENABLE=0): the ranks
are short-lived child processes. Skipped on a box with a single GPU.
"""

import os
import socket
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = Path(__file__).resolve().parent


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_update_modes_rank_agreement_skipped_steps_and_checkpoints_on_two_ranks():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1")
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
               str(HERE / "trainer_ranks.py")]
    done = subprocess.run(command, env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout[-3000:] + done.stderr[-3000:]
    assert "trainer ranks ok: world 2" in done.stdout
