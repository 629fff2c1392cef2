"""Tensor-parallel decode on 2 GPUs: the sharded step with the in-kernel all-reduce must
produce the token of the unsharded step and of the CPU oracle.

Each rank is its own process on its own GPU (kernels that wait on one another
must never share a GPU), launched with torchrun; the test is skipped on a box
with fewer than two GPUs.  All device-side waits are bounded, so a failure is
an error code, not a hang.
"""

import os
import socket
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_decode_matches_single_gpu_and_oracle():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "tp_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, tail
    assert "single-GPU" in r.stdout, tail
