"""GPU: minibatch-sharded training on 2 GPUs of one node (gradient sums over
NVLink: the library's peer-memory all-reduce kernel, NCCL for plain buffers).

Needs at least two visible GPUs; on a single-GPU machine the test is skipped
(the host-side logic of the same path is covered on CPU by test_dist_cpu.py
with two gloo ranks).  NVLS is switched off for the child processes so a rank
that dies in a failed assertion cannot leave multicast state behind.
"""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _gpu_count():
    import torch
    return torch.cuda.device_count()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_two_gpu_training_matches_full_batch_oracle():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "dp_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0 and "DP_PARITY_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(_gpu_count() < 2, reason="needs two GPUs")
def test_all_reduce_gives_up_when_a_rank_does_not_join():
    """Failure made on the host (rank 1 never issues its half of an all-reduce):
    rank 0's kernel runs into its wait limit, reports through the kernel fault
    word, and both ranks carry on with a working communicator."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MG_PEER_WAIT_MS="300")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "dp_timeout_check.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env, cwd=ROOT)
    assert r.returncode == 0 and "DP_TIMEOUT_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
