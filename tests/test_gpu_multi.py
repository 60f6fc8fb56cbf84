"""Tensor-parallel and expert-parallel decode over NCCL on 2+ GPUs: N-GPU result == 1-GPU result.
Skipped on a single-GPU box (the sharding arithmetic is covered on CPU by test_dist_cpu.py)."""
import os
import socket
import subprocess
import sys

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=60).stdout
        return sum(1 for l in out.splitlines() if l.startswith("GPU "))
    except Exception:
        return 0


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


@pytest.mark.parametrize("allreduce", ["peer", "nccl"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_tensor_parallel_matches_single_gpu(world, allreduce):
    if gpu_count() < world:
        pytest.skip("needs %d GPUs" % world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "tp_gpu_worker.py")]
    env = dict(os.environ)
    env.pop("CAI_TP_ALLREDUCE", None)
    if allreduce == "nccl":
        env["CAI_TP_ALLREDUCE"] = "nccl"          # the library all-reduce instead of the peer-memory kernel
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-5000:]
    assert "TP_GPU_OK" in r.stdout


@pytest.mark.parametrize("exchange", ["peer", "nccl"])
@pytest.mark.parametrize("world", [2, 4, 8])
def test_expert_parallel_matches_single_gpu(world, exchange):
    if gpu_count() < world:
        pytest.skip("needs %d GPUs" % world)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()), os.path.join(ROOT, "tests", "ep_gpu_worker.py")]
    env = dict(os.environ)
    env.pop("CAI_EP_EXCHANGE", None)
    if exchange == "nccl":
        env["CAI_EP_EXCHANGE"] = "nccl"           # the library's all-gather + reduce-scatter instead of the peer-memory kernels
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-5000:]
    assert "EP_GPU_OK" in r.stdout
