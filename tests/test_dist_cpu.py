"""world_size-2 gloo test on CPU of the multi-GPU host logic (no GPU)."""
import os
import socket
import subprocess
import sys

from conftest import ROOT


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def test_tensor_parallel_sharding_arithmetic_world_size_2():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "dist_cpu_worker.py")]
    env = dict(os.environ, OMP_NUM_THREADS="2")
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "DIST_CPU_OK" in r.stdout


def test_shard_plan_rejects_uneven_splits():
    import pytest
    from neural_api_b200 import parallel
    with pytest.raises(ValueError):
        parallel.tp_shard_plan(896, 4864, 14, 2, 64, 151936, 0, 4)      # 2 KV heads over 4 ranks
    plan = parallel.tp_shard_plan(5120, 27648, 40, 8, 128, 152064, 7, 8)
    assert plan["q_rows"] == (4480, 5120) and plan["down_cols"] == (24192, 27648) and plan["head_rows"] == (133056, 152064)
