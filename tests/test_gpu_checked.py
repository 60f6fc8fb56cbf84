"""The checked build (libcai_cuda_checked.so, -DCAI_CHECKED): the ordinary kernels with every launch followed by a
synchronize and a look at the device error words, CUDA graphs off, and indices from device-side state that the ordinary
build clamps or skips silently reported as statuses. Run in child processes, because a process binds one of the two
libraries (CAI_CUDA_CHECKED=1 selects the checked one)."""
import os
import subprocess
import sys
import textwrap

import pytest

from conftest import ROOT

pytestmark = pytest.mark.gpu


def _run(args, checked, timeout=900):
    env = dict(os.environ)
    env["CAI_CUDA_CHECKED"] = "1" if checked else "0"
    return subprocess.run([sys.executable] + args, cwd=ROOT, env=env, capture_output=True, text=True, timeout=timeout)


def test_layer_and_model_parity_hold_under_the_checked_build():
    """Every layer-granular entry point against the oracle right after its kernels ran (tests/test_gpu_layers.py), and
    whole models against the oracle and the reference's golden logits (tests/test_gpu_model.py), with the checked
    library: same results, no launch raises anything."""
    r = _run(["-m", "pytest", "tests/test_gpu_layers.py", "tests/test_gpu_model.py", "-x", "-q", "-p", "no:cacheprovider"], checked=True)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout and "failed" not in r.stdout


SCRIPT = textwrap.dedent('''
    import numpy as np
    from neural_api_b200 import _lib
    from neural_api_b200.backend import CudaBackend, CaiError, MoEExpertBank, TYPE_Q8_0
    from oracle import codecs
    lib = _lib.load()
    checked = lib.cai_cuda_is_checked_build()
    be = CudaBackend(0)
    rng = np.random.default_rng(0)
    E, H, I, K, T = 4, 64, 96, 2, 3
    bank = MoEExpertBank(be, E, H, I, TYPE_Q8_0)
    for e in range(E):
        for which, (n, k) in (("up", (I, H)), ("gate", (I, H)), ("down", (H, I))):
            bank.upload(e, which, codecs.quantize_q8_0((rng.standard_normal((n, k)) * 0.05).astype(np.float32)))
    bank.finalize()
    x = rng.standard_normal((T, H)).astype(np.float32)
    ids = np.array([[0, 1], [2, 3], [1, 9]], dtype=np.int32)          # 9: no such expert
    gates = np.full((T, K), 0.5, dtype=np.float32)
    dx, dg = be.to_device(x), be.to_device(gates.reshape(-1))
    dh, dout = be.alloc(T * K * I * 4), be.alloc(T * H * 4)

    def run(id_rows):
        dids = be.to_device(id_rows.reshape(-1))
        try:
            bank.gate_up(dx, dids, T, K, dh)
            bank.down(dh, dids, dg, T, K, dout)
            return dout.read(np.float32, T * H)
        finally:
            dids.free()

    try:
        y = run(ids)
        print("RESULT ok checked=%d finite=%d" % (checked, int(np.isfinite(y).all())))
    except CaiError as e:
        print("RESULT error checked=%d %s" % (checked, e))
    ids[2, 1] = 3
    y = run(ids)                                                       # the context stays usable
    print("AFTER finite=%d" % int(np.isfinite(y).all()))
''')


@pytest.mark.parametrize("checked", [False, True])
def test_an_expert_id_outside_the_bank_is_skipped_silently_or_reported(checked):
    """cai_moe_gate_up_dev takes expert ids from device memory the caller owns. The ordinary build clamps an id that names
    no expert into the bank (no access outside it, like an out-of-range token id in the embedding gather); the checked
    build does the same and reports the id with its bound and the launch site. The next call works in both."""
    r = _run(["-c", SCRIPT], checked=checked, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("RESULT")][0]
    if checked:
        assert "error checked=1" in line and "expert id" in line and "9 outside [0, 4)" in line and "launch at" in line
    else:
        assert line.startswith("RESULT ok checked=0 finite=1")
    assert "AFTER finite=1" in r.stdout
