import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA GPU (run with -m gpu on a B200)")


def load_golden(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"))


def golden_hf_case(name):
    """(config dict, {hf name: fp32 array}, sequences, golden logits) of one pico checkpoint."""
    z = load_golden(name)
    cfg = json.loads(bytes(z["config_json"]).decode())
    tensors = {k[3:]: z[k] for k in z.files if k.startswith("t::")}
    return cfg, tensors, z["sequences"], z["logits"]


@pytest.fixture(scope="session")
def backend():
    """The CUDA backend. No fallback: a missing library or GPU is an error, not a skip."""
    from neural_api_b200.backend import CudaBackend
    b = CudaBackend(0)
    yield b
    b.close()
