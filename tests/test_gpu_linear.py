"""Dequant-fused quantized linear (GEMV path) against the oracle: fp32 compute over
the bit-exact dequantized weights, the path a GGUF Q8_0/Q4_0 import runs in the
reference. Shapes and value laws of the isolated-linear sweep."""
import numpy as np
import pytest

from oracle import codecs
from neural_api_b200.backend import DotProductSharedKernel
from neural_api_b200.configs import LINEAR_BATCHES, LINEAR_SHAPES

pytestmark = pytest.mark.gpu

# max |y - y_ref| <= TOL * RMS(y_ref). fp32 accumulation in a different order from BLAS;
# the budget the decode path is held to is 1e-3.
TOL = 2e-5
# Batches of 9..64 rows (3..8 on large matrices) run on the tensor cores: exact integer codes times activations
# split into two fp16 limbs (22 bits), per-block sums scaled in fp32. Measured ~1e-6 of the output RMS.
TOL_TC = 2e-5


def make_blocks(ggml_type, n, k, seed):
    """Q4_0: nibbles uniform 0..15; Q8_0: int8 uniform [-127,127]; fp16 scale uniform [0.001, 0.05]."""
    rng = np.random.default_rng(seed)
    nblk = n * k // 32
    scale = rng.uniform(0.001, 0.05, nblk).astype(np.float32)
    if ggml_type == codecs.GGML_Q8_0:
        blk = np.empty((nblk, 34), dtype=np.uint8)
        blk[:, 2:] = rng.integers(-127, 128, (nblk, 32), dtype=np.int8).view(np.uint8)
    else:
        blk = np.empty((nblk, 18), dtype=np.uint8)
        blk[:, 2:] = rng.integers(0, 256, (nblk, 16), dtype=np.uint8)
    blk[:, :2] = codecs.single_to_half(scale).view(np.uint8).reshape(-1, 2)
    return blk.reshape(-1)


def rel_err(y, ref):
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
    return float(np.max(np.abs(y.astype(np.float64) - ref))) / max(rms, 1e-30)


@pytest.mark.parametrize("ggml_type", [codecs.GGML_Q8_0, codecs.GGML_Q4_0])
@pytest.mark.parametrize("kn", LINEAR_SHAPES)
def test_linear_sweep_shapes(backend, ggml_type, kn):
    k, n = kn
    blk = make_blocks(ggml_type, n, k, seed=k + n)
    w = codecs.dequantize(ggml_type, blk).reshape(n, k)
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_quant(ggml_type, blk, n, k)
    try:
        rng = np.random.default_rng(7)
        for b in LINEAR_BATCHES:
            x = rng.standard_normal((b, k)).astype(np.float32)
            lin.compute_quant(x)
            y = lin.finish_and_load_result()
            ref = codecs.linear_fp32(w, x)
            assert y.shape == (b, n)
            assert rel_err(y, ref) < (TOL if b <= 8 else TOL_TC), (ggml_type, kn, b, rel_err(y, ref))
    finally:
        lin.unprepare_for_compute()


@pytest.mark.parametrize("ggml_type", [codecs.GGML_Q8_0, codecs.GGML_Q4_0])
@pytest.mark.parametrize("n,k", [(1, 32), (2, 64), (37, 96), (129, 1024), (1000, 2080), (5, 27648)])
@pytest.mark.parametrize("b", [1, 2, 3, 5, 7, 8, 9, 17, 33, 64])
def test_ragged_shapes_and_batches(backend, ggml_type, n, k, b):
    blk = make_blocks(ggml_type, n, k, seed=n * 7 + k)
    w = codecs.dequantize(ggml_type, blk).reshape(n, k)
    rng = np.random.default_rng(b)
    x = rng.standard_normal((b, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_quant(ggml_type, blk, n, k, bias=bias)
    try:
        lin.compute_quant(x)
        y = lin.finish_and_load_result()
        ref = codecs.linear_fp32(w, x, bias)
        assert rel_err(y, ref) < (TOL if b <= 8 else TOL_TC)
    finally:
        lin.unprepare_for_compute()


@pytest.mark.parametrize("ggml_type", [codecs.GGML_Q8_0, codecs.GGML_Q4_0])
@pytest.mark.parametrize("b", [1, 3, 8, 16, 40])
def test_forced_tensor_core_path_any_batch(backend, ggml_type, b):
    """cai_linear_set_path(2): the tcgen05 GEMM for every batch it accepts, ragged N and a half K chunk."""
    n, k = 300, 1056
    blk = make_blocks(ggml_type, n, k, seed=5)
    w = codecs.dequantize(ggml_type, blk).reshape(n, k)
    rng = np.random.default_rng(b)
    x = (rng.standard_normal((b, k)) * rng.uniform(1e-3, 1e3, (b, 1))).astype(np.float32)     # rows of very different scale
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_quant(ggml_type, blk, n, k)
    try:
        lin.set_path(2)
        before = backend.launch_count()
        lin.compute_quant(x)
        assert backend.launch_count() - before in (2, 3)     # activation split + GEMM (+ the sum over K ranges)
        y = lin.finish_and_load_result()
        ref = x.astype(np.float64) @ w.astype(np.float64).T
        for i in range(b):                                   # per row: each has its own scale
            assert rel_err(y[i], ref[i]) < TOL_TC
    finally:
        lin.unprepare_for_compute()


@pytest.mark.parametrize("act", [0, 1, 2, 3])
def test_fused_bias_and_activation_opcodes(backend, act):
    """Opcodes of the reference's fused epilogue: 1 ReLU, 2 sigmoid, 3 tanh."""
    n, k = 200, 256
    blk = make_blocks(codecs.GGML_Q8_0, n, k, seed=11)
    w = codecs.dequantize_q8_0(blk).reshape(n, k) * np.float32(0.02)
    rng = np.random.default_rng(12)
    x = (rng.standard_normal((2, k)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32) * np.float32(0.1)
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_quant(codecs.GGML_Q8_0, blk, n, k, bias=bias)
    try:
        lin.compute_quant(x, act=act)
        y = lin.finish_and_load_result()
        pre = codecs.linear_fp32(codecs.dequantize_q8_0(blk).reshape(n, k), x, bias).astype(np.float64)
        ref = {0: pre, 1: np.maximum(pre, 0), 2: 1 / (1 + np.exp(-pre)), 3: np.tanh(pre)}[act]
        assert np.max(np.abs(y - ref)) < 1e-4
    finally:
        lin.unprepare_for_compute()


@pytest.mark.parametrize("ggml_type,k", [(codecs.GGML_F32, 8), (codecs.GGML_F32, 5), (codecs.GGML_F16, 12), (codecs.GGML_F32, 896)])
def test_unquantized_weights_any_width(backend, ggml_type, k):
    n = 13
    rng = np.random.default_rng(k)
    w = rng.standard_normal((n, k)).astype(np.float32)
    if ggml_type == codecs.GGML_F16:
        data = w.astype(np.float16)
        w = data.astype(np.float32)
        data = data.view(np.uint8)
    else:
        data = w
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_quant(ggml_type, data, n, k)
    try:
        for b in (1, 3, 6):
            x = rng.standard_normal((b, k)).astype(np.float32)
            lin.compute_quant(x)
            assert rel_err(lin.finish_and_load_result(), codecs.linear_fp32(w, x)) < TOL
    finally:
        lin.unprepare_for_compute()


def test_device_resident_chaining(backend):
    """The output buffer of one layer feeds the next without a host round trip
    (the pExternalVBs / ResultBuffer residency of the reference's OpenCL backend)."""
    k, mid, n = 256, 512, 96
    b1 = make_blocks(codecs.GGML_Q8_0, mid, k, seed=1)
    b2 = make_blocks(codecs.GGML_Q4_0, n, mid, seed=2)
    w1 = codecs.dequantize_q8_0(b1).reshape(mid, k)
    w2 = codecs.dequantize_q4_0(b2).reshape(n, mid)
    l1, l2 = DotProductSharedKernel(backend), DotProductSharedKernel(backend)
    l1.prepare_for_compute_quant(codecs.GGML_Q8_0, b1, mid, k)
    l2.prepare_for_compute_quant(codecs.GGML_Q4_0, b2, n, mid)
    try:
        x = np.random.default_rng(3).standard_normal((2, k)).astype(np.float32)
        dx = backend.to_device(x)
        before = backend.launch_count()
        l1.compute_quant(dx, batch=2)
        l2.compute_quant(l1.result_buffer, batch=2)
        assert backend.launch_count() - before == 2
        y = l2.finish_and_load_result()
        ref = codecs.linear_fp32(w2, codecs.linear_fp32(w1, x))
        assert rel_err(y, ref) < 1e-4
        dx.free()
    finally:
        l1.unprepare_for_compute()
        l2.unprepare_for_compute()


def test_errors_are_statuses_not_crashes(backend):
    from neural_api_b200.backend import CaiError
    lin = DotProductSharedKernel(backend)
    with pytest.raises(CaiError, match="multiple of 32"):
        lin.prepare_for_compute_quant(codecs.GGML_Q8_0, np.zeros(34, dtype=np.uint8), 1, 33)
    with pytest.raises(CaiError, match="not supported"):
        lin.prepare_for_compute_quant(30, np.zeros(64, dtype=np.uint8), 1, 32)     # BF16: no reader decodes it
    with pytest.raises(CaiError, match="whole super-blocks"):
        lin.prepare_for_compute_quant(12, np.zeros(144, dtype=np.uint8), 1, 32)    # Q4_K rows are super-blocks of 256
    with pytest.raises(CaiError):
        backend.alloc(1 << 50)                                                     # rejected before cudaMalloc
