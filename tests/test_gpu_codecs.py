"""Bit-exact block dequantization on the GPU (through the resident, repacked layout)
against the oracle and the reference's GGUF fixtures."""
import numpy as np
import pytest

from conftest import load_golden
from oracle import codecs
from neural_api_b200.backend import DotProductSharedKernel

pytestmark = pytest.mark.gpu


def _random_blocks(ggml_type, rows, cols, seed):
    rng = np.random.default_rng(seed)
    nblk = rows * cols // 32
    scale = rng.uniform(0.001, 0.05, nblk).astype(np.float32)
    if ggml_type == codecs.GGML_Q8_0:
        blk = np.empty((nblk, 34), dtype=np.uint8)
        blk[:, 2:] = rng.integers(-127, 128, (nblk, 32)).astype(np.int8).view(np.uint8)
    else:
        blk = np.empty((nblk, 18), dtype=np.uint8)
        blk[:, 2:] = rng.integers(0, 256, (nblk, 16)).astype(np.uint8)
    blk[:, :2] = codecs.single_to_half(scale).view(np.uint8).reshape(-1, 2)
    return blk.reshape(-1)


@pytest.mark.parametrize("ggml_type", [codecs.GGML_Q8_0, codecs.GGML_Q4_0])
@pytest.mark.parametrize("shape", [(1, 32), (3, 96), (64, 896), (257, 4096)])
def test_dequantize_bit_exact(backend, ggml_type, shape):
    rows, cols = shape
    blk = _random_blocks(ggml_type, rows, cols, seed=rows * 1000 + cols)
    got = backend.dequantize(ggml_type, blk, rows, cols)
    want = codecs.dequantize(ggml_type, blk)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequantize_every_half_scale_bit_pattern(backend):
    """Subnormal, zero and huge block scales decode exactly (NeuralHalfToSingle)."""
    bits = np.arange(65536, dtype=np.uint16)
    finite = bits[((bits >> 10) & 0x1F) != 0x1F]
    nblk = finite.size
    blk = np.empty((nblk, 34), dtype=np.uint8)
    blk[:, :2] = finite.view(np.uint8).reshape(-1, 2)
    blk[:, 2:] = np.tile(np.arange(-16, 16, dtype=np.int8).view(np.uint8), (nblk, 1))
    got = backend.dequantize(codecs.GGML_Q8_0, blk.reshape(-1), nblk, 32)
    want = codecs.dequantize_q8_0(blk.reshape(-1))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_f16_and_f32_pass_through(backend):
    rng = np.random.default_rng(5)
    w = rng.standard_normal((7, 24)).astype(np.float32)
    got = backend.dequantize(codecs.GGML_F32, w, 7, 24)
    assert np.array_equal(got, w.reshape(-1))
    h = w.astype(np.float16)
    got = backend.dequantize(codecs.GGML_F16, h.view(np.uint8), 7, 24)
    assert np.array_equal(got, h.astype(np.float32).reshape(-1))


def test_reference_gguf_fixtures_decode_bit_exact(backend):
    for fixture in ("tiny_llama_q8_gguf", "tiny_llama_f16_gguf"):
        z = load_golden(fixture)
        for k in z.files:
            if not k.startswith("raw::"):
                continue
            name = k[5:]
            ty, rows, cols = (int(v) for v in z["meta::" + name])
            got = backend.dequantize(ty, z[k], rows, cols)
            assert np.array_equal(got.view(np.uint32), z["deq::" + name].view(np.uint32)), (fixture, name)


def test_q4_0_known_answer_block(backend):
    k = load_golden("kats")
    got = backend.dequantize(codecs.GGML_Q4_0, k["q4_0_block"], 1, 32)
    assert np.array_equal(got, k["q4_0_expect"])


@pytest.mark.parametrize("ggml_type", [codecs.GGML_Q8_0, codecs.GGML_Q4_0])
def test_resident_linear_weights_dequantize_bit_exact(backend, ggml_type):
    rows, cols = 300, 1792
    blk = _random_blocks(ggml_type, rows, cols, seed=9)
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_quant(ggml_type, blk, rows, cols)
    try:
        got = lin.dequantize_weights()
        want = codecs.dequantize(ggml_type, blk).reshape(rows, cols)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        assert lin.weight_bytes() == blk.size
    finally:
        lin.unprepare_for_compute()
