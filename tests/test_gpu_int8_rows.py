"""The reference's own int8 weight format on the GPU: int8 codes [N][K] with one fp32 scale per output row
(TNNetVolume.QuantizeInt8 / DotProductsTiledInt8, neural/neuralvolume.pas:12471-12562, 12693-12745): the device
quantizer, the linear layer, and whole models that run on int8 rows."""
import numpy as np
import pytest

from neural_api_b200.backend import (DotProductSharedKernel, LlamaModel, StreamingDecoder, make_config, TYPE_F32, TYPE_I8ROW)
from oracle import codecs
from oracle.forward import LlamaConfig, OracleModel, OracleSession, argmax_first

pytestmark = pytest.mark.gpu


def test_device_int8_row_quantizer_equals_the_oracle(backend):
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((70, 640)) * 0.05).astype(np.float32)
    w[3] = 0.0                                                    # all-zero row
    w[4, :6] = [np.nan, np.inf, -np.inf, 3.0, -1.5, 1e-30]
    w[5] = 0.0
    w[5, :3] = [1e-40, -5e-41, 2.5e-41]                           # denormal row maximum
    w[6, :4] = [127.0, 0.5, 1.5, -2.5]                            # exact half-way points: round half to even
    codes, scales = backend.quantize_int8_rows(w)
    ref_codes, ref_scales = codecs.quantize_int8_rows(w)
    assert np.array_equal(scales.view(np.uint32), ref_scales.view(np.uint32))
    assert np.array_equal(codes, ref_codes)


@pytest.mark.parametrize("k,n", [(896, 4864), (5120, 1024), (4864, 896), (80, 33)])
@pytest.mark.parametrize("batch", [1, 2, 4, 16, 64])
def test_int8_row_linear_matches_the_oracle(backend, k, n, batch):
    rng = np.random.default_rng(k + n + batch)
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    codes, scales = codecs.quantize_int8_rows(w)
    bias = rng.standard_normal(n).astype(np.float32) if n == 1024 else None
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_int8(codes, scales, n, k, bias=bias)
    try:
        assert np.array_equal(lin.dequantize_weights().view(np.uint32), codecs.dequantize_int8_rows(codes, scales).view(np.uint32))
        assert lin.weight_bytes() == n * k + 4 * n                # 1 byte per weight + one scale per row
        x = rng.standard_normal((batch, k)).astype(np.float32)
        lin.compute_quant(x)
        y = lin.finish_and_load_result()
        ref = codecs.linear_int8_rows(codes, scales, x, bias)
        rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
        assert float(np.max(np.abs(y - ref))) < 2e-5 * rms
        if batch == 1:
            lin.compute_quant(x, act=1)                            # ReLU opcode of cai_dot_product_int8
            assert float(np.max(np.abs(lin.finish_and_load_result() - np.maximum(ref, 0)))) < 2e-5 * rms
    finally:
        lin.unprepare_for_compute()


def _hf_tensors(kw, rng, std=0.05):
    H, I, V = kw["hidden"], kw["inter"], kw["vocab"]
    qw, kvw = kw["heads"] * kw["head_dim"], kw["kv_heads"] * kw["head_dim"]
    t = {"model.embed_tokens.weight": (V, H), "lm_head.weight": (V, H)}
    for l in range(kw["layers"]):
        p = "model.layers.%d." % l
        t.update({p + "self_attn.q_proj.weight": (qw, H), p + "self_attn.k_proj.weight": (kvw, H), p + "self_attn.v_proj.weight": (kvw, H),
                  p + "self_attn.o_proj.weight": (H, qw), p + "mlp.gate_proj.weight": (I, H), p + "mlp.up_proj.weight": (I, H),
                  p + "mlp.down_proj.weight": (H, I)})
    tensors = {n: (rng.standard_normal(s) * std).astype(np.float32) for n, s in t.items()}
    tensors["model.norm.weight"] = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    for l in range(kw["layers"]):
        p = "model.layers.%d." % l
        tensors[p + "input_layernorm.weight"] = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
        tensors[p + "post_attention_layernorm.weight"] = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    return tensors


def test_model_quantized_to_int8_rows_on_upload_matches_the_oracle(backend):
    """The importer's pQuantizeInt8 route: F32 checkpoint tensors, stored as int8 rows while they are uploaded. The oracle
    quantizes the same tensors with its own QuantizeInt8 and runs on the dequantized rows: logits within 1e-3 of the
    logit RMS and the same greedy tokens; against the unquantized model the drift stays inside the reference's 5e-2
    band (tests/TestNeuralPretrained.pas:4512-4517)."""
    kw = dict(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=640, rms_eps=1e-6, rope_theta=1e4)
    rng = np.random.default_rng(3)
    tensors = _hf_tensors(kw, rng)
    cfg = LlamaConfig(**kw)
    model = LlamaModel(backend, make_config(**kw))
    model.set_int8_weights(True)
    model.upload_hf_tensors(tensors, interleave=True)
    model.finalize()
    q_tensors = {}
    for name, w in tensors.items():
        if w.ndim == 2:
            c, s = codecs.quantize_int8_rows(w)
            q_tensors[name] = codecs.dequantize_int8_rows(c, s)
        else:
            q_tensors[name] = w
    oracle = OracleModel.from_hf_tensors(cfg, q_tensors, interleave=True)
    exact = OracleModel.from_hf_tensors(cfg, tensors, interleave=True)
    # the resident rows are the oracle's rows, byte for byte (rows are quantized before the q/k row permutation moves them)
    buf, ty, rows, cols = model.read_tensor("model.layers.1.mlp.down_proj.weight", 1 << 22)
    assert ty == TYPE_I8ROW
    c_dev, s_dev = codecs.split_int8_rows(buf, rows, cols)
    c_ref, s_ref = codecs.quantize_int8_rows(tensors["model.layers.1.mlp.down_proj.weight"])
    assert np.array_equal(c_dev, c_ref) and np.array_equal(s_dev.view(np.uint32), s_ref.view(np.uint32))
    sess = StreamingDecoder(model, 48)
    osess, esess = OracleSession(oracle, 48), OracleSession(exact, 48)
    try:
        assert not sess.uses_step_kernel                            # the persistent step kernel covers Q8_0 blocks only
        tok = 7
        worst = drift = 0.0
        for _ in range(24):
            logits, amax = sess.step_forward([tok])
            ref = osess.step(tok)
            ex = esess.step(tok)
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            worst = max(worst, float(np.max(np.abs(logits[0] - ref))) / rms)
            drift = max(drift, float(np.max(np.abs(logits[0] - ex))) / float(np.max(np.abs(ex))))
            assert int(amax[0]) == argmax_first(ref)
            tok = int(amax[0])
        assert worst < 1e-3, worst
        assert drift < 5e-2, drift
    finally:
        sess.close()
        model.close()


def test_synthetic_int8_row_model_matches_the_oracle(backend):
    kw = dict(hidden=512, inter=1024, layers=2, heads=8, kv_heads=2, head_dim=64, vocab=1024, rms_eps=1e-6, rope_theta=1e6,
              tie_embeddings=True, qkv_bias=True)
    model = LlamaModel(backend, make_config(**kw))
    model.init_synthetic(TYPE_I8ROW, seed=4, std=0.02)
    model.finalize()
    cfg = LlamaConfig(**kw)
    names = ["model.embed_tokens.weight", "model.norm.weight"]
    for l in range(kw["layers"]):
        p = "model.layers.%d." % l
        names += [p + s for s in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                                  "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight", "mlp.gate_proj.weight",
                                  "mlp.up_proj.weight", "mlp.down_proj.weight", "self_attn.q_proj.bias", "self_attn.k_proj.bias",
                                  "self_attn.v_proj.bias")]
    tensors = {}
    for n in names:
        buf, ty, rows, cols = model.read_tensor(n, 1 << 22)
        if ty == TYPE_I8ROW:
            c, s = codecs.split_int8_rows(buf, rows, cols)
            tensors[n] = codecs.dequantize_int8_rows(c, s)
        else:
            w = codecs.dequantize(ty, buf[:rows * codecs.block_bytes_per_row(ty, cols)])
            tensors[n] = w.reshape(rows, cols) if rows > 1 else w
    oracle = OracleModel.from_hf_tensors(cfg, tensors, interleave=False)
    batch = 3
    sess = StreamingDecoder(model, 40, batch=batch)
    osess = [OracleSession(oracle, 40) for _ in range(batch)]
    rng = np.random.default_rng(9)
    tok = rng.integers(0, kw["vocab"], batch).astype(np.int32)
    try:
        worst = 0.0
        for _ in range(12):
            logits, amax = sess.step_forward(tok)
            nxt = np.empty(batch, dtype=np.int32)
            for b in range(batch):
                ref = osess[b].step(int(tok[b]))
                rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
                worst = max(worst, float(np.max(np.abs(logits[b] - ref))) / rms)
                nxt[b] = argmax_first(ref)
            assert np.array_equal(amax, nxt)
            tok = nxt
        assert worst < 1e-3, worst
    finally:
        sess.close()
        model.close()
