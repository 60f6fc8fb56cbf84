"""The C (AVX2 + OpenMP) restatement of the reference CPU path against the numpy oracle
and the reference's Q8_0 GGUF fixture (no GPU)."""
import json

import numpy as np
import pytest

from conftest import load_golden
from oracle import c_oracle, codecs
from oracle.forward import LlamaConfig, OracleModel, OracleSession

NAME_KIND = {
    "input_layernorm.weight": "attn_norm", "post_attention_layernorm.weight": "ffn_norm",
    "self_attn.q_proj.weight": "q", "self_attn.k_proj.weight": "k", "self_attn.v_proj.weight": "v",
    "self_attn.o_proj.weight": "o", "mlp.up_proj.weight": "up", "mlp.gate_proj.weight": "gate",
    "mlp.down_proj.weight": "down",
}


@pytest.mark.parametrize("ggml_type,quant", [(codecs.GGML_Q8_0, codecs.quantize_q8_0), (codecs.GGML_Q4_0, codecs.quantize_q4_0)])
def test_gemv_and_dequantize(ggml_type, quant):
    rng = np.random.default_rng(0)
    n, k = 77, 896
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    blk = quant(w)
    deq = codecs.dequantize(ggml_type, blk)
    assert np.array_equal(c_oracle.dequantize(ggml_type, blk, n * k).view(np.uint32), deq.view(np.uint32))
    x = rng.standard_normal((3, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    y = c_oracle.gemv(ggml_type, blk, n, k, x, bias)
    ref = codecs.linear_fp32(deq.reshape(n, k), x, bias)
    assert np.max(np.abs(y - ref)) < 2e-5 * np.sqrt(np.mean(ref ** 2)) + 1e-6


def test_forward_on_the_reference_q8_gguf_fixture():
    z = load_golden("tiny_llama_q8_gguf")
    cfgj = json.loads(bytes(z["config_json"]).decode())
    cfg = LlamaConfig.from_hf(cfgj)
    cm = c_oracle.CModel(cfg.hidden, cfg.inter, cfg.layers, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.vocab,
                         cfg.rms_eps, cfg.rope_theta, tie_embeddings=cfg.tie_embeddings)
    tensors = {}
    for key in z.files:
        if not key.startswith("raw::"):
            continue
        name = key[5:]
        ty, rows, cols = (int(v) for v in z["meta::" + name])
        w = codecs.dequantize(ty, z[key])
        tensors[name] = w.reshape(rows, cols) if rows > 1 else w
        data = z[key] if ty != codecs.GGML_F32 else z[key].view(np.float32)
        if name == "model.embed_tokens.weight":
            cm.set_tensor("embed", 0, ty, data)
        elif name == "model.norm.weight":
            cm.set_tensor("final_norm", 0, ty, data)
        else:
            parts = name.split(".", 3)
            cm.set_tensor(NAME_KIND[parts[3]], int(parts[2]), ty, data)
    oracle = OracleModel.from_hf_tensors(cfg, tensors, interleave=False)
    cs = c_oracle.CSession(cm, 12)
    os_ = OracleSession(oracle, 12)
    try:
        for i, t in enumerate([1, 5, 2, 7, 0, 3, 6, 4, 2, 1]):
            a = cs.step(t, i)
            b = os_.step(t, i)
            assert np.max(np.abs(a - b)) < 1e-5
    finally:
        cs.close()
        cm.close()


def test_thread_count_is_reported():
    assert c_oracle.num_threads() >= 1
