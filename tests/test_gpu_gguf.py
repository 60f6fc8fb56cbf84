"""GGUF files through the library on the GPU: the device block decoders bit for bit against the reference's K-quant
fixture, the `gguf` package and the CPU restatement; whole files (the reference's own pico checkpoints and a
hand-written K-quant / legacy-quant qwen2 file) from path to logits."""
import numpy as np
import pytest

import gguf_util as W
from conftest import load_golden
from oracle import gguf_file as GF
from oracle.forward import LlamaConfig, OracleModel, OracleSession
from neural_api_b200.backend import CaiError, DotProductSharedKernel, GGUFReader, LlamaModel, StreamingDecoder

pytestmark = pytest.mark.gpu

ALL_TYPES = (2, 3, 6, 7, 8, 10, 11, 12, 13, 14)


def _fixture(tmp_path, name):
    z = load_golden("gguf_files")
    p = tmp_path / name
    p.write_bytes(bytes(z["file::" + name]))
    return p


@pytest.mark.parametrize("t", ALL_TYPES)
def test_device_decoders_are_bit_exact(backend, t):
    z = load_golden("block_kats")
    raw, want = z["raw::%d" % t], z["deq::%d" % t]
    got = backend.gguf_decode(t, raw, want.size)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    assert np.array_equal(got.view(np.uint32), GF.decode_span(t, raw).view(np.uint32))
    # the codec hook takes the same types
    be = GF.BLOCK[t][1]
    got2 = backend.dequantize(t, raw, want.size // be // 4, be * 4)
    assert np.array_equal(got2.view(np.uint32), want.view(np.uint32))


def test_device_decode_covers_raw_types_and_long_spans(backend):
    rng = np.random.default_rng(5)
    x = rng.standard_normal(1000).astype(np.float32)
    assert np.array_equal(backend.gguf_decode(0, x.view(np.uint8), 1000), x)
    h = rng.integers(0, 1 << 16, 70000, dtype=np.uint16)
    h = h[(h & 0x7C00) != 0x7C00]                                       # every finite half, subnormals included
    assert np.array_equal(backend.gguf_decode(1, h.view(np.uint8), h.size).view(np.uint32),
                          GF.decode_span(1, h.view(np.uint8)).view(np.uint32))
    # more elements than one staged chunk (8 Mi): the chunk seam must fall on a block boundary
    nb = (9 << 20) // 256
    raw = rng.integers(0, 256, (nb, 144), dtype=np.uint8)
    raw[:, 0:2] = np.asarray(rng.standard_normal(nb) * 0.01, dtype=np.float16).view(np.uint8).reshape(nb, 2)
    raw[:, 2:4] = np.asarray(rng.standard_normal(nb) * 0.01, dtype=np.float16).view(np.uint8).reshape(nb, 2)
    got = backend.gguf_decode(12, raw.reshape(-1), nb * 256)
    assert np.array_equal(got.view(np.uint32), GF.dequantize_q4_k(raw.reshape(-1)).view(np.uint32))
    with pytest.raises(CaiError):
        backend.gguf_decode(12, raw.reshape(-1), 100)                   # not a whole number of super-blocks
    with pytest.raises(CaiError):
        backend.gguf_decode(30, raw.reshape(-1), 256)                   # BF16: no decoder in the reference's reader either


def test_kquant_fixture_of_the_reference(backend, tmp_path):
    """TestGGUFKQuantDecodeParity (tests/TestNeuralPretrained.pas:5931-6020): LoadTensorFlat of every tensor of
    tiny_kquant.gguf equals the JSON reference dequantisation (bit for bit here; the reference gates at 1e-6)."""
    z = load_golden("gguf_files")
    r = GGUFReader(_fixture(tmp_path, "tiny_kquant.gguf"))
    try:
        for tname, tid in (("Q4_K", 12), ("Q5_K", 13), ("Q6_K", 14), ("Q2_K", 10)):
            idx = r.find_tensor("kq.%s.weight" % tname)
            assert r.tensor_info(idx)[1] == tid
            x = r.load_tensor(backend, "kq.%s.weight" % tname)
            assert x.shape == (1024,)
            assert np.array_equal(x.view(np.uint32), z["kquant::" + tname].view(np.uint32)), tname
        ref = r.load_tensor(backend, "ref.f32.weight")
        assert ref.shape == (4, 256) and np.array_equal(ref.reshape(-1), z["kquant::ref_f32"])
    finally:
        r.close()


def test_f32_checkpoint_file_reproduces_the_golden_logits(backend, tmp_path):
    """tiny_llama_f32.gguf is the GGUF twin of the pico Llama checkpoint (tests/TestNeuralPretrained.pas:5827-5918):
    loaded from the FILE by the library it must meet the reference's end-to-end gate of 1e-4 on the golden logits."""
    z = load_golden("gguf_files")
    model = LlamaModel.from_gguf(backend, _fixture(tmp_path, "tiny_llama_f32.gguf"))
    assert model.max_positions == 16 and model.cfg.vocab == 11 and model.cfg.tie_embeddings == 0
    sess = StreamingDecoder(model, 16)
    try:
        worst = 0.0
        for s, g in zip(z["tiny_llama::sequences"], z["tiny_llama::logits"]):
            sess.reset()
            for i, t in enumerate(s):
                logits, _ = sess.step_forward([int(t)], [i])
                worst = max(worst, float(np.max(np.abs(logits[0] - g[i]))))
        assert worst < 1e-4, worst
    finally:
        sess.close()
        model.close()


def test_f16_checkpoint_file_stays_in_the_reference_band(backend, tmp_path):
    """The F16 twin: drift below 3e-3 of max |logit| (tests/TestNeuralPretrained.pas:6312-6335)."""
    z = load_golden("gguf_files")
    model = LlamaModel.from_gguf(backend, _fixture(tmp_path, "tiny_llama_f16.gguf"))
    sess = StreamingDecoder(model, 16)
    try:
        drift, mx = 0.0, 0.0
        for s, g in zip(z["tiny_llama::sequences"], z["tiny_llama::logits"]):
            sess.reset()
            for i, t in enumerate(s):
                logits, _ = sess.step_forward([int(t)], [i])
                drift = max(drift, float(np.max(np.abs(logits[0] - g[i]))))
                mx = max(mx, float(np.max(np.abs(g[i]))))
        assert drift / mx < 3e-3
    finally:
        sess.close()
        model.close()


def _oracle_of_file(path):
    g = GF.GGUFFile(path)
    c = GF.llama_config(g)
    cfg = LlamaConfig(hidden=c["hidden"], inter=c["inter"], layers=c["layers"], heads=c["heads"], kv_heads=c["kv_heads"],
                      head_dim=c["head_dim"], vocab=c["vocab"], rms_eps=float(np.float32(c["rms_eps"])),
                      rope_theta=float(np.float32(c["rope_theta"])), tie_embeddings=bool(c["tie_embeddings"]),
                      qkv_bias=bool(c["qkv_bias"]))
    tensors = {}
    for n in g.order:
        hf = GF.hf_name(n)
        if hf is not None:
            tensors[hf] = g.load(n)
    return cfg, OracleModel.from_hf_tensors(cfg, tensors, interleave=False)


def test_q8_checkpoint_file_equals_the_oracle_on_the_same_blocks(backend, tmp_path):
    p = _fixture(tmp_path, "tiny_llama_q8.gguf")
    cfg, oracle = _oracle_of_file(p)
    model = LlamaModel.from_gguf(backend, p)
    sess, osess = StreamingDecoder(model, 12), OracleSession(oracle, 12)
    try:
        for t in [1, 5, 2, 7, 0, 3, 6, 4, 2, 1]:
            logits, _ = sess.step_forward([t])
            ref = osess.step(t)
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            assert np.max(np.abs(logits[0] - ref)) < 1e-4 * max(rms, 1.0)
    finally:
        sess.close()
        model.close()


def _random_blocks(rng, gtype, n_elems, scale):
    bb, be = GF.BLOCK[gtype]
    nb = n_elems // be
    if gtype == 0:
        return (rng.standard_normal(n_elems) * scale).astype(np.float32).view(np.uint8)
    if gtype == 1:
        return (rng.standard_normal(n_elems) * scale).astype(np.float16).view(np.uint8)
    raw = rng.integers(0, 256, (nb, bb), dtype=np.uint8)
    # per-format scale so that the decoded weights have a spread near `scale`
    spread = {2: 8, 3: 8, 6: 16, 7: 16, 8: 74, 10: 30, 11: 60, 12: 300, 13: 600, 14: 1200}[gtype]
    for off in {2: [0], 3: [0, 2], 6: [0], 7: [0, 2], 8: [0], 10: [80, 82], 11: [108], 12: [0, 2], 13: [0, 2], 14: [208]}[gtype]:
        d = np.abs(rng.standard_normal(nb)) * scale / spread + scale / spread / 4
        raw[:, off:off + 2] = d.astype(np.float16).view(np.uint8).reshape(nb, 2)
    return raw.reshape(-1)


def _kquant_qwen2_file(path, seed=11):
    """A two-layer qwen2 file whose matrices use every load-time format; rows of 256 columns so that K-quants fit."""
    rng = np.random.default_rng(seed)
    H, I, L, NH, NKV, V = 256, 512, 3, 4, 2, 96
    hd = H // NH
    tensors = [("token_embd.weight", [H, V], 12, _random_blocks(rng, 12, V * H, 0.05)),
               ("output_norm.weight", [H], 1, (1 + 0.1 * rng.standard_normal(H)).astype(np.float16).view(np.uint8)),
               ("output.weight", [H, V], 14, _random_blocks(rng, 14, V * H, 0.05)),
               ("rope_freqs.weight", [hd // 2], 0, np.ones(hd // 2, np.float32))]      # present in llama.cpp files, unused
    kinds = [("attn_q.weight", [H, NH * hd], 13), ("attn_k.weight", [H, NKV * hd], 10), ("attn_v.weight", [H, NKV * hd], 11),
             ("attn_output.weight", [NH * hd, H], 3), ("ffn_gate.weight", [H, I], 6), ("ffn_up.weight", [H, I], 7),
             ("ffn_down.weight", [I, H], 12)]
    for l in range(L):
        pre = "blk.%d." % l
        for i, (n, dims, t) in enumerate(kinds):
            if l == 1:                                   # second layer: rotate the formats, add the directly resident ones
                t = [14, 8, 2, 12, 13, 10, 11][i]
            if l == 2:                                   # third layer: whole groups in one resident K-quant (fused q|k|v and up|gate)
                t = [14, 14, 14, 13, 13, 13, 12][i]
            tensors.append((pre + n, dims, t, _random_blocks(rng, t, dims[0] * dims[1], 0.04)))
        for n, width in (("attn_q.bias", NH * hd), ("attn_k.bias", NKV * hd), ("attn_v.bias", NKV * hd)):
            tensors.append((pre + n, [width], 0, (0.1 * rng.standard_normal(width)).astype(np.float32)))
        tensors.append((pre + "attn_norm.weight", [H], 0, (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)))
        tensors.append((pre + "ffn_norm.weight", [H], 0, (1 + 0.1 * rng.standard_normal(H)).astype(np.float32)))
    W.write(path, W.llama_meta("qwen2", H, I, L, NH, NKV, 64, eps=1e-6, theta=1000000.0), tensors)


def test_kquant_and_legacy_formats_from_file_to_logits(backend, tmp_path):
    p = tmp_path / "kq_qwen2.gguf"
    _kquant_qwen2_file(p)
    cfg, oracle = _oracle_of_file(p)
    assert cfg.qkv_bias and not cfg.tie_embeddings
    model = LlamaModel.from_gguf(backend, p)
    sess, osess = StreamingDecoder(model, 32), OracleSession(oracle, 32)
    try:
        rng = np.random.default_rng(3)
        for t in rng.integers(0, cfg.vocab, 20):
            logits, _ = sess.step_forward([int(t)])
            ref = osess.step(int(t))
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            assert np.all(np.isfinite(logits))
            assert np.max(np.abs(logits[0] - ref)) < 1e-3 * max(rms, 1.0)
        # the load-time formats are resident as F32, bit-equal to the reader's decode (one of each family)
        for hf, rows, cols in (("model.layers.0.self_attn.o_proj.weight", 256, 256), ("model.layers.1.mlp.down_proj.weight", 256, 512),
                               ("model.layers.0.self_attn.k_proj.weight", 128, 256), ("model.layers.1.mlp.up_proj.weight", 512, 256)):
            buf, ty, r, c = model.read_tensor(hf, rows * cols * 4)
            assert (ty, r, c) == (0, rows, cols)
            assert np.array_equal(buf[:rows * cols * 4].view(np.float32).reshape(rows, cols), oracle_tensor(p, hf))
        # Q4_K / Q5_K / Q6_K stay resident as the file's own super-blocks
        g = GF.GGUFFile(p)
        # ... also as members of a [q|k|v] or [up|gate] group whose formats differ (layer 1: q Q6_K, k Q8_0, v Q4_0;
        # gate Q5_K beside an up matrix decoded from Q2_K): such a group is kept as separate matrices
        for name, hf, tid in (("blk.0.ffn_down.weight", "model.layers.0.mlp.down_proj.weight", 12),
                              ("blk.2.attn_output.weight", "model.layers.2.self_attn.o_proj.weight", 13),
                              ("blk.0.attn_q.weight", "model.layers.0.self_attn.q_proj.weight", 13),
                              ("blk.1.attn_q.weight", "model.layers.1.self_attn.q_proj.weight", 14),
                              ("blk.1.attn_k.weight", "model.layers.1.self_attn.k_proj.weight", 8),
                              ("blk.1.attn_v.weight", "model.layers.1.self_attn.v_proj.weight", 2),
                              ("blk.1.ffn_gate.weight", "model.layers.1.mlp.gate_proj.weight", 13),
                              ("blk.2.ffn_up.weight", "model.layers.2.mlp.up_proj.weight", 13),
                              ("output.weight", "lm_head.weight", 14)):
            raw = g.raw(name)
            buf, ty, r, c = model.read_tensor(hf, raw.size)
            assert ty == tid and np.array_equal(buf[:raw.size], raw)
    finally:
        sess.close()
        model.close()


def oracle_tensor(path, hf):
    g = GF.GGUFFile(path)
    for n in g.order:
        if GF.hf_name(n) == hf:
            return g.load(n)
    raise KeyError(hf)


def test_int8_switch_on_a_kquant_file(backend, tmp_path):
    """pQuantizeInt8 on a K-quant file: the decoded fp32 rows are re-quantized to int8 rows; logits stay within the
    reference's int8 drift gate (5e-2 of max |logit|, tests/TestNeuralPretrained.pas:4465-4525) of the fp32 load."""
    p = tmp_path / "kq_qwen2.gguf"
    _kquant_qwen2_file(p)
    m32 = LlamaModel.from_gguf(backend, p)
    m8 = LlamaModel.from_gguf(backend, p, quantize_int8=True)
    s32, s8 = StreamingDecoder(m32, 16), StreamingDecoder(m8, 16)
    try:
        _, ty, _, _ = m8.read_tensor("model.layers.0.mlp.down_proj.weight", 1 << 20)
        assert ty == 124
        drift, mx = 0.0, 0.0
        for t in (3, 50, 7, 91, 20, 64):
            a, _ = s32.step_forward([t])
            b, _ = s8.step_forward([t])
            drift = max(drift, float(np.max(np.abs(a - b))))
            mx = max(mx, float(np.max(np.abs(a))))
        assert 0 < drift / mx < 5e-2
    finally:
        s32.close(); s8.close(); m32.close(); m8.close()


@pytest.mark.parametrize("gtype", [12, 13, 14, 11, 7])
@pytest.mark.parametrize("batch", [1, 3, 6])
def test_linear_layer_from_kquant_blocks(backend, gtype, batch):
    """cai_linear_create on raw GGUF blocks. Q4_K / Q5_K / Q6_K stay resident and run the K-quant GEMV; the other formats
    are decoded once and run as F32. Either way the product is the fp32 dot over the reference's decoded rows, and the
    resident weights dequantize to those rows bit for bit."""
    rng = np.random.default_rng(9 + gtype)
    n, k = 97, 768                                   # an odd row count: the last warp's second row repeats its first
    raw = _random_blocks(rng, gtype, n * k, 0.05)
    w = GF.decode_span(gtype, raw).reshape(n, k)
    bias = rng.standard_normal(n).astype(np.float32)
    lin = DotProductSharedKernel(backend)
    lin.prepare_for_compute_quant(gtype, raw, n, k, bias=bias)
    assert np.array_equal(lin.dequantize_weights().view(np.uint32), w.view(np.uint32))
    assert lin.weight_bytes() == (raw.size if gtype in (12, 13, 14) else n * k * 4)
    x = rng.standard_normal((batch, k)).astype(np.float32)
    lin.compute_quant(x)
    y = lin.finish_and_load_result()
    ref = x.astype(np.float64) @ w.astype(np.float64).T + bias
    assert np.max(np.abs(y - ref)) < 2e-5 * float(np.sqrt(np.mean(ref ** 2)))
    lin.unprepare_for_compute()


def test_model_load_refusals(backend, tmp_path):
    p = tmp_path / "bad.gguf"
    W.write(p, [("general.architecture", W.STR, "starcoder2")], [])
    with pytest.raises(CaiError, match="not supported"):
        LlamaModel.from_gguf(backend, p)
    # a tensor is missing: finalize refuses, naming it
    t = [("token_embd.weight", [32, 8], 0, np.zeros(256, np.float32)), ("output_norm.weight", [32], 0, np.ones(32, np.float32))]
    W.write(p, W.llama_meta("llama", 32, 64, 1, 2, 2, 16), t)
    with pytest.raises(CaiError):
        LlamaModel.from_gguf(backend, p)
    # a type without a decoder
    t.append(("blk.0.attn_q.weight", [32, 32], 30, np.zeros(2048, np.uint8)))
    W.write(p, W.llama_meta("llama", 32, 64, 1, 2, 2, 16), t)
    with pytest.raises(CaiError, match="unsupported type BF16"):
        LlamaModel.from_gguf(backend, p)
    with pytest.raises(CaiError, match="cannot open"):
        LlamaModel.from_gguf(backend, tmp_path / "missing.gguf")
