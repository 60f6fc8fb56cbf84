"""Pins the CPU oracle against the reference's own golden vectors (no GPU)."""
import json

import numpy as np
import pytest

from conftest import golden_hf_case, load_golden
from oracle import codecs
from oracle.forward import (LlamaConfig, OracleModel, OracleSession, greedy_decode, interleave_rows,
                            rope_interleaved, router_gates, swiglu)


@pytest.mark.parametrize("name", ["tiny_llama", "tiny_qwen2", "tiny_olmoe", "tiny_mixtral"])
@pytest.mark.parametrize("dtype", [np.float64, np.float32])
def test_forward_matches_reference_golden_logits(name, dtype):
    """Gate 1e-4, the reference's own (tests/TestNeuralPretrained.pas:5684-5751)."""
    cfg_json, tensors, seqs, gold = golden_hf_case(name)
    cfg = LlamaConfig.from_hf(cfg_json)
    model = OracleModel.from_hf_tensors(cfg, tensors, dtype=dtype)
    worst = 0.0
    for s, g in zip(seqs, gold):
        sess = OracleSession(model, len(s))
        for i, t in enumerate(s):
            worst = max(worst, float(np.max(np.abs(sess.step(int(t), i) - g[i]))))
    assert worst < 1e-4, worst


def test_q8_gguf_fixture_dequant_and_quantizer_are_bit_exact():
    z = load_golden("tiny_llama_q8_gguf")
    n_q8 = 0
    for k in z.files:
        if not k.startswith("raw::"):
            continue
        name = k[5:]
        ty, rows, cols = (int(v) for v in z["meta::" + name])
        deq = codecs.dequantize(ty, z[k])
        assert np.array_equal(deq.view(np.uint32), z["deq::" + name].view(np.uint32)), name
        if ty == codecs.GGML_Q8_0 and ("twin::" + name) in z.files:
            twin = z["twin::" + name]
            if "q_proj" in name or "k_proj" in name:
                twin = interleave_rows(twin, 16)     # GGUF stores q/k rows interleaved
            assert np.array_equal(codecs.quantize_q8_0(twin), z[k]), name
            n_q8 += 1
    assert n_q8 == 15


def test_f16_gguf_fixture_dequant_is_bit_exact():
    z = load_golden("tiny_llama_f16_gguf")
    for k in z.files:
        if k.startswith("raw::"):
            name = k[5:]
            ty = int(z["meta::" + name][0])
            assert np.array_equal(codecs.dequantize(ty, z[k]).view(np.uint32), z["deq::" + name].view(np.uint32)), name


def _oracle_from_gguf(z, cfg, dtype=np.float32):
    tensors = {}
    for k in z.files:
        if k.startswith("raw::"):
            name = k[5:]
            ty, rows, cols = (int(v) for v in z["meta::" + name])
            w = codecs.dequantize(ty, z[k])
            tensors[name] = w.reshape(rows, cols) if rows > 1 else w
    return OracleModel.from_hf_tensors(cfg, tensors, dtype=dtype, interleave=False)


def test_q8_gguf_drift_against_f32_twin_is_in_the_reference_band():
    """Q8_0 import drift relative to max |logit| in (1e-3, 1.5e-1)
    (tests/TestNeuralPretrained.pas:6343-6438)."""
    z = load_golden("tiny_llama_q8_gguf")
    cfg = LlamaConfig.from_hf(json.loads(bytes(z["config_json"]).decode()))
    q8 = _oracle_from_gguf(z, cfg)
    twin = OracleModel.from_hf_tensors(cfg, {k[6:]: z[k] for k in z.files if k.startswith("twin::")})
    seq = [1, 5, 2, 7, 0, 3, 6, 4]
    a, b = OracleSession(q8, 12), OracleSession(twin, 12)
    drift, mx = 0.0, 0.0
    for i, t in enumerate(seq):
        la, lb = a.step(t, i), b.step(t, i)
        drift = max(drift, float(np.max(np.abs(la - lb))))
        mx = max(mx, float(np.max(np.abs(lb))))
    assert 1e-3 < drift / mx < 1.5e-1, drift / mx


def test_q4_0_known_answer_block():
    k = load_golden("kats")
    assert np.array_equal(codecs.dequantize_q4_0(k["q4_0_block"]), k["q4_0_expect"])


def test_codecs_agree_with_the_gguf_package():
    gq = pytest.importorskip("gguf.quants")
    from gguf import GGMLQuantizationType as T
    rng = np.random.default_rng(0)
    x = (rng.standard_normal((64, 256)) * 0.02).astype(np.float32)
    x[3, :32] = 0.0                                     # an all-zero block
    for ty, quant, deq in ((T.Q8_0, codecs.quantize_q8_0, codecs.dequantize_q8_0),
                           (T.Q4_0, codecs.quantize_q4_0, codecs.dequantize_q4_0)):
        ref = gq.quantize(x, ty)
        mine = quant(x)
        assert np.array_equal(ref.reshape(-1), mine)
        assert np.array_equal(deq(mine), gq.dequantize(ref, ty).reshape(-1))


def test_half_codec_all_bit_patterns():
    bits = np.arange(65536, dtype=np.uint16)
    mine = codecs.half_to_single(bits)
    ref = bits.view(np.float16).astype(np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(mine.view(np.uint32)[ok], ref.view(np.uint32)[ok])
    assert np.all(np.isnan(mine[~ok]))
    # encode: round-to-nearest-even on every normal half, exact round trip
    normal = bits[((bits >> 10) & 0x1F != 0) & ((bits >> 10) & 0x1F != 0x1F)]
    assert np.array_equal(codecs.single_to_half(codecs.half_to_single(normal)), normal)
    rng = np.random.default_rng(1)
    v = (rng.standard_normal(200000) * 0.01).astype(np.float32)
    v = v[np.abs(v) > 1e-4]
    assert np.array_equal(codecs.single_to_half(v), v.astype(np.float16).view(np.uint16))


def test_int8_round_trip_bound():
    """|w - dequant(quant(w))| <= scale/2 (+ the fp16 rounding of the scale)
    (the bound of tests/TestNeuralPretrained.pas:3668-3703 applied to Q8_0 blocks)."""
    rng = np.random.default_rng(2)
    x = (rng.standard_normal((128, 64)) * 0.02).astype(np.float32)
    blk = codecs.quantize_q8_0(x)
    deq = codecs.dequantize_q8_0(blk).reshape(x.shape)
    scale = np.repeat(np.max(np.abs(x.reshape(-1, 32)), axis=1) / 127.0, 32).reshape(x.shape)
    assert np.all(np.abs(deq - x) <= scale * 0.5 + np.abs(x) * 1e-3 + 1e-9)


def test_topk_gate_known_answer():
    k = load_golden("kats")
    order, gates = router_gates(k["topk_in"].astype(np.float32), int(k["topk_k"]), True)
    out = np.zeros(4, dtype=np.float32)
    out[order] = gates
    assert np.allclose(out, k["topk_out"], atol=1e-6)


def test_rope_known_answers():
    """pos 0 is the identity; closed form theta_k = exp(-2k/D ln base)
    (tests/TestNeuralNumerical.pas:15301-15350, tol 1e-5)."""
    hd, base = 8, 10000.0
    theta = np.exp(-2.0 * np.arange(hd // 2) / hd * np.log(base)).astype(np.float32)
    x = np.arange(1, 2 * hd + 1, dtype=np.float32)
    assert np.allclose(rope_interleaved(x, 0, theta, hd), x, atol=0)
    y = rope_interleaved(x, 3, theta, hd).reshape(2, hd // 2, 2)
    xr = x.reshape(2, hd // 2, 2)
    for k in range(hd // 2):
        a = 3 * base ** (-2.0 * k / hd)
        assert np.allclose(y[:, k, 0], np.cos(a) * xr[:, k, 0] - np.sin(a) * xr[:, k, 1], atol=1e-5)
        assert np.allclose(y[:, k, 1], np.sin(a) * xr[:, k, 0] + np.cos(a) * xr[:, k, 1], atol=1e-5)


def test_interleaved_rope_equals_rotate_half_under_the_importer_permutation():
    """tests/TestNeuralPretrained.pas:5262-5327."""
    hd = 8
    rng = np.random.default_rng(3)
    v = rng.standard_normal(hd).astype(np.float64)
    theta = np.exp(-2.0 * np.arange(hd // 2) / hd * np.log(10000.0)).astype(np.float32)
    pos = 5
    half = hd // 2
    hf = np.empty(hd)
    for i in range(half):
        a = np.float64(np.float32(pos) * theta[i])
        hf[i] = v[i] * np.cos(a) - v[i + half] * np.sin(a)
        hf[i + half] = v[i + half] * np.cos(a) + v[i] * np.sin(a)
    mine = rope_interleaved(interleave_rows(v, hd), pos, theta, hd)
    assert np.allclose(mine, interleave_rows(hf, hd), atol=1e-12)


def test_swiglu_packing_known_answer():
    """[up | gate] packing (tests/TestNeuralPretrained.pas:5329-5369)."""
    fused = np.asarray([2.0, -3.0, 0.5, 1.0, -1.0, 0.0], dtype=np.float32)
    up, gate = fused[:3], fused[3:]
    expect = up * (gate / (1.0 + np.exp(-gate)))
    assert np.allclose(swiglu(fused, 3), expect, atol=1e-7)


def test_streamed_equals_full_forward_and_truncate():
    """Cached decode == re-running the prefix (tests/TestNeuralDecode.pas:2996-3094)."""
    cfg_json, tensors, seqs, _ = golden_hf_case("tiny_qwen2")
    cfg = LlamaConfig.from_hf(cfg_json)
    model = OracleModel.from_hf_tensors(cfg, tensors)
    s = [int(t) for t in seqs[0]]
    a = OracleSession(model, 16)
    rows = [a.step(t, i) for i, t in enumerate(s)]
    a.truncate(5)
    again = a.step(s[5], 5)
    assert np.array_equal(again, rows[5])
    toks, _ = greedy_decode(model, s[:4], 4)
    assert len(toks) == 4


def test_int8_kv_cache_row_format_and_drift():
    """The int8 KV row rule of the reference's device kernel (neural/neural.cl:2500-2581): scale = maxabs / 127,
    round half to even, |v - scale * code| <= scale / 2, zero row -> zero codes and unit scale; and a model decoded
    over the int8 cache drifts from the fp32-cache logits by a small, non-zero amount (the reference's own 1e-3
    gate, tests/TestNeuralNumerical.pas:69604-69609, compares two int8-cache implementations, as the GPU test does)."""
    from oracle.forward import quantize_cache_row
    rng = np.random.default_rng(3)
    row = rng.standard_normal(128).astype(np.float32)
    codes, scale = quantize_cache_row(row)
    assert codes.dtype == np.int8 and np.abs(codes).max() == 127 and scale == np.float32(np.abs(row).max() / np.float32(127))
    assert np.all(np.abs(row - scale * codes.astype(np.float32)) <= scale / 2 * (1 + 1e-6))
    half = quantize_cache_row(np.float32([127.0, 0.5, 1.5, 2.5, -0.5, -1.5]))[0]
    assert list(half) == [127, 0, 2, 2, 0, -2]                    # ties to even
    z, zs = quantize_cache_row(np.zeros(64, np.float32))
    assert not z.any() and zs == np.float32(1.0)
    bad, _ = quantize_cache_row(np.float32([1.0, np.nan, np.inf, -np.inf]))
    assert list(bad) == [127, 0, 127, -127]
    cfg_json, tensors, seqs, gold = golden_hf_case("tiny_llama")
    cfg = LlamaConfig.from_hf(cfg_json)
    model = OracleModel.from_hf_tensors(cfg, tensors)
    f32 = OracleSession(model, 16)
    i8 = OracleSession(model, 16, kv_int8=True)
    worst = 0.0
    for t in seqs[0]:
        a, b = f32.step(int(t)), i8.step(int(t))
        worst = max(worst, float(np.max(np.abs(a - b))) / float(np.max(np.abs(a))))
    assert 0 < worst < 1e-1


# ---------------------------------------------------------------------------------------------------------------
# the reference's own int8 weight rows (TNNetVolume.QuantizeInt8, neural/neuralvolume.pas:12471-12562)
# ---------------------------------------------------------------------------------------------------------------
def test_int8_row_quantizer_round_trip_bound_and_edge_values():
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((64, 96)) * 0.05).astype(np.float32)
    codes, scales = codecs.quantize_int8_rows(w)
    back = codecs.dequantize_int8_rows(codes, scales)
    # |dw| <= scale / 2 per row, the reference's own round-trip gate (tests/TestNeuralPretrained.pas:3668-3703)
    assert np.all(np.abs(back - w) <= scales[:, None] * 0.5 * (1 + 1e-5) + 1e-12)
    assert np.all(np.abs(codes.astype(np.int32)).max(axis=1) == 127)          # every row uses the full range
    # NaN -> 0, infinities clamp, a zero row stays zero with scale 0, the maximum ignores non-finite values
    edge = np.zeros((3, 32), dtype=np.float32)
    edge[0, :4] = [np.nan, np.inf, -np.inf, 2.0]
    edge[0, 4] = -1.0
    edge[2, 0] = np.float32(1e-40)                                         # denormal row maximum: scaled in double
    edge[2, 1] = np.float32(-5e-41)
    codes, scales = codecs.quantize_int8_rows(edge)
    assert codes[0, :5].tolist() == [0, 127, -127, 127, -64] and scales[0] == np.float32(2.0) / np.float32(127.0)
    assert not codes[1].any() and scales[1] == 0
    assert codes[2, 0] == 127 and codes[2, 1] == -64 and scales[2] > 0       # -63.5 rounds to the even neighbour
    # round half to even on exact half-way points: v = maxabs * (k + 0.5) / 127 for small k
    row = np.zeros((1, 32), dtype=np.float32)
    row[0, 0] = 127.0
    row[0, 1:5] = [0.5, 1.5, 2.5, -3.5]
    codes, _ = codecs.quantize_int8_rows(row)
    got = codes[0, 1:5].tolist()
    want = [int(np.rint(np.float32(np.float32(v * np.float32(1.0 / 127.0)) * np.float32(127.0)))) for v in (0.5, 1.5, 2.5, -3.5)]
    assert got == want


def test_int8_row_linear_applies_the_scale_after_the_raw_code_sum():
    rng = np.random.default_rng(1)
    w = (rng.standard_normal((8, 64)) * 0.1).astype(np.float32)
    x = rng.standard_normal((2, 64)).astype(np.float32)
    codes, scales = codecs.quantize_int8_rows(w)
    y = codecs.linear_int8_rows(codes, scales, x)
    ref = x.astype(np.float64) @ codecs.dequantize_int8_rows(codes, scales).astype(np.float64).T
    assert np.max(np.abs(y - ref)) < 1e-5
    raw = np.concatenate([codes.view(np.uint8), scales.view(np.uint8).reshape(8, 4)], axis=1).reshape(-1)
    c2, s2 = codecs.split_int8_rows(raw, 8, 64)
    assert np.array_equal(c2, codes) and np.array_equal(s2, scales)
