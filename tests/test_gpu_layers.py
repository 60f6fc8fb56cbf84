"""Layer-granular CUDA shims against the oracle: RMSNorm, RoPE, SwiGLU, router gate,
fused GQA decode attention with its KV cache."""
import numpy as np
import pytest

from conftest import load_golden
from oracle.forward import rms_norm, rope_interleaved, router_gates, softmax_row, swiglu
from neural_api_b200.backend import CaiError, FusedSDPA

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,depth", [(1, 8), (3, 896), (2, 5120), (1, 37)])
def test_rmsnorm(backend, tokens, depth):
    rng = np.random.default_rng(depth)
    x = rng.standard_normal((tokens, depth)).astype(np.float32) * 3
    g = (1 + 0.1 * rng.standard_normal(depth)).astype(np.float32)
    y = backend.rmsnorm(x, g, 1e-6)
    ref = np.stack([rms_norm(r, g, 1e-6) for r in x])
    assert np.max(np.abs(y - ref)) < 1e-5 * np.max(np.abs(ref))


def test_rope_position_zero_is_identity(backend):
    x = np.arange(1, 65, dtype=np.float32).reshape(1, 64)
    assert np.array_equal(backend.rope(x, 16, 0, 10000.0), x)


@pytest.mark.parametrize("head_dim,depth,offset,base", [(4, 8, 3, 1e4), (64, 896, 127, 1e6), (128, 1024, 8191, 1e6)])
def test_rope_matches_closed_form(backend, head_dim, depth, offset, base):
    """pairs (2k,2k+1), theta_k = exp(-2k/D ln base), angle = (t + offset) * theta_k; tol 1e-5
    (tests/TestNeuralNumerical.pas:15301-15350)."""
    rng = np.random.default_rng(offset)
    x = rng.standard_normal((3, depth)).astype(np.float32)
    y = backend.rope(x, head_dim, offset, base)
    theta = np.exp(-2.0 * np.arange(head_dim // 2) / head_dim * np.log(base)).astype(np.float32)
    for t in range(3):
        ref = rope_interleaved(x[t], t + offset, theta, head_dim)
        assert np.max(np.abs(y[t] - ref)) < 1e-5


def test_swiglu_packing_and_extremes(backend):
    x = np.asarray([[2.0, -3.0, 0.5, 1.0, -1.0, 0.0], [1.0, 1.0, 1.0, 100.0, -100.0, -20.0]], dtype=np.float32)
    y = backend.swiglu(x)
    ref = np.stack([swiglu(r, 3) for r in x])
    assert np.all(np.isfinite(y))
    assert np.max(np.abs(y - ref)) < 1e-5
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 2 * 4864)).astype(np.float32) * 4
    assert np.max(np.abs(backend.swiglu(x) - np.stack([swiglu(r, 4864) for r in x]))) < 1e-5


def test_topk_gate_known_answer(backend):
    k = load_golden("kats")
    probs = k["topk_in"].astype(np.float32)
    ids, gates = backend.topk_gate(np.log(probs)[None, :], int(k["topk_k"]), True)
    out = np.zeros(4, dtype=np.float32)
    out[ids[0]] = gates[0]
    assert np.allclose(out, k["topk_out"], atol=1e-6)
    assert list(ids[0]) == [0, 2]


@pytest.mark.parametrize("n_experts,top_k,renorm", [(4, 2, True), (64, 8, False), (64, 8, True), (8, 8, True), (100, 3, False)])
def test_topk_gate_random(backend, n_experts, top_k, renorm):
    rng = np.random.default_rng(n_experts + top_k)
    logits = rng.standard_normal((9, n_experts)).astype(np.float32) * 2
    logits[0, :] = 0.25                      # an all-ties row: lowest indices win
    ids, gates = backend.topk_gate(logits, top_k, renorm)
    for t in range(logits.shape[0]):
        order, ref = router_gates(softmax_row(logits[t]), top_k, renorm)
        assert list(ids[t]) == list(order)
        assert np.max(np.abs(gates[t] - ref)) < 1e-6


def _attn_ref(q, ks, vs, q_heads, kv_heads, hd):
    group = q_heads // kv_heads
    out = np.empty(q_heads * hd, dtype=np.float64)
    for h in range(q_heads):
        g = h // group
        K = np.stack([k[g * hd:(g + 1) * hd] for k in ks]).astype(np.float64)
        V = np.stack([v[g * hd:(g + 1) * hd] for v in vs]).astype(np.float64)
        s = (K @ q[h * hd:(h + 1) * hd].astype(np.float64)) / np.sqrt(hd)
        e = np.exp(s - s.max())
        out[h * hd:(h + 1) * hd] = (e @ V) / e.sum()
    return out


@pytest.mark.parametrize("q_heads,kv_heads,hd,steps,max_ctx", [
    (1, 1, 64, 48, 64),        # the bare single-head d_k=64 layer of the IncrementalDecode example
    (2, 1, 4, 16, 16),         # pico fixtures
    (14, 2, 64, 300, 512),     # Qwen2.5-0.5B grouping (7 query heads per KV head)
    (40, 8, 128, 70, 8192),    # Qwen2.5-32B grouping, long cache -> many context splits
    (16, 16, 128, 33, 2048),   # OLMoE multi-head
    (32, 4, 64, 20, 768),      # TinyLlama
    (3, 1, 20, 9, 16),         # head_dim that is not a multiple of 8
])
def test_fused_sdpa_cached_decode(backend, q_heads, kv_heads, hd, steps, max_ctx):
    rng = np.random.default_rng(q_heads * 100 + hd)
    sdpa = FusedSDPA(backend, q_heads, kv_heads, hd)
    sdpa.begin_incremental_decode(max_ctx)
    try:
        ks, vs = [], []
        qw, kw = q_heads * hd, kv_heads * hd
        for t in range(steps):
            row = rng.standard_normal(qw + 2 * kw).astype(np.float32)
            ks.append(row[qw:qw + kw])
            vs.append(row[qw + kw:])
            out = sdpa.compute_cached_token(row)
            assert sdpa.cache_length == t + 1
            if t in (0, 1, steps // 2, steps - 1):
                ref = _attn_ref(row[:qw], ks, vs, q_heads, kv_heads, hd)
                assert np.max(np.abs(out - ref)) < 2e-5, (t, np.max(np.abs(out - ref)))
        # truncate, then the same row must give the same answer as before
        keep = steps // 2
        sdpa.truncate_cache(keep)
        assert sdpa.cache_length == keep
        row = rng.standard_normal(qw + 2 * kw).astype(np.float32)
        out = sdpa.compute_cached_token(row)
        ref = _attn_ref(row[:qw], ks[:keep] + [row[qw:qw + kw]], vs[:keep] + [row[qw + kw:]], q_heads, kv_heads, hd)
        assert np.max(np.abs(out - ref)) < 2e-5
        with pytest.raises(CaiError):
            sdpa.truncate_cache(keep + 5)
        sdpa.reset_cache()
        assert sdpa.cache_length == 0
    finally:
        sdpa.end_incremental_decode()


def test_fused_sdpa_cache_full_is_an_error(backend):
    sdpa = FusedSDPA(backend, 2, 1, 8)
    sdpa.begin_incremental_decode(3)
    try:
        row = np.ones(32, dtype=np.float32)
        for _ in range(3):
            sdpa.compute_cached_token(row)
        with pytest.raises(CaiError, match="full"):
            sdpa.compute_cached_token(row)
    finally:
        sdpa.end_incremental_decode()


@pytest.mark.parametrize("ggml_type,tokens,n_experts,top_k,hidden,width", [
    (0, 5, 4, 2, 64, 96),            # F32 banks, the shape class of the reference's bank parity test
    (8, 3, 8, 2, 256, 128),          # Q8_0 banks (Mixtral-like top-2)
    (8, 9, 16, 8, 128, 64),          # top-8 of 16 (OLMoE-like routing), more pairs than experts
])
def test_moe_expert_bank_layer_shim(backend, ggml_type, tokens, n_experts, top_k, hidden, width):
    """TNNetMoEExpertBankGateUp / Down through the layer-granular entry points against the per-expert reference graph
    (tests/TestNeuralLayersExtra.pas:7773-7906, tolerance 1e-4): out[t] = sum_j gate_j * down_e(up_e(x) * swish(gate_e(x)))."""
    from neural_api_b200.backend import MoEExpertBank
    from oracle import codecs
    from oracle.forward import router_gates, softmax_row, swiglu
    rng = np.random.default_rng(tokens * 131 + n_experts)
    x = rng.standard_normal((tokens, hidden)).astype(np.float32)
    logits = rng.standard_normal((tokens, n_experts)).astype(np.float32)
    bank = MoEExpertBank(backend, n_experts, hidden, width, ggml_type)
    mats = []
    for e in range(n_experts):
        up = (rng.standard_normal((width, hidden)) * 0.1).astype(np.float32)
        gate = (rng.standard_normal((width, hidden)) * 0.1).astype(np.float32)
        down = (rng.standard_normal((hidden, width)) * 0.1).astype(np.float32)
        if ggml_type == 8:
            blocks = [codecs.quantize_q8_0(m) for m in (up, gate, down)]
            up, gate, down = (codecs.dequantize_q8_0(b).reshape(m.shape) for b, m in zip(blocks, (up, gate, down)))
        else:
            blocks = [up, gate, down]
        for which, b in zip(("up", "gate", "down"), blocks):
            bank.upload(e, which, b)
        mats.append((up, gate, down))
    with pytest.raises(Exception):
        bank.gate_up(backend.to_device(x), backend.to_device(np.zeros(4, np.int32)), tokens, top_k, backend.alloc(16))   # finalize first
    bank.finalize()
    ids, gates = backend.topk_gate(logits, top_k, True)
    want_hidden = np.zeros((tokens * top_k, width), dtype=np.float32)
    want = np.zeros((tokens, hidden), dtype=np.float64)
    for t in range(tokens):
        order, g = router_gates(softmax_row(logits[t]), top_k, True)
        assert list(order) == list(ids[t])
        for j, e in enumerate(order):
            up, gate, down = mats[int(e)]
            fused = np.concatenate([up @ x[t], gate @ x[t]]).astype(np.float32)
            h = swiglu(fused, width)
            want_hidden[t * top_k + j] = h
            want[t] += float(g[j]) * (down.astype(np.float64) @ h.astype(np.float64))
    dx, dids, dg = backend.to_device(x), backend.to_device(ids.reshape(-1)), backend.to_device(gates.reshape(-1))
    dh, dout = backend.alloc(tokens * top_k * width * 4), backend.alloc(tokens * hidden * 4)
    try:
        bank.gate_up(dx, dids, tokens, top_k, dh)
        got_hidden = dh.read(np.float32, tokens * top_k * width).reshape(tokens * top_k, width)
        assert np.max(np.abs(got_hidden - want_hidden)) < 1e-4
        bank.down(dh, dids, dg, tokens, top_k, dout)
        got = dout.read(np.float32, tokens * hidden).reshape(tokens, hidden)
        assert np.max(np.abs(got - want)) < 1e-4
        bank.down(dh, dids, dg, tokens, top_k, dout)                     # the output is overwritten, not accumulated
        assert np.array_equal(dout.read(np.float32, tokens * hidden).reshape(tokens, hidden), got)
    finally:
        for b in (dx, dids, dg, dh, dout):
            b.free()
        bank.close()
