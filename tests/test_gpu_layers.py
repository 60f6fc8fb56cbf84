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
