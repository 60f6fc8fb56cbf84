"""Sliding-window attention and StreamingLLM eviction (TNNetFusedSDPA's Window, EnableEviction) on the layer shim and on
whole sessions, against a float64 attention over the rows the policy keeps and against the oracle."""
import numpy as np
import pytest

from neural_api_b200.backend import CaiError, FusedSDPA, LlamaModel, StreamingDecoder, make_config, TYPE_I8, TYPE_Q8_0
from oracle import codecs
from oracle.forward import LlamaConfig, OracleModel, OracleSession, argmax_first

pytestmark = pytest.mark.gpu


def _attn(q, ks, vs, q_heads, kv_heads, hd):
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


@pytest.mark.parametrize("q_heads,kv_heads,hd", [(14, 2, 64), (8, 8, 128), (3, 1, 20)])
def test_layer_window_and_eviction(backend, q_heads, kv_heads, hd):
    rng = np.random.default_rng(hd)
    qw, kw = q_heads * hd, kv_heads * hd
    steps = 300
    rows = [rng.standard_normal(qw + 2 * kw).astype(np.float32) for _ in range(steps)]
    ks = [r[qw:qw + kw] for r in rows]
    vs = [r[qw + kw:] for r in rows]
    # sliding window of 70 rows in a cache that holds everything
    sd = FusedSDPA(backend, q_heads, kv_heads, hd)
    sd.begin_incremental_decode(steps)
    try:
        sd.set_window(70)
        for t, r in enumerate(rows):
            out = sd.compute_cached_token(r)
            if t in (0, 5, 69, 70, 71, 150, steps - 1):
                lo = max(0, t + 1 - 70)
                ref = _attn(r[:qw], ks[lo:t + 1], vs[lo:t + 1], q_heads, kv_heads, hd)
                assert np.max(np.abs(out - ref)) < 2e-5, t
    finally:
        sd.end_incremental_decode()
    # StreamingLLM: 4 sinks + 60 recent rows in a cache of exactly 64 rows, streamed far past it
    sd = FusedSDPA(backend, q_heads, kv_heads, hd)
    sd.begin_incremental_decode(64)
    try:
        sd.enable_eviction(4, 60)
        for t, r in enumerate(rows):
            out = sd.compute_cached_token(r)
            if t in (0, 63, 64, 65, 123, 124, 200, steps - 1):
                n = t + 1
                keep = list(range(n)) if n <= 64 else list(range(4)) + list(range(n - 60, n))
                ref = _attn(r[:qw], [ks[i] for i in keep], [vs[i] for i in keep], q_heads, kv_heads, hd)
                assert np.max(np.abs(out - ref)) < 2e-5, t
        assert sd.cache_length == steps
        with pytest.raises(CaiError):
            sd.truncate_cache(100)                       # the rows a shorter prefix needs are gone
    finally:
        sd.end_incremental_decode()


def _oracle(model, cfg):
    names = ["model.embed_tokens.weight", "model.norm.weight"]
    for l in range(cfg.layers):
        p = "model.layers.%d." % l
        names += [p + s for s in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                                  "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                  "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")]
    tensors = {}
    for n in names:
        buf, ty, rows, cols = model.read_tensor(n, 1 << 22)
        w = codecs.dequantize(ty, buf[:rows * codecs.block_bytes_per_row(ty, cols)])
        tensors[n] = w.reshape(rows, cols) if rows > 1 else w
    return OracleModel.from_hf_tensors(cfg, tensors, interleave=False)


@pytest.mark.parametrize("kv_type,tol,i8_kernel", [(0, 1e-3, None), (TYPE_I8, 5e-3, "0"), (TYPE_I8, 5e-3, "1")])
def test_session_eviction_and_window_match_the_oracle(backend, monkeypatch, kv_type, tol, i8_kernel):
    """i8_kernel: the int8 cache's CUDA-core kernel ("0") or its integer tensor-core kernel ("1"; the window's first row is
    not on a 32-row boundary, so its tiles take the row-by-row copy path)."""
    if i8_kernel is not None:
        monkeypatch.setenv("CAI_ATTN_I8MMA", i8_kernel)
    kw = dict(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=512, rms_eps=1e-6, rope_theta=1e4,
              tie_embeddings=True)
    model = LlamaModel(backend, make_config(**kw))
    model.init_synthetic(TYPE_Q8_0, seed=6, std=0.05)
    model.finalize()
    cfg = LlamaConfig(**kw)
    oracle = _oracle(model, cfg)
    rng = np.random.default_rng(3)
    toks = rng.integers(0, kw["vocab"], 150)
    try:
        # eviction: 4 sinks + 44 recent rows in a cache of 48, streamed to 150 positions
        sess = StreamingDecoder(model, 48, kv_type=kv_type)
        sess.enable_eviction(4, 44)
        assert not sess.uses_step_kernel
        osess = OracleSession(oracle, 160, kv_int8=(kv_type == TYPE_I8), evict=(4, 44))
        worst = 0.0
        for i, t in enumerate(toks):
            logits, amax = sess.step_forward([int(t)])
            ref = osess.step(int(t))
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            worst = max(worst, float(np.max(np.abs(logits[0] - ref))) / rms)
        assert worst < tol, worst
        assert sess.cache_length() == 150
        sess.close()
        # sliding window of 40 rows, prompt through the chunked prefill
        sess = StreamingDecoder(model, 160, kv_type=kv_type)
        sess.set_window(40)
        osess = OracleSession(oracle, 160, kv_int8=(kv_type == TYPE_I8), window=40)
        sess.prefill([toks[:100]])
        for t in toks[:100]:
            osess.step(int(t))
        worst = 0.0
        for t in toks[100:]:
            logits, amax = sess.step_forward([int(t)])
            ref = osess.step(int(t))
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            worst = max(worst, float(np.max(np.abs(logits[0] - ref))) / rms)
        assert worst < tol, worst
        sess.close()
    finally:
        model.close()
