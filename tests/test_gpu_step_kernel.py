"""The persistent step kernel (one kernel per decode step) against the launch-per-operator path of the same library
and against the oracle, on the shapes the benchmarks run; plus the time-out branches of the device-side waits."""
import os

import numpy as np
import pytest

from neural_api_b200.backend import CaiError, LlamaModel, StreamingDecoder, make_config, TYPE_Q8_0
from neural_api_b200.configs import ARCHS
from oracle import codecs
from oracle.forward import LlamaConfig, OracleModel, OracleSession, argmax_first, rms_norm, rope_interleaved

pytestmark = pytest.mark.gpu


class _env:
    """Sets an environment switch the library reads when a session is created."""

    def __init__(self, name, value):
        self.name, self.value = name, value

    def __enter__(self):
        self.old = os.environ.get(self.name)
        os.environ[self.name] = self.value

    def __exit__(self, *a):
        if self.old is None:
            os.environ.pop(self.name, None)
        else:
            os.environ[self.name] = self.old


SHAPES = {
    # small Qwen2-like: q/k/v biases, 2 query heads per KV head
    "small-bias": dict(hidden=256, inter=512, layers=3, heads=4, kv_heads=2, head_dim=64, vocab=1024, rms_eps=1e-6,
                       rope_theta=1e6, tie_embeddings=True, qkv_bias=True),
    # Qwen2.5-0.5B layers (7 query heads per KV head, hidden 896 = 1.75 chunks), depth cut
    "qwen0.5b-4l": dict(ARCHS["qwen2.5-0.5b"], layers=4),
    # Qwen2.5-32B layer shape (5 query heads per KV head, 27648-wide MLP), depth and vocabulary cut
    "qwen32b-2l": dict(ARCHS["qwen2.5-32b"], layers=2, vocab=4096),
    # one query head per KV head, head_dim 128
    "mha-128": dict(hidden=512, inter=1024, layers=2, heads=4, kv_heads=4, head_dim=128, vocab=512, rms_eps=1e-5,
                    rope_theta=1e4),
}


@pytest.mark.parametrize("shape,ctx,steps", [("small-bias", 40, 12), ("qwen0.5b-4l", 300, 8), ("qwen32b-2l", 700, 4),
                                             ("mha-128", 200, 6)])
def test_step_kernel_matches_launch_per_operator(backend, shape, ctx, steps):
    kw = SHAPES[shape]
    model = LlamaModel(backend, make_config(**kw))
    model.init_synthetic(TYPE_Q8_0, seed=11, std=0.02)
    model.finalize()
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, kw["vocab"], ctx).astype(np.int32)
    results = []
    try:
        for flag in ("1", "0"):
            with _env("CAI_STEP_KERNEL", flag):
                sess = StreamingDecoder(model, ctx + steps + 8)
            try:
                assert sess.uses_step_kernel == (flag == "1")
                sess.prefill([prompt[:-1]])
                tok = int(prompt[-1])
                rows, toks = [], []
                for _ in range(steps):
                    logits, amax = sess.step_forward([tok])
                    rows.append(logits[0].copy())
                    tok = int(amax[0])
                    toks.append(tok)
                dev = sess.decode_greedy([tok], 4)            # the on-device greedy loop
                results.append((rows, toks, dev.reshape(-1).tolist()))
            finally:
                sess.close()
    finally:
        model.close()
    (r1, t1, d1), (r0, t0, d0) = results
    assert t1 == t0 and d1 == d0, (t1, t0, d1, d0)
    for a, b in zip(r1, r0):
        rms = float(np.sqrt(np.mean(b.astype(np.float64) ** 2)))
        assert float(np.max(np.abs(a - b))) < 2e-5 * rms


def _oracle_from_device(model, cfg, names_extra=()):
    names = ["model.embed_tokens.weight", "model.norm.weight"]
    if not cfg.tie_embeddings:
        names.append("lm_head.weight")
    for l in range(cfg.layers):
        p = "model.layers.%d." % l
        names += [p + s for s in ("input_layernorm.weight", "post_attention_layernorm.weight", "self_attn.q_proj.weight",
                                  "self_attn.k_proj.weight", "self_attn.v_proj.weight", "self_attn.o_proj.weight",
                                  "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight")]
        if cfg.qkv_bias:
            names += [p + s for s in ("self_attn.q_proj.bias", "self_attn.k_proj.bias", "self_attn.v_proj.bias")]
    tensors = {}
    cap = max(cfg.vocab, 2 * cfg.inter, cfg.q_width, cfg.hidden) * (max(cfg.hidden, cfg.inter, cfg.q_width) // 32) * 34 + 64
    for n in names:
        buf, ty, rows, cols = model.read_tensor(n, cap)
        w = codecs.dequantize(ty, buf[:rows * codecs.block_bytes_per_row(ty, cols)])
        tensors[n] = w.reshape(rows, cols) if rows > 1 else w
    return OracleModel.from_hf_tensors(cfg, tensors, interleave=False)


def test_benchmark_layer_shape_with_a_long_cache_matches_the_oracle(backend):
    """One layer of the Qwen2.5-32B shape (hidden 5120, 40:8 heads of 128, 27648-wide MLP; vocabulary cut) with 4200
    really cached rows: many context splits, the long down-projection row, the LM head. With ONE layer a position's
    K and V rows depend on its token only, so the oracle's cache is computed for all positions at once with the
    oracle's own operators and its decode steps then run over it."""
    kw = dict(ARCHS["qwen2.5-32b"], layers=1, vocab=4096)
    cfg = LlamaConfig(hidden=kw["hidden"], inter=kw["inter"], layers=1, heads=kw["heads"], kv_heads=kw["kv_heads"],
                      head_dim=kw["head_dim"], vocab=kw["vocab"], rms_eps=kw["rms_eps"], rope_theta=kw["rope_theta"],
                      tie_embeddings=kw.get("tie_embeddings", False), qkv_bias=kw.get("qkv_bias", False))
    model = LlamaModel(backend, make_config(**kw))
    model.init_synthetic(TYPE_Q8_0, seed=3, std=0.02)
    model.finalize()
    n_ctx, n_new = 4200, 3
    rng = np.random.default_rng(5)
    prompt = rng.integers(0, cfg.vocab, n_ctx).astype(np.int32)
    sess = StreamingDecoder(model, n_ctx + n_new + 4)
    try:
        assert sess.uses_step_kernel
        oracle = _oracle_from_device(model, cfg)
        b = oracle.blocks[0]
        osess = OracleSession(oracle, n_ctx + n_new + 4)
        hd = cfg.head_dim
        pre = prompt[:-1]
        X = oracle.embed[pre].astype(np.float32)
        Xn = np.stack([rms_norm(x, b["attn_norm"], cfg.rms_eps) for x in X])
        K = Xn @ b["wk"].T
        V = Xn @ b["wv"].T
        if "bk" in b:
            K = K + b["bk"]
            V = V + b["bv"]
        for t in range(len(pre)):
            osess.k[0, :, t, :] = rope_interleaved(K[t], t, oracle.theta, hd).reshape(cfg.kv_heads, hd)
            osess.v[0, :, t, :] = V[t].reshape(cfg.kv_heads, hd)
        osess.length = len(pre)
        sess.prefill([pre])
        tok = int(prompt[-1])
        for _ in range(n_new):
            logits, amax = sess.step_forward([tok])
            ref = osess.step(tok)
            rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2)))
            assert float(np.max(np.abs(logits[0] - ref))) < 1e-3 * rms
            assert int(amax[0]) == argmax_first(ref)
            tok = int(amax[0])
    finally:
        sess.close()
        model.close()


def test_step_kernel_refuses_a_full_context_on_the_host(backend):
    kw = SHAPES["small-bias"]
    model = LlamaModel(backend, make_config(**kw))
    model.init_synthetic(TYPE_Q8_0, seed=1, std=0.02)
    model.finalize()
    with _env("CAI_STEP_KERNEL", "1"):
        sess = StreamingDecoder(model, 4)
    try:
        assert sess.uses_step_kernel
        for i in range(4):
            sess.step_forward([i])
        with pytest.raises(CaiError, match="context full"):
            sess.step_forward([0])
        sess.truncate_to(2)
        sess.step_forward([5])
        assert sess.cache_length() == 3
    finally:
        sess.close()
        model.close()


@pytest.mark.parametrize("which", [0, 1])
def test_bounded_device_waits_give_up_with_a_status(backend, which):
    """which = 0: the all-reduce kernel waits for a rank that does not exist; 1: the step kernel's grid barrier expects
    one arrival more than there are CTAs. Both must give up after the limit, report CAI_ERR_CUDA, and leave the context
    usable."""
    st = backend.selftest_wait_timeout(which, 2000)            # 2 ms
    assert st == 2                                             # CAI_ERR_CUDA: the error word was raised
    backend.sync()                                             # the word was consumed: the next call is clean
    x = backend.to_device(np.arange(8, dtype=np.float32))
    try:
        assert np.array_equal(x.read(np.float32, 8), np.arange(8, dtype=np.float32))
    finally:
        x.free()
