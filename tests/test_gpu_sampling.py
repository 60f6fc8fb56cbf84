"""Sampling on the device against the restated reference rule: the candidate window (top-k of softmax(logits / T)) and the
weighted draw with nucleus cut, driven by known uniform numbers."""
import ctypes as C

import numpy as np
import pytest

from neural_api_b200.backend import LlamaModel, StreamingDecoder, make_config, TYPE_Q8_0
from oracle.forward import sampler_window, weighted_draw

pytestmark = pytest.mark.gpu

KW = dict(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=5000, rms_eps=1e-6, rope_theta=1e4,
          tie_embeddings=True)


@pytest.fixture(scope="module")
def model(backend):
    m = LlamaModel(backend, make_config(**KW))
    m.init_synthetic(TYPE_Q8_0, seed=12, std=0.05)
    m.finalize()
    yield m
    m.close()


@pytest.mark.parametrize("batch", [1, 3])
@pytest.mark.parametrize("k,temperature", [(1, 1.0), (8, 0.7), (40, 1.3), (64, 1.0)])
def test_candidate_window_matches_the_oracle(model, batch, k, temperature):
    rng = np.random.default_rng(k)
    toks = rng.integers(0, KW["vocab"], (3, batch)).astype(np.int32)
    a = StreamingDecoder(model, 16, batch=batch)
    b = StreamingDecoder(model, 16, batch=batch)
    try:
        for t in toks:
            logits, _ = a.step_forward(t)
            ids, probs = b.step_topk(t, k, temperature)
            for s in range(batch):
                ref_ids, ref_p = sampler_window(logits[s], k, temperature)
                assert np.array_equal(ids[s], ref_ids)
                assert np.max(np.abs(probs[s] - ref_p)) < 1e-6 + 1e-4 * float(ref_p.max())
    finally:
        a.close()
        b.close()


@pytest.mark.parametrize("top_k,top_p,temperature", [(40, 0.0, 1.0), (40, 0.9, 0.8), (8, 0.5, 1.5), (1, 0.0, 1.0)])
def test_sampled_loop_follows_the_weighted_draw_with_known_uniforms(model, top_k, top_p, temperature):
    batch, steps = 2, 12
    rng = np.random.default_rng(top_k)
    u = rng.random((steps, batch)).astype(np.float32)
    first = rng.integers(0, KW["vocab"], batch).astype(np.int32)
    dev = StreamingDecoder(model, 32, batch=batch)
    ref = StreamingDecoder(model, 32, batch=batch)
    try:
        out = dev.decode_sampled(first, steps, temperature=temperature, top_k=top_k, top_p=top_p, uniforms=u)
        tok = first.copy()
        for i in range(steps):
            logits, _ = ref.step_forward(tok)
            nxt = np.empty(batch, dtype=np.int32)
            for s in range(batch):
                ids, probs = sampler_window(logits[s], top_k, temperature)
                nxt[s] = weighted_draw(ids, probs, u[i, s], top_p)
            # a uniform number within float rounding of a boundary of the running sum may fall on either side: then the
            # device's choice must be the neighbouring candidate, and the comparison continues from the device's token
            for s in range(batch):
                if out[i, s] != nxt[s]:
                    ids, probs = sampler_window(logits[s], top_k, temperature)
                    cum = np.cumsum(probs.astype(np.float64))
                    roll = float(u[i, s]) * float(cum[min(len(cum), top_k) - 1])
                    assert np.min(np.abs(cum - roll)) < 1e-5 and int(out[i, s]) in ids.tolist()
            tok = out[i].copy()
        assert dev.cache_length(0) == steps
    finally:
        dev.close()
        ref.close()


def test_keyed_generator_is_reproducible_on_the_host(model, backend):
    batch, steps, seed = 2, 6, 1234
    dev = StreamingDecoder(model, 32, batch=batch)
    twin = StreamingDecoder(model, 32, batch=batch)
    try:
        first = np.asarray([5, 9], dtype=np.int32)
        a = dev.decode_sampled(first, steps, temperature=1.0, top_k=40, top_p=0.95, seed=seed)
        u = np.empty((steps, batch), dtype=np.float32)
        for i in range(steps):
            for s in range(batch):
                x = C.c_float()
                backend._check(backend.lib.cai_sampling_uniform(seed, i + 1, s, C.byref(x)))
                u[i, s] = x.value
        b = twin.decode_sampled(first, steps, temperature=1.0, top_k=40, top_p=0.95, uniforms=u)
        assert np.array_equal(a, b)
        assert len(set(a[:, 0].tolist())) > 1                    # it does sample: not one token repeated
    finally:
        dev.close()
        twin.close()
