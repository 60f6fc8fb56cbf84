"""The allocation-free attention step (cai_sdpa_step_noalloc) against the regular one
(cai_sdpa_step_dev), two calls in a row.

The entry point exists for hosts that are not allowed to allocate GPU memory at call time - a
real-time loop, a plugin living in a fixed arena, a process with a fixed memory budget - so here the test
harness allocates every buffer up front and the call itself only launches kernels; its split-context
scratch is a fixed array inside the library. This file is collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

from neural_api_b200.backend import CaiError, FusedSDPA

pytestmark = pytest.mark.gpu

TOL = 2e-5      # the tolerance of the attention tests


def _attn_fp64(q, ks, vs, q_heads, kv_heads, hd):
    """Plain float64 attention of one query row over the cached rows (the reference the attention tests use)."""
    group = q_heads // kv_heads
    out = np.empty(q_heads * hd, dtype=np.float64)
    for h in range(q_heads):
        g = h // group
        K = np.stack([k[g * hd:(g + 1) * hd] for k in ks]).astype(np.float64)
        V = np.stack([v[g * hd:(g + 1) * hd] for v in vs]).astype(np.float64)
        sc = (K @ q[h * hd:(h + 1) * hd].astype(np.float64)) / np.sqrt(hd)
        e = np.exp(sc - sc.max())
        out[h * hd:(h + 1) * hd] = (e @ V) / e.sum()
    return out


def _run_case(backend, q_heads, kv_heads, hd, max_ctx, prefix):
    lib = backend.lib
    rng = np.random.default_rng(q_heads * 31 + hd)
    qw, kw = q_heads * hd, kv_heads * hd
    rows = [rng.standard_normal(qw + 2 * kw).astype(np.float32) for _ in range(prefix + 2)]
    # reference: the existing entry point, fed every row
    ref = FusedSDPA(backend, q_heads, kv_heads, hd)
    ref.begin_incremental_decode(max_ctx)
    want = [ref.compute_cached_token(r) for r in rows]
    ref.end_incremental_decode()
    # caller-owned buffers for the allocation-free path, filled with the first `prefix` rows
    kc = np.zeros((kv_heads, max_ctx, hd), dtype=np.float32)
    vc = np.zeros_like(kc)
    for t in range(prefix):
        kc[:, t, :] = rows[t][qw:qw + kw].reshape(kv_heads, hd)
        vc[:, t, :] = rows[t][qw + kw:].reshape(kv_heads, hd)
    d_k, d_v = backend.to_device(kc), backend.to_device(vc)
    d_len = backend.to_device(np.asarray([prefix], dtype=np.int32))
    d_row = backend.alloc((qw + 2 * kw) * 4)
    d_out = backend.alloc(qw * 4)
    try:
        for i in range(2):                         # two calls in a row share the built-in scratch
            t = prefix + i
            d_row.write(rows[t])
            d_len.write(np.asarray([t], dtype=np.int32))
            backend._check(lib.cai_sdpa_step_noalloc(backend.ctx, d_row.ptr, d_k.ptr, d_v.ptr, d_len.ptr,
                                                     q_heads, kv_heads, hd, max_ctx, d_out.ptr))
            got = d_out.read(np.float32, qw)
            assert np.max(np.abs(got - want[t])) < TOL, (i, float(np.max(np.abs(got - want[t]))))
            ref = _attn_fp64(rows[t][:qw], [r[qw:qw + kw] for r in rows[:t + 1]], [r[qw + kw:] for r in rows[:t + 1]],
                             q_heads, kv_heads, hd)
            assert np.max(np.abs(got - ref)) < TOL, (i, float(np.max(np.abs(got - ref))))
    finally:
        for b in (d_k, d_v, d_len, d_row, d_out):
            b.free()


@pytest.mark.parametrize("q_heads,kv_heads,hd,max_ctx,prefix", [
    (14, 2, 64, 512, 200),      # many context splits
    (4, 4, 32, 64, 5),          # a single split: the scratch is not touched
    (8, 2, 64, 130, 128),       # the two calls fill the last two slots of the caller's cache (lengths 128 and 129)
])
def test_noalloc_step_matches_regular_step(backend, q_heads, kv_heads, hd, max_ctx, prefix):
    _run_case(backend, q_heads, kv_heads, hd, max_ctx, prefix)


def test_noalloc_rejects_shapes_beyond_the_builtin_scratch(backend):
    dummy = backend.alloc(1024)
    try:
        with pytest.raises(CaiError, match="scratch"):
            backend._check(backend.lib.cai_sdpa_step_noalloc(backend.ctx, dummy.ptr, dummy.ptr, dummy.ptr, dummy.ptr,
                                                             128, 1, 256, 1 << 20, dummy.ptr))
    finally:
        dummy.free()


def test_noalloc_refuses_a_full_cache_without_touching_it(backend):
    """*cache_len_dev == max_ctx leaves no room for the appended row: the kernels must touch neither cache nor output
    and the next cai_dev_sync must report CAI_ERR_STATE; the call after that works again."""
    lib = backend.lib
    q_heads, kv_heads, hd, max_ctx = 4, 2, 64, 16
    qw, kw = q_heads * hd, kv_heads * hd
    rng = np.random.default_rng(3)
    row = rng.standard_normal(qw + 2 * kw).astype(np.float32)
    kc = rng.standard_normal((kv_heads, max_ctx, hd)).astype(np.float32)
    vc = rng.standard_normal((kv_heads, max_ctx, hd)).astype(np.float32)
    sentinel = np.full(qw, 7.0, dtype=np.float32)
    d_k, d_v, d_row, d_out = backend.to_device(kc), backend.to_device(vc), backend.to_device(row), backend.to_device(sentinel)
    d_len = backend.to_device(np.asarray([max_ctx], dtype=np.int32))
    try:
        for bad in (max_ctx, -1):
            d_len.write(np.asarray([bad], dtype=np.int32))
            backend._check(lib.cai_sdpa_step_noalloc(backend.ctx, d_row.ptr, d_k.ptr, d_v.ptr, d_len.ptr,
                                                     q_heads, kv_heads, hd, max_ctx, d_out.ptr))
            with pytest.raises(CaiError) as ei:
                backend.sync()
            assert ei.value.status == 4          # CAI_ERR_STATE
            assert np.array_equal(d_out.read(np.float32, qw), sentinel)
            assert np.array_equal(d_k.read(np.float32, kc.size).reshape(kc.shape), kc)
            assert np.array_equal(d_v.read(np.float32, vc.size).reshape(vc.shape), vc)
        # the last valid slot still works afterwards
        d_len.write(np.asarray([max_ctx - 1], dtype=np.int32))
        backend._check(lib.cai_sdpa_step_noalloc(backend.ctx, d_row.ptr, d_k.ptr, d_v.ptr, d_len.ptr,
                                                 q_heads, kv_heads, hd, max_ctx, d_out.ptr))
        backend.sync()
        ks = [kc[:, t, :].reshape(-1) for t in range(max_ctx - 1)] + [row[qw:qw + kw]]
        vs = [vc[:, t, :].reshape(-1) for t in range(max_ctx - 1)] + [row[qw + kw:]]
        ref = _attn_fp64(row[:qw], ks, vs, q_heads, kv_heads, hd)
        assert np.max(np.abs(d_out.read(np.float32, qw) - ref)) < TOL
    finally:
        for b in (d_k, d_v, d_len, d_row, d_out):
            b.free()
