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
    finally:
        for b in (d_k, d_v, d_len, d_row, d_out):
            b.free()


@pytest.mark.parametrize("q_heads,kv_heads,hd,max_ctx,prefix", [
    (14, 2, 64, 512, 200),      # many context splits
    (4, 4, 32, 64, 5),          # a single split: the scratch is not touched
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
