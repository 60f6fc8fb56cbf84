"""Isolated decode-attention benchmark: `layers` KV caches of one model shape are filled to `ctx - 1` rows through
the layer-granular entry point (cai_sdpa_step_dev), then one step at full context is timed per layer, rotating over
the layers so that the caches (layers x 2 x kv_heads x ctx x head_dim x 4 bytes, chosen larger than L2) stream from
HBM as they do inside a model step.

    python -m neural_api_b200.bench_attention --q-heads 40 --kv-heads 8 --head-dim 128 --ctx 8192 --layers 6

Each timed step is three launches (RoPE + append, split-context decode, combine) issued from Python, so short
contexts measure launch latency; the marginal time per cached row is the kernel's.
"""
import argparse
import json

import numpy as np

from .backend import CudaBackend, FusedSDPA


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--q-heads", type=int, default=40)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=6)
    ap.add_argument("--reps", type=int, default=8)
    a = ap.parse_args()
    b = CudaBackend(0)
    rng = np.random.default_rng(0)
    row = rng.standard_normal((a.q_heads + 2 * a.kv_heads) * a.head_dim).astype(np.float32)
    din = b.to_device(row)
    dout = b.alloc(a.q_heads * a.head_dim * 4)
    layers = []
    for _ in range(a.layers):
        s = FusedSDPA(b, a.q_heads, a.kv_heads, a.head_dim)
        s.begin_incremental_decode(a.ctx)
        layers.append(s)
        for _ in range(a.ctx - 1):
            b._check(b.lib.cai_sdpa_step_dev(s.handle, din.ptr, dout.ptr))
    b.sync()
    times = []
    for _ in range(a.reps):
        for s in layers:
            s.truncate_cache(a.ctx - 1)
        b.sync()
        b.timer_begin()
        for s in layers:
            b._check(b.lib.cai_sdpa_step_dev(s.handle, din.ptr, dout.ptr))
        times.append(b.timer_end() / a.layers)
    times = sorted(times)[1:-1] if len(times) > 2 else times
    ms = float(np.mean(times))
    kv_bytes = 2.0 * a.kv_heads * a.ctx * a.head_dim * 4
    print(json.dumps({"workload": "decode attention q%d kv%d hd%d ctx %d, %d layer caches" % (a.q_heads, a.kv_heads, a.head_dim, a.ctx, a.layers),
                      "us_per_layer_step": ms * 1000.0, "kv_bytes_per_layer": kv_bytes, "gbs": kv_bytes / ms / 1e6}))
    for s in layers:
        s.end_incremental_decode()
    din.free()
    dout.free()


if __name__ == "__main__":
    main()
