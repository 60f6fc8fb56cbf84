"""Worker of the world_size-2 CPU test (gloo): the tensor-parallel sharding arithmetic the CUDA
backend uses (column-split q/k/v/up/gate/head, row-split o/down, sum over ranks with the residual
added on rank 0 only), replayed with the numpy oracle's operators and a gloo all_reduce, must equal
the unsharded oracle. Also exercises the rendezvous helpers. Launched by torch.distributed.run."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from neural_api_b200 import parallel  # noqa: E402
from oracle.forward import (LlamaConfig, OracleModel, OracleSession, rms_norm, rope_interleaved, swiglu)  # noqa: E402


def allreduce(a):
    t = torch.from_numpy(np.ascontiguousarray(a))
    dist.all_reduce(t)
    return t.numpy()


def main():
    rank, world, local_rank, d = parallel.init_process_group("gloo")
    assert d is not None and world == 2
    # rendezvous helpers
    payload = bytes(range(128)) if rank == 0 else bytes(128)
    assert parallel.broadcast_bytes(d, payload, src=0, length=128) == bytes(range(128))
    assert parallel.max_over_ranks(d, float(rank + 1)) == 2.0
    assert parallel.sum_over_ranks(d, 1.0) == 2.0
    covered = []
    for r in range(world):
        covered += list(range(*parallel.shard_range(17, r, world)))
    assert covered == list(range(17))

    cfg = LlamaConfig(hidden=64, inter=128, layers=2, heads=4, kv_heads=2, head_dim=32, vocab=96, rms_eps=1e-6,
                      rope_theta=1e4, qkv_bias=True)
    rng = np.random.default_rng(5)          # same seed on both ranks
    model = OracleModel(cfg, np.float32)
    H, I, qw, kw = cfg.hidden, cfg.inter, cfg.q_width, cfg.kv_width
    g = lambda *s: (rng.standard_normal(s) * 0.1).astype(np.float32)
    model.embed = g(cfg.vocab, H)
    model.lm_head = g(cfg.vocab, H)
    model.final_norm = (1 + g(H)).astype(np.float32)
    for b in model.blocks:
        b.update(attn_norm=(1 + g(H)), ffn_norm=(1 + g(H)), wq=g(qw, H), wk=g(kw, H), wv=g(kw, H), wo=g(H, qw),
                 bq=g(qw), bk=g(kw), bv=g(kw), w_up=g(I, H), w_gate=g(I, H), w_down=g(H, I))
    plan = parallel.tp_shard_plan(H, I, cfg.heads, cfg.kv_heads, cfg.head_dim, cfg.vocab, rank, world)
    hd = cfg.head_dim
    heads_l, kvh_l = cfg.heads // world, cfg.kv_heads // world
    group = cfg.heads // cfg.kv_heads
    max_ctx = 8
    kc = np.zeros((cfg.layers, kvh_l, max_ctx, hd), np.float32)
    vc = np.zeros_like(kc)
    full = OracleSession(model, max_ctx)
    tokens = [3, 17, 42, 9, 77]
    for pos, tok in enumerate(tokens):
        x = model.embed[tok].copy()
        for li, b in enumerate(model.blocks):
            h = rms_norm(x, b["attn_norm"], cfg.rms_eps)
            q = b["wq"][slice(*plan["q_rows"])] @ h + b["bq"][slice(*plan["q_rows"])]
            k = b["wk"][slice(*plan["k_rows"])] @ h + b["bk"][slice(*plan["k_rows"])]
            v = b["wv"][slice(*plan["v_rows"])] @ h + b["bv"][slice(*plan["v_rows"])]
            q = rope_interleaved(q, pos, model.theta, hd)
            k = rope_interleaved(k, pos, model.theta, hd)
            kc[li, :, pos] = k.reshape(kvh_l, hd)
            vc[li, :, pos] = v.reshape(kvh_l, hd)
            att = np.empty(heads_l * hd, np.float32)
            for hq in range(heads_l):
                gq = hq // group
                s = (kc[li, gq, :pos + 1] @ q[hq * hd:(hq + 1) * hd]) * np.float32(1 / np.sqrt(hd))
                e = np.exp(s - s.max())
                att[hq * hd:(hq + 1) * hd] = (e @ vc[li, gq, :pos + 1]) / e.sum()
            part = b["wo"][:, slice(*plan["o_cols"])] @ att
            if rank == 0:
                part = part + x                       # residual rides on one rank only
            x = allreduce(part.astype(np.float32))
            h = rms_norm(x, b["ffn_norm"], cfg.rms_eps)
            fused = np.concatenate([b["w_up"][slice(*plan["up_rows"])] @ h, b["w_gate"][slice(*plan["gate_rows"])] @ h])
            act = swiglu(fused, fused.shape[0] // 2)
            part = b["w_down"][:, slice(*plan["down_cols"])] @ act
            if rank == 0:
                part = part + x
            x = allreduce(part.astype(np.float32))
        h = rms_norm(x, model.final_norm, cfg.rms_eps)
        shard = model.lm_head[slice(*plan["head_rows"])] @ h
        gathered = [torch.zeros(shard.shape[0]) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(shard.astype(np.float32)))
        logits = np.concatenate([t.numpy() for t in gathered])
        ref = full.step(tok, pos)
        err = float(np.max(np.abs(logits - ref)))
        assert err < 1e-5, (pos, err)
    dist.barrier()
    if rank == 0:
        print("DIST_CPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
