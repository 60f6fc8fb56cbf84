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
from oracle.forward import (LlamaConfig, OracleModel, OracleSession, rms_norm, rope_interleaved, router_gates, softmax_row,  # noqa: E402
                            swiglu)


def allreduce(a):
    t = torch.from_numpy(np.ascontiguousarray(a))
    dist.all_reduce(t)
    return t.numpy()


def expert_parallel_check(rank, world):
    """The expert-parallel exchange of one mixture-of-experts layer, replayed with numpy and gloo: every rank owns
    its tokens and a share of the experts; rows [h | ids | gates] are all-gathered, each rank runs the pairs of ITS
    experts for ALL tokens (grouped by expert like the device does), combines them per token, and a reduce-scatter
    returns the sums to the tokens' owners. Must equal the unsharded oracle arithmetic."""
    H, I, E, K, per_rank = 32, 16, 8, 2, 3
    rng = np.random.default_rng(11)         # same seed on every rank: same weights, same tokens
    router = (rng.standard_normal((E, H)) * 0.3).astype(np.float32)
    experts = [dict(up=(rng.standard_normal((I, H)) * 0.2).astype(np.float32), gate=(rng.standard_normal((I, H)) * 0.2).astype(np.float32),
                    down=(rng.standard_normal((H, I)) * 0.2).astype(np.float32)) for _ in range(E)]
    h_all = rng.standard_normal((per_rank * world, H)).astype(np.float32)
    mine = slice(rank * per_rank, (rank + 1) * per_rank)
    # local routing, packed rows, all-gather
    rows = []
    for h in h_all[mine]:
        order, gates = router_gates(softmax_row(router @ h), K, True)
        rows.append(np.concatenate([h, order.astype(np.int32).view(np.float32), gates.astype(np.float32)]))
    packed = torch.from_numpy(np.stack(rows).astype(np.float32))
    gathered = [torch.zeros_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed)
    allrows = np.concatenate([t.numpy() for t in gathered])
    ids = allrows[:, H:H + K].copy().view(np.int32)
    gates = allrows[:, H + K:H + 2 * K]
    assert np.array_equal(allrows[:, :H], h_all)
    lo, hi = parallel.ep_expert_range(E, rank, world)
    pair_out = np.zeros((per_rank * world * K, H), np.float32)
    seen = 0
    for e, pairs in parallel.ep_group_pairs(ids.reshape(-1), lo, hi, tile_rows=4):
        assert lo <= e < hi and 0 < len(pairs) <= 4
        for p in pairs:
            hrow = allrows[p // K, :H]
            fused = np.concatenate([experts[e]["up"] @ hrow, experts[e]["gate"] @ hrow])
            pair_out[p] = experts[e]["down"] @ swiglu(fused, I)
            seen += 1
    assert seen == int(np.sum((ids >= lo) & (ids < hi)))
    part = np.zeros((per_rank * world, H), np.float32)
    for t in range(per_rank * world):
        for k in range(K):
            if lo <= ids[t, k] < hi:
                part[t] += gates[t, k] * pair_out[t * K + k]
    out = torch.zeros(per_rank, H)
    dist.reduce_scatter(out, [torch.from_numpy(part[r * per_rank:(r + 1) * per_rank].copy()) for r in range(world)])
    # unsharded oracle arithmetic for my tokens
    for i, h in enumerate(h_all[mine]):
        order, g = router_gates(softmax_row(router @ h), K, True)
        y = np.zeros(H, np.float32)
        for e_id, gate in zip(order, g):
            ex = experts[int(e_id)]
            fused = np.concatenate([ex["up"] @ h, ex["gate"] @ h])
            y = y + gate * (ex["down"] @ swiglu(fused, I))
        assert float(np.max(np.abs(out[i].numpy() - y))) < 1e-5


def expert_parallel_peer_exchange_check(rank, world):
    """The dispatch / combine rule of the peer-memory exchange (ep_dispatch_kernel / ep_combine_kernel), replayed with numpy:
    a rank reads the ids and gates of every token but the hidden row only of tokens that route to one of ITS experts, and
    a token's owner adds, in rank order, only the partial sums of ranks that host one of the token's experts. Whatever the
    rule says is not read is poisoned with NaN here, so a use of it would show. Must equal the unsharded oracle arithmetic."""
    H, I, E, K, per_rank = 32, 16, 8, 2, 3
    rng = np.random.default_rng(12)
    router = (rng.standard_normal((E, H)) * 0.3).astype(np.float32)
    experts = [dict(up=(rng.standard_normal((I, H)) * 0.2).astype(np.float32), gate=(rng.standard_normal((I, H)) * 0.2).astype(np.float32),
                    down=(rng.standard_normal((H, I)) * 0.2).astype(np.float32)) for _ in range(E)]
    h_all = rng.standard_normal((per_rank * world, H)).astype(np.float32)
    mine = slice(rank * per_rank, (rank + 1) * per_rank)
    rows = []
    for h in h_all[mine]:
        order, gates = router_gates(softmax_row(router @ h), K, True)
        rows.append(np.concatenate([h, order.astype(np.int32).view(np.float32), gates.astype(np.float32)]))
    slot = torch.from_numpy(np.stack(rows).astype(np.float32))          # this rank's dispatch slot
    slots = [torch.zeros_like(slot) for _ in range(world)]
    dist.all_gather(slots, slot)                                         # stands in for the peers' mapped slots
    lo, hi = parallel.ep_expert_range(E, rank, world)
    per = E // world
    allrows = np.full((per_rank * world, H + 2 * K), np.nan, np.float32)
    for r in range(world):
        src = slots[r].numpy()
        for t in range(per_rank):
            row = r * per_rank + t
            allrows[row, H:] = src[t, H:]                                # ids and gates: always
            ids_t = src[t, H:H + K].copy().view(np.int32)
            if np.any((ids_t >= lo) & (ids_t < hi)):
                allrows[row, :H] = src[t, :H]                            # the hidden row: only when an expert of mine is routed to
    ids = allrows[:, H:H + K].copy().view(np.int32)
    gates = allrows[:, H + K:H + 2 * K]
    part = np.zeros((per_rank * world, H), np.float32)
    pair_out = {}
    for e, pairs in parallel.ep_group_pairs(ids.reshape(-1), lo, hi, tile_rows=4):
        for p in pairs:
            hrow = allrows[p // K, :H]
            assert not np.any(np.isnan(hrow))                            # every row a tile touches was pulled
            fused = np.concatenate([experts[e]["up"] @ hrow, experts[e]["gate"] @ hrow])
            pair_out[p] = experts[e]["down"] @ swiglu(fused, I)
    for t in range(per_rank * world):
        for k in range(K):                                               # slots in order, as moe_combine_partial_kernel adds them
            if lo <= ids[t, k] < hi:
                part[t] += gates[t, k] * pair_out[t * K + k]
    cslot = torch.from_numpy(part.copy())                                # this rank's combine slot: partial sums of ALL tokens
    cslots = [torch.zeros_like(cslot) for _ in range(world)]
    dist.all_gather(cslots, cslot)
    x = np.zeros((per_rank, H), np.float32)                              # the residual stream of my tokens (zero here)
    my_ids = ids[mine]
    for t in range(per_rank):
        hosts = sorted(set(int(e) // per for e in my_ids[t]))
        for r in range(world):
            src = cslots[r].numpy().copy()
            if r not in hosts:
                src[:] = np.nan                                          # never read
                continue
            x[t] += src[rank * per_rank + t]
    for i, h in enumerate(h_all[mine]):
        order, g = router_gates(softmax_row(router @ h), K, True)
        y = np.zeros(H, np.float32)
        for e_id, gate in zip(order, g):
            ex = experts[int(e_id)]
            fused = np.concatenate([ex["up"] @ h, ex["gate"] @ h])
            y = y + gate * (ex["down"] @ swiglu(fused, I))
        assert not np.any(np.isnan(x[i]))
        assert float(np.max(np.abs(x[i] - y))) < 1e-5


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
    expert_parallel_check(rank, world)
    expert_parallel_peer_exchange_check(rank, world)
    dist.barrier()
    if rank == 0:
        print("DIST_CPU_OK")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
