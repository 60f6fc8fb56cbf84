"""Host-side plumbing for multi-GPU runs: one process per GPU, torch.distributed
only for rendezvous (rank discovery, handing the communicator id around,
barriers, max-over-ranks timing). The data path never goes through torch.

The reference is single-process / single-device; everything here is new surface.
"""
import os


def env_rank_world():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))


def shard_range(total, rank, world):
    """Contiguous [begin, end) of `total` units owned by `rank` (first ranks take the remainder)."""
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


def tp_shard_plan(hidden, inter, heads, kv_heads, head_dim, vocab, rank, world):
    """Slices of every matrix a tensor-parallel rank keeps. Column-parallel matrices
    (q, k, v, up, gate, lm_head) are split by OUTPUT rows, row-parallel ones (o, down)
    by INPUT columns; after o and down the partial [batch, hidden] results are summed
    over ranks (rank 0 alone adds the residual before the sum). Mirrors the slicing
    cai_model_upload_tensor performs."""
    for name, v in (("heads", heads), ("kv_heads", kv_heads), ("inter", inter), ("vocab", vocab)):
        if v % world:
            raise ValueError("%s=%d does not divide by tp size %d" % (name, v, world))
    qw, kw, il, vl = heads // world * head_dim, kv_heads // world * head_dim, inter // world, vocab // world
    if (qw % 32) or (il % 32):
        raise ValueError("row-parallel shards must be multiples of the 32-element quant block")
    return {
        "q_rows": (rank * qw, (rank + 1) * qw),
        "k_rows": (rank * kw, (rank + 1) * kw),
        "v_rows": (rank * kw, (rank + 1) * kw),
        "o_cols": (rank * qw, (rank + 1) * qw),
        "up_rows": (rank * il, (rank + 1) * il),
        "gate_rows": (rank * il, (rank + 1) * il),
        "down_cols": (rank * il, (rank + 1) * il),
        "head_rows": (rank * vl, (rank + 1) * vl),
    }


def init_process_group(backend=None):
    """Joins the torch.distributed group described by the torchrun environment.
    Returns (rank, world, local_rank, dist or None)."""
    rank, world, local_rank = env_rank_world()
    if world == 1:
        return rank, world, local_rank, None
    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend=backend or "gloo")
    return rank, world, local_rank, dist


def broadcast_bytes(dist, payload, src=0, length=128):
    """Hands `length` bytes from rank `src` to every rank (the NCCL unique id)."""
    import torch
    t = torch.zeros(length, dtype=torch.uint8)
    if dist.get_rank() == src:
        t = torch.tensor(list(payload), dtype=torch.uint8)
    dist.broadcast(t, src=src)
    return bytes(t.tolist())


def max_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(dist, value):
    if dist is None:
        return value
    import torch
    t = torch.tensor([float(value)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def ep_expert_range(n_experts, rank, world):
    """Experts [lo, hi) that rank `rank` of an expert-parallel group keeps (the rule of cai_model_create_ep)."""
    if world < 1 or n_experts % world:
        raise ValueError("n_experts %d does not divide over %d ranks" % (n_experts, world))
    per = n_experts // world
    return rank * per, (rank + 1) * per


def ep_group_pairs(expert_ids, lo, hi, tile_rows=16):
    """Host mirror of the device grouping (op_moe_group): the (token, slot) pairs whose expert lies in [lo, hi),
    grouped by expert in index order and cut into tiles of at most tile_rows pairs; pairs keep their order inside an
    expert. Returns a list of (expert, [pair indices])."""
    tiles = []
    flat = [int(e) for e in expert_ids]
    for e in range(lo, hi):
        mine = [i for i, v in enumerate(flat) if v == e]
        for k in range(0, len(mine), tile_rows):
            tiles.append((e, mine[k:k + tile_rows]))
    return tiles
