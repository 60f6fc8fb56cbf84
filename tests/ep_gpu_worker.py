"""Worker of the multi-GPU expert-parallel test: every rank builds the same synthetic mixture-of-experts model with
its own share of the experts and decodes its own sequences; rank 0 also runs ALL sequences through the unsharded
model on its own GPU. Every rank's logits and greedy tokens must equal the single-GPU rows of its sequences.
Launched by torch.distributed.run, one process per GPU."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402,F401  (first: its NCCL is the one the process loads)
from neural_api_b200 import parallel  # noqa: E402
from neural_api_b200.backend import CudaBackend, LlamaModel, StreamingDecoder, make_config, TYPE_Q8_0  # noqa: E402


def main():
    rank, world, local_rank, dist = parallel.init_process_group("cpu:gloo,cuda:nccl")
    backend = CudaBackend(local_rank)
    uid = backend.comm_unique_id() if rank == 0 else bytes(128)
    uid = parallel.broadcast_bytes(dist, uid, src=0, length=128)
    backend.comm_init(rank, world, uid)
    kw = dict(hidden=256, inter=512, layers=2, heads=4, kv_heads=2, head_dim=64, vocab=512, rms_eps=1e-5, rope_theta=1e4,
              qk_norm=True, n_experts=8, top_k=2, norm_topk=True, moe_inter=128)
    cfg = make_config(**kw)
    model = LlamaModel(backend, cfg, ep_rank=rank, ep_size=world)
    model.init_synthetic(TYPE_Q8_0, seed=5, std=0.05)
    model.finalize()
    per_rank, steps = 3, 8
    rng = np.random.default_rng(1)
    prompt_all = rng.integers(0, kw["vocab"], (per_rank * world, 6)).astype(np.int32)
    prompt = prompt_all[rank * per_rank:(rank + 1) * per_rank]
    sess = StreamingDecoder(model, 32, batch=per_rank)
    sess.prefill(prompt[:, :-1])
    tok = prompt[:, -1].copy()
    my_logits, my_tokens = [], []
    for _ in range(steps):
        logits, amax = sess.step_forward(tok)
        my_logits.append(logits.copy())
        tok = amax.copy()
        my_tokens.append(tok.copy())
    sess.close()
    model.close()
    # every rank checks its own rows against the unsharded model (built on this rank's GPU, after the EP model is gone)
    single = CudaBackend(local_rank)
    m1 = LlamaModel(single, cfg)
    m1.init_synthetic(TYPE_Q8_0, seed=5, std=0.05)
    m1.finalize()
    s1 = StreamingDecoder(m1, 32, batch=per_rank)
    s1.prefill(prompt[:, :-1])
    tok = prompt[:, -1].copy()
    worst, ok = 0.0, 1.0
    for i in range(steps):
        logits, amax = s1.step_forward(tok)
        rms = float(np.sqrt(np.mean(logits.astype(np.float64) ** 2)))
        worst = max(worst, float(np.max(np.abs(logits - my_logits[i]))) / rms)
        if not np.array_equal(amax, my_tokens[i]):
            ok = 0.0
        tok = amax.copy()
    if worst > 1e-4:
        ok = 0.0
    print("EP rank %d worst relative logit difference %.3e over %d ranks" % (rank, worst, world), flush=True)
    s1.close()
    m1.close()
    single.close()
    bad = parallel.sum_over_ranks(dist, 1.0 - ok)
    backend.close()
    if rank == 0:
        print("EP_GPU_OK" if bad < 0.5 else "EP_GPU_MISMATCH")
    dist.destroy_process_group()
    return 0 if bad < 0.5 else 1


if __name__ == "__main__":
    sys.exit(main())
