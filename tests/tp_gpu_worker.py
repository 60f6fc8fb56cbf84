"""Worker of the multi-GPU tensor-parallel test: every rank builds its shard of the same synthetic
model; rank 0 also builds the unsharded model on its own GPU. N-GPU logits and greedy tokens must
equal the 1-GPU result. Launched by torch.distributed.run, one process per GPU."""
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
    kw = dict(hidden=1024, inter=2048, layers=3, heads=16, kv_heads=8, head_dim=64, vocab=4096, rms_eps=1e-6,
              rope_theta=1e6, qkv_bias=True)
    cfg = make_config(**kw)
    model = LlamaModel(backend, cfg, tp_rank=rank, tp_size=world)
    model.init_synthetic(TYPE_Q8_0, seed=7, std=0.02)
    model.finalize()
    batch, steps = 2, 12
    sess = StreamingDecoder(model, 64, batch=batch)
    rng = np.random.default_rng(1)
    prompt = rng.integers(0, kw["vocab"], (batch, 9)).astype(np.int32)
    sess.prefill(prompt[:, :-1])
    tok = prompt[:, -1].copy()
    tp_logits, tp_tokens = [], []
    for _ in range(steps):
        logits, amax = sess.step_forward(tok)
        tp_logits.append(logits.copy())
        tok = amax.copy()
        tp_tokens.append(tok.copy())
    dev_tokens = sess.decode_greedy(tok, 4)           # the on-device greedy loop under TP
    sess.close()
    # one sequence: the persistent step kernel, whose sums over the ranks happen inside the kernel (peer loads)
    os.environ["CAI_STEP_KERNEL"] = "1"
    sess1 = StreamingDecoder(model, 64, batch=1)
    used_step_kernel = sess1.uses_step_kernel
    sess1.prefill(prompt[:1, :-1])
    tok1 = prompt[:1, -1].copy()
    sk_logits, sk_tokens = [], []
    for _ in range(steps):
        logits, amax = sess1.step_forward(tok1)
        sk_logits.append(logits.copy())
        tok1 = amax.copy()
        sk_tokens.append(tok1.copy())
    sk_dev = sess1.decode_greedy(tok1, 4)
    sess1.close()
    os.environ.pop("CAI_STEP_KERNEL", None)
    model.close()
    ok = 1.0
    if rank == 0:
        single = CudaBackend(local_rank)
        m1 = LlamaModel(single, cfg)
        m1.init_synthetic(TYPE_Q8_0, seed=7, std=0.02)
        m1.finalize()
        s1 = StreamingDecoder(m1, 64, batch=batch)
        s1.prefill(prompt[:, :-1])
        tok = prompt[:, -1].copy()
        worst = 0.0
        for i in range(steps):
            logits, amax = s1.step_forward(tok)
            rms = float(np.sqrt(np.mean(logits.astype(np.float64) ** 2)))
            worst = max(worst, float(np.max(np.abs(logits - tp_logits[i]))) / rms)
            if not np.array_equal(amax, tp_tokens[i]):
                ok = 0.0
            tok = amax.copy()
        ref_dev = s1.decode_greedy(tok, 4)
        if not np.array_equal(ref_dev, dev_tokens):
            ok = 0.0
        if worst > 1e-4:
            ok = 0.0
        print("TP worst relative logit difference %.3e over %d ranks" % (worst, world))
        # the one-sequence session against the single-GPU launch-per-operator path
        os.environ["CAI_STEP_KERNEL"] = "0"
        s2 = StreamingDecoder(m1, 64, batch=1)
        os.environ.pop("CAI_STEP_KERNEL", None)
        s2.prefill(prompt[:1, :-1])
        tok = prompt[:1, -1].copy()
        worst1 = 0.0
        for i in range(steps):
            logits, amax = s2.step_forward(tok)
            rms = float(np.sqrt(np.mean(logits.astype(np.float64) ** 2)))
            worst1 = max(worst1, float(np.max(np.abs(logits - sk_logits[i]))) / rms)
            if not np.array_equal(amax, sk_tokens[i]):
                ok = 0.0
            tok = amax.copy()
        if not np.array_equal(s2.decode_greedy(tok, 4), sk_dev):
            ok = 0.0
        s2.close()
        uses_peer = os.environ.get("CAI_TP_ALLREDUCE", "") != "nccl"
        if worst1 > 1e-4 or (uses_peer and not used_step_kernel):
            ok = 0.0
        print("TP step kernel (%s) worst relative logit difference %.3e" % ("on" if used_step_kernel else "off", worst1))
        s1.close()
        m1.close()
        single.close()
    # a failure on ANY rank fails the test: count the ranks that saw one (rank 0 holds the comparison; every rank
    # reports a raised device error word through the exception its failing call threw)
    bad = parallel.sum_over_ranks(dist, 1.0 - ok)
    backend.close()
    if rank == 0:
        print("TP_GPU_OK" if bad < 0.5 else "TP_GPU_MISMATCH")
    dist.destroy_process_group()
    return 0 if bad < 0.5 else 1


if __name__ == "__main__":
    sys.exit(main())
