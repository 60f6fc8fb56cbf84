#!/usr/bin/env python3
"""Decode-throughput benchmark of the CUDA backend.

    python bench.py --gpus 1 --steps 32 --warmup 4
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...        # the CPU restatement of the reference path

A step is one greedy decode step (one token per sequence) of the workload through the
whole layer stack. Default workload: Qwen2.5-32B-shaped dense model, Q8_0 weights
(synthetic N(0, 0.02), seed 3), batch 1, context 8192 filled from random prompt tokens by
cai_session_prefill (64 / batch positions per sequence and step on the tensor-core path; tests hold it
equal to the reference's token-at-a-time prefill), fp32 KV cache; with N > 1 GPUs the attention heads and MLP
columns/rows are sharded tensor-parallel (strong scaling: the job is the same at every N).
The line's `also` block (one GPU) adds the other configurations as side measurements on the same box: Qwen2.5-0.5B
batch 1, TinyLlama-1.1B Q4_0 with 16 sequences, OLMoE-1B-7B batch 64, and the 32B model at batch 64 with the int8 cache.
`--workload linear` is the isolated quantized linear layer, `--workload attention` the isolated decode attention.
Prints ONE JSON line on rank 0.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
import zlib

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

TYPE_BPW = {8: 34.0 / 32.0, 2: 18.0 / 32.0}          # Q8_0, Q4_0 bytes per weight
# DRAM traffic per algorithmic byte, from ncu captures (dram__bytes_read.sum + dram__bytes_write.sum per launch against the
# bytes the launch has to move): the per-operator GEMV on 5120 x 27648 Q8_0 read 150.476 MB and wrote 5.032 MB for
# 150.502 MB of codes and scales; STEP_KERNEL_TRAFFIC is the same ratio for one launch of the persistent step kernel
# (weights + cached K and V rows) on a depth-cut model.
GEMV_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0332
STEP_KERNEL_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.0042    # 1898.532 MB read + 6.480 MB written for 1896.989 MB (2-layer cut, context 2048)
WORKLOAD_DEFAULTS = {
    # arch: (ggml type, seed, batch, context)
    "qwen2.5-32b": (8, 3, 1, 8192),
    "qwen2.5-0.5b": (8, 0, 1, 256),
    "tinyllama-1.1b": (2, 1, 16, 768),
    "olmoe-1b-7b": (8, 2, 64, 2048),
}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device), "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()           # the exact child started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        clocks, reasons = [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 8:
                    continue
                try:
                    clocks.append(float(parts[0]))
                    out["sm_max_mhz"] = float(parts[1])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[4:8]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if clocks:
            out["sm_mhz"] = float(np.median(clocks))
            out["samples"] = len(clocks)
        out["reasons"] = sorted(reasons)
        return out


# --------------------------------------------------------------------------------------
# CPU baseline: the C (AVX2 + OpenMP) restatement of the reference path, bounded sample
# --------------------------------------------------------------------------------------
def _random_blocks(ggml_type, rows, cols, rng, pool):
    """GGUF rows of random codes with sane fp16 scales, tiled from a random pool (values do not
    affect timing; scales are kept finite and small)."""
    nblk = rows * cols // 32
    bb = 34 if ggml_type == 8 else 18
    reps = (nblk * bb + pool.size - 1) // pool.size
    raw = np.tile(pool, reps)[:nblk * bb].reshape(nblk, bb).copy()
    raw[:, 0] = rng.integers(0, 256, 1, dtype=np.uint8)[0]
    raw[:, 1] = 0x10                                  # fp16 exponent ~2^-11: scale ~ 5e-4
    return raw.reshape(-1)


class CpuSample:
    """A few layers + LM head of the workload on the host cores; one step = one token."""

    def __init__(self, arch_kw, ggml_type, ctx):
        from oracle import c_oracle
        self.c = c_oracle
        # all the host threads this process may use, whatever OMP_NUM_THREADS says (torchrun sets it to 1)
        try:
            usable = len(os.sched_getaffinity(0))
        except AttributeError:
            usable = os.cpu_count() or 1
        c_oracle.set_num_threads(usable)
        kw = arch_kw
        if kw.get("n_experts", 0):
            raise RuntimeError("the C restatement covers dense models")
        from neural_api_b200.configs import step_weight_bytes
        full_bytes = step_weight_bytes(kw, TYPE_BPW[ggml_type])
        self.full_layers = kw["layers"]
        self.layers = kw["layers"] if full_bytes < (2 << 30) else 2
        rng = np.random.default_rng(0)
        pool = rng.integers(0, 256, 8 << 20, dtype=np.uint8)
        H, I = kw["hidden"], kw["inter"]
        qw, kvw = kw["heads"] * kw["head_dim"], kw["kv_heads"] * kw["head_dim"]
        m = c_oracle.CModel(H, I, self.layers, kw["heads"], kw["kv_heads"], kw["head_dim"], kw["vocab"],
                            kw.get("rms_eps", 1e-5), kw.get("rope_theta", 1e4), tie_embeddings=True,
                            qkv_bias=kw.get("qkv_bias", False))
        ones = np.ones(H, dtype=np.float32)
        m.set_tensor("embed", 0, ggml_type, _random_blocks(ggml_type, kw["vocab"], H, rng, pool))
        m.set_tensor("final_norm", 0, 0, ones)
        for l in range(self.layers):
            m.set_tensor("attn_norm", l, 0, ones)
            m.set_tensor("ffn_norm", l, 0, ones)
            for kind, rows, cols in (("q", qw, H), ("k", kvw, H), ("v", kvw, H), ("o", H, qw), ("up", I, H),
                                     ("gate", I, H), ("down", H, I)):
                m.set_tensor(kind, l, ggml_type, _random_blocks(ggml_type, rows, cols, rng, pool))
            if kw.get("qkv_bias", False):
                m.set_tensor("bq", l, 0, np.zeros(qw, dtype=np.float32))
                m.set_tensor("bk", l, 0, np.zeros(kvw, dtype=np.float32))
                m.set_tensor("bv", l, 0, np.zeros(kvw, dtype=np.float32))
        self.model = m
        self.ctx = ctx
        self.sess = c_oracle.CSession(m, ctx + 4)
        self.sess.assume_len(ctx)
        self.cores = c_oracle.num_threads()
        self.desc = ("%d of %d layers + LM head at context %d, AVX2+OpenMP C restatement of the reference CPU path, "
                     "layer time scaled x%g" % (self.layers, self.full_layers, ctx, self.full_layers / self.layers))
        self.extrapolated = self.layers != self.full_layers
        self.last_measured_s = 0.0

    def step_seconds(self):
        """Seconds one full decode step would take: sampled layers scaled to the full depth + head."""
        s = self.sess
        s.assume_len(self.ctx)
        t0 = time.perf_counter()
        s.step(1, self.ctx, want_logits=False)
        t1 = time.perf_counter()
        s.assume_len(self.ctx)
        s.step(1, self.ctx, want_logits=True)
        t2 = time.perf_counter()
        layers_t = t1 - t0
        head_t = max((t2 - t1) - layers_t, 0.0)
        self.last_measured_s = t2 - t0                       # what actually ran: two passes over the sampled layers, one head
        return layers_t * (self.full_layers / self.layers) + head_t

    def describe(self):
        """The fields that say how much of the step was measured and how much scaled up."""
        return {"extrapolated": self.extrapolated, "layers_timed": self.layers, "layers_total": self.full_layers,
                "scale": self.full_layers / self.layers, "measured_seconds_per_sample": self.last_measured_s}

    def close(self):
        self.sess.close()
        self.model.close()


def run_reference(args, arch_kw, ggml_type, batch, ctx):
    """--impl reference: the reference's CPU algorithm on the host cores, all threads."""
    sample = CpuSample(arch_kw, ggml_type, ctx)
    for _ in range(args.warmup):
        sample.step_seconds()
    times = [sample.step_seconds() for _ in range(args.steps)]
    extra = sample.describe()
    sample.close()
    sec = float(np.mean(times)) * batch               # sequences run one after another on the CPU path
    value = batch / sec
    line = {
        "impl": "reference", "metric": "decode_tokens_per_s", "value": value, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak" if (args.gpus > 1 and parallel_mode(args) == "dp") else "strong",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, arch_kw, ggml_type, batch, ctx, 1),
        "cpu_baseline": dict({"value": value, "unit": "tokens/s", "cores": sample.cores, "kind": "port", "sample": sample.desc}, **extra),
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    line.update(extra)
    print(json.dumps(line))


def parallel_mode(args):
    if args.parallel != "auto":
        return args.parallel
    return {"qwen2.5-32b": "tp", "olmoe-1b-7b": "ep"}.get(args.workload, "dp")


def workload_config(args, arch_kw, ggml_type, batch, ctx, world):
    return {"workload": "%s-architecture%s %s decode, batch %d%s, context %d, %s KV, fp32 activations"
                        % (args.workload, (" cut to %d layers" % args.layers) if getattr(args, "layers", None) else "",
                           {8: "Q8_0", 2: "Q4_0"}[ggml_type], batch,
                           " per GPU" if (world > 1 and parallel_mode(args) == "dp") else "", ctx,
                           "int8" if getattr(args, "kv", "f32") == "int8" else "fp32"),
            "batch": batch, "context": ctx, "weights": {8: "Q8_0", 2: "Q4_0"}[ggml_type],
            "parallelism": ("%s%d" % (parallel_mode(args), world)) if world > 1 else "single",
            "l2": "inputs larger than L2 (weights streamed once per step)"}


def build_model(backend, rank, world, arch, ggml_type, seed, mode):
    """The synthetic model of a workload: N(0, 0.02) weights from the device generator (keyed by the global element index,
    so shards hold exactly the slices of the unsharded model), quantized on the device."""
    from neural_api_b200.backend import LlamaModel
    from neural_api_b200.configs import arch_config
    tp = world if (world > 1 and mode == "tp") else 1
    ep = world if (world > 1 and mode == "ep") else 1
    model = LlamaModel(backend, arch_config(arch), tp_rank=rank if tp > 1 else 0, tp_size=tp, ep_rank=rank if ep > 1 else 0, ep_size=ep)
    model.init_synthetic(ggml_type, seed=seed, std=0.02)
    model.finalize()
    return model


def run_workload(backend, dist, rank, world, arch, ggml_type, seed, batch, ctx, steps, warmup, do_e2e=True, do_profile=True,
                 mode="tp", kv="f32", model=None, fill="prefill"):
    """Fills the context and measures decode steps. Returns a dict of raw numbers.
    mode "tp": one job, weights sharded over the ranks; "dp": every rank holds the whole model and decodes its own
    batch (different prompts), nothing crosses NVLink; the job's tokens/s is the sum.
    model: a model built by build_model to reuse (else one is built and closed here).
    fill "prefill": the context is produced by cai_session_prefill from random prompt tokens; "zeros": the caches are
    zeroed and declared filled (cai_session_fill_for_benchmark) where a real prefill would take minutes."""
    from neural_api_b200.backend import StreamingDecoder, TYPE_F32, TYPE_I8
    from neural_api_b200.configs import ARCHS, step_weight_bytes
    from neural_api_b200 import parallel
    kw = ARCHS[arch]
    ep = world if (world > 1 and mode == "ep") else 1
    replicas = world if (world > 1 and mode == "dp") else 1
    if ep > 1:
        if batch % ep:
            raise SystemExit("expert parallelism divides the batch over the GPUs: %d sequences, %d GPUs" % (batch, ep))
        batch = batch // ep                   # this rank's sequences; the job's batch is unchanged
        replicas = ep
    own_model = model is None
    if own_model:
        model = build_model(backend, rank, world, arch, ggml_type, seed, mode)
    prof_steps = 2 if do_profile else 0
    max_ctx = ctx + warmup + steps * (2 if do_e2e else 1) + prof_steps + 8
    sess = StreamingDecoder(model, max_ctx, batch=batch, kv_type=TYPE_I8 if kv == "int8" else TYPE_F32)
    rng = np.random.default_rng(seed + (rank if replicas > 1 else 0))   # every replica / expert-parallel rank has its own prompts
    prompt = rng.integers(0, kw["vocab"], (batch, ctx)).astype(np.int32)
    t0 = time.perf_counter()
    if fill == "zeros":
        sess.fill_for_benchmark(ctx - 1)
    elif ctx > 1:
        sess.prefill(prompt[:, :-1])
    prefill_s = time.perf_counter() - t0
    tok = prompt[:, -1].copy()

    def barrier():
        backend.sync()
        if dist is not None:
            parallel.max_over_ranks(dist, 0.0)

    out = sess.decode_greedy(tok, max(warmup, 1))
    first_tokens = [int(t) for t in out[:16, 0]]
    tok = out[-1].copy()
    launches0 = backend.launch_count()
    sampler = ClockSampler(backend.device)
    sampler.start()
    barrier()
    backend.timer_begin()
    out = sess.decode_greedy(tok, steps)
    ms = backend.timer_end()
    barrier()
    clocks = sampler.stop()
    launches = backend.launch_count() - launches0
    ms = parallel.max_over_ranks(dist, ms)
    first_tokens = (first_tokens + [int(t) for t in out[:, 0]])[:16]
    tok = out[-1].copy()
    res = {"ms_total": ms, "ms_per_step": ms / steps, "tokens_per_s": steps * batch * replicas / (ms * 1e-3), "launches": launches,
           "clocks": clocks, "prefill_s": prefill_s, "kv_bytes_step": sess.last_kv_bytes(),
           "weight_bytes_rank": model.step_weight_bytes(), "step_kernel": sess.uses_step_kernel,
           "weight_bytes_job": step_weight_bytes(kw, TYPE_BPW[ggml_type], tokens_per_step=batch),
           # the first 16 greedy tokens of this rank's first sequence: the weights are keyed by global index, so 1, 2, 4 and
           # 8 GPUs should print the same number unless a near-tie of two logits flips
           "tokens_crc": "%08x" % (zlib.crc32(np.asarray(first_tokens, dtype=np.int32).tobytes()) & 0xFFFFFFFF)}
    if do_e2e:
        # the reference-facing call: token ids from host memory in, logits row + argmax back out, every step
        barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            _, amax = sess.step_forward(tok, want_logits=True)
            tok = amax.copy()
        backend.sync()
        e2e_s = parallel.max_over_ranks(dist, time.perf_counter() - t0)
        res["e2e_tokens_per_s"] = steps * batch * replicas / e2e_s
        res["h2d"] = 8 * batch
        res["d2h"] = batch * kw["vocab"] * 4 + 4 * batch
    if do_profile:
        res["profile"] = sess.profile(tok, prof_steps)
        res["profile_steps"] = prof_steps
    sess.close()
    if own_model:
        model.close()
    return res


def tp_parity_check(backend, dist, rank, world, arch, ggml_type):
    """N GPUs against one GPU on a depth-cut model of the same architecture (2 layers, vocabulary cut to 8192 rows): every
    rank steps its tensor-parallel shard, rank 0 then builds the unsharded model on its own GPU and compares logits and
    greedy tokens. Returns ("ok" | "mismatch", worst relative logit difference) on every rank."""
    from neural_api_b200.backend import LlamaModel, StreamingDecoder, make_config
    from neural_api_b200.configs import ARCHS
    from neural_api_b200 import parallel
    kw = dict(ARCHS[arch], layers=2, vocab=8192)
    cfg = make_config(**kw)
    rng = np.random.default_rng(17)
    prompt = rng.integers(0, kw["vocab"], (1, 40)).astype(np.int32)
    steps = 6

    def run(model):
        sess = StreamingDecoder(model, 64)
        sess.prefill(prompt[:, :-1])
        tok = prompt[:, -1].copy()
        rows, toks = [], []
        for _ in range(steps):
            logits, amax = sess.step_forward(tok)
            rows.append(logits[0].copy())
            tok = amax.copy()
            toks.append(int(tok[0]))
        sess.close()
        return rows, toks

    model = LlamaModel(backend, cfg, tp_rank=rank, tp_size=world)
    model.init_synthetic(ggml_type, seed=5, std=0.02)
    model.finalize()
    tp_rows, tp_toks = run(model)
    model.close()
    bad, worst = 0.0, 0.0
    if rank == 0:
        single = LlamaModel(backend, cfg)
        single.init_synthetic(ggml_type, seed=5, std=0.02)
        single.finalize()
        rows, toks = run(single)
        single.close()
        for a, b in zip(tp_rows, rows):
            rms = float(np.sqrt(np.mean(b.astype(np.float64) ** 2)))
            worst = max(worst, float(np.max(np.abs(a - b))) / rms)
        if toks != tp_toks or worst > 1e-4:
            bad = 1.0
    bad = parallel.sum_over_ranks(dist, bad)
    worst = parallel.max_over_ranks(dist, worst)
    return ("ok" if bad < 0.5 else "mismatch"), worst


def run_attention(args):
    """Isolated decode attention: `layers` KV caches of one model shape are filled to ctx - 1 rows through the layer-granular
    entry point (cai_sdpa_step_dev), then one step at full context is timed per layer, rotating over the layers so that the
    caches (chosen larger than L2) stream from HBM as they do inside a model step. Each timed step is three launches
    (RoPE + append, split-context decode, merge of the splits)."""
    from neural_api_b200.backend import CudaBackend, FusedSDPA
    q_heads, kv_heads, head_dim = (int(v) for v in args.heads.lower().split("x"))
    ctx = args.ctx or 8192
    layers = args.batch or 6                               # --batch doubles as the number of layer caches here
    b = CudaBackend(0)
    rng = np.random.default_rng(0)
    row = rng.standard_normal((q_heads + 2 * kv_heads) * head_dim).astype(np.float32)
    din = b.to_device(row)
    dout = b.alloc(q_heads * head_dim * 4)
    caches = []
    for _ in range(layers):
        s = FusedSDPA(b, q_heads, kv_heads, head_dim)
        s.begin_incremental_decode(ctx)
        caches.append(s)
        for _ in range(ctx - 1):
            b._check(b.lib.cai_sdpa_step_dev(s.handle, din.ptr, dout.ptr))
    b.sync()
    times = []
    launches0 = b.launch_count()
    for _ in range(args.warmup + args.steps):
        for s in caches:
            s.truncate_cache(ctx - 1)
        b.sync()
        b.timer_begin()
        for s in caches:
            b._check(b.lib.cai_sdpa_step_dev(s.handle, din.ptr, dout.ptr))
        times.append(b.timer_end() / layers)
    launches = b.launch_count() - launches0
    ms = float(np.mean(times[args.warmup:]))
    kv_bytes = 2.0 * kv_heads * ctx * head_dim * 4
    gbs = kv_bytes / ms / 1e6
    peak, peak_kind = measured_peak_gbs()
    print(json.dumps({"metric": "attention_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
                      "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "isolated decode attention q%d kv%d hd%d context %d, %d layer caches (> L2)"
                                             % (q_heads, kv_heads, head_dim, ctx, layers)},
                      "gpu_launches": launches, "us_per_layer_step": ms * 1000.0,
                      "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "peak_kind": peak_kind,
                                   "traffic": None, "bytes_per_launch": kv_bytes}}))
    for s in caches:
        s.end_incremental_decode()
    din.free()
    dout.free()
    b.close()
    return 0


def run_linear(args):
    """Isolated quantized linear: one resident [N, K] matrix per copy, enough distinct copies to exceed
    the L2 cache, activations and outputs resident on the device. One step = one pass over every copy."""
    from neural_api_b200.backend import CudaBackend, DotProductSharedKernel
    k, n = (int(v) for v in args.kn.lower().split("x"))
    # type -> (ggml id, block bytes, block elements, byte offsets of the block's fp16 scales)
    ggml_type, bb, be, f16_at = {"q8_0": (8, 34, 32, (0,)), "q4_0": (2, 18, 32, (0,)), "q4_k": (12, 144, 256, (0, 2)),
                                 "q5_k": (13, 176, 256, (0, 2)), "q6_k": (14, 210, 256, (208,))}[args.type]
    batch = args.batch or 1
    backend = CudaBackend(0)
    rng = np.random.default_rng(0)
    nblk = n * k // be
    wbytes = nblk * bb
    copies = max(2, int((300 << 20) // wbytes) + 1)
    lins = []
    for c in range(copies):
        blk = rng.integers(0, 256, (nblk, bb), dtype=np.uint8)
        for off in f16_at:
            blk[:, off:off + 2] = np.asarray(rng.uniform(0.001, 0.05, nblk), dtype=np.float16).view(np.uint8).reshape(-1, 2)
        lin = DotProductSharedKernel(backend)
        lin.prepare_for_compute_quant(ggml_type, blk.reshape(-1), n, k)
        lins.append(lin)
    import ctypes as C
    x = backend.to_device(rng.standard_normal((batch, k)).astype(np.float32))
    y = backend.alloc(batch * n * 4)
    handles = (C.c_void_p * copies)(*[lin.handle for lin in lins])
    backend._check(backend.lib.cai_linear_forward_many(handles, copies, x.ptr, batch, y.ptr, args.warmup))
    backend.sync()
    launches0 = backend.launch_count()
    backend.timer_begin()
    backend._check(backend.lib.cai_linear_forward_many(handles, copies, x.ptr, batch, y.ptr, args.steps))
    ms = backend.timer_end()
    launches = backend.launch_count() - launches0
    per_launch_ms = ms / (args.steps * copies)
    alg_bytes = wbytes + 4 * batch * (k + n)
    gbs = alg_bytes / (per_launch_ms * 1e-3) / 1e9
    peak, peak_kind = measured_peak_gbs()
    line = {"metric": "qgemv_hbm_gbs", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": {"workload": "isolated %s linear K=%d N=%d batch %d, %d weight copies (> L2)" % (args.type, k, n, batch, copies)},
            "gpu_launches": launches, "us_per_launch": per_launch_ms * 1e3,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak, "unit": "GB/s", "frac": gbs / peak, "peak_kind": peak_kind,
                         "traffic": None, "bytes_per_launch": alg_bytes}}
    print(json.dumps(line))
    for lin in lins:
        lin.unprepare_for_compute()
    backend.close()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kn", default="5120x27648", help="linear workload: KxN")
    ap.add_argument("--type", default="q8_0", choices=["q8_0", "q4_0", "q4_k", "q5_k", "q6_k"], help="linear workload: block type")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=32)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="qwen2.5-32b", choices=sorted(WORKLOAD_DEFAULTS) + ["linear", "attention"])
    ap.add_argument("--heads", default="40x8x128", help="attention workload: q_heads x kv_heads x head_dim")
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--ctx", type=int, default=None)
    ap.add_argument("--parallel", default="auto", choices=["auto", "tp", "dp", "ep"],
                    help="N > 1: tp = one job sharded tensor-parallel (strong scaling), dp = one replica with its own batch per GPU "
                         "(weak scaling, no collective on the data path), ep = experts sharded, the job's sequences divided over the "
                         "GPUs (strong scaling); auto = tp for qwen2.5-32b, ep for olmoe-1b-7b, dp for the others")
    ap.add_argument("--kv", default="f32", choices=["f32", "int8"],
                    help="KV cache: fp32, or the reference's default int8 rows (codes + one fp32 scale per head and position)")
    ap.add_argument("--fill", default="prefill", choices=["prefill", "zeros"],
                    help="how the context is produced: by cai_session_prefill from random tokens, or declared over zeroed caches "
                         "(large batch x context products, where a real prefill takes minutes; decode timing does not depend on the values)")
    ap.add_argument("--no-extra", action="store_true", help="skip the side measurements of the `also` block and the CPU baseline")
    ap.add_argument("--layers", type=int, default=None,
                    help="depth cut of the architecture (profiling captures on a small case; the workload string says so)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.workload == "linear":
        return run_linear(args)
    if args.workload == "attention":
        return run_attention(args)
    from neural_api_b200.configs import ARCHS
    from neural_api_b200 import parallel
    ggml_type, seed, batch, ctx = WORKLOAD_DEFAULTS[args.workload]
    batch = args.batch or batch
    ctx = args.ctx or ctx
    if args.layers:
        ARCHS[args.workload] = dict(ARCHS[args.workload], layers=args.layers)      # every later look-up sees the cut
    arch_kw = ARCHS[args.workload]
    rank, world, local_rank = parallel.env_rank_world()

    if args.impl == "reference":
        if rank == 0:
            run_reference(args, arch_kw, ggml_type, batch, ctx)
        return 0

    dist = None
    if world > 1:
        import torch  # noqa: F401  (first, so that its NCCL is the one the process loads)
        rank, world, local_rank, dist = parallel.init_process_group("cpu:gloo,cuda:nccl")
    from neural_api_b200.backend import CudaBackend
    backend = CudaBackend(local_rank)
    mode = parallel_mode(args)
    if world > 1 and mode in ("tp", "ep"):
        uid = backend.comm_unique_id() if rank == 0 else bytes(128)
        uid = parallel.broadcast_bytes(dist, uid, src=0, length=128)
        backend.comm_init(rank, world, uid)

    model = build_model(backend, rank, world, args.workload, ggml_type, seed, mode)
    res = run_workload(backend, dist, rank, world, args.workload, ggml_type, seed, batch, ctx, args.steps, args.warmup, mode=mode,
                       kv=args.kv, model=model, fill=args.fill)
    peak, peak_kind = measured_peak_gbs()
    prof = res["profile"]
    lin_ms, lin_n = prof["linear"]
    lin_ms_step = lin_ms / res["profile_steps"]
    step_bytes = res["weight_bytes_rank"] + res["kv_bytes_step"]
    if res["step_kernel"]:
        # One persistent kernel per step: the launch IS the step, so the roofline object is the step's: algorithmic bytes
        # of one launch (this rank's weights + the cached K and V rows it reads) over the launch's device time (CUDA events
        # around the timed steps). The time inside the matrix products, from the kernel's own phase stamps, is kept beside
        # it (`products`), comparable with the per-operator path's figure.
        achieved = step_bytes / (res["ms_per_step"] * 1e-3) / 1e9
        traffic = STEP_KERNEL_TRAFFIC_PER_ALGORITHMIC_BYTE * step_bytes if STEP_KERNEL_TRAFFIC_PER_ALGORITHMIC_BYTE else None
        products = res["weight_bytes_rank"] / (lin_ms_step * 1e-3) / 1e9 if lin_ms_step > 0 else 0.0
        roofline = {"bound": "hbm", "kernel": "step_kernel (one persistent kernel per decode step: products, attention, argmax)",
                    "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic,
                    "bytes_per_launch": step_bytes, "launches_per_step": 1,
                    "products": {"achieved": products, "frac": products / peak, "bytes_per_step": res["weight_bytes_rank"],
                                 "phases_per_step": lin_n / res["profile_steps"], "ms_per_step_in_products": lin_ms_step}}
    else:
        achieved = res["weight_bytes_rank"] / (lin_ms_step * 1e-3) / 1e9 if lin_ms_step > 0 else 0.0
        # DRAM traffic per launch of the dominant kernel: algorithmic bytes per launch x the ratio of
        # (dram__bytes_read.sum + dram__bytes_write.sum) to algorithmic bytes that one ncu capture of the kernel measured
        # on a smaller case (the traffic grows in proportion to the matrix).
        launches_per_step = lin_n / res["profile_steps"] if res["profile_steps"] else 0
        bytes_per_launch = res["weight_bytes_rank"] / launches_per_step if launches_per_step else None
        traffic = GEMV_TRAFFIC_PER_ALGORITHMIC_BYTE * bytes_per_launch if bytes_per_launch else None
        roofline = {"bound": "hbm", "kernel": "gemv_quant_kernel (dequant-fused GEMV, one launch per matrix)", "achieved": achieved, "peak": peak,
                    "unit": "GB/s", "frac": achieved / peak, "peak_kind": peak_kind, "traffic": traffic,
                    "bytes_per_launch": bytes_per_launch, "bytes_per_step": res["weight_bytes_rank"], "launches_per_step": launches_per_step,
                    "ms_per_step_in_kernel": lin_ms_step}
    line = {
        "metric": "decode_tokens_per_s", "value": res["tokens_per_s"], "unit": "tokens/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["ms_per_step"], "higher_is_better": True,
        "scaling": "weak" if (world > 1 and mode == "dp") else "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, arch_kw, ggml_type, batch, ctx, world),
        "clocks": {"sm_mhz": res["clocks"]["sm_mhz"], "sm_max_mhz": res["clocks"]["sm_max_mhz"], "reasons": res["clocks"]["reasons"]},
        "e2e": {"value": res["e2e_tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": res["h2d"], "d2h_bytes_per_step": res["d2h"]},
        "gpu_launches": res["launches"],
        "roofline": roofline,
        "step_roofline": {"bytes_per_step_per_gpu": step_bytes, "achieved_gbs": step_bytes / (res["ms_per_step"] * 1e-3) / 1e9,
                          "frac": step_bytes / (res["ms_per_step"] * 1e-3) / 1e9 / peak, "frac_of_8tbs": step_bytes / (res["ms_per_step"] * 1e-3) / 8e12},
        "profile_ms_per_step": {k: v[0] / res["profile_steps"] for k, v in prof.items()},
        "prefill_s": res["prefill_s"], "tokens_crc": res["tokens_crc"], "step_kernel": res["step_kernel"],
    }
    if world > 1 and mode == "tp":
        # correctness of the sharded path inside the same run: N GPUs against one GPU on a depth-cut model
        model.close()
        model = None
        verdict, worst = tp_parity_check(backend, dist, rank, world, args.workload, ggml_type)
        line["tp_parity"] = verdict
        line["tp_parity_worst_rel_logit_diff"] = worst
    if rank == 0 and world == 1 and not args.no_extra:
        also = {}
        if args.workload == "qwen2.5-32b" and args.batch is None:
            # the metric's second batch size: 64 sequences at the same context on the same weights, int8 cache (69 GB of
            # codes; the fp32 cache of this shape is 275 GB). The context is declared, not prefilled: 64 x 8191 prompt
            # tokens through a 32B model are minutes of prefill; decode timing does not depend on the rows' values.
            try:
                r64 = run_workload(backend, None, 0, 1, args.workload, ggml_type, seed, 64, ctx, 8, 3, do_e2e=True, do_profile=False,
                                   kv="int8", model=model, fill="zeros")
                sb = r64["weight_bytes_rank"] + r64["kv_bytes_step"]
                also["qwen2.5-32b Q8_0 batch 64 context %d int8 KV (context declared, not prefilled)" % ctx] = {
                    "tokens_per_s": r64["tokens_per_s"], "ms_per_step": r64["ms_per_step"], "e2e_tokens_per_s": r64["e2e_tokens_per_s"],
                    "step_hbm_frac": sb / (r64["ms_per_step"] * 1e-3) / 1e9 / peak, "bytes_per_step": sb}
            except Exception as e:
                also["qwen2.5-32b batch 64"] = {"failed": str(e)[:200]}
        model.close()
        model = None
        try:
            sample = CpuSample(arch_kw, ggml_type, ctx)
            sample.step_seconds()
            ts = [sample.step_seconds() for _ in range(3)]
            sec = float(np.median(ts)) * batch
            line["cpu_baseline"] = dict({"value": batch / sec, "unit": "tokens/s", "cores": sample.cores, "kind": "port", "sample": sample.desc},
                                        **sample.describe())
            sample.close()
        except Exception as e:                               # the baseline is reported, never required
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": "failed: %s" % e}
        for name, label, st, wu, fill, kv2 in (
                ("qwen2.5-0.5b", "qwen2.5-0.5b Q8_0 batch 1 context 256", 128, 8, "prefill", "f32"),
                ("tinyllama-1.1b", "tinyllama-1.1b Q4_0 16 sequences context 768", 32, 4, "prefill", "f32"),
                ("olmoe-1b-7b", "olmoe-1b-7b Q8_0 batch 64 context 2048 (context declared, not prefilled)", 16, 4, "zeros", "f32"),
                # the same with the reference's default cache (int8 rows + one scale per row): a quarter of the attention bytes
                ("olmoe-1b-7b", "olmoe-1b-7b Q8_0 batch 64 context 2048 int8 KV (context declared, not prefilled)", 16, 4, "zeros", "int8")):
            if name == args.workload:
                continue
            try:
                t, sd, b2, c2 = WORKLOAD_DEFAULTS[name]
                r2 = run_workload(backend, None, 0, 1, name, t, sd, b2, c2, st, wu, do_e2e=True, do_profile=False, fill=fill, kv=kv2)
                sb = r2["weight_bytes_rank"] + r2["kv_bytes_step"]
                also[label] = {"tokens_per_s": r2["tokens_per_s"], "ms_per_step": r2["ms_per_step"], "e2e_tokens_per_s": r2["e2e_tokens_per_s"],
                               "step_hbm_frac": sb / (r2["ms_per_step"] * 1e-3) / 1e9 / peak, "launches_per_step": r2["launches"] / st,
                               "step_kernel": r2["step_kernel"]}
            except Exception as e:
                also[label] = {"failed": str(e)[:200]}
        line["also"] = also
    if model is not None:
        model.close()
    if rank == 0:
        print(json.dumps(line))
    backend.close()
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
