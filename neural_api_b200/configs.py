"""The synthetic decode workloads (architecture shapes only; weights are random)."""
from .backend import make_config

# name -> keyword arguments of make_config
ARCHS = {
    # Qwen2.5-0.5B: 24 layers, hidden 896, 14 query / 2 KV heads, head_dim 64, SwiGLU 4864,
    # vocab 151936 tied, RMSNorm eps 1e-6, RoPE theta 1e6, q/k/v biases
    "qwen2.5-0.5b": dict(hidden=896, inter=4864, layers=24, heads=14, kv_heads=2, head_dim=64, vocab=151936,
                         rms_eps=1e-6, rope_theta=1e6, tie_embeddings=True, qkv_bias=True),
    # TinyLlama-1.1B: 22 layers, hidden 2048, 32 / 4 heads, head_dim 64, intermediate 5632, vocab 32000
    "tinyllama-1.1b": dict(hidden=2048, inter=5632, layers=22, heads=32, kv_heads=4, head_dim=64, vocab=32000,
                           rms_eps=1e-5, rope_theta=1e4),
    # OLMoE-1B-7B: 16 layers, hidden 2048, 16 heads MHA head_dim 128, 64 experts top-8, expert inter 1024,
    # vocab 50304, q/k norm; router probabilities are not renormalised (norm_topk_prob default false)
    "olmoe-1b-7b": dict(hidden=2048, inter=1024, layers=16, heads=16, kv_heads=16, head_dim=128, vocab=50304,
                        rms_eps=1e-5, rope_theta=1e4, qk_norm=True, n_experts=64, top_k=8, norm_topk=False, moe_inter=1024),
    # Qwen2.5-32B: 64 layers, hidden 5120, 40 / 8 heads, head_dim 128, intermediate 27648, vocab 152064
    "qwen2.5-32b": dict(hidden=5120, inter=27648, layers=64, heads=40, kv_heads=8, head_dim=128, vocab=152064,
                        rms_eps=1e-6, rope_theta=1e6, qkv_bias=True),
}

# isolated quantized linear sweep: (K, N)
LINEAR_SHAPES = [(896, 4864), (3584, 18944), (4096, 14336), (5120, 27648)]
LINEAR_BATCHES = [1, 4, 16, 32, 64]


def arch_config(name, **overrides):
    kw = dict(ARCHS[name])
    kw.update(overrides)
    return make_config(**kw)


def step_weight_bytes(kw, bytes_per_weight, tokens_per_step=1):
    """Algorithmic matrix-weight bytes one decode step streams (codes + scales), all ranks together.
    Dense: every matrix once. MoE: router + the experts `tokens_per_step` tokens can touch at most."""
    H, L, V = kw["hidden"], kw["layers"], kw["vocab"]
    qw, kw_ = kw["heads"] * kw["head_dim"], kw["kv_heads"] * kw["head_dim"]
    attn = (qw + 2 * kw_) * H + H * qw
    if kw.get("n_experts", 0):
        touched = min(kw["n_experts"], tokens_per_step * kw["top_k"])
        mlp = kw["n_experts"] * H + touched * 3 * kw["moe_inter"] * H
    else:
        mlp = 3 * kw["inter"] * H
    return int((L * (attn + mlp) + V * H) * bytes_per_weight)
