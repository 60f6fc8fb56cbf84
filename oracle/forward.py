"""CPU restatement of the reference's Llama-family per-token decode forward
(TEST INFRASTRUCTURE: the checker, never the product).

The reference's layer classes live in a unit that is absent from its checkout
(neural/neuralnetwork.pas), so the forward is restated from the importer that
wires the graph and from the OpenCL twins whose comments say they mirror the
CPU Compute():

  graph / weight conventions  neural/neuralpretrained.pas:16423-16875 (wiring),
                              :14792-14812 (q/k row interleave), :17412-17421
                              (up rows first, gate rows second), :15347-15388 (MoE)
  RMSNorm                     neural/neural.cl:1047-1085   y = gain * (x * inv)
  RoPE                        neural/neural.cl:1517-1542   pairs (2k, 2k+1), fp32 angle
  SwiGLU                      neural/neural.cl:1213-1263   first * (second * sigmoid(second))
  KV append + decode attention neural/neural.cl:2354-2379, 2406-2499
  router softmax              neural/neural.cl:1594-1647
  MoE down bank               neural/neural.cl:2709-2752
  driver loop / argmax        neural/neuralchatengine.pas:683-697, 1466-1505

The session steps ONE token at a time over a KV cache, exactly like
TNNetStreamingDecoder.StepForward (neural/neuraldecode.pas:5696-5712).
`dtype` is float32 for parity runs (the reference computes in fp32) and may be
float64 when pinning against the float64 golden logits.
"""
from dataclasses import dataclass, field
import re
import numpy as np


@dataclass
class LlamaConfig:
    """Subset of TLlamaConfig (neural/neuralpretrained.pas:677-952) the decode path reads."""
    hidden: int
    inter: int
    layers: int
    heads: int
    kv_heads: int
    head_dim: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    tie_embeddings: bool = False
    qkv_bias: bool = False
    qk_norm: bool = False          # OLMoE full-width q/k RMSNorm before RoPE
    n_experts: int = 0             # 0 = dense MLP
    top_k: int = 0
    norm_topk: bool = False
    moe_inter: int = 0

    @property
    def q_width(self):
        return self.heads * self.head_dim

    @property
    def kv_width(self):
        return self.kv_heads * self.head_dim

    @staticmethod
    def from_hf(cfg):
        """Reads the HF config.json keys the importer reads
        (ReadLlamaConfigFromJSONFile, neural/neuralpretrained.pas:13495+; OLMoE
        branch :14152-14210)."""
        mt = cfg.get("model_type", "llama")
        heads = cfg["num_attention_heads"]
        hidden = cfg["hidden_size"]
        n_exp = cfg.get("num_experts", cfg.get("num_local_experts", 0)) or 0
        is_moe = mt in ("olmoe", "mixtral")
        return LlamaConfig(
            hidden=hidden,
            inter=cfg["intermediate_size"],
            layers=cfg["num_hidden_layers"],
            heads=heads,
            kv_heads=cfg.get("num_key_value_heads", heads),
            head_dim=cfg.get("head_dim") or hidden // heads,
            vocab=cfg["vocab_size"],
            rms_eps=cfg.get("rms_norm_eps", 1e-5),
            rope_theta=cfg.get("rope_theta", 10000.0),
            tie_embeddings=bool(cfg.get("tie_word_embeddings", False)),
            qkv_bias=(mt == "qwen2") or bool(cfg.get("attention_bias", False)),
            qk_norm=(mt == "olmoe"),
            n_experts=n_exp if is_moe else 0,
            top_k=cfg.get("num_experts_per_tok", 0) if is_moe else 0,
            # OLMoE reads norm_topk_prob, default False (neuralpretrained.pas:14184);
            # Mixtral always renormalizes.
            norm_topk=(bool(cfg.get("norm_topk_prob", False)) if mt == "olmoe" else (mt == "mixtral")),
            moe_inter=cfg["intermediate_size"] if is_moe else 0,
        )


def interleave_rows(w, head_dim):
    """HF rotate_half row order -> the in-net interleaved order.

    target(h*hd + 2k) <- row(h*hd + k), target(h*hd + 2k + 1) <- row(h*hd + k + hd/2)
    (neural/neuralpretrained.pas:14792-14812). Works on [rows, ...] arrays and on
    1-D bias / gain vectors (:14926-14928, :15233-15243).
    """
    w = np.asarray(w)
    rows = w.shape[0]
    half = head_dim // 2
    idx = np.arange(rows)
    h = idx // head_dim
    r = idx % head_dim
    src = h * head_dim + np.where(r % 2 == 0, r // 2, r // 2 + half)
    return w[src]


_LAYER_RE = re.compile(r"^model\.layers\.(\d+)\.(.+)$")
_EXPERT_RE = re.compile(r"^(?:mlp|block_sparse_moe)\.experts\.(\d+)\.(\w+)\.weight$")


class OracleModel:
    """Weights in the in-net layout, one dict per block."""

    def __init__(self, cfg, dtype=np.float32):
        self.cfg = cfg
        self.dtype = dtype
        self.embed = None
        self.lm_head = None
        self.final_norm = None
        self.blocks = [dict() for _ in range(cfg.layers)]
        hd = cfg.head_dim
        k = np.arange(hd // 2, dtype=np.float64)
        # theta_k = base^(-2k/hd) = exp(-2k/hd * ln base)  (tests/TestNeuralNumerical.pas:15301-15350)
        self.theta = np.exp(-2.0 * k / hd * np.log(cfg.rope_theta)).astype(np.float32)

    def set_tensor(self, name, w, interleave=True):
        """Accepts one tensor under its HF name in HF layout ([out, in] rows).

        interleave=True applies the importer's q/k row permutation; pass False
        for rows that are already in GGUF (llama.cpp-permuted) order, which is
        the in-net order (neural/neuralgguf.pas:428-438 undone by
        neural/neuralpretrained.pas:14792-14812).
        """
        cfg = self.cfg
        w = np.asarray(w, dtype=self.dtype)
        if name == "model.embed_tokens.weight":
            self.embed = w
            return
        if name == "lm_head.weight":
            self.lm_head = w
            return
        if name == "model.norm.weight":
            self.final_norm = w
            return
        m = _LAYER_RE.match(name)
        if not m:
            return  # ignorable buffers such as rotary_emb.inv_freq
        blk = self.blocks[int(m.group(1))]
        rest = m.group(2)
        hd = cfg.head_dim
        perm = (lambda a: interleave_rows(a, hd)) if interleave else (lambda a: a)
        simple = {
            "input_layernorm.weight": "attn_norm",
            "post_attention_layernorm.weight": "ffn_norm",
            "self_attn.v_proj.weight": "wv",
            "self_attn.v_proj.bias": "bv",
            "self_attn.o_proj.weight": "wo",
            "mlp.gate_proj.weight": "w_gate",
            "mlp.up_proj.weight": "w_up",
            "mlp.down_proj.weight": "w_down",
            "mlp.gate.weight": "router",
            "block_sparse_moe.gate.weight": "router",
        }
        permuted = {
            "self_attn.q_proj.weight": "wq",
            "self_attn.k_proj.weight": "wk",
            "self_attn.q_proj.bias": "bq",
            "self_attn.k_proj.bias": "bk",
            "self_attn.q_norm.weight": "q_norm",
            "self_attn.k_norm.weight": "k_norm",
        }
        if rest in simple:
            blk[simple[rest]] = w
            return
        if rest in permuted:
            blk[permuted[rest]] = perm(w)
            return
        e = _EXPERT_RE.match(rest)
        if e:
            kind = {"gate_proj": "gate", "up_proj": "up", "down_proj": "down",
                    "w1": "gate", "w3": "up", "w2": "down"}[e.group(2)]
            blk.setdefault("experts", {}).setdefault(int(e.group(1)), {})[kind] = w

    @staticmethod
    def from_hf_tensors(cfg, tensors, dtype=np.float32, interleave=True):
        m = OracleModel(cfg, dtype)
        for name, w in tensors.items():
            m.set_tensor(name, w, interleave)
        if m.lm_head is None:  # tied head = the embedding rows (neuralpretrained.pas:15655-15671)
            m.lm_head = m.embed
        return m


def rms_norm(x, gain, eps):
    """y = gain * (x * inv), inv = 1/sqrt(mean(x^2) + eps) (neural/neural.cl:1067-1083)."""
    dt = x.dtype.type
    ss = dt(0)
    ss = np.sum(x * x, dtype=x.dtype)
    inv = dt(1.0) / np.sqrt(ss / dt(x.shape[-1]) + dt(eps))
    return gain * (x * inv)


def rope_interleaved(x, pos, theta, head_dim):
    """Rotates channel pairs (2k, 2k+1) of every head by fp32 angle pos*theta_k
    (neural/neural.cl:1534-1541; head-tiled per neural/neuralpretrained.pas:16572-16587)."""
    dt = x.dtype
    heads = x.shape[-1] // head_dim
    v = x.reshape(heads, head_dim // 2, 2)
    angle = (np.float32(pos) * theta).astype(np.float32)     # fp32 product, as on the device twin
    s = np.sin(angle.astype(np.float64)).astype(dt)
    c = np.cos(angle.astype(np.float64)).astype(dt)
    x0 = v[:, :, 0]
    x1 = v[:, :, 1]
    out = np.empty_like(v)
    out[:, :, 0] = c * x0 - s * x1
    out[:, :, 1] = s * x0 + c * x1
    return out.reshape(-1)


def swiglu(fused, half):
    """out[d] = fused[d] * swish(fused[half + d]); first half = up, second = gate.
    Two-branch stable sigmoid (neural/neural.cl:1228-1262)."""
    a = fused[:half]
    b = fused[half:]
    e = np.exp(-np.abs(b))       # exp of a non-positive number: underflows, never overflows
    sig = np.where(b > 0, 1.0 / (1.0 + e), e / (1.0 + e)).astype(fused.dtype)
    return a * (b * sig)


def router_gates(probs, k, renorm):
    """Keep the top-k of a softmax row, zero the rest, renormalise survivors to
    sum 1 when asked (TNNetTopKGate; KAT (0.5,0.1,0.3,0.1), k=2 -> (0.625,0,0.375,0),
    tests/TestNeuralNumerical.pas:75014-75037). Ties: lowest index wins."""
    order = np.argsort(-probs, kind="stable")[:k]
    gates = probs[order]
    if renorm:
        gates = gates / np.sum(gates, dtype=probs.dtype)
    return order, gates


def softmax_row(x):
    """max-shift, exp, sum, divide (neural/neural.cl:1594-1647)."""
    m = np.max(x)
    e = np.exp(x - m)
    return e / np.sum(e, dtype=x.dtype)


def quantize_cache_row(row):
    """The int8 KV-cache row format (neural/neural.cl:2500-2581, the device twin of
    TNNetScaledDotProductAttention.QuantizeCacheRow): one symmetric fp32 scale per (head, position) row,
    scale = maxabs / 127 over the finite magnitudes, codes = clamp(rint(v * (1 / maxabs) * 127), -127, 127) with
    round-half-to-even, multiplied in that order; a row whose maximum is zero or denormal gives zero codes and scale 1;
    NaN -> 0, infinities clamp. Returns (int8 codes, fp32 scale)."""
    v = np.asarray(row, dtype=np.float32)
    a = np.abs(v)
    finite = np.isfinite(a)
    maxabs = np.float32(np.max(a[finite])) if np.any(finite) else np.float32(0.0)
    if maxabs < np.float32(1.1754944e-38):            # below the smallest normal single
        return np.zeros(v.shape, dtype=np.int8), np.float32(1.0)
    recip = np.float32(1.0) / maxabs
    scaled = (v * recip).astype(np.float32) * np.float32(127.0)
    scaled = np.where(np.isnan(v), np.float32(0.0), scaled).astype(np.float32)
    codes = np.clip(np.rint(scaled), -127.0, 127.0).astype(np.int8)        # np.rint rounds half to even
    return codes, np.float32(maxabs / np.float32(127.0))


class OracleSession:
    """One sequence, one KV cache per layer, head-major [kv_head][pos][d]
    (neural/neural.cl:2343-2346). kv_int8 keeps the cache as int8 codes with one fp32 scale per row and folds the
    scales into the score and the value sum exactly like cai_sdpa_decode_int8 (neural/neural.cl:2583-2687)."""

    def __init__(self, model, max_ctx, kv_int8=False, window=0, evict=None):
        """window > 0: every layer attends over the most recent `window` rows (TNNetFusedSDPA's Window, jStart of
        neural/neural.cl:2437-2438). evict = (sinks, recent): StreamingLLM, the first `sinks` rows and the most recent
        `recent` rows stay (TNNetStreamingDecoder.EnableEviction, neural/neuraldecode.pas:1257-1276); rows keep the
        rotation of their original position. The oracle keeps every row and selects; max_ctx bounds positions here."""
        self.window = window
        self.evict = evict
        self.m = model
        cfg = model.cfg
        self.max_ctx = max_ctx
        self.kv_int8 = kv_int8
        if kv_int8:
            self.k = np.zeros((cfg.layers, cfg.kv_heads, max_ctx, cfg.head_dim), dtype=np.int8)
            self.v = np.zeros_like(self.k)
            self.k_scale = np.ones((cfg.layers, cfg.kv_heads, max_ctx), dtype=np.float32)
            self.v_scale = np.ones_like(self.k_scale)
        else:
            self.k = np.zeros((cfg.layers, cfg.kv_heads, max_ctx, cfg.head_dim), dtype=model.dtype)
            self.v = np.zeros_like(self.k)
        self.length = 0

    def reset(self):
        self.length = 0

    def truncate(self, n):
        """TNNetStreamingDecoder.TruncateTo (neural/neuraldecode.pas:5714-5720)."""
        if n < 0 or n > self.length:
            raise ValueError("truncate target outside the committed prefix")
        self.length = n

    def step(self, token, pos=None):
        """One width-1 forward at absolute position `pos` (default: cache length).
        Returns the raw logits row (the importer nets end in raw logits,
        neural/neuralchatengine.pas:1492-1499)."""
        m = self.m
        cfg = m.cfg
        dt = m.dtype
        if pos is None:
            pos = self.length
        slot = self.length
        if slot >= self.max_ctx:
            raise ValueError("context full")
        hd = cfg.head_dim
        group = cfg.heads // cfg.kv_heads
        inv_sqrt = dt(1.0 / np.sqrt(hd))
        x = m.embed[token].astype(dt)             # EncodeZero=1: token 0 is a real row
        for li, b in enumerate(m.blocks):
            h = rms_norm(x, b["attn_norm"], cfg.rms_eps)
            q = b["wq"] @ h
            k = b["wk"] @ h
            v = b["wv"] @ h
            if "bq" in b:
                q = q + b["bq"]
                k = k + b["bk"]
                v = v + b["bv"]
            if cfg.qk_norm:                        # full-width norm before RoPE (neuralpretrained.pas:16520-16530)
                q = rms_norm(q, b["q_norm"], cfg.rms_eps)
                k = rms_norm(k, b["k_norm"], cfg.rms_eps)
            q = rope_interleaved(q, pos, m.theta, hd)
            k = rope_interleaved(k, pos, m.theta, hd)
            if self.kv_int8:
                for g in range(cfg.kv_heads):
                    self.k[li, g, slot], self.k_scale[li, g, slot] = quantize_cache_row(k[g * hd:(g + 1) * hd])
                    self.v[li, g, slot], self.v_scale[li, g, slot] = quantize_cache_row(v[g * hd:(g + 1) * hd])
            else:
                self.k[li, :, slot, :] = k.reshape(cfg.kv_heads, hd)
                self.v[li, :, slot, :] = v.reshape(cfg.kv_heads, hd)
            n = slot + 1
            rows = np.arange(n)
            if self.evict is not None and n > self.evict[0] + self.evict[1]:
                rows = np.concatenate([np.arange(self.evict[0]), np.arange(n - self.evict[1], n)])
            elif self.window > 0 and n > self.window:
                rows = np.arange(n - self.window, n)
            att = np.empty(cfg.q_width, dtype=dt)
            for hq in range(cfg.heads):
                g = hq // group
                qh = q[hq * hd:(hq + 1) * hd]
                if self.kv_int8:
                    # raw code dot, then one scalar per row: kscale * 1/sqrt(d) (neural.cl:2636-2639)
                    sc = (self.k[li, g, rows, :].astype(dt) @ qh) * (self.k_scale[li, g, rows].astype(dt) * inv_sqrt)
                else:
                    sc = (self.k[li, g, rows, :] @ qh) * inv_sqrt    # scale after the dot (neural.cl:2450)
                mx = np.max(sc)
                e = np.exp(sc - mx)
                den = np.sum(e, dtype=dt)
                if self.kv_int8:
                    # (e_j * vscale_j) * code, summed, divided once at the end (neural.cl:2679-2684)
                    att[hq * hd:(hq + 1) * hd] = ((e * self.v_scale[li, g, rows].astype(dt)) @ self.v[li, g, rows, :].astype(dt)) / den
                else:
                    att[hq * hd:(hq + 1) * hd] = (e @ self.v[li, g, rows, :]) / den   # divide once at the end
            x = x + b["wo"] @ att
            h = rms_norm(x, b["ffn_norm"], cfg.rms_eps)
            if cfg.n_experts:
                probs = softmax_row(b["router"] @ h)
                order, gates = router_gates(probs, cfg.top_k, cfg.norm_topk)
                y = np.zeros(cfg.hidden, dtype=dt)
                for e_id, gate in zip(order, gates):
                    ex = b["experts"][int(e_id)]
                    fused = np.concatenate([ex["up"] @ h, ex["gate"] @ h])
                    act = swiglu(fused, fused.shape[0] // 2)
                    y = y + gate * (ex["down"] @ act)            # gate scales the expert OUTPUT
                x = x + y
            else:
                fused = np.concatenate([b["w_up"] @ h, b["w_gate"] @ h])
                act = swiglu(fused, cfg.inter)
                x = x + b["w_down"] @ act
        self.length = slot + 1
        h = rms_norm(x, m.final_norm, cfg.rms_eps)
        return (m.lm_head @ h).astype(dt)


def argmax_first(row):
    """First index of the maximum (ArgMaxRow, neural/neuralchatengine.pas:683-697)."""
    return int(np.argmax(row))


def greedy_decode(model, prompt, n_new, max_ctx=None):
    """The reference's schedule: tokens 0..P-2 one at a time, then token P-1 at
    position P-1 yields the first new token (neural/neuralchatengine.pas:1466-1505).
    Returns (new_tokens, logits rows of the decode steps)."""
    sess = OracleSession(model, max_ctx or (len(prompt) + n_new))
    for i, t in enumerate(prompt[:-1]):
        sess.step(int(t), i)
    tok = int(prompt[-1])
    out, rows = [], []
    for _ in range(n_new):
        logits = sess.step(tok)
        tok = argmax_first(logits)
        out.append(tok)
        rows.append(logits)
    return out, rows


def sampler_window(logits, k, temperature=1.0):
    """The candidate window the reference's samplers work on: scores = softmax(logits / temperature) over the whole row
    (TNNetTemperatureProcessor, neural/neuralchatengine.pas:1387-1388; the samplers take a post-softmax volume), sorted
    descending with ties to the lower id, truncated to the top k (TNNetSamplerBase.SelectTopCandidates,
    neural/neuralvolume.pas:991-1030). Returns (ids, probabilities)."""
    z = np.asarray(logits, dtype=np.float64) / float(temperature)
    z = np.where(np.isnan(z), -np.inf, z)
    p = np.exp(z - np.max(z))
    p = p / p.sum()
    order = np.argsort(-z, kind="stable")[:k]
    return order.astype(np.int32), p[order].astype(np.float32)


def weighted_draw(ids, probs, u, top_p=0.0):
    """TNNetSamplerWeightedTopK.SampleFromSorted (neural/neuralvolume.pas:4749-4785) over a window, optionally cut to the
    nucleus first (the shortest prefix whose mass exceeds top_p): Roll = u * KeptSum; the first candidate whose running
    sum exceeds Roll; the last kept candidate as the numeric-safety fallback. fp32 running sums, as on the device."""
    n_keep = len(ids)
    if 0.0 < top_p < 1.0:
        cum = np.float32(0)
        for j, pj in enumerate(probs):
            cum = np.float32(cum + pj)
            if cum > np.float32(top_p):
                n_keep = j + 1
                break
    kept = np.float32(0)
    for pj in probs[:n_keep]:
        kept = np.float32(kept + pj)
    if not kept > 0:
        return int(ids[0])
    roll = np.float32(np.float32(u) * kept)
    cum = np.float32(0)
    for j in range(n_keep):
        cum = np.float32(cum + probs[j])
        if roll < cum:
            return int(ids[j])
    return int(ids[n_keep - 1])
