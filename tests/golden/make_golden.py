#!/usr/bin/env python3
"""Packs the reference's own golden vectors for the decode hot path into small
.npz fixtures, so that the tests can pin the oracle (and the CUDA path) against
them on machines where the reference checkout is not present.

Run once, in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference

What is packed (all paths relative to the reference root):
  tests/fixtures/tiny_{llama,qwen2,olmoe,mixtral}.safetensors + _config.json +
  _logits.json   pico checkpoints in HF layout with float64-oracle logits for three
                 16-token sequences (gate 1e-4 in tests/TestNeuralPretrained.pas:5684-5751,
                 :7533-7556, :7963+, :8073)
  tests/fixtures/tiny_llama_q8.gguf + tiny_llama_q8.safetensors + _config.json
                 the Q8_0 GGUF twin of an F32 checkpoint (tests/TestNeuralPretrained.pas:6343-6438)
  tests/fixtures/tiny_llama_f16.gguf   the F16 GGUF twin (:6312-6335)
  the hand-rolled one-block Q4_0 known-answer test (:5996-6020): d = 0.5, element e
                 carries nibble (e mod 16)
  the top-k gate known-answer test (tests/TestNeuralNumerical.pas:75014-75037)

The script only READS reference data files (weights, configs, logits); it copies
no reference source code.
"""
import json
import os
import sys

import numpy as np


def load_safetensors(path):
    from safetensors.numpy import load_file
    return load_file(path)


def pack_hf_case(fix, name, out_dir):
    tensors = load_safetensors(os.path.join(fix, name + ".safetensors"))
    cfg = json.load(open(os.path.join(fix, name + "_config.json")))
    gold = json.load(open(os.path.join(fix, name + "_logits.json")))
    payload = {"t::" + k: v for k, v in tensors.items()}
    payload["config_json"] = np.frombuffer(json.dumps(cfg).encode(), dtype=np.uint8)
    payload["sequences"] = np.asarray(gold["sequences"], dtype=np.int32)
    payload["logits"] = np.asarray(gold["logits"], dtype=np.float64)
    np.savez_compressed(os.path.join(out_dir, name + ".npz"), **payload)
    print("packed", name, payload["logits"].shape)


GGUF_TO_HF = {
    "token_embd.weight": "model.embed_tokens.weight",
    "output_norm.weight": "model.norm.weight",
    "output.weight": "lm_head.weight",
}
GGUF_BLK = {
    "attn_norm.weight": "input_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight",
    "attn_k.weight": "self_attn.k_proj.weight",
    "attn_v.weight": "self_attn.v_proj.weight",
    "attn_output.weight": "self_attn.o_proj.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight",
    "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
}


def hf_name(gguf_name):
    """ggml tensor name -> HF name (the rename table of BuildFromGGUFEx,
    neural/neuralpretrained.pas:17804-17848)."""
    if gguf_name in GGUF_TO_HF:
        return GGUF_TO_HF[gguf_name]
    parts = gguf_name.split(".", 2)
    assert parts[0] == "blk"
    return "model.layers.%s.%s" % (parts[1], GGUF_BLK[parts[2]])


def pack_gguf_case(fix, gguf_file, twin_safetensors, cfg_file, out_name, out_dir):
    from gguf import GGUFReader
    from gguf.quants import dequantize
    r = GGUFReader(os.path.join(fix, gguf_file))
    payload = {}
    for t in r.tensors:
        name = hf_name(t.name)
        raw = np.ascontiguousarray(t.data).view(np.uint8).reshape(-1)
        # ggml dims are contiguous-first; rows = product of the others
        cols = int(t.shape[0])
        rows = int(np.prod(t.shape[1:])) if len(t.shape) > 1 else 1
        payload["raw::" + name] = raw
        payload["meta::" + name] = np.asarray([int(t.tensor_type), rows, cols], dtype=np.int64)
        # the gguf package's own dequantisation: an independent check of the codecs
        payload["deq::" + name] = np.asarray(dequantize(t.data, t.tensor_type), dtype=np.float32).reshape(-1)
    if twin_safetensors:
        for k, v in load_safetensors(os.path.join(fix, twin_safetensors)).items():
            payload["twin::" + k] = v
    cfg = json.load(open(os.path.join(fix, cfg_file)))
    payload["config_json"] = np.frombuffer(json.dumps(cfg).encode(), dtype=np.uint8)
    np.savez_compressed(os.path.join(out_dir, out_name + ".npz"), **payload)
    print("packed", out_name, len(r.tensors), "tensors")


def pack_kats(out_dir):
    # One Q4_0 block, d = 0.5, element e carries nibble (e mod 16); expected value
    # 0.5 * ((e mod 16) - 8)  (tests/TestNeuralPretrained.pas:5996-6020).
    blk = np.zeros(18, dtype=np.uint8)
    blk[:2] = np.asarray([0.5], dtype=np.float16).view(np.uint8)
    for b in range(16):
        lo = b % 16            # element b
        hi = (b + 16) % 16     # element b + 16
        blk[2 + b] = lo | (hi << 4)
    expect = np.asarray([0.5 * ((e % 16) - 8) for e in range(32)], dtype=np.float32)
    # top-k gate KAT (tests/TestNeuralNumerical.pas:75014-75037)
    np.savez_compressed(
        os.path.join(out_dir, "kats.npz"),
        q4_0_block=blk, q4_0_expect=expect,
        topk_in=np.asarray([0.5, 0.1, 0.3, 0.1], dtype=np.float32),
        topk_k=np.asarray(2), topk_out=np.asarray([0.625, 0.0, 0.375, 0.0], dtype=np.float32))
    print("packed kats")


def pack_gguf_files(fix, out_dir):
    """The reference's GGUF fixtures as whole files (the C-side reader parses files, not tensors), the K-quant
    reference dequantisations of tests/fixtures/tiny_kquant_ref.json (tests/TestNeuralPretrained.pas:5931-6020) and the
    next-token logits of the F32 checkpoint twin (tiny_llama_logits.json) for the file-to-logits check."""
    payload = {}
    for f in ("tiny_kquant.gguf", "tiny_llama_q8.gguf", "tiny_llama_f16.gguf", "tiny_llama_f32.gguf"):
        payload["file::" + f] = np.frombuffer(open(os.path.join(fix, f), "rb").read(), dtype=np.uint8)
    ref = json.load(open(os.path.join(fix, "tiny_kquant_ref.json")))
    payload["kquant::ref_f32"] = np.asarray(ref["ref_f32"], dtype=np.float32)
    for k, v in ref["dequant"].items():
        payload["kquant::" + k] = np.asarray(v, dtype=np.float32)
    gold = json.load(open(os.path.join(fix, "tiny_llama_logits.json")))
    payload["tiny_llama::sequences"] = np.asarray(gold["sequences"], dtype=np.int32)
    payload["tiny_llama::logits"] = np.asarray(gold["logits"], dtype=np.float64)
    np.savez_compressed(os.path.join(out_dir, "gguf_files.npz"), **payload)
    print("packed gguf_files", sorted(payload))


def pack_block_kats(out_dir):
    """Seeded random blocks of every ggml type the reader decodes, with the `gguf` package's dequantisation of them
    (the external oracle the reference's own fixture generators use, tools/make_kquant_gguf_fixture.py)."""
    from gguf.quants import dequantize
    from gguf.constants import GGMLQuantizationType as T
    geometry = {2: (18, [0]), 3: (20, [0, 2]), 6: (22, [0]), 7: (24, [0, 2]), 8: (34, [0]), 10: (84, [80, 82]),
                11: (110, [108]), 12: (144, [0, 2]), 13: (176, [0, 2]), 14: (210, [208])}
    rng = np.random.default_rng(20240611)
    payload = {}
    n_blocks = 48
    for t, (bb, f16_at) in geometry.items():
        raw = rng.integers(0, 256, size=(n_blocks, bb), dtype=np.uint8)
        for off in f16_at:                       # finite scales, a few subnormal and negative ones among them
            h = (rng.standard_normal(n_blocks) * 0.05).astype(np.float16)
            h[0], h[1], h[2] = np.float16(6e-8), np.float16(-3.1e-5), np.float16(0.0)
            raw[:, off:off + 2] = h.view(np.uint8).reshape(n_blocks, 2)
        payload["raw::%d" % t] = raw.reshape(-1)
        payload["deq::%d" % t] = np.asarray(dequantize(raw.reshape(-1), T(t)), dtype=np.float32).reshape(-1)
    np.savez_compressed(os.path.join(out_dir, "block_kats.npz"), **payload)
    print("packed block_kats", len(payload) // 2, "types")


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    ref = sys.argv[1]
    fix = os.path.join(ref, "tests", "fixtures")
    out_dir = os.path.dirname(os.path.abspath(__file__))
    for name in ("tiny_llama", "tiny_qwen2", "tiny_olmoe", "tiny_mixtral"):
        pack_hf_case(fix, name, out_dir)
    pack_gguf_case(fix, "tiny_llama_q8.gguf", "tiny_llama_q8.safetensors",
                   "tiny_llama_q8_config.json", "tiny_llama_q8_gguf", out_dir)
    pack_gguf_case(fix, "tiny_llama_f16.gguf", None, "tiny_llama_config.json",
                   "tiny_llama_f16_gguf", out_dir)
    pack_kats(out_dir)
    pack_gguf_files(fix, out_dir)
    pack_block_kats(out_dir)


if __name__ == "__main__":
    main()
