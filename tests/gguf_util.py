"""Minimal GGUF writer for the tests: the same kind of hand-written files the reference's own reader tests build
(WriteOneTensorGGUF, tests/TestNeuralPretrained.pas:6037-6083), plus metadata."""
import struct

import numpy as np

U8, I8, U16, I16, U32, I32, F32, BOOL, STR, ARR, U64, I64, F64 = range(13)
_FMT = {U8: "<B", I8: "<b", U16: "<H", I16: "<h", U32: "<I", I32: "<i", F32: "<f", BOOL: "<B", U64: "<Q", I64: "<q", F64: "<d"}


def _s(text):
    b = text.encode()
    return struct.pack("<Q", len(b)) + b


def _value(vtype, v):
    if vtype == STR:
        return _s(v)
    if vtype == ARR:
        etype, items = v
        return struct.pack("<IQ", etype, len(items)) + b"".join(_value(etype, x) for x in items)
    return struct.pack(_FMT[vtype], v)


def gguf_bytes(meta, tensors, version=3, alignment=32, magic=0x46554747, write_alignment_key=False):
    """meta: [(key, value type, value)]; tensors: [(name, ggml dims (contiguous first), ggml type, raw bytes)]."""
    meta = list(meta)
    tensors = [(n, d, t, raw if isinstance(raw, (bytes, bytearray)) else np.ascontiguousarray(raw).reshape(-1).view(np.uint8).tobytes())
               for n, d, t, raw in tensors]
    if write_alignment_key:
        meta.append(("general.alignment", U32, alignment))
    out = struct.pack("<IIQQ", magic, version, len(tensors), len(meta))
    for key, vtype, v in meta:
        out += _s(key) + struct.pack("<I", vtype) + _value(vtype, v)
    offsets, pos = [], 0
    for _, _, _, raw in tensors:
        offsets.append(pos)
        pos += (len(raw) + alignment - 1) // alignment * alignment
    for (name, dims, gtype, raw), off in zip(tensors, offsets):
        out += _s(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        out += struct.pack("<IQ", gtype, off)
    out += b"\0" * ((-len(out)) % alignment)
    for _, _, _, raw in tensors:
        out += bytes(raw) + b"\0" * ((-len(raw)) % alignment)
    return out


def write(path, *args, **kw):
    data = gguf_bytes(*args, **kw)
    with open(path, "wb") as f:
        f.write(data)
    return data


def llama_meta(arch, hidden, inter, layers, heads, kv_heads, ctx, eps=None, theta=None, vocab=None):
    m = [("general.architecture", STR, arch), (arch + ".embedding_length", U32, hidden),
         (arch + ".feed_forward_length", U32, inter), (arch + ".block_count", U32, layers),
         (arch + ".attention.head_count", U32, heads), (arch + ".attention.head_count_kv", U32, kv_heads),
         (arch + ".context_length", U32, ctx)]
    if eps is not None:
        m.append((arch + ".attention.layer_norm_rms_epsilon", F32, eps))
    if theta is not None:
        m.append((arch + ".rope.freq_base", F32, theta))
    if vocab is not None:
        m.append((arch + ".vocab_size", U32, vocab))
    return m
