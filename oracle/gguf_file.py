"""CPU restatement of the reference's GGUF container reader and of its legacy / K-quant block decoders
(TEST INFRASTRUCTURE: the checker of the library's C-side reader, never the product).

Every function cites the reference file:line (paths relative to the reference project root) it restates.

Decoders return float32 in flat row-major order. All arithmetic is single precision with one rounding per
operation, the way the reference's Pascal expressions evaluate: a product `d * sc` is rounded before it meets the
code, and `dl * q - ml` is a rounded multiply followed by a rounded subtract.
"""
import struct
import numpy as np

from .codecs import half_to_single, _blocks, dequantize as _dequantize_basic

QK_K = 256
# ggml type ids (neural/neuralgguf.pas:100-131)
GGML_Q4_1, GGML_Q5_0, GGML_Q5_1 = 3, 6, 7
GGML_Q2_K, GGML_Q3_K, GGML_Q4_K, GGML_Q5_K, GGML_Q6_K = 10, 11, 12, 13, 14

# bytes per block and elements per block (GGMLByteSize / GGMLBlockElems, neural/neuralgguf.pas:375-423)
BLOCK = {0: (4, 1), 1: (2, 1), 2: (18, 32), 3: (20, 32), 6: (22, 32), 7: (24, 32), 8: (34, 32),
         10: (84, 256), 11: (110, 256), 12: (144, 256), 13: (176, 256), 14: (210, 256)}


def _f16(col):
    return half_to_single(np.ascontiguousarray(col).view(np.uint16).reshape(-1))


def _legacy_nibbles(qs):
    """[nb,16] bytes -> [nb,32] nibbles: element e < 16 is the low nibble of byte e, e >= 16 the high nibble of
    byte e - 16 (LegacyNibble, neural/neuralgguf.pas:811-817)."""
    return np.concatenate([qs & 0x0F, qs >> 4], axis=1).astype(np.int32)


def _qh_bits(qh4):
    """[nb,4] bytes (a little-endian 32-bit plane) -> [nb,32] bits, bit e for element e."""
    word = np.ascontiguousarray(qh4).view("<u4").reshape(-1, 1)
    return ((word >> np.arange(32, dtype=np.uint32)[None, :]) & 1).astype(np.int32)


def dequantize_q4_1(raw):
    """20-byte blocks: f16 d, f16 m, 16 nibble bytes; x = d * nibble + m (DequantizeQ4_1, neuralgguf.pas:850-874)."""
    blk = _blocks(raw, 20)
    d, m = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
    q = _legacy_nibbles(blk[:, 4:]).astype(np.float32)
    return ((d[:, None] * q).astype(np.float32) + m[:, None]).astype(np.float32).reshape(-1)


def dequantize_q5_0(raw):
    """22-byte blocks: f16 d, 4 bytes qh, 16 nibble bytes; x = d * ((nibble | bit << 4) - 16)
    (DequantizeQ5_0, neuralgguf.pas:879-908)."""
    blk = _blocks(raw, 22)
    d = _f16(blk[:, 0:2])
    q = _legacy_nibbles(blk[:, 6:]) | (_qh_bits(blk[:, 2:6]) << 4)
    return (d[:, None] * (q - 16).astype(np.float32)).astype(np.float32).reshape(-1)


def dequantize_q5_1(raw):
    """24-byte blocks: f16 d, f16 m, 4 bytes qh, 16 nibble bytes; x = d * (nibble | bit << 4) + m
    (DequantizeQ5_1, neuralgguf.pas:913-945)."""
    blk = _blocks(raw, 24)
    d, m = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
    q = _legacy_nibbles(blk[:, 8:]) | (_qh_bits(blk[:, 4:8]) << 4)
    return ((d[:, None] * q.astype(np.float32)).astype(np.float32) + m[:, None]).astype(np.float32).reshape(-1)


def _scale_min_k4(packed):
    """[nb,12] bytes -> ([nb,8] scales, [nb,8] mins), 6 bits each (DequantizeQ4KScaleMin, neuralgguf.pas:448-465)."""
    d, m, md = packed[:, 0:4], packed[:, 4:8], packed[:, 8:12]
    sc = np.concatenate([d & 0x3F, (md & 0x0F) | ((d >> 2) & 0x30)], axis=1)
    mn = np.concatenate([m & 0x3F, (md >> 4) | ((m >> 2) & 0x30)], axis=1)
    return sc.astype(np.float32), mn.astype(np.float32)


def dequantize_q4_k(raw):
    """144-byte super-blocks of 256: f16 d, f16 dmin, 12 scale bytes, 128 nibble bytes; chunk c of 32 bytes holds
    sub-block 2c in the low and 2c+1 in the high nibble; x = (d*sc)*q - (dmin*mn) (DequantizeQ4K, :474-520)."""
    blk = _blocks(raw, 144)
    nb = blk.shape[0]
    d, dmin = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
    sc, mn = _scale_min_k4(blk[:, 4:16])
    qs = blk[:, 16:].reshape(nb, 4, 32)
    q = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.float32)
    dl = (d[:, None] * sc).astype(np.float32)
    ml = (dmin[:, None] * mn).astype(np.float32)
    return ((dl[:, :, None] * q).astype(np.float32) - ml[:, :, None]).astype(np.float32).reshape(-1)


def dequantize_q5_k(raw):
    """176-byte super-blocks: f16 d, f16 dmin, 12 scale bytes, 32 bytes qh, 128 nibble bytes; sub-block j takes bit j
    of qh byte i as its fifth bit (DequantizeQ5K, :536-590)."""
    blk = _blocks(raw, 176)
    nb = blk.shape[0]
    d, dmin = _f16(blk[:, 0:2]), _f16(blk[:, 2:4])
    sc, mn = _scale_min_k4(blk[:, 4:16])
    qh = blk[:, 16:48]
    qs = blk[:, 48:].reshape(nb, 4, 32)
    ql = np.stack([qs & 0x0F, qs >> 4], axis=2).reshape(nb, 8, 32).astype(np.int32)
    hb = ((qh[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1).astype(np.int32)
    q = (ql | (hb << 4)).astype(np.float32)
    dl = (d[:, None] * sc).astype(np.float32)
    ml = (dmin[:, None] * mn).astype(np.float32)
    return ((dl[:, :, None] * q).astype(np.float32) - ml[:, :, None]).astype(np.float32).reshape(-1)


def _two_bit_plane(qs, nb):
    """[nb,64] bytes -> [nb,256] 2-bit fields: element e = (c, s, p) with c = e div 128, s = (e mod 128) div 32,
    p = e mod 32 sits at shift 2s of byte c*32 + p."""
    qs = qs.reshape(nb, 2, 1, 32)
    sh = np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 4, 1)
    return ((qs >> sh) & 3).reshape(nb, 256).astype(np.int32)


def dequantize_q2_k(raw):
    """84-byte super-blocks: 16 bytes (scale low nibble | min high nibble), 64 bytes of 2-bit codes, f16 d, f16 dmin;
    16 sub-blocks of 16; x = (d*scale)*q - (dmin*min) (DequantizeQ2K, :606-660)."""
    blk = _blocks(raw, 84)
    nb = blk.shape[0]
    scb = blk[:, 0:16]
    d, dmin = _f16(blk[:, 80:82]), _f16(blk[:, 82:84])
    q = _two_bit_plane(blk[:, 16:80], nb).reshape(nb, 16, 16).astype(np.float32)
    dl = (d[:, None] * (scb & 0x0F).astype(np.float32)).astype(np.float32)
    ml = (dmin[:, None] * (scb >> 4).astype(np.float32)).astype(np.float32)
    return ((dl[:, :, None] * q).astype(np.float32) - ml[:, :, None]).astype(np.float32).reshape(-1)


def dequantize_q6_k(raw):
    """210-byte super-blocks: 128 bytes ql, 64 bytes qh, 16 int8 group scales, f16 d; q = (ql | qh << 4) - 32;
    x = (d*scale[g]) * q with g = e div 16 (DequantizeQ6K, :676-738)."""
    blk = _blocks(raw, 210)
    nb = blk.shape[0]
    ql = blk[:, 0:128].reshape(nb, 2, 1, 64)
    ql = ((ql >> np.array([0, 4], dtype=np.uint8).reshape(1, 1, 2, 1)) & 0x0F).reshape(nb, 256).astype(np.int32)
    qh = blk[:, 128:192].reshape(nb, 2, 1, 32)
    qh = ((qh >> np.array([0, 2, 4, 6], dtype=np.uint8).reshape(1, 1, 4, 1)) & 3).reshape(nb, 256).astype(np.int32)
    q = ((ql | (qh << 4)) - 32).reshape(nb, 16, 16).astype(np.float32)
    scales = np.ascontiguousarray(blk[:, 192:208]).view(np.int8).astype(np.float32)
    d = _f16(blk[:, 208:210])
    dl = (d[:, None] * scales).astype(np.float32)
    return (dl[:, :, None] * q).astype(np.float32).reshape(-1)


def dequantize_q3_k(raw):
    """110-byte super-blocks: 32 bytes hmask, 64 bytes of 2-bit codes, 12 bytes of packed 6-bit scales, f16 d;
    scale j = (low nibble of byte j mod 8 (high nibble for j >= 8) | 2 bits of byte 8 + j mod 4 at shift 2*(j div 4))
    - 32; q = ql - 4 when the hmask bit (e div 32) of byte (e mod 32) is clear; x = (d*scale) * q
    (DequantizeQ3K, :762-806)."""
    blk = _blocks(raw, 110)
    nb = blk.shape[0]
    hm = blk[:, 0:32]
    ql = _two_bit_plane(blk[:, 32:96], nb)
    scp = blk[:, 96:108]
    j = np.arange(16)
    lsc = np.where(j[None, :] < 8, scp[:, j & 7] & 0x0F, (scp[:, j & 7] >> 4) & 0x0F).astype(np.int32)
    hsc = ((scp[:, 8 + (j & 3)] >> ((j >> 2) * 2).astype(np.uint8)[None, :]) & 3).astype(np.int32)
    scales = ((lsc | (hsc << 4)) - 32).astype(np.float32)
    d = _f16(blk[:, 108:110])
    hbit = ((hm[:, None, :] >> np.arange(8, dtype=np.uint8)[None, :, None]) & 1).reshape(nb, 256).astype(np.int32)
    q = (ql - ((hbit ^ 1) << 2)).reshape(nb, 16, 16).astype(np.float32)
    dl = (d[:, None] * scales).astype(np.float32)
    return (dl[:, :, None] * q).astype(np.float32).reshape(-1)


_DECODERS = {GGML_Q4_1: dequantize_q4_1, GGML_Q5_0: dequantize_q5_0, GGML_Q5_1: dequantize_q5_1,
             GGML_Q2_K: dequantize_q2_k, GGML_Q3_K: dequantize_q3_k, GGML_Q4_K: dequantize_q4_k,
             GGML_Q5_K: dequantize_q5_k, GGML_Q6_K: dequantize_q6_k}


def decode_span(ggml_type, raw):
    """Raw tensor bytes of any supported type -> float32 (DecodeGGMLSpan, neural/neuralgguf.pas:1471-1523)."""
    if ggml_type in _DECODERS:
        return _DECODERS[ggml_type](raw)
    return _dequantize_basic(ggml_type, raw)


class GGUFError(ValueError):
    pass


class GGUFFile:
    """Header, metadata and tensor table of one GGUF file (TNNetGGUFReader.ParseFile, neural/neuralgguf.pas:1072-1220).

    meta: key -> (value_type, value); arrays become lists. tensors: name -> dict(shape (contiguous axis LAST, i.e.
    the stored dims reversed), type, begin, end) with offsets relative to data_start.
    """

    def __init__(self, path):
        with open(path, "rb") as f:
            self.buf = f.read()
        self.pos = 0
        self.meta, self.tensors, self.order = {}, {}, []
        self._parse()

    def _take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.buf):
            raise GGUFError("gguf: read past the end of file")
        v = struct.unpack_from(fmt, self.buf, self.pos)[0]
        self.pos += size
        return v

    def _string(self):
        n = self._take("<Q")
        if n > len(self.buf) - self.pos:
            raise GGUFError("gguf: string length runs past the end of file")
        s = self.buf[self.pos:self.pos + n].decode("utf-8", "replace")
        self.pos += n
        return s

    _SCALAR = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}

    def _scalar(self, t, key):
        if t == 8:
            return self._string()
        if t not in self._SCALAR:
            raise GGUFError('gguf: metadata key "%s" has unsupported value type %d' % (key, t))
        return self._take(self._SCALAR[t])

    def _parse(self):
        if len(self.buf) < 24:
            raise GGUFError("gguf: file too small")
        if self._take("<I") != 0x46554747:
            raise GGUFError("gguf: bad magic")
        self.version = self._take("<I")
        if self.version not in (2, 3):
            raise GGUFError("gguf: unsupported version %d" % self.version)
        n_tensors, n_kv = self._take("<Q"), self._take("<Q")
        if n_tensors > 0x7FFFFFFF or n_kv > 0x7FFFFFFF:
            raise GGUFError("gguf: implausible header counts")
        for _ in range(n_kv):
            key = self._string()
            if key == "":
                raise GGUFError("gguf: empty metadata key")
            if key in self.meta:
                raise GGUFError('gguf: duplicate metadata key "%s"' % key)
            t = self._take("<I")
            if t == 9:
                et = self._take("<I")
                if et == 9:
                    raise GGUFError('gguf: metadata key "%s" is a nested array' % key)
                cnt = self._take("<Q")
                if cnt > 0x7FFFFFFF:
                    raise GGUFError('gguf: metadata array "%s" is too large' % key)
                self.meta[key] = (9, [self._scalar(et, key) for _ in range(cnt)])
            else:
                self.meta[key] = (t, self._scalar(t, key))
        for _ in range(n_tensors):
            name = self._string()
            if name == "":
                raise GGUFError("gguf: empty tensor name")
            if name in self.tensors:
                raise GGUFError('gguf: duplicate tensor name "%s"' % name)
            nd = self._take("<I")
            if nd < 1 or nd > 8:
                raise GGUFError('gguf: tensor "%s" has implausible n_dims %d' % (name, nd))
            dims = []
            for _ in range(nd):
                v = self._take("<Q")
                if v == 0 or v > 0x7FFFFFFF:
                    raise GGUFError('gguf: tensor "%s" has implausible dimension %d' % (name, v))
                dims.append(v)
            t = self._take("<I")
            n = int(np.prod(np.array(dims, dtype=np.int64)))
            if t in (8, 2, 3, 6, 7) and dims[0] % 32:
                raise GGUFError('gguf: tensor "%s" contiguous dimension is not a multiple of 32' % name)
            if t in (10, 11, 12, 13, 14) and dims[0] % QK_K:
                raise GGUFError('gguf: tensor "%s" contiguous dimension is not a multiple of 256' % name)
            begin = self._take("<Q")
            size = (n // BLOCK[t][1]) * BLOCK[t][0] if t in BLOCK else 0
            self.tensors[name] = dict(shape=dims[::-1], type=t, begin=begin, end=begin + size)
            self.order.append(name)
        align = self.get_int("general.alignment", 32)
        if align < 1 or (align & (align - 1)):
            raise GGUFError("gguf: general.alignment %d is not a positive power of two" % align)
        self.alignment = align
        self.data_start = (self.pos + align - 1) // align * align
        if self.data_start > len(self.buf):
            raise GGUFError("gguf: header ends past the end of the file")
        data_size = len(self.buf) - self.data_start
        for name, t in self.tensors.items():
            if t["begin"] < 0 or t["end"] > data_size:
                raise GGUFError('gguf: tensor "%s" data falls outside the data section' % name)

    # GetMetaInt / GetMetaFloat / GetMetaString (neural/neuralgguf.pas:1263-1314)
    def get_int(self, key, default):
        if key not in self.meta:
            return default
        t, v = self.meta[key]
        if t in (0, 1, 2, 3, 4, 5, 7, 10, 11):
            return int(v)
        raise GGUFError('gguf: metadata key "%s" (type %d) is not an integer' % (key, t))

    def get_float(self, key, default):
        if key not in self.meta:
            return default
        t, v = self.meta[key]
        if t in (6, 12, 0, 1, 2, 3, 4, 5, 10, 11):
            return float(v)
        raise GGUFError('gguf: metadata key "%s" (type %d) is not a number' % (key, t))

    def get_string(self, key, default):
        if key not in self.meta:
            return default
        t, v = self.meta[key]
        if t != 8:
            raise GGUFError('gguf: metadata key "%s" (type %d) is not a string' % (key, t))
        return v

    def raw(self, name):
        t = self.tensors[name]
        return np.frombuffer(self.buf, dtype=np.uint8, count=t["end"] - t["begin"],
                             offset=self.data_start + t["begin"])

    def load(self, name):
        """LoadTensorFlat: the tensor decoded to float32 in its served (row-major) shape."""
        t = self.tensors[name]
        if t["type"] not in BLOCK:
            raise GGUFError('gguf: tensor "%s" has unsupported type %d' % (name, t["type"]))
        return decode_span(t["type"], self.raw(name)).reshape(t["shape"])


# ggml tensor names -> HF names (BuildLlamaFromGGUFEx, neural/neuralpretrained.pas:17573-17600; the qwen2 arm of
# BuildFromGGUFEx, :17804-17848)
_TOP = {"token_embd.weight": "model.embed_tokens.weight", "output_norm.weight": "model.norm.weight",
        "output.weight": "lm_head.weight"}
_BLK = {"attn_norm.weight": "input_layernorm.weight", "attn_q.weight": "self_attn.q_proj.weight",
        "attn_k.weight": "self_attn.k_proj.weight", "attn_v.weight": "self_attn.v_proj.weight",
        "attn_output.weight": "self_attn.o_proj.weight", "ffn_norm.weight": "post_attention_layernorm.weight",
        "ffn_gate.weight": "mlp.gate_proj.weight", "ffn_up.weight": "mlp.up_proj.weight",
        "ffn_down.weight": "mlp.down_proj.weight", "attn_q.bias": "self_attn.q_proj.bias",
        "attn_k.bias": "self_attn.k_proj.bias", "attn_v.bias": "self_attn.v_proj.bias"}


def hf_name(name):
    if name in _TOP:
        return _TOP[name]
    p = name.split(".", 2)
    if len(p) == 3 and p[0] == "blk" and p[2] in _BLK:
        return "model.layers.%s.%s" % (p[1], _BLK[p[2]])
    return None


def llama_config(g):
    """Metadata -> the configuration fields the decode path uses (BuildLlamaFromGGUFEx,
    neural/neuralpretrained.pas:17519-17570; qwen2 arm of BuildFromGGUFEx, :17706-17770)."""
    arch = g.get_string("general.architecture", "")
    if arch not in ("llama", "qwen2"):
        raise GGUFError('GGUF import: general.architecture "%s" is not supported' % arch)

    def req(suffix):
        v = g.get_int(arch + "." + suffix, -1)
        if v <= 0:
            raise GGUFError('GGUF import: metadata key "%s.%s" is missing or not a positive integer' % (arch, suffix))
        return v
    cfg = dict(arch=arch, hidden=req("embedding_length"), inter=req("feed_forward_length"), layers=req("block_count"),
               heads=req("attention.head_count"))
    cfg["kv_heads"] = g.get_int(arch + ".attention.head_count_kv", cfg["heads"])
    cfg["max_positions"] = req("context_length")
    cfg["rms_eps"] = g.get_float(arch + ".attention.layer_norm_rms_epsilon", 1e-5 if arch == "llama" else 1e-6)
    cfg["rope_theta"] = g.get_float(arch + ".rope.freq_base", 10000.0)
    hd = g.get_int(arch + ".attention.key_length", 0)
    vocab = g.get_int(arch + ".vocab_size", 0)
    if vocab <= 0:
        t = g.tensors.get("token_embd.weight")
        if t is not None and len(t["shape"]) == 2:
            vocab = t["shape"][0]
        elif "tokenizer.ggml.tokens" in g.meta:
            vocab = len(g.meta["tokenizer.ggml.tokens"][1])
    if vocab <= 0:
        raise GGUFError("GGUF import: cannot determine the vocab size")
    cfg["vocab"] = vocab
    cfg["tie_embeddings"] = int("output.weight" not in g.tensors)
    if hd <= 0:
        if cfg["hidden"] % cfg["heads"]:
            raise GGUFError("GGUF import: embedding_length is not divisible by head_count")
        hd = cfg["hidden"] // cfg["heads"]
    cfg["head_dim"] = hd
    cfg["qkv_bias"] = int(arch == "qwen2")
    return cfg
