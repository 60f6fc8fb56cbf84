"""CPU restatement of the reference's GGUF block codecs (TEST INFRASTRUCTURE).

This module is the checker, never the product: only tests, the smoke check and
the CPU-baseline leg of the benchmark may import it.

Every function cites the reference file:line (paths relative to the reference
project root) whose behaviour it restates.

Block formats (neural/neuralgguf.pas:100-102, 127-131):
  Q8_0  34 bytes: fp16 scale d, then 32 int8 codes          x[i] = d * q[i]
  Q4_0  18 bytes: fp16 scale d, then 16 bytes of 32 nibbles x[e] = d * (nib(e) - 8)
        element e < 16 is the LOW nibble of byte e, element e >= 16 is the HIGH
        nibble of byte e - 16 (neural/neuralgguf.pas:811-817).
"""
import numpy as np

QK = 32
Q8_0_BLOCK_BYTES = 34
Q4_0_BLOCK_BYTES = 18

# ggml type ids as the GGUF container stores them (neural/neuralgguf.pas:100-131)
GGML_F32 = 0
GGML_F16 = 1
GGML_Q4_0 = 2
GGML_Q8_0 = 8
GGML_I8ROW = 124      # not a ggml id: int8 rows + one fp32 scale per row, host row = K codes then the scale


def half_to_single(bits):
    """IEEE half -> single by bit surgery, subnormals exact.

    Follows NeuralHalfToSingle (neural/neuralvolume.pas:1737-1770): zero keeps
    its sign, subnormal = mantissa * 2^-24, Inf/NaN rebuilt on the all-ones
    exponent, normal = exponent rebias 15 -> 127 and mantissa widened by 13 bits.
    """
    bits = np.asarray(bits, dtype=np.uint16).astype(np.uint32)
    sign = (bits >> 15) & 1
    exp = (bits >> 10) & 0x1F
    man = bits & 0x3FF
    out = np.empty(bits.shape, dtype=np.float32)
    normal_bits = (sign << 31) | ((exp + 112) << 23) | (man << 13)
    infnan_bits = (sign << 31) | (np.uint32(0xFF) << 23) | (man << 13)
    sub = man.astype(np.float32) * np.float32(5.9604644775390625e-8)
    sub = np.where(sign != 0, -sub, sub).astype(np.float32)
    zero_bits = (sign << 31)
    res_bits = np.where(exp == 0x1F, infnan_bits, normal_bits).astype(np.uint32)
    res_bits = np.where((exp == 0) & (man == 0), zero_bits, res_bits).astype(np.uint32)
    out = res_bits.view(np.float32).copy()
    submask = (exp == 0) & (man != 0)
    out[submask] = sub[submask]
    return out


def single_to_half(values):
    """single -> IEEE half, round-to-nearest-even on the dropped 13 bits.

    Follows EncodeF16 (neural/neuralsafetensors.pas:339-396) for every NORMAL
    half result, which is the only range a block scale of finite weights in
    the benchmark configurations reaches (|scale| >= 6.1e-5). The reference's
    subnormal branch rounds half-up instead of half-to-even; that branch is
    restated here too so the oracle agrees with it bit for bit.
    """
    v = np.ascontiguousarray(values, dtype=np.float32)
    bits = v.view(np.uint32)
    sign = ((bits >> 16) & 0x8000).astype(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int64)
    man = (bits & 0x7FFFFF).astype(np.uint32)
    e = exp - 127 + 15
    # normal branch
    half_n = ((np.clip(e, 0, 0x1F).astype(np.uint32) << 10) | (man >> 13)).astype(np.uint32)
    guard = (man & 0x1000) != 0
    sticky_or_odd = ((man & 0xFFF) != 0) | ((half_n & 1) == 1)
    half_n = half_n + (guard & sticky_or_odd).astype(np.uint32)
    # subnormal branch (E in -10..0): implicit one, shift, round on the last dropped bit
    man1 = man | np.uint32(0x800000)
    sh = np.clip(14 - e, 14, 24).astype(np.uint32)
    half_s = (man1 >> sh) + ((man1 >> (sh - 1)) & 1)
    res = np.where(e <= 0, half_s, half_n).astype(np.uint32)
    res = np.where(e < -10, 0, res)
    res = np.where(e >= 0x1F, 0x7C00, res)
    res = np.where((exp == 0xFF) & (man != 0), 0x7E00, res)
    res = np.where((exp == 0xFF) & (man == 0), 0x7C00, res)
    return (sign | res).astype(np.uint16)


def _blocks(raw, block_bytes):
    raw = np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    if raw.size % block_bytes:
        raise ValueError("byte count %d is not a whole number of %d-byte blocks" % (raw.size, block_bytes))
    return raw.reshape(-1, block_bytes)


def dequantize_q8_0(raw):
    """Q8_0 blocks -> float32, x = d * q with ONE fp32 multiply per element.

    Follows the GGML_TYPE_Q8_0 arm of DecodeGGMLSpan
    (neural/neuralgguf.pas:1487-1503): d = DecodeF16(first two bytes), then
    DequantizeInt8(codes, 32, d) = float(code) * d.
    """
    blk = _blocks(raw, Q8_0_BLOCK_BYTES)
    d = half_to_single(blk[:, :2].copy().view(np.uint16).reshape(-1))
    q = blk[:, 2:].view(np.int8).astype(np.float32)
    return (q * d[:, None]).astype(np.float32).reshape(-1)


def q4_0_codes(raw):
    """The 32 nibble values (0..15) of every Q4_0 block, in element order
    (LegacyNibble, neural/neuralgguf.pas:811-817)."""
    blk = _blocks(raw, Q4_0_BLOCK_BYTES)
    qs = blk[:, 2:]
    return np.concatenate([qs & 0x0F, qs >> 4], axis=1)


def dequantize_q4_0(raw):
    """Q4_0 blocks -> float32, x = d * (nibble - 8).

    Follows DequantizeQ4_0 (neural/neuralgguf.pas:822-845): the integer
    (nibble - 8) is converted to single and multiplied by d once.
    """
    blk = _blocks(raw, Q4_0_BLOCK_BYTES)
    d = half_to_single(blk[:, :2].copy().view(np.uint16).reshape(-1))
    codes = q4_0_codes(raw).astype(np.int32) - 8
    return (codes.astype(np.float32) * d[:, None]).astype(np.float32).reshape(-1)


def dequantize_f16(raw):
    """fp16 payload -> float32 (TNNetVolume.DecodeF16, neural/neuralvolume.pas:12584-12628)."""
    raw = np.ascontiguousarray(np.frombuffer(raw, dtype=np.uint8) if not isinstance(raw, np.ndarray) else raw)
    return half_to_single(raw.view(np.uint16).reshape(-1))


def dequantize(ggml_type, raw):
    if ggml_type == GGML_Q8_0:
        return dequantize_q8_0(raw)
    if ggml_type == GGML_Q4_0:
        return dequantize_q4_0(raw)
    if ggml_type == GGML_F16:
        return dequantize_f16(raw)
    if ggml_type == GGML_F32:
        raw = np.ascontiguousarray(raw)
        return raw.view(np.float32).reshape(-1).copy()
    raise ValueError("unsupported ggml type %d" % ggml_type)


def quantize_q8_0(x):
    """float32 [.., K] (K % 32 == 0) -> Q8_0 block bytes.

    Follows the gwQ8_0 arm of TNNetGGUFWriter.AddTensorFlat
    (neural/neuralgguf.pas:1950-1993): scale = absmax / 127 in fp32, stored as
    fp16; inv = 1 / scale computed from the UN-rounded fp32 scale (0 when the
    block is all zero); q = trunc(x * inv +- 0.5) (round half away from zero),
    clamped to [-127, 127].
    """
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, QK)
    absmax = np.max(np.abs(x), axis=1).astype(np.float32)
    scale = (absmax / np.float32(127.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(scale == 0, np.float32(0), np.float32(1.0) / scale).astype(np.float32)
    q = (x * inv[:, None]).astype(np.float32)
    e = np.where(q >= 0, np.trunc(q + np.float32(0.5)), np.trunc(q - np.float32(0.5)))
    e = np.clip(e, -127, 127).astype(np.int8)
    out = np.empty((x.shape[0], Q8_0_BLOCK_BYTES), dtype=np.uint8)
    out[:, :2] = single_to_half(scale).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = e.view(np.uint8)
    return out.reshape(-1)


def quantize_q4_0(x):
    """float32 [.., K] (K % 32 == 0) -> Q4_0 block bytes.

    The reference has NO Q4_0 encoder (its writer emits F32/F16/Q8_0 only,
    neural/neuralgguf.pas:251), so this restates the published ggml rule that
    produces the files the reference reads (quantize_row_q4_0_ref in ggml, the
    same rule the `gguf` Python package implements): take the element with the
    largest magnitude KEEPING ITS SIGN, d = max / -8, id = 1/d (0 if d == 0),
    code = min(15, trunc(x * id + 8.5)); element e < 16 goes to the low nibble
    of byte e, element e >= 16 to the high nibble of byte e - 16.
    """
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, QK)
    idx = np.argmax(np.abs(x), axis=1)
    mx = x[np.arange(x.shape[0]), idx]
    d = (mx / np.float32(-8.0)).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, np.float32(0), np.float32(1.0) / d).astype(np.float32)
    q = np.trunc((x * inv[:, None]).astype(np.float32) + np.float32(8.5))
    q = np.clip(q, 0, 15).astype(np.uint8)
    out = np.empty((x.shape[0], Q4_0_BLOCK_BYTES), dtype=np.uint8)
    out[:, :2] = single_to_half(d).view(np.uint8).reshape(-1, 2)
    out[:, 2:] = q[:, :16] | (q[:, 16:] << 4)
    return out.reshape(-1)


def quantize_int8_rows(w):
    """float32 [rows, K] -> (int8 codes [rows, K], float32 scales [rows]): the reference's own weight format.

    TNNetVolume.MaxAbsFinite + QuantizeInt8, scalar form (neural/neuralvolume.pas:12471-12562): maxabs over the
    finite magnitudes of the row; scale = maxabs / 127; code = Round(v * (1 / maxabs) * 127), the two products in
    that order in single precision, clamped to +-127 (which maps +-Inf), Pascal Round = half to even, NaN -> 0; a
    denormal row maximum scales in double precision (127 / maxabs); an all-zero row keeps zero codes (scale 0).
    """
    w = np.ascontiguousarray(w, dtype=np.float32)
    rows, k = w.shape
    codes = np.zeros((rows, k), dtype=np.int8)
    scales = np.zeros(rows, dtype=np.float32)
    min_single = np.float32(1.1754943508222875e-38)
    for r in range(rows):
        v = w[r]
        a = np.abs(v)
        fin = np.isfinite(a)
        m = np.float32(a[fin].max()) if fin.any() else np.float32(0)
        scales[r] = m / np.float32(127.0)
        if m <= 0:
            continue
        nan = np.isnan(v)
        if m < min_single:
            vc = np.clip(v.astype(np.float64), -float(m), float(m))
            sc = np.rint(vc * (127.0 / float(m)))
        else:
            recip = np.float32(1.0) / m
            with np.errstate(over="ignore", invalid="ignore"):
                sc = ((v * recip).astype(np.float32) * np.float32(127.0)).astype(np.float32)
            sc = np.rint(np.clip(sc, -127.0, 127.0))
        sc = np.where(nan, 0.0, np.clip(sc, -127.0, 127.0))
        codes[r] = sc.astype(np.int8)
    return codes, scales


def linear_int8_rows(codes, scales, x, bias=None):
    """y[b, a] = (sum_i codes[a, i] * x[b, i]) * scales[a] (+ bias): the raw code reduction in fp32 with the row's scale
    applied once after the sum, DotProductsTiledInt8 (neural/neuralvolume.pas:12693-12745). Accumulates in float64 and
    rounds once, so it serves as the exact value both fp32 orders are compared against."""
    acc = x.astype(np.float64) @ codes.astype(np.float64).T
    y = acc * scales.astype(np.float64)[None, :]
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float64)[None, :]
    return y.astype(np.float32)


def split_int8_rows(raw, rows, k):
    """Host rows of the int8-row type ([K code bytes | fp32 scale] per row) -> (int8 codes [rows, K], fp32 scales [rows])."""
    raw = np.ascontiguousarray(raw, dtype=np.uint8)[:rows * (k + 4)].reshape(rows, k + 4)
    return raw[:, :k].copy().view(np.int8), raw[:, k:].copy().view(np.float32).reshape(rows)


def dequantize_int8_rows(codes, scales):
    """DequantizeInt8: code * row scale (one fp32 multiply)."""
    return (codes.astype(np.float32) * scales.astype(np.float32)[:, None]).astype(np.float32)


def block_bytes_per_row(ggml_type, k):
    if ggml_type == GGML_I8ROW:
        return k + 4
    if ggml_type == GGML_Q8_0:
        return k // QK * Q8_0_BLOCK_BYTES
    if ggml_type == GGML_Q4_0:
        return k // QK * Q4_0_BLOCK_BYTES
    if ggml_type == GGML_F16:
        return 2 * k
    if ggml_type == GGML_F32:
        return 4 * k
    raise ValueError("unsupported ggml type %d" % ggml_type)


def linear_fp32(w_deq, x, bias=None):
    """y[b, a] = sum_i w[a, i] * x[b, i] (+ bias[a]) in fp32.

    The FP32-weight linear a GGUF Q8_0/Q4_0 import runs in the reference:
    TNNetVolume.DotProductsTiled (neural/neuralvolume.pas:12127-12423) over the
    dequantized weights, output layout out[b * NumAs + a]
    (neural/neuralvolume.pas:12736). Summation order differs from the AVX lanes
    (BLAS here), which is inside fp32 rounding noise.
    """
    y = np.asarray(x, dtype=np.float32) @ np.asarray(w_deq, dtype=np.float32).T
    if bias is not None:
        y = y + np.asarray(bias, dtype=np.float32)
    return y.astype(np.float32)
