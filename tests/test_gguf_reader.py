"""The C-side GGUF reader (no GPU needed: header, metadata and tensor table are host work) against the CPU
restatement of TNNetGGUFReader, on the reference's own fixture files and on hand-written files; the refusals follow
ParseFile (neural/neuralgguf.pas:1072-1220). Also pins the restated block decoders against the reference's K-quant
fixture and the `gguf` package's dequantisation."""
import struct

import numpy as np
import pytest

import gguf_util as W
from conftest import load_golden
from oracle import gguf_file as GF
from neural_api_b200.backend import GGUFError, GGUFReader

FILES = ["tiny_kquant.gguf", "tiny_llama_q8.gguf", "tiny_llama_f16.gguf", "tiny_llama_f32.gguf"]


def _fixture(tmp_path, name):
    z = load_golden("gguf_files")
    p = tmp_path / name
    p.write_bytes(bytes(z["file::" + name]))
    return p


# ---- the oracle itself -------------------------------------------------------------------------------------------
def test_oracle_decoders_match_the_reference_kquant_fixture(tmp_path):
    """tests/fixtures/tiny_kquant.gguf against tiny_kquant_ref.json (TestGGUFKQuantDecodeParity,
    tests/TestNeuralPretrained.pas:5931-6020): the restated decoders give the reference values bit for bit."""
    z = load_golden("gguf_files")
    g = GF.GGUFFile(_fixture(tmp_path, "tiny_kquant.gguf"))
    for tname in ("Q4_K", "Q5_K", "Q6_K", "Q2_K"):
        x = g.load("kq.%s.weight" % tname).reshape(-1)
        assert np.array_equal(x.view(np.uint32), z["kquant::" + tname].view(np.uint32)), tname
    assert np.array_equal(g.load("ref.f32.weight").reshape(-1), z["kquant::ref_f32"])
    # the source tolerances of the reference test: 4-bit 1.5, 5-bit 0.9, 6-bit 0.6, 2-bit 3.5
    for tname, tol in (("Q4_K", 1.5), ("Q5_K", 0.9), ("Q6_K", 0.6), ("Q2_K", 3.5)):
        assert np.max(np.abs(g.load("kq.%s.weight" % tname).reshape(-1) - z["kquant::ref_f32"])) < tol


def test_oracle_decoders_match_the_gguf_package_on_random_blocks():
    z = load_golden("block_kats")
    for t in (2, 3, 6, 7, 8, 10, 11, 12, 13, 14):
        mine = GF.decode_span(t, z["raw::%d" % t])
        assert np.array_equal(mine.view(np.uint32), z["deq::%d" % t].view(np.uint32)), t


def test_oracle_legacy_and_q3k_closed_forms():
    """Hand-rolled blocks with closed-form values (TestGGUFQ3KAndLegacyDecodeParity,
    tests/TestNeuralPretrained.pas:6022+): element e carries code e mod 16 (4-bit) or e (5-bit)."""
    def f16(v):
        return np.asarray([v], dtype=np.float16)
    d, m = f16(0.3), f16(-1.25)
    df, mf = np.float32(d[0]), np.float32(m[0])
    nib = bytes((e | (e << 4)) & 0xFF for e in range(16))                  # element e and e + 16 both carry e
    q41 = d.tobytes() + m.tobytes() + nib
    want = np.asarray([np.float32(df * np.float32(e % 16)) + mf for e in range(32)], dtype=np.float32)
    assert np.array_equal(GF.dequantize_q4_1(np.frombuffer(q41, dtype=np.uint8)), want)
    # 5-bit: code e in 0..31 -> low nibble e & 15 at the legacy position, bit 4 in the qh plane
    qs = bytearray(16)
    qh = 0
    for e in range(32):
        qs[e % 16] |= (e & 15) << (0 if e < 16 else 4)
        qh |= ((e >> 4) & 1) << e
    q50 = d.tobytes() + struct.pack("<I", qh) + bytes(qs)
    want = np.asarray([df * np.float32(e - 16) for e in range(32)], dtype=np.float32)
    assert np.array_equal(GF.dequantize_q5_0(np.frombuffer(q50, dtype=np.uint8)), want)
    q51 = d.tobytes() + m.tobytes() + struct.pack("<I", qh) + bytes(qs)
    want = np.asarray([np.float32(df * np.float32(e)) + mf for e in range(32)], dtype=np.float32)
    assert np.array_equal(GF.dequantize_q5_1(np.frombuffer(q51, dtype=np.uint8)), want)


# ---- the C-side reader against the oracle ------------------------------------------------------------------------------
@pytest.mark.parametrize("name", FILES)
def test_reader_tables_equal_the_oracle_on_the_reference_fixtures(tmp_path, name):
    p = _fixture(tmp_path, name)
    g = GF.GGUFFile(p)
    r = GGUFReader(p)
    try:
        assert (r.version, r.alignment, r.data_start) == (g.version, g.alignment, g.data_start)
        assert r.tensor_count == len(g.order) and r.meta_count == len(g.meta)
        assert [k for k, _ in r.meta_keys()] == list(g.meta)
        for (k, vt) in r.meta_keys():
            t, v = g.meta[k]
            assert vt == t
            if t == 8:
                assert r.get_meta_string(k, None) == v
            elif t in (6, 12):
                assert r.get_meta_float(k, None) == float(v)
            elif t == 9:
                assert r.get_meta_array_count(k) == len(v)
            else:
                assert r.get_meta_int(k, None) == int(v)
        for i, n in enumerate(g.order):
            name_c, ty, shape, beg, nbytes = r.tensor_info(i)
            t = g.tensors[n]
            assert (name_c, ty, shape, beg, nbytes) == (n, t["type"], list(t["shape"]), t["begin"], t["end"] - t["begin"])
            assert r.find_tensor(n) == i
            assert np.array_equal(r.read_raw(i), g.raw(n))
        assert r.find_tensor("no.such.tensor") == -1 and not r.has_tensor("no.such.tensor")
        assert r.get_meta_int("no.such.key", -7) == -7 and r.get_meta_string("no.such.key", "dflt") == "dflt"
    finally:
        r.close()


@pytest.mark.parametrize("name", FILES[1:])
def test_reader_llama_config_equals_the_oracle(tmp_path, name):
    p = _fixture(tmp_path, name)
    want = GF.llama_config(GF.GGUFFile(p))
    r = GGUFReader(p)
    try:
        cfg, max_pos = r.llama_config()
        got = dict(hidden=cfg.hidden, inter=cfg.inter, layers=cfg.layers, heads=cfg.heads, kv_heads=cfg.kv_heads,
                   head_dim=cfg.head_dim, vocab=cfg.vocab, tie_embeddings=cfg.tie_embeddings, qkv_bias=cfg.qkv_bias)
        assert got == {k: want[k] for k in got}
        assert max_pos == want["max_positions"]
        assert cfg.rms_eps == np.float32(want["rms_eps"]) and cfg.rope_theta == np.float32(want["rope_theta"])
    finally:
        r.close()


def test_reader_metadata_types_and_defaults(tmp_path):
    meta = [("a.u8", W.U8, 200), ("a.i8", W.I8, -5), ("a.u16", W.U16, 60000), ("a.i16", W.I16, -30000),
            ("a.u32", W.U32, 4000000000), ("a.i32", W.I32, -2000000000), ("a.u64", W.U64, 1 << 40), ("a.i64", W.I64, -(1 << 40)),
            ("a.f32", W.F32, 0.5), ("a.f64", W.F64, 1e-300), ("a.bool", W.BOOL, 1), ("a.str", W.STR, "héllo"),
            ("a.arr_s", W.ARR, (W.STR, ["x", "yy", ""])), ("a.arr_i", W.ARR, (W.I32, [1, -2, 3, 4]))]
    p = tmp_path / "meta.gguf"
    W.write(p, meta, [("w", [32], 0, np.zeros(32, np.float32))], version=2, alignment=64, write_alignment_key=True)
    g = GF.GGUFFile(p)
    r = GGUFReader(p)
    try:
        assert r.version == 2 and r.alignment == 64 and r.data_start == g.data_start and r.data_start % 64 == 0
        for k in ("a.u8", "a.i8", "a.u16", "a.i16", "a.u32", "a.i32", "a.u64", "a.i64", "a.bool"):
            assert r.get_meta_int(k, None) == g.get_int(k, None)
            if k != "a.bool":
                assert r.get_meta_float(k, None) == float(g.get_int(k, None))      # ints read as numbers
        assert r.get_meta_float("a.f32", None) == 0.5 and r.get_meta_float("a.f64", None) == 1e-300
        assert r.get_meta_string("a.str", None) == "héllo"
        assert r.get_meta_array_count("a.arr_s") == 3 and r.get_meta_array_count("a.arr_i") == 4
        assert r.get_meta_array_count("absent") == 0
        # a key of another type is an error, as in GetMetaInt / GetMetaString / GetMetaFloat
        with pytest.raises(GGUFError):
            r.get_meta_int("a.f32", 0)
        with pytest.raises(GGUFError):
            r.get_meta_string("a.u8", "")
        with pytest.raises(GGUFError):
            r.get_meta_float("a.str", 0.0)
        with pytest.raises(GGUFError):
            r.get_meta_float("a.bool", 0.0)
        with pytest.raises(GGUFError):
            r.get_meta_array_count("a.u8")
    finally:
        r.close()


def test_reader_serves_dims_reversed(tmp_path):
    p = tmp_path / "dims.gguf"
    W.write(p, [], [("w3", [32, 3, 2], 0, np.zeros(192, np.float32)), ("w1", [64], 8, np.zeros(68, np.uint8))])
    r = GGUFReader(p)
    try:
        assert r.tensor_info(0)[2] == [2, 3, 32] and r.tensor_info(1)[2] == [64]
        assert r.tensor_info(1)[3] == 768 and r.tensor_info(1)[4] == 68
    finally:
        r.close()


def _bad(tmp_path, data, match):
    p = tmp_path / "bad.gguf"
    p.write_bytes(data)
    with pytest.raises(GF.GGUFError):
        GF.GGUFFile(p)                                   # the oracle refuses the same file
    with pytest.raises(GGUFError, match=match):
        GGUFReader(p)


def test_reader_refusals(tmp_path):
    ok_t = [("w", [32], 0, np.zeros(32, np.float32))]
    _bad(tmp_path, b"GGUF" + b"\0" * 8, "too small")
    _bad(tmp_path, W.gguf_bytes([], ok_t, magic=0x12345678), "bad magic")
    _bad(tmp_path, W.gguf_bytes([], ok_t, version=1), "unsupported version 1")
    _bad(tmp_path, W.gguf_bytes([], ok_t, version=4), "unsupported version 4")
    _bad(tmp_path, struct.pack("<IIQQ", 0x46554747, 3, 1 << 40, 0) + b"\0" * 32, "implausible header counts")
    _bad(tmp_path, W.gguf_bytes([("", W.U8, 1)], ok_t), "empty metadata key")
    _bad(tmp_path, W.gguf_bytes([("k", W.U8, 1), ("k", W.U8, 2)], ok_t), "duplicate metadata key")
    _bad(tmp_path, W.gguf_bytes([], ok_t)[:30], "past the end")
    _bad(tmp_path, W.gguf_bytes([("k", W.ARR, (W.ARR, []))], ok_t), "nested array")
    _bad(tmp_path, W.gguf_bytes([], [("", [32], 0, np.zeros(32, np.float32))]), "empty tensor name")
    _bad(tmp_path, W.gguf_bytes([], ok_t + ok_t), "duplicate tensor name")
    _bad(tmp_path, W.gguf_bytes([], [("w", [], 0, b"")]), "implausible n_dims 0")
    _bad(tmp_path, W.gguf_bytes([], [("w", [1] * 9, 0, np.zeros(1, np.float32))]), "implausible n_dims 9")
    _bad(tmp_path, W.gguf_bytes([], [("w", [0], 0, b"")]), "implausible dimension")
    _bad(tmp_path, W.gguf_bytes([], [("w", [1 << 31], 0, b"")]), "implausible dimension")
    _bad(tmp_path, W.gguf_bytes([], [("w", [48], 8, np.zeros(51, np.uint8))]), "not a multiple of the block size 32")
    _bad(tmp_path, W.gguf_bytes([], [("w", [128], 12, np.zeros(72, np.uint8))]), "super-block size 256")
    _bad(tmp_path, W.gguf_bytes([("general.alignment", W.U32, 24)], ok_t, alignment=32), "power of two")
    _bad(tmp_path, W.gguf_bytes([], [("w", [64], 0, np.zeros(64, np.float32))])[:-200], "outside the data section")
    # unknown value type in the metadata
    raw = W.gguf_bytes([("k", W.U8, 1)], ok_t)
    _bad(tmp_path, raw.replace(b"k" + struct.pack("<I", W.U8), b"k" + struct.pack("<I", 13)), "unsupported value type 13")
    # a string whose length runs past the end of the file
    _bad(tmp_path, struct.pack("<IIQQ", 0x46554747, 3, 0, 1) + struct.pack("<Q", 1 << 30) + b"abc" + b"\0" * 16, "runs past the end")
    with pytest.raises(GGUFError, match="cannot open"):
        GGUFReader(tmp_path / "missing.gguf")


def test_reader_keeps_tables_of_undecodable_types_inspectable(tmp_path):
    """A dtype the reader cannot size keeps data_bytes = 0; the table stays readable (neural/neuralgguf.pas:1196-1200)."""
    p = tmp_path / "bf16.gguf"
    W.write(p, [], [("w", [32], 30, np.zeros(64, np.uint8)), ("v", [32], 0, np.ones(32, np.float32))])
    r = GGUFReader(p)
    try:
        assert r.tensor_info(0)[1] == 30 and r.tensor_info(0)[4] == 0
        assert r.tensor_info(1)[4] == 128
    finally:
        r.close()


def test_llama_config_refusals_and_defaults(tmp_path):
    t = [("token_embd.weight", [32, 7], 0, np.zeros(224, np.float32))]
    p = tmp_path / "cfg.gguf"
    W.write(p, W.llama_meta("qwen2", 32, 64, 2, 4, 2, 128), t)
    r = GGUFReader(p)
    cfg, mp = r.llama_config()
    r.close()
    # qwen2 defaults: eps 1e-6, theta 10000, vocab from the embedding rows, tied head, head_dim = hidden / heads, q/k/v biases
    assert (cfg.vocab, cfg.tie_embeddings, cfg.head_dim, cfg.qkv_bias, mp) == (7, 1, 8, 1, 128)
    assert cfg.rms_eps == np.float32(1e-6) and cfg.rope_theta == np.float32(10000.0)
    W.write(p, W.llama_meta("llama", 32, 64, 2, 4, 2, 128), t)
    r = GGUFReader(p)
    cfg, _ = r.llama_config()
    r.close()
    assert cfg.rms_eps == np.float32(1e-5) and cfg.qkv_bias == 0
    for meta, match in (
            ([("general.architecture", W.STR, "gemma2")], "not supported"),
            (W.llama_meta("llama", 32, 64, 2, 4, 2, 128)[:-1], "context_length"),
            (W.llama_meta("llama", 30, 64, 2, 4, 2, 128), "not divisible"),
            (W.llama_meta("llama", 32, 64, 2, 4, 2, 128) + [("llama.rope.scaling.type", W.STR, "yarn")], "not supported"),
            (W.llama_meta("llama", 32, 64, 2, 4, 2, 128) + [("llama.rope.scaling.type", W.STR, "linear"),
                                                           ("llama.rope.scaling.factor", W.F32, 4.0)], "interpolation"),
            (W.llama_meta("qwen2", 32, 64, 2, 4, 2, 128) + [("qwen2.attention.sliding_window", W.U32, 4096)], "sliding-window")):
        W.write(p, meta, t)
        r = GGUFReader(p)
        with pytest.raises(GGUFError, match=match):
            r.llama_config()
        r.close()
    W.write(p, W.llama_meta("llama", 32, 64, 2, 4, 2, 128), [])
    r = GGUFReader(p)
    with pytest.raises(GGUFError, match="vocab size"):
        r.llama_config()
    r.close()
