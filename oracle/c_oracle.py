"""ctypes wrapper of oracle/libcai_oracle.so, the C (AVX2 + OpenMP) restatement of the
reference's CPU decode path. TEST INFRASTRUCTURE and timed CPU baseline only.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcai_oracle.so")

KINDS = {"embed": 0, "head": 1, "final_norm": 2, "attn_norm": 3, "ffn_norm": 4, "q": 5, "k": 6, "v": 7, "o": 8,
         "up": 9, "gate": 10, "down": 11, "bq": 12, "bk": 13, "bv": 14}


class CoConfig(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32),
                ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("vocab", C.c_int32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float), ("tie_embeddings", C.c_int32), ("qkv_bias", C.c_int32)]


def build():
    src = os.path.join(HERE, "cai_oracle.c")
    if not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE], check=True, capture_output=True)
    return LIB_PATH


_lib = None


def load():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        lib = C.CDLL(LIB_PATH)
        lib.co_gemv.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib.co_gemv.restype = None
        lib.co_dequantize.argtypes = [C.c_int, C.c_void_p, C.c_int64, C.c_void_p]
        lib.co_dequantize.restype = None
        lib.co_model_create.argtypes = [C.POINTER(CoConfig)]
        lib.co_model_create.restype = C.c_void_p
        lib.co_model_destroy.argtypes = [C.c_void_p]
        lib.co_model_set_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p]
        lib.co_session_create.argtypes = [C.c_void_p, C.c_int]
        lib.co_session_create.restype = C.c_void_p
        lib.co_session_destroy.argtypes = [C.c_void_p]
        lib.co_session_reset.argtypes = [C.c_void_p]
        lib.co_session_assume_len.argtypes = [C.c_void_p, C.c_int]
        lib.co_session_step.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.co_num_threads.restype = C.c_int
        lib.co_set_num_threads.argtypes = [C.c_int]
        _lib = lib
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def gemv(ggml_type, blocks, n, k, x, bias=None):
    lib = load()
    blocks = np.ascontiguousarray(blocks)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    y = np.empty((x.shape[0], n), dtype=np.float32)
    b = np.ascontiguousarray(bias, dtype=np.float32) if bias is not None else None
    lib.co_gemv(ggml_type, _p(blocks), n, k, _p(x), x.shape[0], _p(b) if b is not None else None, _p(y))
    return y


def dequantize(ggml_type, blocks, n_elems):
    lib = load()
    blocks = np.ascontiguousarray(blocks)
    out = np.empty(n_elems, dtype=np.float32)
    lib.co_dequantize(ggml_type, _p(blocks), n_elems, _p(out))
    return out


class CModel:
    """Dense Llama-family model over GGUF-row tensors in the in-net row order.
    Keeps the numpy buffers alive (the C side references them)."""

    def __init__(self, hidden, inter, layers, heads, kv_heads, head_dim, vocab, rms_eps, rope_theta,
                 tie_embeddings=False, qkv_bias=False):
        self.lib = load()
        self.cfg = CoConfig(hidden, inter, layers, heads, kv_heads, head_dim, vocab, rms_eps, rope_theta,
                            int(tie_embeddings), int(qkv_bias))
        self.handle = self.lib.co_model_create(C.byref(self.cfg))
        self.keep = []

    def set_tensor(self, kind, layer, ggml_type, data):
        data = np.ascontiguousarray(data)
        self.keep.append(data)
        if self.lib.co_model_set_tensor(self.handle, KINDS[kind], layer, ggml_type, _p(data)) != 0:
            raise ValueError("bad tensor %s layer %d" % (kind, layer))

    def close(self):
        if self.handle:
            self.lib.co_model_destroy(self.handle)
            self.handle = None


class CSession:
    def __init__(self, model, max_ctx):
        self.model = model
        self.lib = model.lib
        self.handle = self.lib.co_session_create(model.handle, max_ctx)
        self.vocab = model.cfg.vocab

    def step(self, token, pos, want_logits=True):
        out = np.empty(self.vocab, dtype=np.float32) if want_logits else None
        if self.lib.co_session_step(self.handle, int(token), int(pos), _p(out) if want_logits else None) != 0:
            raise ValueError("step rejected (context full or bad token)")
        return out

    def assume_len(self, n):
        self.lib.co_session_assume_len(self.handle, n)

    def reset(self):
        self.lib.co_session_reset(self.handle)

    def close(self):
        if self.handle:
            self.lib.co_session_destroy(self.handle)
            self.handle = None


def num_threads():
    return load().co_num_threads()


def set_num_threads(n):
    load().co_set_num_threads(n)
