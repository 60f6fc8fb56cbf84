"""Host-side mirror of the reference's device-backend interface for the decode
hot path, written over the C ABI of libcai_cuda.so.

The class and method names follow the reference so that tests read like its
own tests (file:line relative to the reference project root):

  CudaBackend              <- TEasyOpenCL / TNNet.EnableOpenCL   neural/neuralopencl.pas:72-164,
                                                                 neural/neuralchatengine.pas:1156-1157
  DotProductSharedKernel   <- TDotProductSharedKernel            neural/neuralopencl.pas:245-388
  FusedSDPA                <- TNNetFusedSDPA (incremental decode) tests/TestNeuralFusedSDPA.pas:226-236
  LlamaModel               <- BuildLlamaFromTensorReaderWithConfig neural/neuralpretrained.pas:16196-17473
  StreamingDecoder         <- TNNetStreamingDecoder              neural/neuraldecode.pas:1210-1333, 5552-5872
  generate_tokens_streamed <- greedy loop of GenerateFromIds     neural/neuralchatengine.pas:1466-1505

numpy arrays are the host buffers; nothing here computes on the CPU.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import CaiError, LlamaConfigC, SamplingC, TYPE_F16, TYPE_F32, TYPE_I8, TYPE_I8ROW, TYPE_Q4_0, TYPE_Q8_0  # noqa: F401


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p)


class DeviceBuffer:
    """A device allocation owned by a backend (the cl_mem of the OpenCL backend)."""

    def __init__(self, backend, nbytes):
        self.backend = backend
        self.nbytes = int(nbytes)
        p = C.c_void_p()
        backend._check(backend.lib.cai_dev_alloc(backend.ctx, self.nbytes, C.byref(p)))
        self.ptr = p

    def write(self, arr):
        arr = np.ascontiguousarray(arr)
        if arr.nbytes > self.nbytes:
            raise ValueError("host array larger than the device buffer")
        self.backend._check(self.backend.lib.cai_memcpy_h2d(self.backend.ctx, self.ptr, _ptr(arr), arr.nbytes))
        return self

    def read(self, dtype, count):
        out = np.empty(count, dtype=dtype)
        self.backend._check(self.backend.lib.cai_memcpy_d2h(self.backend.ctx, _ptr(out), self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr:
            self.backend.lib.cai_dev_free(self.backend.ctx, self.ptr)
            self.ptr = None


class CudaBackend:
    """One CUDA context on one GPU. Raises if the library or the GPU is missing."""

    def __init__(self, device=0):
        self.lib = _lib.load()
        ctx = C.c_void_p()
        st = self.lib.cai_cuda_init(int(device), C.byref(ctx))
        if st != 0:
            raise CaiError(st, "cai_cuda_init(device=%d) failed: no usable CUDA device" % device)
        self.ctx = ctx
        self.device = device

    def _check(self, status):
        if status != 0:
            buf = C.create_string_buffer(1024)
            self.lib.cai_cuda_last_error(self.ctx, buf, 1024)
            raise CaiError(status, buf.value.decode(errors="replace"))

    def close(self):
        if self.ctx:
            self.lib.cai_cuda_shutdown(self.ctx)
            self.ctx = None

    def device_info(self):
        sm = C.c_int()
        mem = C.c_int64()
        self._check(self.lib.cai_cuda_device_info(self.ctx, C.byref(sm), C.byref(mem)))
        return sm.value, mem.value

    def launch_count(self):
        n = C.c_int64()
        self._check(self.lib.cai_cuda_launch_count(self.ctx, C.byref(n)))
        return n.value

    def alloc(self, nbytes):
        return DeviceBuffer(self, nbytes)

    def to_device(self, arr):
        arr = np.ascontiguousarray(arr)
        return DeviceBuffer(self, max(arr.nbytes, 4)).write(arr)

    def sync(self):
        self._check(self.lib.cai_dev_sync(self.ctx))

    def quantize_int8_rows(self, w):
        """QuantizeInt8 per row on the device: returns (int8 codes [rows, cols], fp32 scales [rows])."""
        w = np.ascontiguousarray(w, dtype=np.float32)
        rows, cols = w.shape
        codes = np.empty((rows, cols), dtype=np.int8)
        scales = np.empty(rows, dtype=np.float32)
        self._check(self.lib.cai_quantize_int8_rows(self.ctx, _ptr(w), rows, cols, _ptr(codes), _ptr(scales)))
        return codes, scales

    def set_wait_limit_us(self, limit_us):
        """Longest device-side wait on another CTA or GPU before a kernel gives up and raises the error word."""
        self._check(self.lib.cai_cuda_set_wait_limit_us(self.ctx, int(limit_us)))

    def selftest_wait_timeout(self, which, limit_us):
        """Makes one bounded device-side wait run out on purpose; returns the status the library reports for it."""
        return int(self.lib.cai_selftest_wait_timeout(self.ctx, int(which), int(limit_us)))

    def timer_begin(self):
        self._check(self.lib.cai_timer_begin(self.ctx))

    def timer_end(self):
        ms = C.c_float()
        self._check(self.lib.cai_timer_end(self.ctx, C.byref(ms)))
        return ms.value

    def flush_l2(self):
        self._check(self.lib.cai_flush_l2(self.ctx))

    # -- codec hook --------------------------------------------------------
    def dequantize(self, ggml_type, blocks, rows, cols):
        blocks = np.ascontiguousarray(blocks)
        out = np.empty(rows * cols, dtype=np.float32)
        self._check(self.lib.cai_dequantize(self.ctx, ggml_type, _ptr(blocks), rows, cols, _ptr(out)))
        return out

    def gguf_decode(self, ggml_type, raw, n_elems):
        """DecodeGGMLSpan on the device: raw block bytes of any ggml type the reader decodes -> fp32."""
        raw = np.ascontiguousarray(raw)
        out = np.empty(n_elems, dtype=np.float32)
        self._check(self.lib.cai_gguf_decode(self.ctx, ggml_type, _ptr(raw), n_elems, _ptr(out)))
        return out

    # -- layer shims on device buffers --------------------------------------
    def rmsnorm(self, x, gain, eps):
        x = np.ascontiguousarray(x, dtype=np.float32)
        tokens, depth = x.shape
        dx, dg = self.to_device(x), self.to_device(np.ascontiguousarray(gain, dtype=np.float32))
        dy = self.alloc(x.nbytes)
        self._check(self.lib.cai_rmsnorm_dev(self.ctx, dx.ptr, dg.ptr, dy.ptr, tokens, depth, eps))
        out = dy.read(np.float32, x.size).reshape(x.shape)
        for b in (dx, dg, dy):
            b.free()
        return out

    def rope(self, x, head_dim, position_offset, theta_base):
        x = np.ascontiguousarray(x, dtype=np.float32)
        tokens, depth = x.shape
        dx = self.to_device(x)
        self._check(self.lib.cai_rope_dev(self.ctx, dx.ptr, tokens, depth, head_dim, position_offset, theta_base))
        out = dx.read(np.float32, x.size).reshape(x.shape)
        dx.free()
        return out

    def swiglu(self, x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        tokens, depth = x.shape
        half = depth // 2
        dx = self.to_device(x)
        dy = self.alloc(tokens * half * 4)
        self._check(self.lib.cai_swiglu_dev(self.ctx, dx.ptr, dy.ptr, tokens, half))
        out = dy.read(np.float32, tokens * half).reshape(tokens, half)
        dx.free()
        dy.free()
        return out

    def topk_gate(self, router_logits, top_k, renorm):
        x = np.ascontiguousarray(router_logits, dtype=np.float32)
        tokens, n_experts = x.shape
        dx = self.to_device(x)
        dids = self.alloc(tokens * top_k * 4)
        dg = self.alloc(tokens * top_k * 4)
        self._check(self.lib.cai_topk_gate_dev(self.ctx, dx.ptr, tokens, n_experts, top_k, int(bool(renorm)), dids.ptr, dg.ptr))
        ids = dids.read(np.int32, tokens * top_k).reshape(tokens, top_k)
        gates = dg.read(np.float32, tokens * top_k).reshape(tokens, top_k)
        for b in (dx, dids, dg):
            b.free()
        return ids, gates

    # -- multi-GPU -----------------------------------------------------------
    def comm_unique_id(self):
        buf = (C.c_ubyte * 128)()
        st = self.lib.cai_comm_unique_id(buf)
        if st != 0:
            raise CaiError(st, "ncclGetUniqueId failed")
        return bytes(buf)

    def comm_init(self, rank, world, unique_id):
        buf = (C.c_ubyte * 128).from_buffer_copy(unique_id)
        self._check(self.lib.cai_comm_init(self.ctx, rank, world, buf))


class DotProductSharedKernel:
    """Resident quantized linear layer: weights uploaded once, immutable.

    prepare_for_compute_quant <- PrepareForComputeInt8 (neuralopencl.pas:844-891)
    compute_quant             <- ComputeInt8 (:946-1056); x may be a host array
                                 (NewVBs = true) or a DeviceBuffer (pExternalVBs)
    finish_and_load_result    <- FinishAndLoadResult (:1058-1104)
    result_buffer             <- ResultBuffer property (:382-387)
    """

    def __init__(self, backend):
        self.backend = backend
        self.handle = None
        self.n = self.k = 0
        self._result = None
        self._result_batch = 0

    def prepare_for_compute_quant(self, ggml_type, blocks, num_as, size, bias=None):
        self.unprepare_for_compute()
        b = self.backend
        blocks = np.ascontiguousarray(blocks)
        h = C.c_void_p()
        bias_p = _ptr(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        b._check(b.lib.cai_linear_create(b.ctx, ggml_type, _ptr(blocks), num_as, size, bias_p, C.byref(h)))
        self.handle, self.n, self.k = h, num_as, size
        return 0

    def prepare_for_compute_int8(self, codes, scales, num_as, size, bias=None):
        """PrepareForComputeInt8 proper (neuralopencl.pas:844-891): the reference's int8 container as it is,
        codes[num_as * size] int8 and one fp32 scale per row (GetInt8QuantData)."""
        self.unprepare_for_compute()
        b = self.backend
        codes = np.ascontiguousarray(codes, dtype=np.int8).reshape(-1)
        scales = np.ascontiguousarray(scales, dtype=np.float32).reshape(-1)
        h = C.c_void_p()
        bias_p = _ptr(np.ascontiguousarray(bias, dtype=np.float32)) if bias is not None else None
        b._check(b.lib.cai_linear_create_int8(b.ctx, _ptr(codes), _ptr(scales), num_as, size, bias_p, C.byref(h)))
        self.handle, self.n, self.k = h, num_as, size
        return 0

    @property
    def quant_ready(self):
        return self.handle is not None

    def weight_bytes(self):
        n = C.c_int64()
        self.backend._check(self.backend.lib.cai_linear_weight_bytes(self.handle, C.byref(n)))
        return n.value

    def set_path(self, path):
        """0 = automatic, 1 = CUDA-core GEMV, 2 = tensor-core GEMM (fails on calls that path does not cover)."""
        self.backend._check(self.backend.lib.cai_linear_set_path(self.handle, int(path)))

    def dequantize_weights(self):
        out = np.empty(self.n * self.k, dtype=np.float32)
        self.backend._check(self.backend.lib.cai_linear_dequantize(self.handle, _ptr(out)))
        return out.reshape(self.n, self.k)

    def compute_quant(self, x, act=0, batch=None):
        """Enqueues y = act(W x + bias). Host input -> result fetched by
        finish_and_load_result; DeviceBuffer input -> result stays in result_buffer."""
        b = self.backend
        if isinstance(x, DeviceBuffer):
            if batch is None:
                raise ValueError("batch is required for a device-resident operand")
            self._ensure_result(batch)
            b._check(b.lib.cai_linear_forward_dev(self.handle, x.ptr, batch, self._result.ptr, act))
            self._host_result = None
        else:
            x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.k)
            batch = x.shape[0]
            y = np.empty((batch, self.n), dtype=np.float32)
            b._check(b.lib.cai_linear_forward(self.handle, _ptr(x), batch, _ptr(y), act))
            self._host_result = y
        self._result_batch = batch

    def _ensure_result(self, batch):
        if self._result is None or self._result.nbytes < batch * self.n * 4:
            if self._result is not None:
                self._result.free()
            self._result = self.backend.alloc(batch * self.n * 4)

    @property
    def result_buffer(self):
        return self._result

    def finish_and_load_result(self):
        if getattr(self, "_host_result", None) is not None:
            return self._host_result
        return self._result.read(np.float32, self._result_batch * self.n).reshape(self._result_batch, self.n)

    def unprepare_for_compute(self):
        if self.handle is not None:
            self.backend.lib.cai_linear_destroy(self.handle)
            self.handle = None
        if self._result is not None:
            self._result.free()
            self._result = None


class FusedSDPA:
    """Fused GQA attention in incremental-decode mode (one token per call)."""

    def __init__(self, backend, q_heads, kv_heads, head_dim):
        self.backend, self.q_heads, self.kv_heads, self.head_dim = backend, q_heads, kv_heads, head_dim
        self.handle = None

    def begin_incremental_decode(self, max_context):
        b = self.backend
        h = C.c_void_p()
        b._check(b.lib.cai_sdpa_create(b.ctx, self.q_heads, self.kv_heads, self.head_dim, max_context, C.byref(h)))
        self.handle = h

    def end_incremental_decode(self):
        if self.handle is not None:
            self.backend.lib.cai_sdpa_destroy(self.handle)
            self.handle = None

    def reset_cache(self):
        self.backend._check(self.backend.lib.cai_sdpa_reset(self.handle))

    def truncate_cache(self, n):
        self.backend._check(self.backend.lib.cai_sdpa_truncate(self.handle, n))

    @property
    def cache_length(self):
        n = C.c_int()
        self.backend._check(self.backend.lib.cai_sdpa_cache_len(self.handle, C.byref(n)))
        return n.value

    def set_window(self, window):
        self.backend._check(self.backend.lib.cai_sdpa_set_window(self.handle, int(window)))

    def enable_eviction(self, sink_tokens, recent_window):
        self.backend._check(self.backend.lib.cai_sdpa_enable_eviction(self.handle, int(sink_tokens), int(recent_window)))

    def compute_cached_token(self, qkv_row):
        """Input row [allQ | allK | allV]; returns q_heads*head_dim outputs."""
        b = self.backend
        row = np.ascontiguousarray(qkv_row, dtype=np.float32).reshape(-1)
        din = b.to_device(row)
        dout = b.alloc(self.q_heads * self.head_dim * 4)
        try:
            b._check(b.lib.cai_sdpa_step_dev(self.handle, din.ptr, dout.ptr))
            return dout.read(np.float32, self.q_heads * self.head_dim)
        finally:
            din.free()
            dout.free()


class MoEExpertBank:
    """TNNetMoEExpertBankGateUp + TNNetMoEExpertBankDown of one layer, resident on the device: per expert the up, gate and
    down matrices; gate_up() emits the selected experts' SwiGLU hidden packed by slot, down() the gate-weighted sum."""

    def __init__(self, backend, n_experts, hidden, expert_width, ggml_type=TYPE_F32):
        self.backend, self.n_experts, self.hidden, self.width = backend, n_experts, hidden, expert_width
        h = C.c_void_p()
        backend._check(backend.lib.cai_moe_bank_create(backend.ctx, n_experts, hidden, expert_width, ggml_type, C.byref(h)))
        self.handle = h

    def upload(self, expert, which, blocks):
        """which: 'up' | 'gate' (rows [expert_width, hidden]) | 'down' (rows [hidden, expert_width])."""
        blocks = np.ascontiguousarray(blocks)
        self.backend._check(self.backend.lib.cai_moe_bank_upload(self.handle, expert, {"up": 0, "gate": 1, "down": 2}[which], _ptr(blocks)))

    def finalize(self):
        self.backend._check(self.backend.lib.cai_moe_bank_finalize(self.handle))

    def gate_up(self, x_dev, slot_expert_dev, tokens, top_k, hidden_out_dev):
        self.backend._check(self.backend.lib.cai_moe_gate_up_dev(self.handle, x_dev.ptr, slot_expert_dev.ptr, tokens, top_k, hidden_out_dev.ptr))

    def down(self, hidden_dev, slot_expert_dev, slot_gate_dev, tokens, top_k, out_dev):
        self.backend._check(self.backend.lib.cai_moe_down_dev(self.handle, hidden_dev.ptr, slot_expert_dev.ptr, slot_gate_dev.ptr,
                                                              tokens, top_k, out_dev.ptr))

    def close(self):
        if self.handle:
            self.backend.lib.cai_moe_bank_destroy(self.handle)
            self.handle = None


class GGUFError(CaiError):
    """A file the reader refused (the reference's EGGUFError)."""


class GGUFReader:
    """TNNetGGUFReader: header, metadata and tensor table of one GGUF file, parsed by the library (no GPU needed to
    open a file or read its tables; decoding a tensor runs on the GPU of the backend passed to load_tensor)."""

    def __init__(self, path):
        self.lib = _lib.load()
        h = C.c_void_p()
        err = C.create_string_buffer(512)
        st = self.lib.cai_gguf_open(str(path).encode(), C.byref(h), err, 512)
        if st != _lib.CAI_OK:
            raise GGUFError(st, err.value.decode(errors="replace"))
        self.handle = h
        ver, al, nm, nt, ds = C.c_int(), C.c_int(), C.c_int64(), C.c_int64(), C.c_int64()
        self._check(self.lib.cai_gguf_info(h, C.byref(ver), C.byref(al), C.byref(nm), C.byref(nt), C.byref(ds)))
        self.version, self.alignment, self.data_start = ver.value, al.value, ds.value
        self.meta_count, self.tensor_count = nm.value, nt.value

    def _check(self, st):
        if st != _lib.CAI_OK:
            buf = C.create_string_buffer(512)
            self.lib.cai_gguf_last_error(self.handle, buf, 512)
            raise GGUFError(st, buf.value.decode(errors="replace"))

    def meta_keys(self):
        out = []
        buf, vt = C.create_string_buffer(512), C.c_int()
        for i in range(self.meta_count):
            self._check(self.lib.cai_gguf_meta_key(self.handle, i, buf, 512, C.byref(vt)))
            out.append((buf.value.decode(), vt.value))
        return out

    def get_meta_int(self, key, default):
        v, found = C.c_int64(), C.c_int()
        self._check(self.lib.cai_gguf_meta_int(self.handle, key.encode(), C.byref(v), C.byref(found)))
        return v.value if found.value else default

    def get_meta_float(self, key, default):
        v, found = C.c_double(), C.c_int()
        self._check(self.lib.cai_gguf_meta_float(self.handle, key.encode(), C.byref(v), C.byref(found)))
        return v.value if found.value else default

    def get_meta_string(self, key, default):
        buf, found = C.create_string_buffer(4096), C.c_int()
        self._check(self.lib.cai_gguf_meta_string(self.handle, key.encode(), buf, 4096, C.byref(found)))
        return buf.value.decode(errors="replace") if found.value else default

    def get_meta_array_count(self, key):
        v = C.c_int64()
        self._check(self.lib.cai_gguf_meta_array_count(self.handle, key.encode(), C.byref(v)))
        return v.value

    def tensor_info(self, index):
        """(name, ggml type, shape with the contiguous axis last, data offset within the data section, bytes)."""
        name, ty, nd = C.create_string_buffer(512), C.c_int(), C.c_int()
        shape = (C.c_int64 * 8)()
        beg, nbytes = C.c_int64(), C.c_int64()
        self._check(self.lib.cai_gguf_tensor_info(self.handle, index, name, 512, C.byref(ty), C.byref(nd), shape,
                                                  C.byref(beg), C.byref(nbytes)))
        return name.value.decode(), ty.value, [int(shape[i]) for i in range(nd.value)], beg.value, nbytes.value

    def find_tensor(self, name):
        v = C.c_int64()
        self._check(self.lib.cai_gguf_find_tensor(self.handle, name.encode(), C.byref(v)))
        return v.value

    def has_tensor(self, name):
        return self.find_tensor(name) >= 0

    def read_raw(self, index):
        nbytes = self.tensor_info(index)[4]
        buf = np.empty(max(nbytes, 1), dtype=np.uint8)
        self._check(self.lib.cai_gguf_read_raw(self.handle, index, _ptr(buf), nbytes))
        return buf[:nbytes]

    def load_tensor(self, backend, name):
        """LoadTensorFlat: the tensor decoded to fp32 on the backend's GPU, in its served shape."""
        idx = self.find_tensor(name)
        if idx < 0:
            raise KeyError(name)
        shape = self.tensor_info(idx)[2]
        n = int(np.prod(shape))
        out = np.empty(n, dtype=np.float32)
        backend._check(self.lib.cai_gguf_load_tensor(backend.ctx, self.handle, idx, _ptr(out), n))
        return out.reshape(shape)

    def llama_config(self):
        """(LlamaConfigC, context_length) from the metadata, as BuildFromGGUFEx derives them."""
        cfg, mp = LlamaConfigC(), C.c_int64()
        self._check(self.lib.cai_gguf_llama_config(self.handle, C.byref(cfg), C.byref(mp)))
        return cfg, mp.value

    def close(self):
        if self.handle:
            self.lib.cai_gguf_close(self.handle)
            self.handle = None


def make_config(hidden, inter, layers, heads, kv_heads, head_dim, vocab, rms_eps=1e-5, rope_theta=10000.0,
                tie_embeddings=False, qkv_bias=False, qk_norm=False, n_experts=0, top_k=0, norm_topk=False, moe_inter=0):
    return LlamaConfigC(hidden, inter, layers, heads, kv_heads, head_dim, vocab, rms_eps, rope_theta,
                        int(tie_embeddings), int(qkv_bias), int(qk_norm), n_experts, top_k, int(norm_topk), moe_inter)


class LlamaModel:
    """The Llama-family graph resident on one GPU (or one tensor-parallel shard)."""

    def __init__(self, backend, cfg, tp_rank=0, tp_size=1, ep_rank=0, ep_size=1):
        """tp_*: tensor-parallel shard of a dense model; ep_*: expert-parallel share of a mixture-of-experts model
        (dense parts replicated, sessions hold this rank's own sequences)."""
        self.backend, self.cfg = backend, cfg
        h = C.c_void_p()
        if ep_size > 1:
            backend._check(backend.lib.cai_model_create_ep(backend.ctx, C.byref(cfg), ep_rank, ep_size, C.byref(h)))
        else:
            backend._check(backend.lib.cai_model_create(backend.ctx, C.byref(cfg), tp_rank, tp_size, C.byref(h)))
        self.handle = h

    @classmethod
    def from_gguf(cls, backend, path, tp_rank=0, tp_size=1, quantize_int8=False):
        """BuildFromGGUFEx: the whole file parsed, decoded and uploaded by the library. Returns the finalized model;
        model.max_positions carries the file's context_length."""
        self = cls.__new__(cls)
        self.backend = backend
        h, cfg, mp = C.c_void_p(), LlamaConfigC(), C.c_int64()
        backend._check(backend.lib.cai_model_load_gguf(backend.ctx, str(path).encode(), tp_rank, tp_size, int(bool(quantize_int8)),
                                                       C.byref(h), C.byref(cfg), C.byref(mp)))
        self.handle, self.cfg, self.max_positions = h, cfg, mp.value
        return self

    def upload_tensor(self, hf_name, ggml_type, data, rows, cols, interleave_head_dim=0):
        data = np.ascontiguousarray(data)
        self.backend._check(self.backend.lib.cai_model_upload_tensor(
            self.handle, hf_name.encode(), ggml_type, _ptr(data), rows, cols, interleave_head_dim))

    def upload_hf_tensors(self, tensors, interleave=True):
        """fp32 HF-layout tensors {name: array}; q/k rows get the importer's interleave."""
        hd = self.cfg.head_dim
        for name, w in tensors.items():
            w = np.ascontiguousarray(w, dtype=np.float32)
            rows, cols = (w.shape if w.ndim == 2 else (1, w.size))
            perm = hd if (interleave and any(s in name for s in ("q_proj", "k_proj", "q_norm", "k_norm"))) else 0
            self.upload_tensor(name, TYPE_F32, w, rows, cols, perm)

    def set_int8_weights(self, on=True):
        """The importer's pQuantizeInt8: F32 matrices uploaded afterwards are stored as int8 rows."""
        self.backend._check(self.backend.lib.cai_model_set_int8_weights(self.handle, int(bool(on))))

    def init_synthetic(self, ggml_type, seed, std=0.02):
        self.backend._check(self.backend.lib.cai_model_init_synthetic(self.handle, ggml_type, seed, std))

    def read_tensor(self, hf_name, max_bytes):
        buf = np.empty(max_bytes, dtype=np.uint8)
        ty, rows, cols = C.c_int(), C.c_int64(), C.c_int64()
        self.backend._check(self.backend.lib.cai_model_read_tensor(
            self.handle, hf_name.encode(), _ptr(buf), max_bytes, C.byref(ty), C.byref(rows), C.byref(cols)))
        return buf, ty.value, rows.value, cols.value

    def finalize(self):
        self.backend._check(self.backend.lib.cai_model_finalize(self.handle))

    def step_weight_bytes(self):
        n = C.c_int64()
        self.backend._check(self.backend.lib.cai_model_step_weight_bytes(self.handle, C.byref(n)))
        return n.value

    def close(self):
        if self.handle:
            self.backend.lib.cai_model_destroy(self.handle)
            self.handle = None


class StreamingDecoder:
    """KV-cached decode session over `batch` independent sequences."""

    def __init__(self, model, max_context, batch=1, kv_type=TYPE_F32):
        """kv_type: TYPE_F32, or TYPE_I8 for the reference's int8 cache (BeginIncrementalDecode(MaxCtx, Int8KV))."""
        self.model, self.backend, self.batch = model, model.backend, batch
        self.vocab = model.cfg.vocab
        h = C.c_void_p()
        self.backend._check(self.backend.lib.cai_session_create(model.handle, max_context, batch, kv_type, C.byref(h)))
        self.handle = h
        self._logits = np.empty((batch, self.vocab), dtype=np.float32)
        self._argmax = np.empty(batch, dtype=np.int32)

    def reset(self, seq=-1):
        self.backend._check(self.backend.lib.cai_session_reset(self.handle, seq))

    def truncate_to(self, n, seq=0):
        self.backend._check(self.backend.lib.cai_session_truncate(self.handle, seq, n))

    def cache_length(self, seq=0):
        n = C.c_int()
        self.backend._check(self.backend.lib.cai_session_cache_len(self.handle, seq, C.byref(n)))
        return n.value

    def enable_eviction(self, sink_tokens, recent_window):
        """StreamingLLM: keep the first sink_tokens rows and the most recent recent_window rows (0, 0 = off)."""
        self.backend._check(self.backend.lib.cai_session_enable_eviction(self.handle, int(sink_tokens), int(recent_window)))

    def set_window(self, window):
        """Sliding-window attention: only the most recent `window` rows (0 = the whole cache)."""
        self.backend._check(self.backend.lib.cai_session_set_window(self.handle, int(window)))

    def fill_for_benchmark(self, n_rows):
        """Zeroes the caches and declares n_rows cached positions per sequence (timing aid; the rows are not the model's)."""
        self.backend._check(self.backend.lib.cai_session_fill_for_benchmark(self.handle, int(n_rows)))

    def step_forward(self, tokens, abs_pos=None, want_logits=True):
        """One width-1 forward per sequence; returns (logits [batch, vocab] or None, argmax [batch])."""
        tok = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch))
        pos = None if abs_pos is None else np.ascontiguousarray(np.asarray(abs_pos, dtype=np.int32).reshape(self.batch))
        self.backend._check(self.backend.lib.cai_session_step(
            self.handle, _ptr(tok), _ptr(pos) if pos is not None else None,
            _ptr(self._logits) if want_logits else None, _ptr(self._argmax)))
        return (self._logits if want_logits else None), self._argmax

    def output(self):
        return self._logits

    def decode_greedy(self, tokens, n_steps):
        tok = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch))
        out = np.empty((n_steps, self.batch), dtype=np.int32)
        self.backend._check(self.backend.lib.cai_session_decode_greedy(self.handle, _ptr(tok), n_steps, _ptr(out)))
        return out

    def step_topk(self, tokens, k, temperature=1.0, abs_pos=None):
        """One step; returns the sampler's candidate window per sequence: (ids [batch, k], probabilities [batch, k])."""
        tok = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch))
        pos = None if abs_pos is None else np.ascontiguousarray(np.asarray(abs_pos, dtype=np.int32).reshape(self.batch))
        ids = np.empty((self.batch, k), dtype=np.int32)
        probs = np.empty((self.batch, k), dtype=np.float32)
        self.backend._check(self.backend.lib.cai_session_step_topk(self.handle, _ptr(tok), _ptr(pos) if pos is not None else None, k,
                                                                  float(temperature), _ptr(ids), _ptr(probs)))
        return ids, probs

    def decode_sampled(self, tokens, n_steps, temperature=1.0, top_k=40, top_p=0.0, seed=0, uniforms=None):
        """The sampled generation loop on the device; uniforms [n_steps, batch] optional (else the keyed generator)."""
        tok = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch))
        opt = SamplingC(float(temperature), int(top_k), float(top_p), int(seed))
        out = np.empty((n_steps, self.batch), dtype=np.int32)
        u = None if uniforms is None else np.ascontiguousarray(np.asarray(uniforms, dtype=np.float32).reshape(n_steps, self.batch))
        self.backend._check(self.backend.lib.cai_session_decode_sampled(self.handle, _ptr(tok), n_steps, C.byref(opt),
                                                                       _ptr(u) if u is not None else None, _ptr(out)))
        return out

    def prefill(self, tokens):
        tok = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch, -1))
        self.backend._check(self.backend.lib.cai_session_prefill(self.handle, _ptr(tok), tok.shape[1]))

    def profile(self, tokens, n_steps):
        """Eager steps with one CUDA event per launch; returns {family: (ms, launches)}."""
        tok = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch))
        ms = (C.c_float * 4)()
        n = (C.c_int64 * 4)()
        self.backend._check(self.backend.lib.cai_session_profile(self.handle, _ptr(tok), n_steps, ms, n))
        return {name: (ms[i], n[i]) for i, name in enumerate(("linear", "attention", "other", "comm"))}

    def snapshot(self):
        self.backend._check(self.backend.lib.cai_session_snapshot(self.handle))

    def restore_snapshot(self):
        self.backend._check(self.backend.lib.cai_session_restore(self.handle))

    def read_kv_row(self, layer, pos, kv_head=0, seq=0, int8=False):
        """One cached row: (k, v) floats for the fp32 cache; (k_codes, v_codes, k_scale, v_scale) for the int8 cache."""
        hd = self.model.cfg.head_dim
        k = np.empty(hd, dtype=np.float32)
        v = np.empty(hd, dtype=np.float32)
        kc = np.empty(hd, dtype=np.int8)
        vc = np.empty(hd, dtype=np.int8)
        sc = np.empty(2, dtype=np.float32)
        self.backend._check(self.backend.lib.cai_session_read_kv_row(self.handle, layer, seq, kv_head, pos, _ptr(k), _ptr(v),
                                                                    _ptr(kc), _ptr(vc), _ptr(sc)))
        return (kc, vc, float(sc[0]), float(sc[1])) if int8 else (k, v)

    def step_trace(self, tokens, cap=4096):
        """One step with the phase trace on; returns (ns since the kernel's first stamp, family per stamp)."""
        tok = np.ascontiguousarray(np.asarray(tokens, dtype=np.int32).reshape(self.batch))
        ns = (C.c_int64 * cap)()
        fam = (C.c_int32 * cap)()
        n = C.c_int()
        self.backend._check(self.backend.lib.cai_session_step_trace(self.handle, _ptr(tok), ns, fam, cap, C.byref(n)))
        return np.asarray(ns[:n.value], dtype=np.int64), np.asarray(fam[:n.value], dtype=np.int32)

    @property
    def uses_step_kernel(self):
        """True when every step of this session is one persistent kernel (False: one kernel per operator)."""
        f = C.c_int()
        self.backend._check(self.backend.lib.cai_session_uses_step_kernel(self.handle, C.byref(f)))
        return bool(f.value)

    def last_kv_bytes(self):
        n = C.c_int64()
        self.backend._check(self.backend.lib.cai_session_last_kv_bytes(self.handle, C.byref(n)))
        return n.value

    def close(self):
        if self.handle:
            self.backend.lib.cai_session_destroy(self.handle)
            self.handle = None


def generate_tokens_streamed(session, prompt, n_new, want_logits=False):
    """The reference's greedy schedule for ONE sequence per batch row: tokens
    0..P-2 are fed one at a time, token P-1 at position P-1 yields the first new
    token. prompt: [batch, P]. Returns (tokens [n_new, batch], logits rows or None)."""
    prompt = np.asarray(prompt, dtype=np.int32).reshape(session.batch, -1)
    if prompt.shape[1] > 1:
        session.prefill(prompt[:, :-1])
    tok = prompt[:, -1].copy()
    out, rows = [], []
    for _ in range(n_new):
        logits, amax = session.step_forward(tok, want_logits=want_logits)
        tok = amax.copy()
        out.append(tok)
        if want_logits:
            rows.append(logits.copy())
    return np.stack(out), (np.stack(rows) if want_logits else None)
