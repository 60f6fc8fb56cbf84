"""ctypes binding of libcai_cuda.so (the declarations of include/cai_cuda.h).

There is no CPU fallback: if the library is missing or a call fails, an
exception is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# CAI_CUDA_CHECKED=1 binds the checked build (same entry points; every launch synchronized and looked at, indices from
# device-side state that the ordinary build clamps silently reported as errors): `python -m neural_api_b200.build --checked`
CHECKED = os.environ.get("CAI_CUDA_CHECKED", "") not in ("", "0")
LIB_PATH = os.path.join(HERE, "libcai_cuda_checked.so" if CHECKED else "libcai_cuda.so")

CAI_OK = 0
TYPE_F32, TYPE_F16, TYPE_Q4_0, TYPE_Q8_0 = 0, 1, 2, 8
TYPE_Q4_1, TYPE_Q5_0, TYPE_Q5_1 = 3, 6, 7                                  # load-time formats: decoded to fp32 on arrival
TYPE_Q2_K, TYPE_Q3_K, TYPE_Q4_K, TYPE_Q5_K, TYPE_Q6_K = 10, 11, 12, 13, 14
TYPE_I8 = 24              # KV cache only: int8 codes + one fp32 scale per row
TYPE_I8ROW = 124          # the reference's int8 weights: int8 codes [N][K] + one fp32 scale per output row
ACT_NONE, ACT_RELU, ACT_SIGMOID, ACT_TANH = 0, 1, 2, 3
STATUS_NAMES = {0: "CAI_OK", 1: "CAI_ERR_INVALID", 2: "CAI_ERR_CUDA", 3: "CAI_ERR_OOM",
                4: "CAI_ERR_STATE", 5: "CAI_ERR_UNSUPPORTED", 6: "CAI_ERR_COMM"}


class CaiError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("%s: %s" % (STATUS_NAMES.get(status, status), message))
        self.status = status
        self.message = message


class SamplingC(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_k", C.c_int32), ("top_p", C.c_float), ("seed", C.c_uint64)]


class LlamaConfigC(C.Structure):
    _fields_ = [("hidden", C.c_int32), ("inter", C.c_int32), ("layers", C.c_int32), ("heads", C.c_int32),
                ("kv_heads", C.c_int32), ("head_dim", C.c_int32), ("vocab", C.c_int32),
                ("rms_eps", C.c_float), ("rope_theta", C.c_float),
                ("tie_embeddings", C.c_int32), ("qkv_bias", C.c_int32), ("qk_norm", C.c_int32),
                ("n_experts", C.c_int32), ("top_k", C.c_int32), ("norm_topk", C.c_int32), ("moe_inter", C.c_int32)]


_P = C.c_void_p
_I = C.c_int
_I64 = C.c_int64
_PP = C.POINTER(C.c_void_p)

# name -> argtypes (restype is always int). Every symbol include/cai_cuda.h declares.
SIGNATURES = {
    "cai_cuda_init": [_I, _PP],
    "cai_cuda_shutdown": [_P],
    "cai_cuda_last_error": [_P, C.c_char_p, _I],
    "cai_cuda_device_info": [_P, C.POINTER(_I), C.POINTER(_I64)],
    "cai_cuda_launch_count": [_P, C.POINTER(_I64)],
    "cai_cuda_is_checked_build": [],
    "cai_cuda_set_wait_limit_us": [_P, C.c_uint],
    "cai_selftest_wait_timeout": [_P, _I, C.c_uint],
    "cai_dev_alloc": [_P, _I64, _PP],
    "cai_dev_free": [_P, _P],
    "cai_memcpy_h2d": [_P, _P, _P, _I64],
    "cai_memcpy_d2h": [_P, _P, _P, _I64],
    "cai_dev_sync": [_P],
    "cai_timer_begin": [_P],
    "cai_timer_end": [_P, C.POINTER(C.c_float)],
    "cai_flush_l2": [_P],
    "cai_dequantize": [_P, _I, _P, _I64, _I64, _P],
    "cai_linear_create": [_P, _I, _P, _I64, _I64, _P, _PP],
    "cai_linear_create_int8": [_P, _P, _P, _I64, _I64, _P, _PP],
    "cai_quantize_int8_rows": [_P, _P, _I64, _I64, _P, _P],
    "cai_linear_destroy": [_P],
    "cai_linear_forward": [_P, _P, _I, _P, _I],
    "cai_linear_forward_dev": [_P, _P, _I, _P, _I],
    "cai_linear_forward_many": [C.POINTER(_P), _I, _P, _I, _P, _I],
    "cai_linear_weight_bytes": [_P, C.POINTER(_I64)],
    "cai_linear_dequantize": [_P, _P],
    "cai_linear_set_path": [_P, _I],
    "cai_rmsnorm_dev": [_P, _P, _P, _P, _I, _I, C.c_float],
    "cai_rope_dev": [_P, _P, _I, _I, _I, _I, C.c_float],
    "cai_swiglu_dev": [_P, _P, _P, _I, _I],
    "cai_topk_gate_dev": [_P, _P, _I, _I, _I, _I, _P, _P],
    "cai_sdpa_create": [_P, _I, _I, _I, _I, _PP],
    "cai_sdpa_destroy": [_P],
    "cai_sdpa_reset": [_P],
    "cai_sdpa_truncate": [_P, _I],
    "cai_sdpa_cache_len": [_P, C.POINTER(_I)],
    "cai_sdpa_set_window": [_P, _I],
    "cai_sdpa_enable_eviction": [_P, _I, _I],
    "cai_sdpa_step_dev": [_P, _P, _P],
    "cai_sdpa_step_noalloc": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P],
    "cai_model_create": [_P, C.POINTER(LlamaConfigC), _I, _I, _PP],
    "cai_model_create_ep": [_P, C.POINTER(LlamaConfigC), _I, _I, _PP],
    "cai_model_destroy": [_P],
    "cai_model_upload_tensor": [_P, C.c_char_p, _I, _P, _I64, _I64, _I],
    "cai_moe_bank_create": [_P, _I, _I, _I, _I, _PP],
    "cai_moe_bank_destroy": [_P],
    "cai_moe_bank_upload": [_P, _I, _I, _P],
    "cai_moe_bank_finalize": [_P],
    "cai_moe_gate_up_dev": [_P, _P, _P, _I, _I, _P],
    "cai_moe_down_dev": [_P, _P, _P, _P, _I, _I, _P],
    "cai_gguf_open": [C.c_char_p, _PP, C.c_char_p, _I],
    "cai_gguf_close": [_P],
    "cai_gguf_last_error": [_P, C.c_char_p, _I],
    "cai_gguf_info": [_P, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I64), C.POINTER(_I64), C.POINTER(_I64)],
    "cai_gguf_meta_key": [_P, _I64, C.c_char_p, _I, C.POINTER(_I)],
    "cai_gguf_meta_int": [_P, C.c_char_p, C.POINTER(_I64), C.POINTER(_I)],
    "cai_gguf_meta_float": [_P, C.c_char_p, C.POINTER(C.c_double), C.POINTER(_I)],
    "cai_gguf_meta_string": [_P, C.c_char_p, C.c_char_p, _I, C.POINTER(_I)],
    "cai_gguf_meta_array_count": [_P, C.c_char_p, C.POINTER(_I64)],
    "cai_gguf_tensor_info": [_P, _I64, C.c_char_p, _I, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I64), C.POINTER(_I64),
                             C.POINTER(_I64)],
    "cai_gguf_find_tensor": [_P, C.c_char_p, C.POINTER(_I64)],
    "cai_gguf_read_raw": [_P, _I64, _P, _I64],
    "cai_gguf_decode": [_P, _I, _P, _I64, _P],
    "cai_gguf_load_tensor": [_P, _P, _I64, _P, _I64],
    "cai_gguf_llama_config": [_P, C.POINTER(LlamaConfigC), C.POINTER(_I64)],
    "cai_model_load_gguf": [_P, C.c_char_p, _I, _I, _I, _PP, C.POINTER(LlamaConfigC), C.POINTER(_I64)],
    "cai_model_set_int8_weights": [_P, _I],
    "cai_model_init_synthetic": [_P, _I, C.c_uint64, C.c_float],
    "cai_model_read_tensor": [_P, C.c_char_p, _P, _I64, C.POINTER(_I), C.POINTER(_I64), C.POINTER(_I64)],
    "cai_model_finalize": [_P],
    "cai_model_step_weight_bytes": [_P, C.POINTER(_I64)],
    "cai_session_create": [_P, _I, _I, _I, _PP],
    "cai_session_destroy": [_P],
    "cai_session_reset": [_P, _I],
    "cai_session_truncate": [_P, _I, _I],
    "cai_session_cache_len": [_P, _I, C.POINTER(_I)],
    "cai_session_fill_for_benchmark": [_P, _I],
    "cai_session_enable_eviction": [_P, _I, _I],
    "cai_session_set_window": [_P, _I],
    "cai_session_step": [_P, _P, _P, _P, _P],
    "cai_session_decode_greedy": [_P, _P, _I, _P],
    "cai_session_step_topk": [_P, _P, _P, _I, C.c_float, _P, _P],
    "cai_session_decode_sampled": [_P, _P, _I, _P, _P, _P],
    "cai_sampling_uniform": [C.c_uint64, C.c_uint64, C.c_uint64, C.POINTER(C.c_float)],
    "cai_session_prefill": [_P, _P, _I],
    "cai_session_profile": [_P, _P, _I, C.POINTER(C.c_float), C.POINTER(_I64)],
    "cai_session_snapshot": [_P],
    "cai_session_restore": [_P],
    "cai_session_logits_dev": [_P, _PP],
    "cai_session_read_kv_row": [_P, _I, _I, _I, _I, _P, _P, _P, _P, _P],
    "cai_session_uses_step_kernel": [_P, C.POINTER(_I)],
    "cai_session_step_trace": [_P, _P, C.POINTER(_I64), C.POINTER(C.c_int32), _I, C.POINTER(_I)],
    "cai_session_last_kv_bytes": [_P, C.POINTER(_I64)],
    "cai_comm_unique_id": [_P],
    "cai_comm_init": [_P, _I, _I, _P],
    "cai_comm_allreduce_dev": [_P, _P, _I64],
}

_lib = None


def load():
    """Loads the shared library once and declares every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            "%s is not built (%s). Run `python -m neural_api_b200.build%s`; "
            "there is no CPU fallback." % (os.path.basename(LIB_PATH), LIB_PATH, " --checked" if CHECKED else ""))
    lib = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.argtypes = argtypes
        fn.restype = C.c_int
    _lib = lib
    return lib
