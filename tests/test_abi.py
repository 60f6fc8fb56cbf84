"""The C-ABI library loads, exports every symbol include/cai_cuda.h declares, and its
host-only paths behave (no compute calls: these tests run without a GPU)."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "cai_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\bint\s+(cai_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    from neural_api_b200 import build
    build.build()                       # compiles only what is stale
    from neural_api_b200 import _lib
    return _lib.load()


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    assert len(names) >= 50
    for must in ("cai_cuda_init", "cai_linear_create", "cai_linear_forward", "cai_session_step", "cai_dequantize",
                 "cai_model_upload_tensor", "cai_comm_init"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_symbols():
        assert hasattr(lib, name), name


def test_binding_table_matches_the_header(lib):
    from neural_api_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_pascal_unit_declares_every_symbol_with_the_header_arity():
    """neuralcuda.pas cannot be compiled here (no Free Pascal), so its external declarations are checked as text:
    one per header symbol, same number of parameters."""
    text = open(os.path.join(ROOT, "include", "cai_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    header = {n: len(a.split(",")) for n, a in re.findall(r"\bint\s+(cai_[a-z0-9_]+)\s*\(([^;]*?)\)\s*;", text, flags=re.S)}
    pas = open(os.path.join(ROOT, "neural_api_b200", "pascal", "neuralcuda.pas")).read()
    decls = dict(re.findall(r"function (cai_[a-z0-9_]+)\((.*?)\): cint; cdecl; external CaiLib;", pas))
    assert sorted(decls) == sorted(header)
    for name, params in decls.items():
        n = 0
        for group in params.split(";"):                      # "a, b: cint" declares two parameters
            n += len(group.split(":")[0].split(","))
        assert n == header[name], name
    for const in ("CAI_TYPE_I8 = 24", "CAI_TYPE_I8ROW = 124", "CAI_TYPE_Q4_K = 12", "CAI_TYPE_Q6_K = 14"):
        assert const in pas


def test_config_struct_layout():
    from neural_api_b200._lib import LlamaConfigC
    assert C.sizeof(LlamaConfigC) == 16 * 4


def test_null_handles_are_rejected_without_touching_a_gpu(lib):
    assert lib.cai_cuda_shutdown(None) == 1
    assert lib.cai_linear_destroy(None) == 1
    assert lib.cai_session_destroy(None) == 1
    assert lib.cai_model_destroy(None) == 1
    assert lib.cai_sdpa_destroy(None) == 1
    assert lib.cai_comm_unique_id(None) == 1


def test_init_on_a_missing_device_returns_a_status(lib):
    ctx = C.c_void_p()
    st = lib.cai_cuda_init(4096, C.byref(ctx))     # no machine has this many GPUs
    assert st == 2 and not ctx.value


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from neural_api_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "absent.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()


def test_checked_twin_exports_the_same_surface_and_says_what_it_is(lib):
    """libcai_cuda_checked.so (-DCAI_CHECKED: every launch synchronized and looked at, silent index clamps reported) has
    the ordinary library's entry points; cai_cuda_is_checked_build tells the two apart without a GPU."""
    from neural_api_b200 import build
    checked = C.CDLL(build.build(checked=True))
    for name in declared_symbols():
        assert hasattr(checked, name), name
    assert checked.cai_cuda_is_checked_build() == 1
    assert lib.cai_cuda_is_checked_build() == 0
