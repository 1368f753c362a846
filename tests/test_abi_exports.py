"""CPU: the shared library loads and exports every symbol include/kanso_cuda.h declares."""
import ctypes
import os
import re

from conftest import ROOT, package


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "kanso_cuda.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(kanso_cuda_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    pkg = package()
    lib_path = pkg.build.build()
    lib = ctypes.CDLL(lib_path)
    syms = declared_symbols()
    assert len(syms) >= 35
    missing = [s for s in syms if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_binding_covers_header():
    kb = package().backend
    assert sorted(kb.PROTOTYPES) == declared_symbols()
    kb.load()


def test_no_gpu_is_an_error_not_a_fallback():
    import torch
    if torch.cuda.is_available():
        return
    kb = package().backend
    try:
        kb.Context(0)
    except kb.KansoError as e:
        assert e.code == kb.ERR_DEVICE and "no CPU fallback" in e.message
    else:
        raise AssertionError("context creation must fail without a GPU")


def test_validate_params_needs_no_device():
    kb = package().backend
    kb.validate_paged_attention_params(kb.PagedAttentionParams(1, 15, 5, 64, 16, 256, 0.125))
    for bad in [kb.PagedAttentionParams(1, 15, 4, 64, 16, 256, 0.125),
                kb.PagedAttentionParams(1, 18, 2, 64, 16, 4, 1.0),
                kb.PagedAttentionParams(1, 8, 2, 384, 16, 4, 1.0),
                kb.PagedAttentionParams(0, 8, 2, 64, 16, 4, 1.0)]:
        try:
            kb.validate_paged_attention_params(bad)
        except kb.KansoError as e:
            assert e.code == kb.ERR_UNSUPPORTED
        else:
            raise AssertionError("invalid params accepted")
