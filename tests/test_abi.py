"""The C-ABI library loads, exports every symbol include/tqb200.h declares and
rejects invalid arguments with the documented status codes (no GPU needed:
validation happens before any CUDA call)."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "tqb200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(tq_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(tq):
    lib = tq._lib.lib()
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in tqb200.h but not exported"
    assert sorted(tq._lib.exported_symbols()) == declared
    assert lib.tq_version() >= 100


def test_struct_layout_matches(tq):
    # tq_flash_decode checks struct_bytes; a mismatch would be reported, not crash
    P = tq._lib.FlashParams()
    P.struct_bytes = ctypes.sizeof(tq._lib.FlashParams) - 8
    assert tq._lib.lib().tq_flash_decode(ctypes.byref(P)) == -7
    assert b"struct_bytes" in tq._lib.lib().tq_last_error_string()


def test_argument_validation_without_gpu(tq):
    L = tq._lib.lib()
    signs = (ctypes.c_float * 128)(*([1.0] * 128))
    bnd = (ctypes.c_float * 7)(*([0.0] * 7))
    null = ctypes.c_void_p(0)
    one = ctypes.c_void_p(16)
    assert L.tq_quantize(one, 1, 1, 1, 128, 100, 3, signs, bnd, one, 13, one, 1, null) == -1
    assert b"power of 2" in L.tq_last_error_string()
    assert L.tq_quantize(one, 1, 1, 1, 128, 128, 5, signs, bnd, one, 13, one, 1, null) == -2
    assert b"Unsupported bit width: 5" in L.tq_last_error_string()
    bad = (ctypes.c_float * 128)(*([0.5] * 128))
    assert L.tq_quantize(one, 1, 1, 1, 128, 128, 3, bad, bnd, one, 13, one, 1, null) == -7
    assert L.tq_quantize(one, 1, 0, 0, 128, 128, 3, signs, bnd, one, 13, one, 1, null) == 0  # empty
    assert L.tq_sparse_v_matvec(one, 1, one, 1, one, 1, 1, 1, bnd, signs, 512, 3, 0.0, 1, one,
                                null, 0, null) == -1
    assert b"dim > 256" in L.tq_last_error_string()
    assert L.tq_sparse_v_matvec(one, 1, one, 1, one, 1, 1, 64, bnd, signs, 128, 3, 0.0, 1, one,
                                null, 0, null) == -5
    assert L.tq_sparse_v_workspace_bytes(28, 32768, 128) == 64 * 28 * 128 * 4


def test_python_wrappers_refuse_cpu_tensors(tq):
    import torch
    x = torch.zeros((4, 128), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        tq.fused_quantize(x, [1.0] * 128, [0.0] * 7, 128, 3)
    with pytest.raises(ValueError, match="expects .n_heads, dim."):
        tq.prerotate_query(torch.zeros((2, 2, 128)), [1.0] * 128)
    with pytest.raises(ValueError, match="block_size"):
        tq.flash_attention_turboquant(x, x, torch.zeros((4, 1)), x, x, None, None, None, 128, 3, 1.0,
                                      block_size=64)
