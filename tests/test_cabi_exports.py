"""The C-ABI library builds, loads without a GPU and exports every symbol include/mpsa.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "mpsa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(?:int|long long)\s+(mpsa_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from mpsa import _lib
    lib = _lib.load()
    names = _declared()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/mpsa.h but not exported"
    assert sorted(_lib.EXPORTS) == names
    assert lib.mpsa_version() >= 100


def test_argument_errors_are_reported_without_a_gpu():
    from mpsa import _lib
    lib = _lib.load()
    # null pointers / bad shapes are rejected before any CUDA call
    rc = lib.mpsa_quant_mx(None, 0, 1, 1, 128, 128, 0, 0, 0, 1.0, 1, None, 0, 0, 0, None, 0, 0, 0,
                           None, None, None, None, None, None)
    assert rc == -1 and "quant_mx" in _lib.last_error()
    rc = lib.mpsa_gemm_block_scaled(None, None, None, None, None, 128, 128, 128, 128, 128, 128, 0, 1, 1, 0, 1.0,
                                    None, None)
    assert rc == -1 and "gemm_block_scaled" in _lib.last_error()
    rc = lib.mpsa_route_band(None, 1, 1, 128, 1, 1, 128, 128, None)
    assert rc == -1


def test_cpu_tensors_are_refused():
    import pytest
    import torch
    import mpsa
    with pytest.raises(ValueError):
        mpsa.quantize_mx(torch.zeros(1, 1, 128, 128, dtype=torch.bfloat16))
