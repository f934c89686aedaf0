"""ctypes binding of libmpsa.so (the C-ABI declared in include/mpsa.h).

There is no CPU fallback: if the library is missing it is built with nvcc; if that fails, or a
call returns an error code, an exception is raised.
"""
import ctypes
import os
import sys

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.environ.get("MPSA_LIB") or os.path.join(_HERE, "libmpsa.so")   # MPSA_LIB: use another build
_lib = None

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

_SIGNATURES = {
    "mpsa_version": ([], c_int),
    "mpsa_last_error": ([ctypes.c_char_p, ctypes.c_ulonglong], c_int),
    "mpsa_selftest_wait_timeout": ([c_void_p, c_ll, c_int, c_void_p], c_int),
    "mpsa_quant_mx": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_float, c_int,
                       c_void_p, c_ll, c_ll, c_ll, c_void_p, c_ll, c_ll, c_ll, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p], c_int),
    "mpsa_quant_mx_centered": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_float, c_void_p, c_int,
                                c_void_p, c_ll, c_ll, c_ll, c_void_p, c_ll, c_ll, c_ll, c_void_p, c_void_p, c_void_p,
                                c_void_p, c_void_p, c_void_p], c_int),
    "mpsa_rope_quant_mx": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_void_p, c_void_p, c_ll, c_float,
                            c_int, c_void_p, c_ll, c_ll, c_ll, c_void_p, c_ll, c_ll, c_ll, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_void_p], c_int),
    "mpsa_col_mean_scratch_floats": ([c_int, c_int, c_int, c_int], c_ll),
    "mpsa_col_mean": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_void_p, c_void_p, c_ll,
                       c_void_p], c_int),
    "mpsa_quant_int8": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_float, c_void_p,
                         c_ll, c_ll, c_ll, c_void_p, c_void_p], c_int),
    "mpsa_prepare_vt": ([c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll,
                         c_void_p], c_int),
    "mpsa_route_band": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p], c_int),
    "mpsa_route_stat": ([c_void_p] * 6 + [c_int] * 6 + [c_void_p, c_void_p], c_int),
    "mpsa_route_online": ([c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p], c_int),
    "mpsa_quant_nvfp4_scratch_floats": ([c_int, c_int], c_int),
    "mpsa_quant_nvfp4": ([c_void_p, c_int, c_int, c_int, c_ll, c_float, c_void_p, c_ll, c_void_p, c_ll, c_void_p,
                          c_void_p, c_void_p], c_int),
    "mpsa_quant_nvfp4_bh": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_float, c_void_p, c_ll,
                             c_void_p, c_void_p, c_void_p, c_void_p], c_int),
    "mpsa_quant_nvfp4_static": ([c_void_p, c_int, c_int, c_int, c_ll, c_float, c_void_p, c_ll, c_void_p, c_void_p,
                                 c_void_p], c_int),
    "mpsa_quant_v_seq": ([c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int,
                          c_void_p, c_void_p, c_void_p, c_void_p, c_void_p], c_int),
    "mpsa_attn_fwd": ([c_void_p] * 13 + [c_int, c_void_p, c_ll, c_ll, c_void_p, c_int, c_void_p] + [c_int] * 10 +
                      [c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p], c_int),
    "mpsa_attn_fwd_routed": ([c_void_p] * 13 + [c_int, c_float, c_void_p, c_int] + [c_void_p] * 4 + [c_int] * 9 +
                             [c_void_p, c_void_p, c_void_p], c_int),
    "mpsa_attn_merge": ([c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_ll, c_int, c_void_p], c_int),
    "mpsa_gemm_block_scaled_batched": ([c_void_p] * 5 + [c_int] * 8 + [c_float, c_void_p, c_void_p], c_int),
    "mpsa_gemm_block_scaled": ([c_void_p] * 5 + [c_int, c_int, c_int, c_ll, c_ll, c_ll, c_int, c_int, c_int, c_int,
                                c_float, c_void_p, c_void_p], c_int),
}
EXPORTS = tuple(_SIGNATURES)


class MpsaError(RuntimeError):
    pass


def lib_path():
    return _LIB_PATH


def load():
    """Load (building first if necessary) the CUDA library.  Raises if it cannot be had."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        sys.path.insert(0, os.path.dirname(_HERE))
        try:
            import build as _build
            _build.build_lib()
        finally:
            sys.path.pop(0)
    if not os.path.exists(_LIB_PATH):
        raise MpsaError(f"{_LIB_PATH} is missing and could not be built; there is no fallback path")
    lib = ctypes.CDLL(_LIB_PATH)
    for name, (args, res) in _SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = res
    _lib = lib
    return lib


def last_error():
    buf = ctypes.create_string_buffer(512)
    load().mpsa_last_error(buf, 512)
    return buf.value.decode(errors="replace")


def check(rc):
    """Turn a C-ABI return code into an exception (ValueError for argument errors)."""
    if rc == 0:
        return
    msg = last_error()
    if rc in (-1, -2):
        raise ValueError(msg)
    raise MpsaError(f"libmpsa error {rc}: {msg}")
