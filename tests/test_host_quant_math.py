"""The per-element quantizer arithmetic that the CUDA kernels execute (csrc/quant_math.h), built
for the host with g++ and checked bit-for-bit against the golden vectors and the oracle.
No GPU needed."""
import ctypes
import os
import subprocess

import numpy as np
import pytest
import torch

from oracle import mx_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
G = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(scope="module")
def hostlib(tmp_path_factory):
    out = str(tmp_path_factory.mktemp("qmh") / "libqmh.so")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off",
           "-I", os.path.join(ROOT, "mp-sparse-attn_b200", "csrc"), "-I", cuda_inc,
           os.path.join(ROOT, "tests", "host", "quant_math_host.cpp"), "-o", out]
    subprocess.run(cmd, check=True)
    return ctypes.CDLL(out)


def _run_mx(lib, x_bf16, s, fp8_fmt=1):
    x = x_bf16.contiguous()
    d = x.shape[-1]
    rows = x.numel() // d
    bits = x.view(torch.int16).numpy().view(np.uint16).reshape(rows, d)
    fp4 = np.empty((rows, d), np.uint8)
    fp8 = np.empty((rows, d), np.uint8)
    s4 = np.empty((rows, d // 32), np.uint8)
    s8 = np.empty((rows, d // 32), np.uint8)
    P = ctypes.c_void_p
    lib.host_quant_mx(P(bits.ctypes.data), ctypes.c_longlong(rows), d, ctypes.c_float(s), fp8_fmt,
                      P(fp4.ctypes.data), P(s4.ctypes.data), P(fp8.ctypes.data), P(s8.ctypes.data))
    shp = tuple(x.shape)
    return fp4.reshape(shp), s4.reshape(shp[:-1] + (d // 32,)), fp8.reshape(shp), s8.reshape(shp[:-1] + (d // 32,))


@pytest.mark.parametrize("tag", ["kat", "d128", "d64"])
def test_kernel_math_matches_reference_golden(hostlib, tag):
    z = np.load(os.path.join(G, "quant_kat.npz"))
    if tag == "kat":
        q = k = torch.from_numpy(z["kat_x"]).view(torch.bfloat16)
    else:
        q = torch.from_numpy(z[f"{tag}_q"]).view(torch.bfloat16)
        k = torch.from_numpy(z[f"{tag}_k"]).view(torch.bfloat16)
    sq = O.q_side_scale(q.shape[-1])
    for side, x, s in (("q", q, sq), ("k", k, 1.0)):
        fp4, s4, fp8, s8 = _run_mx(hostlib, x, s)
        assert np.array_equal(fp4, z[f"{tag}_fp4_{side}"])
        assert np.array_equal(s4, z[f"{tag}_fp4_{side}s"])
        assert np.array_equal(s8, z[f"{tag}_fp8_{side}s"])
        # fp8 element codes: the golden run cannot pin them (interpreter cast), the oracle does
        oc, os_ = O.quant_mxfp8_side(x, s)
        assert np.array_equal(fp8, oc.numpy()) and np.array_equal(s8, os_.numpy())


def test_kernel_math_e4m3_matches_oracle(hostlib):
    q, k, _ = O.make_qkv(11, 1, 2, 1, 128, 128, outliers=5)
    for x, s in ((q, O.q_side_scale(128)), (k, 1.0)):
        _, _, fp8, s8 = _run_mx(hostlib, x, s, fp8_fmt=2)
        oc, os_ = O.quant_mxfp8_side(x, s, "e4m3")
        assert np.array_equal(fp8, oc.numpy()) and np.array_equal(s8, os_.numpy())


def test_kernel_math_int8_matches_golden(hostlib):
    z = np.load(os.path.join(G, "quant_kat.npz"))
    q = torch.from_numpy(z["d128_q"]).view(torch.bfloat16)
    d = q.shape[-1]
    rows = q.numel() // d
    bits = q.contiguous().view(torch.int16).numpy().view(np.uint16).reshape(rows, d)
    codes = np.empty((rows, d), np.int8)
    scales = np.empty((rows, d // 32), np.float32)
    P = ctypes.c_void_p
    hostlib.host_quant_int8(P(bits.ctypes.data), ctypes.c_longlong(rows), d, ctypes.c_float(O.q_side_scale(d)),
                            P(codes.ctypes.data), P(scales.ctypes.data))
    assert np.array_equal(codes.reshape(q.shape), z["d128_i8_q"])
    oc, os_ = O.quant_fpxint8_side(q, O.q_side_scale(d))
    assert np.array_equal(scales.reshape(os_.shape), os_.numpy())


def test_fp4_rne_matches_reference_helper(hostlib):
    z = np.load(os.path.join(G, "mxfp_helpers.npz"))
    x = np.ascontiguousarray(z["fp4_in"])
    finite = np.isfinite(x)
    codes = np.empty(x.shape, np.uint8)
    hostlib.host_fp4_rne(ctypes.c_void_p(x.ctypes.data), ctypes.c_longlong(x.size), ctypes.c_void_p(codes.ctypes.data))
    assert np.array_equal(codes[finite], z["fp4_codes"][finite])
