"""The CPU oracle against vectors the unmodified reference produced ON A B200 (tests/golden/ref_gpu.npz,
written by tests/golden/make_golden_gpu.py): MXFP8 element codes (the Triton CPU interpreter cannot pin
those), MXFP4 codes, E8M0 scale codes, the fused attention output of the reference's "mxfp8" mode and the
output of its block-scaled GEMM kernel.  Runs without a GPU."""
import importlib.util
import os

import numpy as np
import torch

from oracle import mx_oracle as O

G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _gen():
    spec = importlib.util.spec_from_file_location("make_golden_gpu", os.path.join(G, "make_golden_gpu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _cases():
    z = np.load(os.path.join(G, "quant_kat.npz"))
    kat = torch.from_numpy(z["kat_x"]).view(torch.bfloat16)
    yield "kat", kat, kat
    yield "d128", torch.from_numpy(z["d128_q"]).view(torch.bfloat16), torch.from_numpy(z["d128_k"]).view(torch.bfloat16)
    q, k = _gen().quant_inputs_f16()
    yield "f16", q, k


def nonzero_blocks(x):
    """[..., L, D] -> bool [..., L, D]: True where the element's 32-block holds a non-zero value.  On an all-zero
    block the reference divides 0 by 0; what comes out depends on who runs it (the GPU run stores the largest finite
    code, the CPU interpreter the code of -0), so those blocks are compared nowhere."""
    nz = (x.float().reshape(*x.shape[:-1], -1, 32) != 0).any(-1, keepdim=True)
    return nz.expand(*nz.shape[:-1], 32).reshape(x.shape).numpy()


def test_quantizer_codes_equal_the_reference_gpu_run():
    r = np.load(os.path.join(G, "ref_gpu.npz"))
    for tag, q, k in _cases():
        a8, s8q, b8, s8k = O.quant_mxfp8e5(q, k)
        a4, s4q, b4, s4k = O.quant_mxfp4(q, k)
        for side, x, c8, s8, c4, s4 in (("q", q, a8, s8q, a4, s4q), ("k", k, b8, s8k, b4, s4k)):
            m = nonzero_blocks(x)
            assert m.any()
            assert np.array_equal(c8.numpy()[m], r[f"{tag}_fp8_{side}"][m]), (tag, side, "fp8 element codes")
            assert np.array_equal(c4.numpy()[m], r[f"{tag}_fp4_{side}"][m]), (tag, side, "fp4 element codes")
            assert np.array_equal(s8.numpy(), r[f"{tag}_fp8_{side}s"]), (tag, side, "fp8 scale codes")
            assert np.array_equal(s4.numpy(), r[f"{tag}_fp4_{side}s"]), (tag, side, "fp4 scale codes")


def test_attention_oracle_matches_the_reference_kernel_output():
    """ours/mxfp_attn_kernel.py::mxfp_attn_kernel(block_scale_type="mxfp8", skip_thresh=-1e9), non-causal, run on
    a B200: the oracle composed from the reference's pieces must reproduce the kernel it restates.  Tolerance: the
    task's cos >= 0.9999 / rel-L2 <= 1e-2 (measured ~1e-3: the kernel accumulates each tile's P.V in fp16)."""
    r = np.load(os.path.join(G, "ref_gpu.npz"))
    q, k, v = _gen().attn_inputs()
    ref = torch.from_numpy(r["attn_fp8_out"].astype(np.float32))
    out = O.attention_mxfp(q, k, v, causal=False, uniform="fp8", pv_mode="fp16")
    m = O.parity_metrics(out, ref)
    assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2, m


def test_gemm_oracle_matches_the_reference_kernel_output():
    """block_scaled_matmul "mxfp8" (ours/block_scaled_matmul.py:271-296) on a B200 against the oracle's emulation
    and the reference's own PyTorch emulation, at the reference's tolerance (atol = rtol = 1e-3, :440)."""
    r = np.load(os.path.join(G, "ref_gpu.npz"))
    ge = np.load(os.path.join(G, "gemm_emulation.npz"))
    kernel = torch.from_numpy(r["gemm_mxfp8_out"])
    torch.testing.assert_close(kernel, torch.from_numpy(ge["reference"]), atol=1e-3, rtol=1e-3)
    a, b = torch.from_numpy(ge["a_codes"]), torch.from_numpy(ge["b_codes"])
    sa = O.unswizzle_scales(torch.from_numpy(ge["a_scale_tiles"]), a.shape[0], a.shape[1] // 32)
    sb = O.unswizzle_scales(torch.from_numpy(ge["b_scale_tiles"]), b.shape[0], b.shape[1] // 32)
    mine = O.gemm_block_scaled(a, sa, b, sb, "fp8e5", "fp8e5")
    torch.testing.assert_close(kernel, mine, atol=1e-3, rtol=1e-3)
