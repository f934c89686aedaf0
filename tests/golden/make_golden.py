"""Generate the golden vectors under tests/golden/ by RUNNING THE REFERENCE.

Usage (only where the reference checkout is available; pass its path):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference

What is recorded
* ``quant_kat.npz``     - the hand-made 32-element block of known answers and a seeded
                          [1,2,256,128]/[1,1,256,128] bf16 case with outlier K channels and a
                          D=64 case, pushed through the reference's ``quant_mxfp4``,
                          ``quant_mxfp8e5`` and ``quant_fpxint8`` (Triton kernels executed by the
                          Triton CPU interpreter).  For ``quant_mxfp8e5`` only the SCALE codes
                          are kept: the interpreter's fp32->fp8 cast is not the GPU's
                          round-to-nearest-even cast, so its element codes are not a reference.
* ``mxfp_helpers.npz``  - ``ours/mxfp.py``: MXFP4Tensor from-float / to-float / pack / unpack and
                          MXScaleTensor from-float / to-float.
* ``gemm_emulation.npz``- ``ours/block_scaled_matmul.py::initialize_block_scaled_from_tensor``
                          (mxfp8, 128x256x256, seed 42, compute_reference=True): operands, E8M0
                          scale tiles and the PyTorch-emulated product.
"""
import os
import sys

import numpy as np
import torch

os.environ.setdefault("TRITON_INTERPRET", "1")
HERE = os.path.dirname(os.path.abspath(__file__))


def bf16_bits(t):
    return t.contiguous().view(torch.int16).numpy()


def main(ref_root):
    sys.path.insert(0, ref_root)
    from ours.quant_mxint8 import quant_mxfp4, quant_mxfp8e5, quant_fpxint8
    from ours.mxfp import MXFP4Tensor, MXScaleTensor

    out = {}
    # ---- known-answer block -------------------------------------------------------
    blk = torch.tensor([0, 0.1001, 0.124, 0.125, 0.126, 0.25, 0.5, 0.8984, 1, 1.25, 1.2578, 1.5,
                        1.8984, 2, 2.5, 2.5938, 3, 3.9062, 4, 5, 5.0938, 6, 7.9062, 8, 12, 15.875,
                        -0.8984, -1.2578, -5.0938, -15.875, -0.0, 0.3008], dtype=torch.float32)
    rows = torch.stack([blk, blk * 0.25, torch.zeros(32), blk.flip(0) * 3.0])
    # [1,1,128,64]: rows cycle through the 4 patterns, second 32-block is the negated row
    x = torch.cat([rows, -rows], dim=1).repeat(32, 1).reshape(1, 1, 128, 64).to(torch.bfloat16)
    out["kat_x"] = bf16_bits(x)
    a, sa, b, sb = quant_mxfp4(x, x)
    out.update(kat_fp4_q=a.numpy(), kat_fp4_qs=sa.numpy(), kat_fp4_k=b.numpy(), kat_fp4_ks=sb.numpy())
    a, sa, b, sb = quant_mxfp8e5(x, x)
    out.update(kat_fp8_qs=sa.numpy(), kat_fp8_ks=sb.numpy())
    a, sa, b, sb = quant_fpxint8(x, x)
    out.update(kat_i8_q=a.numpy(), kat_i8_qs=sa.numpy(), kat_i8_k=b.numpy(), kat_i8_ks=sb.numpy())

    # ---- seeded tensors -----------------------------------------------------------
    for tag, (hq, hkv, s, d) in {"d128": (2, 1, 256, 128), "d64": (2, 2, 128, 64)}.items():
        g = torch.Generator().manual_seed(1234)
        q = torch.randn(1, hq, s, d, generator=g)
        k = torch.randn(1, hkv, s, d, generator=g)
        idx = torch.randperm(d, generator=g)[:5]
        k[..., idx] *= 20.0
        q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
        out[f"{tag}_q"] = bf16_bits(q)
        out[f"{tag}_k"] = bf16_bits(k)
        a, sa, b, sb = quant_mxfp4(q, k)
        out.update({f"{tag}_fp4_q": a.numpy(), f"{tag}_fp4_qs": sa.numpy(),
                    f"{tag}_fp4_k": b.numpy(), f"{tag}_fp4_ks": sb.numpy()})
        a, sa, b, sb = quant_mxfp8e5(q, k)
        out.update({f"{tag}_fp8_qs": sa.numpy(), f"{tag}_fp8_ks": sb.numpy()})
        a, sa, b, sb = quant_fpxint8(q, k)
        out.update({f"{tag}_i8_q": a.numpy(), f"{tag}_i8_qs": sa.numpy(),
                    f"{tag}_i8_k": b.numpy(), f"{tag}_i8_ks": sb.numpy()})
    np.savez_compressed(os.path.join(HERE, "quant_kat.npz"), **out)

    # ---- ours/mxfp.py helpers -----------------------------------------------------
    g = torch.Generator().manual_seed(7)
    vals = torch.cat([torch.linspace(-7, 7, 225), torch.randn(800, generator=g) * 2.5,
                      torch.tensor([0.0, -0.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, float("inf"),
                                    float("-inf"), float("nan")])]).to(torch.float32)
    vals = vals[: (vals.numel() // 2) * 2]
    t = MXFP4Tensor(data=vals.clone())
    codes = t.data.clone()
    packed = t.to_packed_tensor(dim=0)
    unpacked = t.unpack_packed_tensor(packed, dim=0, original_shape=codes.shape)
    allc = torch.arange(16, dtype=torch.uint8)
    dec = MXFP4Tensor(data=allc, dtype=torch.uint8).to(torch.float32)
    sv = torch.cat([torch.rand(200, generator=g) * 4, torch.tensor([0.0, -1.0, 1.0, 2.0, 0.5, 3e38, 1e-38,
                                                                   float("inf"), float("nan")])])
    st = MXScaleTensor(data=sv.clone())
    sdec = MXScaleTensor(data=torch.ones(1))
    sdec.data = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    np.savez_compressed(os.path.join(HERE, "mxfp_helpers.npz"),
                        fp4_in=vals.numpy(), fp4_codes=codes.numpy(), fp4_packed=packed.numpy(),
                        fp4_unpacked=unpacked.numpy(), fp4_decode16=dec.numpy(),
                        e8m0_in=sv.numpy(), e8m0_codes=st.data.numpy(),
                        e8m0_decode256=sdec.to(torch.float32).numpy())

    # ---- 2-D GEMM emulation -------------------------------------------------------
    from ours.block_scaled_matmul import initialize_block_scaled_from_tensor
    torch.manual_seed(42)
    M, N, K = 128, 256, 256
    a_t = torch.randn((M, K), dtype=torch.float16)
    b_t = torch.randn((N, K), dtype=torch.float16)
    a_s = torch.rand((M // 128, K // 32 // 4, 32, 4, 4)) + 1e-8
    b_s = torch.rand((N // 128, K // 32 // 4, 32, 4, 4)) + 1e-8
    a, sa, b, sb, cfg, (ref, _, _) = initialize_block_scaled_from_tensor(
        a_t, b_t, a_s, b_s, "mxfp8", compute_reference=True)
    np.savez_compressed(os.path.join(HERE, "gemm_emulation.npz"),
                        a_codes=a.view(torch.uint8).numpy(), b_codes=b.view(torch.uint8).numpy(),
                        a_scale_tiles=sa.numpy(), b_scale_tiles=sb.numpy(), reference=ref.numpy(),
                        a_scale_in=a_s.numpy(), b_scale_in=b_s.numpy())
    print("golden vectors written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
