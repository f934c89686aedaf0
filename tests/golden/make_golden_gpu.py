"""Generate tests/golden/ref_gpu.npz by RUNNING THE REFERENCE'S TRITON KERNELS ON A GPU (sm_100).

    python tests/golden/make_golden_gpu.py /path/to/reference [out.npz]

The Triton CPU interpreter does not reproduce the GPU's fp32 -> fp8 cast, and it cannot run
`tl.dot_scaled` at all, so the vectors that pin the MXFP8 element codes, the fused attention output and
the GEMM kernel's output come from a GPU run of the unmodified reference:

* ``quant_mxfp8e5`` / ``quant_mxfp4`` (ours/quant_mxint8.py:223-272, :453-512) on the known-answer block
  and the seeded [1,2,256,128] / [1,1,256,128] bf16 tensors of ``quant_kat.npz`` (same bits: they are read
  from that file), plus a seeded fp16 case: element codes and E8M0 scale codes.
* ``mxfp_attn_kernel(q, k, v, block_scale_type="mxfp8", skip_thresh=-1e9)`` (ours/mxfp_attn_kernel.py:19-74)
  on a seeded B=1 H=2 S=384 D=128 fp16 case (non-causal, every tile processed): the fp16 output.  The
  MXFP4 mode of that wrapper is not run: it packs pairs of heads instead of pairs of depth elements and
  reads out of bounds for the upper half of the heads.
* ``block_scaled_matmul`` in "mxfp8" mode (ours/block_scaled_matmul.py:271-296) on the operands of
  ``gemm_emulation.npz``: the kernel's fp32 output.

Inputs are drawn with the CPU generator, so tests regenerate them bit for bit anywhere.
"""
import os
import sys

import numpy as np
import torch
import torch._dynamo  # noqa: F401  (must be imported before the reference's namespace package `ours` enters sys.modules)

HERE = os.path.dirname(os.path.abspath(__file__))


def attn_inputs():
    """The attention case of ref_gpu.npz: fp16 N(0,1) Q, K, V with 5 K channels scaled x8."""
    g = torch.Generator().manual_seed(77)
    q = torch.randn(1, 2, 384, 128, generator=g)
    k = torch.randn(1, 2, 384, 128, generator=g)
    v = torch.randn(1, 2, 384, 128, generator=g)
    k[..., torch.randperm(128, generator=g)[:5]] *= 8.0
    return q.to(torch.float16), k.to(torch.float16), v.to(torch.float16)


def quant_inputs_f16():
    """fp16 operands of very different magnitude.  The lengths are multiples of the reference's row blocks (128 for Q,
    64 for K): its scale store is not masked, so a ragged last block overwrites the next head's first rows."""
    g = torch.Generator().manual_seed(4321)
    q = (torch.randn(1, 3, 256, 128, generator=g) * 3.0).to(torch.float16)
    k = (torch.randn(1, 3, 192, 128, generator=g) * 0.05).to(torch.float16)
    return q, k


def main(ref_root, out_path):
    if not torch.cuda.is_available():
        raise SystemExit("make_golden_gpu.py needs a CUDA device: it runs the reference's Triton kernels")
    sys.path.insert(0, ref_root)
    from ours.quant_mxint8 import quant_mxfp4, quant_mxfp8e5
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    from ours.block_scaled_matmul import block_scaled_matmul

    z = np.load(os.path.join(HERE, "quant_kat.npz"))
    out = {}
    cases = {"kat": (z["kat_x"], z["kat_x"]), "d128": (z["d128_q"], z["d128_k"])}
    for tag, (qb, kb) in cases.items():
        q = torch.from_numpy(qb).view(torch.bfloat16).cuda()
        k = torch.from_numpy(kb).view(torch.bfloat16).cuda()
        a, sa, b, sb = quant_mxfp8e5(q, k)
        out.update({f"{tag}_fp8_q": a.view(torch.uint8).cpu().numpy(), f"{tag}_fp8_qs": sa.cpu().numpy(),
                    f"{tag}_fp8_k": b.view(torch.uint8).cpu().numpy(), f"{tag}_fp8_ks": sb.cpu().numpy()})
        a, sa, b, sb = quant_mxfp4(q, k)
        out.update({f"{tag}_fp4_q": a.cpu().numpy(), f"{tag}_fp4_qs": sa.cpu().numpy(),
                    f"{tag}_fp4_k": b.cpu().numpy(), f"{tag}_fp4_ks": sb.cpu().numpy()})
    q, k = quant_inputs_f16()
    a, sa, b, sb = quant_mxfp8e5(q.cuda(), k.cuda())
    out.update(f16_fp8_q=a.view(torch.uint8).cpu().numpy(), f16_fp8_qs=sa.cpu().numpy(),
               f16_fp8_k=b.view(torch.uint8).cpu().numpy(), f16_fp8_ks=sb.cpu().numpy())
    a, sa, b, sb = quant_mxfp4(q.cuda(), k.cuda())
    out.update(f16_fp4_q=a.cpu().numpy(), f16_fp4_qs=sa.cpu().numpy(), f16_fp4_k=b.cpu().numpy(), f16_fp4_ks=sb.cpu().numpy())

    q, k, v = attn_inputs()
    o = mxfp_attn_kernel(q.cuda(), k.cuda(), v.cuda(), is_causal=False, block_scale_type="mxfp8", skip_thresh=-1e9)
    torch.cuda.synchronize()
    out["attn_fp8_out"] = o.float().cpu().numpy().astype(np.float16)

    ge = np.load(os.path.join(HERE, "gemm_emulation.npz"))
    a = torch.from_numpy(ge["a_codes"]).cuda().view(torch.float8_e5m2)
    b = torch.from_numpy(ge["b_codes"]).cuda().view(torch.float8_e5m2)
    sa, sb = torch.from_numpy(ge["a_scale_tiles"]).cuda(), torch.from_numpy(ge["b_scale_tiles"]).cuda()
    cfg = {"BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 128, "num_stages": 4, "ELEM_PER_BYTE_A": 1,
           "ELEM_PER_BYTE_B": 1, "VEC_SIZE": 32}
    M, K = a.shape
    N = b.shape[0]
    c = block_scaled_matmul(a, sa, b, sb, torch.float32, M, N, K, cfg)
    torch.cuda.synchronize()
    out["gemm_mxfp8_out"] = c.cpu().numpy()
    out["meta"] = np.array([f"torch {torch.__version__}", f"gpu {torch.cuda.get_device_name(0)}"])
    np.savez_compressed(out_path, **out)
    print("reference GPU vectors written to", out_path)


if __name__ == "__main__":
    if len(sys.argv) not in (2, 3):
        raise SystemExit("usage: python tests/golden/make_golden_gpu.py /path/to/reference [out.npz]")
    main(sys.argv[1], sys.argv[2] if len(sys.argv) == 3 else os.path.join(HERE, "ref_gpu.npz"))
