"""Block quantizers with the signatures of ours/quant_mxint8.py of the reference
(quant_fpxint8 :61, quant_fpxint8_warp :116, quant_mxfp8e5 :223, quant_mxfp4 :453), running as one
hand-written CUDA kernel launch per operand."""
import torch

from mpsa import ops as _ops


def _sides(q, k, sm_scale, tensor_layout):
    if tensor_layout not in ("HND", "NHD"):
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    head_dim = q.shape[-1]
    return _ops.q_side_scale(head_dim, sm_scale), 1.0


def quant_mxfp4(q, k, BLKQ=128, BLKK=64, sm_scale=None, tensor_layout="HND"):
    """-> (q codes uint8 one E2M1 code per byte, q E8M0 scales [b,h,len,D/32], k codes, k scales)."""
    sq, sk = _sides(q, k, sm_scale, tensor_layout)
    a = _ops.quantize_mx(q, sq, want_fp8=False, reference_format=True, kernel_format=False, tensor_layout=tensor_layout)
    b = _ops.quantize_mx(k, sk, want_fp8=False, reference_format=True, kernel_format=False, tensor_layout=tensor_layout)
    return a.fp4_unpacked, a.fp4_scales, b.fp4_unpacked, b.fp4_scales


def quant_mxfp8e5(q, k, BLKQ=128, BLKK=64, sm_scale=None, tensor_layout="HND"):
    """-> (q float8_e5m2, q E8M0 scales, k float8_e5m2, k scales)."""
    sq, sk = _sides(q, k, sm_scale, tensor_layout)
    a = _ops.quantize_mx(q, sq, want_fp4=False, reference_format=True, kernel_format=False, tensor_layout=tensor_layout)
    b = _ops.quantize_mx(k, sk, want_fp4=False, reference_format=True, kernel_format=False, tensor_layout=tensor_layout)
    return a.fp8.view(torch.float8_e5m2), a.fp8_scales, b.fp8.view(torch.float8_e5m2), b.fp8_scales


def quant_mxfp8e4(q, k, BLKQ=128, BLKK=64, sm_scale=None, tensor_layout="HND"):
    """E4M3 variant (emax 8, clamp 448); the reference has no such quantizer."""
    sq, sk = _sides(q, k, sm_scale, tensor_layout)
    a = _ops.quantize_mx(q, sq, want_fp4=False, reference_format=True, kernel_format=False, fp8_elem="e4m3",
                         tensor_layout=tensor_layout)
    b = _ops.quantize_mx(k, sk, want_fp4=False, reference_format=True, kernel_format=False, fp8_elem="e4m3",
                         tensor_layout=tensor_layout)
    return a.fp8.view(torch.float8_e4m3fn), a.fp8_scales, b.fp8.view(torch.float8_e4m3fn), b.fp8_scales


def quant_fpxint8(q, k, BLKQ=128, BLKK=64, sm_scale=None, tensor_layout="HND"):
    """-> (q int8, q fp32 scales [b,h,len,D/32], k int8, k scales)."""
    sq, sk = _sides(q, k, sm_scale, tensor_layout)
    qc, qs = _ops.quantize_int8(q, sq, tensor_layout)
    kc, ks = _ops.quantize_int8(k, sk, tensor_layout)
    return qc, qs, kc, ks


def quant_fpxint8_warp(q, k, BLKQ=128, WARPQ=32, BLKK=64, WARPK=64, tensor_layout="HND"):
    """Same per-32 quantizer with no softmax scale folded into Q (the reference passes 1.0 for both
    sides here, ours/quant_mxint8.py:148, :158).  Scales are returned in the per-32 shape
    [b,h,len,D/32] that the kernel actually produces."""
    if tensor_layout not in ("HND", "NHD"):
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    qc, qs = _ops.quantize_int8(q, 1.0, tensor_layout)
    kc, ks = _ops.quantize_int8(k, 1.0, tensor_layout)
    return qc, qs, kc, ks
