"""Batched block-scaled matmul with the entry points of ours/batched_block_scaled_matmul.py of the reference:
initialize_block_scaled_batched_from_tensor (:239-367) and block_scaled_batched_matmul (:183-236).  All B*H
problems run in one launch of the tcgen05 GEMM kernel."""
import torch

from mpsa import ops as _ops
from .mxfp import MXFP4Tensor, MXScaleTensor

_MODE_OF = {(1, 1, 32): "mxfp8", (2, 2, 32): "mxfp4", (2, 2, 16): "nvfp4"}


def block_scaled_batched_matmul(a_desc, a_scale, b_desc, b_scale, dtype_dst, B, H, M, N, K, configs):
    """a [B,H,M,K/epb], b [B,H,N,K/epb] (K-major both), scales [B,H,rows/128,K/VEC/4,32,4,4] -> C [B,H,M,N];
    dtype_dst in {float32, float16, bfloat16, float8_e5m2}."""
    if dtype_dst not in (torch.float32, torch.float16, torch.bfloat16, torch.float8_e5m2):
        raise ValueError(f"Unsupported dtype: {dtype_dst}")
    key = (configs["ELEM_PER_BYTE_A"], configs["ELEM_PER_BYTE_B"], configs["VEC_SIZE"])
    if key not in _MODE_OF:
        raise ValueError("mixed fp8 x fp4 operands are not supported by this kernel")
    elem = {torch.float8_e4m3fn: "e4m3"}.get(a_desc.dtype, "e5m2")
    belem = {torch.float8_e4m3fn: "e4m3"}.get(b_desc.dtype, "e5m2")
    return _ops.gemm_block_scaled_batched(a_desc, a_scale, b_desc, b_scale, dtype_dst, M, N, K, _MODE_OF[key],
                                          a_elem=elem, b_elem=belem, alpha=float(configs.get("alpha", 1.0)))


def initialize_block_scaled_batched_from_tensor(a_tensor, b_tensor, a_scale, b_scale, block_scale_type="nvfp4",
                                                compute_reference=False):
    """Pack operands [B,H,M,K] / [B,H,N,K] and scale tiles [B,H,rows/128,K/VEC/4,32,4,4] for the kernel.  fp8
    operands are cast to E5M2 (already-fp8 tensors pass through), fp4 operands are E2M1 codes (uint8, one per
    byte) or floats, rounded to nearest even and packed two per byte ALONG K; scales become E8M0 codes (E4M3
    for nvfp4; uint8 codes pass through).  With compute_reference the emulation (A*sa) @ (B*sb)^T is returned as
    well.  Two defects of the reference are not reproduced: it packs fp4 pairs along the head axis (dim=1) and
    its emulation divides by the raw scale codes (ours/batched_block_scaled_matmul.py:288, :352)."""
    B, H, M, K = a_tensor.shape
    B_b, H_b, N, K_b = b_tensor.shape
    assert B == B_b and H == H_b and K == K_b, "A and B need the same batch, heads and K"
    assert block_scale_type in ["nvfp4", "mxfp4", "mxfp8", "mixed"], f"Invalid block scale type: {block_scale_type}"
    if block_scale_type == "mixed":
        raise ValueError("mixed fp8 x fp4 operands are not supported by this kernel")
    VEC_SIZE = 16 if block_scale_type == "nvfp4" else 32
    fp4 = "fp4" in block_scale_type
    expected_a = (B, H, M // 128, K // VEC_SIZE // 4, 32, 4, 4)
    expected_b = (B, H, N // 128, K // VEC_SIZE // 4, 32, 4, 4)
    assert tuple(a_scale.shape) == expected_a, f"a_scale shape {tuple(a_scale.shape)} != {expected_a}"
    assert tuple(b_scale.shape) == expected_b, f"b_scale shape {tuple(b_scale.shape)} != {expected_b}"

    def pack(t):
        if not fp4:
            q = t if t.dtype in (torch.float8_e5m2, torch.float8_e4m3fn) else t.to(torch.float8_e5m2)
            return q, q.to(torch.float32)
        m = MXFP4Tensor(data=t, dtype=torch.uint8) if t.dtype == torch.uint8 else MXFP4Tensor(data=t.to(torch.float32))
        return m.to_packed_tensor(dim=3), m.to(torch.float32)

    a, a_ref = pack(a_tensor)
    b, b_ref = pack(b_tensor)
    if a_scale.dtype == torch.uint8:
        sa, sb = a_scale, b_scale
        sa_ref, sb_ref = _e8m0_to_float(sa), _e8m0_to_float(sb)
    elif block_scale_type == "nvfp4":
        sa8, sb8 = a_scale.to(torch.float8_e4m3fn), b_scale.to(torch.float8_e4m3fn)
        sa_ref, sb_ref = sa8.to(torch.float32), sb8.to(torch.float32)
        sa, sb = sa8.view(torch.uint8), sb8.view(torch.uint8)
    else:
        ma, mb = MXScaleTensor(a_scale.to(torch.float32)), MXScaleTensor(b_scale.to(torch.float32))
        sa, sb = ma.data, mb.data
        sa_ref, sb_ref = ma.to(torch.float32), mb.to(torch.float32)
    configs = {
        "BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 256 if fp4 else 128, "num_stages": 2,
        "ELEM_PER_BYTE_A": 2 if fp4 else 1, "ELEM_PER_BYTE_B": 2 if fp4 else 1, "VEC_SIZE": VEC_SIZE,
    }
    if not compute_reference:
        return a, sa, b, sb, configs, None

    def unpack_scale(t):                            # [B,H,nm,nk,32,4,4] -> [B,H,nm*128,nk*4]
        nm, nk = t.shape[2], t.shape[3]
        return t.permute(0, 1, 2, 5, 4, 3, 6).reshape(B, H, nm * 128, nk * 4)

    ea = unpack_scale(sa_ref).repeat_interleave(VEC_SIZE, dim=3)[:, :, :M, :K]
    eb = unpack_scale(sb_ref).repeat_interleave(VEC_SIZE, dim=3)[:, :, :N, :K]
    reference = torch.matmul(a_ref * ea, (b_ref * eb).transpose(-1, -2))
    return a, sa, b, sb, configs, (reference, a_ref * ea, b_ref * eb)


def _e8m0_to_float(codes):
    t = MXScaleTensor(size=tuple(codes.shape), device=codes.device)
    t.data = codes
    return t.to(torch.float32)
