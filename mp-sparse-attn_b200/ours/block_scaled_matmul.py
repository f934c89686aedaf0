"""Standalone block-scaled GEMM with the entry points of ours/block_scaled_matmul.py of the
reference: initialize_block_scaled_from_tensor (:299-406), block_scaled_matmul (:271-296),
validate_block_scaled_from_tensor (:409-441).  The matmul itself is one tcgen05 kernel launch."""
import torch

from mpsa import ops as _ops
from .mxfp import MXFP4Tensor, MXScaleTensor

_MODE_OF = {(1, 1, 32): "mxfp8", (2, 2, 32): "mxfp4", (2, 2, 16): "nvfp4"}


def supports_block_scaling():
    return torch.cuda.is_available() and torch.cuda.get_device_capability()[0] == 10


def block_scaled_matmul(a_desc, a_scale, b_desc, b_scale, dtype_dst, M, N, K, configs):
    """C[M,N] from packed operands a [M,K/epb], b [N,K/epb] and 5-D scale tiles; dtype_dst in
    {float32, float16, bfloat16, float8_e5m2}."""
    if dtype_dst not in (torch.float32, torch.float16, torch.bfloat16, torch.float8_e5m2):
        raise ValueError(f"Unsupported dtype: {dtype_dst}")
    key = (configs["ELEM_PER_BYTE_A"], configs["ELEM_PER_BYTE_B"], configs["VEC_SIZE"])
    if key not in _MODE_OF:
        raise ValueError("mixed fp8 x fp4 operands are not supported by this kernel")
    mode = _MODE_OF[key]
    elem = {torch.float8_e4m3fn: "e4m3"}.get(a_desc.dtype, "e5m2")
    belem = {torch.float8_e4m3fn: "e4m3"}.get(b_desc.dtype, "e5m2")
    return _ops.gemm_block_scaled(a_desc, a_scale, b_desc, b_scale, dtype_dst, M, N, K, mode,
                                  a_elem=elem, b_elem=belem, alpha=float(configs.get("alpha", 1.0)))


def initialize_block_scaled_from_tensor(a_tensor, b_tensor, a_scale, b_scale, block_scale_type="nvfp4",
                                        compute_reference=False):
    """Pack float operands [M,K] / [N,K] and float scale tiles [rows/128, K/VEC/4, 32,4,4] for the
    kernel: fp8 by cast, fp4 by round-to-nearest-even + 2-per-byte packing along K, scales to
    E8M0 (E4M3 for nvfp4).  With compute_reference the PyTorch emulation (A.sa)@(B.sb)^T is
    returned as well."""
    M, K = a_tensor.shape
    N, K_b = b_tensor.shape
    assert K == K_b, f"K mismatch: A.shape[1]={K} != B.shape[1]={K_b}"
    assert block_scale_type in ["nvfp4", "mxfp4", "mxfp8", "mixed"], f"Invalid block scale type: {block_scale_type}"
    if block_scale_type == "mixed":
        raise ValueError("mixed fp8 x fp4 operands are not supported by this kernel")
    VEC_SIZE = 16 if block_scale_type == "nvfp4" else 32
    fp4 = "fp4" in block_scale_type
    expected_a = (M // 128, K // VEC_SIZE // 4, 32, 4, 4)
    expected_b = (N // 128, K // VEC_SIZE // 4, 32, 4, 4)
    assert tuple(a_scale.shape) == expected_a, f"a_scale shape {tuple(a_scale.shape)} != {expected_a}"
    assert tuple(b_scale.shape) == expected_b, f"b_scale shape {tuple(b_scale.shape)} != {expected_b}"

    def pack(t):
        if not fp4:
            q = t.to(torch.float8_e5m2)
            return q, q.to(torch.float32)
        if t.dtype == torch.uint8:
            m = MXFP4Tensor(data=t, dtype=torch.uint8)
        else:
            m = MXFP4Tensor(data=t.to(torch.float32))
        return m.to_packed_tensor(dim=1), m.to(torch.float32)

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
        "BLOCK_SIZE_M": 128, "BLOCK_SIZE_N": 256, "BLOCK_SIZE_K": 256 if fp4 else 128, "num_stages": 4,
        "ELEM_PER_BYTE_A": 2 if fp4 else 1, "ELEM_PER_BYTE_B": 2 if fp4 else 1, "VEC_SIZE": VEC_SIZE,
    }
    if not compute_reference:
        return a, sa, b, sb, configs, None

    def unpack_scale(t):
        nm, nk = t.shape[0], t.shape[1]
        return t.permute(0, 3, 2, 1, 4).reshape(nm * 128, nk * 4)

    ea = unpack_scale(sa_ref).repeat_interleave(VEC_SIZE, dim=1)[:M, :K]
    eb = unpack_scale(sb_ref).repeat_interleave(VEC_SIZE, dim=1)[:N, :K]
    reference = torch.matmul(a_ref * ea, (b_ref * eb).T)
    return a, sa, b, sb, configs, (reference, a_ref * ea, b_ref * eb)


def _e8m0_to_float(codes):
    t = MXScaleTensor(size=tuple(codes.shape), device=codes.device)
    t.data = codes
    return t.to(torch.float32)


def validate_block_scaled_from_tensor(M, N, K, block_scale_type="nvfp4"):
    device = "cuda"
    VEC_SIZE = 16 if block_scale_type == "nvfp4" else 32
    a_tensor = torch.randn((M, K), dtype=torch.float16, device=device)
    b_tensor = torch.randn((N, K), dtype=torch.float16, device=device)
    a_s = torch.rand((M // 128, K // VEC_SIZE // 4, 32, 4, 4), device=device) + 1e-8
    b_s = torch.rand((N // 128, K // VEC_SIZE // 4, 32, 4, 4), device=device) + 1e-8
    a, sa, b, sb, configs, (reference, _, _) = initialize_block_scaled_from_tensor(
        a_tensor, b_tensor, a_s, b_s, block_scale_type, compute_reference=True)
    output = block_scaled_matmul(a, sa, b, sb, torch.float16, M, N, K, configs)
    torch.testing.assert_close(reference, output.to(torch.float32), atol=1e-3, rtol=1e-3)
    return output
