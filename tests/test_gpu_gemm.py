"""Block-scaled GEMM kernel against the PyTorch emulation (A.sa)(B.sb)^T of the oracle and the
reference's golden emulation output; tolerance atol = rtol = 1e-3 as in the reference's own check
(ours/block_scaled_matmul.py:440) on fp32 output."""
import os

import numpy as np
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _operands(M, N, K, mode, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, generator=g).to(torch.bfloat16)
    return a, b


def _quant_pair(a, b, mode):
    """Quantise with the oracle (CPU) so that the GEMM test does not depend on the CUDA quantizer."""
    if mode == "mxfp8":
        ac, asc = O.quant_mxfp8_side(a, 1.0)
        bc, bsc = O.quant_mxfp8_side(b, 1.0)
        return (ac, asc, "fp8e5"), (bc, bsc, "fp8e5"), ac, bc, 1.0
    if mode == "mxfp4":
        ac, asc = O.quant_mxfp4_side(a, 1.0)
        bc, bsc = O.quant_mxfp4_side(b, 1.0)
        return (ac, asc, "fp4"), (bc, bsc, "fp4"), O.pack_e2m1(ac), O.pack_e2m1(bc), 1.0
    ac, asc, ats = O.quant_nvfp4(a)
    bc, bsc, bts = O.quant_nvfp4(b)
    return (ac, asc, "nvfp4", ats), (bc, bsc, "nvfp4", bts), O.pack_e2m1(ac), O.pack_e2m1(bc), float(ats * bts)


@pytest.mark.parametrize("mode,M,N,K", [
    ("mxfp8", 128, 256, 128), ("mxfp8", 128, 256, 256), ("mxfp8", 256, 512, 1024), ("mxfp8", 200, 300, 384),
    ("mxfp4", 128, 256, 256), ("mxfp4", 256, 256, 1152), ("mxfp4", 130, 100, 128),
    ("nvfp4", 128, 256, 256), ("nvfp4", 256, 384, 832),
    # several tiles in both directions, ragged M and N, a K that ends inside a stage (MXFP4: 384 = 256 + 128)
    ("mxfp8", 512, 1000, 256), ("mxfp4", 300, 900, 384), ("mxfp8", 257, 225, 128), ("mxfp4", 640, 1120, 1024),
])
def test_gemm_matches_emulation(mode, M, N, K):
    import mpsa
    a, b = _operands(M, N, K, mode, seed=1)
    qa, qb, a_dev, b_dev, alpha = _quant_pair(a, b, mode)
    vec = 16 if mode == "nvfp4" else 32
    sa, sb = O.swizzle_scales(qa[1]), O.swizzle_scales(qb[1])
    ref = O.gemm_block_scaled(qa[0], qa[1], qb[0], qb[1], qa[2], qb[2], vec,
                              qa[3] if mode == "nvfp4" else None, qb[3] if mode == "nvfp4" else None)
    out = mpsa.gemm_block_scaled(a_dev.cuda(), sa.cuda(), b_dev.cuda(), sb.cuda(), torch.float32, M, N, K, mode,
                                 alpha=alpha, check=True)
    torch.testing.assert_close(out.cpu(), ref, atol=1e-3, rtol=1e-3)
    m = O.parity_metrics(out.cpu(), ref)
    assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2
    out16 = mpsa.gemm_block_scaled(a_dev.cuda(), sa.cuda(), b_dev.cuda(), sb.cuda(), torch.bfloat16, M, N, K, mode,
                                   alpha=alpha, check=True)
    torch.testing.assert_close(out16.float().cpu(), ref, atol=0.5, rtol=1e-2)


def test_reference_entry_points_and_golden():
    """initialize_block_scaled_from_tensor + block_scaled_matmul on the reference's own validation case
    (128x256x256, mxfp8) against the emulation output recorded from the reference."""
    from ours.block_scaled_matmul import block_scaled_matmul, initialize_block_scaled_from_tensor
    z = np.load(os.path.join(G, "gemm_emulation.npz"))
    torch.manual_seed(42)
    M, N, K = 128, 256, 256
    a_t = torch.randn((M, K), dtype=torch.float16)
    b_t = torch.randn((N, K), dtype=torch.float16)
    a_s, b_s = torch.from_numpy(z["a_scale_in"]), torch.from_numpy(z["b_scale_in"])
    a, sa, b, sb, cfg, (ref, _, _) = initialize_block_scaled_from_tensor(
        a_t.cuda(), b_t.cuda(), a_s.cuda(), b_s.cuda(), "mxfp8", compute_reference=True)
    assert np.array_equal(a.view(torch.uint8).cpu().numpy(), z["a_codes"])
    assert np.array_equal(sa.cpu().numpy(), z["a_scale_tiles"])
    torch.testing.assert_close(ref.cpu(), torch.from_numpy(z["reference"]), atol=1e-3, rtol=1e-3)
    out = block_scaled_matmul(a, sa, b, sb, torch.float32, M, N, K, cfg)
    torch.testing.assert_close(out.cpu(), torch.from_numpy(z["reference"]), atol=1e-3, rtol=1e-3)
    out16 = block_scaled_matmul(a, sa, b, sb, torch.float16, M, N, K, cfg)
    assert out16.dtype == torch.float16
    with pytest.raises(ValueError):
        block_scaled_matmul(a, sa, b, sb, torch.int32, M, N, K, cfg)


def test_quantizer_feeds_gemm_full_k():
    """CUDA quantizer output (codes + scale tiles) straight into the GEMM, K = 8192, linearity in alpha."""
    import mpsa
    M = N = 512
    K = 8192
    a, b = _operands(M, N, K, "mxfp8", seed=1)
    qa = mpsa.quantize_mx(a.cuda().reshape(1, 1, M, K), 1.0)
    qb = mpsa.quantize_mx(b.cuda().reshape(1, 1, N, K), 1.0)
    for mode, ca, cb, fa, fb in (("mxfp8", qa.fp8, qb.fp8, qa.fp8_sf, qb.fp8_sf), ("mxfp4", qa.fp4, qb.fp4, qa.fp4_sf, qb.fp4_sf)):
        out = mpsa.gemm_block_scaled(ca.reshape(M, -1), fa, cb.reshape(N, -1), fb, torch.float32, M, N, K, mode, check=True)
        out2 = mpsa.gemm_block_scaled(ca.reshape(M, -1), fa, cb.reshape(N, -1), fb, torch.float32, M, N, K, mode,
                                      alpha=2.0, check=True)
        assert torch.equal(out2, out * 2)
        if mode == "mxfp8":
            ac, asc = O.quant_mxfp8_side(a, 1.0)
            bc, bsc = O.quant_mxfp8_side(b, 1.0)
            ref = O.gemm_block_scaled(ac, asc, bc, bsc, "fp8e5", "fp8e5")
        else:
            ac, asc = O.quant_mxfp4_side(a, 1.0)
            bc, bsc = O.quant_mxfp4_side(b, 1.0)
            ref = O.gemm_block_scaled(ac, asc, bc, bsc, "fp4", "fp4")
        m = O.parity_metrics(out.cpu(), ref)
        assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2, m
        torch.testing.assert_close(out.cpu(), ref, atol=2e-2, rtol=1e-3)


@pytest.mark.parametrize("mode,M,N,K", [("mxfp8", 128, 256, 256), ("mxfp4", 200, 300, 256), ("mxfp8", 384, 130, 128)])
def test_batched_gemm_equals_per_problem_gemm(mode, M, N, K):
    """One batched launch over [B,H] problems (quantizer output fed straight in, ragged M and N included) gives
    bit for bit what the 2-D entry gives problem by problem."""
    import mpsa
    B, H = 2, 3
    g = torch.Generator().manual_seed(5)
    a = torch.randn(B, H, M, K, generator=g).to(torch.bfloat16).cuda()
    b = torch.randn(B, H, N, K, generator=g).to(torch.bfloat16).cuda()
    qa, qb = mpsa.quantize_mx(a, 1.0), mpsa.quantize_mx(b, 1.0)
    ca, cb, fa, fb = (qa.fp8, qb.fp8, qa.fp8_sf, qb.fp8_sf) if mode == "mxfp8" else (qa.fp4, qb.fp4, qa.fp4_sf, qb.fp4_sf)
    out = mpsa.gemm_block_scaled_batched(ca, fa, cb, fb, torch.float32, M, N, K, mode, check=True)
    assert tuple(out.shape) == (B, H, M, N)
    for i in range(B):
        for j in range(H):
            one = mpsa.gemm_block_scaled(ca[i, j], fa[i, j], cb[i, j], fb[i, j], torch.float32, M, N, K, mode, check=True)
            assert torch.equal(out[i, j], one)


def test_batched_reference_entry_points():
    """initialize_block_scaled_batched_from_tensor + block_scaled_batched_matmul (the reference's batched module)
    against the emulation (A*sa) @ (B*sb)^T, tolerance of the reference's own GEMM check (1e-3, 1e-3)."""
    from ours.batched_block_scaled_matmul import block_scaled_batched_matmul, initialize_block_scaled_batched_from_tensor
    torch.manual_seed(7)
    B, H, M, N, K = 2, 2, 128, 256, 256
    for kind in ("mxfp8", "mxfp4"):
        a_t = torch.randn((B, H, M, K), dtype=torch.float16, device="cuda")
        b_t = torch.randn((B, H, N, K), dtype=torch.float16, device="cuda")
        a_s = torch.rand((B, H, M // 128, K // 32 // 4, 32, 4, 4), device="cuda") + 1e-8
        b_s = torch.rand((B, H, N // 128, K // 32 // 4, 32, 4, 4), device="cuda") + 1e-8
        a, sa, b, sb, cfg, (ref, _, _) = initialize_block_scaled_batched_from_tensor(a_t, b_t, a_s, b_s, kind, compute_reference=True)
        out = block_scaled_batched_matmul(a, sa, b, sb, torch.float32, B, H, M, N, K, cfg)
        torch.testing.assert_close(out, ref, atol=1e-3, rtol=1e-3)
