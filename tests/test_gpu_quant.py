"""CUDA quantizers (through the C-ABI) against the golden vectors and the CPU oracle: bit-exact
codes and scale codes, both the reference output format and the kernel format."""
import os

import numpy as np
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
G = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _gold():
    return np.load(os.path.join(G, "quant_kat.npz"))


@pytest.mark.parametrize("tag", ["kat", "d128", "d64"])
def test_reference_signatures_match_golden(tag):
    from ours.quant_mxint8 import quant_mxfp4, quant_mxfp8e5, quant_fpxint8
    z = _gold()
    if tag == "kat":
        q = k = torch.from_numpy(z["kat_x"]).view(torch.bfloat16)
    else:
        q = torch.from_numpy(z[f"{tag}_q"]).view(torch.bfloat16)
        k = torch.from_numpy(z[f"{tag}_k"]).view(torch.bfloat16)
    qd, kd = q.cuda(), k.cuda()
    a, sa, b, sb = quant_mxfp4(qd, kd)
    assert a.dtype == torch.uint8 and a.shape == q.shape and sa.shape == q.shape[:-1] + (q.shape[-1] // 32,)
    assert np.array_equal(a.cpu().numpy(), z[f"{tag}_fp4_q"]) and np.array_equal(sa.cpu().numpy(), z[f"{tag}_fp4_qs"])
    assert np.array_equal(b.cpu().numpy(), z[f"{tag}_fp4_k"]) and np.array_equal(sb.cpu().numpy(), z[f"{tag}_fp4_ks"])
    a, sa, b, sb = quant_mxfp8e5(qd, kd)
    assert a.dtype == torch.float8_e5m2
    assert np.array_equal(sa.cpu().numpy(), z[f"{tag}_fp8_qs"]) and np.array_equal(sb.cpu().numpy(), z[f"{tag}_fp8_ks"])
    oq, _, ok, _ = O.quant_mxfp8e5(q, k)
    assert torch.equal(a.view(torch.uint8).cpu(), oq) and torch.equal(b.view(torch.uint8).cpu(), ok)
    a, sa, b, sb = quant_fpxint8(qd, kd)
    assert np.array_equal(a.cpu().numpy(), z[f"{tag}_i8_q"]) and np.array_equal(b.cpu().numpy(), z[f"{tag}_i8_k"])
    oa, osa, ob, osb = O.quant_fpxint8(q, k)
    assert torch.equal(sa.cpu(), osa) and torch.equal(sb.cpu(), osb)


@pytest.mark.parametrize("shape,dtype,outliers", [
    ((1, 2, 256, 128), torch.bfloat16, 5),
    ((2, 3, 200, 128), torch.float16, 0),      # ragged: L not a multiple of 128
    ((1, 1, 77, 64), torch.bfloat16, 3),       # D = 64, short
    ((1, 2, 130, 256), torch.float32, 0),      # D = 256 (two scale-tile columns)
])
def test_kernel_format_matches_oracle(shape, dtype, outliers):
    import mpsa
    g = torch.Generator().manual_seed(5)
    x = torch.randn(shape, generator=g)
    if outliers:
        x[..., torch.randperm(shape[-1], generator=g)[:outliers]] *= 20
    x = x.to(dtype)
    x[0, 0, 3, :32] = 0          # an all-zero block
    s = O.q_side_scale(shape[-1])
    r = mpsa.quantize_mx(x.cuda(), s, reference_format=True, kernel_format=True)
    c4, s4 = O.quant_mxfp4_side(x, s)
    c8, s8 = O.quant_mxfp8_side(x, s)
    assert torch.equal(r.fp4_unpacked.cpu(), c4) and torch.equal(r.fp4_scales.cpu(), s4)
    assert torch.equal(r.fp8.cpu(), c8) and torch.equal(r.fp8_scales.cpu(), s8)
    assert torch.equal(r.fp4.cpu(), O.pack_e2m1(c4))
    assert torch.equal(r.fp4_sf.cpu().reshape(O.swizzle_scales(s4).shape), O.swizzle_scales(s4))
    assert torch.equal(r.fp8_sf.cpu().reshape(O.swizzle_scales(s8).shape), O.swizzle_scales(s8))
    # E4M3 variant (no reference counterpart: checked against the oracle's restatement only)
    r = mpsa.quantize_mx(x.cuda(), s, want_fp4=False, reference_format=True, kernel_format=False, fp8_elem="e4m3")
    c8, s8 = O.quant_mxfp8_side(x, s, "e4m3")
    assert torch.equal(r.fp8.cpu(), c8) and torch.equal(r.fp8_scales.cpu(), s8)


def test_nhd_layout_and_strided_input():
    from ours.quant_mxint8 import quant_mxfp4
    g = torch.Generator().manual_seed(9)
    q = torch.randn(2, 192, 4, 128, generator=g).to(torch.bfloat16)   # [B, L, H, D]
    k = torch.randn(2, 192, 2, 128, generator=g).to(torch.bfloat16)
    a, sa, b, sb = quant_mxfp4(q.cuda(), k.cuda(), tensor_layout="NHD")
    assert a.shape == q.shape and sa.shape == (2, 4, 192, 4)
    oa, osa, ob, osb = O.quant_mxfp4(q.transpose(1, 2), k.transpose(1, 2))
    assert torch.equal(a.cpu().transpose(1, 2), oa) and torch.equal(sa.cpu(), osa)
    assert torch.equal(b.cpu().transpose(1, 2), ob) and torch.equal(sb.cpu(), osb)
    with pytest.raises(ValueError):
        quant_mxfp4(q.cuda(), k.cuda(), tensor_layout="XYZ")


def test_full_size_properties():
    """Headline-size Q operand (32 heads x 32768 x 128): properties that need no oracle pass."""
    import mpsa
    g = torch.Generator(device="cuda").manual_seed(2)
    x = torch.randn(1, 32, 32768, 128, generator=g, device="cuda").to(torch.bfloat16)
    r = mpsa.quantize_mx(x, 1.0, reference_format=True, kernel_format=True)
    # scale code == exponent of the block amax - emax + 127 (bf16 input: no rounding edge)
    amax = x.float().abs().reshape(1, 32, 32768, 4, 32).amax(-1)
    e = torch.floor(torch.log2(amax)).to(torch.int32)
    assert torch.equal(r.fp4_scales.to(torch.int32), e - 3 + 127)
    assert torch.equal(r.fp8_scales.to(torch.int32), e - 7 + 127)
    # every block's largest element saturates to +-6 and no code is a NaN pattern
    mag = (r.fp4_unpacked & 7).reshape(1, 32, 32768, 4, 32).amax(-1)
    assert int(mag.min()) == 7
    # packed nibbles reproduce the unpacked codes
    lo, hi = r.fp4 & 0xF, r.fp4 >> 4
    assert torch.equal(torch.stack((lo, hi), -1).flatten(-2), r.fp4_unpacked)
    # dequantised fp8 is within half an E5M2 ulp (2^-3 relative) of the input
    deq = r.fp8.view(torch.float8_e5m2).float() * torch.exp2(r.fp8_scales.float() - 127).repeat_interleave(32, -1)
    err = (deq - x.float()).abs()
    assert float((err / amax.repeat_interleave(32, -1)).max()) <= 2.0 ** -3
    # a 2048-row slice against the oracle, bit exact
    c4, s4 = O.quant_mxfp4_side(x[0, 7, 4096:6144].cpu(), 1.0)
    assert torch.equal(r.fp4_unpacked[0, 7, 4096:6144].cpu(), c4) and torch.equal(r.fp4_scales[0, 7, 4096:6144].cpu(), s4)


@pytest.mark.parametrize("rows,cols,dtype", [(256, 512, torch.bfloat16), (200, 320, torch.float16), (130, 1024, torch.float32)])
def test_nvfp4_quantizer_matches_oracle(rows, cols, dtype):
    """No reference counterpart (parity unpinned): checked against the oracle's restatement of the format."""
    import mpsa
    g = torch.Generator().manual_seed(21)
    x = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
    x[5, 16:32] = 0
    codes, scales, ts = mpsa.quantize_nvfp4(x.cuda())
    oc, osc, ots = O.quant_nvfp4(x)
    assert float(ts.cpu()) == float(ots)
    assert torch.equal(codes.cpu(), O.pack_e2m1(oc))
    assert torch.equal(scales.cpu().reshape(O.swizzle_scales(osc, pad_code=0).shape), O.swizzle_scales(osc, pad_code=0))
    # and straight into the GEMM
    y = (torch.randn(256, cols, generator=g)).to(dtype)
    if cols % 64 == 0 and rows % 1 == 0:
        cy, sy, tsy = mpsa.quantize_nvfp4(y.cuda())
        out = mpsa.gemm_block_scaled(codes, scales, cy, sy, torch.float32, rows, 256, cols, "nvfp4",
                                     alpha=float(ts.cpu()) * float(tsy.cpu()), check=True)
        yc, ysc, yts = O.quant_nvfp4(y)
        ref = O.gemm_block_scaled(oc, osc, yc, ysc, "nvfp4", "nvfp4", 16, ots, yts)
        m = O.parity_metrics(out.cpu(), ref)
        assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2, m


@pytest.mark.parametrize("shape,dtype", [((1, 2, 1300, 128), torch.bfloat16), ((2, 1, 700, 64), torch.float16),
                                         ((1, 1, 513, 128), torch.float32)])
def test_smooth_k_inside_the_quantizer(shape, dtype):
    """The reference's smooth_k is k - k.mean(dim=-2, keepdim=True) ahead of the quantizer
    (ours/mxfp_attn_kernel.py:33-34).  (1) column_mean is the fp32 mean rounded to the input dtype: within one unit in
    the last place of the float64 mean.  (2) Given that mean, the centred quantizer is bit-exact against the oracle
    quantizing the difference that torch's elementwise subtraction leaves (rounded to the input dtype)."""
    import mpsa
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(shape, generator=g) + 0.7 * torch.randn(shape[0], shape[1], 1, shape[3], generator=g)).to(dtype)
    mean = mpsa.column_mean(x.cuda()).cpu()
    assert mean.dtype == torch.float32 and tuple(mean.shape) == (shape[0], shape[1], shape[3])
    assert torch.equal(mean.to(dtype).float(), mean)                       # representable in the input dtype
    ref = x.double().mean(dim=-2)
    ulp = {torch.bfloat16: 2.0 ** -8, torch.float16: 2.0 ** -11, torch.float32: 2.0 ** -22}[dtype]
    assert ((mean.double() - ref).abs() <= ulp * ref.abs() + 1e-6).all()
    xc = (x.float() - mean.unsqueeze(2)).to(dtype)                         # what `k - km` holds, given this km
    r = mpsa.quantize_mx(x.cuda(), 1.0, reference_format=True, kernel_format=True, center=mean.cuda())
    c4, s4 = O.quant_mxfp4_side(xc, 1.0)
    c8, s8 = O.quant_mxfp8_side(xc, 1.0)
    assert torch.equal(r.fp4_unpacked.cpu(), c4) and torch.equal(r.fp4_scales.cpu(), s4)
    assert torch.equal(r.fp8.cpu(), c8) and torch.equal(r.fp8_scales.cpu(), s8)
    assert torch.equal(r.fp4.cpu(), O.pack_e2m1(c4))
    assert torch.equal(r.fp4_sf.cpu().reshape(O.swizzle_scales(s4).shape), O.swizzle_scales(s4))


@pytest.mark.parametrize("shape,dtype,batched", [((1, 2, 300, 128), torch.bfloat16, False), ((2, 2, 130, 64), torch.float16, True),
                                                 ((1, 1, 128, 128), torch.float32, False)])
def test_rotary_embedding_inside_the_quantizer(shape, dtype, batched):
    """quantize_mx(x, rope=(cos, sin)) is bit-exact against the oracle quantizing the rotated tensor (rotate-half
    convention, fp32 arithmetic without fused multiply-add, result rounded to the input dtype)."""
    import mpsa
    B, H, L, D = shape
    g = torch.Generator().manual_seed(12)
    x = torch.randn(shape, generator=g).to(dtype)
    x[0, 0, 5, :32] = 0
    if batched:                                  # per-batch positions
        cs = [O.rope_angles(L, D, offset=17 * b) for b in range(B)]
        cos, sin = torch.stack([c for c, _ in cs]), torch.stack([s_ for _, s_ in cs])
    else:
        cos, sin = O.rope_angles(L, D)
    s = O.q_side_scale(D)
    xr = O.rope_rotate_half(x, cos, sin)
    r = mpsa.quantize_mx(x.cuda(), s, reference_format=True, kernel_format=True, rope=(cos.cuda(), sin.cuda()))
    c4, s4 = O.quant_mxfp4_side(xr, s)
    c8, s8 = O.quant_mxfp8_side(xr, s)
    assert torch.equal(r.fp4_unpacked.cpu(), c4) and torch.equal(r.fp4_scales.cpu(), s4)
    assert torch.equal(r.fp8.cpu(), c8) and torch.equal(r.fp8_scales.cpu(), s8)
    assert torch.equal(r.fp4.cpu(), O.pack_e2m1(c4))
    assert torch.equal(r.fp4_sf.cpu().reshape(O.swizzle_scales(s4).shape), O.swizzle_scales(s4))
    assert torch.equal(r.fp8_sf.cpu().reshape(O.swizzle_scales(s8).shape), O.swizzle_scales(s8))


@pytest.mark.parametrize("shape,dtype", [
    ((1, 2, 1000, 128), torch.bfloat16),       # 7.8 tiles: the last CTA's second and third tile are ragged / absent
    ((2, 3, 384, 128), torch.float16),         # exactly one CTA of three tiles per head
    ((1, 1, 77, 64), torch.bfloat16),          # D = 64, short
    ((1, 2, 130, 256), torch.bfloat16),        # D = 256 (two scale-tile columns)
])
@pytest.mark.parametrize("s", [1.0, 0.1275])
def test_mxfp8_only_kernel_matches_oracle(shape, dtype, s):
    """The MXFP8-only kernel (block maximum on the packed 16-bit patterns, three tiles per CTA) against the oracle, in all
    three of its outputs, and on a strided (NHD) view."""
    import mpsa
    g = torch.Generator().manual_seed(11)
    x = (torch.randn(shape, generator=g) * 3).to(dtype)
    x[0, 0, 5, 32:64] = 0                        # an all-zero block
    x[0, 0, 6, 0] = -0.0
    r = mpsa.quantize_mx(x.cuda(), s, want_fp4=False, reference_format=True, kernel_format=True)
    c8, s8 = O.quant_mxfp8_side(x, s)
    assert torch.equal(r.fp8.cpu(), c8) and torch.equal(r.fp8_scales.cpu(), s8)
    assert torch.equal(r.fp8_sf.cpu().reshape(O.swizzle_scales(s8).shape), O.swizzle_scales(s8))
    both = mpsa.quantize_mx(x.cuda(), s, reference_format=True, kernel_format=True)     # the general kernel
    assert torch.equal(r.fp8, both.fp8) and torch.equal(r.fp8_scales, both.fp8_scales) and torch.equal(r.fp8_sf, both.fp8_sf)
    xt = x.transpose(1, 2).contiguous().cuda()   # [B, L, H, D] storage
    rt = mpsa.quantize_mx(xt, s, want_fp4=False, reference_format=True, kernel_format=False, tensor_layout="NHD")
    assert torch.equal(rt.fp8.cpu().transpose(1, 2), c8) and torch.equal(rt.fp8_scales.cpu(), s8)


@pytest.mark.parametrize("shape", [(1, 2, 640, 128), (2, 1, 300, 128), (1, 2, 200, 64)])
def test_v_quantizer_vector_and_scalar_kernels_agree(shape):
    """16-bit aligned input takes the kernel with 16-byte loads, fp32 input the scalar one: same arithmetic, same bytes
    (the fp32 tensor holds the bf16 values exactly)."""
    import mpsa
    g = torch.Generator().manual_seed(12)
    v = (torch.randn(shape, generator=g) * 2).to(torch.bfloat16)
    v[0, 0, 40:72, 3] = 0                        # an all-zero 32-key block of one head-dim index
    a = mpsa.quantize_v_seq(v.cuda())
    b = mpsa.quantize_v_seq(v.float().cuda())
    assert torch.equal(a.vt8, b.vt8) and torch.equal(a.vt4, b.vt4)
    assert torch.equal(a.v8_sf, b.v8_sf) and torch.equal(a.v4_sf, b.v4_sf)
