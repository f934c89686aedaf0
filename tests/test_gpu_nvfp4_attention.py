"""NVFP4 score tiles in the fused forward (the video-DiT configuration: NVFP4 off the diagonal, MXFP8 on it).

The reference has no NVFP4 path, so the oracle restates the format definition (parity unpinned): quantizer codes,
block scales and the tensor scale must be bit-exact against it, the attention output within cosine >= 0.9999 and
relative L2 <= 1e-2."""
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
COS_MIN, REL_L2_MAX = 0.9999, 1e-2


@pytest.mark.parametrize("shape", [(1, 2, 300, 128), (2, 3, 256, 128), (1, 1, 128, 64)])
def test_batched_nvfp4_quantizer(shape):
    import mpsa
    g = torch.Generator().manual_seed(31)
    x = (torch.randn(*shape, generator=g) * 2).to(torch.bfloat16)
    x[0, 0, 7, 16:32] = 0
    codes, scales, ts = mpsa.quantize_nvfp4_bh(x.cuda(), 0.125)
    oc, osc, ots = O.quant_nvfp4(x, 0.125)
    assert float(ts.cpu()) == float(ots)
    assert torch.equal(codes.cpu(), O.pack_e2m1(oc))
    exp = O.swizzle_scales(osc, pad_code=0)              # [B,H,nt,D/64,32,4,4]
    assert torch.equal(scales.cpu().reshape(exp.shape), exp)


def _run(q, k, v, causal, **kw):
    import mpsa
    return mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=causal, out_dtype=torch.float32, check=True,
                                  fp4_kind="nvfp4", **kw).cpu()


def _check(out, ref, what):
    m = O.parity_metrics(out, ref)
    assert m["cos"] >= COS_MIN and m["rel_l2"] <= REL_L2_MAX, (what, m)


@pytest.mark.parametrize("pv_mode", ["fp16", "requant"])
@pytest.mark.parametrize("causal", [False, True])
def test_nvfp4_tiles(pv_mode, causal):
    q, k, v = O.make_qkv(41, 1, 4, 2, 640, 128, outliers=3)
    for uniform in ("fp4", None):
        ref = O.attention_mxfp(q, k, v, causal=causal, uniform=uniform, pv_mode=pv_mode, fp4_kind="nvfp4")
        _check(_run(q, k, v, causal, uniform=uniform, pv_mode=pv_mode), ref, (pv_mode, causal, uniform))


def test_nvfp4_ragged_and_d64():
    q, k, v = O.make_qkv(42, 1, 2, 2, 330, 64)
    ref = O.attention_mxfp(q, k, v, causal=False, fp4_kind="nvfp4")
    _check(_run(q, k, v, False), ref, "ragged d64")


def test_video_shaped_small():
    """The Wan-like configuration at a small grid: non-causal, 6 x 13 x 20 = 1560 tokens (not a multiple of 128),
    low-frequency component added, NVFP4 off-diagonal / MXFP8 diagonal."""
    q, k, v = O.make_video_qkv(3, 4, (6, 13, 20), 128)
    ref = O.attention_mxfp(q, k, v, causal=False, fp4_kind="nvfp4")
    out = _run(q, k, v, False)
    _check(out, ref, "video")
    print("vs fp32 attention:", O.parity_metrics(out, O.attention_fp32(q, k, v, False)))
