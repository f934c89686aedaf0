"""The forward with the online router inside it (attention_forward_routed: no stand-alone statistic pass) against the
stand-alone form (router_statistic -> precision_map_online -> attention_forward_quantized) and against the CPU oracle:
the precision map must be identical, the outputs equal within the merge's rounding, and the oracle tolerance holds."""
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
COS_MIN, REL_L2_MAX = 0.9999, 1e-2


def _operands(q, k, v):
    import mpsa
    from mpsa import ops
    D = q.shape[-1]
    qq = mpsa.quantize_mx(ops._pad_depth_128(q.cuda()), ops.q_side_scale(D))
    kq = mpsa.quantize_mx(ops._pad_depth_128(k.cuda()), 1.0)
    return qq, kq, mpsa.quantize_v_seq(v.cuda())


@pytest.mark.parametrize("shape,tau", [
    ((1, 4, 2, 1024, 128), 1.02),      # a good share of promoted tiles
    ((1, 4, 2, 1024, 128), 1e9),       # none promoted: nothing is appended to any row's visit list
    ((1, 4, 2, 1024, 128), 0.5),       # every tile promoted, the row's first one included: every MXFP4 tile is done twice
    ((2, 2, 1, 333, 128), 1.0),        # ragged length, two batches
    ((1, 8, 8, 640, 64), 1.05),        # head_dim 64
])
def test_router_inside_the_forward_equals_the_stand_alone_router(shape, tau):
    import mpsa
    from mpsa import ops
    B, Hq, Hkv, S, D = shape
    q, k, v = O.make_qkv(11, B, Hq, Hkv, S, D, outliers=4)
    qq, kq, vq = _operands(q, k, v)
    stat = mpsa.router_statistic(qq, kq, B, Hq, Hkv, S, S, causal=True, check=True)
    pm_ref = mpsa.precision_map_online(stat, S, S, causal=True, band=1, tau=tau)
    out_ref, lse_ref = ops.attention_forward_quantized(qq, kq, vq, B, Hq, Hkv, S, S, D, causal=True, prec_map=pm_ref,
                                                       out_dtype=torch.float32, check=True, return_lse=True)
    out, pm, lse = ops.attention_forward_routed(qq, kq, vq, B, Hq, Hkv, S, S, D, band=1, tau=tau, out_dtype=torch.float32,
                                                check=True, return_map=True, return_lse=True)
    assert int(ops._last_range_flag.item()) == 0
    assert torch.equal(pm, pm_ref), (int((pm != pm_ref).sum()), pm.unique().tolist())
    n_promoted = int(((pm == mpsa.TILE_FP8) & (mpsa.precision_map_band(S, S, True, 1, 128, pm.device) == mpsa.TILE_FP4)).sum())
    if tau == 1e9:
        assert n_promoted == 0
    if tau == 0.5:
        assert int((pm == mpsa.TILE_FP4).sum()) == 0
    m = O.parity_metrics(out.cpu(), out_ref.cpu())
    assert m["rel_l2"] <= 1e-5, (m, n_promoted)                # two passes merged vs one pass: fp32 rounding only
    assert torch.allclose(lse.cpu(), lse_ref.cpu(), rtol=1e-5, atol=1e-4)
    ref = O.attention_mxfp(q, k, v, causal=True, prec_map=pm.cpu(), pv_mode="requant")
    m = O.parity_metrics(out.cpu(), ref)
    assert m["cos"] >= COS_MIN and m["rel_l2"] <= REL_L2_MAX, m


def test_one_call_form_uses_the_router_inside_and_matches_the_stand_alone_form():
    import mpsa
    q, k, v = (t.cuda() for t in O.make_qkv(2, 1, 8, 2, 2048, 128, outliers=5))
    kw = dict(causal=True, pv_mode="requant", router="online", tau=1.05, check=True)
    a = mpsa.attention_forward(q, k, v, out_dtype=torch.bfloat16, **kw)
    b = mpsa.attention_forward(q, k, v, out_dtype=torch.bfloat16, fused_router=False, **kw)
    m = O.parity_metrics(a.float().cpu(), b.float().cpu())
    assert m["rel_l2"] <= 4e-3, m          # bf16 outputs of two different accumulation orders


def test_fallback_when_scores_leave_the_fixed_reference():
    """Later keys 2^64 and more above the first tile's maximum: the forward flags it, and the exact kernel launched behind
    it recomputes the whole output over the final map; the result still matches the oracle,
    and the map is the one the stand-alone router gives."""
    import mpsa
    from mpsa import ops
    q, k, v = O.make_qkv(9, 1, 4, 2, 1024, 128, outliers=3)
    k2 = k.clone().float()
    k2[:, :, 128:] *= 60.0                        # scores of every later tile dwarf the first tile's
    k2 = k2.to(torch.bfloat16)
    qq, kq, vq = _operands(q, k2, v)
    out, pm = ops.attention_forward_routed(qq, kq, vq, 1, 4, 2, 1024, 1024, 128, band=1, tau=1.1, out_dtype=torch.float32,
                                           check=True, return_map=True)
    assert int(ops._last_range_flag.item()) == 1
    assert set(pm.unique().tolist()) <= {0, 1, 2}
    stat = ops.router_statistic(qq, kq, 1, 4, 2, 1024, 1024, causal=True, check=True)
    assert torch.equal(pm, ops.precision_map_online(stat, 1024, 1024, causal=True, band=1, tau=1.1))
    ref = O.attention_mxfp(q, k2, v, causal=True, prec_map=pm.cpu(), pv_mode="requant")
    m = O.parity_metrics(out.cpu(), ref)
    assert m["cos"] >= COS_MIN and m["rel_l2"] <= REL_L2_MAX, m
