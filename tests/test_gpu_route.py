"""Online tile-precision router (statistic kernel + map kernel) against the CPU oracle.

The statistic is a mean of fp32 row maxima of an MXFP4 product: the GPU accumulates the 128 products of a
dot product in another order than the CPU, so it is compared with a tolerance (rel 1e-5 + abs 1e-4 in the log2
domain, written below).  The map is integer work: from the SAME statistic it must be identical; from the
oracle's own statistic it may differ only in cells whose statistic lies within that tolerance of the threshold."""
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-5, 1e-4

CASES = [  # B, Hq, Hkv, S, Skv, D, causal
    (1, 4, 2, 384, 384, 128, True),
    (1, 2, 2, 300, 300, 128, False),     # ragged last tile
    (1, 2, 1, 300, 300, 64, True),       # ragged + causal + D=64 (depth padded to 128)
    (2, 2, 2, 256, 640, 128, True),      # queries are the last 256 of 640 positions
    (1, 2, 2, 1024, 1024, 128, False),
]


def _stat(q, k, S, Skv, D, causal):
    import mpsa
    from mpsa import ops
    B, Hq, Hkv = q.shape[0], q.shape[1], k.shape[1]
    qq = mpsa.quantize_mx(ops._pad_depth_128(q.cuda()), ops.q_side_scale(D, None))
    kq = mpsa.quantize_mx(ops._pad_depth_128(k.cuda()), 1.0)
    return mpsa.router_statistic(qq, kq, B, Hq, Hkv, S, Skv, causal=causal, check=True)


@pytest.mark.parametrize("case", CASES)
def test_statistic_matches_oracle(case):
    B, Hq, Hkv, S, Skv, D, causal = case
    q, _, _ = O.make_qkv(11, B, Hq, Hq, S, D)
    _, k, _ = O.make_qkv(12, B, Hkv, Hkv, Skv, D, outliers=3)
    got = _stat(q, k, S, Skv, D, causal).cpu()
    exp = O.router_statistic_map(q, k, causal=causal)
    assert got.shape == exp.shape
    assert torch.allclose(got, exp, rtol=RTOL, atol=ATOL), (got - exp).abs().max()


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("tau", [0.5, 1.0])
def test_online_map(case, tau):
    import mpsa
    B, Hq, Hkv, S, Skv, D, causal = case
    q, _, _ = O.make_qkv(13, B, Hq, Hq, S, D)
    _, k, _ = O.make_qkv(14, B, Hkv, Hkv, Skv, D, outliers=3)
    stat = _stat(q, k, S, Skv, D, causal)
    got = mpsa.precision_map_online(stat, S, Skv, causal=causal, band=1, tau=tau).cpu()
    # integer work on the same statistic: identical
    assert torch.equal(got, O.precision_map_online(stat.cpu(), S, Skv, causal=causal, band=1, tau=tau))
    # against the oracle's own statistic: only cells on the threshold may differ
    st_o = O.router_statistic_map(q, k, causal=causal)
    exp = O.precision_map_online(st_o, S, Skv, causal=causal, band=1, tau=tau)
    thr = st_o[..., :1] * tau
    near = (st_o - thr).abs() <= RTOL * thr.abs() + ATOL
    assert torch.equal(got[~near], exp[~near])
    assert (got == O.TILE_FP8).any()


def test_attention_with_online_router():
    """The forward with the online map equals the oracle's emulation under the same map."""
    import mpsa
    q, k, v = O.make_qkv(15, 1, 4, 2, 1024, 128, outliers=3)
    stat = _stat(q, k, 1024, 1024, 128, True)
    pm = mpsa.precision_map_online(stat, 1024, 1024, causal=True, band=1, tau=1.0)
    n8 = int((pm == O.TILE_FP8).sum()) - 4 * 8            # promoted beyond the diagonal
    assert 0 < n8 < int((pm != O.TILE_SKIP).sum())
    for pv_mode in ("fp16", "requant"):
        ref = O.attention_mxfp(q, k, v, causal=True, prec_map=pm.cpu(), pv_mode=pv_mode)
        out = mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=True, router="online", tau=1.0,
                                     out_dtype=torch.float32, pv_mode=pv_mode, check=True).cpu()
        m = O.parity_metrics(out, ref)
        assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2, (pv_mode, m)


def test_bad_arguments():
    import mpsa
    st = torch.zeros((1, 1, 2, 3), dtype=torch.float32, device="cuda")
    with pytest.raises(ValueError):
        mpsa.precision_map_online(st, 256, 256, causal=True)


def test_tile_skipping_rule():
    """The reference's router proper: outside the band a tile is processed iff it is the row's first one or its
    statistic reaches skip_thresh times the first tile's.  Map identical to the oracle's from the same statistic;
    the forward under that map equals the oracle's emulation; the reported sparsity counts the dropped tiles."""
    import mpsa
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    q, k, v = O.make_qkv(16, 1, 4, 2, 1024, 128, outliers=3)
    stat = _stat(q, k, 1024, 1024, 128, True)
    pm = mpsa.precision_map_online(stat, 1024, 1024, causal=True, band=1, tau=1.1, skip_thresh=1.0)
    exp = O.precision_map_online(stat.cpu(), 1024, 1024, causal=True, band=1, tau=1.1, skip_thresh=1.0)
    assert torch.equal(pm.cpu(), exp)
    band = O.precision_map_band(8, 8, True, 1)
    dropped = int(((pm.cpu() == O.TILE_SKIP) & (band != O.TILE_SKIP)).sum())
    assert dropped > 0 and bool((pm.cpu()[..., 0] != O.TILE_SKIP).all())
    ref = O.attention_mxfp(q, k, v, causal=True, prec_map=exp, pv_mode="requant")
    out, sparsity = mxfp_attn_kernel(q.cuda(), k.cuda(), v.cuda(), is_causal=True, block_scale_type="online_requant",
                                     skip_thresh=1.0, promote_thresh=1.1, output_dtype=torch.float32, return_sparsity=True)
    m = O.parity_metrics(out.cpu(), ref)
    assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2, m
    assert abs(sparsity - dropped / (4 * 36)) < 1e-6
