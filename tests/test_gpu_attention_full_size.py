"""The headline workload at its own sizes and in its own mode - Llama-3-8B-shaped causal prefill (B=1, Hq=32, Hkv=8,
D=128) at S = 8192 and S = 32768, online router (tau 1.1), P re-quantised to the tile's format - against the CPU oracle on
slices of the very tensors the benchmark draws (seed 2, CPU generator, 5 outlier K channels).  The oracle cannot do the
whole problem in reasonable time, so it gets 256-row slices of two query heads from different KV groups, with all their
keys and with the rows of the precision map the GPU router produced; the router's map itself is checked on those rows
against the oracle's statistic."""
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
COS_MIN, REL_L2_MAX = 0.9999, 1e-2
TAU = 1.1


@pytest.mark.parametrize("S", [8192, 32768])
def test_bench_workload_slices_match_the_oracle(S):
    import mpsa
    from mpsa import ops
    Hq, Hkv, D = 32, 8, 128
    q, k, v = O.make_qkv(2, 1, Hq, Hkv, S, D, outliers=5)
    dq, dk, dv = q.cuda(), k.cuda(), v.cuda()
    qq, kq = mpsa.quantize_mx(dq, ops.q_side_scale(D)), mpsa.quantize_mx(dk, 1.0)
    vq = mpsa.quantize_v_seq(dv)
    stat = mpsa.router_statistic(qq, kq, 1, Hq, Hkv, S, S, causal=True, check=True)
    pm = mpsa.precision_map_online(stat, S, S, causal=True, band=1, tau=TAU)
    out = ops.attention_forward_quantized(qq, kq, vq, 1, Hq, Hkv, S, S, D, causal=True, prec_map=pm,
                                          out_dtype=torch.float32, check=True)
    # the fixed-reference kernel must have been enough: no score left its 2^64 headroom at this size
    assert int(ops._last_range_flag.item()) == 0
    # ... and the one-call form (what the benchmark times: the router runs inside the forward, the promoted tiles
    # are done again in MXFP8 at the end of their row) gives the same result up to fp32 rounding, from the same map
    out2, pm2 = ops.attention_forward_routed(qq, kq, vq, 1, Hq, Hkv, S, S, D, band=1, tau=TAU, out_dtype=torch.float32,
                                             check=True, return_map=True)
    assert int(ops._last_range_flag.item()) == 0
    assert torch.equal(pm, pm2)
    m2 = O.parity_metrics(out2.cpu(), out.cpu())
    assert m2["rel_l2"] <= 1e-5, m2
    out3 = mpsa.attention_forward(dq, dk, dv, causal=True, out_dtype=torch.float32, pv_mode="requant", router="online",
                                  tau=TAU, check=True)
    assert torch.equal(out2, out3)
    pm_c, out_c = pm.cpu(), out.cpu()
    grp = Hq // Hkv
    for h in (3, 17):
        hk = h // grp
        for r0 in (S // 2, S - 256):
            rows = slice(r0, r0 + 256)
            nkeys = r0 + 256
            pm_rows = pm_c[:, h:h + 1, r0 // 128:r0 // 128 + 2, :nkeys // 128]
            ref = O.attention_mxfp(q[:, h:h + 1, rows], k[:, hk:hk + 1, :nkeys], v[:, hk:hk + 1, :nkeys], causal=True,
                                   prec_map=pm_rows, pv_mode="requant")
            m = O.parity_metrics(out_c[:, h:h + 1, rows], ref)
            assert m["cos"] >= COS_MIN and m["rel_l2"] <= REL_L2_MAX, (S, h, r0, m)
            # the map rows: identical to the oracle's map from the oracle's own statistic, except where the statistic
            # lies within the summation-order tolerance of the threshold
            st_o = O.router_statistic_map(q[:, h:h + 1, rows], k[:, hk:hk + 1, :nkeys], causal=True)
            pm_o = O.precision_map_online(st_o, 256, nkeys, causal=True, band=1, tau=TAU)
            diff = pm_o != pm_rows
            if diff.any():
                sink = st_o[..., :1]
                near = (st_o - sink * TAU).abs() <= 1e-5 * st_o.abs() + 1e-4
                assert bool((near | ~diff).all()), (S, h, r0, int(diff.sum()))
