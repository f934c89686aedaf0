"""Fused attention forward against the CPU oracle on the same seeded inputs.

Tolerances (from the task statement): cosine similarity >= 0.9999 and relative L2 <= 1e-2 against
the oracle's MXFP emulation with P in fp16 (the reference's P.V precision); the error against
plain fp32 attention is only reported."""
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu
COS_MIN, REL_L2_MAX = 0.9999, 1e-2


def _run(q, k, v, causal, **kw):
    import mpsa
    out = mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=causal, out_dtype=torch.float32, check=True, **kw)
    return out.cpu()


def _check(out, ref, what):
    m = O.parity_metrics(out, ref)
    assert m["cos"] >= COS_MIN and m["rel_l2"] <= REL_L2_MAX, (what, m)
    return m


@pytest.mark.parametrize("uniform", ["fp8", "fp4", None])
@pytest.mark.parametrize("causal", [False, True])
def test_one_and_two_tiles(uniform, causal):
    for S in (128, 256):
        q, k, v = O.make_qkv(0, 1, 2, 2, S, 128)
        ref = O.attention_mxfp(q, k, v, causal=causal, uniform=uniform)
        _check(_run(q, k, v, causal, uniform=uniform), ref, (S, uniform, causal))


def test_map_is_identical_to_oracle():
    import mpsa
    for (S, Skv, causal, band) in [(1024, 1024, True, 1), (1024, 1024, False, 1), (640, 640, True, 2), (300, 300, True, 1)]:
        got = mpsa.precision_map_band(S, Skv, causal, band).cpu()
        exp = O.precision_map_band(-(-S // 128), -(-Skv // 128), causal, band)
        assert torch.equal(got, exp)
    got = mpsa.precision_map_band(1024, 1024, True, 1, tile=64).cpu()
    assert torch.equal(got, O.precision_map_band(16, 16, True, 1))


def test_plumbing_config_d64():
    """B=1, H=8, S=1024, D=64 causal, seed 0 (128x128 tiles)."""
    q, k, v = O.make_qkv(0, 1, 8, 8, 1024, 64)
    ref = O.attention_mxfp(q, k, v, causal=True)
    out = _run(q, k, v, True)
    _check(out, ref, "cfg1")
    print("vs fp32 attention:", O.parity_metrics(out, O.attention_fp32(q, k, v, True)))


def test_gqa_outliers_causal():
    """Llama-3-8B-like head layout at a small sequence: Hq=8, Hkv=2, D=128, outlier K channels."""
    q, k, v = O.make_qkv(2, 1, 8, 2, 1024, 128, outliers=5)
    ref = O.attention_mxfp(q, k, v, causal=True)
    _check(_run(q, k, v, True), ref, "gqa")


def test_ragged_lengths_and_custom_map():
    q, k, v = O.make_qkv(3, 2, 2, 1, 333, 128)
    for causal in (False, True):
        ref = O.attention_mxfp(q, k, v, causal=causal)
        _check(_run(q, k, v, causal), ref, ("ragged", causal))
    # arbitrary per-(batch, head) map: checkerboard of FP8 / FP4 tiles, non causal
    B, H, S = 2, 2, 512
    q, k, v = O.make_qkv(4, B, H, H, S, 128)
    g = torch.Generator().manual_seed(1)
    pm = torch.randint(1, 3, (B, H, 4, 4), generator=g, dtype=torch.uint8)
    ref = O.attention_mxfp(q, k, v, causal=False, prec_map=pm)
    _check(_run(q, k, v, False, prec_map=pm.cuda()), ref, "custom map")
    # skipped tiles in a non-causal map, and a row tile with nothing to attend to -> zeros
    pm[:, :, 1, :] = 0
    pm[:, :, 2, 1] = 0
    ref = O.attention_mxfp(q, k, v, causal=False, prec_map=pm)
    out = _run(q, k, v, False, prec_map=pm.cuda())
    assert float(out[:, :, 128:256].abs().max()) == 0.0
    keep = torch.ones(S, dtype=torch.bool)
    keep[128:256] = False
    _check(out[:, :, keep], ref[:, :, keep], "skips")


def test_reference_entry_points():
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    from ours.mxfp_attn import mxfp_attn
    q, k, v = O.make_qkv(5, 1, 4, 4, 512, 128, dtype=torch.float16)
    for bst, uni in (("mxfp4", "fp4"), ("mxfp8", "fp8")):
        ref = O.attention_mxfp(q, k, v, causal=False, uniform=uni)
        o = mxfp_attn_kernel(q.cuda(), k.cuda(), v.cuda(), is_causal=False, block_scale_type=bst, skip_thresh=-1e9)
        assert o.dtype == torch.float16 and o.shape == q.shape
        m = O.parity_metrics(o.float().cpu(), ref)
        assert m["cos"] >= COS_MIN and m["rel_l2"] <= REL_L2_MAX, m
    o = mxfp_attn(q.cuda(), k.cuda(), v.cuda(), is_causal=True, smooth_k=False, block_scale_type="diag",
                  output_dtype=torch.bfloat16)
    ref = O.attention_mxfp(q, k, v, causal=True)
    m = O.parity_metrics(o.float().cpu(), ref)
    assert o.dtype == torch.bfloat16 and m["cos"] >= 0.9999 and m["rel_l2"] <= 1.5e-2, m
    # NHD layout
    o2 = mxfp_attn_kernel(q.transpose(1, 2).contiguous().cuda(), k.transpose(1, 2).contiguous().cuda(),
                          v.transpose(1, 2).contiguous().cuda(), is_causal=False, tensor_layout="NHD",
                          block_scale_type="mxfp8")
    ref = O.attention_mxfp(q, k, v, causal=False, uniform="fp8")
    m = O.parity_metrics(o2.transpose(1, 2).float().cpu(), ref)
    assert m["cos"] >= COS_MIN and m["rel_l2"] <= REL_L2_MAX, m
    with pytest.raises(AssertionError):
        mxfp_attn_kernel(torch.zeros(1, 1, 128, 96, device="cuda", dtype=torch.float16),
                         torch.zeros(1, 1, 128, 96, device="cuda", dtype=torch.float16),
                         torch.zeros(1, 1, 128, 96, device="cuda", dtype=torch.float16))


def test_long_sequence_slice_and_properties():
    """S = 8192 with the Llama-like layout: a slice of query rows of one head against the oracle,
    and row-stochastic behaviour (V = ones -> O = ones) over the whole output."""
    import mpsa
    q, k, v = O.make_qkv(2, 1, 8, 2, 8192, 128, outliers=5)
    out = mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=True, out_dtype=torch.float32, check=True)
    h = 5
    rows = slice(8192 - 256, 8192)
    ref = O.attention_mxfp(q[:, h:h + 1, rows], k[:, h // 4:h // 4 + 1], v[:, h // 4:h // 4 + 1], causal=True,
                           prec_map=O.precision_map_band(64, 64, True)[62:64])
    _check(out[:, h:h + 1, rows].cpu(), ref, "slice")
    ones = torch.ones_like(v)
    o1 = mpsa.attention_forward(q.cuda(), k.cuda(), ones.cuda(), causal=True, out_dtype=torch.float32, check=True)
    assert float((o1 - 1).abs().max()) < 2e-3


# ---- quantised P.V (P re-quantised to the tile's format, V quantised along the sequence) -------------
def test_v_quantizer_matches_oracle():
    import mpsa
    g = torch.Generator().manual_seed(8)
    for (B, H, S, D) in [(1, 2, 256, 128), (2, 1, 200, 128), (1, 2, 128, 64)]:
        v = (torch.randn(B, H, S, D, generator=g) * 1.7).to(torch.bfloat16)
        v[0, 0, 32:64, 5] = 0                      # an all-zero block
        r = mpsa.quantize_v_seq(v.cuda())
        for fmt, codes, sf in (("fp8e5", r.vt8.cpu(), r.v8_sf.cpu()), ("fp4", r.vt4.cpu(), r.v4_sf.cpu())):
            oc, osc = O.quant_v_seq(v, fmt)        # [B,H,D,S] codes, [B,H,D,S/32] scales
            pad = r.vt8.shape[-1]
            nblk = osc.shape[-1]                   # the oracle pads a ragged tail to a whole 32-key block
            got = (O.unpack_e2m1(codes) if fmt == "fp4" else codes)[..., :nblk * 32]
            assert torch.equal(got, oc)
            # scale tiles: rows = d, columns = key blocks; one tile per 128 keys
            tiles = sf.reshape(B, H, pad // 128, 32, 4, 4)
            for kt in range(pad // 128):
                for blk in range(4):
                    kb = kt * 4 + blk
                    if kb >= nblk:
                        continue
                    col = tiles[:, :, kt, :, :, blk]                  # [B,H,32,4]: d = i4*32 + i32
                    flat = col.permute(0, 1, 3, 2).reshape(B, H, 128)[..., :D]
                    assert torch.equal(flat, osc[..., kb]), (fmt, kt, blk)


@pytest.mark.parametrize("uniform", ["fp8", "fp4", None])
@pytest.mark.parametrize("causal", [False, True])
def test_requant_pv_small(uniform, causal):
    for S in (128, 384):
        q, k, v = O.make_qkv(0, 1, 2, 2, S, 128)
        ref = O.attention_mxfp(q, k, v, causal=causal, uniform=uniform, pv_mode="requant")
        out = _run(q, k, v, causal, uniform=uniform, pv_mode="requant")
        _check(out, ref, ("requant", S, uniform, causal))


def test_requant_pv_gqa_outliers_and_ragged():
    q, k, v = O.make_qkv(2, 1, 8, 2, 1024, 128, outliers=5)
    ref = O.attention_mxfp(q, k, v, causal=True, pv_mode="requant")
    out = _run(q, k, v, True, pv_mode="requant")
    _check(out, ref, "requant gqa")
    print("requant vs fp32 attention:", O.parity_metrics(out, O.attention_fp32(q, k, v, True)))
    q, k, v = O.make_qkv(3, 2, 2, 1, 333, 128)
    ref = O.attention_mxfp(q, k, v, causal=True, pv_mode="requant")
    _check(_run(q, k, v, True, pv_mode="requant"), ref, "requant ragged")
    q, k, v = O.make_qkv(0, 1, 4, 4, 512, 64)
    ref = O.attention_mxfp(q, k, v, causal=True, pv_mode="requant")
    _check(_run(q, k, v, True, pv_mode="requant"), ref, "requant d64")


def test_host_tensors_are_streamed():
    """CPU tensors through the reference-facing call: chunked over KV groups on three streams, same result as the
    device call on the same inputs (bit for bit: the chunks are independent units of the path)."""
    import mpsa
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    q, k, v = O.make_qkv(7, 2, 8, 2, 512, 128, outliers=3)
    dev_out = mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=True, out_dtype=torch.bfloat16,
                                     pv_mode="requant", check=True).cpu()
    for _ in range(2):                            # second call reuses the staging buffers
        host_out = mxfp_attn_kernel(q, k, v, is_causal=True, block_scale_type="diag_requant", output_dtype=torch.bfloat16)
        assert not host_out.is_cuda and torch.equal(host_out, dev_out)     # no synchronisation: the call returned the data
    buf = torch.empty_like(host_out).pin_memory()
    r = mxfp_attn_kernel(q, k, v, is_causal=True, block_scale_type="diag_requant", output_dtype=torch.bfloat16, out=buf)
    assert r is buf and torch.equal(buf, dev_out)
    # the non-blocking form hands back the event to wait on
    buf2 = torch.zeros_like(buf).pin_memory()
    r2, done = mpsa.attention_forward_host(q, k, v, causal=True, out=buf2, out_dtype=torch.bfloat16, pv_mode="requant",
                                           non_blocking=True)
    done.synchronize()
    assert r2 is buf2 and torch.equal(buf2, dev_out)


def test_block_scale_type_names_are_checked():
    """The reference asserts the set of block_scale_type names (ours/mxfp_attn_kernel.py:452); a name outside the
    set of this library raises instead of silently running another format."""
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    q, k, v = (t.cuda() for t in O.make_qkv(1, 1, 2, 2, 256, 128))
    for name in ("mixed", "mxfp6", "MXFP8", ""):
        with pytest.raises(ValueError):
            mxfp_attn_kernel(q, k, v, block_scale_type=name)
    o = mxfp_attn_kernel(q, k, v, block_scale_type="nvfp4", output_dtype=torch.float32)
    ref = O.attention_mxfp(q.cpu(), k.cpu(), v.cpu(), causal=False, uniform="fp4", fp4_kind="nvfp4")
    _check(o.cpu(), ref, "nvfp4 by name")


def test_fixed_reference_kernel_and_its_fallback():
    """Quantised P.V runs with the row reference fixed after the first key tile; the exact kernel is its conditional
    fallback.  (1) On ordinary data both give the same output.  (2) When later keys push the scores more than 2^64
    above the first tile's maximum, the fallback must take over: the result still matches the oracle."""
    import mpsa
    from mpsa import ops
    q, k, v = O.make_qkv(9, 1, 4, 2, 1024, 128, outliers=3)

    def run(q, k, v, lazy):
        sq = ops.q_side_scale(128)
        qq, kq = mpsa.quantize_mx(q.cuda(), sq), mpsa.quantize_mx(k.cuda(), 1.0)
        vq = mpsa.quantize_v_seq(v.cuda())
        return ops.attention_forward_quantized(qq, kq, vq, 1, 4, 2, 1024, 1024, 128, causal=True, out_dtype=torch.float32,
                                               check=True, lazy=lazy).cpu()

    a, b = run(q, k, v, True), run(q, k, v, False)
    assert torch.allclose(a, b, rtol=1e-5, atol=1e-6), (a - b).abs().max()
    _check(a, O.attention_mxfp(q, k, v, causal=True, pv_mode="requant"), "fixed reference")
    k2 = k.clone().float()
    k2[:, :, 128:] *= 60.0                       # scores of every later tile dwarf the first tile's
    k2 = k2.to(torch.bfloat16)
    ref = O.attention_mxfp(q, k2, v, causal=True, pv_mode="requant")
    out = run(q, k2, v, True)
    assert torch.isfinite(out).all()
    _check(out, ref, "fallback")
    assert torch.allclose(out, run(q, k2, v, False), rtol=1e-5, atol=1e-6)


def test_fixed_reference_is_not_abandoned_on_ragged_shapes():
    """The padding rows of a ragged last query tile hold no data: they must not trigger the exact-kernel fallback."""
    import mpsa
    from mpsa import ops
    for S, causal in ((1560, False), (300, True)):
        q, k, v = O.make_qkv(10, 1, 2, 2, S, 128)
        out = mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=causal, pv_mode="requant", out_dtype=torch.float32, check=True)
        assert int(ops._last_range_flag.item()) == 0
        _check(out.cpu(), O.attention_mxfp(q, k, v, causal=causal, pv_mode="requant"), ("ragged", S))


@pytest.mark.parametrize("pv_mode", ["fp16", "requant"])
def test_merge_in_the_epilogue(pv_mode):
    """A forward over the second half of the keys, given the partial result over the first half, writes the merged
    result itself: it must equal the separate merge pass, and the attention over all keys up to quantisation of
    V in halves (V's block scales do not depend on the split: its blocks are 32 keys long)."""
    import mpsa
    from mpsa import ops
    B, Hq, Hkv, S, D = 1, 4, 2, 512, 128
    q, k, v = O.make_qkv(12, B, Hq, Hkv, S, D, outliers=2)
    qq = mpsa.quantize_mx(q.cuda(), ops.q_side_scale(D))
    halves = []
    for sl in (slice(0, S // 2), slice(S // 2, S)):
        vh = v[:, :, sl].contiguous().cuda()
        halves.append((mpsa.quantize_mx(k[:, :, sl].contiguous().cuda(), 1.0),
                       mpsa.quantize_v_seq(vh) if pv_mode == "requant" else ops.prepare_vt(vh)))
    kw = dict(causal=False, uniform="fp4", out_dtype=torch.float32, check=True)
    a0, l0 = ops.attention_forward_quantized(qq, *halves[0], B, Hq, Hkv, S, S // 2, D, return_lse=True, **kw)
    a1, l1 = ops.attention_forward_quantized(qq, *halves[1], B, Hq, Hkv, S, S // 2, D, return_lse=True, **kw)
    fused, lf = ops.attention_forward_quantized(qq, *halves[1], B, Hq, Hkv, S, S // 2, D, merge_with=(a0, l0), **kw)
    acc, lacc = a0.clone(), l0.clone()
    mpsa.attention_merge(acc, lacc, a1, l1)
    assert torch.allclose(fused, acc, rtol=1e-5, atol=1e-6), (fused - acc).abs().max()
    assert torch.allclose(lf, lacc, rtol=1e-6, atol=1e-5)
    ref = O.attention_mxfp(q, k, v, causal=False, uniform="fp4", pv_mode=pv_mode)
    _check(fused.cpu(), ref, ("merged", pv_mode))
    # an empty earlier result (lse = -inf) leaves the plain forward
    z, lz = torch.zeros_like(a0), torch.full_like(l0, float("-inf"))
    alone, _ = ops.attention_forward_quantized(qq, *halves[1], B, Hq, Hkv, S, S // 2, D, merge_with=(z, lz), **kw)
    assert torch.allclose(alone, a1, rtol=1e-6, atol=1e-7)


def test_smooth_k_through_the_reference_entry_point():
    """mxfp_attn_kernel(..., smooth_k=True) on device tensors centres K inside the quantizer; the result must match the
    oracle run on K minus the same mean (a shift of K along the sequence moves every score of a row equally)."""
    import mpsa
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    q, k, v = O.make_qkv(13, 1, 4, 2, 384, 128, outliers=2)
    k = (k.float() + 1.5).to(torch.bfloat16)                    # a mean worth removing
    o = mxfp_attn_kernel(q.cuda(), k.cuda(), v.cuda(), is_causal=True, smooth_k=True, block_scale_type="diag",
                         output_dtype=torch.float32)
    mpsa.check_status()
    mean = mpsa.column_mean(k.cuda()).cpu()
    kc = (k.float() - mean.unsqueeze(2)).to(torch.bfloat16)
    _check(o.cpu(), O.attention_mxfp(q, kc, v, causal=True), "smooth_k")


def test_rotary_embedding_fused_into_the_quantizers():
    """attention_forward(..., rope=(cos, sin)) on un-rotated q and k equals the oracle on the rotated tensors."""
    import mpsa
    q, k, v = O.make_qkv(14, 1, 4, 2, 384, 128)
    cos, sin = O.rope_angles(384, 128)
    out = mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=True, out_dtype=torch.float32, check=True,
                                 rope=(cos.cuda(), sin.cuda()))
    ref = O.attention_mxfp(O.rope_rotate_half(q, cos, sin), O.rope_rotate_half(k, cos, sin), v, causal=True)
    _check(out.cpu(), ref, "rope")


def test_persisted_kv_block_feeds_the_forward(tmp_path):
    """K and V quantised once, packed into the persisted byte form on the device, written to a file, read back and
    unpacked as views: the forward gives bit-identical output to the one on the live operands."""
    import mpsa
    from mpsa import kvstore, ops
    B, Hq, Hkv, S, D = 1, 4, 2, 640, 128
    q, k, v = O.make_qkv(15, B, Hq, Hkv, S, D, outliers=2)
    qq = mpsa.quantize_mx(q.cuda(), ops.q_side_scale(D))
    kq, vq = mpsa.quantize_mx(k.cuda(), 1.0), mpsa.quantize_v_seq(v.cuda())
    kw = dict(causal=True, out_dtype=torch.float32, check=True)
    direct = ops.attention_forward_quantized(qq, kq, vq, B, Hq, Hkv, S, S, D, **kw)
    path = str(tmp_path / "kv.mpsakv")
    n = kvstore.save_kv(path, kq, vq)
    assert n == kvstore.packed_size(kq, vq)
    k2, v2, h = kvstore.load_kv(path, device="cuda")
    assert (h["S"], h["Hkv"], h["pitch"]) == (S, Hkv, 640) and torch.equal(k2.fp4, kq.fp4) and torch.equal(v2.v4_sf, vq.v4_sf)
    again = ops.attention_forward_quantized(qq, k2, v2, B, Hq, Hkv, S, S, D, **kw)
    assert torch.equal(direct, again)


@pytest.mark.parametrize("pv_mode", ["fp16", "requant"])
def test_prepared_kv_is_reused(pv_mode):
    """prepare_kv once, attention_forward(kv=...) for two different query blocks: same bits as the calls that
    quantise K and V themselves (online router included)."""
    import mpsa
    q, k, v = O.make_qkv(16, 1, 4, 2, 512, 128, outliers=2)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    kw = dict(causal=True, pv_mode=pv_mode, router="online", tau=1.1, out_dtype=torch.float32, check=True)
    kv = mpsa.prepare_kv(kd, vd, pv_mode=pv_mode)
    assert torch.equal(mpsa.attention_forward(qd, None, None, kv=kv, **kw), mpsa.attention_forward(qd, kd, vd, **kw))
    q2 = qd[:, :, 256:].contiguous()               # the last 256 queries against all keys
    assert torch.equal(mpsa.attention_forward(q2, None, None, kv=kv, **kw), mpsa.attention_forward(q2, kd, vd, **kw))
    with pytest.raises(ValueError):
        mpsa.attention_forward(qd, None, None, kv=kv, fp4_kind="nvfp4", **kw)
