"""Host-side logic that needs no GPU: the chunk plan of the host-memory pipeline."""
import itertools

from mpsa.ops import _host_chunks


def test_host_chunks_cover_every_head_once_in_order():
    for B, Hkv, grp in itertools.product((1, 2), (1, 2, 8), (1, 2, 4, 7)):
        chunks = _host_chunks(B, Hkv, grp)
        seen = []
        for b, g, h0, nh in chunks:
            assert 0 <= b < B and 0 <= g < Hkv and nh >= 1 and 0 <= h0 and h0 + nh <= grp
            seen += [(b, g, h) for h in range(h0, h0 + nh)]
        assert seen == [(b, g, h) for b in range(B) for g in range(Hkv) for h in range(grp)]
        # a KV group's pieces are consecutive and start at its first head (K and V are uploaded with the first piece)
        for i, (b, g, h0, nh) in enumerate(chunks):
            if h0 > 0:
                pb, pg, ph0, pnh = chunks[i - 1]
                assert (pb, pg) == (b, g) and ph0 + pnh == h0


def test_host_chunks_cut_first_and_last_group_finer():
    chunks = _host_chunks(1, 8, 4)
    assert [c[3] for c in chunks[:3]] == [1, 1, 2] and [c[3] for c in chunks[-3:]] == [2, 1, 1]
    assert all(c[3] == 4 for c in chunks[3:-3])
    assert _host_chunks(1, 1, 4) == [(0, 0, 0, 4)]          # a single group is not cut


def test_oracle_router_statistic_equals_a_naive_loop():
    """The vectorised router statistic of the oracle against a tile-by-tile restatement of its definition
    (mean over the query rows of the row maximum over the visible keys; rows without a visible key count 0)."""
    import torch
    from oracle import mx_oracle as O
    for (S, Skv, causal, D) in [(300, 300, True, 64), (256, 640, True, 128), (200, 330, False, 128)]:
        q, _, _ = O.make_qkv(21, 1, 2, 2, S, D)
        _, k, _ = O.make_qkv(22, 1, 1, 1, Skv, D, outliers=2)
        got = O.router_statistic_map(q, k, causal=causal)
        qc, qs = O.quant_mxfp4_side(q, O.q_side_scale(D))
        kc, ks = O.quant_mxfp4_side(k, 1.0)
        qd, kd = O.dequant(qc, qs, "fp4").float(), O.dequant(kc, ks, "fp4").float()
        off = Skv - S
        for h in range(2):
            s = qd[0, h] @ kd[0, 0].T
            for i in range(-(-S // 128)):
                for j in range(-(-Skv // 128)):
                    rows = range(i * 128, min(S, i * 128 + 128))
                    tot = 0.0
                    for r in rows:
                        cols = [c for c in range(j * 128, min(Skv, j * 128 + 128)) if (not causal) or c <= r + off]
                        if cols:
                            tot += float(s[r, cols].max())
                    exp = tot / len(rows)
                    assert abs(float(got[0, h, i, j]) - exp) <= 1e-4 * max(1.0, abs(exp)), (S, Skv, causal, h, i, j)


def test_oracle_online_map_rules():
    import torch
    from oracle import mx_oracle as O
    stat = torch.tensor([[[[4.0, 0, 0, 0], [4.0, 5.0, 0, 0], [4.0, 3.0, 9.0, 0], [4.0, 4.4, 1.0, 2.0]]]])
    m = O.precision_map_online(stat, 512, 512, causal=True, band=1, tau=1.1)
    assert m[0, 0].tolist() == [[1, 0, 0, 0], [2, 1, 0, 0], [2, 2, 1, 0], [2, 1, 2, 1]]
    m = O.precision_map_online(stat, 512, 512, causal=True, band=1, tau=1.1, skip_thresh=0.5)
    assert m[0, 0].tolist() == [[1, 0, 0, 0], [2, 1, 0, 0], [2, 2, 1, 0], [2, 1, 0, 1]]      # the first tile and the band are never dropped


def test_oracle_rotary_embedding_is_the_rotate_half_rule():
    """The oracle's restatement against the formula written the way transformers writes it:
    x * cos + rotate_half(x) * sin with cos / sin repeated over the two halves."""
    import torch
    from oracle import mx_oracle as O
    g = torch.Generator().manual_seed(21)
    x = torch.randn(2, 3, 40, 64, generator=g).to(torch.bfloat16)
    cos, sin = O.rope_angles(40, 64, offset=5)
    assert cos.shape == (40, 32) and float(cos[0, 0]) == float(torch.cos(torch.tensor(5.0)))
    cc, ss = torch.cat([cos, cos], -1), torch.cat([sin, sin], -1)
    rot = torch.cat([-x[..., 32:].float(), x[..., :32].float()], -1)
    ref = (x.float() * cc + rot * ss).to(torch.bfloat16)
    assert torch.equal(O.rope_rotate_half(x, cos, sin), ref)
    # per-batch angles
    cb, sb = torch.stack([cos, cos.flip(0)]), torch.stack([sin, sin.flip(0)])
    y = O.rope_rotate_half(x, cb, sb)
    assert torch.equal(y[0], ref[0]) and not torch.equal(y[1], ref[1])
    # a rotation keeps the norm of every (x1[i], x2[i]) pair
    xf = torch.randn(1, 1, 40, 64, generator=g)
    yf = O.rope_rotate_half(xf, cos, sin)
    n0 = xf[..., :32] ** 2 + xf[..., 32:] ** 2
    n1 = yf[..., :32] ** 2 + yf[..., 32:] ** 2
    assert torch.allclose(n0, n1, rtol=1e-5, atol=1e-6)
