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
