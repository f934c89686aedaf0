"""The persisted form of a quantised K/V block: byte layout, round trip, zero-copy views and header validation
(host logic only: the sections are opaque bytes here, the kernels that make and read them are tested on the GPU)."""
import struct

import pytest
import torch

from mpsa import kvstore, ops


def _fake(B=1, H=2, S=300, D=128, pitch=384, fp4_kind="mxfp4", forms=("fp8", "fp4"), with_v=True, seed=0):
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape: torch.randint(0, 256, shape, dtype=torch.uint8, generator=g)
    nt = -(-S // 128)
    kq = ops.QuantizedOperand(fp8_elem="e5m2", fp4_kind=fp4_kind)
    if "fp8" in forms:
        kq.fp8, kq.fp8_sf = r(B, H, S, D), r(B, H, nt, 1, 512)
    if "fp4" in forms:
        kq.fp4, kq.fp4_sf = r(B, H, S, D // 2), r(B, H, nt, 2 if fp4_kind == "nvfp4" else 1, 512)
    if fp4_kind == "nvfp4":
        kq.fp4_ts = torch.tensor([0.0123], dtype=torch.float32)
    vq = None
    if with_v:
        vq = ops.QuantizedV(r(B, H, D, pitch) if "fp8" in forms else None, r(B, H, pitch // 128, 512) if "fp8" in forms else None,
                            r(B, H, D, pitch // 2) if "fp4" in forms else None, r(B, H, pitch // 128, 512) if "fp4" in forms else None,
                            "e5m2")
    return kq, vq


def _same(a, b):
    return (a is None and b is None) or torch.equal(a, b)


@pytest.mark.parametrize("fp4_kind,forms,with_v", [("mxfp4", ("fp8", "fp4"), True), ("mxfp4", ("fp4",), True),
                                                  ("nvfp4", ("fp8", "fp4"), True), ("mxfp4", ("fp8", "fp4"), False)])
def test_round_trip_and_layout(fp4_kind, forms, with_v):
    kq, vq = _fake(fp4_kind=fp4_kind, forms=forms, with_v=with_v)
    buf = kvstore.pack_kv(kq, vq)
    assert buf.dtype == torch.uint8 and buf.numel() == kvstore.packed_size(kq, vq) and buf.numel() % 256 == 0
    assert bytes(buf[:8].numpy().tobytes()) == kvstore.MAGIC
    h = kvstore.read_header(buf)
    assert (h["B"], h["Hkv"], h["S"], h["D"]) == (1, 2, 300, 128) and h["fp4_kind"] == fp4_kind
    assert h["pitch"] == (384 if with_v else 0)
    ends = 0
    for name, (off, n) in sorted(h["sections"].items(), key=lambda kv: kv[1][0]):
        assert off % 256 == 0 and off >= ends          # aligned, in order, not overlapping
        ends = off + n
    k2, v2, _ = kvstore.unpack_kv(buf)
    for f in ("fp8", "fp8_sf", "fp4", "fp4_sf"):
        assert _same(getattr(kq, f), getattr(k2, f)), f
    assert k2.fp8_elem == "e5m2" and k2.fp4_kind == fp4_kind
    if fp4_kind == "nvfp4":
        assert float(k2.fp4_ts) == pytest.approx(0.0123)
    if with_v:
        for f in ("vt8", "v8_sf", "vt4", "v4_sf"):
            assert _same(getattr(vq, f), getattr(v2, f)), f
    else:
        assert v2 is None
    # views, not copies
    first = k2.fp8 if k2.fp8 is not None else k2.fp4
    first.view(-1)[0] ^= 0xFF
    assert not torch.equal(buf, kvstore.pack_kv(kq, vq))


def test_file_round_trip(tmp_path):
    kq, vq = _fake(seed=3)
    path = str(tmp_path / "block.mpsakv")
    n = kvstore.save_kv(path, kq, vq)
    assert n == kvstore.packed_size(kq, vq)
    k2, v2, h = kvstore.load_kv(path)
    assert torch.equal(k2.fp4, kq.fp4) and torch.equal(v2.vt8, vq.vt8) and h["S"] == 300


def test_pack_into_a_given_buffer_and_errors():
    kq, vq = _fake()
    n = kvstore.packed_size(kq, vq)
    out = torch.zeros(n + 512, dtype=torch.uint8)
    buf = kvstore.pack_kv(kq, vq, out=out)
    assert buf.data_ptr() == out.data_ptr() and buf.numel() == n
    with pytest.raises(ValueError):
        kvstore.pack_kv(kq, vq, out=torch.zeros(n - 1, dtype=torch.uint8))
    with pytest.raises(ValueError):
        kvstore.pack_kv(ops.QuantizedOperand(), None)
    vq.fp8_elem = "e4m3"
    with pytest.raises(ValueError):
        kvstore.pack_kv(kq, vq)


def test_header_validation():
    kq, vq = _fake()
    buf = kvstore.pack_kv(kq, vq)
    bad = buf.clone(); bad[0] = 0
    with pytest.raises(ValueError, match="magic"):
        kvstore.read_header(bad)
    with pytest.raises(ValueError):
        kvstore.read_header(buf[:64])
    with pytest.raises(ValueError, match="truncated"):
        kvstore.unpack_kv(buf[:buf.numel() - 256].clone())
    bad = buf.clone()                                  # a section offset that is not aligned
    raw = bytearray(bad[128:152].numpy().tobytes())
    tag, off, n = struct.unpack("<3q", raw)
    bad[128:152] = torch.frombuffer(bytearray(struct.pack("<3q", tag, off + 8, n)), dtype=torch.uint8)
    with pytest.raises(ValueError):
        kvstore.read_header(bad)
    bad = buf.clone()                                  # a shape the sections cannot hold
    bad[16:20] = torch.frombuffer(bytearray(struct.pack("<i", 301)), dtype=torch.uint8)
    with pytest.raises(ValueError):
        kvstore.unpack_kv(bad)
    bad = buf.clone()                                  # pitch smaller than the keys
    bad[24:28] = torch.frombuffer(bytearray(struct.pack("<i", 128)), dtype=torch.uint8)
    with pytest.raises(ValueError):
        kvstore.read_header(bad)
