"""Persisted form of a quantised K/V block: one flat byte buffer = a fixed header, a table of sections and the
sections themselves (codes and 128x4 scale tiles exactly as the kernels read them), so that a block quantised
once can be kept (a KV cache on disk or in host memory), shipped between GPUs, and handed back to the fused forward
without touching the 16-bit tensors again.  The reference keeps nothing: it re-quantises K on every call
(ours/mxfp_attn_kernel.py:41-55) and holds V in fp16 (:29-31).

Layout (little endian):
  bytes 0..7     magic  b"MPSAKV01"
  bytes 8..63    14 x int32: B, Hkv, S (keys), D (depth as quantised: 128), V pitch (keys per V^T row), fp8 element
                 (0 e5m2, 1 e4m3), fp4 kind (0 mxfp4, 1 nvfp4), number of sections, then 6 reserved zeros
  bytes 64..67   float32 NVFP4 tensor scale of K (0 when unused)
  bytes 68..127  zero
  bytes 128..    section table: per section 3 x int64 (tag, offset, length), offsets from the start of the buffer and
                 multiples of 256 (every section starts 256-byte aligned: TMA and 16-byte vector loads need 16)
  tags           1 K fp8 codes, 2 K fp8 scale tiles, 3 K fp4 codes, 4 K fp4 scale tiles,
                 5 V^T fp8 codes, 6 V^T fp8 scale tiles, 7 V^T fp4 codes, 8 V^T fp4 scale tiles
Sections that a producer did not make (the ring ships the FP4 forms only) are simply absent.
unpack_kv returns views into the buffer: nothing is copied, on the host or on the device."""
from __future__ import annotations

import struct
from typing import Optional, Tuple

import torch

MAGIC = b"MPSAKV01"
HEADER_BYTES = 128
ALIGN = 256
_TAGS = {"k8": 1, "k8_sf": 2, "k4": 3, "k4_sf": 4, "vt8": 5, "v8_sf": 6, "vt4": 7, "v4_sf": 8}
_FP8 = {"e5m2": 0, "e4m3": 1}
_FP4 = {"mxfp4": 0, "nvfp4": 1}


def _round_up(n: int, a: int = ALIGN) -> int:
    return -(-n // a) * a


def _sections(kq, vq):
    out = []
    for name, t in (("k8", kq.fp8), ("k8_sf", kq.fp8_sf), ("k4", kq.fp4), ("k4_sf", kq.fp4_sf)):
        if t is not None:
            out.append((name, t))
    if vq is not None:
        for name, t in (("vt8", vq.vt8), ("v8_sf", vq.v8_sf), ("vt4", vq.vt4), ("v4_sf", vq.v4_sf)):
            if t is not None:
                out.append((name, t))
    return out


def packed_size(kq, vq) -> int:
    """Bytes pack_kv needs for these operands."""
    secs = _sections(kq, vq)
    n = _round_up(HEADER_BYTES + 24 * len(secs))
    for _, t in secs:
        n += _round_up(t.numel() * t.element_size())
    return n


def pack_kv(kq, vq=None, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """kq: QuantizedOperand of K [B,Hkv,S,128] in kernel format; vq: QuantizedV (or None).  -> uint8 tensor on the
    operands' device holding header + sections.  `out`: a uint8 buffer of at least packed_size bytes to fill."""
    secs = _sections(kq, vq)
    if not secs:
        raise ValueError("nothing to pack")
    codes = kq.fp8 if kq.fp8 is not None else kq.fp4
    if codes is None or codes.dim() != 4:
        raise ValueError("K codes must be [B, Hkv, S, bytes per row]")
    B, Hkv, S = codes.shape[:3]
    D = codes.shape[3] * (1 if kq.fp8 is not None else 2)
    pitch = 0
    if vq is not None:
        pitch = vq.vt8.shape[-1] if vq.vt8 is not None else vq.vt4.shape[-1] * 2
        if vq.fp8_elem != kq.fp8_elem:
            raise ValueError("K and V use different fp8 element formats")
    dev = codes.device
    total = packed_size(kq, vq)
    if out is None:
        out = torch.empty(total, dtype=torch.uint8, device=dev)
    elif out.dtype != torch.uint8 or out.numel() < total or out.device != dev or not out.is_contiguous():
        raise ValueError(f"out must be a contiguous uint8 buffer of at least {total} bytes on the operands' device")
    ts = float(kq.fp4_ts.item()) if (kq.fp4_kind == "nvfp4" and kq.fp4_ts is not None) else 0.0
    head = bytearray(_round_up(HEADER_BYTES + 24 * len(secs)))
    head[0:8] = MAGIC
    struct.pack_into("<14i", head, 8, B, Hkv, S, D, pitch, _FP8[kq.fp8_elem], _FP4[kq.fp4_kind], len(secs), 0, 0, 0, 0, 0, 0)
    struct.pack_into("<f", head, 64, ts)
    off = len(head)
    for i, (name, t) in enumerate(secs):
        n = t.numel() * t.element_size()
        struct.pack_into("<3q", head, HEADER_BYTES + 24 * i, _TAGS[name], off, n)
        off += _round_up(n)
    out[:len(head)].copy_(torch.frombuffer(head, dtype=torch.uint8))
    off = len(head)
    for name, t in secs:
        n = t.numel() * t.element_size()
        if not t.is_contiguous():
            raise ValueError(f"section {name} is not contiguous")
        out[off:off + n].copy_(t.reshape(-1).view(torch.uint8))
        off += _round_up(n)
    return out[:total]


def read_header(buf: torch.Tensor) -> dict:
    """Parse and validate the header of a packed buffer (host or device tensor); raises ValueError on anything odd."""
    if buf.dtype != torch.uint8 or buf.dim() != 1 or buf.numel() < HEADER_BYTES:
        raise ValueError("a packed K/V buffer is a 1-D uint8 tensor of at least 128 bytes")
    head = bytes(buf[:HEADER_BYTES].cpu().numpy().tobytes())
    if head[:8] != MAGIC:
        raise ValueError("not a packed K/V buffer (bad magic)")
    B, Hkv, S, D, pitch, fp8, fp4, nsec = struct.unpack_from("<8i", head, 8)
    if min(B, Hkv, S, D) <= 0 or fp8 not in (0, 1) or fp4 not in (0, 1) or not (0 < nsec <= len(_TAGS)) or \
            pitch < 0 or pitch % 128 or (pitch and pitch < S):
        raise ValueError("corrupt K/V header")
    table_end = HEADER_BYTES + 24 * nsec
    if buf.numel() < table_end:
        raise ValueError("truncated K/V buffer (section table)")
    table = bytes(buf[HEADER_BYTES:table_end].cpu().numpy().tobytes())
    names = {v: k for k, v in _TAGS.items()}
    sections = {}
    for i in range(nsec):
        tag, off, n = struct.unpack_from("<3q", table, 24 * i)
        if tag not in names or names[tag] in sections or off % ALIGN or off < table_end or n <= 0 or off + n > buf.numel():
            raise ValueError("corrupt or truncated K/V buffer (section table)")
        sections[names[tag]] = (off, n)
    return dict(B=B, Hkv=Hkv, S=S, D=D, pitch=pitch, fp8_elem="e5m2" if fp8 == 0 else "e4m3",
                fp4_kind="mxfp4" if fp4 == 0 else "nvfp4", fp4_ts=struct.unpack_from("<f", head, 64)[0],
                sections=sections)


def unpack_kv(buf: torch.Tensor) -> Tuple[object, object, dict]:
    """-> (QuantizedOperand of K, QuantizedV or None, header).  The tensors are views of `buf`; absent V^T forms come
    back as None (attention_forward_quantized needs both forms of V: a caller that ships one form supplies a
    placeholder for the other, as the ring does)."""
    from . import ops
    h = read_header(buf)
    if buf.data_ptr() % 16:
        raise ValueError("a packed K/V buffer must start 16-byte aligned")
    B, Hkv, S, D, pitch = h["B"], h["Hkv"], h["S"], h["D"], h["pitch"]
    nt = -(-S // 128)
    m4 = 2 if h["fp4_kind"] == "nvfp4" else 1
    want = {"k8": (B, Hkv, S, D), "k8_sf": (B, Hkv, nt, D // 128, 512), "k4": (B, Hkv, S, D // 2),
            "k4_sf": (B, Hkv, nt, m4 * (D // 128), 512),
            "vt8": (B, Hkv, D, pitch), "v8_sf": (B, Hkv, pitch // 128, 512),
            "vt4": (B, Hkv, D, pitch // 2), "v4_sf": (B, Hkv, pitch // 128, 512)}
    t = {}
    for name, (off, n) in h["sections"].items():
        shape = want[name]
        size = 1
        for d in shape:
            size *= d
        if size != n:
            raise ValueError(f"section {name} has {n} bytes, the header's shape needs {size}")
        t[name] = buf[off:off + n].view(shape)
    kq = ops.QuantizedOperand(fp8=t.get("k8"), fp8_sf=t.get("k8_sf"), fp4=t.get("k4"), fp4_sf=t.get("k4_sf"),
                              fp8_elem=h["fp8_elem"], fp4_kind=h["fp4_kind"])
    if h["fp4_kind"] == "nvfp4":
        kq.fp4_ts = torch.tensor([h["fp4_ts"]], dtype=torch.float32, device=buf.device)
    vq = None
    if any(name in t for name in ("vt8", "vt4")):
        vq = ops.QuantizedV(t.get("vt8"), t.get("v8_sf"), t.get("vt4"), t.get("v4_sf"), h["fp8_elem"])
    return kq, vq, h


def save_kv(path: str, kq, vq=None) -> int:
    """Write the packed form to a file; returns the number of bytes."""
    buf = pack_kv(kq, vq).cpu()
    buf.numpy().tofile(path)
    return buf.numel()


def load_kv(path: str, device=None) -> Tuple[object, object, dict]:
    """Read a file written by save_kv; with `device` the buffer is moved there in one copy before it is unpacked."""
    import numpy as np
    buf = torch.from_numpy(np.fromfile(path, dtype=np.uint8))
    if device is not None:
        buf = buf.to(device)
    return unpack_kv(buf)
