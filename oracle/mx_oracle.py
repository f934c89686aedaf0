"""CPU oracle for the diagonal-tiled mixed-precision (MXFP) attention path.

TEST INFRASTRUCTURE ONLY.  This module is a CPU restatement (eager PyTorch on
CPU tensors, fp32 arithmetic) of the algorithm implemented by the reference
project's ``ours/`` directory.  It exists so that the CUDA kernels can be checked
bit-for-bit (quantizer codes, scale codes, precision map) or within a stated
tolerance (attention / GEMM outputs).  Nothing in the shipped package imports it;
only the tests, the smoke entry and the benchmark's CPU-baseline leg do.

Pinning status
--------------
* MXFP4 quantizer, E8M0 scales of both MX quantizers, the int8 quantizer, the
  E2M1/E8M0 helper classes and the 2-D block-scaled GEMM emulation are PINNED:
  ``tests/golden/*.npz`` holds outputs of the reference's own code
  (``ours/quant_mxint8.py`` run under the Triton CPU interpreter,
  ``ours/mxfp.py`` and ``ours/block_scaled_matmul.py`` run eagerly) and
  ``tests/test_oracle_golden.py`` compares this file with them.
* MXFP8(E5M2) element codes: the reference casts with Triton's fp32->fp8e5
  conversion, which is round-to-nearest-even on the GPU; the CPU interpreter's
  cast is not faithful (drops the mantissa carry), so codes are pinned to
  torch's RNE ``.to(torch.float8_e5m2)`` and only the scale codes to the
  reference run.
* PARITY UNPINNED (no counterpart in the reference, restated from the format
  definitions): the E4M3 variant of the MXFP8 quantizer, the NVFP4 quantizer,
  the precision map (band rule), causal masking / GQA inside the MXFP kernel,
  the sequence-axis V quantizer and the re-quantised P mode.

Every function cites the reference file:line it follows.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

LOG2E = 1.44269504  # constant used by the reference, ours/quant_mxint8.py:494

# precision-map cell values
TILE_SKIP, TILE_FP8, TILE_FP4 = 0, 1, 2

_E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)


# --------------------------------------------------------------------------------------
# element / scale decoders  (ours/mxfp.py:44-77, :275-284)
# --------------------------------------------------------------------------------------
def decode_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """uint8 codes (S<<3|E<<1|M, one per byte) -> fp32.  ours/mxfp.py:44-77."""
    c = codes.to(torch.int64)
    mag = _E2M1_VALUES[c & 7]
    return torch.where((c & 8) != 0, -mag, mag)


def decode_e8m0(codes: torch.Tensor) -> torch.Tensor:
    """E8M0 -> fp32 = 2^(e-127); 255 -> NaN.  ours/mxfp.py:275-284."""
    e = codes.to(torch.float32)
    v = torch.pow(torch.tensor(2.0), e - 127.0)
    return torch.where(codes == 255, torch.full_like(v, float("nan")), v)


def decode_e5m2(codes: torch.Tensor) -> torch.Tensor:
    return codes.view(torch.float8_e5m2).to(torch.float32)


def decode_e4m3(codes: torch.Tensor) -> torch.Tensor:
    return codes.view(torch.float8_e4m3fn).to(torch.float32)


def encode_e2m1_rne(values: torch.Tensor) -> torch.Tensor:
    """fp32 -> E2M1 codes, round-to-nearest-even, saturating.  ours/mxfp.py:84-170.

    Ties between neighbours go to the candidate with mantissa bit 0; NaN/Inf
    saturate to 6; zeros keep their sign.
    """
    s = torch.signbit(values).to(torch.uint8)
    a = values.abs().to(torch.float32)
    a = torch.where(torch.isnan(a) | torch.isinf(a), torch.full_like(a, 6.0), a)
    # midpoints between consecutive candidates; "<=" goes down when the lower
    # candidate has an even mantissa (indices 0,2,4,6), "<" otherwise.
    idx = torch.zeros_like(a, dtype=torch.int64)
    mids = [0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0]
    for i, m in enumerate(mids):
        lower_even = (i % 2) == 0
        idx = idx + ((a > m) if lower_even else (a >= m)).to(torch.int64)
    return ((s << 3) | idx.to(torch.uint8)).to(torch.uint8)


def encode_e8m0(values: torch.Tensor) -> torch.Tensor:
    """fp32 -> E8M0 = clamp(floor(log2 v)+127, 0, 254); <=0/NaN/Inf -> 255.
    ours/mxfp.py:286-307."""
    v = values.to(torch.float32)
    bad = torch.isnan(v) | torch.isinf(v) | (v <= 0)
    e = torch.floor(torch.log2(torch.where(bad, torch.ones_like(v), v))) + 127.0
    e = e.to(torch.int32).clamp(0, 254).to(torch.uint8)
    return torch.where(bad, torch.full_like(e, 255), e)


def pack_e2m1(codes: torch.Tensor) -> torch.Tensor:
    """Two codes per byte along the last axis, low nibble first.  ours/mxfp.py:172-205."""
    lo = codes[..., 0::2]
    hi = codes[..., 1::2]
    return ((hi << 4) | lo).to(torch.uint8)


def unpack_e2m1(packed: torch.Tensor) -> torch.Tensor:
    """Inverse of :func:`pack_e2m1`.  ours/mxfp.py:207-236."""
    lo = packed & 0xF
    hi = (packed >> 4) & 0xF
    return torch.stack((lo, hi), dim=-1).reshape(*packed.shape[:-1], packed.shape[-1] * 2)


# --------------------------------------------------------------------------------------
# MX block quantizers  (ours/quant_mxint8.py)
# --------------------------------------------------------------------------------------
def _mx_prepare(x: torch.Tensor, s: float, emax: int, vec: int = 32, min_sh: Optional[float] = None):
    """Shared front end of the MX quantizers: fp32 multiply by the fp32 scalar ``s``,
    32-element groups along the last axis, shared exponent and E8M0 code.
    ours/quant_mxint8.py:295-309 (fp4) / :183-197 (fp8), scale code :347-351 / :215-219.
    ``min_sh`` (not in the reference): lower clamp of the shared exponent, for operands such as softmax
    probabilities whose blocks can be smaller than the smallest E8M0 scale.
    """
    d = x.shape[-1]
    assert d % vec == 0
    xf = x.to(torch.float32) * torch.tensor(s, dtype=torch.float32)
    g = xf.reshape(*x.shape[:-1], d // vec, vec)
    amax = g.abs().amax(dim=-1, keepdim=True)
    sh = torch.floor(torch.log2(amax)) - float(emax)
    if min_sh is not None:
        sh = torch.clamp(sh, min=min_sh)
    scale = torch.exp2(sh)
    y = g / scale
    e = torch.floor(torch.log2(scale)) + 127.0
    e8 = torch.clamp(e, 0, 254)
    e8 = torch.where(torch.isnan(e8), torch.zeros_like(e8), e8).to(torch.uint8).squeeze(-1)
    return y, e8, amax


def quant_mxfp4_side(x: torch.Tensor, s: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """One side (Q or K) of ``quant_mxfp4``: uint8 E2M1 codes (one per byte) and E8M0
    scales per 32 elements of the last axis.  ours/quant_mxint8.py:276-351.

    The element rule is the reference's own (not round-to-nearest-even):
    sign = not (y >= 0); exp by thresholds 1, 2, 4 (:321-323); mantissa bit set iff
    the value normalised by 2^(exp-1) exceeds 1.25, or 0.25 when exp == 0 (:326-328).
    A block whose amax is 0 produces NaN (0/0), hence sign 1, exp 0, mantissa 0 = code 8
    and scale code 0.
    """
    y, e8, _ = _mx_prepare(x, s, emax=3)
    y = torch.clamp(y, -6.0, 6.0)
    sign = torch.where(y >= 0, 0, 1)
    a = y.abs()
    exp = torch.where(a >= 2.0, torch.where(a >= 4.0, 3, 2), torch.where(a >= 1.0, 1, 0))
    norm = a / torch.exp2((exp - 1).to(torch.float32))
    man = torch.where(exp == 0, torch.where(norm > 0.25, 1, 0), torch.where(norm > 1.25, 1, 0))
    code = ((sign << 3) | (exp << 1) | man).to(torch.uint8)
    return code.reshape(x.shape), e8


def quant_mxfp8_side(x: torch.Tensor, s: float = 1.0, elem: str = "e5m2",
                     zero_block_code: Optional[int] = 0, min_sh: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """One side of ``quant_mxfp8e5``: fp8 codes (as uint8) + E8M0 scales.
    ours/quant_mxint8.py:164-221: emax_elem = 7 (:191), clamp +-57344 (:203), cast to E5M2 (:205).

    ``elem="e4m3"`` is the variant the reference does not have (PARITY UNPINNED):
    emax 8, clamp +-448, cast to float8_e4m3fn.

    All-zero blocks: the reference divides 0 by 0 and stores the NaN pattern; the CUDA
    path stores ``zero_block_code`` (0) instead, because a NaN element would poison the
    attention row.  Pass ``zero_block_code=None`` for the reference behaviour.
    """
    if elem == "e5m2":
        emax, lim, dt = 7, 57344.0, torch.float8_e5m2
    elif elem == "e4m3":
        emax, lim, dt = 8, 448.0, torch.float8_e4m3fn
    else:
        raise ValueError(elem)
    y, e8, amax = _mx_prepare(x, s, emax=emax, min_sh=min_sh)
    yq = torch.clamp(y, -lim, lim).to(dt).view(torch.uint8)
    if zero_block_code is not None:
        yq = torch.where(amax == 0, torch.full_like(yq, zero_block_code), yq)
    return yq.reshape(x.shape), e8


def rope_rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding in the rotate-half convention (what transformers applies to Q and K before the attention
    call the reference patches, evaluate/llama/modify_sparse_attn.py): with x1 / x2 the halves of the last axis,
    y1 = x1 cos - x2 sin, y2 = x2 cos + x1 sin.  x [B,H,L,D]; cos / sin fp32 [L,D/2] or [B,L,D/2].  fp32 products and
    sum (no fused multiply-add), result in x's dtype.  No reference counterpart with this rounding: unpinned."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    if cos.dim() == 3:
        cos, sin = cos.unsqueeze(1), sin.unsqueeze(1)
    y1 = x1 * cos - x2 * sin
    y2 = x2 * cos + x1 * sin
    return torch.cat([y1, y2], dim=-1).to(x.dtype)


def rope_angles(L: int, D: int, base: float = 10000.0, offset: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos / sin fp32 [L, D/2] of position * base^(-2i/D), positions offset .. offset+L-1."""
    inv = base ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)
    ang = torch.arange(offset, offset + L, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang), torch.sin(ang)


def q_side_scale(head_dim: int, sm_scale: Optional[float] = None) -> float:
    """Softmax scale folded into Q by every quantizer: sm_scale * log2(e), passed to the
    kernel as an fp32 scalar.  ours/quant_mxint8.py:479-480, :494."""
    if sm_scale is None:
        sm_scale = head_dim ** -0.5
    return float(torch.tensor(sm_scale * LOG2E, dtype=torch.float32))


def quant_mxfp4(q, k, BLKQ=128, BLKK=64, sm_scale=None):
    """ours/quant_mxint8.py:453-512 (HND layout)."""
    qc, qs = quant_mxfp4_side(q, q_side_scale(q.shape[-1], sm_scale))
    kc, ks = quant_mxfp4_side(k, 1.0)
    return qc, qs, kc, ks


def quant_mxfp8e5(q, k, BLKQ=128, BLKK=64, sm_scale=None):
    """ours/quant_mxint8.py:223-272 (HND layout)."""
    qc, qs = quant_mxfp8_side(q, q_side_scale(q.shape[-1], sm_scale))
    kc, ks = quant_mxfp8_side(k, 1.0)
    return qc, qs, kc, ks


def quant_fpxint8_side(x: torch.Tensor, s: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-32 int8 quantizer.  ours/quant_mxint8.py:21-58: scale = amax/127 + 1e-7 (:46-47),
    round half away from zero by adding 0.5*sign and truncating (:51-52); the stored
    scale goes through an E5M2 round trip (:57)."""
    d = x.shape[-1]
    xf = x.to(torch.float32) * torch.tensor(s, dtype=torch.float32)
    g = xf.reshape(*x.shape[:-1], d // 32, 32)
    sc = g.abs().amax(dim=-1, keepdim=True) / 127.0
    sc = sc + 0.0000001
    y = g / sc
    y = y + 0.5 * torch.where(y >= 0, 1.0, -1.0)
    codes = y.to(torch.int8)  # C-style truncation
    sc8 = sc.squeeze(-1).to(torch.float8_e5m2).to(torch.float32)
    return codes.reshape(x.shape), sc8


def quant_fpxint8(q, k, BLKQ=128, BLKK=64, sm_scale=None):
    """ours/quant_mxint8.py:61-114."""
    qc, qs = quant_fpxint8_side(q, q_side_scale(q.shape[-1], sm_scale))
    kc, ks = quant_fpxint8_side(k, 1.0)
    return qc, qs, kc, ks


def quant_nvfp4(x: torch.Tensor, s: float = 1.0):
    """NVFP4 (PARITY UNPINNED; the reference has only the GEMM mode string,
    ours/block_scaled_matmul.py:321-324): 16-element blocks, E4M3 block scales, one fp32
    tensor scale.  ts = amax_tensor/(6*448); block scale = e4m3_rne(amax_blk/(6*ts));
    codes = E2M1 RNE of x/(scale*ts)."""
    xf = x.to(torch.float32) * torch.tensor(s, dtype=torch.float32)
    d = x.shape[-1]
    g = xf.reshape(*x.shape[:-1], d // 16, 16)
    tmax = xf.abs().amax()
    ts = (tmax / torch.tensor(6.0 * 448.0)).to(torch.float32)
    ts = torch.where(ts == 0, torch.ones_like(ts), ts)
    bmax = g.abs().amax(dim=-1, keepdim=True)
    sc8 = torch.clamp(bmax / (6.0 * ts), max=448.0).to(torch.float8_e4m3fn)
    scf = sc8.to(torch.float32) * ts
    y = torch.where(scf == 0, torch.zeros_like(g), g / torch.where(scf == 0, torch.ones_like(scf), scf))
    codes = encode_e2m1_rne(y)
    return codes.reshape(x.shape), sc8.view(torch.uint8).squeeze(-1), ts


# --------------------------------------------------------------------------------------
# scale-factor tile layout  (ours/mxfp_attn_kernel.py:56-57, ours/block_scaled_matmul.py:382-384)
# --------------------------------------------------------------------------------------
def swizzle_scales(scales: torch.Tensor, pad_code: int = 127) -> torch.Tensor:
    """[..., L, C] row-major block scales -> [..., ceil(L/128), ceil(C/4), 32, 4, 4] where
    element (row r, column c) of a 128x4 chunk sits at [r % 32][r // 32][c], i.e. byte
    ``(r%32)*16 + (r//32)*4 + c`` of a 512-byte tile.  ours/mxfp_attn_kernel.py:56-57.
    Rows/columns beyond the tensor are filled with ``pad_code`` (E8M0 1.0)."""
    *lead, L, C = scales.shape
    Lp, Cp = -(-L // 128) * 128, -(-C // 4) * 4
    s = torch.full((*lead, Lp, Cp), pad_code, dtype=scales.dtype)
    s[..., :L, :C] = scales
    n = len(lead)
    s = s.reshape(*lead, Lp // 128, 4, 32, Cp // 4, 4)
    perm = list(range(n)) + [n + 0, n + 3, n + 2, n + 1, n + 4]
    return s.permute(*perm).contiguous()


def unswizzle_scales(sw: torch.Tensor, L: int, C: int) -> torch.Tensor:
    """Inverse of :func:`swizzle_scales` (ours/block_scaled_matmul.py:382-384)."""
    *lead, nl, nc, _, _, _ = sw.shape
    n = len(lead)
    perm = list(range(n)) + [n + 0, n + 3, n + 2, n + 1, n + 4]
    s = sw.permute(*perm).reshape(*lead, nl * 128, nc * 4)
    return s[..., :L, :C].contiguous()


# --------------------------------------------------------------------------------------
# block-scaled GEMM emulation  (ours/block_scaled_matmul.py:374-392)
# --------------------------------------------------------------------------------------
def dequant(codes: torch.Tensor, scales: torch.Tensor, fmt: str, vec: int = 32,
            tensor_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """codes [.., L, D] (one per byte) x scales [.., L, D/vec] -> fp32 [.., L, D]."""
    if fmt in ("fp4", "mxfp4", "nvfp4"):
        v = decode_e2m1(codes)
    elif fmt in ("fp8e5", "e5m2", "mxfp8"):
        v = decode_e5m2(codes)
    elif fmt in ("fp8e4", "e4m3"):
        v = decode_e4m3(codes)
    else:
        raise ValueError(fmt)
    if fmt == "nvfp4":
        sc = decode_e4m3(scales)
        if tensor_scale is not None:
            sc = sc * tensor_scale
    else:
        sc = decode_e8m0(scales)
    return v * sc.repeat_interleave(vec, dim=-1)


def gemm_block_scaled(a_codes, a_scales, b_codes, b_scales, fmt_a: str, fmt_b: str,
                      vec: int = 32, a_ts=None, b_ts=None) -> torch.Tensor:
    """C[M,N] = (A*sa) @ (B*sb)^T in fp32.  ours/block_scaled_matmul.py:387-392."""
    a = dequant(a_codes, a_scales, fmt_a, vec, a_ts)
    b = dequant(b_codes, b_scales, fmt_b, vec, b_ts)
    return a @ b.transpose(-1, -2)


# --------------------------------------------------------------------------------------
# precision map (no counterpart in the reference; PARITY UNPINNED)
# --------------------------------------------------------------------------------------
def precision_map_band(n_q_tiles: int, n_k_tiles: int, causal: bool, band: int = 1,
                       off_tiles: int = 0) -> torch.Tensor:
    """uint8 [n_q_tiles, n_k_tiles]: FP8 iff |i-j| < band, else FP4; causal => j>i SKIP.
    ``off_tiles`` = (Skv - S) / tile shifts the diagonal when the queries are the last S of Skv
    positions.  The causal tile range follows the two-stage loop of ours/online_routing.py:68-77."""
    i = torch.arange(n_q_tiles)[:, None] + off_tiles
    j = torch.arange(n_k_tiles)[None, :]
    m = torch.where((i - j).abs() < band, TILE_FP8, TILE_FP4).to(torch.uint8)
    if causal:
        m = torch.where(j > i, torch.tensor(TILE_SKIP, dtype=torch.uint8), m)
    return m


def router_statistic(s_tile: torch.Tensor) -> torch.Tensor:
    """sum_rows(max_cols S) / rows of one score tile.  ours/mxfp_attn_kernel.py:272-280."""
    return s_tile.amax(dim=-1).sum(dim=-1) / s_tile.shape[-2]


def router_statistic_map(q: torch.Tensor, k: torch.Tensor, *, causal: bool, sm_scale: Optional[float] = None,
                         tile: int = 128) -> torch.Tensor:
    """float32 [B,Hq,nq,nk]: router_statistic of every visible tile of S = dequant(Q4) @ dequant(K4)^T (the
    reference quantizer's MXFP4 operands, log2 domain; ours/mxfp_attn_kernel.py:262-280).  Keys beyond the
    end and, if causal, above the query are left out of the row maximum; a row without a visible key counts
    as 0; cells entirely above the causal diagonal hold 0.  The masking is this build's: the reference's
    statistic exists only in its non-causal kernel."""
    B, Hq, S, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    sq = q_side_scale(D, sm_scale)
    qc, qs = quant_mxfp4_side(q, sq)
    kc, ks = quant_mxfp4_side(k, 1.0)
    qd = dequant(qc, qs, "fp4").float()
    kd = dequant(kc, ks, "fp4").float()
    nq, nk = -(-S // tile), -(-Skv // tile)
    off = Skv - S
    stat = torch.zeros((B, Hq, nq, nk), dtype=torch.float32)
    rows = torch.arange(S)
    cols = torch.arange(Skv)
    vis = (cols[None, :] <= rows[:, None] + off) if causal else torch.ones((S, Skv), dtype=torch.bool)
    ninf = torch.tensor(float("-inf"))
    n_rows = torch.clamp(S - torch.arange(nq) * tile, max=tile).to(torch.float32)       # valid rows per query tile
    for b in range(B):
        for h in range(Hq):
            s = qd[b, h] @ kd[b, h // (Hq // Hkv)].T
            s = torch.where(vis, s, ninf)
            s = torch.nn.functional.pad(s, (0, nk * tile - Skv, 0, nq * tile - S), value=float("-inf"))
            mx = s.view(nq, tile, nk, tile).amax(dim=-1)                                   # [nq, tile, nk] row maxima
            mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)                   # no visible key: counts 0
            stat[b, h] = mx.sum(dim=1) / n_rows[:, None]
    return stat


def precision_map_online(stat: torch.Tensor, S: int, Skv: int, *, causal: bool, band: int = 1, tau: float = 1.0,
                         tile: int = 128, skip_thresh: Optional[float] = None) -> torch.Tensor:
    """uint8 [B,Hq,nq,nk]: the band map, plus FP8 for every other visible tile with
    stat[i,j] >= stat[i,0] * tau (first key tile = the reference statistic, ours/mxfp_attn_kernel.py:272-276)."""
    B, Hq, nq, nk = stat.shape
    base = precision_map_band(nq, nk, causal, band, (Skv - S) // tile)
    if causal:
        # tiles the (end-aligned, possibly ragged) diagonal leaves entirely masked
        i = torch.arange(nq)[:, None]
        j = torch.arange(nk)[None, :]
        last_q = torch.clamp((i + 1) * tile - 1, max=S - 1)
        base = torch.where(j * tile > last_q + (Skv - S), torch.tensor(TILE_SKIP, dtype=torch.uint8), base)
    promote = stat >= stat[..., :1] * tau
    m = base.expand(B, Hq, nq, nk).clone()
    m[(m == TILE_FP4) & promote] = TILE_FP8
    if skip_thresh is not None:
        # the reference's router: a tile is processed iff it is the first one or stat >= sink * skip_thresh
        # (ours/mxfp_attn_kernel.py:276-280); tiles inside the band are never dropped here
        keep = stat >= stat[..., :1] * skip_thresh
        keep[..., 0] = True
        outside = base.expand(B, Hq, nq, nk) == TILE_FP4
        m[outside & ~keep] = TILE_SKIP
    return m


# --------------------------------------------------------------------------------------
# V operand preparation for P.V (sequence-axis blocks; PARITY UNPINNED)
# --------------------------------------------------------------------------------------
def quant_v_seq(v: torch.Tensor, fmt: str):
    """Quantise V [.., S, D] with 32-element blocks running along the SEQUENCE axis (the
    contraction axis of P.V).  Returns codes [.., D, S] (transposed, one per byte) and
    scales [.., D, S/32].  RNE element rule for fp4 (OCP MX), RNE cast for fp8."""
    vt = v.transpose(-1, -2).contiguous()
    if vt.shape[-1] % 32:                          # a ragged tail is zero-padded to a whole block
        vt = torch.nn.functional.pad(vt.float(), (0, 32 - vt.shape[-1] % 32))
    if fmt == "fp4":
        y, e8, amax = _mx_prepare(vt, 1.0, emax=2)
        codes = encode_e2m1_rne(torch.where(amax == 0, torch.zeros_like(y), y)).reshape(vt.shape)
        return codes, e8
    return quant_mxfp8_side(vt, 1.0, "e4m3" if fmt == "fp8e4" else "e5m2")


# --------------------------------------------------------------------------------------
# fused attention forward emulation
# --------------------------------------------------------------------------------------
def attention_mxfp(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool,
                   tile: int = 128, band: int = 1, prec_map: Optional[torch.Tensor] = None,
                   fp8_elem: str = "e5m2", pv_mode: str = "fp16", sm_scale: Optional[float] = None,
                   out_dtype: torch.dtype = torch.float32, uniform: Optional[str] = None,
                   return_scores: bool = False, fp4_kind: str = "mxfp4"):
    """Emulation of the fused forward, composed from the reference's pieces.

    q [B,Hq,S,D], k/v [B,Hkv,Skv,D] (bf16/fp16/fp32 CPU tensors).
    1. Q and K are quantised to BOTH MXFP8 and MXFP4 with the reference quantizers
       (softmax scale * log2e folded into Q; ours/quant_mxint8.py:494).
    2. S = (Qd*sq) @ (Kd*sk)^T in fp32 (ours/block_scaled_matmul.py:387-392), tile by tile
       from the FP8 or the FP4 operands as the precision map says; SKIP tiles and, on
       causal diagonal tiles, keys above the query are masked (the -1e6 add of
       ours/online_routing.py:113-115 is -inf here).
    3. m = rowmax, P = exp2(S - m), l = sum P from the unrounded fp32 P
       (ours/mxfp_attn_kernel.py:320-328).
    4. pv_mode "fp16": P -> fp16, V -> fp16, O = P@V (:339-340).  pv_mode "requant": P =
       exp2(S - ceil(m)) is block-quantised per 32 keys in the tile's format (MXFP8 by the
       rule of ours/quant_mxint8.py:164-221, MXFP4 by the OCP rule with round-to-nearest-even)
       and V per 32 keys along the sequence (no counterpart in the reference).
    5. O = O / l (:355), cast to out_dtype.
    GQA: kv head = q head // (Hq/Hkv) (ours/online_routing.py:160).
    ``uniform`` = "fp8" | "fp4" forces one format for every non-skipped tile.
    ``fp4_kind`` = "nvfp4": the FP4 tiles of S come from NVFP4 operands (quant_nvfp4 over the whole of Q and
    of K): S = (codes*block scales) @ (codes*block scales)^T in fp32, then times fp32(ts_q * ts_k).  P.V keeps
    the MX formats.  PARITY UNPINNED (no NVFP4 in the reference).
    """
    B, Hq, S, D = q.shape
    _, Hkv, Skv, _ = k.shape
    grp = Hq // Hkv
    sq = q_side_scale(D, sm_scale)
    q8c, q8s = quant_mxfp8_side(q, sq, fp8_elem)
    q4c, q4s = quant_mxfp4_side(q, sq)
    k8c, k8s = quant_mxfp8_side(k, 1.0, fp8_elem)
    k4c, k4s = quant_mxfp4_side(k, 1.0)
    f8 = "fp8e5" if fp8_elem == "e5m2" else "fp8e4"
    Q8, Q4 = dequant(q8c, q8s, f8), dequant(q4c, q4s, "fp4")
    K8, K4 = dequant(k8c, k8s, f8), dequant(k4c, k4s, "fp4")
    s4_scale = None
    if fp4_kind == "nvfp4":
        qc, qs, qts = quant_nvfp4(q, sq)
        kc, ks, kts = quant_nvfp4(k, 1.0)
        Q4 = decode_e2m1(qc) * decode_e4m3(qs).repeat_interleave(16, dim=-1)
        K4 = decode_e2m1(kc) * decode_e4m3(ks).repeat_interleave(16, dim=-1)
        s4_scale = (qts.double() * kts.double()).to(torch.float32)
    elif fp4_kind != "mxfp4":
        raise ValueError(fp4_kind)
    nq, nk = -(-S // tile), -(-Skv // tile)
    if prec_map is None:
        prec_map = precision_map_band(nq, nk, causal, band, (Skv - S) // tile)
        if uniform is not None:
            code = TILE_FP8 if uniform == "fp8" else TILE_FP4
            prec_map = torch.where(prec_map == TILE_SKIP, prec_map,
                                   torch.tensor(code, dtype=torch.uint8))
    if prec_map.dim() == 2:
        prec_map = prec_map.expand(B, Hq, nq, nk)
    vf = v.to(torch.float16).to(torch.float32) if pv_mode == "fp16" else v.to(torch.float32)
    out = torch.empty(B, Hq, S, D, dtype=torch.float32)
    scores = torch.empty(B, Hq, S, Skv, dtype=torch.float32) if return_scores else None
    for b in range(B):
        for h in range(Hq):
            hk = h // grp
            pm = prec_map[b, h]
            cell = pm.repeat_interleave(tile, 0).repeat_interleave(tile, 1)[:S, :Skv]
            S8 = Q8[b, h] @ K8[b, hk].T
            S4 = Q4[b, h] @ K4[b, hk].T
            if s4_scale is not None:
                S4 = S4 * s4_scale
            sc = torch.where(cell == TILE_FP8, S8, S4)
            mask = cell == TILE_SKIP
            if causal:
                mask = mask | (torch.arange(Skv)[None, :] > torch.arange(S)[:, None] + (Skv - S))
            sc = sc.masked_fill(mask, float("-inf"))
            if return_scores:
                scores[b, h] = sc
            m = sc.amax(dim=-1, keepdim=True)
            if pv_mode == "requant":
                # P is block-quantised with power-of-two scales, so an integral change of the
                # reference changes scale codes only; the integral reference makes the element
                # codes independent of how an implementation tracks the running maximum.
                m = torch.ceil(m)
            p = torch.exp2(sc - m)
            l = p.sum(dim=-1, keepdim=True)
            if pv_mode == "fp16":
                o = p.to(torch.float16).to(torch.float32) @ vf[b, hk]
            elif pv_mode == "requant":
                o = _pv_requant(p, v[b, hk], cell, tile, f8)
            else:
                raise ValueError(pv_mode)
            out[b, h] = o / l
    out = out.to(out_dtype)
    return (out, scores) if return_scores else out


def _pv_requant(p: torch.Tensor, v: torch.Tensor, cell: torch.Tensor, tile: int, f8: str):
    """P block-quantised per 32 keys (format of the tile) times V block-quantised per 32
    keys along the sequence.  PARITY UNPINNED."""
    S, Skv = p.shape
    if Skv % 32:                                   # masked tail keys have P = 0: pad to a whole block
        p = torch.nn.functional.pad(p, (0, 32 - Skv % 32))
        cell = torch.nn.functional.pad(cell, (0, 32 - Skv % 32), value=int(cell[0, -1]))
    v8c, v8s = quant_v_seq(v, f8)
    v4c, v4s = quant_v_seq(v, "fp4")
    V8 = dequant(v8c, v8s, f8).T
    V4 = dequant(v4c, v4s, "fp4").T
    # the kernel clamps P's shared exponent at -126 (probabilities below that carry no weight)
    p8c, p8s = quant_mxfp8_side(p, 1.0, "e5m2" if f8 == "fp8e5" else "e4m3", min_sh=-126.0)
    y, e8, amax = _mx_prepare(p, 1.0, emax=2, min_sh=-126.0)
    p4c = encode_e2m1_rne(torch.where(amax == 0, torch.zeros_like(y), y)).reshape(p.shape)
    P8, P4 = dequant(p8c, p8s, f8), dequant(p4c, e8, "fp4")
    is8 = cell == TILE_FP8
    o = torch.where(is8, P8, torch.zeros_like(P8)) @ V8
    o = o + torch.where(is8, torch.zeros_like(P4), P4) @ V4
    return o


def attention_fp32(q, k, v, causal: bool, sm_scale: Optional[float] = None) -> torch.Tensor:
    """Plain fp32 softmax attention (the 'bf16 SDPA' error reference), GQA aware."""
    B, Hq, S, D = q.shape
    Hkv = k.shape[1]
    if sm_scale is None:
        sm_scale = D ** -0.5
    kf = k.float().repeat_interleave(Hq // Hkv, dim=1)
    vf = v.float().repeat_interleave(Hq // Hkv, dim=1)
    sc = (q.float() @ kf.transpose(-1, -2)) * sm_scale
    if causal:
        Skv = k.shape[2]
        mask = torch.arange(Skv)[None, :] > torch.arange(S)[:, None] + (Skv - S)
        sc = sc.masked_fill(mask, float("-inf"))
    return torch.softmax(sc, dim=-1) @ vf


def parity_metrics(x: torch.Tensor, ref: torch.Tensor) -> dict:
    """Cosine similarity, relative L1 (spas_sage_attn/utils.py:25-36) and relative L2."""
    a, b = x.double().flatten(), ref.double().flatten()
    cos = float((a @ b) / (a.norm() * b.norm() + 1e-300))
    l1 = float((a - b).abs().sum() / (b.abs().sum() + 1e-300))
    l2 = float((a - b).norm() / (b.norm() + 1e-300))
    return {"cos": cos, "rel_l1": l1, "rel_l2": l2, "max_abs": float((a - b).abs().max())}


# --------------------------------------------------------------------------------------
# seeded synthetic inputs of the benchmark configurations
# --------------------------------------------------------------------------------------
def make_qkv(seed: int, B: int, Hq: int, Hkv: int, S: int, D: int, outliers: int = 0,
             dtype=torch.bfloat16):
    """fp32 randn in the order Q, K, V from a CPU generator, cast to ``dtype``; optional
    ``outliers`` K channels (fixed seeded indices, drawn after V) scaled x20."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    q = torch.randn(B, Hq, S, D, generator=g)
    k = torch.randn(B, Hkv, S, D, generator=g)
    v = torch.randn(B, Hkv, S, D, generator=g)
    if outliers:
        idx = torch.randperm(D, generator=g)[:outliers]
        k[..., idx] *= 20.0
    return q.to(dtype), k.to(dtype), v.to(dtype)


def make_video_qkv(seed: int, H: int, grid: Tuple[int, int, int], D: int, dtype=torch.bfloat16):
    """Synthetic stand-in for video-DiT self-attention inputs: B=1, S = f*h*w tokens laid out row-major over
    the (f, h, w) latent grid.  Q, K, V are N(0,1) (drawn in that order from one CPU generator) plus, each
    separately, a smooth component low[t, c] = (2/8) * sum_{i<8} sin(2*pi*<w_i, pos(t)> + phi[i, c]) with integer
    wave vectors w_i in {0..3}^3, pos(t) = (f/F, h/Hh, w/W) and phases phi ~ U[0, 2*pi) per head and channel,
    which correlates neighbouring tokens."""
    F, Hh, W = grid
    S = F * Hh * W
    g = torch.Generator(device="cpu").manual_seed(seed)
    base = [torch.randn(1, H, S, D, generator=g) for _ in range(3)]
    ff, hh, ww = torch.meshgrid(torch.arange(F) / F, torch.arange(Hh) / Hh, torch.arange(W) / W, indexing="ij")
    pos = torch.stack([ff.reshape(-1), hh.reshape(-1), ww.reshape(-1)], dim=-1)          # [S, 3]
    out = []
    for x in base:
        wv = torch.randint(0, 4, (8, 3), generator=g).to(torch.float32)
        phi = torch.rand(8, H, 1, D, generator=g) * (2 * torch.pi)
        arg = 2 * torch.pi * (pos @ wv.T)                                                  # [S, 8]
        low = torch.zeros(H, S, D)
        for i in range(8):
            low += torch.sin(arg[:, i].reshape(1, S, 1) + phi[i])
        out.append((x + 0.25 * low.unsqueeze(0)).to(dtype))
    return tuple(out)
