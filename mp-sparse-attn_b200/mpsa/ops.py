"""Tensor-level operations on top of the C-ABI.  torch supplies device memory and streams; all
arithmetic runs in the hand-written sm_100a kernels of libmpsa.so."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib

TILE_SKIP, TILE_FP8, TILE_FP4 = 0, 1, 2
LOG2E = 1.44269504  # ours/quant_mxint8.py:494

_IN_DTYPE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_OUT_DTYPE = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2, torch.float8_e5m2: 3}
_FP8_QUANT = {"e5m2": 1, "e4m3": 2}
_FP8_DESC = {"e5m2": 1, "e4m3": 0}
_status = {}
_last_range_flag = None


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("mpsa operations need CUDA tensors; there is no CPU path")


def status_word(device) -> torch.Tensor:
    """Per-device int32 word the kernels write when one of their bounded waits expires.  It lives in pinned host memory
    (reachable from the device under unified addressing: the kernels touch it only after a wait has already failed
    1024 probes), so the host can look at it before every launch without synchronising."""
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status:
        _status[key] = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _status[key]


_WAIT_NAMES = {1: "TMA bytes", 2: "tensor-core commit", 3: "pipeline hand-off"}


def _raise_if_failed(device):
    """Raise if a kernel that has already finished on `device` recorded an expired wait.  No synchronisation: called by
    the wrappers before they launch, so that a failure surfaces at the next call at the latest instead of being carried
    along silently (a kernel that finds the word set gives up its own long waits too)."""
    w = status_word(device)
    code = int(w[0])
    if code != 0:
        w.zero_()
        raise _lib.MpsaError(f"a kernel gave up waiting (status {code}: {_WAIT_NAMES.get(code, '?')})")


def check_status(device=None):
    """Synchronise the device and raise if a kernel recorded an expired wait (1 TMA, 2 MMA, 3 pipeline)."""
    dev = torch.cuda.current_device() if device is None else device
    torch.cuda.synchronize(dev)
    _raise_if_failed(dev)


def q_side_scale(head_dim: int, sm_scale: Optional[float] = None) -> float:
    """sm_scale * log2(e), the factor the reference folds into Q (ours/quant_mxint8.py:479-494)."""
    if sm_scale is None:
        sm_scale = head_dim ** -0.5
    return sm_scale * LOG2E


@dataclass
class QuantizedOperand:
    """One side (Q or K) quantised for the tensor cores; any field may be None if not requested."""
    fp8: Optional[torch.Tensor] = None          # uint8 [B,H,L,D]
    fp8_sf: Optional[torch.Tensor] = None       # uint8 [B,H,ceil(L/128),ceil(D/128),512]
    fp4: Optional[torch.Tensor] = None          # uint8 [B,H,L,D/2] packed
    fp4_sf: Optional[torch.Tensor] = None
    fp8_scales: Optional[torch.Tensor] = None   # uint8 [B,H,L,D/32] row-major (reference format)
    fp4_scales: Optional[torch.Tensor] = None
    fp4_unpacked: Optional[torch.Tensor] = None  # uint8 [B,H,L,D] one code per byte (reference format)
    fp8_elem: str = "e5m2"
    fp4_kind: str = "mxfp4"                     # "nvfp4": fp4_sf holds E4M3 scale tiles [B,H,ceil(L/128),D/64,512]
    fp4_ts: Optional[torch.Tensor] = None       # NVFP4: the fp32 tensor scale (1-element tensor)


def _bhld(x: torch.Tensor, tensor_layout: str):
    """Logical (B,H,L,D) view parameters of a HND or NHD tensor: sizes and element strides."""
    if x.dim() != 4:
        raise ValueError("expected a 4-D tensor")
    if x.stride(-1) != 1:
        x = x.contiguous()
    if tensor_layout == "HND":
        B, H, L, D = x.shape
        sb, sh, sl = x.stride(0), x.stride(1), x.stride(2)
    elif tensor_layout == "NHD":
        B, L, H, D = x.shape
        sb, sh, sl = x.stride(0), x.stride(2), x.stride(1)
    else:
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    return x, (B, H, L, D), (sb, sh, sl)


def column_mean(x: torch.Tensor, tensor_layout: str = "HND") -> torch.Tensor:
    """Mean over the sequence, fp32 [B,H,D] holding values rounded to x's dtype: the vector "smooth K" subtracts
    (ours/mxfp_attn_kernel.py:33-34)."""
    _require_cuda(x)
    if x.dtype not in _IN_DTYPE:
        raise ValueError(f"unsupported input dtype {x.dtype}")
    x, (B, H, L, D), (sb, sh, sl) = _bhld(x, tensor_layout)
    lib = _lib.load()
    n = lib.mpsa_col_mean_scratch_floats(B, H, L, D)
    mean = torch.empty((B, H, D), dtype=torch.float32, device=x.device)
    scratch = torch.empty(n, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = lib.mpsa_col_mean(x.data_ptr(), _IN_DTYPE[x.dtype], B, H, L, D, sb, sh, sl, mean.data_ptr(), scratch.data_ptr(),
                               n, _stream())
    _lib.check(rc)
    return mean


def quantize_mx(x: torch.Tensor, scale: float = 1.0, *, want_fp8=True, want_fp4=True, reference_format=False,
                kernel_format=True, fp8_elem="e5m2", tensor_layout="HND", center=None, rope=None) -> QuantizedOperand:
    """Quantise one operand along its last axis in 32-element MX blocks (one kernel launch).

    reference_format: emit what ours/quant_mxint8.py returns (fp4 one code per byte, row-major
    scales, shaped like the input).  kernel_format: emit packed fp4 and 128x4 scale tiles.
    center: optional fp32 [B,H,D] from column_mean, subtracted from every row before quantising.
    rope: optional (cos, sin), fp32 [L, D/2] or [B, L, D/2]: the rotary embedding (rotate-half convention) is applied to
    every row first, in the same pass (D 64 or 128)."""
    _require_cuda(x)
    if x.dtype not in _IN_DTYPE:
        raise ValueError(f"unsupported input dtype {x.dtype}")
    x, (B, H, L, D), (sb, sh, sl) = _bhld(x, tensor_layout)
    dev = x.device
    out = QuantizedOperand(fp8_elem=fp8_elem)
    u8 = dict(dtype=torch.uint8, device=dev)
    nl, nd = -(-L // 128), -(-D // 128)
    o8 = (0, 0, 0)
    o4 = (0, 0, 0)

    def _strides(t):
        return (t.stride(0), t.stride(1), t.stride(2)) if tensor_layout == "HND" else \
            (t.stride(0), t.stride(2), t.stride(1))

    if want_fp8:
        out.fp8 = torch.empty(x.shape, **u8)
        o8 = _strides(out.fp8)
        if reference_format:
            out.fp8_scales = torch.empty((B, H, L, D // 32), **u8)
        if kernel_format:
            out.fp8_sf = torch.empty((B, H, nl, nd, 512), **u8)
    if want_fp4:
        if reference_format:
            out.fp4_unpacked = torch.empty(x.shape, **u8)
            o4 = _strides(out.fp4_unpacked)
            out.fp4_scales = torch.empty((B, H, L, D // 32), **u8)
        if kernel_format:
            out.fp4 = torch.empty((B, H, L, D // 2), **u8)
            out.fp4_sf = torch.empty((B, H, nl, nd, 512), **u8)
    outs = (_ptr(out.fp8), *o8, _ptr(out.fp4_unpacked), *o4, _ptr(out.fp8_scales), _ptr(out.fp4_scales),
            _ptr(out.fp4), _ptr(out.fp8_sf), _ptr(out.fp4_sf), _stream())
    with torch.cuda.device(dev):
        if rope is not None:
            cos, sin = rope
            if center is not None:
                raise ValueError("rope and center do not combine: the mean would have to be that of the rotated tensor")
            if cos.shape != sin.shape or cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.device != dev or \
                    sin.device != dev or tuple(cos.shape[-2:]) != (L, D // 2) or cos.dim() not in (2, 3) or \
                    (cos.dim() == 3 and cos.shape[0] != B) or not cos.is_contiguous() or not sin.is_contiguous():
                raise ValueError("rope = (cos, sin): contiguous fp32 [L, D/2] or [B, L, D/2] on x's device")
            rc = _lib.load().mpsa_rope_quant_mx(x.data_ptr(), _IN_DTYPE[x.dtype], B, H, L, D, sb, sh, sl, cos.data_ptr(),
                                                sin.data_ptr(), L * (D // 2) if cos.dim() == 3 else 0, float(scale),
                                                _FP8_QUANT[fp8_elem], *outs)
        elif center is None:
            rc = _lib.load().mpsa_quant_mx(x.data_ptr(), _IN_DTYPE[x.dtype], B, H, L, D, sb, sh, sl, float(scale),
                                           _FP8_QUANT[fp8_elem], *outs)
        else:
            if center.dtype != torch.float32 or tuple(center.shape) != (B, H, D) or not center.is_contiguous() or \
                    center.device != dev:
                raise ValueError("center must be a contiguous fp32 [B, H, D] tensor on x's device")
            rc = _lib.load().mpsa_quant_mx_centered(x.data_ptr(), _IN_DTYPE[x.dtype], B, H, L, D, sb, sh, sl, float(scale),
                                                    center.data_ptr(), _FP8_QUANT[fp8_elem], *outs)
    _lib.check(rc)
    return out


def quantize_int8(x: torch.Tensor, scale: float = 1.0, tensor_layout="HND"):
    """Per-32 int8 codes and fp32 scales of one operand (ours/quant_mxint8.py:21-58)."""
    _require_cuda(x)
    x, (B, H, L, D), (sb, sh, sl) = _bhld(x, tensor_layout)
    codes = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    oc = (codes.stride(0), codes.stride(1), codes.stride(2)) if tensor_layout == "HND" else \
        (codes.stride(0), codes.stride(2), codes.stride(1))
    scales = torch.empty((B, H, L, D // 32), dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        rc = _lib.load().mpsa_quant_int8(x.data_ptr(), _IN_DTYPE[x.dtype], B, H, L, D, sb, sh, sl, float(scale),
                                         codes.data_ptr(), *oc, scales.data_ptr(), _stream())
    _lib.check(rc)
    return codes, scales


def quantize_nvfp4(x: torch.Tensor, scale: float = 1.0):
    """NVFP4 quantisation of a 2-D operand [rows, K] along K: packed E2M1 codes [rows, K/2], E4M3 block
    scales as 128x4 tiles [ceil(rows/128), K/64, 512] and the fp32 tensor scale (a 1-element tensor)."""
    _require_cuda(x)
    if x.dim() != 2:
        raise ValueError("quantize_nvfp4 expects a 2-D tensor")
    if x.stride(-1) != 1:
        x = x.contiguous()
    rows, cols = x.shape
    lib = _lib.load()
    n = lib.mpsa_quant_nvfp4_scratch_floats(rows, cols)
    dev = x.device
    scratch = torch.empty(max(n, 1), dtype=torch.float32, device=dev)
    codes = torch.empty((rows, cols // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((-(-rows // 128), cols // 64, 512), dtype=torch.uint8, device=dev)
    ts = torch.empty(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = lib.mpsa_quant_nvfp4(x.data_ptr(), _IN_DTYPE[x.dtype], rows, cols, x.stride(0), float(scale),
                                  scratch.data_ptr(), scratch.numel(), codes.data_ptr(), codes.stride(0),
                                  scales.data_ptr(), ts.data_ptr(), _stream())
    _lib.check(rc)
    return codes, scales, ts


def quantize_nvfp4_bh(x: torch.Tensor, scale: float = 1.0):
    """NVFP4 quantisation of an attention operand [B,H,L,D] along D with ONE tensor scale: packed codes
    [B,H,L,D/2], E4M3 scale tiles [B,H,ceil(L/128),D/64,512] (tiles restart at every head), tensor scale."""
    _require_cuda(x)
    x, (B, H, L, D), (sb, sh, sl) = _bhld(x, "HND")
    dev = x.device
    nl = -(-L // 128)
    scratch = torch.empty(B * H * nl * -(-D // 512), dtype=torch.float32, device=dev)
    codes = torch.empty((B, H, L, D // 2), dtype=torch.uint8, device=dev)
    scales = torch.empty((B, H, nl, D // 64, 512), dtype=torch.uint8, device=dev)
    ts = torch.empty(1, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        rc = _lib.load().mpsa_quant_nvfp4_bh(x.data_ptr(), _IN_DTYPE[x.dtype], B, H, L, D, sb, sh, sl, float(scale),
                                             scratch.data_ptr(), scratch.numel(), codes.data_ptr(), scales.data_ptr(),
                                             ts.data_ptr(), _stream())
    _lib.check(rc)
    return codes, scales, ts


def quantize_qk(x: torch.Tensor, scale: float = 1.0, *, fp8_elem="e5m2", fp4_kind="mxfp4", smooth=False,
                rope=None) -> QuantizedOperand:
    """Q or K (depth already padded to 128) in both precisions of the fused forward: MXFP8 and either MXFP4
    (one pass for both) or NVFP4 (a second quantizer).  smooth: subtract the mean over the sequence first
    (the reference's smooth_k), inside the MX quantizer."""
    if fp4_kind not in ("mxfp4", "nvfp4"):
        raise ValueError(f"unknown fp4_kind {fp4_kind!r}")
    center = None
    if rope is not None and (smooth or fp4_kind != "mxfp4"):
        raise ValueError("the fused rotary embedding goes with MXFP4/MXFP8 operands and without smooth_k")
    if smooth:
        center = column_mean(x)
        if fp4_kind == "nvfp4":                    # the NVFP4 quantizer has no centred form: it gets the difference
            x = (x.float() - center.unsqueeze(2)).to(x.dtype)
            center = None
    if fp4_kind == "mxfp4":
        return quantize_mx(x, scale, fp8_elem=fp8_elem, center=center, rope=rope)
    out = quantize_mx(x, scale, want_fp4=False, fp8_elem=fp8_elem)
    out.fp4, out.fp4_sf, out.fp4_ts = quantize_nvfp4_bh(x, scale)
    out.fp4_kind = "nvfp4"
    return out


def v_pitch(Skv: int) -> int:
    """Default number of keys per row of a V^T buffer: Skv rounded up to 128.  The kernels take the pitch as an
    argument (any multiple of 128 that holds Skv), so a caller may lay several blocks side by side in one buffer."""
    return -(-Skv // 128) * 128


def prepare_vt(v: torch.Tensor, pad: Optional[int] = None) -> torch.Tensor:
    """V [B,H,Skv,D] -> fp16 V^T [B,H,D,Skv_pad] (Skv_pad = v_pitch(Skv) unless given, zero filled)."""
    _require_cuda(v)
    if v.stride(-1) != 1:
        v = v.contiguous()
    B, H, Skv, D = v.shape
    pad = v_pitch(Skv) if pad is None else pad
    vt = torch.empty((B, H, D, pad), dtype=torch.float16, device=v.device)
    with torch.cuda.device(v.device):
        rc = _lib.load().mpsa_prepare_vt(v.data_ptr(), _IN_DTYPE[v.dtype], vt.data_ptr(), B, H, Skv, D, pad,
                                         v.stride(0), v.stride(1), v.stride(2), _stream())
    _lib.check(rc)
    return vt


@dataclass
class QuantizedV:
    """V quantised along the sequence for a quantised P.V (both formats, transposed)."""
    vt8: torch.Tensor       # uint8 [B,H,D,Skv_pad]
    v8_sf: torch.Tensor     # uint8 [B,H,Skv_pad/128,512]
    vt4: torch.Tensor       # uint8 [B,H,D,Skv_pad/2]
    v4_sf: torch.Tensor
    fp8_elem: str = "e5m2"


def quantize_v_seq(v: torch.Tensor, fp8_elem: str = "e5m2", pad: Optional[int] = None) -> QuantizedV:
    """V [B,H,Skv,D] -> MXFP8 and MXFP4 V^T with 32-key blocks along the sequence (one launch)."""
    _require_cuda(v)
    if v.stride(-1) != 1:
        v = v.contiguous()
    B, H, Skv, D = v.shape
    pad = v_pitch(Skv) if pad is None else pad
    u8 = dict(dtype=torch.uint8, device=v.device)
    out = QuantizedV(torch.empty((B, H, D, pad), **u8), torch.empty((B, H, pad // 128, 512), **u8),
                     torch.empty((B, H, D, pad // 2), **u8), torch.empty((B, H, pad // 128, 512), **u8), fp8_elem)
    with torch.cuda.device(v.device):
        rc = _lib.load().mpsa_quant_v_seq(v.data_ptr(), _IN_DTYPE[v.dtype], B, H, Skv, D, pad, v.stride(0), v.stride(1),
                                          v.stride(2), _FP8_QUANT[fp8_elem], out.vt8.data_ptr(), out.v8_sf.data_ptr(),
                                          out.vt4.data_ptr(), out.v4_sf.data_ptr(), _stream())
    _lib.check(rc)
    return out


def precision_map_band(S: int, Skv: int, causal: bool, band: int = 1, tile: int = 128, device="cuda") -> torch.Tensor:
    """uint8 [ceil(S/tile), ceil(Skv/tile)]: FP8 within `band` tiles of the diagonal, FP4 elsewhere,
    SKIP above the causal diagonal."""
    nq, nk = -(-S // tile), -(-Skv // tile)
    m = torch.empty((nq, nk), dtype=torch.uint8, device=device)
    with torch.cuda.device(m.device):
        rc = _lib.load().mpsa_route_band(m.data_ptr(), nq, nk, tile, int(causal), band, S, Skv, _stream())
    _lib.check(rc)
    return m


def router_statistic(qq: "QuantizedOperand", kq: "QuantizedOperand", B: int, Hq: int, Hkv: int, S: int, Skv: int,
                     *, causal: bool, check: bool = False) -> torch.Tensor:
    """float32 [B,Hq,nq,nk]: mean over the query rows of the row maximum of every visible 128 x 128 tile of
    the MXFP4 score matrix (ours/mxfp_attn_kernel.py:272-280).  Cells above the causal diagonal hold 0."""
    if qq.fp4 is None or kq.fp4 is None:
        raise ValueError("router_statistic needs the MXFP4 form of Q and K")
    dev = qq.fp4.device
    nq, nk = -(-S // 128), -(-Skv // 128)
    stat = torch.empty((B, Hq, nq, nk), dtype=torch.float32, device=dev)
    scratch = torch.empty((B, Hq, nq, nk, 4), dtype=torch.float32, device=dev)
    _raise_if_failed(dev)
    status = status_word(dev)
    with torch.cuda.device(dev):
        rc = _lib.load().mpsa_route_stat(qq.fp4.data_ptr(), qq.fp4_sf.data_ptr(), kq.fp4.data_ptr(), kq.fp4_sf.data_ptr(),
                                         stat.data_ptr(), scratch.data_ptr(), B, Hq, Hkv, S, Skv, int(causal), status.data_ptr(),
                                         _stream())
    _lib.check(rc)
    if check:
        check_status(dev)
    return stat


def precision_map_online(stat: torch.Tensor, S: int, Skv: int, *, causal: bool, band: int = 1, tau: float = 1.0,
                         skip_thresh: Optional[float] = None) -> torch.Tensor:
    """uint8 [B,Hq,nq,nk] from router_statistic: band rule, plus FP8 for every other visible tile whose statistic
    reaches `tau` times that of the row's first key tile.  skip_thresh (the reference's use of the statistic,
    ours/mxfp_attn_kernel.py:276-297): a tile outside the band is processed only if it is the row's first one or its
    statistic reaches skip_thresh times the first tile's; otherwise it is SKIP."""
    B, Hq, nq, nk = stat.shape
    if (nq, nk) != (-(-S // 128), -(-Skv // 128)) or stat.dtype != torch.float32:
        raise ValueError("stat must be float32 [B, Hq, ceil(S/128), ceil(Skv/128)]")
    stat = stat.contiguous()
    m = torch.empty((B, Hq, nq, nk), dtype=torch.uint8, device=stat.device)
    with torch.cuda.device(stat.device):
        rc = _lib.load().mpsa_route_online(m.data_ptr(), stat.data_ptr(), B, Hq, S, Skv, int(causal), band, float(tau),
                                           0.0 if skip_thresh is None else float(skip_thresh), int(skip_thresh is not None),
                                           _stream())
    _lib.check(rc)
    return m


def _pad_depth_128(x: torch.Tensor) -> torch.Tensor:
    D = x.shape[-1]
    if D == 128:
        return x
    return torch.nn.functional.pad(x, (0, 128 - D))


def prepare_kv(k: torch.Tensor, v: torch.Tensor, *, pv_mode: str = "fp16", fp8_elem: str = "e5m2", fp4_kind: str = "mxfp4",
               smooth_k: bool = False, rope=None):
    """The key/value side of attention_forward on its own: K quantised in both precisions (depth padded to 128) and V
    prepared for the chosen P.V mode.  The pair can be kept - in memory, or through mpsa.kvstore - and given to
    attention_forward(kv=...) any number of times, so K and V are read in 16 bits once."""
    _require_cuda(k, v)
    if k.shape[-1] not in (64, 128):
        raise ValueError("headdim should be in [64, 128].")
    if rope is not None and k.shape[-1] != 128:
        raise ValueError("the fused rotary embedding needs head_dim 128")
    kq = quantize_qk(_pad_depth_128(k), 1.0, fp8_elem=fp8_elem, fp4_kind=fp4_kind, smooth=smooth_k, rope=rope)
    if pv_mode == "fp16":
        vt = prepare_vt(v)
    elif pv_mode == "requant":
        vt = quantize_v_seq(v, fp8_elem)
    else:
        raise ValueError(f"unknown pv_mode {pv_mode!r}")
    return kq, vt


def attention_forward(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool, band: int = 1,
                      prec_map: Optional[torch.Tensor] = None, uniform: Optional[str] = None,
                      sm_scale: Optional[float] = None, fp8_elem: str = "e5m2",
                      out_dtype: torch.dtype = torch.bfloat16, pv_mode: str = "fp16", check: bool = False,
                      router: str = "band", tau: float = 1.0, fp4_kind: str = "mxfp4",
                      skip_thresh: Optional[float] = None, return_sparsity: bool = False, smooth_k: bool = False,
                      rope=None, kv=None, fused_router: bool = True):
    """Quantise Q/K (both MXFP8 and MXFP4 in one pass each), prepare V, build the precision map and
    run the fused forward.  q [B,Hq,S,D], k/v [B,Hkv,Skv,D]; D in {64, 128}.
    smooth_k: subtract K's mean over the sequence inside the K quantizer (softmax is unchanged by it: every score
    of a row moves by the same amount).
    rope: (cos, sin) fp32 [Skv, D/2] (or [B, Skv, D/2]): q and k arrive WITHOUT their rotary embedding and the
    quantizers apply it (queries take the last S positions); D = 128.
    kv: the pair from prepare_kv (or mpsa.kvstore) in place of k and v, which may then be None; pv_mode follows the
    kind of V given, and smooth_k / the K side of rope have been applied when the pair was made.

    router "band": the static diagonal-band map.  router "online": every tile whose MXFP4 statistic reaches `tau`
    times that of the row's first key tile is promoted to MXFP8.  Causal with quantised P.V: the router runs inside
    the forward (attention_forward_routed; fused_router=False forces the stand-alone form).  Otherwise one extra MXFP4
    pass over the score tiles (router_statistic) and precision_map_online build the map first; with skip_thresh it also
    drops the tiles the reference's router would drop.  return_sparsity: also return the share of visible tiles dropped.

    pv_mode "fp16": P and V in fp16, the P.V precision of the reference kernel.
    pv_mode "requant": P is re-quantised to the tile's MX format and V is quantised along the sequence.
    fp4_kind "nvfp4": the FP4 tiles of Q.K^T use NVFP4 operands (16-element blocks, E4M3 scales, one tensor scale per
    operand) instead of MXFP4; P.V keeps the MX formats."""
    if kv is not None:
        _require_cuda(q)
        kq, vt = kv
        codes = kq.fp8 if kq.fp8 is not None else kq.fp4
        if codes is None or codes.dim() != 4 or codes.shape[0] != q.shape[0]:
            raise ValueError("kv = (QuantizedOperand of K [B,Hkv,Skv,...], V^T or QuantizedV)")
        Hkv, Skv = codes.shape[1], codes.shape[2]
        if kq.fp4_kind != fp4_kind or kq.fp8_elem != fp8_elem:
            raise ValueError("kv was prepared with another fp4_kind / fp8_elem than this call asks for")
    else:
        _require_cuda(q, k, v)
        _, Hkv, Skv, _ = k.shape
    B, Hq, S, D = q.shape
    if D not in (64, 128):
        raise ValueError("headdim should be in [64, 128].")
    sq = q_side_scale(D, sm_scale)
    rope_q = None
    if rope is not None:
        if D != 128:
            raise ValueError("the fused rotary embedding needs head_dim 128")
        rope_q = tuple(t[..., Skv - S:, :].contiguous() for t in rope)
    qq = quantize_qk(_pad_depth_128(q), sq, fp8_elem=fp8_elem, fp4_kind=fp4_kind, rope=rope_q)
    if kv is None:
        kq, vt = prepare_kv(k, v, pv_mode=pv_mode, fp8_elem=fp8_elem, fp4_kind=fp4_kind, smooth_k=smooth_k, rope=rope)
    if router == "online":
        if fp4_kind != "mxfp4":
            raise ValueError("the online router reads MXFP4 operands")
        if prec_map is not None or uniform is not None:
            raise ValueError("router='online' builds its own precision map")
        if fused_router and causal and skip_thresh is None and isinstance(vt, QuantizedV) and not return_sparsity:
            # the router runs inside the forward: no stand-alone statistic pass
            return attention_forward_routed(qq, kq, vt, B, Hq, Hkv, S, Skv, D, band=band, tau=tau, out_dtype=out_dtype,
                                            check=check)
        stat = router_statistic(qq, kq, B, Hq, Hkv, S, Skv, causal=causal, check=check)
        prec_map = precision_map_online(stat, S, Skv, causal=causal, band=band, tau=tau, skip_thresh=skip_thresh)
    elif router != "band":
        raise ValueError(f"unknown router {router!r}")
    elif skip_thresh is not None:
        raise ValueError("skip_thresh needs router='online'")
    out = attention_forward_quantized(qq, kq, vt, B, Hq, Hkv, S, Skv, D, causal=causal, band=band,
                                      prec_map=prec_map, uniform=uniform, out_dtype=out_dtype, check=check)
    if not return_sparsity:
        return out
    # share of the causally visible tiles that the router dropped
    band_map = precision_map_band(S, Skv, causal, band, 128, q.device)
    pm = band_map if prec_map is None else prec_map
    visible = int((band_map != TILE_SKIP).sum()) * (pm.numel() // band_map.numel())
    return out, 1.0 - float((pm != TILE_SKIP).sum()) / max(visible, 1)


def attention_forward_quantized(qq: QuantizedOperand, kq: QuantizedOperand, vt, B: int, Hq: int,
                                Hkv: int, S: int, Skv: int, D: int, *, causal: bool, band: int = 1,
                                prec_map: Optional[torch.Tensor] = None, uniform: Optional[str] = None,
                                out_dtype: torch.dtype = torch.bfloat16, check: bool = False, return_lse: bool = False,
                                lazy: bool = True, merge_with=None):
    """The fused forward on operands that are already quantised (depth padded to 128) and a V^T from
    prepare_vt (fp16 P.V) or a QuantizedV from quantize_v_seq (quantised P.V).  Both formats of Q and K
    must be present unless `uniform` restricts the map to one."""
    requant = isinstance(vt, QuantizedV)
    dev = vt.vt8.device if requant else vt.device
    nq, nk = -(-S // 128), -(-Skv // 128)
    if prec_map is None:
        prec_map = precision_map_band(S, Skv, causal, band, 128, dev)
        if uniform is not None:
            code = TILE_FP8 if uniform == "fp8" else TILE_FP4
            prec_map = torch.where(prec_map == TILE_SKIP, prec_map, torch.full_like(prec_map, code))
    if prec_map.dtype != torch.uint8 or tuple(prec_map.shape[-2:]) != (nq, nk):
        raise ValueError(f"precision map must be uint8 [..., {nq}, {nk}]")
    prec_map = prec_map.contiguous()
    if prec_map.dim() == 2:
        msb = msh = 0
    elif prec_map.dim() == 4:
        if tuple(prec_map.shape[:2]) != (B, Hq):
            raise ValueError("4-D precision map must be [B, Hq, nq, nk]")
        msb, msh = prec_map.stride(0), prec_map.stride(1)
    else:
        raise ValueError("precision map must be 2-D or 4-D")
    if out_dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported dtype: {out_dtype}")

    # A format the map never selects may be absent; the kernel still maps both, so stand in a
    # zero buffer of the right size (never a smaller one: the TMA map spans rows x row-bytes).
    def _codes(t, rows, row_bytes):
        return t if t is not None else torch.zeros((rows, row_bytes), dtype=torch.uint8, device=dev)
    q8, q4 = _codes(qq.fp8, B * Hq * S, 128), _codes(qq.fp4, B * Hq * S, 64)
    k8, k4 = _codes(kq.fp8, B * Hkv * Skv, 128), _codes(kq.fp4, B * Hkv * Skv, 64)
    q8s = qq.fp8_sf if qq.fp8_sf is not None else qq.fp4_sf
    q4s = qq.fp4_sf if qq.fp4_sf is not None else qq.fp8_sf
    k8s = kq.fp8_sf if kq.fp8_sf is not None else kq.fp4_sf
    k4s = kq.fp4_sf if kq.fp4_sf is not None else kq.fp8_sf
    for t, rows, rb in ((q8, B * Hq * S, 128), (q4, B * Hq * S, 64), (k8, B * Hkv * Skv, 128), (k4, B * Hkv * Skv, 64)):
        if t.numel() != rows * rb or not t.is_contiguous():
            raise ValueError("quantised operand has the wrong size (depth must be padded to 128)")
    if qq.fp4_kind != kq.fp4_kind:
        raise ValueError("Q and K use different FP4 kinds")
    nvf4 = qq.fp4_kind == "nvfp4"
    fp4_scale = 0.0
    if nvf4:
        if qq.fp4 is None or kq.fp4 is None or qq.fp8 is None or kq.fp8 is None:
            raise ValueError("NVFP4 score tiles need both the MXFP8 and the NVFP4 form of Q and K")
        fp4_scale = float(qq.fp4_ts.item()) * float(kq.fp4_ts.item())
    m4 = 2 if nvf4 else 1                          # 512-byte FP4 scale tiles per 128 rows
    for t, n in ((q8s, B * Hq * nq), (q4s, B * Hq * nq * m4), (k8s, B * Hkv * nk), (k4s, B * Hkv * nk * m4)):
        if t.numel() != n * 512 or not t.is_contiguous():
            raise ValueError("scale tiles have the wrong size")
    skv_pad = (vt.vt8 if requant else vt).shape[-1]      # keys per V^T row: any multiple of 128 that holds Skv
    if skv_pad % 128 or skv_pad < nk * 128:
        raise ValueError("V^T rows must hold a multiple of 128 keys, at least Skv")
    if requant:
        if tuple(vt.vt8.shape) != (B, Hkv, D, skv_pad) or tuple(vt.vt4.shape) != (B, Hkv, D, skv_pad // 2) or \
                vt.v8_sf.numel() != B * Hkv * (skv_pad // 128) * 512 or vt.v4_sf.numel() != B * Hkv * (skv_pad // 128) * 512:
            raise ValueError("quantised V has the wrong shape")
        if vt.fp8_elem != qq.fp8_elem:
            raise ValueError("Q/K and V use different fp8 element formats")
        vptrs = (None, vt.vt8.data_ptr(), vt.v8_sf.data_ptr(), vt.vt4.data_ptr(), vt.v4_sf.data_ptr(), 1)
    else:
        if tuple(vt.shape) != (B, Hkv, D, skv_pad) or vt.dtype != torch.float16 or not vt.is_contiguous():
            raise ValueError("vt must be contiguous fp16 [B, Hkv, D, keys per row]")
        vptrs = (vt.data_ptr(), None, None, None, None, 0)
    if (qq.fp8 is None or kq.fp8 is None) and uniform != "fp4":
        raise ValueError("MXFP8 operands missing but the precision map may select FP8 tiles")
    if (qq.fp4 is None or kq.fp4 is None) and uniform != "fp8":
        raise ValueError("MXFP4 operands missing but the precision map may select FP4 tiles")
    acc_in = lse_in = None
    if merge_with is not None:
        # (acc, lse) of an earlier partial result over other keys: the kernel's epilogue merges instead of a second pass
        acc_in, lse_in = merge_with
        if acc_in.dtype != torch.float32 or tuple(acc_in.shape) != (B, Hq, S, D) or not acc_in.is_contiguous() or \
                lse_in.dtype != torch.float32 or tuple(lse_in.shape) != (B, Hq, S) or not lse_in.is_contiguous():
            raise ValueError("merge_with = (fp32 [B,Hq,S,D], fp32 [B,Hq,S]), both contiguous")
        out_dtype, return_lse = torch.float32, True
    out = torch.empty((B, Hq, S, D), dtype=out_dtype, device=dev)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev) if return_lse else None
    _raise_if_failed(dev)
    st = status_word(dev)
    # quantised P.V: a per-call word lets the library run the fixed-reference kernel with the exact one as its
    # conditional fallback (same results, see include/mpsa.h)
    flag = torch.zeros(1, dtype=torch.int32, device=dev) if (requant and lazy) else None
    global _last_range_flag
    _last_range_flag = flag                       # kept for inspection: non-zero after the call = the exact kernel took over
    with torch.cuda.device(dev):
        rc = _lib.load().mpsa_attn_fwd(
            q8.data_ptr(), q8s.data_ptr(), q4.data_ptr(), q4s.data_ptr(),
            k8.data_ptr(), k8s.data_ptr(), k4.data_ptr(), k4s.data_ptr(),
            *vptrs, prec_map.data_ptr(), msb, msh, out.data_ptr(), _OUT_DTYPE[out_dtype], _ptr(lse),
            B, Hq, Hkv, S, Skv, D, skv_pad, int(causal), _FP8_DESC[qq.fp8_elem], int(nvf4), fp4_scale,
            _ptr(flag), _ptr(acc_in), _ptr(lse_in), st.data_ptr(), _stream())
    _lib.check(rc)
    if check:
        check_status(dev)
    return (out, lse) if return_lse else out


def attention_forward_routed(qq: QuantizedOperand, kq: QuantizedOperand, vq: "QuantizedV", B: int, Hq: int, Hkv: int, S: int,
                             Skv: int, D: int, *, band: int = 1, tau: float = 1.0, out_dtype: torch.dtype = torch.bfloat16,
                             check: bool = False, return_map: bool = False, return_lse: bool = False, stages: int = 15,
                             return_stat: bool = False):
    """The causal forward with the online router inside it (quantised P.V, MXFP4/MXFP8 operands): no stand-alone
    statistic pass.  A tile the router promotes is done again in MXFP8 by the same CTA after the row's own tiles (its
    MXFP4 result is left out).  Same precision map as precision_map_online(router_statistic(...), tau=tau).
    stages: mask of the launches to make (1 band map, 2 forward, 8 the conditional exact forward behind it; 4 is ignored) -
    a subset is for timing a stage alone.  return_stat: also the router statistic of the tiles outside the band (fp32
    [B,Hq,nq,nk], zero elsewhere)."""
    if not isinstance(vq, QuantizedV):
        raise ValueError("the routed forward needs V quantised along the sequence (quantize_v_seq)")
    if qq.fp4_kind != "mxfp4" or kq.fp4_kind != "mxfp4":
        raise ValueError("the online router reads MXFP4 operands")
    for t in (qq.fp8, qq.fp4, qq.fp8_sf, qq.fp4_sf, kq.fp8, kq.fp4, kq.fp8_sf, kq.fp4_sf):
        if t is None:
            raise ValueError("the routed forward needs both the MXFP8 and the MXFP4 form of Q and K")
    if out_dtype not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported dtype: {out_dtype}")
    if Skv < S:
        raise ValueError("causal attention needs Skv >= S")
    dev = vq.vt8.device
    nq, nk = -(-S // 128), -(-Skv // 128)
    skv_pad = vq.vt8.shape[-1]
    if qq.fp8.numel() != B * Hq * S * 128 or kq.fp8.numel() != B * Hkv * Skv * 128 or tuple(vq.vt8.shape) != (B, Hkv, D, skv_pad):
        raise ValueError("quantised operands have the wrong size (depth must be padded to 128)")
    pm = torch.empty((B, Hq, nq, nk), dtype=torch.uint8, device=dev)
    out = torch.empty((B, Hq, S, D), dtype=out_dtype, device=dev)
    lse = torch.empty((B, Hq, S), dtype=torch.float32, device=dev)
    lse_final = torch.empty((B, Hq, S), dtype=torch.float32, device=dev) if return_lse else None
    stat = torch.zeros((B, Hq, nq, nk), dtype=torch.float32, device=dev) if return_stat else None
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    global _last_range_flag
    _last_range_flag = flag
    _raise_if_failed(dev)
    st = status_word(dev)
    with torch.cuda.device(dev):
        rc = _lib.load().mpsa_attn_fwd_routed(
            qq.fp8.data_ptr(), qq.fp8_sf.data_ptr(), qq.fp4.data_ptr(), qq.fp4_sf.data_ptr(),
            kq.fp8.data_ptr(), kq.fp8_sf.data_ptr(), kq.fp4.data_ptr(), kq.fp4_sf.data_ptr(),
            vq.vt8.data_ptr(), vq.v8_sf.data_ptr(), vq.vt4.data_ptr(), vq.v4_sf.data_ptr(),
            pm.data_ptr(), int(band), float(tau), out.data_ptr(), _OUT_DTYPE[out_dtype], lse.data_ptr(), _ptr(lse_final),
            _ptr(stat), None, B, Hq, Hkv, S, Skv, D, skv_pad, _FP8_DESC[qq.fp8_elem], int(stages), flag.data_ptr(),
            st.data_ptr(), _stream())
    _lib.check(rc)
    if check:
        check_status(dev)
    res = (out,)
    if return_map:
        res += (pm,)
    if return_lse:
        res += (lse_final,)
    if return_stat:
        res += (stat,)
    return res[0] if len(res) == 1 else res


def attention_merge(acc: torch.Tensor, lse_acc: torch.Tensor, part: torch.Tensor, lse_part: torch.Tensor) -> None:
    """In-place merge of a partial attention result (part, lse_part) into (acc fp32, lse_acc): the result is
    the softmax-weighted combination over the union of the two key sets."""
    _require_cuda(acc, lse_acc, part, lse_part)
    D = acc.shape[-1]
    rows = acc.numel() // D
    if acc.dtype != torch.float32 or lse_acc.dtype != torch.float32 or lse_part.dtype != torch.float32:
        raise ValueError("accumulator and lse tensors must be fp32")
    if part.shape != acc.shape or lse_acc.numel() != rows or lse_part.numel() != rows:
        raise ValueError("shape mismatch between accumulator and partial result")
    if not (acc.is_contiguous() and part.is_contiguous() and lse_acc.is_contiguous() and lse_part.is_contiguous()):
        raise ValueError("attention_merge needs contiguous tensors")
    with torch.cuda.device(acc.device):
        rc = _lib.load().mpsa_attn_merge(acc.data_ptr(), lse_acc.data_ptr(), part.data_ptr(), _OUT_DTYPE[part.dtype],
                                         lse_part.data_ptr(), rows, D, _stream())
    _lib.check(rc)


def diagonal_tiled_attention(q, k, v, causal=True, pv_mode="requant"):
    """README-level entry of the reference project: diagonal tiles in MXFP8, the rest in MXFP4, P
    re-quantised to the tile's format before P.V."""
    return attention_forward(q, k, v, causal=causal, pv_mode=pv_mode,
                             out_dtype=q.dtype if q.dtype != torch.float32 else torch.float32)


class _HostPipeline:
    """Streams and staging buffers of attention_forward_host for one device and one problem shape."""

    def __init__(self, dev, grp, S, Skv, D, dtype, slots=2):
        self.h2d, self.d2h = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        # chunks alternate between two compute streams: the short kernels that open a chunk (quantizers, router) run
        # in the tail of the previous chunk's forward instead of behind it
        self.compute = [torch.cuda.Stream(dev), torch.cuda.Stream(dev)]
        self.q = [torch.empty((1, grp, S, D), dtype=dtype, device=dev) for _ in range(slots)]
        self.kv = [(torch.empty((1, 1, Skv, D), dtype=dtype, device=dev), torch.empty((1, 1, Skv, D), dtype=dtype, device=dev))
                   for _ in range(slots)]
        self.q_loaded = [torch.cuda.Event() for _ in range(slots)]     # the slot's queries have arrived
        self.q_consumed = [torch.cuda.Event() for _ in range(slots)]   # the forward that read them is done
        self.kv_loaded = [torch.cuda.Event() for _ in range(slots)]
        self.kv_consumed = [[] for _ in range(slots)]                   # one event per piece that read the slot


_host_pipes = {}


def _host_chunks(B, Hkv, grp):
    """(batch, KV group, first q-head of the group, number of q-heads) in processing order.  A KV group is the
    unit; the first and the last group are cut into smaller pieces so that the pipeline fills and drains quickly."""
    out = []
    n = B * Hkv
    for i in range(n):
        b, g = divmod(i, Hkv)
        if grp >= 4 and n > 1 and i == 0:
            sizes = [1, 1, grp - 2]
        elif grp >= 4 and n > 1 and i == n - 1:
            sizes = [grp - 2, 1, 1]
        else:
            sizes = [grp]
        h = 0
        for sz in sizes:
            out.append((b, g, h, sz))
            h += sz
    return out


def attention_forward_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool, out: Optional[torch.Tensor] = None,
                           device=None, out_dtype: torch.dtype = torch.bfloat16, non_blocking: bool = False, **kw):
    """The fused forward for operands that live in (pinned) HOST memory: q [B,Hq,S,D], k/v [B,Hkv,S,D] CPU tensors,
    result a pinned CPU tensor [B,Hq,S,D].  The work is cut into (batch, KV group) chunks - independent units of
    the path - and pipelined over copy and compute streams: while chunk i is computed, the inputs of chunk i+1 cross
    PCIe and the output of chunk i-1 goes back, so that a call costs about max(copy, compute) rather than their sum.
    Keyword arguments are those of attention_forward.

    The call returns when the result IS in `out`: it waits (on the host, for this call's last copy only) before
    returning.  non_blocking=True returns at once with (out, event) instead; `out` may be read after
    event.synchronize() - or after any later synchronisation of the current stream, which is ordered behind the copies."""
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("attention_forward_host expects CPU tensors; use attention_forward for device tensors")
    B, Hq, S, D = q.shape
    Hkv, Skv = k.shape[1], k.shape[2]
    if Hq % Hkv:
        raise ValueError("Hq must be a multiple of Hkv")
    grp = Hq // Hkv
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    q, k, v = (t if t.is_contiguous() else t.contiguous() for t in (q, k, v))
    q, k, v = (t if t.is_pinned() else t.pin_memory() for t in (q, k, v))
    if out is None:
        out = torch.empty((B, Hq, S, D), dtype=out_dtype).pin_memory()
    elif out.is_cuda or out.dtype != out_dtype or tuple(out.shape) != (B, Hq, S, D) or not out.is_contiguous():
        raise ValueError("out must be a contiguous CPU tensor [B,Hq,S,D] of out_dtype")
    key = (dev.index, grp, S, Skv, D, q.dtype)
    pipe = _host_pipes.get(key)
    if pipe is None:
        _host_pipes.clear()                       # one shape at a time: the staging buffers are large
        pipe = _host_pipes[key] = _HostPipeline(dev, grp, S, Skv, D, q.dtype)
    main = torch.cuda.current_stream(dev)
    start = torch.cuda.Event()
    start.record(main)
    pipe.h2d.wait_event(start)                    # the caller's earlier work on these buffers comes first
    pipe.d2h.wait_event(start)
    for cs in pipe.compute:
        cs.wait_event(start)
    for used in pipe.kv_consumed:
        used.clear()
    keep = []
    chunks = _host_chunks(B, Hkv, grp)
    n_kv = -1                                      # KV groups uploaded so far - 1
    for n, (b, g, h0, nh) in enumerate(chunks):
        qs = n % len(pipe.q)
        dq = pipe.q[qs][:, :nh]
        new_kv = h0 == 0
        if new_kv:
            n_kv += 1
        ks = n_kv % len(pipe.kv)
        dk, dv = pipe.kv[ks]
        with torch.cuda.stream(pipe.h2d):
            if new_kv:
                for e in pipe.kv_consumed[ks]:     # every piece of the group that held this slot has read K and V
                    pipe.h2d.wait_event(e)
                pipe.kv_consumed[ks].clear()
                dk.copy_(k[b:b + 1, g:g + 1], non_blocking=True)
                dv.copy_(v[b:b + 1, g:g + 1], non_blocking=True)
                pipe.kv_loaded[ks].record(pipe.h2d)
            if n >= len(pipe.q):
                pipe.h2d.wait_event(pipe.q_consumed[qs])
            dq.copy_(q[b:b + 1, g * grp + h0:g * grp + h0 + nh], non_blocking=True)
            pipe.q_loaded[qs].record(pipe.h2d)
        cs = pipe.compute[n % len(pipe.compute)]
        cs.wait_event(pipe.kv_loaded[ks])
        cs.wait_event(pipe.q_loaded[qs])
        with torch.cuda.stream(cs):
            o = attention_forward(dq, dk, dv, causal=causal, out_dtype=out_dtype, **kw)
        pipe.q_consumed[qs].record(cs)
        done = torch.cuda.Event()
        done.record(cs)
        pipe.kv_consumed[ks].append(done)
        with torch.cuda.stream(pipe.d2h):
            pipe.d2h.wait_event(done)
            out[b:b + 1, g * grp + h0:g * grp + h0 + nh].copy_(o, non_blocking=True)
        keep.append(o)                            # alive until the copies are ordered behind `main` below
    fin = torch.cuda.Event()
    fin.record(pipe.d2h)
    main.wait_event(fin)
    for o in keep:
        o.record_stream(pipe.d2h)
    if non_blocking:
        return out, fin
    fin.synchronize()
    _raise_if_failed(dev)
    return out


_GEMM_MODE = {"mxfp8": 0, "mxfp4": 1, "nvfp4": 2}


def gemm_block_scaled(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
                      out_dtype: torch.dtype, M: int, N: int, K: int, mode: str, *, a_elem="e5m2", b_elem="e5m2",
                      alpha: float = 1.0, check: bool = False) -> torch.Tensor:
    """C[M,N] = alpha * (A.sa)(B.sb)^T.  a [M,K/epb] / b [N,K/epb] bytes (uint8 or float8), scales as 128x4
    tiles [rows/128, K/vec/4, 32,4,4] (uint8 E8M0, or E4M3 bytes for nvfp4)."""
    _require_cuda(a, b, a_scale, b_scale)
    if mode not in _GEMM_MODE:
        raise ValueError(f"Invalid block scale type: {mode}")
    if out_dtype not in _OUT_DTYPE:
        raise ValueError(f"Unsupported dtype: {out_dtype}")
    if a.stride(-1) != 1:
        a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    a_scale, b_scale = a_scale.contiguous(), b_scale.contiguous()
    c = torch.empty((M, N), dtype=out_dtype, device=a.device)
    _raise_if_failed(a.device)
    st = status_word(a.device)
    with torch.cuda.device(a.device):
        rc = _lib.load().mpsa_gemm_block_scaled(
            a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), c.data_ptr(), M, N, K,
            a.stride(0) * a.element_size(), b.stride(0) * b.element_size(), c.stride(0), _GEMM_MODE[mode],
            _FP8_DESC[a_elem], _FP8_DESC[b_elem], _OUT_DTYPE[out_dtype], float(alpha), st.data_ptr(), _stream())
    _lib.check(rc)
    if check:
        check_status(a.device)
    return c


def gemm_block_scaled_batched(a: torch.Tensor, a_scale: torch.Tensor, b: torch.Tensor, b_scale: torch.Tensor,
                              out_dtype: torch.dtype, M: int, N: int, K: int, mode: str, *, a_elem="e5m2", b_elem="e5m2",
                              alpha: float = 1.0, check: bool = False) -> torch.Tensor:
    """C[..., M, N] = alpha * (A.sa)(B.sb)^T for every leading index: a [..., M, K/epb], b [..., N, K/epb] bytes,
    scale tiles [..., rows/128, K/vec/4, 32,4,4]; one launch for all problems."""
    _require_cuda(a, b, a_scale, b_scale)
    if mode not in _GEMM_MODE:
        raise ValueError(f"Invalid block scale type: {mode}")
    if out_dtype not in _OUT_DTYPE:
        raise ValueError(f"Unsupported dtype: {out_dtype}")
    lead = tuple(a.shape[:-2])
    if tuple(b.shape[:-2]) != lead:
        raise ValueError("a and b need the same leading (batch) dimensions")
    batch = 1
    for d in lead:
        batch *= d
    a, b, a_scale, b_scale = a.contiguous(), b.contiguous(), a_scale.contiguous(), b_scale.contiguous()
    epb = 1 if mode == "mxfp8" else 2
    vec = 16 if mode == "nvfp4" else 32
    if a.shape[-2] != M or b.shape[-2] != N or a.shape[-1] * a.element_size() != K // epb or b.shape[-1] * b.element_size() != K // epb:
        raise ValueError("operand shapes do not match M, N, K")
    for t, rows in ((a_scale, M), (b_scale, N)):
        if t.numel() * t.element_size() != batch * (-(-rows // 128)) * (K // vec // 4) * 512:
            raise ValueError("scale tiles have the wrong size")
    c = torch.empty((*lead, M, N), dtype=out_dtype, device=a.device)
    _raise_if_failed(a.device)
    st = status_word(a.device)
    with torch.cuda.device(a.device):
        rc = _lib.load().mpsa_gemm_block_scaled_batched(
            a.data_ptr(), a_scale.data_ptr(), b.data_ptr(), b_scale.data_ptr(), c.data_ptr(), batch, M, N, K,
            _GEMM_MODE[mode], _FP8_DESC[a_elem], _FP8_DESC[b_elem], _OUT_DTYPE[out_dtype], float(alpha), st.data_ptr(),
            _stream())
    _lib.check(rc)
    if check:
        check_status(a.device)
    return c
