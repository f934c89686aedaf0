"""Fused MXFP attention with the entry points of ours/mxfp_attn_kernel.py of the reference:
mxfp_attn_kernel (:19-74) and block_scaled_batched_attn (:362-423)."""
import torch

from mpsa import ops as _ops


@torch.compiler.disable
def mxfp_attn_kernel(q, k, v, attn_mask=None, dropout_p=0.0,
                     is_causal=False, scale=None, smooth_k=False, attention_sink=False, tensor_layout="HND",
                     output_dtype=torch.float16, return_sparsity=False, block_scale_type="mxfp4", skip_thresh=None, out=None,
                     promote_thresh=None):
    """q [B,Hq,S,D], k/v [B,Hkv,Skv,D] (HND) or [B,S,H,D] (NHD) -> o in q's layout.

    block_scale_type: "mxfp4" / "mxfp8" quantise every tile of Q.K^T to that format (the two modes
    of the reference that run); "nvfp4" does the same with NVFP4 operands; "diag" keeps the diagonal tiles in MXFP8 and the rest in MXFP4; "diag_requant"
    additionally re-quantises P to the tile's format before P.V (V quantised along the sequence);
    "online" / "online_requant" are the same two with the online router on top of the diagonal rule: a tile
    is also MXFP8 if its MXFP4 statistic reaches promote_thresh (default 1.1) times that of the row's first key
    tile, and, when skip_thresh is given, a tile outside the band is dropped unless it is the row's first one or
    its statistic reaches skip_thresh times the first tile's - the reference's rule
    (ours/mxfp_attn_kernel.py:272-297).  return_sparsity then also returns the share of visible tiles dropped.
    attn_mask, dropout_p and attention_sink are accepted and ignored, as in the reference wrapper, and so are
    skip_thresh and return_sparsity outside the online modes; is_causal, scale and output_dtype are honoured
    (the reference ignores them).  Any other block_scale_type raises ValueError, "mixed" included (not built).
    Host (CPU) tensors are streamed through the GPU and the call returns when the result is in host memory."""
    host = not v.is_cuda
    if host and tensor_layout != "HND":
        raise ValueError("host tensors are taken in the HND layout only")
    if not host:
        torch.cuda.set_device(v.device)
    if tensor_layout == "NHD":
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    elif tensor_layout != "HND":
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    if q.dtype == torch.float32:
        q, k = q.to(torch.float16), k.to(torch.float16)      # ours/mxfp_attn_kernel.py:28-29
    if smooth_k and host:
        k = k - k.mean(dim=-2, keepdim=True)                 # :33-34; device tensors: inside the K quantizer, below
    assert q.shape[-1] in [64, 128], "headdim should be in [64, 128]."
    fp4_kind = "mxfp4"
    if block_scale_type == "mxfp4":
        uniform = "fp4"
    elif block_scale_type == "mxfp8":
        uniform = "fp8"
    elif block_scale_type == "nvfp4":
        # every tile of Q.K^T in NVFP4 (16-element blocks, E4M3 scales, one tensor scale per operand)
        uniform, fp4_kind = "fp4", "nvfp4"
    elif block_scale_type in ("diag", "diag_requant", "online", "online_requant"):
        uniform = None
    elif block_scale_type == "mixed":
        # the reference's fp8 Q x fp4 K mode (ours/mxfp_attn_kernel.py:170, :264-265) has no kernel here
        raise ValueError("block_scale_type 'mixed' (MXFP8 Q x MXFP4 K) is not built; use 'diag' for per-tile mixed precision")
    else:
        raise ValueError(f"Invalid block scale type: {block_scale_type}")      # the reference asserts the set (:452)
    online = block_scale_type.startswith("online")
    kw = dict(causal=bool(is_causal), uniform=uniform, sm_scale=scale, out_dtype=output_dtype,
              pv_mode="requant" if block_scale_type.endswith("requant") else "fp16",
              router="online" if online else "band",
              tau=(1.1 if promote_thresh is None else float(promote_thresh)) if online else 1.0,
              skip_thresh=skip_thresh if online else None, fp4_kind=fp4_kind)
    if host:
        o = _ops.attention_forward_host(q, k, v, out=out, **kw)      # `out`: a pinned CPU tensor to fill (optional)
    else:
        if out is not None:
            raise ValueError("out= is for host tensors only")
        o = _ops.attention_forward(q, k, v, return_sparsity=bool(return_sparsity and online), smooth_k=bool(smooth_k), **kw)
        if return_sparsity and online:
            o, sparsity = o
            return (o.transpose(1, 2) if tensor_layout == "NHD" else o), sparsity
    return o.transpose(1, 2) if tensor_layout == "NHD" else o


def block_scaled_batched_attn(a_desc, a_scale, b_desc, b_scale, v_ori, dtype_dst, B, H, M, N, K, configs, STAGE=1,
                              skip_thresh=None):
    """Attention from already-quantised operands in the reference's formats: a/b fp8 [B,H,L,K]
    (float8_e5m2) or packed fp4 [B,H,L,K/2], scales as 128x4 tiles [B,H,L/128,K/32/4,32,4,4]
    (K must be 128), v [B,H,N,K].  STAGE 1 = full attention; STAGE 3 = causal."""
    if dtype_dst not in (torch.float32, torch.float16, torch.bfloat16):
        raise ValueError(f"Unsupported dtype: {dtype_dst}")
    if K != 128:
        raise ValueError("pre-quantised operands need head_dim 128")
    fp4 = configs["ELEM_PER_BYTE_A"] == 2
    elem = "e4m3" if a_desc.dtype == torch.float8_e4m3fn else "e5m2"

    def operand(codes, scales):
        c = codes.view(torch.uint8).contiguous()
        s = scales.view(torch.uint8).contiguous().reshape(B, H, -1, 1, 512)
        if fp4:
            return _ops.QuantizedOperand(fp4=c, fp4_sf=s, fp8_elem=elem)
        return _ops.QuantizedOperand(fp8=c, fp8_sf=s, fp8_elem=elem)

    Hkv = v_ori.shape[1]
    return _ops.attention_forward_quantized(operand(a_desc, a_scale), operand(b_desc, b_scale),
                                            _ops.prepare_vt(v_ori), B, H, Hkv, M, N, K, causal=(STAGE == 3),
                                            uniform="fp4" if fp4 else "fp8", out_dtype=dtype_dst)
