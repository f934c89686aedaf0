"""Hook for Hugging Face `transformers` models: registers the diagonal-tiled mixed-precision forward as an attention
implementation, so that a model built with ``attn_implementation="mpsa"`` runs its prefill through it.

The reference wires its kernels into models by replacing attention modules (evaluate/llama/modify_sparse_attn.py:15-136,
spas_sage_attn/autotune.py:143-158) and never hooks the MXFP kernel in; `transformers` now has a registry for exactly
this, which needs no module surgery:

    import mpsa.hf                       # registers "mpsa"
    model = AutoModelForCausalLM.from_pretrained(..., attn_implementation="mpsa")

What is routed to the kernel: calls without an explicit attention mask (or with the plain causal pattern the model
announces through ``is_causal``), head_dim 64 or 128, more than one query token.  Everything else - decoding steps,
padding masks, dropout, other head dims - goes to the library's own SDPA implementation, unchanged.
"""
from typing import Optional

import torch

from . import ops

PV_MODE = "requant"        # "fp16" for the reference's P.V precision
ROUTER = "band"            # "online" adds the statistic pass
TAU = 1.1
SMOOTH_K = False           # True: subtract K's mean over the sequence inside the K quantizer (the default of the reference's mxfp_attn)


def mpsa_attention_forward(module: torch.nn.Module, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                           attention_mask: Optional[torch.Tensor], dropout: float = 0.0, scaling: Optional[float] = None,
                           is_causal: Optional[bool] = None, **kwargs):
    """query [B,Hq,S,D], key/value [B,Hkv,Skv,D] (GQA heads are NOT repeated) -> (output [B,S,Hq,D], None)."""
    from transformers.integrations.sdpa_attention import sdpa_attention_forward
    is_causal = is_causal if is_causal is not None else getattr(module, "is_causal", True)
    B, Hq, S, D = query.shape
    usable = (query.is_cuda and attention_mask is None and dropout == 0.0 and S > 1 and D in (64, 128)
              and key.shape[2] >= S and Hq % key.shape[1] == 0
              and query.dtype in (torch.float16, torch.bfloat16, torch.float32))
    if not usable:
        return sdpa_attention_forward(module, query, key, value, attention_mask, dropout=dropout, scaling=scaling,
                                      is_causal=is_causal, **kwargs)
    out = ops.attention_forward(query, key, value, causal=bool(is_causal), sm_scale=scaling, out_dtype=query.dtype
                                if query.dtype != torch.float32 else torch.float32, pv_mode=PV_MODE,
                                router=ROUTER, tau=TAU, smooth_k=SMOOTH_K)
    return out.transpose(1, 2).contiguous(), None


def register(name: str = "mpsa") -> str:
    """Register the forward under `name` in transformers' attention registry (idempotent)."""
    from transformers import AttentionInterface
    AttentionInterface.register(name, mpsa_attention_forward)
    try:                                   # newer versions also keep a registry of mask builders per implementation
        from transformers import AttentionMaskInterface
        from transformers.masking_utils import sdpa_mask
        AttentionMaskInterface.register(name, sdpa_mask)
    except Exception:
        pass
    return name


register()
