"""Model-side hooks in the reference project's own style: an attention object with the call signature of its
`SparseAttentionMeansim` (spas_sage_attn/autotune.py:358-383), a `kernel_selection` entry for the MXFP kernel
(spas_sage_attn/autotune.py:143-158 knows "spargeattn_triton", "spargeattn_cuda" and "online_routing" only), and the
Wan video-DiT patch (evaluate/modify_model/modify_wan.py:97-135), which replaces every block's self-attention forward.

    from mpsa.model_hooks import MixedPrecisionAttention, add_mxfp_kernel, set_mpsa_attn_wan
    layer.self_attn.sparse_attention = MixedPrecisionAttention()      # evaluate/llama/modify_sparse_attn.py:124
    add_mxfp_kernel(SparseAttentionMeansim)                           # kernel_name="mxfp" now dispatches here
    set_mpsa_attn_wan(wan_model)                                       # needs the `wan` package for its rope_apply

The `transformers` registry hook is in mpsa/hf.py.  Nothing here imports the reference or the `wan` package at
import time.
"""
from typing import Callable, Optional

import torch

from . import ops

KERNEL_NAME = "mxfp"


def mxfp_kernel(q, k, v, mask=None, is_causal=False, smooth_k=True, scale=None, tensor_layout="HND", return_sparsity=False,
                block_scale_type="diag_requant", skip_thresh=None, **ignored):
    """The callable `kernel_selection("mxfp")` returns: the reference's kernel-call convention
    (spas_sage_attn/autotune.py:361-383: q, k, v, mask positional; is_causal, smooth_k, scale, tensor_layout,
    return_sparsity by name; the SpargeAttn thresholds it also passes are accepted and ignored)."""
    from ours.mxfp_attn_kernel import mxfp_attn_kernel
    return mxfp_attn_kernel(q, k, v, attn_mask=mask, is_causal=is_causal, scale=scale, smooth_k=smooth_k,
                            tensor_layout=tensor_layout, output_dtype=q.dtype if q.dtype != torch.float32 else torch.float32,
                            return_sparsity=return_sparsity, block_scale_type=block_scale_type, skip_thresh=skip_thresh)


class MixedPrecisionAttention(torch.nn.Module):
    """Drop-in for an instance of the reference's SparseAttentionMeansim: same forward signature, no tuning state.
    block_scale_type as in ours.mxfp_attn_kernel ("diag", "diag_requant", "online", "online_requant", "mxfp8", "mxfp4",
    "nvfp4")."""

    def __init__(self, block_scale_type: str = "diag_requant", smooth_k: bool = True, skip_thresh: Optional[float] = None,
                 kernel_name: str = KERNEL_NAME):
        super().__init__()
        self.block_scale_type = block_scale_type
        self.smooth_k = smooth_k
        self.skip_thresh = skip_thresh
        self.kernel_name = kernel_name

    def kernel_selection(self, kernel_name=None):
        if kernel_name is None or kernel_name == KERNEL_NAME:
            return mxfp_kernel
        raise ValueError(f"not support kernel name: {kernel_name}")

    @torch.no_grad()
    def forward(self, q, k, v, mask=None, is_causal=False, scale=None, tensor_layout="HND", tune_mode=False, smooth_k=None,
                return_sparsity=False):
        if tune_mode:
            raise ValueError("the mixed-precision kernel has no hyper-parameters to tune")
        kernel = self.kernel_selection(self.kernel_name)
        return kernel(q, k, v, mask, is_causal=is_causal, smooth_k=self.smooth_k if smooth_k is None else smooth_k, scale=scale,
                      tensor_layout=tensor_layout, return_sparsity=return_sparsity, block_scale_type=self.block_scale_type,
                      skip_thresh=self.skip_thresh)


def add_mxfp_kernel(attention_class) -> None:
    """Teach a class with the reference's `kernel_selection(self, kernel_name)` method (SparseAttentionMeansim) the name
    "mxfp": instances built with kernel_name="mxfp" then call this library.  Idempotent."""
    inner = attention_class.kernel_selection
    if getattr(inner, "_mpsa_patched", False):
        return

    def kernel_selection(self, kernel_name=None):
        if kernel_name == KERNEL_NAME:
            return mxfp_kernel
        return inner(self, kernel_name)

    kernel_selection._mpsa_patched = True
    attention_class.kernel_selection = kernel_selection


def _wan_self_attention_forward(rope_apply: Callable):
    @torch.no_grad()
    def forward(self, x, seq_lens, grid_sizes, freqs):
        """x [B, L, C]; seq_lens [B]; grid_sizes [B, 3]; freqs: rotary table (evaluate/modify_model/modify_wan.py:98-125)."""
        b, s, n, d = *x.shape[:2], self.num_heads, self.head_dim
        if tuple(getattr(self, "window_size", (-1, -1))) != (-1, -1):
            raise ValueError("windowed attention is not supported")
        if seq_lens.shape[0] != 1:
            raise ValueError("one sequence per call (no variable-length batches)")
        q = self.norm_q(self.q(x)).view(b, s, n, d)
        k = self.norm_k(self.k(x)).view(b, s, n, d)
        v = self.v(x).view(b, s, n, d)
        q, k = rope_apply(q, grid_sizes, freqs), rope_apply(k, grid_sizes, freqs)
        half = (torch.float16, torch.bfloat16)
        q, k, v = (t if t.dtype in half else t.to(torch.bfloat16) for t in (q, k, v))
        o = self.inner_attention(q, k.to(q.dtype), v.to(q.dtype), is_causal=False, tensor_layout="NHD")
        return self.o(o.to(x.dtype).flatten(2))
    return forward


def set_mpsa_attn_wan(model, rope_apply: Optional[Callable] = None, block_scale_type: str = "diag_requant",
                      smooth_k: bool = True) -> int:
    """Every block's self-attention of a Wan model (`model.blocks[i].self_attn` with q/k/v/o projections, norm_q/norm_k,
    num_heads, head_dim) computes its attention with this library from now on; returns the number of blocks patched.
    rope_apply: the model family's rotary function (default: wan.modules.model.rope_apply)."""
    if rope_apply is None:
        from wan.modules.model import rope_apply as _rope_apply      # the model's own package
        rope_apply = _rope_apply
    fwd = _wan_self_attention_forward(rope_apply)
    n = 0
    for block in model.blocks:
        block.self_attn.inner_attention = MixedPrecisionAttention(block_scale_type=block_scale_type, smooth_k=smooth_k)
        block.self_attn.forward = fwd.__get__(block.self_attn, type(block.self_attn))
        n += 1
    return n
