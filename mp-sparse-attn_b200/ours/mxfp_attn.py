"""`mxfp_attn` with the superset signature of ours/mxfp_attn.py:30-78 of the reference.  There the
function stops after Q.K^T; here it is the full fused attention (same as mxfp_attn_kernel)."""
import torch

from .mxfp_attn_kernel import mxfp_attn_kernel


@torch.compiler.disable
def mxfp_attn(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, scale=None, smooth_k=True,
              attention_sink=False, tensor_layout="HND", output_dtype=torch.float16, return_sparsity=False,
              skip_thresh=None, block_scale_type="mxfp4", BLKQ=128, compute_reference=False):
    return mxfp_attn_kernel(q, k, v, attn_mask=attn_mask, dropout_p=dropout_p, is_causal=is_causal, scale=scale,
                            smooth_k=smooth_k, attention_sink=attention_sink, tensor_layout=tensor_layout,
                            output_dtype=output_dtype, return_sparsity=return_sparsity,
                            block_scale_type=block_scale_type, skip_thresh=skip_thresh)
