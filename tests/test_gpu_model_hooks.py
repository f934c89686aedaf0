"""The reference-style model hooks on a GPU: a SparseAttentionMeansim-shaped object and a Wan-shaped block run their
attention through the library; results stay close to exact attention (MXFP4 scores: loose tolerance)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_attention_object_in_both_layouts():
    from mpsa import model_hooks as H, ops
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn(1, 4, 384, 128, generator=g) for _ in range(3))
    v = v + 2.0                                    # values with a mean: zero-mean V under a flat softmax leaves only noise to compare
    q, k, v = (t.to(torch.bfloat16).cuda() for t in (q, k, v))
    att = H.MixedPrecisionAttention(block_scale_type="diag_requant", smooth_k=True)
    for causal in (True, False):
        ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=causal)
        o = att(q, k, v, is_causal=causal)
        o2 = att(q.transpose(1, 2).contiguous(), k.transpose(1, 2).contiguous(), v.transpose(1, 2).contiguous(),
                 is_causal=causal, tensor_layout="NHD")
        assert o.shape == q.shape and o2.shape == (1, 384, 4, 128) and o.dtype == q.dtype
        assert torch.equal(o2.transpose(1, 2), o)
        # the object adds nothing of its own: same bytes as the reference-named entry point with the same settings
        from ours.mxfp_attn_kernel import mxfp_attn_kernel
        direct = mxfp_attn_kernel(q, k, v, is_causal=causal, smooth_k=True, output_dtype=q.dtype, block_scale_type="diag_requant")
        assert torch.equal(o, direct)
        cos = torch.nn.functional.cosine_similarity(o.float().flatten(), ref.flatten(), dim=0).item()
        assert cos >= 0.98, (causal, cos)          # MXFP4 scores, P and V against exact attention
    ops.check_status()


def test_wan_shaped_block():
    from mpsa import model_hooks as H, ops
    import importlib.util, os
    spec = importlib.util.spec_from_file_location("_hooks_cpu", os.path.join(os.path.dirname(__file__), "test_model_hooks_cpu.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _Wan = mod._Wan
    torch.manual_seed(1)
    model = _Wan(dim=256, heads=2, n=2).cuda().to(torch.bfloat16)
    x = torch.randn(1, 640, 256, device="cuda", dtype=torch.bfloat16)
    att = model.blocks[0].self_attn
    q, k, v = (m(x).view(1, 640, 2, 128).transpose(1, 2).float() for m in (att.q, att.k, att.v))
    ref = att.o(torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).flatten(2).to(torch.bfloat16))
    assert H.set_mpsa_attn_wan(model, rope_apply=lambda t, g, f: t) == 2
    y = att(x, torch.tensor([640]), torch.tensor([[4, 10, 16]]), None)
    cos = torch.nn.functional.cosine_similarity(y.float().flatten(), ref.float().flatten(), dim=0).item()
    assert y.shape == x.shape and cos >= 0.95, cos
    ops.check_status()
