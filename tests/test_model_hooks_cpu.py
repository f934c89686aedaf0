"""Host logic of the reference-style model hooks: the kernel_selection entry and the Wan patch's plumbing (no GPU: the
attention call itself is replaced by a recorder)."""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "mp-sparse-attn_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


class _MeansimLike:
    """Shape of the reference class (spas_sage_attn/autotune.py:143-158): names it knows, ValueError otherwise."""

    def kernel_selection(self, kernel_name=None):
        if kernel_name == "online_routing":
            return "online_routing_attn"
        raise ValueError(f"not support kernel name: {kernel_name}")


def test_kernel_selection_learns_the_mxfp_name():
    from mpsa import model_hooks as H
    obj = _MeansimLike()
    with pytest.raises(ValueError):
        obj.kernel_selection("mxfp")
    H.add_mxfp_kernel(_MeansimLike)
    H.add_mxfp_kernel(_MeansimLike)                      # idempotent
    assert obj.kernel_selection("mxfp") is H.mxfp_kernel
    assert obj.kernel_selection("online_routing") == "online_routing_attn"
    with pytest.raises(ValueError):
        obj.kernel_selection("nonsense")
    att = H.MixedPrecisionAttention()
    assert att.kernel_selection() is H.mxfp_kernel and att.kernel_selection("mxfp") is H.mxfp_kernel
    with pytest.raises(ValueError):
        att.kernel_selection("spargeattn_cuda")
    with pytest.raises(ValueError):
        att(torch.zeros(1), torch.zeros(1), torch.zeros(1), tune_mode=True)


class _SelfAttn(torch.nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.num_heads, self.head_dim, self.window_size = heads, dim // heads, (-1, -1)
        self.q, self.k, self.v, self.o = (torch.nn.Linear(dim, dim) for _ in range(4))
        self.norm_q, self.norm_k = torch.nn.Identity(), torch.nn.Identity()


class _Block(torch.nn.Module):
    def __init__(self, dim, heads):
        super().__init__()
        self.self_attn = _SelfAttn(dim, heads)


class _Wan(torch.nn.Module):
    def __init__(self, dim=64, heads=2, n=3):
        super().__init__()
        self.blocks = torch.nn.ModuleList(_Block(dim, heads) for _ in range(n))


def test_wan_patch_plumbing(monkeypatch):
    from mpsa import model_hooks as H
    seen = []

    def fake_kernel(q, k, v, mask, **kw):
        seen.append((tuple(q.shape), kw["tensor_layout"], kw["is_causal"], kw["block_scale_type"]))
        return torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2).float(), k.transpose(1, 2).float(),
                                                                v.transpose(1, 2).float()).transpose(1, 2).to(q.dtype)

    monkeypatch.setattr(H, "mxfp_kernel", fake_kernel)
    torch.manual_seed(0)
    model = _Wan()
    rope_calls = []
    rope = lambda t, g, f: (rope_calls.append(1), t)[1]
    assert H.set_mpsa_attn_wan(model, rope_apply=rope, block_scale_type="diag") == 3
    x = torch.randn(1, 40, 64)
    att = model.blocks[1].self_attn
    y = att(x, torch.tensor([40]), torch.tensor([[2, 4, 5]]), None)
    assert y.shape == x.shape and len(rope_calls) == 2
    assert seen == [((1, 40, 2, 32), "NHD", False, "diag")]
    # same numbers as the unpatched arithmetic (the recorder computes exact attention; inputs pass through bf16)
    q, k, v = (m(x).view(1, 40, 2, 32).transpose(1, 2) for m in (att.q, att.k, att.v))
    ref = att.o(torch.nn.functional.scaled_dot_product_attention(q, k, v).transpose(1, 2).flatten(2))
    assert torch.allclose(y, ref, atol=3e-2, rtol=3e-2)
    with pytest.raises(ValueError):
        att(torch.randn(2, 40, 64), torch.tensor([40, 40]), torch.tensor([[2, 4, 5]] * 2), None)
