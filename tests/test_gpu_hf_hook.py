"""The transformers hook: a tiny random-init Llama runs its prefill through the mixed-precision forward when built with
attn_implementation="mpsa"; logits stay close to the SDPA model's (the tolerance is loose: MXFP4 scores in every layer)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_llama_prefill_through_the_hook(monkeypatch):
    transformers = pytest.importorskip("transformers")
    import mpsa.hf
    from mpsa import ops
    cfg = transformers.LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=2, head_dim=128, max_position_embeddings=2048)
    torch.manual_seed(0)
    ref = transformers.LlamaForCausalLM._from_config(copy.deepcopy(cfg), attn_implementation="sdpa").to("cuda", torch.bfloat16).eval()
    ours = transformers.LlamaForCausalLM._from_config(copy.deepcopy(cfg), attn_implementation="mpsa").to("cuda", torch.bfloat16).eval()
    assert ref.config._attn_implementation == "sdpa" and ours.config._attn_implementation == "mpsa"
    ours.load_state_dict(ref.state_dict())
    calls = []
    real = ops.attention_forward
    monkeypatch.setattr(ops, "attention_forward", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    x = torch.randint(0, 512, (1, 640), device="cuda")
    with torch.no_grad():
        a = ref(x).logits.float()
        b = ours(x).logits.float()
    assert len(calls) == cfg.num_hidden_layers            # every layer's prefill went through the kernel
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert cos >= 0.98, cos
    mpsa.hf.ops.check_status()
