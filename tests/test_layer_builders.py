"""Single-layer builders of each decoder family: the pieces must match the layers of the family's whole-model builder."""
import pytest
import torch

import importlib
from torchtune_b200.modules.peft import LoRALinear

_TINY = dict(vocab_size=64, num_layers=1, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=16)
_FAMILIES = {
    "llama2": ("llama2_mlp", "lora_llama2_self_attention", "lora_llama2_mlp", dict(intermediate_dim=48)),
    "llama3": ("llama3_mlp", "lora_llama3_self_attention", "lora_llama3_mlp", dict(intermediate_dim=48)),
    "llama3_1": ("llama3_mlp", "lora_llama3_attention", "lora_llama3_mlp", dict(intermediate_dim=48)),
    "llama3_2": ("llama3_mlp", "lora_llama3_2_self_attention", "lora_llama3_mlp", dict(intermediate_dim=48)),
    "mistral": ("mistral_mlp", "lora_mistral_self_attention", "lora_mistral_mlp", dict(intermediate_dim=48)),
    "phi3": ("phi3_mlp", "lora_phi3_self_attention", "lora_phi3_mlp", dict(intermediate_dim=48)),
    "qwen2": ("qwen2_mlp", "lora_qwen2_self_attention", "lora_qwen2_mlp", dict(intermediate_dim=48)),
    "qwen3": ("qwen3_mlp", "lora_qwen3_self_attention", "lora_qwen3_mlp", dict(intermediate_dim=48, head_dim=8, q_norm=True, k_norm=True)),
    "gemma": ("gemma_mlp", "lora_gemma_self_attention", "lora_gemma_mlp", dict(intermediate_dim=48, head_dim=8)),
    "gemma2": ("gemma2_mlp", "lora_gemma2_self_attention", "lora_gemma2_mlp", dict(intermediate_dim=48, head_dim=8)),
}


def _shapes(module):
    return {k: tuple(v.shape) for k, v in module.state_dict().items()}


@pytest.mark.parametrize("family", sorted(_FAMILIES))
def test_layer_pieces_match_the_whole_model(family):
    mlp_name, attn_name, lora_mlp_name, extra = _FAMILIES[family]
    pkg = importlib.import_module(f"torchtune_b200.models.{family}")
    full = getattr(pkg, family)(**_TINY, **extra)
    layer = full.layers[0]

    mlp = getattr(pkg, mlp_name)(32, 48)
    assert _shapes(mlp) == _shapes(layer.mlp)
    assert type(mlp.activation) is type(layer.mlp.activation)

    lora_full = getattr(pkg, f"lora_{family}")(["q_proj", "v_proj"], apply_lora_to_mlp=True, lora_rank=4, lora_alpha=8.0, **_TINY, **extra)
    attn_extra = {k: v for k, v in extra.items() if k != "intermediate_dim"}
    attn = getattr(pkg, attn_name)(["q_proj", "v_proj"], embed_dim=32, num_heads=4, num_kv_heads=2, max_seq_len=16, lora_rank=4, lora_alpha=8.0, **attn_extra)
    assert _shapes(attn) == _shapes(lora_full.layers[0].attn)
    assert isinstance(attn.q_proj, LoRALinear) and not isinstance(attn.k_proj, LoRALinear)

    lora_mlp = getattr(pkg, lora_mlp_name)(dim=32, hidden_dim=48, lora_rank=4, lora_alpha=8.0)
    assert _shapes(lora_mlp) == _shapes(lora_full.layers[0].mlp)

    x = torch.randn(2, 5, 32)
    assert attn(x, x).shape == x.shape and lora_mlp(x).shape == x.shape


def test_attention_builder_rejects_no_modules_and_unknown_arguments():
    from torchtune_b200.models.llama3 import lora_llama3_self_attention

    with pytest.raises(ValueError):
        lora_llama3_self_attention([], embed_dim=32, num_heads=4, num_kv_heads=2, max_seq_len=16, lora_rank=4, lora_alpha=8.0)
    with pytest.raises(TypeError):
        lora_llama3_self_attention(["q_proj"], embed_dim=32, num_heads=4, num_kv_heads=2, max_seq_len=16, lora_rank=4, lora_alpha=8.0, not_an_argument=1)


def test_family_attention_classes_match_the_whole_model_layers():
    from torchtune_b200.models.gemma2 import gemma2
    from torchtune_b200.models.gemma2._attention import Gemma2Attention
    from torchtune_b200.models.qwen3 import qwen3
    from torchtune_b200.models.qwen3._attention import Qwen3Attention
    from torchtune_b200.modules import RMSNorm, RotaryPositionalEmbeddings
    from torchtune_b200.modules.linear import Linear

    torch.manual_seed(0)
    x = torch.randn(2, 12, 32)

    full = gemma2(**_TINY, intermediate_dim=48, head_dim=8, sliding_window_size=4, query_pre_attn_scalar=16, hidden_capping_value=20.0).eval()
    layer = full.layers[0]  # even layers carry the window
    ref = layer.attn
    mine = Gemma2Attention(embed_dim=32, num_heads=4, num_kv_heads=2, head_dim=8, q_proj=Linear(32, 32, bias=False), k_proj=Linear(32, 16, bias=False),
                           v_proj=Linear(32, 16, bias=False), output_proj=Linear(32, 32, bias=False),
                           pos_embeddings=RotaryPositionalEmbeddings(dim=8, max_seq_len=16, base=10_000), max_seq_len=16, sliding_window_size=4,
                           softcapping=20.0, query_pre_attn_scalar=16).eval()
    mine.load_state_dict(ref.state_dict())
    want = ref(x, x, mask=layer.mask_mod(None, 2, 12))
    assert torch.allclose(mine(x, x), want, atol=1e-5)
    assert not torch.allclose(mine(x, x), ref(x, x), atol=1e-5)  # the window changes the result at this length

    fullq = qwen3(**_TINY, intermediate_dim=48, head_dim=8, q_norm=True, k_norm=True).eval()
    refq = fullq.layers[0].attn
    mineq = Qwen3Attention(embed_dim=32, num_heads=4, num_kv_heads=2, head_dim=8, q_proj=Linear(32, 32, bias=True), k_proj=Linear(32, 16, bias=True),
                           v_proj=Linear(32, 16, bias=True), output_proj=Linear(32, 32, bias=False), pos_embeddings=refq.pos_embeddings,
                           q_norm=RMSNorm(8, eps=1e-5), k_norm=RMSNorm(8, eps=1e-5), max_seq_len=16).eval()
    mineq.load_state_dict(refq.state_dict())
    assert mineq.qk_norm_before_rope
    assert torch.allclose(mineq(x, x), refq(x, x), atol=1e-6)


def test_clip_and_llama4_layer_pieces():
    from torch import nn

    from torchtune_b200.models.clip._component_builders import clip_mlp, lora_clip_attention, lora_clip_mlp
    from torchtune_b200.models.llama4._component_builders import llama4_mlp, lora_llama4_mlp, lora_llama4_self_attention
    from torchtune_b200.modules import RotaryPositionalEmbeddings

    x = torch.randn(2, 7, 32)
    attn = lora_clip_attention(["q_proj", "output_proj"], embed_dim=32, head_dim=8, num_heads=4, num_kv_heads=4, attn_bias=True, lora_rank=4, lora_alpha=8.0)
    assert isinstance(attn.q_proj, LoRALinear) and isinstance(attn.output_proj, LoRALinear) and not isinstance(attn.k_proj, LoRALinear)
    assert attn.k_proj.bias is not None and attn(x, x).shape == x.shape
    mlp = lora_clip_mlp(in_dim=32, out_dim=32, hidden_dim=64, activation=nn.GELU(), lora_rank=4, lora_alpha=8.0)
    plain = clip_mlp(32, 32, 64, nn.GELU())
    base_keys = {k for k in mlp.state_dict() if "lora" not in k}
    assert base_keys == set(plain.state_dict()) and mlp(x).shape == x.shape

    rope = RotaryPositionalEmbeddings(dim=8, max_seq_len=16, base=500_000)
    a4 = lora_llama4_self_attention(["q_proj", "v_proj"], rope, head_dim=8, embed_dim=32, num_heads=4, num_kv_heads=2, max_seq_len=16, lora_rank=4, lora_alpha=8.0)
    assert isinstance(a4.v_proj, LoRALinear) and a4(x, x).shape == x.shape
    m4 = lora_llama4_mlp(dim=32, hidden_dim=48, lora_rank=4, lora_alpha=8.0)
    assert {k for k in m4.state_dict() if "lora" not in k} == set(llama4_mlp(32, 48).state_dict()) and m4(x).shape == x.shape
    with pytest.raises(ValueError):
        lora_clip_attention([], embed_dim=32, head_dim=8, num_heads=4, num_kv_heads=4, lora_rank=4, lora_alpha=8.0)
