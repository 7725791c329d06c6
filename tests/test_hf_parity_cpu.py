"""Every decoder family against the `transformers` implementation of the same architecture: a tiny random model is written with
``save_pretrained``, read through this package's Hugging Face checkpointer, loaded into this package's builder, and the logits are
compared; then the weights are saved back in Hugging Face format and read by `transformers` again."""
import glob
import os

import pytest
import torch

transformers = pytest.importorskip("transformers")

from torchtune_b200.training import FullModelHFCheckpointer  # noqa: E402

_D = dict(vocab_size=128, hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4)
_T = dict(vocab_size=128, num_layers=2, num_heads=4, embed_dim=64, intermediate_dim=96, max_seq_len=64)
_LLAMA3_ROPE = lambda factor: dict(rope_type="llama3", factor=factor, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192)  # noqa: E731


def _llama2():
    from torchtune_b200.models.llama2 import llama2

    cfg = transformers.LlamaConfig(**_D, num_key_value_heads=4, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0, tie_word_embeddings=False)
    return transformers.LlamaForCausalLM, cfg, "LLAMA2", lambda: llama2(**_T, num_kv_heads=4)


def _llama3_1():
    from torchtune_b200.models.llama3_1 import llama3_1

    cfg = transformers.LlamaConfig(**_D, num_key_value_heads=2, max_position_embeddings=16384, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=_LLAMA3_ROPE(8.0), tie_word_embeddings=False)
    return transformers.LlamaForCausalLM, cfg, "LLAMA3", lambda: llama3_1(**_T, num_kv_heads=2, rope_base=500000, scale_factor=8)


def _llama3_2():
    from torchtune_b200.models.llama3_2 import llama3_2

    cfg = transformers.LlamaConfig(**_D, num_key_value_heads=2, max_position_embeddings=16384, rms_norm_eps=1e-5, rope_theta=500000.0, rope_scaling=_LLAMA3_ROPE(32.0), tie_word_embeddings=True)
    return transformers.LlamaForCausalLM, cfg, "LLAMA3_2", lambda: llama3_2(**_T, num_kv_heads=2)


def _mistral():
    from torchtune_b200.models.mistral import mistral

    cfg = transformers.MistralConfig(**_D, num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0, sliding_window=None, head_dim=16)
    return transformers.MistralForCausalLM, cfg, "MISTRAL", lambda: mistral(**_T, num_kv_heads=2)


def _qwen2(tie):
    def make():
        from torchtune_b200.models.qwen2 import qwen2

        cfg = transformers.Qwen2Config(**_D, num_key_value_heads=2, max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=tie)
        return transformers.Qwen2ForCausalLM, cfg, "QWEN2", lambda: qwen2(**_T, num_kv_heads=2, norm_eps=1e-6, tie_word_embeddings=tie)

    return make


def _qwen3():
    from torchtune_b200.models.qwen3 import qwen3

    cfg = transformers.Qwen3Config(**_D, num_key_value_heads=2, head_dim=32, max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, attention_bias=False)
    return transformers.Qwen3ForCausalLM, cfg, "QWEN3", lambda: qwen3(**_T, num_kv_heads=2, head_dim=32, norm_eps=1e-6, q_proj_bias=False, k_proj_bias=False, v_proj_bias=False, q_norm=True, k_norm=True)


def _gemma():
    from torchtune_b200.models.gemma import gemma

    cfg = transformers.GemmaConfig(**_D, num_key_value_heads=1, head_dim=32, max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=10000.0, hidden_activation="gelu_pytorch_tanh")
    return transformers.GemmaForCausalLM, cfg, "GEMMA", lambda: gemma(**_T, head_dim=32, num_kv_heads=1)


def _gemma2():
    from torchtune_b200.models.gemma2 import gemma2

    cfg = transformers.Gemma2Config(**_D, num_key_value_heads=2, head_dim=32, max_position_embeddings=64, rms_norm_eps=1e-6, rope_theta=10000.0, query_pre_attn_scalar=24, sliding_window=8,
                                    attn_logit_softcapping=20.0, final_logit_softcapping=10.0, attn_implementation="eager")
    return transformers.Gemma2ForCausalLM, cfg, "GEMMA2", lambda: gemma2(**_T, head_dim=32, num_kv_heads=2, hidden_capping_value=20.0, final_capping_value=10.0, sliding_window_size=8, query_pre_attn_scalar=24)


def _phi3():
    from torchtune_b200.models.phi3 import phi3

    cfg = transformers.Phi3Config(**_D, num_key_value_heads=4, max_position_embeddings=64, original_max_position_embeddings=64, rms_norm_eps=1e-5, rope_theta=10000.0, pad_token_id=0, tie_word_embeddings=False)
    return transformers.Phi3ForCausalLM, cfg, "PHI3_MINI", lambda: phi3(**_T, num_kv_heads=4)


_CASES = {"llama2": _llama2, "llama3_1": _llama3_1, "llama3_2_tied": _llama3_2, "mistral": _mistral, "qwen2": _qwen2(False), "qwen2_tied": _qwen2(True), "qwen3": _qwen3,
          "gemma": _gemma, "gemma2": _gemma2, "phi3": _phi3}


@pytest.mark.parametrize("case", sorted(_CASES))
def test_logits_match_transformers_and_weights_round_trip(case, tmp_path):
    hf_cls, cfg, model_type, build = _CASES[case]()
    torch.manual_seed(0)
    hf = hf_cls(cfg).eval().float()
    src = tmp_path / "hf"
    hf.save_pretrained(src, safe_serialization=True)
    files = sorted(os.path.basename(f) for f in glob.glob(str(src / "*.safetensors")))
    ck = FullModelHFCheckpointer(checkpoint_dir=str(src), checkpoint_files=files, model_type=model_type, output_dir=str(tmp_path / "out"))
    state = ck.load_checkpoint()["model"]
    mine = build().eval()
    mine.load_state_dict(state)  # strict: every key of the model is provided and nothing is left over

    tokens = torch.randint(0, cfg.vocab_size, (2, 17))  # longer than the sliding window of the case that has one
    with torch.no_grad():
        want = hf(input_ids=tokens).logits
        got = mine(tokens)
    assert torch.allclose(got, want, atol=2e-6, rtol=1e-5), (got - want).abs().max()

    # back to the Hugging Face layout; `transformers` must read the same weights it wrote
    ck.save_checkpoint({"model": mine.state_dict()}, epoch=0)
    written = sorted(glob.glob(str(tmp_path / "out" / "epoch_0" / "*.safetensors")))
    assert written
    from safetensors.torch import load_file

    back = {}
    for f in written:
        back.update(load_file(f))
    original = hf.state_dict()
    tied = getattr(cfg, "tie_word_embeddings", False)
    for key, value in original.items():
        if key == "lm_head.weight" and (tied or key not in back):
            continue
        assert key in back, key
        assert torch.equal(back[key], value), key


def test_gemma2_logit_cap_in_the_fused_loss_and_the_reference_graph():
    from torchtune_b200.models.gemma2 import gemma2
    from torchtune_b200.modules.loss import LinearCrossEntropyLoss

    kw = dict(**_T, head_dim=32, num_kv_heads=2, hidden_capping_value=20.0, final_capping_value=2.0, sliding_window_size=8, query_pre_attn_scalar=24)
    torch.manual_seed(0)
    model = gemma2(**kw)
    with torch.no_grad():
        model.tok_embeddings.weight.mul_(40.0)  # logits well beyond the cap, so that it matters
    tokens = torch.randint(0, 128, (2, 12))
    labels = torch.randint(0, 128, (2, 12))
    labels[0, :3] = -100

    logits = model(tokens)
    peak = float(logits.detach().abs().max())
    assert 1.5 < peak <= 2.0
    want = torch.nn.functional.cross_entropy(logits.reshape(-1, 128), labels.reshape(-1), ignore_index=-100)
    want.backward()
    want_grad = model.layers[0].mlp.w1.weight.grad.clone()
    model.zero_grad()

    loss_fn = LinearCrossEntropyLoss(num_output_chunks=4)
    loss_fn.set_model_output(model)
    assert loss_fn.logit_softcap == 2.0
    got = loss_fn(model(tokens), labels)
    got.backward()
    assert torch.allclose(got, want, atol=1e-5)
    assert torch.allclose(model.layers[0].mlp.w1.weight.grad, want_grad, atol=1e-6)

    # cap_logits=False builds the reference's graph: the cap is on the normalised hidden state, the logits are not bounded
    torch.manual_seed(0)
    ref_graph = gemma2(**kw, cap_logits=False)
    assert ref_graph.logit_softcap == 0.0 and ref_graph.norm.cap_hidden
    assert set(ref_graph.state_dict()) == set(model.state_dict())
    hidden = ref_graph.norm(torch.randn(1, 3, 64) * 50)
    assert float(hidden.abs().max()) <= 2.0


def test_every_consumer_of_hidden_states_applies_the_logit_cap():
    """Several paths skip the decoder's output layer and project hidden states themselves (preference optimisation, evaluation
    log-likelihoods, early-exit loss, distillation, the GRPO loss).  With a soft-capped decoder each must give what the decoder's own
    capped logits give."""
    import torch.nn.functional as F

    from torchtune_b200 import ops, rlhf
    from torchtune_b200.dev.rl import LinearGRPOLoss
    from torchtune_b200.engine.preference import sequence_logprobs
    from torchtune_b200.models.gemma2 import gemma2
    from torchtune_b200.modules.early_exit_loss import early_exit_loss, uniform_loss_scale

    kw = dict(**_T, head_dim=32, num_kv_heads=2, hidden_capping_value=20.0, final_capping_value=2.0, sliding_window_size=8, query_pre_attn_scalar=24)
    torch.manual_seed(0)
    model = gemma2(**kw).eval()
    with torch.no_grad():
        model.tok_embeddings.weight.mul_(40.0)
    tokens = torch.randint(0, 128, (2, 12))
    labels = tokens.clone()
    labels[:, :3] = -100
    assert ops.logit_softcap_of(model) == 2.0

    with torch.no_grad():
        logits = model(tokens)
        model.skip_output_layer = True
        hidden = model(tokens)
        model.skip_output_layer = False
    uncapped = F.linear(hidden, model.tok_embeddings.weight)
    assert float(uncapped.abs().max()) > 4.0 and float(logits.abs().max()) <= 2.0  # the cap matters here

    # preference optimisation
    want = rlhf.get_batch_log_probs(logits, labels, label_pad_token_id=-100)
    got, _ = sequence_logprobs(model, tokens, labels)
    assert torch.allclose(got, want, atol=1e-4)

    # operator level, and the GRPO loss built on it
    lp = ops.token_logprobs(hidden[:, :-1], model.tok_embeddings.weight, labels[:, 1:], -100, 4, softcap=2.0)
    ref_lp = torch.log_softmax(logits[:, :-1].float(), -1).gather(-1, labels[:, 1:].clamp_min(0).unsqueeze(-1)).squeeze(-1) * (labels[:, 1:] != -100)
    assert torch.allclose(lp, ref_lp, atol=1e-5)
    grpo = LinearGRPOLoss()
    grpo.set_model_output(model)
    model.skip_output_layer = False
    assert grpo.logit_softcap == 2.0
    out = grpo(hidden[:, :-1], labels[:, 1:].clamp_min(0), ref_lp, torch.ones(2), padding_masks=labels[:, 1:] != -100)
    assert torch.allclose(out[-1] * (labels[:, 1:] != -100), ref_lp, atol=1e-5)

    # early-exit loss over the last layer only equals plain cross entropy over the capped logits
    with torch.no_grad():
        pre_norm = model.layers[1](model.layers[0](model.tok_embeddings(tokens), mask=model.layers[0].mask_mod(None, 2, 12)))
        ee = early_exit_loss(model, {1: pre_norm}, labels, torch.nn.CrossEntropyLoss(ignore_index=-100), loss_scale_fn=uniform_loss_scale)
    ce = F.cross_entropy(logits.reshape(-1, 128), labels.reshape(-1), ignore_index=-100)
    assert torch.allclose(ee, ce, atol=1e-4)

    # what distillation uses for both student and teacher
    assert torch.allclose(model.unembed_normed(hidden), logits, atol=1e-5)
