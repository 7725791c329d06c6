"""Generation utilities and RLHF maths on CPU against closed-form / brute-force references."""
import math

import pytest
import torch
import torch.nn.functional as F

from torchtune_b200 import generation, rlhf
from torchtune_b200.models.llama2 import llama2
from torchtune_b200.rlhf.loss import DPOLoss, PPOLoss, RSOLoss


def _tiny():
    torch.manual_seed(0)
    return llama2(vocab_size=97, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32, max_seq_len=64, intermediate_dim=64).eval()


def test_padding_mask_helpers():
    pad = torch.tensor([[False, False, True, True], [True, True, True, True]])
    mask = generation.get_causal_mask_from_padding_mask(pad)
    assert mask.shape == (2, 4, 4)
    assert mask[0, 3].tolist() == [False, False, True, True]
    assert mask[0, 0].tolist() == [True, False, False, False]  # a padded row still attends to itself
    pos = generation.get_position_ids_from_padding_mask(pad)
    assert pos.tolist() == [[0, 0, 0, 1], [0, 1, 2, 3]]


def test_sample_greedy_and_topk():
    logits = torch.tensor([[0.1, 5.0, 0.2, 0.3]])
    assert generation.sample(logits, temperature=1e-6, top_k=1).item() == 1
    q = torch.ones(1, 4)
    assert generation.sample(logits, temperature=1.0, top_k=1, q=q).item() == 1


def test_generate_kv_cache_matches_full_forward():
    model = _tiny()
    prompt = torch.randint(1, 97, (2, 5))
    out_nc, logits_nc = generation.generate(model, prompt, max_generated_tokens=6, top_k=1, temperature=1e-6)
    model.setup_caches(batch_size=2, dtype=torch.float32, decoder_max_seq_len=16)
    out_c, logits_c = generation.generate(model, prompt, max_generated_tokens=6, top_k=1, temperature=1e-6)
    assert torch.equal(out_nc, out_c)
    assert torch.allclose(logits_nc, logits_c, atol=1e-4)


def test_generate_stop_tokens_pad_after_stop():
    model = _tiny()
    prompt = torch.randint(1, 97, (1, 4))
    out, _ = generation.generate(model, prompt, max_generated_tokens=8, top_k=1, temperature=1e-6)
    stop = int(out[0, 5])
    out2, _ = generation.generate(model, prompt, max_generated_tokens=8, top_k=1, temperature=1e-6, stop_tokens=[stop], pad_id=0)
    assert out2[0, 5] == stop or stop in out2[0, 4:6].tolist()
    first = out2[0, 4:].tolist().index(stop)
    assert all(t == 0 for t in out2[0, 4 + first + 1 :].tolist())


def test_truncate_at_first_stop_token():
    seq = torch.tensor([[869, 30, 869], [2, 30, 869], [13, 30, 5], [13, 2, 20]])
    mask, out = rlhf.truncate_sequence_at_first_stop_token(seq, torch.tensor([2, 869]), fill_value=0)
    assert out.tolist() == [[869, 0, 0], [2, 0, 0], [13, 30, 5], [13, 2, 0]]
    assert mask.tolist() == [[False, True, True], [False, True, True], [False, False, False], [False, False, True]]


def test_batch_log_probs_matches_loop():
    torch.manual_seed(1)
    logits = torch.randn(3, 7, 11)
    labels = torch.randint(0, 11, (3, 7))
    labels[0, :3] = -100
    labels[2, 5:] = -100
    got = rlhf.get_batch_log_probs(logits, labels)
    avg = rlhf.get_batch_log_probs(logits, labels, return_average_logprobs=True)
    for b in range(3):
        tot, n = 0.0, 0
        for t in range(1, 7):
            if labels[b, t] != -100:
                tot += F.log_softmax(logits[b, t - 1], -1)[labels[b, t]].item()
                n += 1
        assert got[b].item() == pytest.approx(tot, abs=1e-4)
        assert avg[b].item() == pytest.approx(tot / n, abs=1e-4)
    with pytest.raises(ValueError):
        rlhf.get_batch_log_probs(logits, labels[:, :-1])


def test_logprob_helpers_agree():
    logits = torch.randn(4, 6, 13)
    seq = torch.randint(0, 13, (4, 6))
    a = rlhf.logits_to_logprobs(logits, seq, temperature=0.7)
    b = rlhf.batched_logits_to_logprobs(logits, seq, temperature=0.7, chunk_size=3)
    assert torch.allclose(a, b, atol=1e-6)
    assert rlhf.truncate_sequence_for_logprobs(logits, 3).shape == (4, 3, 13)
    assert torch.equal(rlhf.truncate_sequence_for_logprobs(logits, 3), logits[:, 2:5])


def test_dpo_and_rso_losses():
    pol = rlhf.ChosenRejectedOutputs(torch.tensor([-1.0, -2.0]), torch.tensor([-3.0, -1.0]))
    ref = rlhf.ChosenRejectedOutputs(torch.tensor([-1.5, -2.0]), torch.tensor([-2.0, -1.0]))
    loss, cr, rr = DPOLoss(beta=0.1)(pol, ref)
    delta = torch.tensor([(-1.0 + 3.0) - (-1.5 + 2.0), 0.0])
    assert torch.allclose(loss, -F.logsigmoid(0.1 * delta))
    assert torch.allclose(cr, torch.tensor([0.05, 0.0])) and torch.allclose(rr, torch.tensor([-0.1, 0.0]))
    ls, _, _ = DPOLoss(beta=0.1, label_smoothing=0.2)(pol, ref)
    assert torch.allclose(ls, -0.8 * F.logsigmoid(0.1 * delta) - 0.2 * F.logsigmoid(-0.1 * delta))
    hinge, _, _ = RSOLoss(gamma=0.5)(pol, ref)
    assert torch.allclose(hinge, torch.relu(1 - 0.5 * delta))


def test_ppo_loss_identity_policy():
    lp = torch.randn(2, 5)
    adv = torch.randn(2, 5)
    vals = torch.randn(2, 5)
    rets = torch.randn(2, 5)
    loss, pl, vl, ratio, clip = PPOLoss(value_coeff=0.1)(lp, lp, adv, vals, vals, rets)
    assert ratio.item() == pytest.approx(1.0)
    assert clip.item() == 0.0
    assert pl.item() == pytest.approx(-adv.mean().item(), abs=1e-6)
    assert vl.item() == pytest.approx(0.5 * ((vals - rets) ** 2).mean().item(), abs=1e-6)
    assert loss.item() == pytest.approx(pl.item() + 0.1 * vl.item(), abs=1e-6)


def test_ppo_loss_clipping_and_masks():
    old = torch.zeros(1, 4)
    new = torch.tensor([[math.log(2.0), math.log(0.5), 0.0, 0.0]])
    adv = torch.tensor([[1.0, -1.0, 1.0, 1.0]])
    mask = torch.tensor([[True, True, True, False]])
    z = torch.zeros(1, 4)
    _, pl, _, _, clip = PPOLoss(epsilon=0.2)(old, new, adv, z, z, z, padding_masks=mask, value_padding_masks=mask)
    # token0: ratio 2 → clipped to 1.2 → loss -1.2 ; token1: ratio .5, adv<0 → clipped .8 → loss .8 ; token2: -1
    assert pl.item() == pytest.approx((-1.2 + 0.8 - 1.0) / 3, abs=1e-5)
    assert clip.item() == pytest.approx(2 / 3, abs=1e-5)


def test_rewards_and_gae():
    scores = torch.tensor([1.0, 2.0])
    lp = torch.tensor([[0.1, 0.2, 0.3], [0.3, 0.2, 0.1]])
    ref = torch.zeros(2, 3)
    total, kl, klr = rlhf.get_rewards_ppo(scores, lp, ref, 0.5, valid_score_idxs=torch.tensor([2, 0]))
    assert torch.allclose(kl, lp) and torch.allclose(klr, -0.5 * lp)
    assert total[0, 2].item() == pytest.approx(1.0 - 0.15) and total[1, 0].item() == pytest.approx(2.0 - 0.15)
    values = torch.tensor([[1.0, 2.0, 3.0]])
    rewards = torch.tensor([[0.5, 0.5, 0.5]])
    g, l = 0.9, 0.8
    adv, ret = rlhf.estimate_advantages(values, rewards, g, l)
    d2 = 0.5 - 3.0
    d1 = 0.5 + g * 3.0 - 2.0
    d0 = 0.5 + g * 2.0 - 1.0
    a2 = d2
    a1 = d1 + g * l * a2
    a0 = d0 + g * l * a1
    raw = torch.tensor([[a0, a1, a2]])
    assert torch.allclose(ret, raw + values, atol=1e-6)
    assert torch.allclose(adv, rlhf.whiten(raw), atol=1e-6)


def test_penalty_mask_and_whiten():
    pad = torch.tensor([[False, False, True], [False, False, False]])
    lens = torch.tensor([2, 3])
    assert rlhf.get_reward_penalty_mask(pad, lens, penalise_no_eos=True).tolist() == [False, True]
    assert rlhf.get_reward_penalty_mask(pad, lens, penalise_no_eos=False, min_response_length=3).tolist() == [True, False]
    x = torch.randn(4, 9) * 3 + 2
    w = rlhf.whiten(x, shift_mean=False)
    assert w.mean().abs() < 1e-5 and w.var().item() == pytest.approx(1.0, abs=1e-4)
    assert rlhf.whiten(x).mean().item() == pytest.approx(x.mean().item(), abs=1e-4)  # default adds the mean back (reference semantics)
    m = torch.ones_like(x, dtype=torch.bool)
    assert torch.allclose(rlhf.whiten(x, m), rlhf.whiten(x), atol=1e-5)  # second positional argument is the mask


def test_reward_codec_roundtrip():
    from torchtune_b200.rlhf.utils import reward_hf_to_tune, reward_tune_to_hf

    sd = {
        "model.embed_tokens.weight": torch.randn(10, 8),
        "model.layers.0.self_attn.q_proj.weight": torch.randn(8, 8),
        "model.layers.0.self_attn.k_proj.weight": torch.randn(4, 8),
        "model.norm.weight": torch.randn(8),
        "score.weight": torch.randn(1, 8),
    }
    t = reward_hf_to_tune(sd, num_heads=2, num_kv_heads=1, dim=8)
    assert "output.weight" in t and "tok_embeddings.weight" in t
    back = reward_tune_to_hf(t, num_heads=2, num_kv_heads=1, dim=8)
    assert back.keys() == sd.keys()
    for k in sd:
        assert torch.equal(back[k], sd[k])


def test_preference_step_trains_adapters_only():
    """One DPO step through the engine's PreferenceStep: the reference pass runs with adapters disabled, only adapter
    parameters move, and the loss of the first step equals -log(sigmoid(0)) because policy and reference coincide (LoRA B = 0)."""
    from torchtune_b200.engine.preference import PreferenceStep
    from torchtune_b200.models.llama3 import lora_llama3
    from torchtune_b200.modules.peft import get_adapter_params, set_trainable_params
    from torchtune_b200.rlhf.loss import DPOLoss

    torch.manual_seed(0)
    model = lora_llama3(lora_attn_modules=["q_proj", "v_proj"], apply_lora_to_mlp=True, vocab_size=64, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=32,
                        max_seq_len=64, intermediate_dim=64, lora_rank=4, lora_alpha=8.0)
    set_trainable_params(model, get_adapter_params(model))
    frozen = {n: p.detach().clone() for n, p in model.named_parameters() if not p.requires_grad}
    opt = torch.optim.AdamW([p for p in model.parameters() if p.requires_grad], lr=1e-2)
    step = PreferenceStep(model, DPOLoss(beta=0.1), opt, torch.device("cpu"))
    prompt = torch.randint(0, 64, (3, 5))
    tokens = torch.cat([torch.cat([prompt, prompt]), torch.randint(0, 64, (6, 11))], dim=1)
    labels = tokens.clone()
    labels[:, :5] = -100
    first = step({"tokens": tokens, "labels": labels})
    assert abs(float(first) - 0.6931472) < 1e-4
    for _ in range(5):
        last = step({"tokens": tokens, "labels": labels})
    assert float(last) < float(first)  # the adapters learn to prefer the chosen halves
    assert float(step.last_stats["rewards/accuracies"]) > 0.5
    for n, p in model.named_parameters():
        if not p.requires_grad:
            assert torch.equal(p, frozen[n])
