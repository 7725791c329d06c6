"""GRPO losses against hand-computed values and the dev GRPO recipe end to end on CPU."""
import json
import re

import pytest
import torch

from helpers import run_tune, write_tiny_hf_checkpoint
from tokenizer_assets import write_sentencepiece_model
from torchtune_b200.dev.grpo import GRPOCompletionLoss, GRPOLoss, GRPOSimpleLoss, extract_tags, shaped_correctness_reward
from torchtune_b200.models.llama2 import llama2

ARCH = dict(vocab_size=200, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=64, max_seq_len=512, intermediate_dim=128, norm_eps=1e-5)


def test_grpo_losses_closed_form():
    old = torch.zeros(2, 3)
    new = torch.log(torch.tensor([[2.0, 1.0, 0.5], [1.0, 1.0, 1.0]]))
    ref = new.clone()  # zero KL
    adv = torch.tensor([1.0, -1.0])
    mask = torch.tensor([[True, True, True], [True, True, False]])
    loss, policy, kl, ratios, clip = GRPOLoss(epsilon=0.2, kl_coeff=0.1)(old, new, ref, adv, mask)
    # row 0 (adv 1): min(r, clip(r)) = 1.2, 1, 0.5 ; row 1 (adv -1): -1, -1 (third masked)
    assert policy.item() == pytest.approx((1.2 + 1 + 0.5 - 1 - 1) / 5, abs=1e-5)
    assert kl.item() == pytest.approx(0.0, abs=1e-7) and loss.item() == pytest.approx(-policy.item(), abs=1e-6)
    assert clip.item() == pytest.approx(1 / 5, abs=1e-6)
    _, policy_c, _, ratios_c, _ = GRPOCompletionLoss(epsilon=0.2)(old, new, ref, adv, mask)
    assert ratios_c.item() == pytest.approx(1.0) and policy_c.item() == pytest.approx(0.0, abs=1e-6)
    lp = torch.randn(2, 3, requires_grad=True)
    loss_s, policy_s, kl_s, _, _ = GRPOSimpleLoss(kl_coeff=0.0)(lp.detach(), lp, lp.detach(), adv, mask)
    loss_s.backward()
    # d/dlogp of -exp(lp - sg(lp))·A = -A per token, averaged per sequence then over sequences
    assert torch.allclose(lp.grad, torch.tensor([[-1 / 6] * 3, [1 / 4, 1 / 4, 0.0]]), atol=1e-6)


def test_reward_shaping():
    assert extract_tags("<think>a</think><answer> 7 </answer>") == {"think": ["a"], "answer": ["7"]}
    assert shaped_correctness_reward("42", "6*7=<<6*7=42>>42</think> <answer>42</answer>") == (100.0, 1.0)
    assert shaped_correctness_reward("42", "</think> <answer>$42</answer>") == (20.0, 0.0)
    assert shaped_correctness_reward("42", "no tags at all") == (10.0, 0.0)


def test_grpo_recipe_single_process(tmp_path, tune_path, monkeypatch):
    ckpt = tmp_path / "policy"
    write_tiny_hf_checkpoint(ckpt, arch=ARCH, builder=llama2)
    (tmp_path / "tok").mkdir()
    sp = write_sentencepiece_model(tmp_path / "tok", vocab_size=200)
    qa = tmp_path / "qa.json"
    qa.write_text(json.dumps([{"question": f"what is {i} plus {i}", "answer": str(2 * i)} for i in range(8)]))
    out = tmp_path / "out"
    run_tune(tune_path, f"run dev/grpo_full_finetune_distributed --config tiny/llama2_grpo checkpointer.checkpoint_dir={ckpt} tokenizer.path={sp} dataset.data_files={qa} output_dir={out} metric_logger.filename=log.txt", monkeypatch)
    text = (out / "logs" / "log.txt").read_text()
    for name in ("loss", "policy_loss", "kl_loss", "rewards", "successes", "response_lengths", "approx_policy_kl"):
        vals = [float(x) for x in re.findall(rf"\b{name}:(\S+)", text)]
        assert len(vals) == 2 and all(v == v for v in vals), (name, vals)
    assert (out / "epoch_0" / "model-00001-of-00001.safetensors").exists()


def test_grpo_chunked_output_loss_matches_unchunked_and_plain_formula():
    """Chunked logits give the same loss, statistics, log-probs and gradients as the whole tensor, and both equal the formula
    written out on full log-softmax."""
    import torch

    from torchtune_b200.dev.grpo import GRPOWithChunkedOutputLoss

    torch.manual_seed(0)
    bg, length, vocab = 6, 12, 40
    logits = torch.randn(bg, length, vocab, requires_grad=True)
    targets = torch.randint(0, vocab, (bg, length))
    ref = torch.log_softmax(torch.randn(bg, length, vocab), -1).gather(-1, targets[..., None]).squeeze(-1)
    adv = torch.randn(bg)
    mask = torch.rand(bg, length) > 0.3
    mask[:, 0] = True
    fn = GRPOWithChunkedOutputLoss(num_output_chunks=4, kl_coeff=0.2)

    whole = fn(logits, targets, ref, adv, mask)
    g_whole, = torch.autograd.grad(whole[0], logits)
    parts = fn(list(logits.chunk(4, dim=1)), targets, ref, adv, mask)
    g_parts, = torch.autograd.grad(parts[0], logits)
    for a, b in zip(whole, parts):
        torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(g_whole, g_parts, rtol=1e-5, atol=1e-7)

    logp = torch.log_softmax(logits.detach().double(), -1).gather(-1, targets[..., None]).squeeze(-1)
    d = ref.double() - logp
    kl = torch.exp(d) - d - 1
    m = mask.double()
    per_seq = ((-(adv.double()[:, None] - 0.2 * kl)) * m).sum(1) / m.sum(1)
    torch.testing.assert_close(whole[0].double(), per_seq.mean(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(whole[2].double(), ((kl * m).sum(1) / m.sum(1)).mean(), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(whole[5].double(), logp, rtol=1e-5, atol=1e-6)
    assert whole[3].item() == 1.0 and whole[4].item() == 0.0
