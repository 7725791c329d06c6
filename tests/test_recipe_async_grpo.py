"""Asynchronous GRPO: rewards, the fused linear GRPO loss, the weight hand-over and the whole topology (two inference workers,
post-processing, trainer, parameter server) end to end on CPU."""
import json
import re

import pytest
import torch

from helpers import run_tune, write_tiny_hf_checkpoint
from tokenizer_assets import write_sentencepiece_model
from torchtune_b200.dev.rl import LinearGRPOLoss
from torchtune_b200.dev.rl.datatypes import Trajectory
from torchtune_b200.dev.rl.rewards import FormattedMathCorrectnessReward, RewardOutput, ThinkingAnswerFormattingReward, answers_match
from torchtune_b200.dev.rl.workers import ParameterServer, ReplayBuffer, WeightUpdateReceiver
from torchtune_b200.models.llama2 import llama2

ARCH = dict(vocab_size=200, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=64, max_seq_len=512, intermediate_dim=128, norm_eps=1e-5)


def test_rewards_and_answer_matching():
    assert answers_match("1234", "the total is $1,234.00") and answers_match("0.5", "1/2") and not answers_match("12", "13")
    math = FormattedMathCorrectnessReward("answer", positive_reward=10.0)
    out = math(None, ["<think>x</think><answer>42</answer>", "42 somewhere <answer>41</answer>", "nothing"], ["42", "42", "42"])
    assert out.total_reward.tolist() == [10.0, 5.0, 0.0] and out.successes.tolist() == [1.0, 0.0, 0.0]
    fmt = ThinkingAnswerFormattingReward("think", "answer", positive_reward=1.0)
    out = fmt(None, ["<think>\na\n</think>\n<answer>\n1\n</answer>\n", "<think>a</think> <answer>1</answer>", "<answer>1</answer><think>a</think>"], ["1"] * 3)
    assert out.total_reward.tolist() == [2.0, 1.0, 0.0]
    assert set(out.log("r")) == {"r/formatting", "r/formatting/successes", "r/formatting/soft_format_reward", "r/formatting/strict_format_reward"}
    assert isinstance(out, RewardOutput)


def test_linear_grpo_loss_matches_the_formula_on_full_logits():
    torch.manual_seed(0)
    bg, length, dim, vocab = 4, 10, 16, 48
    model = torch.nn.Module()
    model.output = torch.nn.Linear(dim, vocab, bias=False)
    hidden = torch.randn(bg, length, dim, requires_grad=True)
    targets = torch.randint(0, vocab, (bg, length))
    ref = torch.log_softmax(torch.randn(bg, length, vocab), -1).gather(-1, targets[..., None]).squeeze(-1)
    adv = torch.randn(bg)
    keep = torch.rand(bg, length) > 0.3
    keep[:, 0] = True
    fn = LinearGRPOLoss(num_output_chunks=3, kl_coeff=0.2)
    fn.set_model_output(model)
    assert model.skip_output_layer
    loss, policy, kl, ratios, clipfrac, logp = fn(hidden, targets, ref, adv, keep)
    g, = torch.autograd.grad(loss, hidden)

    h2 = hidden.detach().clone().requires_grad_()
    lp = torch.log_softmax(model.output(h2).float(), -1).gather(-1, targets[..., None]).squeeze(-1)
    d = ref - lp
    per_tok = -(torch.exp(lp - lp.detach()) * adv[:, None] - 0.2 * (torch.exp(d) - d - 1))
    m = keep.float()
    want = ((per_tok * m).sum(1) / m.sum(1)).mean()
    g2, = torch.autograd.grad(want, h2)
    assert loss.item() == pytest.approx(want.item(), rel=1e-5, abs=1e-6)
    torch.testing.assert_close(g, g2, rtol=1e-4, atol=1e-6)
    torch.testing.assert_close(logp[keep], lp.detach()[keep], rtol=1e-4, atol=1e-5)
    assert ratios.item() == 1.0 and clipfrac.item() == 0.0 and kl.item() >= 0.0 and policy.item() == policy.item()


def test_parameter_server_versions_and_replay_buffer():
    a, b = torch.nn.Linear(4, 4), torch.nn.Linear(4, 4)
    server = ParameterServer(a.state_dict())
    recv = WeightUpdateReceiver(server, b)
    assert not recv.maybe_update() and recv.version == 0  # nothing published yet
    with torch.no_grad():
        a.weight.add_(1.0)
    assert server.publish(a.state_dict()) == 1
    assert recv.maybe_update() and recv.version == 1 and torch.equal(a.weight, b.weight)
    assert not recv.maybe_update()

    buf = ReplayBuffer(max_size=2)
    mk = lambda v, width: Trajectory(query_responses=torch.ones(2, 3 + width, dtype=torch.long), responses=torch.ones(2, width, dtype=torch.long), logprobs=torch.zeros(2, width),  # noqa: E731
                                     ref_logprobs=torch.zeros(2, width), query_response_padding_masks=torch.ones(2, 3 + width, dtype=torch.bool), seq_lens=torch.tensor([width, 1]),
                                     answers=["x", "x"], policy_version=v, advantages=torch.zeros(2))
    assert buf.extend(mk(3, 4)) and buf.extend(mk(5, 6))
    assert not buf.extend(mk(7, 2), should_stop=lambda: True)  # full: gives up when told to stop
    batch = buf.sample(2)
    assert batch.query_responses.shape == (4, 9) and batch.policy_version == 3 and batch.responses.shape == (4, 6)
    assert buf.sample(1, should_stop=lambda: True) is None


@pytest.mark.timeout(600)
@pytest.mark.parametrize("backend", ["thread", "process"])
def test_async_grpo_recipe_end_to_end(tmp_path, tune_path, monkeypatch, backend):
    """``process``: the inference workers are child processes feeding a multiprocessing queue and pulling weights from the
    shared-memory parameter server; ``thread``: every role is a thread of the controller."""
    ckpt = tmp_path / "policy"
    write_tiny_hf_checkpoint(ckpt, arch=ARCH, builder=llama2)
    (tmp_path / "tok").mkdir()
    sp = write_sentencepiece_model(tmp_path / "tok", vocab_size=200)
    qa = tmp_path / "qa.json"
    qa.write_text(json.dumps([{"question": f"what is {i} plus {i}", "answer": str(2 * i)} for i in range(8)]))
    out = tmp_path / "out"
    # child processes run truly in parallel and fill the queues before the first weights are published, so that run is longer:
    # later batches are then sampled after a publish
    steps = 3 if backend == "thread" else 10
    run_tune(tune_path, f"run dev/async_grpo_full_finetune_distributed --config tiny/async_grpo base_model_path={ckpt} tokenizer.path={sp} dataset.data_files={qa} output_dir={out} "
                        f"metric_logger.filename=log.txt orchestration.backend={backend} orchestration.num_steps={steps}", monkeypatch)
    text = (out / "logs" / "log.txt").read_text()
    losses = [float(x) for x in re.findall(r"train/loss:(\S+)", text)]
    assert len(losses) == steps and all(v == v for v in losses), losses
    for name in ("train/kl_loss", "train/policy_staleness", "postprocessing/groups", "rewards/formatting", "rewards/math_correctness", "inference/worker_0/policy_version"):
        assert re.search(rf"{re.escape(name)}:", text), name
    # weights were published and picked up: some inference worker reports a policy version above zero
    versions = [float(x) for x in re.findall(r"inference/worker_\d/policy_version:(\S+)", text)]
    assert max(versions) >= 1
    assert (out / "epoch_0" / "model-00001-of-00001.safetensors").exists()
