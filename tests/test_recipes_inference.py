"""generate / quantize / eleuther_eval recipes on CPU with a tiny Llama-2 and a generated
sentencepiece tokenizer."""
import json
from pathlib import Path

import pytest
import torch

from helpers import fixed_init_, run_tune, write_tiny_hf_checkpoint
from tokenizer_assets import write_sentencepiece_model
from torchtune_b200.evaluation import EvalLM
from torchtune_b200.models.llama2 import llama2, llama2_tokenizer

ARCH = dict(vocab_size=200, num_layers=2, num_heads=4, num_kv_heads=2, embed_dim=64, max_seq_len=256, intermediate_dim=128, norm_eps=1e-5)
MODEL_ARGS = " ".join(f"model.{k}={v}" for k, v in ARCH.items())


def _common(tmp_path):
    ckpt = tmp_path / "ckpt"
    write_tiny_hf_checkpoint(ckpt, arch=ARCH, builder=llama2)
    (tmp_path / "tok").mkdir(exist_ok=True)
    sp = write_sentencepiece_model(tmp_path / "tok", vocab_size=200)
    return (
        f"model._component_=torchtune_b200.models.llama2.llama2 {MODEL_ARGS} checkpointer.checkpoint_dir={ckpt} "
        f"checkpointer.checkpoint_files=[model-00001-of-00001.safetensors] device=cpu dtype=fp32 output_dir={tmp_path / 'out'}"
    ), sp


def test_generate_recipe(tmp_path, tune_path, monkeypatch, caplog):
    common, sp = _common(tmp_path)
    run_tune(tune_path, f"run generate --config generation {common} tokenizer.path={sp} max_new_tokens=12 prompt.user=hello top_k=5", monkeypatch)
    assert "tokens/sec" in caplog.text


def test_quantize_then_load(tmp_path, tune_path, monkeypatch):
    common, _ = _common(tmp_path)
    run_tune(tune_path, f"run quantize --config quantization {common} quantizer.groupsize=32", monkeypatch)
    out = tmp_path / "out" / "model-00001-of-00001-8da4w.pt"
    sd = torch.load(out)
    packed = [k for k in sd if k.endswith("weight_packed")]
    assert packed and all(sd[k].dtype == torch.uint8 for k in packed)
    assert sd["tok_embeddings.weight"].dtype == torch.float32


def test_eval_lm_scores_match_manual(tmp_path):
    (tmp_path / "tok").mkdir(exist_ok=True)
    sp = write_sentencepiece_model(tmp_path / "tok", vocab_size=200)
    tok = llama2_tokenizer(str(sp))
    model = llama2(**ARCH)
    fixed_init_(model, std=0.3)
    lm = EvalLM(model, tok, device=torch.device("cpu"), dtype=torch.float32, batch_size=2)
    reqs = [("the quick brown", " fox jumps"), ("hello", " world"), ("a b c ", "d")]
    got = lm.loglikelihood(reqs)
    for (ctx, cont), (ll, greedy) in zip(reqs, got):
        c, k = lm._encode_pair(ctx, cont)
        ids = torch.tensor([c + k])
        logp = torch.log_softmax(model(ids)[0].float(), -1)
        want = sum(logp[len(c) - 1 + i, t].item() for i, t in enumerate(k))
        assert ll == pytest.approx(want, abs=1e-3)
        assert greedy == all(logp[len(c) - 1 + i].argmax().item() == t for i, t in enumerate(k))
    assert lm.loglikelihood_rolling(["the quick brown fox"])[0] < 0
    text = lm.generate_until([("hello", {"until": ["\n"], "max_gen_toks": 8})])[0]
    assert isinstance(text, str) and "\n" not in text


def test_eleuther_eval_recipe_jsonl(tmp_path, tune_path, monkeypatch, caplog):
    common, sp = _common(tmp_path)
    task = tmp_path / "mc.jsonl"
    docs = [{"query": f"question {i} answer:", "choices": [" yes", " no", " maybe so"], "gold": i % 3} for i in range(6)]
    task.write_text("\n".join(json.dumps(d) for d in docs))
    run_tune(tune_path, f"run eleuther_eval --config eleuther_evaluation {common} tokenizer.path={sp} tasks=[{task}] batch_size=4 limit=5", monkeypatch)
    assert "acc_norm" in caplog.text and "'n': 5" in caplog.text


def test_generate_v2_recipe_and_its_tensor_parallel_twin_decode_the_same_text(tmp_path, tune_path, monkeypatch, caplog):
    """dev/generate_v2 on one process, then dev/generate_v2_distributed on two gloo ranks (decoder split over the ranks, per-rank
    KV caches): greedy decoding must give the same completion."""
    import os
    import re
    import subprocess
    import sys

    common, sp = _common(tmp_path)
    args = f"{common} tokenizer.path={sp} tokenizer.max_seq_len=128 max_new_tokens=10 prompt.user=hello prompt.system=null temperature=0.0 top_k=null"
    run_tune(tune_path, f"run dev/generate_v2 --config llama2/generation_v2 {args}", monkeypatch)
    assert "tokens/sec" in caplog.text
    single = re.findall(r"\n\n(.*)\n\n", caplog.text)[-1]
    root = Path(tune_path).resolve().parents[2]
    env = dict(os.environ, PYTHONPATH=str(root), MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    res = subprocess.run([sys.executable, str(root / "tune"), "run", "--nnodes=1", "--nproc_per_node=2", "--master-addr=127.0.0.1", "--master-port=29597", "dev/generate_v2_distributed",
                          "--config", "llama2/generation_v2"] + args.split(), cwd=str(root), env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert len(single) > 0 and f"\n\n{single}\n" in res.stdout + res.stderr, (single, (res.stdout + res.stderr)[-1500:])


def test_prompt_to_messages_and_step_visibility():
    from torchtune_b200.engine.inference import CachedDecoder, prompt_to_messages

    msgs = prompt_to_messages({"system": "be brief", "user": {"text": "hi"}, "ipython": None})
    assert [m.role for m in msgs] == ["system", "user", "assistant"] and msgs[-1].text_content == ""
    with pytest.raises(ValueError):
        prompt_to_messages({"user": {"image": "x.png"}})
    dec = CachedDecoder(lambda *a, **k: None, torch.device("cpu"), total=6, temperature=0.0, top_k=None, stop_tokens=[])
    assert dec.visibility(0, 3)[0].tolist() == torch.tril(torch.ones(6, 6, dtype=torch.bool))[:3].tolist()
    assert dec.visibility(4, 1)[0, 0].tolist() == [True] * 5 + [False]


def test_eval_lm_chat_template(tmp_path):
    """The harness' chat mode: turns are wrapped by the tokenizer's prompt template, a generation prompt is opened, and a tokenizer
    without any template is refused."""
    (tmp_path / "tok").mkdir(exist_ok=True)
    sp = write_sentencepiece_model(tmp_path / "tok", vocab_size=200)
    model = llama2(**ARCH)
    lm = EvalLM(model, llama2_tokenizer(str(sp)), device=torch.device("cpu"), dtype=torch.float32)  # Llama-2 tokenizers carry the [INST] template
    text = lm.apply_chat_template([{"role": "system", "content": "be brief"}, {"role": "user", "content": "hello"}])
    assert text.startswith("[INST] <<SYS>>\nbe brief\n<</SYS>>\n\nhello [/INST]")
    assert lm.chat_template() == "Llama2ChatTemplate" and lm.tokenizer_name == "Llama2Tokenizer"

    bare = llama2_tokenizer(str(sp), prompt_template=None)
    bare.prompt_template = None
    with pytest.raises(ValueError, match="prompt template"):
        EvalLM(model, bare, device=torch.device("cpu"), dtype=torch.float32).apply_chat_template([{"role": "user", "content": "x"}])
