"""Evaluation front-end for causal language models.

The reference wraps its models in the EleutherAI harness' HF model class
(recipes/eleuther_eval.py:60-470).  :class:`EvalLM` implements the three request types of
that harness — ``loglikelihood``, ``loglikelihood_rolling`` and ``generate_until`` — directly
on this package's decoder, tokenizer and KV-cache generation, so it works with or without the
harness installed:

* with ``lm_eval`` importable, :func:`run_lm_eval` adapts an :class:`EvalLM` to the harness'
  ``LM`` interface and runs the named tasks;
* without it, :func:`evaluate_jsonl_task` scores multiple-choice tasks stored as JSON lines
  (``{"query": str, "choices": [str, …], "gold": int}``) with length-normalised accuracy.

Continuation log-likelihoods use the fused ``hidden → log-prob`` operator, so ``[batch, seq,
vocab]`` logits are not materialised.
"""
from __future__ import annotations

import json
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import generation, ops
from ..modules.common_utils import delete_kv_caches


class EvalLM:
    def __init__(self, model: nn.Module, tokenizer: Any, *, device: torch.device, dtype: torch.dtype = torch.bfloat16, max_seq_length: int = 4096, batch_size: int = 8, enable_kv_cache: bool = True):
        self.model, self.tokenizer = model.eval(), tokenizer
        self.device, self.dtype = device, dtype
        self.max_seq_length, self.batch_size, self.enable_kv_cache = max_seq_length, batch_size, enable_kv_cache
        self.pad_id = getattr(tokenizer, "pad_id", 0)
        self.eos_id = getattr(tokenizer, "eos_id", None)

    # -- chat formatting (the harness calls these when a task is run with ``apply_chat_template``) -----------------------
    @property
    def tokenizer_name(self) -> str:
        return type(self.tokenizer).__name__

    def chat_template(self, chat_template: Any = False) -> str:
        """Identifies the template in the harness' result cache; the text itself comes from :meth:`apply_chat_template`."""
        template = getattr(self.tokenizer, "prompt_template", None)
        return type(template).__name__ if template is not None else ""

    def apply_chat_template(self, chat_history: List[Dict[str, str]], add_generation_prompt: bool = True) -> str:
        """One string for a list of ``{"role", "content"}`` turns (parity: recipes/eleuther_eval.py:392-403): the tokenizer's prompt
        template wraps each turn, or a Hugging Face tokenizer renders its own chat template."""
        template = getattr(self.tokenizer, "prompt_template", None)
        if template is not None:
            from ..data import Message

            turns = [Message(role=t["role"], content=t["content"]) for t in chat_history]
            if add_generation_prompt and (not turns or turns[-1].role != "assistant"):
                turns.append(Message(role="assistant", content=""))
            return "".join(m.text_content for m in template(turns, inference=True))
        if hasattr(self.tokenizer, "render_template"):
            return self.tokenizer.render_template(chat_history, add_eos=False)
        raise ValueError("You can't use a tokenizer without a prompt template and apply_chat_template: True. Use HuggingFaceModelTokenizer if you do not require a custom one.")

    # -- tokenisation -------------------------------------------------------------------
    def tok_encode(self, text: str, add_bos: bool = False) -> List[int]:
        return self.tokenizer.encode(text, add_bos=add_bos, add_eos=False)

    def tok_decode(self, tokens: Sequence[int]) -> str:
        return self.tokenizer.decode(list(tokens))

    def _encode_pair(self, context: str, continuation: str) -> Tuple[List[int], List[int]]:
        # trailing spaces of the context belong to the continuation (harness convention)
        n_spaces = len(context) - len(context.rstrip())
        if n_spaces > 0:
            continuation = context[-n_spaces:] + continuation
            context = context[:-n_spaces]
        whole = self.tok_encode(context + continuation, add_bos=True)
        ctx = self.tok_encode(context, add_bos=True)
        return ctx, whole[len(ctx) :]

    # -- scoring ------------------------------------------------------------------------
    @torch.inference_mode()
    def _score(self, rows: List[Tuple[List[int], List[int]]]) -> List[Tuple[float, bool]]:
        """Each row is (context tokens, continuation tokens); returns the summed continuation
        log-probability and whether the continuation is the greedy decode."""
        out: List[Tuple[float, bool]] = []
        core = getattr(self.model, "decoder", self.model)
        for i in range(0, len(rows), self.batch_size):
            chunk = rows[i : i + self.batch_size]
            seqs = []
            for ctx, cont in chunk:
                full = (ctx + cont)[-(self.max_seq_length + 1) :]
                seqs.append(full)
            width = max(len(s) for s in seqs)
            tokens = torch.full((len(seqs), width), self.pad_id, dtype=torch.long)
            labels = torch.full((len(seqs), width), -100, dtype=torch.long)
            for r, (s, (_, cont)) in enumerate(zip(seqs, chunk)):
                tokens[r, : len(s)] = torch.tensor(s)
                n = min(len(cont), len(s) - 1)
                labels[r, len(s) - n : len(s)] = torch.tensor(s[len(s) - n :])
            tokens, labels = tokens.to(self.device), labels.to(self.device)
            prev = getattr(core, "skip_output_layer", False)
            core.skip_output_layer = True
            try:
                hidden = self.model(tokens)
            finally:
                core.skip_output_layer = prev
            weight = core.output.weight if hasattr(core.output, "weight") else core.output.tied_module.weight
            h, y = hidden[:, :-1].contiguous(), labels[:, 1:].contiguous()
            logp = ops.token_logprobs(h, weight, y, -100, softcap=ops.logit_softcap_of(core))
            sums = logp.sum(-1).tolist()
            # greedy check on the continuation positions only
            mask = y != -100
            greedy = torch.zeros(len(seqs), dtype=torch.bool)
            sel = h[mask]
            if sel.numel():
                pred = torch.nn.functional.linear(sel, weight).argmax(-1)
                ok = torch.zeros_like(mask)
                ok[mask] = pred == y[mask]
                greedy = (ok | ~mask).all(-1).cpu()
            out.extend((float(s), bool(g)) for s, g in zip(sums, greedy.tolist()))
        return out

    def loglikelihood(self, requests: Iterable[Tuple[str, str]]) -> List[Tuple[float, bool]]:
        return self._score([self._encode_pair(c, k) for c, k in requests])

    def loglikelihood_rolling(self, requests: Iterable[str]) -> List[float]:
        res = []
        for text in requests:
            toks = self.tok_encode(text, add_bos=True)
            total = 0.0
            # disjoint windows; each window is conditioned on its own first token only
            for lo in range(0, max(len(toks) - 1, 1), self.max_seq_length):
                window = toks[lo : lo + self.max_seq_length + 1]
                if len(window) < 2:
                    break
                total += self._score([(window[:1], window[1:])])[0][0]
            res.append(total)
        return res

    # -- generation ---------------------------------------------------------------------
    @torch.inference_mode()
    def generate_until(self, requests: Iterable[Tuple[str, Dict[str, Any]]]) -> List[str]:
        outs = []
        for context, kwargs in requests:
            until = kwargs.get("until") or []
            until = [until] if isinstance(until, str) else list(until)
            max_new = int(kwargs.get("max_gen_toks", 256))
            temperature = float(kwargs.get("temperature", 0.0))
            if kwargs.get("do_sample") is False:
                temperature = 0.0
            toks = self.tok_encode(context, add_bos=True)[-(self.max_seq_length - max_new) :]
            prompt = torch.tensor(toks, dtype=torch.long, device=self.device)
            if self.enable_kv_cache:
                with self.device:
                    self.model.setup_caches(batch_size=1, dtype=self.dtype, decoder_max_seq_len=len(toks) + max_new)
            try:
                gen, _ = generation.generate(
                    self.model, prompt, max_generated_tokens=max_new, pad_id=self.pad_id,
                    temperature=temperature if temperature > 0 else 1e-6, top_k=None if temperature > 0 else 1,
                    stop_tokens=getattr(self.tokenizer, "stop_tokens", None) or ([self.eos_id] if self.eos_id is not None else None),
                )
            finally:
                if self.enable_kv_cache:
                    delete_kv_caches(self.model)
            text = self.tok_decode(gen[0, len(toks) :].tolist())
            for stop in until:
                if stop and stop in text:
                    text = text.split(stop)[0]
            outs.append(text)
        return outs


def evaluate_jsonl_task(lm: EvalLM, path: str, limit: Optional[int] = None) -> Dict[str, float]:
    """Multiple-choice accuracy (raw and byte-length normalised) over a JSON-lines file."""
    docs = [json.loads(line) for line in open(path) if line.strip()]
    if limit is not None:
        docs = docs[: int(limit)]
    requests, spans = [], []
    for d in docs:
        spans.append((len(requests), len(d["choices"])))
        requests.extend((d["query"], c) for c in d["choices"])
    scores = lm.loglikelihood(requests)
    acc = acc_norm = 0
    for d, (lo, n) in zip(docs, spans):
        ll = torch.tensor([s for s, _ in scores[lo : lo + n]])
        lens = torch.tensor([max(len(c.encode()), 1) for c in d["choices"]], dtype=torch.float)
        acc += int(ll.argmax().item() == d["gold"])
        acc_norm += int((ll / lens).argmax().item() == d["gold"])
    n = max(len(docs), 1)
    return {"acc": acc / n, "acc_norm": acc_norm / n, "n": len(docs)}


def run_lm_eval(lm: EvalLM, tasks: List[str], limit: Optional[int] = None, **kwargs: Any) -> Dict[str, Any]:
    """Run harness tasks through ``lm`` (requires the ``lm_eval`` package)."""
    try:
        from lm_eval.api.model import LM
        from lm_eval.evaluator import evaluate
        from lm_eval.tasks import TaskManager, get_task_dict
    except ImportError as exc:  # pragma: no cover - depends on the environment
        raise ImportError("the EleutherAI evaluation harness is not installed: use JSON-lines tasks (tasks: [file.jsonl]) or install `lm_eval`") from exc

    class _Adapter(LM):  # pragma: no cover - exercised only with the harness installed
        def loglikelihood(self, requests):
            return lm.loglikelihood([r.args for r in requests])

        def loglikelihood_rolling(self, requests):
            return lm.loglikelihood_rolling([r.args[0] for r in requests])

        def generate_until(self, requests):
            return lm.generate_until([r.args for r in requests])

        @property
        def tokenizer_name(self):
            return lm.tokenizer_name

        def chat_template(self, chat_template=False):
            return lm.chat_template(chat_template)

        def apply_chat_template(self, chat_history, add_generation_prompt=True):
            return lm.apply_chat_template(chat_history, add_generation_prompt)

    task_dict = get_task_dict(tasks, TaskManager(include_path=kwargs.pop("include_path", None)))
    return evaluate(_Adapter(), task_dict, limit=limit, **kwargs)
