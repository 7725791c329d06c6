"""Evaluation front-end for vision-language models (reference: the ``_VLMEvalWrapper`` around the EleutherAI harness'
multimodal model class, recipes/eleuther_eval.py:43-283).

:class:`EvalVLM` answers the harness' one multimodal request type, ``generate_until`` on (text with image tags, images): the
text is split at the tags, the images are interleaved, the model's transform builds tokens, tiles and the cross-attention
mask, and decoding is greedy on the self- and cross-attention KV caches, one sample at a time (as in the reference, which
refuses batches above one and any sampling).  Decoding goes through :class:`~torchtune_b200.engine.inference.CachedDecoder`,
so the attention masks are per-step visibility rows, not a ``[max_len, max_len]`` triangle.

Two ways to use it, like the text front-end: :func:`run_lm_eval_multimodal` adapts it to the harness when ``lm_eval`` is
installed; :func:`evaluate_multimodal_jsonl` scores a JSON-lines task (``{"query": "… <image> …", "images": [path, …],
"answer": str}`` — exact match after whitespace / case normalisation, plus a "contains" score) without any extra package.
"""
from __future__ import annotations

import json
from typing import Any, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
from torch import nn

from .. import utils
from ..data import Message, format_content_with_images, load_image, padded_collate_tiled_images_and_mask
from ..modules.common_utils import delete_kv_caches


class EvalVLM:
    def __init__(self, model: nn.Module, transform: Any, *, device: torch.device, dtype: torch.dtype = torch.bfloat16, max_seq_length: int = 4096, batch_size: int = 1,
                 enable_kv_cache: bool = True, image_tag: str = "<image>", max_images_per_sample: int = 7):
        self.model, self.transform = model.eval(), transform
        self.device, self.dtype, self.max_seq_length, self.batch_size = device, dtype, int(max_seq_length), int(batch_size)
        self.enable_kv_cache = True  # multimodal decoding always runs on the caches (image features are cached after the prefill)
        self.image_tag, self.max_images_per_sample = image_tag, int(max_images_per_sample)

    # properties the harness reads
    rank, world_size, truncation = 0, 1, True
    max_length = property(lambda self: self.max_seq_length)
    eos_token_id = property(lambda self: self.transform.tokenizer.eos_id)
    eot_token_id = property(lambda self: getattr(self.transform.tokenizer, "eot_id", self.transform.tokenizer.eos_id))

    def tok_encode(self, text: str, **_: Any) -> List[int]:
        return self.transform.tokenizer.encode(text, add_bos=False, add_eos=False)

    def tok_decode(self, tokens: Any, skip_special_tokens: bool = True) -> str:
        tokens = [tokens] if isinstance(tokens, int) else list(tokens)
        try:
            return self.transform.tokenizer.decode(tokens, skip_special_tokens=skip_special_tokens)
        except TypeError:
            return self.transform.tokenizer.decode(tokens)

    def encode_sample(self, text: str, images: Sequence[Any]) -> Dict[str, Any]:
        """One (text, images) pair → the collated single-sample batch (tokens left-padded, tiles padded to the per-sample
        image budget)."""
        rgb = [im.convert("RGB") if getattr(im, "mode", "RGB") != "RGB" else im for im in images]
        messages = [Message(role="user", content=format_content_with_images(text, image_tag=self.image_tag, images=rgb)), Message(role="assistant", content="")]
        sample = self.transform({"messages": messages}, inference=True)
        return padded_collate_tiled_images_and_mask([sample], pad_direction="left", pad_max_images=self.max_images_per_sample, pad_max_tiles=self.transform.max_num_tiles)

    @torch.inference_mode()
    def generate(self, text: str, images: Sequence[Any], max_gen_toks: int = 256, left_truncate_len: Optional[int] = None) -> List[int]:
        from ..engine.inference import CachedDecoder

        batch = self.encode_sample(text, images)
        prompt = batch.pop("tokens")
        if left_truncate_len is not None:
            prompt = prompt[:, -left_truncate_len:]
            batch["encoder_mask"] = batch["encoder_mask"][:, -left_truncate_len:]
        seq_len = prompt.shape[1]
        total = min(self.max_seq_length, seq_len + int(max_gen_toks))
        utils.batch_to_device(batch, self.device)
        with self.device:
            self.model.setup_caches(batch_size=1, dtype=self.dtype, encoder_max_seq_len=self.transform.image_seq_len * self.max_images_per_sample, decoder_max_seq_len=total)
        try:
            decoder = CachedDecoder(self.model, self.device, total, temperature=0.0, top_k=None, stop_tokens=self.transform.stop_tokens)
            return decoder.run(prompt.to(self.device), int(max_gen_toks), prefill_extras=batch, step_extras={"encoder_mask": batch["encoder_mask"][:, -1:]})
        finally:
            delete_kv_caches(self.model)

    def generate_until(self, requests: Iterable[Tuple[str, Sequence[Any], Dict[str, Any]]]) -> List[str]:
        outs = []
        for text, images, kwargs in requests:
            if kwargs.get("do_sample") or float(kwargs.get("temperature", 0.0) or 0.0) != 0.0:
                raise RuntimeError("Any decoding strategy other than greedy is not supported.")
            until = kwargs.get("until") or []
            until = [until] if isinstance(until, str) else list(until)
            out = self.tok_decode(self.generate(text, images, int(kwargs.get("max_gen_toks", 256))))
            for stop in until:
                if stop and stop in out:
                    out = out.split(stop)[0]
            outs.append(out)
        return outs


def _norm(text: str) -> str:
    return " ".join(text.lower().split()).strip(" .")


def evaluate_multimodal_jsonl(lm: EvalVLM, path: str, limit: Optional[int] = None, max_gen_toks: int = 32) -> Dict[str, float]:
    """Exact-match and containment accuracy of greedy answers over a JSON-lines file of ``{"query", "images", "answer"}``
    records (``images``: file paths or URLs, one per ``<image>`` tag of the query)."""
    docs = [json.loads(line) for line in open(path) if line.strip()]
    if limit is not None:
        docs = docs[: int(limit)]
    exact = contains = 0
    for d in docs:
        images = [load_image(p) for p in d.get("images", [])]
        got = _norm(lm.generate_until([(d["query"], images, {"max_gen_toks": max_gen_toks})])[0])
        want = _norm(str(d["answer"]))
        exact += int(got == want)
        contains += int(bool(want) and want in got)
    n = max(len(docs), 1)
    return {"exact_match": exact / n, "contains": contains / n, "n": len(docs)}


def run_lm_eval_multimodal(lm: EvalVLM, tasks: List[str], limit: Optional[int] = None, **kwargs: Any) -> Dict[str, Any]:
    """Run multimodal harness tasks (e.g. ``mmmu_val_science``) through ``lm`` (requires the ``lm_eval`` package)."""
    try:
        from lm_eval.api.model import LM
        from lm_eval.evaluator import evaluate
        from lm_eval.tasks import TaskManager, get_task_dict
    except ImportError as exc:  # pragma: no cover - depends on the environment
        raise ImportError("the EleutherAI evaluation harness is not installed: use JSON-lines tasks (tasks: [file.jsonl]) or install `lm_eval`") from exc

    class _Adapter(LM):  # pragma: no cover - exercised only with the harness installed
        MULTIMODAL = True

        def loglikelihood(self, requests):
            raise NotImplementedError("multimodal tasks are generation tasks")

        loglikelihood_rolling = loglikelihood

        def generate_until(self, requests):
            reqs = []
            for r in requests:
                context, gen_kwargs, aux = r.args if len(r.args) == 3 else (*r.args, {})
                reqs.append((context, list(aux.get("visual", [])), gen_kwargs))
            return lm.generate_until(reqs)

    task_dict = get_task_dict(tasks, TaskManager(include_path=kwargs.pop("include_path", None)))
    return evaluate(_Adapter(), task_dict, limit=limit, **kwargs)
