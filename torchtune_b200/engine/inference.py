"""Single-conversation decoding shared by the ``dev/generate_v2*`` recipes (reference behaviour:
recipes/dev/generate_v2.py:28-243 and recipes/dev/generate_v2_distributed.py:40-270).

Pieces:

* :func:`prompt_to_messages` — the config's ``prompt`` section (role → text, or role → ``{image, text}``) as messages that end
  with an open assistant turn;
* :class:`CachedDecoder` — the decode loop on a KV cache.  Attention visibility is described per step by *one row per new
  token* (``key position ≤ token position``), built from an ``arange``; no ``[total, total]`` triangular matrix is ever
  materialised, and the rows go through the attention kernel's boolean-mask path;
* :class:`SingleTurnGenerator` — model + transform + the multimodal batch plumbing for deep-fusion (cross-attention) and
  early-fusion (image tokens spliced into the sequence) models, on one device or tensor-parallel over all ranks
  (``tensor_parallel=True``: the decoder — also the decoder inside an early-fusion model — is sliced with
  :func:`~torchtune_b200.parallel.tp_model.tensor_parallelize`; every rank samples with the same seed).
"""
from __future__ import annotations

import time
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch
from torch import nn

from .. import config, training, utils
from ..config import DictConfig, OmegaConf
from ..data import Message, load_image, padded_collate, padded_collate_tiled_images_and_mask
from ..generation import sample
from ..modules.model_fusion import DeepFusionModel, EarlyFusionModel


def _content_parts(content: Any) -> List[Dict[str, Any]]:
    if isinstance(content, str):
        return [{"type": "text", "content": content}]
    if not isinstance(content, dict) or "text" not in content:
        raise ValueError("a prompt entry is either a string or a mapping with a `text` key (and optionally `image`)")
    parts = [{"type": "image", "content": load_image(content["image"])}] if content.get("image") is not None else []
    return parts + [{"type": "text", "content": content["text"]}]


def prompt_to_messages(prompt: Dict[str, Any]) -> List[Message]:
    """``{system: …, user: …}`` (insertion order is turn order; ``None`` entries are skipped) → messages plus an empty assistant
    turn for the model to fill."""
    turns = [Message(role=role, content=_content_parts(content)) for role, content in prompt.items() if content is not None]
    return turns + [Message(role="assistant", content="")]


class CachedDecoder:
    """Token-by-token decoding of one sequence.  ``forward(tokens, mask=…, input_pos=…, **extras)`` must return logits
    ``[1, s, vocab]`` and keep its own KV cache of ``total`` positions."""

    def __init__(self, forward: Callable[..., torch.Tensor], device: torch.device, total: int, temperature: float, top_k: Optional[int], stop_tokens: Iterable[int]):
        self.forward, self.device, self.total = forward, device, int(total)
        self.temperature, self.top_k, self.stop_tokens = temperature, top_k, set(int(t) for t in stop_tokens)
        self._keys = torch.arange(self.total, device=device)

    def visibility(self, first: int, count: int) -> torch.Tensor:
        """``[1, count, total]`` booleans: the token at position ``first + i`` sees the cache slots ``0 … first + i``."""
        pos = torch.arange(first, first + count, device=self.device)
        return (self._keys[None, :] <= pos[:, None]).unsqueeze(0)

    def run(self, prompt: torch.Tensor, max_new_tokens: int, prefill_extras: Optional[Dict[str, Any]] = None, step_extras: Optional[Dict[str, Any]] = None) -> List[int]:
        n = prompt.shape[1]
        pos = torch.arange(n, device=self.device).unsqueeze(0)
        logits = self.forward(prompt, mask=self.visibility(0, n), input_pos=pos, **(prefill_extras or {}))[:, -1]
        out: List[int] = []
        for _ in range(max_new_tokens):
            token = sample(logits, temperature=self.temperature, top_k=self.top_k)
            out.append(int(token.item()))
            if out[-1] in self.stop_tokens or n >= self.total - 1:
                break
            logits = self.forward(token.view(1, 1), mask=self.visibility(n, 1), input_pos=torch.full((1, 1), n, device=self.device), **(step_extras or {}))[:, -1]
            n += 1
        return out


class _TPDecoderShim(nn.Module):
    """Gives a tensor-parallel decoder the calling convention an :class:`EarlyFusionModel` expects from its decoder."""

    def __init__(self, tp_decoder: nn.Module):
        super().__init__()
        self.tp_decoder = tp_decoder
        self.tok_embeddings = tp_decoder.tok_embeddings

    def setup_caches(self, *args: Any, **kwargs: Any) -> None:
        self.tp_decoder.setup_caches(*args, **kwargs)

    def caches_are_setup(self) -> bool:
        return self.tp_decoder.caches_are_setup()

    def caches_are_enabled(self) -> bool:
        return self.tp_decoder.caches_are_enabled()

    def reset_caches(self) -> None:
        self.tp_decoder.reset_caches()

    def forward(self, tokens=None, *, mask=None, input_pos=None, input_embeds=None, **_: Any) -> torch.Tensor:
        return self.tp_decoder.forward_inference(tokens, mask=mask, input_pos=input_pos, input_embeds=input_embeds)


class SingleTurnGenerator:
    def __init__(self, cfg: DictConfig, tensor_parallel: bool = False) -> None:
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(dtype=cfg.get("dtype"), device=self._device)
        self._logger = utils.get_logger(cfg.get("log_level", "INFO"))
        self._tp = None
        self._rank = 0
        if tensor_parallel:
            import torch.distributed as dist

            if not dist.is_initialized():
                dist.init_process_group("nccl" if self._device.type == "cuda" else "gloo", **({"device_id": self._device} if self._device.type == "cuda" else {}))
            self._rank = dist.get_rank()
            torch.manual_seed(int(cfg.get("seed") if cfg.get("seed") is not None else 1234))  # every rank must draw the same tokens
        else:
            training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode"))
        self._tensor_parallel = tensor_parallel

    def setup(self, cfg: DictConfig) -> None:
        ckpt = config.instantiate(cfg.checkpointer).load_checkpoint()
        if self._tensor_parallel:
            model = self._build_tensor_parallel(cfg, ckpt[training.MODEL_KEY])
        else:
            with training.set_default_dtype(self._dtype), self._device:
                model = config.instantiate(cfg.model)
            model.load_state_dict(ckpt[training.MODEL_KEY])
            model = model.eval()
        self.model = model
        self.model_transform = config.instantiate(cfg.tokenizer)
        if self._rank == 0:
            self._logger.info(f"Model was initialized with precision {self._dtype}" + (f" over {self._tp.world} ranks." if self._tp is not None else "."))

    def _build_tensor_parallel(self, cfg: DictConfig, state_dict: Dict[str, Any]) -> nn.Module:
        """The model is built without storage and the decoder is given storage and values layer by layer while it is split, so a
        decoder larger than one GPU (Llama-4 Scout: 218 GB in bf16) never exists in full on a rank; the encoders of an early-fusion
        model stay whole on every rank."""
        from ..parallel.tp import TensorParallelContext
        from ..parallel.tp_model import tensor_parallelize
        from ..training._distributed import LayerwisePreparer

        with training.set_default_dtype(self._dtype), torch.device("meta"):
            model = config.instantiate(cfg.model)
        fusion = isinstance(model, EarlyFusionModel)
        decoder = model.decoder if fusion else model
        decoder_state = {k[len("decoder."):]: v for k, v in state_dict.items() if k.startswith("decoder.")} if fusion else state_dict
        self._tp = TensorParallelContext(self._device, max_rows_per_rank=128, max_width=decoder.tok_embeddings.embedding_dim)
        sliced = tensor_parallelize(decoder, self._tp, prepare_layer=LayerwisePreparer(self._device, state_dict=decoder_state)).eval()
        if not fusion:
            return sliced
        whole = LayerwisePreparer(self._device, state_dict=state_dict)
        for name, encoder in model.encoders.items():
            whole(encoder, f"encoders.{name}.")
        model.decoder = _TPDecoderShim(sliced)
        return model.eval()

    # ------------------------------------------------------------------ batches
    def _multimodal_extras(self, inputs: Dict[str, Any], seq_len: int):
        """``(prompt tokens [1, s], extras of the prefill call, extras of every later call)`` for the three model kinds."""
        model, tf = self.model, self.model_transform
        if isinstance(model, DeepFusionModel):
            batch = padded_collate_tiled_images_and_mask([inputs], pad_direction="left", pad_max_images=1, pad_max_tiles=tf.max_num_tiles)
            prompt = batch.pop("tokens")
            batch["encoder_mask"] = batch["encoder_mask"][:, :seq_len]
            utils.batch_to_device(batch, self._device)
            # after the prefill the image features live in the cross-attention KV cache: later steps pass only the last mask row
            return prompt.to(self._device), batch, {"encoder_mask": batch["encoder_mask"][:, -1:]}
        if isinstance(model, EarlyFusionModel):
            prompt = padded_collate([{"tokens": inputs["tokens"]}], pad_direction="left", keys_to_pad=["tokens"], padding_idx=tf.pad_id)["tokens"]
            images = torch.cat(inputs["encoder_input"]["vision"]["images"]).to(self._device)
            return prompt.to(self._device), {"encoder_input": {"vision": {"images": images}}}, {}
        raise TypeError(f"{type(model).__name__} takes no images")

    def _forward(self) -> Callable[..., torch.Tensor]:
        if self._tp is not None and not isinstance(self.model, EarlyFusionModel):
            return self.model.forward_inference
        return self.model

    @torch.inference_mode()
    def generate(self, cfg: DictConfig) -> str:
        messages = prompt_to_messages(OmegaConf.to_container(cfg.prompt))
        multimodal = any(m.contains_media for m in messages)
        inputs = self.model_transform({"messages": messages}, inference=True)
        seq_len = len(inputs["tokens"])
        total = seq_len + int(cfg.max_new_tokens)
        with self._device:
            cache_kwargs = dict(batch_size=1, dtype=self._dtype, decoder_max_seq_len=total)
            if multimodal and isinstance(self.model, DeepFusionModel):
                cache_kwargs["encoder_max_seq_len"] = self.model_transform.image_seq_len
            self.model.setup_caches(**cache_kwargs)
        if multimodal:
            prompt, prefill_extras, step_extras = self._multimodal_extras(inputs, seq_len)
        else:
            prompt, prefill_extras, step_extras = torch.tensor(inputs["tokens"], device=self._device).unsqueeze(0), {}, {}
        decoder = CachedDecoder(self._forward(), self._device, total, cfg.temperature, cfg.get("top_k"), self.model_transform.stop_tokens)
        t0 = time.perf_counter()
        generated = decoder.run(prompt, int(cfg.max_new_tokens), prefill_extras, step_extras)
        if self._device.type == "cuda":
            torch.cuda.synchronize(self._device)
        dt = time.perf_counter() - t0
        text = self.model_transform.decode(generated)
        if self._rank == 0:
            self._logger.info(f"\n\n{text}\n")
            self.log_metrics(total_time=dt, tokens_per_second=len(generated) / dt)
        return text

    def log_metrics(self, total_time: float, tokens_per_second: float) -> None:
        nbytes = sum(t.numel() * t.element_size() for t in list(self.model.parameters()) + list(self.model.buffers()))
        self._logger.info(f"Time for inference: {total_time:.02f} sec total, {tokens_per_second:.02f} tokens/sec")
        self._logger.info(f"Bandwidth achieved: {nbytes * tokens_per_second / 1e9:.02f} GB/s" + (" per rank" if self._tp is not None else ""))
        if self._device.type == "cuda":
            self._logger.info(f"Max memory allocated: {training.get_memory_stats(device=self._device)['peak_memory_alloc']:.02f} GiB")

    def cleanup(self) -> None:
        if self._tp is not None:
            import torch.distributed as dist

            self._tp.close()
            dist.destroy_process_group()
