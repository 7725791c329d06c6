# tune-recipe: distributed=false
"""Single-prompt generation for text and image+text models (deep- and early-fusion).

    tune run dev/generate_v2 --config llama2/generation_v2 prompt.user="Hello"

Parity: recipes/dev/generate_v2.py:30-250 of the reference.  The prompt is a single-turn conversation given in the
config (``prompt.system`` / ``prompt.user``; ``prompt.user`` may be ``{image: <path or url>, text: …}``); the model's
transform turns it into tokens (+ image tiles and the cross-attention mask); decoding runs one token at a time on
the KV cache and stops at a stop token.
"""
import sys
import time
from typing import Any, Dict, List

import torch

from torchtune_b200 import config, training, utils
from torchtune_b200.config import DictConfig, OmegaConf
from torchtune_b200.data import Message, load_image, padded_collate, padded_collate_tiled_images_and_mask
from torchtune_b200.generation import sample
from torchtune_b200.modules.model_fusion import DeepFusionModel, EarlyFusionModel


class SingleTurnYAMLToMessages:
    """``{system: str, user: str | {image: loc, text: str}}`` → messages ending with an empty assistant turn."""

    def __call__(self, prompt: Dict[str, Any]) -> List[Message]:
        messages = []
        for role, content in prompt.items():
            if content is None:
                continue
            if isinstance(content, str):
                parts = [{"type": "text", "content": content}]
            elif "image" in content:
                parts = [{"type": "image", "content": load_image(content["image"])}, {"type": "text", "content": content["text"]}]
            else:
                assert "text" in content, "Multiple entries per role expect at least a text key"
                parts = [{"type": "text", "content": content["text"]}]
            messages.append(Message(role=role, content=parts))
        messages.append(Message(role="assistant", content=""))
        return messages


class InferenceRecipe:
    def __init__(self, cfg: DictConfig) -> None:
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(dtype=cfg.get("dtype"), device=self._device)
        self._logger = utils.get_logger(cfg.get("log_level", "INFO"))
        training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode"))

    def setup(self, cfg: DictConfig) -> None:
        ckpt = config.instantiate(cfg.checkpointer).load_checkpoint()
        with training.set_default_dtype(self._dtype), self._device:
            model = config.instantiate(cfg.model)
        model.load_state_dict(ckpt[training.MODEL_KEY])
        self.model = model.eval()
        self._logger.info(f"Model was initialized with precision {self._dtype}.")
        self.model_transform = config.instantiate(cfg.tokenizer)
        self.to_messages = SingleTurnYAMLToMessages()

    def log_metrics(self, total_time: float, tokens_per_second: float) -> None:
        nbytes = sum(p.numel() * p.element_size() for p in self.model.parameters()) + sum(b.numel() * b.element_size() for b in self.model.buffers())
        self._logger.info(f"Time for inference: {total_time:.02f} sec total, {tokens_per_second:.02f} tokens/sec")
        self._logger.info(f"Bandwidth achieved: {nbytes * tokens_per_second / 1e9:.02f} GB/s")
        if self._device.type == "cuda":
            stats = training.get_memory_stats(device=self._device)
            self._logger.info(f"Max memory allocated: {stats['peak_memory_alloc']:.02f} GiB")

    @torch.inference_mode()
    def generate(self, cfg: DictConfig) -> str:
        messages = self.to_messages(OmegaConf.to_container(cfg.prompt))
        multimodal = any(m.contains_media for m in messages)
        inputs = self.model_transform({"messages": messages}, inference=True)
        seq_len = len(inputs["tokens"])
        total = seq_len + cfg.max_new_tokens
        with self._device:
            self.model.setup_caches(batch_size=1, dtype=self._dtype, encoder_max_seq_len=self.model_transform.image_seq_len if multimodal else None, decoder_max_seq_len=total)
        causal = torch.tril(torch.ones(total, total, dtype=torch.bool, device=self._device))
        positions = torch.arange(total, device=self._device)
        batch: Dict[str, Any] = {}
        if isinstance(self.model, DeepFusionModel) and multimodal:
            batch = padded_collate_tiled_images_and_mask([inputs], pad_direction="left", pad_max_images=1, pad_max_tiles=self.model_transform.max_num_tiles)
            batch["encoder_mask"] = batch["encoder_mask"][:, :seq_len]
            prompt = batch.pop("tokens").to(self._device)
        elif isinstance(self.model, EarlyFusionModel) and multimodal:
            batch = padded_collate([{"tokens": inputs["tokens"]}], pad_direction="left", keys_to_pad=["tokens"], padding_idx=self.model_transform.pad_id)
            batch["encoder_input"] = {"vision": {"images": torch.cat(inputs["encoder_input"]["vision"]["images"]).to(self._device)}}
            prompt = batch.pop("tokens").to(self._device)
        else:
            prompt = torch.tensor(inputs["tokens"], device=self._device).unsqueeze(0)
        batch["mask"] = causal[None, :seq_len]
        batch["input_pos"] = positions[None, :seq_len]
        utils.batch_to_device(batch, self._device)

        generated: List[int] = []
        t0 = time.perf_counter()
        logits = self.model(prompt, **batch)[:, -1]
        token = sample(logits, temperature=cfg.temperature, top_k=cfg.get("top_k"))
        generated.append(token.item())
        if multimodal:
            batch.pop("encoder_input", None)  # image features live in the cross-attention KV cache / the spliced prefix now
            if "encoder_mask" in batch:
                batch["encoder_mask"] = batch["encoder_mask"][:, -1:]
        for _ in range(cfg.max_new_tokens):
            if token.item() in self.model_transform.stop_tokens:
                break
            batch["input_pos"] = positions[None, seq_len : seq_len + 1]
            batch["mask"] = causal[None, seq_len : seq_len + 1, :]
            logits = self.model(token.view(1, 1), **batch)[:, -1]
            token = sample(logits, temperature=cfg.temperature, top_k=cfg.get("top_k"))
            generated.append(token.item())
            seq_len += 1
            if seq_len >= total - 1:
                break
        if self._device.type == "cuda":
            torch.cuda.synchronize(self._device)
        dt = time.perf_counter() - t0
        text = self.model_transform.decode(generated)
        self._logger.info(f"\n\n{text}\n")
        self.log_metrics(total_time=dt, tokens_per_second=len(generated) / dt)
        return text


@config.parse
def main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="InferenceRecipe", cfg=cfg)
    recipe = InferenceRecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.generate(cfg=cfg)


if __name__ == "__main__":
    sys.exit(main())
