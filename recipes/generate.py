# tune-recipe: distributed=false
"""Text generation from a fine-tuned (optionally quantised) checkpoint.

    tune run generate --config generation prompt.user="Tell me a joke."

Parity: recipes/generate.py:29-220 of the reference — same config keys (``prompt.system`` /
``prompt.user``, ``max_new_tokens``, ``temperature``, ``top_k``, ``enable_kv_cache``,
``quantizer``).  Decoding uses the package's KV-cache attention path; the time to first token
and tokens/s are logged.
"""
import itertools
import sys
import time
from typing import Any, Dict, List, Optional

import torch

from torchtune_b200 import config, generation, training, utils
from torchtune_b200.config import DictConfig
from torchtune_b200.data import Message

logger = utils.get_logger("DEBUG")


class InferenceRecipe:
    def __init__(self, cfg: DictConfig) -> None:
        self._device = utils.get_device(device=cfg.get("device"))
        self._dtype = training.get_dtype(dtype=cfg.get("dtype"), device=self._device)
        self._quantizer = config.instantiate(cfg.quantizer) if cfg.get("quantizer") is not None else None
        self._quantization_mode = training.get_quantizer_mode(self._quantizer)
        training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode"))

    def setup(self, cfg: DictConfig) -> None:
        checkpointer = config.instantiate(cfg.checkpointer)
        ckpt = checkpointer.load_checkpoint()
        self._model = self._setup_model(cfg.model, ckpt[training.MODEL_KEY])
        self._tokenizer = config.instantiate(cfg.tokenizer)

    def _setup_model(self, model_cfg: DictConfig, state_dict: Dict[str, Any]) -> torch.nn.Module:
        with training.set_default_dtype(self._dtype), self._device:
            model = config.instantiate(model_cfg)
        model.load_state_dict(state_dict)
        if self._quantization_mode is not None:
            # weights are stored in full precision; quantise after loading
            model = self._quantizer.quantize(model) if hasattr(self._quantizer, "quantize") else self._quantizer.convert(self._quantizer.prepare(model))
            model = model.to(device=self._device)
        else:
            training.validate_expected_param_dtype(model.named_parameters(), dtype=self._dtype)
        logger.info(f"Model is initialized with precision {self._dtype}.")
        return model.eval()

    def convert_prompt_to_tokens(self, prompt: Any) -> List[int]:
        """A plain string becomes a user turn; a mapping may carry ``system`` and ``user``."""
        if isinstance(prompt, str):
            prompt = {"user": prompt}
        messages = []
        if prompt.get("system"):
            messages.append(Message(role="system", content=prompt["system"]))
        messages.append(Message(role="user", content=prompt["user"]))
        messages.append(Message(role="assistant", content=""))
        if hasattr(self._tokenizer, "tokenize_messages"):
            try:
                return self._tokenizer.tokenize_messages(messages, add_end_tokens=False)[0]
            except TypeError:
                return self._tokenizer.tokenize_messages(messages[:-1], add_eos=False)[0]
        return self._tokenizer.encode(prompt["user"], add_bos=True, add_eos=False)

    @torch.inference_mode()
    def generate(self, cfg: DictConfig) -> str:
        tokens = self.convert_prompt_to_tokens(cfg.prompt)
        prompt = torch.tensor(tokens, dtype=torch.int, device=self._device)
        total_len = prompt.numel() + cfg.max_new_tokens
        if cfg.get("enable_kv_cache", True):
            with self._device:
                self._model.setup_caches(batch_size=1, dtype=self._dtype, decoder_max_seq_len=total_len)
        t0 = time.perf_counter()
        generated, _ = generation.generate(
            model=self._model,
            prompt=prompt,
            max_generated_tokens=cfg.max_new_tokens,
            pad_id=getattr(self._tokenizer, "pad_id", 0),
            temperature=cfg.temperature,
            top_k=cfg.get("top_k"),
            stop_tokens=getattr(self._tokenizer, "stop_tokens", None),
        )
        if self._device.type == "cuda":
            torch.cuda.synchronize(self._device)
        dt = time.perf_counter() - t0
        out_tokens = generated[0].tolist()
        text = self._tokenizer.decode(out_tokens)
        logger.info(text)
        n_new = len(out_tokens) - prompt.numel()
        model_bytes = sum(p.numel() * p.element_size() for p in itertools.chain(self._model.parameters(), self._model.buffers()))
        tps = n_new / dt if dt > 0 else float("inf")
        logger.info(f"Time for inference: {dt:.02f} sec total, {tps:.02f} tokens/sec")
        logger.info(f"Bandwidth achieved: {model_bytes * tps / 1e9:.02f} GB/s")
        if self._device.type == "cuda":
            logger.info(f"Memory used: {torch.cuda.max_memory_allocated(self._device) / 1e9:.02f} GB")
        return text


@config.parse
def main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="InferenceRecipe", cfg=cfg)
    recipe = InferenceRecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.generate(cfg=cfg)


if __name__ == "__main__":
    sys.exit(main())
