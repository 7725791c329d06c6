# tune-recipe: distributed=false
"""Evaluate a checkpoint on language-model benchmarks.

    tune run eleuther_eval --config eleuther_evaluation tasks=["truthfulqa_mc2","hellaswag"]

Parity: recipes/eleuther_eval.py:60-580 of the reference (config keys ``tasks``, ``limit``,
``batch_size``, ``max_seq_length``, ``enable_kv_cache``, ``quantizer``, ``include_path``).
Task names are run through the EleutherAI harness when it is installed; entries ending in
``.jsonl`` are files scored by the built-in evaluators, which need no extra package.  Text models
go through :class:`torchtune_b200.evaluation.EvalLM` (multiple-choice log-likelihood tasks),
vision-language models (deep-fusion, e.g. Llama-3.2-Vision with ``llama3_2_vision/11B_evaluation``)
through :class:`torchtune_b200.evaluation.EvalVLM` (greedy generation from text + images; config
keys ``image_tag``, ``max_images_per_sample``).
"""
import sys
import time
from typing import Any, Dict

import torch

from torchtune_b200 import config, training, utils
from torchtune_b200.config import DictConfig
from torchtune_b200.evaluation import EvalLM, EvalVLM, evaluate_jsonl_task, evaluate_multimodal_jsonl, run_lm_eval, run_lm_eval_multimodal
from torchtune_b200.modules.model_fusion import DeepFusionModel

logger = utils.get_logger("DEBUG")


class EleutherEvalRecipe:
    def __init__(self, cfg: DictConfig) -> None:
        self.device = utils.get_device(device=cfg.get("device"))
        self.dtype = training.get_dtype(dtype=cfg.get("dtype"), device=self.device)
        self.logger = logger
        training.set_seed(seed=cfg.get("seed"), debug_mode=cfg.get("cudnn_deterministic_mode"))
        self.limit = cfg.get("limit")
        self.tasks = list(cfg.tasks)
        self.batch_size = cfg.get("batch_size", 8)
        self.enable_kv_cache = cfg.get("enable_kv_cache", True)
        self.include_path = cfg.get("include_path")
        self.max_seq_length = cfg.get("max_seq_length", 4096)
        self.apply_chat_template = bool(cfg.get("chat_template", False))

    def setup(self, cfg: DictConfig) -> None:
        quantizer = config.instantiate(cfg.quantizer) if cfg.get("quantizer") is not None else None
        mode = training.get_quantizer_mode(quantizer)
        checkpointer = config.instantiate(cfg.checkpointer)
        if mode is not None and "qat" in mode:
            raise ValueError("You have specified a quantizer with 'QAT' - QAT quantizers should only be used during quantization aware training and when quantizing models. Please use the corresponding post-training quantizer e.g. Int8DynActInt4WeightQuantizer for Int8DynActInt4WeightQATQuantizer.")
        ckpt = checkpointer.load_checkpoint()
        with training.set_default_dtype(self.dtype), self.device:
            model = config.instantiate(cfg.model)
        model.load_state_dict(ckpt[training.MODEL_KEY])
        if mode is not None:
            model = quantizer.quantize(model).to(device=self.device)
        self.logger.info(f"Model is initialized with precision {self.dtype}.")
        self.model = model.eval()
        self.tokenizer = config.instantiate(cfg.tokenizer)
        self.multimodal = isinstance(self.model, DeepFusionModel)
        if self.multimodal:
            if mode is not None:
                raise ValueError("quantized evaluation is implemented for text models")
            self.eval_lm = EvalVLM(self.model, self.tokenizer, device=self.device, dtype=self.dtype, max_seq_length=self.max_seq_length, batch_size=self.batch_size,
                                   image_tag=cfg.get("image_tag", "<image>"), max_images_per_sample=cfg.get("max_images_per_sample", 7))
            return
        self.eval_lm = EvalLM(self.model, self.tokenizer, device=self.device, dtype=self.dtype, max_seq_length=self.max_seq_length, batch_size=self.batch_size, enable_kv_cache=self.enable_kv_cache)

    def evaluate(self) -> Dict[str, Any]:
        t0 = time.time()
        results: Dict[str, Any] = {}
        harness_tasks = [t for t in self.tasks if not str(t).endswith(".jsonl")]
        for t in self.tasks:
            if str(t).endswith(".jsonl"):
                results[str(t)] = (evaluate_multimodal_jsonl if self.multimodal else evaluate_jsonl_task)(self.eval_lm, str(t), self.limit)
        if harness_tasks:
            self.logger.info(f"Running evaluation on the following tasks: {harness_tasks}")
            out = (run_lm_eval_multimodal if self.multimodal else run_lm_eval)(self.eval_lm, harness_tasks, limit=self.limit, include_path=self.include_path, **({"apply_chat_template": True} if self.apply_chat_template else {}))
            results.update(out.get("results", out))
        self.logger.info(f"Eval completed in {time.time() - t0:.02f} seconds.")
        if self.device.type == "cuda":
            self.logger.info(f"Max memory allocated: {torch.cuda.max_memory_allocated() / 1e9:.02f} GB")
        for task, metrics in results.items():
            self.logger.info(f"{task}: {metrics}")
        return results


@config.parse
def recipe_main(cfg: DictConfig) -> None:
    config.log_config(recipe_name="EleutherEvalRecipe", cfg=cfg)
    recipe = EleutherEvalRecipe(cfg=cfg)
    recipe.setup(cfg=cfg)
    recipe.evaluate()


if __name__ == "__main__":
    sys.exit(recipe_main())
