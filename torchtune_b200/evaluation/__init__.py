from .harness import EvalLM, evaluate_jsonl_task, run_lm_eval
from .vlm import EvalVLM, evaluate_multimodal_jsonl, run_lm_eval_multimodal

__all__ = ["EvalLM", "EvalVLM", "evaluate_jsonl_task", "evaluate_multimodal_jsonl", "run_lm_eval", "run_lm_eval_multimodal"]
