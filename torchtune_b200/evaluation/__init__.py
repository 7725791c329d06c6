from .harness import EvalLM, evaluate_jsonl_task, run_lm_eval

__all__ = ["EvalLM", "evaluate_jsonl_task", "run_lm_eval"]
