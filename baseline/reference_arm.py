"""Runs the unmodified reference implementation (installed under ``baseline/_ref``) on the
benchmark configuration."""
from __future__ import annotations


def run(args, model_cfg, seq_len, doc_len, batch_per_gpu, lr, ClockSampler, timed_loop, dist_env) -> dict:
    return {"impl": "reference", "unavailable": "reference arm not wired up yet"}
