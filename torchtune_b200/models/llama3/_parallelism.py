"""Tensor-parallel layout of the Llama-style decoder, in the declarative form recipe configs name through
``tensor_parallel_plan._component_`` (reference plans: torchtune/models/llama3/_parallelism.py:33-131).

The reference hands such a plan to DTensor's ``parallelize_module``.  Here the layout is *built in*:
:func:`torchtune_b200.parallel.tp_model.tensor_parallelize` constructs the sharded model directly and its collective GEMMs assume
exactly this plan, so the functions below return a description — module-path pattern → style — that
:func:`validate_tp_plan` checks against what the engine implements.  A config that names one of them therefore keeps working, and a
plan that asks for something else is refused instead of being silently ignored.
"""
from __future__ import annotations

from typing import Dict, Optional

from torch import nn

# styles
COLUMN = "column_parallel"  # weight rows (output features) split; input rows gathered from the sequence shards (all-gather → GEMM)
ROW = "row_parallel"  # weight columns (input features) split; partial outputs summed and scattered by rows (GEMM → reduce-scatter)
SEQUENCE = "sequence_parallel"  # module runs on this rank's token rows; parameters replicated, gradients summed over the group
REPLICATED_ROWS = "replicated_weight_row_sharded_tokens"  # replicated table / head applied to this rank's token rows

_BASE: Dict[str, str] = {
    "tok_embeddings": REPLICATED_ROWS,
    "norm": SEQUENCE,
    "output": REPLICATED_ROWS,
    "layers.*.sa_norm": SEQUENCE,
    "layers.*.mlp_norm": SEQUENCE,
    "layers.*.attn.q_proj": COLUMN,
    "layers.*.attn.k_proj": COLUMN,
    "layers.*.attn.v_proj": COLUMN,
    "layers.*.attn.output_proj": ROW,
    "layers.*.mlp.w1": COLUMN,
    "layers.*.mlp.w3": COLUMN,
    "layers.*.mlp.w2": ROW,
}


def base_llama_tp_plan(model: Optional[nn.Module] = None, *, enable_fp8_training: bool = False) -> Dict[str, str]:
    """Plan of a text decoder (``TransformerDecoder``).  With ``enable_fp8_training`` the column / row projections run with fp8
    operands (tensorwise scales per shard); the layout itself is the same."""
    return _fp8_llama_tp_plan() if enable_fp8_training else dict(_BASE)


def _fp8_llama_tp_plan() -> Dict[str, str]:
    return {k: (v + "+fp8" if v in (COLUMN, ROW) else v) for k, v in _BASE.items()}


def decoder_only_tp_plan(model: Optional[nn.Module] = None, *, enable_fp8_training: bool = False) -> Dict[str, str]:
    """The same plan addressed through the ``decoder.`` prefix of an early-fusion model (encoders are left alone)."""
    return {f"decoder.{k}": v for k, v in base_llama_tp_plan(model, enable_fp8_training=enable_fp8_training).items()}


def validate_tp_plan(plan: Optional[Dict[str, str]]) -> None:
    """Raise if ``plan`` asks for a layout other than the built-in one (after dropping a ``decoder.`` prefix and ``+fp8``)."""
    if not plan:
        return
    import re

    moe = {"layers.*.mlp": "gather_rows_in_scatter_sum_rows_out", "layers.*.mlp.router.gate": "replicated", "layers.*.mlp.experts": "expert_tensor_parallel",
           "layers.*.mlp.shared_expert.w1": COLUMN, "layers.*.mlp.shared_expert.w3": COLUMN, "layers.*.mlp.shared_expert.w2": ROW}
    for key, style in plan.items():
        k = key[len("decoder."):] if key.startswith("decoder.") else key
        k = re.sub(r"^layers\.\d+\.", "layers.*.", k)  # plans may name every layer (mixture-of-experts models differ per layer)
        want = _BASE.get(k, moe.get(k))
        if want is None:
            raise ValueError(f"tensor_parallel_plan names {key!r}, which the tensor-parallel engine does not shard")
        if str(style).replace("+fp8", "") != want:
            raise ValueError(f"tensor_parallel_plan wants {key!r} as {style!r}; the engine implements {want!r}")


def decoder_only_tp_training_plan(model: Optional[nn.Module] = None, *, enable_fp8_training: bool = False) -> Dict[str, str]:
    """Training plan of an early-fusion model's decoder (sequence-sharded activations)."""
    return decoder_only_tp_plan(model, enable_fp8_training=enable_fp8_training)


def decoder_only_tp_inference_plan(model: Optional[nn.Module] = None) -> Dict[str, str]:
    """Inference plan: the same weight split; activations stay replicated and every row-parallel projection is followed by an
    all-reduce (``TPDecoder.forward_inference``), so norms and embeddings are plain replicated modules."""
    return {k: ("replicated" if v in (SEQUENCE, REPLICATED_ROWS) else v) for k, v in decoder_only_tp_plan(model).items()}
