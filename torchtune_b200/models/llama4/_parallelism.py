"""Tensor-parallel plans of the Llama-4 decoder (reference: torchtune/models/llama4/_parallelism.py:26-189): attention as in
the dense Llama plan; MoE layers under *expert tensor parallelism* (router replicated, every expert's width split, shared expert
split like a dense MLP); dense MLP layers (Maverick's odd layers) column / row parallel.  Plans are descriptions checked against
the layout :func:`torchtune_b200.parallel.tp_model.tensor_parallelize` builds (see ``models/llama3/_parallelism.py``)."""
from __future__ import annotations

from typing import Dict, Optional

from torch import nn

from ...modules.moe._parallelism import ExpertTensorParallel, NoParallel, PrepareModuleInputOutput
from ..llama3._parallelism import COLUMN, REPLICATED_ROWS, ROW, SEQUENCE


def _layers(model: Optional[nn.Module]):
    core = getattr(model, "decoder", model)
    return list(getattr(core, "layers", [])) if core is not None else []


def decoder_only_tp_training_plan(model: Optional[nn.Module] = None, *, enable_fp8_training: bool = False) -> Dict[str, object]:
    fp8 = "+fp8" if enable_fp8_training else ""
    plan: Dict[str, object] = {"decoder.tok_embeddings": REPLICATED_ROWS, "decoder.norm": SEQUENCE, "decoder.output": REPLICATED_ROWS}
    for i, layer in enumerate(_layers(model)):
        p = f"decoder.layers.{i}"
        plan.update({f"{p}.sa_norm": SEQUENCE, f"{p}.mlp_norm": SEQUENCE, f"{p}.attn.q_proj": COLUMN + fp8, f"{p}.attn.k_proj": COLUMN + fp8, f"{p}.attn.v_proj": COLUMN + fp8,
                     f"{p}.attn.output_proj": ROW + fp8})
        mlp = getattr(getattr(layer, "inner", layer), "mlp", None)
        if hasattr(mlp, "experts"):
            plan.update({f"{p}.mlp": PrepareModuleInputOutput(input_layouts=("rows",), desired_input_layouts=("replicated",), output_layouts=("partial",), desired_output_layouts=("rows",)),
                         f"{p}.mlp.router.gate": NoParallel(), f"{p}.mlp.experts": ExpertTensorParallel()})
            if getattr(mlp, "shared_expert", None) is not None:
                plan.update({f"{p}.mlp.shared_expert.w1": COLUMN + fp8, f"{p}.mlp.shared_expert.w3": COLUMN + fp8, f"{p}.mlp.shared_expert.w2": ROW + fp8})
        else:
            plan.update({f"{p}.mlp.w1": COLUMN + fp8, f"{p}.mlp.w3": COLUMN + fp8, f"{p}.mlp.w2": ROW + fp8})
    return plan


def decoder_only_tp_inference_plan(model: Optional[nn.Module] = None) -> Dict[str, object]:
    """The same weight split with replicated activations (norms and embeddings are plain replicated modules; every row-parallel
    projection and the MoE layer are followed by an all-reduce)."""
    out = {}
    for k, v in decoder_only_tp_training_plan(model).items():
        out[k] = "replicated" if str(v) in (SEQUENCE, REPLICATED_ROWS) else v
    return out


def decoder_only_tp_plan(model: Optional[nn.Module] = None, *, enable_fp8_training: bool = False, inference: bool = False) -> Dict[str, object]:
    if inference:
        if enable_fp8_training:
            raise ValueError("fp8 training plans are for training")
        return decoder_only_tp_inference_plan(model)
    return decoder_only_tp_training_plan(model, enable_fp8_training=enable_fp8_training)
