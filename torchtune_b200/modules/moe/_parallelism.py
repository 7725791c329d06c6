"""Parallel styles of mixture-of-experts layers, in the declarative form tensor-parallel plans use (reference:
torchtune/modules/moe/_parallelism.py:26-250, DTensor ``ParallelStyle`` subclasses applied by ``parallelize_module``).

Here the sharded MoE modules are built directly (:class:`torchtune_b200.parallel.tp_model.TPMoE` for expert *tensor*
parallelism, :class:`torchtune_b200.parallel.ep.ExpertParallelMoE` for expert parallelism), so a style object is a description:
it names what the engine does with the module it is attached to, and :func:`torchtune_b200.models.llama3._parallelism.validate_tp_plan`
checks a plan against the built-in layout.  Each style can also be *applied* to a stand-alone ``MoE`` / experts module, which
returns the corresponding sharded module of this package — the counterpart of calling ``parallelize_module`` with a single entry.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Optional, Tuple

from torch import nn


@dataclass(frozen=True)
class ParallelStyleSpec:
    style: str

    def __str__(self) -> str:  # plans compare styles as strings
        return self.style


class ExpertTensorParallel(ParallelStyleSpec):
    """Every rank keeps all experts but ``hidden / tp`` of each expert's width (gate / up split on their last dimension, down
    on its first); tokens are gathered, routed identically everywhere and the partial layer outputs are summed and scattered
    back by rows."""

    def __init__(self, *, input_layouts: Any = None, output_layouts: Any = None, use_local_output: bool = True):
        super().__init__("expert_tensor_parallel")

    def apply(self, moe: nn.Module, tp) -> nn.Module:
        from ...parallel.tp_model import TPMoE

        return TPMoE(moe, tp)


class ExpertParallel(ParallelStyleSpec):
    """Experts spread over the ranks (``num_experts / ep`` each); routed token rows travel to the owning rank and back over
    peer memory.  No counterpart in the reference, which has no expert parallelism."""

    def __init__(self) -> None:
        super().__init__("expert_parallel")

    def apply(self, moe: nn.Module, ep) -> nn.Module:
        from ...parallel.ep import ExpertParallelMoE

        return ExpertParallelMoE(moe, ep)


class NoParallel(ParallelStyleSpec):
    """The module (the router's gate) is replicated and sees replicated inputs; its gradient is summed over the group."""

    def __init__(self, *, input_layout: Any = None, output_layout: Any = None, use_local_output: bool = True):
        super().__init__("replicated")

    def apply(self, module: nn.Module, ctx: Any = None) -> nn.Module:
        return module


class PrepareModuleInputOutput(ParallelStyleSpec):
    """Layout changes around a module: sequence-sharded rows are gathered on the way in, partial results are summed and
    scattered by rows on the way out — what the MoE layer under expert tensor parallelism does with its activations."""

    def __init__(self, *, input_layouts: Optional[Tuple] = None, desired_input_layouts: Optional[Tuple] = None, input_kwarg_layouts: Optional[dict] = None,
                 desired_input_kwarg_layouts: Optional[dict] = None, use_local_input: bool = True, output_layouts: Optional[Tuple] = None, desired_output_layouts: Optional[Tuple] = None,
                 use_local_output: bool = True):
        super().__init__("gather_rows_in_scatter_sum_rows_out")
        for a, b, what in ((input_layouts, desired_input_layouts, "input"), (output_layouts, desired_output_layouts, "output")):
            if (a is None) != (b is None) or (a is not None and len(a) != len(b)):
                raise ValueError(f"{what}_layouts and desired_{what}_layouts should have same length!")

    def apply(self, module: nn.Module, ctx: Any = None) -> nn.Module:
        return module
