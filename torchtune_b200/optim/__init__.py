from .adamw import AdamW
from .adamw8bit import AdamW8bit

__all__ = ["AdamW", "AdamW8bit"]


def resident_optimizer(params, optimizer_class="torch.optim.AdamW", *, offload_gradients: bool = False, **kwargs):
    """Stand-in for ``torchao.optim.CPUOffloadOptimizer`` in configs written for the reference's memory-saving recipes: builds
    ``optimizer_class(params, **kwargs)`` on the device.  Nothing is moved to the host — 180 GB of device memory hold the optimizer
    state of every model these single-device configs target; ``offload_gradients`` is accepted and has no effect."""
    if isinstance(optimizer_class, str):
        from ..config._resolve import get_component_from_path

        optimizer_class = get_component_from_path(optimizer_class)
    return optimizer_class(params, **kwargs)


__all__ += ["resident_optimizer"]
