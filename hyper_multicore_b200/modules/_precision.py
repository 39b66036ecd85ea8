"""Keep FP32 control parameters FP32 under Module.to(dtype) (reference: hyper_multicore/modules/_precision.py:22-53)."""

from __future__ import annotations

from collections.abc import Callable, Iterable

import torch


def preserve_fp32_parameters(module: torch.nn.Module, transform: Callable, names: Iterable[str]) -> Callable:
    """Wrap the function handed to Module._apply so the named parameters (and their existing
    gradients) follow device moves but never leave FP32."""
    keep = set()
    for name in names:
        parameter = getattr(module, name, None)
        if parameter is None:
            continue
        keep.add(id(parameter))
        if parameter.grad is not None:
            keep.add(id(parameter.grad))

    def apply(tensor: torch.Tensor) -> torch.Tensor:
        moved = transform(tensor)
        if id(tensor) not in keep or moved.dtype == torch.float32:
            return moved
        if tensor.is_meta:
            return moved.to(dtype=torch.float32)
        return tensor.to(device=moved.device, dtype=torch.float32)

    return apply
