"""Helpers for the MXFP8 weight contract of MegaMoeExperts(precision="mxfp8").

The executor expects each expert weight as its original BF16 root tensor [e, M, N] carrying the
physical fields of the reference's contract as attributes (docs/mega_moe.md:169-200):
``col_data`` / ``col_scale [e, M/64, N, 2]`` (32-blocks along M, used forward) and ``row_data`` /
``row_scale [e, M, N/64, 2]`` (32-blocks along N, used backward). The caller owns quantisation;
``attach_mx_fields`` does it on the GPU with this library's quantiser.
"""

from __future__ import annotations

import torch

from . import kernels


def attach_mx_fields(root: torch.Tensor) -> torch.Tensor:
    """Quantise ``root`` (BF16 [e, M, N], CUDA) along both axes and store the fields on it."""
    if root.dtype != torch.bfloat16 or root.ndim != 3:
        raise TypeError("attach_mx_fields expects a BF16 [experts, M, N] tensor")
    fields = kernels.mx_quant_weight(root.detach())
    for name, value in fields.items():
        setattr(root, name, value)
    return root
