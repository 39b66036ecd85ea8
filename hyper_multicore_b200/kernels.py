"""Typed Python entry points over the C ABI: one function per ``hmc_*`` kernel.

Every function takes CUDA tensors the caller allocated, checks nothing the native side already
checks, and enqueues on torch's current stream.
"""

from __future__ import annotations

import ctypes

import torch

from . import _lib
from ._lib import (HMC_EPI_STORE_BF16, HMC_EPI_STORE_F32, HMC_EPI_SWIGLU, HMC_EPI_SWIGLU_GRAD,
                   HMC_GEMM_RAGGED_K, HMC_GEMM_RAGGED_M, HMC_MAJOR_K, HMC_MAJOR_MN, GroupedGemmArgs)


def _require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    device = None
    for tensor in tensors:
        if tensor is None:
            continue
        if not tensor.is_cuda:
            raise _lib.HmcError("hyper_multicore_b200 kernels need CUDA tensors; there is no CPU path")
        device = tensor.device if device is None else device
        if tensor.device != device:
            raise ValueError("all tensors must be on one CUDA device")
    assert device is not None
    return device


def grouped_gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    group_ends: torch.Tensor,
    *,
    mode: int,
    b_major: int = HMC_MAJOR_MN,
    epilogue: int = HMC_EPI_STORE_BF16,
    aux: torch.Tensor | None = None,
    ready_counters: torch.Tensor | None = None,
    ready_budget_ns: int = 0,
    status: torch.Tensor | None = None,
    max_ctas: int = 0,
) -> None:
    """Launch the tcgen05 grouped GEMM.

    RAGGED_M: ``a`` [rows, k]; ``b`` [groups, k, n_cols] (MN) or [groups, n_cols, k] (K); ``c`` [rows, *].
    RAGGED_K: ``a`` [rows, m]; ``b`` [rows, n]; ``c`` [groups, m, n] BF16 or FP32.
    """
    device = _require_cuda(a, b, c, group_ends, aux, ready_counters, status)
    args = GroupedGemmArgs()
    args.mode = mode
    args.epilogue = epilogue
    args.groups = group_ends.numel()
    args.max_ctas = max_ctas
    args.rows = a.shape[0]
    if mode == HMC_GEMM_RAGGED_M:
        args.a_major = HMC_MAJOR_K
        args.b_major = b_major
        args.k = a.shape[1]
        n_cols = b.shape[2] if b_major == HMC_MAJOR_MN else b.shape[1]
        args.n = n_cols // 2 if epilogue == HMC_EPI_SWIGLU else n_cols
        args.m = 0
    else:
        args.a_major = HMC_MAJOR_MN
        args.b_major = HMC_MAJOR_MN
        args.m = a.shape[1]
        args.n = b.shape[1]
        args.k = 0
    args.a = a.data_ptr()
    args.b = b.data_ptr()
    args.c = c.data_ptr()
    args.aux = _lib.ptr(aux)
    args.group_ends = group_ends.data_ptr()
    args.ready_counters = _lib.ptr(ready_counters)
    args.ready_budget_ns = ready_budget_ns
    args.status = _lib.ptr(status)
    with torch.cuda.device(device):
        _lib.check(_lib.load().hmc_grouped_gemm(ctypes.byref(args), _lib.stream_ptr(device)))
