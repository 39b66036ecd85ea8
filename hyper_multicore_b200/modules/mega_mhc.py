"""MegaMhc: shifted single-pass mHC block boundary (four residual streams).

Same parameters, shapes, dtypes and errors as the reference (hyper_multicore/modules/mega_mhc/
module.py:44-185, function.py:318-365, hyper_multicore/modules/mega_mhc_common.py:28-226,
hyper_multicore/modules/mega_mhc_grad/function.py:117-203). The Ascend buffer-size bounds on the
hidden size (5760 for training, 12288 forward) do not apply; hidden % 128 == 0 is kept.
"""

from __future__ import annotations

from collections.abc import Callable
from typing import Any

import torch
from torch.autograd.function import once_differentiable

from .. import kernels
from ._precision import preserve_fp32_parameters

MHC_STREAMS = 4
MHC_MAPPINGS = MHC_STREAMS * MHC_STREAMS + 2 * MHC_STREAMS
MHC_SINKHORN_ITERS = 20
DEFAULT_TOKEN_TILE = 32


def validate_mega_mhc_hidden_size(hidden_size: int) -> None:
    if not isinstance(hidden_size, int) or isinstance(hidden_size, bool) or hidden_size <= 0:
        raise ValueError(f"hidden_size must be a positive integer, got {hidden_size!r}.")
    if hidden_size % 128:
        raise ValueError(f"hidden_size must be divisible by 128, got {hidden_size}.")


def validate_mega_mhc_inputs(previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix,
                             phi, alpha, bias, norm_weight, num_iters, token_tile) -> None:
    """Shape, dtype and device contract (mega_mhc_common.py:28-201)."""
    if not isinstance(residual, torch.Tensor):
        raise TypeError("residual must be a Tensor.")
    if residual.ndim < 3 or residual.shape[-2] != MHC_STREAMS:
        raise ValueError(f"residual must end in [{MHC_STREAMS}, H], got {tuple(residual.shape)}.")
    lead, hidden = tuple(residual.shape[:-2]), residual.shape[-1]
    spec = {
        "previous_output": (previous_output, (*lead, hidden), torch.bfloat16),
        "residual": (residual, tuple(residual.shape), torch.bfloat16),
        "previous_pre_mix": (previous_pre_mix, (*lead, MHC_STREAMS), torch.float32),
        "previous_post_mix": (previous_post_mix, (*lead, MHC_STREAMS), torch.float32),
        "previous_residual_mix": (previous_residual_mix, (*lead, MHC_STREAMS, MHC_STREAMS), torch.float32),
        "phi": (phi, (MHC_MAPPINGS, MHC_STREAMS * hidden), torch.float32),
        "alpha": (alpha, (3,), torch.float32),
        "bias": (bias, (MHC_MAPPINGS,), torch.float32),
        "norm_weight": (norm_weight, (hidden,), torch.bfloat16),
    }
    for name, (value, shape, _) in spec.items():
        if not isinstance(value, torch.Tensor):
            raise TypeError(f"{name} must be a Tensor.")
        if tuple(value.shape) != shape:
            raise ValueError(f"{name} must have shape {shape}, got {tuple(value.shape)}.")
    if num_iters != MHC_SINKHORN_ITERS:
        raise ValueError(f"initial HyperMegaMhc requires num_iters={MHC_SINKHORN_ITERS}, got {num_iters}.")
    validate_mega_mhc_hidden_size(hidden)
    if not isinstance(token_tile, int) or isinstance(token_tile, bool) or token_tile <= 0:
        raise ValueError(f"token_tile must be a positive integer, got {token_tile!r}.")
    if residual.numel() == 0:
        raise ValueError("HyperMegaMhc requires at least one token.")
    if residual.device.type != "cuda":
        raise TypeError(f"HyperMegaMhc requires CUDA tensors, got {residual.device}.")
    for name, (value, _, dtype) in spec.items():
        if value.dtype != dtype:
            raise TypeError(f"{name} must have dtype {dtype}, got {value.dtype}.")
        if value.device != residual.device:
            raise ValueError(f"{name} must be on {residual.device}, got {value.device}.")


def _forward(inputs, hc_eps, norm_eps, num_iters, need_backward):
    """Allocate outputs and caches in the reference's order (torch/ops.py:230-268, 313-369) and launch."""
    previous_output, residual = inputs[0], inputs[1]
    lead, hidden = tuple(residual.shape[:-2]), residual.shape[-1]
    tokens = residual.numel() // (MHC_STREAMS * hidden)
    device = residual.device
    contiguous = [t.contiguous() for t in inputs]
    f32 = dict(dtype=torch.float32, device=device)
    new_residual = torch.empty((tokens, MHC_STREAMS, hidden), dtype=residual.dtype, device=device)
    next_pre = torch.empty((tokens, MHC_STREAMS), **f32)
    next_post = torch.empty((tokens, MHC_STREAMS), **f32)
    next_mix = torch.empty((tokens, MHC_STREAMS * MHC_STREAMS), **f32)
    block_input = torch.empty((tokens, hidden), dtype=residual.dtype, device=device)
    hc_before_norm = torch.empty((tokens, MHC_MAPPINGS), **f32)
    inv_rms = torch.empty((tokens, 1), **f32)
    mixed_input = torch.empty((tokens, hidden), dtype=residual.dtype, device=device)
    rms_rstd = torch.empty((tokens, 1), **f32)
    kernels.mega_mhc_out(*contiguous, new_residual, next_pre, next_post, next_mix, block_input, hc_before_norm,
                         inv_rms, None, None, mixed_input, rms_rstd, hc_eps=hc_eps, norm_eps=norm_eps,
                         num_iters=num_iters, need_backward=need_backward)
    outputs = (new_residual.reshape(*lead, MHC_STREAMS, hidden), next_pre.reshape(*lead, MHC_STREAMS),
               next_post.reshape(*lead, MHC_STREAMS), next_mix.reshape(*lead, MHC_STREAMS, MHC_STREAMS),
               block_input.reshape(*lead, hidden))
    return outputs, (new_residual, hc_before_norm, inv_rms, mixed_input, rms_rstd), contiguous


class _HyperMegaMhcFunction(torch.autograd.Function):
    """Fused forward with its matching native backward (function.py:205-315)."""

    @staticmethod
    def forward(ctx, *args):  # pylint: disable=arguments-differ
        inputs, (hc_eps, norm_eps, num_iters) = args[:9], args[9:12]
        outputs, cache, contiguous = _forward(inputs, hc_eps, norm_eps, num_iters, need_backward=True)
        ctx.save_for_backward(*contiguous, *cache)
        ctx.config = (hc_eps, num_iters)
        ctx.shapes = [t.shape for t in inputs]
        return outputs

    @staticmethod
    @once_differentiable
    def backward(ctx, *grad_outputs):  # pylint: disable=arguments-differ
        saved = ctx.saved_tensors
        inputs, (new_residual, hc_before_norm, inv_rms, mixed_input, rms_rstd) = saved[:9], saved[9:]
        residual = inputs[1]
        hidden = residual.shape[-1]
        tokens = residual.numel() // (MHC_STREAMS * hidden)
        device = residual.device
        f32 = dict(dtype=torch.float32, device=device)
        shapes = [(tokens, MHC_STREAMS, hidden), (tokens, MHC_STREAMS), (tokens, MHC_STREAMS),
                  (tokens, MHC_STREAMS * MHC_STREAMS), (tokens, hidden)]
        dtypes = [residual.dtype, torch.float32, torch.float32, torch.float32, residual.dtype]
        grads = [torch.zeros(shape, dtype=dtype, device=device) if g is None
                 else g.reshape(shape).to(dtype).contiguous()
                 for g, shape, dtype in zip(grad_outputs, shapes, dtypes)]
        names = ("previous_output", "residual", "previous_pre_mix", "previous_post_mix", "previous_residual_mix",
                 "phi", "alpha", "bias", "norm_weight")
        tensors = dict(zip(names, inputs))
        tensors.update(new_residual=new_residual, hc_before_norm=hc_before_norm, inv_rms=inv_rms,
                       mixed_input=mixed_input, rms_rstd=rms_rstd, grad_new_residual=grads[0],
                       grad_next_pre_mix=grads[1], grad_next_post_mix=grads[2], grad_next_residual_mix=grads[3],
                       grad_block_input=grads[4])
        result = dict(
            grad_previous_output=torch.empty((tokens, hidden), dtype=residual.dtype, device=device),
            grad_residual=torch.empty((tokens, MHC_STREAMS, hidden), dtype=residual.dtype, device=device),
            grad_previous_pre_mix=torch.empty((tokens, MHC_STREAMS), **f32),
            grad_previous_post_mix=torch.empty((tokens, MHC_STREAMS), **f32),
            grad_previous_residual_mix=torch.empty((tokens, MHC_STREAMS * MHC_STREAMS), **f32),
            grad_phi=torch.empty((MHC_MAPPINGS, MHC_STREAMS * hidden), **f32), grad_alpha=torch.empty((3,), **f32),
            grad_bias=torch.empty((MHC_MAPPINGS,), **f32), grad_norm_weight=torch.empty((hidden,), **f32))
        tensors.update(result)
        hc_eps, num_iters = ctx.config
        kernels.mega_mhc_grad_out(tensors, hc_eps=hc_eps, num_iters=num_iters)
        ordered = [result["grad_previous_output"], result["grad_residual"], result["grad_previous_pre_mix"],
                   result["grad_previous_post_mix"], result["grad_previous_residual_mix"], result["grad_phi"],
                   result["grad_alpha"], result["grad_bias"], result["grad_norm_weight"]]
        out = []
        for grad, shape, source, needed in zip(ordered, ctx.shapes, inputs, ctx.needs_input_grad[:9]):
            out.append(grad.reshape(shape).to(source.dtype) if needed else None)
        return (*out, None, None, None, None)


def hyper_mega_mhc(previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix, phi, alpha,
                   bias, norm_weight, *, hc_eps: float = 1e-6, norm_eps: float = 1e-6,
                   num_iters: int = MHC_SINKHORN_ITERS, need_backward: bool = True,
                   token_tile: int = DEFAULT_TOKEN_TILE):
    """Run the fused shifted boundary with its matching autograd backward."""
    inputs = (previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix, phi, alpha,
              bias, norm_weight)
    validate_mega_mhc_inputs(*inputs, num_iters, token_tile)
    if need_backward and torch.is_grad_enabled() and any(t.requires_grad for t in inputs):
        return _HyperMegaMhcFunction.apply(*inputs, hc_eps, norm_eps, num_iters, token_tile)
    return _forward(inputs, hc_eps, norm_eps, num_iters, need_backward=False)[0]


class MegaMhc(torch.nn.Module):
    """Own the current layer's mapping predictor and input RMSNorm weight."""

    def __init__(self, hidden_size: int, *, hc_eps: float = 1e-6, norm_eps: float = 1e-6,
                 num_iters: int = MHC_SINKHORN_ITERS, token_tile: int = DEFAULT_TOKEN_TILE,
                 device: Any | None = None) -> None:
        super().__init__()
        validate_mega_mhc_hidden_size(hidden_size)
        if num_iters != MHC_SINKHORN_ITERS:
            raise ValueError(f"MegaMhc requires num_iters={MHC_SINKHORN_ITERS}, got {num_iters}.")
        if not isinstance(token_tile, int) or isinstance(token_tile, bool) or token_tile <= 0:
            raise ValueError(f"token_tile must be a positive integer, got {token_tile!r}.")
        self.hidden_size = hidden_size
        self.hc_eps = float(hc_eps)
        self.norm_eps = float(norm_eps)
        self.num_iters = num_iters
        self.token_tile = token_tile
        factory = {"device": device, "dtype": torch.float32}
        self.phi = torch.nn.Parameter(torch.empty((MHC_MAPPINGS, MHC_STREAMS * hidden_size), **factory))
        self.alpha = torch.nn.Parameter(torch.ones((3,), **factory))
        self.bias = torch.nn.Parameter(torch.zeros((MHC_MAPPINGS,), **factory))
        self.norm_weight = torch.nn.Parameter(torch.ones((hidden_size,), device=device, dtype=torch.bfloat16))
        torch.nn.init.normal_(self.phi, mean=0.0, std=(MHC_STREAMS * hidden_size) ** -0.5)

    def _apply(self, fn: Callable, recurse: bool = True):
        return super()._apply(preserve_fp32_parameters(self, fn, ("phi", "alpha", "bias")), recurse=recurse)

    @classmethod
    def from_module(cls, module: torch.nn.Module) -> "MegaMhc":
        """Share the Parameters of an existing four-stream shifted mHC module (module.py:105-132)."""
        configuration = {}
        for name in ("hidden_size", "hc_eps", "norm_eps", "num_iters"):
            if not hasattr(module, name):
                raise ValueError(f"source mHC module must expose {name}")
            configuration[name] = getattr(module, name)
        phi = getattr(module, "phi", None)
        if not isinstance(phi, torch.nn.Parameter):
            raise TypeError("source phi must be an FP32 Parameter [24, 4H]")
        result = cls(**configuration, device=phi.device)
        for name in ("phi", "alpha", "bias", "norm_weight"):
            parameter = getattr(module, name, None)
            expected = getattr(result, name)
            if (not isinstance(parameter, torch.nn.Parameter) or parameter.shape != expected.shape
                    or parameter.dtype != expected.dtype or parameter.device != expected.device):
                raise ValueError(f"source {name} must match shape={tuple(expected.shape)}, dtype={expected.dtype}")
            setattr(result, name, parameter)
        return result

    def forward(self, previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix):
        """Returns (new_residual, next_pre_mix, next_post_mix, next_residual_mix, block_input)."""
        return hyper_mega_mhc(previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix,
                              self.phi, self.alpha, self.bias, self.norm_weight, hc_eps=self.hc_eps,
                              norm_eps=self.norm_eps, num_iters=self.num_iters, token_tile=self.token_tile)
