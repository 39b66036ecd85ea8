"""MegaGate: router projection + top-k routing.

Same constructor, parameters, outputs and error behaviour as the reference module
(hyper_multicore/modules/mega_gate/module.py:79-289, function.py:96-207). Every scoring function
runs through the CUDA Route / RouteGrad kernels (the reference's native path covers sqrtsoftplus
only and falls back to Torch otherwise, module.py:266-271).
"""

from __future__ import annotations

import math
from collections.abc import Callable
from typing import Any

import torch
from torch.autograd.function import once_differentiable

from .. import kernels
from ._precision import preserve_fp32_parameters

_SCORING = ("sqrtsoftplus", "softmax", "sigmoid")


def route(logits, text_bias, vision_bias, image_mask, use_vision_bias, top_k, scale, scoring, n_group=0,
          topk_group=0):
    """Allocate the five Route outputs and launch (mirror of ops._mega_gate_route)."""
    tokens, experts = logits.shape
    device = logits.device
    weights = torch.empty((tokens, top_k), dtype=torch.float32, device=device)
    indices = torch.empty((tokens, top_k), dtype=torch.int64, device=device)
    scores = torch.empty((tokens, experts), dtype=torch.float32, device=device)
    selected = torch.empty((tokens, top_k), dtype=torch.float32, device=device)
    denominator = torch.empty((tokens, 1), dtype=torch.float32, device=device)
    kernels.gate_route_out(logits, text_bias, vision_bias, image_mask, use_vision_bias, top_k, scale, scoring,
                           weights, indices, scores, selected, denominator, n_group, topk_group)
    return weights, indices, scores, selected, denominator


class _ProjectFunction(torch.autograd.Function):
    """FP32 projection with the Torch matmul backward the reference relies on (function.py:175-178)."""

    @staticmethod
    def forward(ctx, hidden, weight):  # pylint: disable=arguments-differ
        ctx.save_for_backward(hidden, weight)
        return kernels.gate_project(hidden, weight)

    @staticmethod
    def backward(ctx, grad_logits):  # pylint: disable=arguments-differ
        hidden, weight = ctx.saved_tensors
        grad_hidden = grad_weight = None
        if ctx.needs_input_grad[0]:
            grad_hidden = (grad_logits @ weight.float()).to(hidden.dtype)
        if ctx.needs_input_grad[1]:
            grad_weight = (grad_logits.t() @ hidden.float()).to(weight.dtype)
        return grad_hidden, grad_weight


class _RouteFunction(torch.autograd.Function):
    """Differentiate Route with respect to the logits only; first order (function.py:96-160)."""

    @staticmethod
    def forward(ctx, logits, text_bias, vision_bias, image_mask, use_vision_bias, top_k, scale, scoring,  # pylint: disable=arguments-differ
                n_group=0, topk_group=0):
        ctx.set_materialize_grads(False)
        weights, indices, scores, selected, denominator = route(
            logits, text_bias.detach(), vision_bias.detach(), image_mask, use_vision_bias, top_k, scale, scoring,
            n_group, topk_group)
        ctx.save_for_backward(logits, indices, scores, selected, denominator)
        ctx.config = (top_k, scale, scoring)
        ctx.mark_non_differentiable(indices)
        return weights, indices

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_weights, grad_indices):  # pylint: disable=arguments-differ
        del grad_indices
        if grad_weights is None or not ctx.needs_input_grad[0]:
            return (None,) * 10
        logits, indices, scores, selected, denominator = ctx.saved_tensors
        top_k, scale, scoring = ctx.config
        grad_logits = torch.empty_like(logits)
        kernels.gate_route_grad_out(logits, scores, selected, denominator, indices, grad_weights.contiguous().float(),
                                    top_k, scale, scoring, grad_logits)
        return (grad_logits,) + (None,) * 9


class _GateFunction(torch.autograd.Function):
    """Projection and Route as one launch; the backward of ``_RouteFunction`` followed by ``_ProjectFunction``'s."""

    @staticmethod
    def forward(ctx, hidden, weight, text_bias, vision_bias, image_mask, use_vision_bias, top_k, scale, scoring):  # pylint: disable=arguments-differ
        ctx.set_materialize_grads(False)
        logits, weights, indices, scores, selected, denominator = kernels.gate_project_route(
            hidden, weight, text_bias.detach(), vision_bias.detach(), image_mask, use_vision_bias, top_k, scale, scoring)
        ctx.save_for_backward(hidden, weight, logits, indices, scores, selected, denominator)
        ctx.config = (top_k, scale, scoring)
        ctx.mark_non_differentiable(indices)
        return logits, weights, indices

    @staticmethod
    @once_differentiable
    def backward(ctx, grad_logits, grad_weights, grad_indices):  # pylint: disable=arguments-differ
        del grad_indices
        hidden, weight, logits, indices, scores, selected, denominator = ctx.saved_tensors
        top_k, scale, scoring = ctx.config
        total = None
        if grad_weights is not None:
            total = torch.empty_like(logits)
            kernels.gate_route_grad_out(logits, scores, selected, denominator, indices,
                                        grad_weights.contiguous().float(), top_k, scale, scoring, total)
        if grad_logits is not None:
            total = grad_logits if total is None else total + grad_logits
        grad_hidden = grad_weight = None
        if total is not None:
            if ctx.needs_input_grad[0]:
                grad_hidden = (total @ weight.float()).to(hidden.dtype)
            if ctx.needs_input_grad[1]:
                grad_weight = (total.t() @ hidden.float()).to(weight.dtype)
        return (grad_hidden, grad_weight) + (None,) * 7


class MegaGate(torch.nn.Module):
    """Project hidden states and select experts."""

    def __init__(self, *, hidden_size: int, num_experts: int, top_k: int, scoring_func: str,
                 routed_scaling_factor: float, vision_enabled: bool = False,
                 initializer_range: float = 0.02, n_group: int | None = None, topk_group: int | None = None) -> None:
        """``n_group`` / ``topk_group`` are an extension the reference does not have: each token may only
        select experts from the ``topk_group`` best of ``n_group`` equal contiguous expert groups (group
        score = sum of the two largest biased scores of the group)."""
        super().__init__()
        if (n_group is None) != (topk_group is None):
            raise ValueError("n_group and topk_group go together")
        if n_group is not None:
            if not 1 <= n_group <= 32 or num_experts % n_group:
                raise ValueError("n_group must be in [1, 32] and divide num_experts")
            if not 1 <= topk_group <= n_group or top_k > topk_group * (num_experts // n_group):
                raise ValueError("topk_group must be in [1, n_group] and leave at least top_k experts")
        self.n_group = int(n_group or 0)
        self.topk_group = int(topk_group or 0)
        if hidden_size <= 0 or num_experts <= 0:
            raise ValueError("hidden_size and num_experts must be positive")
        if top_k <= 0 or top_k > num_experts:
            raise ValueError("top_k must be in [1, num_experts]")
        if scoring_func not in _SCORING:
            raise ValueError(f"unsupported scoring_func: {scoring_func!r}")
        if not math.isfinite(routed_scaling_factor):
            raise ValueError("routed_scaling_factor must be finite")
        if not math.isfinite(initializer_range) or initializer_range < 0.0:
            raise ValueError("initializer_range must be finite and nonnegative")
        self.hidden_size = int(hidden_size)
        self.num_experts = int(num_experts)
        self.top_k = int(top_k)
        self.scoring_func = scoring_func
        self.routed_scaling_factor = float(routed_scaling_factor)
        self.initializer_range = float(initializer_range)
        self.weight = torch.nn.Parameter(torch.empty(num_experts, hidden_size))
        self.bias = torch.nn.Parameter(torch.empty(num_experts, dtype=torch.float32))
        if vision_enabled:
            self.bias_vl = torch.nn.Parameter(torch.empty(num_experts, dtype=torch.float32))
        else:
            self.register_parameter("bias_vl", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        """Normal projection weight, zero correction biases."""
        torch.nn.init.normal_(self.weight, mean=0.0, std=self.initializer_range)
        torch.nn.init.zeros_(self.bias)
        if self.bias_vl is not None:
            torch.nn.init.zeros_(self.bias_vl)

    @classmethod
    def from_module(cls, module: torch.nn.Module, **configuration: Any) -> "MegaGate":
        """Bind an existing router's Parameters without copying them (module.py:141-179)."""
        weight = getattr(module, "weight", None)
        if not isinstance(weight, torch.nn.Parameter) or weight.ndim != 2:
            raise ValueError("source router requires a weight Parameter shaped [num_experts, hidden_size]")
        options = {}
        for name in ("top_k", "scoring_func", "routed_scaling_factor"):
            value = configuration.pop(name, getattr(module, name, None))
            if value is None:
                raise ValueError(f"Provide {name} or expose it on the source router")
            options[name] = value
        bias_vl = getattr(module, "bias_vl", None)
        vision_enabled = configuration.pop("vision_enabled", bias_vl is not None)
        if bias_vl is not None and not vision_enabled:
            raise ValueError("source bias_vl requires vision_enabled=True")
        result = cls(hidden_size=weight.shape[1], num_experts=weight.shape[0], vision_enabled=vision_enabled,
                     **options, **configuration).to(device=weight.device)
        result.weight = weight
        for name in ("bias", "bias_vl"):
            value = getattr(module, name, None)
            if value is not None:
                if (not isinstance(value, torch.nn.Parameter) or value.shape != (weight.shape[0],)
                        or value.dtype != torch.float32 or value.device != weight.device):
                    raise ValueError(f"source {name} must be an FP32 Parameter [num_experts] on the weight device")
                setattr(result, name, value)
        return result

    def _apply(self, fn: Callable, recurse: bool = True):
        return super()._apply(preserve_fp32_parameters(self, fn, ("bias", "bias_vl")), recurse=recurse)

    def forward(self, hidden_states: torch.Tensor, image_mask: torch.Tensor | None = None):
        """Returns (logits [T,E] fp32, routing_weights [T,K] fp32, expert_indices [T,K] int64)."""
        if image_mask is not None and self.bias_vl is None:
            raise ValueError("image_mask requires vision_enabled=True when constructing MegaGate")
        if image_mask is not None and image_mask.shape != hidden_states.shape[:2]:
            raise ValueError("image_mask must have shape [batch, sequence]")
        if not hidden_states.is_cuda:
            raise TypeError("MegaGate on the sm_100a backend requires CUDA tensors (there is no CPU path)")
        flattened = hidden_states.reshape(-1, self.hidden_size)
        tokens = flattened.shape[0]
        device = flattened.device
        if tokens == 0:
            return (torch.empty((0, self.num_experts), dtype=torch.float32, device=device),
                    torch.empty((0, self.top_k), dtype=torch.float32, device=device),
                    torch.empty((0, self.top_k), dtype=torch.int64, device=device))
        use_vision = image_mask is not None and self.bias_vl is not None
        if use_vision:
            if image_mask.dtype != torch.bool:
                raise TypeError("image_mask must be a BOOL tensor")
            if not image_mask.is_contiguous():
                raise ValueError("image_mask must be contiguous for native MegaGate")
            mask = image_mask.view(-1)
        else:
            mask = None
        needs_grad = torch.is_grad_enabled() and (flattened.requires_grad or self.weight.requires_grad)
        text_bias = self.bias.detach().float()
        vision_bias = self.bias_vl.detach().float() if use_vision else text_bias
        if kernels.gate_route_fusable(flattened, self.weight, self.n_group):
            # one launch: the projection's epilogue routes the token whose logits it holds
            if needs_grad:
                return _GateFunction.apply(flattened, self.weight, text_bias, vision_bias, mask, use_vision, self.top_k,
                                           self.routed_scaling_factor, self.scoring_func)
            return kernels.gate_project_route(flattened, self.weight, text_bias, vision_bias, mask, use_vision,
                                              self.top_k, self.routed_scaling_factor, self.scoring_func)[:3]
        if needs_grad:
            logits = _ProjectFunction.apply(flattened, self.weight)
            weights, indices = _RouteFunction.apply(logits, text_bias, vision_bias, mask, use_vision, self.top_k,
                                                    self.routed_scaling_factor, self.scoring_func, self.n_group,
                                                    self.topk_group)
        else:
            logits = kernels.gate_project(flattened, self.weight)
            weights, indices = route(logits, text_bias, vision_bias, mask, use_vision, self.top_k,
                                     self.routed_scaling_factor, self.scoring_func, self.n_group,
                                     self.topk_group)[:2]
        return logits, weights, indices
