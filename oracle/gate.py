"""MegaGate oracle (CPU, torch fp32).

Restates MegaGate._torch_forward (hyper_multicore/modules/mega_gate/module.py:189-227) and the
independent golden of the reference's system test (tests/torch/_test_mega_gate.py:291-333).
"""

from __future__ import annotations

import torch
from torch.nn import functional as F


def scores_from_logits(logits: torch.Tensor, scoring: str) -> torch.Tensor:
    """module.py:199-206."""
    if scoring == "sqrtsoftplus":
        return F.softplus(logits).sqrt()
    if scoring == "softmax":
        return logits.softmax(dim=-1)
    if scoring == "sigmoid":
        return logits.sigmoid()
    raise ValueError(f"unsupported scoring_func: {scoring!r}")


def group_limit(biased: torch.Tensor, n_group: int, topk_group: int) -> torch.Tensor:
    """Extension with no counterpart in the reference (it has no expert groups): keep only the experts
    of the `topk_group` best of `n_group` equal contiguous groups; a group's score is the sum of its two
    largest biased scores (the largest for single-expert groups); ties go to the lower group."""
    tokens, experts = biased.shape
    grouped = biased.view(tokens, n_group, experts // n_group)
    group_scores = grouped.topk(min(2, grouped.shape[-1]), dim=-1).values.sum(dim=-1)
    # stable descending order = ties to the lower group index
    order = torch.sort(group_scores, dim=-1, descending=True, stable=True).indices[:, :topk_group]
    keep = torch.zeros(tokens, n_group, dtype=torch.bool).scatter_(1, order, True)
    return biased.masked_fill(~keep.unsqueeze(-1).expand_as(grouped).reshape(tokens, experts), float("-inf"))


def route_from_logits(logits, bias, bias_vl, image_mask, top_k, scoring, scale, n_group=0, topk_group=0):
    """module.py:208-227: bias only selects; weights come from the unbiased scores."""
    scores = scores_from_logits(logits.float(), scoring)
    correction = bias.float()
    if image_mask is not None and bias_vl is not None:
        correction = torch.where(image_mask.reshape(-1, 1), bias_vl.float().unsqueeze(0), bias.float().unsqueeze(0))
    biased = scores + correction
    if n_group:
        biased = group_limit(biased, n_group, topk_group)
    indices = torch.topk(biased, top_k, dim=-1, sorted=False).indices
    selected = scores.gather(1, indices)
    denominator = selected.sum(dim=-1, keepdim=True) + 1.0e-20
    weights = selected / denominator if top_k > 1 else selected
    return {
        "weights": weights * scale,
        "indices": indices,
        "scores": scores,
        "biased": biased,
        "selected": selected,
        "denominator": denominator,
    }


def gate_forward(hidden, weight, bias, bias_vl, image_mask, top_k, scoring, scale, n_group=0, topk_group=0):
    """module.py:195-198 projection + route."""
    logits = F.linear(hidden.reshape(-1, hidden.shape[-1]).float(), weight.float())
    out = route_from_logits(logits, bias, bias_vl, image_mask, top_k, scoring, scale, n_group, topk_group)
    out["logits"] = logits
    return out


def route_grad(logits, indices, grad_weights, top_k, scoring, scale):
    """Autograd of the route expression for fixed indices (function.py:138-160 contract)."""
    logits = logits.detach().clone().float().requires_grad_(True)
    scores = scores_from_logits(logits, scoring)
    selected = scores.gather(1, indices)
    denominator = selected.sum(dim=-1, keepdim=True) + 1.0e-20
    weights = (selected / denominator if top_k > 1 else selected) * scale
    return torch.autograd.grad(weights, logits, grad_outputs=grad_weights)[0]


def topk_margin(biased: torch.Tensor, top_k: int) -> torch.Tensor:
    """Gap between the K-th and (K+1)-th biased score per row; rows under 1e-6 may legitimately
    resolve differently between CPU and GPU transcendental implementations."""
    if top_k >= biased.shape[1]:
        return torch.full((biased.shape[0],), float("inf"))
    top = torch.topk(biased, top_k + 1, dim=-1, sorted=True).values
    return top[:, top_k - 1] - top[:, top_k]
