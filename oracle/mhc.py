"""MegaMHC oracle (CPU, torch fp32 math on BF16 activations).

Restates tests/common/multicore/mega_mhc_golden.py: _sinkhorn (29-36), _predict_mappings (39-76),
torch_mega_mhc (79-142); the backward is torch autograd of that forward, as in
tests/common/multicore/mega_mhc_grad_golden.py:117-193 (norm_weight gradient returned FP32).
"""

from __future__ import annotations

import torch

STREAMS = 4


def sinkhorn(logits: torch.Tensor, num_iters: int, eps: float) -> torch.Tensor:
    """mega_mhc_golden.py:29-36."""
    current = torch.softmax(logits.float(), dim=-1) + eps
    current = current / (current.sum(dim=-2, keepdim=True) + eps)
    for _ in range(1, num_iters):
        current = current / (current.sum(dim=-1, keepdim=True) + eps)
        current = current / (current.sum(dim=-2, keepdim=True) + eps)
    return current


def predict_mappings(residual, phi, alpha, bias, *, hc_eps, norm_eps, num_iters):
    """mega_mhc_golden.py:39-76."""
    lead = residual.shape[:-2]
    res = residual.float()
    normalized = res * torch.rsqrt(res.square().mean(dim=(-2, -1), keepdim=True) + norm_eps)
    logits = torch.matmul(normalized.flatten(-2), phi.float().transpose(-1, -2))
    pre_l, post_l, mix_l = torch.split(logits, (STREAMS, STREAMS, STREAMS * STREAMS), dim=-1)
    pre_b, post_b, mix_b = torch.split(bias.float(), (STREAMS, STREAMS, STREAMS * STREAMS))
    pre = torch.sigmoid(pre_l * alpha[0].float() + pre_b) + hc_eps
    post = 2.0 * torch.sigmoid(post_l * alpha[1].float() + post_b)
    mix = sinkhorn((mix_l * alpha[2].float() + mix_b).reshape(*lead, STREAMS, STREAMS), num_iters, hc_eps)
    return pre, post, mix


def mega_mhc(previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix, phi, alpha,
             bias, norm_weight, *, hc_eps=1e-6, norm_eps=1e-6, num_iters=20):
    """mega_mhc_golden.py:122-142."""
    res = residual.float()
    new_residual = (
        torch.einsum("...ji,...jh->...ih", previous_residual_mix.float(), res)
        + previous_post_mix.float().unsqueeze(-1) * previous_output.float().unsqueeze(-2)
    ).to(residual.dtype)
    next_pre, next_post, next_mix = predict_mappings(
        new_residual, phi, alpha, bias, hc_eps=hc_eps, norm_eps=norm_eps, num_iters=num_iters)
    mixed = (new_residual.float() * previous_pre_mix.float().unsqueeze(-1)).sum(dim=-2)
    block = mixed * torch.rsqrt(mixed.square().mean(dim=-1, keepdim=True) + norm_eps)
    block = (block * norm_weight.float()).to(residual.dtype)
    return new_residual, next_pre, next_post, next_mix, block


def mega_mhc_grad(grads, inputs, *, hc_eps=1e-6, norm_eps=1e-6, num_iters=20):
    """mega_mhc_grad_golden.py:165-193. ``grads``: 5 output gradients; ``inputs``: the 9 forward inputs."""
    with torch.enable_grad():
        leaves = tuple(v.detach().clone().requires_grad_(True) for v in inputs)
        outputs = mega_mhc(*leaves, hc_eps=hc_eps, norm_eps=norm_eps, num_iters=num_iters)
        result = torch.autograd.grad(outputs, leaves, grad_outputs=tuple(grads))
    return (*result[:-1], result[-1].float())
