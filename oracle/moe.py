"""MoE expert-FFN oracle (CPU, torch): the reference's TorchExperts CPU branch.

Restates tests/common/multicore/moe_reference.py:170-181 (per-expert loop, BF16 F.linear,
BF16-rounded activation, probabilities after FC2 with a BF16 round of the weighted value,
BF16 index_add in ascending expert order) on EIO-packed weights
(W1 = [E, H, 2I] = gate | up, W2 = [E, I, H]; converter tests/torch/_test_mega_moe.py:197-216),
and the sharper FP32 weight-gradient reference tests/common/multicore/fp32_expert_reference.py:8-37.
"""

from __future__ import annotations

import torch
from torch.nn import functional as F


def swiglu(gate, up, swiglu_limit=None, clamp_after_silu=False):
    """FP32 SwiGLU with the optional clamp of docs/mega_moe.md:258-272 (gate clipped from above before or
    after SiLU, up clipped to [-L, L]; torch.clamp passes gradients on the boundary, as the text requires)."""
    gate, up = gate.float(), up.float()
    if swiglu_limit is None:
        return F.silu(gate) * up
    if clamp_after_silu:
        return F.silu(gate).clamp(max=swiglu_limit) * up.clamp(-swiglu_limit, swiglu_limit)
    return F.silu(gate.clamp(max=swiglu_limit)) * up.clamp(-swiglu_limit, swiglu_limit)


def experts_forward(hidden, topk_ids, topk_weights, w1, w2, *, swiglu_limit=None, clamp_after_silu=False,
                    apply_probs_before_fc2=False):
    """Differentiable forward. hidden [T,H] bf16; w1 [E,H,2I]; w2 [E,I,H]; returns [T,H] bf16.

    With apply_probs_before_fc2 the two BF16 roundings of docs/mega_moe.md:274-281 are kept
    (a0 = bf16(act); fc2 input = bf16(fp32(a0) * p)) and the Top-K rows are summed unweighted
    (backends/bf16/autograd.py:133-135)."""
    num_experts, _, two_i = w1.shape
    inter = two_i // 2
    gate_w = w1[:, :, :inter].transpose(1, 2)  # [E, I, H] = [out, in]
    up_w = w1[:, :, inter:].transpose(1, 2)
    down_w = w2.transpose(1, 2)  # [E, H, I]
    output = hidden * 0 + topk_weights.sum() * 0
    for expert in range(num_experts):
        rows, slots = torch.where(topk_ids == expert)
        source = hidden.index_select(0, rows)
        gate = F.linear(source, gate_w[expert])
        up = F.linear(source, up_w[expert])
        activation = swiglu(gate, up, swiglu_limit, clamp_after_silu).to(hidden.dtype)
        if apply_probs_before_fc2:
            activation = (activation.float() * topk_weights[rows, slots, None].float()).to(hidden.dtype)
            weighted = F.linear(activation, down_w[expert])
        else:
            value = F.linear(activation, down_w[expert])
            weighted = (value.float() * topk_weights[rows, slots, None]).to(hidden.dtype)
        output = output.index_add(0, rows, weighted)
    return output


def experts_forward_backward(hidden, topk_ids, topk_weights, w1, w2, grad_output, **options):
    """Forward + backward through torch autograd on CPU; returns output, dX, dProbs, dW1, dW2."""
    hidden = hidden.detach().clone().requires_grad_(True)
    probs = topk_weights.detach().clone().float().requires_grad_(True)
    w1 = w1.detach().clone().requires_grad_(True)
    w2 = w2.detach().clone().requires_grad_(True)
    output = experts_forward(hidden, topk_ids, probs, w1, w2, **options)
    output.backward(grad_output)
    return {
        "output": output.detach(),
        "grad_hidden": hidden.grad,
        "grad_probs": probs.grad,
        "grad_w1": w1.grad,
        "grad_w2": w2.grad,
    }


def fp32_expert(tokens, gate_up, down):
    """fp32_expert_reference.py:8-37 for the EIO layout."""
    tokens, gate_up, down = (v.detach().cpu().float() for v in (tokens, gate_up, down))
    projection = (tokens @ gate_up).bfloat16().float()
    gate, up = projection.chunk(2, dim=-1)
    silu = F.silu(gate)
    activation = (silu * up).bfloat16().float()
    output = (activation @ down).bfloat16()
    grad_output = (2 * output.float() / output.numel()).bfloat16().float()
    grad_activation = (grad_output @ down.T).bfloat16().float()
    sigmoid = gate.sigmoid()
    grad_gate = (grad_activation * up * sigmoid * (1 + gate * (1 - sigmoid))).bfloat16().float()
    grad_up = (grad_activation * silu).bfloat16().float()
    grad_projection = torch.cat((grad_gate, grad_up), dim=-1)
    return output, tokens.T @ grad_projection, activation.T @ grad_output
