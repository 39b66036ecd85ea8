"""MXFP8 oracle (CPU, torch). PARITY UNPINNED: the reference has no numeric golden for MXFP8.

The reference quantises with a third-party CANN operator (`dynamic_mx_quant_with_dual_axis`,
scale_alg=1, RINT) whose source is not part of that project, and its own replay test checks only
finiteness and determinism (tests/torch/_replay_mega_moe_arch35.py:92-107). This oracle therefore
states the rule this build uses - the OCP Microscaling one - and evaluates the reference's expert
FFN dataflow (backends/mxfp8/graph.py:140-154) on de-quantised operands:

  shared exponent of a 32-block = floor(log2(max |x|)) - 8, stored biased by 127 as UE8M0
  element = round-to-nearest-even(x / 2^exponent) to E4M3, saturating at +-448; zero block -> scale 1

Forward:  Xq(row) . W1(col) -> U (bf16) -> Act = bf16(silu(g) * u) -> Actq(row) . W2(col) -> Y (bf16)
Backward: dYq(row) . W2(row)^T -> dA (bf16) -> dU (bf16) -> dUq(row) . W1(row)^T -> dX (bf16)
          dW2 = Actq(col)^T . dYq(col),  dW1 = Xq(col)^T . dUq(col)   ("col" = blocks down the rows)
"""

from __future__ import annotations

import torch
from torch.nn import functional as F


def quantize(x: torch.Tensor, axis: int):
    """Returns (e4m3 tensor, biased uint8 exponents with size/32 along ``axis``)."""
    x = x.float().movedim(axis, -1)
    lead = x.shape[:-1]
    blocks = x.reshape(*lead, x.shape[-1] // 32, 32)
    amax = blocks.abs().amax(dim=-1)
    _, exponent = torch.frexp(amax)  # amax = m * 2^exponent, m in [0.5, 1)
    biased = (exponent - 1 - 8 + 127).clamp(0, 254)
    biased = torch.where(amax > 0, biased, torch.full_like(biased, 127))
    scale = torch.pow(2.0, (biased - 127).float()).unsqueeze(-1)
    q = (blocks / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    q = q.reshape(*lead, -1).movedim(-1, axis)
    return q, biased.to(torch.uint8).movedim(-1, axis) if axis != x.dim() - 1 else biased.to(torch.uint8)


def dequantize(q: torch.Tensor, biased: torch.Tensor, axis: int) -> torch.Tensor:
    scale = torch.pow(2.0, biased.float() - 127).repeat_interleave(32, dim=axis)
    return q.float() * scale


def fake_quant(x: torch.Tensor, axis: int) -> torch.Tensor:
    """Quantise and de-quantise along ``axis`` (length padded with zeros to a multiple of 32)."""
    size = x.shape[axis]
    pad = (-size) % 32
    if pad:
        shape = list(x.shape)
        shape[axis] = pad
        x = torch.cat((x.float(), torch.zeros(shape)), dim=axis)
    q, s = quantize(x, axis)
    return dequantize(q, s, axis).narrow(axis, 0, size)


def reference_weight_fields(weight: torch.Tensor) -> dict:
    """The reference's physical MX fields of a BF16 weight [e, m, n] (docs/mega_moe.md:169-200):
    col_data / col_scale [e, m/64, n, 2] with 32-blocks along m, row_data / row_scale [e, m, n/64, 2]
    with 32-blocks along n."""
    experts, m, n = weight.shape
    col_q, col_s = quantize(weight, 1)  # [e, m/32, n]
    row_q, row_s = quantize(weight, 2)  # [e, m, n/32]
    return {
        "col_data": col_q, "col_scale": col_s.reshape(experts, m // 64, 2, n).permute(0, 1, 3, 2).contiguous(),
        "row_data": row_q, "row_scale": row_s.reshape(experts, m, n // 64, 2).contiguous(),
    }


def experts_forward_backward(hidden, topk_ids, topk_weights, w1, w2, grad_output):
    """MoE forward + backward on MXFP8 operands; w1 [E,H,2I], w2 [E,I,H] are the BF16 logical weights."""
    tokens, hid = hidden.shape
    num_experts, _, two_i = w1.shape
    inter = two_i // 2
    bf = torch.bfloat16
    w1_col, w1_row = fake_quant(w1, 1), fake_quant(w1, 2)
    w2_col, w2_row = fake_quant(w2, 1), fake_quant(w2, 2)
    output = torch.zeros(tokens, hid, dtype=bf)
    grad_hidden = torch.zeros(tokens, hid)
    grad_probs = torch.zeros_like(topk_weights, dtype=torch.float32)
    grad_w1 = torch.zeros(w1.shape, dtype=bf)
    grad_w2 = torch.zeros(w2.shape, dtype=bf)
    for expert in range(num_experts):
        rows, slots = torch.where(topk_ids == expert)
        if rows.numel() == 0:
            continue
        x = hidden[rows]
        probs = topk_weights[rows, slots].float()
        u = (fake_quant(x, 1) @ w1_col[expert]).to(bf)
        gate, up = u.float()[:, :inter], u.float()[:, inter:]
        act = (F.silu(gate) * up).to(bf)
        y = (fake_quant(act, 1) @ w2_col[expert]).to(bf)
        weighted = (y.float() * probs[:, None]).to(bf)
        output = output.index_add(0, rows, weighted)
        # backward
        g = grad_output[rows].float()
        grad_probs[rows, slots] = (g * y.float()).sum(-1)
        dy = (g * probs[:, None]).to(bf)
        d_act = (fake_quant(dy, 1) @ w2_row[expert].T).to(bf).float()
        sig = torch.sigmoid(gate)
        d_u = torch.cat(((d_act * up * sig * (1 + gate * (1 - sig))).to(bf), (d_act * gate * sig).to(bf)), dim=-1)
        d_x = (fake_quant(d_u, 1) @ w1_row[expert].T).to(bf)
        grad_hidden.index_add_(0, rows, d_x.float())
        grad_w2[expert] = (fake_quant(act, 0).T @ fake_quant(dy, 0)).to(bf)
        grad_w1[expert] = (fake_quant(x, 0).T @ fake_quant(d_u, 0)).to(bf)
    return {"output": output, "grad_hidden": grad_hidden.to(bf), "grad_probs": grad_probs, "grad_w1": grad_w1,
            "grad_w2": grad_w2}
