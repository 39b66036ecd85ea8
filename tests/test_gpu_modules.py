"""GPU: MegaGate and MegaMhc modules (forward + autograd) against the oracle."""

import pytest
import torch

from oracle import gate as ogate
from oracle import mhc as omhc
from tests.helpers import cosine, rel_l2, sorted_sets

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("scoring", ["sqrtsoftplus", "softmax", "sigmoid"])
@pytest.mark.parametrize("vision", [False, True])
def test_mega_gate_forward_backward(cuda_device, scoring, vision):
    from hyper_multicore_b200 import MegaGate

    torch.manual_seed(11)
    hidden, experts, top_k, scale = 256, 64, 6, 2.5
    gate = MegaGate(hidden_size=hidden, num_experts=experts, top_k=top_k, scoring_func=scoring,
                    routed_scaling_factor=scale, vision_enabled=vision, initializer_range=0.2)
    with torch.no_grad():
        gate.bias.uniform_(-0.1, 0.1)
        if vision:
            gate.bias_vl.uniform_(-0.1, 0.1)
    x = torch.randn(2, 40, hidden).bfloat16()
    mask = (torch.rand(2, 40) < 0.3) if vision else None
    ref = ogate.gate_forward(x, gate.weight.detach(), gate.bias.detach(), gate.bias_vl.detach() if vision else None,
                             mask, top_k, scoring, scale)
    gate = gate.to(cuda_device)
    assert gate.bias.dtype == torch.float32
    xd = x.to(cuda_device).requires_grad_(True)
    logits, weights, indices = gate(xd, None if mask is None else mask.to(cuda_device))
    assert logits.dtype == torch.float32 and weights.dtype == torch.float32 and indices.dtype == torch.int64
    torch.testing.assert_close(logits.detach().cpu(), ref["logits"], rtol=1e-5, atol=1e-6)
    got_idx, got_w = sorted_sets(indices.cpu(), weights.detach().cpu())
    ref_idx, ref_w = sorted_sets(ref["indices"], ref["weights"])
    safe = ogate.topk_margin(ref["biased"], top_k) > 1e-5
    assert torch.equal(got_idx[safe], ref_idx[safe])
    torch.testing.assert_close(got_w[safe], ref_w[safe], rtol=1e-5, atol=1e-6)
    # backward through weights and logits, against torch autograd of the oracle expression
    g_w = torch.randn(80, top_k)
    g_l = torch.randn(80, experts) * 0.1
    torch.autograd.backward((weights, logits), (g_w.to(cuda_device), g_l.to(cuda_device)))
    xr = x.clone().float().requires_grad_(True)
    wr = gate.weight.detach().cpu().clone().requires_grad_(True)
    logits_r = torch.nn.functional.linear(xr.reshape(-1, hidden), wr)
    scores = ogate.scores_from_logits(logits_r, scoring)
    selected = scores.gather(1, indices.cpu())
    weights_r = selected / (selected.sum(-1, keepdim=True) + 1e-20) * scale
    torch.autograd.backward((weights_r, logits_r), (g_w, g_l))
    assert rel_l2(gate.weight.grad.cpu(), wr.grad) < 1e-4
    assert rel_l2(xd.grad.cpu().float(), xr.grad) < 1e-2  # BF16 rounding of the hidden-state gradient


def test_mega_gate_errors(cuda_device):
    from hyper_multicore_b200 import MegaGate

    with pytest.raises(ValueError, match="top_k must be in"):
        MegaGate(hidden_size=8, num_experts=4, top_k=5, scoring_func="softmax", routed_scaling_factor=1.0)
    with pytest.raises(ValueError, match="unsupported scoring_func"):
        MegaGate(hidden_size=8, num_experts=4, top_k=2, scoring_func="relu", routed_scaling_factor=1.0)
    gate = MegaGate(hidden_size=8, num_experts=4, top_k=2, scoring_func="softmax", routed_scaling_factor=1.0)
    gate = gate.to(cuda_device)
    x = torch.randn(1, 3, 8, device=cuda_device)
    with pytest.raises(ValueError, match="requires vision_enabled=True"):
        gate(x, torch.zeros(1, 3, dtype=torch.bool, device=cuda_device))
    empty = gate(torch.randn(1, 0, 8, device=cuda_device))
    assert empty[0].shape == (0, 4) and empty[2].shape == (0, 2)


@pytest.mark.parametrize("lead,hidden", [((5,), 128), ((2, 21), 256)])
def test_mega_mhc_module_autograd(cuda_device, lead, hidden):
    from hyper_multicore_b200 import MegaMhc

    torch.manual_seed(7)
    module = MegaMhc(hidden)
    with torch.no_grad():
        module.bias.normal_(0, 0.1)
        module.alpha.copy_(torch.tensor([1.0, 0.8, 1.2]))
        module.norm_weight.copy_((1 + 0.02 * torch.randn(hidden)).bfloat16())
    inputs = (torch.randn(*lead, hidden).bfloat16(), torch.randn(*lead, 4, hidden).bfloat16(),
              torch.sigmoid(torch.randn(*lead, 4)), 2 * torch.sigmoid(torch.randn(*lead, 4)),
              torch.softmax(torch.randn(*lead, 4, 4), dim=-1))
    params = (module.phi.detach().clone(), module.alpha.detach().clone(), module.bias.detach().clone(),
              module.norm_weight.detach().clone())
    grads = (torch.randn(*lead, 4, hidden).bfloat16() * 0.1, torch.randn(*lead, 4) * 0.1, torch.randn(*lead, 4) * 0.1,
             torch.randn(*lead, 4, 4) * 0.1, torch.randn(*lead, hidden).bfloat16() * 0.1)
    ref_out = omhc.mega_mhc(*inputs, *params)
    ref_grad = omhc.mega_mhc_grad(grads, (*inputs, *params))
    module = module.to(cuda_device).bfloat16()  # dtype conversion must keep phi / alpha / bias FP32
    assert module.phi.dtype == torch.float32 and module.norm_weight.dtype == torch.bfloat16
    dev_in = [t.to(cuda_device).requires_grad_(True) for t in inputs]
    out = module(*dev_in)
    for got, expected in zip(out, ref_out):
        assert got.shape == expected.shape
        assert cosine(got.detach().cpu().float(), expected.float()) > 0.9999
    torch.autograd.backward(out, [g.to(cuda_device) for g in grads])
    got_grads = [t.grad for t in dev_in] + [module.phi.grad, module.alpha.grad, module.bias.grad,
                                             module.norm_weight.grad]
    for index, (got, expected) in enumerate(zip(got_grads, ref_grad)):
        assert got.shape == expected.shape, index
        assert rel_l2(got.cpu().float(), expected.float()) <= 2e-2, index
    no_grad_out = module(*[t.detach() for t in dev_in])
    assert torch.equal(no_grad_out[0], out[0])
    with pytest.raises(ValueError, match="divisible by 128"):
        MegaMhc(100)
    with pytest.raises(ValueError, match="previous_pre_mix must have shape"):
        module(dev_in[0], dev_in[1], dev_in[2][..., :3], dev_in[3], dev_in[4])
