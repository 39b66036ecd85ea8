"""GPU: the operator-level wrappers (names and contracts of the reference's hyper_multicore/torch/ops.py)."""

import numpy as np
import pytest
import torch

from oracle import gate as ogate
from oracle import mhc as omhc
from oracle import route as oroute
from tests.helpers import cosine, rel_l2

pytestmark = pytest.mark.gpu


def test_versions():
    from hyper_multicore_b200 import ops

    assert ops.mega_moe_transport_version() == 2
    assert ops.worker_queue_layout_version() == 2


def test_gate_route_ops_and_checks(cuda_device):
    from hyper_multicore_b200 import ops

    dev = cuda_device
    torch.manual_seed(2302)
    logits = torch.randn(257, 33) * 3
    zero = torch.zeros(33)
    placeholder = torch.zeros(1, dtype=torch.bool, device=dev)
    out = ops._mega_gate_route(logits.to(dev), zero.to(dev), zero.to(dev), placeholder, None, None, top_k=6,
                               routed_scaling_factor=2.5, use_vision_bias=False)
    expected = torch.nn.functional.softplus(logits).sqrt()
    torch.testing.assert_close(out[2].cpu(), expected, rtol=2e-7, atol=1e-30)
    assert out[1].dtype == torch.int64 and out[4].shape == (257, 1)
    ref = ogate.route_from_logits(logits, zero, None, None, 6, "sqrtsoftplus", 2.5)
    upstream = ((ref["indices"].float() + 1) / 33) / 2
    grad = ops._mega_gate_route_grad(logits.to(dev), ref["scores"].to(dev), ref["selected"].to(dev),
                                     ref["denominator"].to(dev), ref["indices"].to(dev), upstream.to(dev), None, None,
                                     top_k=6, routed_scaling_factor=2.5)
    torch.testing.assert_close(grad.cpu(), ogate.route_grad(logits, ref["indices"], upstream, 6, "sqrtsoftplus", 2.5),
                               rtol=1e-5, atol=1e-6)
    with pytest.raises(RuntimeError, match="top_k must be in"):
        ops._mega_gate_route(logits.to(dev), zero.to(dev), zero.to(dev), placeholder, top_k=34,
                             routed_scaling_factor=1.0, use_vision_bias=False)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        ops._mega_gate_route(logits.to(dev).t(), zero.to(dev), zero.to(dev), placeholder, top_k=2,
                             routed_scaling_factor=1.0, use_vision_bias=False)
    with pytest.raises(RuntimeError, match="finite"):
        ops._mega_gate_route(logits.to(dev), zero.to(dev), zero.to(dev), placeholder, top_k=2,
                             routed_scaling_factor=float("inf"), use_vision_bias=False)


def test_permute_ops_round_trip(cuda_device):
    from hyper_multicore_b200 import ops

    dev = cuda_device
    torch.manual_seed(0)
    tokens, top_k, hidden, experts = 129, 3, 64, 7
    x = torch.randn(tokens, hidden).bfloat16()
    ids = torch.stack([torch.randperm(experts)[:top_k] for _ in range(tokens)])
    output = torch.empty(tokens * top_k, hidden, dtype=torch.bfloat16, device=dev)
    mapping = torch.empty(tokens * top_k, dtype=torch.int32, device=dev)
    ops.moe_token_permute_out(x.to(dev), ids.to(dev), output, mapping)
    ref_map, ref_src, _ = oroute.permutation(ids.numpy(), experts)
    assert np.array_equal(mapping.cpu().numpy(), ref_map)
    assert torch.equal(output.cpu(), x[torch.from_numpy(ref_src).long() // top_k])
    probs = torch.rand(tokens, top_k)
    out2 = torch.empty_like(output)
    out_p = torch.empty(tokens * top_k, device=dev)
    ops.moe_token_permute_from_mapping_out(x.to(dev), mapping, probs.to(dev), out2, out_p)
    assert torch.equal(out2, output)
    grad_out = torch.randn(tokens, hidden).bfloat16().to(dev)
    grad_perm = torch.empty_like(output)
    grad_probs = torch.empty(tokens, top_k, device=dev)
    ops.mega_moe_unpermute_grad_out(output, grad_out, mapping, probs.to(dev), grad_perm, grad_probs)
    back = ops.moe_token_permute_grad(grad_perm, mapping, tokens, top_k)
    expected = (grad_out.float().cpu().unsqueeze(1) * probs.unsqueeze(-1)).bfloat16().float().sum(1)
    torch.testing.assert_close(back.cpu().float(), expected, rtol=2e-2, atol=2e-2)
    table = torch.tensor([[1, 2, 3, 4], [5, 6, 7, 8]], dtype=torch.int32, device=dev)
    meta = ops.route_offsets(table, 1, 0, hidden_size=16)
    assert meta["dispatch_target_off"].tolist() == [1, 8, 3, 14] and meta["group_list"].tolist() == [10, 22]
    assert meta["dispatch_src_off_elements"].tolist() == [0, 80, 176, 288]
    with pytest.raises(RuntimeError, match="must be contiguous"):
        ops.moe_token_permute_out(x.to(dev).t().contiguous().t(), ids.to(dev), output, mapping)


def test_mhc_ops_bsnd(cuda_device):
    from hyper_multicore_b200 import ops
    from tests.test_gpu_mhc import NAMES_OUT, make_inputs

    dev = cuda_device
    tokens, hidden = 48, 256
    inputs = make_inputs(tokens, hidden, seed=4)
    ref = omhc.mega_mhc(*inputs)
    bsnd = [inputs[0].reshape(1, tokens, hidden), inputs[1].reshape(1, tokens, 4, hidden), inputs[2].reshape(1, tokens, 4),
            inputs[3].reshape(1, tokens, 4), inputs[4].reshape(1, tokens, 4, 4), *inputs[5:]]
    outs = ops.hyper_mega_mhc(*[t.to(dev) for t in bsnd], None, None, None, need_backward=True)
    assert len(outs) == 11 and outs[3].shape == (1, tokens, 4, 4) and outs[7].shape == (40, 1, tokens, 4)
    for name, got, expected in zip(NAMES_OUT, outs[:5], ref):
        assert cosine(got.cpu().float().reshape(expected.shape), expected.float()) > 0.9999, name
    grads = (torch.randn(tokens, 4, hidden).bfloat16() * 0.1, torch.randn(tokens, 4) * 0.1, torch.randn(tokens, 4) * 0.1,
             torch.randn(tokens, 4, 4) * 0.1, torch.randn(tokens, hidden).bfloat16() * 0.1)
    ref_grad = omhc.mega_mhc_grad(grads, inputs)
    d = [t.to(dev) for t in bsnd]
    g = [t.to(dev) for t in grads]
    new_residual, hc_before_norm, inv_rms, sum_out, norm_out, mixed_input, rms_rstd = outs[0], *outs[5:]
    result = ops.hyper_mega_mhc_grad(g[4], g[2], g[3], new_residual, d[5], d[6], d[7], d[2], hc_before_norm, inv_rms,
                                     sum_out, norm_out, g[1], mixed_input, rms_rstd, d[8], g[0], d[1], d[0], d[3], d[4],
                                     None, None, None)
    order = (1, 5, 6, 7, 0, 2, 3, 4, 8)  # position of each returned gradient among the forward inputs
    for got, index in zip(result, order):
        assert rel_l2(got.cpu().float().reshape(ref_grad[index].shape), ref_grad[index].float()) <= 2e-2, index
    with pytest.raises(ValueError, match="BSND"):
        ops.hyper_mega_mhc(*[t.to(dev) for t in inputs], None, None, None, need_backward=False)
