"""GPU parity at the sizes of the benchmark configurations, each against the CPU oracle.

The oracle's cost is what bounds these cases: the expert FFN golden is nearly flat in the token count (a few
seconds for the whole 4096-token problem), the router and the route preparation are cheap at any size, and
the residual mix is token-wise independent, so a slice of a full-size run is checked.
"""

import numpy as np
import pytest
import torch

import bench
import bench_side
from oracle import compare, gate as ogate, mhc as omhc, moe as omoe, mxfp8 as omx, route as oroute
from tests.helpers import rel_l2, sorted_sets
from tests.test_gpu_mhc import NAMES_IN, check_backward, check_forward, run_backward, run_forward

pytestmark = pytest.mark.gpu


def test_moe_layer_at_the_benchmark_shape(cuda_device):
    """4096 tokens, hidden 4096, 32 experts, softmax top-4, intermediate 1536 (the expert-parallel BF16
    configuration's per-rank problem, the shape bench.py times): forward + backward against the golden."""
    from hyper_multicore_b200 import MegaMoeExperts

    dev = cuda_device
    shape = bench.SHAPES["c2"]
    x, ids, probs, grad, w1, w2 = bench.make_inputs(shape, 0, 1)
    ref = omoe.experts_forward_backward(x, ids, probs, w1, w2, grad)
    module = MegaMoeExperts(hidden_size=shape.hidden, intermediate_size=shape.inter, num_experts=shape.num_experts(1),
                            top_k=shape.top_k)
    xd = x.to(dev).requires_grad_(True)
    pd = probs.to(dev).requires_grad_(True)
    w1d, w2d = w1.to(dev).requires_grad_(True), w2.to(dev).requires_grad_(True)
    out = module(xd, ids.to(dev), pd, expert_weights=(w1d, w2d))
    out.backward(grad.to(dev))
    module.check_status()
    for name, got in (("output", out), ("grad_hidden", xd.grad), ("grad_probs", pd.grad), ("grad_w1", w1d.grad),
                      ("grad_w2", w2d.grad)):
        compare.check(name, got, ref[name])


def test_multimodal_gate_and_route_preparation_end_to_end(cuda_device):
    """6144 text + 2048 vision tokens, hidden 4096, two routers' biases over 64 experts, top-6 softmax:
    MegaGate, then the per-expert counts and the expert-major permutation. Expert sets are exact wherever
    the oracle's top-k margin exceeds 1e-6 on the same FP32 logits; counts and mapping are bit-exact
    against the integer oracle on the indices the GPU produced."""
    from hyper_multicore_b200 import MegaGate, kernels as K

    dev = cuda_device
    cfg = bench_side.GATE
    x, weight, bias, bias_vl, mask = bench_side.gate_inputs(0)
    tokens = x.shape[1]
    assert tokens == 8192 and cfg["experts"] == 64 and cfg["top_k"] == 6
    gate = MegaGate(hidden_size=cfg["hidden"], num_experts=cfg["experts"], top_k=cfg["top_k"], scoring_func=cfg["scoring"],
                    routed_scaling_factor=cfg["scale"], vision_enabled=True).to(dev)
    with torch.no_grad():
        gate.weight.copy_(weight)
        gate.bias.copy_(bias)
        gate.bias_vl.copy_(bias_vl)
        logits, weights, indices = gate(x.to(dev), mask.to(dev))
    # the projection keeps FP32 accuracy (the reference's logits tolerance)
    exact = x[0].double() @ weight.double().T
    torch.testing.assert_close(logits.cpu().double(), exact, rtol=1e-5, atol=1e-5)
    ref = ogate.route_from_logits(logits.cpu(), bias, bias_vl, mask.reshape(-1), cfg["top_k"], cfg["scoring"], cfg["scale"])
    safe = ogate.topk_margin(ref["biased"], cfg["top_k"]) > 1e-6
    got_idx, got_w = sorted_sets(indices.cpu(), weights.cpu())
    ref_idx, ref_w = sorted_sets(ref["indices"], ref["weights"])
    flips = (got_idx != ref_idx).any(dim=-1)
    assert not (flips & safe).any(), f"{int((flips & safe).sum())} index flips on rows with a clear top-k margin"
    torch.testing.assert_close(got_w[~flips], ref_w[~flips], rtol=1e-5, atol=1e-6)
    mapping, sources, row_experts, counts, _ = K.moe_sort_routes(indices, cfg["experts"])
    ids_np = indices.cpu().numpy()
    assert np.array_equal(counts.cpu().numpy(), oroute.counts(ids_np, cfg["experts"]))
    ref_map, ref_src, ref_exp = oroute.permutation(ids_np, cfg["experts"])
    assert np.array_equal(mapping.cpu().numpy(), ref_map)
    assert np.array_equal(sources.cpu().numpy(), ref_src)
    assert np.array_equal(row_experts.cpu().numpy(), ref_exp)


def test_residual_mix_slice_of_a_full_size_run(cuda_device):
    """16384 tokens x 4 streams x hidden 7168 on the GPU; tokens are independent, so a 1024-token slice is
    checked against the oracle with the reference's thresholds (forward outputs, and the gradients of the
    five per-token inputs; the parameter gradients sum over all tokens and are covered at smaller sizes)."""
    dev = cuda_device
    tokens, hidden, sample = bench_side.MHC["tokens"], bench_side.MHC["hidden"], 1024
    inputs, grads = bench_side.mhc_inputs(0, tokens, hidden, device=dev)
    dev_in, out, cache = run_forward(inputs, dev)
    got = run_backward(dev_in, out, cache, grads, dev)
    first = slice(5000, 5000 + sample)  # an interior slice: offsets into every buffer are exercised
    cpu_in = tuple(t[first].cpu() if t.shape[:1] == (tokens,) else t.cpu() for t in inputs)
    cpu_grads = tuple(g[first].cpu() for g in grads)
    ref = omhc.mega_mhc(*cpu_in)
    check_forward({name: value[first] for name, value in out.items()}, ref)
    ref_grads = omhc.mega_mhc_grad(cpu_grads, cpu_in)
    per_token = len(NAMES_IN) - 4  # previous_output, residual and the three previous mixes
    check_backward([g[first] for g in got[:per_token]], ref_grads[:per_token])


def test_mxfp8_layer_at_the_expert_parallel_shape(cuda_device):
    """Hidden 7168, intermediate 2048 (the EP=8 MXFP8 configuration's expert shape) on 4 experts, 1024
    tokens, top-2, against the OCP-MX oracle (parity unpinned: the reference holds no MXFP8 numerics)."""
    from hyper_multicore_b200 import MegaMoeExperts
    from hyper_multicore_b200.mxfp8 import attach_mx_fields

    dev = cuda_device
    tokens, hidden, inter, experts, top_k = 1024, 7168, 2048, 4, 2
    g = torch.Generator().manual_seed(7168)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    probs, ids = torch.topk(torch.randn(tokens, experts, generator=g).sigmoid(), top_k, dim=-1)
    probs = (probs / probs.sum(-1, keepdim=True)).contiguous()
    w1 = (torch.randn(experts, hidden, 2 * inter, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(experts, inter, hidden, generator=g) * 0.02).bfloat16()
    grad = torch.randn(tokens, hidden, generator=g).bfloat16()
    ref = omx.experts_forward_backward(x, ids, probs, w1, w2, grad)
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            precision="mxfp8")
    w1d = attach_mx_fields(w1.to(dev).requires_grad_(True))
    w2d = attach_mx_fields(w2.to(dev).requires_grad_(True))
    xd, pd = x.to(dev).requires_grad_(True), probs.to(dev).requires_grad_(True)
    out = module(xd, ids.to(dev), pd, expert_weights=(w1d, w2d))
    out.backward(grad.to(dev))
    module.check_status()
    for name, got, limit in (("output", out, 1e-2), ("grad_hidden", xd.grad, 3e-2), ("grad_probs", pd.grad, 3e-2),
                             ("grad_w1", w1d.grad, 3e-2), ("grad_w2", w2d.grad, 3e-2)):
        error = rel_l2(got.detach().cpu().float(), ref[name].float())
        assert error <= limit, (name, error)


def test_mxfp8_replay_checks_of_the_reference(cuda_device):
    """What the reference's own MXFP8 replay pins (tests/torch/_replay_mega_moe_arch35.py:92-107): two
    forward + backward passes agree with rtol = 0, everything is finite, and experts without rows get
    exact-zero weight gradients."""
    from hyper_multicore_b200 import MegaMoeExperts
    from hyper_multicore_b200.mxfp8 import attach_mx_fields

    dev = cuda_device
    tokens, hidden, inter, experts, top_k = 777, 512, 256, 8, 2
    g = torch.Generator().manual_seed(35)
    x = torch.randn(tokens, hidden, generator=g).bfloat16().to(dev)
    logits = torch.randn(tokens, experts, generator=g)
    logits[:, [2, 5]] = -1e9  # two experts stay empty
    probs, ids = torch.topk(logits.softmax(-1), top_k, dim=-1)
    w1 = attach_mx_fields((torch.randn(experts, hidden, 2 * inter, generator=g) * 0.05).bfloat16().to(dev).requires_grad_(True))
    w2 = attach_mx_fields((torch.randn(experts, inter, hidden, generator=g) * 0.05).bfloat16().to(dev).requires_grad_(True))
    grad = torch.randn(tokens, hidden, generator=g).bfloat16().to(dev)
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            precision="mxfp8")
    passes = []
    for _ in range(2):
        xd, pd = x.clone().requires_grad_(True), probs.to(dev).requires_grad_(True)
        w1.grad = w2.grad = None
        out = module(xd, ids.to(dev), pd, expert_weights=(w1, w2))
        out.backward(grad)
        passes.append((out.detach().clone(), xd.grad.clone(), pd.grad.clone(), w1.grad.clone(), w2.grad.clone()))
    module.check_status()
    for first, second in zip(*passes):
        assert torch.isfinite(first.float()).all()
        assert torch.equal(first, second), "two passes over the same inputs must agree bit for bit"
    for empty in (2, 5):
        assert (passes[0][3][empty] == 0).all() and (passes[0][4][empty] == 0).all()
    assert (passes[0][3][0] != 0).any()
