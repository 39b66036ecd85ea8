"""GPU parity: MegaGate Route / RouteGrad / projection against the oracle and the reference fixtures."""

import pytest
import torch

from oracle import gate as ogate
from tests.helpers import load_cases, sorted_sets

pytestmark = pytest.mark.gpu


def _route(K, logits, bias, bias_vl, mask, top_k, scale, scoring):
    dev = logits.device
    tokens, experts = logits.shape
    out = dict(
        weights=torch.empty(tokens, top_k, device=dev), indices=torch.empty(tokens, top_k, dtype=torch.int64, device=dev),
        route_scores=torch.empty(tokens, experts, device=dev), selected=torch.empty(tokens, top_k, device=dev),
        denominator=torch.empty(tokens, 1, device=dev))
    use_vision = mask is not None
    K.gate_route_out(logits, bias, bias_vl if use_vision else bias, mask, use_vision, top_k, scale, scoring, **out)
    return out


def _check_against(K, dev, logits_cpu, bias, bias_vl, mask, top_k, scale, scoring):
    ref = ogate.route_from_logits(logits_cpu, bias, bias_vl, mask, top_k, scoring, scale)
    got = _route(K, logits_cpu.to(dev), bias.to(dev), None if bias_vl is None else bias_vl.to(dev),
                 None if mask is None else mask.to(dev), top_k, scale, scoring)
    torch.cuda.synchronize()
    torch.testing.assert_close(got["route_scores"].cpu(), ref["scores"], rtol=1e-5, atol=1e-6)
    margin = ogate.topk_margin(ref["biased"], top_k)
    safe = margin > 1e-6
    got_idx, got_w = sorted_sets(got["indices"].cpu(), got["weights"].cpu())
    ref_idx, ref_w = sorted_sets(ref["indices"], ref["weights"])
    flips = (got_idx != ref_idx).any(dim=-1)
    assert not (flips & safe).any(), f"{int((flips & safe).sum())} index flips on rows with a clear top-k margin"
    keep = ~flips
    torch.testing.assert_close(got_w[keep], ref_w[keep], rtol=1e-5, atol=1e-6)
    # every row holds top_k distinct experts
    assert (got_idx[:, 1:] != got_idx[:, :-1]).all()
    return got, ref, int(flips.sum())


@pytest.mark.parametrize("scoring", ["sqrtsoftplus", "softmax", "sigmoid"])
def test_route_matches_reference_fixture(cuda_device, scoring):
    from hyper_multicore_b200 import kernels as K

    for case in load_cases("gate"):
        if case["scoring"] != scoring:
            continue
        tokens, hidden, experts, top_k, vision = (int(v) for v in case["config"])
        scale = float(case["scale"][0])
        got, _, flips = _check_against(K, cuda_device, case["logits"], case["bias"],
                                       case["bias_vl"] if vision else None, case["mask"] if vision else None,
                                       top_k, scale, scoring)
        assert flips == 0
        got_idx, got_w = sorted_sets(got["indices"].cpu(), got["weights"].cpu())
        ref_idx, ref_w = sorted_sets(case["indices"], case["weights"])
        assert torch.equal(got_idx, ref_idx)
        torch.testing.assert_close(got_w, ref_w, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("scoring,experts,top_k", [("sqrtsoftplus", 33, 6), ("softmax", 64, 6), ("sigmoid", 256, 8),
                                                    ("sqrtsoftplus", 384, 1), ("softmax", 1000, 17)])
@pytest.mark.parametrize("tokens", [1, 17, 129])
def test_route_shapes(cuda_device, scoring, experts, top_k, tokens):
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(experts * 7 + tokens)
    logits = torch.randn(tokens, experts) * 3
    bias = torch.empty(experts).uniform_(-0.5, 0.5)
    bias_vl = torch.empty(experts).uniform_(-0.5, 0.5)
    mask = torch.rand(tokens) < 0.5
    _check_against(K, cuda_device, logits, bias, bias_vl, mask, top_k, 2.5, scoring)
    _check_against(K, cuda_device, logits, bias, None, None, top_k, 1.0, scoring)


def test_score_operation_order_edge_values(cuda_device):
    """Softplus threshold and tiny-exponential branches (tests/torch/_test_mega_gate.py:722-749)."""
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(2302)
    logits = torch.randn(64, 32) * 3
    logits[0, :8] = torch.tensor([-80.0, -20.0, -1e-7, 0.0, 20.0 - 2 ** -19, 20.0, 20.0 + 2 ** -19, 80.0])
    zero = torch.zeros(32)
    got = _route(K, logits.to(cuda_device), zero.to(cuda_device), None, None, 6, 2.5, "sqrtsoftplus")
    expected = torch.nn.functional.softplus(logits).sqrt()
    torch.testing.assert_close(got["route_scores"].cpu(), expected, rtol=2e-7, atol=1e-30)


def test_exact_ties_take_the_lower_expert(cuda_device):
    from hyper_multicore_b200 import kernels as K

    logits = torch.zeros(5, 40)
    got = _route(K, logits.to(cuda_device), torch.zeros(40, device=cuda_device), None, None, 4, 1.0, "sigmoid")
    assert got["indices"].cpu().tolist() == [[0, 1, 2, 3]] * 5
    torch.testing.assert_close(got["weights"].cpu(), torch.full((5, 4), 0.25))


@pytest.mark.parametrize("scoring", ["sqrtsoftplus", "softmax", "sigmoid"])
@pytest.mark.parametrize("top_k", [1, 6])
def test_route_grad_given_identical_forward_state(cuda_device, scoring, top_k):
    """RouteGrad against torch autograd on the same forward state (tests/torch/_test_mega_gate.py:752-777)."""
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(2302)
    logits = torch.randn(257, 33)
    ref = ogate.route_from_logits(logits, torch.zeros(33), None, None, top_k, scoring, 2.5)
    upstream = ((ref["indices"].float() + 1) / 33) / 2
    expected = ogate.route_grad(logits, ref["indices"], upstream, top_k, scoring, 2.5)
    grad = torch.empty(257, 33, device=cuda_device)
    K.gate_route_grad_out(logits.to(cuda_device), ref["scores"].to(cuda_device), ref["selected"].to(cuda_device),
                          ref["denominator"].to(cuda_device), ref["indices"].to(cuda_device),
                          upstream.to(cuda_device), top_k, 2.5, scoring, grad)
    torch.testing.assert_close(grad.cpu(), expected, rtol=1e-5, atol=1e-6)


def test_route_grad_matches_reference_fixture(cuda_device):
    from hyper_multicore_b200 import kernels as K

    for case in load_cases("gate"):
        tokens, hidden, experts, top_k, vision = (int(v) for v in case["config"])
        scale = float(case["scale"][0])
        ref = ogate.route_from_logits(case["logits"], case["bias"], case["bias_vl"] if vision else None,
                                      case["mask"] if vision else None, top_k, case["scoring"], scale)
        order = {tuple(sorted(r)) for r in ref["indices"].tolist()}
        assert order == {tuple(sorted(r)) for r in case["indices"].tolist()}
        # selected / denominator must follow the fixture's index order for the gradient to line up
        selected = ref["scores"].gather(1, case["indices"])
        denominator = selected.sum(dim=-1, keepdim=True) + 1e-20
        grad = torch.empty(tokens, experts, device=cuda_device)
        K.gate_route_grad_out(case["logits"].to(cuda_device), ref["scores"].to(cuda_device),
                              selected.to(cuda_device), denominator.to(cuda_device),
                              case["indices"].to(cuda_device), case["grad_weights"].to(cuda_device), top_k, scale,
                              case["scoring"], grad)
        torch.testing.assert_close(grad.cpu(), case["grad_logits"], rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("x_dtype,w_dtype", [(torch.bfloat16, torch.float32), (torch.float32, torch.float32),
                                              (torch.bfloat16, torch.bfloat16)])
def test_projection_is_fp32_accurate(cuda_device, x_dtype, w_dtype):
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(3)
    x = torch.randn(200, 1000).to(x_dtype)
    w = (torch.randn(70, 1000) * 0.02).to(w_dtype)
    ref = torch.nn.functional.linear(x.double(), w.double()).float()
    got = K.gate_project(x.to(cuda_device), w.to(cuda_device)).cpu()  # tcgen05 (promoted) where eligible
    torch.testing.assert_close(got, ref, rtol=1e-5, atol=1e-6)
    fma = K.gate_project(x.to(cuda_device), w.to(cuda_device), use_tensor_cores=False).cpu()
    torch.testing.assert_close(fma, ref, rtol=1e-5, atol=3e-6)
    loose = K.gate_project(x.to(cuda_device), w.to(cuda_device), use_tensor_cores="unpromoted").cpu()
    torch.testing.assert_close(loose, ref, rtol=1e-5, atol=1e-5 * float(ref.abs().max()))
    for case in load_cases("gate"):
        got = K.gate_project(case["hidden"].to(cuda_device), case["weight"].to(cuda_device)).cpu()
        torch.testing.assert_close(got, case["logits"], rtol=1e-5, atol=1e-6)


def test_projection_follows_in_place_weight_updates(cuda_device):
    """The BF16 parts of the weight are kept with the weight tensor between calls and split again after an
    in-place update (an optimiser step): the logits must follow the new values, and an unchanged weight must
    reproduce its logits bit for bit from the kept parts."""
    from hyper_multicore_b200 import kernels as K

    g = torch.Generator().manual_seed(11)
    x = torch.randn(256, 512, generator=g).bfloat16().to(cuda_device)
    w = (torch.randn(64, 512, generator=g) * 0.05).to(cuda_device)
    first = K.gate_project(x, w)
    again = K.gate_project(x, w)
    assert torch.equal(first, again)
    with torch.no_grad():
        w.add_(torch.randn(64, 512, generator=g).to(cuda_device) * 0.05)
    updated = K.gate_project(x, w)
    exact = x.double() @ w.double().T
    torch.testing.assert_close(updated.double(), exact, rtol=1e-5, atol=1e-5)
    assert not torch.equal(first, updated)
    assert torch.equal(updated, K.gate_project(x, w))


def test_projection_at_the_multimodal_gate_shape(cuda_device):
    """8192 tokens x hidden 4096 x 64 experts: the tensor-core path against a float64 reference."""
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(9)
    x = torch.randn(8192, 4096, device=cuda_device).bfloat16()
    x[6144:] = (x[6144:].float() * torch.empty(4096, device=cuda_device).uniform_(0.5, 2.0)).bfloat16()
    w = torch.randn(64, 4096, device=cuda_device) * 0.02
    ref = (x.double() @ w.double().T).float()
    # default: tcgen05 with the accumulation chain cut every 128 elements of K - inside the reference's
    # logits tolerance against a float64 result, and bit-identical from run to run
    got = K.gate_project(x, w)
    torch.testing.assert_close(got, ref, rtol=1e-5, atol=2e-6)
    assert torch.equal(got, K.gate_project(x, w))
    # FP32 FMAs accumulate 4096 terms in one chain; the three-GEMM tensor-core variant even more loosely
    torch.testing.assert_close(K.gate_project(x, w, use_tensor_cores=False), ref, rtol=1e-5, atol=3e-5)
    torch.testing.assert_close(K.gate_project(x, w, use_tensor_cores="unpromoted"), ref, rtol=1e-5,
                               atol=1e-5 * float(ref.abs().max()))
    # 256 experts (four expert tiles per token tile), hidden 7168
    x2 = torch.randn(1000, 7168, device=cuda_device).bfloat16()
    w2 = torch.randn(256, 7168, device=cuda_device) * 0.02
    torch.testing.assert_close(K.gate_project(x2, w2), (x2.double() @ w2.double().T).float(), rtol=1e-5, atol=4e-6)


@pytest.mark.parametrize("experts,n_group,topk_group,top_k,scoring", [(256, 8, 4, 8, "sigmoid"), (64, 4, 2, 6, "softmax"),
                                                                      (48, 16, 5, 3, "sqrtsoftplus"), (32, 32, 8, 8, "sigmoid")])
def test_group_limited_routing(cuda_device, experts, n_group, topk_group, top_k, scoring):
    """Group-limited selection (an extension: the reference has no expert groups): 256 experts in 8 groups,
    4 groups per token, top-8 is the expert-parallel MXFP8 configuration's router. Checked against the
    oracle's restatement; every selected expert must lie in one of the chosen groups."""
    from hyper_multicore_b200 import MegaGate, kernels as K

    g = torch.Generator().manual_seed(experts + n_group)
    tokens = 777
    logits = torch.randn(tokens, experts, generator=g) * 2
    bias = torch.randn(experts, generator=g) * 0.1
    ref = ogate.route_from_logits(logits, bias, None, None, top_k, scoring, 2.5, n_group, topk_group)
    dev = cuda_device
    out = dict(
        weights=torch.empty(tokens, top_k, device=dev), indices=torch.empty(tokens, top_k, dtype=torch.int64, device=dev),
        route_scores=torch.empty(tokens, experts, device=dev), selected=torch.empty(tokens, top_k, device=dev),
        denominator=torch.empty(tokens, 1, device=dev))
    K.gate_route_out(logits.to(dev), bias.to(dev), bias.to(dev), None, False, top_k, 2.5, scoring, **out,
                     n_group=n_group, topk_group=topk_group)
    got_idx, got_w = sorted_sets(out["indices"].cpu(), out["weights"].cpu())
    ref_idx, ref_w = sorted_sets(ref["indices"], ref["weights"])
    # rows whose group choice or top-k boundary is a near tie may legitimately differ between CPU and GPU exp()
    flips = (got_idx != ref_idx).any(dim=-1)
    assert flips.float().mean() < 0.01, f"{int(flips.sum())} of {tokens} rows differ"
    torch.testing.assert_close(got_w[~flips], ref_w[~flips], rtol=1e-5, atol=1e-6)
    groups_per_row = torch.tensor([len(set((row // (experts // n_group)).tolist())) for row in out["indices"].cpu()])
    assert (groups_per_row <= topk_group).all()
    # module level: the extension arguments reach the kernel, validation rejects impossible settings
    gate = MegaGate(hidden_size=64, num_experts=experts, top_k=top_k, scoring_func=scoring, routed_scaling_factor=1.0,
                    n_group=n_group, topk_group=topk_group).to(dev)
    _, _, idx = gate(torch.randn(2, 50, 64, device=dev).bfloat16())
    assert ((idx // (experts // n_group)).sort(dim=-1).values.diff(dim=-1) != 0).sum(dim=-1).max() < topk_group
    with pytest.raises(ValueError):
        MegaGate(hidden_size=64, num_experts=experts, top_k=top_k, scoring_func=scoring, routed_scaling_factor=1.0,
                 n_group=n_group)
    with pytest.raises(ValueError):
        MegaGate(hidden_size=64, num_experts=experts, top_k=top_k, scoring_func=scoring, routed_scaling_factor=1.0,
                 n_group=7, topk_group=1)


@pytest.mark.parametrize("scoring", ["sqrtsoftplus", "softmax", "sigmoid"])
@pytest.mark.parametrize("tokens,experts,top_k,vision,w_dtype", [
    (1000, 64, 6, True, torch.float32),     # two K-slices per token tile, ragged last tile
    (20000, 64, 8, False, torch.float32),   # one K-slice
    (300, 48, 48, True, torch.float32),     # every expert selected, experts not a multiple of 32
    (129, 20, 1, False, torch.float32),     # top-1: weights are not normalised
    (4096, 32, 4, True, torch.bfloat16),    # BF16 router weight (one part)
    (777, 33, 5, True, torch.float32),      # odd expert count: scalar stores
])
def test_fused_projection_and_route_equal_the_two_launches_bit_for_bit(cuda_device, scoring, tokens, experts, top_k,
                                                                       vision, w_dtype):
    """The projection's epilogue routes the token it holds: all six outputs equal projection-then-Route exactly."""
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(tokens + experts)
    dev = cuda_device
    x = torch.randn(tokens, 512, device=dev).bfloat16()
    w = (torch.randn(experts, 512, device=dev) * 0.2).to(w_dtype)
    bias = torch.empty(experts, device=dev).uniform_(-0.1, 0.1)
    bias_vl = torch.empty(experts, device=dev).uniform_(-0.1, 0.1)
    mask = (torch.rand(tokens, device=dev) < 0.3) if vision else None
    assert K.gate_route_fusable(x, w)
    fused = K.gate_project_route(x, w, bias, bias_vl if vision else bias, mask, vision, top_k, 2.5, scoring)
    logits = K.gate_project(x, w)
    two = _route(K, logits, bias, bias_vl, mask, top_k, 2.5, scoring)
    torch.cuda.synchronize()
    assert torch.equal(fused[0], logits)
    for got, name in zip(fused[1:], ("weights", "indices", "route_scores", "selected", "denominator")):
        assert torch.equal(got, two[name]), name
    # and the Route itself against the oracle on the same logits
    ref = ogate.route_from_logits(logits.cpu(), bias.cpu(), bias_vl.cpu() if vision else None,
                                  None if mask is None else mask.cpu(), top_k, scoring, 2.5)
    safe = ogate.topk_margin(ref["biased"], top_k) > 1e-6
    got_idx, got_w = sorted_sets(fused[2].cpu(), fused[1].cpu())
    ref_idx, ref_w = sorted_sets(ref["indices"], ref["weights"])
    assert torch.equal(got_idx[safe], ref_idx[safe])
    torch.testing.assert_close(got_w[safe], ref_w[safe], rtol=1e-5, atol=1e-6)


def test_fused_route_is_limited_to_one_expert_tile_without_groups(cuda_device):
    from hyper_multicore_b200 import kernels as K

    x = torch.randn(256, 64, device=cuda_device).bfloat16()
    assert K.gate_route_fusable(x, torch.randn(64, 64, device=cuda_device))
    assert not K.gate_route_fusable(x, torch.randn(65, 64, device=cuda_device))
    assert not K.gate_route_fusable(x, torch.randn(64, 64, device=cuda_device), n_group=4)
    assert not K.gate_route_fusable(x.float(), torch.randn(64, 64, device=cuda_device))
    assert not K.gate_route_fusable(x[:100], torch.randn(64, 64, device=cuda_device))


@pytest.mark.parametrize("scoring", ["sqrtsoftplus", "softmax", "sigmoid"])
def test_module_gradients_do_not_depend_on_the_fusion(cuda_device, scoring, monkeypatch):
    """MegaGate with the one-launch forward and with projection and Route apart: same outputs, same gradients."""
    from hyper_multicore_b200 import MegaGate

    torch.manual_seed(23)
    gate = MegaGate(hidden_size=256, num_experts=64, top_k=6, scoring_func=scoring, routed_scaling_factor=2.5,
                    vision_enabled=True, initializer_range=0.2).to(cuda_device)
    with torch.no_grad():
        gate.bias.uniform_(-0.1, 0.1)
        gate.bias_vl.uniform_(-0.1, 0.1)
    x = torch.randn(2, 192, 256, device=cuda_device).bfloat16()
    mask = torch.rand(2, 192, device=cuda_device) < 0.3
    g_w = torch.randn(384, 6, device=cuda_device)
    g_l = torch.randn(384, 64, device=cuda_device) * 0.1
    results = []
    for fused in ("1", "0"):
        monkeypatch.setenv("HMC_GATE_FUSED_ROUTE", fused)
        gate.weight.grad = None
        xd = x.clone().requires_grad_(True)
        logits, weights, indices = gate(xd, mask)
        torch.autograd.backward((weights, logits), (g_w, g_l))
        results.append((logits.detach(), weights.detach(), indices, xd.grad, gate.weight.grad.clone()))
    one, two = results
    for a, b in zip(one[:3], two[:3]):
        assert torch.equal(a, b)
    torch.testing.assert_close(one[3].float(), two[3].float(), rtol=1e-6, atol=1e-7)
    torch.testing.assert_close(one[4], two[4], rtol=1e-6, atol=1e-7)
    # only the weights' gradient, and only the logits'
    for pick in (0, 1):
        monkeypatch.setenv("HMC_GATE_FUSED_ROUTE", "1")
        xd = x.clone().requires_grad_(True)
        logits, weights, _ = gate(xd, mask)
        (weights if pick == 0 else logits).backward(g_w if pick == 0 else g_l)
        assert torch.isfinite(xd.grad.float()).all()
