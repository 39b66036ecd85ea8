"""GPU parity: MegaMoeExperts forward + backward (EP=1) against the reference's CPU golden path."""

import pytest
import torch

from oracle import compare, moe as omoe
from tests.helpers import load_cases

pytestmark = pytest.mark.gpu


def run_module(case, dev, layout="EIO", numerics=None):
    from hyper_multicore_b200 import MegaMoeExperts

    tokens, hidden = case["hidden"].shape
    experts, _, two_i = case["w1"].shape
    top_k = case["topk_ids"].shape[1]
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=two_i // 2, num_experts=experts, top_k=top_k,
                            numerics_options=numerics)
    x = case["hidden"].to(dev).requires_grad_(True)
    probs = case["topk_weights"].to(dev).float().requires_grad_(True)
    w1, w2 = case["w1"].to(dev), case["w2"].to(dev)
    if layout == "EOI":
        w1, w2 = w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous()
    w1.requires_grad_(True)
    w2.requires_grad_(True)
    out = module(x, case["topk_ids"].to(dev), probs, expert_weights=(w1, w2))
    out.backward(case["grad_output"].to(dev))
    module.check_status()
    grad_w1, grad_w2 = w1.grad, w2.grad
    if layout == "EOI":
        grad_w1, grad_w2 = grad_w1.transpose(1, 2), grad_w2.transpose(1, 2)
    return {"output": out.detach().cpu(), "grad_hidden": x.grad.cpu(), "grad_probs": probs.grad.cpu(),
            "grad_w1": grad_w1.cpu(), "grad_w2": grad_w2.cpu()}, module


def check(got, ref, **allowance):
    """The reference's tolerance with the one documented allowance (oracle/compare.py)."""
    for name in ("output", "grad_hidden", "grad_probs", "grad_w1", "grad_w2"):
        compare.check(name, got[name], ref[name], **allowance)


@pytest.mark.parametrize("layout", ["EIO", "EOI"])
def test_matches_reference_fixture(cuda_device, layout):
    for case in load_cases("moe"):
        got, module = run_module(case, cuda_device, layout)
        check(got, case)
        assert len(module.state_dict()) == 0  # the executor owns no parameters


def make_case(tokens, hidden, inter, experts, top_k, seed, dead_expert=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    router = torch.randn(experts, hidden, generator=g) * 0.02
    logits = x.float() @ router.T
    if dead_expert is not None:
        logits[:, dead_expert] = -1e9
    weights, ids = torch.topk(logits.softmax(-1), top_k, dim=-1)
    w1 = (torch.randn(experts, hidden, 2 * inter, generator=g) * 0.02).bfloat16()
    w2 = (torch.randn(experts, inter, hidden, generator=g) * 0.02).bfloat16()
    grad = torch.randn(tokens, hidden, generator=g).bfloat16()
    return {"hidden": x, "topk_ids": ids, "topk_weights": weights, "w1": w1, "w2": w2, "grad_output": grad}


@pytest.mark.parametrize("tokens,hidden,inter,experts,top_k", [(1, 64, 64, 4, 1), (17, 128, 64, 4, 2),
                                                               (129, 256, 128, 8, 3), (512, 1024, 2048, 16, 2)])
def test_matches_oracle(cuda_device, tokens, hidden, inter, experts, top_k):
    """The last shape is the single-rank MoE configuration: 512 tokens, H=1024, 16 experts, top-2, I=2048."""
    case = make_case(tokens, hidden, inter, experts, top_k, seed=tokens, dead_expert=1 if experts > 4 else None)
    ref = omoe.experts_forward_backward(case["hidden"], case["topk_ids"], case["topk_weights"], case["w1"],
                                        case["w2"], case["grad_output"])
    got, _ = run_module(case, cuda_device)
    check(got, ref)
    if experts > 4:
        assert (got["grad_w1"][1] == 0).all() and (got["grad_w2"][1] == 0).all(), "cold expert gradient must be exact zero"


def test_float32_partial_weight_gradients(cuda_device):
    from hyper_multicore_b200 import MegaMoeNumericsOptions

    case = make_case(200, 128, 128, 4, 2, seed=5)
    ref = omoe.experts_forward_backward(case["hidden"], case["topk_ids"], case["topk_weights"], case["w1"],
                                        case["w2"], case["grad_output"])
    got, module = run_module(case, cuda_device, numerics=MegaMoeNumericsOptions(partial_weight_grad_dtype="float32"))
    check(got, ref)


@pytest.mark.parametrize("limit,after_silu,before_fc2", [(1.0, False, False), (1.0, True, False),
                                                         (None, False, True), (1.25, False, True), (1.25, True, True)])
@pytest.mark.parametrize("layout", ["EIO", "EOI"])
def test_numerics_options(cuda_device, limit, after_silu, before_fc2, layout):
    """SwiGLU clamp before / after SiLU and probabilities applied before FC2 (docs/mega_moe.md:258-308 of
    the reference). Weights are five times larger than elsewhere so that outputs are O(1) and the limits
    sit inside the spread of the gate / up values (std about 1.6): a large share of the entries is clipped."""
    from hyper_multicore_b200 import MegaMoeNumericsOptions

    case = make_case(300, 256, 128, 8, 3, seed=11, dead_expert=2)
    case["w1"], case["w2"] = (case["w1"].float() * 5).bfloat16(), (case["w2"].float() * 5).bfloat16()
    options = dict(swiglu_limit=limit, clamp_after_silu=after_silu, apply_probs_before_fc2=before_fc2)
    ref = omoe.experts_forward_backward(case["hidden"], case["topk_ids"], case["topk_weights"], case["w1"],
                                        case["w2"], case["grad_output"], **options)
    plain = omoe.experts_forward_backward(case["hidden"], case["topk_ids"], case["topk_weights"], case["w1"],
                                          case["w2"], case["grad_output"])
    if limit is not None:
        assert (ref["output"].float() - plain["output"].float()).abs().max() > 0.2, "the clamp must matter here"
    got, module = run_module(case, cuda_device, layout, numerics=MegaMoeNumericsOptions(**options))
    # five times larger weights: dX terms of several units, whose BF16 ulp (0.03) is ten times the absolute
    # tolerance, so more sums that cancel miss it (seen: 21 to 41 of 76800 elements, worst 2.0 x the bound)
    check(got, ref, stray_fraction=1e-3)
    assert module.swiglu_limit == limit and module.clamp_after_silu == after_silu
    assert module.apply_probs_before_fc2 == before_fc2
    assert (got["grad_w1"][2] == 0).all() and (got["grad_w2"][2] == 0).all()


def test_repeated_calls_and_activation_checkpoint(cuda_device):
    """Two forwards before any backward (saved tensors must be owned copies), then checkpoint replay."""
    from hyper_multicore_b200 import MegaMoeExperts
    from torch.utils.checkpoint import checkpoint

    dev = cuda_device
    case_a, case_b = make_case(96, 128, 64, 4, 2, seed=1), make_case(64, 128, 64, 4, 2, seed=2)
    module = MegaMoeExperts(hidden_size=128, intermediate_size=64, num_experts=4, top_k=2)
    w1 = case_a["w1"].to(dev).requires_grad_(True)
    w2 = case_a["w2"].to(dev).requires_grad_(True)
    outs, leaves = [], []
    for case in (case_a, case_b):
        x = case["hidden"].to(dev).requires_grad_(True)
        p = case["topk_weights"].to(dev).requires_grad_(True)
        outs.append(module(x, case["topk_ids"].to(dev), p, expert_weights=(w1, w2)))
        leaves.append((x, p))
    (outs[0].float().sum() + outs[1].float().sum()).backward()
    ref_a = omoe.experts_forward_backward(case_a["hidden"], case_a["topk_ids"], case_a["topk_weights"], case_a["w1"],
                                          case_a["w2"], torch.ones(96, 128).bfloat16())
    compare.check("grad_hidden", leaves[0][0].grad, ref_a["grad_hidden"])
    x = case_a["hidden"].to(dev).requires_grad_(True)
    p = case_a["topk_weights"].to(dev).requires_grad_(True)
    ids = case_a["topk_ids"].to(dev)
    out = checkpoint(lambda a, b: module(a, ids, b, expert_weights=(w1, w2)), x, p, use_reentrant=False)
    out.float().sum().backward()
    compare.check("grad_hidden (checkpoint replay)", x.grad, ref_a["grad_hidden"])
    module.check_status()


def test_shared_execution_resources(cuda_device):
    """Two layers on one workspace, both forwards before either backward; a closed member cannot run and
    the workspace goes with the last member (reference: docs/mega_moe.md:329-366)."""
    from hyper_multicore_b200 import MegaMoeExperts

    dev = cuda_device
    cases = [make_case(120, 128, 64, 4, 2, seed=21), make_case(77, 128, 64, 4, 2, seed=22)]
    layers = [MegaMoeExperts(hidden_size=128, intermediate_size=64, num_experts=4, top_k=2) for _ in cases]
    MegaMoeExperts.share_execution_resources(layers)
    state = []
    for layer, case in zip(layers, cases):
        x = case["hidden"].to(dev).requires_grad_(True)
        p = case["topk_weights"].to(dev).requires_grad_(True)
        w1 = case["w1"].to(dev).requires_grad_(True)
        w2 = case["w2"].to(dev).requires_grad_(True)
        out = layer(x, case["topk_ids"].to(dev), p, expert_weights=(w1, w2))
        state.append((out, x, p, w1, w2))
    assert layers[0]._workspace is layers[1]._workspace and layers[0]._workspace is not None
    for (out, x, p, w1, w2), case in reversed(list(zip(state, cases))):
        out.backward(case["grad_output"].to(dev))
        ref = omoe.experts_forward_backward(case["hidden"], case["topk_ids"], case["topk_weights"], case["w1"],
                                            case["w2"], case["grad_output"])
        check({"output": out.detach().cpu(), "grad_hidden": x.grad.cpu(), "grad_probs": p.grad.cpu(),
               "grad_w1": w1.grad.cpu(), "grad_w2": w2.grad.cpu()}, ref)
    layers[0].check_status()
    layers[0].close()
    assert layers[1]._workspace is not None
    with pytest.raises(RuntimeError, match="closed multicore modules cannot execute"):
        layers[0](state[0][1], cases[0]["topk_ids"].to(dev), state[0][2], expert_weights=(state[0][3], state[0][4]))
    layers[1].close()
    assert layers[1]._group.closed


def test_validation_errors(cuda_device):
    from hyper_multicore_b200 import MegaMoeExperts

    dev = cuda_device
    module = MegaMoeExperts(hidden_size=64, intermediate_size=64, num_experts=4, top_k=2)
    case = make_case(8, 64, 64, 4, 2, seed=3)
    args = (case["hidden"].to(dev), case["topk_ids"].to(dev), case["topk_weights"].to(dev))
    good = (case["w1"].to(dev), case["w2"].to(dev))
    with pytest.raises(ValueError, match="expert_weights must have EIO shapes"):
        module(*args, expert_weights=(good[0][:, :32], good[1]))
    with pytest.raises(TypeError, match="must all use BF16"):
        module(*args, expert_weights=(good[0].float(), good[1].float()))
    with pytest.raises(ValueError, match="topk_ids must have shape"):
        module(args[0], args[1][:, :1], args[2], expert_weights=good)
    with pytest.raises(TypeError, match="BF16 CUDA hidden states"):
        module(args[0].float(), args[1], args[2], expert_weights=good)
    with pytest.raises(ValueError, match="outside that range"):
        module(args[0], args[1] + 3, args[2], expert_weights=good)
    module._status.zero_()  # the rejected call left a bad-index report behind
    out = module(*args, expert_weights=good)
    assert out.shape == args[0].shape and out.dtype == torch.bfloat16
    with pytest.raises(ValueError, match="gate_up_weight must have shape"):  # layout is bound by the first call
        module(*args, expert_weights=(good[0].transpose(1, 2).contiguous(), good[1].transpose(1, 2).contiguous()))
