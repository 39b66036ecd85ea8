"""GPU parity: MegaMHC forward / backward against the oracle, with the reference's thresholds."""

import pytest
import torch

from oracle import mhc as omhc
from tests.helpers import cosine, load_cases, rel_l2

pytestmark = pytest.mark.gpu

NAMES_IN = ("previous_output", "residual", "previous_pre_mix", "previous_post_mix", "previous_residual_mix",
            "phi", "alpha", "bias", "norm_weight")
NAMES_OUT = ("new_residual", "next_pre_mix", "next_post_mix", "next_residual_mix", "block_input")


def make_inputs(tokens, hidden, seed):
    """Inputs as tests/torch/benchmark_mega_mhc.py:37-45 draws them."""
    g = torch.Generator().manual_seed(seed)
    rn = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    return (rn(tokens, hidden).bfloat16(), rn(tokens, 4, hidden).bfloat16(), torch.sigmoid(rn(tokens, 4)),
            2 * torch.sigmoid(rn(tokens, 4)), torch.softmax(rn(tokens, 4, 4), dim=-1),
            rn(24, 4 * hidden) * (4 * hidden) ** -0.5, torch.tensor([1.0, 0.8, 1.2]), rn(24) * 0.1,
            (1 + 0.02 * rn(hidden)).bfloat16())


def run_forward(inputs, dev, need_backward=True):
    from hyper_multicore_b200 import _lib, kernels as K

    dev_in = [t.to(dev) for t in inputs]
    residual = dev_in[1]
    tokens, _, hidden = residual.shape
    f32 = dict(dtype=torch.float32, device=dev)
    out = dict(new_residual=torch.empty_like(residual), next_pre_mix=torch.empty(tokens, 4, **f32),
               next_post_mix=torch.empty(tokens, 4, **f32), next_residual_mix=torch.empty(tokens, 16, **f32),
               block_input=torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev))
    cache = dict(hc_before_norm=torch.empty(tokens, 24, **f32), inv_rms=torch.empty(tokens, 1, **f32),
                 sum_out=torch.empty(40, 1, tokens, 4, **f32), norm_out=torch.empty(40, 1, tokens, 4, 4, **f32),
                 mixed_input=torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev),
                 rms_rstd=torch.empty(tokens, 1, **f32))
    status = _lib.new_status(dev)
    K.mega_mhc_out(*dev_in, *out.values(), *cache.values(), hc_eps=1e-6, norm_eps=1e-6, num_iters=20,
                   need_backward=need_backward, status=status)
    _lib.raise_on_status(status, "mhc forward")
    return dev_in, out, cache


def check_forward(out, ref):
    """Thresholds of tests/torch/benchmark_mega_mhc.py:80-92."""
    for name, expected in zip(NAMES_OUT, ref):
        got = out[name].cpu().float().reshape(expected.shape)
        cos_min, mae_max = (0.9999, 2e-3) if name == "block_input" else (0.99999, 2e-4)
        assert cosine(got, expected.float()) >= cos_min, name
        assert float((got - expected.float()).abs().mean()) <= mae_max, name


def run_backward(dev_in, out, cache, grads, dev):
    from hyper_multicore_b200 import _lib, kernels as K

    tokens, _, hidden = dev_in[1].shape
    f32 = dict(dtype=torch.float32, device=dev)
    tensors = dict(zip(NAMES_IN, dev_in))
    tensors.update(new_residual=out["new_residual"], hc_before_norm=cache["hc_before_norm"],
                   inv_rms=cache["inv_rms"], mixed_input=cache["mixed_input"], rms_rstd=cache["rms_rstd"])
    g = [t.to(dev) for t in grads]
    tensors.update(grad_new_residual=g[0], grad_next_pre_mix=g[1], grad_next_post_mix=g[2],
                   grad_next_residual_mix=g[3].reshape(tokens, 16).contiguous(), grad_block_input=g[4])
    result = dict(grad_previous_output=torch.empty_like(dev_in[0]), grad_residual=torch.empty_like(dev_in[1]),
                  grad_previous_pre_mix=torch.empty(tokens, 4, **f32),
                  grad_previous_post_mix=torch.empty(tokens, 4, **f32),
                  grad_previous_residual_mix=torch.empty(tokens, 4, 4, **f32),
                  grad_phi=torch.empty(24, 4 * hidden, **f32), grad_alpha=torch.empty(3, **f32),
                  grad_bias=torch.empty(24, **f32), grad_norm_weight=torch.empty(hidden, **f32))
    tensors.update(result)
    status = _lib.new_status(dev)
    K.mega_mhc_grad_out(tensors, hc_eps=1e-6, num_iters=20, status=status)
    _lib.raise_on_status(status, "mhc backward")
    return [result[k] for k in ("grad_previous_output", "grad_residual", "grad_previous_pre_mix",
                                "grad_previous_post_mix", "grad_previous_residual_mix", "grad_phi", "grad_alpha",
                                "grad_bias", "grad_norm_weight")]


def check_backward(got, ref):
    """Thresholds of tests/torch/benchmark_mega_mhc_grad.py:107-111."""
    for name, value, expected in zip(NAMES_IN, got, ref):
        value = value.cpu().float().reshape(expected.shape)
        assert rel_l2(value, expected.float()) <= 2e-2, (name, rel_l2(value, expected.float()))
        assert cosine(value, expected.float()) >= 0.999, name


def test_forward_and_backward_match_reference_fixture(cuda_device):
    for case in load_cases("mhc"):
        inputs = tuple(case[f"in_{n}"] for n in NAMES_IN)
        dev_in, out, cache = run_forward(inputs, cuda_device)
        check_forward(out, [case[f"out_{n}"] for n in NAMES_OUT])
        grads = [case[f"gout_{n}"] for n in NAMES_OUT]
        got = run_backward(dev_in, out, cache, grads, cuda_device)
        check_backward(got, [case[f"gin_{n}"] for n in NAMES_IN])


@pytest.mark.parametrize("tokens,hidden", [(1, 128), (33, 256), (257, 1024), (64, 7168)])
def test_forward_and_backward_match_oracle(cuda_device, tokens, hidden):
    inputs = make_inputs(tokens, hidden, seed=tokens + hidden)
    ref = omhc.mega_mhc(*inputs)
    dev_in, out, cache = run_forward(inputs, cuda_device)
    check_forward(out, ref)
    g = torch.Generator().manual_seed(99)
    grads = (torch.randn(tokens, 4, hidden, generator=g).bfloat16() * 0.1, torch.randn(tokens, 4, generator=g) * 0.1,
             torch.randn(tokens, 4, generator=g) * 0.1, torch.randn(tokens, 4, 4, generator=g) * 0.1,
             torch.randn(tokens, hidden, generator=g).bfloat16() * 0.1)
    got = run_backward(dev_in, out, cache, grads, cuda_device)
    check_backward(got, omhc.mega_mhc_grad(grads, inputs))


def test_sinkhorn_outputs_are_doubly_stochastic_at_full_size(cuda_device):
    """Size-independent property at a large token count: rows and columns of next_residual_mix sum to 1,
    new_residual is linear in previous_output through previous_post_mix."""
    tokens, hidden = 4096, 7168
    inputs = make_inputs(tokens, hidden, seed=1)
    _, out, _ = run_forward(inputs, cuda_device, need_backward=False)
    mix = out["next_residual_mix"].reshape(tokens, 4, 4)
    torch.testing.assert_close(mix.sum(dim=-2), torch.ones(tokens, 4, device=cuda_device), rtol=0, atol=1e-3)
    # the last Sinkhorn step normalises columns; rows are only as close to 1 as 20 iterations converge
    torch.testing.assert_close(mix.sum(dim=-1), torch.ones(tokens, 4, device=cuda_device), rtol=0, atol=2e-2)
    sample = slice(0, 16)
    ref = omhc.mega_mhc(*(t[sample] if t.shape[:1] == (tokens,) else t for t in inputs))
    # FP32 summation order may differ from the CPU einsum: allow rare one-ulp BF16 flips only
    mismatch = (out["new_residual"][sample].cpu() != ref[0]).float().mean()
    assert float(mismatch) < 1e-3
