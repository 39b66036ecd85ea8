"""Generate tests/golden/*.npz by running the reference's own Python golden path on CPU.

Run in a container that has the reference checked out:

    REFERENCE_ROOT=/path/to/hyper-multicore python tests/golden/make_golden.py

The fixtures are small seeded cases; BF16 tensors are stored as their raw int16 bit patterns
(key suffix ``__bf16``). The GPU box never needs the reference: tests read only the .npz files.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REFERENCE_ROOT = os.environ.get("REFERENCE_ROOT")
if not REFERENCE_ROOT:
    raise SystemExit("set REFERENCE_ROOT to a checkout of the reference project")
sys.path.insert(0, REFERENCE_ROOT)

from hyper_multicore.modules.mega_gate.module import MegaGate  # noqa: E402  pylint: disable=wrong-import-position
from hyper_multicore.modules.mega_moe.route import _compute_route_metadata, _expert_capacity  # noqa: E402
from hyper_multicore.modules.mega_moe.spec import MegaMoeSpec  # noqa: E402
from tests.common.multicore.mega_mhc_golden import torch_mega_mhc  # noqa: E402
from tests.common.multicore.mega_mhc_grad_golden import torch_mega_mhc_grad  # noqa: E402
from tests.common.multicore.moe_reference import TorchExperts  # noqa: E402


def pack(**tensors) -> dict:
    out = {}
    for name, value in tensors.items():
        if isinstance(value, torch.Tensor):
            value = value.detach()
            if value.dtype == torch.bfloat16:
                out[name + "__bf16"] = value.contiguous().view(torch.int16).numpy()
            else:
                out[name] = value.contiguous().numpy()
        else:
            out[name] = np.asarray(value)
    return out


def gate_cases() -> None:
    cases = {}
    configs = [
        ("sqrtsoftplus", 48, 64, 16, 6, 2.5, False),
        ("sqrtsoftplus", 33, 64, 40, 1, 1.0, True),
        ("softmax", 48, 64, 16, 3, 1.0, True),
        ("softmax", 31, 96, 64, 6, 1.0, False),
        ("sigmoid", 48, 64, 16, 4, 1.5, True),
        ("sigmoid", 20, 128, 256, 8, 2.5, False),
    ]
    for index, (scoring, tokens, hidden, experts, top_k, scale, vision) in enumerate(configs):
        torch.manual_seed(100 + index)
        gate = MegaGate(hidden_size=hidden, num_experts=experts, top_k=top_k, scoring_func=scoring,
                        routed_scaling_factor=scale, vision_enabled=vision, initializer_range=0.2)
        with torch.no_grad():
            gate.bias.uniform_(-0.1, 0.1)
            if vision:
                gate.bias_vl.uniform_(-0.1, 0.1)
        hidden_states = torch.randn(1, tokens, hidden).bfloat16()
        mask = (torch.rand(1, tokens) < 0.4) if vision else None
        logits, weights, indices = gate._torch_forward(hidden_states, mask)  # pylint: disable=protected-access
        grad_weights = torch.randn_like(weights)
        grad_logits = torch.autograd.grad(weights, logits, grad_outputs=grad_weights)[0]
        prefix = f"case{index}_"
        for key, value in pack(
            hidden=hidden_states.reshape(tokens, hidden), weight=gate.weight, bias=gate.bias,
            bias_vl=gate.bias_vl if vision else torch.zeros(experts),
            mask=mask.reshape(-1) if vision else torch.zeros(tokens, dtype=torch.bool),
            logits=logits, weights=weights, indices=indices, grad_weights=grad_weights, grad_logits=grad_logits,
        ).items():
            cases[prefix + key] = value
        cases[prefix + "config"] = np.array([tokens, hidden, experts, top_k, int(vision)], dtype=np.int64)
        cases[prefix + "scale"] = np.array([scale], dtype=np.float64)
        cases[prefix + "scoring"] = np.array(scoring)
    cases["num_cases"] = np.array(len(configs))
    np.savez_compressed(HERE / "gate.npz", **cases)


def _spec(ep_size: int, rank: int, experts: int) -> MegaMoeSpec:
    return MegaMoeSpec(local_num_tokens=128, hidden_size=1, intermediate_size=128, num_experts=experts, top_k=2,
                       initial_capacity_factor=None, receive_capacity=1 << 20, ep_size=ep_size, ep_group=None,
                       rank_id=rank, num_cube_cores=1)


def route_cases() -> None:
    cases = {}
    rng = np.random.default_rng(7)
    tables = [np.array([[1, 2, 3, 4], [5, 6, 7, 8]], dtype=np.int32),  # the reference's known-answer table
              np.array([[0, 0, 0, 0], [3, 1, 2, 0]], dtype=np.int32)]   # ragged, with an empty source
    for ep, experts in ((1, 8), (2, 16), (4, 32), (8, 64), (8, 256)):
        table = rng.integers(0, 50, size=(ep, experts)).astype(np.int32)
        table[rng.random(table.shape) < 0.2] = 0
        tables.append(table)
    count = 0
    for table in tables:
        ep, experts = table.shape
        tensor = torch.from_numpy(table)
        for rank in range(ep):
            spec = _spec(ep, rank, experts)
            capacity, maximum = _expert_capacity(tensor, spec)
            meta = _compute_route_metadata(tensor[rank], tensor, None, spec, capacity)
            prefix = f"case{count}_"
            cases[prefix + "table"] = table
            cases[prefix + "rank"] = np.array(rank)
            cases[prefix + "capacity"] = np.array([capacity, maximum])
            for name in ("dispatch_src_off", "dispatch_target_off", "dispatch_size", "combine_src_off",
                         "combine_target_off", "combine_size", "group_list"):
                cases[prefix + name] = getattr(meta, name).numpy()
            count += 1
    cases["num_cases"] = np.array(count)
    np.savez_compressed(HERE / "route.npz", **cases)


def moe_cases() -> None:
    cases = {}
    configs = [(40, 64, 128, 4, 2), (33, 128, 64, 8, 3)]  # tokens, hidden, intermediate, experts, top_k
    for index, (tokens, hidden, inter, experts, top_k) in enumerate(configs):
        torch.manual_seed(300 + index)
        model = TorchExperts(hidden, inter, experts)
        with torch.no_grad():
            for parameter in model.parameters():
                parameter.normal_(0.0, 0.05)
        model = model.bfloat16()
        x = torch.randn(tokens, hidden).bfloat16().requires_grad_(True)
        router = torch.randn(tokens, experts)
        if index == 1:
            router[:, 5] = -1e9  # expert 5 receives nothing
        probs_all = router.softmax(dim=-1)
        topk_weights, topk_ids = torch.topk(probs_all, top_k, dim=-1)
        topk_weights = topk_weights.detach().clone().requires_grad_(True)
        output = model(x, topk_ids, topk_weights)
        grad_output = torch.randn(tokens, hidden).bfloat16()
        output.backward(grad_output)
        # EIO packing (tests/torch/_test_mega_moe.py:197-216): W1 = [E, H, 2I] = gate | up, W2 = [E, I, H]
        w1 = torch.cat((model.w1, model.w3), dim=1).transpose(1, 2).contiguous()
        w2 = model.w2.transpose(1, 2).contiguous()
        grad_w1 = torch.cat((model.w1.grad, model.w3.grad), dim=1).transpose(1, 2).contiguous()
        grad_w2 = model.w2.grad.transpose(1, 2).contiguous()
        prefix = f"case{index}_"
        for key, value in pack(hidden=x, topk_ids=topk_ids, topk_weights=topk_weights, w1=w1, w2=w2,
                               grad_output=grad_output, output=output, grad_hidden=x.grad,
                               grad_probs=topk_weights.grad, grad_w1=grad_w1, grad_w2=grad_w2).items():
            cases[prefix + key] = value
    cases["num_cases"] = np.array(len(configs))
    np.savez_compressed(HERE / "moe.npz", **cases)


def mhc_cases() -> None:
    cases = {}
    configs = [(6, 128), (9, 256)]
    for index, (tokens, hidden) in enumerate(configs):
        torch.manual_seed(500 + index)
        previous_output = torch.randn(tokens, hidden).bfloat16()
        residual = torch.randn(tokens, 4, hidden).bfloat16()
        pre = torch.sigmoid(torch.randn(tokens, 4))
        post = 2 * torch.sigmoid(torch.randn(tokens, 4))
        mix = torch.softmax(torch.randn(tokens, 4, 4), dim=-1)
        phi = torch.randn(24, 4 * hidden) * (4 * hidden) ** -0.5
        alpha = torch.tensor([1.0, 0.8, 1.2])
        bias = torch.randn(24) * 0.1
        norm_weight = (1 + 0.02 * torch.randn(hidden)).bfloat16()
        inputs = (previous_output, residual, pre, post, mix, phi, alpha, bias, norm_weight)
        outputs = torch_mega_mhc(*inputs)
        grads = (torch.randn(tokens, 4, hidden).bfloat16() * 0.1, torch.randn(tokens, 4) * 0.1,
                 torch.randn(tokens, 4) * 0.1, torch.randn(tokens, 4, 4) * 0.1,
                 torch.randn(tokens, hidden).bfloat16() * 0.1)
        gradients = torch_mega_mhc_grad(*grads, *inputs)
        prefix = f"case{index}_"
        names_in = ("previous_output", "residual", "previous_pre_mix", "previous_post_mix",
                    "previous_residual_mix", "phi", "alpha", "bias", "norm_weight")
        names_out = ("new_residual", "next_pre_mix", "next_post_mix", "next_residual_mix", "block_input")
        packed = {}
        packed.update({f"in_{n}": v for n, v in zip(names_in, inputs)})
        packed.update({f"out_{n}": v for n, v in zip(names_out, outputs)})
        packed.update({f"gout_{n}": v for n, v in zip(names_out, grads)})
        packed.update({f"gin_{n}": v for n, v in zip(names_in, gradients)})
        for key, value in pack(**packed).items():
            cases[prefix + key] = value
    cases["num_cases"] = np.array(len(configs))
    np.savez_compressed(HERE / "mhc.npz", **cases)


if __name__ == "__main__":
    torch.set_num_threads(1)
    gate_cases()
    route_cases()
    moe_cases()
    mhc_cases()
    for path in sorted(HERE.glob("*.npz")):
        print(path.name, path.stat().st_size, "bytes")
