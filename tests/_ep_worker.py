"""Worker of the multi-GPU expert-parallel test: one process per GPU, launched by torch.distributed.run.

Every rank regenerates all ranks' seeded inputs, runs MegaMoeExperts over its own tokens with its own
expert shard, and checks outputs and gradients against the CPU oracle evaluated on the concatenated
global batch (the reference's multi-rank golden replicates rows the same way,
tests/common/multicore/moe_reference.py:37-75).
"""

import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import compare, moe as omoe  # noqa: E402


def make_rank_inputs(rank, tokens, hidden, experts, top_k, seed):
    g = torch.Generator().manual_seed(seed * 100 + rank)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    logits = torch.randn(tokens, experts, generator=g)
    weights, ids = torch.topk(logits.softmax(-1), top_k, dim=-1)
    grad = torch.randn(tokens, hidden, generator=g).bfloat16()
    return x, ids, weights.contiguous(), grad


def check(name, got, expected):
    """The reference's tolerance with the one documented allowance (oracle/compare.py)."""
    compare.check(f"[rank {os.environ.get('RANK')}] {name}", got, expected)


def scenario_mx(module, rank, world, device, token_counts, hidden, inter, experts, top_k, seed):
    """MXFP8 backend across ranks against the MX oracle on the concatenated batch. Rows of one
    expert arrive source-rank-major, which is the row order of the concatenated batch, so the
    token-axis quantisation blocks of the weight gradients line up with the oracle's."""
    from hyper_multicore_b200.mxfp8 import attach_mx_fields
    from oracle import mxfp8 as omx
    from tests.helpers import rel_l2

    local = experts // world
    gw = torch.Generator().manual_seed(seed)
    w1_all = (torch.randn(experts, hidden, 2 * inter, generator=gw) * 0.05).bfloat16()
    w2_all = (torch.randn(experts, inter, hidden, generator=gw) * 0.05).bfloat16()
    per_rank = [make_rank_inputs(r, token_counts[r], hidden, experts, top_k, seed) for r in range(world)]
    x, ids, probs, grad = per_rank[rank]
    dist.barrier()  # the oracle below takes a different time on every rank; start the GPU call together
    w1 = attach_mx_fields(w1_all[rank * local:(rank + 1) * local].contiguous().to(device).requires_grad_(True))
    w2 = attach_mx_fields(w2_all[rank * local:(rank + 1) * local].contiguous().to(device).requires_grad_(True))
    xd = x.to(device).requires_grad_(True)
    pd = probs.to(device).requires_grad_(True)
    out = module(xd, ids.to(device), pd, expert_weights=(w1, w2))
    out.backward(grad.to(device))
    module.check_status()
    ref = omx.experts_forward_backward(
        torch.cat([p[0] for p in per_rank]), torch.cat([p[1] for p in per_rank]),
        torch.cat([p[2] for p in per_rank]), w1_all, w2_all, torch.cat([p[3] for p in per_rank]))
    start = sum(token_counts[:rank])
    rows = slice(start, start + token_counts[rank])
    experts_slice = slice(rank * local, (rank + 1) * local)
    for name, got, expected, limit in (
            ("output", out, ref["output"][rows], 1e-2), ("grad_hidden", xd.grad, ref["grad_hidden"][rows], 3e-2),
            ("grad_probs", pd.grad, ref["grad_probs"][rows], 3e-2),
            ("grad_w1", w1.grad, ref["grad_w1"][experts_slice], 3e-2),
            ("grad_w2", w2.grad, ref["grad_w2"][experts_slice], 3e-2)):
        if expected.numel():
            error = rel_l2(got.detach().cpu().float(), expected.float())
            assert error <= limit, (name, error)


def scenario(module, rank, world, device, token_counts, hidden, inter, experts, top_k, seed, layout, **options):
    local = experts // world
    gw = torch.Generator().manual_seed(seed)
    w1_all = (torch.randn(experts, hidden, 2 * inter, generator=gw) * 0.05).bfloat16()
    w2_all = (torch.randn(experts, inter, hidden, generator=gw) * 0.05).bfloat16()
    per_rank = [make_rank_inputs(r, token_counts[r], hidden, experts, top_k, seed) for r in range(world)]
    x, ids, probs, grad = per_rank[rank]
    dist.barrier()  # the oracle below takes a different time on every rank; start the GPU call together
    w1 = w1_all[rank * local:(rank + 1) * local]
    w2 = w2_all[rank * local:(rank + 1) * local]
    if layout == "EOI":
        w1, w2 = w1.transpose(1, 2), w2.transpose(1, 2)
    w1 = w1.contiguous().to(device).requires_grad_(True)
    w2 = w2.contiguous().to(device).requires_grad_(True)
    xd = x.to(device).requires_grad_(True)
    pd = probs.to(device).requires_grad_(True)
    out = module(xd, ids.to(device), pd, expert_weights=(w1, w2))
    out.backward(grad.to(device))
    module.check_status()
    ref = omoe.experts_forward_backward(
        torch.cat([p[0] for p in per_rank]), torch.cat([p[1] for p in per_rank]),
        torch.cat([p[2] for p in per_rank]), w1_all, w2_all, torch.cat([p[3] for p in per_rank]), **options)
    start = sum(token_counts[:rank])
    rows = slice(start, start + token_counts[rank])
    check("output", out, ref["output"][rows])
    check("grad_hidden", xd.grad, ref["grad_hidden"][rows])
    check("grad_probs", pd.grad, ref["grad_probs"][rows])
    gw1, gw2 = w1.grad, w2.grad
    if layout == "EOI":
        gw1, gw2 = gw1.transpose(1, 2), gw2.transpose(1, 2)
    check("grad_w1", gw1, ref["grad_w1"][rank * local:(rank + 1) * local])
    check("grad_w2", gw2, ref["grad_w2"][rank * local:(rank + 1) * local])


def main():
    from hyper_multicore_b200 import MegaMoeExperts

    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    # the CPU oracle runs in every rank: share the host cores instead of oversubscribing them
    torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))
    hidden, inter, experts, top_k = 256, 128, 8 * world // 2 if world > 2 else 8, 2
    for layout in ("EIO", "EOI"):
        module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                                ep_group=dist.group.WORLD)
        even = [96] * world
        ragged = [40 + 57 * r for r in range(world)]
        empty_first = [0] + [64] * (world - 1)
        grown = [700] * world  # exceeds the first workspace: collective re-allocation
        for index, counts in enumerate((even, ragged, even, empty_first, grown)):
            scenario(module, rank, world, device, counts, hidden, inter, experts, top_k, seed=10 + index,
                     layout=layout)
        state = module.debug_state()
        assert state["ep"] == world and state["generation"] >= 10, state
        module.close()
    # Failure convergence with the operator queued ahead of the table read-back: one rank brings expert weights of
    # the wrong shape. It raises its own error; every other rank learns of it from the validity header, its queued
    # kernels do nothing (the route guard saw the flag on the device) and it raises too. The next call is healthy.
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            ep_group=dist.group.WORLD)
    scenario(module, rank, world, device, [96] * world, hidden, inter, experts, top_k, seed=40, layout="EIO")
    x, ids, probs, _ = make_rank_inputs(rank, 96, hidden, experts, top_k, 41)
    local = experts // world
    good = (torch.zeros(local, hidden, 2 * inter, dtype=torch.bfloat16, device=device),
            torch.zeros(local, inter, hidden, dtype=torch.bfloat16, device=device))
    bad = (good[0][:, :, :inter].contiguous(), good[1])
    try:
        module(x.to(device), ids.to(device), probs.to(device), expert_weights=bad if rank == world - 1 else good)
    except ValueError as error:
        expected = "gate_up_weight must have shape" if rank == world - 1 else "invalid inputs on EP rank"
        assert expected in str(error), str(error)
    else:
        raise AssertionError("every rank must reject a call with invalid inputs on one rank")
    torch.cuda.synchronize()
    module.check_status()
    scenario(module, rank, world, device, [80] * world, hidden, inter, experts, top_k, seed=42, layout="EIO")
    module.close()
    # two serial layers on one peer-mapped workspace
    shared = [MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                             ep_group=dist.group.WORLD) for _ in range(2)]
    MegaMoeExperts.share_execution_resources(shared)
    for index, layer in enumerate(shared + shared):
        scenario(layer, rank, world, device, [64 + 32 * index] * world, hidden, inter, experts, top_k,
                 seed=70 + index, layout="EIO")
    assert shared[0]._workspace is shared[1]._workspace
    shared[0].close()
    assert shared[1]._workspace is not None
    shared[1].close()
    # pull dispatch: owners fetch their rows from the sources' published buffers
    from hyper_multicore_b200 import MegaMoeNumericsOptions, MegaMoeTuningOptions

    pull = MegaMoeTuningOptions(dispatch_mode="pull")
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            ep_group=dist.group.WORLD, tuning_options=pull)
    for index, counts in enumerate(([96] * world, [40 + 57 * r for r in range(world)], [0] + [64] * (world - 1),
                                    [500] * world)):
        scenario(module, rank, world, device, counts, hidden, inter, experts, top_k, seed=80 + index, layout="EIO")
    assert module._workspace.pull
    module.close()
    before = dict(swiglu_limit=0.5, clamp_after_silu=False, apply_probs_before_fc2=True)
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            ep_group=dist.group.WORLD, tuning_options=pull,
                            numerics_options=MegaMoeNumericsOptions(**before))
    for index, counts in enumerate(([96] * world, [40 + 57 * r for r in range(world)])):
        scenario(module, rank, world, device, counts, hidden, inter, experts, top_k, seed=90 + index, layout="EOI",
                 **before)
    module.close()
    # numerics options: clamped SwiGLU with the probabilities travelling with the rows (before FC2)

    options = dict(swiglu_limit=0.5, clamp_after_silu=True, apply_probs_before_fc2=True)
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            ep_group=dist.group.WORLD, numerics_options=MegaMoeNumericsOptions(**options))
    for index, counts in enumerate(([96] * world, [40 + 57 * r for r in range(world)], [0] + [64] * (world - 1))):
        scenario(module, rank, world, device, counts, hidden, inter, experts, top_k, seed=50 + index, layout="EIO",
                 **options)
    module.close()
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            ep_group=dist.group.WORLD, precision="mxfp8")
    for index, counts in enumerate(([96] * world, [40 + 57 * r for r in range(world)], [0] + [200] * (world - 1))):
        scenario_mx(module, rank, world, device, counts, hidden, inter, experts, top_k, seed=30 + index)
    module.close()
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            ep_group=dist.group.WORLD, precision="mxfp8", tuning_options=pull)
    scenario_mx(module, rank, world, device, [40 + 57 * r for r in range(world)], hidden, inter, experts, top_k, seed=33)
    module.close()
    dist.barrier()
    if rank == 0:
        print(f"EP={world} ok", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    try:
        main()
    except BaseException:  # pylint: disable=broad-except
        import traceback

        text = f"[rank {os.environ.get('RANK')}] " + traceback.format_exc()
        print(text, flush=True)
        log_dir = os.environ.get("HMC_TEST_LOG_DIR")
        if log_dir:
            Path(log_dir).mkdir(parents=True, exist_ok=True)
            (Path(log_dir) / f"ep_worker_rank{os.environ.get('RANK')}.log").write_text(text)
        raise
