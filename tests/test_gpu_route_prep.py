"""GPU parity (bit-exact): histogram, stable expert-major sort, offsets, row movement."""

import numpy as np
import pytest
import torch

from oracle import route as oroute
from tests.helpers import load_cases

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens,top_k,experts,dtype", [
    (0, 2, 4, torch.int64), (1, 1, 1, torch.int32), (17, 2, 4, torch.int64), (128, 4, 32, torch.int32),
    (129, 3, 7, torch.int64), (4096, 4, 32, torch.int64), (8192, 8, 256, torch.int32), (5000, 6, 1000, torch.int64),
    (60000, 8, 64, torch.int32)])
def test_sort_routes_is_bit_exact(cuda_device, tokens, top_k, experts, dtype):
    """Up to a few hundred thousand routes the sort is one cooperative launch (per-warp counters up to 256 experts,
    warps taking turns beyond); the 480000-route case needs more chunks than are resident at once and takes the
    three-kernel path."""
    from hyper_multicore_b200 import _lib, kernels as K

    rng = np.random.default_rng(tokens + experts)
    weights = rng.random(experts) ** 3 + 1e-3  # skewed loads, some experts nearly empty
    ids = rng.choice(experts, size=(tokens, top_k), p=weights / weights.sum()) if tokens else np.zeros((0, top_k), int)
    if experts > 3 and tokens:
        ids[ids == 2] = 3  # expert 2 is empty
    status = _lib.new_status(cuda_device)
    mapping, sources, row_experts, counts, cumulative = K.moe_sort_routes(
        torch.from_numpy(ids).to(dtype).to(cuda_device), experts, status=status)
    ref_map, ref_src, ref_exp = oroute.permutation(ids, experts)
    ref_counts = oroute.counts(ids, experts)
    assert np.array_equal(mapping.cpu().numpy(), ref_map)
    assert np.array_equal(counts.cpu().numpy(), ref_counts)
    assert np.array_equal(cumulative.cpu().numpy(), ref_counts.astype(np.int64).cumsum())
    if tokens:
        assert np.array_equal(sources.cpu().numpy(), ref_src)
        assert np.array_equal(row_experts.cpu().numpy(), ref_exp)
    assert np.array_equal(K.moe_histogram(torch.from_numpy(ids).to(dtype).to(cuda_device), experts).cpu().numpy(),
                          ref_counts)
    _lib.raise_on_status(status, "sort")


def test_bad_expert_id_is_reported_not_faulted(cuda_device):
    from hyper_multicore_b200 import _lib, kernels as K

    ids = torch.tensor([[0, 1], [9, 1]], device=cuda_device)
    status = _lib.new_status(cuda_device)
    K.moe_sort_routes(ids, 4, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 4


def test_route_offsets_match_reference_fixture(cuda_device):
    from hyper_multicore_b200 import kernels as K

    for case in load_cases("route"):
        table = case["table"].to(cuda_device)
        rank = int(case["rank"])
        out = K.route_offsets(table, rank)
        for name in ("dispatch_src_off", "dispatch_target_off", "dispatch_size", "combine_src_off",
                     "combine_target_off", "combine_size", "group_list"):
            assert torch.equal(out[name].cpu(), case[name]), name
            assert out[name].dtype == case[name].dtype
        ep, experts = table.shape
        local = experts // ep
        totals = out["totals"].cpu().tolist()
        assert totals[0] == int(case["table"][rank].sum())
        assert totals[1] == int(case["table"][:, rank * local:(rank + 1) * local].sum())


@pytest.mark.parametrize("tokens,top_k,hidden,experts", [(1, 1, 8, 1), (17, 2, 64, 4), (129, 4, 1024, 8), (512, 2, 1024, 16)])
def test_row_movement_round_trips(cuda_device, tokens, top_k, hidden, experts):
    from hyper_multicore_b200 import _lib, kernels as K

    torch.manual_seed(tokens)
    dev = cuda_device
    x = torch.randn(tokens, hidden).bfloat16()
    ids = torch.stack([torch.randperm(experts)[:top_k] for _ in range(tokens)])
    probs = torch.rand(tokens, top_k)
    mapping, sources, _, _, _ = K.moe_sort_routes(ids.to(dev), experts)
    ref_map, ref_src, _ = oroute.permutation(ids.numpy(), experts)
    rows = tokens * top_k
    guard = 3
    status = _lib.new_status(dev)
    # gather form (moe_token_permute_out) with guard rows around the output
    out = torch.full((rows + 2 * guard, hidden), 7.0, dtype=torch.bfloat16, device=dev)
    K.moe_gather_rows(x.to(dev), sources, top_k, out[guard:guard + rows])
    expected = x[torch.from_numpy(ref_src).long() // top_k]
    assert torch.equal(out[guard:guard + rows].cpu(), expected)
    assert (out[:guard] == 7).all() and (out[guard + rows:] == 7).all()
    # scatter form (moe_token_permute_from_mapping_out): bit-preserving copy of rows and probabilities
    out2 = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)
    out_p = torch.empty(rows, device=dev)
    K.moe_permute_from_mapping(x.to(dev), mapping, probs.to(dev), top_k, out2, out_p, status=status)
    assert torch.equal(out2.cpu(), expected)
    assert torch.equal(out_p.cpu()[torch.from_numpy(ref_map).long()], probs.reshape(-1))
    # weighted un-permutation, golden order: BF16 round per term, BF16 accumulate in expert order
    y = torch.randn(rows, hidden).bfloat16()
    restored = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
    K.moe_unpermute(y.to(dev), mapping, probs.to(dev), tokens, top_k, restored, status=status)
    ref = torch.zeros(tokens, hidden, dtype=torch.bfloat16)
    map_t = torch.from_numpy(ref_map).long().reshape(tokens, top_k)
    for e in range(experts):
        t_idx, k_idx = torch.where(ids == e)
        weighted = (y[map_t[t_idx, k_idx]].float() * probs[t_idx, k_idx, None]).bfloat16()
        ref = ref.index_add(0, t_idx, weighted)
    assert torch.equal(restored.cpu(), ref)
    # its backward
    g = torch.randn(tokens, hidden).bfloat16()
    gperm = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)
    gprob = torch.empty(tokens, top_k, device=dev)
    K.moe_unpermute_grad(y.to(dev), g.to(dev), mapping, probs.to(dev), top_k, gperm, gprob, status=status)
    ref_gperm = torch.empty(rows, hidden, dtype=torch.bfloat16)
    ref_gperm[map_t.reshape(-1)] = (g.float().repeat_interleave(top_k, 0) * probs.reshape(-1, 1)).bfloat16()
    assert torch.equal(gperm.cpu(), ref_gperm)
    ref_gprob = (g.float().unsqueeze(1) * y[map_t].float()).sum(-1)
    torch.testing.assert_close(gprob.cpu(), ref_gprob, rtol=1e-4, atol=1e-4)
    # K-sum of permuted gradients
    gx = torch.empty(tokens, hidden, dtype=torch.bfloat16, device=dev)
    K.moe_token_permute_grad(gperm, mapping, tokens, top_k, gx, status=status)
    torch.testing.assert_close(gx.cpu().float(), ref_gperm[map_t].float().sum(1), rtol=1e-2, atol=1e-2)
    _lib.raise_on_status(status, "row movement")


def test_zero_empty_expert_gradients(cuda_device):
    from hyper_multicore_b200 import kernels as K

    first = torch.ones(4, 8, 16, dtype=torch.bfloat16, device=cuda_device)
    second = torch.ones(4, 16, 8, dtype=torch.float32, device=cuda_device)
    cumulative = torch.tensor([0, 5, 5, 9], dtype=torch.int64, device=cuda_device)
    K.zero_empty_expert_grad(first, second, cumulative)
    assert first.sum(dim=(1, 2)).cpu().tolist() == [0, 128, 0, 128]
    assert second.sum(dim=(1, 2)).cpu().tolist() == [0, 128, 0, 128]


@pytest.mark.parametrize("ep,experts", [(1, 4), (2, 8), (4, 32), (8, 256)])
def test_send_order_visits_local_expert_zero_of_every_destination_first(cuda_device, ep, experts):
    """Prefix of a rank's segments in the order a GEMM-carried dispatch sends them: local expert le of the
    destinations rank + 1, rank + 2, ..., rank, for le = 0, 1, ... (every owner's first experts complete first)."""
    from hyper_multicore_b200 import kernels as K

    rng = np.random.default_rng(ep * 1000 + experts)
    table = rng.integers(0, 50, size=(ep, experts), dtype=np.int32)
    local = experts // ep
    for rank in range(ep):
        off = K.route_offsets(torch.from_numpy(table).to(cuda_device), rank)
        expected, run = [], 0
        for le in range(local):
            for dd in range(ep):
                expected.append(run)
                run += int(table[rank, ((rank + 1 + dd) % ep) * local + le])
        expected.append(run)
        assert off["send_order_start"].cpu().tolist() == expected
        assert run == int(table[rank].sum())
