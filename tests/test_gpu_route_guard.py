"""GPU: the device-side admission check of an expert-parallel call and the skip flag its kernels honour.

The module queues the MoE operator before it has read the count table back; `hmc_route_guard` decides on the
device, from the same table on every rank, whether the call may run, and mirrors table, status words and
decision to pinned host memory for the host's deferred validation.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _table(counts, header, dev):
    """{counts[ep][experts]; header[ep][4]} as the count exchange lays it out."""
    ep = len(counts)
    flat = [c for row in counts for c in row] + [h for r in range(ep) for h in header[r]]
    return torch.tensor(flat, dtype=torch.int32, device=dev)


@pytest.mark.parametrize("case,capacity,routed_limit,invalid_rank,expected", [
    ("fits", 100, 100, None, 0), ("exact fit", 23, 24, None, 0), ("rank 1 receives too many rows", 22, 100, None, 1),
    ("rank 0 routes too many rows", 100, 23, None, 1), ("rank 1 flagged its inputs invalid", 100, 100, 1, 1)])
def test_route_guard_decision_and_host_mirror(cuda_device, case, capacity, routed_limit, invalid_rank, expected):
    from hyper_multicore_b200 import _lib, kernels as K

    dev = cuda_device
    ep, experts = 2, 4
    counts = [[5, 6, 7, 6], [1, 2, 9, 1]]  # rank 0 routes 24 rows, rank 1 13; rank 0 receives 14, rank 1 23
    header = [[0, 12, 1, 0], [0, 7, 1, 0]]
    if invalid_rank is not None:
        header[invalid_rank][0] = 1
    table = _table(counts, header, dev)
    status = _lib.new_status(dev)
    status[2] = 41  # the mirror carries the status words as they are
    flag = torch.full((1,), -1, dtype=torch.int32, device=dev)
    mirror = torch.full((ep * (experts + 4) + _lib.HMC_STATUS_WORDS + 1,), -5, dtype=torch.int32).pin_memory()
    K.route_guard(table, ep, experts, capacity, routed_limit, status, flag, mirror)
    torch.cuda.synchronize()
    assert flag.item() == expected, case
    words = mirror.tolist()
    assert words[:ep * (experts + 4)] == table.cpu().tolist()
    assert words[ep * (experts + 4):-1] == status.cpu().tolist()
    assert words[-1] == expected


def test_kernels_given_a_set_flag_do_nothing(cuda_device):
    """A grouped GEMM (tiles and dispatch warps), the stand-alone dispatch and the bounded wait all return at once
    when the flag is set: no store, no wait, no status word; with the flag cleared the same calls do their work."""
    from hyper_multicore_b200 import _lib, kernels as K

    dev = cuda_device
    rows, k, n, experts = 300, 128, 256, 2
    counts = torch.tensor([[180, 120]], dtype=torch.int32, device=dev)
    off = K.route_offsets(counts, 0)
    a = torch.randn(rows, k, device=dev).bfloat16()
    w = (torch.randn(experts, k, n, device=dev) * 0.05).bfloat16()
    expert_of_row = torch.cat([torch.zeros(180), torch.ones(120)]).int().to(dev)
    status = _lib.new_status(dev)
    lib = _lib.load()
    stream = torch.cuda.current_stream(dev).cuda_stream
    for value in (1, 0):
        flag = torch.tensor([value], dtype=torch.int32, device=dev)
        received = torch.zeros(rows, k, device=dev, dtype=torch.bfloat16)
        c = torch.full((rows, n), 7.0, device=dev, dtype=torch.bfloat16)
        ctrl = torch.zeros(_lib.HMC_CTRL_WORDS, dtype=torch.int32, device=dev)
        peers = (ctypes.c_void_p * 1)(received.data_ptr())
        peer_ctrl = (ctypes.c_void_p * 1)(ctrl.data_ptr())
        K._call("hmc_ep_publish_ready", dev, peer_ctrl, 1, 0, 1)
        sending = K._dispatch_struct(a, None, expert_of_row, off["dispatch_src_off"], off["dispatch_target_off"], rows=rows,
                                     top_k=1, ep=1, local_experts=experts, capacity_rows=rows, peer_buffers=peers,
                                     peer_ctrl=peer_ctrl, local_ctrl=ctrl, generation=1, status=status,
                                     budget_ns=1_000_000_000, rank=0)
        sending.skip_flag = flag.data_ptr()
        args = _lib.GroupedGemmArgs()
        args.mode, args.a_major, args.b_major, args.epilogue = K.HMC_GEMM_RAGGED_M, K.HMC_MAJOR_K, K.HMC_MAJOR_MN, 0
        args.groups, args.rows, args.n, args.k = experts, rows, n, k
        args.a, args.b, args.c = received.data_ptr(), w.data_ptr(), c.data_ptr()
        args.group_ends = off["group_list"].data_ptr()
        args.ready_counters, args.ready_budget_ns = ctrl.data_ptr(), 1_000_000_000
        args.status = status.data_ptr()
        args.dispatch = ctypes.cast(ctypes.pointer(sending), ctypes.c_void_p)
        args.skip_flag = flag.data_ptr()
        _lib.check(lib.hmc_grouped_gemm(ctypes.byref(args), stream))
        # a wait for a counter nothing advances: skipped with the flag, satisfied by the dispatch without it
        _lib.check(lib.hmc_ep_wait_unless(ctrl.data_ptr(), 180, 50_000_000, status.data_ptr(), flag.data_ptr(), stream))
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0, status.tolist()
        if value:
            assert not received.any() and (c == 7).all() and not ctrl[:experts].any()
        else:
            assert torch.equal(received, a) and ctrl[:experts].tolist() == [180, 120]
            ref = torch.cat([a[:180].float() @ w[0].float(), a[180:].float() @ w[1].float()])
            torch.testing.assert_close(c.float(), ref, rtol=2e-2, atol=2e-3 * max(1.0, float(ref.abs().max())))
        # the stand-alone dispatch kernel honours the flag as well
        received.zero_()
        ctrl[:experts].zero_()
        _lib.check(lib.hmc_ep_dispatch(ctypes.byref(sending), stream))
        torch.cuda.synchronize()
        assert bool(received.any()) == (value == 0)
