"""GPU: tcgen05 grouped GEMM, every operand layout and fused epilogue, against an FP32 torch reference."""

import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL, ATOL = 2e-2, 2e-3  # the reference's MoE tolerance (tests/torch/_test_mega_moe.py:38-39)


def _ends(counts, dev):
    return torch.tensor(counts, dtype=torch.int64).cumsum(0).to(dev)


def _starts(counts):
    return [0] + torch.tensor(counts).cumsum(0).tolist()


def _close(got, ref):
    torch.testing.assert_close(got.float(), ref.float(), rtol=RTOL, atol=ATOL * max(1.0, float(ref.abs().max())))


@pytest.mark.parametrize("tile_mode", [1, 2])  # 128-row tiles on one CTA, 256-row tiles on a CTA pair
@pytest.mark.parametrize("b_major", [0, 1])
@pytest.mark.parametrize("counts,k,n", [([128], 64, 256), ([100, 0, 300, 129, 1], 512, 512),
                                        ([100, 0, 300, 129, 1], 200, 328), ([0, 0, 5], 64, 8),
                                        ([700, 1, 0, 900], 1024, 2048)])
def test_ragged_m_plain(cuda_device, tile_mode, b_major, counts, k, n):
    from hyper_multicore_b200 import _lib, kernels as K

    torch.manual_seed(sum(counts) + k)
    dev = cuda_device
    rows, groups, guard = sum(counts), len(counts), 7
    a = torch.randn(rows + guard, k, device=dev).bfloat16()
    w = (torch.randn(groups, k, n, device=dev) * 0.05).bfloat16()
    b = w if b_major == K.HMC_MAJOR_MN else w.transpose(1, 2).contiguous()
    c = torch.full((rows + guard, n), 7.0, device=dev, dtype=torch.bfloat16)
    status = _lib.new_status(dev)
    K.grouped_gemm(a, b, c, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M, b_major=b_major, status=status,
                   tile_mode=tile_mode)
    starts = _starts(counts)
    ref = torch.cat([a[starts[g]:starts[g + 1]].float() @ w[g].float() for g in range(groups)])
    _close(c[:rows], ref)
    assert (c[rows:] == 7).all(), "rows past the last group were written"
    _lib.raise_on_status(status, "grouped gemm")


@pytest.mark.parametrize("tile_mode", [1, 2])
@pytest.mark.parametrize("b_major", [0, 1])
@pytest.mark.parametrize("inter", [384, 200])
def test_ragged_m_swiglu_forward_and_backward_epilogues(cuda_device, tile_mode, b_major, inter):
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(inter)
    dev = cuda_device
    counts, k = [257, 64, 0, 511], 1024
    rows, groups = sum(counts), len(counts)
    starts = _starts(counts)
    a = torch.randn(rows, k, device=dev).bfloat16()
    w = (torch.randn(groups, k, 2 * inter, device=dev) * 0.03).bfloat16()
    b = w if b_major == K.HMC_MAJOR_MN else w.transpose(1, 2).contiguous()
    u = torch.empty(rows, 2 * inter, device=dev, dtype=torch.bfloat16)
    act = torch.empty(rows, inter, device=dev, dtype=torch.bfloat16)
    K.grouped_gemm(a, b, u, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M, b_major=b_major,
                   epilogue=K.HMC_EPI_SWIGLU, aux=act, tile_mode=tile_mode)
    ref_u = torch.cat([a[starts[g]:starts[g + 1]].float() @ w[g].float() for g in range(groups)])
    _close(u, ref_u)
    ub = u.float()  # activation is defined on the BF16-rounded projection
    _close(act, torch.nn.functional.silu(ub[:, :inter]) * ub[:, inter:])
    # backward epilogue: acc = dAct = dY @ W2^T, fused SwiGLU gradient against the saved U
    hidden = 512
    dy = torch.randn(rows, hidden, device=dev).bfloat16()
    w2 = (torch.randn(groups, hidden, inter, device=dev) * 0.03).bfloat16()  # logical [K=hidden, N=inter]
    b2 = w2 if b_major == K.HMC_MAJOR_MN else w2.transpose(1, 2).contiguous()
    du = torch.empty(rows, 2 * inter, device=dev, dtype=torch.bfloat16)
    K.grouped_gemm(dy, b2, du, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M, b_major=b_major,
                   epilogue=K.HMC_EPI_SWIGLU_GRAD, aux=u, tile_mode=tile_mode)
    d_act = torch.cat([dy[starts[g]:starts[g + 1]].float() @ w2[g].float() for g in range(groups)]).bfloat16().float()
    gate, up = ub[:, :inter], ub[:, inter:]
    sig = torch.sigmoid(gate)
    ref_du = torch.cat([d_act * up * sig * (1 + gate * (1 - sig)), d_act * gate * sig], dim=-1)
    _close(du, ref_du)


@pytest.mark.parametrize("tile_mode", [0, 1])  # 1: one-CTA tiles; otherwise CTA pairs on 256 x 256 tiles where m % 256 == 0
@pytest.mark.parametrize("f32", [False, True])
@pytest.mark.parametrize("counts,m,n", [([64], 128, 256), ([128, 0, 65, 1, 300], 256, 512),
                                        ([128, 0, 65, 1, 300], 200, 328), ([0, 0], 128, 256),
                                        ([128, 0, 65, 1, 300], 256, 328), ([0, 0, 0], 512, 256),
                                        ([77, 16, 0, 500, 33, 7], 512, 768), ([399] * 24 + [0, 1000], 1024, 1280)])
def test_ragged_k_weight_gradient(cuda_device, f32, counts, m, n, tile_mode):
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(m + n)
    dev = cuda_device
    rows, groups = sum(counts), len(counts)
    a = torch.randn(rows + 5, m, device=dev).bfloat16()
    b = (torch.randn(rows + 5, n, device=dev) * 0.1).bfloat16()
    a[rows:] = float("nan")  # rows past the last group must never leak into a product
    b[rows:] = float("nan")
    c = torch.full((groups, m, n), 3.0, device=dev, dtype=torch.float32 if f32 else torch.bfloat16)
    K.grouped_gemm(a, b, c, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_K,
                   epilogue=K.HMC_EPI_STORE_F32 if f32 else K.HMC_EPI_STORE_BF16, tile_mode=tile_mode)
    starts = _starts(counts)
    ref = torch.stack([a[starts[g]:starts[g + 1]].float().T @ b[starts[g]:starts[g + 1]].float() for g in range(groups)])
    _close(c, ref)
    for g, count in enumerate(counts):
        if count == 0:
            assert (c[g] == 0).all(), "a cold expert must get an exact-zero gradient"


def test_full_size_linearity(cuda_device):
    """Size-independent property at the benchmark's GEMM1 shape: C(a1 + a2) == C(a1) + C(a2) within BF16."""
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(0)
    dev = cuda_device
    counts = [512] * 32
    rows, k, n = sum(counts), 4096, 3072
    w = (torch.randn(32, k, n, device=dev) * 0.02).bfloat16()
    a1 = torch.randn(rows, k, device=dev).bfloat16()
    a2 = (a1 * 0.5).bfloat16()  # exactly representable, so a1 + a2 = 1.5 * a1 has one rounding
    outs = []
    for a in (a1, a2, (a1.float() + a2.float()).bfloat16()):
        c = torch.empty(rows, n, device=dev, dtype=torch.bfloat16)
        K.grouped_gemm(a, w, c, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M)
        outs.append(c.float())
    _close(outs[2], outs[0] + outs[1])
    spot = torch.randint(0, rows, (64,), device=dev)
    ref = torch.stack([a1[r].float() @ w[int(r) // 512].float() for r in spot])
    _close(outs[0][spot], ref)


def test_arrival_counters_gate_the_groups(cuda_device):
    """Counters already at their expected value let every group through; a counter that nothing
    advances makes the bounded wait run out and sets the status words instead of hanging."""
    from hyper_multicore_b200 import _lib, kernels as K

    dev = cuda_device
    counts = [130, 70]
    a = torch.randn(200, 64, device=dev).bfloat16()
    w = torch.randn(2, 64, 256, device=dev).bfloat16()
    c = torch.zeros(200, 256, device=dev, dtype=torch.bfloat16)
    ready = torch.tensor(counts, dtype=torch.int32, device=dev)
    status = _lib.new_status(dev)
    K.grouped_gemm(a, w, c, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M, ready_counters=ready, status=status,
                   ready_budget_ns=200_000_000)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0
    _close(c[:130], a[:130].float() @ w[0].float())
    ready[1] = 69  # one row of group 1 never "arrives"
    K.grouped_gemm(a, w, c, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M, ready_counters=ready, status=status,
                   ready_budget_ns=50_000_000)
    torch.cuda.synchronize()
    words = status.tolist()
    assert words[0] == 2 and words[1:4] == [1, 70, 69]
    # the context is still healthy
    status.zero_()
    ready[1] = 70
    K.grouped_gemm(a, w, c, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M, ready_counters=ready, status=status)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0


def test_late_rows_do_not_look_like_a_pipeline_fault(cuda_device):
    """The producer may wait for a peer's rows for the whole arrival budget; the MMA and epilogue warps
    behind it must outlast that wait. Here the internal barrier budget (20 ms) runs out long before the
    missing row "arrives" (the host advances the counter, which lives in pinned host memory, after
    0.3 s) and well inside the arrival budget (5 s): the GEMM must finish with a clean status."""
    import time

    from hyper_multicore_b200 import _lib, kernels as K

    dev = cuda_device
    counts = [130, 70]
    a = torch.randn(200, 64, device=dev).bfloat16()
    w = torch.randn(2, 64, 256, device=dev).bfloat16()
    for tile_mode in (1, 2):
        c = torch.zeros(200, 256, device=dev, dtype=torch.bfloat16)
        ready = torch.tensor([130, 69], dtype=torch.int32).pin_memory()
        status = _lib.new_status(dev)
        torch.cuda.synchronize()
        K.grouped_gemm(a, w, c, _ends(counts, dev), mode=K.HMC_GEMM_RAGGED_M, ready_counters=ready, status=status,
                       ready_budget_ns=5_000_000_000, pipe_budget_ns=20_000_000, tile_mode=tile_mode)
        time.sleep(0.3)
        ready[1] = 70
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0, status.tolist()
        _close(c[130:], a[130:].float() @ w[1].float())


def test_ready_flag_that_nobody_publishes_times_out(cuda_device):
    """A dispatch towards a generation no peer has declared itself ready for gives up after its budget with
    HMC_STATUS_TIMEOUT_READY {peer, expected, seen}; the kernel returns, and the next, published, call
    on the same control block is healthy."""
    import ctypes

    from hyper_multicore_b200 import _lib, kernels as K

    dev = cuda_device
    rows, hidden, experts = 64, 128, 4
    tokens = torch.randn(rows, hidden, device=dev).bfloat16()
    expert_of_row = torch.arange(rows, device=dev, dtype=torch.int32) // (rows // experts)
    counts = torch.full((1, experts), rows // experts, dtype=torch.int32, device=dev)
    off = K.route_offsets(counts, 0)
    ctrl = torch.zeros(_lib.HMC_CTRL_WORDS, dtype=torch.int32, device=dev)
    received = torch.zeros(rows, hidden, device=dev, dtype=torch.bfloat16)
    peers = (ctypes.c_void_p * 1)(received.data_ptr())
    peer_ctrl = (ctypes.c_void_p * 1)(ctrl.data_ptr())
    status = _lib.new_status(dev)

    def dispatch(generation):
        K.ep_dispatch(tokens, None, expert_of_row, off["dispatch_src_off"], off["dispatch_target_off"], rows=rows,
                      top_k=1, ep=1, local_experts=experts, capacity_rows=rows, peer_buffers=peers,
                      peer_ctrl=peer_ctrl, local_ctrl=ctrl, generation=generation, status=status,
                      budget_ns=20_000_000)
        torch.cuda.synchronize()

    dispatch(5)  # the ready word still holds 0
    words = status.tolist()
    assert words[0] == 3 and words[1:4] == [0, 5, 0], words
    assert not received.any(), "no row may be stored towards a peer that is not ready"
    status.zero_()
    K._call("hmc_ep_publish_ready", dev, peer_ctrl, 1, 0, 5)
    dispatch(5)
    assert status.tolist()[0] == 0
    assert torch.equal(received, tokens)
    assert ctrl[:experts].tolist() == [rows // experts] * experts


@pytest.mark.parametrize("tile_mode", [1, 2])
@pytest.mark.parametrize("hidden", [256, 1000])
def test_dispatch_warps_feed_the_gemm_that_carries_them(cuda_device, tile_mode, hidden):
    """A row-ragged GEMM with a fused dispatch: extra warps of the same launch gather this rank's rows into
    the receive buffer and advance the arrival counters its tile producers wait on. One rank stands for
    the group (every expert is local), so rows, counters and results can be checked exactly."""
    import ctypes

    from hyper_multicore_b200 import _lib, kernels as K

    torch.manual_seed(hidden + tile_mode)
    dev = cuda_device
    tokens, top_k, experts, n = 300, 2, 4, 256
    x = torch.randn(tokens, hidden, device=dev).bfloat16()
    ids = torch.stack([torch.randperm(experts, device=dev)[:top_k] for _ in range(tokens)]).int()
    mapping, sources, row_experts, counts, _ = K.moe_sort_routes(ids, experts)
    off = K.route_offsets(counts.view(1, experts), 0)
    rows = tokens * top_k
    w = (torch.randn(experts, hidden, n, device=dev) * 0.05).bfloat16()
    received = torch.zeros(rows, hidden, device=dev, dtype=torch.bfloat16)
    c = torch.zeros(rows, n, device=dev, dtype=torch.bfloat16)
    ctrl = torch.zeros(_lib.HMC_CTRL_WORDS, dtype=torch.int32, device=dev)
    peers = (ctypes.c_void_p * 1)(received.data_ptr())
    peer_ctrl = (ctypes.c_void_p * 1)(ctrl.data_ptr())
    status = _lib.new_status(dev)
    K._call("hmc_ep_publish_ready", dev, peer_ctrl, 1, 0, 1)
    sending = dict(tokens=x, source_of_row=sources, expert_of_row=row_experts, dispatch_src_off=off["dispatch_src_off"],
                   dispatch_target_off=off["dispatch_target_off"], rows=rows, top_k=top_k, ep=1, local_experts=experts,
                   capacity_rows=rows, peer_buffers=peers, peer_ctrl=peer_ctrl, local_ctrl=ctrl, generation=1,
                   status=status, budget_ns=2_000_000_000, rank=0, send_order_start=off["send_order_start"])
    K.grouped_gemm(received, w, c, off["group_list"], mode=K.HMC_GEMM_RAGGED_M, ready_counters=ctrl[:experts],
                   ready_budget_ns=2_000_000_000, status=status, tile_mode=tile_mode, dispatch=sending)
    torch.cuda.synchronize()
    assert status.tolist()[0] == 0, status.tolist()
    expected_rows = x[(sources // top_k).long()]
    assert torch.equal(received, expected_rows), "the dispatch warps must deliver every row to its slot"
    assert ctrl[:experts].tolist() == counts.tolist(), "every expert's arrival counter must reach its row count"
    starts = [0] + counts.cumsum(0).tolist()
    ref = torch.cat([expected_rows[starts[g]:starts[g + 1]].float() @ w[g].float() for g in range(experts)])
    _close(c, ref)
