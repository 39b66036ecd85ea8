"""GPU: MXFP8 quantisers, block-scaled GEMM and the MXFP8 MegaMoeExperts backend.

Parity is UNPINNED by the reference (no numeric MXFP8 golden exists there): these tests compare with
oracle/mxfp8.py, the CPU statement of the OCP Microscaling rule this build uses. Quantised bytes and
scales must match the oracle bit for bit; GEMM results within rel-L2 1e-2 (outputs) / 3e-2 (gradients).
"""

import pytest
import torch

from oracle import mxfp8 as omx
from tests.helpers import rel_l2

pytestmark = pytest.mark.gpu


def _unpack_row_atoms(atoms, pad_blocks, width):
    """atoms [width/128][pad_blocks][32][4][4] -> biased exponents [pad_blocks*128, width/32]."""
    a = atoms.view(width // 128, pad_blocks, 32, 4, 4).permute(1, 3, 2, 0, 4)  # [pb, r4, r32, cb, kk]
    return a.reshape(pad_blocks * 128, width // 32)


def _unpack_col_atoms(atoms, pad_blocks, width):
    """atoms [pad_blocks][width/128][32][4][4] -> biased exponents [pad_blocks*4, width]."""
    a = atoms.view(pad_blocks, width // 128, 32, 4, 4).permute(0, 4, 1, 3, 2)  # [pb, kk, cb, c4, c32]
    return a.reshape(pad_blocks * 4, width)


def _padded_starts(counts):
    starts, block = [], 0
    for c in counts:
        starts.append(block * 128)
        block += (c + 127) // 128
    return starts


@pytest.mark.parametrize("counts,width", [([128], 128), ([100, 0, 300, 129, 1], 256), ([5, 700], 384)])
def test_plain_quantiser_is_bit_exact(cuda_device, counts, width):
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(sum(counts))
    rows = sum(counts)
    x = (torch.randn(rows, width) * torch.rand(rows, 1) * 4).bfloat16()
    x[0, :32] = 0  # an all-zero block takes scale 1
    ends = torch.tensor(counts, dtype=torch.int64).cumsum(0)
    q = K.mx_quant(x.to(cuda_device), ends.to(cuda_device), width, want_row=True, want_col=True)
    torch.cuda.synchronize()
    row_scale = _unpack_row_atoms(q.row_scale.cpu(), q.pad_blocks, width)
    col_scale = _unpack_col_atoms(q.col_scale.cpu(), q.pad_blocks, width)
    row_data = q.row_data.cpu().view(torch.float8_e4m3fn)
    col_data = q.col_data.cpu().view(torch.float8_e4m3fn)
    starts = _padded_starts(counts)
    first = 0
    for g, count in enumerate(counts):
        if count == 0:
            continue
        seg = x[first:first + count].float()
        first += count
        ref_q, ref_s = omx.quantize(seg, 1)
        got = slice(starts[g], starts[g] + count)
        assert torch.equal(row_data[got].view(torch.uint8), ref_q.view(torch.uint8))
        assert torch.equal(row_scale[got], ref_s)
        padded = (count + 127) // 128 * 128
        seg_pad = torch.cat((seg, torch.zeros(padded - count, width)))
        ref_q, ref_s = omx.quantize(seg_pad, 0)
        got = slice(starts[g], starts[g] + padded)
        assert torch.equal(col_data[got].view(torch.uint8), ref_q.view(torch.uint8))
        assert torch.equal(col_scale[starts[g] // 32:(starts[g] + padded) // 32], ref_s)


def test_fused_swiglu_quantisers_match_the_oracle(cuda_device):
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(3)
    counts, inter = [70, 0, 200], 128
    rows = sum(counts)
    u = torch.randn(rows, 2 * inter).bfloat16()
    d_act = torch.randn(rows, inter).bfloat16()
    ends = torch.tensor(counts, dtype=torch.int64).cumsum(0).to(cuda_device)
    dense = torch.empty(rows, inter, dtype=torch.bfloat16, device=cuda_device)
    K.mx_quant(u.to(cuda_device), ends, inter, kind=K.HMC_MXQ_SWIGLU, dense=dense)
    gate, up = u.float()[:, :inter], u.float()[:, inter:]
    act = (torch.nn.functional.silu(gate) * up).bfloat16()
    torch.testing.assert_close(dense.cpu().float(), act.float(), rtol=1e-2, atol=1e-2)
    dense2 = torch.empty(rows, 2 * inter, dtype=torch.bfloat16, device=cuda_device)
    q = K.mx_quant(d_act.to(cuda_device), ends, 2 * inter, kind=K.HMC_MXQ_SWIGLU_GRAD, aux=u.to(cuda_device),
                   dense=dense2)
    sig = torch.sigmoid(gate)
    ref = torch.cat((d_act.float() * up * sig * (1 + gate * (1 - sig)), d_act.float() * gate * sig), -1).bfloat16()
    torch.testing.assert_close(dense2.cpu().float(), ref.float(), rtol=1e-2, atol=1e-2)
    # the quantised copy is the quantisation of exactly the dense values the kernel produced
    starts = _padded_starts(counts)
    got_q = q.row_data.cpu().view(torch.float8_e4m3fn)
    got_s = _unpack_row_atoms(q.row_scale.cpu(), q.pad_blocks, 2 * inter)
    first = 0
    for g, count in enumerate(counts):
        if count:
            ref_q, ref_s = omx.quantize(dense2.cpu()[first:first + count].float(), 1)
            assert torch.equal(got_q[starts[g]:starts[g] + count].view(torch.uint8), ref_q.view(torch.uint8))
            assert torch.equal(got_s[starts[g]:starts[g] + count], ref_s)
        first += count


def test_weight_fields_follow_the_reference_contract(cuda_device):
    from hyper_multicore_b200 import kernels as K

    torch.manual_seed(5)
    w = (torch.randn(3, 256, 384) * 0.02).bfloat16()
    got = K.mx_quant_weight(w.to(cuda_device))
    ref = omx.reference_weight_fields(w)
    for name in ("col_data", "row_data"):
        assert got[name].dtype == torch.float8_e4m3fn and got[name].shape == (3, 256, 384)
        assert torch.equal(got[name].cpu().view(torch.uint8), ref[name].view(torch.uint8)), name
    assert got["col_scale"].shape == (3, 4, 384, 2) and got["row_scale"].shape == (3, 256, 6, 2)
    for name in ("col_scale", "row_scale"):
        assert torch.equal(got[name].cpu(), ref[name]), name


def make_case(tokens, hidden, inter, experts, top_k, seed, dead_expert=None):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(tokens, hidden, generator=g).bfloat16()
    logits = torch.randn(tokens, experts, generator=g)
    if dead_expert is not None:
        logits[:, dead_expert] = -1e9
    weights, ids = torch.topk(logits.softmax(-1), top_k, dim=-1)
    w1 = (torch.randn(experts, hidden, 2 * inter, generator=g) * 0.05).bfloat16()
    w2 = (torch.randn(experts, inter, hidden, generator=g) * 0.05).bfloat16()
    grad = torch.randn(tokens, hidden, generator=g).bfloat16()
    return {"hidden": x, "topk_ids": ids, "topk_weights": weights.contiguous(), "w1": w1, "w2": w2, "grad_output": grad}


@pytest.mark.parametrize("tokens,hidden,inter,experts,top_k", [(64, 128, 128, 4, 2), (300, 256, 128, 8, 3),
                                                               (512, 1024, 2048, 16, 2)])
def test_mxfp8_experts_forward_backward(cuda_device, tokens, hidden, inter, experts, top_k):
    from hyper_multicore_b200 import MegaMoeExperts
    from hyper_multicore_b200.mxfp8 import attach_mx_fields

    dev = cuda_device
    case = make_case(tokens, hidden, inter, experts, top_k, seed=tokens, dead_expert=1)
    ref = omx.experts_forward_backward(case["hidden"], case["topk_ids"], case["topk_weights"], case["w1"], case["w2"],
                                       case["grad_output"])
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            precision="mxfp8")
    w1 = attach_mx_fields(case["w1"].to(dev).requires_grad_(True))
    w2 = attach_mx_fields(case["w2"].to(dev).requires_grad_(True))
    x = case["hidden"].to(dev).requires_grad_(True)
    p = case["topk_weights"].to(dev).requires_grad_(True)
    out = module(x, case["topk_ids"].to(dev), p, expert_weights=(w1, w2))
    out2 = module(x.detach(), case["topk_ids"].to(dev), p.detach(), expert_weights=(w1, w2))
    assert torch.equal(out.detach(), out2), "forward must be deterministic"
    out.backward(case["grad_output"].to(dev))
    module.check_status()
    got = {"output": out, "grad_hidden": x.grad, "grad_probs": p.grad, "grad_w1": w1.grad, "grad_w2": w2.grad}
    for name, limit in (("output", 1e-2), ("grad_hidden", 3e-2), ("grad_probs", 3e-2), ("grad_w1", 3e-2),
                        ("grad_w2", 3e-2)):
        value = got[name].detach().cpu().float()
        assert torch.isfinite(value).all(), name
        assert rel_l2(value, ref[name].float()) <= limit, (name, rel_l2(value, ref[name].float()))
    assert (w1.grad[1] == 0).all() and (w2.grad[1] == 0).all(), "cold expert gradients must be exact zeros"


@pytest.mark.parametrize("counts", [[300, 0, 129, 640, 1, 256], [128], [1000, 385]])
def test_cta_pair_tiles_equal_one_cta_tiles_bit_for_bit(cuda_device, counts):
    """The 256 x 256 CTA-pair kernel and the 128 x 128 kernel accumulate the same products in the same order,
    so all three layouts (NN forward, NT for dA / dX, TN for the weight gradients) must agree exactly; the
    one-CTA kernel is the one checked against the oracle above. Groups with an odd number of 128-row blocks
    leave half a pair tile empty; a group without rows gets exact-zero weight gradients."""
    from hyper_multicore_b200 import kernels as K

    dev = cuda_device
    g = torch.Generator().manual_seed(len(counts))
    experts, rows, k, n = len(counts), sum(counts), 512, 768
    ends = torch.tensor(counts, dtype=torch.int64).cumsum(0).to(dev)
    x = torch.randn(rows, k, generator=g).bfloat16().to(dev)
    dy = torch.randn(rows, n, generator=g).bfloat16().to(dev)
    w = (torch.randn(experts, k, n, generator=g) * 0.05).bfloat16().to(dev)
    fields = K.mx_quant_weight(w)
    xq = K.mx_quant(x, ends, k, want_row=True, want_col=True)
    dyq = K.mx_quant(dy, ends, n, want_row=True, want_col=True)
    status = torch.zeros(4, dtype=torch.int32, device=dev)

    def both(run, shape, dtype=torch.bfloat16):
        outs = []
        for tile_mode in (1, 2):
            c = torch.full(shape, 7.0, dtype=dtype, device=dev)
            run(c, tile_mode)
            outs.append(c)
        assert int(status[0]) == 0, status.tolist()
        assert torch.isfinite(outs[0].float()).all() and outs[0].float().abs().sum() > 0
        assert torch.equal(outs[0], outs[1])

    # NN: y = x @ w, scales of w along its rows (the contraction)
    col_atoms = K.mx_pack_weight_scale(fields["col_scale"], 0, experts, k, n)
    both(lambda c, tm: K.mx_gemm(xq.row_data, xq.row_scale, fields["col_data"], col_atoms, c, ends, mode=K.HMC_GEMM_RAGGED_M,
                                 rows=rows, pad_blocks=xq.pad_blocks, n=n, k=k, b_major=K.HMC_MAJOR_MN, status=status,
                                 tile_mode=tm), (rows, n))
    # NT: dx = dy @ w^T, scales of w along its columns
    row_atoms = K.mx_pack_weight_scale(fields["row_scale"], 1, experts, k, n)
    both(lambda c, tm: K.mx_gemm(dyq.row_data, dyq.row_scale, fields["row_data"], row_atoms, c, ends, mode=K.HMC_GEMM_RAGGED_M,
                                 rows=rows, pad_blocks=dyq.pad_blocks, n=k, k=n, b_major=K.HMC_MAJOR_K, status=status,
                                 tile_mode=tm), (rows, k))
    # TN: dw = x^T @ dy per group, both operands quantised down the rows
    for epilogue, dtype in ((K.HMC_EPI_STORE_BF16, torch.bfloat16), (K.HMC_EPI_STORE_F32, torch.float32)):
        both(lambda c, tm: K.mx_gemm(xq.col_data, xq.col_scale, dyq.col_data, dyq.col_scale, c, ends, mode=K.HMC_GEMM_RAGGED_K,
                                     rows=rows, pad_blocks=xq.pad_blocks, m=k, n=n, epilogue=epilogue, status=status,
                                     tile_mode=tm), (experts, k, n), dtype)


@pytest.mark.parametrize("counts", [[300, 0, 129, 640, 1, 256], [128], [1000, 385]])
def test_swiglu_quantising_epilogue_equals_gemm_then_quantiser(cuda_device, counts):
    """GEMM1 with the SwiGLU + dual-axis quantisation in its epilogue writes the same U and, bit for bit, the
    same quantised activation (both axes, data and scales, padding rows of every used block included) as the
    plain GEMM followed by the stand-alone SwiGLU quantiser."""
    from hyper_multicore_b200 import kernels as K

    dev = cuda_device
    g = torch.Generator().manual_seed(17 + len(counts))
    experts, rows, k, inter = len(counts), sum(counts), 512, 384
    ends = torch.tensor(counts, dtype=torch.int64).cumsum(0).to(dev)
    x = torch.randn(rows, k, generator=g).bfloat16().to(dev)
    w = (torch.randn(experts, k, 2 * inter, generator=g) * 0.08).bfloat16().to(dev)
    fields = K.mx_quant_weight(w)
    atoms = K.mx_pack_weight_scale(fields["col_scale"], 0, experts, k, 2 * inter)
    xq = K.mx_quant(x, ends, k, want_row=True)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    common = dict(mode=K.HMC_GEMM_RAGGED_M, rows=rows, pad_blocks=xq.pad_blocks, n=2 * inter, k=k, b_major=K.HMC_MAJOR_MN,
                  status=status)
    u_plain = torch.zeros(rows, 2 * inter, dtype=torch.bfloat16, device=dev)
    K.mx_gemm(xq.row_data, xq.row_scale, fields["col_data"], atoms, u_plain, ends, **common)
    ref = K.mx_quant(u_plain, ends, inter, kind=K.HMC_MXQ_SWIGLU, want_row=True, want_col=True)
    u_fused = torch.zeros_like(u_plain)
    got = K.MxActivations(rows, experts, inter, dev, want_row=True, want_col=True)
    K.mx_gemm(xq.row_data, xq.row_scale, fields["col_data"], atoms, u_fused, ends, epilogue=K.HMC_EPI_SWIGLU_MXQ, act=got,
              **common)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    assert torch.equal(u_plain, u_fused) and u_plain.float().abs().sum() > 0
    used = sum((c + 127) // 128 for c in counts)  # blocks that hold rows; the spare ones behind them are never written
    assert got.pad_blocks == ref.pad_blocks
    assert torch.equal(got.row_data[:used * 128], ref.row_data[:used * 128])
    assert torch.equal(got.col_data[:used * 128], ref.col_data[:used * 128])
    row_atoms = lambda q: q.row_scale.view(inter // 128, q.pad_blocks, 512)[:, :used]
    col_atoms = lambda q: q.col_scale.view(q.pad_blocks, inter // 128, 512)[:used]
    assert torch.equal(row_atoms(got), row_atoms(ref))
    assert torch.equal(col_atoms(got), col_atoms(ref))


@pytest.mark.parametrize("counts", [[300, 0, 129, 640, 1, 256], [128], [1000, 385]])
@pytest.mark.parametrize("want_da", [True, False])
def test_swiglu_grad_quantising_epilogue_equals_gemm_then_quantiser(cuda_device, counts, want_da):
    """dA = dY . W2^T with the SwiGLU-grad + dual-axis quantisation in its epilogue gives, bit for bit, the
    quantised dU = [dgate | dup] of the plain GEMM followed by the stand-alone SwiGLU-grad quantiser, and the
    same dAct when that is asked for."""
    from hyper_multicore_b200 import kernels as K

    dev = cuda_device
    g = torch.Generator().manual_seed(29 + len(counts))
    experts, rows, hidden, inter = len(counts), sum(counts), 384, 256
    ends = torch.tensor(counts, dtype=torch.int64).cumsum(0).to(dev)
    dy = torch.randn(rows, hidden, generator=g).bfloat16().to(dev)
    u = torch.randn(rows, 2 * inter, generator=g).bfloat16().to(dev)
    w2 = (torch.randn(experts, inter, hidden, generator=g) * 0.08).bfloat16().to(dev)
    fields = K.mx_quant_weight(w2)
    atoms = K.mx_pack_weight_scale(fields["row_scale"], 1, experts, inter, hidden)
    dyq = K.mx_quant(dy, ends, hidden, want_row=True)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    common = dict(mode=K.HMC_GEMM_RAGGED_M, rows=rows, pad_blocks=dyq.pad_blocks, n=inter, k=hidden, b_major=K.HMC_MAJOR_K,
                  status=status)
    da_plain = torch.zeros(rows, inter, dtype=torch.bfloat16, device=dev)
    K.mx_gemm(dyq.row_data, dyq.row_scale, fields["row_data"], atoms, da_plain, ends, **common)
    ref = K.mx_quant(da_plain, ends, 2 * inter, kind=K.HMC_MXQ_SWIGLU_GRAD, aux=u, want_row=True, want_col=True)
    da_fused = torch.zeros_like(da_plain) if want_da else None
    got = K.MxActivations(rows, experts, 2 * inter, dev, want_row=True, want_col=True)
    K.mx_gemm(dyq.row_data, dyq.row_scale, fields["row_data"], atoms, da_fused, ends, epilogue=K.HMC_EPI_SWIGLU_GRAD_MXQ,
              act=got, aux=u, **common)
    torch.cuda.synchronize()
    assert int(status[0]) == 0, status.tolist()
    if want_da:
        assert torch.equal(da_plain, da_fused)
    assert da_plain.float().abs().sum() > 0
    used = sum((c + 127) // 128 for c in counts)
    assert torch.equal(got.row_data[:used * 128], ref.row_data[:used * 128])
    assert torch.equal(got.col_data[:used * 128], ref.col_data[:used * 128])
    width = 2 * inter
    assert torch.equal(got.row_scale.view(width // 128, got.pad_blocks, 512)[:, :used],
                       ref.row_scale.view(width // 128, ref.pad_blocks, 512)[:, :used])
    assert torch.equal(got.col_scale.view(got.pad_blocks, width // 128, 512)[:used],
                       ref.col_scale.view(ref.pad_blocks, width // 128, 512)[:used])


def test_requantised_weights_replace_cached_scale_factors(cuda_device):
    """One module, weights updated in place and re-quantised between calls (an optimiser step): the new
    field tensors tend to land in the memory the old ones just freed, and fresh weights may even get a
    recycled id(). The packed scale factors must follow the new fields, not a cache entry."""
    from hyper_multicore_b200 import MegaMoeExperts
    from hyper_multicore_b200.mxfp8 import attach_mx_fields

    dev = cuda_device
    tokens, hidden, inter, experts, top_k = 96, 256, 128, 4, 2
    module = MegaMoeExperts(hidden_size=hidden, intermediate_size=inter, num_experts=experts, top_k=top_k,
                            precision="mxfp8")
    w1 = w2 = None
    for seed in (30, 31, 32, 33):
        case = make_case(tokens, hidden, inter, experts, top_k, seed=seed)
        case["w1"] = (case["w1"].float() * (1.0 + seed % 3)).bfloat16()  # different scale factors every round
        ref = omx.experts_forward_backward(case["hidden"], case["topk_ids"], case["topk_weights"], case["w1"],
                                           case["w2"], case["grad_output"])
        if seed % 2 == 0 or w1 is None:  # fresh tensors ...
            w1 = case["w1"].to(dev).requires_grad_(True)
            w2 = case["w2"].to(dev).requires_grad_(True)
        else:  # ... or the same tensors updated in place
            with torch.no_grad():
                w1.copy_(case["w1"].to(dev))
                w2.copy_(case["w2"].to(dev))
            w1.grad = w2.grad = None
        attach_mx_fields(w1)
        attach_mx_fields(w2)
        x = case["hidden"].to(dev).requires_grad_(True)
        p = case["topk_weights"].to(dev).requires_grad_(True)
        out = module(x, case["topk_ids"].to(dev), p, expert_weights=(w1, w2))
        out.backward(case["grad_output"].to(dev))
        module.check_status()
        for name, value, limit in (("output", out, 1e-2), ("grad_hidden", x.grad, 3e-2), ("grad_w1", w1.grad, 3e-2)):
            error = rel_l2(value.detach().cpu().float(), ref[name].float())
            assert error <= limit, (seed, name, error)
        del x, p, out


def test_mxfp8_validation(cuda_device):
    from hyper_multicore_b200 import MegaMoeExperts, MegaMoeNumericsOptions

    with pytest.raises(ValueError, match="does not support clamp"):
        MegaMoeExperts(hidden_size=128, intermediate_size=128, num_experts=4, top_k=2, precision="mxfp8",
                       numerics_options=MegaMoeNumericsOptions(swiglu_limit=7.0))
    with pytest.raises(ValueError, match="multiples of 128"):
        MegaMoeExperts(hidden_size=192, intermediate_size=128, num_experts=4, top_k=2, precision="mxfp8")
    module = MegaMoeExperts(hidden_size=128, intermediate_size=128, num_experts=4, top_k=2, precision="mxfp8")
    case = make_case(16, 128, 128, 4, 2, seed=1)
    args = [case[k].to(cuda_device) for k in ("hidden", "topk_ids", "topk_weights")]
    with pytest.raises(ValueError, match="missing required col data/scale"):
        module(*args, expert_weights=(case["w1"].to(cuda_device), case["w2"].to(cuda_device)))
