"""Typed Python entry points over the C ABI: one function per ``hmc_*`` kernel.

Every function takes CUDA tensors the caller allocated, checks nothing the native side already
checks, and enqueues on torch's current stream.
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from ._lib import (HMC_EPI_STORE_BF16, HMC_EPI_STORE_F32, HMC_EPI_SWIGLU, HMC_EPI_SWIGLU_GRAD, HMC_EPI_SWIGLU_GRAD_MXQ, HMC_EPI_SWIGLU_MXQ,
                   HMC_GEMM_RAGGED_K, HMC_GEMM_RAGGED_M, HMC_MAJOR_K, HMC_MAJOR_MN, GroupedGemmArgs)


def _require_cuda(*tensors: torch.Tensor | None) -> torch.device:
    device = None
    for tensor in tensors:
        if tensor is None:
            continue
        if not tensor.is_cuda:
            raise _lib.HmcError("hyper_multicore_b200 kernels need CUDA tensors; there is no CPU path")
        device = tensor.device if device is None else device
        if tensor.device != device:
            raise ValueError("all tensors must be on one CUDA device")
    assert device is not None
    return device


def grouped_gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    c: torch.Tensor,
    group_ends: torch.Tensor,
    *,
    mode: int,
    b_major: int = HMC_MAJOR_MN,
    epilogue: int = HMC_EPI_STORE_BF16,
    aux: torch.Tensor | None = None,
    ready_counters: torch.Tensor | None = None,
    ready_budget_ns: int = 0,
    status: torch.Tensor | None = None,
    max_ctas: int = 0,
    tile_mode: int = 0,
    swiglu_clamp: int = 0,
    swiglu_limit: float = 0.0,
    row_probs: torch.Tensor | None = None,
    row_dot: torch.Tensor | None = None,
    combine: dict | None = None,
    pipe_budget_ns: int = 0,
    dispatch: dict | None = None,
) -> None:
    """Launch the tcgen05 grouped GEMM.

    ``swiglu_clamp`` / ``swiglu_limit`` select the clamped SwiGLU of the SwiGLU epilogues;
    ``row_probs`` (float32 [rows]) weights the activation before FC2 and, in the SwiGLU-grad
    epilogue, ``row_dot`` (float32 [rows], zeroed by the caller) receives the probability gradient.
    ``combine`` (RAGGED_M, BF16 stores) sends the result rows from the epilogue to the routed buffers of
    their source ranks: keys segment_start, combine_target_off (device int64), peer_buffers, peer_ctrl
    (ctypes pointer arrays), ep, local_experts, target_rows_limit; ``c`` may then be None.

    ``dispatch`` (RAGGED_M with ``ready_counters``): the keyword arguments of ``ep_dispatch`` plus ``rank``;
    extra warps of the GEMM then send this rank's rows while its tiles wait for the rows it receives.

    RAGGED_M: ``a`` [rows, k]; ``b`` [groups, k, n_cols] (MN) or [groups, n_cols, k] (K); ``c`` [rows, *].
    RAGGED_K: ``a`` [rows, m]; ``b`` [rows, n]; ``c`` [groups, m, n] BF16 or FP32.
    """
    device = _require_cuda(a, b, c, group_ends, aux, status, row_probs, row_dot)
    if ready_counters is not None and not (ready_counters.is_cuda or ready_counters.is_pinned()):
        raise ValueError("ready_counters must live in device memory or in pinned (device-visible) host memory")
    if c is None and combine is None:
        raise ValueError("grouped_gemm needs an output tensor unless its rows are combined to their sources")
    for name, plane in (("row_probs", row_probs), ("row_dot", row_dot)):
        if plane is not None and (plane.dtype != torch.float32 or not plane.is_contiguous() or plane.numel() < a.shape[0]):
            raise ValueError(f"{name} must be a contiguous float32 tensor with one entry per row")
    args = GroupedGemmArgs()
    args.mode = mode
    args.epilogue = epilogue
    args.groups = group_ends.numel()
    args.max_ctas = max_ctas
    args.tile_mode = tile_mode
    args.rows = a.shape[0]
    if mode == HMC_GEMM_RAGGED_M:
        args.a_major = HMC_MAJOR_K
        args.b_major = b_major
        args.k = a.shape[1]
        n_cols = b.shape[2] if b_major == HMC_MAJOR_MN else b.shape[1]
        args.n = n_cols // 2 if epilogue == HMC_EPI_SWIGLU else n_cols
        args.m = 0
    else:
        args.a_major = HMC_MAJOR_MN
        args.b_major = HMC_MAJOR_MN
        args.m = a.shape[1]
        args.n = b.shape[1]
        args.k = 0
    args.a = a.data_ptr()
    args.b = b.data_ptr()
    args.c = _lib.ptr(c)
    args.aux = _lib.ptr(aux)
    args.group_ends = group_ends.data_ptr()
    args.ready_counters = _lib.ptr(ready_counters)
    args.ready_budget_ns = ready_budget_ns
    args.status = _lib.ptr(status)
    args.swiglu_clamp = swiglu_clamp
    args.swiglu_limit = swiglu_limit
    args.row_probs = _lib.ptr(row_probs)
    args.row_dot = _lib.ptr(row_dot)
    args.pipe_budget_ns = pipe_budget_ns
    fused = None
    if combine is not None:
        fused = _lib.GemmCombine()
        fused.segment_start = combine["segment_start"].data_ptr()
        fused.combine_target_off = combine["combine_target_off"].data_ptr()
        fused.peer_buffers = ctypes.cast(combine["peer_buffers"], ctypes.c_void_p)
        fused.peer_ctrl = ctypes.cast(combine["peer_ctrl"], ctypes.c_void_p)
        fused.ep, fused.local_experts = combine["ep"], combine["local_experts"]
        fused.target_rows_limit = combine["target_rows_limit"]
        args.combine = ctypes.cast(ctypes.pointer(fused), ctypes.c_void_p)
    sending = None
    if dispatch is not None:
        sending = _dispatch_struct(**dispatch)
        args.dispatch = ctypes.cast(ctypes.pointer(sending), ctypes.c_void_p)
    with torch.cuda.device(device):
        _lib.check(_lib.load().hmc_grouped_gemm(ctypes.byref(args), _lib.stream_ptr(device)))


def store_words(dst: torch.Tensor, src: torch.Tensor) -> None:
    """dst[:] = src for int32 tensors, by a kernel. ``dst`` may be pinned host memory: the read-back then
    does not wait behind bulk device-to-host copies queued in a copy engine."""
    if dst.dtype != torch.int32 or src.dtype != torch.int32 or dst.numel() < src.numel():
        raise ValueError("store_words copies int32 words into a tensor at least as large")
    if not (dst.is_cuda or dst.is_pinned()):
        raise ValueError("store_words writes device or pinned host memory")
    device = _require_cuda(src)
    _call("hmc_store_words", device, dst.data_ptr(), src.data_ptr(), src.numel())


def store_words_pair(dst: torch.Tensor, first: torch.Tensor, second: torch.Tensor) -> None:
    """dst = [first | second] for int32 tensors, by ONE kernel (see ``store_words``)."""
    if any(t.dtype != torch.int32 for t in (dst, first, second)) or dst.numel() < first.numel() + second.numel():
        raise ValueError("store_words_pair copies int32 words into a tensor at least as large")
    if not (dst.is_cuda or dst.is_pinned()):
        raise ValueError("store_words_pair writes device or pinned host memory")
    device = _require_cuda(first, second)
    _call("hmc_store_words_pair", device, dst.data_ptr(), first.data_ptr(), first.numel(), second.data_ptr(), second.numel())


def grouped_gemm_combine_units(n: int) -> int:
    """Counter increments per result row of a fused-combine GEMM with ``n`` output columns."""
    return int(_lib.load().hmc_grouped_gemm_combine_units(n))


def _call(name: str, device: torch.device, *args) -> None:
    with torch.cuda.device(device):
        _lib.check(getattr(_lib.load(), name)(*args, _lib.stream_ptr(device)))


# ------------------------------------------------------------------------------------------- gate
_GATE_DEFAULT = "1"  # promoted tcgen05 projection for eligible inputs; HMC_GATE_TENSOR_CORES=0 selects FP32 FMAs


def gate_project(x: torch.Tensor, weight: torch.Tensor, use_tensor_cores: bool | str | None = None) -> torch.Tensor:
    """FP32 logits [T, E] = float(x [T, H]) @ float(weight [E, H]).T.

    BF16 hidden states (at least 128 tokens, H a multiple of 8) go through tcgen05 with the weight split
    into three BF16 parts and the accumulation chain of the dominant part cut every 128 elements of K
    ("promoted"); everything else, or ``use_tensor_cores=False`` / HMC_GATE_TENSOR_CORES=0, takes the FP32-FMA
    kernel. ``use_tensor_cores="unpromoted"`` (HMC_GATE_TENSOR_CORES=unpromoted) is the three-GEMM variant
    whose full-length accumulation leaves about 2e-5 absolute error at H = 4096.
    """
    if use_tensor_cores is None:
        use_tensor_cores = {"0": False, "1": True}.get(os.environ.get("HMC_GATE_TENSOR_CORES", _GATE_DEFAULT),
                                                       os.environ.get("HMC_GATE_TENSOR_CORES"))
    device = _require_cuda(x, weight)
    for name, tensor in (("hidden states", x), ("weight", weight)):
        if tensor.dtype not in (torch.bfloat16, torch.float32):
            raise TypeError(f"MegaGate {name} must be BF16 or FP32, got {tensor.dtype}")
    x = x.contiguous()
    weight = weight.contiguous()
    logits = torch.empty((x.shape[0], weight.shape[0]), dtype=torch.float32, device=device)
    eligible = x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.shape[0] >= 128
    if eligible and use_tensor_cores == "unpromoted":
        need = _lib.load().hmc_gate_project_workspace_bytes(x.shape[0], x.shape[1], weight.shape[0])
        workspace = torch.empty(need, dtype=torch.uint8, device=device)
        _call("hmc_gate_project_tc", device, x.data_ptr(), weight.data_ptr(), int(weight.dtype == torch.bfloat16),
              x.shape[0], x.shape[1], weight.shape[0], logits.data_ptr(), workspace.data_ptr(), need)
        return logits
    if eligible and use_tensor_cores:
        workspace, fresh, keep = _gate_weight_parts(weight, x.shape[1], device)
        _call("hmc_gate_project_promoted", device, x.data_ptr(), weight.data_ptr() if fresh else None,
              int(weight.dtype == torch.bfloat16), x.shape[0], x.shape[1], weight.shape[0], logits.data_ptr(),
              workspace.data_ptr(), workspace.numel(), None)
        keep()
        return logits
    _call("hmc_gate_project", device, x.data_ptr(), int(x.dtype == torch.bfloat16), weight.data_ptr(),
          int(weight.dtype == torch.bfloat16), x.shape[0], x.shape[1], weight.shape[0], logits.data_ptr())
    return logits


def _gate_weight_parts(weight: torch.Tensor, hidden: int, device: torch.device):
    """Workspace holding the BF16 parts of ``weight``, whether the kernel has to fill it, and a call that keeps it.

    The parts stay with the weight tensor until it is written to again (its version counter moves with every
    in-place update, e.g. an optimiser step).
    """
    need = _lib.load().hmc_gate_project_promoted_workspace_bytes(hidden, weight.shape[0])
    cached = getattr(weight, "_hmc_gate_parts", None)
    fresh = cached is None or cached[0] != weight._version or cached[1].device != device or cached[1].numel() != need
    if fresh:
        cached = (weight._version, torch.empty(need, dtype=torch.uint8, device=device))

    def keep() -> None:
        if fresh:
            try:
                weight._hmc_gate_parts = cached
            except (AttributeError, RuntimeError):  # a tensor that takes no attributes: split again next time
                pass

    return cached[1], fresh, keep


def gate_route_fusable(x: torch.Tensor, weight: torch.Tensor, n_group: int = 0) -> bool:
    """True when projection and Route run as one launch (``gate_project_route``): BF16 hidden states that take
    the promoted tcgen05 projection, at most 64 experts, no group limit."""
    if os.environ.get("HMC_GATE_TENSOR_CORES", _GATE_DEFAULT) != "1" or os.environ.get("HMC_GATE_FUSED_ROUTE", "1") != "1":
        return False
    if not (x.is_cuda and x.dtype == torch.bfloat16 and x.ndim == 2 and x.shape[1] % 8 == 0 and x.shape[0] >= 128):
        return False
    if weight.dtype not in (torch.bfloat16, torch.float32):
        return False
    return bool(_lib.load().hmc_gate_project_route_supported(weight.shape[0], n_group))


def gate_project_route(x, weight, text_bias, vision_bias, image_mask, use_vision_bias, top_k, scale, scoring):
    """Projection and Route in one launch; the caller checks ``gate_route_fusable`` first.

    Returns (logits [T, E], weights [T, K], indices [T, K] int64, route_scores [T, E], selected [T, K],
    denominator [T, 1]), bit for bit what ``gate_project`` followed by ``gate_route_out`` produce.
    """
    device = _require_cuda(x, weight, text_bias, vision_bias)
    x = x.contiguous()
    weight = weight.contiguous()
    tokens, experts = x.shape[0], weight.shape[0]
    f32 = {"dtype": torch.float32, "device": device}
    logits = torch.empty((tokens, experts), **f32)
    weights = torch.empty((tokens, top_k), **f32)
    indices = torch.empty((tokens, top_k), dtype=torch.int64, device=device)
    scores = torch.empty((tokens, experts), **f32)
    selected = torch.empty((tokens, top_k), **f32)
    denominator = torch.empty((tokens, 1), **f32)
    args = _lib.GateRouteArgs()
    args.logits = None
    args.text_bias = text_bias.data_ptr()
    args.vision_bias = vision_bias.data_ptr()
    args.image_mask = _lib.ptr(image_mask) if use_vision_bias else None
    args.use_vision_bias = int(bool(use_vision_bias))
    args.experts = experts
    args.top_k = top_k
    args.scoring = _lib.HMC_SCORE[scoring]
    args.tokens = tokens
    args.scale = scale
    args.weights = weights.data_ptr()
    args.indices = indices.data_ptr()
    args.route_scores = scores.data_ptr()
    args.selected = selected.data_ptr()
    args.denominator = denominator.data_ptr()
    args.n_group, args.topk_group = 0, 0
    workspace, fresh, keep = _gate_weight_parts(weight, x.shape[1], device)
    _call("hmc_gate_project_route", device, x.data_ptr(), weight.data_ptr() if fresh else None,
          int(weight.dtype == torch.bfloat16), x.shape[1], logits.data_ptr(), workspace.data_ptr(), workspace.numel(),
          ctypes.byref(args), None)
    keep()
    return logits, weights, indices, scores, selected, denominator


def gate_route_out(logits, text_bias, vision_bias, image_mask, use_vision_bias, top_k, scale, scoring,
                   weights, indices, route_scores, selected, denominator, n_group=0, topk_group=0) -> None:
    """Top-k Route on FP32 logits into caller-owned outputs (``n_group`` > 0: group-limited selection)."""
    device = _require_cuda(logits, text_bias, vision_bias, weights, indices, route_scores, selected, denominator)
    args = _lib.GateRouteArgs()
    args.logits = logits.data_ptr()
    args.text_bias = text_bias.data_ptr()
    args.vision_bias = vision_bias.data_ptr()
    args.image_mask = _lib.ptr(image_mask) if use_vision_bias else None
    args.use_vision_bias = int(bool(use_vision_bias))
    args.experts = logits.shape[1]
    args.top_k = top_k
    args.scoring = _lib.HMC_SCORE[scoring]
    args.tokens = logits.shape[0]
    args.scale = scale
    args.weights = weights.data_ptr()
    args.indices = indices.data_ptr()
    args.route_scores = route_scores.data_ptr()
    args.selected = selected.data_ptr()
    args.denominator = denominator.data_ptr()
    args.n_group, args.topk_group = n_group, topk_group
    _call("hmc_gate_route", device, ctypes.byref(args))


def gate_route_grad_out(logits, route_scores, selected, denominator, indices, grad_weights, top_k, scale,
                        scoring, grad_logits, status=None) -> None:
    """RouteGrad into a caller-owned FP32 [T, E] gradient."""
    device = _require_cuda(logits, route_scores, selected, denominator, indices, grad_weights, grad_logits)
    args = _lib.GateRouteGradArgs()
    args.logits = logits.data_ptr()
    args.route_scores = route_scores.data_ptr()
    args.selected = selected.data_ptr()
    args.denominator = denominator.data_ptr()
    args.indices = indices.data_ptr()
    args.grad_weights = grad_weights.data_ptr()
    args.experts = logits.shape[1]
    args.top_k = top_k
    args.scoring = _lib.HMC_SCORE[scoring]
    args.tokens = logits.shape[0]
    args.scale = scale
    args.grad_logits = grad_logits.data_ptr()
    args.status = _lib.ptr(status)
    _call("hmc_gate_route_grad", device, ctypes.byref(args))


# ------------------------------------------------------------------------------------ route prep
def moe_histogram(indices: torch.Tensor, experts: int, status=None) -> torch.Tensor:
    """INT32 histogram of expert ids."""
    device = _require_cuda(indices)
    flat = indices.reshape(-1).contiguous()
    counts = torch.empty(experts, dtype=torch.int32, device=device)
    _call("hmc_moe_histogram", device, flat.data_ptr(), int(flat.dtype == torch.int64), flat.numel(), experts,
          counts.data_ptr(), _lib.ptr(status))
    return counts


def moe_sort_routes(indices: torch.Tensor, experts: int, *, want_sources: bool = True, status=None):
    """Stable expert-major sort of the flat (token, slot) routes.

    Returns (mapping[T*K] i32, source_of_row[T*K] i32 | None, expert_of_row | None, counts[E] i32,
    cumulative[E] i64).
    """
    device = _require_cuda(indices)
    if indices.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"expert indices must be int32 or int64, got {indices.dtype}")
    flat = indices.reshape(-1).contiguous()
    entries = flat.numel()
    lib = _lib.load()
    workspace = torch.empty(max(1, lib.hmc_moe_sort_workspace_bytes(entries, experts)), dtype=torch.uint8,
                            device=device)
    mapping = torch.empty(entries, dtype=torch.int32, device=device)
    sources = torch.empty(entries, dtype=torch.int32, device=device) if want_sources else None
    row_experts = torch.empty(entries, dtype=torch.int32, device=device) if want_sources else None
    counts = torch.empty(experts, dtype=torch.int32, device=device)
    cumulative = torch.empty(experts, dtype=torch.int64, device=device)
    _call("hmc_moe_sort_routes", device, flat.data_ptr(), int(flat.dtype == torch.int64), entries, experts,
          workspace.data_ptr(), workspace.numel(), mapping.data_ptr(), _lib.ptr(sources), _lib.ptr(row_experts),
          counts.data_ptr(), cumulative.data_ptr(), _lib.ptr(status))
    return mapping, sources, row_experts, counts, cumulative


def moe_gather_rows(tokens: torch.Tensor, source_of_row: torch.Tensor, top_k: int, out: torch.Tensor) -> None:
    """out[row] = tokens[source_of_row[row] // top_k]."""
    device = _require_cuda(tokens, source_of_row, out)
    _call("hmc_moe_gather_rows", device, tokens.data_ptr(), source_of_row.data_ptr(), source_of_row.numel(), top_k,
          tokens.shape[1], out.data_ptr())


def moe_permute_from_mapping(tokens, mapping, probs, top_k, out, out_probs, status=None) -> None:
    """out[mapping[t*K+k]] = tokens[t]; out_probs[mapping[t*K+k]] = probs[t, k]."""
    device = _require_cuda(tokens, mapping, out)
    _call("hmc_moe_permute_from_mapping", device, tokens.data_ptr(), mapping.data_ptr(), _lib.ptr(probs),
          tokens.shape[0], top_k, tokens.shape[1], out.data_ptr(), _lib.ptr(out_probs), _lib.ptr(status))


def moe_unpermute(permuted, mapping, probs, num_tokens, top_k, out, status=None) -> None:
    """Weighted K-sum of expert-major rows back to token order."""
    device = _require_cuda(permuted, mapping, out)
    _call("hmc_moe_unpermute", device, permuted.data_ptr(), mapping.data_ptr(), _lib.ptr(probs), num_tokens, top_k,
          permuted.shape[1], permuted.shape[0], out.data_ptr(), _lib.ptr(status))


def moe_unpermute_grad(permuted, grad_out, mapping, probs, top_k, grad_permuted, grad_probs, status=None) -> None:
    """grad_permuted[row] = bf16(grad_out[t] * p); grad_probs[t,k] = <grad_out[t], permuted[row]>."""
    device = _require_cuda(grad_out, mapping, probs, grad_permuted)
    _call("hmc_moe_unpermute_grad", device, _lib.ptr(permuted), grad_out.data_ptr(), mapping.data_ptr(),
          probs.data_ptr(), grad_out.shape[0], top_k, grad_out.shape[1], grad_permuted.data_ptr(),
          _lib.ptr(grad_probs), _lib.ptr(status))


def moe_token_permute_grad(grad_permuted, mapping, num_tokens, top_k, grad_tokens, status=None) -> None:
    """grad_tokens[t] = sum_k grad_permuted[mapping[t*K+k]]."""
    device = _require_cuda(grad_permuted, mapping, grad_tokens)
    _call("hmc_moe_token_permute_grad", device, grad_permuted.data_ptr(), mapping.data_ptr(), num_tokens, top_k,
          grad_permuted.shape[1], grad_tokens.data_ptr(), _lib.ptr(status))


def zero_empty_expert_grad(first, second, cumulative) -> None:
    """Zero the per-expert slices whose cumulative row count did not advance."""
    device = _require_cuda(first, second, cumulative)
    experts = cumulative.numel()
    _call("hmc_zero_empty_expert_grad", device, first.data_ptr(), first.numel() // experts * first.element_size(),
          _lib.ptr(second), 0 if second is None else second.numel() // experts * second.element_size(),
          cumulative.data_ptr(), experts)


def route_offsets(counts_by_source: torch.Tensor, rank: int):
    """Row-unit push-mode descriptors from the gathered [EP, E] INT32 count table."""
    device = _require_cuda(counts_by_source)
    ep, experts = counts_by_source.shape
    local = experts // ep
    i64 = dict(dtype=torch.int64, device=device)
    i32 = dict(dtype=torch.int32, device=device)
    out = {
        "dispatch_src_off": torch.empty(experts, **i64),
        "dispatch_target_off": torch.empty(experts, **i64),
        "dispatch_size": torch.empty(experts, **i32),
        "combine_src_off": torch.empty(ep * local, **i64),
        "combine_target_off": torch.empty(ep * local, **i64),
        "combine_size": torch.empty(ep * local, **i32),
        "group_list": torch.empty(local, **i64),
        "totals": torch.empty(2, **i64),
        "recv_segment_start": torch.empty(ep * local, **i64),
        "send_order_start": torch.empty(experts + 1, **i64),
    }
    _call("hmc_route_offsets", device, counts_by_source.contiguous().data_ptr(), ep, experts, rank,
          *(out[k].data_ptr() for k in ("dispatch_src_off", "dispatch_target_off", "dispatch_size",
                                        "combine_src_off", "combine_target_off", "combine_size", "group_list",
                                        "totals", "recv_segment_start", "send_order_start")))
    return out


# -------------------------------------------------------------------------------------------- mHC
def mega_mhc_out(previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix, phi, alpha,
                 bias, norm_weight, new_residual, next_pre_mix, next_post_mix, next_residual_mix, block_input,
                 hc_before_norm, inv_rms, sum_out, norm_out, mixed_input, rms_rstd, *, hc_eps, norm_eps, num_iters,
                 need_backward, status=None) -> None:
    """Shifted single-pass mHC forward into caller-owned outputs and caches."""
    device = _require_cuda(previous_output, residual, phi, new_residual)
    hidden = residual.shape[-1]
    tokens = residual.numel() // (4 * hidden)
    lib = _lib.load()
    workspace = torch.empty(lib.hmc_mega_mhc_workspace_bytes(tokens, hidden), dtype=torch.uint8, device=device)
    args = _lib.MegaMhcArgs()
    args.tokens, args.hidden = tokens, hidden
    for name, tensor in (("previous_output", previous_output), ("residual", residual),
                         ("previous_pre_mix", previous_pre_mix), ("previous_post_mix", previous_post_mix),
                         ("previous_residual_mix", previous_residual_mix), ("phi", phi), ("alpha", alpha),
                         ("bias", bias), ("norm_weight", norm_weight), ("new_residual", new_residual),
                         ("next_pre_mix", next_pre_mix), ("next_post_mix", next_post_mix),
                         ("next_residual_mix", next_residual_mix), ("block_input", block_input),
                         ("hc_before_norm", hc_before_norm), ("inv_rms", inv_rms), ("sum_out", sum_out),
                         ("norm_out", norm_out), ("mixed_input", mixed_input), ("rms_rstd", rms_rstd),
                         ("workspace", workspace), ("status", status)):
        setattr(args, name, _lib.ptr(tensor))
    args.workspace_bytes = workspace.numel()
    args.hc_eps, args.norm_eps, args.num_iters, args.need_backward = hc_eps, norm_eps, num_iters, int(need_backward)
    _call("hmc_mega_mhc", device, ctypes.byref(args))


def mega_mhc_grad_out(tensors: dict, *, hc_eps: float, num_iters: int, status=None) -> None:
    """mHC backward; ``tensors`` maps every pointer field of ``hmc_mega_mhc_grad_args`` to a tensor."""
    residual = tensors["residual"]
    device = _require_cuda(residual)
    hidden = residual.shape[-1]
    tokens = residual.numel() // (4 * hidden)
    lib = _lib.load()
    workspace = torch.empty(lib.hmc_mega_mhc_grad_workspace_bytes(tokens, hidden), dtype=torch.uint8, device=device)
    args = _lib.MegaMhcGradArgs()
    args.tokens, args.hidden = tokens, hidden
    for name, _ in _lib.MegaMhcGradArgs._fields_:  # pylint: disable=protected-access
        if name in tensors:
            setattr(args, name, _lib.ptr(tensors[name]))
    args.workspace = workspace.data_ptr()
    args.workspace_bytes = workspace.numel()
    args.hc_eps, args.num_iters = hc_eps, num_iters
    args.status = _lib.ptr(status)
    _call("hmc_mega_mhc_grad", device, ctypes.byref(args))


# --------------------------------------------------------------------------------- EP transport
def ep_dispatch(tokens, source_of_row, expert_of_row, dispatch_src_off, dispatch_target_off, *, rows, top_k, ep,
                local_experts, capacity_rows, peer_buffers, peer_ctrl, local_ctrl, generation, status=None,
                budget_ns=0, max_ctas=0, row_values=None, value_index=None, value_plane_offset=0) -> None:
    """Push expert-major rows (or gathered token rows) into their owners' receive buffers.

    ``row_values`` (float32) adds one scalar per row, read at ``value_index[j]`` when an index is
    given, and stored in the float plane ``value_plane_offset`` bytes into each owner's buffer.
    """
    device = _require_cuda(tokens, expert_of_row, dispatch_src_off, dispatch_target_off, local_ctrl, row_values,
                           value_index)
    args = _dispatch_struct(tokens, source_of_row, expert_of_row, dispatch_src_off, dispatch_target_off, rows=rows,
                            top_k=top_k, ep=ep, local_experts=local_experts, capacity_rows=capacity_rows,
                            peer_buffers=peer_buffers, peer_ctrl=peer_ctrl, local_ctrl=local_ctrl,
                            generation=generation, status=status, budget_ns=budget_ns, max_ctas=max_ctas,
                            row_values=row_values, value_index=value_index, value_plane_offset=value_plane_offset)
    _call("hmc_ep_dispatch", device, ctypes.byref(args))


def _dispatch_struct(tokens, source_of_row, expert_of_row, dispatch_src_off, dispatch_target_off, *, rows, top_k, ep,
                     local_experts, capacity_rows, peer_buffers, peer_ctrl, local_ctrl, generation, status=None,
                     budget_ns=0, max_ctas=0, row_values=None, value_index=None, value_plane_offset=0, rank=0,
                     send_order_start=None):
    """``hmc_ep_dispatch_args`` from tensors (``rank`` matters only when the dispatch rides inside a GEMM)."""
    if row_values is not None and (row_values.dtype != torch.float32 or not row_values.is_contiguous()):
        raise ValueError("row_values must be a contiguous float32 tensor")
    args = _lib.EpDispatchArgs()
    args.tokens = tokens.data_ptr()
    args.source_of_row = _lib.ptr(source_of_row)
    args.expert_of_row = expert_of_row.data_ptr()
    args.dispatch_src_off = dispatch_src_off.data_ptr()
    args.dispatch_target_off = dispatch_target_off.data_ptr()
    args.rows, args.top_k, args.hidden = rows, top_k, tokens.shape[1]
    args.ep, args.local_experts, args.capacity_rows = ep, local_experts, capacity_rows
    args.peer_buffers = ctypes.cast(peer_buffers, ctypes.c_void_p)
    args.peer_ctrl = ctypes.cast(peer_ctrl, ctypes.c_void_p)
    args.local_ctrl = local_ctrl.data_ptr()
    args.generation, args.max_ctas, args.budget_ns = generation, max_ctas, budget_ns
    args.status = _lib.ptr(status)
    args.row_values, args.value_index = _lib.ptr(row_values), _lib.ptr(value_index)
    args.value_plane_offset = value_plane_offset
    args.rank = rank
    args.send_order_start = _lib.ptr(send_order_start)
    return args


def ep_combine(results, segment_start, combine_target_off, *, rows, ep, local_experts, target_rows_limit,
               peer_buffers, peer_ctrl, local_ctrl, generation, status=None, budget_ns=0, max_ctas=0,
               result_values=None, value_plane_offset=0) -> None:
    """Return result rows (and optionally one float per row) to the routed buffers of their source ranks."""
    device = _require_cuda(results, segment_start, combine_target_off, local_ctrl, result_values)
    if result_values is not None and (result_values.dtype != torch.float32 or not result_values.is_contiguous()):
        raise ValueError("result_values must be a contiguous float32 tensor")
    args = _lib.EpCombineArgs()
    args.results = results.data_ptr()
    args.segment_start = segment_start.data_ptr()
    args.combine_target_off = combine_target_off.data_ptr()
    args.rows, args.hidden, args.ep, args.local_experts = rows, results.shape[1], ep, local_experts
    args.target_rows_limit = target_rows_limit
    args.peer_buffers = ctypes.cast(peer_buffers, ctypes.c_void_p)
    args.peer_ctrl = ctypes.cast(peer_ctrl, ctypes.c_void_p)
    args.local_ctrl = local_ctrl.data_ptr()
    args.generation, args.max_ctas, args.budget_ns = generation, max_ctas, budget_ns
    args.status = _lib.ptr(status)
    args.result_values = _lib.ptr(result_values)
    args.value_plane_offset = value_plane_offset
    _call("hmc_ep_combine", device, ctypes.byref(args))


def ep_publish_source(peer_ctrl, ep: int, rank: int, generation: int, device: torch.device) -> None:
    """Tell every peer that this rank's source buffer holds the rows of ``generation`` (pull dispatch)."""
    _call("hmc_ep_publish_source", device, peer_ctrl, ep, rank, generation)


def ep_pull(out, segment_start, source_row_off, *, rows, ep, local_experts, source_rows_limit, peer_sources,
            local_ctrl, generation, status=None, budget_ns=0, max_ctas=0, out_values=None,
            value_plane_offset=0) -> None:
    """Fetch this rank's rows from the published source buffers of their source ranks."""
    device = _require_cuda(out, segment_start, source_row_off, local_ctrl, out_values)
    args = _lib.EpPullArgs()
    args.peer_sources = ctypes.cast(peer_sources, ctypes.c_void_p)
    args.source_row_off = source_row_off.data_ptr()
    args.segment_start = segment_start.data_ptr()
    args.out = out.data_ptr()
    args.out_values = _lib.ptr(out_values)
    args.rows, args.hidden, args.ep, args.local_experts = rows, out.shape[1], ep, local_experts
    args.source_rows_limit, args.value_plane_offset = source_rows_limit, value_plane_offset
    args.local_ctrl = local_ctrl.data_ptr()
    args.generation, args.max_ctas, args.budget_ns = generation, max_ctas, budget_ns
    args.status = _lib.ptr(status)
    _call("hmc_ep_pull", device, ctypes.byref(args))


def route_guard(table_block: torch.Tensor, ep: int, experts: int, capacity_rows: int, routed_limit: int, status,
                skip_flag: torch.Tensor, host_mirror: torch.Tensor) -> None:
    """Device-side admission check of one expert-parallel call + mirror of table, status words and decision
    to pinned host memory (``hmc_route_guard``)."""
    device = _require_cuda(table_block, skip_flag, status)
    if not host_mirror.is_pinned() or host_mirror.numel() < ep * (experts + 4) + _lib.HMC_STATUS_WORDS + 1:
        raise ValueError("host_mirror must be pinned int32 memory of ep * (experts + 4) + 9 words")
    _call("hmc_route_guard", device, table_block.data_ptr(), ep, experts, capacity_rows, routed_limit, _lib.ptr(status),
          skip_flag.data_ptr(), host_mirror.data_ptr())


def ep_wait(counter: torch.Tensor, expected: int, status=None, budget_ns: int = 0) -> None:
    """Stream-ordered bounded wait until ``counter[0] >= expected``."""
    device = _require_cuda(counter)
    _call("hmc_ep_wait", device, counter.data_ptr(), expected, budget_ns, _lib.ptr(status))


# ---------------------------------------------------------------------------------------- MXFP8
HMC_MXQ_PLAIN, HMC_MXQ_SWIGLU, HMC_MXQ_SWIGLU_GRAD = 0, 1, 2


def mx_pad_blocks(rows: int, groups: int) -> int:
    """Upper bound of the 128-row blocks of the padded expert-major layout."""
    return (rows + 127) // 128 + groups


def _combine_struct(combine: dict):
    fused = _lib.GemmCombine()
    fused.segment_start = combine["segment_start"].data_ptr()
    fused.combine_target_off = combine["combine_target_off"].data_ptr()
    fused.peer_buffers = ctypes.cast(combine["peer_buffers"], ctypes.c_void_p)
    fused.peer_ctrl = ctypes.cast(combine["peer_ctrl"], ctypes.c_void_p)
    fused.ep, fused.local_experts = combine["ep"], combine["local_experts"]
    fused.target_rows_limit = combine["target_rows_limit"]
    return fused


def mx_gemm_combine_units(n: int) -> int:
    """Counter increments per result row of a fused-combine MX GEMM with ``n`` output columns."""
    return int(_lib.load().hmc_mx_gemm_combine_units(n))


def mx_gemm(a, a_scale, b, b_scale, c, group_ends, *, mode, rows, pad_blocks, n, k=0, m=0,
            b_major=HMC_MAJOR_MN, epilogue=HMC_EPI_STORE_BF16, status=None, max_ctas=0, combine=None,
            tile_mode=0, act: "MxActivations | None" = None, aux=None) -> None:
    """Block-scaled FP8 grouped GEMM; see ``hmc_mx_gemm_args`` for the operand layouts. ``combine`` as in
    ``grouped_gemm``: the rows leave the epilogue for their source ranks and ``c`` may be None. ``tile_mode``:
    0 = 256 x 256 CTA-pair tiles where the shape allows, 1 = 128 x 128 tiles, 2 = pairs or an error.
    ``epilogue=HMC_EPI_SWIGLU_MXQ``: ``c`` = U [rows, n] and ``act`` (an ``MxActivations`` of width n / 2 with both
    axes) receives the quantised bf16(silu(gate) * up). ``epilogue=HMC_EPI_SWIGLU_GRAD_MXQ``: the accumulator is
    dAct [rows, n], ``aux`` = the saved U [rows, 2n], ``act`` (width 2n) receives the quantised dU and ``c`` (dAct)
    may be None."""
    device = _require_cuda(a, a_scale, b, b_scale, c, group_ends, status)
    args = _lib.MxGemmArgs()
    args.mode, args.b_major, args.epilogue = mode, b_major, epilogue
    args.groups, args.max_ctas, args.tile_mode = group_ends.numel(), max_ctas, tile_mode
    args.rows, args.pad_blocks, args.m, args.n, args.k = rows, pad_blocks, m, n, k
    args.a, args.a_scale = a.data_ptr(), a_scale.data_ptr()
    args.b, args.b_scale = b.data_ptr(), b_scale.data_ptr()
    args.c = _lib.ptr(c)
    args.group_ends = group_ends.data_ptr()
    args.status = _lib.ptr(status)
    if act is not None:
        args.act_row_data, args.act_row_scale = act.row_data.data_ptr(), act.row_scale.data_ptr()
        args.act_col_data, args.act_col_scale = _lib.ptr(act.col_data), _lib.ptr(act.col_scale)
    args.aux = _lib.ptr(aux)
    fused = None
    if combine is not None:
        fused = _combine_struct(combine)
        args.combine = ctypes.cast(ctypes.pointer(fused), ctypes.c_void_p)
    _call("hmc_mx_gemm", device, ctypes.byref(args))


def ep_wait_groups(counters: torch.Tensor, group_ends: torch.Tensor, status=None, budget_ns: int = 0) -> None:
    """Stream-ordered bounded wait until every group's arrival counter covers its rows."""
    device = _require_cuda(counters, group_ends)
    _call("hmc_ep_wait_groups", device, counters.data_ptr(), group_ends.data_ptr(), group_ends.numel(), budget_ns,
          _lib.ptr(status))


class MxActivations:
    """Quantised activations in the padded expert-major layout (see ``hmc_mx_quant_args``)."""

    def __init__(self, rows: int, groups: int, width: int, device, *, want_row: bool, want_col: bool) -> None:
        self.rows, self.width = rows, width
        self.pad_blocks = mx_pad_blocks(rows, groups)
        u8 = dict(dtype=torch.uint8, device=device)
        pad_rows = self.pad_blocks * 128
        atoms = self.pad_blocks * (width // 128) * 512
        self.row_data = torch.empty((pad_rows, width), **u8) if want_row else None
        self.row_scale = torch.empty(atoms, **u8) if want_row else None
        self.col_data = torch.empty((pad_rows, width), **u8) if want_col else None
        self.col_scale = torch.empty(atoms, **u8) if want_col else None


def mx_quant(src, group_ends, width, *, kind=HMC_MXQ_PLAIN, aux=None, want_row=True, want_col=False,
             dense=None) -> MxActivations:
    """Quantise expert-major BF16 rows (optionally through SwiGLU / SwiGLU-grad) to MXFP8."""
    device = _require_cuda(src, group_ends, aux, dense)
    rows, groups = src.shape[0], group_ends.numel()
    out = MxActivations(rows, groups, width, device, want_row=want_row, want_col=want_col)
    args = _lib.MxQuantArgs()
    args.kind, args.groups = kind, groups
    args.rows, args.pad_blocks, args.width = rows, out.pad_blocks, width
    args.src, args.aux, args.group_ends = src.data_ptr(), _lib.ptr(aux), group_ends.data_ptr()
    args.row_data, args.row_scale = _lib.ptr(out.row_data), _lib.ptr(out.row_scale)
    args.col_data, args.col_scale = _lib.ptr(out.col_data), _lib.ptr(out.col_scale)
    args.dense = _lib.ptr(dense)
    _call("hmc_mx_quant", device, ctypes.byref(args))
    return out


def mx_quant_weight(weight: torch.Tensor, *, want_col: bool = True, want_row: bool = True) -> dict:
    """BF16 weight [e, m, n] -> the reference's physical MX fields (col_* blocks along m, row_* along n)."""
    device = _require_cuda(weight)
    experts, m, n = weight.shape
    weight = weight.contiguous()
    out = {}
    if want_col:
        out["col_data"] = torch.empty((experts, m, n), dtype=torch.float8_e4m3fn, device=device)
        out["col_scale"] = torch.empty((experts, m // 64, n, 2), dtype=torch.uint8, device=device)
    if want_row:
        out["row_data"] = torch.empty((experts, m, n), dtype=torch.float8_e4m3fn, device=device)
        out["row_scale"] = torch.empty((experts, m, n // 64, 2), dtype=torch.uint8, device=device)
    _call("hmc_mx_quant_weight", device, weight.data_ptr(), experts, m, n, _lib.ptr(out.get("col_data")),
          _lib.ptr(out.get("col_scale")), _lib.ptr(out.get("row_data")), _lib.ptr(out.get("row_scale")))
    return out


def mx_pack_weight_scale(scale: torch.Tensor, axis: int, experts: int, m: int, n: int) -> torch.Tensor:
    """Reference scale tensor (col_scale: axis 0, row_scale: axis 1) -> scale-factor atoms for the GEMM."""
    device = _require_cuda(scale)
    atoms = torch.empty(experts * m * n // 32, dtype=torch.uint8, device=device)
    _call("hmc_mx_pack_weight_scale", device, scale.data_ptr(), axis, experts, m, n, atoms.data_ptr())
    return atoms
