"""Operator-level wrappers with the names, argument order and allocation rules of the reference's
``hyper_multicore/torch/ops.py`` (the drop-in boundary of the module layer).

Each function validates like the reference's C++ binding did (contiguity, dtype, device, extents),
allocates exactly the outputs the reference wrapper allocated, and launches through the C ABI.
``runtime_config``, ``all_event_counters`` and ``diagnostic_buffer`` are accepted and ignored:
tiles are scheduled on the device, so there is no serialised host schedule to pass.
"""

from __future__ import annotations

import ctypes
import math
from dataclasses import dataclass
from typing import Any

import torch

from . import _lib, kernels

_MHC_STREAMS = 4


def _check(condition: bool, message: str) -> None:
    """TORCH_CHECK equivalent: the reference's bindings raise RuntimeError."""
    if not condition:
        raise RuntimeError(message)


def _check_cuda_contiguous(name: str, tensor: torch.Tensor, dtype=None) -> None:
    _check(isinstance(tensor, torch.Tensor), f"{name} must be a Tensor")
    _check(tensor.is_cuda, f"{name} must be a CUDA tensor")
    _check(tensor.is_contiguous(), f"{name} must be contiguous")
    if dtype is not None:
        _check(tensor.dtype == dtype, f"{name} must have dtype {dtype}, got {tensor.dtype}")


def mega_moe_transport_version() -> int:
    """reference: torch/csrc/registration.cpp:21."""
    from . import _lib

    return _lib.load().hmc_mega_moe_transport_version()


def worker_queue_layout_version() -> int:
    """reference: torch/csrc/registration.cpp:22."""
    from . import _lib

    return _lib.load().hmc_worker_queue_layout_version()


# --------------------------------------------------------------------------------------- MegaGate
def _mega_gate_route(logits, text_bias, vision_bias, image_mask, runtime_config=None, diagnostic_buffer=None, *,
                     top_k: int, routed_scaling_factor: float, use_vision_bias: bool, scoring_func: str = "sqrtsoftplus",
                     diagnostics=None):
    """reference: torch/ops.py:954-1012, checks torch/csrc/mega_gate.cpp:40-61.

    Returns (weights [T,K] f32, indices [T,K] i64, route_scores [T,E] f32, selected [T,K] f32,
    denominator [T,1] f32). ``scoring_func`` extends the native op to softmax and sigmoid.
    """
    del runtime_config, diagnostic_buffer, diagnostics
    _check_cuda_contiguous("logits", logits, torch.float32)
    _check(logits.ndim == 2 and logits.shape[0] > 0, "logits must be a non-empty [tokens, experts] tensor")
    tokens, experts = logits.shape
    for name, bias in (("text_bias", text_bias), ("vision_bias", vision_bias)):
        _check_cuda_contiguous(name, bias, torch.float32)
        _check(tuple(bias.shape) == (experts,) and bias.device == logits.device, f"{name} must be [experts] on the logits device")
    _check(1 <= top_k <= experts, "top_k must be in [1, expert_count]")
    _check(math.isfinite(routed_scaling_factor), "routed_scaling_factor must be finite")
    _check(not logits.requires_grad, "mega_gate_route does not record autograd; use MegaGate")
    if use_vision_bias:
        _check_cuda_contiguous("image_mask", image_mask, torch.bool)
        _check(image_mask.numel() == tokens, "image_mask must have one entry per token")
    from .modules.mega_gate import route

    return route(logits, text_bias, vision_bias, image_mask if use_vision_bias else None, bool(use_vision_bias),
                 int(top_k), float(routed_scaling_factor), scoring_func)


def _mega_gate_route_grad(logits, route_scores, selected_scores, normalization_denominator, expert_indices,
                          grad_routing_weights, runtime_config=None, diagnostic_buffer=None, *, top_k: int,
                          routed_scaling_factor: float, scoring_func: str = "sqrtsoftplus") -> torch.Tensor:
    """reference: torch/ops.py:1015-1044, checks torch/csrc/mega_gate.cpp:132-176."""
    del runtime_config, diagnostic_buffer
    tokens, experts = logits.shape
    _check_cuda_contiguous("logits", logits, torch.float32)
    _check_cuda_contiguous("route_scores", route_scores, torch.float32)
    _check_cuda_contiguous("selected_scores", selected_scores, torch.float32)
    _check_cuda_contiguous("normalization_denominator", normalization_denominator, torch.float32)
    _check_cuda_contiguous("expert_indices", expert_indices, torch.int64)
    _check_cuda_contiguous("grad_routing_weights", grad_routing_weights, torch.float32)
    _check(tuple(route_scores.shape) == (tokens, experts), "route_scores must match logits")
    _check(tuple(selected_scores.shape) == (tokens, top_k) and tuple(expert_indices.shape) == (tokens, top_k)
           and tuple(grad_routing_weights.shape) == (tokens, top_k), "top-k tensors must be [tokens, top_k]")
    _check(normalization_denominator.numel() == tokens, "normalization_denominator must be [tokens, 1]")
    grad_logits = torch.empty_like(logits)
    kernels.gate_route_grad_out(logits, route_scores, selected_scores, normalization_denominator, expert_indices,
                                grad_routing_weights, int(top_k), float(routed_scaling_factor), scoring_func, grad_logits)
    return grad_logits


# ------------------------------------------------------------------------------ MoE row helpers
def moe_token_permute_out(tokens, indices, output, mapping) -> None:
    """reference: torch/ops.py:493-509, checks torch/csrc/moe_token_permute_out.cpp:25-48.

    ``output[mapping[t * K + k]] = tokens[t]`` with rows expert-major, stable by flat index.
    """
    _check_cuda_contiguous("tokens", tokens)
    _check_cuda_contiguous("indices", indices)
    _check_cuda_contiguous("output", output, tokens.dtype)
    _check_cuda_contiguous("mapping", mapping, torch.int32)
    _check(tokens.ndim == 2 and indices.ndim == 2 and indices.shape[0] == tokens.shape[0], "indices must be [tokens, top_k]")
    _check(indices.dtype in (torch.int32, torch.int64), "indices must be INT32 or INT64")
    rows = indices.numel()
    _check(tuple(output.shape) == (rows, tokens.shape[1]) and mapping.numel() == rows,
           "output must be [tokens * top_k, hidden] and mapping [tokens * top_k]")
    _check(output.data_ptr() != tokens.data_ptr(), "output must not overlap tokens")
    experts = int(indices.max().item()) + 1 if rows else 1
    result, sources, _, _, _ = kernels.moe_sort_routes(indices, experts)
    mapping.copy_(result)
    if rows:
        kernels.moe_gather_rows(tokens, sources, indices.shape[1], output)


def moe_token_permute_from_mapping_out(tokens, mapping, probabilities, output, output_probabilities) -> None:
    """reference: torch/ops.py:512-528 (utilities.asc:162-209): bit-preserving expansion through an existing map."""
    _check_cuda_contiguous("tokens", tokens)
    _check_cuda_contiguous("mapping", mapping, torch.int32)
    _check_cuda_contiguous("probabilities", probabilities, torch.float32)
    _check_cuda_contiguous("output", output, tokens.dtype)
    _check_cuda_contiguous("output_probabilities", output_probabilities, torch.float32)
    top_k = mapping.numel() // max(tokens.shape[0], 1)
    _check(mapping.numel() == tokens.shape[0] * top_k and probabilities.numel() == mapping.numel(),
           "mapping and probabilities must hold tokens * top_k entries")
    _check(output.shape[0] == mapping.numel() and output_probabilities.numel() == mapping.numel(),
           "outputs must have tokens * top_k rows")
    kernels.moe_permute_from_mapping(tokens, mapping, probabilities, top_k, output, output_probabilities)


def mega_moe_unpermute_grad_out(permuted_tokens, grad_output, sorted_indices, probs, grad_permuted, grad_probs) -> None:
    """reference: torch/ops.py:531-551 (torch/csrc/mega_moe_unpermute.cpp:56-65)."""
    for name, tensor in (("permuted_tokens", permuted_tokens), ("grad_output", grad_output), ("grad_permuted", grad_permuted)):
        _check_cuda_contiguous(name, tensor, torch.bfloat16)
    _check_cuda_contiguous("sorted_indices", sorted_indices, torch.int32)
    _check_cuda_contiguous("probs", probs, torch.float32)
    _check_cuda_contiguous("grad_probs", grad_probs, torch.float32)
    top_k = probs.shape[-1]
    _check(sorted_indices.numel() == grad_output.shape[0] * top_k, "sorted_indices must hold tokens * top_k entries")
    kernels.moe_unpermute_grad(permuted_tokens, grad_output, sorted_indices, probs, top_k, grad_permuted, grad_probs)


def moe_token_permute_grad(grad_permuted_tokens, sorted_indices, num_tokens: int, top_k: int) -> torch.Tensor:
    """reference: torch/ops.py:931-951 (torch/csrc/moe_token_permute_grad.cpp:29-38). Returns owned [T, H]."""
    _check_cuda_contiguous("grad_permuted_tokens", grad_permuted_tokens, torch.bfloat16)
    _check_cuda_contiguous("sorted_indices", sorted_indices, torch.int32)
    _check(sorted_indices.numel() == num_tokens * top_k, "sorted_indices must hold num_tokens * top_k entries")
    out = torch.empty((num_tokens, grad_permuted_tokens.shape[1]), dtype=grad_permuted_tokens.dtype,
                      device=grad_permuted_tokens.device)
    kernels.moe_token_permute_grad(grad_permuted_tokens, sorted_indices, num_tokens, top_k, out)
    return out


def zero_empty_expert_gradients(first, second, cumulative_groups) -> None:
    """reference: torch/ops.py:1047-1057 (torch/csrc/mega_moe_utilities.cpp:64-92)."""
    _check_cuda_contiguous("first", first)
    _check_cuda_contiguous("second", second)
    _check_cuda_contiguous("cumulative_groups", cumulative_groups, torch.int64)
    _check(first.shape[0] == cumulative_groups.numel() == second.shape[0], "one gradient slice per local expert")
    kernels.zero_empty_expert_grad(first, second, cumulative_groups)


def route_offsets(counts, rank: int, ub_bytes: int = 0, hidden_size: int = 1) -> dict:
    """reference: torch/ops.py:1060-1064 (utilities.asc:89-151). Returns the named row-unit descriptors
    (the reference packs them into two flat tensors); ``hidden_size`` > 1 adds element-unit copies."""
    del ub_bytes
    _check_cuda_contiguous("counts", counts, torch.int32)
    _check(counts.ndim == 2 and counts.shape[1] % counts.shape[0] == 0, "counts must be [ep, experts]")
    rows = kernels.route_offsets(counts, int(rank))
    if hidden_size != 1:
        for name in ("dispatch_src_off", "dispatch_target_off", "dispatch_size", "combine_src_off",
                     "combine_target_off", "combine_size"):
            rows[name + "_elements"] = rows[name] * hidden_size
    return rows


# -------------------------------------------------------------------------------- MegaMoE operators
@dataclass
class MoeTransport:
    """Peer-mapped endpoints of one expert-parallel group member (``hmc_moe_transport``): what the
    reference keeps in its symmetric workspace (hyper_multicore/modules/mega_moe/workspace.py:48-75)."""

    ep: int
    rank: int
    peer_dispatch: Any            # ctypes array of ep pointers: receive (pull: source) buffer of every rank
    peer_combine: Any | None      # ctypes array of ep pointers: routed buffer of every rank
    peer_ctrl: Any                # ctypes array of ep pointers: control blocks
    dispatch_rows_limit: int
    combine_rows_limit: int = 0
    dispatch_plane_offset: int = 0
    combine_plane_offset: int = 0
    generation: int = 0
    dispatch_mode: str = "push"
    wait_budget_ns: int = 0
    copy_stream: torch.cuda.Stream | None = None

    def as_struct(self) -> "_lib.MoeTransport":
        out = _lib.MoeTransport()
        out.ep, out.rank = self.ep, self.rank
        out.peer_dispatch = ctypes.cast(self.peer_dispatch, ctypes.c_void_p)
        out.peer_combine = ctypes.cast(self.peer_combine, ctypes.c_void_p) if self.peer_combine is not None else None
        out.peer_ctrl = ctypes.cast(self.peer_ctrl, ctypes.c_void_p)
        out.dispatch_rows_limit, out.combine_rows_limit = self.dispatch_rows_limit, self.combine_rows_limit
        out.dispatch_plane_offset, out.combine_plane_offset = self.dispatch_plane_offset, self.combine_plane_offset
        out.generation = self.generation
        out.dispatch_mode = _lib.HMC_MOE_DISPATCH[self.dispatch_mode]
        out.wait_budget_ns = self.wait_budget_ns
        out.copy_stream = self.copy_stream.cuda_stream if self.copy_stream is not None else None
        return out


@dataclass
class MegaMoeLaunch:
    """What the reference encodes in its tiling tensors, workspaces and RuntimeConfig blobs, as plain fields:
    shapes, layout, numerics, the route tensors the device-side scheduling reads, the owned copies and the
    optional token-order prologue / epilogue (see ``hmc_mega_moe_args`` / ``hmc_mega_moe_grad_args``)."""

    transport: MoeTransport
    intermediate_size: int
    top_k: int
    routed_rows: int
    received_rows: int
    weight_layout: str = "EIO"
    swiglu_clamp: int = 0
    swiglu_limit: float = 0.0
    fuse_dispatch: bool = True
    probs_before_fc2: bool = False
    status: torch.Tensor | None = None
    dispatch_src_index: torch.Tensor | None = None
    expert_of_row: torch.Tensor | None = None
    recv_segment_start: torch.Tensor | None = None
    send_order_start: torch.Tensor | None = None
    mapping: torch.Tensor | None = None
    topk_probs: torch.Tensor | None = None
    # forward
    route_probs: torch.Tensor | None = None
    row_probs: torch.Tensor | None = None
    saved_dispatch: torch.Tensor | None = None
    saved_combine: torch.Tensor | None = None
    saved_row_probs: torch.Tensor | None = None
    output: torch.Tensor | None = None
    skip_flag: torch.Tensor | None = None
    # backward
    weight_grad_f32: bool = False
    row_dot: torch.Tensor | None = None
    grad_output: torch.Tensor | None = None
    grad_probs: torch.Tensor | None = None
    grad_hidden: torch.Tensor | None = None
    # MXFP8
    pad_blocks: int = 0


def _ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def _check_rows(name: str, tensor: torch.Tensor | None, width: int, dtype=torch.bfloat16) -> None:
    if tensor is None:
        return
    _check_cuda_contiguous(name, tensor, dtype)
    _check(tensor.ndim == 2 and tensor.shape[1] == width, f"{name} must be [rows, {width}], got {tuple(tensor.shape)}")


def _launch_native(name: str, args, device: torch.device, launches: int) -> None:
    del launches  # counted by the native library itself
    with torch.cuda.device(device):
        _lib.check(getattr(_lib.load(), name)(ctypes.byref(args), _lib.stream_ptr(device)))


def mega_moe(dispatch_target, dispatch_target_off, dispatch_src, dispatch_src_off, dispatch_size, up_proj_weight,
             up_proj_glist, up_proj_y, swiglu_out, down_proj_weight, down_proj_glist, down_proj_y, combine_target,
             combine_target_off, combine_src_off, combine_size, gmm_workspace, up_proj_tiling, swiglu_tiling,
             down_proj_tiling, runtime_config, all_event_counters, rank_id: int, ep: int, expert_num: int,
             hidden_size: int, seq_size: int, *, launch: MegaMoeLaunch) -> None:
    """MoE-FFN forward operator; reference: torch/ops.py:554-649 (schema torch/csrc/registration.cpp:30-60).

    Writes in place to dispatch_target, up_proj_y, swiglu_out, down_proj_y (one rank) or combine_target
    (expert parallel); every buffer is the caller's. ``gmm_workspace``, the tiling tensors and
    ``runtime_config`` are accepted and not read; ``launch`` carries their content as plain fields.
    Offsets are in rows.
    """
    del gmm_workspace, up_proj_tiling, swiglu_tiling, down_proj_tiling, runtime_config
    inter = launch.intermediate_size
    _check_rows("dispatch_target", dispatch_target, hidden_size)
    _check_rows("dispatch_src", dispatch_src, hidden_size)
    _check_rows("up_proj_y", up_proj_y, 2 * inter)
    _check_rows("swiglu_out", swiglu_out, inter)
    _check_rows("down_proj_y", down_proj_y, hidden_size)
    _check_rows("combine_target", combine_target, hidden_size)
    for name, weight in (("up_proj_weight", up_proj_weight), ("down_proj_weight", down_proj_weight)):
        _check_cuda_contiguous(name, weight, torch.bfloat16)
    _check_cuda_contiguous("up_proj_glist", up_proj_glist, torch.int64)
    _check(up_proj_glist.numel() == expert_num // ep, "up_proj_glist must hold one cumulative count per local expert")
    _check(down_proj_glist is up_proj_glist or down_proj_glist.data_ptr() == up_proj_glist.data_ptr(),
           "both projections walk the same group list")
    _check_cuda_contiguous("all_event_counters", all_event_counters, torch.int32)
    rows = max(launch.received_rows, 1)
    _check(up_proj_y.shape[0] >= rows and swiglu_out.shape[0] >= rows and dispatch_target.shape[0] >= rows,
           "dispatch_target, up_proj_y and swiglu_out must hold the received rows")
    args = _lib.MegaMoeArgs()
    transport = launch.transport.as_struct()
    args.dispatch_target, args.dispatch_target_off = _ptr(dispatch_target), _ptr(dispatch_target_off)
    args.dispatch_src, args.dispatch_src_off, args.dispatch_size = _ptr(dispatch_src), _ptr(dispatch_src_off), _ptr(dispatch_size)
    args.up_proj_weight, args.up_proj_glist = _ptr(up_proj_weight), _ptr(up_proj_glist)
    args.up_proj_y, args.swiglu_out = _ptr(up_proj_y), _ptr(swiglu_out)
    args.down_proj_weight, args.down_proj_glist, args.down_proj_y = _ptr(down_proj_weight), _ptr(down_proj_glist), _ptr(down_proj_y)
    args.combine_target, args.combine_target_off = _ptr(combine_target), _ptr(combine_target_off)
    args.combine_src_off, args.combine_size = _ptr(combine_src_off), _ptr(combine_size)
    args.all_event_counters, args.diagnostic_buffer = _ptr(all_event_counters), _ptr(launch.status)
    args.rank_id, args.ep, args.expert_num, args.hidden_size, args.seq_size = rank_id, ep, expert_num, hidden_size, seq_size
    args.intermediate_size, args.top_k = inter, launch.top_k
    args.routed_rows, args.received_rows = launch.routed_rows, launch.received_rows
    args.weight_layout = _lib.HMC_MOE_LAYOUT[launch.weight_layout]
    args.swiglu_clamp, args.swiglu_limit = launch.swiglu_clamp, launch.swiglu_limit
    args.fuse_dispatch, args.probs_before_fc2 = int(launch.fuse_dispatch), int(launch.probs_before_fc2)
    args.dispatch_src_index, args.expert_of_row = _ptr(launch.dispatch_src_index), _ptr(launch.expert_of_row)
    args.recv_segment_start, args.send_order_start = _ptr(launch.recv_segment_start), _ptr(launch.send_order_start)
    args.route_probs, args.row_probs = _ptr(launch.route_probs), _ptr(launch.row_probs)
    args.transport = ctypes.cast(ctypes.pointer(transport), ctypes.c_void_p)
    args.saved_dispatch, args.saved_combine = _ptr(launch.saved_dispatch), _ptr(launch.saved_combine)
    args.saved_row_probs = _ptr(launch.saved_row_probs)
    args.mapping, args.topk_probs, args.output = _ptr(launch.mapping), _ptr(launch.topk_probs), _ptr(launch.output)
    args.skip_flag = _ptr(launch.skip_flag)
    _launch_native("hmc_mega_moe", args, dispatch_target.device, 6)


def mega_moe_grad(dispatch_target, dispatch_target_off, dy, dispatch_src_off, dispatch_size, hidden, hidden_dw, w2,
                  act_grad_y, gate, grad_gate, w1, gate_dx, grad_x, combine_target_off, combine_src_off, combine_size,
                  permute_out, gate_dw, group_list, act_grad_tiling, gate_grad_tiling, w1_grad_tiling, w2_grad_tiling,
                  swiglu_grad_tiling, gmm_workspace, swiglu_grad_workspace, runtime_config, all_event_counters,
                  rank_id: int, ep: int, expert_num: int, hidden_size: int, seq_size: int, *,
                  launch: MegaMoeLaunch) -> None:
    """MoE-FFN backward operator; reference: torch/ops.py:652-737 (schema torch/csrc/registration.cpp:70-107).

    ``hidden`` is the saved SwiGLU output, ``gate`` the saved up-projection, ``permute_out`` the saved received
    rows; writes hidden_dw (dW2), grad_gate (dU), gate_dx (dX rows, one rank) or grad_x (combine target),
    gate_dw (dW1). ``act_grad_y`` is accepted and not written: the activation gradient stays in the accumulator
    of the fused SwiGLU-grad epilogue. Tiling tensors, workspaces and ``runtime_config`` are not read.
    """
    del act_grad_y, act_grad_tiling, gate_grad_tiling, w1_grad_tiling, w2_grad_tiling, swiglu_grad_tiling
    del gmm_workspace, swiglu_grad_workspace, runtime_config
    inter = launch.intermediate_size
    _check_rows("dispatch_target", dispatch_target, hidden_size)
    _check_rows("dy", dy, hidden_size)
    _check_rows("hidden", hidden, inter)
    _check_rows("gate", gate, 2 * inter)
    _check_rows("grad_gate", grad_gate, 2 * inter)
    _check_rows("gate_dx", gate_dx, hidden_size)
    _check_rows("grad_x", grad_x, hidden_size)
    _check_rows("permute_out", permute_out, hidden_size)
    for name, weight in (("w1", w1), ("w2", w2)):
        _check_cuda_contiguous(name, weight, torch.bfloat16)
    grad_dtype = torch.float32 if launch.weight_grad_f32 else torch.bfloat16
    for name, grad in (("hidden_dw", hidden_dw), ("gate_dw", gate_dw)):
        if grad is not None:
            _check_cuda_contiguous(name, grad, grad_dtype)
    _check(hidden_dw is None or hidden_dw.shape == w2.shape, "hidden_dw must have the shape of w2")
    _check(gate_dw is None or gate_dw.shape == w1.shape, "gate_dw must have the shape of w1")
    _check_cuda_contiguous("group_list", group_list, torch.int64)
    _check_cuda_contiguous("all_event_counters", all_event_counters, torch.int32)
    args = _lib.MegaMoeGradArgs()
    transport = launch.transport.as_struct()
    args.dispatch_target, args.dispatch_target_off = _ptr(dispatch_target), _ptr(dispatch_target_off)
    args.dy, args.dispatch_src_off, args.dispatch_size = _ptr(dy), _ptr(dispatch_src_off), _ptr(dispatch_size)
    args.hidden, args.hidden_dw, args.w2 = _ptr(hidden), _ptr(hidden_dw), _ptr(w2)
    args.gate, args.grad_gate, args.w1 = _ptr(gate), _ptr(grad_gate), _ptr(w1)
    args.gate_dx, args.grad_x = _ptr(gate_dx), _ptr(grad_x)
    args.combine_target_off, args.combine_src_off, args.combine_size = _ptr(combine_target_off), _ptr(combine_src_off), _ptr(combine_size)
    args.permute_out, args.gate_dw, args.group_list = _ptr(permute_out), _ptr(gate_dw), _ptr(group_list)
    args.all_event_counters, args.diagnostic_buffer = _ptr(all_event_counters), _ptr(launch.status)
    args.rank_id, args.ep, args.expert_num, args.hidden_size, args.seq_size = rank_id, ep, expert_num, hidden_size, seq_size
    args.intermediate_size, args.top_k = inter, launch.top_k
    args.routed_rows, args.received_rows = launch.routed_rows, launch.received_rows
    args.weight_layout = _lib.HMC_MOE_LAYOUT[launch.weight_layout]
    args.swiglu_clamp, args.swiglu_limit = launch.swiglu_clamp, launch.swiglu_limit
    args.fuse_dispatch, args.weight_grad_f32 = int(launch.fuse_dispatch), int(launch.weight_grad_f32)
    args.probs_before_fc2 = int(launch.probs_before_fc2)
    args.dispatch_src_index, args.expert_of_row = _ptr(launch.dispatch_src_index), _ptr(launch.expert_of_row)
    args.recv_segment_start, args.send_order_start = _ptr(launch.recv_segment_start), _ptr(launch.send_order_start)
    args.row_probs, args.row_dot = _ptr(launch.row_probs), _ptr(launch.row_dot)
    args.transport = ctypes.cast(ctypes.pointer(transport), ctypes.c_void_p)
    args.grad_output, args.saved_combine = _ptr(launch.grad_output), _ptr(launch.saved_combine)
    args.mapping, args.topk_probs = _ptr(launch.mapping), _ptr(launch.topk_probs)
    args.grad_probs, args.grad_hidden = _ptr(launch.grad_probs), _ptr(launch.grad_hidden)
    _launch_native("hmc_mega_moe_grad", args, dy.device, 9)


def mega_moe_mxfp8_abi_version() -> int:
    """reference: torch/csrc/mega_moe_mxfp8.cpp (the loader asserts version 3)."""
    return _lib.load().hmc_mega_moe_mxfp8_abi_version()


_MX_FORWARD_BUFFERS = (
    "dispatch_buffer", "dispatch_target_off", "source_buffer", "dispatch_src_off", "dispatch_size", "w1_col_data",
    "group_list", "up", "a_row", "w2_col_data", "group_list2", "down", "routed_buffer", "combine_target_off",
    "combine_src_off", "combine_size", "x_row", "x_scale", "x_col", "x_col_scale", "a_scale", "a_col", "a_col_scale",
    "w1_col_scale", "w2_col_scale")
_MX_BACKWARD_BUFFERS = (
    "dispatch", "dispatch_target_off", "source", "dispatch_src_off", "dispatch_size", "a_col", "dw2", "w2_row_data", "da",
    "up", "du_row", "w1_row_data", "dx", "routed_buffer", "combine_target_off", "combine_src_off", "combine_size", "x_col",
    "dw1", "group_list", "dy_row", "dy_scale", "dy_col", "dy_col_scale", "a_col_scale", "w2_row_scale", "du_scale",
    "du_col", "du_col_scale", "w1_row_scale", "x_col_scale")


def _mx_common(args, launch: MegaMoeLaunch, events, rank_id, ep, expert_num, hidden_size, seq_size):
    transport = launch.transport.as_struct()
    args.all_event_counters, args.diagnostic_buffer = _ptr(events), _ptr(launch.status)
    args.rank_id, args.ep, args.expert_num, args.hidden_size, args.seq_size = rank_id, ep, expert_num, hidden_size, seq_size
    args.intermediate_size, args.top_k = launch.intermediate_size, launch.top_k
    args.routed_rows, args.received_rows, args.pad_blocks = launch.routed_rows, launch.received_rows, launch.pad_blocks
    args.expert_of_row, args.recv_segment_start = _ptr(launch.expert_of_row), _ptr(launch.recv_segment_start)
    args.transport = ctypes.cast(ctypes.pointer(transport), ctypes.c_void_p)
    args.saved_combine = _ptr(launch.saved_combine)
    args.mapping, args.topk_probs = _ptr(launch.mapping), _ptr(launch.topk_probs)
    args.skip_flag = _ptr(launch.skip_flag)
    return transport  # kept alive by the caller until the native call returns


def mega_moe_mxfp8(buffers, runtime_config, events, diagnostic, launch_metadata, *, rank_id: int, ep: int,
                   expert_num: int, hidden_size: int, seq_size: int, launch: MegaMoeLaunch) -> None:
    """MXFP8 MoE-FFN forward operator; reference schema torch/csrc/mega_moe_mxfp8.cpp:36-42. ``buffers`` is the
    reference's list in its order (backends/mxfp8/execution.py:88-96; the two trailing plan tensors may be
    omitted; weight scales are scale-factor atoms). ``runtime_config`` and ``launch_metadata`` are not read."""
    del runtime_config, diagnostic, launch_metadata
    _check(len(buffers) >= len(_MX_FORWARD_BUFFERS), f"mega_moe_mxfp8 takes {len(_MX_FORWARD_BUFFERS)} buffers")
    args = _lib.MegaMoeMxfp8Args()
    device = None
    for name, tensor in zip(_MX_FORWARD_BUFFERS, buffers):
        if tensor is not None:
            _check(tensor.is_cuda and tensor.is_contiguous(), f"{name} must be a contiguous CUDA tensor")
            device = tensor.device
        setattr(args, name, _ptr(tensor))
    keep = _mx_common(args, launch, events, rank_id, ep, expert_num, hidden_size, seq_size)
    args.dispatch_src_index, args.output = _ptr(launch.dispatch_src_index), _ptr(launch.output)
    _launch_native("hmc_mega_moe_mxfp8", args, device, 7)
    del keep


def mega_moe_mxfp8_grad(buffers, runtime_config, events, diagnostic, launch_metadata, *, rank_id: int, ep: int,
                        expert_num: int, hidden_size: int, seq_size: int, launch: MegaMoeLaunch) -> None:
    """MXFP8 MoE-FFN backward operator; ``buffers`` in the order of backends/mxfp8/execution.py:147-155."""
    del runtime_config, diagnostic, launch_metadata
    _check(len(buffers) >= len(_MX_BACKWARD_BUFFERS), f"mega_moe_mxfp8_grad takes {len(_MX_BACKWARD_BUFFERS)} buffers")
    args = _lib.MegaMoeMxfp8GradArgs()
    device = None
    for name, tensor in zip(_MX_BACKWARD_BUFFERS, buffers):
        if tensor is not None:
            _check(tensor.is_cuda and tensor.is_contiguous(), f"{name} must be a contiguous CUDA tensor")
            device = tensor.device
        setattr(args, name, _ptr(tensor))
    keep = _mx_common(args, launch, events, rank_id, ep, expert_num, hidden_size, seq_size)
    args.weight_grad_f32 = int(launch.weight_grad_f32)
    args.grad_output, args.grad_probs, args.grad_hidden = _ptr(launch.grad_output), _ptr(launch.grad_probs), _ptr(launch.grad_hidden)
    _launch_native("hmc_mega_moe_mxfp8_grad", args, device, 11)
    del keep


# ------------------------------------------------------------------------------------------- mHC
def _allocate_hyper_mega_mhc_forward_cache(residual: torch.Tensor, num_iters: int):
    """The six backward intermediates in the reference's order (torch/ops.py:230-268)."""
    batch, sequence, streams, hidden = residual.shape
    mix = streams * streams + 2 * streams
    f32 = dict(dtype=torch.float32, device=residual.device)
    return (torch.empty((batch, sequence, mix), **f32), torch.empty((batch, sequence, 1), **f32),
            torch.empty((2 * num_iters, batch, sequence, streams), **f32),
            torch.empty((2 * num_iters, batch, sequence, streams, streams), **f32),
            torch.empty((batch, sequence, hidden), dtype=residual.dtype, device=residual.device),
            torch.empty((batch, sequence, 1), **f32))


def hyper_mega_mhc(previous_output, residual, previous_pre_mix, previous_post_mix, previous_residual_mix, phi, alpha,
                   bias, norm_weight, runtime_config=None, all_event_counters=None, diagnostic_buffer=None, *,
                   hc_eps: float = 1e-6, norm_eps: float = 1e-6, num_iters: int = 20, need_backward: bool,
                   diagnostics=None):
    """reference: torch/ops.py:270-369. BSND inputs; returns the five outputs followed by the six caches."""
    del runtime_config, all_event_counters, diagnostic_buffer, diagnostics
    if residual.ndim != 4:
        raise ValueError(f"residual must be BSND [B, S, 4, H], got {tuple(residual.shape)}.")
    batch, sequence, streams, hidden = residual.shape
    _check(streams == _MHC_STREAMS, "residual must have four streams")
    f32 = dict(dtype=torch.float32, device=residual.device)
    new_residual = torch.empty_like(residual)
    next_pre = torch.empty((batch, sequence, streams), **f32)
    next_post = torch.empty_like(next_pre)
    next_mix = torch.empty((batch, sequence, streams * streams), **f32)
    block_input = torch.empty((batch, sequence, hidden), dtype=residual.dtype, device=residual.device)
    cache = _allocate_hyper_mega_mhc_forward_cache(residual, num_iters)
    inputs = [t.contiguous() for t in (previous_output, residual, previous_pre_mix, previous_post_mix,
                                       previous_residual_mix, phi, alpha, bias, norm_weight)]
    kernels.mega_mhc_out(*inputs, new_residual, next_pre, next_post, next_mix, block_input, *cache, hc_eps=hc_eps,
                         norm_eps=norm_eps, num_iters=num_iters, need_backward=need_backward)
    return (new_residual, next_pre, next_post, next_mix.reshape(batch, sequence, streams, streams), block_input, *cache)


def hyper_mega_mhc_grad(grad_hin_placeholder, grad_h_post, grad_h_res, x, phi, alpha, bias, previous_pre,
                        hc_before_norm, inv_rms, sum_out, norm_out, grad_current_pre, mixed_input, rms_rstd,
                        norm_weight, direct_grad_x, previous_residual, previous_output, previous_post,
                        previous_residual_mix, runtime_config=None, all_event_counters=None, diagnostic_buffer=None, *,
                        hc_eps: float = 1e-6, grad_block_input=None, diagnostics=None):
    """reference: torch/ops.py:397-490, argument order of the native backward ABI.

    ``x`` is the forward new_residual, ``direct_grad_x`` its direct gradient, ``grad_current_pre /
    grad_h_post / grad_h_res`` the gradients of the predicted mappings. The gradient of block_input,
    which the reference folds into ``grad_hin_placeholder``, may also be given as ``grad_block_input``.
    Returns (grad_residual, grad_phi, grad_alpha, grad_bias, grad_previous_output, grad_previous_pre,
    grad_previous_post, grad_previous_residual_mix, grad_norm_weight fp32).
    """
    del runtime_config, all_event_counters, diagnostic_buffer, diagnostics, sum_out, norm_out
    block_grad = grad_block_input if grad_block_input is not None else grad_hin_placeholder
    hidden = previous_residual.shape[-1]
    tokens = previous_residual.numel() // (_MHC_STREAMS * hidden)
    f32 = dict(dtype=torch.float32, device=previous_residual.device)
    result = dict(
        grad_residual=torch.empty_like(previous_residual), grad_phi=torch.empty_like(phi),
        grad_alpha=torch.empty_like(alpha), grad_bias=torch.empty_like(bias),
        grad_previous_output=torch.empty_like(previous_output), grad_previous_pre_mix=torch.empty_like(previous_pre),
        grad_previous_post_mix=torch.empty_like(previous_post),
        grad_previous_residual_mix=torch.empty_like(previous_residual_mix),
        grad_norm_weight=torch.empty(norm_weight.shape, **f32))
    tensors = dict(
        grad_new_residual=direct_grad_x.contiguous(), grad_next_pre_mix=grad_current_pre.contiguous(),
        grad_next_post_mix=grad_h_post.contiguous(), grad_next_residual_mix=grad_h_res.reshape(tokens, 16).contiguous(),
        grad_block_input=block_grad.contiguous(), new_residual=x.contiguous(), hc_before_norm=hc_before_norm,
        inv_rms=inv_rms, mixed_input=mixed_input, rms_rstd=rms_rstd, previous_output=previous_output.contiguous(),
        residual=previous_residual.contiguous(), previous_pre_mix=previous_pre.contiguous(),
        previous_post_mix=previous_post.contiguous(), previous_residual_mix=previous_residual_mix.contiguous(),
        phi=phi, alpha=alpha, bias=bias, norm_weight=norm_weight, **result)
    kernels.mega_mhc_grad_out(tensors, hc_eps=hc_eps, num_iters=20)
    return tuple(result.values())
