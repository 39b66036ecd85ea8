"""MegaMoeExperts: router-selected SwiGLU experts with expert parallelism, on B200.

Public contract of the reference executor (hyper_multicore/modules/mega_moe/module.py:164-535):
parameterless module, expert weights borrowed per call in EIO ([e,H,2I],[e,I,H]) or EOI
([e,2I,H],[e,H,I]) layout, probabilities applied after FC2, one host synchronisation per call
(the count table), every EP rank calls in the same order.

Data flow of one forward (reference call stack: module.py:497-535, autograd.py:576-679):
  sort routes -> count all-gather -> offsets -> [per-call counters zeroed, ready published]
  -> dispatch rows to their owners (peer stores + per-expert arrival counters)
  -> grouped GEMM1 with fused SwiGLU, gated per expert on the arrival counters -> grouped GEMM2
  -> combine rows back to their sources -> weighted K-sum in token order.
Backward mirrors it with dY / dX and the four gradient GEMMs (autograd.py:681-763).
"""

from __future__ import annotations

import ctypes
import itertools
import math
import os
import struct
import weakref
from typing import Any

import torch
import torch.distributed as dist

from ... import _lib, kernels, ops
from ...symm import PeerWorkspace, align_rows
from .numerics import MegaMoeNumericsOptions, MegaMoeSchedulerOptions, MegaMoeTuningOptions
from .route import PreparedRoute, prepare_route, validate_topk_inputs

_COMMUNICATION_SPLIT = 128


class _InvalidExpertWeights(ValueError):
    """Shape / device / layout error of the borrowed expert weights."""


class _InvalidExpertWeightType(TypeError):
    """dtype error of the borrowed expert weights."""


def _validate_swiglu_limit(limit: Any) -> None:
    ok = limit is None
    if not ok and isinstance(limit, (int, float)) and not isinstance(limit, bool):
        try:
            encoded = struct.unpack("<f", struct.pack("<f", float(limit)))[0]
            ok = math.isfinite(limit) and math.isfinite(encoded) and encoded > 0
        except (OverflowError, struct.error):
            ok = False
    if not ok:
        raise ValueError(
            f"swiglu_limit must be None or a finite positive float32-representable number, got {limit!r}.")


def _resolve_ep_size(ep_group: Any | None) -> int:
    if ep_group is not None:
        if not dist.is_initialized():
            raise ValueError("Initialize torch.distributed before passing ep_group")
        return dist.get_world_size(ep_group)
    if dist.is_initialized() and dist.get_world_size() > 1:
        raise ValueError("Pass ep_group explicitly for distributed MegaMoeExperts")
    return 1


def _resolve_options(precision, numerics_options, tuning_options):
    if numerics_options is not None and not isinstance(numerics_options, MegaMoeNumericsOptions):
        raise TypeError("numerics_options must be MegaMoeNumericsOptions or None")
    if tuning_options is not None and not isinstance(tuning_options, MegaMoeTuningOptions):
        raise TypeError("tuning_options must be MegaMoeTuningOptions or None")
    numerics = numerics_options or MegaMoeNumericsOptions()
    tuning = tuning_options or MegaMoeTuningOptions()
    for name in ("apply_probs_before_fc2", "clamp_after_silu"):
        if not isinstance(getattr(numerics, name), bool):
            raise TypeError(f"{name} must be a boolean")
    if precision not in ("bf16", "mxfp8"):
        raise ValueError("MegaMoE precision must be bf16 or mxfp8")
    if precision == "mxfp8" and (numerics.swiglu_limit is not None or numerics.apply_probs_before_fc2):
        raise ValueError("MXFP8 does not support clamp or before-FC2 probability weighting")
    if numerics.partial_weight_grad_dtype not in (None, "native", "float32"):
        raise ValueError("partial_weight_grad_dtype must be native, float32 or None")
    _validate_swiglu_limit(numerics.swiglu_limit)
    if tuning.dispatch_mode not in ("push", "pull"):
        raise ValueError(f"dispatch_mode must be 'push' or 'pull', got {tuning.dispatch_mode!r}")
    for name in ("initial_capacity_factor", "capacity_growth_factor"):
        value = getattr(tuning, name)
        if value is not None:
            if tuning.dispatch_mode == "pull":
                raise ValueError("pull dispatch rejects explicit capacity factors")
            if isinstance(value, bool) or not isinstance(value, (int, float)) or not math.isfinite(value) or value < 1:
                raise ValueError(f"{name} must be a finite number >= 1, got {value!r}")
    scheduler = tuning.scheduler or MegaMoeSchedulerOptions()
    if not isinstance(scheduler, MegaMoeSchedulerOptions):
        raise TypeError("scheduler must be MegaMoeSchedulerOptions or None")
    if scheduler.lowering not in ("auto", "dense", "compact"):
        raise ValueError(f"unknown lowering {scheduler.lowering!r}")
    # Device-side tile scheduling replaces the reference's host task graph: its Ascend-only knobs
    # have no counterpart, so only their defaults are accepted.
    if (scheduler.policy is not None or scheduler.queue_ready_lookahead is not None or scheduler.batch_experts
            or scheduler.nominal_schedule or scheduler.lowering == "compact"):
        raise ValueError("scheduler options other than the defaults do not apply to the sm_100a backend")
    return numerics, tuning


class _LocalWorkspace:
    """Control block of a single-rank executor: rows never leave the GPU, so only the counters,
    the ready flag and a one-entry peer table are needed."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.ep, self.rank, self.group = 1, 0, None
        self.ctrl = torch.zeros(_lib.HMC_CTRL_WORDS, dtype=torch.int32, device=device)
        self.peer_ctrl = (ctypes.c_void_p * 1)(self.ctrl.data_ptr())
        self.generation = 0

    def next_generation(self) -> int:
        """Generation of the next operator call (the operator clears the counters and publishes it)."""
        self.generation += 1
        return self.generation

    def close(self) -> None:
        """Nothing to release explicitly."""


class _ResourceGroup:
    """Workspace owned jointly by the serial modules of one group
    (reference: _ExecutionResourceGroup, hyper_multicore/modules/module.py:262-345, 408-430)."""

    def __init__(self, key: tuple) -> None:
        self.key = key
        self.members: set[int] = set()
        self.workspace: Any | None = None
        self.control: Any | None = None  # PeerControl of an EP group: control block + count-exchange table
        self.closed = False
        self.shared = False
        self.sequence = next(_GROUP_SEQUENCE)  # creation order: the same on every rank
        _GROUPS.add(self)


_GROUPS: "weakref.WeakSet[_ResourceGroup]" = weakref.WeakSet()
_GROUP_SEQUENCE = itertools.count()
_DESTROY_HOOKED = False


def _close_all_groups() -> None:
    """Release every live workspace; every rank reaches this in the same order."""
    for group in sorted(_GROUPS, key=lambda g: g.sequence):
        if not group.closed and (group.workspace is not None or group.control is not None):
            if group.workspace is not None:
                group.workspace.close()
                group.workspace = None
            if group.control is not None:
                group.control.close()
                group.control = None
            group.closed = True


def _hook_process_group_destruction() -> None:
    """Workspaces map peer memory through the process group's ranks: release them before the group
    goes away (reference: hyper_multicore/_automatic.py:55-124, docs/mega_moe.md:348-356)."""
    global _DESTROY_HOOKED  # pylint: disable=global-statement
    if _DESTROY_HOOKED:
        return
    original = dist.destroy_process_group

    def destroy_process_group(group=None):
        if group is None or group is dist.group.WORLD:
            _close_all_groups()
        return original(group)

    dist.destroy_process_group = destroy_process_group
    _DESTROY_HOOKED = True


class _MegaMoeFunction(torch.autograd.Function):
    """Forward / backward of the routed expert FFN on already prepared routes."""

    @staticmethod
    def forward(ctx, hidden, probs, w1, w2, module, route: PreparedRoute):  # pylint: disable=arguments-differ
        ctx.module = module
        ctx.route = route
        # grad mode is off inside Function.forward: whether a backward can follow is what the inputs say
        module._backward_expected = any(ctx.needs_input_grad[:4])  # pylint: disable=protected-access
        run = module._run_forward_mx if module.precision == "mxfp8" else module._run_forward  # pylint: disable=protected-access
        out, saved = run(hidden, probs, w1, w2, route)
        ctx.save_for_backward(hidden, probs, w1, w2, *saved)
        return out

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, grad_output):  # pylint: disable=arguments-differ
        hidden, probs, w1, w2, *saved = ctx.saved_tensors
        run = ctx.module._run_backward_mx if ctx.module.precision == "mxfp8" else ctx.module._run_backward  # pylint: disable=protected-access
        grads = run(grad_output.contiguous(), hidden, probs, w1, w2, *saved, ctx.route,
                    need_weight_grads=(ctx.needs_input_grad[2], ctx.needs_input_grad[3]))
        grad_hidden, grad_probs, grad_w1, grad_w2 = grads
        return (grad_hidden if ctx.needs_input_grad[0] else None,
                grad_probs if ctx.needs_input_grad[1] else None,
                grad_w1 if ctx.needs_input_grad[2] else None,
                grad_w2 if ctx.needs_input_grad[3] else None, None, None)


class MegaMoeExperts(torch.nn.Module):
    """Execute router-selected local experts; the caller owns the expert parameters."""

    def __init__(self, *, hidden_size: int, intermediate_size: int, num_experts: int, top_k: int,
                 ep_group: Any | None = None, precision: str = "bf16",
                 numerics_options: MegaMoeNumericsOptions | None = None,
                 tuning_options: MegaMoeTuningOptions | None = None, expert_placement: Any | None = None) -> None:
        super().__init__()
        numerics, tuning = _resolve_options(precision, numerics_options, tuning_options)
        if expert_placement is not None and getattr(expert_placement, "strategy", "none") != "none":
            raise ValueError("adaptive expert placement (HotReplica) is not part of the sm_100a backend")
        ep_size = _resolve_ep_size(ep_group)
        for name, value in (("hidden_size", hidden_size), ("intermediate_size", intermediate_size),
                            ("num_experts", num_experts), ("top_k", top_k), ("ep_size", ep_size)):
            if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
                raise ValueError(f"{name} must be a positive integer, got {value!r}.")
        if top_k > num_experts:
            raise ValueError(f"top_k ({top_k}) cannot exceed num_experts ({num_experts}).")
        if num_experts % ep_size:
            raise ValueError(f"num_experts ({num_experts}) must be divisible by ep_size ({ep_size}).")
        for name, split in (("dispatch_split", tuning.dispatch_split), ("combine_split", tuning.combine_split)):
            if (not isinstance(split, int) or isinstance(split, bool) or split <= 0
                    or split % _COMMUNICATION_SPLIT):
                raise ValueError(
                    f"{name} must be a positive integer multiple of {_COMMUNICATION_SPLIT}, got {split!r}.")
        if hidden_size % 8 or intermediate_size % 8:
            raise ValueError("hidden_size and intermediate_size must be multiples of 8 (16-byte BF16 rows)")
        if precision == "mxfp8" and (hidden_size % 128 or intermediate_size % 128):
            raise ValueError("precision='mxfp8' needs hidden_size and intermediate_size to be multiples of 128 "
                             "on the sm_100a backend (the reference requires multiples of 64)")
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.num_experts = num_experts
        self.top_k = top_k
        self.ep_size = ep_size
        self.local_experts = num_experts // ep_size
        self._ep_group = ep_group
        self._rank = dist.get_rank(ep_group) if ep_group is not None else 0
        self._precision = precision
        self._numerics = numerics
        self._tuning = tuning
        self._pull = tuning.dispatch_mode == "pull" and ep_size > 1
        self._layout: str | None = None
        self._scale_atoms: dict = {}
        # Budget of every cross-rank device wait (ready flags, arrival and combine counters). A rank
        # that is late by more than this makes its peers give up with a status word instead of hanging.
        self._wait_budget_ns = int(float(os.environ.get("HMC_EP_WAIT_SECONDS", "60")) * 1e9)
        self._backward_expected = False
        # push dispatch rides inside the GEMM that consumes the rows; HMC_MOE_FUSED_DISPATCH=0 launches the
        # stand-alone dispatch kernel ahead of it instead
        self._fuse_dispatch = os.environ.get("HMC_MOE_FUSED_DISPATCH", "1") != "0"
        # queue the operator ahead of the count-table read-back (HMC_MOE_DEFERRED_ROUTE=0: read it first)
        self._defer_route = os.environ.get("HMC_MOE_DEFERRED_ROUTE", "1") != "0"
        self._group = _ResourceGroup(self._compatibility_key())
        self._group.members.add(id(self))
        self._closed = False
        self._status: torch.Tensor | None = None
        if ep_size > 1:
            _hook_process_group_destruction()
        local, hidden, inter = self.local_experts, hidden_size, intermediate_size
        self._weight_shapes = {
            "EIO": ((local, hidden, inter * 2), (local, inter, hidden)),
            "EOI": ((local, inter * 2, hidden), (local, hidden, inter)),
        }

    # ------------------------------------------------------------------ read-only properties
    @property
    def precision(self) -> str:
        return self._precision

    @property
    def swiglu_limit(self) -> float | None:
        return self._numerics.swiglu_limit

    @property
    def clamp_after_silu(self) -> bool:
        return self._numerics.clamp_after_silu

    @property
    def apply_probs_before_fc2(self) -> bool:
        return self._numerics.apply_probs_before_fc2

    # ------------------------------------------------------------------ execution resources
    @property
    def _workspace(self):
        return self._group.workspace

    @_workspace.setter
    def _workspace(self, value) -> None:
        self._group.workspace = value

    def _compatibility_key(self) -> tuple:
        """Normalised configuration two modules must share to use one workspace: field values, not
        option-object identity (reference: docs/mega_moe.md:337-342)."""
        numerics, tuning = self._numerics, self._tuning
        return (type(self).__name__, self.hidden_size, self.intermediate_size, self.num_experts, self.top_k,
                self.ep_size, id(self._ep_group), self._precision,
                (numerics.partial_weight_grad_dtype, numerics.swiglu_limit, numerics.clamp_after_silu,
                 numerics.apply_probs_before_fc2),
                (tuning.dispatch_mode, tuning.dispatch_split, tuning.combine_split, tuning.initial_capacity_factor,
                 tuning.capacity_growth_factor))

    @classmethod
    def share_execution_resources(cls, modules) -> None:
        """Share one workspace among compatible modules that execute serially; must be called
        before any of them runs (reference: hyper_multicore/modules/module.py:262-323)."""
        members = tuple(modules)
        if not members:
            raise ValueError("shared multicore execution requires at least one module.")
        if len({id(member) for member in members}) != len(members):
            raise ValueError("shared multicore execution cannot contain duplicate modules.")
        if any(not isinstance(member, cls) for member in members):
            raise TypeError(f"all shared modules must be {cls.__name__} instances, "
                            f"got {[type(member).__name__ for member in members]}.")
        if any(member._closed or member._group.closed for member in members):  # pylint: disable=protected-access
            raise RuntimeError("closed multicore modules cannot share execution resources.")
        if len({type(member) for member in members}) != 1:
            raise TypeError("shared multicore execution requires one concrete module type.")
        first = members[0]._group  # pylint: disable=protected-access
        if all(member._group is first for member in members):  # pylint: disable=protected-access
            return
        for member in members:
            group = member._group  # pylint: disable=protected-access
            if group.key != first.key:
                raise ValueError("shared multicore modules must have identical configuration and scope.")
            if group.workspace is not None or len(group.members) != 1:
                raise RuntimeError("execution resources must be shared before first use or previous grouping.")
        first.shared = True
        for member in members[1:]:
            member._group.members.discard(id(member))  # pylint: disable=protected-access
            member._group = first  # pylint: disable=protected-access
            first.members.add(id(member))

    # ------------------------------------------------------------------ validation
    def _infer_layout(self, shape1, shape2) -> str:
        for layout, shapes in self._weight_shapes.items():
            if (shape1, shape2) == shapes:
                return layout
        raise _InvalidExpertWeights(
            f"expert_weights must have EIO shapes {self._weight_shapes['EIO']} or EOI shapes "
            f"{self._weight_shapes['EOI']}, got {(shape1, shape2)}.")

    def _validate_mx_weights(self, hidden: torch.Tensor, weight1, weight2) -> None:
        """MXFP8 roots carry their physical fields as attributes (reference: backends/mxfp8/weights.py:36-86)."""
        shapes = self._weight_shapes["EIO"]
        for name, root, (experts, rows, cols) in (("gate_up_weight", weight1, shapes[0]), ("down_weight", weight2, shapes[1])):
            if not isinstance(root, torch.Tensor):
                raise _InvalidExpertWeightType("MegaMoE MXFP8 weights require an original tensor root with physical MX storage.")
            if tuple(root.shape) not in ((experts, rows, cols), (experts * rows, cols)):
                raise _InvalidExpertWeights(
                    f"MegaMoE MXFP8 root shape {tuple(root.shape)} does not match expert shape {(experts, rows, cols)}.")
            if root.device != hidden.device:
                raise _InvalidExpertWeights("expert weights and hidden states must be on the same GPU.")
            data, scale = getattr(root, "col_data", None), getattr(root, "col_scale", None)
            if data is None or scale is None:
                raise _InvalidExpertWeights(f"MegaMoE MXFP8 current root ({name}) is missing required col data/scale.")
            self._check_mx_pair(data, scale, root, (experts, rows, cols), "col")
        self._pending_layout = "EIO"

    @staticmethod
    def _check_mx_pair(data, scale, root, shape, direction):
        experts, rows, cols = shape
        if data.dtype != torch.float8_e4m3fn or scale.dtype != torch.uint8:
            raise _InvalidExpertWeightType("MegaMoE MXFP8 physical storage requires E4M3FN data and packed uint8 E8M0 scales.")
        if not data.is_contiguous() or not scale.is_contiguous():
            raise _InvalidExpertWeights("MX physical data and scale must be contiguous; implicit copies are forbidden")
        if data.device != root.device or scale.device != root.device:
            raise _InvalidExpertWeights("MX physical data, scales and current root must share a device")
        if data.numel() != experts * rows * cols or scale.numel() != experts * rows * cols // 32:
            raise _InvalidExpertWeights(f"MX {direction} data/scale sizes do not match expert shape {shape}")

    def _validate_weights(self, hidden: torch.Tensor, expert_weights) -> None:
        try:
            weight1, weight2 = expert_weights
            shape1, shape2 = tuple(weight1.shape), tuple(weight2.shape)
        except (AttributeError, TypeError, ValueError) as error:
            raise _InvalidExpertWeights("expert_weights must contain two tensors") from error
        if self._precision == "mxfp8":
            self._validate_mx_weights(hidden, weight1, weight2)
            return
        if self._layout is None:
            layout = self._infer_layout(shape1, shape2)
        else:
            layout = self._layout
            expected1, expected2 = self._weight_shapes[layout]
            if shape1 != expected1:
                raise _InvalidExpertWeights(f"gate_up_weight must have shape {expected1}, got {shape1}.")
            if shape2 != expected2:
                raise _InvalidExpertWeights(f"down_weight must have shape {expected2}, got {shape2}.")
        if weight1.device != hidden.device or weight2.device != hidden.device:
            raise _InvalidExpertWeights("expert weights and hidden states must be on the same GPU.")
        if weight1.dtype != hidden.dtype or weight2.dtype != hidden.dtype:
            raise _InvalidExpertWeightType("expert weights and hidden states must all use BF16.")
        if not weight1.is_contiguous() or not weight2.is_contiguous():
            raise _InvalidExpertWeights("expert weights must be contiguous for zero-copy execution.")
        self._pending_layout = layout

    def _validate_forward_inputs(self, hidden_states, topk_ids, topk_weights, tokens_per_expert, expert_weights):
        if not isinstance(hidden_states, torch.Tensor) or hidden_states.dtype != torch.bfloat16 or \
                not hidden_states.is_cuda:
            raise TypeError("MegaMoeExperts requires BF16 CUDA hidden states.")
        if hidden_states.ndim < 2 or hidden_states.shape[-1] != self.hidden_size:
            raise ValueError(
                "hidden_states must have at least two dimensions and configured hidden size "
                f"{self.hidden_size}, got {tuple(hidden_states.shape)}.")
        hidden_flat = hidden_states.reshape(-1, self.hidden_size)
        route_shape = (hidden_flat.shape[0], self.top_k)
        if tuple(topk_ids.shape) != route_shape:
            raise ValueError(f"topk_ids must have shape {route_shape}, got {tuple(topk_ids.shape)}.")
        if tuple(topk_weights.shape) != route_shape:
            raise ValueError(f"topk_weights must have shape {route_shape}, got {tuple(topk_weights.shape)}.")
        if tokens_per_expert is not None:
            if tuple(tokens_per_expert.shape) != (self.num_experts,):
                raise ValueError(
                    f"tokens_per_expert must have shape ({self.num_experts},), got {tuple(tokens_per_expert.shape)}.")
            if tokens_per_expert.dtype not in (torch.int32, torch.int64):
                raise TypeError(f"tokens_per_expert must be int32 or int64, got {tokens_per_expert.dtype}.")
        validate_topk_inputs(hidden_flat, topk_ids, topk_weights)
        limit = (2 ** 31 - 1) // max(self.hidden_size, self.top_k)
        if hidden_flat.shape[0] > limit:
            raise ValueError(f"token count {hidden_flat.shape[0]} exceeds the INT32 addressing limit {limit}")
        self._validate_weights(hidden_flat, expert_weights)
        return hidden_flat.contiguous()

    # ------------------------------------------------------------------ resources
    def _ensure_workspace(self, device: torch.device, route: PreparedRoute):
        if self.ep_size == 1:
            if self._workspace is None:
                self._workspace = _LocalWorkspace(device)
            return self._workspace
        need_capacity, need_routed = route.max_received_rows, route.max_routed_rows
        workspace = self._workspace
        if self._pull:
            # Owners fetch into plain local tensors: the peer-mapped memory holds each rank's own rows
            # (source buffer + routed buffer), so a hot expert never makes it grow.
            if workspace is None or need_routed > workspace.routed_rows:
                generation = 0
                if workspace is not None:
                    generation = workspace.generation
                    workspace.close()
                self._workspace = PeerWorkspace(self._ep_group, self.hidden_size, need_routed, need_routed, device,
                                                pull=True, control=self._group.control)
                self._workspace.generation = generation
            return self._workspace
        if workspace is not None and need_capacity <= workspace.capacity_rows and need_routed <= workspace.routed_rows:
            return workspace
        # Every rank sees the same gathered table, so every rank takes this branch together.
        growth = self._tuning.capacity_growth_factor or 1.25
        initial = self._tuning.initial_capacity_factor or 1.25
        if workspace is None:
            capacity = max(need_capacity, math.ceil(min(initial, self.ep_size) * need_routed))
            routed = need_routed
            generation = 0
        else:
            capacity = max(need_capacity, math.ceil(workspace.capacity_rows * growth))
            routed = max(need_routed, workspace.routed_rows)
            generation = workspace.generation
            workspace.close()
        bound = self.ep_size * align_rows(need_routed)
        if need_capacity > bound:
            # cannot happen for real routes: a rank receives at most every rank's tokens * top_k rows
            # (reference: _grow_receive_capacity, hyper_multicore/modules/mega_moe/spec.py:113-119)
            raise ValueError("MegaMoe route exceeds the lossless token bound")
        capacity = max(need_capacity, min(capacity, bound))
        self._workspace = PeerWorkspace(self._ep_group, self.hidden_size, capacity, routed, device,
                                        control=self._group.control)
        self._workspace.generation = generation
        return self._workspace

    def close(self) -> None:
        """Release this member; the workspace goes with the last member of its group. Collective over
        the EP group when ep_size > 1: every rank closes in the same order, with no call in flight
        (reference: hyper_multicore/modules/module.py:408-430)."""
        if self._closed:
            return
        group = self._group
        group.members.discard(id(self))
        if not group.members and not group.closed:
            if group.workspace is not None:
                group.workspace.close()
                group.workspace = None
            if group.control is not None:
                group.control.close()
                group.control = None
            group.closed = True
        self._closed = True

    def debug_state(self) -> dict:
        """Workspace sizes and the last device status words (synchronises)."""
        state = {"layout": self._layout, "ep_size": self.ep_size}
        if isinstance(self._workspace, PeerWorkspace):
            state.update(self._workspace.debug_state())
        if self._status is not None:
            state["status"] = self._status.tolist()
        return state

    def check_status(self) -> None:
        """Raise if a bounded device wait ran out or an index was rejected (synchronises)."""
        if self._status is not None:
            _lib.raise_on_status(self._status, "MegaMoeExperts")

    @staticmethod
    def _takes_part_in_autograd(hidden_states, topk_weights, expert_weights) -> bool:
        try:
            tensors = (hidden_states, topk_weights, *expert_weights)
        except TypeError:
            tensors = (hidden_states, topk_weights)
        return torch.is_grad_enabled() and any(isinstance(t, torch.Tensor) and t.requires_grad for t in tensors)

    # ------------------------------------------------------------------ forward
    def forward(self, hidden_states: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor, *,
                expert_weights: tuple[torch.Tensor, torch.Tensor],
                tokens_per_expert: torch.Tensor | None = None) -> torch.Tensor:
        """Route token states through the configured experts; returns the input shape and dtype."""
        weight_error: Exception | None = None
        try:
            hidden_flat = self._validate_forward_inputs(hidden_states, topk_ids, topk_weights, tokens_per_expert,
                                                        expert_weights)
        except (_InvalidExpertWeights, _InvalidExpertWeightType) as error:
            if self.ep_size == 1:
                raise
            # A rank-local weight error is deferred until every rank has joined the count
            # exchange, so that no peer is left waiting (reference: module.py:474-495).
            weight_error = error
            hidden_flat = hidden_states.reshape(-1, self.hidden_size).contiguous()
        if self._closed or self._group.closed:
            raise RuntimeError("closed multicore modules cannot execute.")
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("MegaMoe dynamic tokens and workspace growth do not support graph capture")
        device = hidden_flat.device
        if self._status is None:
            self._status = _lib.new_status(device)
        if self.ep_size > 1 and self._group.control is None and os.environ.get("HMC_COUNT_EXCHANGE", "device") != "nccl":
            from ...symm import PeerControl  # pylint: disable=import-outside-toplevel

            self._group.control = PeerControl(self._ep_group, self.num_experts, device)  # collective, once
        # Steady state of a push group: the operator is queued WITHOUT waiting for the count table. The route
        # guard decides on the device whether the call fits the live workspace; the table is validated below,
        # once everything is queued (the first call and pull dispatch size buffers from the table; the MXFP8
        # backend sizes its per-call buffers for the workspace's capacity instead of the rows received).
        workspace = self._workspace
        defer = None
        if (self._defer_route and self.ep_size > 1 and not self._pull
                and isinstance(workspace, PeerWorkspace) and self._group.control is not None):
            defer = (workspace.capacity_rows, workspace.routed_rows)
        route = prepare_route(hidden_flat, topk_ids.contiguous(), num_experts=self.num_experts, top_k=self.top_k,
                              ep_size=self.ep_size, rank=self._rank, group=self._ep_group,
                              invalid=weight_error is not None, status=self._status,
                              autograd=self._takes_part_in_autograd(hidden_states, topk_weights, expert_weights),
                              control=self._group.control, budget_ns=self._wait_budget_ns, defer_limits=defer)
        if weight_error is not None:
            if route.deferred is not None:
                # the peers have queued this call (as a no-op: the route guard saw this rank's flag) and moved on
                # to the next generation; keep step with them
                workspace.next_generation()
            raise weight_error
        if route.status_words is not None:
            # read together with the count table: earlier kernels' status words are final
            if route.status_words[0] != 0:
                code = route.status_words[0]
                raise _lib.HmcError(f"MegaMoeExperts: device status {code} ({_lib.STATUS_NAMES.get(code, '?')}), "
                                    f"detail {route.status_words[1:4]}")
        elif route.pending is None and route.deferred is None:
            # prepare_route just synchronised with the device, so earlier kernels' status words are final
            self.check_status()
        if self._layout is None:
            self._layout = self._pending_layout
        if route.deferred is None:
            self._ensure_workspace(device, route)
        weight1, weight2 = expert_weights
        probs = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
        out = _MegaMoeFunction.apply(hidden_flat, probs.contiguous(), weight1, weight2, self, route)
        if route.deferred is not None and route.resolve():
            # the call did not fit the workspace: it was a no-op on every rank; grow together and run it again
            route.skip_flag = None
            self._ensure_workspace(device, route)
            out = _MegaMoeFunction.apply(hidden_flat, probs.contiguous(), weight1, weight2, self, route)
        try:
            route.finish()
        except ValueError:
            self._status.zero_()  # the rejected ids also set the status words; the call is over
            raise
        return out.reshape(hidden_states.shape)

    def _swiglu_options(self) -> dict:
        """Clamp arguments of the SwiGLU epilogues (reference: docs/mega_moe.md:258-272)."""
        limit = self._numerics.swiglu_limit
        if limit is None:
            return {}
        clamp = _lib.HMC_CLAMP_AFTER_SILU if self._numerics.clamp_after_silu else _lib.HMC_CLAMP_BEFORE_SILU
        return {"swiglu_clamp": clamp, "swiglu_limit": float(limit)}

    def _copy_stream(self, device: torch.device) -> torch.cuda.Stream:
        stream = getattr(self, "_side_stream", None)
        if stream is None or stream.device != device:
            stream = self._side_stream = torch.cuda.Stream(device=device)
        return stream

    def _local_rows(self, rows: int, device: torch.device):
        """Single-rank receive buffer: [rows, H] BF16 followed by one float per row."""
        row_bytes = self.hidden_size * 2
        raw = torch.empty(rows * (row_bytes + 4), dtype=torch.uint8, device=device)
        return (raw[:rows * row_bytes].view(torch.bfloat16).view(rows, self.hidden_size),
                raw[rows * row_bytes:].view(torch.float32), rows * row_bytes)

    def _transport(self, workspace, generation: int, device: torch.device, local_buffer: torch.Tensor | None = None,
                   local_plane_offset: int = 0) -> ops.MoeTransport:
        """Endpoints of this call: the peer-mapped workspace of an EP group, or, on a single rank, the
        call's own receive buffer standing in for "the owner's buffer"."""
        if self.ep_size == 1:
            return ops.MoeTransport(
                ep=1, rank=0, peer_dispatch=(ctypes.c_void_p * 1)(_lib.ptr(local_buffer)), peer_combine=None,
                peer_ctrl=workspace.peer_ctrl, dispatch_rows_limit=0 if local_buffer is None else local_buffer.shape[0],
                dispatch_plane_offset=local_plane_offset, generation=generation, wait_budget_ns=self._wait_budget_ns)
        pull = self._pull
        return ops.MoeTransport(
            ep=self.ep_size, rank=self._rank, peer_dispatch=workspace.peer_source if pull else workspace.peer_expert,
            peer_combine=workspace.peer_routed, peer_ctrl=workspace.peer_ctrl,
            dispatch_rows_limit=workspace.routed_rows if pull else workspace.capacity_rows,
            combine_rows_limit=workspace.routed_rows,
            dispatch_plane_offset=workspace.source_plane_offset if pull else workspace.expert_plane_offset,
            combine_plane_offset=workspace.routed_plane_offset, generation=generation,
            dispatch_mode="pull" if pull else "push", wait_budget_ns=self._wait_budget_ns,
            copy_stream=self._copy_stream(device))

    def _launch(self, route: PreparedRoute, transport: ops.MoeTransport, **fields) -> ops.MegaMoeLaunch:
        off = route.offsets
        return ops.MegaMoeLaunch(
            transport=transport, intermediate_size=self.intermediate_size, top_k=self.top_k,
            routed_rows=route.routed_rows, received_rows=route.received_rows, weight_layout=self._layout or "EIO",
            fuse_dispatch=self._fuse_dispatch, probs_before_fc2=self._numerics.apply_probs_before_fc2,
            status=self._status, expert_of_row=route.expert_of_row,
            recv_segment_start=off["recv_segment_start"], send_order_start=off["send_order_start"],
            mapping=route.mapping, **self._swiglu_options(), **fields)

    def _run_forward(self, hidden, probs, w1, w2, route: PreparedRoute):
        """One call of the forward operator (reference: ops.mega_moe, torch/ops.py:554-649, issued by
        backends/bf16/autograd.py:576-679): dispatch, GEMM1 + SwiGLU, GEMM2, combine, and the Top-K sum."""
        workspace = self._workspace
        device = hidden.device
        received, routed_rows = route.received_rows, route.routed_rows
        inter, hid = self.intermediate_size, self.hidden_size
        bf16 = dict(dtype=torch.bfloat16, device=device)
        before_fc2 = self._numerics.apply_probs_before_fc2
        ep1, pull = self.ep_size == 1, self._pull
        off = route.offsets
        rows = max(received, 1)
        # One rank owns every expert and nothing travels with the rows: the dispatch is a local gather with
        # nothing to wait for (the reference short-circuits peer == self the same way, rma.h:205-208).
        local_gather = ep1 and not before_fc2
        generation = 0 if local_gather else workspace.next_generation()
        row_probs = None
        if ep1:
            if before_fc2:
                dispatch_target, row_probs, plane = self._local_rows(rows, device)
            else:
                dispatch_target, plane = torch.empty(rows, hid, **bf16), 0
            transport = self._transport(workspace, generation, device, dispatch_target, plane)
        else:
            transport = self._transport(workspace, generation, device)
            if pull:
                # owners fetch into a plain local tensor of exactly the received size
                dispatch_target = torch.empty(rows, hid, **bf16)
                row_probs = torch.empty(rows, dtype=torch.float32, device=device) if before_fc2 else None
            else:
                dispatch_target = workspace.expert_buffer
                row_probs = workspace.expert_values if before_fc2 else None
        up_proj = torch.empty(rows, 2 * inter, **bf16)
        activation = torch.empty(rows, inter, **bf16)
        down_proj = torch.empty(rows, hid, **bf16) if ep1 else None
        out = torch.empty(hidden.shape[0], hid, **bf16)
        # Owned copies: the peer-mapped buffers are rewritten by the next call on any rank
        # (reference: autograd.py:655-663 saves a dispatch copy and clones the combine output).
        push_ep = not ep1 and not pull
        saved_received = torch.empty(rows, hid, **bf16) if push_ep else dispatch_target[:rows]
        routed_out = down_proj if ep1 else torch.empty(max(routed_rows, 1), hid, **bf16)
        saved_probs = None
        if before_fc2:
            saved_probs = torch.empty(rows, dtype=torch.float32, device=device) if push_ep else row_probs[:rows]
        launch = self._launch(
            route, transport, dispatch_src_index=route.source_of_row,
            route_probs=probs.reshape(-1) if before_fc2 else None, row_probs=row_probs,
            saved_dispatch=saved_received if push_ep else None, saved_combine=None if ep1 else routed_out,
            saved_row_probs=saved_probs if (before_fc2 and push_ep) else None,
            topk_probs=None if before_fc2 else probs, output=out, skip_flag=route.skip_flag)
        ops.mega_moe(dispatch_target, off["dispatch_target_off"], hidden, off["dispatch_src_off"], off["dispatch_size"],
                     w1, off["group_list"], up_proj, activation, w2, off["group_list"], down_proj,
                     None if ep1 else workspace.routed_buffer, off["combine_target_off"], off["combine_src_off"],
                     off["combine_size"], None, None, None, None, None, workspace.ctrl, self._rank, self.ep_size,
                     self.num_experts, hid, hidden.shape[0], launch=launch)
        if before_fc2:
            saved_last = saved_probs if saved_probs is not None else torch.empty(0, device=device)
        else:
            saved_last = routed_out
        return out, (saved_received, up_proj, activation, saved_last)

    def _run_backward(self, grad_output, hidden, probs, w1, w2, received_x, up_proj, activation, saved_last,
                      route: PreparedRoute, need_weight_grads):
        """One call of the backward operator (reference: ops.mega_moe_grad, torch/ops.py:652-737, issued by
        backends/bf16/autograd.py:681-763). `saved_last` is the routed forward output (probabilities after
        FC2, needed for their gradient) or the received per-row probabilities (probabilities before FC2)."""
        workspace = self._workspace
        device = hidden.device
        received, routed_rows = route.received_rows, route.routed_rows
        inter, hid = self.intermediate_size, self.hidden_size
        bf16 = dict(dtype=torch.bfloat16, device=device)
        off = route.offsets
        tokens = hidden.shape[0]
        rows = max(received, 1)
        before_fc2 = self._numerics.apply_probs_before_fc2
        ep1, pull = self.ep_size == 1, self._pull
        f32_partials = self._numerics.partial_weight_grad_dtype == "float32"
        wdtype = torch.float32 if f32_partials else torch.bfloat16
        grad_w1 = torch.empty(w1.shape, dtype=wdtype, device=device) if need_weight_grads[0] else None
        grad_w2 = torch.empty(w2.shape, dtype=wdtype, device=device) if need_weight_grads[1] else None
        grad_up = torch.empty(rows, 2 * inter, **bf16)
        grad_hidden = torch.empty(tokens, hid, **bf16)
        grad_probs = torch.empty(tokens, self.top_k, dtype=torch.float32, device=device)
        # With the probability gradient travelling back (before FC2) the rows return through the combine
        # kernel, which carries the float plane; otherwise they leave from the dX GEMM's epilogue.
        fused_combine = not ep1 and not before_fc2
        grad_x_rows = None if fused_combine else torch.empty(rows, hid, **bf16)
        fields = dict(weight_grad_f32=f32_partials, grad_probs=grad_probs, grad_hidden=grad_hidden)
        plane = 0
        if before_fc2:
            # dY rows are plain copies of the token gradients (reference: _stage_backward_source,
            # backends/bf16/autograd.py:138-150); the gather is fused into the dispatch.
            generation = workspace.next_generation()
            dy_source = grad_output
            fields.update(dispatch_src_index=route.source_of_row, row_probs=saved_last,
                          row_dot=torch.empty(rows, dtype=torch.float32, device=device))
            if ep1:
                dispatch_target, _, plane = self._local_rows(rows, device)
            else:
                dispatch_target = torch.empty(rows, hid, **bf16) if pull else workspace.expert_buffer
        else:
            fields.update(grad_output=grad_output, saved_combine=saved_last, topk_probs=probs)
            if ep1:
                # the source's expert-major order IS the owner's order: the dY rows are used in place
                generation = 0
                dy_source = dispatch_target = torch.empty(max(routed_rows, 1), hid, **bf16)
            else:
                generation = workspace.next_generation()
                # pull: dY is written straight into the published source buffer; the owners fetch it
                dy_source = workspace.source_buffer if pull else torch.empty(max(routed_rows, 1), hid, **bf16)
                dispatch_target = torch.empty(rows, hid, **bf16) if pull else workspace.expert_buffer
        transport = self._transport(workspace, generation, device, dispatch_target if ep1 else None, plane)
        launch = self._launch(route, transport, **fields)
        ops.mega_moe_grad(dispatch_target, off["dispatch_target_off"], dy_source, off["dispatch_src_off"],
                          off["dispatch_size"], activation, grad_w2, w2, None, up_proj, grad_up, w1, grad_x_rows,
                          None if ep1 else workspace.routed_buffer, off["combine_target_off"], off["combine_src_off"],
                          off["combine_size"], received_x, grad_w1, off["group_list"], None, None, None, None, None,
                          None, None, None, workspace.ctrl, self._rank, self.ep_size, self.num_experts, hid, tokens,
                          launch=launch)
        if grad_w1 is not None and grad_w1.dtype != w1.dtype:
            grad_w1 = grad_w1.to(w1.dtype)
        if grad_w2 is not None and grad_w2.dtype != w2.dtype:
            grad_w2 = grad_w2.to(w2.dtype)
        return grad_hidden, grad_probs, grad_w1, grad_w2

    # ------------------------------------------------------------------ MXFP8 backend
    def _atoms(self, root: torch.Tensor, direction: str, shape) -> torch.Tensor:
        """Scale-factor atoms of one weight axis, re-packed only when the scale tensor changed."""
        scale = getattr(root, f"{direction}_scale", None)
        data = getattr(root, f"{direction}_data", None)
        if scale is None or data is None:
            raise ValueError(f"MegaMoE MXFP8 current root is missing required {direction} data/scale.")
        self._check_mx_pair(data, scale, root, shape, direction)
        # An entry is valid only for the very tensor object it was packed from (held weakly: an id() or a
        # data_ptr() can come back for new weights once the old ones are freed) at the same version.
        key = (id(scale), direction)
        version = scale._version  # pylint: disable=protected-access
        cached = self._scale_atoms.get(key)
        if cached is None or cached[0]() is not scale or cached[1] != version:
            for stale in [k for k, entry in self._scale_atoms.items() if entry[0]() is None]:
                del self._scale_atoms[stale]
            experts, rows, cols = shape
            atoms = kernels.mx_pack_weight_scale(scale, 0 if direction == "col" else 1, experts, rows, cols)
            self._scale_atoms[key] = cached = (weakref.ref(scale), version, atoms)
        return cached[2]

    def _mx_buffers(self, rows: int, groups: int, width: int, device, *, want_col: bool):
        """Row- and (optionally) column-quantised planes of one activation in the padded expert-major layout."""
        pad_blocks = kernels.mx_pad_blocks(rows, groups)
        acts = kernels.MxActivations(rows, groups, width, device, want_row=True, want_col=want_col)
        assert acts.pad_blocks == pad_blocks
        return acts

    def _mx_transport(self, workspace, route: PreparedRoute, device, local_buffer):
        ep1 = self.ep_size == 1
        generation = 0 if ep1 else workspace.next_generation()
        return self._transport(workspace, generation, device, local_buffer if ep1 else None)

    def _run_forward_mx(self, hidden, probs, root1, root2, route: PreparedRoute):
        """One call of the MXFP8 forward operator: dispatch -> quant X -> GEMM1 -> SwiGLU + quant -> GEMM2 ->
        combine -> K-sum (reference: ops.mega_moe_mxfp8 issued by backends/mxfp8/execution.py:64-118, graph
        backends/mxfp8/graph.py:140-146)."""
        workspace = self._workspace
        device = hidden.device
        inter, hid, local = self.intermediate_size, self.hidden_size, self.local_experts
        received, routed_rows = route.received_rows, route.routed_rows
        rows = max(received, 1)
        bf16 = dict(dtype=torch.bfloat16, device=device)
        off = route.offsets
        training = self._backward_expected
        ep1, pull = self.ep_size == 1, self._pull
        dispatch_buffer = workspace.expert_buffer if (not ep1 and not pull) else torch.empty(rows, hid, **bf16)
        transport = self._mx_transport(workspace, route, device, dispatch_buffer)
        up_proj = torch.empty(rows, 2 * inter, **bf16)
        down_proj = torch.empty(rows, hid, **bf16) if ep1 else None
        x_q = self._mx_buffers(received, local, hid, device, want_col=training)
        act_q = self._mx_buffers(received, local, inter, device, want_col=training)
        routed_out = down_proj if ep1 else torch.empty(max(routed_rows, 1), hid, **bf16)
        out = torch.empty(hidden.shape[0], hid, **bf16)
        launch = self._launch(route, transport, dispatch_src_index=route.source_of_row, pad_blocks=x_q.pad_blocks,
                              saved_combine=None if ep1 else routed_out, topk_probs=probs, output=out,
                              skip_flag=route.skip_flag)
        buffers = [
            dispatch_buffer, off["dispatch_target_off"], hidden, off["dispatch_src_off"], off["dispatch_size"],
            root1.col_data, off["group_list"], up_proj, act_q.row_data, root2.col_data, off["group_list"], down_proj,
            None if ep1 else workspace.routed_buffer, off["combine_target_off"], off["combine_src_off"],
            off["combine_size"], x_q.row_data, x_q.row_scale, x_q.col_data, x_q.col_scale, act_q.row_scale,
            act_q.col_data, act_q.col_scale, self._atoms(root1, "col", (local, hid, 2 * inter)),
            self._atoms(root2, "col", (local, inter, hid)),
        ]
        ops.mega_moe_mxfp8(buffers, None, workspace.ctrl, None, None, rank_id=self._rank, ep=self.ep_size,
                           expert_num=self.num_experts, hidden_size=hid, seq_size=hidden.shape[0], launch=launch)
        empty = torch.empty(0, dtype=torch.uint8, device=device)
        keep = training and received > 0
        saved = (up_proj, routed_out,
                 x_q.col_data if keep else empty, x_q.col_scale if keep else empty,
                 act_q.col_data if keep else empty, act_q.col_scale if keep else empty)
        return out, saved

    def _run_backward_mx(self, grad_output, hidden, probs, root1, root2, up_proj, routed_out, x_col, x_col_scale,
                         act_col, act_col_scale, route: PreparedRoute, need_weight_grads):
        """One call of the MXFP8 backward operator: dY rows -> dispatch -> quant -> dA -> SwiGLU-grad + quant ->
        dX, dW2, dW1 -> combine -> K-sum (reference: ops.mega_moe_mxfp8_grad issued by
        backends/mxfp8/execution.py:120-164, graph backends/mxfp8/graph.py:147-154)."""
        workspace = self._workspace
        device = hidden.device
        inter, hid, local = self.intermediate_size, self.hidden_size, self.local_experts
        received, routed_rows = route.received_rows, route.routed_rows
        rows = max(received, 1)
        tokens = hidden.shape[0]
        bf16 = dict(dtype=torch.bfloat16, device=device)
        off = route.offsets
        ep1, pull = self.ep_size == 1, self._pull
        grad_routed = torch.empty(max(routed_rows, 1), hid, **bf16)
        grad_probs = torch.empty(tokens, self.top_k, dtype=torch.float32, device=device)
        grad_hidden = torch.empty(tokens, hid, **bf16)
        f32_partials = self._numerics.partial_weight_grad_dtype == "float32"
        wdtype = torch.float32 if f32_partials else torch.bfloat16
        shape1, shape2 = (local, hid, 2 * inter), (local, inter, hid)
        grad_w1 = torch.empty(shape1, dtype=wdtype, device=device) if need_weight_grads[0] else None
        grad_w2 = torch.empty(shape2, dtype=wdtype, device=device) if need_weight_grads[1] else None
        want_col = grad_w1 is not None or grad_w2 is not None
        if ep1:
            dispatch = grad_routed  # already in the owner's (= the source's) order
        else:
            dispatch = torch.empty(rows, hid, **bf16) if pull else workspace.expert_buffer
        transport = self._mx_transport(workspace, route, device, dispatch)
        dy_q = self._mx_buffers(received, local, hid, device, want_col=want_col)
        du_q = self._mx_buffers(received, local, 2 * inter, device, want_col=want_col)
        grad_act = torch.empty(rows, inter, **bf16)
        grad_x_rows = torch.empty(rows, hid, **bf16) if ep1 else None
        launch = self._launch(route, transport, pad_blocks=dy_q.pad_blocks, weight_grad_f32=f32_partials,
                              grad_output=grad_output, saved_combine=routed_out, topk_probs=probs, grad_probs=grad_probs,
                              grad_hidden=grad_hidden)
        have_saved = received > 0
        buffers = [
            dispatch, off["dispatch_target_off"], grad_routed, off["dispatch_src_off"], off["dispatch_size"],
            act_col if have_saved else None, grad_w2, root2.row_data, grad_act, up_proj, du_q.row_data, root1.row_data,
            grad_x_rows, None if ep1 else workspace.routed_buffer, off["combine_target_off"], off["combine_src_off"],
            off["combine_size"], x_col if have_saved else None, grad_w1, off["group_list"], dy_q.row_data, dy_q.row_scale,
            dy_q.col_data, dy_q.col_scale, act_col_scale if have_saved else None, self._atoms(root2, "row", shape2),
            du_q.row_scale, du_q.col_data, du_q.col_scale, self._atoms(root1, "row", shape1),
            x_col_scale if have_saved else None,
        ]
        ops.mega_moe_mxfp8_grad(buffers, None, workspace.ctrl, None, None, rank_id=self._rank, ep=self.ep_size,
                                expert_num=self.num_experts, hidden_size=hid, seq_size=tokens, launch=launch)
        if grad_w1 is not None:
            grad_w1 = grad_w1.to(root1.dtype).reshape(root1.shape)
        if grad_w2 is not None:
            grad_w2 = grad_w2.to(root2.dtype).reshape(root2.shape)
        return grad_hidden, grad_probs, grad_w1, grad_w2
