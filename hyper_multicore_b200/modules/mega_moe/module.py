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

from ... import _lib, kernels
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

    def begin_call(self) -> int:
        self.generation += 1
        self.ctrl[:_lib.HMC_CTRL_READY].zero_()
        kernels._call("hmc_ep_publish_ready", self.device, self.peer_ctrl, 1, 0, self.generation)  # pylint: disable=protected-access
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
        route = prepare_route(hidden_flat, topk_ids.contiguous(), num_experts=self.num_experts, top_k=self.top_k,
                              ep_size=self.ep_size, rank=self._rank, group=self._ep_group,
                              invalid=weight_error is not None, status=self._status,
                              autograd=self._takes_part_in_autograd(hidden_states, topk_weights, expert_weights),
                              control=self._group.control, budget_ns=self._wait_budget_ns)
        if weight_error is not None:
            raise weight_error
        if route.status_words is not None:
            # read together with the count table: earlier kernels' status words are final
            if route.status_words[0] != 0:
                code = route.status_words[0]
                raise _lib.HmcError(f"MegaMoeExperts: device status {code} ({_lib.STATUS_NAMES.get(code, '?')}), "
                                    f"detail {route.status_words[1:4]}")
        elif route.pending is None:
            # prepare_route just synchronised with the device, so earlier kernels' status words are final
            self.check_status()
        if self._layout is None:
            self._layout = self._pending_layout
        self._ensure_workspace(device, route)
        weight1, weight2 = expert_weights
        probs = topk_weights if topk_weights.dtype == torch.float32 else topk_weights.float()
        out = _MegaMoeFunction.apply(hidden_flat, probs.contiguous(), weight1, weight2, self, route)
        try:
            route.finish()
        except ValueError:
            self._status.zero_()  # the rejected ids also set the status words; the call is over
            raise
        return out.reshape(hidden_states.shape)

    def _peer_tables(self, workspace, expert_buffer: torch.Tensor):
        if isinstance(workspace, PeerWorkspace):
            return workspace.peer_expert, workspace.peer_routed, workspace.peer_ctrl
        return (ctypes.c_void_p * 1)(expert_buffer.data_ptr()), None, workspace.peer_ctrl

    def _swiglu_options(self) -> dict:
        """Clamp arguments of the SwiGLU epilogues (reference: docs/mega_moe.md:258-272)."""
        limit = self._numerics.swiglu_limit
        if limit is None:
            return {}
        clamp = _lib.HMC_CLAMP_AFTER_SILU if self._numerics.clamp_after_silu else _lib.HMC_CLAMP_BEFORE_SILU
        return {"swiglu_clamp": clamp, "swiglu_limit": float(limit)}

    def _pull_rows(self, workspace, route: PreparedRoute, generation: int, fill, values=None):
        """Pull dispatch: `fill(rows)` writes this rank's expert-major rows into its source buffer, the
        buffer is published, and this rank fetches the rows of its own experts from every source
        (reference: owner-initiated GET, docs/design/mega_moe_design.md:33-35). Returns the received
        rows (a local tensor of exactly the received size) and, with `values`, their per-row scalars."""
        device = workspace.device
        routed = route.routed_rows
        if routed > 0:
            fill(workspace.source_buffer[:routed])
            if values is not None:
                workspace.source_values[:routed].copy_(values)
        kernels.ep_publish_source(workspace.peer_ctrl, self.ep_size, self._rank, generation, device)
        rows = max(route.received_rows, 1)
        out = torch.empty(rows, self.hidden_size, dtype=torch.bfloat16, device=device)
        out_values = torch.empty(rows, dtype=torch.float32, device=device) if values is not None else None
        off = route.offsets
        kernels.ep_pull(out, off["recv_segment_start"], off["combine_target_off"], rows=route.received_rows,
                        ep=self.ep_size, local_experts=self.local_experts, source_rows_limit=workspace.routed_rows,
                        peer_sources=workspace.peer_source, local_ctrl=workspace.ctrl, generation=generation,
                        status=self._status, budget_ns=self._wait_budget_ns, out_values=out_values,
                        value_plane_offset=workspace.source_plane_offset)
        return out, out_values

    def _fused_combine(self, workspace, off, peer_routed, peer_ctrl) -> dict | None:
        """Arguments that make a GEMM's epilogue return its rows to their source ranks."""
        if self.ep_size == 1:
            return None
        return {"segment_start": off["recv_segment_start"], "combine_target_off": off["combine_target_off"],
                "peer_buffers": peer_routed, "peer_ctrl": peer_ctrl, "ep": self.ep_size,
                "local_experts": self.local_experts, "target_rows_limit": workspace.routed_rows}

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

    def _run_forward(self, hidden, probs, w1, w2, route: PreparedRoute):
        workspace = self._workspace
        device = hidden.device
        eio = self._layout == "EIO"
        b_major = kernels.HMC_MAJOR_MN if eio else kernels.HMC_MAJOR_K
        received, routed_rows = route.received_rows, route.routed_rows
        inter, hid = self.intermediate_size, self.hidden_size
        bf16 = dict(dtype=torch.bfloat16, device=device)
        before_fc2 = self._numerics.apply_probs_before_fc2
        off = route.offsets
        pull = self._pull
        generation = workspace.begin_call() if self.ep_size > 1 else 0
        if self.ep_size == 1 and not before_fc2:
            # One rank owns every expert: the owner's order is the source's expert-major order, so the
            # dispatch is a local gather with nothing to wait for (the reference short-circuits
            # peer == self to a local copy the same way, rma.h:205-208).
            expert_buffer = torch.empty(max(received, 1), hid, **bf16)
            expert_values = None
            if routed_rows > 0:
                kernels.moe_gather_rows(hidden, route.source_of_row, self.top_k, expert_buffer[:routed_rows])
            peer_routed = peer_ctrl = None
        elif pull:
            sorted_probs = probs.reshape(-1).index_select(0, route.source_of_row.long()) if before_fc2 else None
            expert_buffer, expert_values = self._pull_rows(
                workspace, route, generation,
                lambda rows_out: kernels.moe_gather_rows(hidden, route.source_of_row, self.top_k, rows_out),
                values=sorted_probs)
            _, peer_routed, peer_ctrl = self._peer_tables(workspace, expert_buffer)
        else:
            if self.ep_size == 1:
                generation = workspace.begin_call()
                expert_buffer, expert_values, plane_offset = self._local_rows(max(received, 1), device)
                capacity = expert_buffer.shape[0]
            else:
                expert_buffer, expert_values = workspace.expert_buffer, workspace.expert_values
                capacity, plane_offset = workspace.capacity_rows, workspace.expert_plane_offset
            peer_expert, peer_routed, peer_ctrl = self._peer_tables(workspace, expert_buffer)
            travelling = dict(row_values=probs.reshape(-1), value_index=route.source_of_row,
                              value_plane_offset=plane_offset) if before_fc2 else {}
            kernels.ep_dispatch(hidden, route.source_of_row, route.expert_of_row, off["dispatch_src_off"],
                                off["dispatch_target_off"], rows=routed_rows, top_k=self.top_k, ep=self.ep_size,
                                local_experts=self.local_experts, capacity_rows=capacity, peer_buffers=peer_expert,
                                peer_ctrl=peer_ctrl, local_ctrl=workspace.ctrl, generation=generation,
                                status=self._status, budget_ns=self._wait_budget_ns, **travelling)
        rows = max(received, 1)
        up_proj = torch.empty(rows, 2 * inter, **bf16)
        activation = torch.empty(rows, inter, **bf16)
        down_proj = torch.empty(rows, hid, **bf16) if self.ep_size == 1 else None
        x_recv = expert_buffer[:rows]
        row_probs = expert_values[:rows] if before_fc2 else None
        # pulled / locally gathered rows are complete in stream order and live in a tensor of their own
        local_gather = self.ep_size == 1 and not before_fc2
        arrival = None if (pull or local_gather) else \
            workspace.ctrl[_lib.HMC_CTRL_ARRIVAL:_lib.HMC_CTRL_ARRIVAL + self.local_experts]
        saved_received = torch.empty_like(x_recv) if (self.ep_size > 1 and not pull) else x_recv
        if received > 0:
            kernels.grouped_gemm(x_recv, w1, up_proj, off["group_list"], mode=kernels.HMC_GEMM_RAGGED_M,
                                 b_major=b_major, epilogue=kernels.HMC_EPI_SWIGLU, aux=activation,
                                 ready_counters=arrival, ready_budget_ns=self._wait_budget_ns, status=self._status,
                                 row_probs=row_probs, **self._swiglu_options())
            if self.ep_size > 1 and not pull:
                # GEMM1 has waited for every expert's rows: the owned copy of the received rows (the
                # symmetric buffer is rewritten by the next call) runs on a side stream beside GEMM2.
                side = self._copy_stream(device)
                side.wait_stream(torch.cuda.current_stream(device))
                with torch.cuda.stream(side):
                    saved_received.copy_(x_recv)
            kernels.grouped_gemm(activation, w2, None if self.ep_size > 1 else down_proj, off["group_list"],
                                 mode=kernels.HMC_GEMM_RAGGED_M, b_major=b_major, status=self._status,
                                 combine=self._fused_combine(workspace, off, peer_routed, peer_ctrl))
        if self.ep_size == 1:
            routed_out = down_proj
            saved_received = x_recv
            saved_probs = row_probs
        else:
            # The result rows left the GEMM2 epilogue for their sources; wait for this rank's own.
            kernels.ep_wait(workspace.ctrl[_lib.HMC_CTRL_COMBINE:],
                            routed_rows * kernels.grouped_gemm_combine_units(hid), status=self._status,
                            budget_ns=self._wait_budget_ns)
            # Owned copies: the symmetric buffers are rewritten by the next call on any rank
            # (reference: autograd.py:655-663 saves a dispatch copy and clones the combine output).
            # They are made on a side stream, beside the K-sum below; this stream joins it before
            # the call returns.
            live_routed = workspace.routed_buffer[:max(routed_rows, 1)]
            routed_out = torch.empty_like(live_routed)
            saved_probs = (row_probs if pull else torch.empty_like(row_probs)) if before_fc2 else None
            main = torch.cuda.current_stream(device)
            side = self._copy_stream(device)
            side.wait_stream(main)
            with torch.cuda.stream(side):
                routed_out.copy_(live_routed)
                if before_fc2 and not pull:
                    saved_probs.copy_(row_probs)
        out = torch.empty(hidden.shape[0], hid, **bf16)
        live = routed_out if self.ep_size == 1 else live_routed
        if before_fc2:
            # The rows are already weighted: the Top-K rows of a token are summed as they are
            # (reference: _restore_unweighted_output, backends/bf16/autograd.py:133-135).
            # in ascending expert order with a BF16 rounding per addition, like the golden's index_add
            kernels.moe_unpermute(live, route.mapping, None, hidden.shape[0], self.top_k, out, status=self._status)
            saved_last = saved_probs if saved_probs is not None else torch.empty(0, device=device)
        else:
            kernels.moe_unpermute(live, route.mapping, probs, hidden.shape[0], self.top_k, out,
                                  status=self._status)
            saved_last = routed_out
        if self.ep_size > 1:
            torch.cuda.current_stream(device).wait_stream(self._copy_stream(device))
        return out, (saved_received, up_proj, activation, saved_last)

    def _run_backward(self, grad_output, hidden, probs, w1, w2, received_x, up_proj, activation, saved_last,
                      route: PreparedRoute, need_weight_grads):
        """`saved_last` is the routed forward output (probabilities after FC2, needed for their
        gradient) or the received per-row probabilities (probabilities before FC2)."""
        workspace = self._workspace
        device = hidden.device
        eio = self._layout == "EIO"
        received, routed_rows = route.received_rows, route.routed_rows
        inter, hid = self.intermediate_size, self.hidden_size
        bf16 = dict(dtype=torch.bfloat16, device=device)
        off = route.offsets
        tokens = hidden.shape[0]
        rows = max(received, 1)
        before_fc2 = self._numerics.apply_probs_before_fc2
        grad_probs = None
        generation = peer_routed = peer_ctrl = None
        if before_fc2:
            # dYe rows are plain copies of the token gradients (reference: _stage_backward_source,
            # backends/bf16/autograd.py:138-150); the gather is fused into the dispatch.
            row_probs = saved_last
            generation = workspace.begin_call()
            if self._pull:
                dy_recv, _ = self._pull_rows(
                    workspace, route, generation,
                    lambda rows_out: kernels.moe_gather_rows(grad_output, route.source_of_row, self.top_k, rows_out))
                _, peer_routed, peer_ctrl = self._peer_tables(workspace, dy_recv)
                arrival = None
            else:
                if self.ep_size == 1:
                    expert_buffer, _, _ = self._local_rows(rows, device)
                    capacity = rows
                else:
                    expert_buffer, capacity = workspace.expert_buffer, workspace.capacity_rows
                peer_expert, peer_routed, peer_ctrl = self._peer_tables(workspace, expert_buffer)
                kernels.ep_dispatch(grad_output, route.source_of_row, route.expert_of_row, off["dispatch_src_off"],
                                    off["dispatch_target_off"], rows=routed_rows, top_k=self.top_k, ep=self.ep_size,
                                    local_experts=self.local_experts, capacity_rows=capacity,
                                    peer_buffers=peer_expert, peer_ctrl=peer_ctrl, local_ctrl=workspace.ctrl,
                                    generation=generation, status=self._status, budget_ns=self._wait_budget_ns)
                dy_recv = expert_buffer[:rows]
                arrival = workspace.ctrl[_lib.HMC_CTRL_ARRIVAL:_lib.HMC_CTRL_ARRIVAL + self.local_experts]
            row_dot = torch.zeros(rows, dtype=torch.float32, device=device)
        else:
            row_probs = row_dot = None
            grad_probs = torch.empty(tokens, self.top_k, dtype=torch.float32, device=device)
            if self._pull:
                # dYe is written straight into the published source buffer; the owners fetch it
                generation = workspace.begin_call()
                dy_recv, _ = self._pull_rows(
                    workspace, route, generation,
                    lambda rows_out: kernels.moe_unpermute_grad(saved_last, grad_output, route.mapping, probs,
                                                                self.top_k, rows_out, grad_probs,
                                                                status=self._status))
                _, peer_routed, peer_ctrl = self._peer_tables(workspace, dy_recv)
                arrival = None
            else:
                # dYe (source's expert-major order) and dProbs
                grad_routed = torch.empty(max(routed_rows, 1), hid, **bf16)
                kernels.moe_unpermute_grad(saved_last, grad_output, route.mapping, probs, self.top_k, grad_routed,
                                           grad_probs, status=self._status)
            if self._pull:
                pass
            elif self.ep_size == 1:
                # One rank owns every expert: the source's expert-major order IS the owner's order
                # (the reference short-circuits peer == self the same way, rma.h:205-208), so the
                # rows are used in place and nothing has to arrive.
                dy_recv = grad_routed[:rows]
                arrival = None
            else:
                generation = workspace.begin_call()
                expert_buffer = workspace.expert_buffer
                peer_expert, peer_routed, peer_ctrl = self._peer_tables(workspace, expert_buffer)
                kernels.ep_dispatch(grad_routed, None, route.expert_of_row, off["dispatch_src_off"],
                                    off["dispatch_target_off"], rows=routed_rows, top_k=self.top_k, ep=self.ep_size,
                                    local_experts=self.local_experts, capacity_rows=workspace.capacity_rows,
                                    peer_buffers=peer_expert, peer_ctrl=peer_ctrl, local_ctrl=workspace.ctrl,
                                    generation=generation, status=self._status, budget_ns=self._wait_budget_ns)
                dy_recv = expert_buffer[:rows]
                arrival = workspace.ctrl[_lib.HMC_CTRL_ARRIVAL:_lib.HMC_CTRL_ARRIVAL + self.local_experts]
        grad_up = torch.empty(rows, 2 * inter, **bf16)
        # With the probability gradient travelling back (before FC2) the rows return through the combine
        # kernel, which carries the float plane; otherwise they leave from the dX GEMM's epilogue.
        fused = None if (self.ep_size == 1 or before_fc2) else self._fused_combine(workspace, off, peer_routed, peer_ctrl)
        grad_x_rows = torch.empty(rows, hid, **bf16) if fused is None else None
        f32_partials = self._numerics.partial_weight_grad_dtype == "float32"
        wdtype = torch.float32 if f32_partials else torch.bfloat16
        wepi = kernels.HMC_EPI_STORE_F32 if f32_partials else kernels.HMC_EPI_STORE_BF16
        grad_w1 = torch.empty(w1.shape, dtype=wdtype, device=device) if need_weight_grads[0] else None
        grad_w2 = torch.empty(w2.shape, dtype=wdtype, device=device) if need_weight_grads[1] else None
        # Transposed use of the weights: EIO W2 [e, I, H] is the K-major B of dA = dY . W2^T; EOI the reverse.
        bt_major = kernels.HMC_MAJOR_K if eio else kernels.HMC_MAJOR_MN
        if received > 0:
            kernels.grouped_gemm(dy_recv, w2, grad_up, off["group_list"], mode=kernels.HMC_GEMM_RAGGED_M,
                                 b_major=bt_major, epilogue=kernels.HMC_EPI_SWIGLU_GRAD, aux=up_proj,
                                 ready_counters=arrival, ready_budget_ns=self._wait_budget_ns, status=self._status,
                                 row_probs=row_probs, row_dot=row_dot, **self._swiglu_options())
            kernels.grouped_gemm(grad_up, w1, grad_x_rows, off["group_list"], mode=kernels.HMC_GEMM_RAGGED_M,
                                 b_major=bt_major, status=self._status, combine=fused)
        if grad_w2 is not None:
            # The arrival wait of the dA GEMM above orders this kernel after the rows have landed.
            # With probabilities before FC2, `activation` is the weighted input FC2 actually saw.
            a_op, b_op = (activation, dy_recv) if eio else (dy_recv, activation)
            kernels.grouped_gemm(a_op, b_op, grad_w2, off["group_list"], mode=kernels.HMC_GEMM_RAGGED_K, epilogue=wepi,
                                 status=self._status)
        if grad_w1 is not None:
            a_op, b_op = (received_x, grad_up) if eio else (grad_up, received_x)
            kernels.grouped_gemm(a_op, b_op, grad_w1, off["group_list"], mode=kernels.HMC_GEMM_RAGGED_K, epilogue=wepi,
                                 status=self._status)
        if self.ep_size == 1:
            returned, returned_dot = grad_x_rows, row_dot
        elif fused is not None:
            kernels.ep_wait(workspace.ctrl[_lib.HMC_CTRL_COMBINE:],
                            routed_rows * kernels.grouped_gemm_combine_units(hid), status=self._status,
                            budget_ns=self._wait_budget_ns)
            returned, returned_dot = workspace.routed_buffer, None
        else:
            kernels.ep_combine(grad_x_rows, off["recv_segment_start"], off["combine_target_off"], rows=received,
                               ep=self.ep_size, local_experts=self.local_experts,
                               target_rows_limit=workspace.routed_rows, peer_buffers=peer_routed,
                               peer_ctrl=peer_ctrl, local_ctrl=workspace.ctrl, generation=generation,
                               status=self._status, budget_ns=self._wait_budget_ns, result_values=row_dot,
                               value_plane_offset=workspace.routed_plane_offset)
            kernels.ep_wait(workspace.ctrl[_lib.HMC_CTRL_COMBINE:], routed_rows, status=self._status, budget_ns=self._wait_budget_ns)
            returned, returned_dot = workspace.routed_buffer, workspace.routed_values
        grad_hidden = torch.empty(tokens, hid, **bf16)
        kernels.moe_token_permute_grad(returned, route.mapping, tokens, self.top_k, grad_hidden, status=self._status)
        if before_fc2:
            # the probability gradient of route (t, k) sits at that route's row of the source order
            # (reference: backends/bf16/autograd.py:725-730)
            grad_probs = returned_dot.index_select(0, route.mapping.long()).view(tokens, self.top_k)
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

    def _mx_exchange(self, source, source_of_row, route, generation_hint=None):
        """Dispatch rows to their owners and wait until every local expert's rows have landed."""
        workspace = self._workspace
        device = source.device
        received, routed_rows = route.received_rows, route.routed_rows
        if self.ep_size == 1 and source_of_row is None:
            return source[:max(received, 1)], None, None, None  # already in the owner's order
        if self.ep_size == 1:
            # one rank owns every expert: the dispatch is a local gather into the owner's (= the source's) order
            rows_in = torch.empty(max(received, 1), self.hidden_size, dtype=torch.bfloat16, device=device)
            if routed_rows > 0:
                kernels.moe_gather_rows(source, source_of_row, self.top_k, rows_in[:routed_rows])
            return rows_in, None, None, None
        generation = workspace.begin_call()
        if self._pull:
            if source_of_row is not None:
                fill = lambda rows_out: kernels.moe_gather_rows(source, source_of_row, self.top_k, rows_out)  # noqa: E731
            else:
                fill = lambda rows_out: rows_out.copy_(source[:rows_out.shape[0]])  # noqa: E731
            rows_in, _ = self._pull_rows(workspace, route, generation, fill)
            _, peer_routed, peer_ctrl = self._peer_tables(workspace, rows_in)
            return rows_in, generation, peer_routed, peer_ctrl
        if self.ep_size == 1:
            expert_buffer = torch.empty(max(received, 1), self.hidden_size, dtype=torch.bfloat16, device=device)
            capacity = expert_buffer.shape[0]
        else:
            expert_buffer = workspace.expert_buffer
            capacity = workspace.capacity_rows
        peer_expert, peer_routed, peer_ctrl = self._peer_tables(workspace, expert_buffer)
        off = route.offsets
        kernels.ep_dispatch(source, source_of_row, route.expert_of_row, off["dispatch_src_off"],
                            off["dispatch_target_off"], rows=routed_rows, top_k=self.top_k, ep=self.ep_size,
                            local_experts=self.local_experts, capacity_rows=capacity, peer_buffers=peer_expert,
                            peer_ctrl=peer_ctrl, local_ctrl=workspace.ctrl, generation=generation,
                            status=self._status, budget_ns=self._wait_budget_ns)
        arrival = workspace.ctrl[_lib.HMC_CTRL_ARRIVAL:_lib.HMC_CTRL_ARRIVAL + self.local_experts]
        kernels.ep_wait_groups(arrival, off["group_list"], status=self._status, budget_ns=self._wait_budget_ns)
        return expert_buffer[:max(received, 1)], generation, peer_routed, peer_ctrl

    def _mx_return(self, rows_tensor, route, generation, peer_routed, peer_ctrl, width=None):
        """Combine result rows back to their sources (identity at ep_size == 1). With `rows_tensor` None
        the rows already left from the producing GEMM's epilogue (`width` columns): only wait for this
        rank's own rows."""
        if self.ep_size == 1:
            return rows_tensor
        workspace = self._workspace
        off = route.offsets
        if rows_tensor is None:
            kernels.ep_wait(workspace.ctrl[_lib.HMC_CTRL_COMBINE:],
                            route.routed_rows * kernels.mx_gemm_combine_units(width), status=self._status,
                            budget_ns=self._wait_budget_ns)
            return workspace.routed_buffer
        kernels.ep_combine(rows_tensor, off["recv_segment_start"], off["combine_target_off"], rows=route.received_rows,
                           ep=self.ep_size, local_experts=self.local_experts,
                           target_rows_limit=workspace.routed_rows, peer_buffers=peer_routed, peer_ctrl=peer_ctrl,
                           local_ctrl=workspace.ctrl, generation=generation, status=self._status, budget_ns=self._wait_budget_ns)
        kernels.ep_wait(workspace.ctrl[_lib.HMC_CTRL_COMBINE:], route.routed_rows, status=self._status, budget_ns=self._wait_budget_ns)
        return workspace.routed_buffer

    def _run_forward_mx(self, hidden, probs, root1, root2, route: PreparedRoute):
        """dispatch -> quant X -> GEMM1 -> SwiGLU + quant -> GEMM2 -> combine -> K-sum
        (reference graph: backends/mxfp8/graph.py:140-146)."""
        device = hidden.device
        inter, hid, local = self.intermediate_size, self.hidden_size, self.local_experts
        received = route.received_rows
        rows = max(received, 1)
        bf16 = dict(dtype=torch.bfloat16, device=device)
        ends = route.offsets["group_list"]
        training = self._backward_expected
        x_recv, generation, peer_routed, peer_ctrl = self._mx_exchange(hidden, route.source_of_row, route)
        up_proj = torch.empty(rows, 2 * inter, **bf16)
        fused = self._fused_combine(self._workspace, route.offsets, peer_routed, peer_ctrl)
        down_proj = torch.empty(rows, hid, **bf16) if fused is None else None
        x_q = act_q = None
        if received > 0:
            x_q = kernels.mx_quant(x_recv[:received], ends, hid, want_row=True, want_col=training)
            kernels.mx_gemm(x_q.row_data, x_q.row_scale, root1.col_data, self._atoms(root1, "col", (local, hid, 2 * inter)),
                            up_proj, ends, mode=kernels.HMC_GEMM_RAGGED_M, rows=received, pad_blocks=x_q.pad_blocks,
                            n=2 * inter, k=hid, b_major=kernels.HMC_MAJOR_MN, status=self._status)
            act_q = kernels.mx_quant(up_proj[:received], ends, inter, kind=kernels.HMC_MXQ_SWIGLU, want_row=True,
                                     want_col=training)
            kernels.mx_gemm(act_q.row_data, act_q.row_scale, root2.col_data, self._atoms(root2, "col", (local, inter, hid)),
                            down_proj, ends, mode=kernels.HMC_GEMM_RAGGED_M, rows=received, pad_blocks=act_q.pad_blocks,
                            n=hid, k=inter, b_major=kernels.HMC_MAJOR_MN, status=self._status, combine=fused)
        returned = self._mx_return(down_proj, route, generation, peer_routed, peer_ctrl, width=hid)
        routed_out = returned if self.ep_size == 1 else returned[:max(route.routed_rows, 1)].clone()
        out = torch.empty(hidden.shape[0], hid, **bf16)
        kernels.moe_unpermute(routed_out, route.mapping, probs, hidden.shape[0], self.top_k, out, status=self._status)
        empty = torch.empty(0, dtype=torch.uint8, device=device)
        saved = (up_proj, routed_out,
                 x_q.col_data if x_q is not None and training else empty,
                 x_q.col_scale if x_q is not None and training else empty,
                 act_q.col_data if act_q is not None and training else empty,
                 act_q.col_scale if act_q is not None and training else empty)
        return out, saved

    def _run_backward_mx(self, grad_output, hidden, probs, root1, root2, up_proj, routed_out, x_col, x_col_scale,
                         act_col, act_col_scale, route: PreparedRoute, need_weight_grads):
        """dispatch dY -> quant -> dA -> SwiGLU-grad + quant -> dX, dW2, dW1 -> combine
        (reference graph: backends/mxfp8/graph.py:147-154)."""
        device = hidden.device
        inter, hid, local = self.intermediate_size, self.hidden_size, self.local_experts
        received, routed_rows = route.received_rows, route.routed_rows
        rows = max(received, 1)
        tokens = hidden.shape[0]
        bf16 = dict(dtype=torch.bfloat16, device=device)
        ends = route.offsets["group_list"]
        grad_routed = torch.empty(max(routed_rows, 1), hid, **bf16)
        grad_probs = torch.empty(tokens, self.top_k, dtype=torch.float32, device=device)
        kernels.moe_unpermute_grad(routed_out, grad_output, route.mapping, probs, self.top_k, grad_routed, grad_probs,
                                   status=self._status)
        dy_recv, generation, peer_routed, peer_ctrl = self._mx_exchange(grad_routed, None, route)
        f32_partials = self._numerics.partial_weight_grad_dtype == "float32"
        wdtype = torch.float32 if f32_partials else torch.bfloat16
        wepi = kernels.HMC_EPI_STORE_F32 if f32_partials else kernels.HMC_EPI_STORE_BF16
        shape1, shape2 = (local, hid, 2 * inter), (local, inter, hid)
        grad_w1 = torch.empty(shape1, dtype=wdtype, device=device) if need_weight_grads[0] else None
        grad_w2 = torch.empty(shape2, dtype=wdtype, device=device) if need_weight_grads[1] else None
        fused = self._fused_combine(self._workspace, route.offsets, peer_routed, peer_ctrl)
        grad_x_rows = torch.empty(rows, hid, **bf16) if fused is None else None
        if received > 0:
            want_col = grad_w1 is not None or grad_w2 is not None
            dy_q = kernels.mx_quant(dy_recv[:received], ends, hid, want_row=True, want_col=want_col)
            grad_act = torch.empty(rows, inter, **bf16)
            # W2 [e, I, H] row-quantised (blocks along H) is the K-major B of dA = dY . W2^T
            kernels.mx_gemm(dy_q.row_data, dy_q.row_scale, root2.row_data, self._atoms(root2, "row", shape2), grad_act,
                            ends, mode=kernels.HMC_GEMM_RAGGED_M, rows=received, pad_blocks=dy_q.pad_blocks, n=inter,
                            k=hid, b_major=kernels.HMC_MAJOR_K, status=self._status)
            du_q = kernels.mx_quant(grad_act[:received], ends, 2 * inter, kind=kernels.HMC_MXQ_SWIGLU_GRAD,
                                    aux=up_proj[:received], want_row=True, want_col=want_col)
            kernels.mx_gemm(du_q.row_data, du_q.row_scale, root1.row_data, self._atoms(root1, "row", shape1), grad_x_rows,
                            ends, mode=kernels.HMC_GEMM_RAGGED_M, rows=received, pad_blocks=du_q.pad_blocks, n=hid,
                            k=2 * inter, b_major=kernels.HMC_MAJOR_K, status=self._status, combine=fused)
            if grad_w2 is not None:
                kernels.mx_gemm(act_col, act_col_scale, dy_q.col_data, dy_q.col_scale, grad_w2, ends,
                                mode=kernels.HMC_GEMM_RAGGED_K, rows=received, pad_blocks=dy_q.pad_blocks, m=inter, n=hid,
                                epilogue=wepi, status=self._status)
            if grad_w1 is not None:
                kernels.mx_gemm(x_col, x_col_scale, du_q.col_data, du_q.col_scale, grad_w1, ends,
                                mode=kernels.HMC_GEMM_RAGGED_K, rows=received, pad_blocks=du_q.pad_blocks, m=hid,
                                n=2 * inter, epilogue=wepi, status=self._status)
        else:
            for grad in (grad_w1, grad_w2):
                if grad is not None:
                    grad.zero_()
        returned = self._mx_return(grad_x_rows, route, generation, peer_routed, peer_ctrl, width=hid)
        grad_hidden = torch.empty(tokens, hid, **bf16)
        kernels.moe_token_permute_grad(returned, route.mapping, tokens, self.top_k, grad_hidden, status=self._status)
        if grad_w1 is not None:
            grad_w1 = grad_w1.to(root1.dtype).reshape(root1.shape)
        if grad_w2 is not None:
            grad_w2 = grad_w2.to(root2.dtype).reshape(root2.shape)
        return grad_hidden, grad_probs, grad_w1, grad_w2
