"""Host side of MegaMoE route preparation.

Follows prepare_topk_route / _prepare_dynamic_route of the reference
(hyper_multicore/modules/mega_moe/route.py:939-971): permutation index + histogram on the device,
one asynchronous count all-gather carrying a small validity header (route.py:850-878), one host
read-back of the count table for validation and capacity (route.py:585-622, 248-263), offset
descriptors computed on the device (route.py:309-390).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist

from ... import kernels

_HEADER = 3  # [invalid, local tokens, takes part in autograd] ahead of the per-expert counts
_PINNED: dict = {}  # (device, experts) -> pinned int32 staging for single-rank validation


@dataclass
class PreparedRoute:
    """Everything one forward/backward pair needs to address rows."""

    mapping: torch.Tensor          # [T*K] int32: destination row of flat (token, slot)
    source_of_row: torch.Tensor    # [T*K] int32: inverse permutation
    expert_of_row: torch.Tensor    # [T*K] int32
    counts_by_source: Any          # host copy of the gathered table (None for single-rank calls)
    offsets: dict[str, torch.Tensor]
    routed_rows: int               # tokens * top_k on this rank
    received_rows: int             # rows this rank's experts receive
    max_received_rows: int         # over the group
    max_routed_rows: int           # over the group
    pending: Any = None            # single-rank calls: (event, pinned counts + status words) checked by finish()
    status_words: Any = None       # multi-rank calls with the device exchange: status words read with the table
    deferred: Any = None           # multi-rank calls queued ahead of the table read-back: see resolve()
    skip_flag: Any = None          # device int32 the operator's kernels honour (set by the route guard)

    def resolve(self, what: str = "MegaMoeExperts") -> bool:
        """Deferred multi-rank calls validate here, after the operator has been queued.

        The route guard decided on the device, identically on every rank, whether the call may run (no rank
        flagged invalid inputs, nobody receives or routes more rows than the workspace holds) and mirrored the
        count table, the status words and its decision to pinned host memory. Waiting for that copy does not
        wait for the GEMMs queued behind it. Every rank reads the same table, so every rank raises the same
        error here, or learns together that the workspace must grow (returns True: the queued operator was a
        no-op on every rank and the caller runs the call again after growing).
        """
        if self.deferred is None:
            return False
        event, mirror, ep_size, num_experts, top_k, rank = self.deferred
        self.deferred = None
        event.synchronize()
        flat = mirror.tolist()
        body = ep_size * num_experts
        host = [flat[body + 4 * r: body + 4 * r + _HEADER] + flat[r * num_experts:(r + 1) * num_experts]
                for r in range(ep_size)]
        table_words = ep_size * (num_experts + 4)
        status = flat[table_words:table_words + 8]
        skipped = bool(flat[table_words + 8])
        if status[0] != 0:
            from ... import _lib

            raise _lib.HmcError(f"{what}: device status {status[0]} ({_lib.STATUS_NAMES.get(status[0], '?')}), "
                                f"detail {status[1:4]}")
        host_counts = check_gathered_rows(host, top_k, num_experts)  # raises on every rank together
        local = num_experts // ep_size
        received = [sum(sum(row[d * local:(d + 1) * local]) for row in host_counts) for d in range(ep_size)]
        routed = [sum(row) for row in host_counts]
        self.counts_by_source = host_counts
        self.received_rows = received[rank]
        self.max_received_rows, self.max_routed_rows = max(received), max(routed)
        return skipped

    def finish(self, what: str = "MegaMoeExperts") -> None:
        """Single-rank calls validate here, after the layer's kernels have been queued.

        The counts and the status words were copied to pinned host memory right after the sort, so
        waiting for that copy does not wait for the GEMMs queued behind it. Out-of-range expert ids
        were dropped by the sort (mapping -1, no rows), so the queued kernels touched nothing bad.
        """
        if self.pending is None:
            return
        event, pinned, experts, expected = self.pending
        self.pending = None
        event.synchronize()
        words = pinned.tolist()
        routed = sum(words[:experts])
        if routed != expected:
            raise ValueError(
                f"topk_ids must hold expert ids in [0, {experts}): {expected - routed} routes fell outside that range.")
        status = words[experts:]
        if status[0] != 0:
            from ... import _lib

            raise _lib.HmcError(f"{what}: device status {status[0]} ({_lib.STATUS_NAMES.get(status[0], '?')}), "
                                f"detail {status[1:4]}")


def validate_topk_inputs(hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> None:
    """Metadata-only checks (reference: route.py:160-183)."""
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"topk_ids must be int32 or int64, got {topk_ids.dtype}.")
    if not topk_weights.is_floating_point():
        raise TypeError(f"topk_weights must be floating point, got {topk_weights.dtype}.")
    if topk_ids.device != hidden.device or topk_weights.device != hidden.device:
        raise ValueError("hidden_states, topk_ids and topk_weights must be on one device.")


def check_gathered_rows(host: list[list[int]], top_k: int, num_experts: int) -> list[list[int]]:
    """Validate the gathered table [invalid, local tokens, autograd, counts...] of every EP rank.

    Every rank holds the same rows, so every rank takes the same decision and raises the same error
    together: nobody is left waiting in a collective or in a device wait
    (reference: _validate_dynamic_rows, hyper_multicore/modules/mega_moe/route.py:585-593, and the
    validity header of 850-868). Returns the per-rank count rows. Pure host logic: runs on plain lists.
    """
    if any(row[0] for row in host):
        bad = [r for r, row in enumerate(host) if row[0]]
        raise ValueError(f"MegaMoeExperts received invalid inputs on EP rank(s) {bad}; all ranks reject the call.")
    if len({row[2] for row in host}) != 1:
        # a rank that skips backward would leave its peers waiting in theirs
        raise RuntimeError("MegaMoe autograd participation differs across EP ranks")
    host_counts = [row[_HEADER:] for row in host]
    # A rank whose counts do not add up to its tokens * top_k dropped out-of-range expert ids, and ALL
    # ranks reject the call (a peer that went on would wait for rows that never come).
    short = [r for r, row in enumerate(host) if sum(host_counts[r]) != row[1] * top_k]
    if short:
        missing = sum(host[r][1] * top_k - sum(host_counts[r]) for r in short)
        raise ValueError(
            f"topk_ids must hold expert ids in [0, {num_experts}): {missing} routes fell outside that range "
            f"on EP rank(s) {short}; all ranks reject the call.")
    return host_counts


def prepare_route(hidden: torch.Tensor, topk_ids: torch.Tensor, *, num_experts: int, top_k: int, ep_size: int,
                  rank: int, group: Any | None, invalid: bool = False, status=None,
                  autograd: bool = False, control: Any | None = None, budget_ns: int = 0,
                  defer_limits: tuple[int, int] | None = None) -> PreparedRoute:
    """Sort the routes, exchange counts, derive offsets. Collective when ep_size > 1.

    ``defer_limits`` = (receive capacity, routed capacity) of the live workspace: the host does not wait for the
    count table. The route guard takes the admission decision on the device, `received_rows` of the result is the
    capacity (an upper bound), and `resolve()` validates the mirrored table once the operator has been queued."""
    device = hidden.device
    tokens = hidden.shape[0]
    mapping, sources, row_experts, counts, _ = kernels.moe_sort_routes(topk_ids, num_experts, status=status)
    if ep_size == 1 and status is not None:
        # One rank owns every expert: every size the host needs is tokens * top_k, so nothing waits for
        # the device here. Counts and status travel to pinned memory and are checked by finish().
        table = counts.view(1, num_experts)
        offsets = kernels.route_offsets(table, rank)
        key = (device, num_experts)
        pinned = _PINNED.get(key)
        if pinned is None:
            pinned = _PINNED[key] = torch.empty(num_experts + status.numel(), dtype=torch.int32).pin_memory()
        # written by kernels, not by a copy engine: this read-back must not queue behind the caller's
        # own bulk device-to-host copies
        kernels.store_words_pair(pinned, counts, status)
        event = torch.cuda.Event()
        event.record()
        routed = tokens * top_k
        return PreparedRoute(
            mapping=mapping, source_of_row=sources, expert_of_row=row_experts, counts_by_source=None,
            offsets=offsets, routed_rows=routed, received_rows=routed, max_received_rows=routed,
            max_routed_rows=routed, pending=(event, pinned, num_experts, routed))
    if control is not None:
        # Device-initiated exchange through the peer-mapped count table: one kernel instead of staging a
        # payload and enqueueing a host collective; the header words travel as kernel arguments.
        table, block = control.exchange(counts, (int(invalid), tokens, int(autograd)), status, budget_ns)
        offsets = kernels.route_offsets(table, rank)
        if defer_limits is not None:
            words = block.numel() + 8 + 1
            key = ("mirror", device, words)
            slot = _PINNED.get(key)
            if slot is None:
                # two mirrors in turn: a call's mirror is read by resolve() before the call after next writes it
                slot = _PINNED[key] = [torch.empty(words, dtype=torch.int32).pin_memory() for _ in range(2)] + [0]
            slot[2] ^= 1
            mirror = slot[slot[2]]
            flag = control.skip_flag
            kernels.route_guard(block, ep_size, num_experts, defer_limits[0], defer_limits[1], status, flag, mirror)
            event = torch.cuda.Event()
            event.record()
            return PreparedRoute(
                mapping=mapping, source_of_row=sources, expert_of_row=row_experts, counts_by_source=None,
                offsets=offsets, routed_rows=tokens * top_k, received_rows=defer_limits[0],
                max_received_rows=defer_limits[0], max_routed_rows=tokens * top_k,
                deferred=(event, mirror, ep_size, num_experts, top_k, rank), skip_flag=flag)
        words = status.numel() if status is not None else 0
        key = ("table", device, block.numel() + words)
        staged = _PINNED.get(key)
        if staged is None:
            staged = _PINNED[key] = torch.empty(block.numel() + words, dtype=torch.int32).pin_memory()
        kernels.store_words(staged[:block.numel()], block)
        if words:
            kernels.store_words(staged[block.numel():], status)
        torch.cuda.current_stream(device).synchronize()  # the one host synchronisation of the call
        flat = staged.tolist()
        read_status = flat[block.numel():] if words else None
        body = ep_size * num_experts
        host = [flat[body + 4 * r: body + 4 * r + _HEADER] + flat[r * num_experts:(r + 1) * num_experts]
                for r in range(ep_size)]
    else:
        read_status = None
        payload = torch.empty(_HEADER + num_experts, dtype=torch.int32, device=device)
        if ep_size > 1:
            # header staged in pinned memory: a plain torch.tensor(..., device=...) copies synchronously
            key = ("header", device)
            stage = _PINNED.get(key)
            if stage is None:
                stage = _PINNED[key] = torch.empty(_HEADER, dtype=torch.int32).pin_memory()
            stage[0], stage[1], stage[2] = int(invalid), tokens, int(autograd)
            payload[:_HEADER].copy_(stage, non_blocking=True)
        else:
            payload[:_HEADER] = 0
        payload[_HEADER:] = counts
        if ep_size > 1:
            gathered = torch.empty(ep_size * (_HEADER + num_experts), dtype=torch.int32, device=device)
            work = dist.all_gather_into_tensor(gathered, payload, group=group, async_op=True)
            work.wait()
            table_with_header = gathered.view(ep_size, _HEADER + num_experts)
        else:
            table_with_header = payload.view(1, _HEADER + num_experts)
        table = table_with_header[:, _HEADER:].contiguous()
        offsets = kernels.route_offsets(table, rank)
        host = table_with_header.tolist()  # the one host synchronisation of the call
    host_counts = check_gathered_rows(host, top_k, num_experts)
    local = num_experts // ep_size
    received = [sum(sum(row[d * local:(d + 1) * local]) for row in host_counts) for d in range(ep_size)]
    routed = [sum(row) for row in host_counts]
    return PreparedRoute(
        mapping=mapping, source_of_row=sources, expert_of_row=row_experts, counts_by_source=host_counts,
        offsets=offsets, routed_rows=tokens * top_k, received_rows=received[rank],
        max_received_rows=max(received), max_routed_rows=max(routed), status_words=read_status)
