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

_HEADER = 3  # [invalid, local tokens, reserved] ahead of the per-expert counts


@dataclass
class PreparedRoute:
    """Everything one forward/backward pair needs to address rows."""

    mapping: torch.Tensor          # [T*K] int32: destination row of flat (token, slot)
    source_of_row: torch.Tensor    # [T*K] int32: inverse permutation
    expert_of_row: torch.Tensor    # [T*K] int32
    counts_by_source: list[list[int]]  # host copy of the gathered table
    offsets: dict[str, torch.Tensor]
    routed_rows: int               # tokens * top_k on this rank
    received_rows: int             # rows this rank's experts receive
    max_received_rows: int         # over the group
    max_routed_rows: int           # over the group


def validate_topk_inputs(hidden: torch.Tensor, topk_ids: torch.Tensor, topk_weights: torch.Tensor) -> None:
    """Metadata-only checks (reference: route.py:160-183)."""
    if topk_ids.dtype not in (torch.int32, torch.int64):
        raise TypeError(f"topk_ids must be int32 or int64, got {topk_ids.dtype}.")
    if not topk_weights.is_floating_point():
        raise TypeError(f"topk_weights must be floating point, got {topk_weights.dtype}.")
    if topk_ids.device != hidden.device or topk_weights.device != hidden.device:
        raise ValueError("hidden_states, topk_ids and topk_weights must be on one device.")


def prepare_route(hidden: torch.Tensor, topk_ids: torch.Tensor, *, num_experts: int, top_k: int, ep_size: int,
                  rank: int, group: Any | None, invalid: bool = False, status=None) -> PreparedRoute:
    """Sort the routes, exchange counts, derive offsets. Collective when ep_size > 1."""
    device = hidden.device
    tokens = hidden.shape[0]
    mapping, sources, row_experts, counts, _ = kernels.moe_sort_routes(topk_ids, num_experts, status=status)
    payload = torch.empty(_HEADER + num_experts, dtype=torch.int32, device=device)
    payload[:_HEADER] = torch.tensor([int(invalid), tokens, 0], dtype=torch.int32, device=device) \
        if ep_size > 1 else 0
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
    if any(row[0] for row in host):
        bad = [r for r, row in enumerate(host) if row[0]]
        raise ValueError(f"MegaMoeExperts received invalid inputs on EP rank(s) {bad}; all ranks reject the call.")
    host_counts = [row[_HEADER:] for row in host]
    if sum(host_counts[rank]) != tokens * top_k:
        raise ValueError(
            f"topk_ids must hold expert ids in [0, {num_experts}): {tokens * top_k - sum(host_counts[rank])} "
            "routes fell outside that range.")
    local = num_experts // ep_size
    received = [sum(sum(row[d * local:(d + 1) * local]) for row in host_counts) for d in range(ep_size)]
    routed = [sum(row) for row in host_counts]
    return PreparedRoute(
        mapping=mapping, source_of_row=sources, expert_of_row=row_experts, counts_by_source=host_counts,
        offsets=offsets, routed_rows=tokens * top_k, received_rows=received[rank],
        max_received_rows=max(received), max_routed_rows=max(routed))
