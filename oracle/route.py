"""Route-preparation oracle (CPU, numpy integers): histogram, expert-major permutation, offsets.

Restates hyper_multicore/modules/mega_moe/route.py: _resolve_counts (186-211),
_expert_capacity (248-263), _compute_route_metadata torch form (351-390), and the permutation
contract of utilities.asc:162-209 (mapping[token * top_k + slot] = destination row, rows
expert-major). Intra-expert order is this build's choice: stable by flat index.
"""

from __future__ import annotations

import numpy as np


def counts(topk_ids: np.ndarray, num_experts: int) -> np.ndarray:
    """route.py:193-197."""
    return np.bincount(topk_ids.reshape(-1).astype(np.int64), minlength=num_experts).astype(np.int32)


def permutation(topk_ids: np.ndarray, num_experts: int):
    """Stable counting sort over flat index t*K+k. Returns (mapping, source_of_row, expert_of_row)."""
    flat = topk_ids.reshape(-1).astype(np.int64)
    order = np.argsort(flat, kind="stable")
    mapping = np.empty(flat.size, dtype=np.int32)
    mapping[order] = np.arange(flat.size, dtype=np.int32)
    return mapping, order.astype(np.int32), flat[order].astype(np.int32)


def expert_capacity(counts_by_source: np.ndarray, ep: int, rank: int):
    """route.py:248-263."""
    experts = counts_by_source.shape[1]
    local = experts // ep
    loads = counts_by_source.reshape(ep, ep, local).sum(axis=(0, 2))
    return max(1, int(loads[rank])), int(loads.max())


def route_metadata(counts_by_source: np.ndarray, ep: int, rank: int) -> dict:
    """route.py:351-390, push mode, row units."""
    table = counts_by_source.astype(np.int64)
    experts = table.shape[1]
    local = experts // ep
    source_prefix = table.cumsum(axis=1) - table
    destination_layout = table.reshape(ep, ep, local).transpose(1, 2, 0)
    destination_flat = destination_layout.reshape(ep, -1)
    destination_prefix = (destination_flat.cumsum(axis=1) - destination_flat).reshape(ep, local, ep)
    local_prefix = destination_prefix[rank]
    local_counts = destination_layout[rank]
    lo, hi = rank * local, (rank + 1) * local
    return {
        "dispatch_src_off": source_prefix[rank].astype(np.int64),
        "dispatch_target_off": destination_prefix[:, :, rank].reshape(-1).astype(np.int64),
        "dispatch_size": table[rank].astype(np.int32),
        "combine_src_off": local_prefix.T.reshape(-1).astype(np.int64),
        "combine_target_off": source_prefix[:, lo:hi].reshape(-1).astype(np.int64),
        "combine_size": table[:, lo:hi].reshape(-1).astype(np.int32),
        "group_list": (local_prefix[:, -1] + local_counts[:, -1]).astype(np.int64),
    }
