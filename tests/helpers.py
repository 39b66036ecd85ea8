"""Shared test helpers: golden fixture loading and tolerance checks."""

from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

GOLDEN = Path(__file__).resolve().parent / "golden"


def load_cases(name: str) -> list[dict]:
    """Load tests/golden/<name>.npz into one dict per case; BF16 arrays come back as torch.bfloat16."""
    with np.load(GOLDEN / f"{name}.npz", allow_pickle=False) as data:
        count = int(data["num_cases"])
        cases = [dict() for _ in range(count)]
        for key in data.files:
            if key == "num_cases":
                continue
            prefix, _, field = key.partition("_")
            index = int(prefix[4:])
            array = data[key]
            if field.endswith("__bf16"):
                cases[index][field[:-6]] = torch.from_numpy(array.copy()).view(torch.bfloat16)
            elif array.dtype.kind in "US":
                cases[index][field] = str(array)
            else:
                cases[index][field] = torch.from_numpy(array.copy())
    return cases


def sorted_sets(indices: torch.Tensor, *others: torch.Tensor):
    """Sort each row's expert ids and carry companion tensors along (order-free top-k compare)."""
    order = indices.argsort(dim=-1)
    return (indices.gather(1, order), *(o.gather(1, order) for o in others))


def cosine(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().flatten()
    b = b.double().flatten()
    return float((a @ b) / (a.norm() * b.norm() + 1e-300))


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a = a.double().flatten()
    b = b.double().flatten()
    return float((a - b).norm() / (b.norm() + 1e-300))
