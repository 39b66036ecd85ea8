"""Numerical and tuning options of MegaMoeExperts.

Same names, defaults and validation behaviour as the reference's frozen dataclasses
(hyper_multicore/modules/mega_moe/numerics.py:21-50, hyper_multicore/experimental/_mega_moe.py:21-75).
Options that only name Ascend scheduling concepts are accepted at their defaults and rejected
otherwise, the way the reference's arch35 path rejects them (docs/mega_moe.md:417-423).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Literal


@dataclass(frozen=True)
class MegaMoeNumericsOptions:
    """Activation and probability semantics of one MegaMoeExperts instance."""

    partial_weight_grad_dtype: Literal["native", "float32"] | None = None
    swiglu_limit: float | None = None
    clamp_after_silu: bool = False
    apply_probs_before_fc2: bool = False


@dataclass(frozen=True)
class MegaMoeSchedulerOptions:
    """Experimental scheduling knobs of the reference; none applies to device-side scheduling."""

    policy: str | None = None
    queue_ready_lookahead: int | None = None
    batch_experts: bool | None = None
    nominal_schedule: bool | None = None
    lowering: Literal["auto", "dense", "compact"] = "auto"


@dataclass(frozen=True)
class MegaMoeTuningOptions:
    """Execution policies that do not change model semantics."""

    dispatch_mode: Literal["push", "pull"] = "push"
    initial_capacity_factor: float | None = None
    capacity_growth_factor: float | None = None
    dispatch_split: int = 128
    combine_split: int = 128
    scheduler: MegaMoeSchedulerOptions | None = None
