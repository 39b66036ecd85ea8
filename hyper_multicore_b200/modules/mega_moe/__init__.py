"""MegaMoE expert executor."""

from .module import MegaMoeExperts
from .numerics import MegaMoeNumericsOptions, MegaMoeSchedulerOptions, MegaMoeTuningOptions

__all__ = ["MegaMoeExperts", "MegaMoeNumericsOptions", "MegaMoeSchedulerOptions", "MegaMoeTuningOptions"]
