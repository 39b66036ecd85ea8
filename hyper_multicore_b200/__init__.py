"""B200 (sm_100a) implementation of the hyper_multicore MegaMoE / MegaGate / MegaMHC hot path.

Public names follow the reference package (hyper_multicore/__init__.py:31-35).
"""

__version__ = "0.1.0"

_EXPORTS = {
    "MegaMoeExperts": ("hyper_multicore_b200.modules.mega_moe", "MegaMoeExperts"),
    "MegaMoeNumericsOptions": ("hyper_multicore_b200.modules.mega_moe", "MegaMoeNumericsOptions"),
    "MegaMoeTuningOptions": ("hyper_multicore_b200.modules.mega_moe", "MegaMoeTuningOptions"),
    "MegaMoeSchedulerOptions": ("hyper_multicore_b200.modules.mega_moe", "MegaMoeSchedulerOptions"),
    "MegaGate": ("hyper_multicore_b200.modules.mega_gate", "MegaGate"),
    "MegaMhc": ("hyper_multicore_b200.modules.mega_mhc", "MegaMhc"),
    "hyper_mega_mhc": ("hyper_multicore_b200.modules.mega_mhc", "hyper_mega_mhc"),
}

__all__ = sorted(_EXPORTS)


def __getattr__(name: str):
    """Import lazily so that `import hyper_multicore_b200` stays cheap."""
    if name in _EXPORTS:
        import importlib

        module, attribute = _EXPORTS[name]
        return getattr(importlib.import_module(module), attribute)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
