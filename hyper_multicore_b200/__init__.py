"""B200 (sm_100a) implementation of the hyper_multicore MegaMoE / MegaGate / MegaMHC hot path."""

__version__ = "0.1.0"
