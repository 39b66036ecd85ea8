"""Host-side mirror of the reference's module layer for the MegaMoE / MegaGate / MegaMHC path."""
