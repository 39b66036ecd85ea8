"""CPU: the C-ABI library loads and exports every symbol include/hmc_b200.h declares."""

import ctypes
import re
from pathlib import Path

from hyper_multicore_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def _declared_symbols() -> set[str]:
    header = (ROOT / "include" / "hmc_b200.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return set(re.findall(r"\b(hmc_[a-z0-9_]+)\s*\(", header))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 20
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in hmc_b200.h but missing from the library"


def test_python_binding_covers_the_header():
    assert _declared_symbols() == set(_lib.SIGNATURES)


def test_versions_and_error_text():
    lib = _lib.load()
    assert lib.hmc_abi_version() == 1
    # The reference loader asserts these two layout versions (torch/csrc/registration.cpp:21-22).
    assert lib.hmc_mega_moe_transport_version() == 2
    assert lib.hmc_worker_queue_layout_version() == 2
    assert isinstance(lib.hmc_last_error(), bytes)


def test_argument_checks_fail_without_touching_a_device():
    lib = _lib.load()
    assert lib.hmc_grouped_gemm(None, None) == -1
    assert b"null args" in lib.hmc_last_error()
    args = _lib.GateRouteArgs()
    args.tokens = 0
    assert lib.hmc_gate_route(ctypes.byref(args), None) == -1
    assert b"tokens must be positive" in lib.hmc_last_error()
    assert lib.hmc_route_offsets(None, 2, 5, 0, None, None, None, None, None, None, None, None, None, None) == -1


def test_struct_sizes_match_the_header_layout():
    # 8 int32 + 4 int64 + 6 pointers + uint64 + pointer
    assert ctypes.sizeof(_lib.GroupedGemmArgs) == 8 * 4 + 4 * 8 + 6 * 8 + 8 + 8 + 2 * 4 + 3 * 8
