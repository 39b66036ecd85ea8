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


def test_python_constants_equal_the_header_defines():
    """Every integer ``#define HMC_*`` of the header that the binding names too has the same value there."""
    header = (ROOT / "include" / "hmc_b200.h").read_text()
    defines = {name: int(value, 0) for name, value in re.findall(r"^#define\s+(HMC_[A-Z0-9_]+)\s+(-?(?:0x[0-9a-fA-F]+|\d+))\b",
                                                                header, flags=re.M)}
    shared = [name for name in defines if isinstance(getattr(_lib, name, None), int)]
    assert len(shared) >= 15, shared
    for name in shared:
        assert getattr(_lib, name) == defines[name], (name, getattr(_lib, name), defines[name])


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
    assert lib.hmc_route_offsets(None, 2, 5, 0, None, None, None, None, None, None, None, None, None, None, None) == -1


STRUCTS = {
    "hmc_gemm_combine": "GemmCombine", "hmc_grouped_gemm_args": "GroupedGemmArgs", "hmc_mx_gemm_args": "MxGemmArgs",
    "hmc_mx_quant_args": "MxQuantArgs", "hmc_gate_route_args": "GateRouteArgs",
    "hmc_gate_route_grad_args": "GateRouteGradArgs", "hmc_mega_mhc_args": "MegaMhcArgs",
    "hmc_mega_mhc_grad_args": "MegaMhcGradArgs", "hmc_ep_dispatch_args": "EpDispatchArgs",
    "hmc_ep_combine_args": "EpCombineArgs", "hmc_ep_pull_args": "EpPullArgs", "hmc_ep_exchange_args": "EpExchangeArgs",
    "hmc_moe_transport": "MoeTransport", "hmc_mega_moe_args": "MegaMoeArgs", "hmc_mega_moe_grad_args": "MegaMoeGradArgs",
    "hmc_mega_moe_mxfp8_args": "MegaMoeMxfp8Args", "hmc_mega_moe_mxfp8_grad_args": "MegaMoeMxfp8GradArgs",
}


def test_struct_layouts_match_the_header(tmp_path):
    """The header compiles as plain C, and every ctypes mirror has the size and the field offsets the C
    compiler gives the struct it mirrors (field names are the same on both sides)."""
    import shutil
    import subprocess

    if shutil.which("gcc") is None:
        import pytest

        pytest.skip("no C compiler")
    header = (ROOT / "include" / "hmc_b200.h").read_text()
    declared = set(re.findall(r"^} (hmc_[a-z0-9_]+);", header, flags=re.M))
    assert declared == set(STRUCTS), "every struct of the header needs a ctypes mirror listed here"
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{ROOT / "include" / "hmc_b200.h"}"', "int main(void) {"]
    for c_name, py_name in STRUCTS.items():
        lines.append(f'  printf("{c_name} size %zu\\n", sizeof({c_name}));')
        for field, _ in getattr(_lib, py_name)._fields_:  # pylint: disable=protected-access
            lines.append(f'  printf("{c_name} {field} %zu\\n", offsetof({c_name}, {field}));')
    lines += ["  return 0;", "}"]
    source = tmp_path / "layout.c"
    source.write_text("\n".join(lines))
    binary = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-o", str(binary), str(source)], check=True)
    output = subprocess.run([str(binary)], check=True, capture_output=True, text=True).stdout
    for line in output.splitlines():
        c_name, field, value = line.split()
        mirror = getattr(_lib, STRUCTS[c_name])
        expected = ctypes.sizeof(mirror) if field == "size" else getattr(mirror, field).offset
        assert int(value) == expected, f"{c_name}.{field}: header {value}, ctypes {expected}"
