"""Build libhmc_b200.so in-tree with nvcc for sm_100a (no torch headers, plain C ABI)."""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
PACKAGE = CSRC.parent
LIBRARY = PACKAGE / "libhmc_b200.so"
OBJ_DIR = CSRC / "build"
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
                "-Xptxas", "-v"]


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(dep.stat().st_mtime > stamp for dep in deps)


def _compile(source: Path, headers: list[Path], verbose: bool) -> Path:
    obj = OBJ_DIR / (source.stem + ".o")
    if _stale(obj, [source, *headers]):
        cmd = ["nvcc", *ARCH_FLAGS, *COMMON_FLAGS, "-c", str(source), "-o", str(obj)]
        result = subprocess.run(cmd, capture_output=True, text=True)
        log = OBJ_DIR / (source.stem + ".ptxas.log")
        log.write_text(result.stderr)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed for {source.name}:\n{result.stderr}")
        if verbose:
            print(f"[hmc build] compiled {source.name}")
    return obj


def build(verbose: bool = False) -> Path:
    """Compile every .cu under csrc/ and link the shared library next to the package."""
    OBJ_DIR.mkdir(exist_ok=True)
    headers = [*CSRC.glob("*.cuh"), PACKAGE.parent / "include" / "hmc_b200.h"]
    sources = _sources()
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        objects = list(pool.map(lambda s: _compile(s, headers, verbose), sources))
    if _stale(LIBRARY, objects):
        cmd = ["nvcc", *ARCH_FLAGS, "-shared", "-o", str(LIBRARY), *map(str, objects), "-lcudart"]
        result = subprocess.run(cmd, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stderr}")
        if verbose:
            print(f"[hmc build] linked {LIBRARY}")
    return LIBRARY


if __name__ == "__main__":
    build(verbose=True)
    sys.exit(0)
