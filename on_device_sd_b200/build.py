"""Builds libb200moe.so in-tree with nvcc for sm_100a (no other architecture is supported).

    python -m on_device_sd_b200.build [--force] [--verbose]

The shared library lands next to this file so that it travels with the source tree; nothing
is installed into site-packages and no JIT cache is used.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "libb200moe.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr", "--extended-lambda",
]


def _defines() -> list[str]:
    d = []
    if (CSRC / "ffn_int4.cuh").exists():
        d.append("-DB200MOE_WITH_INT4")
    if (CSRC / "ffn_umma.cuh").exists():
        d.append("-DB200MOE_WITH_UMMA")
    return d


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PKG.parent / "include" / "b200moe.h", Path(__file__)]
    return any(p.stat().st_mtime > t for p in deps)


def nvcc_path() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; libb200moe.so cannot be built")


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not _stale():
        return LIB
    cmd = [nvcc_path(), *NVCC_FLAGS, *_defines(), "-I", str(PKG.parent / "include"), "-o", str(LIB)]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += [str(s) for s in _sources()]
    cmd += ["-lcuda"] if (CSRC / "ffn_umma.cuh").exists() else []
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed building libb200moe.so:\n" + res.stderr[-4000:])
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIB)
