"""Build the in-tree CUDA library ``sparkinfer_b200/_b12x_b200.so`` for sm_100a.

    python -m sparkinfer_b200.build [--force] [--verbose]

nvcc cross-compiles without a GPU. The object is rebuilt when any source under ``csrc/`` or
the public header is newer than it.
"""

from __future__ import annotations

import argparse
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
HEADER = PKG.parent / "include" / "b12x_b200.h"
OUTPUT = PKG / "_b12x_b200.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-shared", "-Xcompiler", "-fPIC",
    "--fmad=false",  # the quantizers must round every product; nothing else is FMA-bound
]


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def dependencies() -> list[Path]:
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [HEADER]


def needs_build() -> bool:
    if not OUTPUT.exists():
        return True
    built = OUTPUT.stat().st_mtime
    return any(dep.stat().st_mtime > built for dep in dependencies())


def build(force: bool = False, verbose: bool = False) -> Path:
    if not force and not needs_build():
        return OUTPUT
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    cmd = [nvcc, *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(OUTPUT), *map(str, sources())]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}): {' '.join(cmd)}")
    return OUTPUT


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args()
    print(build(force=args.force, verbose=args.verbose))


if __name__ == "__main__":
    main()
