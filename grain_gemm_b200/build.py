"""Build ``libgrain_b200.so`` for sm_100a with nvcc and record what it was built from.

The library is built in-tree, next to this file, together with ``build.json`` (compiler
target, ABI version and the SHA-256 of every source file).  The loader refuses a library
whose manifest does not match the sources beside it, the same provenance rule as the
reference's native bridges (``src/grain_gemm/kernels/moe_gather.py:29-55`` there).

    python -m grain_gemm_b200.build
"""

from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
HEADER = PACKAGE.parent / "include" / "grain_gemm_b200.h"
LIBRARY = PACKAGE / "libgrain_b200.so"
MANIFEST = PACKAGE / "build.json"
ABI_VERSION = 4
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
         "-Xcompiler", "-fPIC", "-shared"]


def sources():
    return sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cuh")) + [HEADER]


def source_hashes():
    return {path.name: hashlib.sha256(path.read_bytes()).hexdigest() for path in sources()}


def find_nvcc():
    candidates = [os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"]
    for candidate in candidates:
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or add the CUDA toolkit to PATH")


def is_current():
    if not LIBRARY.is_file() or not MANIFEST.is_file():
        return False
    try:
        manifest = json.loads(MANIFEST.read_text())
    except (OSError, ValueError):
        return False
    return (manifest.get("abi_version") == ABI_VERSION
            and manifest.get("source_sha256") == source_hashes())


def build_library(force=False, verbose=False):
    """Compile the library unless an up-to-date one is already in place."""
    if not force and is_current():
        return LIBRARY
    nvcc = find_nvcc()
    with tempfile.TemporaryDirectory(dir=PACKAGE) as scratch:
        output = Path(scratch) / LIBRARY.name
        command = [nvcc, *ARCH_FLAGS, *FLAGS, "-o", str(output), str(CSRC / "abi.cu")]
        if verbose:
            command.insert(1, "-Xptxas=-v")
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"nvcc failed:\n{result.stdout}\n{result.stderr}")
        if verbose:
            print(result.stderr)
        os.replace(output, LIBRARY)
    MANIFEST.write_text(json.dumps({
        "architecture": "sm_100",
        "compiler_architecture": "sm_100a",
        "abi_version": ABI_VERSION,
        "flags": ARCH_FLAGS + FLAGS,
        "source_sha256": source_hashes(),
    }, indent=1) + "\n")
    return LIBRARY


if __name__ == "__main__":
    build_library(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(LIBRARY)
