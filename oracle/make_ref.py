"""Installs the unmodified reference package into ``oracle/_ref`` (git-ignored).  TEST INFRASTRUCTURE.

The reference's own GPU path on a B200 is its Triton backend (``backend="triton"``, which its
``auto`` policy selects for compute capability 10.0: ``src/grain_gemm/gemm.py:104-119``,
``src/grain_gemm/moe.py:242-251``).  Installed beside the oracle it serves two purposes on a GPU
box, both in the tests and the benchmark's context figures only, never in the product:

* a second, bit-level oracle: full-size BF16/FP32 GEMM outputs and whole ``moe_ffn`` results of
  the reference itself (the one place where libdevice ``expf`` is evaluated);
* the "what a user of the reference gets on this GPU today" timing next to ours.

Nothing is copied into the repository's history: the install goes through pip from the
read-only reference tree (``GRAIN_REFERENCE``, default: a ``reference`` folder beside this
repository) via a temporary copy,
``--no-deps``, and lands in ``oracle/_ref`` only.  Only its Triton kernels are ever called; the
reference's native (CuTe/CUTLASS) sources are removed from the install and never built.

    python oracle/make_ref.py
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
import tempfile
from pathlib import Path

HERE = Path(__file__).resolve().parent
TARGET = HERE / "_ref"


def reference_root() -> Path:
    return Path(os.environ.get("GRAIN_REFERENCE", str(HERE.parents[1] / "reference")))


def is_installed() -> bool:
    return (TARGET / "grain_gemm" / "__init__.py").is_file()


def install(force: bool = False) -> bool:
    """Install when the reference tree is present; returns whether ``oracle/_ref`` is usable."""
    root = reference_root()
    if is_installed() and not force:
        return True
    if not (root / "pyproject.toml").is_file():
        return False
    with tempfile.TemporaryDirectory() as scratch:
        copy = Path(scratch) / "reference"
        shutil.copytree(root, copy, ignore=shutil.ignore_patterns(".git", "benchmarks", "experiments",
                                                                   "docs", "tests"))
        command = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index",
                   "--no-build-isolation", "--no-deps", "--upgrade", "--target", str(TARGET), str(copy)]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            sys.stderr.write(result.stdout + result.stderr)
            return False
    # Only the Python/Triton side is used: the package's C++/CUDA sources are not needed.
    shutil.rmtree(TARGET / "grain_gemm" / "kernels" / "csrc", ignore_errors=True)
    return is_installed()


def load():
    """Import the installed reference under the name ``grain_gemm_reference`` (the repository has
    its own ``grain_gemm`` drop-in package; the two must not be confused).  None when absent."""
    import importlib.util

    if not is_installed():
        return None
    name = "grain_gemm_reference"
    if name in sys.modules:
        return sys.modules[name]
    package = TARGET / "grain_gemm"
    spec = importlib.util.spec_from_file_location(name, package / "__init__.py",
                                                  submodule_search_locations=[str(package)])
    module = importlib.util.module_from_spec(spec)
    sys.modules[name] = module
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    ok = install(force="--force" in sys.argv)
    print(TARGET if ok else "reference not installed")
    sys.exit(0 if ok else 1)
