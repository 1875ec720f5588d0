"""Build recipe for the sm_100a shared library (``fuseml_b200/lib/libfuseml_sm100.so``).

The library is compiled in-tree with ``nvcc`` for ``sm_100a`` only; it is the
single native artefact of the package and is loaded through ``ctypes`` by
:mod:`fuseml_b200._native`.  Run ``python -m fuseml_b200.build`` (or call
:func:`build`) after changing anything under ``fuseml_b200/csrc``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libfuseml_sm100.so"
STAMP = LIB_DIR / "libfuseml_sm100.stamp"

SOURCES = ["fuseml_sm100.cu", "host_plan.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-lineinfo",
    "-shared", "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the sm_100a library cannot be built")
    return exe


def source_digest() -> str:
    """SHA-256 over every file the library is built from (sources + headers + flags)."""
    h = hashlib.sha256()
    files = sorted(CSRC.glob("*")) + [PKG_DIR.parent / "include" / "fuseml_sm100.h"]
    for f in files:
        if f.suffix in {".cu", ".cuh", ".cpp", ".h"}:
            h.update(f.name.encode())
            h.update(f.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    return LIB_PATH.exists() and STAMP.exists() and STAMP.read_text().strip() == source_digest()


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile the library if it is missing or older than its sources."""
    if not force and is_current():
        return LIB_PATH
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    cmd = [_nvcc(), *NVCC_FLAGS]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    cmd += ["-o", str(LIB_PATH)] + [str(CSRC / s) for s in SOURCES]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed ({proc.returncode}):\n{proc.stdout}\n{proc.stderr}")
    if verbose:
        sys.stderr.write(proc.stderr)
    STAMP.write_text(source_digest() + "\n")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
