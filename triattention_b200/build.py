"""Ahead-of-time build of the sm_100a C-ABI library (``libtriattn_sm100a.so``, next to this file).

The reference JIT-compiles per detected architecture (``triattention/kernels/extension.py:28-54``);
this build targets sm_100a only, cross-compiles without a GPU, and keeps the reference's
``-O3 --use_fast_math -lineinfo`` flags so that approximate division / exp2 lower identically.

Usage:  python -m triattention_b200.build [--force] [--verbose]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import shutil
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIBRARY = ROOT / "libtriattn_sm100a.so"
SOURCES = ("abi.cu", "kv_write.cu", "decode.cu", "prefill.cu", "tasks.cu")
FLAGS = ("-O3", "-std=c++17", "--use_fast_math", "-lineinfo", "-gencode", "arch=compute_100a,code=sm_100a",
         "-Xcompiler", "-fPIC")


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the sm_100a library cannot be built")
    return found


def _digest() -> str:
    h = hashlib.sha256()
    for path in sorted(CSRC.iterdir()):
        if path.suffix in (".cu", ".cuh", ".h"):
            h.update(path.name.encode())
            h.update(path.read_bytes())
    h.update(" ".join(FLAGS).encode())
    return h.hexdigest()[:16]


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile every .cu for sm_100a into one shared object; skip when sources are unchanged."""
    stamp = ROOT / "build" / "stamp.txt"
    want = _digest()
    if LIBRARY.is_file() and stamp.is_file() and stamp.read_text().strip() == want and not force:
        return LIBRARY
    obj_dir = ROOT / "build"
    obj_dir.mkdir(exist_ok=True)
    objects, procs = [], []
    for name in SOURCES:
        obj = obj_dir / (Path(name).stem + ".o")
        cmd = [nvcc(), *FLAGS, "-I", str(CSRC), "-c", str(CSRC / name), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((name, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    failed = []
    for name, proc in procs:
        out, _ = proc.communicate()
        if verbose or proc.returncode:
            print(f"--- {name}\n{out}")
        if proc.returncode:
            failed.append(name)
    if failed:
        raise RuntimeError(f"nvcc failed for {failed}")
    subprocess.run([nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objects, "-o", str(LIBRARY)], check=True)
    stamp.write_text(want + "\n")
    return LIBRARY


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args()
    print(build_library(args.force, args.verbose))
    os._exit(0)
