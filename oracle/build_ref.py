"""Build the reference's own CUDA extension into ``oracle/_ref/`` (test infrastructure only).

The reference ships no CPU implementation and no sm_100 kernel: on a B200 its loader
(``triattention/kernels/extension.py:23-25,45``) compiles ``kernels/cuda/prefill_sm80.cu`` with
``-O3 --use_fast_math -gencode=arch=compute_100,code=sm_100``.  This recipe runs the same nvcc
command line directly on the reference's source files where they lie (nothing is copied into
this repository) and writes one pybind11 module, ``oracle/_ref/triattention_ref.so``.

The module can only *run* on a GPU.  GPU parity tests import it as the authoritative oracle and
``tests/golden/make_golden.py`` uses it to record golden vectors.  Product code never imports it.

The reference checkout is named by ``--reference`` or the ``TRIATTENTION_REFERENCE`` environment variable; without
either, a directory called ``reference`` beside this repository is used if it holds the sources.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--force]
"""
from __future__ import annotations

import argparse
import hashlib
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT = HERE / "_ref"
NAME = "triattention_ref"


def find_reference() -> Path | None:
    """The reference checkout: $TRIATTENTION_REFERENCE, else a `reference` directory beside this repository."""
    named = os.environ.get("TRIATTENTION_REFERENCE")
    for candidate in ([Path(named)] if named else []) + [HERE.parent.parent / "reference"]:
        if (candidate / "triattention" / "kernels" / "cuda" / "prefill_sm80.cu").is_file():
            return candidate
    return None


def command(reference: Path) -> list[str]:
    import torch
    from torch.utils import cpp_extension as ce

    cuda_dir = reference / "triattention" / "kernels" / "cuda"
    cmd = ["nvcc", "-O3", "-std=c++17", "--use_fast_math", "-lineinfo",
           "-gencode=arch=compute_100,code=sm_100", *ce.COMMON_NVCC_FLAGS,
           "-Xcompiler", "-fPIC", "-shared", f"-DTORCH_EXTENSION_NAME={NAME}", "-DTORCH_API_INCLUDE_EXTENSION_H",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in [*ce.include_paths(), sysconfig.get_paths()["include"], str(cuda_dir)]:
        cmd += ["-I", inc]
    cmd += [str(cuda_dir / "prefill_sm80.cu"), "-o", str(OUT / f"{NAME}.so")]
    for lib in ce.library_paths():
        cmd += ["-L", lib, f"-Xlinker=-rpath={lib}"]
    cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python"]
    return cmd


def digest(reference: Path) -> str:
    cuda_dir = reference / "triattention" / "kernels" / "cuda"
    h = hashlib.sha256()
    for name in ("prefill_sm80.cu", "common_device.cuh", "common_host.cuh"):
        h.update((cuda_dir / name).read_bytes())
    return h.hexdigest()[:16]


def build(reference: Path, force: bool = False) -> Path | None:
    """Compile if the sources are present and the stamp is stale; return the .so path or None."""
    so, stamp = OUT / f"{NAME}.so", OUT / "stamp.txt"
    if not (reference / "triattention" / "kernels" / "cuda" / "prefill_sm80.cu").is_file():
        return so if so.is_file() else None
    want = digest(reference)
    if so.is_file() and stamp.is_file() and stamp.read_text().strip() == want and not force:
        return so
    OUT.mkdir(exist_ok=True)
    subprocess.run(command(reference), check=True)
    stamp.write_text(want + "\n")
    return so


def load():
    """Import the built module (GPU tests / golden generation only)."""
    import importlib.util

    import torch  # noqa: F401  (the module links against libtorch)

    so = OUT / f"{NAME}.so"
    if not so.is_file():
        raise FileNotFoundError(f"{so} is missing; run oracle/build_ref.py where the reference is mounted")
    spec = importlib.util.spec_from_file_location(NAME, so)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--reference", default=None)
    parser.add_argument("--force", action="store_true")
    args = parser.parse_args()
    where = Path(args.reference) if args.reference else find_reference()
    path = build(where, args.force) if where is not None else None
    print(path if path else "reference sources not found; nothing built")
    sys.exit(0)
