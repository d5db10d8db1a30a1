"""Build the probe library (``tests/probe/libtriattn_probe.so``) for sm_100a: the test-only operand-layout probe
(umma_probe.cu) and the measurement-only INT8 tensor-peak kernel that bench.py times (i8_peak.cu).

Usage:  python tests/probe/build_probe.py [--force]
"""
from __future__ import annotations

import argparse
import ctypes
import hashlib
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
LIBRARY = HERE / "libtriattn_probe.so"

_P, _I, _U = ctypes.c_void_p, ctypes.c_int, ctypes.c_uint32
ARGTYPES = [_P, _I, _P, _I, _U, _U, _U, _U, _U, _U, _U, _U, _U, _I, _I, _I, _P, _P, _P]


def build(force: bool = False) -> Path:
    from triattention_b200.build import CSRC, FLAGS, nvcc
    sources = [HERE / "umma_probe.cu", HERE / "i8_peak.cu"]
    h = hashlib.sha256()
    for path in sources + [CSRC / name for name in ("tcgen05.cuh", "common.cuh", "abi_internal.h")]:
        h.update(path.read_bytes())
    stamp, want = HERE / "stamp.txt", h.hexdigest()[:16]
    if LIBRARY.is_file() and stamp.is_file() and stamp.read_text().strip() == want and not force:
        return LIBRARY
    subprocess.run([nvcc(), *FLAGS, "-I", str(CSRC), "-shared", *map(str, sources), "-o", str(LIBRARY)], check=True)
    stamp.write_text(want + "\n")
    return LIBRARY


def load() -> ctypes.CDLL:
    if not LIBRARY.is_file():
        raise FileNotFoundError(f"{LIBRARY} is missing; run tests/probe/build_probe.py")
    lib = ctypes.CDLL(str(LIBRARY))
    lib.tri_umma_probe.argtypes, lib.tri_umma_probe.restype = ARGTYPES, ctypes.c_int
    lib.tri_probe_last_error.argtypes, lib.tri_probe_last_error.restype = [], ctypes.c_char_p
    lib.tri_i8_peak.argtypes = [_I, _I, ctypes.POINTER(ctypes.c_int64), _P, _P]
    lib.tri_i8_peak.restype = ctypes.c_int
    return lib


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    print(build(parser.parse_args().force))
