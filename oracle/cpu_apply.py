"""ctypes wrapper of the oracle's threaded CPU applier (``apply_segments.c``). Test infrastructure only."""

import ctypes
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "liboracle_apply.so"


def build() -> Path:
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    return LIB


def load():
    if not LIB.is_file():
        build()
    lib = ctypes.CDLL(str(LIB))
    lib.rlt_oracle_apply.restype = ctypes.c_int64
    lib.rlt_oracle_apply.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int]
    return lib


def apply(triples: np.ndarray, threads: int) -> int:
    """Copy every (src address, dst address, bytes) row of an int64 [n, 3] array of REAL host addresses."""
    triples = np.ascontiguousarray(triples, np.int64)
    n = load().rlt_oracle_apply(triples.ctypes.data, len(triples), threads)
    if n < 0:
        raise ValueError("bad segment list")
    return int(n)
