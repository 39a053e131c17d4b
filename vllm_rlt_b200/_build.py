"""In-tree build of the native code: the C-ABI CUDA library and the torch op library.

Everything is compiled for sm_100a only, with explicit ``nvcc`` / ``g++``
commands, into files that sit inside the package directory so that they travel
with a source snapshot. Nothing is cached outside the tree.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
INCLUDE = ROOT / "include"

LIB_NAME = "librlt_kv_handoff.so"
OPS_NAME = "_C.so"

CUDA_SOURCES = ["lib.cu", "kv_table_copy.cu", "kv_segment_copy.cu", "kv_finalize.cu", "tensor_transfer.cu",
                "kv_signal.cu", "peer.cu"]
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for candidate in (os.environ.get("CUDA_HOME"), "/usr/local/cuda"):
        if candidate and (Path(candidate) / "bin" / "nvcc").is_file():
            return str(Path(candidate) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found is None:
        raise RuntimeError("nvcc not found: the KV-handoff kernels cannot be built")
    return found


def _fingerprint(command: list[str], inputs: list[Path]) -> str:
    """Hash of everything a build step depends on: the command line and the bytes of every input file."""
    h = hashlib.sha256()
    h.update("\0".join(command).encode())
    for path in inputs:
        h.update(b"\0" + path.name.encode() + b"\0")
        h.update(path.read_bytes())
    return h.hexdigest()


def _stamp(target: Path) -> Path:
    return target.with_name(target.name + ".stamp")


def _stale(target: Path, fingerprint: str) -> bool:
    """A binary is reused only if the stamp written beside it by the build that made it carries the same
    fingerprint and the binary's own hash: a binary compiled from other sources, with other flags, or
    replaced since, is rebuilt whatever its modification time says."""
    stamp = _stamp(target)
    if not target.is_file() or not stamp.is_file():
        return True
    recorded = stamp.read_text().split()
    return recorded != [fingerprint, hashlib.sha256(target.read_bytes()).hexdigest()]


def _record(target: Path, fingerprint: str) -> None:
    _stamp(target).write_text(f"{fingerprint} {hashlib.sha256(target.read_bytes()).hexdigest()}\n")


def _run(cmd: list[str], show: bool = False) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build step failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if show:
        print(proc.stdout + proc.stderr)


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """Compile the C-ABI library (no torch types, static cudart)."""
    target = PACKAGE / LIB_NAME
    sources = [CSRC / s for s in CUDA_SOURCES]
    deps = sources + [CSRC / "common.cuh", INCLUDE / "rlt_kv_handoff.h"]
    flags = [*ARCH, "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden"]
    fingerprint = _fingerprint(flags, deps)
    if force or verbose or _stale(target, fingerprint):
        cmd = [_nvcc(), *flags, f"-I{INCLUDE}", "-shared", "-o", str(target), *map(str, sources), "-ldl"]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        _run(cmd, show=verbose)
        _record(target, fingerprint)
    return target


def build_ops(force: bool = False) -> Path:
    """Compile the torch op library that registers ``torch.ops.vllm_rlt.kv_*`` over the C ABI."""
    import torch
    from torch.utils import cpp_extension

    target = PACKAGE / OPS_NAME
    source = CSRC / "torch_bindings.cpp"
    deps = [source, CSRC / "ops.h", INCLUDE / "rlt_kv_handoff.h", PACKAGE / LIB_NAME]
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    flags = ["-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_EXTENSION_NAME=_C",
             f"torch={torch.__version__}"]
    fingerprint = _fingerprint(flags, deps)
    if force or _stale(target, fingerprint):
        includes = [f"-I{p}" for p in cpp_extension.include_paths("cuda")] + [f"-I{INCLUDE}", f"-I{CSRC}"]
        import sysconfig

        includes.append(f"-I{sysconfig.get_paths()['include']}")
        torch_lib = Path(torch.__file__).parent / "lib"
        cmd = ["g++", *flags[:-1], *includes, str(source), "-o", str(target),
               f"-L{PACKAGE}", "-l:" + LIB_NAME, f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-lc10",
               "-ltorch_cuda", "-lc10_cuda", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
        _run(cmd)
        _record(target, fingerprint)
    return target


def build_all(force: bool = False) -> None:
    build_library(force)
    build_ops(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", PACKAGE / LIB_NAME, PACKAGE / OPS_NAME)
