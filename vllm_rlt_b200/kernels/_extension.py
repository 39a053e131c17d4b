"""Load the torch op library once. Same contract as the reference's loader (vllm_rlt/kernels/_extension.py:8-23):
a library that was never built is reported as unavailable (and that answer is cached), any other import error
propagates, and nothing here creates a CUDA context."""

from functools import cache
from importlib import import_module


@cache
def try_load_extension() -> bool:
    try:
        import_module("vllm_rlt_b200._C")
    except ModuleNotFoundError as exc:
        if exc.name != "vllm_rlt_b200._C":
            raise
        return False
    return True


def load_extension() -> None:
    if not try_load_extension():
        raise RuntimeError("Native KV-handoff ops are not built: run `python -m vllm_rlt_b200._build`.")
