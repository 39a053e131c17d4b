"""ctypes view of the C ABI declared in ``include/rlt_kv_handoff.h``.

The library must already be built in-tree (``python -m vllm_rlt_b200._build``).
Loading fails loudly when it is missing: there is no fallback path.
"""

from __future__ import annotations

import ctypes as C
from functools import cache
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
LIB_PATH = PACKAGE / "librlt_kv_handoff.so"

RLT_OK = 0
RLT_E_INVALID, RLT_E_GEOMETRY, RLT_E_LIMIT, RLT_E_CUDA, RLT_E_ALIGN = -1, -2, -3, -4, -5
STATUS_OK, STATUS_BAD_RANGE, STATUS_BAD_BLOCK, STATUS_BAD_PLANE, STATUS_TIMEOUT, STATUS_STALL = 0, 1, 2, 3, 4, 5
STATUS_WORDS = 4
MODE_ALL_PLANES, MODE_DEDUP, MODE_EXIT_ONLY = 0, 1, 2
MAX_REQUESTS = 4096
MAX_SEGMENTS = 4096
MAX_WAIT_NS = 2_000_000_000
IPC_HANDLE_BYTES = 64


class RltRegion(C.Structure):
    _fields_ = [
        ("key", C.c_void_p),
        ("value", C.c_void_p),
        ("block_bytes", C.c_int64),
        ("layer_bytes", C.c_int64),
        ("token_bytes", C.c_int64),
    ]


class RltPool(C.Structure):
    _fields_ = [
        ("codes", RltRegion),
        ("scales", RltRegion),
        ("num_blocks", C.c_int32),
        ("block_size", C.c_int32),
        ("num_layers", C.c_int32),
        ("num_planes", C.c_int32),
    ]


class RltBatch(C.Structure):
    _fields_ = [
        ("num_requests", C.c_int32),
        ("table_width", C.c_int32),
        ("src_tables", C.c_void_p),
        ("dst_tables", C.c_void_p),
        ("tok_begin", C.c_void_p),
        ("tok_end", C.c_void_p),
        ("exit_planes", C.c_void_p),
        ("exit_offsets", C.c_void_p),
        ("exit_count", C.c_int64),
    ]


class RltHostBatch(C.Structure):
    _fields_ = [
        ("num_requests", C.c_int32),
        ("table_width", C.c_int32),
        ("src_planes", C.c_int32),
        ("dst_planes", C.c_int32),
        ("src_tables", C.c_void_p),
        ("dst_tables", C.c_void_p),
        ("tok_begin", C.c_void_p),
        ("tok_end", C.c_void_p),
    ]


class RltOptions(C.Structure):
    _fields_ = [
        ("mode", C.c_int32),
        ("layer_begin", C.c_int32),
        ("layer_end", C.c_int32),
        ("wire_planes", C.c_int32),
        ("status", C.c_void_p),
        ("grid_limit", C.c_int32),
        ("variant", C.c_int32),
        ("workspace", C.c_void_p),
        ("workspace_bytes", C.c_int64),
        ("plane_begin", C.c_int32),
        ("plane_end", C.c_int32),
        ("deep_layer_mask", C.c_uint64),
    ]


# name -> (restype, argtypes); one entry per RLT_API declaration in the header.
SIGNATURES = {
    "rlt_version": (C.c_int, []),
    "rlt_error_string": (C.c_char_p, [C.c_int]),
    "rlt_last_cuda_error": (C.c_int, []),
    "rlt_kernel_launches": (C.c_int64, []),
    "rlt_kv_handoff": (C.c_int, [C.POINTER(RltPool), C.POINTER(RltPool), C.POINTER(RltBatch), C.POINTER(RltOptions), C.c_void_p]),
    "rlt_kv_handoff_host": (C.c_int, [C.POINTER(RltPool), C.POINTER(RltPool), C.POINTER(RltHostBatch), C.POINTER(RltOptions), C.c_void_p]),
    "rlt_kv_host_batch_limit": (C.c_int64, []),
    "rlt_kv_dedup_workspace_bytes": (C.c_int64, [C.c_int32, C.c_int32, C.c_int32]),
    "rlt_kv_packed_bytes": (C.c_int64, [C.POINTER(RltPool), C.c_int64, C.c_int32, C.c_int32]),
    "rlt_kv_pack": (C.c_int, [C.POINTER(RltPool), C.POINTER(RltBatch), C.POINTER(RltOptions), C.c_void_p, C.c_int64, C.c_void_p]),
    "rlt_kv_pack_dedup_static": (C.c_int, [C.POINTER(RltPool), C.POINTER(RltBatch), C.POINTER(RltOptions), C.c_void_p, C.c_int64, C.c_void_p]),
    "rlt_kv_static_plan_entries": (C.c_int64, []),
    "rlt_kv_scatter": (C.c_int, [C.c_void_p, C.c_int64, C.POINTER(RltPool), C.POINTER(RltBatch), C.POINTER(RltOptions), C.c_void_p]),
    "rlt_kv_finalize": (C.c_int, [C.POINTER(RltPool), C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_uint64, C.c_void_p, C.c_void_p]),
    "rlt_tensor_transfer": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "rlt_tensor_copy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_void_p]),
    "rlt_kv_push": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "rlt_kv_copy_segments": (C.c_int, [C.c_void_p, C.c_int32, C.c_void_p]),
    "rlt_kv_signal": (C.c_int, [C.c_void_p, C.c_uint64, C.c_void_p]),
    "rlt_kv_wait": (C.c_int, [C.c_void_p, C.c_uint64, C.c_int64, C.c_void_p, C.c_void_p]),
    "rlt_kv_post": (C.c_int, [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]),
    "rlt_host_register": (C.c_int, [C.c_void_p, C.c_size_t, C.POINTER(C.c_void_p)]),
    "rlt_host_unregister": (C.c_int, [C.c_void_p]),
    "rlt_peer_enable": (C.c_int, [C.c_int, C.c_int]),
    "rlt_peer_can_access": (C.c_int, [C.c_int, C.c_int]),
    "rlt_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_int64)]),
    "rlt_ipc_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "rlt_ipc_close": (C.c_int, [C.c_void_p]),
}


@cache
def load() -> C.CDLL:
    """Load the C-ABI library once and attach prototypes. Raises if it is not built."""
    if not LIB_PATH.is_file():
        raise RuntimeError(
            f"{LIB_PATH.name} is not built: run `python -m vllm_rlt_b200._build`. "
            "The KV handoff has no CPU or PyTorch fallback."
        )
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    return lib


OPS_PATH = PACKAGE / "_C.so"


def ops_built() -> bool:
    """Whether the torch op library sits in the tree. Looks at the file only: nothing is loaded, no CUDA context."""
    return OPS_PATH.is_file()


@cache
def load_ops():
    """Register ``torch.ops.vllm_rlt.kv_*`` by loading the in-tree op library; returns the op namespace.

    The reference finds its op library by importing ``vllm_rlt._C`` and treats a missing module as "optional
    kernels absent" (vllm_rlt/kernels/_extension.py:8-23). These ops are not optional: a library that was never
    built raises here, and a library that exists but cannot be loaded (wrong torch, missing symbol) lets the
    loader's own error through. A successful load is remembered; a failure is not, so a later build is picked up.
    """
    if not ops_built():
        raise RuntimeError(
            f"{OPS_PATH.name} is not built: run `python -m vllm_rlt_b200._build`. "
            "The KV-handoff ops have CUDA implementations only."
        )
    import torch

    torch.ops.load_library(str(OPS_PATH))
    return torch.ops.vllm_rlt


class RltError(RuntimeError):
    def __init__(self, code: int, where: str):
        lib = load()
        text = lib.rlt_error_string(code).decode()
        extra = f" (cudaError {lib.rlt_last_cuda_error()})" if code == RLT_E_CUDA else ""
        super().__init__(f"{where}: {text}{extra}")
        self.code = code


def check(code: int, where: str) -> None:
    if code != RLT_OK:
        if code in (RLT_E_INVALID, RLT_E_GEOMETRY, RLT_E_LIMIT, RLT_E_ALIGN):
            raise ValueError(str(RltError(code, where)))
        raise RltError(code, where)
