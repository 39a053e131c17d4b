"""Python face of the KV-handoff kernels: argument checking and the C-ABI calls.

These wrappers play the role that ``vllm_rlt/kernels/activation.py`` plays for
the reference's one native op: validate on the host, then launch on the
caller's current CUDA stream without synchronising. There is no fallback: if
the native library is not built, or no CUDA device is present, the calls raise.

Reference behaviour that is kept: bad ranges and tables raise ``ValueError``
with the messages of ``kv_segments`` (vllm_rlt/pd/transport.py:29-47).
"""

from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Sequence

import numpy as np
import torch

from .. import _lib
from .._lib import MODE_ALL_PLANES, MODE_DEDUP, MODE_EXIT_ONLY  # noqa: F401  (re-exported)


def _stream_ptr(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


# --------------------------------------------------------------------------- pools


@dataclass(frozen=True)
class Region:
    """One K/V tensor pair as raw pointers and byte strides (``_kv_region``, vllm_rlt/pd/transport.py:18-26)."""

    key_ptr: int
    value_ptr: int
    block_bytes: int
    layer_bytes: int
    token_bytes: int

    @classmethod
    def of(cls, key: torch.Tensor, value: torch.Tensor) -> "Region":
        if key.shape != value.shape or key.dtype != value.dtype or key.device != value.device:
            raise ValueError("key and value tensors must agree in shape, dtype and device")
        if key.dim() < 4 or not key.is_contiguous() or not value.is_contiguous():
            raise ValueError("pool tensors must be contiguous [blocks, layers, block_size, ...]")
        e = key.element_size()
        return cls(key.data_ptr(), value.data_ptr(), key.stride(0) * e, key.stride(1) * e, key.stride(2) * e)

    def rebased(self, key_ptr: int, value_ptr: int) -> "Region":
        return Region(key_ptr, value_ptr, self.block_bytes, self.layer_bytes, self.token_bytes)

    def as_struct(self) -> _lib.RltRegion:
        return _lib.RltRegion(self.key_ptr, self.value_ptr, self.block_bytes, self.layer_bytes, self.token_bytes)


_NO_REGION = _lib.RltRegion(None, None, 0, 0, 0)


@dataclass(frozen=True)
class PoolView:
    """Geometry and addresses of one paged KV pool, local or mapped from a peer GPU.

    ``scales`` is set only when scale tensors travel: a dynamic-scale FP8 pool.
    A fixed-scale FP8 pool keeps its (constant) scale tensors out of the handoff,
    as the reference does (vllm_rlt/pd/transport.py:132-137).
    """

    codes: Region
    scales: Region | None
    num_blocks: int
    block_size: int
    num_layers: int
    num_planes: int
    device: int
    keepalive: tuple = field(default=(), compare=False, repr=False)

    @classmethod
    def from_tensors(cls, key, value, num_planes, key_scale=None, value_scale=None) -> "PoolView":
        if not key.is_cuda:
            raise ValueError("KV pools must live on a CUDA device: the handoff has no CPU path")
        codes = Region.of(key, value)
        scales = None
        keep = (key, value)
        if key_scale is not None:
            if key_scale.shape != key.shape[:-1] or key_scale.dtype != torch.float32:
                raise ValueError("scale tensors must be float32 [blocks, layers, block_size, kv_heads]")
            scales = Region.of(key_scale, value_scale)
            keep += (key_scale, value_scale)
        return cls(codes, scales, key.shape[0], key.shape[2], key.shape[1], int(num_planes), key.device.index, keep)

    @classmethod
    def from_cache(cls, cache) -> "PoolView":
        """From a ``KVCacheManager``-shaped object (vllm_rlt/core/kv_cache_manager.py:261-271)."""
        dynamic = cache.key_scale is not None and cache.fp8_scale is None
        return cls.from_tensors(
            cache.key_cache,
            cache.value_cache,
            cache.storage_depths,
            cache.key_scale if dynamic else None,
            cache.value_scale if dynamic else None,
        )

    def as_struct(self) -> _lib.RltPool:
        return _lib.RltPool(
            self.codes.as_struct(),
            self.scales.as_struct() if self.scales is not None else _NO_REGION,
            self.num_blocks,
            self.block_size,
            self.num_layers,
            self.num_planes,
        )

    @property
    def row_bytes(self) -> int:
        return self.codes.token_bytes + (self.scales.token_bytes if self.scales is not None else 0)

    def payload_bytes(self, tokens: int, planes: int, layers: int | None = None) -> int:
        """Algorithmic payload of ``tokens`` tokens over ``planes`` planes."""
        return 2 * (self.num_layers if layers is None else layers) * self.row_bytes * tokens * planes


# --------------------------------------------------------------------------- batches


class _Staging:
    """One pinned host buffer; reusable once the copy that read it has completed."""

    def __init__(self, capacity: int):
        self.buffer = torch.empty(capacity, dtype=torch.uint8, pin_memory=True)
        self.event = None

    def free(self) -> bool:
        return self.event is None or self.event.query()

    def release(self) -> None:
        self.event = torch.cuda.Event()
        self.event.record()


class _PinnedPool:
    """Pinned staging buffers are costly to allocate (a driver call each), so they are kept and reused."""

    def __init__(self):
        self.buffers: list[_Staging] = []

    def acquire(self, size: int) -> _Staging:
        for b in self.buffers:
            if b.buffer.numel() >= size and b.free():
                b.event = None
                return b
        capacity = 1 << max(16, (size - 1).bit_length())
        b = _Staging(capacity)
        if len(self.buffers) < 64:
            self.buffers.append(b)
        return b


_PINNED = _PinnedPool()


class HandoffBatch:
    """Per-request tables and ranges, staged in pinned memory and copied to the device once.

    ``src_tables[r]`` / ``dst_tables[r]`` are the per-plane block tables of request
    ``r`` (``plane_block_tables``); ``ranges[r]`` is its token range; ``exit_planes[r]``
    (optional) holds one zero-based exit plane per token position of the request.
    Validation mirrors ``kv_segments``: same conditions, same messages.
    """

    def __init__(
        self,
        src_tables: Sequence[Sequence[Sequence[int]]] | None,
        dst_tables: Sequence[Sequence[Sequence[int]]] | None,
        ranges: Sequence[tuple[int, int]],
        *,
        block_size: int,
        exit_planes: Sequence[Sequence[int]] | None = None,
        src_blocks: int | None = None,
        dst_blocks: int | None = None,
        device=None,
        stream=None,
    ):
        n = len(ranges)
        if n < 1:
            raise ValueError("a handoff batch needs at least one request")
        if n > _lib.MAX_REQUESTS:
            raise ValueError(f"a handoff batch holds at most {_lib.MAX_REQUESTS} requests")
        self.num_requests = n
        self.block_size = block_size
        bounds = np.asarray(ranges, dtype=np.int64).reshape(n, 2)
        begin, end = bounds[:, 0], bounds[:, 1]
        if ((begin < 0) | (begin >= end)).any():
            raise ValueError("invalid KV range")
        self.ranges = [(int(s), int(e)) for s, e in bounds]
        self.total_tokens = int((end - begin).sum())
        # Per side: one int32 array [requests, planes, pages], zero-padded to the longest table. The checks are those of
        # the reference's planner, done on whole arrays.
        sides, width = [], 1
        for tables, limit in ((src_tables, src_blocks), (dst_tables, dst_blocks)):
            if tables is None:
                sides.append(None)
                continue
            if len(tables) != n:
                raise ValueError("one table set per request is required")
            planes = len(tables[0])
            if any(len(req) != planes for req in tables):
                raise ValueError("requests of one batch must have the same number of planes")
            pages0 = len(tables[0][0])
            if all(len(table) == pages0 for req in tables for table in req):
                # tables of one length (a single request, or a chunk's trimmed tables): one conversion, no padding
                padded = np.asarray(tables, dtype=np.int32).reshape(n, planes, pages0)
                if (end > pages0 * block_size).any():
                    raise ValueError("KV range exceeds allocation")
                pages_max = pages0
            else:
                rows = [table for req in tables for table in req]
                lens = np.fromiter(map(len, rows), np.int64, count=n * planes).reshape(n, planes)
                pages = lens[:, 0]
                if (end > lens.min(axis=1) * block_size).any():
                    raise ValueError("KV range exceeds allocation")
                if (lens != pages[:, None]).any():
                    raise ValueError("the planes of one request must have tables of equal length")
                total = int(lens.sum())
                if isinstance(rows[0], np.ndarray):
                    flat = np.concatenate(rows).astype(np.int32, copy=False)
                else:
                    flat = np.fromiter((b for table in rows for b in table), np.int32, count=total)
                pages_max = int(pages.max())
                padded = np.zeros((n, planes, pages_max), np.int32)
                # a boolean mask is filled in row-major order, which is the order of the flat array
                padded.reshape(n * planes, pages_max)[np.arange(pages_max) < lens.reshape(-1)[:, None]] = flat
            width = max(width, pages_max)
            sides.append((padded, limit))
        self.table_width = width
        arrays = []
        used = None
        for side in sides:
            if side is None:
                arrays.append(None)
                continue
            a, limit = side
            if a.shape[2] < width:  # the two sides share one width
                wider = np.zeros((n, a.shape[1], width), np.int32)
                wider[:, :, : a.shape[2]] = a
                a = wider
            # negative ids compare as huge unsigned numbers; the padding (0) is a valid id, so the mask of
            # pages that the ranges touch is only needed when something looks wrong
            bad = a < 0 if limit is None else a.view(np.uint32) >= limit
            if bad.any():
                if used is None:
                    cols = np.arange(width)
                    used = (cols >= (begin // block_size)[:, None]) & (cols <= ((end - 1) // block_size)[:, None])
                if (bad & used[:, None, :]).any():
                    raise ValueError("physical block outside registered pool")
            arrays.append(np.ascontiguousarray(a))
        self.src_planes = arrays[0].shape[1] if arrays[0] is not None else 0
        self.dst_planes = arrays[1].shape[1] if arrays[1] is not None else 0
        exit_parts = offsets = None
        exit_count = 0
        if exit_planes is not None:
            if len(exit_planes) != n:
                raise ValueError("one exit-plane array per request is required")
            exit_parts = [np.asarray(e, np.int32) for e in exit_planes]
            counts = np.fromiter(map(len, exit_parts), np.int64, count=n)
            if any(e.ndim != 1 for e in exit_parts) or (counts < end).any():
                raise ValueError("exit planes must cover every token position up to the range end")
            offsets = np.cumsum(counts) - counts
            exit_count = int(counts.sum())
        # One pinned staging buffer, one host-to-device copy; int64 data first for alignment. The exit planes,
        # the largest piece, are gathered straight into the staging buffer.
        pieces = [("exit_offsets", offsets), ("src_tables", arrays[0]), ("dst_tables", arrays[1]),
                  ("tok_begin", begin.astype(np.int32)), ("tok_end", end.astype(np.int32))]
        layout, size = {}, 0
        for name, a in pieces:
            if a is None:
                continue
            size = (size + 15) & ~15
            layout[name] = (size, a)
            size += a.nbytes
        if exit_parts is not None:
            size = (size + 15) & ~15
            layout["exit_planes"] = (size, None)
            size += 4 * exit_count
        self.metadata_bytes = size
        device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        staging = _PINNED.acquire(size)
        host = staging.buffer.numpy()
        for name, (at, a) in layout.items():
            if a is not None:
                host[at : at + a.nbytes] = a.reshape(-1).view(np.uint8)
            elif exit_count:
                np.concatenate(exit_parts, out=host[at : at + 4 * exit_count].view(np.int32))
        self._dev = torch.empty(size, dtype=torch.uint8, device=device)
        with torch.cuda.device(device), torch.cuda.stream(stream if stream is not None else torch.cuda.current_stream(device)):
            self._dev.copy_(staging.buffer[:size], non_blocking=True)
            staging.release()
        exits = exit_parts
        base = self._dev.data_ptr()
        self._ptr = {name: base + at for name, (at, _) in layout.items()}
        self.has_exit = exits is not None
        self.exit_count = exit_count

    @classmethod
    def from_device(cls, src_tables, dst_tables, tok_begin, tok_end, *, block_size: int, exit_planes=None,
                    exit_offsets=None) -> "HandoffBatch":
        """A batch whose arrays already sit in device memory, for instance block tables and exit planes that a peer
        sent over NCCL: nothing is staged, copied or read back. ``src_tables`` / ``dst_tables`` are contiguous int32
        ``[requests, planes, width]`` (either may be None), ``tok_begin`` / ``tok_end`` int32 ``[requests]``,
        ``exit_planes`` int32 with one entry per token and ``exit_offsets`` int64 ``[requests]``. No host-side
        validation is possible; the kernels check ranges, block ids and exit planes and report through the status words.
        """
        tables = src_tables if src_tables is not None else dst_tables
        if tables is None or tables.dim() != 3:
            raise ValueError("block tables must be [requests, planes, width]")
        n, _, width = tables.shape
        if not 1 <= n <= _lib.MAX_REQUESTS:
            raise ValueError(f"a handoff batch holds 1 to {_lib.MAX_REQUESTS} requests")
        checks = [(src_tables, torch.int32, "src_tables"), (dst_tables, torch.int32, "dst_tables"),
                  (tok_begin, torch.int32, "tok_begin"), (tok_end, torch.int32, "tok_end"),
                  (exit_planes, torch.int32, "exit_planes"), (exit_offsets, torch.int64, "exit_offsets")]
        for t, dtype, name in checks:
            if t is not None and (not t.is_cuda or t.dtype != dtype or not t.is_contiguous()):
                raise ValueError(f"{name} must be a contiguous CUDA {dtype} tensor")
        if src_tables is not None and dst_tables is not None and (src_tables.shape[0] != n or dst_tables.shape[0] != n or
                                                                  src_tables.shape[2] != dst_tables.shape[2]):
            raise ValueError("source and destination tables must agree in requests and width")
        if tok_begin.numel() != n or tok_end.numel() != n:
            raise ValueError("one token range per request is required")
        if (exit_planes is None) != (exit_offsets is None) or (exit_offsets is not None and exit_offsets.numel() != n):
            raise ValueError("exit_planes and exit_offsets come as a pair, one offset per request")
        self = cls.__new__(cls)
        self.num_requests, self.table_width, self.block_size = n, width, block_size
        self.ranges, self.total_tokens = None, None
        self.src_planes = src_tables.shape[1] if src_tables is not None else 0
        self.dst_planes = dst_tables.shape[1] if dst_tables is not None else 0
        self.metadata_bytes = 0
        self._dev = (src_tables, dst_tables, tok_begin, tok_end, exit_planes, exit_offsets)  # keeps them alive
        names = ("src_tables", "dst_tables", "tok_begin", "tok_end", "exit_planes", "exit_offsets")
        self._ptr = {name: t.data_ptr() for name, t in zip(names, self._dev) if t is not None}
        self.has_exit = exit_planes is not None
        self.exit_count = exit_planes.numel() if exit_planes is not None else 0
        return self

    def as_struct(self) -> _lib.RltBatch:
        g = self._ptr.get
        return _lib.RltBatch(
            self.num_requests, self.table_width, g("src_tables"), g("dst_tables"),
            g("tok_begin"), g("tok_end"), g("exit_planes"), g("exit_offsets"), self.exit_count,
        )


def new_status(device=None) -> torch.Tensor:
    """A zeroed int32 status word array the kernels report data errors into."""
    return torch.zeros(_lib.STATUS_WORDS, dtype=torch.int32, device=device or "cuda")


_STATUS_TEXT = {
    _lib.STATUS_BAD_RANGE: "KV range exceeds allocation",
    _lib.STATUS_BAD_BLOCK: "physical block outside registered pool",
    _lib.STATUS_BAD_PLANE: "exit plane outside the pool's planes",
    _lib.STATUS_TIMEOUT: "timed out waiting for the peer's completion flag",
    _lib.STATUS_STALL: "a bulk copy did not complete within the wait limit",
}


def raise_for_status(status: torch.Tensor) -> None:
    """Synchronising read of a status array; raises like the reference's planner would have."""
    words = status.tolist()
    if words[0] == _lib.STATUS_OK:
        return
    text = _STATUS_TEXT.get(words[0], f"device status {words[0]}")
    if words[0] == _lib.STATUS_STALL:
        raise RuntimeError(f"{text} (CTA {words[1]}, warp {words[2]})")
    if words[0] == _lib.STATUS_TIMEOUT:
        raise TimeoutError(f"{text} (last value {words[1]})")
    raise ValueError(f"{text} (request {words[1]}, detail {words[2]}, {words[3]})")


def _options(mode, layer_begin, layer_end, wire_planes, status, grid_limit, variant, workspace=None,
             plane_begin=0, plane_end=0, deep_layer_mask=0) -> _lib.RltOptions:
    if workspace is not None and (workspace.dtype != torch.uint8 or not workspace.is_contiguous() or not workspace.is_cuda):
        raise ValueError("workspace must be a contiguous CUDA uint8 tensor")
    return _lib.RltOptions(
        int(mode), int(layer_begin), int(layer_end), int(wire_planes),
        status.data_ptr() if status is not None else None, int(grid_limit), int(variant),
        workspace.data_ptr() if workspace is not None else None, workspace.numel() if workspace is not None else 0,
        int(plane_begin), int(plane_end), int(deep_layer_mask),
    )


def dedup_workspace(batch: "HandoffBatch", planes: int, device=None) -> torch.Tensor:
    """Scratch tensor for pack/scatter in ``MODE_DEDUP`` (holds the wire plan of the batch)."""
    n = _lib.load().rlt_kv_dedup_workspace_bytes(batch.num_requests, batch.table_width, planes)
    if n < 0:
        _lib.check(int(n), "rlt_kv_dedup_workspace_bytes")
    return torch.empty(int(n), dtype=torch.uint8, device=device or "cuda")


def dedup_wire_tokens(workspace: torch.Tensor) -> int:
    """(token, plane) pairs on the wire of the last dedup pack/scatter that used ``workspace`` (synchronises)."""
    return int(workspace[:8].view(torch.int64).item())


# --------------------------------------------------------------------------- ops


def kv_handoff(src: PoolView, dst: PoolView, batch: HandoffBatch, *, mode=MODE_ALL_PLANES,
               layer_begin=0, layer_end=0, plane_begin=0, plane_end=0, deep_layers=None, status=None, stream=None,
               grid_limit=0, variant=0) -> None:
    """Pool-to-pool handoff of a batch, straight from source blocks to destination blocks.

    ``layer_begin/layer_end`` and ``plane_begin/plane_end`` restrict the launch to a slice of layers and
    destination planes (0, 0 = everything), which is what layer-by-layer streaming uses. ``deep_layers`` lists
    the layers carried for planes >= 1 (a recurrent-depth model's recurrent layers); plane 0 carries them all.
    """
    lib = _lib.load()
    mask = 0
    if deep_layers is not None:
        for layer in deep_layers:
            if not 0 <= layer < min(src.num_layers, 64):
                raise ValueError("recurrent_layers must be valid cache layer indices")
            mask |= 1 << layer
        if mask == 0:
            raise ValueError("recurrent_layers must be nonempty and unique")
    s, d, b = src.as_struct(), dst.as_struct(), batch.as_struct()
    o = _options(mode, layer_begin, layer_end, 0, status, grid_limit, variant, None, plane_begin, plane_end, mask)
    _lib.check(lib.rlt_kv_handoff(C.byref(s), C.byref(d), C.byref(b), C.byref(o), _stream_ptr(stream)), "rlt_kv_handoff")


def host_batch_limit() -> int:
    """Largest sum of table and range bytes ``kv_handoff_host`` accepts."""
    return int(_lib.load().rlt_kv_host_batch_limit())


def kv_handoff_host(src: PoolView, dst: PoolView, src_tables: np.ndarray, dst_tables: np.ndarray, tok_begin: np.ndarray,
                    tok_end: np.ndarray, *, layer_begin=0, layer_end=0, plane_begin=0, plane_end=0, status=None,
                    stream=None) -> None:
    """All-planes handoff of a small batch whose tables are host arrays: the library stages them in a slot of its own
    and queues copy and launch on ``stream`` (``rlt_kv_handoff_host``); the arrays are free again on return.

    ``src_tables`` / ``dst_tables`` are C-contiguous int32 ``[requests, planes, width]`` of one width, ``tok_begin`` /
    ``tok_end`` int32 ``[requests]``. Nothing is validated on the host beyond shapes; the kernel checks block ids and
    ranges and reports through ``status``. Raises ``ValueError`` with the library's limit message when the batch does
    not fit a staging slot."""
    arrays = (src_tables, dst_tables, tok_begin, tok_end)
    if any(a.dtype != np.int32 or not a.flags.c_contiguous for a in arrays):
        raise ValueError("host tables and ranges must be C-contiguous int32 arrays")
    n, src_planes, width = src_tables.shape
    if dst_tables.shape[0] != n or dst_tables.shape[2] != width or tok_begin.shape != (n,) or tok_end.shape != (n,):
        raise ValueError("source and destination tables must agree in requests and width, one range per request")
    hb = _lib.RltHostBatch(n, width, src_planes, dst_tables.shape[1], src_tables.ctypes.data, dst_tables.ctypes.data,
                           tok_begin.ctypes.data, tok_end.ctypes.data)
    s, d = src.as_struct(), dst.as_struct()
    o = _options(MODE_ALL_PLANES, layer_begin, layer_end, 0, status, 0, 0, None, plane_begin, plane_end, 0)
    _lib.check(_lib.load().rlt_kv_handoff_host(C.byref(s), C.byref(d), C.byref(hb), C.byref(o), _stream_ptr(stream)),
               "rlt_kv_handoff_host")


def packed_bytes(pool: PoolView, total_tokens: int, wire_planes: int, layers: int | None = None) -> int:
    lib = _lib.load()
    s = pool.as_struct()
    n = lib.rlt_kv_packed_bytes(C.byref(s), total_tokens, wire_planes, pool.num_layers if layers is None else layers)
    if n < 0:
        _lib.check(int(n), "rlt_kv_packed_bytes")
    return int(n)


def kv_pack(src: PoolView, batch: HandoffBatch, out: torch.Tensor, *, mode=MODE_ALL_PLANES, layer_begin=0,
            layer_end=0, wire_planes=0, status=None, stream=None, grid_limit=0, variant=0, workspace=None) -> None:
    """Gather a batch into ``out`` (uint8, contiguous) in the reference's segment order."""
    if out.dtype != torch.uint8 or not out.is_contiguous() or not out.is_cuda:
        raise ValueError("packed buffer must be a contiguous CUDA uint8 tensor")
    lib = _lib.load()
    s, b = src.as_struct(), batch.as_struct()
    o = _options(mode, layer_begin, layer_end, wire_planes, status, grid_limit, variant, workspace)
    _lib.check(lib.rlt_kv_pack(C.byref(s), C.byref(b), C.byref(o), out.data_ptr(), out.numel(), _stream_ptr(stream)), "rlt_kv_pack")


def kv_pack_to(src: PoolView, batch: HandoffBatch, out_ptr: int, out_bytes: int, *, mode=MODE_ALL_PLANES, layer_begin=0,
               layer_end=0, wire_planes=0, status=None, stream=None, grid_limit=0, variant=0, workspace=None) -> None:
    """``kv_pack`` into raw memory, typically a staging buffer on the decode GPU mapped through a peer pointer:
    the gather and the push over NVLink become one kernel and nothing is staged on the prefill side."""
    lib = _lib.load()
    s, b = src.as_struct(), batch.as_struct()
    o = _options(mode, layer_begin, layer_end, wire_planes, status, grid_limit, variant, workspace)
    _lib.check(lib.rlt_kv_pack(C.byref(s), C.byref(b), C.byref(o), out_ptr, out_bytes, _stream_ptr(stream)), "rlt_kv_pack")


def kv_scatter(packed: torch.Tensor, dst: PoolView, batch: HandoffBatch, *, mode=MODE_ALL_PLANES, layer_begin=0,
               layer_end=0, wire_planes=0, status=None, stream=None, grid_limit=0, variant=0, workspace=None) -> None:
    """Write a packed image into the destination blocks of a batch."""
    if packed.dtype != torch.uint8 or not packed.is_contiguous() or not packed.is_cuda:
        raise ValueError("packed buffer must be a contiguous CUDA uint8 tensor")
    lib = _lib.load()
    d, b = dst.as_struct(), batch.as_struct()
    o = _options(mode if mode == MODE_DEDUP else MODE_ALL_PLANES, layer_begin, layer_end, wire_planes, status,
                 grid_limit, variant, workspace)
    _lib.check(lib.rlt_kv_scatter(packed.data_ptr(), packed.numel(), C.byref(d), C.byref(b), C.byref(o), _stream_ptr(stream)), "rlt_kv_scatter")


def kv_finalize(pool: PoolView, tables: torch.Tensor, rows: torch.Tensor, *, layers=None, status=None, stream=None) -> None:
    """Copy each row's exit-plane K/V (and scales) into every deeper plane.

    ``tables`` is the pool's device ``int32 [requests, planes, width]``; ``rows`` is a device
    ``int32 [n, 3]`` of (request index, exit plane, token position); ``layers`` lists the layers to
    copy (default all; pass the model's recurrent layers for boundary-KV models). For scale tensors
    to be copied the view must carry them: build it with ``PoolView.from_tensors(..., key_scale,
    value_scale)`` also for a fixed-scale pool.
    """
    for t, name, cols in ((tables, "tables", None), (rows, "rows", 3)):
        if t.dtype != torch.int32 or not t.is_contiguous() or not t.is_cuda:
            raise ValueError(f"{name} must be a contiguous CUDA int32 tensor")
    if tables.dim() != 3 or tables.shape[1] != pool.num_planes:
        raise ValueError("tables must be [requests, planes, width] with the pool's plane count")
    if rows.dim() != 2 or rows.shape[1] != 3:
        raise ValueError("rows must be [n, 3]: request index, exit plane, token position")
    mask = 0
    if layers is not None:
        for layer in layers:
            if not 0 <= layer < pool.num_layers:
                raise ValueError("recurrent_layers must be valid cache layer indices")
            mask |= 1 << layer
        if mask == 0:
            raise ValueError("recurrent_layers must be nonempty and unique")
    s = pool.as_struct()
    _lib.check(
        _lib.load().rlt_kv_finalize(C.byref(s), tables.data_ptr(), tables.shape[0], tables.shape[2], rows.data_ptr(),
                                    rows.shape[0], mask, status.data_ptr() if status is not None else None,
                                    _stream_ptr(stream)),
        "rlt_kv_finalize",
    )


def kv_push(src_ptr: int, dst_ptr: int, nbytes: int, *, stream=None) -> None:
    """Copy one byte range; ``dst_ptr`` may be a peer mapping."""
    _lib.check(_lib.load().rlt_kv_push(src_ptr, dst_ptr, nbytes, _stream_ptr(stream)), "rlt_kv_push")


def kv_copy_segments(segments: torch.Tensor, *, stream=None) -> None:
    """Copy ``int64 [n, 3]`` (source address, destination address, bytes) triples held on the device."""
    if segments.dtype != torch.int64 or segments.dim() != 2 or segments.shape[1] != 3 or not segments.is_contiguous():
        raise ValueError("segments must be a contiguous int64 [n, 3] tensor")
    if not segments.is_cuda:
        raise ValueError("segments must live on the device")
    _lib.check(_lib.load().rlt_kv_copy_segments(segments.data_ptr(), segments.shape[0], _stream_ptr(stream)), "rlt_kv_copy_segments")


def kv_signal(flag_ptr: int, value: int, *, stream=None) -> None:
    _lib.check(_lib.load().rlt_kv_signal(flag_ptr, value, _stream_ptr(stream)), "rlt_kv_signal")


def kv_wait(flag_ptr: int, value: int, timeout_ns: int, status: torch.Tensor, *, stream=None) -> None:
    _lib.check(_lib.load().rlt_kv_wait(flag_ptr, value, timeout_ns, status.data_ptr(), _stream_ptr(stream)), "rlt_kv_wait")


def kernel_launches() -> int:
    return int(_lib.load().rlt_kernel_launches())
