"""Per-submission metadata on its way to the GPU: pinned host rows that kernels read where they lie.

The runner-facing names and contracts are those of vllm-rlt's staging helpers (vllm_rlt/worker/tensors.py:95-280 and
:368-419: ``UvaBuffer``, ``UvaBufferPool``, ``UvaBackedTensor``, ``StagedInputTensor``, ``StagedWriteTensor``), so code
written against them runs unchanged; what stands behind the names is this library's. Nothing here waits for the GPU
or decides when host memory may be overwritten: whoever submits work retires a slot's readers before the slot comes
round again (two submissions may be in flight, vllm_rlt/worker/submission_queue.py:5).

Mechanism. All host memory is page-locked, and page-locked memory is visible to the device at the same address, so
the transfer kernels of this library (``rlt_tensor_copy``, ``rlt_tensor_transfer``) take a host row range as their
source directly: publishing a snapshot costs one CPU copy and no launch. A consumer that must not touch host memory (a
CUDA-graph input) asks for ``use_uva=False`` and gets a device mirror filled by ``rlt_tensor_copy`` on the current
stream. Row capacity doubles on demand, slot by slot. There is no CPU destination: the device is always CUDA.
"""

from __future__ import annotations

import torch

from .tensors import TensorTransfer, copy_tensor

IN_FLIGHT = 2  # submissions whose snapshots may still be read


def _resolve(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError("staging targets a CUDA device: this library has no CPU path")
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def _capacity_for(rows: int) -> int:
    """Smallest power of two that holds ``rows`` (1 for none)."""
    return 1 << max(rows - 1, 0).bit_length()


class UvaBuffer:
    """Pinned rows plus, on request, a device mirror of them."""

    def __init__(self, shape, dtype, device, *, use_uva=True, target=None):
        self.device = _resolve(device)
        self.use_uva = bool(use_uva)
        self.cpu = torch.empty(shape, dtype=dtype, pin_memory=True)
        if target is not None:
            same = target.shape == self.cpu.shape and target.dtype == self.cpu.dtype and target.device == self.device
            if not same:
                raise ValueError("fallback target must match buffer shape, dtype and device")
        self._mirror = target if not self.use_uva else None

    @property
    def np(self):
        """The rows as a NumPy array (bfloat16 has no NumPy form: fill that dtype through ``.cpu``)."""
        return self.cpu.numpy()

    def rows(self, count=None):
        return self.cpu if count is None else self.cpu.narrow(0, 0, count)

    def stage(self, count=None):
        """What a kernel should read for the first ``count`` rows: the pinned rows themselves, or the mirror after
        queueing its refresh on the current stream. Returns at once; the rows stay owned by the caller's submission."""
        host = self.rows(count)
        if self.use_uva:
            return host
        if self._mirror is None:
            self._mirror = torch.empty(self.cpu.shape, dtype=self.cpu.dtype, device=self.device)
        mirror = self._mirror if count is None else self._mirror.narrow(0, 0, count)
        if host.numel() > 0:
            copy_tensor(host, mirror)
        return mirror

    def regrown(self, rows: int) -> "UvaBuffer":
        """A fresh buffer of the same kind with room for ``rows`` rows (contents are not carried over: a snapshot is
        always written whole)."""
        return UvaBuffer((_capacity_for(rows), *self.cpu.shape[1:]), self.cpu.dtype, self.device, use_uva=self.use_uva)


class UvaBufferPool:
    """``max_concurrency`` buffers handed out in turn. ``index`` names the one the next ``acquire`` returns."""

    def __init__(self, shape, dtype, device, *, use_uva=True, max_concurrency=IN_FLIGHT):
        if max_concurrency < 1:
            raise ValueError("UVA pool capacity must be positive")
        self.buffers = []
        while len(self.buffers) < max_concurrency:
            self.buffers.append(UvaBuffer(shape, dtype, device, use_uva=use_uva))
        self.index = 0

    @property
    def device(self) -> torch.device:
        return self.buffers[0].device

    def acquire(self, count=None):
        """The buffer whose turn it is, replaced by a larger one first if ``count`` rows do not fit."""
        turn, self.index = self.index, (self.index + 1) % len(self.buffers)
        if count is not None and self.buffers[turn].cpu.shape[0] < count:
            self.buffers[turn] = self.buffers[turn].regrown(count)
        return self.buffers[turn]

    def _snapshot(self, source):
        """Copy a CPU tensor into the next buffer; returns ``(buffer, rows written)``."""
        if source.device.type != "cpu":
            raise ValueError("UVA snapshot source must be a CPU tensor")
        if tuple(source.shape[1:]) != tuple(self.buffers[0].cpu.shape[1:]):
            raise ValueError("UVA snapshot trailing dimensions do not match")
        rows = source.shape[0]
        buffer = self.acquire(rows)
        buffer.rows(rows).copy_(source)
        return buffer, rows

    def stage(self, source):
        """Snapshot ``source`` and return the kernel-readable form of the snapshot."""
        buffer, rows = self._snapshot(source)
        return buffer.stage(rows)

    def copy_to_gpu(self, source, out=None):
        """Snapshot ``source`` and queue its transfer into ``out`` (or into a new device tensor), read straight from
        the snapshot."""
        if out is not None and (out.shape != source.shape or out.device != self.device):
            raise ValueError("output must match the input shape and configured device")
        buffer, rows = self._snapshot(source)
        if out is None:
            out = torch.empty(source.shape, dtype=source.dtype, device=self.device)
        if source.numel() > 0:
            copy_tensor(buffer.rows(rows).reshape(-1), out.reshape(-1) if out.is_contiguous() else out)
        return out


class UvaBackedTensor:
    """CPU state that changes between submissions; ``publish`` freezes its current value in the next pinned slot
    (one CPU copy) and returns that slot's rows for kernels to read."""

    def __init__(self, shape, dtype, device, *, max_concurrency=IN_FLIGHT):
        self.pool = UvaBufferPool(shape, dtype, device, max_concurrency=max_concurrency)
        self.cpu = torch.empty(shape, dtype=dtype)

    @property
    def np(self):
        return self.cpu.numpy()

    def publish(self, count=None):
        live = self.cpu if count is None else self.cpu.narrow(0, 0, count)
        frozen = self.pool.acquire(live.shape[0]).rows(live.shape[0])
        frozen.copy_(live)
        return frozen


class StagedInputTensor:
    """A flat typed array assembled on the CPU piece by piece and sent to the device once per submission.

    ``append`` hands back the CPU slice that received the values. Slices are positions in the flat array: they stay
    valid when the array grows, and the device tensor that ``upload`` returns holds the same values at the same
    positions. Consecutive uploads alternate between device tensors, so the previous submission can still read its own.
    """

    def __init__(self, dtype, device, *, use_uva=True):
        self.dtype, self.use_uva = dtype, use_uva
        self.device = _resolve(device)
        self.pool = UvaBufferPool(0, dtype, self.device)
        self.targets: list[torch.Tensor | None] = [None for _ in self.pool.buffers]
        self.cpu = torch.empty(0, dtype=dtype)
        self.count = 0

    def reset(self):
        self.count = 0

    def _reserve(self, extra: int) -> slice:
        where = slice(self.count, self.count + extra)
        if where.stop > self.cpu.shape[0]:
            roomier = torch.empty(_capacity_for(where.stop), dtype=self.dtype)
            roomier[: self.count] = self.cpu[: self.count]
            self.cpu = roomier
        self.count = where.stop
        return where

    def append(self, values):
        on_device = isinstance(values, torch.Tensor) and values.device.type != "cpu"
        if on_device:
            raise ValueError("staged input values must be CPU-owned")
        where = self._reserve(len(values))
        piece = self.cpu[where]  # taken after a possible growth
        piece.copy_(torch.as_tensor(values, dtype=self.dtype))
        return piece

    def upload(self):
        turn = self.pool.index
        frozen = self.pool.acquire(self.count).rows(self.count)
        frozen.copy_(self.cpu[: self.count])
        if self.targets[turn] is None or self.targets[turn].shape[0] < self.count:
            self.targets[turn] = torch.empty(_capacity_for(self.count), dtype=self.dtype, device=self.device)
        sent = self.targets[turn][: self.count]
        if self.count:
            copy_tensor(frozen, sent)
        return sent


class StagedWriteTensor:
    """Small writes into rows of a device tensor the caller owns, gathered on the CPU and applied by ONE segmented
    launch per ``submit``. The values are taken at ``stage_write`` time; the launch reads them from a pinned snapshot."""

    def __init__(self, tensor, initial_writes, initial_values, *, use_uva=True):
        self.gpu = tensor
        self.writes = initial_writes
        self.contents = UvaBufferPool(initial_values, tensor.dtype, tensor.device, max_concurrency=1)
        self.transfers = TensorTransfer(initial_writes, tensor.dtype, tensor.device)
        self.values: list = []
        self.targets: list[torch.Tensor] = []

    def reset(self):
        self.values, self.targets = [], []
        self.transfers.reset()

    def stage_write(self, index, start, values):
        if len(values) == 0:
            return
        if isinstance(values, torch.Tensor):
            if values.device.type != "cpu":
                raise ValueError("staged values must be CPU-owned")
            values = values.tolist()
        row = self.gpu[index]
        if row.ndim != 1 or start < 0 or start + len(values) > row.shape[0]:
            raise ValueError("staged write range is outside the target row")
        self.targets.append(row[start : start + len(values)])
        self.values += values

    def submit(self):
        if not self.targets:
            return
        frozen = self.contents.acquire(len(self.values)).rows(len(self.values))
        frozen.copy_(torch.tensor(self.values, dtype=frozen.dtype))
        if self.transfers.capacity < len(self.targets):
            self.transfers = TensorTransfer(_capacity_for(len(self.targets)), self.gpu.dtype, self.gpu.device)
        self.transfers.reset()
        begin = 0
        for target in self.targets:
            self.transfers.append(frozen[begin : begin + target.shape[0]], target)
            begin += target.shape[0]
        self.transfers.submit()
