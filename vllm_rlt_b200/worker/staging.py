"""Host-side staging for per-submission metadata: pinned snapshots the device reads in place, and batched writes.

Counterparts of the reference's ``UvaBuffer``, ``UvaBufferPool``, ``UvaBackedTensor``, ``StagedInputTensor`` and
``StagedWriteTensor`` (vllm_rlt/worker/tensors.py:95-280, :368-419), with the same method names and the same
ownership rule: none of these objects synchronises or decides when its storage may be overwritten; the
submission owner retires a slot's readers before the slot comes round again.

How they work here. A snapshot is a slot of pinned host memory. Pinned memory is mapped into the device's address
space, so a kernel of this library can read a snapshot where it lies (``use_uva=True``, the default): staging
costs one CPU copy and no launch. With ``use_uva=False`` the slot is copied to a device tensor of the same
shape with ``rlt_tensor_copy`` on the current stream, for consumers that must not touch host memory (a CUDA
graph input). Slots rotate round-robin; a slot grows to the next power of two when a submission needs more
rows than it has, and only that slot. Destinations are CUDA tensors: there is no CPU path.
"""

from __future__ import annotations

import torch

from .tensors import TensorTransfer, copy_tensor

SLOTS = 2  # submissions that may be in flight at once (MAX_CONCURRENT_SUBMISSIONS, vllm_rlt/worker/submission_queue.py:5)


def _cuda_device(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise ValueError("staging targets a CUDA device: this library has no CPU path")
    return torch.device("cuda", torch.cuda.current_device()) if device.index is None else device


def _rows_for(count: int) -> int:
    return 1 << max(0, (count - 1).bit_length())


class UvaBuffer:
    """One pinned snapshot slot with a kernel-readable view of it."""

    def __init__(self, shape, dtype, device, *, use_uva=True, target=None):
        self.device = _cuda_device(device)
        self.use_uva = bool(use_uva)
        self.cpu = torch.empty(shape, dtype=dtype, pin_memory=True)
        if target is not None and (target.shape != self.cpu.shape or target.dtype != dtype or target.device != self.device):
            raise ValueError("fallback target must match buffer shape, dtype and device")
        self._device_copy = None if self.use_uva else target

    @property
    def np(self):
        """NumPy view of the slot (bfloat16 has none: write that dtype through ``.cpu``)."""
        return self.cpu.numpy()

    def stage(self, count=None):
        """The first ``count`` rows as something a kernel can read: the slot itself, or its device copy queued on
        the current stream. Does not wait and does not make the slot reusable."""
        host = self.cpu if count is None else self.cpu[:count]
        if self.use_uva:
            return host
        if self._device_copy is None:
            self._device_copy = torch.empty_like(self.cpu, device=self.device)
        view = self._device_copy if count is None else self._device_copy[:count]
        if host.numel():
            copy_tensor(host, view)
        return view


class UvaBufferPool:
    """Rotating snapshot slots; ``acquire`` hands out the next one, grown if the submission needs more rows."""

    def __init__(self, shape, dtype, device, *, use_uva=True, max_concurrency=SLOTS):
        if max_concurrency < 1:
            raise ValueError("UVA pool capacity must be positive")
        self.buffers = [UvaBuffer(shape, dtype, device, use_uva=use_uva) for _ in range(max_concurrency)]
        self.index = 0

    def acquire(self, count=None):
        slot = self.buffers[self.index]
        if count is not None and count > slot.cpu.shape[0]:
            grown = (_rows_for(count), *slot.cpu.shape[1:])
            slot = self.buffers[self.index] = UvaBuffer(grown, slot.cpu.dtype, slot.device, use_uva=slot.use_uva)
        self.index = (self.index + 1) % len(self.buffers)
        return slot

    def _snapshot(self, source):
        if source.device.type != "cpu":
            raise ValueError("UVA snapshot source must be a CPU tensor")
        if source.shape[1:] != self.buffers[0].cpu.shape[1:]:
            raise ValueError("UVA snapshot trailing dimensions do not match")
        slot = self.acquire(len(source))
        slot.cpu[: len(source)].copy_(source)
        return slot

    def stage(self, source):
        """Snapshot a CPU tensor into the next slot and return its kernel-readable view."""
        return self._snapshot(source).stage(len(source))

    def copy_to_gpu(self, source, out=None):
        """Snapshot a CPU tensor and queue its copy into a new device tensor, or into ``out``."""
        device = self.buffers[0].device
        if out is not None and (out.shape != source.shape or out.device != device):
            raise ValueError("output must match the input shape and configured device")
        snapshot = self._snapshot(source).cpu[: len(source)]
        if out is None:
            out = torch.empty(source.shape, dtype=source.dtype, device=device)
        if snapshot.numel():
            copy_tensor(snapshot.reshape(-1), out.reshape(-1) if out.is_contiguous() else out)
        return out


class UvaBackedTensor:
    """Mutable CPU state published as rotating pinned snapshots: ``publish`` is one CPU copy, nothing else."""

    def __init__(self, shape, dtype, device, *, max_concurrency=SLOTS):
        self.cpu = torch.empty(shape, dtype=dtype)
        self.pool = UvaBufferPool(shape, dtype, device, max_concurrency=max_concurrency)

    @property
    def np(self):
        return self.cpu.numpy()

    def publish(self, count=None):
        source = self.cpu if count is None else self.cpu[:count]
        snapshot = self.pool.acquire(len(source)).cpu[: len(source)]
        snapshot.copy_(source)
        return snapshot


class StagedInputTensor:
    """Append CPU values piece by piece, then upload the whole flat array once per submission.

    ``append`` returns the CPU slice that now holds the values; its offsets stay valid through growth, and the same
    slice taken on the tensor ``upload`` returns holds the same values on the device."""

    def __init__(self, dtype, device, *, use_uva=True):
        self.dtype, self.device, self.use_uva = dtype, _cuda_device(device), use_uva
        self.cpu = torch.empty(0, dtype=dtype)
        self.pool = UvaBufferPool(0, dtype, self.device)
        self.targets = [None] * SLOTS
        self.count = 0

    def reset(self):
        self.count = 0

    def append(self, values):
        if isinstance(values, torch.Tensor) and values.device.type != "cpu":
            raise ValueError("staged input values must be CPU-owned")
        begin, end = self.count, self.count + len(values)
        if end > self.cpu.numel():
            bigger = torch.empty(_rows_for(end), dtype=self.dtype)
            bigger[:begin] = self.cpu[:begin]
            self.cpu = bigger
        piece = self.cpu[begin:end]
        piece.copy_(values if isinstance(values, torch.Tensor) else torch.tensor(values, dtype=self.dtype))
        self.count = end
        return piece

    def upload(self):
        which = self.pool.index
        slot = self.pool.acquire(self.count)
        snapshot = slot.cpu[: self.count]
        snapshot.copy_(self.cpu[: self.count])
        target = self.targets[which]
        if target is None or target.numel() < slot.cpu.numel():
            target = self.targets[which] = torch.empty(slot.cpu.numel(), dtype=self.dtype, device=self.device)
        if self.count:
            copy_tensor(snapshot, target[: self.count])
        return target[: self.count]


class StagedWriteTensor:
    """Collect small writes into rows of a caller-owned device tensor; ``submit`` snapshots the values and moves
    all of them with one segmented launch. Values are copied when staged: later changes by the caller do not
    reach the device."""

    def __init__(self, tensor, initial_writes, initial_values, *, use_uva=True):
        self.gpu = tensor
        self.contents = UvaBufferPool(initial_values, tensor.dtype, tensor.device, max_concurrency=1)
        self.writes = initial_writes
        self.transfers = TensorTransfer(initial_writes, tensor.dtype, tensor.device)
        self.reset()

    def stage_write(self, index, start, values):
        count = len(values)
        if not count:
            return
        row = self.gpu[index]
        if row.ndim != 1 or start < 0 or start + count > row.numel():
            raise ValueError("staged write range is outside the target row")
        if isinstance(values, torch.Tensor):
            if values.device.type != "cpu":
                raise ValueError("staged values must be CPU-owned")
            values = values.tolist()
        self.values.extend(values)
        self.targets.append(row[start : start + count])

    def submit(self):
        if not self.values:
            return
        total = len(self.values)
        snapshot = self.contents.acquire(total).cpu[:total]
        snapshot.copy_(torch.tensor(self.values, dtype=snapshot.dtype))
        if len(self.targets) > self.transfers.capacity:
            self.transfers = TensorTransfer(_rows_for(len(self.targets)), self.gpu.dtype, self.gpu.device)
        self.transfers.reset()
        at = 0
        for target in self.targets:
            self.transfers.append(snapshot[at : at + target.numel()], target)
            at += target.numel()
        self.transfers.submit()

    def reset(self):
        self.values, self.targets = [], []
        self.transfers.reset()
