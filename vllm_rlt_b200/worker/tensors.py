"""Typed tensor transfer on one device (or from pinned host memory to the device) over the native kernels.

Same contract as the reference's ``copy_tensor`` and ``TensorTransfer``
(vllm_rlt/worker/tensors.py:35-87, :282-365): equal-sized contiguous tensors for the flat copy, batches of
disjoint 1-D/2-D copies of one (source type, target type) pair for the segmented one, the five transfer
dtypes, and the same ``ValueError`` conditions, including the refusal of copies between two different CUDA
devices (those go through the handoff connector). There is no CPU or PyTorch fallback here: targets must be
CUDA tensors and host sources must be pinned.
"""

from __future__ import annotations

import torch

from .. import _lib

_DTYPES = {torch.int32: 0, torch.int64: 1, torch.float16: 2, torch.bfloat16: 3, torch.float32: 4}


def _check_source(source: torch.Tensor, device: torch.device) -> None:
    if source.is_cuda:
        if source.device != device:
            raise ValueError("cross-device transfers require an explicit connector")
    elif not source.is_pinned():
        raise ValueError("host sources must be pinned: this transfer has no pageable-memory path")


def copy_tensor(source: torch.Tensor, target: torch.Tensor, *, secondary: torch.Tensor | None = None) -> torch.Tensor:
    """Copy contiguous values to their final storage, optionally writing a second typed output."""
    if source.numel() != target.numel() or not source.is_contiguous() or not target.is_contiguous():
        raise ValueError("copy_tensor requires equal-sized contiguous tensors")
    if secondary is not None and (
        secondary.numel() != source.numel() or not secondary.is_contiguous() or secondary.device != target.device
    ):
        raise ValueError("secondary output must match target size and device")
    if source.dtype not in _DTYPES or target.dtype not in _DTYPES or (secondary is not None and secondary.dtype not in _DTYPES):
        raise ValueError("unsupported transfer dtype")
    if not target.is_cuda:
        raise ValueError("transfer destination must be a CUDA tensor")
    _check_source(source, target.device)
    if source.numel() == 0:
        return target
    with torch.cuda.device(target.device):
        _lib.check(
            _lib.load().rlt_tensor_copy(
                source.data_ptr(), target.data_ptr(), secondary.data_ptr() if secondary is not None else None,
                source.numel(), _DTYPES[source.dtype], _DTYPES[target.dtype],
                _DTYPES[secondary.dtype] if secondary is not None else 0, torch.cuda.current_stream().cuda_stream),
            "rlt_tensor_copy",
        )
    return target


class TensorTransfer:
    """One typed batch of disjoint 1-D/2-D copies with borrowed tensor references.

    ``append`` records a copy, ``submit`` launches the whole batch as one kernel, ``reset`` forgets it.
    Descriptors are written into a pinned table that the kernel reads through its device mapping, so a
    submission needs no separate host-to-device copy. The table and the tensors of a submitted batch must
    stay untouched until the work queued behind ``submit`` has completed.
    """

    def __init__(self, capacity: int, dtype: torch.dtype, device, *, target_dtype: torch.dtype | None = None):
        self.dtype, self.target_dtype = dtype, target_dtype or dtype
        if self.dtype not in _DTYPES or self.target_dtype not in _DTYPES:
            raise ValueError("unsupported transfer dtype")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("transfer destination must be a CUDA device")
        self.capacity = capacity
        self.table = torch.zeros((capacity, 8), dtype=torch.int64, pin_memory=True)
        self.table_np = self.table.numpy()
        self.reset()

    def reset(self) -> None:
        self.copies: list[tuple[torch.Tensor, torch.Tensor]] = []
        self.max_rows = self.max_cols = 0

    def append(self, source: torch.Tensor, target: torch.Tensor) -> None:
        if source.shape != target.shape or source.ndim not in (1, 2):
            raise ValueError("transfer requires matching 1D/2D shapes")
        if source.dtype != self.dtype or target.dtype != self.target_dtype:
            raise ValueError("transfer dtype does not match its batch")
        if target.device != self.device:
            raise ValueError("transfer destination must be on the configured device")
        if source.is_cuda and source.device != self.device:
            raise ValueError("transfer source must be on the configured device")
        _check_source(source, self.device)
        if source.numel() == 0:
            return
        if len(self.copies) == self.capacity:
            raise ValueError("transfer batch is full")
        rows, cols = (1, source.shape[0]) if source.ndim == 1 else source.shape
        self.copies.append((source, target))
        self.max_rows, self.max_cols = max(self.max_rows, rows), max(self.max_cols, cols)

    def submit(self) -> None:
        if not self.copies:
            return
        for index, (source, target) in enumerate(self.copies):
            src = source.unsqueeze(0) if source.ndim == 1 else source
            dst = target.unsqueeze(0) if target.ndim == 1 else target
            self.table_np[index] = (src.data_ptr(), dst.data_ptr(), *src.shape, *src.stride(), *dst.stride())
        with torch.cuda.device(self.device):
            _lib.check(
                _lib.load().rlt_tensor_transfer(
                    self.table.data_ptr(), len(self.copies), self.max_rows, self.max_cols, _DTYPES[self.dtype],
                    _DTYPES[self.target_dtype], torch.cuda.current_stream().cuda_stream),
                "rlt_tensor_transfer",
            )
