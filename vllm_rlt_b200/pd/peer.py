"""Peer-memory handles: how a prefill worker gets a writable pointer into the decode worker's pools.

The reference registers its pools with a NIXL agent and ships the agent's metadata in the
start-up handshake (vllm_rlt/pd/transport.py:131-154). Here every pool tensor is exported
as a CUDA IPC handle plus a byte offset, small enough to ride in the same handshake message
(``startup_info()["info"]``); the peer opens the handle once and adds the offset.
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib


def export_tensor(t: torch.Tensor) -> dict:
    """IPC handle (hex) and offset of a CUDA tensor's storage; valid while the tensor lives."""
    if not t.is_cuda:
        raise ValueError("only CUDA tensors can be exported to a peer")
    handle = (C.c_uint8 * _lib.IPC_HANDLE_BYTES)()
    offset = C.c_int64(0)
    with torch.cuda.device(t.device):
        _lib.check(_lib.load().rlt_ipc_export(t.data_ptr(), handle, C.byref(offset)), "rlt_ipc_export")
    return {"handle": bytes(handle).hex(), "offset": int(offset.value), "bytes": t.numel() * t.element_size(),
            "device": t.device.index}


class PeerMapping:
    """Allocations of other processes mapped into this one; one open per distinct handle."""

    def __init__(self):
        self._bases: dict[str, int] = {}

    def pointer(self, exported: dict) -> int:
        key = exported["handle"]
        base = self._bases.get(key)
        if base is None:
            raw = (C.c_uint8 * _lib.IPC_HANDLE_BYTES).from_buffer_copy(bytes.fromhex(key))
            out = C.c_void_p()
            _lib.check(_lib.load().rlt_ipc_open(raw, C.byref(out)), "rlt_ipc_open")
            base = self._bases[key] = int(out.value)
        return base + exported["offset"]

    def close(self) -> None:
        """Unmap everything. Call on the writer before the owner frees its memory."""
        lib = _lib.load()
        for base in self._bases.values():
            _lib.check(lib.rlt_ipc_close(base), "rlt_ipc_close")
        self._bases.clear()


def enable_peer_access(device: int, peer: int) -> None:
    """Single-process form: let ``device`` address memory of ``peer`` directly."""
    lib = _lib.load()
    ok = lib.rlt_peer_can_access(device, peer)
    if ok < 0:
        _lib.check(ok, "rlt_peer_can_access")
    if ok == 0:
        raise RuntimeError(f"device {device} cannot access memory of device {peer}")
    _lib.check(lib.rlt_peer_enable(device, peer), "rlt_peer_enable")
