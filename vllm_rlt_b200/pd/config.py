"""Deployment limits of the PD handoff; field names and checks follow ``PDConfig`` (vllm_rlt/pd/config.py:6-51).

The three transfer limits keep their meaning as bounds on one submission: bytes per launch,
bytes in flight per worker, and descriptors per launch (descriptor path only).
"""

import math
from dataclasses import dataclass


@dataclass(frozen=True)
class PDConfig:
    prefill_devices: tuple[int, ...] = (0,)
    decode_devices: tuple[int, ...] = (1,)
    max_pending_requests: int = 256
    transfer_chunk_bytes: int = 256 * 1024**2
    max_inflight_bytes: int = 2 * 1024**3
    max_transfer_descriptors: int = 256
    max_control_messages: int = 32
    startup_timeout: float = 300.0
    request_timeout: float = 300.0
    shutdown_timeout: float = 30.0
    backend: str = "B200_P2P"
    max_receiving_requests: int = 32
    max_draining_requests: int = 8

    def __post_init__(self):
        if not self.prefill_devices or not self.decode_devices:
            raise ValueError("PD requires nonempty prefill and decode device pools")
        devices = tuple(self.prefill_devices) + tuple(self.decode_devices)
        if any(type(d) is not int or d < 0 for d in devices) or len(set(devices)) != len(devices):
            raise ValueError("PD devices must be distinct nonnegative CUDA device indices")
        for name in ("max_receiving_requests", "max_draining_requests"):
            value = getattr(self, name)
            if type(value) is not int or value < 0:
                raise ValueError(f"{name} must be a nonnegative integer")
        for name in ("max_pending_requests", "transfer_chunk_bytes", "max_inflight_bytes",
                     "max_transfer_descriptors", "max_control_messages"):
            value = getattr(self, name)
            if type(value) is not int or value < 1:
                raise ValueError(f"{name} must be a positive integer")
        if self.transfer_chunk_bytes > self.max_inflight_bytes:
            raise ValueError("transfer_chunk_bytes exceeds max_inflight_bytes")
        for name in ("startup_timeout", "request_timeout", "shutdown_timeout"):
            value = getattr(self, name)
            if not math.isfinite(value) or value <= 0:
                raise ValueError(f"{name} must be positive and finite")
        if not self.backend:
            raise ValueError("transport backend must be specified")
