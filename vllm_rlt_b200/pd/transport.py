"""Transport of the PD handoff: same surface as the reference's ``NixlConnector``, B200 data plane.

``B200Transport`` can be handed to an unmodified ``PDStageConnector`` in place of
``NixlConnector`` (vllm_rlt/pd/transport.py:115-243): it has the same ``info`` keys, ``peers``,
``pending``, ``inflight_bytes``, the three metrics, and ``connect / submit / poll / busy / close``
with the same return values and exceptions. What differs is underneath:

* registration: pool tensors are exported as CUDA IPC handles (``info["metadata"]``) instead of
  NIXL agent metadata; the writer maps them lazily on its first submission to a peer;
* ``submit``: the descriptor lists become one ``rlt_kv_copy_segments`` launch whose stores go
  straight into the peer's pool, followed on the same stream by an ``rlt_kv_post`` of the
  ``(transfer id, sequence)`` notification into the receiver's mailbox;
* ``submit_tables`` (an addition): the connector passes block tables and a token range and the
  GPU does the walk itself (``rlt_kv_handoff``); no descriptor list is built at all;
* ``poll``: completion is a CUDA event per ticket; notifications are read from a mailbox in
  POSIX shared memory that the peer's GPU writes, so the receiver polls without any CUDA call.

Device work is behind a small backend object so that the bookkeeping (budget, tickets,
time-outs, mailbox protocol) is testable without a GPU.
"""

from __future__ import annotations

import struct
import time
from collections import deque
from dataclasses import dataclass
from multiprocessing import shared_memory

import numpy as np

SLOT_BYTES = 64
BODY_BYTES = 56
LANES = 16
SLOTS = 256
LANE_BYTES = SLOT_BYTES * (1 + SLOTS)  # one header slot (consumed counter) + the ring
TID_MAX = BODY_BYTES - 8


@dataclass
class Transfer:
    """One submission in flight (vllm_rlt/pd/transport.py:9-15)."""

    handle: object
    transfer_id: str
    sequence: int
    size: int
    submitted: float
    keepalive: tuple = ()


def _kv_region(key, value) -> dict:
    """Byte geometry of a K/V tensor pair (vllm_rlt/pd/transport.py:18-26)."""
    e = key.element_size()
    return dict(key_ptr=key.data_ptr(), value_ptr=value.data_ptr(), block_bytes=key.stride(0) * e,
                layer_bytes=key.stride(1) * e, token_bytes=key.stride(2) * e)


# ------------------------------------------------------------------------------------ mailbox


class Mailbox:
    """Receiver-owned ring of 64-byte notification slots in POSIX shared memory, one lane per sender.

    Lane layout: slot 0 is a header whose first 8 bytes hold the count of messages the receiver
    has consumed; slots 1..SLOTS are the ring. Message ``n`` (1-based) of a lane lives in ring slot
    ``(n - 1) % SLOTS`` and carries stamp ``n`` in its first 8 bytes; the body is
    ``[sequence u32][tid length u32][tid bytes]``. The sender's GPU writes body then stamp
    (``rlt_kv_post``); the receiver's host reads stamp then body.
    """

    def __init__(self, name: str | None = None):
        self.owner = name is None
        if self.owner:
            self.shm = shared_memory.SharedMemory(create=True, size=LANES * LANE_BYTES)
            self.shm.buf[:] = bytes(len(self.shm.buf))
        else:
            self.shm = shared_memory.SharedMemory(name=name)
        self.name = self.shm.name
        self.words = np.frombuffer(self.shm.buf, dtype=np.uint64)
        self.bytes = np.frombuffer(self.shm.buf, dtype=np.uint8)
        self.next = [1] * LANES  # receiver: next stamp expected per lane

    @staticmethod
    def lane_of(device: int) -> int:
        return device % LANES

    @staticmethod
    def slot_offset(lane: int, n: int) -> int:
        return lane * LANE_BYTES + SLOT_BYTES * (1 + (n - 1) % SLOTS)

    @staticmethod
    def encode(transfer_id: str, sequence: int) -> bytes:
        raw = transfer_id.encode()
        if len(raw) > TID_MAX:
            raise ValueError(f"transfer id longer than {TID_MAX} bytes")
        return struct.pack("<II", sequence, len(raw)) + raw.ljust(TID_MAX, b"\0")

    def consumed(self, lane: int) -> int:
        return int(self.words[lane * LANE_BYTES // 8])

    def drain(self, lane: int):
        """Receiver: yield ``(transfer id, sequence)`` of every message that has arrived on a lane."""
        while True:
            n = self.next[lane]
            at = self.slot_offset(lane, n)
            if int(self.words[at // 8]) != n:
                return
            sequence, length = struct.unpack_from("<II", self.bytes, at + 8)
            tid = bytes(self.bytes[at + 16 : at + 16 + min(length, TID_MAX)]).decode()
            self.next[lane] = n + 1
            self.words[lane * LANE_BYTES // 8] = n  # lets the sender reuse the slot
            yield tid, sequence

    def close(self):
        if self.shm is None:
            return
        self.words = self.bytes = None
        shm, self.shm = self.shm, None
        try:
            shm.close()
        finally:
            if self.owner:
                try:
                    shm.unlink()
                except FileNotFoundError:
                    pass

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


# ------------------------------------------------------------------------------------ device backend


class CudaBackend:
    """The device side of the transport: peer mappings, launches, events.

    Every launch goes to one transfer stream owned by the backend, so copies never queue behind the model's
    compute. ``device_ordered`` tells the connector that a submission may be handed a producer event to wait
    for *on the device*: the copy is queued at once and starts when the event fires, with no host poll in between.
    """

    device_ordered = True

    def __init__(self, device):
        import torch

        from . import peer as peerlib

        self.torch = torch
        self.device = torch.device(device)
        self.mapping = peerlib.PeerMapping()
        self.peerlib = peerlib
        self._mailboxes: dict[str, tuple[Mailbox, int]] = {}
        self.stream = torch.cuda.Stream(self.device)

    def _on_stream(self):
        return self.torch.cuda.stream(self.stream)

    def order_after(self, event) -> None:
        """Make everything submitted from now on wait (on the device) for ``event``."""
        if event is not None:
            self.stream.wait_event(event)

    def export(self, tensor) -> dict:
        e = self.peerlib.export_tensor(tensor)
        e["ptr"] = tensor.data_ptr()
        return e

    def translator(self, peer_info: dict):
        """Function mapping an address in the peer's address space to one this process can write."""
        spans = []
        same_process = peer_info["metadata"].get("pid") == _pid()
        for e in peer_info["metadata"]["tensors"]:
            base = e["ptr"] if same_process else self.mapping.pointer(e)
            spans.append((e["ptr"], e["ptr"] + e["bytes"], base))
        if same_process and peer_info["device"] != self.device.index:
            self.peerlib.enable_peer_access(self.device.index, peer_info["device"])

        def translate(address: int, nbytes: int) -> int:
            for lo, hi, base in spans:
                if lo <= address and address + nbytes <= hi:
                    return base + (address - lo)
            raise ValueError("remote descriptor outside the peer's registered memory")

        return translate

    def mailbox_pointer(self, name: str) -> tuple[Mailbox, int]:
        """Open a peer's mailbox and make it writable from this device."""
        import ctypes as C

        from .. import _lib

        hit = self._mailboxes.get(name)
        if hit is None:
            box = Mailbox(name)
            host = C.addressof(C.c_char.from_buffer(box.shm.buf))
            out = C.c_void_p()
            with self.torch.cuda.device(self.device):
                _lib.check(_lib.load().rlt_host_register(host, len(box.shm.buf), C.byref(out)), "rlt_host_register")
            hit = self._mailboxes[name] = (box, int(out.value), host)
        return hit[0], hit[1]

    def copy_segments(self, triples):
        from ..kernels import kv_handoff as kh

        torch = self.torch
        host = torch.tensor(triples, dtype=torch.int64).reshape(-1, 3).pin_memory()
        keep = []
        with torch.cuda.device(self.device), self._on_stream():
            for at in range(0, len(host), kh._lib.MAX_SEGMENTS):
                dev = host[at : at + kh._lib.MAX_SEGMENTS].to(self.device, non_blocking=True)
                kh.kv_copy_segments(dev)
                keep.append(dev)
        return (host, *keep)

    def handoff(self, cache, peer_info, translate, requests, *, mode=0, layer_begin=0, layer_end=0,
                exit_planes=None, status=None):
        """One table-driven launch for ``requests`` = [(source tables, target tables, start, end), ...]."""
        from ..kernels import kv_handoff as kh

        src = kh.PoolView.from_cache(cache)
        codes = src.codes.rebased(translate(peer_info["key_ptr"], 1), translate(peer_info["value_ptr"], 1))
        scales = None
        if src.scales is not None:
            sr = peer_info["scale_region"]
            scales = src.scales.rebased(translate(sr["key_ptr"], 1), translate(sr["value_ptr"], 1))
        planes = 1 if mode == kh.MODE_EXIT_ONLY else peer_info["depths"]
        dst = kh.PoolView(codes, scales, peer_info["num_blocks"], peer_info["block_size"], peer_info["num_layers"],
                          planes, peer_info["device"])
        with self.torch.cuda.device(self.device), self._on_stream():
            batch = kh.HandoffBatch(
                [r[0] for r in requests], [r[1] for r in requests], [(r[2], r[3]) for r in requests],
                block_size=src.block_size, exit_planes=exit_planes, src_blocks=src.num_blocks,
                dst_blocks=dst.num_blocks, device=self.device)
            kh.kv_handoff(src, dst, batch, mode=mode, layer_begin=layer_begin, layer_end=layer_end, status=status)
        return (batch,)

    def post(self, slot_ptr: int, body: bytes, stamp: int):
        import ctypes as C

        from .. import _lib

        with self.torch.cuda.device(self.device):
            buf = (C.c_uint8 * BODY_BYTES).from_buffer_copy(body)
            _lib.check(_lib.load().rlt_kv_post(slot_ptr, buf, stamp, self.stream.cuda_stream), "rlt_kv_post")

    def event(self):
        ev = self.torch.cuda.Event()
        with self.torch.cuda.device(self.device):
            ev.record(self.stream)
        return ev

    def close(self):
        import ctypes as C  # noqa: F401

        from .. import _lib

        for box, _, host in self._mailboxes.values():
            _lib.check(_lib.load().rlt_host_unregister(host), "rlt_host_unregister")
            box.close()
        self._mailboxes.clear()
        self.mapping.close()


def _pid() -> int:
    import os

    return os.getpid()


# ------------------------------------------------------------------------------------ transport


class B200Transport:
    def __init__(self, name, cache, hidden, config, *, backend=None, lane=None):
        self.config = config
        self.name = name
        self.cache = cache
        self.backend = backend if backend is not None else CudaBackend(cache.key_cache.device)
        # True: submissions may carry a producer event that the copy waits for on the device (``after=``)
        self.device_ordered = getattr(self.backend, "device_ordered", False) is True
        self.storage = (cache.key_cache, cache.value_cache, hidden)
        # Dynamic scales travel with their rows; a fixed scale is checked in the handshake instead
        # (vllm_rlt/pd/transport.py:132-137).
        scale_region = None
        if cache.key_scale is not None and cache.fp8_scale is None:
            self.storage += (cache.key_scale, cache.value_scale)
            scale_region = _kv_region(cache.key_scale, cache.value_scale)
        self.mailbox = Mailbox()
        k = cache.key_cache
        self.info = dict(
            **_kv_region(k, cache.value_cache),
            agent=name,
            metadata=dict(tensors=[self.backend.export(t) for t in self.storage], mailbox=self.mailbox.name, pid=_pid(),
                          lane=None),
            hidden_ptr=hidden.data_ptr(),
            hidden_bytes=hidden.stride(0) * hidden.element_size(),
            device=k.device.index if k.device.index is not None else 0,
            num_blocks=cache.num_blocks,
            block_size=cache.block_size,
            num_layers=cache.num_layers,
            depths=cache.storage_depths,
            kv_dtype=str(k.dtype),
            fp8_scale=cache.fp8_scale,
            scale_region=scale_region,
        )
        # Mailbox lane this worker writes on at every receiver: its device index unless told otherwise
        # (workers of one deployment never share a device, vllm_rlt/pd/config.py:31-33).
        self.info["metadata"]["lane"] = Mailbox.lane_of(self.info["device"] if lane is None else lane)
        self.peers: dict[str, dict] = {}
        self._lane_agent: dict[int, str] = {}
        self._writer: dict[str, dict] = {}  # per peer: translate fn, mailbox, next stamp
        self.pending: deque[Transfer] = deque()
        self.inflight_bytes = 0
        self.bytes_sent = 0
        self.transfers = 0
        self.transfer_seconds = 0.0

    # -- handshake ---------------------------------------------------------------------------

    def connect(self, peer):
        """Geometry equality as in vllm_rlt/pd/transport.py:162-180, same messages."""
        strides = ("block_bytes", "layer_bytes", "token_bytes")
        for key in ("block_size", "num_layers", "depths", "hidden_bytes", "kv_dtype", *strides):
            if peer[key] != self.info[key]:
                raise ValueError(f"PD KV geometry mismatch: {key}")
        if peer["fp8_scale"] != self.info["fp8_scale"]:
            raise ValueError("P and D must use the same calibrated FP8 scale")
        mine, theirs = self.info["scale_region"], peer["scale_region"]
        if (mine is None) != (theirs is None) or (mine is not None and any(mine[k] != theirs[k] for k in strides)):
            raise ValueError("PD KV scale geometry mismatch")
        name = peer["agent"]
        lane = peer["metadata"]["lane"]
        if self._lane_agent.get(lane, name) != name:
            raise ValueError(f"peer {name!r} shares mailbox lane {lane} with another connected worker")
        self._lane_agent[lane] = name
        self.peers[name] = peer

    def _writer_state(self, peer_name: str) -> dict:
        state = self._writer.get(peer_name)
        if state is None:
            peer = self.peers[peer_name]
            box, box_ptr = self.backend.mailbox_pointer(peer["metadata"]["mailbox"])
            state = self._writer[peer_name] = dict(
                translate=self.backend.translator(peer), box=box, box_ptr=box_ptr,
                lane=self.info["metadata"]["lane"], stamp=0,
            )
        return state

    # -- submission --------------------------------------------------------------------------

    def _admit(self, size: int, state: dict) -> bool:
        if size > self.config.transfer_chunk_bytes:
            raise ValueError("transfer exceeds configured chunk size")
        if self.inflight_bytes + size > self.config.max_inflight_bytes:
            return False
        # the receiver must have consumed the slot this message will reuse
        return state["stamp"] - state["box"].consumed(state["lane"]) < SLOTS

    def _finish_submit(self, state, transfer_id, sequence, size, keepalive) -> bool:
        state["stamp"] += 1
        at = Mailbox.slot_offset(state["lane"], state["stamp"])
        self.backend.post(state["box_ptr"] + at, Mailbox.encode(transfer_id, sequence), state["stamp"])
        ticket = Transfer(self.backend.event(), transfer_id, sequence, size, time.monotonic(), keepalive)
        self.pending.append(ticket)
        self.inflight_bytes += size
        return True

    def submit(self, transfer_id, sequence, peer, local, remote, size, *, after=None):
        """WRITE the local ranges onto the remote ranges and notify the peer (vllm_rlt/pd/transport.py:182-201).

        ``after`` (device-ordered backends only): a producer event the copy waits for on the device.
        """
        state = self._writer_state(peer)
        if not self._admit(size, state):
            return False
        self._order_after(after)
        if len(local) != len(remote):
            raise ValueError("incompatible source/target KV geometry")
        translate = state["translate"]
        triples = []
        for (src, n, _), (dst, m, _) in zip(local, remote):
            if n != m:
                raise ValueError("incompatible source/target KV geometry")
            triples.append((src, translate(dst, n), n))
        keep = self.backend.copy_segments(triples) if triples else ()
        return self._finish_submit(state, transfer_id, sequence, size, keep)

    def _order_after(self, event) -> None:
        if event is None:
            return
        if not self.device_ordered:
            raise ValueError("this backend cannot wait for an event on the device; submit once it has fired")
        self.backend.order_after(event)

    def submit_tables(self, transfer_id, sequence, peer, requests, size, *, mode=0, layer_begin=0, layer_end=0,
                      exit_planes=None, extra=(), status=None, after=None):
        """Table-driven form of ``submit``: ``requests`` is a list of ``(source tables, target tables,
        start, end)`` and the GPU walks the tables itself; ``extra`` holds plain ``(source address,
        peer address, bytes)`` ranges that ride along (the final hidden-state row)."""
        state = self._writer_state(peer)
        if not self._admit(size, state):
            return False
        self._order_after(after)
        translate = state["translate"]
        keep = tuple(self.backend.handoff(self.cache, self.peers[peer], translate, requests, mode=mode,
                                          layer_begin=layer_begin, layer_end=layer_end, exit_planes=exit_planes,
                                          status=status))
        if extra:
            keep += tuple(self.backend.copy_segments([(s, translate(d, n), n) for s, d, n in extra]))
        return self._finish_submit(state, transfer_id, sequence, size, keep)

    # -- progress ----------------------------------------------------------------------------

    def poll(self):
        remaining = deque()
        finished = []
        now = time.monotonic()
        for ticket in self.pending:
            if now - ticket.submitted > self.config.request_timeout:
                raise TimeoutError("KV write timed out; registered memory must be quarantined")
            if not ticket.handle.query():
                remaining.append(ticket)
                continue
            ticket.handle = None
            ticket.keepalive = ()
            self.inflight_bytes -= ticket.size
            self.bytes_sent += ticket.size
            self.transfers += 1
            self.transfer_seconds += time.monotonic() - ticket.submitted
            finished.append(ticket)
        self.pending = remaining
        notifications = []
        for lane, agent in self._lane_agent.items():
            for tid, sequence in self.mailbox.drain(lane):
                notifications.append((agent, tid, sequence))
        return finished, notifications

    def busy(self, transfer_id):
        return any(t.transfer_id == transfer_id for t in self.pending)

    def close(self):
        if self.pending:
            raise RuntimeError("cannot deregister memory with in-flight transfers")
        self._writer.clear()
        self.backend.close()
        self.mailbox.close()
        self.peers.clear()
