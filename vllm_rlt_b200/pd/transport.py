"""Transport of the PD handoff: same surface as the reference's ``NixlConnector``, B200 data plane.

``B200Transport`` can be handed to an unmodified ``PDStageConnector`` in place of
``NixlConnector`` (vllm_rlt/pd/transport.py:115-243): it has the same ``info`` keys, ``peers``,
``pending``, ``inflight_bytes``, the three metrics, and ``connect / submit / poll / busy / close``
with the same return values and exceptions. What differs is underneath:

* registration: pool tensors are exported as CUDA IPC handles (``info["metadata"]``) instead of
  NIXL agent metadata; a worker maps a peer's tensors lazily on first use;
* ``submit``: the descriptor lists become one ``rlt_kv_copy_segments`` launch whose stores go
  straight into the peer's pool, followed on the same stream by an ``rlt_kv_post`` of the
  ``(transfer id, sequence)`` notification into the receiver's mailbox;
* ``submit_tables`` (an addition): the connector passes block tables and a token range and the
  GPU does the walk itself (``rlt_kv_handoff``); no descriptor list is built at all;
* ``poll``: completion is a CUDA event per ticket; notifications are read from a mailbox in
  POSIX shared memory that the peer's GPU writes, so the receiver polls without any CUDA call.

Two directions for ``submit_tables``. *Push*: the sender's GPU runs the handoff kernel with the receiver's pool
behind peer pointers and then posts "landed". *Pull* (the default): the sender writes the chunk's descriptor
(both sides' block tables, the token range, the hidden-state row) into a descriptor ring in the receiver's
mailbox from the host and, behind the producer's event on its transfer stream, posts a 64-byte "offer"; the
receiver's ``poll()`` finds the offer, runs the same kernel on its own transfer stream with the *sender's* pool
behind peer pointers, reports ``(peer, tid, seq)`` as received when that launch's event has fired, and posts
"pulled" into the sender's mailbox, which completes the sender's ticket (``busy()`` stays true until then, so the
source KV cannot be released under a reader). NVLink read responses carry less protocol overhead than writes,
so a pair moves about 9 % more payload per second this way; the coordinator and the connector protocol are
untouched because the tables travel P->D inside the transport. No load is ever issued with cluster multicast.

Device work is behind a small backend object so that the bookkeeping (budget, tickets,
time-outs, mailbox protocol) is testable without a GPU.
"""

from __future__ import annotations

import os
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
RING_BYTES = 256 * 1024  # descriptor ring of one lane
LANE_BYTES = SLOT_BYTES * (1 + SLOTS) + RING_BYTES  # header slot (consumed counter), message ring, descriptor ring
RING_OFFSET = SLOT_BYTES * (1 + SLOTS)
TID_MAX = 40

# what a message says (one byte of its header)
LANDED = 0  # push: the chunk's bytes are in your pool
OFFER = 1   # pull: the chunk is ready in my pool; its descriptor is in my lane's descriptor ring
PULLED = 2  # pull: I have read the chunk you offered; you may let go of it


@dataclass
class Transfer:
    """One submission in flight (vllm_rlt/pd/transport.py:9-15)."""

    handle: object
    transfer_id: str
    sequence: int
    size: int
    submitted: float
    keepalive: tuple = ()
    started: object = None        # event on the transfer stream: the copy (or the offer) has begun
    started_at: float | None = None  # host time of the first poll that found it begun


@dataclass
class Message:
    kind: int
    transfer_id: str
    sequence: int
    descriptor: bytes = b""
    count: int = 1  # consecutive sequence numbers, starting at ``sequence``, that this one message stands for


class _RemoteCompletion:
    """Ticket handle of an offered chunk: done when the peer has said "pulled"."""

    def __init__(self):
        self.done = False

    def query(self) -> bool:
        return self.done


def _kv_region(key, value) -> dict:
    """Byte geometry of a K/V tensor pair (vllm_rlt/pd/transport.py:18-26)."""
    e = key.element_size()
    return dict(key_ptr=key.data_ptr(), value_ptr=value.data_ptr(), block_bytes=key.stride(0) * e,
                layer_bytes=key.stride(1) * e, token_bytes=key.stride(2) * e)


# ------------------------------------------------------------------------------------ chunk descriptors


def encode_chunk(requests, extra, *, mode=0, layer_begin=0, layer_end=0, plane_begin=0, plane_end=0) -> bytes:
    """A pull offer's descriptor: what the receiver needs to run the launch itself.

    ``requests`` is ``[(source tables, target tables, start, end)]``; each request's tables are cut down to the
    pages the range touches and the range is rebased onto them (block tables are only ever indexed by page, so
    the kernel's result is the same), which keeps a descriptor proportional to the chunk, not to the prompt.
    ``extra`` is ``[(source address, target address, bytes)]``.
    """
    out = [struct.pack("<8I", len(requests), len(extra), mode, layer_begin, layer_end, plane_begin, plane_end, 0)]
    for source, target, start, end in requests:
        if not source or not target or start < 0 or start >= end:
            raise ValueError("invalid KV range")
        page = min(len(table) for table in (*source, *target))
        out.append(struct.pack("<2I2q", len(source), len(target), start, end))
        out.append(struct.pack("<I", page))
        for table in (*source, *target):
            out.append(np.asarray(table[:page], dtype=np.int32).tobytes())
    for src, dst, n in extra:
        out.append(struct.pack("<3q", src, dst, n))
    return b"".join(out)


def decode_chunk(raw: bytes):
    """Inverse of ``encode_chunk``: ``(requests, extra, options)`` with the launch options as a dict."""
    n_req, n_extra, mode, layer_begin, layer_end, plane_begin, plane_end, _ = struct.unpack_from("<8I", raw, 0)
    at = 32
    requests = []
    for _ in range(n_req):
        src_planes, dst_planes, start, end = struct.unpack_from("<2I2q", raw, at)
        at += 24
        (pages,) = struct.unpack_from("<I", raw, at)
        at += 4
        tables = []
        for _ in range(src_planes + dst_planes):
            tables.append(np.frombuffer(raw, dtype=np.int32, count=pages, offset=at))
            at += 4 * pages
        requests.append((tuple(tables[:src_planes]), tuple(tables[src_planes:]), start, end))
    extra = []
    for _ in range(n_extra):
        extra.append(struct.unpack_from("<3q", raw, at))
        at += 24
    return requests, extra, dict(mode=mode, layer_begin=layer_begin, layer_end=layer_end, plane_begin=plane_begin,
                                 plane_end=plane_end)


def trim_request(source, target, start, end, block_size):
    """Cut a request's tables to the pages ``[start, end)`` touches and rebase the range onto them."""
    first, last = start // block_size, (end - 1) // block_size
    cut = lambda tables: tuple(table[first : last + 1] for table in tables)  # noqa: E731
    return cut(source), cut(target), start - first * block_size, end - first * block_size


class _RingWriter:
    """Sender-side allocator of one lane's descriptor ring in a peer's mailbox. Regions are handed out in ring
    order and become reusable when the receiver has consumed the message (stamp) they belong to."""

    def __init__(self, size: int = RING_BYTES):
        self.size = size
        self.head = 0
        self.live: deque[tuple[int, int, int]] = deque()  # (stamp, start, end) oldest first

    def reserve(self, nbytes: int, stamp: int, consumed: int):
        if nbytes > self.size:
            raise ValueError("chunk descriptor larger than the descriptor ring")
        while self.live and self.live[0][0] <= consumed:
            self.live.popleft()
        if not self.live:
            start = self.head if self.head + nbytes <= self.size else 0
        else:
            tail = self.live[0][1]  # where the oldest live region starts
            if tail < self.head:  # live bytes are [tail, head): free are [head, size) and [0, tail)
                if self.head + nbytes <= self.size:
                    start = self.head
                elif nbytes <= tail:
                    start = 0
                else:
                    return None
            elif self.head + nbytes <= tail:  # live bytes wrap around the end: free are [head, tail)
                start = self.head
            else:
                return None
        self.head = start + nbytes
        self.live.append((stamp, start, start + nbytes))
        return start


# ------------------------------------------------------------------------------------ mailbox


class Mailbox:
    """Receiver-owned notification slots and descriptor rings in POSIX shared memory, one lane per sender.

    Lane layout: slot 0 is a header whose first 8 bytes hold the count of messages the receiver
    has consumed; slots 1..SLOTS are the message ring; ``RING_BYTES`` of descriptor ring follow. Message ``n``
    (1-based) of a lane lives in ring slot ``(n - 1) % SLOTS`` and carries stamp ``n`` in its first 8 bytes; the
    body is ``[sequence u32][tid length u8][kind u8][count u16][descriptor offset u32][descriptor bytes u32][tid]``;
    ``count`` consecutive sequence numbers starting at ``sequence`` share the message (chunks that left as one launch).
    The sender writes body then stamp - its GPU with ``rlt_kv_post`` when the message must follow device work,
    its CPU otherwise; the receiver's host reads stamp then body. A descriptor is written by the sender's CPU
    before the message that names it is posted, and read by the receiver before it counts the message consumed.
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
    def encode(transfer_id: str, sequence: int, kind: int = LANDED, descriptor: tuple[int, int] = (0, 0),
               count: int = 1) -> bytes:
        raw = transfer_id.encode()
        if len(raw) > TID_MAX:
            raise ValueError(f"transfer id longer than {TID_MAX} bytes")
        if not 1 <= count < 1 << 16:
            raise ValueError("a message stands for 1 to 65535 sequence numbers")
        return struct.pack("<IBBHII", sequence, len(raw), kind, count, *descriptor) + raw.ljust(TID_MAX, b"\0")

    def consumed(self, lane: int) -> int:
        return int(self.words[lane * LANE_BYTES // 8])

    def write_descriptor(self, lane: int, offset: int, raw: bytes) -> None:
        at = lane * LANE_BYTES + RING_OFFSET + offset
        self.bytes[at : at + len(raw)] = np.frombuffer(raw, dtype=np.uint8)

    def post_from_host(self, lane: int, n: int, body: bytes) -> None:
        """The CPU form of ``rlt_kv_post``: body first, stamp last (program order is store order on x86)."""
        at = self.slot_offset(lane, n)
        self.bytes[at + 8 : at + SLOT_BYTES] = np.frombuffer(body, dtype=np.uint8)
        self.words[at // 8] = n

    def drain(self, lane: int):
        """Receiver: yield a ``Message`` for everything that has arrived on a lane, in order."""
        while True:
            n = self.next[lane]
            at = self.slot_offset(lane, n)
            if int(self.words[at // 8]) != n:
                return
            sequence, length, kind, count, d_off, d_len = struct.unpack_from("<IBBHII", self.bytes, at + 8)
            tid = bytes(self.bytes[at + 24 : at + 24 + min(length, TID_MAX)]).decode()
            descriptor = b""
            if d_len:
                base = lane * LANE_BYTES + RING_OFFSET + d_off
                descriptor = bytes(self.bytes[base : base + d_len])
            self.next[lane] = n + 1
            self.words[lane * LANE_BYTES // 8] = n  # lets the sender reuse the slot and the descriptor's bytes
            yield Message(kind, tid, sequence, descriptor, max(1, count))

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
        self._views: dict[tuple, tuple] = {}
        self._host_limit = None  # bytes of tables one call of the library's own staging takes
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

    def copy_ranges(self, triples):
        """A few plain (source, destination, bytes) ranges, one ``rlt_kv_push`` launch each: no descriptor table to
        build, pin and upload, which matters for the single hidden-state row that rides on a chunk."""
        from ..kernels import kv_handoff as kh

        with self.torch.cuda.device(self.device), self._on_stream():
            for src, dst, n in triples:
                kh.kv_push(src, dst, n)
        return ()

    def handoff(self, cache, peer_info, translate, requests, *, mode=0, layer_begin=0, layer_end=0,
                plane_begin=0, plane_end=0, exit_planes=None, status=None, pull=False, before_launch=None):
        """One table-driven launch for ``requests`` = [(source tables, target tables, start, end), ...], optionally
        of one slice of layers and destination planes (0, 0 = all).

        Push: the local pool is the source and the peer's pool, behind translated pointers, the destination.
        ``pull=True``: the peer's pool is the source and the local pool the destination (plain peer loads)."""
        from ..kernels import kv_handoff as kh

        # the two pool views of a (peer, direction, plane count) never change: build them once
        key = (peer_info["agent"], pull, mode == kh.MODE_EXIT_ONLY)
        views = self._views.get(key)
        if views is None:
            mine = kh.PoolView.from_cache(cache)
            codes = mine.codes.rebased(translate(peer_info["key_ptr"], 1), translate(peer_info["value_ptr"], 1))
            scales = None
            if mine.scales is not None:
                sr = peer_info["scale_region"]
                scales = mine.scales.rebased(translate(sr["key_ptr"], 1), translate(sr["value_ptr"], 1))
            if pull:
                theirs = kh.PoolView(codes, scales, peer_info["num_blocks"], peer_info["block_size"], peer_info["num_layers"],
                                     peer_info["depths"], peer_info["device"])
                if mode == kh.MODE_EXIT_ONLY and mine.num_planes != 1:
                    raise ValueError("an exit-only pull needs a single-plane destination pool")
                views = (theirs, mine)
            else:
                planes = 1 if mode == kh.MODE_EXIT_ONLY else peer_info["depths"]
                theirs = kh.PoolView(codes, scales, peer_info["num_blocks"], peer_info["block_size"], peer_info["num_layers"],
                                     planes, peer_info["device"])
                views = (mine, theirs)
            self._views[key] = views
        src, dst = views
        if exit_planes is None and status is None and mode == kh.MODE_ALL_PLANES:
            host = self._host_tables(requests, src, dst)
            if host is not None:  # a chunk's worth of tables: staged and launched by one call into the library
                with self.torch.cuda.device(self.device):
                    if before_launch is not None:
                        before_launch()
                    kh.kv_handoff_host(src, dst, *host, layer_begin=layer_begin, layer_end=layer_end,
                                       plane_begin=plane_begin, plane_end=plane_end, stream=self.stream)
                return ()
        with self.torch.cuda.device(self.device), self._on_stream():
            batch = kh.HandoffBatch(
                [r[0] for r in requests], [r[1] for r in requests], [(r[2], r[3]) for r in requests],
                block_size=src.block_size, exit_planes=exit_planes, src_blocks=src.num_blocks,
                dst_blocks=dst.num_blocks, device=self.device)
            if before_launch is not None:
                before_launch()  # the tables are staged: what follows is the launch itself
            kh.kv_handoff(src, dst, batch, mode=mode, layer_begin=layer_begin, layer_end=layer_end,
                          plane_begin=plane_begin, plane_end=plane_end, status=status)
        return (batch,)

    def _host_tables(self, requests, src, dst):
        """``(source tables, destination tables, begin, end)`` as int32 arrays for ``kv_handoff_host``, or None when
        the batch is not of that kind (tables of different lengths, too large for a staging slot) or when anything
        about it looks wrong: the general path then finds the error and words it as the reference does."""
        import numpy as np

        try:
            source = np.asarray([r[0] for r in requests], dtype=np.int32)
            target = np.asarray([r[1] for r in requests], dtype=np.int32)
        except (ValueError, OverflowError):
            return None
        if source.ndim != 3 or target.ndim != 3 or source.shape[1] != src.num_planes or target.shape[1] != dst.num_planes:
            return None
        begin = np.asarray([r[2] for r in requests], dtype=np.int64)
        end = np.asarray([r[3] for r in requests], dtype=np.int64)
        # a decode worker reserves pages for the tokens it will generate, so its tables run past the prompt's: tables
        # are only ever indexed by the pages a range touches, and both sides are cut to the shorter one
        width = min(source.shape[2], target.shape[2])
        if width < 1:
            return None
        if source.shape[2] != width:
            source = np.ascontiguousarray(source[:, :, :width])
        if target.shape[2] != width:
            target = np.ascontiguousarray(target[:, :, :width])
        if self._host_limit is None:
            from ..kernels import kv_handoff as kh

            self._host_limit = kh.host_batch_limit()
        if source.nbytes + target.nbytes + 8 * len(requests) > self._host_limit:
            return None
        suspicious = ((begin < 0) | (begin >= end) | (end > source.shape[2] * src.block_size)).any() \
            or (source.view(np.uint32) >= src.num_blocks).any() or (target.view(np.uint32) >= dst.num_blocks).any()
        if suspicious:
            return None
        return source, target, begin.astype(np.int32), end.astype(np.int32)

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

    marker = event  # an event at the current end of the transfer stream, used to tell when queued work begins

    def timed_event(self):
        """Like ``event`` but usable with ``elapsed_time`` (device time between two of them)."""
        ev = self.torch.cuda.Event(enable_timing=True)
        with self.torch.cuda.device(self.device):
            ev.record(self.stream)
        return ev

    def close(self):
        from .. import _lib

        boxes, self._mailboxes = self._mailboxes, {}
        self._views = {}
        for box, _, host in boxes.values():
            _lib.check(_lib.load().rlt_host_unregister(host), "rlt_host_unregister")
            box.close()
        self.mapping.close()

    def __del__(self):
        # a backend that is dropped without close() must still unregister what it registered: the mailbox mappings
        # go away with their objects, and a registration left behind would cover whatever is mapped there next
        try:
            self.close()
        except Exception:
            pass


def _pid() -> int:
    import os

    return os.getpid()


# ------------------------------------------------------------------------------------ transport


@dataclass
class _Pull:
    """A chunk this worker is reading out of a peer's pool."""

    event: object
    peer: str
    transfer_id: str
    sequence: int
    size: int
    keepalive: tuple = ()
    reported: bool = False  # (peer, tid, seq) has been handed to the connector; "pulled" may still be unsent
    count: int = 1          # consecutive sequence numbers the launch covers
    begun: object = None    # timing event recorded before the launch (backends that can time on the device)


def default_direction() -> str:
    """``RLT_KV_DIRECTION`` (``pull`` or ``push``) if set, else pull."""
    value = os.environ.get("RLT_KV_DIRECTION", "pull").strip().lower()
    if value not in ("pull", "push"):
        raise ValueError("RLT_KV_DIRECTION must be 'pull' or 'push'")
    return value


class B200Transport:
    def __init__(self, name, cache, hidden, config, *, backend=None, lane=None, direction=None):
        self.config = config
        self.name = name
        self.cache = cache
        self.backend = backend if backend is not None else CudaBackend(cache.key_cache.device)
        # True: submissions may carry a producer event that the copy waits for on the device (``after=``)
        self.device_ordered = getattr(self.backend, "device_ordered", False) is True
        self.direction = default_direction() if direction is None else direction
        if self.direction not in ("pull", "push"):
            raise ValueError("direction must be 'pull' or 'push'")
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
        self._link: dict[str, dict] = {}  # per peer: address translation, its mailbox, next stamp, descriptor ring
        self.pending: deque[Transfer] = deque()
        self._offered: dict[tuple[str, str, int], _RemoteCompletion] = {}
        self._pulls: list[_Pull] = []
        self.inflight_bytes = 0
        self.bytes_sent = 0
        self.bytes_received = 0
        self.pull_seconds = 0.0  # device time this worker's GPU spent reading peers' pools
        self.pull_rates: deque[float] = deque(maxlen=4096)  # GB/s of each pull launch, device-timed
        self.transfers = 0
        self.transfer_seconds = 0.0
        # RLT_KV_TRACE=<directory>: every step of every chunk with the host's monotonic clock (which all processes of
        # a host share), written to <directory>/<worker name>.jsonl at close(); off by default
        self._trace_dir = os.environ.get("RLT_KV_TRACE")
        self._trace: list[tuple] = []

    def _note(self, what: str, transfer_id: str, sequence: int) -> None:
        if self._trace_dir:
            self._trace.append((time.monotonic(), what, transfer_id, sequence))

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

    def _peer_link(self, peer_name: str) -> dict:
        link = self._link.get(peer_name)
        if link is None:
            peer = self.peers[peer_name]
            box, box_ptr = self.backend.mailbox_pointer(peer["metadata"]["mailbox"])
            link = self._link[peer_name] = dict(
                translate=self.backend.translator(peer), box=box, box_ptr=box_ptr,
                lane=self.info["metadata"]["lane"], stamp=0, ring=_RingWriter(),
            )
        return link

    # -- submission --------------------------------------------------------------------------

    def _slot_free(self, link: dict) -> bool:
        """The receiver must have consumed the message whose slot the next one reuses."""
        return link["stamp"] - link["box"].consumed(link["lane"]) < SLOTS

    def _admit(self, size: int, link: dict) -> bool:
        if size > self.config.transfer_chunk_bytes:
            raise ValueError("transfer exceeds configured chunk size")
        if self.inflight_bytes + size > self.config.max_inflight_bytes:
            return False
        return self._slot_free(link)

    def _post(self, link: dict, body: bytes, *, from_host: bool = False) -> None:
        link["stamp"] += 1
        if from_host:
            link["box"].post_from_host(link["lane"], link["stamp"], body)
        else:
            at = Mailbox.slot_offset(link["lane"], link["stamp"])
            self.backend.post(link["box_ptr"] + at, body, link["stamp"])

    def _ticket(self, handle, transfer_id, sequence, size, keepalive, started) -> bool:
        now = time.monotonic()
        begun = now if started is None or started.query() else None  # nothing ahead of it on the transfer stream
        self.pending.append(Transfer(handle, transfer_id, sequence, size, now, keepalive, started, begun))
        self.inflight_bytes += size
        return True

    def _order_after(self, event):
        """Queue what follows behind ``event`` on the transfer stream; returns an event that fires when the
        transfer stream has got past that wait, i.e. when this submission's own work begins."""
        if event is not None:
            if not self.device_ordered:
                raise ValueError("this backend cannot wait for an event on the device; submit once it has fired")
            self.backend.order_after(event)
        return self.backend.marker()

    def submit(self, transfer_id, sequence, peer, local, remote, size, *, after=None):
        """WRITE the local ranges onto the remote ranges and notify the peer (vllm_rlt/pd/transport.py:182-201).

        ``after`` (device-ordered backends only): a producer event the copy waits for on the device.
        """
        link = self._peer_link(peer)
        if not self._admit(size, link):
            return False
        body = Mailbox.encode(transfer_id, sequence, LANDED)
        if len(local) != len(remote):
            raise ValueError("incompatible source/target KV geometry")
        translate = link["translate"]
        triples = []
        for (src, n, _), (dst, m, _) in zip(local, remote):
            if n != m:
                raise ValueError("incompatible source/target KV geometry")
            triples.append((src, translate(dst, n), n))
        started = self._order_after(after)
        keep = self.backend.copy_segments(triples) if triples else ()
        self._post(link, body)
        return self._ticket(self.backend.event(), transfer_id, sequence, size, keep, started)

    def submit_tables(self, transfer_id, sequence, peer, requests, size, *, mode=0, layer_begin=0, layer_end=0,
                      plane_begin=0, plane_end=0, exit_planes=None, extra=(), status=None, after=None, parts=None):
        """Table-driven form of ``submit``: ``requests`` is a list of ``(source tables, target tables,
        start, end)`` and the GPU walks the tables itself; ``extra`` holds plain ``(source address,
        peer address, bytes)`` ranges that ride along (the final hidden-state row).

        ``parts`` lets several chunks that are ready together leave as ONE launch: a list of ``(sequence, size)``
        with consecutive sequence numbers starting at ``sequence`` and sizes adding up to ``size``. Each part keeps
        its own ticket, its own share of the in-flight budget and its own notification at the receiver; only the
        launch, the staging of the tables and the mailbox message are shared.

        In the pull direction nothing is copied here: the chunk is offered and the peer reads it (see the module
        docstring); the tickets complete when the peer says so. Launches that carry per-token exit planes or a
        status array are always pushed (a descriptor does not carry them).
        """
        link = self._peer_link(peer)
        parts = [(sequence, size)] if parts is None else list(parts)
        if [s for s, _ in parts] != list(range(sequence, sequence + len(parts))) or sum(n for _, n in parts) != size:
            raise ValueError("parts must be consecutive sequence numbers whose sizes add up to the submission")
        for _, n in parts:
            if n > self.config.transfer_chunk_bytes:
                raise ValueError("transfer exceeds configured chunk size")
        if self.inflight_bytes + size > self.config.max_inflight_bytes or not self._slot_free(link):
            return False
        where = dict(mode=mode, layer_begin=layer_begin, layer_end=layer_end, plane_begin=plane_begin, plane_end=plane_end)
        if self.direction == "pull" and exit_planes is None and status is None:
            return self._offer(link, transfer_id, parts, requests, extra, where, after)
        body = Mailbox.encode(transfer_id, sequence, LANDED, count=len(parts))
        translate = link["translate"]
        started = self._order_after(after)
        keep = tuple(self.backend.handoff(self.cache, self.peers[peer], translate, requests, exit_planes=exit_planes,
                                          status=status, **where))
        if extra:
            keep += tuple(self.backend.copy_ranges([(s, translate(d, n), n) for s, d, n in extra]))
        self._post(link, body)
        done = self.backend.event()
        for seq, n in parts:
            self._ticket(done, transfer_id, seq, n, keep, started)
        return True

    def _offer(self, link, transfer_id, parts, requests, extra, where, after) -> bool:
        page = self.info["block_size"]
        raw = encode_chunk([trim_request(*r, page) for r in requests], extra, **where)
        box = link["box"]
        at = link["ring"].reserve(len(raw), link["stamp"] + 1, box.consumed(link["lane"]))
        if at is None:
            return False  # the peer has not yet read the descriptors ahead of this one: retry later
        first = parts[0][0]
        body = Mailbox.encode(transfer_id, first, OFFER, (at, len(raw)), count=len(parts))
        box.write_descriptor(link["lane"], at, raw)
        started = self._order_after(after)  # the offer leaves when the producer's event has fired
        self._post(link, body)
        self._note("offer queued", transfer_id, first)
        handle = self._offered[(self._agent_of(link), transfer_id, first)] = _RemoteCompletion()
        for seq, n in parts:
            self._ticket(handle, transfer_id, seq, n, (), started)
        return True

    def _agent_of(self, link) -> str:
        return next(name for name, other in self._link.items() if other is link)

    # -- progress ----------------------------------------------------------------------------

    def _begin_pull(self, agent: str, message: Message) -> None:
        """Run the launch an offer describes, on this worker's transfer stream, reading the peer's pool."""
        requests, extra, where = decode_chunk(message.descriptor)
        link = self._peer_link(agent)
        translate = link["translate"]
        timed = getattr(self.backend, "timed_event", None)
        begun = None

        def staged():  # called between staging the tables and the launch: device time counts from here
            nonlocal begun
            begun = timed() if timed is not None else None
            self._note("pull tables staged", message.transfer_id, message.sequence)

        self._note("pull decoded", message.transfer_id, message.sequence)
        keep = ()
        if requests:
            keep = tuple(self.backend.handoff(self.cache, self.peers[agent], translate, requests, pull=True,
                                              before_launch=staged, **where))
        elif timed is not None:
            begun = timed()
        self._note("pull tables launched", message.transfer_id, message.sequence)
        size = 0
        if extra:
            keep += tuple(self.backend.copy_ranges([(translate(s, n), d, n) for s, d, n in extra]))
            size += sum(n for _, _, n in extra)
        layers = (where["layer_end"] or self.info["num_layers"]) - where["layer_begin"]
        row = self.info["token_bytes"] + (self.info["scale_region"]["token_bytes"] if self.info["scale_region"] else 0)
        for _, target, start, end in requests:
            planes = (where["plane_end"] or len(target)) - where["plane_begin"]
            size += (end - start) * planes * 2 * layers * row
        done = timed() if timed is not None else self.backend.event()
        self._pulls.append(_Pull(done, agent, message.transfer_id, message.sequence, size, keep, count=message.count,
                                 begun=begun))
        self._note("pull launched", message.transfer_id, message.sequence)

    def poll(self):
        remaining = deque()
        finished = []
        notifications = []
        for lane, agent in self._lane_agent.items():
            for message in self.mailbox.drain(lane):
                if message.kind == LANDED:
                    self._note("landed seen", message.transfer_id, message.sequence)
                    notifications += [(agent, message.transfer_id, message.sequence + k) for k in range(message.count)]
                elif message.kind == OFFER:
                    self._note("offer seen", message.transfer_id, message.sequence)
                    self._begin_pull(agent, message)
                elif message.kind == PULLED:
                    handle = self._offered.pop((agent, message.transfer_id, message.sequence), None)
                    self._note("pulled seen", message.transfer_id, message.sequence)
                    if handle is not None:
                        handle.done = True
        # chunks this worker is reading: report each once its launch has finished, then tell its owner
        still = []
        for pull in self._pulls:
            if not pull.reported and pull.event.query():
                pull.reported = True
                pull.keepalive = ()
                self._note("pull finished", pull.transfer_id, pull.sequence)
                self.bytes_received += pull.size
                if pull.begun is not None:
                    seconds = pull.begun.elapsed_time(pull.event) * 1e-3  # device time of the launch(es)
                    self.pull_seconds += seconds
                    if seconds > 0:
                        self.pull_rates.append(pull.size / seconds / 1e9)
                notifications += [(pull.peer, pull.transfer_id, pull.sequence + k) for k in range(pull.count)]
            if pull.reported:
                link = self._peer_link(pull.peer)
                if self._slot_free(link):
                    self._post(link, Mailbox.encode(pull.transfer_id, pull.sequence, PULLED, count=pull.count), from_host=True)
                    continue
            still.append(pull)
        self._pulls = still
        now = time.monotonic()
        for ticket in self.pending:
            if ticket.started_at is None and (ticket.started is None or ticket.started.query()):
                ticket.started_at = now
                self._note("copy or offer begun", ticket.transfer_id, ticket.sequence)  # time-outs and transfer time count from when the copy could begin,
                #                          not from when it was queued behind the prefill that produces the KV
            if ticket.started_at is not None and now - ticket.started_at > self.config.request_timeout:
                raise TimeoutError("KV write timed out; registered memory must be quarantined")
            if ticket.started_at is None or not ticket.handle.query():
                remaining.append(ticket)
                continue
            ticket.keepalive = ()
            self.inflight_bytes -= ticket.size
            self.bytes_sent += ticket.size
            self.transfers += 1
            self.transfer_seconds += time.monotonic() - ticket.started_at
            self._note("ticket done", ticket.transfer_id, ticket.sequence)
            finished.append(ticket)
        self.pending = remaining
        return finished, notifications

    def busy(self, transfer_id):
        return any(t.transfer_id == transfer_id for t in self.pending)

    @property
    def reading(self) -> bool:
        """True while this worker still reads a peer's pool or owes it a "pulled" message."""
        return bool(self._pulls)

    def close(self):
        if self.pending or self._pulls:
            raise RuntimeError("cannot deregister memory with in-flight transfers")
        if self._trace_dir and self._trace:
            import json

            os.makedirs(self._trace_dir, exist_ok=True)
            with open(os.path.join(self._trace_dir, f"{self.name}.jsonl"), "a") as out:
                for row in self._trace:
                    out.write(json.dumps(row) + "\n")
            self._trace = []
        self._link.clear()
        self.backend.close()
        self.mailbox.close()
        self.peers.clear()
