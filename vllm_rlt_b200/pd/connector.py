"""Per-worker transfer state machine of the PD handoff, speaking the reference's ``TransferConnector`` protocol.

This class takes the place of the reference's ``PDStageConnector`` (vllm_rlt/pd/connector.py:49-455)
behind the unchanged protocol of vllm_rlt/engine/connector.py:9-83. The stage engine, the scheduler
and the deployment coordinator keep calling the same methods with the same meaning; the control
verbs (``connect, reserve, prefill, cancel, cancel_safe, commit, ack, abort``) and the notifications
(``connected, reserved, prefill_started, prefill_complete, commit, received, activated, released,
rejected``) are the reference's, as are the error messages callers match on.

What changes is what a queued chunk is. The reference turns a token range into two Python lists of
byte descriptors (``kv_segments`` on both sides, ``partition_segments``) and submits them one list at
a time. Here a chunk is a ``TableChunk``: block tables of both sides plus a token range, cut so that
its payload stays under ``transfer_chunk_bytes``. One chunk is one ``rlt_kv_handoff`` launch in which
the GPU walks the tables itself, and one ``(transfer id, sequence)`` notification. Sequence numbers,
one notification per submitted chunk and ``commit.count == next_sequence`` are kept.

The object asks the engine to change request, compute or KV state (``reserve_transfer``,
``accept_import``, ``release_transfer_compute``, ``release_transfer``, ``suspend_transfer``); it owns
only transfer bookkeeping and the hidden-state staging rows.
"""

from __future__ import annotations

import hashlib
import json
import time
from collections import deque
from dataclasses import asdict, dataclass, field, is_dataclass, replace


@dataclass
class TableChunk:
    """One bounded submission: tokens ``[start, end)`` of every plane, by block table."""

    event: object
    sequence: int
    source_tables: tuple
    target_tables: tuple
    start: int
    end: int
    size: int
    hidden: tuple | None = None  # (source address, target address, bytes) of the final hidden row


@dataclass
class RequestTransfer:
    """Bookkeeping of one transfer generation; field names follow vllm_rlt/pd/connector.py:17-46."""

    tid: str
    request: object
    slot: int
    peer: str
    outgoing: bool = False
    trace_id: str | None = None
    target_tables: tuple = ()
    target_slot: int = 0
    cached_tokens: int = 0
    target_cached_tokens: int = 0
    chunks: deque = field(default_factory=deque)
    transfer_boundary_count: int = 0
    transfer_boundary_first: tuple | None = None
    transfer_boundary_last: tuple | None = None
    transfer_overlaps: int = 0
    submitted_since_compute: bool = False
    received: set = field(default_factory=set)
    next_sequence: int = 0
    expected: int | None = None
    committed: bool = False
    cancelled: bool = False
    ready: bool = False
    active: bool = False
    cancel_confirmed: bool = False
    compute_done: bool = False
    last_event: object = None
    acknowledged: bool = False
    started: float = field(default_factory=time.monotonic)


def _phase_name(phase) -> str:
    return str(getattr(phase, "name", phase)).upper()


def _event_done(event) -> bool:
    return event is None or bool(event.query())


class PDStageConnector:
    def __init__(self, engine, hidden, transport, config, *, notify):
        self.engine = engine
        self.cache = engine.cache_manager
        self.hidden = hidden
        self.transport = transport
        self.config = config
        self.notify = notify
        self.transfers: dict[str, RequestTransfer] = {}
        self.free_slots = list(range(len(hidden) - 1, -1, -1))
        self.transfer_cursor = 0
        self.prefill_tokens = 0
        self._verbs = {
            "connect": self._on_connect,
            "reserve": self._on_reserve,
            "prefill": self._on_reserve,
            "cancel": lambda c: self.cancel(c["tid"]),
            "cancel_safe": lambda c: self.cancel_safe(c["tid"]),
            "commit": lambda c: self.commit(c["tid"], c["count"]),
            "ack": lambda c: self.acknowledge(c["tid"]),
        }

    # ------------------------------------------------------------------ construction / handshake

    @classmethod
    def create(cls, engine, *, config, notify, transport_factory=None):
        """Allocate the staging rows on the stage's device and register the pools with the transport.

        Row count as in vllm_rlt/pd/connector.py:62-76: one per schedulable sequence, plus the
        receive window on a decode stage and the drain window on a prefill stage.
        """
        import torch

        from .transport import B200Transport

        stage = engine.stage_config
        rows = engine.scheduler.config.max_num_seqs
        if stage.produces_tokens:
            rows += config.max_receiving_requests
        if stage.accepts_prompt:
            rows += config.max_draining_requests
        anchor = next(engine.model.parameters())
        hidden = torch.empty((rows, engine.model.config.hidden_size), device=anchor.device, dtype=anchor.dtype)
        factory = transport_factory or B200Transport
        return cls(engine, hidden, factory(stage.stage_id, engine.cache_manager, hidden, config), config, notify=notify)

    def startup_info(self):
        """Transport info plus a fingerprint of model config, weights, dtype, layout and attention
        (vllm_rlt/pd/connector.py:78-98); the coordinator refuses workers whose fingerprints differ."""
        import torch

        weights = hashlib.sha256()
        for tensor in self.engine.model.state_dict().values():
            weights.update(tensor.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes())
        anchor = next(self.engine.model.parameters())
        model_config = self.engine.model.config
        described = dict(
            model=asdict(model_config) if is_dataclass(model_config) else dict(vars(model_config)),
            weights=weights.hexdigest(),
            dtype=str(anchor.dtype).removeprefix("torch."),
            layout=self.cache.layout,
            attention=self.cache.attention_info,
        )
        fingerprint = hashlib.sha256(json.dumps(described, sort_keys=True).encode()).hexdigest()
        return dict(info=self.transport.info, fingerprint=fingerprint, transfer_slots=len(self.hidden))

    @property
    def has_pending(self):
        return bool(self.transfers or self.transport.pending)

    # ------------------------------------------------------------------ control verbs

    def command(self, command):
        kind = command["kind"]
        handler = self._verbs.get(kind)
        if handler is not None:
            handler(command)
            return True
        if kind == "abort" and command["request_id"] in self.transfers:
            raise ValueError("transferred requests must use the transfer cancellation protocol")
        return False

    def _on_connect(self, command):
        for peer in command["peers"]:
            self.transport.connect(peer)
        self.notify("connected")

    def _on_reserve(self, command):
        self.reserve(
            command["tid"], command["tokens"], command["params"],
            receiving=command["kind"] == "reserve",
            peer=command["peer"],
            trace_id=command.get("trace_id"),
            target_tables=command.get("tables", ()),
            target_slot=command.get("slot", 0),
            target_cached_tokens=command.get("cached_tokens", 0),
        )

    def close(self):
        if self.has_pending:
            raise RuntimeError("cannot close a connector with pending transfers")
        self.transport.close()
        return dict(
            prefill_tokens=self.prefill_tokens,
            bytes_sent=self.transport.bytes_sent,
            transfers=self.transport.transfers,
            transfer_seconds=self.transport.transfer_seconds,
        )

    # ------------------------------------------------------------------ StageConnector part

    def exports(self, request):
        t = self.transfers.get(request.request_id)
        return t is not None and t.request is request and t.outgoing

    def can_schedule(self, request):
        """Back-pressure for an exporting request: its queue is drained, its last event has fired, and the
        in-flight budget has room (vllm_rlt/pd/connector.py:175-186). Never mutates anything."""
        if not self.exports(request):
            return True
        t = self.transfers[request.request_id]
        return bool(
            not t.cancelled
            and not t.chunks
            and _event_done(t.last_event)
            and self.transport.inflight_bytes < self.config.max_inflight_bytes
        )

    def prefill_submitted(self, request, *, phase, start, progress, event, stream):
        import torch

        t = self.transfers[request.request_id]
        if t.request is not request:
            raise RuntimeError("stale transfer generation")
        name = _phase_name(phase)
        wavefront = getattr(self.engine.scheduler.config, "wavefront_chunked_prefill", False)
        if name == "PREFILLING_PRELUDE" or (name == "PREFILLING_RECURRENT" and wavefront):
            # The transfer overlapped this compute step if it is on the wire now or went out since the last one.
            t.transfer_overlaps += bool(self.transport.busy(t.tid) or t.submitted_since_compute)
        t.submitted_since_compute = False
        if not progress.chunk_complete:
            t.last_event = event
            return
        stream = stream or torch.cuda.current_stream(self.cache.device)
        with torch.cuda.stream(stream):
            if event is not None:
                stream.wait_event(event)
            if progress.prompt_complete:
                self.hidden[t.slot].copy_(request.hidden_state)
            ready = torch.cuda.Event()
            ready.record(stream)
        t.last_event = ready
        self.prefill_tokens += request.num_prefilled_tokens - start
        self.queue_chunk(t, start, request.num_prefilled_tokens, ready, progress.prompt_complete)
        t.compute_done = progress.prompt_complete

    # ------------------------------------------------------------------ planning

    def _token_plane_bytes(self) -> int:
        info = self.transport.info
        per = info["token_bytes"]
        if info.get("scale_region") is not None:
            per += info["scale_region"]["token_bytes"]
        return 2 * info["num_layers"] * per

    def queue_chunk(self, transfer, start, end, event, final):
        """Cut tokens ``[start, end)`` into table chunks no larger than ``transfer_chunk_bytes``.

        The prefix skip (``start = max(start, target_cached_tokens)``) and the boundary
        bookkeeping are those of vllm_rlt/pd/connector.py:220-229; the hidden row rides with the
        last chunk when ``final`` (:232-241).
        """
        info = self.transport.info
        peer = self.transport.peers[transfer.peer]
        tables = self.cache.plane_block_tables(transfer.tid)
        start = max(start, transfer.target_cached_tokens)
        pieces = []
        if start < end:
            span = (start, end)
            if transfer.transfer_boundary_first is None:
                transfer.transfer_boundary_first = span
            transfer.transfer_boundary_last = span
            transfer.transfer_boundary_count += 1
            if len(tables) != len(transfer.target_tables):
                raise ValueError("incompatible source/target KV geometry")
            page = info["block_size"]
            for table, target in zip(tables, transfer.target_tables):
                if end > len(table) * page or end > len(target) * page:
                    raise ValueError("KV range exceeds allocation")
            per_token = self._token_plane_bytes() * len(tables)
            step = max(1, self.config.transfer_chunk_bytes // per_token)
            at = start
            while at < end:
                stop = min(end, at + step)
                pieces.append((at, stop, (stop - at) * per_token))
                at = stop
        hidden = None
        if final:
            size = info["hidden_bytes"]
            hidden = (info["hidden_ptr"] + transfer.slot * size, peer["hidden_ptr"] + transfer.target_slot * size, size)
            if not pieces or pieces[-1][2] + size > self.config.transfer_chunk_bytes:
                pieces.append((end, end, 0))
        for index, (lo, hi, size) in enumerate(pieces):
            last = index == len(pieces) - 1
            transfer.chunks.append(TableChunk(
                event, transfer.next_sequence, tuple(tables), tuple(transfer.target_tables), lo, hi,
                size + (hidden[2] if hidden and last else 0), hidden if last else None,
            ))
            transfer.next_sequence += 1
        if self._device_ordered():
            # No need to wait for the next progress() pass: queue the copies now, behind the producer's event
            # on the device, for as long as the in-flight budget admits them.
            while transfer.chunks and not transfer.cancelled and self._submit_chunk(transfer):
                pass

    def _device_ordered(self) -> bool:
        return getattr(self.transport, "device_ordered", False) is True

    # ------------------------------------------------------------------ lifecycle

    def reserve(self, tid, tokens, params, *, receiving, peer, trace_id=None, target_tables=(), target_slot=0,
                target_cached_tokens=0):
        """One local request and one staging row per transfer generation (vllm_rlt/pd/connector.py:248-305)."""
        if tid in self.transfers:
            raise RuntimeError("duplicate transfer generation")
        role = self.engine.stage_config.role
        if not self.free_slots:
            self.notify("rejected", tid=tid, role=role)
            return
        # The prefill side only produces prompt KV and never samples; the decode side owns sampling.
        effective = params if receiving else replace(params, max_tokens=1)
        request = self.engine.reserve_transfer(tid, tokens, effective, receiving=receiving, trace_id=trace_id)
        if request is None:
            self.notify("rejected", tid=tid, role=role)
            return
        t = RequestTransfer(tid, request, self.free_slots.pop(), peer, outgoing=not receiving, trace_id=trace_id)
        t.cached_tokens = request.num_prefilled_tokens
        self.transfers[tid] = t
        if receiving:
            self.notify("reserved", tid=tid, tables=self.cache.plane_block_tables(tid), slot=t.slot,
                        cached_tokens=t.cached_tokens)
            return
        t.target_tables, t.target_slot, t.target_cached_tokens = target_tables, target_slot, target_cached_tokens
        if t.cached_tokens > target_cached_tokens:
            # The prefill side already holds more of the prompt than the decode side: send that part now.
            import torch

            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(self.cache.device))
            self.queue_chunk(t, target_cached_tokens, t.cached_tokens, event, False)
        self.notify("prefill_started", tid=tid)

    def _forget(self, t):
        self.free_slots.append(t.slot)
        del self.transfers[t.tid]
        self.notify("released", tid=t.tid, role=self.engine.stage_config.role)

    def _remove(self, t):
        if t.tid not in self.engine.scheduler.requests or self.engine.release_transfer(t.request):
            self._forget(t)

    def output_finished(self, request_id):
        t = self.transfers.get(request_id)
        if t is None:
            return
        self._mark_active(t)
        if request_id not in self.engine.scheduler.requests:
            self._forget(t)

    def _mark_active(self, t):
        if not t.active:
            t.active = True
            self.notify("activated", tid=t.tid, seconds=time.monotonic() - t.started)

    def cancel(self, transfer_id):
        t = self.transfers.get(transfer_id)
        if t is None:
            self.notify("released", tid=transfer_id, role=self.engine.stage_config.role)
            return
        t.cancelled = True
        if t.outgoing:
            t.chunks.clear()
            self.engine.suspend_transfer(t.request)
        elif t.ready:
            self._remove(t)  # every expected write was seen, so no remote writer is left

    def cancel_safe(self, transfer_id):
        t = self.transfers.get(transfer_id)
        if t is None:
            return
        if not t.cancelled:
            raise RuntimeError("unexpected cancellation acknowledgement")
        if t.outgoing:
            raise RuntimeError("source cancellation must drain local and remote accesses")
        t.cancel_confirmed = True
        self._remove(t)

    def commit(self, transfer_id, count):
        t = self.transfers.get(transfer_id)
        if t is None or t.cancelled:
            return
        if t.outgoing:
            raise RuntimeError("commit requires an incoming transfer")
        if t.expected is not None and t.expected != count:
            raise RuntimeError("conflicting transfer commit")
        if type(count) is not int or count <= 0:
            raise RuntimeError("invalid transfer commit count")
        t.expected = count

    def acknowledge(self, transfer_id):
        t = self.transfers.get(transfer_id)
        if t is None:
            return
        if not t.outgoing:
            raise RuntimeError("acknowledgement requires an outgoing transfer")
        t.acknowledged = True

    # ------------------------------------------------------------------ progress

    def progress(self):
        self.cache.poll_prefixes()
        self._take_notifications()
        order = list(self.transfers.values())
        if order:
            pivot = self.transfer_cursor % len(order)
            order = order[pivot:] + order[:pivot]
            self.transfer_cursor += 1
        for t in order:
            if t.outgoing:
                self._advance_outgoing(t)
            else:
                self._advance_incoming(t)
        # Fill the in-flight budget: further round-robin passes while any transfer still gets a chunk out.
        live = [t for t in order if t.outgoing and not t.cancelled]
        while live:
            sent = [self._submit_chunk(t) for t in live]
            if not any(sent):
                break
            live = [t for t in live if t.chunks]
        for t in order:
            if not t.outgoing or t.cancelled:
                continue
            if t.compute_done and not t.chunks and not t.committed:
                t.committed = True
                self.notify("commit", tid=t.tid, count=t.next_sequence)
            if t.acknowledged and t.committed and t.request.compute_released and not self.transport.busy(t.tid):
                self._remove(t)

    def _take_notifications(self):
        _, notifications = self.transport.poll()
        for peer, tid, sequence in notifications:
            t = self.transfers.get(tid)
            if t is None or t.cancelled:
                continue  # an old generation must not activate a reused request id
            if t.outgoing or peer != t.peer or type(sequence) is not int or sequence < 0:
                raise RuntimeError("invalid transfer completion")
            if t.ready and sequence not in t.received:
                raise RuntimeError("late KV write after decode activation")
            t.received.add(sequence)

    def _advance_outgoing(self, t):
        if t.cancelled:
            # The staging row may still be read by a queued copy: wait for local and remote users.
            if not self.transport.busy(t.tid) and _event_done(t.last_event):
                self._remove(t)
            return
        if (t.compute_done and not t.request.compute_released
                and self.engine.release_transfer_compute(t.request, ready_event=t.last_event)):
            self.notify(
                "prefill_complete", tid=t.tid,
                boundaries=(t.transfer_boundary_first, t.transfer_boundary_last, t.transfer_boundary_count),
                overlaps=t.transfer_overlaps,
            )
        self._submit_chunk(t)

    def _advance_incoming(self, t):
        if t.cancelled:
            if t.ready or t.cancel_confirmed:
                self._remove(t)
            return
        if t.ready:
            if t.request.request_id not in self.engine.scheduler.requests:
                self._forget(t)
            elif not t.active and _phase_name(t.request.phase) != "RECEIVING":
                self._mark_active(t)
            return
        if t.expected is None:
            return
        if any(seq >= t.expected for seq in t.received):
            raise RuntimeError("unexpected transfer sequence")
        if len(t.received) == t.expected:
            if not self.engine.accept_import(t.request, self.hidden[t.slot], cached_tokens=t.cached_tokens):
                raise RuntimeError("stale import activation")
            t.ready = True
            self.notify("received", tid=t.tid)

    def _submit_chunk(self, t):
        """Put the transfer's next chunk on the wire once its event has fired; True if one went out."""
        if not t.chunks:
            return False
        chunk = t.chunks[0]
        if isinstance(chunk, TableChunk):
            ordered = self._device_ordered()
            if not ordered and not chunk.event.query():
                return False
            sent = self._submit_tables(t, chunk, after=chunk.event if ordered else None)
        else:
            # a caller-built descriptor chunk: (event, sequence, local, remote, size)
            event, sequence, local, remote, size = chunk
            sent = event.query() and self.transport.submit(t.tid, sequence, t.peer, local, remote, size)
        if not sent:
            return False
        t.chunks.popleft()
        t.submitted_since_compute = True
        return True

    def _submit_tables(self, t, chunk, after=None):
        extra = [chunk.hidden] if chunk.hidden is not None else []
        ordered = {} if after is None else {"after": after}
        if chunk.start >= chunk.end:  # nothing but the hidden row
            local = [(s, n, self.transport.info["device"]) for s, _, n in extra]
            remote = [(d, n, self.transport.peers[t.peer]["device"]) for _, d, n in extra]
            return self.transport.submit(t.tid, chunk.sequence, t.peer, local, remote, chunk.size, **ordered)
        requests = [(chunk.source_tables, chunk.target_tables, chunk.start, chunk.end)]
        return self.transport.submit_tables(t.tid, chunk.sequence, t.peer, requests, chunk.size, extra=extra, **ordered)
