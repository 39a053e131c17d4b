"""Per-worker transfer state machine of the PD handoff, speaking the reference's ``TransferConnector`` protocol.

This class takes the place of the reference's ``PDStageConnector`` (vllm_rlt/pd/connector.py:49-455)
behind the unchanged protocol of vllm_rlt/engine/connector.py:9-83. The stage engine, the scheduler
and the deployment coordinator keep calling the same methods with the same meaning; the control
verbs (``connect, reserve, prefill, cancel, cancel_safe, commit, ack, abort``) and the notifications
(``connected, reserved, prefill_started, prefill_complete, commit, received, activated, released,
rejected``) are the reference's, as are the error messages callers match on.

How it is built. Every transfer generation is a ``RequestTransfer`` record whose fields are the reference's
(its tests and the coordinator read and set them). What a record is *doing* is a ``Stage``, derived from those
fields, and each of the two roles owns a table ``{Stage: step}``:

* ``Exporter`` (a prefill worker's outgoing transfers): COMPUTING -> DRAINING -> COMMITTED -> retired, with
  UNWINDING for a cancelled export that must outlive its last local and remote reader;
* ``Importer`` (a decode worker's incoming transfers): COLLECTING -> LANDED -> SERVING -> retired, with
  ABANDONED for a cancelled import that waits for the coordinator's "writers have stopped".

``progress()`` polls the transport once, lets the importer book the arrivals, gives every transfer one step of
its role's table in a rotating order, then lets the exporter fill the in-flight budget round-robin and settle
commits and retirements.

What a queued chunk is. The reference turns a token range into two Python lists of byte descriptors
(``kv_segments`` on both sides, ``partition_segments``) and submits them one list at a time. Here a chunk is a
``TableChunk``: block tables of both sides plus a token range (optionally one layer group of one plane), cut so
that its payload stays under ``transfer_chunk_bytes``. One chunk is one ``rlt_kv_handoff`` launch in which the
GPU walks the tables itself, and one ``(transfer id, sequence)`` notification. Sequence numbers, one notification
per submitted chunk and ``commit.count == next_sequence`` are kept.

Layer streaming. ``layer_written(request, plane=, layer=, event=)`` is an optional producer hook beside the
protocol: a model runner that calls it after queuing a layer's KV writes lets the slice leave while later layers
still compute; ``prefill_submitted`` then only sends what is left. Nobody calling it changes nothing.

The object asks the engine to change request, compute or KV state (``reserve_transfer``,
``accept_import``, ``release_transfer_compute``, ``release_transfer``, ``suspend_transfer``); it owns
only transfer bookkeeping and the hidden-state staging rows.
"""

from __future__ import annotations

import enum
import hashlib
import json
import time
from collections import deque
from dataclasses import asdict, dataclass, field, is_dataclass, replace


@dataclass
class TableChunk:
    """One bounded submission: tokens ``[start, end)`` by block table, of every plane and layer unless sliced."""

    event: object
    sequence: int
    source_tables: tuple
    target_tables: tuple
    start: int
    end: int
    size: int
    hidden: tuple | None = None  # (source address, target address, bytes) of the final hidden row
    planes: tuple[int, int] | None = None  # destination plane slice [begin, end), None = every plane
    layers: tuple[int, int] | None = None  # layer slice [begin, end), None = every layer


@dataclass
class RequestTransfer:
    """Bookkeeping of one transfer generation. The fields up to ``started`` are those of the reference's record
    (vllm_rlt/pd/connector.py:17-46), which its tests and tools construct and poke directly."""

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
    # layer streaming: per destination plane, how many layers of the current prefill window have left already
    streamed_layers: dict = field(default_factory=dict)
    streamed_window: tuple | None = None
    stream_refused: tuple | None = None  # a window whose early slices were withdrawn: it leaves whole at the chunk's end

    def note_range(self, start: int, end: int) -> None:
        """Remember the first and last token range put on the wire, and how many there were."""
        if self.transfer_boundary_first is None:
            self.transfer_boundary_first = (start, end)
        self.transfer_boundary_last = (start, end)
        self.transfer_boundary_count += 1


class Stage(enum.Enum):
    """What a transfer generation is doing, as far as this worker is concerned."""

    # outgoing
    COMPUTING = "prompt still being computed; finished ranges leave as they are queued"
    DRAINING = "prompt computed; queued chunks are still going out"
    COMMITTED = "every chunk is out and the count is announced; waits for ack, compute release, last reader"
    UNWINDING = "cancelled export: waits for its local and remote readers to finish"
    # incoming
    COLLECTING = "reserved; notifications are being counted against the announced total"
    LANDED = "complete and handed to the engine; waits for a compute slot"
    SERVING = "admitted to compute; the record lives until the request leaves the scheduler"
    ABANDONED = "cancelled import: waits for proof that no writer is left"


def stage_of(t: RequestTransfer) -> Stage:
    if t.outgoing:
        if t.cancelled:
            return Stage.UNWINDING
        if t.committed:
            return Stage.COMMITTED
        return Stage.DRAINING if t.compute_done else Stage.COMPUTING
    if t.cancelled:
        return Stage.ABANDONED
    if not t.ready:
        return Stage.COLLECTING
    return Stage.SERVING if t.active else Stage.LANDED


def _phase_name(phase) -> str:
    return str(getattr(phase, "name", phase)).upper()


def _fired(event) -> bool:
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
        self.free_slots = [*range(len(hidden))][::-1]
        self.transfer_cursor = 0
        self.prefill_tokens = 0
        self.stream_layers = 4  # layers per slice that ``layer_written`` lets go at once
        self.stream_whole_planes = False  # True: a plane leaves in one piece, the last plane in two (few launches per step)
        self.layer_watch = None  # set by ``create`` when this worker reports its KV writes itself (pd/layer_watch.py)
        self._early_arrivals: list = []  # arrivals a poll inside a step brought in (see ``report_layer``)
        self.exporter = Exporter(self)
        self.importer = Importer(self)
        self._control = {
            "connect": lambda c: self._connect(c["peers"]),
            "reserve": lambda c: self._reserve_from(c, receiving=True),
            "prefill": lambda c: self._reserve_from(c, receiving=False),
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
        rows += config.max_receiving_requests if stage.produces_tokens else 0
        rows += config.max_draining_requests if stage.accepts_prompt else 0
        anchor = next(engine.model.parameters())
        hidden = torch.empty((rows, engine.model.config.hidden_size), device=anchor.device, dtype=anchor.dtype)
        make = transport_factory or B200Transport
        connector = cls(engine, hidden, make(stage.stage_id, engine.cache_manager, hidden, config), config, notify=notify)
        from . import layer_watch

        if layer_watch.wanted() and stage.accepts_prompt and layer_watch.eligible(connector):
            connector.layer_watch = layer_watch.LayerWatch(connector).install()
            connector.stream_whole_planes = True
        return connector

    def startup_info(self):
        """Transport info plus a fingerprint of model config, weights, dtype, layout and attention
        (vllm_rlt/pd/connector.py:78-98); the coordinator refuses workers whose fingerprints differ."""
        import torch

        model = self.engine.model
        weights = hashlib.sha256()
        for tensor in model.state_dict().values():
            weights.update(tensor.detach().contiguous().view(torch.uint8).cpu().numpy().tobytes())
        settings = model.config
        identity = {
            "model": asdict(settings) if is_dataclass(settings) else dict(vars(settings)),
            "weights": weights.hexdigest(),
            "dtype": str(next(model.parameters()).dtype).removeprefix("torch."),
            "layout": self.cache.layout,
            "attention": self.cache.attention_info,
        }
        fingerprint = hashlib.sha256(json.dumps(identity, sort_keys=True).encode()).hexdigest()
        return {"info": self.transport.info, "fingerprint": fingerprint, "transfer_slots": len(self.hidden)}

    @property
    def has_pending(self):
        return bool(self.transfers or self.transport.pending or getattr(self.transport, "reading", False) is True)

    # ------------------------------------------------------------------ control verbs

    def command(self, command):
        kind = command["kind"]
        if kind in self._control:
            self._control[kind](command)
            return True
        if kind == "abort" and command["request_id"] in self.transfers:
            raise ValueError("transferred requests must use the transfer cancellation protocol")
        return False

    def _connect(self, peers):
        for peer in peers:
            self.transport.connect(peer)
        self.notify("connected")

    def _reserve_from(self, command, *, receiving):
        self.reserve(command["tid"], command["tokens"], command["params"], receiving=receiving, peer=command["peer"],
                     trace_id=command.get("trace_id"), target_tables=command.get("tables", ()),
                     target_slot=command.get("slot", 0), target_cached_tokens=command.get("cached_tokens", 0))

    def close(self):
        if self.has_pending:
            raise RuntimeError("cannot close a connector with pending transfers")
        self.transport.close()
        t = self.transport
        metrics = {"prefill_tokens": self.prefill_tokens, "bytes_sent": t.bytes_sent, "transfers": t.transfers,
                   "transfer_seconds": t.transfer_seconds}
        if self.layer_watch is not None:
            self.layer_watch.remove()
            metrics["streamed_slices"] = self.layer_watch.reported
            metrics["stream_host_seconds"] = self.layer_watch.host_seconds
            if self.layer_watch.failure is not None:
                metrics["stream_failure"] = self.layer_watch.failure
        received = getattr(t, "bytes_received", 0)
        if isinstance(received, int) and received:  # the pull direction: what this worker's GPU read, and for how long
            rates = sorted(getattr(t, "pull_rates", ()))
            metrics.update(bytes_received=received, pull_seconds=t.pull_seconds,
                           pull_gbps_p50=rates[len(rates) // 2] if rates else 0.0)
        return metrics

    # ------------------------------------------------------------------ StageConnector part

    def _export_of(self, request):
        t = self.transfers.get(request.request_id)
        return t if t is not None and t.outgoing and t.request is request else None

    def exports(self, request):
        return self._export_of(request) is not None

    def can_schedule(self, request):
        """Back-pressure for an exporting request (vllm_rlt/pd/connector.py:175-186): it may compute again once
        nothing of it is queued, its last event has fired and the in-flight budget has room. Mutates nothing."""
        t = self._export_of(request)
        if t is None:
            return True
        if t.cancelled or t.chunks or not _fired(t.last_event):
            return False
        return self.transport.inflight_bytes < self.config.max_inflight_bytes

    def prefill_submitted(self, request, *, phase, start, progress, event, stream):
        """The engine has queued one prefill step of an exporting request
        (vllm_rlt/engine/connector.py:18-33, vllm_rlt/pd/connector.py:188-218)."""
        t = self.transfers[request.request_id]
        if t.request is not request:
            raise RuntimeError("stale transfer generation")
        self.exporter.step_submitted(t, _phase_name(phase), start, progress, event, stream)

    def layer_written(self, request, *, plane, layer, event=None, start=None, end=None):
        """Optional producer hook: the KV writes of ``layer`` at destination plane ``plane`` for the tokens
        ``[start, end)`` of the request's current prefill window have been queued, all earlier layers of that plane
        too, and ``event`` (recorded by the caller after them) covers them. Returns True if a slice was queued.

        ``start`` / ``end`` default to the window ``[num_prefilled_tokens, ...)`` the engine reports with the next
        ``prefill_submitted``; callers that know the window pass it. Slices are cut at ``stream_layers`` layers.
        """
        t = self._export_of(request)
        if t is None or t.cancelled:
            return False
        return self.exporter.layer_written(t, plane, layer, event, start, end)

    def report_layer(self, request_id, plane, layer, start, end, *, event=None) -> bool:
        """``layer_written`` for a reporter that sits inside the model's forward (pd/layer_watch.py): it knows the
        request by id, passes the window it saw, and must never get an exception back. A plane that is written a
        second time inside one window withdraws the window from streaming: what left early may be stale, so the whole
        window leaves at the chunk's end, as without streaming."""
        t = self.transfers.get(request_id)
        if t is None or not t.outgoing or t.cancelled or t.compute_done:
            return False
        window = (max(start, t.target_cached_tokens), end)
        if window[0] >= window[1] or t.stream_refused == window:
            return False
        if t.streamed_window == window and layer + 1 <= t.streamed_layers.get(plane, 0):
            t.streamed_window, t.streamed_layers, t.stream_refused = None, {}, window
            return False
        if not 0 <= plane < len(t.target_tables) or not 0 <= layer < self.transport.info["num_layers"]:
            return False
        if 2 * self.transport.inflight_bytes > self.config.max_inflight_bytes:
            # tickets are normally returned by progress(), between steps; a step that streams more than the budget
            # holds would stall its own later slices, so finished ones are returned here and what the poll brought
            # in is kept for the next progress()
            self._early_arrivals += self.transport.poll()[1]
        return self.exporter.layer_written(t, plane, layer, event, start, end)

    # ------------------------------------------------------------------ planning

    def _row_bytes(self) -> int:
        """Bytes of one token of one layer of K or V, scales included when they travel."""
        info = self.transport.info
        scales = info.get("scale_region")
        return info["token_bytes"] + (scales["token_bytes"] if scales is not None else 0)

    def queue_chunk(self, transfer, start, end, event, final):
        """Queue tokens ``[start, end)`` of every plane behind ``event``; with ``final`` the hidden row rides on the
        last chunk. Same contract as vllm_rlt/pd/connector.py:220-246: the decode side's cached prefix is skipped
        and every chunk gets the next sequence number."""
        self.exporter.queue_range(transfer, start, end, event, final)

    def _device_ordered(self) -> bool:
        return getattr(self.transport, "device_ordered", False) is True

    # ------------------------------------------------------------------ lifecycle

    def reserve(self, tid, tokens, params, *, receiving, peer, trace_id=None, target_tables=(), target_slot=0,
                target_cached_tokens=0):
        """One local request and one staging row per transfer generation (vllm_rlt/pd/connector.py:248-305)."""
        if tid in self.transfers:
            raise RuntimeError("duplicate transfer generation")
        role = self.engine.stage_config.role
        request = None
        if self.free_slots:
            # a prefill worker only produces prompt KV and never samples: one token of budget is all it needs
            wanted = params if receiving else replace(params, max_tokens=1)
            request = self.engine.reserve_transfer(tid, tokens, wanted, receiving=receiving, trace_id=trace_id)
        if request is None:
            self.notify("rejected", tid=tid, role=role)
            return
        t = RequestTransfer(tid, request, self.free_slots.pop(), peer, outgoing=not receiving, trace_id=trace_id,
                            cached_tokens=request.num_prefilled_tokens)
        self.transfers[tid] = t
        (self.importer if receiving else self.exporter).opened(t, target_tables, target_slot, target_cached_tokens)

    def _forget(self, t):
        self.free_slots.append(t.slot)
        del self.transfers[t.tid]
        self.notify("released", tid=t.tid, role=self.engine.stage_config.role)

    def _remove(self, t):
        """Retire a generation: the engine lets go of request and KV first, unless it no longer knows the request."""
        if t.tid in self.engine.scheduler.requests and not self.engine.release_transfer(t.request):
            return
        self._forget(t)

    def _trace(self, what, tid):
        note = getattr(self.transport, "_note", None)  # the transport's optional chunk trace (RLT_KV_TRACE)
        if callable(note) and getattr(self.transport, "_trace_dir", None):
            note(what, tid, -1)

    def _announce_active(self, t):
        if t.active:
            return
        t.active = True
        self.notify("activated", tid=t.tid, seconds=time.monotonic() - t.started)

    def output_finished(self, request_id):
        t = self.transfers.get(request_id)
        if t is None:
            return
        self._announce_active(t)
        if request_id not in self.engine.scheduler.requests:
            self._forget(t)

    def cancel(self, transfer_id):
        t = self.transfers.get(transfer_id)
        if t is None:
            self.notify("released", tid=transfer_id, role=self.engine.stage_config.role)
            return
        t.cancelled = True
        (self.exporter if t.outgoing else self.importer).cancelled(t)

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
        self._trace("commit arrived", transfer_id)

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
        _, arrivals = self.transport.poll()
        if self._early_arrivals:
            arrivals, self._early_arrivals = self._early_arrivals + list(arrivals), []
        self.importer.book(arrivals)
        turn = list(self.transfers.values())
        if turn:
            first = self.transfer_cursor % len(turn)
            turn = turn[first:] + turn[:first]
            self.transfer_cursor += 1
        for t in turn:
            role = self.exporter if t.outgoing else self.importer
            role.table[stage_of(t)](t)
        self.exporter.fill_budget(turn)
        self.exporter.settle(turn)

    def _submit_chunk(self, t):
        """Put the transfer's next chunk on the wire once its event allows; True if one went out."""
        return self.exporter.send_next(t)


class Exporter:
    """Outgoing side: ranges of a prompt leave as the prefill finishes them; the source is retired in two steps."""

    def __init__(self, connector: PDStageConnector):
        self.c = connector
        self.table = {
            Stage.COMPUTING: self.send_next,
            Stage.DRAINING: self.drain,
            Stage.COMMITTED: self.drain,
            Stage.UNWINDING: self.unwind,
        }

    # -- opening and cancelling

    def opened(self, t, target_tables, target_slot, target_cached_tokens):
        c = self.c
        t.target_tables, t.target_slot, t.target_cached_tokens = target_tables, target_slot, target_cached_tokens
        if t.cached_tokens > target_cached_tokens:
            # this worker already holds more of the prompt than the decode side (its own prefix cache): that part
            # can leave at once, behind whatever the compute stream has queued so far
            import torch

            marker = torch.cuda.Event()
            marker.record(torch.cuda.current_stream(c.cache.device))
            c.queue_chunk(t, target_cached_tokens, t.cached_tokens, marker, False)
        c.notify("prefill_started", tid=t.tid)

    def cancelled(self, t):
        t.chunks.clear()
        self.c.engine.suspend_transfer(t.request)

    # -- the engine's reports

    def step_submitted(self, t, phase, start, progress, event, stream):
        import torch

        c = self.c
        wavefront = getattr(c.engine.scheduler.config, "wavefront_chunked_prefill", False)
        if phase == "PREFILLING_PRELUDE" or (wavefront and phase == "PREFILLING_RECURRENT"):
            # the transfer overlapped this compute step if it is on the wire now or went out since the last one
            t.transfer_overlaps += bool(c.transport.busy(t.tid) or t.submitted_since_compute)
        t.submitted_since_compute = False
        if not progress.chunk_complete:
            t.last_event = event
            return
        request = t.request
        lane = stream or torch.cuda.current_stream(c.cache.device)
        with torch.cuda.stream(lane):
            if event is not None:
                lane.wait_event(event)
            if progress.prompt_complete:
                c.hidden[t.slot].copy_(request.hidden_state)
            ready = torch.cuda.Event()
            ready.record(lane)
        t.last_event = ready
        end = request.num_prefilled_tokens
        c.prefill_tokens += end - start
        c.queue_chunk(t, start, end, ready, progress.prompt_complete)
        t.compute_done = progress.prompt_complete

    def layer_written(self, t, plane, layer, event, start, end):
        c = self.c
        info = c.transport.info
        layers_total = info["num_layers"]
        if not 0 <= layer < layers_total or not 0 <= plane < len(t.target_tables):
            raise ValueError("layer or plane outside the pool")
        request = t.request
        lo = request.num_prefilled_tokens if start is None else start
        hi = len(request.prompt_token_ids) if end is None else end
        lo = max(lo, t.target_cached_tokens)
        if lo >= hi:
            return False
        if t.streamed_window != (lo, hi):
            t.streamed_window, t.streamed_layers = (lo, hi), {}
        sent = t.streamed_layers.get(plane, 0)
        if layer + 1 <= sent:
            raise ValueError("layers of a plane must be reported in increasing order")
        group = max(1, int(c.stream_layers))
        if c.stream_whole_planes:
            # Only what is still to move when the step ends counts as latency: a plane leaves in one piece after its
            # last layer, and the last plane in two, so that its final ``stream_layers`` layers are all that is left.
            cut = layers_total - group
            early = plane + 1 == len(t.target_tables) and layer + 1 == cut and cut > sent
            if not early and layer + 1 < layers_total:
                return False
        elif layer + 1 - sent < group and layer + 1 < layers_total:
            return False
        if event is None:
            import torch

            event = torch.cuda.Event()
            event.record(torch.cuda.current_stream(c.cache.device))
        tables = c.cache.plane_block_tables(t.tid)
        self._enqueue(t, tables, lo, hi, event, planes=(plane, plane + 1), layers=(sent, layer + 1))
        t.streamed_layers[plane] = layer + 1
        t.last_event = event
        self.flush(t)
        return True

    # -- planning

    def queue_range(self, t, start, end, event, final):
        c = self.c
        info = c.transport.info
        start = max(start, t.target_cached_tokens)
        tables = c.cache.plane_block_tables(t.tid)
        if start < end:
            t.note_range(start, end)
            if len(tables) != len(t.target_tables):
                raise ValueError("incompatible source/target KV geometry")
            if t.streamed_window == (start, end):
                # layer_written already sent part of this window: only the layers it did not reach are left
                for plane in range(len(tables)):
                    sent = t.streamed_layers.get(plane, 0)
                    if sent < info["num_layers"]:
                        self._enqueue(t, tables, start, end, event, planes=(plane, plane + 1),
                                      layers=(sent, info["num_layers"]))
                t.streamed_window, t.streamed_layers = None, {}
            else:
                self._enqueue(t, tables, start, end, event)
        if final:
            self._attach_hidden(t, tables, end, event)
        self.flush(t)

    def _enqueue(self, t, tables, start, end, event, *, planes=None, layers=None):
        """Cut ``[start, end)`` (of a plane / layer slice, if given) into chunks under ``transfer_chunk_bytes``:
        by tokens while one token fits, by plane and then by layer group when even one token is too large."""
        c = self.c
        info = c.transport.info
        page = info["block_size"]
        for table in (*tables, *t.target_tables):
            if end > len(table) * page:
                raise ValueError("KV range exceeds allocation")
        limit = c.config.transfer_chunk_bytes
        plane_lo, plane_hi = planes or (0, len(tables))
        layer_lo, layer_hi = layers or (0, info["num_layers"])
        row = 2 * c._row_bytes()  # K and V of one token of one layer
        slices = [(planes, layers)]
        if (plane_hi - plane_lo) * (layer_hi - layer_lo) * row > limit:
            if row > limit:
                raise ValueError("transfer_chunk_bytes is smaller than one token row of one layer")
            per_layer_group = limit // row
            slices = [((plane, plane + 1), (at, min(layer_hi, at + per_layer_group)))
                      for plane in range(plane_lo, plane_hi) for at in range(layer_lo, layer_hi, per_layer_group)]
        for plane_slice, layer_slice in slices:
            p0, p1 = plane_slice or (0, len(tables))
            l0, l1 = layer_slice or (0, info["num_layers"])
            per_token = (p1 - p0) * (l1 - l0) * row
            step = max(1, limit // per_token)
            for at in range(start, end, step):
                stop = min(end, at + step)
                t.chunks.append(TableChunk(event, t.next_sequence, tuple(tables), tuple(t.target_tables), at, stop,
                                           (stop - at) * per_token, None, plane_slice, layer_slice))
                t.next_sequence += 1

    def _attach_hidden(self, t, tables, end, event):
        """The final hidden-state row rides on the last queued chunk if it fits, else goes alone."""
        c = self.c
        info, peer = c.transport.info, c.transport.peers[t.peer]
        size = info["hidden_bytes"]
        row = (info["hidden_ptr"] + t.slot * size, peer["hidden_ptr"] + t.target_slot * size, size)
        last = t.chunks[-1] if t.chunks else None
        if isinstance(last, TableChunk) and last.event is event and last.size + size <= c.config.transfer_chunk_bytes:
            last.hidden, last.size = row, last.size + size
            return
        t.chunks.append(TableChunk(event, t.next_sequence, tuple(tables), tuple(t.target_tables), end, end, size, row))
        t.next_sequence += 1

    # -- sending

    def flush(self, t):
        """With a device-ordered transport nothing waits for the next ``progress()``: queue the copies now, behind
        the producer's event on the device, for as long as the in-flight budget admits them."""
        if self.c._device_ordered():
            while t.chunks and not t.cancelled and self.send_next(t):
                pass

    def send_next(self, t):
        """Put the head of the transfer's queue on the wire: a caller-built descriptor chunk alone, table chunks
        together with every chunk behind them that is ready at the same moment (one launch, see ``_group``)."""
        if not t.chunks:
            return False
        head = t.chunks[0]
        if not isinstance(head, TableChunk):
            if not self._send_descriptors(t, head):
                return False
            taken = 1
        else:
            taken = self._send_table_chunks(t)
        for _ in range(taken):
            t.chunks.popleft()
        t.submitted_since_compute = t.submitted_since_compute or taken > 0
        return taken > 0

    def _group(self, t):
        """The table chunks at the head of the queue that can leave as one launch: same producer event, same plane and
        layer slice, token ranges that continue one another (a trailing hidden-row-only chunk joins too), and as
        many of them as the in-flight budget has room for (always at least the first)."""
        head = t.chunks[0]
        room = self.c.config.max_inflight_bytes - self.c.transport.inflight_bytes
        group, total, end = [], 0, head.start
        for chunk in t.chunks:
            if not isinstance(chunk, TableChunk):
                break
            same_launch = (chunk.event is head.event and chunk.planes == head.planes and chunk.layers == head.layers
                           and chunk.source_tables == head.source_tables and chunk.target_tables == head.target_tables)
            if not same_launch or chunk.start != end:  # a hidden-row-only chunk sits at the end of its range
                break
            if group and (total + chunk.size > room or len(group) == 255):
                break
            group.append(chunk)
            total += chunk.size
            end = max(end, chunk.end)
            if chunk.hidden is not None:
                break  # the hidden row closes a prompt: nothing follows it
        return group

    def _send_descriptors(self, t, chunk):
        """A caller-built descriptor chunk, the reference's form: (event, sequence, local, remote, size)."""
        event, sequence, local, remote, size = chunk
        return event.query() and self.c.transport.submit(t.tid, sequence, t.peer, local, remote, size)

    def _send_table_chunks(self, t):
        """Submit the head group; returns how many chunks went out (0: not now)."""
        transport = self.c.transport
        head = t.chunks[0]
        behind = {}
        if self.c._device_ordered():
            behind["after"] = head.event
        elif not head.event.query():
            return 0
        group = self._group(t)
        riders = [c.hidden for c in group if c.hidden is not None]
        start, end = group[0].start, max(c.end for c in group)
        total = sum(c.size for c in group)
        if start >= end:  # nothing but the hidden row
            here, there = transport.info["device"], transport.peers[t.peer]["device"]
            sent = transport.submit(t.tid, head.sequence, t.peer, [(s, n, here) for s, _, n in riders],
                                    [(d, n, there) for _, d, n in riders], head.size, **behind)
            return 1 if sent else 0
        where = {}
        if head.planes is not None:
            where.update(plane_begin=head.planes[0], plane_end=head.planes[1])
        if head.layers is not None:
            where.update(layer_begin=head.layers[0], layer_end=head.layers[1])
        if len(group) > 1:
            where["parts"] = [(c.sequence, c.size) for c in group]
        sent = transport.submit_tables(t.tid, head.sequence, t.peer, [(head.source_tables, head.target_tables, start, end)],
                                       total, extra=riders, **where, **behind)
        return len(group) if sent else 0

    # -- table steps

    def drain(self, t):
        c = self.c
        if (t.compute_done and not t.request.compute_released
                and c.engine.release_transfer_compute(t.request, ready_event=t.last_event)):
            c.notify("prefill_complete", tid=t.tid, overlaps=t.transfer_overlaps,
                     boundaries=(t.transfer_boundary_first, t.transfer_boundary_last, t.transfer_boundary_count))
            c._trace("prefill_complete sent", t.tid)
        self.send_next(t)

    def unwind(self, t):
        # the staging row may still be read by a queued copy, the KV by the peer: both must be over
        if not self.c.transport.busy(t.tid) and _fired(t.last_event):
            self.c._remove(t)

    # -- after everyone has had a turn

    def fill_budget(self, turn):
        """Further round-robin passes over the live exports while any of them still gets a chunk out."""
        live = [t for t in turn if t.outgoing and not t.cancelled and t.tid in self.c.transfers]
        while live:
            went = [self.send_next(t) for t in live]
            if True not in went:
                return
            live = [t for t in live if t.chunks]

    def settle(self, turn):
        c = self.c
        for t in turn:
            if not t.outgoing or t.cancelled or t.tid not in c.transfers:
                continue
            if not t.committed and t.compute_done and not t.chunks:
                t.committed = True
                c.notify("commit", tid=t.tid, count=t.next_sequence)
                c._trace("commit sent", t.tid)
            if t.committed and t.acknowledged and t.request.compute_released and not c.transport.busy(t.tid):
                c._remove(t)


class Importer:
    """Incoming side: count arrivals against the announced total, hand the request to the engine, keep the record
    until the request has left the scheduler."""

    def __init__(self, connector: PDStageConnector):
        self.c = connector
        self.table = {
            Stage.COLLECTING: self.collect,
            Stage.LANDED: self.watch,
            Stage.SERVING: self.watch,
            Stage.ABANDONED: self.abandon,
        }

    def opened(self, t, *_):
        c = self.c
        c.notify("reserved", tid=t.tid, tables=c.cache.plane_block_tables(t.tid), slot=t.slot, cached_tokens=t.cached_tokens)

    def cancelled(self, t):
        if t.ready:
            self.c._remove(t)  # every expected write was seen, so no remote writer is left

    def book(self, arrivals):
        for peer, tid, sequence in arrivals:
            t = self.c.transfers.get(tid)
            if t is None or t.cancelled:
                continue  # a generation that is gone must not activate whoever reuses its request id
            if t.outgoing or peer != t.peer or type(sequence) is not int or sequence < 0:
                raise RuntimeError("invalid transfer completion")
            if t.ready and sequence not in t.received:
                raise RuntimeError("late KV write after decode activation")
            t.received.add(sequence)

    def collect(self, t):
        c = self.c
        if t.expected is None:
            return
        if t.received and max(t.received) >= t.expected:
            raise RuntimeError("unexpected transfer sequence")
        if len(t.received) < t.expected:
            return
        c._trace("all chunks landed", t.tid)
        if not c.engine.accept_import(t.request, c.hidden[t.slot], cached_tokens=t.cached_tokens):
            raise RuntimeError("stale import activation")
        t.ready = True
        c.notify("received", tid=t.tid)
        c._trace("received sent", t.tid)

    def watch(self, t):
        c = self.c
        if t.request.request_id not in c.engine.scheduler.requests:
            c._forget(t)
        elif not t.active and _phase_name(t.request.phase) != "RECEIVING":
            c._announce_active(t)

    def abandon(self, t):
        if t.ready or t.cancel_confirmed:
            self.c._remove(t)
