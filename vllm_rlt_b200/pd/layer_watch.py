"""Layer streaming without a source edit: reports a prefill worker's KV writes to its connector as they are queued.

``PDStageConnector.layer_written`` is the hook a model runner calls after the KV write of a layer
(vllm_rlt/models/ouro.py:185 is the call site a maintainer would use). Where the runner is not edited, this module gets
the same information from the cache manager itself: every eager prefill traversal writes its K/V rows through
``KVCacheManager._write_prepared(layer, batch, k, v)`` (vllm_rlt/core/kv_cache_manager.py:848-886) with a ``KVMetadata``
batch whose host rows say which request, depth and positions the rows belong to (vllm_rlt/worker/metadata.py:21-41).
``LayerWatch`` wraps that one bound method ON THE WORKER'S OWN CACHE MANAGER INSTANCE, lets the write go ahead
unchanged and then tells the connector "layer L of plane P of request R, tokens [a, b), is queued".

It is switched on per worker with ``RLT_KV_STREAM=1`` and only where reporting early is safe:

* a depth owns its plane (``last_exited`` storage: plane = depth). In a layout where several depths write one plane a
  row is rewritten later in the same step, so nothing may leave early;
* prefill is not wavefront-chunked (there one step advances several windows of a request at different depths, which the
  connector's one-window bookkeeping would answer by sending everything twice).

Everything else (graph-captured steps, which go through the runner's own device cache object; batches without host
rows; requests that are not being exported; rows that are not one contiguous range) is simply not reported, and the
next ``prefill_submitted`` sends whatever was not streamed, as it always does.
"""

from __future__ import annotations

import os
import time


def wanted() -> bool:
    return os.environ.get("RLT_KV_STREAM", "").strip().lower() in ("1", "true", "yes", "on", "alternate")


def alternate() -> bool:
    """``RLT_KV_STREAM=alternate``: every second request streams, the others leave at the chunk's end as usual. For
    measuring what streaming costs and saves inside ONE process, where run-to-run differences cannot blur it."""
    return os.environ.get("RLT_KV_STREAM", "").strip().lower() == "alternate"


def eligible(connector) -> bool:
    """Whether this worker's storage and scheduler allow layers to leave early (see the module docstring)."""
    cache = connector.cache
    depths = getattr(cache, "max_loops", None)
    plane_of = getattr(cache, "_plane", None)
    if not isinstance(depths, int) or not callable(plane_of) or not callable(getattr(cache, "_write_prepared", None)):
        return False
    if len({plane_of(d) for d in range(depths)}) != depths:
        return False
    return not getattr(connector.engine.scheduler.config, "wavefront_chunked_prefill", False)


class LayerWatch:
    """Stands in for ``cache._write_prepared`` on one cache manager instance."""

    def __init__(self, connector):
        self.connector = connector
        self.cache = connector.cache
        self.write = self.cache._write_prepared  # the bound original
        self.shadowed = self.cache.__dict__.get("_write_prepared")  # normally None: the original is the class's method
        self.plan_of = None   # the batch object the plan below was made for
        self.plan = ()        # [(request id, plane, first token, end token)]
        self.reported = 0     # slices that left early, for the metrics
        self.host_seconds = 0.0  # time this object added to the forward, for the metrics
        self.failure = None   # what made this object stop reporting, if anything did
        self.alternate = alternate()
        self.order = {}       # request id -> the order in which requests were first seen (alternate mode)
        self.event_factory = None  # None: the connector records a CUDA event on the current stream when a slice leaves

    def install(self) -> "LayerWatch":
        self.cache._write_prepared = self
        return self

    def remove(self) -> None:
        if self.cache.__dict__.get("_write_prepared") is self:
            if self.shadowed is None:
                del self.cache.__dict__["_write_prepared"]
            else:
                self.cache._write_prepared = self.shadowed

    def __call__(self, layer, batch, k, v):
        self.write(layer, batch, k, v)
        rows = getattr(batch, "rows", None)
        if not rows or not self.connector.transfers:
            return
        if self.failure is not None:
            return
        began = time.perf_counter()
        try:
            if self.plan_of is not batch:  # one descriptor serves every layer of a traversal: plan once
                self.plan_of, self.plan = batch, self._plan(batch)
            for request_id, plane, start, end in self.plan:
                if self.alternate and self.order.setdefault(request_id, len(self.order)) % 2 == 0:
                    continue  # even-numbered requests (the first is number 0) do not stream
                event = self.event_factory() if self.event_factory is not None else None
                if self.connector.report_layer(request_id, plane, layer, start, end, event=event):
                    self.reported += 1
        except Exception as error:  # noqa: BLE001 - the KV write itself succeeded: the model's forward must go on
            # Streaming is an extra. Whatever went wrong, stop reporting for good and take back what was streamed of
            # the windows that are open, so that each leaves whole at its chunk's end, where the ordinary path runs
            # (and raises, if the cause is still there, in a place that is prepared for it).
            self.failure = f"{type(error).__name__}: {error}"
            for transfer in self.connector.transfers.values():
                transfer.streamed_window, transfer.streamed_layers = None, {}
        self.host_seconds += time.perf_counter() - began

    def _plan(self, batch):
        """``(request id, plane, first token, end token)`` for every (request, depth) of the batch whose rows are one
        gap-free run of tokens. The rows are taken apart with C-speed tools: this runs inside the model's forward."""
        rows = batch.rows
        if len(batch.allocations) == 1:
            # One request: every row is its row. A prefill chunk is laid out as one ascending run of positions at one
            # depth; the two ends, the middle and the count are looked at instead of every row (the scan below costs a
            # fraction of a millisecond per depth, inside a forward that is bound by its host thread).
            (request_id, _), count = batch.allocations[0], len(rows)
            (_, depth, first), (_, mid_depth, middle), (_, last_depth, last) = rows[0], rows[count // 2], rows[-1]
            if depth == mid_depth == last_depth and last - first + 1 == count and middle == first + count // 2:
                return ((request_id, self.cache._plane(depth), first, last + 1),)
            return ()
        import numpy as np

        allocations, depths, positions = zip(*rows)
        names = {id(allocation): request_id for request_id, allocation in batch.allocations}
        count = len(positions)
        owner = np.fromiter(map(id, allocations), np.int64, count)
        depth = np.asarray(depths, dtype=np.int64)
        position = np.asarray(positions, dtype=np.int64)
        plan = []
        if (owner == owner[0]).all() and (depth == depth[0]).all():  # one request at one depth: the usual prefill step
            groups = [(int(owner[0]), int(depth[0]), position)]
        else:
            groups = []
            for who in dict.fromkeys(owner.tolist()):
                mine = owner == who
                for level in dict.fromkeys(depth[mine].tolist()):
                    groups.append((who, level, position[mine & (depth == level)]))
        for who, level, tokens in groups:
            request_id = names.get(who)
            start, end = int(tokens.min()), int(tokens.max()) + 1
            if request_id is not None and end - start == len(tokens) and (np.sort(tokens) == np.arange(start, end)).all():
                plan.append((request_id, self.cache._plane(level), start, end))
        return tuple(plan)
