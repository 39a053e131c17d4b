"""Connector + transport, prefill worker and decode worker in one process, on CPU tensors.

The whole control sequence of a handoff (vllm_rlt/pd/engine.py:197-240 drives it in a deployment):
reserve on D -> prefill on P -> chunks -> commit -> received -> ack -> released, with the messages
relayed by hand the way the coordinator relays them. Destination bytes are compared with the oracle.
"""

from contextlib import nullcontext
from dataclasses import dataclass
from types import SimpleNamespace

import pytest
import torch

from tests.fakes import FakeBackend, FakeEngine, FakeEvent

DIRECTIONS = ["push", "pull"]
from vllm_rlt_b200.core.kv_pool import KVPool
from vllm_rlt_b200.pd.config import PDConfig
from vllm_rlt_b200.pd.connector import PDStageConnector, TableChunk
from vllm_rlt_b200.pd.transport import B200Transport


@pytest.fixture(autouse=True)
def no_cuda(monkeypatch):
    monkeypatch.setattr(torch.cuda, "current_stream", lambda device=None: SimpleNamespace(wait_event=lambda e: None))
    monkeypatch.setattr(torch.cuda, "stream", lambda stream: nullcontext())

    class ReadyEvent(FakeEvent):
        def record(self, stream=None):
            pass

    monkeypatch.setattr(torch.cuda, "Event", ReadyEvent)


class Worker:
    """One stage worker: pool, engine stand-in (or the real ``TransferStage``), transport, connector."""

    def __init__(self, role, config, lane, *, blocks=64, fp8=False, seed=0, device="cpu", direction="push",
                 stage=False, prefix_caching=False, shape=(3, 2, 8), page=4, planes=2, hidden_size=16):
        self.pool = KVPool(*shape, blocks, page, planes, device=device, kv_cache_dtype="fp8_e4m3" if fp8 else "auto",
                           enable_prefix_caching=prefix_caching)
        gen = torch.Generator().manual_seed(seed)
        for t in (self.pool.key_cache, self.pool.value_cache):
            raw = t.view(torch.uint8)
            raw.copy_(torch.randint(0, 256, raw.shape, dtype=torch.uint8, generator=gen) if role == "prefill" else torch.full(raw.shape, 0xA5, dtype=torch.uint8))
        if fp8:
            for t in (self.pool.key_scale, self.pool.value_scale):
                t.copy_(torch.rand(t.shape, generator=gen) if role == "prefill" else torch.full(t.shape, -1.0))
        import random

        random.Random(seed).shuffle(self.pool._free_blocks)
        if stage:
            from vllm_rlt_b200.core.admission import StageSettings, TransferStage

            self.pool.layout, self.pool.attention_info = "last_exited", {"backend": "torch"}
            self.engine = TransferStage(role, self.pool, settings=StageSettings(max_num_seqs=4, prefill_chunk_size=2 * page),
                                        hidden_size=hidden_size)
        else:
            self.engine = FakeEngine(role, self.pool, hidden_size=hidden_size)
        self.messages = []
        hidden = torch.zeros(6, hidden_size, device=device)
        backend = FakeBackend() if device == "cpu" else None
        self.transport = B200Transport(f"{role}-0", self.pool, hidden, config, backend=backend, lane=lane, direction=direction)
        self.connector = PDStageConnector(self.engine, hidden, self.transport, config,
                                          notify=lambda kind, **f: self.messages.append(dict(kind=kind, **f)))

    def take(self, kind):
        hits = [m for m in self.messages if m["kind"] == kind]
        self.messages = [m for m in self.messages if m["kind"] != kind]
        return hits


def make_pair(config=None, **kw):
    config = config or PDConfig()
    p, d = Worker("prefill", config, 0, seed=1, **kw), Worker("decode", config, 1, seed=2, **kw)
    assert p.connector.command(dict(kind="connect", peers=[d.transport.info]))
    assert d.connector.command(dict(kind="connect", peers=[p.transport.info]))
    assert p.take("connected") and d.take("connected")
    return p, d


def pool_rows(pool, tables, start, end):
    out = []
    tensors = [pool.key_cache, pool.value_cache] + ([pool.key_scale, pool.value_scale] if pool.key_scale is not None else [])
    for table in tables:
        for t in range(start, end):
            for x in tensors:
                out.append(x[table[t // 4], :, t % 4].contiguous().view(torch.uint8).reshape(-1))
    return torch.cat(out)


@dataclass
class Params:
    """Stands in for SamplingParams: the connector only narrows ``max_tokens`` on the prefill side."""

    max_tokens: int = 4


def run_handoff(p, d, tid, tokens, *, chunks=((0, None),)):
    """Relay the control messages by hand; returns the source request and the decode side's reservation."""
    prompt = list(range(1, tokens + 1))
    d.connector.command(dict(kind="reserve", tid=tid, tokens=prompt, params=Params(), peer="prefill-0"))
    (reserved,) = d.take("reserved")
    p.connector.command(dict(kind="prefill", tid=tid, tokens=prompt, params=Params(), peer="decode-0",
                             tables=reserved["tables"], slot=reserved["slot"], cached_tokens=reserved["cached_tokens"]))
    assert p.take("prefill_started")
    request = p.engine.scheduler.requests[tid]
    assert p.connector.exports(request)
    done = 0
    for start, end in chunks:
        end = tokens if end is None else end
        request.num_prefilled_tokens = end
        final = end == tokens
        if final:
            request.hidden_state = torch.full((16,), float(len(tid)))
        progress = SimpleNamespace(chunk_complete=True, prompt_complete=final)
        p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=start, progress=progress, event=None, stream=None)
        done = end
        p.connector.progress()
        d.connector.progress()
    p.connector.progress()  # a pulled chunk completes on the source once the reader has said so
    assert done == tokens
    return request, reserved


@pytest.mark.parametrize("direction", DIRECTIONS)
@pytest.mark.parametrize("fp8", [False, True])
def test_full_handoff_sequence_moves_exactly_the_prompt_kv(fp8, direction):
    p, d = make_pair(fp8=fp8, direction=direction)
    before = [t.clone() for t in (d.pool.key_cache, d.pool.value_cache)]
    request, reserved = run_handoff(p, d, "req-1", 10, chunks=((0, 6), (6, None)))
    (commit,) = p.take("commit")
    assert commit["count"] == 2  # two prefill chunks, each under the byte limit: two submissions
    (complete,) = p.take("prefill_complete")
    assert complete["boundaries"] == ((0, 6), (6, 10), 2)
    assert request.compute_released
    # the coordinator relays the commit to D; D has already seen both notifications
    d.connector.command(dict(kind="commit", tid="req-1", count=commit["count"]))
    d.connector.progress()
    assert d.take("received") == [dict(kind="received", tid="req-1")]
    st, dt = p.pool.plane_block_tables("req-1"), reserved["tables"]
    assert torch.equal(pool_rows(p.pool, st, 0, 10), pool_rows(d.pool, dt, 0, 10))
    assert torch.equal(d.engine.imported["req-1"], torch.full((16,), 5.0))
    # nothing outside the request's rows changed on D: rows of other blocks still hold the sentinel
    used = {b for table in dt for b in table}
    for t, old in zip((d.pool.key_cache, d.pool.value_cache), before):
        for block in set(range(d.pool.num_blocks)) - used:
            assert torch.equal(t[block].view(torch.uint8), old[block].view(torch.uint8))
        tail_block = dt[0][2]  # tokens 8..9 live here; offsets 2..3 were never written
        assert (t[tail_block, :, 2:].view(torch.uint8) == 0xA5).all()
    # activation and retirement
    d.engine.admit("req-1")
    d.connector.progress()
    assert d.take("activated")
    p.connector.command(dict(kind="ack", tid="req-1"))
    p.connector.progress()
    assert p.take("released") == [dict(kind="released", tid="req-1", role="prefill")]
    assert p.pool.num_used_blocks == 0 and not p.connector.transfers
    del d.engine.scheduler.requests["req-1"]
    d.connector.output_finished("req-1")
    assert d.take("released")
    assert not d.connector.has_pending
    metrics = p.connector.close()
    assert metrics["transfers"] == 2 and metrics["prefill_tokens"] == 10
    assert metrics["bytes_sent"] == 10 * 2 * 2 * 3 * (2 * 8 * (1 if fp8 else 2) + (2 * 4 if fp8 else 0)) + 16 * 4
    d.connector.close()


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_chunks_respect_the_byte_limit_and_sequence_numbers_are_dense(direction):
    per_token = 2 * 3 * 2 * 8 * 2 * 2  # K,V x layers x heads x dim x bf16 x planes = 384 B
    config = PDConfig(transfer_chunk_bytes=3 * per_token + 10, max_inflight_bytes=1 << 20)
    p, d = make_pair(config, direction=direction)
    run_handoff(p, d, "r", 12)
    (commit,) = p.take("commit")
    assert commit["count"] == 5  # 12 tokens in pieces of 3 -> 4 full KV chunks, and the hidden row alone in a fifth
    d.connector.command(dict(kind="commit", tid="r", count=5))
    d.connector.progress()
    assert d.take("received")
    mover = (d if direction == "pull" else p).transport.backend  # whose device ran the table-driven launches
    kinds = [c[0] if isinstance(c, tuple) else "segments" for c in mover.copies]
    assert kinds.count("tables") == 1  # five tickets and five notifications, but chunks ready together are one launch
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("r"), 0, 12),
                       pool_rows(d.pool, d.pool.plane_block_tables("r"), 0, 12))
    run_handoff(p, d, "s", 11)  # last piece has room for the hidden row: it rides along
    assert p.take("commit")[0]["count"] == 4


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_prefix_already_on_the_decode_side_is_skipped(direction):
    p, d = make_pair(direction=direction)
    prompt = list(range(8))
    d.connector.command(dict(kind="reserve", tid="r", tokens=prompt, params=Params(), peer="prefill-0"))
    (reserved,) = d.take("reserved")
    d.pool._allocations["r"].prefix = 4  # the decode side found the first block in its prefix cache
    p.connector.command(dict(kind="prefill", tid="r", tokens=prompt, params=Params(), peer="decode-0",
                             tables=reserved["tables"], slot=reserved["slot"], cached_tokens=4))
    request = p.engine.scheduler.requests["r"]
    request.num_prefilled_tokens, request.hidden_state = 8, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    chunk = p.connector.transfers["r"].chunks[0]
    assert isinstance(chunk, TableChunk) and (chunk.start, chunk.end) == (4, 8)
    p.connector.progress()
    assert p.take("prefill_complete")[0]["boundaries"] == ((4, 8), (4, 8), 1)
    d.connector.transfers["r"].cached_tokens = 4
    d.connector.command(dict(kind="commit", tid="r", count=p.take("commit")[0]["count"]))
    d.connector.progress()
    d.connector.progress()
    assert d.take("received")
    dt = reserved["tables"]
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("r"), 4, 8), pool_rows(d.pool, dt, 4, 8))
    assert (d.pool.key_cache[dt[0][0]].view(torch.uint8) == 0xA5).all()  # the cached block was not rewritten


def test_backpressure_and_cancellation_keep_resources_until_safe():
    config = PDConfig(transfer_chunk_bytes=400, max_inflight_bytes=400)
    p, d = make_pair(config)
    p.transport.backend.complete_immediately = False
    request, _ = run_handoff(p, d, "r", 6)
    t = p.connector.transfers["r"]
    assert p.transport.inflight_bytes > 0 and t.chunks  # one chunk on the wire, the rest waits for budget
    assert not p.connector.can_schedule(request)
    p.connector.command(dict(kind="cancel", tid="r"))
    assert not t.chunks and p.engine.suspended == ["r"]
    p.connector.progress()
    assert "r" in p.connector.transfers  # still on the wire: the slot and the KV stay
    for ev in p.transport.backend.events:
        ev.done = True
    p.connector.progress()
    assert p.take("released") and p.pool.num_used_blocks == 0
    # the decode side drops the import only after the coordinator confirms the writer stopped
    d.connector.command(dict(kind="cancel", tid="r"))
    d.connector.progress()
    assert "r" in d.connector.transfers
    p.connector.cancel_safe("missing")  # unknown generations are ignored
    d.connector.transfers["r"].cancelled = False
    with pytest.raises(RuntimeError, match="unexpected cancellation acknowledgement"):
        d.connector.cancel_safe("r")
    d.connector.transfers["r"].cancelled = True
    d.connector.command(dict(kind="cancel_safe", tid="r"))
    assert d.take("released") and d.pool.num_used_blocks == 0


def test_rejection_when_the_decode_pool_is_full_and_protocol_errors():
    p, d = make_pair(blocks=8)
    d.connector.command(dict(kind="reserve", tid="ok", tokens=list(range(12)), params=Params(), peer="prefill-0"))
    assert d.take("reserved")
    d.connector.command(dict(kind="reserve", tid="big", tokens=list(range(8)), params=Params(), peer="prefill-0"))
    assert d.take("rejected") == [dict(kind="rejected", tid="big", role="decode")]
    assert "big" not in d.connector.transfers and len(d.connector.free_slots) == 5
    with pytest.raises(RuntimeError, match="duplicate transfer generation"):
        d.connector.reserve("ok", [1], Params(), receiving=True, peer="prefill-0")
    with pytest.raises(RuntimeError, match="invalid transfer commit"):
        d.connector.commit("ok", 0)
    with pytest.raises(RuntimeError, match="acknowledgement requires an outgoing transfer"):
        d.connector.acknowledge("ok")
    with pytest.raises(ValueError, match="cancellation protocol"):
        d.connector.command(dict(kind="abort", request_id="ok"))
    assert d.connector.command(dict(kind="stats")) is False
    with pytest.raises(RuntimeError, match="pending transfers"):
        d.connector.close()


# ----------------------------------------------------------------------------- layer streaming, small chunks, real admission


def handoff_ready(p, d, tid, tokens):
    prompt = list(range(1, tokens + 1))
    d.connector.command(dict(kind="reserve", tid=tid, tokens=prompt, params=Params(), peer="prefill-0"))
    (reserved,) = d.take("reserved")
    p.connector.command(dict(kind="prefill", tid=tid, tokens=prompt, params=Params(), peer="decode-0",
                             tables=reserved["tables"], slot=reserved["slot"], cached_tokens=reserved["cached_tokens"]))
    assert p.take("prefill_started")
    return p.engine.scheduler.requests[tid], reserved


def settle(p, d, rounds=3):
    for _ in range(rounds):
        p.connector.progress()
        d.connector.progress()


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_layers_reported_one_by_one_leave_early_and_the_tail_is_one_slice(direction):
    """A producer that reports each (plane, layer) as written gets slices out before the step ends: after the last
    layer only that layer's slice is left to move, ``prefill_submitted`` adds nothing but the hidden row, and the
    destination is complete."""
    p, d = make_pair(direction=direction)
    request, reserved = handoff_ready(p, d, "s", 10)
    p.connector.stream_layers = 2
    t = p.connector.transfers["s"]
    sent_before_step_end = 0
    for plane in range(2):
        for layer in range(3):
            went = p.connector.layer_written(request, plane=plane, layer=layer, event=FakeEvent(), start=0, end=10)
            assert went == (layer >= 1)  # groups of two layers: 0-1 leave together; the last layer never waits
            sent_before_step_end += went
    assert sent_before_step_end == 4 and t.next_sequence == 4 and t.streamed_layers == {0: 3, 1: 3}
    request.num_prefilled_tokens, request.hidden_state = 10, torch.full((16,), 3.0)
    p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    (commit,) = p.take("commit")
    assert commit["count"] == 5  # four slices left while the step ran; its end only adds the hidden row
    assert p.take("prefill_complete")[0]["boundaries"] == ((0, 10), (0, 10), 1)
    d.connector.command(dict(kind="commit", tid="s", count=5))
    settle(p, d)
    assert d.take("received")
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("s"), 0, 10), pool_rows(d.pool, reserved["tables"], 0, 10))
    assert torch.equal(d.engine.imported["s"], torch.full((16,), 3.0))
    with pytest.raises(ValueError, match="increasing order"):
        request.num_prefilled_tokens = 0
        p.connector.layer_written(request, plane=0, layer=1, event=FakeEvent(), start=0, end=10)
        p.connector.layer_written(request, plane=0, layer=0, event=FakeEvent(), start=0, end=10)


def cache_that_writes(pool, depths=2):
    """Gives a pool the three things the layer watch looks at on a cache manager: how many depths there are, which
    plane a depth is stored in, and the prepared write every traversal goes through (here it only counts calls)."""
    pool.max_loops, pool._plane, pool.writes = depths, (lambda depth: depth), []
    pool._write_prepared = lambda layer, batch, k, v: pool.writes.append(layer)
    return pool


def traversal(pool, request_id, depth, start, end, layers=3):
    """One depth of a prefill step as the model drives it: one prepared batch, every layer written through it."""
    allocation = object()
    batch = SimpleNamespace(rows=tuple((allocation, depth, t) for t in range(start, end)), allocations=((request_id, allocation),))
    for layer in range(layers):
        pool._write_prepared(layer, batch, None, None)


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_a_watched_cache_reports_its_own_writes_and_the_step_end_sends_only_the_rest(direction):
    from vllm_rlt_b200.pd import layer_watch

    p, d = make_pair(direction=direction)
    cache_that_writes(p.pool)
    assert layer_watch.eligible(p.connector)
    watch = layer_watch.LayerWatch(p.connector).install()
    watch.event_factory = FakeEvent
    p.connector.stream_layers = 2
    request, reserved = handoff_ready(p, d, "s", 10)
    traversal(p.pool, "s", 0, 0, 10)
    traversal(p.pool, "s", 1, 0, 10)
    traversal(p.pool, "stranger", 0, 0, 4)  # not an export: written, not reported
    assert p.pool.writes == [0, 1, 2] * 3 and watch.reported == 4
    assert p.connector.transfers["s"].streamed_layers == {0: 3, 1: 3}
    request.num_prefilled_tokens, request.hidden_state = 10, torch.full((16,), 3.0)
    p.connector.prefill_submitted(request, phase="PREFILL", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    (commit,) = p.take("commit")
    assert commit["count"] == 5  # four slices while the step ran, the hidden row at its end
    d.connector.command(dict(kind="commit", tid="s", count=5))
    settle(p, d)
    assert d.take("received")
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("s"), 0, 10), pool_rows(d.pool, reserved["tables"], 0, 10))
    watch.remove()
    assert "_write_prepared" in p.pool.__dict__ and p.pool._write_prepared is not watch  # the stand-in of this test is back


def test_planes_can_leave_whole_and_the_last_in_two_pieces_so_that_a_step_costs_few_launches():
    from vllm_rlt_b200.pd import layer_watch

    p, d = make_pair()
    cache_that_writes(p.pool)
    watch = layer_watch.LayerWatch(p.connector).install()
    watch.event_factory = FakeEvent
    p.connector.stream_layers, p.connector.stream_whole_planes = 1, True
    request, reserved = handoff_ready(p, d, "s", 10)
    traversal(p.pool, "s", 0, 0, 10)
    assert watch.reported == 1  # plane 0 in one piece, after its last layer
    traversal(p.pool, "s", 1, 0, 10)
    assert watch.reported == 3  # the last plane in two pieces: layers 0-1, then the last layer
    request.num_prefilled_tokens, request.hidden_state = 10, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILL", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    (commit,) = p.take("commit")
    d.connector.command(dict(kind="commit", tid="s", count=commit["count"]))
    settle(p, d)
    assert commit["count"] == 4 and d.take("received")  # three early slices and the hidden row
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("s"), 0, 10), pool_rows(d.pool, reserved["tables"], 0, 10))


def test_a_plane_written_twice_in_one_window_withdraws_the_window_and_the_step_end_sends_all_of_it():
    from vllm_rlt_b200.pd import layer_watch

    p, d = make_pair()
    cache_that_writes(p.pool)
    watch = layer_watch.LayerWatch(p.connector).install()
    watch.event_factory = FakeEvent
    p.connector.stream_layers = 2
    request, reserved = handoff_ready(p, d, "s", 6)
    traversal(p.pool, "s", 0, 0, 6)
    assert watch.reported == 2
    traversal(p.pool, "s", 0, 0, 6)  # the same plane again: what left may be stale
    t = p.connector.transfers["s"]
    assert watch.reported == 2 and t.streamed_window is None and t.stream_refused == (0, 6)
    request.num_prefilled_tokens, request.hidden_state = 6, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILL", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    (commit,) = p.take("commit")
    assert commit["count"] == 3  # the two early slices and the whole window again, which carries the hidden row
    d.connector.command(dict(kind="commit", tid="s", count=3))
    settle(p, d)
    assert d.take("received")
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("s"), 0, 6), pool_rows(d.pool, reserved["tables"], 0, 6))


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_a_step_that_streams_more_than_the_budget_holds_gets_its_tickets_back_inside_the_step(direction):
    """One plane of this request is 1,920 bytes and the budget 2,000: without returning tickets inside the step the
    second plane would wait for the next progress(); the watch's report polls when half the budget is taken."""
    from vllm_rlt_b200.pd import layer_watch

    config = PDConfig(transfer_chunk_bytes=1000, max_inflight_bytes=2000)
    p, d = make_pair(config, direction=direction)
    p.transport.device_ordered = True  # as on a device: submissions leave when they are reported, not at the next progress()
    cache_that_writes(p.pool)
    watch = layer_watch.LayerWatch(p.connector).install()
    watch.event_factory = FakeEvent
    p.connector.stream_layers, p.connector.stream_whole_planes = 1, True
    request, reserved = handoff_ready(p, d, "s", 10)
    t = p.connector.transfers["s"]
    traversal(p.pool, "s", 0, 0, 10)
    assert watch.reported == 1 and not t.chunks  # plane 0 is on its way
    if direction == "pull":
        d.connector.progress()  # the decode worker reads the offered chunk and says so
    traversal(p.pool, "s", 1, 0, 10)
    assert watch.reported == 3 and not t.chunks  # both pieces of plane 1 left during the step: nothing is queued
    request.num_prefilled_tokens, request.hidden_state = 10, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILL", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    (commit,) = p.take("commit")
    d.connector.command(dict(kind="commit", tid="s", count=commit["count"]))
    settle(p, d)
    assert d.take("received")
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("s"), 0, 10), pool_rows(d.pool, reserved["tables"], 0, 10))


def test_an_error_inside_the_watch_stops_streaming_and_never_reaches_the_forward():
    from vllm_rlt_b200.pd import layer_watch

    p, d = make_pair()
    cache_that_writes(p.pool)
    watch = layer_watch.LayerWatch(p.connector).install()
    watch.event_factory = FakeEvent
    p.connector.stream_layers = 2
    request, reserved = handoff_ready(p, d, "s", 10)
    traversal(p.pool, "s", 0, 0, 10)
    assert watch.reported == 2
    original = p.connector.report_layer
    p.connector.report_layer = lambda *a, **k: (_ for _ in ()).throw(RuntimeError("boom"))
    traversal(p.pool, "s", 1, 0, 10)  # the writes still happen, nothing is raised
    p.connector.report_layer = original
    assert watch.failure == "RuntimeError: boom" and p.pool.writes == [0, 1, 2] * 2
    assert p.connector.transfers["s"].streamed_window is None
    traversal(p.pool, "s", 1, 0, 10)
    assert watch.reported == 2  # it stays off
    request.num_prefilled_tokens, request.hidden_state = 10, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILL", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    (commit,) = p.take("commit")
    d.connector.command(dict(kind="commit", tid="s", count=commit["count"]))
    settle(p, d)
    assert d.take("received")
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("s"), 0, 10), pool_rows(d.pool, reserved["tables"], 0, 10))


def test_the_watch_reads_requests_planes_and_token_runs_off_a_batch():
    from vllm_rlt_b200.pd.layer_watch import LayerWatch

    watch = LayerWatch.__new__(LayerWatch)
    watch.cache = SimpleNamespace(_plane=lambda depth: depth)
    a, b = object(), object()
    one = SimpleNamespace(rows=tuple((a, 2, t) for t in range(40, 140)), allocations=(("s", a),))
    assert watch._plan(one) == (("s", 2, 40, 140),)
    gap = SimpleNamespace(rows=tuple((a, 2, t) for t in (*range(40, 90), *range(91, 141))), allocations=(("s", a),))
    assert watch._plan(gap) == ()  # not one run of tokens: nothing is reported, the chunk leaves at its end
    mixed = SimpleNamespace(rows=tuple((a, 1 + (t > 100), t) for t in range(40, 140)), allocations=(("s", a),))
    assert watch._plan(mixed) == ()  # two depths in one batch of one request
    two = SimpleNamespace(rows=tuple((a, 1, t) for t in range(100, 1100)) + tuple((b, 0, t) for t in range(0, 1000))
                          + tuple((b, 1, t) for t in (5, 7)), allocations=(("s", a), ("q", b)))
    assert sorted(watch._plan(two)) == [("q", 0, 0, 1000), ("s", 1, 100, 1100)]  # q's two stray rows at depth 1 are no run


def test_the_watch_is_refused_where_depths_share_a_plane_or_prefill_is_wavefront_chunked(monkeypatch):
    from vllm_rlt_b200.pd import layer_watch

    p, _ = make_pair()
    cache_that_writes(p.pool)
    assert layer_watch.eligible(p.connector)
    p.pool._plane = lambda depth: 0  # every depth stored in one plane: rows are rewritten within a step
    assert not layer_watch.eligible(p.connector)
    p.pool._plane = lambda depth: depth
    p.engine.scheduler.config.wavefront_chunked_prefill = True
    assert not layer_watch.eligible(p.connector)
    monkeypatch.setenv("RLT_KV_STREAM", "1")
    assert layer_watch.wanted()
    monkeypatch.setenv("RLT_KV_STREAM", "0")
    assert not layer_watch.wanted()


def test_nobody_calling_the_layer_hook_changes_nothing_and_a_non_exporting_request_is_ignored():
    p, d = make_pair()
    request, reserved = handoff_ready(p, d, "q", 6)
    stranger = SimpleNamespace(request_id="other")
    assert p.connector.layer_written(stranger, plane=0, layer=0) is False
    assert d.connector.layer_written(d.engine.scheduler.requests["q"], plane=0, layer=0) is False  # imports do not stream
    request.num_prefilled_tokens, request.hidden_state = 6, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    assert p.take("commit")[0]["count"] == 1


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_a_chunk_limit_below_one_token_splits_by_plane_and_layer_instead_of_failing(direction):
    """One token over all planes and layers is 384 B here; with a 200-byte limit the reference's planner would cut
    inside the token, so must this one: by plane, then by layer group."""
    config = PDConfig(transfer_chunk_bytes=200, max_inflight_bytes=1 << 20)
    p, d = make_pair(config, direction=direction)
    request, reserved = handoff_ready(p, d, "w", 5)
    request.num_prefilled_tokens, request.hidden_state = 5, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d, rounds=6)
    (commit,) = p.take("commit")
    # per plane: 3 layers x 64 B -> layer groups of 3 (192 B <= 200), one token each: 2 planes x 5 tokens, + the hidden row
    assert commit["count"] == 2 * 5 + 1
    d.connector.command(dict(kind="commit", tid="w", count=commit["count"]))
    settle(p, d)
    assert d.take("received")
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("w"), 0, 5), pool_rows(d.pool, reserved["tables"], 0, 5))
    too_small = PDConfig(transfer_chunk_bytes=60, max_inflight_bytes=1 << 20)
    p2, d2 = make_pair(too_small, direction=direction)
    request, _ = handoff_ready(p2, d2, "x", 2)
    request.num_prefilled_tokens = 2
    with pytest.raises(ValueError, match="smaller than one token row"):
        p2.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                       progress=SimpleNamespace(chunk_complete=True, prompt_complete=False), event=None, stream=None)


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_decode_side_prefix_hit_travels_with_the_reservation_and_is_skipped_by_the_source(direction):
    """The real admission hook on both sides: D imported a prompt earlier and cached its pages; a second prompt that
    shares two pages is reserved with cached_tokens = 8, the source skips those tokens, bytes_sent drops by the prefix
    and the shared blocks keep their bytes."""
    config = PDConfig()
    p = Worker("prefill", config, 0, seed=1, direction=direction, stage=True)
    d = Worker("decode", config, 1, seed=2, direction=direction, stage=True, prefix_caching=True)
    # a fresh pool hands out ascending block ids, which makes the shared blocks easy to recognise below
    for w in (p, d):
        w.pool._free_blocks.sort(reverse=True)
    assert p.connector.command(dict(kind="connect", peers=[d.transport.info]))
    assert d.connector.command(dict(kind="connect", peers=[p.transport.info]))

    def run(tid, prompt):
        d.connector.command(dict(kind="reserve", tid=tid, tokens=prompt, params=Params(), peer="prefill-0"))
        (reserved,) = d.take("reserved")
        p.connector.command(dict(kind="prefill", tid=tid, tokens=prompt, params=Params(), peer="decode-0",
                                 tables=reserved["tables"], slot=reserved["slot"], cached_tokens=reserved["cached_tokens"]))
        request = p.engine.requests[tid]
        p.engine.begin_prefill(request)
        p.engine.end_prefill(request, torch.full((16,), 2.0))
        p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                      progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
        settle(p, d)
        (commit,) = p.take("commit")
        d.connector.command(dict(kind="commit", tid=tid, count=commit["count"]))
        settle(p, d)
        assert d.take("received")
        p.connector.command(dict(kind="ack", tid=tid))
        settle(p, d)
        assert p.take("released")
        return reserved

    first = run("one", list(range(1, 14)))   # 13 tokens: pages 0-2 become cached on D (the last token's page is not)
    assert first["cached_tokens"] == 0
    sent_first = p.transport.bytes_sent
    shared = [bytes(d.pool.key_cache[b].view(torch.uint8).reshape(-1).tolist()) for b in first["tables"][0][:2]]
    second = run("two", list(range(1, 9)) + [40, 41, 42, 43, 44])  # shares two pages (8 tokens) with the first
    assert second["cached_tokens"] == 8
    assert [list(t[:2]) for t in second["tables"]] == [list(t[:2]) for t in first["tables"]]  # the same physical blocks
    per_token = 2 * 3 * 2 * 8 * 2 * 2
    assert sent_first == 13 * per_token + 64 and p.transport.bytes_sent - sent_first == (13 - 8) * per_token + 64
    assert shared == [bytes(d.pool.key_cache[b].view(torch.uint8).reshape(-1).tolist()) for b in second["tables"][0][:2]]
    src = p.pool  # the source freed its blocks on release; compare what D holds for tokens 8.. with a fresh gather instead
    assert d.engine.requests["two"].num_prefilled_tokens == 13 and d.pool._allocations["two"].imported == 13


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_what_the_layer_hook_did_not_reach_leaves_at_the_end_of_the_step(direction):
    p, d = make_pair(direction=direction)
    request, reserved = handoff_ready(p, d, "h", 7)
    p.connector.stream_layers = 2
    assert not p.connector.layer_written(request, plane=0, layer=0, event=FakeEvent(), start=0, end=7)
    assert p.connector.layer_written(request, plane=0, layer=1, event=FakeEvent(), start=0, end=7)  # plane 0, layers 0-1
    request.num_prefilled_tokens, request.hidden_state = 7, torch.ones(16)
    p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=None, stream=None)
    settle(p, d)
    (commit,) = p.take("commit")
    assert commit["count"] == 3  # the early slice, plane 0's last layer, the whole of plane 1 (+ the hidden row on it)
    d.connector.command(dict(kind="commit", tid="h", count=3))
    settle(p, d)
    assert d.take("received")
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("h"), 0, 7), pool_rows(d.pool, reserved["tables"], 0, 7))
