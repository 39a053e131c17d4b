"""The connector driving the real transport and kernels: a prefill and a decode worker on one GPU.

Same hand-relayed control sequence as tests/test_connector_cpu.py, but every chunk is a real
``rlt_kv_handoff`` launch, the hidden row a real segment copy, and every notification is written by the
GPU into the decode worker's mailbox.
"""

import time
from types import SimpleNamespace

import pytest
import torch

from tests.test_connector_cpu import DIRECTIONS, Params, Worker, pool_rows

pytestmark = pytest.mark.gpu


def pump(p, d, until, limit=20.0):
    deadline = time.monotonic() + limit
    while not until() and time.monotonic() < deadline:
        p.connector.progress()
        d.connector.progress()
    assert until()


@pytest.mark.parametrize("direction", DIRECTIONS)
@pytest.mark.parametrize("fp8", [False, True])
def test_handoff_through_connector_transport_and_kernels(fp8, direction):
    from vllm_rlt_b200.pd.config import PDConfig

    per_token = 2 * 3 * (2 * 8 * (1 if fp8 else 2) + (2 * 4 if fp8 else 0)) * 2
    config = PDConfig(transfer_chunk_bytes=5 * per_token + 100, max_inflight_bytes=16 * per_token)
    p = Worker("prefill", config, 0, seed=1, fp8=fp8, device="cuda:0", direction=direction)
    d = Worker("decode", config, 1, seed=2, fp8=fp8, device="cuda:0", direction=direction)
    p.connector.command(dict(kind="connect", peers=[d.transport.info]))
    d.connector.command(dict(kind="connect", peers=[p.transport.info]))
    tokens = 23
    prompt = list(range(tokens))
    d.connector.command(dict(kind="reserve", tid="req", tokens=prompt, params=Params(), peer="prefill-0"))
    (reserved,) = d.take("reserved")
    p.connector.command(dict(kind="prefill", tid="req", tokens=prompt, params=Params(), peer="decode-0",
                             tables=reserved["tables"], slot=reserved["slot"], cached_tokens=0))
    request = p.engine.scheduler.requests["req"]
    sentinel_before = d.pool.key_cache.clone()
    for start, end in ((0, 9), (9, 16), (16, tokens)):
        request.num_prefilled_tokens = end
        final = end == tokens
        if final:
            request.hidden_state = torch.full((16,), 3.0, device="cuda:0")
        event = torch.cuda.Event()
        event.record()
        p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=start,
                                      progress=SimpleNamespace(chunk_complete=True, prompt_complete=final),
                                      event=event, stream=None)
        p.connector.progress()
    pump(p, d, lambda: bool([m for m in p.messages if m["kind"] == "commit"]))
    (commit,) = p.take("commit")
    assert commit["count"] == 6  # 9, 7 and 7 tokens in pieces of at most 5: 2 + 2 + 2 submissions
    d.connector.command(dict(kind="commit", tid="req", count=commit["count"]))
    pump(p, d, lambda: bool([m for m in d.messages if m["kind"] == "received"]))
    torch.cuda.synchronize()
    st, dt = p.pool.plane_block_tables("req"), reserved["tables"]
    assert torch.equal(pool_rows(p.pool, st, 0, tokens).cpu(), pool_rows(d.pool, dt, 0, tokens).cpu())
    assert torch.equal(d.engine.imported["req"].cpu(), torch.full((16,), 3.0))
    used = {b for table in dt for b in table}
    for block in set(range(d.pool.num_blocks)) - used:
        assert torch.equal(d.pool.key_cache[block].view(torch.uint8), sentinel_before[block].view(torch.uint8))
    assert (d.pool.key_cache[dt[0][5], :, 3:].view(torch.uint8) == 0xA5).all()  # token 23 of block 5 never written
    d.engine.admit("req")
    p.connector.command(dict(kind="ack", tid="req"))
    pump(p, d, lambda: not p.connector.transfers and bool([m for m in d.messages if m["kind"] == "activated"]))
    assert p.pool.num_used_blocks == 0
    del d.engine.scheduler.requests["req"]
    d.connector.output_finished("req")
    metrics = p.connector.close()
    assert metrics["transfers"] == 6 and metrics["bytes_sent"] == tokens * per_token + 16 * 4
    d.connector.close()


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_chunks_leave_behind_the_producer_event_without_another_progress_pass(direction):
    """The reference submits a chunk only when a later ``progress()`` pass finds its event fired (the commit tail,
    vllm_rlt/pd/config.py:10-15). Here the copies are queued at once behind the event on the device: the decode
    side receives every notification although the prefill worker's host never runs ``progress()`` again."""
    from vllm_rlt_b200.pd.config import PDConfig

    per_token = 2 * 3 * (2 * 8 * 2) * 2
    config = PDConfig(transfer_chunk_bytes=6 * per_token, max_inflight_bytes=64 * per_token)
    p = Worker("prefill", config, 0, seed=1, device="cuda:0", direction=direction)
    d = Worker("decode", config, 1, seed=2, device="cuda:0", direction=direction)
    p.connector.command(dict(kind="connect", peers=[d.transport.info]))
    d.connector.command(dict(kind="connect", peers=[p.transport.info]))
    tokens = 20
    d.connector.command(dict(kind="reserve", tid="req", tokens=list(range(tokens)), params=Params(), peer="prefill-0"))
    (reserved,) = d.take("reserved")
    p.connector.command(dict(kind="prefill", tid="req", tokens=list(range(tokens)), params=Params(), peer="decode-0",
                             tables=reserved["tables"], slot=reserved["slot"], cached_tokens=0))
    request = p.engine.scheduler.requests["req"]
    request.num_prefilled_tokens = tokens
    request.hidden_state = torch.ones(16, device="cuda:0")
    compute = torch.cuda.Stream()
    with torch.cuda.stream(compute):
        torch.cuda._sleep(int(0.15 * 1.9e9))  # the "prefill" is still running for ~150 ms
        event = torch.cuda.Event()
        event.record(compute)
    p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True),
                                  event=event, stream=compute)
    transfer = p.connector.transfers["req"]
    assert not transfer.chunks and transfer.next_sequence == 4  # 20 tokens in pieces of 6, all queued already
    assert not event.query()  # ... while the producer has not finished
    incoming = d.connector.transfers["req"]
    deadline = time.monotonic() + 20
    while len(incoming.received) < 4 and time.monotonic() < deadline:
        d.connector.progress()  # only the decode side's host runs
    assert incoming.received == {0, 1, 2, 3} and event.query()
    torch.cuda.synchronize()
    assert torch.equal(pool_rows(p.pool, p.pool.plane_block_tables("req"), 0, tokens).cpu(),
                       pool_rows(d.pool, reserved["tables"], 0, tokens).cpu())
    # the control messages still follow the protocol once the prefill host runs again
    p.connector.progress()
    assert p.take("commit") == [dict(kind="commit", tid="req", count=4)]
    d.connector.command(dict(kind="commit", tid="req", count=4))
    d.connector.progress()
    assert d.take("received")
    d.engine.admit("req")
    p.connector.command(dict(kind="ack", tid="req"))
    pump(p, d, lambda: not p.connector.transfers)
    del d.engine.scheduler.requests["req"]
    d.connector.output_finished("req")
    p.connector.close()
    d.connector.close()


def oracle_of(worker, base):
    """An ``OraclePool`` holding the same bytes and block tables as a worker's device pool."""
    from oracle import handoff_oracle as ho

    pool = worker.pool
    o = ho.OraclePool(pool.num_layers, pool.num_kv_heads, pool.head_dim, pool.num_blocks, pool.block_size, pool.storage_depths,
                      element=2, base=base)
    o.key.data[...] = pool.key_cache.view(torch.uint8).cpu().numpy().reshape(o.key.data.shape)
    o.value.data[...] = pool.value_cache.view(torch.uint8).cpu().numpy().reshape(o.value.data.shape)
    return o


def device_bytes(pool):
    return [t.contiguous().view(torch.uint8).reshape(-1).cpu().numpy() for t in (pool.key_cache, pool.value_cache)]


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_layers_reported_by_the_producer_stream_through_the_connector_and_the_tail_is_one_slice(direction):
    """A stand-in model runner reports every (plane, layer) as it "writes" it (a timed sleep per layer on the compute
    stream). Slices leave behind each report's event while later layers still run; when the last layer's report is in,
    one slice per plane is all that is left, and the destination pool equals the oracle's byte for byte."""
    import numpy as np

    from oracle import handoff_oracle as ho
    from vllm_rlt_b200.pd.config import PDConfig

    config = PDConfig()
    shape = dict(shape=(8, 4, 64), page=16, planes=2, blocks=48)
    p = Worker("prefill", config, 0, seed=1, device="cuda:0", direction=direction, **shape)
    d = Worker("decode", config, 1, seed=2, device="cuda:0", direction=direction, **shape)
    p.connector.command(dict(kind="connect", peers=[d.transport.info]))
    d.connector.command(dict(kind="connect", peers=[p.transport.info]))
    tokens = 70
    d.connector.command(dict(kind="reserve", tid="req", tokens=list(range(tokens)), params=Params(), peer="prefill-0"))
    (reserved,) = d.take("reserved")
    p.connector.command(dict(kind="prefill", tid="req", tokens=list(range(tokens)), params=Params(), peer="decode-0",
                             tables=reserved["tables"], slot=reserved["slot"], cached_tokens=0))
    request = p.engine.scheduler.requests["req"]
    P, D = oracle_of(p, 1 << 30), oracle_of(d, 1 << 40)
    ho.handoff_rows(P, D, p.pool.plane_block_tables("req"), reserved["tables"], 0, tokens)
    p.connector.stream_layers = 3
    compute = torch.cuda.Stream()
    transfer = p.connector.transfers["req"]
    launched = []
    with torch.cuda.stream(compute):
        for plane in range(2):
            for layer in range(8):
                torch.cuda._sleep(int(0.004 * 1.9e9))  # one layer of "prefill" at this depth
                event = torch.cuda.Event()
                event.record(compute)
                launched.append(p.connector.layer_written(request, plane=plane, layer=layer, event=event, start=0, end=tokens))
        end_of_compute = torch.cuda.Event()
        end_of_compute.record(compute)
    # layers 0-2, 3-5 and the last group 6-7 of either plane: six slices, the last of them queued with the last layer
    assert launched == [False, False, True, False, False, True, False, True] * 2 and transfer.next_sequence == 6
    assert not transfer.chunks  # each slice was handed to the transport at once, behind its event
    request.num_prefilled_tokens, request.hidden_state = tokens, torch.full((16,), 2.0, device="cuda:0")
    p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True),
                                  event=end_of_compute, stream=compute)
    assert transfer.next_sequence == 7  # nothing of the KV was left for the end of the step: only the hidden row
    pump(p, d, lambda: bool([m for m in p.messages if m["kind"] == "commit"]))
    assert p.take("commit") == [dict(kind="commit", tid="req", count=7)]
    d.connector.command(dict(kind="commit", tid="req", count=7))
    pump(p, d, lambda: bool([m for m in d.messages if m["kind"] == "received"]))
    torch.cuda.synchronize()
    for got, want in zip(device_bytes(d.pool), (D.key.data.reshape(-1), D.value.data.reshape(-1))):
        assert np.array_equal(got, want)
    assert torch.equal(d.engine.imported["req"].cpu(), torch.full((16,), 2.0))
    d.engine.admit("req")
    p.connector.command(dict(kind="ack", tid="req"))
    pump(p, d, lambda: not p.connector.transfers)
    del d.engine.scheduler.requests["req"]
    d.connector.output_finished("req")
    per_token = 2 * 8 * 4 * 64 * 2 * 2
    assert p.connector.close()["bytes_sent"] == tokens * per_token + 16 * 4
    d.connector.close()


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_a_watched_cache_streams_rows_that_are_only_written_while_the_step_runs(direction):
    """The layer watch on a real device. The source pool starts EMPTY (zeros); a stand-in for the cache manager's
    prepared write copies each layer's rows into it on the compute stream, behind a sleep, and the watch reports the
    write from inside that call with an event it records itself. A slice that did not wait for its event would carry
    zeros: the destination must equal the oracle's handoff of the complete source, byte for byte."""
    import numpy as np

    from oracle import handoff_oracle as ho
    from vllm_rlt_b200.pd import layer_watch
    from vllm_rlt_b200.pd.config import PDConfig

    shape = dict(shape=(8, 4, 64), page=16, planes=2, blocks=48)
    p = Worker("prefill", PDConfig(), 0, seed=1, device="cuda:0", direction=direction, **shape)
    d = Worker("decode", PDConfig(), 1, seed=2, device="cuda:0", direction=direction, **shape)
    p.connector.command(dict(kind="connect", peers=[d.transport.info]))
    d.connector.command(dict(kind="connect", peers=[p.transport.info]))
    tokens = 70
    d.connector.command(dict(kind="reserve", tid="req", tokens=list(range(tokens)), params=Params(), peer="prefill-0"))
    (reserved,) = d.take("reserved")
    p.connector.command(dict(kind="prefill", tid="req", tokens=list(range(tokens)), params=Params(), peer="decode-0",
                             tables=reserved["tables"], slot=reserved["slot"], cached_tokens=0))
    request = p.engine.scheduler.requests["req"]
    P, D = oracle_of(p, 1 << 30), oracle_of(d, 1 << 40)
    tables = p.pool.plane_block_tables("req")
    ho.handoff_rows(P, D, tables, reserved["tables"], 0, tokens)
    full = [p.pool.key_cache.clone(), p.pool.value_cache.clone()]
    for t in (p.pool.key_cache, p.pool.value_cache):
        t.zero_()
    positions = torch.arange(tokens, device="cuda:0")

    def write_prepared(layer, batch, k, v):  # what a model's attention layer does: this layer's rows of this depth
        plane = batch.rows[0][1]
        blocks = torch.tensor(tables[plane], device="cuda:0")[positions // 16]
        torch.cuda._sleep(int(0.003 * 1.9e9))
        for cache, source in zip((p.pool.key_cache, p.pool.value_cache), full):
            cache[blocks, layer, positions % 16] = source[blocks, layer, positions % 16]

    p.pool.max_loops, p.pool._plane, p.pool._write_prepared = 2, (lambda depth: depth), write_prepared
    assert layer_watch.eligible(p.connector)
    watch = layer_watch.LayerWatch(p.connector).install()
    p.connector.stream_layers, p.connector.stream_whole_planes = 2, True
    compute = torch.cuda.Stream()
    allocation = object()
    with torch.cuda.stream(compute):
        for depth in range(2):
            batch = SimpleNamespace(rows=tuple((allocation, depth, t) for t in range(tokens)), allocations=(("req", allocation),))
            for layer in range(8):
                p.pool._write_prepared(layer, batch, None, None)
        end_of_compute = torch.cuda.Event()
        end_of_compute.record(compute)
    transfer = p.connector.transfers["req"]
    assert watch.reported == 3 and not transfer.chunks  # plane 0 whole, plane 1 in two pieces, each behind its own event
    request.num_prefilled_tokens, request.hidden_state = tokens, torch.full((16,), 2.0, device="cuda:0")
    p.connector.prefill_submitted(request, phase="PREFILL", start=0,
                                  progress=SimpleNamespace(chunk_complete=True, prompt_complete=True),
                                  event=end_of_compute, stream=compute)
    pump(p, d, lambda: bool([m for m in p.messages if m["kind"] == "commit"]))
    (commit,) = p.take("commit")
    assert commit["count"] == 4  # the three slices and the hidden row
    d.connector.command(dict(kind="commit", tid="req", count=4))
    pump(p, d, lambda: bool([m for m in d.messages if m["kind"] == "received"]))
    torch.cuda.synchronize()
    for got, want in zip(device_bytes(d.pool), (D.key.data.reshape(-1), D.value.data.reshape(-1))):
        assert np.array_equal(got, want)
    d.engine.admit("req")
    p.connector.command(dict(kind="ack", tid="req"))
    pump(p, d, lambda: not p.connector.transfers)
    del d.engine.scheduler.requests["req"]
    d.connector.output_finished("req")
    watch.remove()
    p.connector.close()
    d.connector.close()


@pytest.mark.parametrize("direction", DIRECTIONS)
def test_a_prefix_resident_on_the_decode_side_is_reserved_skipped_and_left_untouched(direction):
    """The decode-side reservation hook end to end on the device (mirrors tests/test_pd.py:626-687 and
    tests/test_stage_engine.py:595-648 of the reference): D imports a prompt, which publishes its pages; a second
    prompt sharing 4 pages is reserved with ``cached_tokens`` = 64 on the shared physical blocks, P starts at token 64,
    ``bytes_sent`` is smaller by the prefix, the shared blocks keep their bytes and the whole pool equals the oracle's."""
    import numpy as np

    from oracle import handoff_oracle as ho
    from vllm_rlt_b200.pd.config import PDConfig

    config = PDConfig()
    shape = dict(shape=(4, 4, 64), page=16, planes=2, blocks=64, stage=True)
    p = Worker("prefill", config, 0, seed=1, device="cuda:0", direction=direction, **shape)
    d = Worker("decode", config, 1, seed=2, device="cuda:0", direction=direction, prefix_caching=True, **shape)
    p.connector.command(dict(kind="connect", peers=[d.transport.info]))
    d.connector.command(dict(kind="connect", peers=[p.transport.info]))
    P, D = oracle_of(p, 1 << 30), oracle_of(d, 1 << 40)
    per_token = 2 * 4 * 4 * 64 * 2 * 2

    def run(tid, prompt):
        d.connector.command(dict(kind="reserve", tid=tid, tokens=prompt, params=Params(), peer="prefill-0"))
        (reserved,) = d.take("reserved")
        p.connector.command(dict(kind="prefill", tid=tid, tokens=prompt, params=Params(), peer="decode-0",
                                 tables=reserved["tables"], slot=reserved["slot"], cached_tokens=reserved["cached_tokens"]))
        request = p.engine.requests[tid]
        p.engine.begin_prefill(request)
        p.engine.end_prefill(request, torch.full((16,), 1.0, device="cuda:0"))
        event = torch.cuda.Event()
        event.record()
        ho.handoff_rows(P, D, p.pool.plane_block_tables(tid), reserved["tables"], reserved["cached_tokens"], len(prompt))
        p.connector.prefill_submitted(request, phase="PREFILLING_RECURRENT", start=0,
                                      progress=SimpleNamespace(chunk_complete=True, prompt_complete=True), event=event, stream=None)
        pump(p, d, lambda: bool([m for m in p.messages if m["kind"] == "commit"]))
        (commit,) = p.take("commit")
        d.connector.command(dict(kind="commit", tid=tid, count=commit["count"]))
        pump(p, d, lambda: bool([m for m in d.messages if m["kind"] == "received"]))
        d.take("received")
        p.connector.command(dict(kind="ack", tid=tid))
        pump(p, d, lambda: tid not in p.connector.transfers)
        return reserved

    first = run("one", list(range(1, 101)))          # 100 tokens: pages 0..5 become cached on D
    assert first["cached_tokens"] == 0 and p.transport.bytes_sent == 100 * per_token + 64
    second = run("two", list(range(1, 65)) + list(range(500, 540)))   # shares 4 whole pages = 64 tokens
    assert second["cached_tokens"] == 64
    assert [list(t[:4]) for t in second["tables"]] == [list(t[:4]) for t in first["tables"]]
    assert p.transport.bytes_sent == (100 + 104 - 64) * per_token + 2 * 64
    assert d.pool._allocations["two"].imported == 104 and d.engine.requests["two"].num_prefilled_tokens == 104
    torch.cuda.synchronize()
    for got, want in zip(device_bytes(d.pool), (D.key.data.reshape(-1), D.value.data.reshape(-1))):
        assert np.array_equal(got, want)  # includes the shared blocks: written once, by the first import
    d.transport.close()  # the reader unmaps before the owner lets go (the imports stay reserved on D)
    p.transport.close()
