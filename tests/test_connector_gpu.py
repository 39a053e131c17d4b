"""The connector driving the real transport and kernels: a prefill and a decode worker on one GPU.

Same hand-relayed control sequence as tests/test_connector_cpu.py, but every chunk is a real
``rlt_kv_handoff`` launch, the hidden row a real segment copy, and every notification is written by the
GPU into the decode worker's mailbox.
"""

import time
from types import SimpleNamespace

import pytest
import torch

from tests.test_connector_cpu import Params, Worker, pool_rows

pytestmark = pytest.mark.gpu


def pump(p, d, until, limit=20.0):
    deadline = time.monotonic() + limit
    while not until() and time.monotonic() < deadline:
        p.connector.progress()
        d.connector.progress()
    assert until()


@pytest.mark.parametrize("fp8", [False, True])
def test_handoff_through_connector_transport_and_kernels(fp8):
    from vllm_rlt_b200.pd.config import PDConfig

    per_token = 2 * 3 * (2 * 8 * (1 if fp8 else 2) + (2 * 4 if fp8 else 0)) * 2
    config = PDConfig(transfer_chunk_bytes=5 * per_token + 100, max_inflight_bytes=16 * per_token)
    p = Worker("prefill", config, 0, seed=1, fp8=fp8, device="cuda:0")
    d = Worker("decode", config, 1, seed=2, fp8=fp8, device="cuda:0")
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


def test_chunks_leave_behind_the_producer_event_without_another_progress_pass():
    """The reference submits a chunk only when a later ``progress()`` pass finds its event fired (the commit tail,
    vllm_rlt/pd/config.py:10-15). Here the copies are queued at once behind the event on the device: the decode
    side receives every notification although the prefill worker's host never runs ``progress()`` again."""
    from vllm_rlt_b200.pd.config import PDConfig

    per_token = 2 * 3 * (2 * 8 * 2) * 2
    config = PDConfig(transfer_chunk_bytes=6 * per_token, max_inflight_bytes=64 * per_token)
    p = Worker("prefill", config, 0, seed=1, device="cuda:0")
    d = Worker("decode", config, 1, seed=2, device="cuda:0")
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
