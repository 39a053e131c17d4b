"""Transport bookkeeping without a GPU: handshake, budget, tickets, time-outs, the mailbox protocol.

Mirrors what the reference pins for its NIXL transport with a fake agent (tests/test_pd.py:810-870)
and what its connector tests expect of a transport (tests/test_transfer_connector.py:15-27).
"""

import pytest
import torch

from tests.fakes import FakeBackend, cpu_cache
from vllm_rlt_b200.pd import transport as tr
from vllm_rlt_b200.pd.config import PDConfig


def make_pair(config=None, **cache_kw):
    config = config or PDConfig()
    pc, dc = cpu_cache(**cache_kw), cpu_cache(**cache_kw)
    pc.key_cache.view(torch.uint8).random_(0, 256)
    pc.value_cache.view(torch.uint8).random_(0, 256)
    p = tr.B200Transport("p0", pc, torch.zeros(2, 16), config, backend=FakeBackend())
    d = tr.B200Transport("d0", dc, torch.zeros(2, 16), config, backend=FakeBackend(), lane=1)
    p.connect(d.info)
    d.connect(p.info)
    return p, d


def block_range(info, block, nbytes=None):
    n = info["block_bytes"] if nbytes is None else nbytes
    return (info["key_ptr"] + block * info["block_bytes"], n, info["device"])


def test_info_has_every_key_the_connector_and_coordinator_read():
    p, d = make_pair()
    want = {"key_ptr", "value_ptr", "block_bytes", "layer_bytes", "token_bytes", "agent", "metadata", "hidden_ptr",
            "hidden_bytes", "device", "num_blocks", "block_size", "num_layers", "depths", "kv_dtype", "fp8_scale",
            "scale_region"}
    assert want <= set(p.info)
    assert p.info["agent"] == "p0" and p.info["scale_region"] is None
    assert p.info["block_bytes"] == 3 * 4 * 2 * 8 * 2 and p.info["token_bytes"] == 32
    assert p.peers == {"d0": d.info}
    for t in (p, d):
        t.close()


def test_write_lands_and_receiver_is_notified_in_order():
    p, d = make_pair()
    local = [block_range(p.info, 3), block_range(p.info, 5, 64)]
    remote = [block_range(d.info, 7), block_range(d.info, 1, 64)]
    size = sum(n for _, n, _ in local)
    assert p.submit("tid-a", 0, "d0", local, remote, size)
    assert p.submit("tid-a", 1, "d0", local[:1], remote[:1], local[0][1])
    assert p.busy("tid-a") and not p.busy("other") and p.inflight_bytes == size + local[0][1]
    finished, notes = p.poll()
    assert [t.sequence for t in finished] == [0, 1] and notes == []
    assert p.inflight_bytes == 0 and p.bytes_sent == size + local[0][1] and p.transfers == 2 and not p.pending
    _, notes = d.poll()
    assert notes == [("p0", "tid-a", 0), ("p0", "tid-a", 1)]
    assert d.poll()[1] == []
    src, dst = p.cache.key_cache.view(torch.uint8), d.cache.key_cache.view(torch.uint8)
    assert torch.equal(dst[7], src[3])
    assert torch.equal(dst[1].reshape(-1)[:64], src[5].reshape(-1)[:64])
    assert int(dst[1].reshape(-1)[64:].sum()) == 0
    for t in (p, d):
        t.close()


def test_budget_refuses_without_raising_and_chunk_limit_raises():
    config = PDConfig(transfer_chunk_bytes=400, max_inflight_bytes=600)
    p, d = make_pair(config)
    p.backend.complete_immediately = False
    seg = lambda n: ([block_range(p.info, 0, n)], [block_range(d.info, 0, n)], n)  # noqa: E731
    with pytest.raises(ValueError, match="exceeds configured chunk size"):
        p.submit("t", 0, "d0", *seg(401))
    assert p.submit("t", 0, "d0", *seg(384))
    assert p.submit("t", 1, "d0", *seg(384)) is False  # would exceed the in-flight budget: retry later
    assert p.inflight_bytes == 384 and len(p.pending) == 1
    assert p.poll()[0] == []
    with pytest.raises(RuntimeError, match="in-flight"):
        p.close()
    p.backend.events[0].done = True
    assert len(p.poll()[0]) == 1
    assert p.submit("t", 1, "d0", *seg(384))
    p.backend.events[1].done = True
    p.poll()
    for t in (p, d):
        t.close()


def test_a_write_that_never_completes_times_out():
    config = PDConfig(request_timeout=0.01)
    p, d = make_pair(config)
    p.backend.complete_immediately = False
    assert p.submit("t", 0, "d0", [block_range(p.info, 0, 64)], [block_range(d.info, 0, 64)], 64)
    import time

    time.sleep(0.05)
    with pytest.raises(TimeoutError, match="quarantined"):
        p.poll()


def test_descriptor_outside_registered_memory_is_rejected():
    p, d = make_pair()
    bad = [(d.info["key_ptr"] + d.info["block_bytes"] * d.info["num_blocks"] - 8, 64, 1)]
    with pytest.raises(ValueError, match="outside the peer's registered memory"):
        p.submit("t", 0, "d0", [block_range(p.info, 0, 64)], bad, 64)
    with pytest.raises(ValueError, match="incompatible source/target KV geometry"):
        p.submit("t", 0, "d0", [block_range(p.info, 0, 64)], [block_range(d.info, 0, 32)], 64)
    for t in (p, d):
        t.close()


@pytest.mark.parametrize("key", ["block_size", "num_layers", "depths", "hidden_bytes", "kv_dtype", "token_bytes"])
def test_handshake_rejects_geometry_mismatch(key):
    p, d = make_pair()
    peer = dict(d.info, agent="d1", metadata=dict(d.info["metadata"], lane=2))
    peer[key] = "x" if key == "kv_dtype" else peer[key] + 1
    with pytest.raises(ValueError, match=f"PD KV geometry mismatch: {key}"):
        p.connect(peer)
    for t in (p, d):
        t.close()


def test_handshake_rejects_scale_mismatch():
    a = tr.B200Transport("a", cpu_cache(fp8=True), torch.zeros(1, 8), PDConfig(), backend=FakeBackend())
    b = tr.B200Transport("b", cpu_cache(fp8=True, fp8_scale=0.5), torch.zeros(1, 8), PDConfig(), backend=FakeBackend())
    c = tr.B200Transport("c", cpu_cache(fp8=True, fp8_scale=0.25), torch.zeros(1, 8), PDConfig(), backend=FakeBackend())
    assert a.info["scale_region"] is not None and b.info["scale_region"] is None
    assert len(a.storage) == 5 and len(b.storage) == 3  # dynamic scales are registered, fixed ones are not
    with pytest.raises(ValueError, match="same calibrated FP8 scale"):
        a.connect(b.info)
    with pytest.raises(ValueError, match="same calibrated FP8 scale"):
        b.connect(c.info)
    b.connect(dict(b.info, agent="b2", metadata=dict(b.info["metadata"], lane=1)))
    with pytest.raises(ValueError, match="shares mailbox lane"):
        b.connect(dict(b.info, agent="b3", metadata=dict(b.info["metadata"], lane=1)))
    for t in (a, b, c):
        t.close()


def test_mailbox_wraps_and_applies_back_pressure():
    p, d = make_pair()
    one = ([block_range(p.info, 0, 16)], [block_range(d.info, 0, 16)], 16)
    for seq in range(tr.SLOTS):
        assert p.submit("t", seq, "d0", *one)
        p.poll()
    assert p.submit("t", tr.SLOTS, "d0", *one) is False  # ring full until the receiver drains it
    _, notes = d.poll()
    assert [s for _, _, s in notes] == list(range(tr.SLOTS))
    for seq in range(tr.SLOTS, tr.SLOTS + 10):
        assert p.submit("t", seq, "d0", *one)
    p.poll()
    assert [s for _, _, s in d.poll()[1]] == list(range(tr.SLOTS, tr.SLOTS + 10))
    with pytest.raises(ValueError, match="transfer id longer"):
        p.submit("x" * 60, 0, "d0", *one)
    for t in (p, d):
        t.close()


def test_config_validation_matches_reference_rules():
    for bad in (dict(prefill_devices=(0,), decode_devices=(0,)), dict(prefill_devices=()), dict(max_inflight_bytes=0),
                dict(transfer_chunk_bytes=100, max_inflight_bytes=50), dict(request_timeout=float("inf")), dict(backend="")):
        with pytest.raises(ValueError):
            PDConfig(**bad)
    c = PDConfig()
    assert c.max_inflight_bytes >= 24 * 4 * 2 * 2048 * 16 * 128 * 2  # a 2048-token Ouro-1.4B prompt stays in flight whole


# ----------------------------------------------------------------------------- pull direction


def make_pull_pair(config=None, **cache_kw):
    config = config or PDConfig()
    pc, dc = cpu_cache(**cache_kw), cpu_cache(**cache_kw)
    pc.key_cache.view(torch.uint8).random_(0, 256)
    pc.value_cache.view(torch.uint8).random_(0, 256)
    p = tr.B200Transport("p0", pc, torch.arange(32, dtype=torch.float32).reshape(2, 16), config, backend=FakeBackend(), direction="pull")
    d = tr.B200Transport("d0", dc, torch.zeros(2, 16), config, backend=FakeBackend(), lane=1, direction="pull")
    p.connect(d.info)
    d.connect(p.info)
    return p, d


def test_an_offered_chunk_is_read_by_the_peer_and_completes_only_when_it_says_so():
    p, d = make_pull_pair()
    src_tables, dst_tables = ((3, 5), (7, 9), (11, 13), (2, 4)), ((1, 0), (6, 8), (10, 12), (14, 15))
    hidden = (p.info["hidden_ptr"] + 64, d.info["hidden_ptr"], 64)
    size = 6 * 4 * 2 * 3 * 32 + 64
    assert p.submit_tables("tid", 0, "d0", [(src_tables, dst_tables, 1, 7)], size, extra=[hidden])
    assert p.busy("tid") and p.inflight_bytes == size and not p.backend.copies  # nothing moved on the source
    assert p.poll() == ([], []) and p.busy("tid")
    assert not d.reading
    _, notes = d.poll()  # finds the offer, reads the chunk (the fake copies at once), reports it, acknowledges
    assert notes == [("p0", "tid", 0)] and d.bytes_received == size and not d.reading
    assert [c[0] for c in d.backend.copies if isinstance(c, tuple)] == ["tables"]
    finished, notes = p.poll()
    assert [t.sequence for t in finished] == [0] and notes == [] and not p.busy("tid")
    assert p.bytes_sent == size and p.inflight_bytes == 0 and p.transfers == 1
    for plane in range(4):
        for t in range(1, 7):
            a = p.cache.key_cache[src_tables[plane][t // 4], :, t % 4].view(torch.uint8)
            b = d.cache.key_cache[dst_tables[plane][t // 4], :, t % 4].view(torch.uint8)
            assert torch.equal(a, b)
    assert int(d.cache.key_cache[dst_tables[0][0], :, 0].view(torch.uint8).sum()) == 0  # token 0 was not in the range
    assert torch.equal(d.storage[2][0], p.storage[2][1])  # the hidden row came along
    for t in (p, d):
        t.close()


def test_a_reader_that_has_not_finished_keeps_the_source_busy_and_blocks_close():
    p, d = make_pull_pair()
    d.backend.complete_immediately = False
    tables = ((0,), (1,), (2,), (3,))
    assert p.submit_tables("t", 0, "d0", [(tables, tables, 0, 4)], 4 * 4 * 2 * 3 * 32)
    assert d.poll() == ([], []) and d.reading
    assert p.poll() == ([], []) and p.busy("t")
    with pytest.raises(RuntimeError, match="in-flight"):
        d.close()
    d.backend.events[-1].done = True
    assert d.poll()[1] == [("p0", "t", 0)] and not d.reading
    assert len(p.poll()[0]) == 1
    for t in (p, d):
        t.close()


def test_descriptors_are_cut_to_the_pages_of_the_chunk_and_round_trip():
    source = (tuple(range(100, 140)), tuple(range(200, 240)))
    target = (tuple(range(300, 340)), tuple(range(400, 440)))
    s, t, lo, hi = tr.trim_request(source, target, 70, 101, 16)
    assert (lo, hi) == (6, 37) and s == ((104, 105, 106), (204, 205, 206)) and t == ((304, 305, 306), (404, 405, 406))
    raw = tr.encode_chunk([(s, t, lo, hi)], [(1 << 40, 1 << 41, 64)], mode=0, layer_begin=2, layer_end=5, plane_begin=1, plane_end=2)
    assert len(raw) < 200
    requests, extra, where = tr.decode_chunk(raw)
    assert [[list(x) for x in side] for side in requests[0][:2]] == [[list(x) for x in s], [list(x) for x in t]]
    assert requests[0][2:] == (6, 37) and extra == [(1 << 40, 1 << 41, 64)]
    assert where == dict(mode=0, layer_begin=2, layer_end=5, plane_begin=1, plane_end=2)
    with pytest.raises(ValueError, match="invalid KV range"):
        tr.encode_chunk([(s, t, 5, 5)], [])


def test_the_descriptor_ring_applies_back_pressure_and_reuses_space_in_order():
    ring = tr._RingWriter(size=100)
    assert ring.reserve(40, 1, 0) == 0 and ring.reserve(40, 2, 0) == 40
    assert ring.reserve(40, 3, 0) is None          # 20 bytes at the end, nothing consumed: no room
    assert ring.reserve(40, 3, 1) == 0             # message 1 consumed: its bytes are free again (wraps to the front)
    assert ring.reserve(30, 4, 1) is None          # would run into message 2's bytes
    assert ring.reserve(30, 4, 3) == 40            # everything consumed: continues after the last region
    with pytest.raises(ValueError, match="larger than the descriptor ring"):
        ring.reserve(101, 5, 4)
    p, d = make_pull_pair()
    wide = tuple(tuple(range(i, i + 4)) for i in (0, 4, 8, 12))
    sent = 0
    while p.submit_tables("t", sent, "d0", [(wide, wide, 0, 16)], 16 * 4 * 2 * 3 * 32):
        sent += 1
        assert sent <= tr.SLOTS  # the message ring fills first with descriptors this small
    assert sent == tr.SLOTS
    assert len(d.poll()[1]) == sent
    assert p.submit_tables("t", sent, "d0", [(wide, wide, 0, 16)], 16 * 4 * 2 * 3 * 32)
    d.poll()
    assert d.reading      # the source has not read its 256 "pulled" messages yet: the 257th waits for a slot
    p.poll()
    d.poll()
    assert not d.reading
    p.poll()
    assert not p.pending
    for t in (p, d):
        t.close()


def test_time_outs_and_transfer_time_count_from_when_the_copy_could_begin():
    """A chunk queued behind a long prefill is not a slow transfer: the clock starts when the transfer stream gets
    to it, not when it was queued."""
    import time

    config = PDConfig(request_timeout=0.05)
    p, d = make_pair(config)
    p.backend.hold_start = True
    p.backend.complete_immediately = False
    assert p.submit("t", 0, "d0", [block_range(p.info, 0, 64)], [block_range(d.info, 0, 64)], 64)
    time.sleep(0.12)
    assert p.poll() == ([], [])                    # twice the time-out has passed, but the copy has not begun
    p.backend.markers[-1].done = True
    assert p.poll() == ([], [])                    # begun now: the clock starts here
    p.backend.events[-1].done = True
    finished, _ = p.poll()
    assert len(finished) == 1 and p.transfer_seconds < 0.05
    assert p.submit("t", 1, "d0", [block_range(p.info, 0, 64)], [block_range(d.info, 0, 64)], 64)
    p.backend.markers[-1].done = True
    p.poll()
    time.sleep(0.12)
    with pytest.raises(TimeoutError, match="quarantined"):
        p.poll()


@pytest.mark.parametrize("direction", ["push", "pull"])
def test_chunks_submitted_together_share_one_launch_but_keep_their_tickets_and_notifications(direction):
    config = PDConfig(transfer_chunk_bytes=3000, max_inflight_bytes=7000)
    pc, dc = cpu_cache(), cpu_cache()
    pc.key_cache.view(torch.uint8).random_(0, 256)
    p = tr.B200Transport("p0", pc, torch.zeros(2, 16), config, backend=FakeBackend(), direction=direction)
    d = tr.B200Transport("d0", dc, torch.zeros(2, 16), config, backend=FakeBackend(), lane=1, direction=direction)
    p.connect(d.info)
    d.connect(p.info)
    tables = ((0, 1), (2, 3), (4, 5), (6, 7))
    per_token = 4 * 2 * 3 * 32
    request = [(tables, tables, 0, 8)]
    with pytest.raises(ValueError, match="consecutive sequence numbers"):
        p.submit_tables("t", 4, "d0", request, 8 * per_token, parts=[(4, 3 * per_token), (6, 5 * per_token)])
    with pytest.raises(ValueError, match="add up"):
        p.submit_tables("t", 4, "d0", request, 8 * per_token, parts=[(4, 3 * per_token), (5, 3 * per_token)])
    with pytest.raises(ValueError, match="exceeds configured chunk size"):
        p.submit_tables("t", 4, "d0", request, 8 * per_token, parts=[(4, 4 * per_token), (5, 4 * per_token)])
    parts = [(4, 3 * per_token), (5, 3 * per_token), (6, 2 * per_token)]
    assert p.submit_tables("t", 4, "d0", request, 8 * per_token, parts=parts)
    assert len(p.pending) == 3 and p.inflight_bytes == 8 * per_token
    assert p.submit_tables("t", 7, "d0", request, 8 * per_token, parts=[(7, 3 * per_token), (8, 3 * per_token), (9, 2 * per_token)]) is False
    notes = []
    for _ in range(3):
        notes += d.poll()[1]
        p.poll()
    assert notes == [("p0", "t", 4), ("p0", "t", 5), ("p0", "t", 6)]
    mover = d if direction == "pull" else p
    assert [c[0] for c in mover.backend.copies if isinstance(c, tuple)] == ["tables"]  # one launch for the three
    assert p.transfers == 3 and p.bytes_sent == 8 * per_token and not p.pending and p.inflight_bytes == 0
    assert torch.equal(dc.key_cache[:8].view(torch.uint8), pc.key_cache[:8].view(torch.uint8))
    assert int(dc.key_cache[8:].view(torch.uint8).sum()) == 0
    for t in (p, d):
        t.close()
