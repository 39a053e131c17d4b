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
