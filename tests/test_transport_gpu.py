"""The transport on a real GPU: descriptor-list WRITE, table-driven WRITE, GPU-written notifications."""

import random
import time

import pytest
import torch

from oracle import handoff_oracle as ho

pytestmark = pytest.mark.gpu


def make_pool(device, blocks=64, fp8=False, seed=0, fill=True):
    from vllm_rlt_b200.core.kv_pool import KVPool

    pool = KVPool(3, 4, 32, blocks, 16, 2, device=device, kv_cache_dtype="fp8_e4m3" if fp8 else "auto")
    gen = torch.Generator(device=device).manual_seed(seed)
    for t in (pool.key_cache, pool.value_cache):
        if fill:
            t.view(torch.uint8).random_(0, 256, generator=gen)
        else:
            t.view(torch.uint8).fill_(0xA5)
    if fp8:
        for t in (pool.key_scale, pool.value_scale):
            if fill:
                t.uniform_(0.01, 0.1, generator=gen)
            else:
                t.view(torch.uint8).fill_(0xA5)
    random.Random(seed).shuffle(pool._free_blocks)
    return pool


def expected_destination(P, D, requests):
    """Independent statement with torch indexing: destination rows <- source rows, everything else untouched."""
    want = [t.clone() for t in tensors(D)]
    for rid, start, end in requests:
        st, dt = P.plane_block_tables(rid), D.plane_block_tables(rid)
        for plane in range(len(st)):
            for t in range(start, end):
                for w, a in zip(want, tensors(P)):
                    w[dt[plane][t // 16], :, t % 16] = a[st[plane][t // 16], :, t % 16]
    return want


def tensors(pool):
    out = [pool.key_cache, pool.value_cache]
    if pool.key_scale is not None and pool.fp8_scale is None:
        out += [pool.key_scale, pool.value_scale]
    return out


def drain(p, d, want_notes):
    notes = []
    deadline = time.monotonic() + 20
    while (p.pending or len(notes) < want_notes) and time.monotonic() < deadline:
        p.poll()
        notes += d.poll()[1]
    assert not p.pending
    return notes


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("two_gpus", [False, True])
def test_descriptor_and_table_paths_write_the_same_bytes(fp8, two_gpus):
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd.config import PDConfig
    from vllm_rlt_b200.pd.transport import B200Transport

    if two_gpus and torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    dev_p, dev_d = "cuda:0", "cuda:1" if two_gpus else "cuda:0"
    config = PDConfig(transfer_chunk_bytes=1 << 20, max_inflight_bytes=8 << 20, max_transfer_descriptors=7)
    P = make_pool(dev_p, fp8=fp8, seed=1)
    requests = [("a", 0, 40), ("b", 5, 16), ("c", 16, 33)]
    lengths = {"a": 40, "b": 16, "c": 33}
    results = []
    for path in ("descriptors", "tables"):
        D = make_pool(dev_d, fp8=fp8, seed=2, fill=False)
        for rid in lengths:
            if not P.has_allocation(rid):
                assert P.allocate(rid, lengths[rid])
            assert D.reserve_transfer(rid, lengths[rid]) is not None
        hidden_p = torch.arange(4 * 64, dtype=torch.bfloat16, device=dev_p).reshape(4, 64)
        hidden_d = torch.zeros(4, 64, dtype=torch.bfloat16, device=dev_d)
        p = B200Transport("p0", P, hidden_p, config)
        d = B200Transport("d0", D, hidden_d, config, lane=9)  # one GPU may play both workers: distinct lanes
        p.connect(d.info)
        d.connect(p.info)
        want = expected_destination(P, D, requests)
        sent, seq = 0, 0
        status = kh.new_status(dev_p)
        for rid, start, end in requests:
            if path == "descriptors":
                source = ho.kv_segments(p.info, P.plane_block_tables(rid), start, end)
                target = ho.kv_segments(p.peers["d0"], D.plane_block_tables(rid), start, end)
                source, target = list(source), list(target)
                hb = p.info["hidden_bytes"]
                source.append((p.info["hidden_ptr"] + 1 * hb, hb, p.info["device"]))
                target.append((d.info["hidden_ptr"] + 2 * hb, hb, d.info["device"]))
                for local, remote, size in ho.partition_segments(source, target, config.transfer_chunk_bytes, config.max_transfer_descriptors):
                    while not p.submit(rid, seq, "d0", local, remote, size):
                        p.poll()
                    sent += size
                    seq += 1
            else:
                batch = [(P.plane_block_tables(rid), D.plane_block_tables(rid), start, end)]
                size = kh.PoolView.from_cache(P).payload_bytes(end - start, 2)
                hb = p.info["hidden_bytes"]
                extra = [(p.info["hidden_ptr"] + 1 * hb, d.info["hidden_ptr"] + 2 * hb, hb)]
                while not p.submit_tables(rid, seq, "d0", batch, size + hb, extra=extra, status=status):
                    p.poll()
                sent += size + hb
                seq += 1
        notes = drain(p, d, seq)
        kh.raise_for_status(status)
        assert [(a, s) for a, _, s in notes] == [("p0", i) for i in range(seq)]
        assert p.bytes_sent == sent and p.transfers == seq and p.inflight_bytes == 0
        torch.cuda.synchronize()
        for got, exp in zip(tensors(D), want):
            assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8))
        assert torch.equal(hidden_d[2].cpu(), hidden_p[1].cpu()) and int(hidden_d[[0, 1, 3]].abs().sum()) == 0
        results.append([t.clone() for t in tensors(D)])
        p.close()
        d.close()
        for rid in lengths:
            D.unpin_transfer(rid, rid)
            D.free(rid)
    for a, b in zip(*results):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))


def test_notification_is_only_visible_after_the_bytes():
    """The mailbox stamp is posted on the stream that carried the copy: once the receiver's host sees the
    notification, the destination already holds the data (checked right after the first sighting)."""
    from vllm_rlt_b200.pd.config import PDConfig
    from vllm_rlt_b200.pd.transport import B200Transport

    P = make_pool("cuda:0", blocks=512, seed=3)
    D = make_pool("cuda:0", blocks=512, seed=4, fill=False)
    assert P.allocate("a", 4096) and D.reserve_transfer("a", 4096) is not None
    cfg = PDConfig()
    p = B200Transport("p0", P, torch.zeros(1, 8, device="cuda:0"), cfg)
    d = B200Transport("d0", D, torch.zeros(1, 8, device="cuda:0"), cfg, lane=9)
    p.connect(d.info)
    d.connect(p.info)
    source = list(ho.kv_segments(p.info, P.plane_block_tables("a"), 0, 4096))
    target = list(ho.kv_segments(p.peers["d0"], D.plane_block_tables("a"), 0, 4096))
    parts = list(ho.partition_segments(source, target, cfg.transfer_chunk_bytes, cfg.max_transfer_descriptors))
    for seq, (local, remote, size) in enumerate(parts):
        assert p.submit("a", seq, "d0", local, remote, size)
    seen = []
    deadline = time.monotonic() + 20
    while len(seen) < len(parts) and time.monotonic() < deadline:
        seen += d.poll()[1]
    assert len(seen) == len(parts)
    last_dst = D.plane_block_tables("a")[1][-1]
    last_src = P.plane_block_tables("a")[1][-1]
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):  # a stream that is not ordered after the copy
        same = torch.equal(D.value_cache[last_dst].view(torch.uint8), P.value_cache[last_src].view(torch.uint8))
    assert same
    while p.pending:
        p.poll()
    p.close()
    d.close()


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("two_gpus", [False, True])
def test_offered_chunks_are_pulled_by_the_receiver_and_acknowledged(fp8, two_gpus):
    """The pull direction of ``submit_tables``: the sender only offers (behind an event), the receiver's GPU reads the
    sender's pool through peer pointers, reports the chunk when its own launch has finished and acknowledges it."""
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd.config import PDConfig
    from vllm_rlt_b200.pd.transport import B200Transport

    if two_gpus and torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    dev_p, dev_d = "cuda:0", "cuda:1" if two_gpus else "cuda:0"
    config = PDConfig(transfer_chunk_bytes=1 << 20, max_inflight_bytes=8 << 20)
    P = make_pool(dev_p, fp8=fp8, seed=1)
    D = make_pool(dev_d, fp8=fp8, seed=2, fill=False)
    requests = [("a", 0, 40), ("b", 5, 16), ("c", 16, 33)]
    for rid, n in {"a": 40, "b": 16, "c": 33}.items():
        assert P.allocate(rid, n) and D.reserve_transfer(rid, n) is not None
    hidden_p = torch.arange(4 * 64, dtype=torch.bfloat16, device=dev_p).reshape(4, 64)
    hidden_d = torch.zeros(4, 64, dtype=torch.bfloat16, device=dev_d)
    p = B200Transport("p0", P, hidden_p, config, direction="pull")
    d = B200Transport("d0", D, hidden_d, config, lane=9, direction="pull")
    p.connect(d.info)
    d.connect(p.info)
    want = expected_destination(P, D, requests)
    launches = kh.kernel_launches()
    with torch.cuda.device(dev_p):
        producer = torch.cuda.Stream()
        with torch.cuda.stream(producer):
            torch.cuda._sleep(int(0.05 * 1.9e9))  # the KV is "written" 50 ms from now
            ready = torch.cuda.Event()
            ready.record(producer)
    sent = 0
    hb = p.info["hidden_bytes"]
    for seq, (rid, start, end) in enumerate(requests):
        size = kh.PoolView.from_cache(P).payload_bytes(end - start, 2) + hb
        extra = [(p.info["hidden_ptr"] + 1 * hb, d.info["hidden_ptr"] + 2 * hb, hb)]
        assert p.submit_tables(rid, seq, "d0", [(P.plane_block_tables(rid), D.plane_block_tables(rid), start, end)], size,
                               extra=extra, after=ready)
        sent += size
    assert d.poll() == ([], []) and not ready.query()  # nothing is offered before the producer's event has fired
    assert all(p.busy(rid) for rid, _, _ in requests)
    notes = drain(p, d, len(requests))
    assert sorted((a, t, s) for a, t, s in notes) == [("p0", "a", 0), ("p0", "b", 1), ("p0", "c", 2)]
    assert p.bytes_sent == sent == d.bytes_received and p.transfers == 3 and p.inflight_bytes == 0 and not d.reading
    assert kh.kernel_launches() - launches == 3 * 3  # per chunk: the offer's post on P; the handoff and the hidden copy on D
    torch.cuda.synchronize(dev_d)
    for got, exp in zip(tensors(D), want):
        assert torch.equal(got.view(torch.uint8), exp.view(torch.uint8))
    assert torch.equal(hidden_d[2].cpu(), hidden_p[1].cpu()) and int(hidden_d[[0, 1, 3]].abs().sum()) == 0
    d.close()  # the reader unmaps the source pool before its owner lets go of it
    p.close()
