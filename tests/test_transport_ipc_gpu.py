"""Two processes, as in a deployment: the decode worker owns its pool and mailbox, the prefill worker maps them.

The processes exchange only the transport's ``info`` dict (what the coordinator relays in the
``connect`` command). KV bytes go through the CUDA IPC mapping, notifications through the
shared-memory mailbox that the prefill GPU writes and the decode host polls. One GPU suffices:
nothing on the device waits for the other process.
"""

import time

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _pool(seed, fill, fp8=False):
    import random

    from vllm_rlt_b200.core.kv_pool import KVPool

    pool = KVPool(3, 4, 32, 64, 16, 2, device="cuda:0", kv_cache_dtype="fp8_e4m3" if fp8 else "auto")
    gen = torch.Generator(device="cuda:0").manual_seed(seed)
    tensors = [pool.key_cache, pool.value_cache] + ([pool.key_scale, pool.value_scale] if fp8 else [])
    for t in tensors:
        raw = t.view(torch.uint8)
        if fill:
            raw.random_(0, 256, generator=gen)
        else:
            raw.fill_(0xA5)
    random.Random(seed).shuffle(pool._free_blocks)
    return pool, tensors


def _decode_worker(conn, fp8):
    from vllm_rlt_b200.pd.config import PDConfig
    from vllm_rlt_b200.pd.transport import B200Transport

    try:
        torch.cuda.set_device(0)
        pool, tensors = _pool(2, fill=False, fp8=fp8)
        lengths = conn.recv()
        tables = {rid: pool.reserve_transfer(rid, n) for rid, n in lengths.items()}
        hidden = torch.zeros(4, 64, dtype=torch.bfloat16, device="cuda:0")
        d = B200Transport("d0", pool, hidden, PDConfig(), lane=9)
        conn.send(dict(info=d.info, tables=tables))
        d.connect(conn.recv())
        expected = conn.recv()
        notes, deadline = [], time.monotonic() + 30
        while len(notes) < expected and time.monotonic() < deadline:
            notes += d.poll()[1]
        torch.cuda.synchronize()
        conn.send(dict(notes=notes, pool=[t.contiguous().view(torch.uint8).cpu() for t in tensors], hidden=hidden.cpu()))
        conn.recv()  # the writer has unmapped: now the owner may free
        d.close()
        conn.send("closed")
    except Exception as exc:  # surface the failure in the parent
        conn.send(dict(error=repr(exc)))
        raise


@pytest.mark.parametrize("direction", ["push", "pull"])
@pytest.mark.parametrize("fp8", [False, True])
def test_cross_process_write_and_notification(fp8, direction):
    from oracle import handoff_oracle as ho
    from vllm_rlt_b200.pd.config import PDConfig
    from vllm_rlt_b200.pd.transport import B200Transport

    ctx = mp.get_context("spawn")
    parent, child = ctx.Pipe()
    proc = ctx.Process(target=_decode_worker, args=(child, fp8))
    proc.start()
    try:
        pool, tensors = _pool(1, fill=True, fp8=fp8)
        lengths = {"a": 40, "b": 17}
        for rid, n in lengths.items():
            assert pool.allocate(rid, n)
        parent.send(lengths)
        hello = parent.recv()
        assert "error" not in hello, hello
        hidden = torch.arange(4 * 64, dtype=torch.bfloat16, device="cuda:0").reshape(4, 64)
        cfg = PDConfig(transfer_chunk_bytes=1 << 20, max_transfer_descriptors=5)
        # "b" goes by tables: pushed by this process's GPU, or offered and pulled by the decode worker's
        p = B200Transport("p0", pool, hidden, cfg, direction=direction)
        p.connect(hello["info"])
        parent.send(p.info)
        seq = 0
        # request "a" by descriptor lists, request "b" by tables; the hidden row rides with "b"
        source = list(ho.kv_segments(p.info, pool.plane_block_tables("a"), 3, 40))
        target = list(ho.kv_segments(p.peers["d0"], hello["tables"]["a"], 3, 40))
        for local, remote, size in ho.partition_segments(source, target, cfg.transfer_chunk_bytes, cfg.max_transfer_descriptors):
            while not p.submit("a", seq, "d0", local, remote, size):
                p.poll()
            seq += 1
        hb = p.info["hidden_bytes"]
        extra = [(p.info["hidden_ptr"] + 3 * hb, hello["info"]["hidden_ptr"] + 1 * hb, hb)]
        size = 17 * 2 * 2 * 3 * (4 * 32 * (1 if fp8 else 2) + (16 if fp8 else 0)) + hb
        assert p.submit_tables("b", seq, "d0", [(pool.plane_block_tables("b"), hello["tables"]["b"], 0, 17)], size, extra=extra)
        seq += 1
        parent.send(seq)
        result = parent.recv()
        assert "error" not in result, result
        assert [(peer, s) for peer, _, s in result["notes"]] == [("p0", i) for i in range(seq)]
        assert [tid for _, tid, _ in result["notes"]] == ["a"] * (seq - 1) + ["b"]
        while p.pending:
            p.poll()
        # expected destination: sentinel everywhere except the rows of the two ranges
        for got, src_t in zip(result["pool"], tensors):
            want = torch.full_like(got, 0xA5)
            src_b = src_t.contiguous().view(torch.uint8).cpu()
            for rid, lo, hi in (("a", 3, 40), ("b", 0, 17)):
                for plane in range(2):
                    for t in range(lo, hi):
                        sb, db = pool.plane_block_tables(rid)[plane][t // 16], hello["tables"][rid][plane][t // 16]
                        want[db, :, t % 16] = src_b[sb, :, t % 16]
            assert torch.equal(got, want)
        assert torch.equal(result["hidden"][1], hidden[3].cpu()) and int(result["hidden"][[0, 2, 3]].abs().sum()) == 0
        p.close()  # unmap before the owner frees
        parent.send("unmapped")
        assert parent.recv() == "closed"
    finally:
        proc.join(timeout=60)
        if proc.is_alive():
            proc.terminate()
    assert proc.exitcode == 0
