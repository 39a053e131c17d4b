"""The multi-rank metadata exchange on CPU: two gloo ranks, decode tables and handles reach the prefill rank."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

from vllm_rlt_b200.pd import exchange


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        is_prefill, index, partners = exchange.pairing(rank, world)
        lengths, planes, width, page = [9, 16, 3], 2, 4, 4
        tables_msg = torch.zeros((len(lengths), planes, width), dtype=torch.int32)
        handles_msg = torch.zeros((2, exchange.HANDLE_ROW), dtype=torch.uint8)
        if not is_prefill:
            tables = [[[10 * r + p + j for j in range(-(-n // page))] for p in range(planes)] for r, n in enumerate(lengths)]
            tables_msg.copy_(exchange.encode_tables(tables, planes, width))
            exported = [{"handle": bytes([rank, k] * 32).hex(), "offset": 4096 * k + 48} for k in range(2)]
            handles_msg.copy_(exchange.encode_handles(exported))
        all_tables, all_handles = exchange.all_gather_metadata(tables_msg, handles_msg)
        if is_prefill:
            got_tables = exchange.decode_tables(all_tables[partners[0]], lengths, page)
            got_handles = exchange.decode_handles(all_handles[partners[0]])
            out.put((rank, got_tables, got_handles))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_rank_exchange_delivers_tables_and_handles():
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    rank, tables, handles = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert rank == 0
    assert tables == [[[0, 1, 2], [1, 2, 3]], [[10, 11, 12, 13], [11, 12, 13, 14]], [[20], [21]]]
    assert handles == [{"handle": bytes([1, 0] * 32).hex(), "offset": 48}, {"handle": bytes([1, 1] * 32).hex(), "offset": 4144}]


def test_pairing_for_even_and_uneven_splits():
    assert exchange.pairing(0, 2) == (True, 0, [1])
    assert exchange.pairing(1, 2) == (False, 0, [0])
    assert [exchange.pairing(r, 8)[2] for r in range(8)] == [[4], [5], [6], [7], [0], [1], [2], [3]]
    # 2P:6D - each prefill rank feeds three decode ranks; 6P:2D - three prefill ranks share one decode rank
    assert exchange.pairing(0, 8, 2) == (True, 0, [2, 4, 6])
    assert exchange.pairing(1, 8, 2) == (True, 1, [3, 5, 7])
    assert exchange.pairing(5, 8, 2) == (False, 3, [1])
    assert exchange.pairing(7, 8, 6) == (False, 1, [1, 3, 5])
    assert exchange.pairing(4, 8, 6) == (True, 4, [6])
    with pytest.raises(ValueError):
        exchange.pairing(0, 1)
    with pytest.raises(ValueError):
        exchange.pairing(0, 4, 4)


def test_table_codec_round_trip_and_errors():
    tables = [[[5, 6, 7], [8, 9, 1]], [[2], [3]]]
    msg = exchange.encode_tables(tables, 2, 3)
    assert msg.dtype == torch.int32 and tuple(msg.shape) == (2, 2, 3)
    assert exchange.decode_tables(msg, [12, 4], 4) == tables
    with pytest.raises(ValueError):
        exchange.encode_tables(tables, 3, 3)
    with pytest.raises(ValueError):
        exchange.encode_tables(tables, 2, 2)


def _lonely(rank, port, out):
    import datetime

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=2, timeout=datetime.timedelta(seconds=3))
        out.put("joined")
    except Exception as exc:
        out.put(type(exc).__name__)


def test_a_worker_that_never_joins_ends_the_exchange_with_an_error_not_a_hang():
    """Failure injection on the host: the peer of a two-rank exchange is simply never started."""
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    proc = ctx.Process(target=_lonely, args=(0, _free_port(), out))
    proc.start()
    got = out.get(timeout=90)
    proc.join(timeout=30)
    assert got != "joined"


def test_pull_edges_agree_on_both_ends_for_every_split():
    """Both ends of a P->D edge derive the same flag slots and request lists from the pairing alone, every request
    of every prefill rank is on exactly one edge, and no two edges share a flag word."""
    from vllm_rlt_b200.pd import exchange

    for world in (2, 3, 4, 5, 8):
        for prefill in range(1, world):
            for num_requests in (1, 2, 7, 64):
                plans = {r: exchange.pull_edges(r, world, prefill, num_requests) for r in range(world)}
                fan = max(len(exchange.pairing(r, world, prefill)[2]) for r in range(world))
                for p in range(prefill):
                    sent = sorted(i for e in plans[p] for i in e["requests"])
                    assert sent == list(range(num_requests))
                    assert len({e["done_slot"] for e in plans[p]}) == len(plans[p])
                    for e in plans[p]:
                        assert e["prefill"] == p and 0 <= e["done_slot"] < fan and 0 <= e["ready_slot"] < fan
                        assert e in plans[e["decode"]]  # the decode rank sees the very same edge
                for d in range(prefill, world):
                    assert len({e["ready_slot"] for e in plans[d]}) == len(plans[d])
                    for e in plans[d]:
                        assert e["decode"] == d and e in plans[e["prefill"]]


def _verify_worker(rank, world, port, out, damage):
    """Rank 0 owns a source pool, rank 1 the destination after a handoff written with loops; they run the same
    whole-transfer check the multi-GPU benchmark runs, over gloo instead of NCCL."""
    import torch.distributed as dist

    from tests.test_verify_cpu import SMALL, make_pool, plain_handoff
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.pd import verify

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        w = workloads.last_exited_exit_only(SMALL, requests=3, min_len=5, max_len=19, partial_fraction=0.7, mode="dedup", seed=5)
        src = make_pool(SMALL, w.src_blocks, SMALL.planes, seed=1)  # both ranks can build it: seeded
        everything = list(range(len(w.lengths)))
        if rank == 0:
            ok, nbytes = verify.verify_over_group(src, True, [(1, w, everything, None)], mode="dedup", device="cpu")
        else:
            dst = make_pool(SMALL, w.dst_blocks, w.dst_planes, fill=verify.FILL_BYTE)
            plain_handoff(src, dst, w, "dedup")
            if damage:
                dst.key_cache.view(torch.uint8)[int(w.dst_tables[0][0][0]), 0, 0, 0, 0] ^= 1
            ok, nbytes = verify.verify_over_group(dst, False, [(0, w, everything, [w.dst_tables[i] for i in everything])],
                                                  mode="dedup", device="cpu")
        out.put((rank, ok, nbytes, w.payload_bytes))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("damage", [False, True])
def test_whole_transfer_verification_over_two_ranks(damage):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_verify_worker, args=(r, 2, port, out, damage)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(out.get(timeout=180) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok, nbytes, payload in results:  # both ranks learn the same verdict and the same byte count
        assert ok == (not damage)
        assert nbytes == (0 if damage else payload)
