"""The benchmark's own workload at its full size (64 requests, 149,439 tokens, 29.4 GB of payload), checked through
properties that do not need the CPU oracle: every destination row equals the source row torch indexing selects, rows
outside the ranges keep the sentinel, and pack followed by scatter lands the same bytes as the direct handoff.

Needs about 165 GiB of device memory; skipped where that much is not free.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def untouched_rows_keep_the_sentinel(w, dst):
    """Token slots of each request's last block that lie beyond its range end were never written."""
    bs = w.shape.block_size
    for r, (_, end) in enumerate(w.ranges):
        used = end % bs
        if used == 0:
            continue
        for plane in range(w.dst_planes):
            block = int(np.asarray(w.dst_tables[r][plane])[(end - 1) // bs])
            for t in (dst.key_cache, dst.value_cache):
                if not bool((t[block, :, used:].view(torch.uint8) == 0xA5).all()):
                    return False
    return True


def test_full_size_exit_only_handoff_and_pack_scatter_round_trip():
    import bench
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.kernels import kv_handoff as kh

    torch.cuda.empty_cache()
    free, _ = torch.cuda.mem_get_info(0)
    w = workloads.last_exited_exit_only(requests=64, mode="exit_only")
    need = (w.src_blocks + w.dst_blocks) * w.shape.block_bytes + w.payload_bytes + (2 << 30)
    if free < need:
        pytest.skip(f"needs {need / 2**30:.0f} GiB of free device memory")
    device = torch.device("cuda", 0)
    src, dst = bench.build_device_side(w, device, 11)
    sv, dv = kh.PoolView.from_cache(src), kh.PoolView.from_cache(dst)
    batch = kh.HandoffBatch(w.src_tables, w.dst_tables, w.ranges, block_size=w.shape.block_size, exit_planes=w.exit_planes,
                            src_blocks=w.src_blocks, dst_blocks=w.dst_blocks, device=device)
    status = kh.new_status(device)

    kh.kv_handoff(sv, dv, batch, mode=kh.MODE_EXIT_ONLY, status=status)
    kh.raise_for_status(status)
    assert bench.spot_check(w, src, dst)  # every row of every request
    assert untouched_rows_keep_the_sentinel(w, dst)
    direct = [int(t.view(torch.uint8).view(torch.int64).sum()) for t in (dst.key_cache, dst.value_cache)]

    # the same bytes through the wire image
    for t in (dst.key_cache, dst.value_cache):
        t.view(torch.uint8).fill_(0xA5)
    size = kh.packed_bytes(sv, batch.total_tokens, 1)
    assert size == w.payload_bytes
    packed = torch.empty(size, dtype=torch.uint8, device=device)
    kh.kv_pack(sv, batch, packed, mode=kh.MODE_EXIT_ONLY, status=status)
    kh.kv_scatter(packed, dv, batch, status=status)
    kh.raise_for_status(status)
    del packed
    assert bench.spot_check(w, src, dst)
    assert untouched_rows_keep_the_sentinel(w, dst)
    # a checksum of the whole destination pool (wrapping 64-bit sums): identical after both routes
    assert [int(t.view(torch.uint8).view(torch.int64).sum()) for t in (dst.key_cache, dst.value_cache)] == direct
    del src, dst
    torch.cuda.empty_cache()


def test_the_reference_cpu_case_at_its_stated_size_against_the_oracle():
    """The configuration the reference itself can run on a CPU, at its stated size: Ouro-1.4B-shaped per-depth KV
    (24 layers x 4 planes, 16 KV heads of 128, bf16 N(0,1)), 8 requests with prompt lengths U[128, 1024], block 16,
    two independent pools of 4,096 blocks with seeded random block tables. The oracle plans every request with the
    reference's segment walk and partitioning and writes the descriptors on the CPU; the GPU does the direct handoff and,
    separately, gather -> pack -> scatter. Every block a table names is compared byte for byte (rows past a range's
    end must still hold the fill byte), and every other block of the destination pool must still be all fill bytes.
    The oracle's pools are allocated lazily and only the named blocks are ever touched on the host."""
    from oracle import handoff_oracle as ho
    from tests.conftest import oracle_pool
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh

    layers, heads, dim, blocks, page, planes = shape = (24, 16, 128, 4096, 16, 4)
    pool_bytes = 2 * blocks * layers * page * heads * dim * 2
    if torch.cuda.mem_get_info(0)[0] < 4 * pool_bytes:
        pytest.skip("needs about 52 GiB of free device memory")
    rng = np.random.default_rng(20240)
    lengths = [int(n) for n in rng.integers(128, 1025, size=8)]

    def tables_for(seed):
        order = np.random.default_rng(seed).permutation(blocks).tolist()
        out = []
        for n in lengths:
            pages = -(-n // page)
            claim = [order.pop() for _ in range(planes * pages)]
            out.append([claim[p * pages : (p + 1) * pages] for p in range(planes)])
        return out

    src_tables, dst_tables = tables_for(1), tables_for(2)
    src = KVPool(layers, heads, dim, blocks, page, planes, device="cuda")
    gen = torch.Generator(device="cuda").manual_seed(7)
    src.key_cache.normal_(generator=gen)
    src.value_cache.normal_(generator=gen)

    def fresh_destination():
        pool = KVPool(layers, heads, dim, blocks, page, planes, device="cuda")
        for t in (pool.key_cache, pool.value_cache):
            t.view(torch.uint8).fill_(0xA5)
        return pool

    # the oracle's side: the named source blocks come from the device, the named destination blocks start as fill bytes
    P = oracle_pool("bf16", shape)
    D = oracle_pool("bf16", shape, device=1, base=1 << 40)
    used_src = sorted({b for request in src_tables for table in request for b in table})
    used_dst = sorted({b for request in dst_tables for table in request for b in table})
    for host, device_tensor in ((P.key, src.key_cache), (P.value, src.value_cache)):
        taken = device_tensor[torch.tensor(used_src, device="cuda")].view(torch.uint8).cpu().numpy()
        host.data[used_src] = taken.reshape(len(used_src), *host.data.shape[1:])
    for host in (D.key, D.value):
        host.data[used_dst] = 0xA5
    moved = sum(ho.handoff_reference(P, D, s, d, 0, n) for s, d, n in zip(src_tables, dst_tables, lengths))
    assert moved == sum(lengths) * planes * 2 * layers * heads * dim * 2

    def equals_the_oracle(pool):
        named = torch.tensor(used_dst, device="cuda")
        others = torch.ones(blocks, dtype=torch.bool, device="cuda")
        others[named] = False
        for host, device_tensor in ((D.key, pool.key_cache), (D.value, pool.value_cache)):
            got = device_tensor[named].view(torch.uint8).cpu().numpy().reshape(len(used_dst), -1)
            if not np.array_equal(got, host.data[used_dst].reshape(len(used_dst), -1)):
                return False
            if not bool((device_tensor[others].view(torch.uint8) == 0xA5).all()):
                return False
        return True

    sv = kh.PoolView.from_cache(src)
    batch = kh.HandoffBatch(src_tables, dst_tables, [(0, n) for n in lengths], block_size=page, src_blocks=blocks, dst_blocks=blocks)
    status = kh.new_status()
    direct = fresh_destination()
    kh.kv_handoff(sv, kh.PoolView.from_cache(direct), batch, status=status)
    kh.raise_for_status(status)
    assert equals_the_oracle(direct)
    del direct

    size = kh.packed_bytes(sv, batch.total_tokens, planes)
    assert size == moved
    packed = torch.empty(size, dtype=torch.uint8, device="cuda")
    kh.kv_pack(sv, batch, packed, status=status)
    first = ho.pack_rows(P, src_tables[0], 0, lengths[0])  # the wire image starts with the first request's rows
    assert np.array_equal(packed[: first.size].cpu().numpy(), first)
    through_the_wire = fresh_destination()
    kh.kv_scatter(packed, kh.PoolView.from_cache(through_the_wire), batch, status=status)
    kh.raise_for_status(status)
    assert equals_the_oracle(through_the_wire)
