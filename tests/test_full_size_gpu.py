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
