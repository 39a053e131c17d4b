"""The pool's allocator and decode-side reservation hook on CPU tensors, pinned to the reference's behaviour.

Mirrors tests/test_pd.py:26-53 of the reference (lease-deferred free, import publication) and checks block-table
order against a trace recorded from the reference's ``KVCacheManager`` (tests/golden/allocation.json).
"""

import pytest
import torch

from tests.conftest import golden_json
from vllm_rlt_b200.core.kv_pool import KVPool


def make(blocks=16, planes=4, page=4, **kw):
    return KVPool(2, 1, 8, blocks, page, planes, device="cpu", dtype=torch.float32, **kw)


def test_block_table_order_matches_the_reference_trace():
    for case in golden_json("allocation.json"):
        layers, heads, dim, blocks, page, planes = case["shape"]
        pool = KVPool(layers, heads, dim, blocks, page, planes, device="cpu", dtype=torch.float32)
        for step in case["trace"]:
            if step["op"] == "alloc":
                assert pool.allocate(step["rid"], step["tokens"]) == step["ok"]
                assert [list(t) for t in pool.plane_block_tables(step["rid"])] == step["tables"]
            else:
                pool.free(step["rid"])
        assert pool.num_free_blocks == case["free"]


def test_transfer_lease_defers_free_until_last_reader():
    pool = make()
    assert pool.allocate("a", 8)
    pool.pin_transfer("a", "x")
    pool.pin_transfer("a", "y")
    pool.free("a")
    assert pool.num_used_blocks == 8
    with pytest.raises(RuntimeError, match="scheduled for release"):
        pool.pin_transfer("a", "z")
    pool.unpin_transfer("a", "x")
    assert pool.num_used_blocks == 8
    pool.unpin_transfer("a", "y")
    assert pool.num_used_blocks == 0
    pool.free("a")


def test_receive_publishes_only_once_and_within_capacity():
    pool = make()
    pool.allocate("a", 8)
    with pytest.raises(ValueError, match="exceeds reserved capacity"):
        pool.mark_imported_prefix("a", 9)
    pool.mark_imported_prefix("a", 7)
    with pytest.raises(RuntimeError, match="already initialized"):
        pool.mark_imported_prefix("a", 7)
    pool.allocate("b", 4)
    with pytest.raises(RuntimeError, match="already initialized"):
        pool.mark_imported_prefix("b", 4, start=2)  # the allocation holds no cached prefix of 2 tokens


def test_reservation_hook_allocates_pins_and_rejects_when_full():
    pool = make(blocks=8, planes=2)
    tables = pool.reserve_transfer("t1", 9)  # 3 pages x 2 planes
    assert tables == ((0, 1, 2), (3, 4, 5)) and pool.has_transfer_lease("t1")
    assert pool.reserve_transfer("t2", 8) is None  # 4 blocks needed, 2 free: rejected, nothing leaked
    assert pool.num_used_blocks == 6 and not pool.has_allocation("t2")
    with pytest.raises(ValueError, match="already owns KV blocks"):
        pool.reserve_transfer("t1", 1)
    with pytest.raises(ValueError, match="physical KV blocks"):
        pool.allocate("huge", 400)
    pool.free("t1")  # deferred: the transfer still holds its lease
    assert pool.num_used_blocks == 6
    pool.unpin_transfer("t1", "t1")
    assert pool.num_used_blocks == 0
    shared = KVPool(2, 1, 8, 8, 4, 4, device="cpu", dtype=torch.float32, layout="shared")
    assert shared.storage_depths == 1 and shared.required_blocks(9) == 3
    fp8 = KVPool(2, 1, 8, 8, 4, 2, device="cpu", kv_cache_dtype="fp8_e4m3", fp8_scale=0.5)
    assert fp8.key_cache.dtype == torch.float8_e4m3fn and float(fp8.key_scale.flatten()[0]) == 0.5
    with pytest.raises(ValueError):
        KVPool(2, 1, 8, 8, 4, 2, device="cpu", fp8_scale=0.5)
