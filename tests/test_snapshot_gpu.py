"""Preemption snapshots through the segment-copy kernel: same host layout as the reference's, bit-exact."""

import random

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kv,scale", [("auto", None), ("fp8_e4m3", None), ("fp8_e4m3", 0.5)])
def test_snapshot_matches_block_indexing_and_restore_round_trips(kv, scale):
    from vllm_rlt_b200.core.kv_pool import KVPool

    pool = KVPool(3, 4, 32, 64, 16, 3, device="cuda", kv_cache_dtype=kv, fp8_scale=scale)
    gen = torch.Generator(device="cuda").manual_seed(5)
    tensors = [pool.key_cache, pool.value_cache] + ([pool.key_scale, pool.value_scale] if kv != "auto" and scale is None else [])
    for t in tensors:
        t.view(torch.uint8).random_(0, 256, generator=gen)
    random.Random(1).shuffle(pool._free_blocks)
    assert pool.allocate("a", 70)
    blocks = [b for table in pool.plane_block_tables("a") for b in table]
    snap = pool.snapshot("a")
    assert snap.pages == 5 and snap.max_tokens == 70 and snap.keys.is_pinned()
    # the reference's statement: keys[row] = key_cache[block] (vllm_rlt/core/kv_cache_manager.py:637-643)
    assert torch.equal(snap.keys.view(torch.uint8), pool.key_cache[blocks].cpu().view(torch.uint8))
    assert torch.equal(snap.values.view(torch.uint8), pool.value_cache[blocks].cpu().view(torch.uint8))
    if kv != "auto":
        assert torch.equal(snap.key_scales.view(torch.uint8), pool.key_scale[blocks].cpu().view(torch.uint8))
        assert torch.equal(snap.value_scales.view(torch.uint8), pool.value_scale[blocks].cpu().view(torch.uint8))
    else:
        assert snap.key_scales is None
    before = [t.clone() for t in (pool.key_cache, pool.value_cache)]
    pool.free("a")
    assert pool.allocate("other", 30) and pool.allocate("a", 70)  # comes back in different blocks
    new_blocks = [b for table in pool.plane_block_tables("a") for b in table]
    assert new_blocks != blocks
    pool.restore("a", snap)
    torch.cuda.synchronize()
    assert torch.equal(pool.key_cache[new_blocks].view(torch.uint8), before[0][blocks].view(torch.uint8))
    assert torch.equal(pool.value_cache[new_blocks].view(torch.uint8), before[1][blocks].view(torch.uint8))
    untouched = sorted(set(range(64)) - set(new_blocks))
    assert torch.equal(pool.key_cache[untouched].view(torch.uint8), before[0][untouched].view(torch.uint8))


def test_snapshot_and_restore_refusals_match_the_reference():
    from vllm_rlt_b200.core.kv_pool import KVPool

    pool = KVPool(2, 2, 8, 32, 4, 2, device="cuda")
    assert pool.reserve_transfer("leased", 8) is not None
    with pytest.raises(RuntimeError, match="cannot snapshot KV during a transfer"):
        pool.snapshot("leased")
    assert pool.allocate("a", 8) and pool.allocate("b", 12) and pool.allocate("c", 8)
    snap = pool.snapshot("a")
    with pytest.raises(ValueError, match="capacity does not match"):
        pool.restore("b", snap)
    pool.mark_imported_prefix("c", 8)
    with pytest.raises(RuntimeError, match="already holds KV"):
        pool.restore("c", snap)
    fp8 = KVPool(2, 2, 8, 32, 4, 2, device="cuda", kv_cache_dtype="fp8_e4m3")
    assert fp8.allocate("a", 8)
    with pytest.raises(ValueError, match="dtype does not match"):
        fp8.restore("a", snap)
