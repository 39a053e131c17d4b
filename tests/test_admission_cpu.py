"""The decode-side reservation hook (admission plan + prefix-aware allocation + lifecycle verbs) on CPU,
replayed against traces recorded from the reference's own ``StageEngine`` (tests/golden/reservation.json, written by
tests/golden/make_golden.py), and the properties the reference's tests pin for it
(tests/test_stage_engine.py:82-92, :138-154, :595-648 there)."""

from dataclasses import dataclass

import pytest
import torch

from tests.conftest import golden_json
from tests.fakes import FakeEvent
from vllm_rlt_b200.core.admission import Phase, StageSettings, TransferStage
from vllm_rlt_b200.core.kv_pool import KVPool


@dataclass
class Params:
    max_tokens: int


def stage_for(case, role="decode"):
    cache = dict(case["cache"])
    pool = KVPool(2, 1, 8, cache.pop("num_blocks"), cache.pop("block_size"), case["planes"], device="cpu",
                  dtype=torch.float32, **cache)
    settings = StageSettings(max_num_seqs=case["max_num_seqs"], prefill_chunk_size=case["prefill_chunk_size"])
    return TransferStage(role, pool, settings=settings)


@pytest.mark.parametrize("case", golden_json("reservation.json"), ids=lambda c: c["name"])
def test_reservations_replay_the_reference_trace(case):
    stage = stage_for(case)
    pool = stage.cache_manager
    live = {}
    for step in case["trace"]:
        rid = step["rid"]
        if step["op"] == "reserve":
            request = stage.reserve_transfer(rid, step["tokens"], Params(step["max_tokens"]), receiving=True)
            assert (request is not None) == step["ok"], step
            if request is None:
                assert rid not in stage.requests and not pool.has_allocation(rid)
            else:
                live[rid] = request
                assert request.phase is Phase.RECEIVING and pool.has_transfer_lease(rid)
                assert request.num_prefilled_tokens == step["cached_tokens"], step
                assert [list(t) for t in pool.plane_block_tables(rid)] == step["tables"], step
        elif step["op"] == "accept":
            request = live[rid]
            assert stage.accept_import(request, torch.zeros(4), cached_tokens=request.num_prefilled_tokens) is step["ok"]
            assert [list(page) for page in pool._prefixes.values()] == step["cached_pages"], step
        else:
            assert stage.release_transfer(live.pop(rid))
        assert pool.num_free_blocks == step["free"], step
        assert len(pool._free_blocks) == step["free_list"], step


def test_a_rejected_reservation_evicts_no_cached_page():
    case = next(c for c in golden_json("reservation.json") if c["name"] == "eviction")
    stage = stage_for(case)
    pool = stage.cache_manager
    a = stage.reserve_transfer("a", list(range(1, 10)), Params(1), receiving=True)
    stage.accept_import(a, torch.zeros(4))
    stage.release_transfer(a)
    cached = list(pool._prefixes.values())
    assert cached and pool.num_free_blocks == 32
    hold = stage.reserve_transfer("hold", list(range(30, 43)), Params(1), receiving=True)  # 16 blocks
    # needs 20 more blocks; 8 free + 8 evictable would not be enough: nothing may be evicted for it
    assert stage.reserve_transfer("big", [(5 * i) % 59 + 2 for i in range(17)], Params(1), receiving=True) is None
    assert list(pool._prefixes.values()) == cached and hold is not None


def test_import_activation_checks_identity_phase_and_prefix_start():
    case = golden_json("reservation.json")[0]
    stage = stage_for(case)
    pool = stage.cache_manager
    first = stage.reserve_transfer("g", list(range(1, 14)), Params(2), receiving=True)
    stage.release_transfer(first)
    second = stage.reserve_transfer("g", list(range(1, 14)), Params(2), receiving=True)
    assert not stage.accept_import(first, torch.zeros(4))          # a stale generation activates nothing
    with pytest.raises(RuntimeError, match="already initialized"):
        stage.accept_import(second, torch.zeros(4), cached_tokens=4)  # the reservation had no prefix hit
    assert stage.accept_import(second, torch.zeros(4), cached_tokens=0)
    with pytest.raises(ValueError, match="not awaiting an import"):
        stage.accept_import(second, torch.zeros(4))
    assert second.phase is Phase.RECEIVING and pool.has_transfer_lease("g")  # leased until a compute slot is granted
    granted = stage.grant_compute()
    assert granted == [second] and second.phase is Phase.DECODE and not pool.has_transfer_lease("g")
    stage.finish(second)
    # only cached pages remain, and those count as free because they can be evicted
    assert pool.num_used_blocks == 0 and pool.num_blocks - len(pool._free_blocks) == len(pool._prefixes) * pool.storage_depths


def test_compute_slots_are_granted_oldest_first_up_to_the_limit():
    case = dict(golden_json("reservation.json")[0], max_num_seqs=2)
    stage = stage_for(case)
    reqs = [stage.reserve_transfer(f"r{i}", [i + 1, i + 2, i + 3], Params(1), receiving=True) for i in range(3)]
    for r in reversed(reqs):
        stage.accept_import(r, torch.zeros(4))
    assert [r.request_id for r in stage.grant_compute()] == ["r2", "r1"]
    assert stage.grant_compute() == []
    stage.finish(reqs[2])
    assert [r.request_id for r in stage.grant_compute()] == ["r0"]


def test_source_retirement_is_two_steps_with_identity_checks():
    case = golden_json("reservation.json")[1]
    stage = stage_for(case, role="prefill")
    pool = stage.cache_manager
    request = stage.reserve_transfer("s", list(range(1, 9)), Params(1), receiving=False)
    assert request.phase is Phase.WAITING and pool.has_transfer_lease("s")
    event = FakeEvent(done=False)
    with pytest.raises(ValueError, match="not awaiting transfer completion"):
        stage.release_transfer_compute(request, ready_event=event)
    stage.begin_prefill(request)
    stage.end_prefill(request, torch.ones(4))
    assert not stage.release_transfer_compute(request, ready_event=event)  # the staging read is not done
    event.done = True
    assert stage.release_transfer_compute(request, ready_event=event)
    assert request.compute_released and request.hidden_state is None and pool.has_transfer_lease("s")
    assert stage.release_transfer(request) and pool.num_used_blocks == 0 and "s" not in stage.requests
    assert not stage.release_transfer(request)  # a second call finds another (or no) generation
    again = stage.reserve_transfer("s", list(range(1, 9)), Params(1), receiving=False)
    assert not stage.release_transfer_compute(request, ready_event=event) and again.phase is Phase.WAITING
    stage.suspend_transfer(again)
    assert again.phase is Phase.TRANSFERRING


def test_growth_and_frontier_arguments_are_validated():
    pool = KVPool(2, 1, 8, 16, 4, 2, device="cpu", dtype=torch.float32, incremental_allocation=True)
    assert pool.allocate("a", 16, initial_tokens=5)
    assert pool.allocated_blocks("a") == 4 and [len(t) for t in pool.plane_block_tables("a")] == [2, 2]
    assert pool.ensure_capacity("a", 8) and pool.allocated_blocks("a") == 4
    assert pool.ensure_capacity("a", 13) and [list(t) for t in pool.plane_block_tables("a")] == [[0, 1, 4, 5], [2, 3, 6, 7]]
    with pytest.raises(ValueError, match="exceeds logical capacity"):
        pool.ensure_capacity("a", 17)
    assert pool.allocate("b", 16, initial_tokens=16)
    assert not pool.ensure_capacity("a", 16) or pool.num_free_blocks == 0
    with pytest.raises(ValueError, match="invalid initial KV frontier"):
        pool.allocate("c", 4, initial_tokens=5)
    with pytest.raises(ValueError, match="prefix exceeds initial KV frontier"):
        pool.allocate("c", 8, initial_tokens=4, prefix=((0, 2), (1, 3)))
    with pytest.raises(ValueError, match="prefix caching requires last_exited"):
        KVPool(2, 1, 8, 16, 4, 2, device="cpu", layout="shared", enable_prefix_caching=True)
