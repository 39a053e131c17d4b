"""GPU parity of the batched exit-depth propagation against pools the reference itself finalized."""

import numpy as np
import pytest
import torch

from tests.conftest import golden_json, golden_npz, load_pool, oracle_pool
from tests.gpu_support import GpuPool, assert_pools_equal

pytestmark = pytest.mark.gpu


def full_view(gp):
    """Pool view that always carries the scale tensors: finalize copies them for fixed-scale pools too."""
    from vllm_rlt_b200.kernels.kv_handoff import PoolView

    return PoolView.from_tensors(gp.key_cache, gp.value_cache, gp.storage_depths, gp.key_scale, gp.value_scale)


@pytest.mark.parametrize("case", golden_json("finalize.json"), ids=lambda c: c["name"])
def test_finalize_reproduces_the_reference_pool(case):
    from vllm_rlt_b200.kernels import kv_handoff as kh

    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"], recurrent_layers=case["recurrent_layers"])
    load_pool(P, arrays, "src_before_")
    gp = GpuPool(P)
    reqs = case["requests"]
    planes = case["shape"][5]
    width = max(len(t) for r in reqs for t in r["src_tables"])
    tables = np.zeros((len(reqs), planes, width), np.int32)
    rows = []
    for i, r in enumerate(reqs):
        for p, t in enumerate(r["src_tables"]):
            tables[i, p, : len(t)] = t
        rows += [(i, e, pos) for pos, e in enumerate(r["exit_planes"])]
    status = kh.new_status()
    before = kh.kernel_launches()
    kh.kv_finalize(full_view(gp), torch.from_numpy(tables).cuda(), torch.tensor(rows, dtype=torch.int32, device="cuda"),
                   layers=case["recurrent_layers"], status=status)
    assert kh.kernel_launches() == before + 1  # K, V and scales in one launch
    kh.raise_for_status(status)
    load_pool(P, arrays, "src_after_")
    assert_pools_equal(gp, P)


def test_finalize_matches_the_oracle_on_a_larger_seeded_pool_and_is_idempotent():
    import random

    from vllm_rlt_b200.kernels import kv_handoff as kh

    rng, nrng = random.Random(4), np.random.default_rng(4)
    P = oracle_pool("fp8", (4, 16, 128, 96, 16, 4))
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    lengths = [70, 33, 16]
    for i, n in enumerate(lengths):
        assert P.allocate(f"r{i}", n)
    gp = GpuPool(P)
    width = max(-(-n // 16) for n in lengths)
    tables = np.zeros((3, 4, width), np.int32)
    rows = []
    for i, n in enumerate(lengths):
        for p, t in enumerate(P.plane_block_tables(f"r{i}")):
            tables[i, p, : len(t)] = t
        for pos in range(n):
            e = rng.randrange(4)
            rows.append((i, e, pos))
            P.finalize_token(f"r{i}", pos, e)
    rng.shuffle(rows)
    t_tables, t_rows = torch.from_numpy(tables).cuda(), torch.tensor(rows, dtype=torch.int32, device="cuda")
    status = kh.new_status()
    for _ in range(2):
        kh.kv_finalize(full_view(gp), t_tables, t_rows, status=status)
        kh.raise_for_status(status)
        assert_pools_equal(gp, P)


def test_finalize_reports_rows_it_cannot_apply():
    from vllm_rlt_b200.kernels import kv_handoff as kh

    P = oracle_pool("bf16", (2, 2, 8, 16, 4, 3))
    P.fill_random(np.random.default_rng(0))
    P.allocate("a", 8)
    gp = GpuPool(P)
    tables = torch.tensor([[list(t) for t in P.plane_block_tables("a")]], dtype=torch.int32, device="cuda")
    rows = torch.tensor([(0, 1, 2), (0, 7, 3)], dtype=torch.int32, device="cuda")  # exit plane 7 does not exist
    status = kh.new_status()
    kh.kv_finalize(full_view(gp), tables, rows, status=status)
    with pytest.raises(ValueError, match="exit plane outside"):
        kh.raise_for_status(status)
    P.finalize_token("a", 2, 1)  # the valid row was still applied, the bad one skipped
    assert_pools_equal(gp, P)
    with pytest.raises(ValueError, match="recurrent_layers"):
        kh.kv_finalize(full_view(gp), tables, rows, layers=[5])


@pytest.mark.parametrize("planes", [2, 32, 64, 65])
def test_finalize_with_many_planes_fills_every_deeper_plane(planes):
    """Up to 64 planes one unit loads a row once and stores it to every deeper plane; beyond that the
    unit-per-target kernel runs. Both must leave the pool the oracle's ``finalize_token`` leaves."""
    import random

    from vllm_rlt_b200.kernels import kv_handoff as kh

    rng = random.Random(planes)
    lengths = [9, 4, 1]
    page = 4
    blocks = sum(-(-n // page) for n in lengths) * planes + 2
    P = oracle_pool("fp8", (3, 2, 16, blocks, page, planes))
    P.fill_random(np.random.default_rng(planes))
    P.shuffle_free_list(rng)
    for i, n in enumerate(lengths):
        assert P.allocate(f"r{i}", n)
    gp = GpuPool(P)
    width = max(-(-n // page) for n in lengths)
    tables = np.zeros((len(lengths), planes, width), np.int32)
    rows = []
    for i, n in enumerate(lengths):
        for p, t in enumerate(P.plane_block_tables(f"r{i}")):
            tables[i, p, : len(t)] = t
        for pos in range(n):
            e = rng.choice([0, planes - 1, rng.randrange(planes)])
            rows.append((i, e, pos))
            P.finalize_token(f"r{i}", pos, e)
    status = kh.new_status()
    kh.kv_finalize(full_view(gp), torch.from_numpy(tables).cuda(), torch.tensor(rows, dtype=torch.int32, device="cuda"),
                   status=status)
    kh.raise_for_status(status)
    assert_pools_equal(gp, P)
