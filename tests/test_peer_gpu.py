"""Two GPUs in one process: the handoff kernel with one pool behind a peer pointer, in both directions.

Push = the kernel runs on the source GPU and stores into the other GPU's pool; pull = the kernel runs on the
destination GPU and loads from the other GPU's pool. Either way the destination must equal the reference's
destination on the golden fixtures, byte for byte over the whole pool. Nothing here waits on another rank:
one process issues every launch and synchronises both devices.
"""

import pytest
import torch

from tests.conftest import golden_json, golden_npz, load_pool, oracle_pool
from tests.gpu_support import GpuPool, assert_pools_equal
from tests.test_kv_handoff_gpu import sentinel_destination

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from vllm_rlt_b200.pd import peer

    peer.enable_peer_access(0, 1)
    peer.enable_peer_access(1, 0)


@pytest.mark.parametrize("case", golden_json("handoff.json"), ids=lambda c: c["name"])
@pytest.mark.parametrize("direction", ["push", "pull"])
@pytest.mark.parametrize("variant", [0, 3, 5])
def test_cross_gpu_handoff_equals_reference_destination(two_gpus, case, direction, variant):
    from vllm_rlt_b200.kernels import kv_handoff as k

    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    D = oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40)
    load_pool(P, arrays, "src_")
    load_pool(D, arrays, "dst_before_")
    gp, gd = GpuPool(P, device="cuda:0"), GpuPool(D, device="cuda:1")
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    run_on = 0 if direction == "push" else 1
    reqs = case["requests"]
    with torch.cuda.device(run_on):
        status = k.new_status(f"cuda:{run_on}")
        batch = k.HandoffBatch(
            [r["src_tables"] for r in reqs], [r["dst_tables"] for r in reqs],
            [(r["start"], r["end"]) for r in reqs], block_size=P.block_size,
            src_blocks=P.num_blocks, dst_blocks=D.num_blocks, device=f"cuda:{run_on}",
        )
        k.kv_handoff(gp.view(), gd.view(), batch, status=status, variant=variant)
        torch.cuda.synchronize(run_on)
        k.raise_for_status(status)
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)
    # the source is read-only in both directions
    load_pool(P, arrays, "src_")
    assert_pools_equal(gp, P)


# exit-only needs every layer in every plane: the recurrent-layer fixtures are left to the single-GPU tests
FULL_DEPTH = [c for c in golden_json("finalize.json") if c["recurrent_layers"] is None]


@pytest.mark.parametrize("case", FULL_DEPTH, ids=lambda c: c["name"])
@pytest.mark.parametrize("direction", ["push", "pull"])
def test_cross_gpu_exit_only_takes_each_token_at_its_exit_plane(two_gpus, case, direction):
    from oracle import handoff_oracle as ho
    from vllm_rlt_b200.kernels import kv_handoff as k

    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    load_pool(P, arrays, "src_after_")
    D = sentinel_destination(case["kind"], case["shape"], planes=1)
    reqs = case["requests"]
    ranges = [(0, r["tokens"]) for r in reqs]
    exits = [r["exit_planes"] for r in reqs]
    one = [[r["dst_tables"][0]] for r in reqs]
    gp, gd = GpuPool(P, device="cuda:0"), GpuPool(D, device="cuda:1")
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    run_on = 0 if direction == "push" else 1
    with torch.cuda.device(run_on):
        status = k.new_status(f"cuda:{run_on}")
        batch = k.HandoffBatch([r["src_tables"] for r in reqs], one, ranges, block_size=P.block_size,
                               exit_planes=exits, device=f"cuda:{run_on}")
        k.kv_handoff(gp.view(), gd.view(), batch, mode=k.MODE_EXIT_ONLY, status=status)
        torch.cuda.synchronize(run_on)
        k.raise_for_status(status)
    for r, tables in zip(reqs, one):
        ho.handoff_rows(P, D, r["src_tables"], tables, 0, r["tokens"], mode=ho.MODE_EXIT_ONLY, exit_planes=r["exit_planes"])
    assert_pools_equal(gd, D)


@pytest.mark.parametrize("case", FULL_DEPTH, ids=lambda c: c["name"])
@pytest.mark.parametrize("direction", ["push", "pull"])
def test_cross_gpu_dedup_rebuilds_the_reference_destination(two_gpus, case, direction):
    """Dedup between two GPUs: rows up to each token's exit plane are read once and stored to every plane they
    fill; the destination equals what the reference wrote by sending all planes."""
    from vllm_rlt_b200.kernels import kv_handoff as k

    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    load_pool(P, arrays, "src_after_")
    D = sentinel_destination(case["kind"], case["shape"])
    reqs = case["requests"]
    gp, gd = GpuPool(P, device="cuda:0"), GpuPool(D, device="cuda:1")
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    run_on = 0 if direction == "push" else 1
    with torch.cuda.device(run_on):
        status = k.new_status(f"cuda:{run_on}")
        batch = k.HandoffBatch([r["src_tables"] for r in reqs], [r["dst_tables"] for r in reqs],
                               [(0, r["tokens"]) for r in reqs], block_size=P.block_size,
                               exit_planes=[r["exit_planes"] for r in reqs], device=f"cuda:{run_on}")
        k.kv_handoff(gp.view(), gd.view(), batch, mode=k.MODE_DEDUP, status=status)
        torch.cuda.synchronize(run_on)
        k.raise_for_status(status)
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)
