"""GPU parity: the CUDA kernels, called through the C ABI, against the CPU oracle and the golden fixtures.

Bit-exact everywhere (the handoff is a byte mover). Every comparison is over the
whole destination pool, which was pre-filled with a sentinel, so a stray write is
caught as well as a missing one (the "no other byte changes" property pinned by
tests/test_tensor_transfer.py:64-74 in the reference).
"""

import random

import numpy as np
import pytest
import torch

from oracle import handoff_oracle as ho
from tests.conftest import golden_json, golden_npz, load_pool, oracle_pool
from tests.gpu_support import GpuPool, assert_pools_equal

pytestmark = pytest.mark.gpu

# kernel flavours: 0 = register path (16-byte loads/stores), 3 and 4 = cp.async.bulk rings of 8 x 4 KiB / 4 x 8 KiB,
# 5 = register path with 32-byte loads/stores, 6 = register path with the pool-to-pool dedup walking destination planes
# (the default walks source planes and fans each row out; see the fan-out tests below)
VARIANTS = [0, 3, 4, 5, 6]


def kh():
    from vllm_rlt_b200.kernels import kv_handoff

    return kv_handoff


def sentinel_destination(kind, shape, planes=None):
    s = list(shape)
    if planes is not None:
        s[5] = planes
    D = oracle_pool(kind, s, device=1, base=1 << 40)
    fixed = [t.data.copy() for t in (D.key_scale, D.value_scale)] if D.fp8 and D.fixed_scale is not None else None
    D.fill_sentinel()
    if fixed is not None:
        D.key_scale.data[...] = fixed[0]
        D.value_scale.data[...] = fixed[1]
    return D


# ----------------------------------------------------------------------------- golden fixtures


@pytest.mark.parametrize("case", golden_json("handoff.json"), ids=lambda c: c["name"])
@pytest.mark.parametrize("batched", [True, False])
@pytest.mark.parametrize("variant", VARIANTS)
def test_handoff_equals_reference_destination(case, batched, variant):
    k = kh()
    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    D = oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40)
    load_pool(P, arrays, "src_")
    load_pool(D, arrays, "dst_before_")
    gp, gd = GpuPool(P), GpuPool(D)
    reqs = case["requests"]
    status = k.new_status()
    groups = [reqs] if batched else [[r] for r in reqs]
    for group in groups:
        batch = k.HandoffBatch(
            [r["src_tables"] for r in group], [r["dst_tables"] for r in group],
            [(r["start"], r["end"]) for r in group], block_size=P.block_size,
            src_blocks=P.num_blocks, dst_blocks=D.num_blocks,
        )
        k.kv_handoff(gp.view(), gd.view(), batch, status=status, variant=variant)
    k.raise_for_status(status)
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)


@pytest.mark.parametrize("case", golden_json("handoff.json"), ids=lambda c: c["name"])
@pytest.mark.parametrize("longer", ["source", "destination"])
def test_tables_of_one_length_per_side_with_sides_of_different_length(case, longer):
    """Requests sent one at a time have tables of one length per side, which the batch converts in one step; a side
    whose tables run past the range (pages a later chunk will use) must not change what is copied."""
    k = kh()
    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    D = oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40)
    load_pool(P, arrays, "src_")
    load_pool(D, arrays, "dst_before_")
    gp, gd = GpuPool(P), GpuPool(D)
    status = k.new_status()
    for r in case["requests"]:
        src = [np.asarray(t, np.int32) for t in r["src_tables"]]
        dst = [np.asarray(t, np.int32) for t in r["dst_tables"]]
        pad = np.zeros(3, np.int32)  # block 0 is a valid id; the range never reaches these pages
        if longer == "source":
            src = [np.concatenate([t, pad]) for t in src]
        else:
            dst = [np.concatenate([t, pad]) for t in dst]
        batch = k.HandoffBatch([src], [dst], [(r["start"], r["end"])], block_size=P.block_size,
                               src_blocks=P.num_blocks, dst_blocks=D.num_blocks)
        assert batch.table_width == max(len(src[0]), len(dst[0]))
        k.kv_handoff(gp.view(), gd.view(), batch, status=status)
    k.raise_for_status(status)
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)


@pytest.mark.parametrize("case", golden_json("handoff.json"), ids=lambda c: c["name"])
def test_handoff_from_host_tables_equals_reference_destination(case):
    """``rlt_kv_handoff_host``: the library stages the tables itself. One request per call, the calls repeated so
    that the staging ring (16 slots) wraps; the arrays are overwritten right after each call returns."""
    k = kh()
    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    D = oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40)
    load_pool(P, arrays, "src_")
    load_pool(D, arrays, "dst_before_")
    gp, gd = GpuPool(P), GpuPool(D)
    status = k.new_status()
    for _ in range(7):  # every launch writes the same bytes; with 3 - 4 requests per case the ring wraps
        for r in case["requests"]:
            src = np.ascontiguousarray(np.asarray(r["src_tables"], np.int32)[None])
            dst = np.ascontiguousarray(np.asarray(r["dst_tables"], np.int32)[None])
            begin, end = np.asarray([r["start"]], np.int32), np.asarray([r["end"]], np.int32)
            k.kv_handoff_host(gp.view(), gd.view(), src, dst, begin, end, status=status)
            for a in (src, dst, begin, end):
                a[...] = -7  # the call has copied them: nothing may read these arrays any more
    k.raise_for_status(status)
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)


def test_host_tables_larger_than_a_staging_slot_are_refused():
    k = kh()
    case = golden_json("handoff.json")[0]
    P = oracle_pool(case["kind"], case["shape"])
    gp = GpuPool(P)
    width = k.host_batch_limit() // (4 * 2 * P.planes) + 1
    tables = np.zeros((1, P.planes, width), np.int32)
    one = np.zeros(1, np.int32)
    with pytest.raises(ValueError, match="limit"):
        k.kv_handoff_host(gp.view(), gp.view(), tables, tables, one, one + 1)


@pytest.mark.parametrize("case", golden_json("handoff.json"), ids=lambda c: c["name"])
@pytest.mark.parametrize("variant", VARIANTS)
def test_pack_equals_reference_wire_and_scatter_inverts_it(case, variant):
    k = kh()
    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    D = oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40)
    load_pool(P, arrays, "src_")
    load_pool(D, arrays, "dst_before_")
    gp, gd = GpuPool(P), GpuPool(D)
    reqs = case["requests"]
    batch = k.HandoffBatch(
        [r["src_tables"] for r in reqs], [r["dst_tables"] for r in reqs],
        [(r["start"], r["end"]) for r in reqs], block_size=P.block_size,
    )
    size = k.packed_bytes(gp.view(), batch.total_tokens, P.planes)
    assert size == arrays["packed"].size
    packed = torch.full((size + 64,), 0x5A, dtype=torch.uint8, device="cuda")
    status = k.new_status()
    k.kv_pack(gp.view(), batch, packed[:size], status=status, variant=variant)
    k.raise_for_status(status)
    got = packed.cpu().numpy()
    assert np.array_equal(got[:size], arrays["packed"])
    assert (got[size:] == 0x5A).all()
    k.kv_scatter(packed[:size], gd.view(), batch, status=status, variant=variant)
    k.raise_for_status(status)
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)


@pytest.mark.parametrize("case", golden_json("finalize.json"), ids=lambda c: c["name"])
def test_exit_plane_modes_on_reference_finalized_source(case):
    k = kh()
    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"], recurrent_layers=case["recurrent_layers"])
    load_pool(P, arrays, "src_after_")
    gp = GpuPool(P)
    reqs = case["requests"]
    ranges = [(0, r["tokens"]) for r in reqs]
    exits = [r["exit_planes"] for r in reqs]
    # all planes and dedup both reproduce the reference destination
    for mode in (k.MODE_ALL_PLANES, k.MODE_DEDUP):
        if mode == k.MODE_DEDUP and case["recurrent_layers"] is not None:
            continue
        D = sentinel_destination(case["kind"], case["shape"])
        gd = GpuPool(D)
        batch = k.HandoffBatch([r["src_tables"] for r in reqs], [r["dst_tables"] for r in reqs], ranges,
                               block_size=P.block_size, exit_planes=exits)
        status = k.new_status()
        k.kv_handoff(gp.view(), gd.view(), batch, mode=mode, status=status)
        k.raise_for_status(status)
        load_pool(D, arrays, "dst_after_")
        assert_pools_equal(gd, D)
    if case["recurrent_layers"] is not None:
        return
    # exit only: single-plane destination, checked against the row-level oracle
    D1 = sentinel_destination(case["kind"], case["shape"], planes=1)
    gd1 = GpuPool(D1)
    one = [[r["dst_tables"][0]] for r in reqs]
    batch = k.HandoffBatch([r["src_tables"] for r in reqs], one, ranges, block_size=P.block_size, exit_planes=exits)
    status = k.new_status()
    k.kv_handoff(gp.view(), gd1.view(), batch, mode=k.MODE_EXIT_ONLY, status=status)
    k.raise_for_status(status)
    for r, tables in zip(reqs, one):
        ho.handoff_rows(P, D1, r["src_tables"], tables, 0, r["tokens"], mode=ho.MODE_EXIT_ONLY, exit_planes=r["exit_planes"])
    assert_pools_equal(gd1, D1)
    # exit-only pack: the wire image is the row oracle's
    size = k.packed_bytes(gp.view(), batch.total_tokens, 1)
    packed = torch.zeros(size, dtype=torch.uint8, device="cuda")
    k.kv_pack(gp.view(), batch, packed, mode=k.MODE_EXIT_ONLY, status=status)
    k.raise_for_status(status)
    want = np.concatenate([
        ho.pack_rows(P, r["src_tables"], 0, r["tokens"], mode=ho.MODE_EXIT_ONLY, exit_planes=r["exit_planes"]) for r in reqs
    ])
    assert np.array_equal(packed.cpu().numpy(), want)


# ----------------------------------------------------------------------------- seeded cases vs the oracle

SHAPES = {
    # name: (kind, (layers, kv_heads, head_dim, blocks, block_size, planes))
    "ouro_bf16_small": ("bf16", (4, 16, 128, 96, 16, 4)),       # 4 KiB rows, vec16
    "ouro_fp8_small": ("fp8", (4, 16, 128, 96, 16, 4)),         # 2 KiB code rows + 64 B scale rows
    "huginn_rows": ("bf16", (3, 55, 96, 48, 16, 2)),            # 10,560 B rows: 16-B aligned, not a power of two
    "huginn_fp8_rows": ("fp8", (2, 55, 96, 40, 16, 2)),         # 220 B scale rows: 4-byte path
    "odd_rows": ("fp8", (3, 1, 3, 40, 8, 2)),                   # 3 B code rows (byte path), 4 B scale rows
    "block32": ("bf16", (2, 2, 8, 40, 32, 3)),
    "block1": ("bf16", (2, 2, 8, 64, 1, 2)),
    "shared_single_plane": ("bf16", (3, 2, 16, 40, 16, 1)),
}


def random_requests(rng, pool_src, pool_dst, count, max_tokens):
    reqs = []
    for i in range(count):
        tokens = rng.randint(1, max_tokens)
        if not (pool_src.allocate(f"r{i}", tokens) and pool_dst.allocate(f"r{i}", tokens)):
            break
        start = rng.choice([0, 0, rng.randrange(tokens)])
        end = rng.choice([tokens, tokens, rng.randint(start + 1, tokens)])
        reqs.append((f"r{i}", tokens, start, end))
    assert reqs
    return reqs


@pytest.mark.parametrize("name", list(SHAPES))
@pytest.mark.parametrize("mode_name", ["all", "dedup", "exit_only"])
@pytest.mark.parametrize("variant", VARIANTS)
def test_seeded_handoff_matches_oracle(name, mode_name, variant):
    k = kh()
    kind, shape = SHAPES[name]
    planes = shape[5]
    seed = hash((name, mode_name)) & 0xFFFF
    rng, nrng = random.Random(seed), np.random.default_rng(seed)
    P = oracle_pool(kind, shape)
    dst_planes = 1 if mode_name == "exit_only" else planes
    D = sentinel_destination(kind, shape, planes=dst_planes)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    D.shuffle_free_list(rng)
    per_request = shape[3] // (max(planes, 1) * 3)
    reqs = random_requests(rng, P, D, 3, max(1, per_request * shape[4] - 1))
    mode = {"all": ho.MODE_ALL_PLANES, "dedup": ho.MODE_DEDUP, "exit_only": ho.MODE_EXIT_ONLY}[mode_name]
    exits = None
    if mode != ho.MODE_ALL_PLANES:
        exits = [[rng.randrange(planes) for _ in range(t)] for _, t, _, _ in reqs]
        for (rid, t, _, _), e in zip(reqs, exits):
            for pos in range(t):
                P.finalize_token(rid, pos, e[pos])
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch(
        [P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
        [(s, e) for _, _, s, e in reqs], block_size=P.block_size, exit_planes=exits,
        src_blocks=P.num_blocks, dst_blocks=D.num_blocks,
    )
    status = k.new_status()
    k.kv_handoff(gp.view(), gd.view(), batch, mode=mode, status=status, variant=variant)
    k.raise_for_status(status)
    moved = 0
    for i, (rid, _, s, e) in enumerate(reqs):
        moved += ho.handoff_rows(P, D, P.plane_block_tables(rid), D.plane_block_tables(rid), s, e,
                                 mode=mode, exit_planes=None if exits is None else exits[i])
    assert moved == gp.view().payload_bytes(batch.total_tokens, dst_planes)
    assert_pools_equal(gd, D)
    if mode == ho.MODE_DEDUP:
        # on a finalized source, dedup and all-planes agree (what makes dedup a valid wire saving)
        D2 = sentinel_destination(kind, shape)
        D2._free, D2.tables = [], dict(D.tables)
        for rid, _, s, e in reqs:
            ho.handoff_reference(P, D2, P.plane_block_tables(rid), D2.plane_block_tables(rid), s, e)
        assert_pools_equal(gd, D2)


@pytest.mark.parametrize("name", ["ouro_bf16_small", "ouro_fp8_small", "huginn_fp8_rows", "odd_rows"])
@pytest.mark.parametrize("variant", VARIANTS)
def test_layer_slices_compose_to_the_full_handoff(name, variant):
    """Layer-by-layer streaming: slices [0,1), [1,3), [3,L) together equal one full handoff."""
    k = kh()
    kind, shape = SHAPES[name]
    rng, nrng = random.Random(11), np.random.default_rng(11)
    P = oracle_pool(kind, shape)
    D = sentinel_destination(kind, shape)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    D.shuffle_free_list(rng)
    reqs = random_requests(rng, P, D, 2, 3 * shape[4] + 5)
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch(
        [P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
        [(s, e) for _, _, s, e in reqs], block_size=P.block_size,
    )
    layers = shape[0]
    cuts = sorted({0, 1, min(3, layers), layers})
    status = k.new_status()
    for lo, hi in zip(cuts, cuts[1:]):
        k.kv_handoff(gp.view(), gd.view(), batch, layer_begin=lo, layer_end=hi, status=status, variant=variant)
        for rid, _, s, e in reqs:
            ho.handoff_rows(P, D, P.plane_block_tables(rid), D.plane_block_tables(rid), s, e, layer_begin=lo, layer_end=hi)
        assert_pools_equal(gd, D)
    k.raise_for_status(status)
    # and the packed image of a slice is the oracle's
    lo, hi = cuts[1], cuts[2] if len(cuts) > 2 else layers
    if hi > lo:
        size = k.packed_bytes(gp.view(), batch.total_tokens, P.planes, hi - lo)
        packed = torch.zeros(size, dtype=torch.uint8, device="cuda")
        k.kv_pack(gp.view(), batch, packed, layer_begin=lo, layer_end=hi, status=status, variant=variant)
        k.raise_for_status(status)
        want = np.concatenate([ho.pack_rows(P, P.plane_block_tables(r), s, e, layer_begin=lo, layer_end=hi) for r, _, s, e in reqs])
        assert np.array_equal(packed.cpu().numpy(), want)


@pytest.mark.parametrize("variant", VARIANTS)
def test_many_requests_cross_the_scan_tile(variant):
    """More requests than threads in a CTA, so the request prefix sums span several scan tiles."""
    k = kh()
    kind, shape = "bf16", (2, 2, 8, 2400, 4, 2)
    rng, nrng = random.Random(5), np.random.default_rng(5)
    P, D = oracle_pool(kind, shape), sentinel_destination(kind, shape)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    D.shuffle_free_list(rng)
    reqs = []
    for i in range(600):
        tokens = rng.randint(1, 7)
        assert P.allocate(f"r{i}", tokens) and D.allocate(f"r{i}", tokens)
        start = rng.randrange(tokens)
        reqs.append((f"r{i}", tokens, start, rng.randint(start + 1, tokens)))
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch(
        [P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
        [(s, e) for _, _, s, e in reqs], block_size=P.block_size,
    )
    status = k.new_status()
    k.kv_handoff(gp.view(), gd.view(), batch, status=status, variant=variant)
    k.raise_for_status(status)
    for rid, _, s, e in reqs:
        ho.handoff_rows(P, D, P.plane_block_tables(rid), D.plane_block_tables(rid), s, e)
    assert_pools_equal(gd, D)
    size = k.packed_bytes(gp.view(), batch.total_tokens, P.planes)
    packed = torch.zeros(size, dtype=torch.uint8, device="cuda")
    k.kv_pack(gp.view(), batch, packed, status=status, variant=variant)
    k.raise_for_status(status)
    want = np.concatenate([ho.pack_rows(P, P.plane_block_tables(r), s, e) for r, _, s, e in reqs])
    assert np.array_equal(packed.cpu().numpy(), want)


# ----------------------------------------------------------------------------- errors


def test_bad_block_id_is_reported_and_skipped_not_written():
    k = kh()
    kind, shape = "bf16", (2, 2, 8, 16, 4, 2)
    P, D = oracle_pool(kind, shape), sentinel_destination(kind, shape)
    P.fill_random(np.random.default_rng(0))
    P.allocate("a", 8)
    D.allocate("a", 8)
    gp, gd = GpuPool(P), GpuPool(D)
    src = [list(t) for t in P.plane_block_tables("a")]
    src[1][1] = 99  # outside the pool; host validation is bypassed by not passing src_blocks
    batch = k.HandoffBatch([src], [D.plane_block_tables("a")], [(0, 8)], block_size=4)
    status = k.new_status()
    k.kv_handoff(gp.view(), gd.view(), batch, status=status)
    with pytest.raises(ValueError, match="physical block outside registered pool"):
        k.raise_for_status(status)
    assert status.tolist()[:1] == [2] and status.tolist()[3] == 99
    # every other row arrived; the rows of the bad block kept the sentinel
    tables = P.plane_block_tables("a")
    ho.handoff_rows(P, D, tables, D.plane_block_tables("a"), 0, 8)
    bad_dst = D.plane_block_tables("a")[1][1]
    for t in D.tensors():
        t.data[bad_dst] = 0xA5
    assert_pools_equal(gd, D)
    with pytest.raises(ValueError, match="physical block outside registered pool"):
        k.HandoffBatch([src], [D.plane_block_tables("a")], [(0, 8)], block_size=4, src_blocks=16)


def test_host_validation_matches_reference_errors():
    k = kh()
    tables = [[[0, 1, 2]]]
    for rng_ in [(-1, 3), (3, 3), (5, 2)]:
        with pytest.raises(ValueError, match="invalid KV range"):
            k.HandoffBatch(tables, tables, [rng_], block_size=4)
    with pytest.raises(ValueError, match="KV range exceeds allocation"):
        k.HandoffBatch(tables, tables, [(0, 13)], block_size=4)
    P = oracle_pool("bf16", (2, 2, 8, 16, 4, 1))
    D = oracle_pool("bf16", (2, 2, 16, 16, 4, 1))
    batch = k.HandoffBatch(tables, tables, [(0, 12)], block_size=4)
    with pytest.raises(ValueError, match="geometry"):
        k.kv_handoff(GpuPool(P).view(), GpuPool(D).view(), batch)


# ----------------------------------------------------------------------------- dedup wire image


def dedup_case(kind, shape, seed, lengths):
    rng, nrng = random.Random(seed), np.random.default_rng(seed)
    planes = shape[5]
    P, D = oracle_pool(kind, shape), sentinel_destination(kind, shape)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    D.shuffle_free_list(rng)
    reqs, exits = [], []
    for i, n in enumerate(lengths):
        assert P.allocate(f"r{i}", n) and D.allocate(f"r{i}", n)
        start = rng.choice([0, rng.randrange(n)])
        end = rng.randint(start + 1, n)
        e = [rng.randrange(planes) for _ in range(n)]
        for pos in range(n):
            P.finalize_token(f"r{i}", pos, e[pos])
        reqs.append((f"r{i}", start, end))
        exits.append(e)
    return P, D, reqs, exits


@pytest.mark.parametrize("name", ["ouro_bf16_small", "ouro_fp8_small", "huginn_fp8_rows", "odd_rows", "block32"])
@pytest.mark.parametrize("variant", VARIANTS)
def test_dedup_wire_carries_only_executed_planes_and_scatter_rebuilds_the_rest(name, variant):
    k = kh()
    kind, shape = SHAPES[name]
    page, planes = shape[4], shape[5]
    P, D, reqs, exits = dedup_case(kind, shape, 21, [3 * page + 5, page, 2 * page - 1])
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch(
        [P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
        [(s, e) for _, s, e in reqs], block_size=page, exit_planes=exits,
    )
    want = np.concatenate([
        ho.pack_rows(P, P.plane_block_tables(r), s, e, mode=ho.MODE_DEDUP, exit_planes=exits[i])
        for i, (r, s, e) in enumerate(reqs)
    ])
    pairs = sum(exits[i][t] + 1 for i, (_, s, e) in enumerate(reqs) for t in range(s, e))
    full = k.packed_bytes(gp.view(), batch.total_tokens, planes)
    assert want.size == k.packed_bytes(gp.view(), pairs, 1) < full
    workspace = k.dedup_workspace(batch, planes)
    packed = torch.full((full,), 0x5A, dtype=torch.uint8, device="cuda")
    status = k.new_status()
    k.kv_pack(gp.view(), batch, packed, mode=k.MODE_DEDUP, status=status, workspace=workspace, variant=variant)
    k.raise_for_status(status)
    assert k.dedup_wire_tokens(workspace) == pairs
    got = packed.cpu().numpy()
    assert np.array_equal(got[: want.size], want)
    assert (got[want.size :] == 0x5A).all()
    # the receiver plans from the same exit planes and rebuilds every plane
    workspace2 = k.dedup_workspace(batch, planes)
    k.kv_scatter(packed[: want.size], gd.view(), batch, mode=k.MODE_DEDUP, status=status, workspace=workspace2, variant=variant)
    k.raise_for_status(status)
    for i, (r, s, e) in enumerate(reqs):
        ho.handoff_reference(P, D, P.plane_block_tables(r), D.plane_block_tables(r), s, e)
    assert_pools_equal(gd, D)


def test_dedup_pack_needs_a_workspace_of_the_stated_size():
    k = kh()
    kind, shape = SHAPES["ouro_bf16_small"]
    P, D, reqs, exits = dedup_case(kind, shape, 3, [20])
    gp = GpuPool(P)
    batch = k.HandoffBatch([P.plane_block_tables("r0")], None, [(0, 20)], block_size=16, exit_planes=exits)
    packed = torch.zeros(k.packed_bytes(gp.view(), 20, 4), dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="invalid argument"):
        k.kv_pack(gp.view(), batch, packed, mode=k.MODE_DEDUP)
    small = torch.zeros(32, dtype=torch.uint8, device="cuda")
    with pytest.raises(ValueError, match="size limit"):
        k.kv_pack(gp.view(), batch, packed, mode=k.MODE_DEDUP, workspace=small)


@pytest.mark.parametrize("mode_name", ["all", "dedup"])
def test_plane_and_layer_slices_tile_the_full_handoff(mode_name):
    """Per-depth streaming: every (plane slice, layer slice) launch moves exactly its part; together they are the handoff."""
    k = kh()
    kind, shape = SHAPES["ouro_fp8_small"]
    planes, layers = shape[5], shape[0]
    P, D, reqs, exits = dedup_case(kind, shape, 33, [45, 16, 7])
    mode = ho.MODE_ALL_PLANES if mode_name == "all" else ho.MODE_DEDUP
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch(
        [P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
        [(s, e) for _, s, e in reqs], block_size=shape[4], exit_planes=exits,
    )
    status = k.new_status()
    for p0, p1 in ((0, 1), (1, 3), (3, planes)):
        for l0, l1 in ((0, 2), (2, layers)):
            k.kv_handoff(gp.view(), gd.view(), batch, mode=mode, layer_begin=l0, layer_end=l1, plane_begin=p0,
                         plane_end=p1, status=status)
            for i, (r, s, e) in enumerate(reqs):
                st, dt = P.plane_block_tables(r), D.plane_block_tables(r)
                for plane in range(p0, p1):
                    for t in range(s, e):
                        sp = ho.source_plane(mode, plane, exits[i][t])
                        for a, b in zip(P.tensors(), D.tensors()):
                            b.data[dt[plane][t // 16], l0:l1, t % 16] = a.data[st[sp][t // 16], l0:l1, t % 16]
            assert_pools_equal(gd, D)
    k.raise_for_status(status)
    D2 = sentinel_destination(kind, shape)
    D2._free, D2.tables = [], dict(D.tables)
    for r, s, e in reqs:
        ho.handoff_reference(P, D2, P.plane_block_tables(r), D2.plane_block_tables(r), s, e)
    assert_pools_equal(gd, D2)
    with pytest.raises(ValueError, match="invalid argument"):
        k.kv_handoff(gp.view(), gd.view(), batch, plane_begin=2, plane_end=planes + 1)


def test_benchmark_shape_checked_row_by_row_with_torch_indexing():
    """The benchmark's own shape (Ouro-1.4B, 16-token blocks, 4 KiB rows) at a size the oracle would take minutes
    for: every destination row of every request is compared with the source row torch indexing selects."""
    import bench
    from vllm_rlt_b200 import workloads

    k = kh()
    for mode_name, mode in (("exit_only", k.MODE_EXIT_ONLY), ("dedup", k.MODE_DEDUP), ("all", k.MODE_ALL_PLANES)):
        w = workloads.last_exited_exit_only(requests=6, min_len=200, max_len=900, mode=mode_name)
        src, dst = bench.build_device_side(w, torch.device("cuda", 0), 7)
        batch = k.HandoffBatch(w.src_tables, w.dst_tables, w.ranges, block_size=16, exit_planes=w.exit_planes)
        status = k.new_status()
        if mode_name == "dedup":
            # dedup equals all-planes only on a finalized source: make planes beyond each exit a copy first
            width = max(len(t) for r in w.src_tables for t in r)
            tables = torch.zeros((len(w.lengths), 4, width), dtype=torch.int32)
            for i, r in enumerate(w.src_tables):
                for p, t in enumerate(r):
                    tables[i, p, : len(t)] = torch.from_numpy(np.asarray(t))
            rows = torch.tensor([(i, int(e), pos) for i, ex in enumerate(w.exit_planes) for pos, e in enumerate(ex)], dtype=torch.int32)
            k.kv_finalize(k.PoolView.from_cache(src), tables.cuda(), rows.cuda(), status=status)
        k.kv_handoff(k.PoolView.from_cache(src), k.PoolView.from_cache(dst), batch, mode=mode, status=status)
        k.raise_for_status(status)
        assert bench.spot_check(w, src, dst)
        if mode_name == "dedup":
            w_all = workloads.Workload(w.shape, w.lengths, w.ranges, w.src_tables, w.dst_tables, None, w.src_blocks,
                                       w.dst_blocks, w.dst_planes, extra=dict(mode="all"))
            assert bench.spot_check(w_all, src, dst)  # same bytes as the reference's all-planes handoff
        del src, dst
        torch.cuda.empty_cache()


@pytest.mark.parametrize("mode_name", ["all", "dedup"])
def test_recurrent_depth_model_carries_only_its_recurrent_layers_in_deeper_planes(mode_name):
    """Golden pools of a manager built with ``recurrent_layers=(2, 3)``: plane 0 moves whole, planes >= 1 move only
    layers 2 and 3 (the only ones ``finalize_token`` maintains there); the other rows keep the sentinel."""
    k = kh()
    case = [c for c in golden_json("finalize.json") if c["recurrent_layers"] is not None][0]
    arrays = golden_npz(case["name"])
    shape, deep = case["shape"], case["recurrent_layers"]
    P = oracle_pool(case["kind"], shape, recurrent_layers=deep)
    load_pool(P, arrays, "src_after_")
    D = sentinel_destination(case["kind"], shape)
    gp, gd = GpuPool(P), GpuPool(D)
    reqs = case["requests"]
    batch = k.HandoffBatch([r["src_tables"] for r in reqs], [r["dst_tables"] for r in reqs],
                           [(0, r["tokens"]) for r in reqs], block_size=shape[4],
                           exit_planes=[r["exit_planes"] for r in reqs])
    mode = k.MODE_ALL_PLANES if mode_name == "all" else k.MODE_DEDUP
    status = k.new_status()
    k.kv_handoff(gp.view(), gd.view(), batch, mode=mode, deep_layers=deep, status=status)
    k.raise_for_status(status)
    full = sentinel_destination(case["kind"], shape)
    load_pool(full, arrays, "dst_after_")  # the reference's all-layer, all-plane destination
    page = shape[4]
    for r in reqs:
        for plane, table in enumerate(r["dst_tables"]):
            layers = range(shape[0]) if plane == 0 else deep
            for t in range(r["tokens"]):
                for a, b in zip(full.tensors(), D.tensors()):
                    for layer in layers:
                        b.data[table[t // page], layer, t % page] = a.data[table[t // page], layer, t % page]
    assert_pools_equal(gd, D)


# ----------------------------------------------------------------------------- pool-to-pool dedup, fan-out walk


@pytest.mark.parametrize("planes,page,fp8", [(32, 16, False), (8, 64, True), (2, 1, False), (64, 4, False)])
def test_dedup_fan_out_reads_each_row_once_and_fills_every_deeper_plane(planes, page, fp8):
    """Many planes, geometric exits: the default dedup handoff (one unit per SOURCE plane, rows of tokens that
    stop there stored to every deeper plane) equals the oracle and the walk over destination planes (variant 6)."""
    k = kh()
    kind = "fp8" if fp8 else "bf16"
    lengths = [3 * page + 1, page, 2 * page - 1, 1]
    blocks = sum(-(-n // page) for n in lengths) * planes + 3
    shape = (3, 2, 16, blocks, page, planes)
    rng, nrng = random.Random(planes * 131 + page), np.random.default_rng(planes)
    P, D = oracle_pool(kind, shape), sentinel_destination(kind, shape)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    D.shuffle_free_list(rng)
    reqs, exits = [], []
    for i, n in enumerate(lengths):
        assert P.allocate(f"r{i}", n) and D.allocate(f"r{i}", n)
        e = [min(planes - 1, int(nrng.geometric(0.25)) - 1) for _ in range(n)]
        e[0], e[-1] = planes - 1, 0  # both ends of the range occur
        for pos in range(n):
            P.finalize_token(f"r{i}", pos, e[pos])
        start = rng.choice([0, rng.randrange(n)])
        reqs.append((f"r{i}", start, rng.randint(start + 1, n)))
        exits.append(e)
    results = []
    for variant in (0, 6):
        gp, gd = GpuPool(P), GpuPool(D)
        batch = k.HandoffBatch(
            [P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
            [(s, e) for _, s, e in reqs], block_size=page, exit_planes=exits,
            src_blocks=P.num_blocks, dst_blocks=D.num_blocks)
        status = k.new_status()
        k.kv_handoff(gp.view(), gd.view(), batch, mode=k.MODE_DEDUP, status=status, variant=variant)
        k.raise_for_status(status)
        results.append(gd)
        assert_pools_equal(gp, P)  # the source is only read
    for i, (r, s, e) in enumerate(reqs):
        ho.handoff_rows(P, D, P.plane_block_tables(r), D.plane_block_tables(r), s, e, mode=ho.MODE_DEDUP, exit_planes=exits[i])
    for gd in results:
        assert_pools_equal(gd, D)


def test_dedup_fan_out_reports_bad_exit_planes_and_bad_deeper_blocks():
    k = kh()
    kind, shape = "bf16", (2, 2, 8, 24, 4, 3)
    P, D = oracle_pool(kind, shape), sentinel_destination(kind, shape)
    P.fill_random(np.random.default_rng(5))
    P.allocate("a", 8)
    D.allocate("a", 8)
    tables_s, tables_d = P.plane_block_tables("a"), D.plane_block_tables("a")
    good = [0, 1, 2, 0, 1, 2, 0, 1]
    for pos, e in enumerate(good):
        P.finalize_token("a", pos, e)

    # an exit plane outside [0, planes): reported, that token is skipped on every plane, the others arrive
    for bad in (-1, 3):
        D.fill_sentinel()
        gp, gd = GpuPool(P), GpuPool(D)
        exits = list(good)
        exits[5] = bad
        batch = k.HandoffBatch([tables_s], [tables_d], [(0, 8)], block_size=4, exit_planes=[exits])
        status = k.new_status()
        k.kv_handoff(gp.view(), gd.view(), batch, mode=k.MODE_DEDUP, status=status)
        with pytest.raises(ValueError, match="exit plane"):
            k.raise_for_status(status)
        assert status.tolist()[0] == 3 and status.tolist()[3] == bad
        ho.handoff_rows(P, D, tables_s, tables_d, 0, 5, mode=ho.MODE_DEDUP, exit_planes=exits)
        ho.handoff_rows(P, D, tables_s, tables_d, 6, 8, mode=ho.MODE_DEDUP, exit_planes=exits)
        assert_pools_equal(gd, D)

    # a block id outside the pool on a deeper destination plane: reported; that plane's block keeps the sentinel,
    # the rows of the valid planes arrive
    D.fill_sentinel()
    gp, gd = GpuPool(P), GpuPool(D)
    broken = [list(t) for t in tables_d]
    broken[2][0] = 77
    batch = k.HandoffBatch([tables_s], [broken], [(0, 8)], block_size=4, exit_planes=[good])
    status = k.new_status()
    k.kv_handoff(gp.view(), gd.view(), batch, mode=k.MODE_DEDUP, status=status)
    with pytest.raises(ValueError, match="physical block outside registered pool"):
        k.raise_for_status(status)
    assert status.tolist()[0] == 2 and status.tolist()[3] == 77
    ho.handoff_rows(P, D, tables_s, tables_d, 0, 8, mode=ho.MODE_DEDUP, exit_planes=good)
    for t in D.tensors():
        t.data[tables_d[2][0]] = 0xA5
    assert_pools_equal(gd, D)


@pytest.mark.parametrize("variant", [0, 3])
def test_dedup_scatter_reports_a_negative_exit_plane_and_skips_the_token(variant):
    """A token whose exit plane is negative has no row on the wire: the scatter reports it, writes nothing for it and
    touches no block outside the request's own."""
    k = kh()
    kind, shape = SHAPES["ouro_bf16_small"]
    page, planes = shape[4], shape[5]
    P, D, reqs, exits = dedup_case(kind, shape, 8, [2 * page + 3])
    (rid, s, e), = reqs
    gp, gd = GpuPool(P), GpuPool(D)
    bad = [list(exits[0])]
    bad[0][s] = -1
    batch = k.HandoffBatch([P.plane_block_tables(rid)], [D.plane_block_tables(rid)], [(s, e)], block_size=page, exit_planes=bad)
    packed = torch.zeros(k.packed_bytes(gp.view(), e - s, planes), dtype=torch.uint8, device="cuda")
    status = k.new_status()
    k.kv_scatter(packed, gd.view(), batch, mode=k.MODE_DEDUP, status=status, workspace=k.dedup_workspace(batch, planes),
                 variant=variant)
    with pytest.raises(ValueError, match="exit plane"):
        k.raise_for_status(status)
    assert status.tolist()[0] == 3 and status.tolist()[2] == s and status.tolist()[3] == -1
    own = sorted(b for table in D.plane_block_tables(rid) for b in table)
    others = np.setdiff1d(np.arange(D.num_blocks), own)
    for t in gd.tensors():
        assert (t.view(torch.uint8)[torch.from_numpy(others).cuda()] == 0xA5).all()
    # the bad token's own rows kept the sentinel on every plane
    for plane, table in enumerate(D.plane_block_tables(rid)):
        assert (gd.key_cache.view(torch.uint8)[table[s // page], :, s % page] == 0xA5).all()


@pytest.mark.parametrize("variant", [0, 3])
def test_dedup_pack_reports_a_negative_exit_plane_and_leaves_the_token_off_the_wire(variant):
    """The pack side of the case above: the token has no row on any plane, so nothing that builds rows sees it; the
    pack must still report it, and the image must hold exactly the other tokens' rows."""
    k = kh()
    kind, shape = SHAPES["ouro_bf16_small"]
    page, planes = shape[4], shape[5]
    P, D, reqs, exits = dedup_case(kind, shape, 8, [2 * page + 3])
    (rid, s, e), = reqs
    gp = GpuPool(P)
    bad = [list(exits[0])]
    bad[0][s] = -1
    batch = k.HandoffBatch([P.plane_block_tables(rid)], None, [(s, e)], block_size=page, exit_planes=bad)
    want = ho.pack_rows(P, P.plane_block_tables(rid), s, e, mode=ho.MODE_DEDUP, exit_planes=bad[0])
    full = k.packed_bytes(gp.view(), e - s, planes)
    packed = torch.full((full,), 0x5A, dtype=torch.uint8, device="cuda")
    status = k.new_status()
    k.kv_pack(gp.view(), batch, packed, mode=k.MODE_DEDUP, status=status, workspace=k.dedup_workspace(batch, planes),
              variant=variant)
    with pytest.raises(ValueError, match="exit plane"):
        k.raise_for_status(status)
    assert status.tolist() == [3, 0, s, -1]
    got = packed.cpu().numpy()
    assert np.array_equal(got[: want.size], want) and (got[want.size :] == 0x5A).all()


@pytest.mark.parametrize("mode_name", ["exit_only", "dedup", "dedup_pack"])
def test_an_exit_array_shorter_than_the_ranges_is_reported_and_never_read_past(mode_name):
    """RltBatch.exit_count bounds every read of exit_planes: a request whose offset + range end runs past the
    array is reported as a bad range and skipped as a whole; the requests before it arrive untouched by that."""
    k = kh()
    kind, shape = SHAPES["ouro_bf16_small"]
    page, planes = shape[4], shape[5]
    P, D, reqs, exits = dedup_case(kind, shape, 13, [page + 2, 2 * page + 1])
    reqs = [(r, 0, e) for r, _, e in reqs]
    if mode_name == "exit_only":
        D = sentinel_destination(kind, shape, planes=1)
        for (r, _, _), n in zip(reqs, [page + 2, 2 * page + 1]):
            assert D.allocate(r, n)
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch([P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
                           [(s, e) for _, s, e in reqs], block_size=page, exit_planes=exits)
    assert batch.exit_count == len(exits[0]) + len(exits[1])
    batch.exit_count = len(exits[0]) + reqs[1][2] - 1  # one entry short of the second request's range end
    status = k.new_status()
    if mode_name == "dedup_pack":
        full = k.packed_bytes(gp.view(), batch.total_tokens, planes)
        packed = torch.full((full,), 0x5A, dtype=torch.uint8, device="cuda")
        k.kv_pack(gp.view(), batch, packed, mode=k.MODE_DEDUP, status=status, workspace=k.dedup_workspace(batch, planes))
        want = ho.pack_rows(P, P.plane_block_tables(reqs[0][0]), 0, reqs[0][2], mode=ho.MODE_DEDUP, exit_planes=exits[0])
        got = packed.cpu().numpy()
        assert np.array_equal(got[: want.size], want) and (got[want.size :] == 0x5A).all()
    else:
        mode = k.MODE_EXIT_ONLY if mode_name == "exit_only" else k.MODE_DEDUP
        k.kv_handoff(gp.view(), gd.view(), batch, mode=mode, status=status)
        r, s, e = reqs[0]
        ho.handoff_rows(P, D, P.plane_block_tables(r), D.plane_block_tables(r), s, e,
                        mode=ho.MODE_EXIT_ONLY if mode_name == "exit_only" else ho.MODE_DEDUP, exit_planes=exits[0])
        assert_pools_equal(gd, D)
    with pytest.raises(ValueError, match="KV range exceeds allocation"):
        k.raise_for_status(status)
    assert status.tolist()[:2] == [1, 1]
