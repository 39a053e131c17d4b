"""Seeded random geometries: every path (direct, pack, scatter, dedup wire) and every kernel flavour against the oracle.

Shapes are drawn to hit the corners the fixed tests do not enumerate: block sizes from 1 to 64, rows that are
16-byte, 4-byte and odd multiples, one to five planes, layer and plane slices, ranges that start and end mid-block.
"""

import random

import numpy as np
import pytest
import torch

from oracle import handoff_oracle as ho
from tests.conftest import oracle_pool
from tests.gpu_support import GpuPool, assert_pools_equal
from tests.test_kv_handoff_gpu import sentinel_destination

pytestmark = pytest.mark.gpu

VARIANTS = [0, 1, 2, 3, 4, 5, 6]


def draw(seed):
    rng = random.Random(seed)
    kind = rng.choice(["bf16", "bf16", "fp8", "fp8", "fp8_fixed", "f32"])
    layers, heads = rng.randint(1, 5), rng.randint(1, 4)
    dim = rng.choice([3, 4, 8, 12, 16, 20, 32, 64])
    page = rng.choice([1, 2, 3, 4, 7, 8, 16, 16, 32, 64])
    planes = rng.randint(1, 5)
    lengths = [rng.randint(1, 3 * page + 3) for _ in range(rng.randint(1, 4))]
    blocks = sum(-(-n // page) for n in lengths) * planes + rng.randint(0, 5)
    return rng, kind, (layers, heads, dim, blocks, page, planes), lengths


@pytest.mark.parametrize("seed", range(48))
def test_random_geometry(seed):
    from vllm_rlt_b200.kernels import kv_handoff as k

    rng, kind, shape, lengths = draw(seed)
    layers, _, _, _, page, planes = shape
    nrng = np.random.default_rng(seed)
    mode = rng.choice([ho.MODE_ALL_PLANES, ho.MODE_DEDUP, ho.MODE_EXIT_ONLY])
    dst_planes = 1 if mode == ho.MODE_EXIT_ONLY else planes
    variant = rng.choice(VARIANTS)
    P = oracle_pool(kind, shape)
    D = sentinel_destination(kind, shape, planes=dst_planes)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    D.shuffle_free_list(rng)
    reqs, exits = [], []
    for i, n in enumerate(lengths):
        assert P.allocate(f"r{i}", n) and D.allocate(f"r{i}", n)
        start = rng.choice([0, rng.randrange(n)])
        reqs.append((f"r{i}", start, rng.randint(start + 1, n)))
        e = [rng.randrange(planes) for _ in range(n)]
        exits.append(e)
        if mode != ho.MODE_ALL_PLANES:
            for pos in range(n):
                P.finalize_token(f"r{i}", pos, e[pos])
    use_exits = exits if mode != ho.MODE_ALL_PLANES else None
    l0 = rng.randrange(layers)
    l1 = rng.randint(l0 + 1, layers)
    p0 = rng.randrange(dst_planes)
    p1 = rng.randint(p0 + 1, dst_planes)
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch(
        [P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
        [(s, e) for _, s, e in reqs], block_size=page, exit_planes=use_exits,
        src_blocks=P.num_blocks, dst_blocks=D.num_blocks,
    )
    status = k.new_status()

    # 1. a (layer, plane) slice of the direct handoff
    k.kv_handoff(gp.view(), gd.view(), batch, mode=mode, layer_begin=l0, layer_end=l1, plane_begin=p0, plane_end=p1,
                 status=status, variant=variant)
    for i, (r, s, e) in enumerate(reqs):
        st, dt = P.plane_block_tables(r), D.plane_block_tables(r)
        for plane in range(p0, p1):
            for t in range(s, e):
                sp = ho.source_plane(mode, plane, exits[i][t] if use_exits else planes - 1)
                for a, b in zip(P.tensors(), D.tensors()):
                    b.data[dt[plane][t // page], l0:l1, t % page] = a.data[st[sp][t // page], l0:l1, t % page]
    k.raise_for_status(status)
    assert_pools_equal(gd, D)

    # 2. the rest of the handoff in one launch: the destination now equals the full handoff
    k.kv_handoff(gp.view(), gd.view(), batch, mode=mode, status=status, variant=variant)
    for i, (r, s, e) in enumerate(reqs):
        ho.handoff_rows(P, D, P.plane_block_tables(r), D.plane_block_tables(r), s, e, mode=mode,
                        exit_planes=exits[i] if use_exits else None)
    k.raise_for_status(status)
    assert_pools_equal(gd, D)

    # 3. pack (all / exit-only / dedup wire) equals the oracle's image; scatter of it reproduces the destination
    wire_planes = 1 if mode == ho.MODE_EXIT_ONLY else planes
    want = np.concatenate([
        ho.pack_rows(P, P.plane_block_tables(r), s, e, mode=mode, exit_planes=exits[i] if use_exits else None,
                     layer_begin=l0, layer_end=l1)
        for i, (r, s, e) in enumerate(reqs)])
    full = k.packed_bytes(gp.view(), batch.total_tokens, wire_planes, l1 - l0)
    packed = torch.full((max(full, 16),), 0x5A, dtype=torch.uint8, device="cuda")
    ws = k.dedup_workspace(batch, planes) if mode == ho.MODE_DEDUP else None
    k.kv_pack(gp.view(), batch, packed, mode=mode, layer_begin=l0, layer_end=l1, status=status, workspace=ws, variant=variant)
    k.raise_for_status(status)
    got = packed.cpu().numpy()
    assert np.array_equal(got[: want.size], want)
    assert (got[want.size :] == 0x5A).all()
    D3 = sentinel_destination(kind, shape, planes=dst_planes)
    D3._free, D3.tables = [], dict(D.tables)
    gd3 = GpuPool(D3)
    ws2 = k.dedup_workspace(batch, planes) if mode == ho.MODE_DEDUP else None
    k.kv_scatter(packed[: max(want.size, 16)], gd3.view(), batch, mode=mode if mode == ho.MODE_DEDUP else 0,
                 layer_begin=l0, layer_end=l1, status=status, workspace=ws2, variant=variant)
    k.raise_for_status(status)
    for i, (r, s, e) in enumerate(reqs):
        ho.handoff_rows(P, D3, P.plane_block_tables(r), D3.plane_block_tables(r), s, e, mode=mode,
                        exit_planes=exits[i] if use_exits else None, layer_begin=l0, layer_end=l1)
    assert_pools_equal(gd3, D3)
