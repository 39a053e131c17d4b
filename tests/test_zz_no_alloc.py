"""The allocation-free dedup pack (``rlt_kv_pack_dedup_static``) against the ordinary entry point.

Some callers cannot allocate at all once they are serving: a stage worker that gave every free byte
of HBM to its KV pool at start-up would see a later ``cudaMalloc`` for the wire-plan scratch fail, or
stall the device mid-serving. For them the library keeps the plan in an array of its own image. This
test calls that entry point through the C ABI twice in a row, on two different batches, and requires
the packed bytes to equal those of ``rlt_kv_pack`` with a caller-provided workspace and the CPU oracle's
dedup wire image, bit for bit (the tolerance of every handoff test: none). It also checks the claim in
the entry point's name: the device's free memory, as the driver reports it, is the same before and
after a call. The file name sorts last so that a run that stops at the first failure has already run
everything else.
"""

import ctypes as C
import random

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def make_case(seed, lengths, planes=4, page=16):
    from oracle import handoff_oracle as ho
    from tests.gpu_support import GpuPool

    rng, nrng = random.Random(seed), np.random.default_rng(seed)
    P = ho.OraclePool(3, 4, 32, 64, page, planes, element=2)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    tables, ranges, exits = [], [], []
    for i, n in enumerate(lengths):
        assert P.allocate(f"r{i}", n)
        tables.append(P.plane_block_tables(f"r{i}"))
        start = rng.randrange(n)
        ranges.append((start, rng.randint(start + 1, n)))
        exits.append([rng.randrange(planes) for _ in range(n)])
    return GpuPool(P), tables, ranges, exits, P


def test_static_scratch_pack_equals_the_workspace_pack_on_two_calls_in_a_row():
    from vllm_rlt_b200 import _lib
    from vllm_rlt_b200.kernels import kv_handoff as kh

    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    from oracle import handoff_oracle as ho

    for call, (seed, lengths) in enumerate(((1, [40, 16, 23]), (2, [64, 5]))):
        pool, tables, ranges, exits, P = make_case(seed, lengths)
        view = pool.view()
        batch = kh.HandoffBatch(tables, None, ranges, block_size=16, exit_planes=exits)
        size = kh.packed_bytes(view, batch.total_tokens, 4)
        want = torch.full((size,), 0x5A, dtype=torch.uint8, device="cuda")
        got = torch.full((size,), 0x5A, dtype=torch.uint8, device="cuda")
        status = kh.new_status()
        workspace = kh.dedup_workspace(batch, 4)
        kh.kv_pack(view, batch, want, mode=kh.MODE_DEDUP, status=status, workspace=workspace)
        s, b = view.as_struct(), batch.as_struct()
        o = _lib.RltOptions(kh.MODE_DEDUP, 0, 0, 0, status.data_ptr(), 0, 0, None, 0)
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # cudaMemGetInfo: what the driver has left, not torch's cache
        rc = lib.rlt_kv_pack_dedup_static(C.byref(s), C.byref(b), C.byref(o), got.data_ptr(), size, stream)
        assert rc == _lib.RLT_OK, lib.rlt_error_string(rc)
        torch.cuda.synchronize()
        if call > 0:  # the first call on a device may place the library's image, array included; later ones take nothing
            assert torch.cuda.mem_get_info()[0] == free_before
        kh.raise_for_status(status)
        oracle = np.concatenate([ho.pack_rows(P, tables[i], lo, hi, mode=ho.MODE_DEDUP, exit_planes=exits[i])
                                 for i, (lo, hi) in enumerate(ranges)])
        image = got.cpu().numpy()
        assert np.array_equal(image[: oracle.size], oracle) and (image[oracle.size :] == 0x5A).all()
        pairs = sum(exits[i][t] + 1 for i, (lo, hi) in enumerate(ranges) for t in range(lo, hi))
        assert kh.dedup_wire_tokens(workspace) == pairs
        assert torch.equal(got, want)
        assert int((got != 0x5A).sum()) > 0


def test_static_scratch_rejects_batches_beyond_its_size_and_other_modes():
    from vllm_rlt_b200 import _lib
    from vllm_rlt_b200.kernels import kv_handoff as kh

    lib = _lib.load()
    limit = lib.rlt_kv_static_plan_entries()
    assert limit == 1 << 20
    pool, tables, ranges, exits, _ = make_case(3, [20])
    view = pool.view()
    batch = kh.HandoffBatch(tables, None, ranges, block_size=16, exit_planes=exits)
    out = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    s, b = view.as_struct(), batch.as_struct()
    o = _lib.RltOptions(kh.MODE_DEDUP, 0, 0, 0, None, 0, 0, None, 0)
    b.table_width = limit // (b.num_requests * 4) + 1  # one entry too many
    assert lib.rlt_kv_pack_dedup_static(C.byref(s), C.byref(b), C.byref(o), out.data_ptr(), out.numel(), None) == _lib.RLT_E_LIMIT
    b = batch.as_struct()
    o.mode = kh.MODE_ALL_PLANES
    assert lib.rlt_kv_pack_dedup_static(C.byref(s), C.byref(b), C.byref(o), out.data_ptr(), out.numel(), None) == _lib.RLT_E_INVALID
