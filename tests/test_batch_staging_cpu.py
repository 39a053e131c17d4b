"""The host side of ``HandoffBatch``: what is staged for the device, checked without a GPU.

The pinned-buffer pool and the device copy are replaced by plain CPU tensors; the staged bytes are then compared with
arrays built the slow, obvious way (nested loops), and the planner's error messages with the reference's.
"""

import contextlib
import random

import numpy as np
import pytest
import torch


@pytest.fixture
def kh(monkeypatch):
    from vllm_rlt_b200.kernels import kv_handoff

    class Staging:
        def __init__(self, size):
            self.buffer = torch.zeros(size, dtype=torch.uint8)

        def release(self):
            pass

    class Pool:
        def acquire(self, size):
            return Staging(size)

    monkeypatch.setattr(kv_handoff, "_PINNED", Pool())
    monkeypatch.setattr(torch.cuda, "device", lambda d: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "stream", lambda s: contextlib.nullcontext())
    monkeypatch.setattr(torch.cuda, "current_stream", lambda d=None: None)
    return kv_handoff


def staged(batch, name, dtype, count):
    at = batch._ptr[name] - batch._dev.data_ptr()
    return batch._dev.numpy()[at : at + count * np.dtype(dtype).itemsize].view(dtype)


def draw(seed, as_arrays):
    rng = random.Random(seed)
    page = rng.choice([1, 4, 16])
    planes_s, planes_d = rng.randint(1, 4), rng.randint(1, 4)
    n = rng.randint(1, 9)
    src, dst, ranges, exits = [], [], [], []
    for _ in range(n):
        tokens = rng.randint(1, 6 * page)
        pages = -(-tokens // page) + rng.randint(0, 2)  # tables may be longer than the range needs
        mk = (lambda v: np.asarray(v, np.int32)) if as_arrays else list
        src.append([mk([rng.randrange(500) for _ in range(pages)]) for _ in range(planes_s)])
        dst.append([mk([rng.randrange(500) for _ in range(pages)]) for _ in range(planes_d)])
        start = rng.randrange(tokens)
        ranges.append((start, rng.randint(start + 1, tokens)))
        exits.append(mk([rng.randrange(planes_s) for _ in range(tokens + rng.randint(0, 3))]))
    return page, src, dst, ranges, exits


@pytest.mark.parametrize("seed", range(24))
@pytest.mark.parametrize("as_arrays", [False, True])
def test_staged_bytes_are_the_padded_tables_ranges_and_exit_planes(kh, seed, as_arrays):
    page, src, dst, ranges, exits = draw(seed, as_arrays)
    with_exits = seed % 3 != 0
    b = kh.HandoffBatch(src, dst, ranges, block_size=page, exit_planes=exits if with_exits else None,
                        src_blocks=500, dst_blocks=500, device="cpu")
    n = len(ranges)
    width = max(len(t[0]) for t in src + dst)
    assert (b.num_requests, b.table_width, b.total_tokens) == (n, width, sum(e - s for s, e in ranges))
    assert b.ranges == [(int(s), int(e)) for s, e in ranges] and b.has_exit == with_exits
    for name, tables in (("src_tables", src), ("dst_tables", dst)):
        planes = len(tables[0])
        got = staged(b, name, np.int32, n * planes * width).reshape(n, planes, width)
        for r in range(n):
            for p in range(planes):
                row = list(tables[r][p])
                assert got[r, p, : len(row)].tolist() == [int(x) for x in row]
                assert not got[r, p, len(row) :].any()
    assert staged(b, "tok_begin", np.int32, n).tolist() == [s for s, _ in ranges]
    assert staged(b, "tok_end", np.int32, n).tolist() == [e for _, e in ranges]
    if with_exits:
        offsets = staged(b, "exit_offsets", np.int64, n).tolist()
        flat = staged(b, "exit_planes", np.int32, sum(len(e) for e in exits))
        at = 0
        for r, e in enumerate(exits):
            assert offsets[r] == at
            assert flat[at : at + len(e)].tolist() == [int(x) for x in e]
            at += len(e)
    else:
        assert "exit_planes" not in b._ptr and "exit_offsets" not in b._ptr
    assert all(at % 16 == 0 for at in (p - b._dev.data_ptr() for p in b._ptr.values()))


def test_host_checks_raise_what_the_reference_planner_raises(kh):
    t = [[[0, 1, 2]]]
    mk = lambda *a, **k: kh.HandoffBatch(*a, block_size=4, device="cpu", **k)  # noqa: E731
    for bad in [(-1, 3), (3, 3), (5, 2)]:
        with pytest.raises(ValueError, match="invalid KV range"):
            mk(t, t, [bad])
    with pytest.raises(ValueError, match="KV range exceeds allocation"):
        mk(t, t, [(0, 13)])
    with pytest.raises(ValueError, match="planes of one request must have tables of equal length"):
        mk([[[0, 1, 2], [0, 1, 2, 3]]], None, [(0, 8)])
    with pytest.raises(ValueError, match="same number of planes"):
        mk([[[0, 1, 2]], [[0, 1], [2, 3]]], None, [(0, 8), (0, 8)])
    with pytest.raises(ValueError, match="at least one request"):
        mk(t, t, [])
    # a block id outside the pool only matters on pages the range touches
    with pytest.raises(ValueError, match="physical block outside registered pool"):
        mk([[[0, 99, 2]]], None, [(0, 12)], src_blocks=16)
    with pytest.raises(ValueError, match="physical block outside registered pool"):
        mk([[[0, -1, 2]]], None, [(0, 12)])
    mk([[[0, 99, 2]]], None, [(0, 4)], src_blocks=16)
    mk([[[0, 99, 2]]], None, [(8, 12)], src_blocks=16)
    with pytest.raises(ValueError, match="exit planes must cover"):
        mk(t, t, [(0, 12)], exit_planes=[[0, 1]])
    with pytest.raises(ValueError, match="one exit-plane array per request"):
        mk(t, t, [(0, 12)], exit_planes=[[0] * 12, [1] * 3])
