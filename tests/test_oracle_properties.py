"""Size-independent properties of the planner restatement, on generated inputs.

These hold for the reference's ``kv_segments`` / ``coalesce_segments`` / ``partition_segments``
(vllm_rlt/pd/transport.py:29-112) by construction; the golden fixtures pin the exact lists, the properties
cover the input space the fixtures do not enumerate.
"""

import random

from hypothesis import given, settings
from hypothesis import strategies as st

from oracle import handoff_oracle as ho


def byte_map(pairs):
    """Expand ``(source address, target address, bytes)`` triples into the ordered list of byte moves."""
    return [(s + i, d + i) for s, d, n in pairs for i in range(n)]


@st.composite
def segment_lists(draw):
    count = draw(st.integers(1, 12))
    source, target = [], []
    s_at, d_at = 1000, 9000
    for _ in range(count):
        n = draw(st.integers(1, 40))
        # sometimes adjacent on one side, both sides or neither; sometimes another device
        s_at += draw(st.sampled_from([0, 0, 3, 64]))
        d_at += draw(st.sampled_from([0, 0, 5, 128]))
        source.append((s_at, n, draw(st.sampled_from([0, 0, 0, 2]))))
        target.append((d_at, n, 1))
        s_at += n
        d_at += n
    return source, target


@settings(max_examples=150, deadline=None)
@given(segment_lists(), st.integers(1, 97), st.integers(1, 6))
def test_partition_moves_every_byte_once_in_order_and_obeys_both_limits(lists, byte_limit, descriptor_limit):
    source, target = lists
    want = byte_map((s, d, n) for (s, n, _), (d, _, _) in zip(source, target))
    got = []
    chunks = list(ho.partition_segments(source, target, byte_limit, descriptor_limit))
    for local, remote, size in chunks:
        assert len(local) == len(remote) <= descriptor_limit
        assert size == sum(n for _, n, _ in local) == sum(n for _, n, _ in remote) <= byte_limit
        assert all(n > 0 for _, n, _ in local)
        got += byte_map((s, d, n) for (s, n, _), (d, _, _) in zip(local, remote))
    assert got == want
    # every chunk but the last is full on one of the two limits
    for local, _, size in chunks[:-1]:
        assert size == byte_limit or len(local) == descriptor_limit


@settings(max_examples=150, deadline=None)
@given(segment_lists())
def test_coalesce_keeps_the_byte_moves_and_never_merges_across_a_gap_or_a_device(lists):
    source, target = lists
    merged = list(ho.coalesce_segments(source, target))
    assert byte_map((s, d, n) for s, d, n, _, _ in merged) == byte_map(
        (s, d, n) for (s, n, _), (d, _, _) in zip(source, target))
    for a, b in zip(merged, merged[1:]):
        adjacent = a[0] + a[2] == b[0] and a[1] + a[2] == b[1] and a[3] == b[3] and a[4] == b[4]
        assert not adjacent  # anything mergeable was merged


@st.composite
def pools_and_ranges(draw):
    page = draw(st.sampled_from([1, 2, 4, 16]))
    layers = draw(st.integers(1, 3))
    planes = draw(st.integers(1, 4))
    tokens = draw(st.integers(1, 5 * page))
    fp8 = draw(st.booleans())
    pages = -(-tokens // page)
    blocks = pages * planes + draw(st.integers(0, 3))
    start = draw(st.integers(0, tokens - 1))
    end = draw(st.integers(start + 1, tokens))
    seed = draw(st.integers(0, 1000))
    return page, layers, planes, tokens, fp8, blocks, start, end, seed


@settings(max_examples=120, deadline=None)
@given(pools_and_ranges())
def test_segments_cover_exactly_the_rows_of_the_range(case):
    page, layers, planes, tokens, fp8, blocks, start, end, seed = case
    pool = ho.OraclePool(layers, 2, 4, blocks, page, planes, element=1 if fp8 else 2, fp8=fp8)
    pool.shuffle_free_list(random.Random(seed))
    assert pool.allocate("r", tokens)
    tables = pool.plane_block_tables("r")
    segments = list(ho.kv_segments(pool.info(), tables, start, end))
    assert sum(n for _, n, _ in segments) == ho.payload_bytes(pool, end - start, planes)
    # the bytes named are exactly the (plane, layer, token) rows of the range, each once
    want = set()
    for t in pool.tensors():
        row = t.data.shape[-1]
        for table in tables:
            for tok in range(start, end):
                for layer in range(layers):
                    origin = t.base + ((table[tok // page] * layers + layer) * page + tok % page) * row
                    want.update(range(origin, origin + row))
    got = [a + i for a, n, _ in segments for i in range(n)]
    assert len(got) == len(set(got)) and set(got) == want
    # the same walk on another pool yields segments of the same sizes in the same order: what lets source and
    # target lists be zipped
    other = ho.OraclePool(layers, 2, 4, blocks, page, planes, element=1 if fp8 else 2, fp8=fp8, base=1 << 40, device=1)
    other.shuffle_free_list(random.Random(seed + 1))
    assert other.allocate("r", tokens)
    mirror = list(ho.kv_segments(other.info(), other.plane_block_tables("r"), start, end))
    assert [n for _, n, _ in mirror] == [n for _, n, _ in segments]


# ----------------------------------------------------------------------------- differential check against the reference

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REFERENCE = Path(os.environ.get("VLLM_RLT_REFERENCE", str(ROOT.parent / "reference")))


def seeded_planner_cases(count=60):
    """Plain-data planner inputs: pool geometry as an ``info`` dict, tables, a range, and partition limits."""
    cases = []
    for seed in range(count):
        rng = random.Random(seed)
        page = rng.choice([1, 2, 4, 16])
        layers, planes = rng.randint(1, 3), rng.randint(1, 4)
        tokens = rng.randint(1, 5 * page)
        pages = -(-tokens // page)
        blocks = pages * planes + rng.randint(0, 3)
        row = rng.choice([8, 24, 64])
        infos, tables = [], []
        for side in range(2):
            order = list(range(blocks))
            rng.shuffle(order)
            tables.append([order[p * pages : (p + 1) * pages] for p in range(planes)])
            base = (side + 1) << 32
            info = dict(key_ptr=base, value_ptr=base + (1 << 28), block_bytes=layers * page * row, layer_bytes=page * row,
                        token_bytes=row, device=side, num_blocks=blocks, block_size=page, num_layers=layers, scale_region=None)
            if rng.random() < 0.5:
                info["scale_region"] = dict(key_ptr=base + (2 << 28), value_ptr=base + (3 << 28), block_bytes=layers * page * 4,
                                            layer_bytes=page * 4, token_bytes=4)
            infos.append(info)
        if infos[0]["scale_region"] is None or infos[1]["scale_region"] is None:
            infos[0]["scale_region"] = infos[1]["scale_region"] = None
        start = rng.randrange(tokens)
        cases.append(dict(infos=infos, tables=tables, start=start, end=rng.randint(start + 1, tokens),
                          byte_limit=rng.choice([64, 333, 4096, 1 << 20]), descriptor_limit=rng.choice([1, 3, 256])))
    return cases


def run_planner(module, cases):
    out = []
    for c in cases:
        source = list(module.kv_segments(c["infos"][0], c["tables"][0], c["start"], c["end"]))
        target = list(module.kv_segments(c["infos"][1], c["tables"][1], c["start"], c["end"]))
        chunks = [[list(map(list, local)), list(map(list, remote)), size]
                  for local, remote, size in module.partition_segments(source, target, c["byte_limit"], c["descriptor_limit"])]
        out.append(dict(source=list(map(list, source)), chunks=chunks))
    return out


@pytest.mark.skipif(not (REFERENCE / "vllm_rlt" / "pd" / "transport.py").is_file(), reason="reference checkout not present")
def test_planner_restatement_equals_the_reference_on_seeded_inputs():
    """Runs the reference's own ``kv_segments`` and ``partition_segments`` in a child process on 60 seeded inputs
    and compares every segment and every chunk with the restatement's."""
    code = ("import json, sys; sys.path[:0] = [%r, %r]; from tests.test_oracle_properties import seeded_planner_cases, run_planner; "
            "from vllm_rlt.pd import transport; print(json.dumps(run_planner(transport, seeded_planner_cases())))"
            % (str(ROOT), str(REFERENCE)))
    done = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=str(ROOT))
    assert done.returncode == 0, done.stderr[-2000:]
    theirs = json.loads(done.stdout.strip().splitlines()[-1])
    ours = json.loads(json.dumps(run_planner(ho, seeded_planner_cases())))
    assert ours == theirs
