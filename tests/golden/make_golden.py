"""Generate the golden fixtures in this folder by running the reference itself on CPU.

Run once, in a container where the reference checkout is importable:

    python tests/golden/make_golden.py --reference <vllm-rlt checkout>

The fixtures (``*.json`` and ``*.npz`` beside this file) are committed; the
tests never import the reference. Every fixture is produced by reference code
only: ``KVCacheManager`` for pools, tables, writes and ``finalize_token``;
``kv_segments`` / ``partition_segments`` for the plan; a byte copy over the
pools' ``uint8`` views for the write itself (the one correct result of a WRITE
of those descriptors).
"""

import argparse
import json
import os
import random
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent


def as_bytes(t):
    import torch

    return t.detach().contiguous().view(torch.uint8).numpy().copy()


def pool_tensors(cache):
    out = {"key": cache.key_cache, "value": cache.value_cache}
    if cache.key_scale is not None:
        out["key_scale"] = cache.key_scale
        out["value_scale"] = cache.value_scale
    return out


def region_info(cache, device=0):
    from vllm_rlt.pd.transport import _kv_region

    scale_region = None
    if cache.key_scale is not None and cache.fp8_scale is None:
        scale_region = _kv_region(cache.key_scale, cache.value_scale)
    return dict(
        **_kv_region(cache.key_cache, cache.value_cache),
        device=device,
        num_blocks=cache.num_blocks,
        block_size=cache.block_size,
        num_layers=cache.num_layers,
        depths=cache.storage_depths,
        scale_region=scale_region,
    )


def name_segments(cache, segments):
    """(address, n, dev) -> (tensor name, byte offset, n) so fixtures hold no process addresses."""
    spans = []
    for name, t in pool_tensors(cache).items():
        spans.append((t.data_ptr(), t.data_ptr() + t.numel() * t.element_size(), name))
    out = []
    for address, n, _ in segments:
        for lo, hi, name in spans:
            if lo <= address and address + n <= hi:
                out.append([name, address - lo, n])
                break
        else:
            raise AssertionError("segment outside pool")
    return out


def geometry(cache):
    info = region_info(cache)
    g = {k: info[k] for k in ("block_bytes", "layer_bytes", "token_bytes")}
    if info["scale_region"] is not None:
        g["scale"] = {k: info["scale_region"][k] for k in ("block_bytes", "layer_bytes", "token_bytes")}
    return g


def make_cache(kind, *shape, **kw):
    import torch
    from vllm_rlt.core.kv_cache_manager import KVCacheManager

    if kind == "bf16":
        return KVCacheManager(*shape, dtype=torch.bfloat16, **kw)
    if kind == "f32":
        return KVCacheManager(*shape, **kw)
    if kind == "fp8":
        return KVCacheManager(*shape, dtype=torch.bfloat16, kv_cache_dtype="fp8_e4m3", **kw)
    if kind == "fp8_fixed":
        return KVCacheManager(*shape, dtype=torch.bfloat16, kv_cache_dtype="fp8_e4m3", fp8_scale=0.5, **kw)
    raise ValueError(kind)


def randomize(cache, gen):
    """Random payload written through uint8 views (FP8 codes avoid NaN encodings)."""
    import torch

    for name, t in pool_tensors(cache).items():
        raw = t.view(torch.uint8)
        if name.endswith("scale"):
            if cache.fp8_scale is None:
                t.copy_(torch.empty(t.shape).uniform_(0.01, 0.1, generator=gen))
            continue
        data = torch.randint(0, 256, raw.shape, dtype=torch.uint8, generator=gen)
        if cache.kv_cache_dtype == "fp8_e4m3":
            data[(data & 0x7F) == 0x7F] = 0x3C
        raw.copy_(data)


def byte_copy(src_cache, dst_cache, local, remote):
    import torch

    def locate(cache, address, n):
        for t in pool_tensors(cache).values():
            lo = t.data_ptr()
            if lo <= address and address + n <= lo + t.numel() * t.element_size():
                return t.view(torch.uint8).reshape(-1)[address - lo : address - lo + n]
        raise AssertionError

    for (s, n, _), (d, m, _) in zip(local, remote, strict=True):
        assert n == m
        locate(dst_cache, d, n).copy_(locate(src_cache, s, n))


# ------------------------------------------------------------------------------ cases


def segment_cases():
    """Planner output for the shapes the reference's own tests pin (tests/test_pd.py:56-87)."""
    from vllm_rlt.pd.transport import kv_segments, partition_segments

    cases = []
    specs = [
        ("f32", (3, 2, 8, 24, 4, 4), 9, 2, 9, 333, 3),
        ("fp8", (3, 2, 8, 24, 4, 4), 9, 2, 9, 333, 3),
        ("fp8_fixed", (3, 2, 8, 24, 4, 4), 9, 2, 9, 333, 3),
        ("bf16", (3, 2, 8, 24, 4, 4), 9, 2, 9, 10**9, 256),
        ("bf16", (3, 2, 8, 24, 4, 4), 9, 0, 8, 10**9, 256),
        ("bf16", (2, 4, 16, 64, 16, 2), 100, 17, 95, 4096, 5),
        ("fp8", (2, 4, 16, 64, 16, 2), 100, 0, 100, 10**9, 256),
    ]
    for kind, shape, tokens, start, end, byte_limit, desc_limit in specs:
        cache = make_cache(kind, *shape)
        assert cache.allocate("a", tokens)
        tables = cache.plane_block_tables("a")
        info = region_info(cache)
        segs = list(kv_segments(info, tables, start, end))
        parts = list(partition_segments(segs, segs, byte_limit, desc_limit))
        cases.append(
            dict(
                kind=kind,
                shape=list(shape),
                tokens=tokens,
                start=start,
                end=end,
                byte_limit=byte_limit,
                descriptor_limit=desc_limit,
                tables=[list(t) for t in tables],
                geometry=geometry(cache),
                segments=name_segments(cache, segs),
                partition=[[name_segments(cache, local), n] for local, _, n in parts],
            )
        )
    return cases


def partition_cases():
    """Coalesce/partition known answers, the inputs of tests/test_pd.py:97-115 run through the reference."""
    from vllm_rlt.pd.transport import partition_segments

    source = [(1000, 100, 0), (1100, 100, 0), (1200, 100, 0), (5000, 50, 0)]
    target = [(7000, 100, 1), (7100, 100, 1), (9000, 100, 1), (9100, 50, 1)]
    out = []
    for byte_limit, desc_limit in [(10**6, 256), (120, 256), (10**6, 2), (100, 1), (75, 3)]:
        parts = list(partition_segments(source, target, byte_limit, desc_limit))
        out.append(
            dict(
                source=source,
                target=target,
                byte_limit=byte_limit,
                descriptor_limit=desc_limit,
                parts=[[list(map(list, l)), list(map(list, r)), n] for l, r, n in parts],
            )
        )
    rng = random.Random(7)
    for _ in range(6):
        source, target, s, d = [], [], 10_000, 90_000
        for _ in range(rng.randrange(1, 12)):
            n = rng.choice([16, 64, 100, 384])
            s += rng.choice([0, 0, 32])
            d += rng.choice([0, 0, 48])
            source.append((s, n, 0))
            target.append((d, n, 1))
            s += n
            d += n
        byte_limit, desc_limit = rng.choice([64, 200, 10**6]), rng.choice([1, 2, 256])
        parts = list(partition_segments(source, target, byte_limit, desc_limit))
        out.append(
            dict(
                source=source,
                target=target,
                byte_limit=byte_limit,
                descriptor_limit=desc_limit,
                parts=[[list(map(list, l)), list(map(list, r)), n] for l, r, n in parts],
            )
        )
    bad = None
    try:
        list(partition_segments(source, target[:-1], 10**6, 256))
    except ValueError as exc:
        bad = str(exc)
    return dict(cases=out, length_mismatch_error=bad)


def handoff_cases(out_dir):
    """Two independent pools with shuffled free lists; reference plan + byte copy; full pools saved."""
    import torch
    from vllm_rlt.pd.transport import kv_segments, partition_segments

    index = []
    specs = [
        ("bf16", (3, 2, 8, 64, 4, 4), [(9, 2, 9), (16, 0, 16), (5, 0, 5)], 333, 3),
        ("fp8", (3, 2, 8, 64, 4, 4), [(9, 2, 9), (16, 0, 16), (7, 3, 7)], 10**6, 256),
        ("fp8_fixed", (3, 2, 8, 64, 4, 4), [(9, 2, 9), (12, 0, 12)], 10**6, 256),
        ("bf16", (4, 2, 16, 96, 16, 4), [(100, 0, 100), (33, 16, 33), (64, 0, 64), (17, 5, 16)], 8192, 7),
        ("bf16", (2, 5, 24, 40, 8, 1), [(30, 0, 30), (9, 1, 9)], 10**6, 256),
    ]
    for n, (kind, shape, requests, byte_limit, desc_limit) in enumerate(specs):
        gen = torch.Generator().manual_seed(1000 + n)
        P, D = make_cache(kind, *shape), make_cache(kind, *shape)
        random.Random(2000 + n).shuffle(P._free_blocks)
        random.Random(3000 + n).shuffle(D._free_blocks)
        randomize(P, gen)
        for tname, t in pool_tensors(D).items():
            if tname.endswith("scale") and D.fp8_scale is not None:
                continue  # a fixed-scale pool keeps its constant scales; they do not travel
            t.view(torch.uint8).fill_(0xA5)
        d_before = {k: as_bytes(v) for k, v in pool_tensors(D).items()}
        meta = []
        for i, (tokens, start, end) in enumerate(requests):
            rid = f"r{i}"
            assert P.allocate(rid, tokens) and D.allocate(rid, tokens)
            st, dt = P.plane_block_tables(rid), D.plane_block_tables(rid)
            source = list(kv_segments(region_info(P, 0), st, start, end))
            target = list(kv_segments(region_info(D, 1), dt, start, end))
            moved = 0
            for local, remote, size in partition_segments(source, target, byte_limit, desc_limit):
                byte_copy(P, D, local, remote)
                moved += size
            meta.append(
                dict(
                    tokens=tokens,
                    start=start,
                    end=end,
                    src_tables=[list(t) for t in st],
                    dst_tables=[list(t) for t in dt],
                    bytes=moved,
                    packed_offset=None,
                )
            )
        # Wire image: concatenation of the source segments, request by request.
        packed = []
        for m in meta:
            st = [tuple(t) for t in m["src_tables"]]
            m["packed_offset"] = int(sum(len(p) for p in packed))
            for address, size, _ in kv_segments(region_info(P, 0), st, m["start"], m["end"]):
                for t in pool_tensors(P).values():
                    lo = t.data_ptr()
                    if lo <= address and address + size <= lo + t.numel() * t.element_size():
                        packed.append(
                            t.view(torch.uint8).reshape(-1)[address - lo : address - lo + size].numpy().copy()
                        )
        name = f"handoff_{n}_{kind}"
        arrays = {f"src_{k}": as_bytes(v) for k, v in pool_tensors(P).items()}
        arrays.update({f"dst_before_{k}": v for k, v in d_before.items()})
        arrays.update({f"dst_after_{k}": as_bytes(v) for k, v in pool_tensors(D).items()})
        arrays["packed"] = np.concatenate(packed)
        np.savez_compressed(out_dir / f"{name}.npz", **arrays)
        index.append(
            dict(
                name=name,
                kind=kind,
                shape=list(shape),
                byte_limit=byte_limit,
                descriptor_limit=desc_limit,
                requests=meta,
                free_src_seed=2000 + n,
                free_dst_seed=3000 + n,
            )
        )
    return index


def finalize_cases(out_dir):
    """``write`` every executed plane, ``finalize_token`` at a per-token exit plane, then a full handoff.

    Saves the source pool before and after finalize and the destination after
    the reference all-planes handoff: the dedup and exit-only modes are checked
    against these.
    """
    import torch
    from vllm_rlt.pd.transport import kv_segments, partition_segments

    index = []
    specs = [
        ("bf16", (3, 2, 8, 64, 4, 4), None, [11, 6]),
        ("fp8", (3, 2, 8, 64, 4, 4), None, [9, 8]),
        ("fp8_fixed", (2, 2, 8, 64, 4, 3), None, [7]),
        ("bf16", (6, 3, 8, 96, 4, 4), (2, 3), [10, 5]),
    ]
    for n, (kind, shape, recurrent, lengths) in enumerate(specs):
        gen = torch.Generator().manual_seed(4000 + n)
        rng = random.Random(5000 + n)
        kw = {} if recurrent is None else dict(recurrent_layers=recurrent)
        P, D = make_cache(kind, *shape, **kw), make_cache(kind, *shape, **kw)
        rng.shuffle(P._free_blocks)
        rng.shuffle(D._free_blocks)
        layers, heads, dim, _, _, planes = shape
        for t in pool_tensors(D).values():
            t.view(torch.uint8).fill_(0xA5)
        if D.fp8_scale is not None:
            D.key_scale.fill_(D.fp8_scale)
            D.value_scale.fill_(D.fp8_scale)
        for t in pool_tensors(P).values():
            t.view(torch.uint8).fill_(0x11)
        if P.fp8_scale is not None:
            P.key_scale.fill_(P.fp8_scale)
            P.value_scale.fill_(P.fp8_scale)
        meta = []
        exits = []
        for i, tokens in enumerate(lengths):
            rid = f"r{i}"
            assert P.allocate(rid, tokens) and D.allocate(rid, tokens)
            e = [rng.randrange(planes) for _ in range(tokens)]
            exits.append(e)
            for pos in range(tokens):
                for depth in range(e[pos] + 1):
                    for layer in range(layers):
                        k = torch.randn(1, heads, dim, generator=gen).to(torch.bfloat16)
                        v = torch.randn(1, heads, dim, generator=gen).to(torch.bfloat16)
                        P.write(layer, [rid], [depth], [pos], k, v)
        before = {f"src_before_{k}": as_bytes(v) for k, v in pool_tensors(P).items()}
        for i, tokens in enumerate(lengths):
            for pos in range(tokens):
                P.finalize_token(f"r{i}", pos, exits[i][pos])
        for i, tokens in enumerate(lengths):
            rid = f"r{i}"
            st, dt = P.plane_block_tables(rid), D.plane_block_tables(rid)
            source = list(kv_segments(region_info(P, 0), st, 0, tokens))
            target = list(kv_segments(region_info(D, 1), dt, 0, tokens))
            for local, remote, _ in partition_segments(source, target, 10**9, 256):
                byte_copy(P, D, local, remote)
            meta.append(
                dict(
                    tokens=tokens,
                    exit_planes=exits[i],
                    src_tables=[list(t) for t in st],
                    dst_tables=[list(t) for t in dt],
                )
            )
        name = f"finalize_{n}_{kind}"
        arrays = dict(before)
        arrays.update({f"src_after_{k}": as_bytes(v) for k, v in pool_tensors(P).items()})
        arrays.update({f"dst_after_{k}": as_bytes(v) for k, v in pool_tensors(D).items()})
        np.savez_compressed(out_dir / f"{name}.npz", **arrays)
        index.append(
            dict(
                name=name,
                kind=kind,
                shape=list(shape),
                recurrent_layers=None if recurrent is None else list(recurrent),
                requests=meta,
            )
        )
    return index


def allocation_cases():
    """Block-table order of ``allocate`` / ``free`` (vllm_rlt/core/kv_cache_manager.py:339-359, :420-461, :501-509)."""
    out = []
    cache = make_cache("f32", 2, 1, 8, 40, 4, 3)
    trace = []
    for op, rid, tokens in [
        ("alloc", "a", 9),
        ("alloc", "b", 4),
        ("free", "a", 0),
        ("alloc", "c", 13),
        ("alloc", "d", 1),
        ("free", "b", 0),
        ("alloc", "e", 8),
    ]:
        if op == "alloc":
            ok = cache.allocate(rid, tokens)
            trace.append(dict(op=op, rid=rid, tokens=tokens, ok=ok, tables=[list(t) for t in cache.plane_block_tables(rid)]))
        else:
            cache.free(rid)
            trace.append(dict(op=op, rid=rid))
    out.append(dict(shape=[2, 1, 8, 40, 4, 3], trace=trace, free=len(cache._free_blocks)))
    return out


def reservation_cases():
    """Traces of the reference's decode-side reservation hook: ``StageEngine.reserve_transfer`` (which plans the
    admission, allocates and pins), ``accept_import`` (which publishes the imported prompt to the prefix cache) and
    ``release_transfer``, on a real ``StageEngine`` with a tiny CPU model. Every step records what the connector
    would see (tables, prefix hit) and the pool's free-block count, so an implementation of the hook can be replayed
    against it. Prompts are lists of token ids below the tiny model's vocabulary of 64; ``max_tokens`` drives the
    growth budget."""
    import torch

    from tests.helpers import tiny_ouro_config
    from vllm_rlt import CacheConfig, SamplingParams, SchedulerConfig
    from vllm_rlt.engine.stage_config import StageConfig
    from vllm_rlt.engine.stage_engine import StageEngine
    from vllm_rlt.models import OuroForCausalLM

    scenarios = {
        # D holds a 3-page prefix from an earlier import; the next prompts share 3, 1 and 0 pages of it
        "prefix_hits": dict(
            cache=dict(num_blocks=64, block_size=4, enable_prefix_caching=True), chunk=8, seqs=4,
            steps=[("reserve", "a", list(range(1, 14)), 3), ("accept", "a"),
                   ("reserve", "b", list(range(1, 13)) + [40, 41, 42], 2), ("reserve", "c", list(range(1, 6)) + [50, 51, 52, 53], 1),
                   ("reserve", "d", [55, 56, 57, 58, 59], 4), ("accept", "b"), ("release", "a"), ("release", "c"),
                   ("reserve", "e", list(range(1, 13)) + [40, 41, 42, 43, 44], 1), ("release", "b"), ("release", "d"), ("release", "e")]),
        # a pool too small for two prompts at once: the second reservation is rejected whole and succeeds after a release
        "rejection_leaves_nothing": dict(
            cache=dict(num_blocks=24, block_size=4), chunk=8, seqs=4,
            steps=[("reserve", "a", list(range(1, 16)), 2), ("reserve", "b", list(range(20, 31)), 2), ("release", "a"),
                   ("reserve", "b", list(range(20, 31)), 2), ("release", "b")]),
        # incremental allocation without preemption: an import's future decode growth stays budgeted
        "growth_budget": dict(
            cache=dict(num_blocks=16, block_size=2, incremental_allocation=True), chunk=2, seqs=2,
            steps=[("reserve", "import", [1, 2], 7), ("reserve", "other", [3, 4], 1), ("release", "import"),
                   ("reserve", "other", [3, 4], 1), ("release", "other")]),
        # cached pages held only by the cache count as free, are budgeted when claimed, and are evicted oldest-first
        "eviction": dict(
            cache=dict(num_blocks=32, block_size=4, enable_prefix_caching=True), chunk=8, seqs=4,
            steps=[("reserve", "a", list(range(1, 10)), 1), ("accept", "a"), ("release", "a"),
                   ("reserve", "b", list(range(1, 10)), 1), ("release", "b"),
                   ("reserve", "big", [(7 * i) % 61 + 2 for i in range(27)], 2), ("release", "big"),
                   ("reserve", "c", list(range(1, 10)), 1), ("release", "c")]),
    }
    out = []
    for name, sc in scenarios.items():
        config = tiny_ouro_config()
        torch.manual_seed(0)
        engine = StageEngine(
            OuroForCausalLM(config), stage_config=StageConfig(role="decode"),
            cache_config=CacheConfig(sc["cache"]["num_blocks"], sc["cache"]["block_size"],
                                     **{k: v for k, v in sc["cache"].items() if k not in ("num_blocks", "block_size")}),
            scheduler_config=SchedulerConfig(max_num_seqs=sc["seqs"], prefill_chunk_size=sc["chunk"]),
        )
        cache = engine.cache_manager
        live, trace = {}, []
        try:
            for step in sc["steps"]:
                op, rid = step[0], step[1]
                if op == "reserve":
                    _, _, tokens, max_tokens = step
                    request = engine.reserve_transfer(rid, tokens, SamplingParams(max_tokens=max_tokens, ignore_eos=True), receiving=True)
                    row = dict(op=op, rid=rid, tokens=tokens, max_tokens=max_tokens, ok=request is not None)
                    if request is not None:
                        live[rid] = request
                        row.update(cached_tokens=request.num_prefilled_tokens,
                                   tables=[list(t) for t in cache.plane_block_tables(rid)])
                    else:
                        row.update(kept_request=engine.has_request(rid), kept_allocation=cache.has_allocation(rid))
                elif op == "accept":
                    ok = engine.accept_import(live[rid], torch.zeros(config.hidden_size), cached_tokens=live[rid].num_prefilled_tokens)
                    row = dict(op=op, rid=rid, ok=bool(ok), cached_pages=[list(b) for b in cache._prefixes.values()])
                else:
                    engine.release_transfer(live.pop(rid))
                    row = dict(op=op, rid=rid)
                row["free"] = cache.num_free_blocks
                row["free_list"] = len(cache._free_blocks)
                trace.append(row)
        finally:
            engine.close()
        out.append(dict(name=name, planes=cache.storage_depths, cache=sc["cache"], prefill_chunk_size=sc["chunk"],
                        max_num_seqs=sc["seqs"], trace=trace))
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("VLLM_RLT_REFERENCE", str(HERE.parents[2] / "reference")),
                    help="path of the vllm-rlt checkout (default: $VLLM_RLT_REFERENCE or a sibling of this repository)")
    ap.add_argument("--out", default=str(HERE), help="directory the fixtures are written to (default: beside this script)")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    import torch

    torch.set_num_threads(1)
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    (out / "segments.json").write_text(json.dumps(segment_cases(), indent=0))
    (out / "partition.json").write_text(json.dumps(partition_cases(), indent=0))
    (out / "handoff.json").write_text(json.dumps(handoff_cases(out), indent=0))
    (out / "finalize.json").write_text(json.dumps(finalize_cases(out), indent=0))
    (out / "allocation.json").write_text(json.dumps(allocation_cases(), indent=0))
    (out / "reservation.json").write_text(json.dumps(reservation_cases(), indent=0))
    print("golden fixtures written to", out)


if __name__ == "__main__":
    main()
