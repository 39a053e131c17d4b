"""Multi-GPU handoff harness: prefill GPUs push KV to decode GPUs over NVLink.

One process per GPU (torchrun). The first ``P`` ranks are prefill workers that own source pools,
the rest are decode workers that own destination pools; ``P`` defaults to half the ranks and can be
any split (2:6, 4:4, 6:2 ...). Requests of a prefill worker are routed round-robin over its decode
partners. Every P->D edge is independent: there is no collective on the data path. NCCL carries only
the metadata a real deployment exchanges on its control channel (``reserved`` -> ``prefill``,
vllm_rlt/pd/engine.py:197-214): the decode side's block tables and the IPC handles of its pools and
flags. KV bytes go from the prefill GPU's SMs straight into the decode GPU's pool through peer
pointers (plain per-thread stores), followed by a release-store of a completion flag in the decode
GPU's memory that the decode side waits on with a bounded wait.

Two timed modes: the default hands a finished batch off in one launch per edge; ``--streaming``
replays a layer-by-layer prefill (a timed dummy kernel per layer) and streams each (depth, layer
group) behind it, reporting how long after the prefill's end the last byte lands.
"""

from __future__ import annotations

import json
import os
import random
import statistics
import time

MODES = {"exit_only": 2, "dedup": 1, "all": 0}


POOL_LIMIT_BYTES = 165 << 30  # what one pool may take of a 180 GB GPU


def make_workload(args, prefill_index: int, lengths=None, wave: int = 0):
    """The workload of one prefill worker; every rank can rebuild any worker's from its index.

    All workers get the same prompt lengths (those of worker 0), so that per-GPU work is identical at
    every N (weak scaling); block tables and exit planes are seeded per worker. ``wave`` selects one of several
    independent draws, for workloads whose full request count does not fit the pools at once. A workload whose source or
    destination pool cannot fit one GPU is refused here, before anything is allocated.
    """
    w = _make_workload(args, prefill_index, lengths, wave)
    if w.exit_planes is None and getattr(args, "mode", "all") != "all":
        raise SystemExit(f"workload {getattr(args, 'workload', 'ouro1p4b')!r} has no per-token exit planes: run it with --mode all")
    for side, blocks in (("source", w.src_blocks), ("destination", w.dst_blocks)):
        need = blocks * w.shape.block_bytes
        if need > POOL_LIMIT_BYTES:
            raise SystemExit(f"workload {getattr(args, 'workload', 'ouro1p4b')!r} with {len(w.lengths)} requests needs a "
                             f"{need / 2**30:.0f} GiB {side} pool; run it in waves with a smaller --requests")
    return w


def _make_workload(args, prefill_index: int, lengths=None, wave: int = 0):
    from vllm_rlt_b200 import workloads as wl

    if lengths is None and prefill_index != 0:
        lengths = _make_workload(args, 0, None, wave).lengths
    seed = wl.SEED_BASE + 1 + 17 * prefill_index + 1009 * wave  # a wave is another draw of the same distribution
    name = getattr(args, "workload", "ouro1p4b")
    if name == "ouro1p4b":
        return wl.last_exited_exit_only(wl.OURO_1P4B, requests=args.requests, mode=args.mode, seed=seed, lengths=lengths)
    if name == "ouro2p6b":
        return wl.last_exited_exit_only(wl.OURO_2P6B, requests=args.requests, mode=args.mode, seed=seed, lengths=lengths)
    if name == "ouro2p6b_fp8_shared":
        # FP8 e4m3 with travelling float32 scales; "SHARED for loops >= 2" = two planes (loop 1, loops 2..4)
        shape = wl.KVShape("ouro-2.6b-fp8 planes[0,1,1,1]", 48, 16, 128, 2, fp8=True)
        return wl.per_depth_all_planes(shape, requests=args.requests, min_len=1024, max_len=8192, seed=seed,
                                       log_uniform=True, lengths=lengths)
    if name == "ouro2p6b_4k":
        # per-request latency probe: 4096-token Ouro-2.6B-shaped prompts
        if args.mode == "all":
            return wl.per_depth_all_planes(wl.OURO_2P6B, requests=args.requests, min_len=4096, max_len=4096, seed=seed)
        return wl.last_exited_exit_only(wl.OURO_2P6B, requests=args.requests, min_len=4096, max_len=4096,
                                        partial_fraction=0.0, mode=args.mode, seed=seed)
    if name == "ouro2p6b_fp8_4k":
        shape = wl.OURO_2P6B_FP8 if args.mode != "all" else wl.KVShape("ouro-2.6b-fp8 single plane", 48, 16, 128, 1, fp8=True)
        if args.mode == "all":
            return wl.per_depth_all_planes(shape, requests=args.requests, min_len=4096, max_len=4096, seed=seed)
        return wl.last_exited_exit_only(shape, requests=args.requests, min_len=4096, max_len=4096, partial_fraction=0.0,
                                        mode=args.mode, seed=seed)
    if name == "huginn":
        return wl.recurrent_depth_dedup(wl.HUGINN_3P5B, requests=args.requests, seed=seed, lengths=lengths)
    if name == "huginn_recurrent":
        # prelude (layers 0-1) and coda (6-7) KV exist once; only the core layers 2-5 have one copy per recurrence
        return wl.recurrent_depth_dedup(wl.HUGINN_3P5B, requests=args.requests, seed=seed, lengths=lengths,
                                        deep_layers=(2, 3, 4, 5))
    if name == "ouro2p6b_chunk":
        # one 2048-token prefill chunk per request, all planes (what a WCPB step finishes)
        # half of the requests already have a 4096-token prefix on the decode side: only the chunk after it moves
        return wl.per_depth_all_planes(wl.OURO_2P6B, requests=args.requests, min_len=2048, max_len=2048,
                                       seed=wl.SEED_BASE + 5, resident_prefix=4096, resident_fraction=0.5)
    raise SystemExit(f"unknown workload {name}")


def run_multi(args, rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist

    import bench
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd import exchange
    from vllm_rlt_b200.pd import peer as peerlib
    from vllm_rlt_b200.pd.streaming import LayerStreamer

    if world != args.gpus:
        raise SystemExit("--gpus must equal WORLD_SIZE")
    n_prefill = args.prefill or world // 2
    n_decode = world - n_prefill
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    exchange.init_process_group_quietly(device)
    is_prefill, index, partners = exchange.pairing(rank, world, n_prefill)
    mode = MODES[args.mode]

    def assigned(p_index: int, d_rank: int, w):
        """Requests of prefill worker p_index that go to decode rank d_rank (round-robin over its partners)."""
        _, _, p_partners = exchange.pairing(p_index, world, n_prefill)
        return [i for i in range(len(w.lengths)) if p_partners[i % len(p_partners)] == d_rank]

    # ---- workloads: a prefill rank builds its own; a decode rank rebuilds those of its sources ----
    if is_prefill:
        w = make_workload(args, index)
        shape = w.shape
        sources = []
    else:
        sources = partners  # prefill ranks (== prefill indices) that send to this decode rank
        per_source = {p: make_workload(args, p) for p in sources}
        w = next(iter(per_source.values()))
        shape = w.shape
    s = shape
    dst_planes = w.dst_planes
    deep = w.extra.get("deep_layers")
    fan_in = max(len(exchange.pairing(r, world, n_prefill)[2]) for r in range(n_prefill, world))
    width = -(-max(getattr(args, "max_len", 0) or 0, max(w.lengths)) // s.block_size)
    width_t = torch.tensor([width], device=device)
    dist.all_reduce(width_t, op=dist.ReduceOp.MAX)
    width = int(width_t.item())
    kw = dict(device=device, kv_cache_dtype="fp8_e4m3" if s.fp8 else "auto")
    n_req = len(w.lengths)

    # ---- set-up: pools, decode-side reservation, metadata exchange over NCCL ----------------
    table_msg = torch.zeros((fan_in, n_req, dst_planes, width), dtype=torch.int32, device=device)
    n_handles = (4 if s.fp8 else 2) + fan_in
    handle_msg = torch.zeros((n_handles, exchange.HANDLE_ROW), dtype=torch.uint8, device=device)
    if is_prefill:
        src = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, **kw)
        bench.fill_source(src, s, workloads.SEED_BASE + index)
    else:
        total_blocks = 0
        for p, wp in per_source.items():
            total_blocks += sum(-(-wp.lengths[i] // s.block_size) for i in assigned(p, rank, wp)) * dst_planes
        dst = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, max(total_blocks, 1), s.block_size, dst_planes,
                     layout="last_exited", **kw)
        for t in (dst.key_cache, dst.value_cache):
            t.view(torch.uint8).fill_(0xA5)
        # decode-side allocation hook: seeded permutation of the free list, one reservation per incoming request
        random.Random(workloads.SEED_BASE + 1000 + index).shuffle(dst._free_blocks)
        reserved = {}
        for slot, p in enumerate(sources):
            wp = per_source[p]
            tables = [[] for _ in range(n_req)]
            for i in assigned(p, rank, wp):
                got = dst.reserve_transfer(f"p{p}-r{i}", wp.lengths[i])
                assert got is not None
                tables[i] = got
                reserved[(p, i)] = got
            padded = [t if t else [[] for _ in range(dst_planes)] for t in tables]
            table_msg[slot].copy_(exchange.encode_tables(padded, dst_planes, width))
        flags = torch.zeros(fan_in, dtype=torch.int64, device=device)
        exported = [dst.key_cache, dst.value_cache] + ([dst.key_scale, dst.value_scale] if s.fp8 else [])
        rows = [peerlib.export_tensor(t) for t in exported]
        flag_export = peerlib.export_tensor(flags)
        for slot in range(fan_in):
            rows.append(dict(flag_export, offset=flag_export["offset"] + 8 * slot))
        handle_msg.copy_(exchange.encode_handles(rows))
    all_tables, all_handles = exchange.all_gather_metadata(table_msg, handle_msg)
    blocks_msg = torch.tensor([0 if is_prefill else dst.num_blocks], device=device)
    all_blocks = [torch.zeros_like(blocks_msg) for _ in range(world)]
    dist.all_gather(all_blocks, blocks_msg)
    torch.cuda.synchronize()

    status = kh.new_status(device)
    mapping = peerlib.PeerMapping()
    edges = []  # prefill side: one entry per decode partner
    if is_prefill:
        sv = kh.PoolView.from_cache(src)
        for d_rank in partners:
            d_sources = exchange.pairing(d_rank, world, n_prefill)[2]
            slot = d_sources.index(rank)
            mine = assigned(index, d_rank, w)
            if not mine:
                continue
            decoded = exchange.decode_tables(all_tables[d_rank][slot], w.lengths, s.block_size)
            ptrs = [mapping.pointer(e) for e in exchange.decode_handles(all_handles[d_rank])]
            n_pool = 4 if s.fp8 else 2
            scales = sv.scales.rebased(ptrs[2], ptrs[3]) if s.fp8 else None
            d_blocks = int(all_blocks[d_rank].item())
            dv = kh.PoolView(sv.codes.rebased(ptrs[0], ptrs[1]), scales, d_blocks, s.block_size, s.num_layers, dst_planes, -1)
            sub = dict(
                src_tables=[w.src_tables[i] for i in mine], dst_tables=[decoded[i] for i in mine],
                ranges=[w.ranges[i] for i in mine],
                exit_planes=None if w.exit_planes is None else [w.exit_planes[i] for i in mine],
            )
            edge = dict(d_rank=d_rank, dv=dv, flag_ptr=ptrs[n_pool + slot], sub=sub, mine=mine,
                        payload=workloads.subset(w, mine).payload_bytes)

            def make_batch(sub=sub):
                return kh.HandoffBatch(sub["src_tables"], sub["dst_tables"], sub["ranges"], block_size=s.block_size,
                                       exit_planes=sub["exit_planes"], src_blocks=w.src_blocks, device=device)

            edge["make_batch"] = make_batch
            edge["batch"] = make_batch()
            edges.append(edge)
    my_payload = sum(e["payload"] for e in edges)
    counter = 0

    def step():
        nonlocal counter
        counter += 1
        if is_prefill:
            for e in edges:
                kh.kv_handoff(sv, e["dv"], e["batch"], mode=mode, status=status, variant=args.variant, deep_layers=deep)
                kh.kv_signal(e["flag_ptr"], counter)
        else:
            for slot in range(len(sources)):
                kh.kv_wait(flags.data_ptr() + 8 * slot, counter, kh._lib.MAX_WAIT_NS, status)

    # ---- streaming replay: a dummy prefill of `layer_us` per layer and depth, handoff slices behind it ----
    def streaming_step(layer_us: float, layers_per_slice: int):
        """Returns (prefill end event, handoff end event, compute stream) for one chunk pass on a prefill rank."""
        nonlocal counter
        counter += 1
        if not is_prefill:
            for slot in range(len(sources)):
                kh.kv_wait(flags.data_ptr() + 8 * slot, counter, kh._lib.MAX_WAIT_NS, status)
            return None
        compute = torch.cuda.current_stream(device)
        streamers = [LayerStreamer(sv, e["dv"], e["batch"], mode=mode, layers_per_slice=layers_per_slice,
                                   status=status, variant=args.variant) for e in edges]
        for st in streamers:
            st.stream.wait_stream(compute)
        cycles = int(layer_us * 1e-6 * 1.9e9)
        for plane in range(dst_planes):
            for layer in range(s.num_layers):
                torch.cuda._sleep(cycles)  # stands in for one layer of prefill compute at this depth
                for st in streamers:
                    st.layer_done(plane, layer, producer_stream=compute)
        prefill_end = torch.cuda.Event(enable_timing=True)
        prefill_end.record(compute)
        ends = [st.finish(e["flag_ptr"], counter) for st, e in zip(streamers, edges)]
        for st in streamers:
            compute.wait_stream(st.stream)
        return prefill_end, ends, sum(st.launched for st in streamers)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    kh.raise_for_status(status)
    dist.barrier()
    torch.cuda.synchronize()

    sampler = bench.ClockSampler(bench.visible_device_index(local)) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    dist.barrier()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    launches0 = kh.kernel_launches()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    events = []
    t0.record(stream)
    for _ in range(args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        step()
        b.record(stream)
        events.append((a, b))
    t1.record(stream)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    launches = kh.kernel_launches() - launches0
    kh.raise_for_status(status)
    clocks = sampler.stop() if sampler else None
    total_ms = torch.tensor([t0.elapsed_time(t1)], device=device)
    dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
    kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
    # per-GPU rates: egress of a prefill GPU, ingress of a decode GPU (bytes it received / its wait time)
    egress = torch.tensor([my_payload / (kernel_ms * 1e-3) / 1e9 if is_prefill else float("inf")], device=device)
    dist.all_reduce(egress, op=dist.ReduceOp.MIN)
    k_ms = torch.tensor([kernel_ms if is_prefill else 0.0], device=device)
    dist.all_reduce(k_ms, op=dist.ReduceOp.MAX)
    n_launch = torch.tensor([launches], device=device)
    dist.all_reduce(n_launch)
    payload_all = torch.tensor([float(my_payload)], device=device, dtype=torch.float64)
    dist.all_reduce(payload_all)

    # ---- verification: every transferred row of every tensor (K, V, FP8 scales), by checksum over NCCL
    from vllm_rlt_b200.pd import verify

    if is_prefill:
        checks = [(e["d_rank"], w, e["mine"], None) for e in edges]
        verified, verified_bytes = verify.verify_over_group(src, True, checks, mode=args.mode, deep=deep, device=device)
    else:
        checks = []
        for p in sources:
            mine = assigned(p, rank, per_source[p])
            checks.append((p, per_source[p], mine, [reserved[(p, i)] for i in mine]))
        verified, verified_bytes = verify.verify_over_group(dst, False, checks, mode=args.mode, deep=deep, device=device)

    # ---- end to end on the prefill side: host tables -> device, launch, flag, status read back
    e2e = []
    for i in range(args.warmup + args.steps):
        dist.barrier()
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        counter += 1
        if is_prefill:
            for e in edges:
                b = e["make_batch"]()
                kh.kv_handoff(sv, e["dv"], b, mode=mode, status=status, variant=args.variant, deep_layers=deep)
                kh.kv_signal(e["flag_ptr"], counter)
        else:
            for slot in range(len(sources)):
                kh.kv_wait(flags.data_ptr() + 8 * slot, counter, kh._lib.MAX_WAIT_NS, status)
        kh.raise_for_status(status)
        if i >= args.warmup:
            e2e.append(time.perf_counter() - t_start)
    e2e_s = torch.tensor([statistics.mean(e2e)], device=device, dtype=torch.float64)
    dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)

    # ---- per-request latency on every prefill rank's first edge: launch + flag, on the prefill stream
    lat = []
    if is_prefill and edges:
        e = edges[0]
        for r in range(min(len(e["mine"]), 32)):
            sub = e["sub"]
            b = kh.HandoffBatch([sub["src_tables"][r]], [sub["dst_tables"][r]], [sub["ranges"][r]], block_size=s.block_size,
                                exit_planes=None if sub["exit_planes"] is None else [sub["exit_planes"][r]], device=device)
            kh.kv_handoff(sv, e["dv"], b, mode=mode, status=status, variant=args.variant, deep_layers=deep)
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            kh.kv_handoff(sv, e["dv"], b, mode=mode, status=status, variant=args.variant, deep_layers=deep)
            counter += 1
            kh.kv_signal(e["flag_ptr"], counter)
            z.record(stream)
            torch.cuda.synchronize()
            lat.append(a.elapsed_time(z))
        # keep the decode side's expected counter in step for what follows
    counter_t = torch.tensor([counter], device=device)
    dist.all_reduce(counter_t, op=dist.ReduceOp.MAX)
    counter = int(counter_t.item())
    if is_prefill:
        for e in edges:
            kh.kv_signal(e["flag_ptr"], counter)
    torch.cuda.synchronize()
    dist.barrier()

    # ---- streaming replay -------------------------------------------------------------------
    streaming = None
    if getattr(args, "streaming", False):
        tails, fulls, slices = [], [], 0
        for i in range(2 + args.steps):
            dist.barrier()
            torch.cuda.synchronize()
            out = streaming_step(args.layer_us, args.layers_per_slice)
            torch.cuda.synchronize()
            kh.raise_for_status(status)
            if is_prefill and i >= 2:
                prefill_end, ends, slices = out
                tails.append(max(prefill_end.elapsed_time(z) for z in ends))
        # the same pass without streaming: the handoff starts only when the whole prefill has finished
        for i in range(2 + args.steps):
            dist.barrier()
            torch.cuda.synchronize()
            counter += 1
            if is_prefill:
                torch.cuda._sleep(int(args.layer_us * 1e-6 * 1.9e9) * s.num_layers * dst_planes)
                a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream)
                for e in edges:
                    kh.kv_handoff(sv, e["dv"], e["batch"], mode=mode, status=status, variant=args.variant, deep_layers=deep)
                    kh.kv_signal(e["flag_ptr"], counter)
                z.record(stream)
            else:
                for slot in range(len(sources)):
                    kh.kv_wait(flags.data_ptr() + 8 * slot, counter, kh._lib.MAX_WAIT_NS, status)
            torch.cuda.synchronize()
            kh.raise_for_status(status)
            if is_prefill and i >= 2:
                fulls.append(a.elapsed_time(z))
        tail = torch.tensor([statistics.median(tails) if tails else 0.0], device=device)
        full = torch.tensor([statistics.median(fulls) if fulls else 0.0], device=device)
        dist.all_reduce(tail, op=dist.ReduceOp.MAX)
        dist.all_reduce(full, op=dist.ReduceOp.MAX)
        streaming = {
            "tail_ms_after_prefill_end": float(tail.item()), "unstreamed_ms_after_prefill_end": float(full.item()),
            "simulated_prefill_ms": args.layer_us * 1e-3 * s.num_layers * dst_planes, "layer_us": args.layer_us,
            "layers_per_slice": args.layers_per_slice, "slices_per_pass": slices,
            "what": "max over prefill ranks of the median time from the end of the simulated prefill to the completion flag",
        }

    torch.cuda.synchronize()
    dist.barrier()
    if is_prefill:
        mapping.close()  # writers unmap before receivers free
    dist.barrier()

    if rank == 0:
        ms_per_step = float(total_ms.item()) / args.steps
        total_payload = float(payload_all.item())
        value = total_payload / (ms_per_step * 1e-3) / 1e9
        per_gpu = float(egress.item())
        # the busier side bounds an uneven split: n_prefill egress links feed n_decode ingress links
        links = min(n_prefill, n_decode)
        per_link = value / links
        line = {
            "metric": bench.METRIC, "value": value, "unit": bench.UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "scaling_note": "N=1 is the intra-device pool-to-pool handoff (HBM-bound); N>=2 moves the same per-pair workload "
                            "between N/2 prefill and N/2 decode GPUs (NVLink-bound, 900 GB/s nominal per pair): N=2, 4, 8 "
                            "scale with one another, N=1 is a different bound",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": bench.config_of(w, args, {
                "split": f"{n_prefill}P:{n_decode}D", "variant": args.variant, "workload_name": getattr(args, "workload", "ouro1p4b"),
                "per_prefill_worker": w.description, "payload_bytes": total_payload,
                "transport": "peer stores over NVLink (CUDA IPC mapping), completion flag per step"}),
            "roofline": {"bound": "nvlink", "achieved": per_link, "peak": bench.NVLINK_NOMINAL_GBS, "unit": "GB/s",
                         "frac": per_link / bench.NVLINK_NOMINAL_GBS,
                         "traffic": w.payload_bytes * bench.NVLINK_WRITE_OVERHEAD,
                         "traffic_source": "link bytes per launch: nvltx__bytes.sum / nvltx__bytes_data_user.sum = 1.1875 from an "
                                           "ncu capture of the same kernel writing to a peer, scaled by the payload",
                         "peak_source": "nominal NVLink 5 rate per direction per GPU (no driver-measured link peak exists); a plain peer-to-peer memcpy between two B200s reached 770 GB/s",
                         "frac_of_peer_memcpy_770": per_link / bench.NVLINK_PEER_MEMCPY_GBS,
                         "kernel": "table_copy_kernel", "algorithmic_bytes_per_launch": w.payload_bytes,
                         "kernel_ms": float(k_ms.item()), "frac_of_nominal_900": per_link / bench.NVLINK_NOMINAL_GBS,
                         "raw_link_gbps": per_link * bench.NVLINK_WRITE_OVERHEAD,
                         "raw_link_frac_of_900": per_link * bench.NVLINK_WRITE_OVERHEAD / 900.0,
                         "raw_link_note": "NVLink carries 18.75 % of protocol bytes on top of written payload (ncu nvltx__bytes "
                                          "counters of this kernel)",
                         "what": "aggregate payload rate / min(prefill, decode) GPUs: the per-GPU link rate of the busier side"},
            "per_pair_gbps": per_link, "slowest_prefill_gpu_egress_gbps": per_gpu,
            "e2e": {"value": total_payload / float(e2e_s.item()) / 1e9, "unit": bench.UNIT,
                    "h2d_bytes_per_step": sum(e["batch"].metadata_bytes for e in edges), "d2h_bytes_per_step": 16,
                    "ms_per_step": float(e2e_s.item()) * 1e3},
            "p50_latency_ms": statistics.median(lat),
            "latency_ms": {"p50": statistics.median(lat), "max": max(lat), "min": min(lat),
                           "what": "rank 0, one launch + completion flag per request, CUDA events on the prefill stream"},
            "gpu_launches": int(n_launch.item()), "clocks": clocks,
            "verified": verified and verified_bytes == int(total_payload), "verified_bytes": verified_bytes,
            "verified_how": "64-bit position-weighted checksums of every transferred row of K, V and the FP8 scale tensors per "
                            "(request, destination plane, tensor), compared between the prefill and the decode GPU over NCCL; "
                            "plus the fill byte in the unowned slots of partially filled blocks",
        }
        if streaming:
            line["streaming"] = streaming
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()
