"""Multi-GPU handoff harness: N/2 prefill GPUs push KV to N/2 decode GPUs over NVLink.

One process per GPU (torchrun). Rank ``p`` in the first half is a prefill worker that owns a
source pool; rank ``p + N/2`` is its decode worker and owns the destination pool. The pairs
are independent: there is no collective on the data path. NCCL carries only the metadata a
real deployment exchanges on its control channel (``reserved`` -> ``prefill`` messages,
vllm_rlt/pd/engine.py:197-214): the decode side's block tables and the IPC handles of its
pools. KV bytes go from the prefill GPU's SMs straight into the decode GPU's pool through
peer pointers (plain per-thread stores), followed by a release-store of a
completion flag in the decode GPU's memory that the decode side waits on with a bounded wait.
"""

from __future__ import annotations

import json
import os
import random
import statistics
import time

import numpy as np



def run_multi(args, rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist

    import bench
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd import exchange
    from vllm_rlt_b200.pd import peer as peerlib

    if world != args.gpus or world % 2:
        raise SystemExit("--gpus must equal WORLD_SIZE and be even for a P:D split")
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    pairs = world // 2
    is_prefill, pair, partners = exchange.pairing(rank, world)
    partner = partners[0]

    # Same per-pair workload at every N (weak scaling); each pair gets its own seed.
    w = workloads.last_exited_exit_only(requests=args.requests, mode=args.mode, seed=workloads.SEED_BASE + 1 + 17 * pair)
    s = w.shape
    mode = {"exit_only": kh.MODE_EXIT_ONLY, "dedup": kh.MODE_DEDUP, "all": kh.MODE_ALL_PLANES}[args.mode]
    kw = dict(device=device, kv_cache_dtype="fp8_e4m3" if s.fp8 else "auto")
    width = max(len(t) for req in w.dst_tables for t in req)

    # ---- set-up: pools, decode-side reservation, metadata exchange over NCCL ----------------
    table_msg = torch.zeros((len(w.lengths), w.dst_planes, width), dtype=torch.int32, device=device)
    handle_msg = torch.zeros((3, exchange.HANDLE_ROW), dtype=torch.uint8, device=device)  # key, value, flag
    if is_prefill:
        src = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, **kw)
        gen = torch.Generator(device=device).manual_seed(workloads.SEED_BASE + pair)
        src.key_cache.normal_(generator=gen)
        src.value_cache.normal_(generator=gen)
        flag = None
    else:
        dst = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.dst_blocks, s.block_size,
                     w.dst_planes, layout="last_exited", **kw)
        for t in (dst.key_cache, dst.value_cache):
            t.view(torch.uint8).fill_(0xA5)
        # decode-side allocation hook: a seeded permutation of the free list, then one reservation per request
        random.Random(workloads.SEED_BASE + 1000 + pair).shuffle(dst._free_blocks)
        tables = []
        for i, n in enumerate(w.lengths):
            got = dst.reserve_transfer(f"r{i}", n)
            assert got is not None
            tables.append(got)
        table_msg.copy_(exchange.encode_tables(tables, w.dst_planes, width))
        flag = torch.zeros(1, dtype=torch.int64, device=device)
        handle_msg.copy_(exchange.encode_handles([peerlib.export_tensor(t) for t in (dst.key_cache, dst.value_cache, flag)]))
    all_tables, all_handles = exchange.all_gather_metadata(table_msg, handle_msg)
    torch.cuda.synchronize()

    status = kh.new_status(device)
    mapping = peerlib.PeerMapping()
    if is_prefill:
        dst_tables = exchange.decode_tables(all_tables[partner], w.lengths, s.block_size)
        ptrs = [mapping.pointer(e) for e in exchange.decode_handles(all_handles[partner])]
        sv = kh.PoolView.from_cache(src)
        dv = kh.PoolView(sv.codes.rebased(ptrs[0], ptrs[1]), None, w.dst_blocks, s.block_size, s.num_layers, w.dst_planes, -1)
        flag_ptr = ptrs[2]

        def make_batch():
            return kh.HandoffBatch(w.src_tables, dst_tables, w.ranges, block_size=s.block_size, exit_planes=w.exit_planes,
                                   src_blocks=w.src_blocks, dst_blocks=w.dst_blocks, device=device)

        batch = make_batch()
    counter = 0

    def step():
        nonlocal counter
        counter += 1
        if is_prefill:
            kh.kv_handoff(sv, dv, batch, mode=mode, status=status, variant=args.variant)
            kh.kv_signal(flag_ptr, counter)
        else:
            kh.kv_wait(flag.data_ptr(), counter, kh._lib.MAX_WAIT_NS, status)

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
    k_ms = torch.tensor([kernel_ms if is_prefill else 0.0], device=device)
    dist.all_reduce(k_ms, op=dist.ReduceOp.MAX)
    n_launch = torch.tensor([launches], device=device)
    dist.all_reduce(n_launch)

    # ---- verification: prefill gathers what the first tokens of request 0 should hold, decode compares
    sample = min(64, w.lengths[0])
    expect = torch.zeros((2, sample, s.num_layers, s.num_kv_heads, s.head_dim), dtype=torch.bfloat16, device=device)
    ok = torch.ones(1, device=device)
    for plane in range(w.dst_planes):
        if is_prefill:
            pos = torch.arange(sample, device=device)
            if w.exit_planes is None:
                sp = torch.full((sample,), plane, device=device)
            else:
                e = torch.tensor(np.asarray(w.exit_planes[0][:sample]), device=device)
                sp = e if args.mode == "exit_only" else torch.clamp(e, max=plane)
            st = torch.tensor(np.stack(w.src_tables[0]), device=device)
            sb = st[sp, pos // s.block_size]
            expect[0] = src.key_cache[sb, :, pos % s.block_size]
            expect[1] = src.value_cache[sb, :, pos % s.block_size]
            dist.send(expect, partner)
        else:
            dist.recv(expect, partner)
            pos = torch.arange(sample, device=device)
            db = torch.tensor(tables[0][plane], device=device)[pos // s.block_size]
            same = torch.equal(dst.key_cache[db, :, pos % s.block_size].view(torch.int16), expect[0].view(torch.int16)) and \
                torch.equal(dst.value_cache[db, :, pos % s.block_size].view(torch.int16), expect[1].view(torch.int16))
            ok *= float(same)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)

    # ---- end to end on the prefill side: host tables -> device, launch, flag, status read back
    e2e = []
    for i in range(args.warmup + args.steps):
        dist.barrier()
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        counter += 1
        if is_prefill:
            b = make_batch()
            kh.kv_handoff(sv, dv, b, mode=mode, status=status, variant=args.variant)
            kh.kv_signal(flag_ptr, counter)
        else:
            kh.kv_wait(flag.data_ptr(), counter, kh._lib.MAX_WAIT_NS, status)
        kh.raise_for_status(status)
        if i >= args.warmup:
            e2e.append(time.perf_counter() - t_start)
    e2e_s = torch.tensor([statistics.mean(e2e)], device=device, dtype=torch.float64)
    dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)

    # ---- per-request latency on pair 0: launch + flag, observed on the prefill stream
    lat = []
    if is_prefill:
        for r in range(min(len(w.lengths), 32)):
            one = workloads.subset(w, [r])
            b = kh.HandoffBatch(one.src_tables, [dst_tables[r]], one.ranges, block_size=s.block_size,
                                exit_planes=one.exit_planes, device=device)
            kh.kv_handoff(sv, dv, b, mode=mode, status=status, variant=args.variant)
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            kh.kv_handoff(sv, dv, b, mode=mode, status=status, variant=args.variant)
            counter += 1
            kh.kv_signal(flag_ptr, counter)
            z.record(stream)
            torch.cuda.synchronize()
            lat.append(a.elapsed_time(z))
    torch.cuda.synchronize()
    dist.barrier()
    if is_prefill:
        mapping.close()  # writers unmap before receivers free
    dist.barrier()

    if rank == 0:
        ms_per_step = float(total_ms.item()) / args.steps
        total_payload = w.payload_bytes * pairs  # every pair has the same token count distribution parameters
        value = total_payload / (ms_per_step * 1e-3) / 1e9
        per_pair = w.payload_bytes / (float(k_ms.item()) * 1e-3) / 1e9
        line = {
            "metric": bench.METRIC, "value": value, "unit": bench.UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": bench.config_of(w, args, {"split": f"{pairs}P:{pairs}D", "variant": args.variant,
                                                "transport": "peer stores over NVLink (CUDA IPC mapping), completion flag per step"}),
            "roofline": {"bound": "nvlink", "achieved": per_pair, "peak": bench.NVLINK_MEASURED_GBS, "unit": "GB/s",
                         "frac": per_pair / bench.NVLINK_MEASURED_GBS, "traffic": None,
                         "peak_source": "measured peer copy on this pool, 770 GB/s per direction (nominal 900)",
                         "kernel": "table_copy_kernel", "algorithmic_bytes_per_launch": w.payload_bytes,
                         "kernel_ms": float(k_ms.item()), "frac_of_nominal_900": per_pair / 900.0},
            "per_pair_gbps": per_pair,
            "e2e": {"value": total_payload / float(e2e_s.item()) / 1e9, "unit": bench.UNIT,
                    "h2d_bytes_per_step": batch.metadata_bytes, "d2h_bytes_per_step": 16,
                    "ms_per_step": float(e2e_s.item()) * 1e3},
            "latency_ms": {"p50": statistics.median(lat), "max": max(lat), "min": min(lat),
                           "what": "pair 0, one launch + completion flag per request, CUDA events on the prefill stream"},
            "gpu_launches": int(n_launch.item()), "clocks": clocks, "verified": bool(ok.item() == 1.0),
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()
