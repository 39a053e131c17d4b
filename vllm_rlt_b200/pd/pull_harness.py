"""Multi-GPU handoff, pull direction: the decode GPU reads the prefill GPU's pool over NVLink.

Same deployment shape, workloads, metadata exchange and timing rules as ``harness.run_multi`` (the push
direction), with the kernel on the other side of the link: the prefill worker only posts a "KV ready" flag
behind its producer, the decode worker waits for it (bounded), runs ``rlt_kv_handoff`` with the *source*
pool given as peer pointers and its own pool as destination, and posts a "done" flag into the prefill GPU's
memory so that the source blocks may be released.

Why it exists: NVLink charges writes 18.75 % of protocol bytes and read responses 12.5 %, and the read
requests travel on the opposite, otherwise idle direction. Measured with the link counters on this kernel:
push 713 GB/s of payload (847 GB/s raw), pull 769 GB/s of payload (865 GB/s raw) per pair. The price is
that the copy runs on the decode GPU's SMs instead of the prefill GPU's.
"""

from __future__ import annotations

import gc
import json
import os
import random
import statistics
import time

import numpy as np


def wire_bytes(w, requests, mode: str) -> int:
    """Bytes of the given requests of a workload that the decode GPU loads from the prefill pool."""
    from vllm_rlt_b200 import workloads

    sub = workloads.subset(w, list(requests))
    if mode != "dedup" or sub.exit_planes is None:
        return sub.payload_bytes
    deep = sub.extra.get("deep_layers")
    s = sub.shape
    per_layer = s.token_plane_bytes // s.num_layers
    total = 0
    for exits, (lo, hi) in zip(sub.exit_planes, sub.ranges):
        reach = np.minimum(np.asarray(exits[lo:hi], dtype=np.int64) + 1, sub.dst_planes)  # planes read per token
        if deep:
            total += int((s.token_plane_bytes + (reach - 1) * len(deep) * per_layer).sum())
        else:
            total += int(reach.sum()) * s.token_plane_bytes
    return total


def merge_waves(lines: list[dict], samples: list[float]) -> dict:
    """One benchmark line for several waves of one workload: a step is one pass over every wave, so times and bytes
    add up, rates are totals over totals, and the latency percentiles are over the requests of all waves."""
    out = dict(lines[0])
    ms = sum(x["ms_per_step"] for x in lines)
    payload = sum(x["config"]["payload_bytes"] for x in lines)
    link = sum(x["link_bytes"] for x in lines)
    pairs = lines[0]["value"] / lines[0]["per_pair_gbps"]
    out["ms_per_step"] = ms
    out["value"] = payload / (ms * 1e-3) / 1e9
    out["per_pair_gbps"] = out["value"] / pairs
    out["link_bytes"] = link
    out["link_gbps_per_pair"] = out["per_pair_gbps"] * link / payload
    out["config"] = dict(lines[0]["config"], waves=len(lines), requests=sum(x["config"]["requests"] for x in lines),
                         tokens=sum(x["config"]["tokens"] for x in lines), payload_bytes=payload,
                         wave_note="the request count does not fit the pools at once: independent draws of the workload "
                                   "run one after another, each on fresh pools; every wave is verified")
    roof = dict(lines[0]["roofline"])
    roof["achieved"] = out["link_gbps_per_pair"]
    roof["frac"] = roof["achieved"] / roof["peak"]
    roof["frac_of_nominal_900"] = roof["frac"]
    roof["kernel_ms"] = sum(x["roofline"]["kernel_ms"] for x in lines)
    roof["algorithmic_bytes_per_launch"] = sum(x["roofline"]["algorithmic_bytes_per_launch"] for x in lines)
    roof["traffic"] = sum(x["roofline"]["traffic"] for x in lines)
    out["roofline"] = roof
    e2e_ms = sum(x["e2e"]["ms_per_step"] for x in lines)
    out["e2e"] = dict(lines[0]["e2e"], value=payload / (e2e_ms * 1e-3) / 1e9, ms_per_step=e2e_ms,
                      h2d_bytes_per_step=sum(x["e2e"]["h2d_bytes_per_step"] for x in lines),
                      d2h_bytes_per_step=sum(x["e2e"]["d2h_bytes_per_step"] for x in lines))
    out["p50_latency_ms"] = statistics.median(samples)
    out["latency_ms"] = dict(lines[0]["latency_ms"], p50=statistics.median(samples), max=max(samples), min=min(samples),
                             requests=len(samples))
    out["gpu_launches"] = sum(x["gpu_launches"] for x in lines)
    out["verified"] = all(x["verified"] for x in lines)
    out["verified_bytes"] = sum(x["verified_bytes"] for x in lines)
    return out


def run_pull(args, rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist

    import bench
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd import exchange
    from vllm_rlt_b200.pd import peer as peerlib
    from vllm_rlt_b200.pd.harness import MODES, make_workload

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

    def partners_of(r):
        return exchange.pairing(r, world, n_prefill)[2]

    def assigned(p_rank: int, d_rank: int, w):
        return exchange.assigned_requests(p_rank, d_rank, world, n_prefill, len(w.lengths))

    def one_wave(wave: int):
        if is_prefill:
            w = make_workload(args, index, wave=wave)
            per_source = {}
        else:
            per_source = {p: make_workload(args, p, wave=wave) for p in partners}
            w = next(iter(per_source.values()))
        s = w.shape
        dst_planes = w.dst_planes
        deep = w.extra.get("deep_layers")
        kw = dict(device=device, kv_cache_dtype="fp8_e4m3" if s.fp8 else "auto")
        fan = max(len(partners_of(r)) for r in range(world))

        # ---- set-up: pools, reservation on the decode side, handles of pools and flags to everyone --------------
        handle_msg = torch.zeros((4 + fan, exchange.HANDLE_ROW), dtype=torch.uint8, device=device)
        flags = torch.zeros(fan, dtype=torch.int64, device=device)  # prefill: "done" per partner; decode: "ready" per source
        if is_prefill:
            pool = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, **kw)
            bench.fill_source(pool, s, workloads.SEED_BASE + index)
        else:
            total_blocks = sum(
                sum(-(-wp.lengths[i] // s.block_size) for i in assigned(p, rank, wp)) * dst_planes for p, wp in per_source.items())
            pool = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, max(total_blocks, 1), s.block_size, dst_planes, **kw)
            for t in (pool.key_cache, pool.value_cache):
                t.view(torch.uint8).fill_(0xA5)
            random.Random(workloads.SEED_BASE + 1000 + index).shuffle(pool._free_blocks)
            reserved = {}
            for p, wp in per_source.items():
                for i in assigned(p, rank, wp):
                    reserved[(p, i)] = pool.reserve_transfer(f"p{p}-r{i}", wp.lengths[i])
                    assert reserved[(p, i)] is not None
        tensors = [pool.key_cache, pool.value_cache] + ([pool.key_scale, pool.value_scale] if s.fp8 else [])
        rows = [peerlib.export_tensor(t) for t in tensors]
        rows += [rows[0]] * (4 - len(rows))
        flag_export = peerlib.export_tensor(flags)
        rows += [dict(flag_export, offset=flag_export["offset"] + 8 * j) for j in range(fan)]
        handle_msg.copy_(exchange.encode_handles(rows))
        all_handles = [torch.zeros_like(handle_msg) for _ in range(world)]
        dist.all_gather(all_handles, handle_msg)
        # The prefill workers' block tables and per-token exit planes travel to the decode workers over NCCL, as a
        # deployment would send them on its control channel: a decode worker pulls with the tables it RECEIVED, not
        # with ones it could rebuild from the seed. (All workers share the prompt lengths, so the messages are equal-sized.)
        width = -(-max(w.lengths) // s.block_size)
        src_msg = torch.zeros((len(w.lengths), s.planes, width), dtype=torch.int32, device=device)
        exit_msg = torch.zeros(max(1, sum(w.lengths)), dtype=torch.int32, device=device)
        if is_prefill:
            src_msg.copy_(exchange.encode_tables(w.src_tables, s.planes, width))
            if w.exit_planes is not None:
                exit_msg.copy_(torch.from_numpy(np.concatenate([np.asarray(e, np.int32) for e in w.exit_planes])))
        all_src, all_exits = exchange.all_gather_metadata(src_msg, exit_msg)
        torch.cuda.synchronize()
        received = {}
        if not is_prefill:
            for p_rank, wp in per_source.items():
                tables = exchange.decode_tables(all_src[p_rank], wp.lengths, s.block_size)
                exits = None
                if wp.exit_planes is not None:
                    flat = all_exits[p_rank].cpu().numpy()
                    ends = np.cumsum(wp.lengths)
                    exits = [flat[e - n : e] for e, n in zip(ends, wp.lengths)]
                received[p_rank] = (tables, exits)

        status = kh.new_status(device)
        mapping = peerlib.PeerMapping()
        edges = []
        plan = exchange.pull_edges(rank, world, n_prefill, len(w.lengths))
        if is_prefill:
            for edge in plan:
                ptrs = [mapping.pointer(e) for e in exchange.decode_handles(all_handles[edge["decode"]])]
                mine = edge["requests"]
                edges.append(dict(ready_ptr=ptrs[4 + edge["ready_slot"]], done=flags.data_ptr() + 8 * edge["done_slot"], mine=mine,
                                  payload=workloads.subset(w, mine).payload_bytes))
        else:
            dv = kh.PoolView.from_cache(pool)
            for edge in plan:
                p, mine = edge["prefill"], edge["requests"]
                wp = per_source[p]
                ptrs = [mapping.pointer(e) for e in exchange.decode_handles(all_handles[p])]
                scales = dv.scales.rebased(ptrs[2], ptrs[3]) if s.fp8 else None
                sv = kh.PoolView(dv.codes.rebased(ptrs[0], ptrs[1]), scales, wp.src_blocks, s.block_size, s.num_layers, s.planes, -1)
                got_tables, got_exits = received[p]
                sub = dict(src=[got_tables[i] for i in mine], dst=[reserved[(p, i)] for i in mine],
                           ranges=[wp.ranges[i] for i in mine],
                           exits=None if got_exits is None else [got_exits[i] for i in mine])

                def make_batch(sub=sub, wp=wp):
                    return kh.HandoffBatch(sub["src"], sub["dst"], sub["ranges"], block_size=s.block_size, exit_planes=sub["exits"],
                                           src_blocks=wp.src_blocks, dst_blocks=pool.num_blocks, device=device)

                edges.append(dict(sv=sv, ready=flags.data_ptr() + 8 * edge["ready_slot"], done_ptr=ptrs[4 + edge["done_slot"]], sub=sub,
                                  make_batch=make_batch, batch=make_batch(), mine=mine, source=p,
                                  payload=workloads.subset(wp, mine).payload_bytes))
        my_payload = sum(e["payload"] for e in edges) if not is_prefill else 0
        # bytes that cross the link: in dedup mode each row is read once (planes up to the token's exit plane) and the
        # deeper planes are filled on the decode GPU from the same load
        my_wire = sum(wire_bytes(per_source[e["source"]], e["mine"], args.mode) for e in edges) if not is_prefill else 0
        counter = 0

        def step(fresh_batches=False):
            nonlocal counter
            counter += 1
            if is_prefill:
                for e in edges:
                    kh.kv_signal(e["ready_ptr"], counter)  # behind the producer of the KV on this stream
                for e in edges:
                    kh.kv_wait(e["done"], counter, kh._lib.MAX_WAIT_NS, status)  # the source may be released after this
            else:
                for e in edges:
                    b = e["make_batch"]() if fresh_batches else e["batch"]
                    kh.kv_wait(e["ready"], counter, kh._lib.MAX_WAIT_NS, status)
                    kh.kv_handoff(e["sv"], dv, b, mode=mode, status=status, variant=args.variant, deep_layers=deep)
                    kh.kv_signal(e["done_ptr"], counter)

        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        kh.raise_for_status(status)
        dist.barrier()
        sampler = bench.ClockSampler(bench.visible_device_index(local)) if rank == world - 1 else None
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
        clock_box = [clocks]
        dist.broadcast_object_list(clock_box, src=world - 1)
        total_ms = torch.tensor([t0.elapsed_time(t1)], device=device)
        dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)
        kernel_ms = statistics.mean(a.elapsed_time(b) for a, b in events)
        k_ms = torch.tensor([kernel_ms if not is_prefill else 0.0], device=device)
        dist.all_reduce(k_ms, op=dist.ReduceOp.MAX)
        n_launch = torch.tensor([launches], device=device)
        dist.all_reduce(n_launch)
        payload_all = torch.tensor([float(my_payload), float(my_wire)], device=device, dtype=torch.float64)
        dist.all_reduce(payload_all)

        # ---- verification: every transferred row of every tensor (K, V, FP8 scales), by checksum over NCCL
        from vllm_rlt_b200.pd import verify

        if is_prefill:
            checks = [(e["decode"], w, e["requests"], None) for e in plan]
        else:
            checks = [(e["source"], per_source[e["source"]], e["mine"], e["sub"]["dst"]) for e in edges]
        verified, verified_bytes = verify.verify_over_group(pool, is_prefill, checks, mode=args.mode, deep=deep, device=device)

        # ---- end to end: every step the prefill worker stages its block tables and exit planes from pinned host memory
        # and sends them to the decode worker over NCCL (the deployment's metadata exchange); the decode worker stages its
        # own tables and ranges from the host, launches straight from the received device arrays, and the status is read back
        def pinned(array):
            return torch.from_numpy(np.ascontiguousarray(array)).pin_memory()

        for e in edges:
            mine = e["mine"]
            wp = w if is_prefill else per_source[e["source"]]
            lengths = [wp.lengths[i] for i in mine]
            shape = (len(mine), s.planes, width)
            e["wire"] = dict(src=torch.zeros(shape, dtype=torch.int32, device=device),
                             exits=torch.zeros(max(1, sum(lengths)), dtype=torch.int32, device=device))
            if is_prefill:
                e["host"] = dict(src=pinned(exchange.encode_tables([wp.src_tables[i] for i in mine], s.planes, width).numpy()),
                                 exits=None if wp.exit_planes is None else
                                 pinned(np.concatenate([np.asarray(wp.exit_planes[i], np.int32) for i in mine])))
            else:
                ends = np.cumsum(lengths)
                e["host"] = dict(dst=pinned(exchange.encode_tables(e["sub"]["dst"], dst_planes, width).numpy()),
                                 begin=pinned(np.asarray([r[0] for r in e["sub"]["ranges"]], np.int32)),
                                 end=pinned(np.asarray([r[1] for r in e["sub"]["ranges"]], np.int32)),
                                 offsets=pinned((ends - np.asarray(lengths)).astype(np.int64)))
            e["has_exits"] = wp.exit_planes is not None

        def e2e_step():
            nonlocal counter
            counter += 1
            staged = 0
            if is_prefill:
                for e in edges:
                    e["wire"]["src"].copy_(e["host"]["src"], non_blocking=True)
                    staged += e["host"]["src"].numel() * 4
                    dist.send(e["wire"]["src"], e["decode"])
                    if e["has_exits"]:
                        e["wire"]["exits"].copy_(e["host"]["exits"], non_blocking=True)
                        staged += e["host"]["exits"].numel() * 4
                        dist.send(e["wire"]["exits"], e["decode"])
                    kh.kv_signal(e["ready_ptr"], counter)
                for e in edges:
                    kh.kv_wait(e["done"], counter, kh._lib.MAX_WAIT_NS, status)
            else:
                for e in edges:
                    dist.recv(e["wire"]["src"], e["source"])
                    if e["has_exits"]:
                        dist.recv(e["wire"]["exits"], e["source"])
                    mine_dev = {k: v.to(device, non_blocking=True) for k, v in e["host"].items()}
                    staged += sum(v.numel() * v.element_size() for v in e["host"].values())
                    b = kh.HandoffBatch.from_device(e["wire"]["src"], mine_dev["dst"], mine_dev["begin"], mine_dev["end"],
                                                    block_size=s.block_size,
                                                    exit_planes=e["wire"]["exits"] if e["has_exits"] else None,
                                                    exit_offsets=mine_dev["offsets"] if e["has_exits"] else None)
                    kh.kv_wait(e["ready"], counter, kh._lib.MAX_WAIT_NS, status)
                    kh.kv_handoff(e["sv"], dv, b, mode=mode, status=status, variant=args.variant, deep_layers=deep)
                    kh.kv_signal(e["done_ptr"], counter)
                    e["last_batch"] = (b, mine_dev)
            return staged

        if is_prefill:
            for e, planned in zip(edges, plan):
                e["decode"] = planned["decode"]
        e2e, staged_now = [], 0
        for i in range(args.warmup + args.steps):
            dist.barrier()
            torch.cuda.synchronize()
            t_start = time.perf_counter()
            staged_now = e2e_step()
            kh.raise_for_status(status)
            if i >= args.warmup:
                e2e.append(time.perf_counter() - t_start)
        e2e_s = torch.tensor([statistics.mean(e2e)], device=device, dtype=torch.float64)
        dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
        staged_bytes = torch.tensor([staged_now], device=device)
        dist.all_reduce(staged_bytes)
        # the destination was written once more by the end-to-end steps, from tables that crossed NCCL: check it again
        verified_e2e, verified_e2e_bytes = verify.verify_over_group(pool, is_prefill, checks, mode=args.mode, deep=deep, device=device)
        verified = verified and verified_e2e and verified_e2e_bytes == verified_bytes

        # ---- per-request latency between rank 0 and its first partner: ready flag -> pull -> done flag, timed on the prefill
        # stream. The decode worker knows a request from its reservation on, so it queues wait -> pull -> done ahead of
        # time; the prefill worker gives it a few milliseconds to do so before it raises the flag (the wait is bounded).
        lat = []
        first_d = partners_of(0)[0]
        probe = min(int(getattr(args, "latency_requests", 16) or 16), len(assigned(0, first_d, w if rank == 0 else (per_source.get(0) or w))))
        for r in range(probe):
            for repeat in range(2):
                dist.barrier()
                torch.cuda.synchronize()
                counter += 1
                if rank == 0:
                    e = edges[0]
                    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    time.sleep(0.004)
                    a.record(stream)
                    kh.kv_signal(e["ready_ptr"], counter)
                    kh.kv_wait(e["done"], counter, kh._lib.MAX_WAIT_NS, status)
                    z.record(stream)
                    torch.cuda.synchronize()
                    if repeat:
                        lat.append(a.elapsed_time(z))
                elif rank == first_d:
                    e = next(x for x in edges if x["source"] == 0)
                    sub = e["sub"]
                    b = kh.HandoffBatch([sub["src"][r]], [sub["dst"][r]], [sub["ranges"][r]], block_size=s.block_size,
                                        exit_planes=None if sub["exits"] is None else [sub["exits"][r]], device=device)
                    kh.kv_wait(e["ready"], counter, kh._lib.MAX_WAIT_NS, status)
                    kh.kv_handoff(e["sv"], dv, b, mode=mode, status=status, variant=args.variant, deep_layers=deep)
                    kh.kv_signal(e["done_ptr"], counter)
                    torch.cuda.synchronize()
        kh.raise_for_status(status)
        torch.cuda.synchronize()
        dist.barrier()
        mapping.close()
        dist.barrier()

        if rank == 0:
            ms_per_step = float(total_ms.item()) / args.steps
            total_payload, total_wire = (float(x) for x in payload_all.tolist())
            value = total_payload / (ms_per_step * 1e-3) / 1e9
            links = min(n_prefill, n_decode)
            per_pair = value / links
            per_link = per_pair * total_wire / total_payload  # what the link carries per pair
            line = {
                "metric": bench.METRIC, "value": value, "unit": bench.UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "scaling_note": "N=1 is the intra-device pool-to-pool handoff (HBM-bound); N>=2 moves the same per-pair workload "
                                "between N/2 prefill and N/2 decode GPUs (NVLink-bound, 900 GB/s nominal per pair): N=2, 4, 8 "
                                "scale with one another, N=1 is a different bound",
                "vs_baseline": None, "dtype": "u8", "data": "synthetic",
                "config": bench.config_of(w, args, {
                    "split": f"{n_prefill}P:{n_decode}D", "variant": args.variant, "workload_name": args.workload,
                    "per_prefill_worker": w.description, "payload_bytes": total_payload,
                    "transport": "decode GPU pulls through peer pointers over NVLink (CUDA IPC mapping); ready and done flags per step; "
                                 "the prefill workers' block tables and exit planes reach the decode workers over NCCL"}),
                "roofline": {"bound": "nvlink", "achieved": per_link, "peak": bench.NVLINK_NOMINAL_GBS, "unit": "GB/s",
                             "frac": per_link / bench.NVLINK_NOMINAL_GBS,
                             "traffic": total_wire / max(1, n_decode) * bench.NVLINK_READ_OVERHEAD,
                             "traffic_source": "link bytes per launch: nvlrx__bytes.sum / nvlrx__bytes_data_user.sum = 1.125 from an "
                                               "ncu capture of the same kernel reading from a peer, scaled by the bytes read",
                             "peak_source": "nominal NVLink 5 rate per direction per GPU (no driver-measured link peak exists); a plain peer-to-peer memcpy between two B200s reached 770 GB/s",
                             "frac_of_peer_memcpy_770": per_link / bench.NVLINK_PEER_MEMCPY_GBS,
                             "kernel": "table_fan_kernel" if args.mode == "dedup" else "table_copy_kernel",
                             "algorithmic_bytes_per_launch": total_wire / max(1, n_decode),
                             "kernel_ms": float(k_ms.item()), "frac_of_nominal_900": per_link / bench.NVLINK_NOMINAL_GBS,
                             "raw_link_gbps": per_link * bench.NVLINK_READ_OVERHEAD,
                             "raw_link_frac_of_900": per_link * bench.NVLINK_READ_OVERHEAD / 900.0,
                             "raw_link_note": "read responses carry 12.5 % of protocol bytes on top of the payload (ncu nvlrx__bytes "
                                              "counters of this kernel); requests use the opposite direction",
                             "what": "bytes that cross NVLink per second / min(prefill, decode) GPUs: the per-GPU link rate of the "
                                     "busier side; equals the payload rate except in dedup mode, where only the rows up to each "
                                     "token's exit plane cross the link and `value` counts every destination byte"},
                "per_pair_gbps": per_pair, "link_bytes": total_wire, "link_gbps_per_pair": per_link,
                "e2e": {"value": total_payload / float(e2e_s.item()) / 1e9, "unit": bench.UNIT,
                        "h2d_bytes_per_step": int(staged_bytes.item()), "d2h_bytes_per_step": 16 * world, "ms_per_step": float(e2e_s.item()) * 1e3,
                        "note": "every step: the prefill worker stages its block tables and exit planes from pinned host memory and "
                                "sends them to the decode worker over NCCL; the decode worker stages its own tables and ranges, "
                                "waits for the ready flag, pulls, raises the done flag; both read their status words back"},
                "p50_latency_ms": statistics.median(lat),
                "latency_ms": {"p50": statistics.median(lat), "max": max(lat), "min": min(lat),
                               "what": "rank 0 -> its first decode partner: ready flag, pull, done flag; CUDA events on the prefill stream; "
                                       "the decode side has its wait and pull queued before the flag is raised"},
                "gpu_launches": int(n_launch.item()), "clocks": clock_box[0],
                "verified": verified and verified_bytes == int(total_payload), "verified_bytes": verified_bytes,
                "verified_how": "64-bit position-weighted checksums of every transferred row of K, V and the FP8 scale tensors per "
                                "(request, destination plane, tensor): source rows gathered with torch indexing on the prefill GPU, "
                                "destination rows on the decode GPU, tables compared over NCCL; plus the fill byte in the unowned "
                                "slots of partially filled blocks",
            }
            return line, lat
        return None, None

    waves = max(1, int(getattr(args, "waves", 1) or 1))
    lines, samples = [], []
    for wave in range(waves):
        line, lat = one_wave(wave)
        torch.cuda.synchronize()
        gc.collect()  # the wave's closures form reference cycles that would keep its pools alive into the next wave
        torch.cuda.empty_cache()
        dist.barrier()
        if rank == 0:
            lines.append(line)
            samples += lat
    if rank == 0:
        print(json.dumps(lines[0] if waves == 1 else merge_waves(lines, samples)), flush=True)
    dist.destroy_process_group()
