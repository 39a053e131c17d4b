"""Pack -> push -> scatter over NVLink, with a wire image that carries each KV row only once.

The direct handoff (``harness.run_multi``) writes every destination row over the link. When tokens left
the recurrence early, the planes beyond a token's exit plane are copies of one row, so most of those bytes
are redundant on the wire. Here the prefill GPU gathers the batch into the dedup wire image *directly in a
staging buffer on the decode GPU* (the pack kernel's destination is a peer pointer, so gather and push are
one kernel and nothing is staged on the prefill side), posts a flag, and the decode GPU scatters the image
into its own block tables, rebuilding the copies at HBM speed. Two staging buffers alternate; the decode side
tells the prefill side through a flag in the prefill GPU's memory when a buffer may be overwritten. All waits
are bounded. NCCL carries only tables, IPC handles and sizes.

One prefill rank per decode rank (N/2 : N/2).
"""

from __future__ import annotations

import json
import os
import random

import numpy as np


def run_staged(args, rank: int, world: int) -> None:
    import torch
    import torch.distributed as dist

    import bench
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd import exchange
    from vllm_rlt_b200.pd import peer as peerlib
    from vllm_rlt_b200.pd.harness import MODES, make_workload

    if world != args.gpus or world % 2:
        raise SystemExit("the staged path needs an even --gpus equal to WORLD_SIZE")
    local = int(os.environ.get("LOCAL_RANK", rank))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    exchange.init_process_group_quietly(device)
    pairs = world // 2
    is_prefill, index, partners = exchange.pairing(rank, world)
    partner = partners[0]
    w = make_workload(args, index if is_prefill else partner)
    s = w.shape
    mode = MODES[args.mode]
    wire_mode = mode  # exit_only and all pack as they are; dedup packs the dedup image
    planes = w.dst_planes
    kw = dict(device=device, kv_cache_dtype="fp8_e4m3" if s.fp8 else "auto")
    ptb = s.token_plane_bytes
    if args.mode == "dedup":
        pairs_on_wire = sum(int(np.minimum(np.asarray(e[lo:hi]) + 1, s.planes).sum()) for e, (lo, hi) in zip(w.exit_planes, w.ranges))
    else:
        pairs_on_wire = w.tokens * planes
    wire_bytes = pairs_on_wire * ptb
    width = -(-max(w.lengths) // s.block_size)

    table_msg = torch.zeros((len(w.lengths), planes, width), dtype=torch.int32, device=device)
    handle_msg = torch.zeros((4, exchange.HANDLE_ROW), dtype=torch.uint8, device=device)  # flag, staging 0, staging 1
    if is_prefill:
        src = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, **kw)
        bench.fill_source(src, s, workloads.SEED_BASE + index)
        if w.exit_planes is not None and args.mode == "dedup":
            # a LAST_EXITED source holds copies beyond each exit plane (what finalize leaves behind)
            tables = torch.zeros((len(w.lengths), s.planes, width), dtype=torch.int32)
            for i, r in enumerate(w.src_tables):
                for p, t in enumerate(r):
                    tables[i, p, : len(t)] = torch.from_numpy(np.asarray(t))
            rows = torch.from_numpy(np.concatenate([
                np.stack([np.full(len(e), i, np.int32), np.asarray(e, np.int32), np.arange(len(e), dtype=np.int32)], 1)
                for i, e in enumerate(w.exit_planes)])).to(device)
            view = kh.PoolView.from_tensors(src.key_cache, src.value_cache, s.planes, src.key_scale, src.value_scale)
            for at in range(0, len(rows), 1 << 16):
                kh.kv_finalize(view, tables.to(device), rows[at : at + (1 << 16)].contiguous())
        back = torch.zeros(1, dtype=torch.int64, device=device)  # "decode has consumed step k"
        handle_msg[0].copy_(exchange.encode_handles([peerlib.export_tensor(back)])[0])
    else:
        dst = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.dst_blocks, s.block_size, planes, **kw)
        for t in (dst.key_cache, dst.value_cache):
            t.view(torch.uint8).fill_(0xA5)
        random.Random(workloads.SEED_BASE + 1000 + index).shuffle(dst._free_blocks)
        reserved = [dst.reserve_transfer(f"r{i}", n) for i, n in enumerate(w.lengths)]
        table_msg.copy_(exchange.encode_tables(reserved, planes, width))
        flag = torch.zeros(1, dtype=torch.int64, device=device)
        staging = [torch.empty(wire_bytes, dtype=torch.uint8, device=device) for _ in range(2)]
        handle_msg[:3].copy_(exchange.encode_handles([peerlib.export_tensor(t) for t in (flag, *staging)]))
    all_tables, all_handles = exchange.all_gather_metadata(table_msg, handle_msg)
    torch.cuda.synchronize()

    status = kh.new_status(device)
    mapping = peerlib.PeerMapping()
    if is_prefill:
        ptrs = [mapping.pointer(e) for e in exchange.decode_handles(all_handles[partner])[:3]]
        flag_ptr, staging_ptrs = ptrs[0], ptrs[1:3]
        sv = kh.PoolView.from_cache(src)
        batch = kh.HandoffBatch(w.src_tables, None, w.ranges, block_size=s.block_size, exit_planes=w.exit_planes,
                                src_blocks=w.src_blocks, device=device)
        workspace = kh.dedup_workspace(batch, s.planes, device) if args.mode == "dedup" else None
    else:
        back_ptr = mapping.pointer(exchange.decode_handles(all_handles[partner])[0])
        dv = kh.PoolView.from_cache(dst)
        batch = kh.HandoffBatch(None, reserved, w.ranges, block_size=s.block_size,
                                exit_planes=w.exit_planes if args.mode == "dedup" else None,
                                dst_blocks=w.dst_blocks, device=device)
        workspace = kh.dedup_workspace(batch, planes, device) if args.mode == "dedup" else None
    step_no = 0

    def step():
        nonlocal step_no
        step_no += 1
        k, b = step_no, step_no % 2
        if is_prefill:
            if k > 2:  # the buffer was last used by step k - 2: wait until the decode side has scattered it
                kh.kv_wait(back.data_ptr(), k - 2, kh._lib.MAX_WAIT_NS, status)
            kh.kv_pack_to(sv, batch, staging_ptrs[b], wire_bytes, mode=wire_mode, status=status, workspace=workspace,
                          variant=args.variant)
            kh.kv_signal(flag_ptr, k)
        else:
            kh.kv_wait(flag.data_ptr(), k, kh._lib.MAX_WAIT_NS, status)
            kh.kv_scatter(staging[b], dv, batch, mode=mode if args.mode == "dedup" else kh.MODE_ALL_PLANES, status=status,
                          workspace=workspace, variant=args.variant)
            kh.kv_signal(back_ptr, k)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    kh.raise_for_status(status)
    dist.barrier()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream()
    launches0 = kh.kernel_launches()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record(stream)
    for _ in range(args.steps):
        step()
    t1.record(stream)
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    kh.raise_for_status(status)
    launches = torch.tensor([kh.kernel_launches() - launches0], device=device)
    dist.all_reduce(launches)
    total_ms = torch.tensor([t0.elapsed_time(t1)], device=device)
    dist.all_reduce(total_ms, op=dist.ReduceOp.MAX)

    # verification: every transferred row of every tensor, by checksum over NCCL
    from vllm_rlt_b200.pd import verify

    everything = list(range(len(w.lengths)))
    if is_prefill:
        verified, verified_bytes = verify.verify_over_group(src, True, [(partner, w, everything, None)], mode=args.mode, device=device)
    else:
        verified, verified_bytes = verify.verify_over_group(dst, False, [(partner, w, everything, reserved)], mode=args.mode,
                                                            device=device)
    torch.cuda.synchronize()
    dist.barrier()
    mapping.close()
    dist.barrier()
    if rank == 0:
        ms = float(total_ms.item()) / args.steps
        payload = w.payload_bytes * pairs
        line = {
            "metric": bench.METRIC, "value": payload / (ms * 1e-3) / 1e9, "unit": bench.UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": bench.config_of(w, args, {
                "split": f"{pairs}P:{pairs}D", "path": "pack into peer staging -> flag -> scatter (double buffered)",
                "wire_bytes_per_pair": wire_bytes, "payload_bytes": payload,
                "wire_fraction_of_payload": wire_bytes / w.payload_bytes}),
            "roofline": {"bound": "nvlink", "achieved": wire_bytes / (ms * 1e-3) / 1e9, "peak": bench.NVLINK_NOMINAL_GBS,
                         "unit": "GB/s", "frac": wire_bytes / (ms * 1e-3) / 1e9 / bench.NVLINK_NOMINAL_GBS, "traffic": None,
                         "peak_source": "nominal NVLink 5 rate per direction per GPU",
                         "what": "bytes that actually cross NVLink per pair / time; `value` counts the destination bytes rebuilt"},
            "per_pair_gbps": w.payload_bytes / (ms * 1e-3) / 1e9, "e2e": None,
            "gpu_launches": int(launches.item()),
            "verified": verified and verified_bytes == int(payload), "verified_bytes": verified_bytes,
        }
        print(json.dumps(line), flush=True)
    dist.destroy_process_group()
