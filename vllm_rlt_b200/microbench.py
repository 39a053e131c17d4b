"""Times every kernel of the library on one GPU with synthetic inputs and prints one JSON line per kernel.

    python -m vllm_rlt_b200.microbench [--requests 8]

Bytes are the algorithmic bytes each kernel must move (read + written); rates are to be read against the
HBM copy peak of the device. The headline handoff kernel is measured by ``bench.py``; this covers the rest:
pack, scatter, the dedup wire (plan + pack, plan + rebuilding scatter), finalize, segment copy, push and the
typed tensor transfers.
"""

from __future__ import annotations

import argparse
import json
import statistics

import numpy as np
import torch


def timed(fn, reps=7, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


def report(name, nbytes, ms, **extra):
    print(json.dumps(dict(kernel=name, algorithmic_bytes=int(nbytes), ms=round(ms, 4), gbps=round(nbytes / ms / 1e6, 1), **extra)), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=8)
    args = ap.parse_args()

    from . import workloads
    from .core.kv_pool import KVPool
    from .kernels import kv_handoff as kh
    from .worker.tensors import TensorTransfer, copy_tensor

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = workloads.last_exited_exit_only(requests=args.requests, mode="dedup")
    s = w.shape
    src = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, device=dev)
    dst = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.dst_blocks, s.block_size, s.planes, device=dev)
    src.key_cache.normal_()
    src.value_cache.normal_()
    sv, dv = kh.PoolView.from_cache(src), kh.PoolView.from_cache(dst)
    status = kh.new_status(dev)
    batch = kh.HandoffBatch(w.src_tables, w.dst_tables, w.ranges, block_size=s.block_size, exit_planes=w.exit_planes, device=dev)
    tokens, ptb = w.tokens, s.token_plane_bytes
    exits = np.concatenate(w.exit_planes)
    pairs = int((exits + 1).sum())

    # finalize first: it makes the planes beyond each exit plane copies, which dedup relies on
    width = batch.table_width
    tables = torch.zeros((len(w.lengths), s.planes, width), dtype=torch.int32)
    for i, r in enumerate(w.src_tables):
        for p, t in enumerate(r):
            tables[i, p, : len(t)] = torch.from_numpy(np.asarray(t))
    tables = tables.to(dev)
    rows = torch.from_numpy(np.concatenate([
        np.stack([np.full(len(e), i, np.int32), np.asarray(e, np.int32), np.arange(len(e), dtype=np.int32)], 1)
        for i, e in enumerate(w.exit_planes)])).to(dev)
    copies = int((s.planes - 1 - exits).sum())
    ms = timed(lambda: kh.kv_finalize(sv, tables, rows, status=status))
    sources = int((exits < s.planes - 1).sum())
    report("finalize_fan_kernel", (sources + copies) * ptb, ms, rows=len(rows), source_rows=sources, copied_rows=copies,
           note="each exit row with deeper planes is read once and written once per deeper plane")

    full = kh.packed_bytes(sv, tokens, s.planes)
    packed = torch.empty(full, dtype=torch.uint8, device=dev)
    ms = timed(lambda: kh.kv_pack(sv, batch, packed, status=status))
    report("table_copy_kernel pack all planes", 2 * full, ms)
    ms = timed(lambda: kh.kv_scatter(packed, dv, batch, status=status))
    report("table_copy_kernel scatter all planes", 2 * full, ms)
    ws = kh.dedup_workspace(batch, s.planes, dev)
    wire = pairs * ptb
    ms = timed(lambda: kh.kv_pack(sv, batch, packed, mode=kh.MODE_DEDUP, status=status, workspace=ws))
    report("dedup plan (3 kernels) + table_copy_kernel pack dedup", 2 * wire, ms, wire_fraction=round(wire / full, 3))
    ms = timed(lambda: kh.kv_scatter(packed[:wire], dv, batch, mode=kh.MODE_DEDUP, status=status, workspace=ws))
    report("dedup plan (3 kernels) + table_fan_kernel scatter dedup", wire + full, ms,
           note="reads the wire image once, writes every plane")
    kh.raise_for_status(status)

    # explicit ranges
    block = src.key_cache.stride(0) * 2
    blocks = min(256, w.src_blocks, w.dst_blocks)
    segs = torch.tensor([(src.key_cache.data_ptr() + i * block, dst.key_cache.data_ptr() + (blocks - 1 - i) * block, block)
                         for i in range(blocks)], dtype=torch.int64, device=dev)
    ms = timed(lambda: kh.kv_copy_segments(segs))
    report("segment_copy_kernel (256 block-sized ranges)", 2 * blocks * block, ms)
    n = min(1 << 30, src.key_cache.numel() * 2)
    ms = timed(lambda: kh.kv_push(src.key_cache.data_ptr(), dst.key_cache.data_ptr(), n))
    report("push_kernel (one range)", 2 * n, ms)

    # typed transfers
    ids = torch.randint(0, 2**40, (1 << 26,), dtype=torch.int64, device=dev)
    out32 = torch.empty(1 << 26, dtype=torch.int32, device=dev)
    ms = timed(lambda: copy_tensor(ids, out32))
    report("flat_transfer_kernel int64 -> int32", (8 + 4) << 26, ms)
    hidden = torch.randn(4096, 2048, device=dev, dtype=torch.bfloat16)
    staged = torch.empty(4096, 2048, device=dev, dtype=torch.bfloat16)
    tt = TensorTransfer(64, torch.bfloat16, dev)
    for i in range(64):
        tt.append(hidden[i * 64 : (i + 1) * 64], staged[(63 - i) * 64 : (64 - i) * 64])
    ms = timed(tt.submit)
    report("segmented_transfer_kernel (64 copies of 64 x 2048 bf16)", 2 * hidden.numel() * 2, ms)


if __name__ == "__main__":
    main()
