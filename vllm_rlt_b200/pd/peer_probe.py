"""One process, two GPUs: hand a small batch from a pool on ``cuda:0`` to a pool on ``cuda:1`` over NVLink.

    python -m vllm_rlt_b200.pd.peer_probe [--requests 2]

The smallest cross-GPU use of the library (peer access enabled inside one process, no IPC, no flags). It prints
the device-timed rate and checks the destination; it is also the program to put under a profiler to see the
link counters of the handoff kernel, since it has a single rank and nothing waits on anything.
"""

from __future__ import annotations

import argparse
import json
import statistics


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--mode", default="exit_only", choices=["exit_only", "all", "dedup"])
    ap.add_argument("--variant", type=int, default=0, help="kernel flavour (RltOptions.variant)")
    ap.add_argument("--pull", action="store_true", help="run the kernel on the destination GPU and read the source over the link")
    args = ap.parse_args()

    import torch

    import bench
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd import peer

    if torch.cuda.device_count() < 2:
        raise SystemExit("needs two GPUs")
    peer.enable_peer_access(0, 1)
    peer.enable_peer_access(1, 0)
    run_on = 1 if args.pull else 0
    torch.cuda.set_device(0)
    w = workloads.last_exited_exit_only(requests=args.requests, mode=args.mode)
    s = w.shape
    src = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, device="cuda:0")
    dst = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.dst_blocks, s.block_size, w.dst_planes, device="cuda:1")
    bench.fill_source(src, s, 3)
    for t in (dst.key_cache, dst.value_cache):
        t.view(torch.uint8).fill_(0xA5)
    torch.cuda.synchronize(1)
    sv, dv = kh.PoolView.from_cache(src), kh.PoolView.from_cache(dst)
    torch.cuda.synchronize(0)
    torch.cuda.set_device(run_on)
    batch = kh.HandoffBatch(w.src_tables, w.dst_tables, w.ranges, block_size=s.block_size, exit_planes=w.exit_planes,
                            device=f"cuda:{run_on}")
    status = kh.new_status(f"cuda:{run_on}")
    mode = {"exit_only": kh.MODE_EXIT_ONLY, "all": kh.MODE_ALL_PLANES, "dedup": kh.MODE_DEDUP}[args.mode]
    times = []
    for i in range(1 + args.steps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        kh.kv_handoff(sv, dv, batch, mode=mode, status=status, variant=args.variant)
        b.record()
        torch.cuda.synchronize(run_on)
        if i:
            times.append(a.elapsed_time(b))
    kh.raise_for_status(status)
    torch.cuda.set_device(0)
    # compare on the destination device: bring the expected rows of request 0 over with a plain copy
    n = min(64, w.lengths[0])
    import numpy as np

    pos = torch.arange(n, device="cuda:0")
    e = torch.tensor(np.asarray(w.exit_planes[0][:n]), device="cuda:0").long() if w.exit_planes is not None else None
    ok = True
    for plane in range(w.dst_planes):
        sp = e if args.mode == "exit_only" else torch.clamp(e, max=plane) if args.mode == "dedup" else torch.full((n,), plane, device="cuda:0")
        st = torch.tensor(np.stack([np.asarray(t) for t in w.src_tables[0]]), device="cuda:0").long()
        want = src.key_cache[st[sp, pos // s.block_size], :, pos % s.block_size].to("cuda:1")
        db = torch.tensor(np.asarray(w.dst_tables[0][plane]), device="cuda:1").long()[(pos // s.block_size).to("cuda:1")]
        got = dst.key_cache[db, :, (pos % s.block_size).to("cuda:1")]
        ok = ok and bool(torch.equal(want.view(torch.int16), got.view(torch.int16)))
    ms = statistics.median(times)
    # bytes that must cross the link: in dedup mode with the kernel on the destination GPU, rows up to each exit plane
    link = w.payload_bytes
    if args.mode == "dedup" and args.pull:
        link = sum(int(np.minimum(np.asarray(x[lo:hi]) + 1, w.dst_planes).sum()) for x, (lo, hi) in zip(w.exit_planes, w.ranges)) * s.token_plane_bytes
    print(json.dumps({"link_bytes": link, "direction": "pull (kernel on the destination GPU)" if args.pull else "push (kernel on the source GPU)",
                      "payload_bytes": w.payload_bytes, "ms": ms, "gbps": w.payload_bytes / ms / 1e6, "verified": ok}), flush=True)


if __name__ == "__main__":
    main()
