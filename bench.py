"""KV-handoff benchmark: GB/s of the prefill->decode KV handoff on B200, with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0). A step is one pass of the handoff over the
whole synthetic batch. At N=1 the workload is the intra-device pool-to-pool
handoff of a LAST_EXITED Ouro-1.4B-shaped source (64 requests, per-token exit
planes, exit-only into a single-plane pool). Inputs are synthetic and larger
than L2, so no cache flush is needed between iterations.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "kv_handoff_gbps"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
NVLINK_MEASURED_GBS = 770.0
# link bytes per payload byte for writes over NVLink (ncu: nvltx__bytes.sum / nvltx__bytes_data_user.sum of the handoff kernel)
NVLINK_WRITE_OVERHEAD = 1.1875
# the same for read responses when the destination GPU pulls (ncu: nvlrx__bytes.sum / nvlrx__bytes_data_user.sum)
NVLINK_READ_OVERHEAD = 1.125
# DRAM traffic per algorithmic byte of table_copy_kernel, from the ncu capture summarised under profiles/
TRAFFIC_PER_ALGORITHMIC_BYTE = 0.98


# ------------------------------------------------------------------------------- helpers


def measured_peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            return float(data["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.device_index = device_index
        self.proc = None
        self.lines: list[str] = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.device_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, max_clock, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                clocks.append(float(parts[1]))
                max_clock = float(parts[2])
            except ValueError:
                continue
            for name, value in zip(names, parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(clocks) if clocks else None,
            "sm_max_mhz": max_clock,
            "samples": len(clocks),
            "reasons": sorted(reasons),
        }


def visible_device_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


# ------------------------------------------------------------------------------- workload on the GPU


def build_device_side(w, device, seed):
    """Pools on the device, source filled with N(0,1) bf16 (or random non-NaN e4m3 + U[0.01,0.1] scales)."""
    import torch

    from vllm_rlt_b200.core.kv_pool import KVPool

    s = w.shape
    kw = dict(device=device, kv_cache_dtype="fp8_e4m3" if s.fp8 else "auto")
    src = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, **kw)
    dst = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.dst_blocks, s.block_size, w.dst_planes, **kw)
    fill_source(src, s, seed)
    for t in (dst.key_cache, dst.value_cache):
        t.view(torch.uint8).fill_(0xA5)
    return src, dst


def fill_source(src, shape, seed):
    """N(0,1) bf16 values, or random e4m3 bytes without the NaN encodings plus U[0.01, 0.1] float32 scales."""
    import torch

    gen = torch.Generator(device=src.device).manual_seed(seed)
    if shape.fp8:
        for t in (src.key_cache, src.value_cache):
            raw = t.view(torch.uint8).reshape(-1)
            raw.random_(0, 256, generator=gen)
            for at in range(0, raw.numel(), 1 << 30):  # in pieces: the mask would otherwise double the footprint
                piece = raw[at : at + (1 << 30)]
                piece.masked_fill_((piece & 0x7F) == 0x7F, 0x3C)
        for t in (src.key_scale, src.value_scale):
            t.uniform_(0.01, 0.1, generator=gen)
    else:
        src.key_cache.normal_(generator=gen)
        src.value_cache.normal_(generator=gen)


def spot_check(w, src, dst, requests=None):
    """Independent check with torch indexing: destination rows equal the selected source rows.

    By default every row of every request is compared (one request at a time, so the temporaries stay small).
    """
    import numpy as np
    import torch

    ok = True
    bs = w.shape.block_size
    for r in (range(len(w.lengths)) if requests is None else requests):
        n = w.ranges[r][1]
        pos = torch.arange(n, device=src.device)
        for plane in range(w.dst_planes):
            if w.exit_planes is None:
                sp = torch.full((n,), plane, device=src.device)
            else:
                e = torch.tensor(np.asarray(w.exit_planes[r][:n]), device=src.device)
                sp = e if w.extra["mode"] == "exit_only" else torch.minimum(e, torch.full_like(e, plane))
            st = torch.tensor(np.stack(w.src_tables[r]), device=src.device)
            dt = torch.tensor(np.asarray(w.dst_tables[r][plane]), device=src.device)
            sb = st[sp, pos // bs]
            db = dt[pos // bs]
            pairs = [(src.key_cache, dst.key_cache), (src.value_cache, dst.value_cache)]
            if src.key_scale is not None:
                pairs += [(src.key_scale, dst.key_scale), (src.value_scale, dst.value_scale)]
            for a, b in pairs:
                va = a[sb, :, pos % bs].contiguous().view(torch.uint8)
                vb = b[db, :, pos % bs].contiguous().view(torch.uint8)
                ok = ok and bool(torch.equal(va, vb))
    return ok


# ------------------------------------------------------------------------------- CPU baseline (oracle)


class CpuSample:
    """The CPU restatement of the reference path on a bounded slice of the workload.

    The reference always sends every plane of a prompt (it has no exit-plane selection), so the
    sample is the all-planes handoff of the workload's first requests, cut off at ``max_tokens``
    tokens in total: Python planner (kv_segments on both sides + partition_segments, as the
    reference runs it) and a threaded memcpy of the resulting descriptors. Pools are touched
    once at set-up so that first-touch page faults stay out of the timing.
    """

    def __init__(self, w, max_tokens=1024):
        import random

        from oracle import handoff_oracle as ho

        self.ho = ho
        s = w.shape
        self.cores = len(os.sched_getaffinity(0))
        lengths, left = [], max_tokens
        for n in w.lengths:
            if left <= 0:
                break
            lengths.append(min(n, left))
            left -= lengths[-1]
        self.lengths = lengths
        blocks = sum(-(-n // s.block_size) for n in lengths) * s.planes
        kw = dict(element=s.element, fp8=s.fp8)
        self.P = ho.OraclePool(s.num_layers, s.num_kv_heads, s.head_dim, blocks, s.block_size, s.planes, base=1 << 30, **kw)
        self.D = ho.OraclePool(s.num_layers, s.num_kv_heads, s.head_dim, blocks, s.block_size, s.planes, base=1 << 44, device=1, **kw)
        rng = random.Random(1)
        self.P.shuffle_free_list(rng)
        self.D.shuffle_free_list(rng)
        for i, n in enumerate(lengths):
            assert self.P.allocate(f"r{i}", n) and self.D.allocate(f"r{i}", n)
        for pool, byte in ((self.P, 0x3C), (self.D, 0xA5)):
            for t in pool.tensors():
                t.data[...] = byte
        self.spans = sorted((t.base, t.flat.ctypes.data, t.flat.size) for pool in (self.P, self.D) for t in pool.tensors())
        self.payload = sum(ho.payload_bytes(self.P, n, s.planes) for n in lengths)
        self.plan_s = self.apply_s = 0.0
        self.reps = 0
        self.single_s = None  # one repetition with one copy thread, as a stage worker of the reference runs

    def _real(self, address):
        for base, ptr, size in self.spans:
            if base <= address < base + size:
                return ptr + (address - base)
        raise ValueError("address outside pools")

    def run_once(self, threads=None):
        import numpy as np

        from oracle import cpu_apply

        ho, P, D = self.ho, self.P, self.D
        t0 = time.perf_counter()
        triples = []
        for i, n in enumerate(self.lengths):
            src = ho.kv_segments(P.info(), P.plane_block_tables(f"r{i}"), 0, n)
            dst = ho.kv_segments(D.info(), D.plane_block_tables(f"r{i}"), 0, n)
            for local, remote, _ in ho.partition_segments(src, dst, 256 * 1024**2, 256):
                triples.extend((self._real(a), self._real(b), m) for (a, m, _), (b, _, _) in zip(local, remote))
        arr = np.array(triples, np.int64)
        t1 = time.perf_counter()
        moved = cpu_apply.apply(arr, self.cores if threads is None else threads)
        t2 = time.perf_counter()
        assert moved == self.payload
        if threads is not None:
            self.single_s = t2 - t0
            return t2 - t0
        self.plan_s += t1 - t0
        self.apply_s += t2 - t1
        self.reps += 1
        return t2 - t0

    def result(self):
        import numpy as np

        first_src = self.P.plane_block_tables("r0")[0][0]
        first_dst = self.D.plane_block_tables("r0")[0][0]
        ok = all(np.array_equal(a.data[first_src], b.data[first_dst]) for a, b in zip(self.P.tensors(), self.D.tensors()))
        total = self.plan_s + self.apply_s
        return {
            "value": self.payload * self.reps / total / 1e9,
            "unit": UNIT,
            "cores": self.cores,
            "kind": "port",
            "single_thread_value": None if self.single_s is None else self.payload / self.single_s / 1e9,
            "single_thread_note": "same sample with one copy thread: the reference's stage workers run with "
                                  "torch.set_num_threads(1) (vllm_rlt/engine/worker.py:38)",
            "sample": (f"all-planes handoff of the first {len(self.lengths)} request(s) cut at {sum(self.lengths)} tokens "
                       f"({self.payload / 1e9:.2f} GB payload), {self.reps} repetitions; Python planner "
                       f"{self.plan_s / self.reps * 1e3:.1f} ms + {self.cores}-thread memcpy {self.apply_s / self.reps * 1e3:.1f} ms "
                       f"per repetition; pools pre-touched; byte-exact: {ok}"),
        }


def cpu_baseline_sample(w, budget_s=10.0, max_tokens=1024):
    sample = CpuSample(w, max_tokens)
    t_end = time.perf_counter() + budget_s
    while sample.reps < 3 or (time.perf_counter() < t_end and sample.reps < 200):
        sample.run_once()
    sample.run_once(threads=1)
    return sample.result()


# ------------------------------------------------------------------------------- arms


def config_of(w, args, extra=None):
    c = {
        "workload": w.description,
        "requests": len(w.lengths),
        "tokens": w.tokens,
        "payload_bytes": w.payload_bytes,
        "mode": w.extra.get("mode"),
        "l2": "inputs larger than L2 (no flush needed)",
    }
    if extra:
        c.update(extra)
    return c


def run_reference(args, rank, world):
    from vllm_rlt_b200 import workloads

    if rank != 0:
        return
    w = workloads.last_exited_exit_only(requests=args.requests)
    sample = CpuSample(w, args.cpu_tokens)
    times = []
    for i in range(args.warmup + args.steps):
        if i == args.warmup:
            sample.plan_s = sample.apply_s = 0.0
            sample.reps = 0
        dt = sample.run_once()
        if i >= args.warmup:
            times.append(dt)
    sample.run_once(threads=1)
    last = sample.result()
    value = last["value"]
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": statistics.mean(times) * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
        "config": config_of(w, args), "cpu_baseline": last,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_single(args):
    import numpy as np
    import torch

    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.kernels import kv_handoff as kh

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    from vllm_rlt_b200.pd.harness import make_workload

    w = make_workload(args, 0)
    need = (w.src_blocks + w.dst_blocks) * w.shape.block_bytes
    free, _ = torch.cuda.mem_get_info()
    if need + (6 << 30) > free:
        raise SystemExit(f"workload needs {need / 2**30:.1f} GiB of pools but only {free / 2**30:.1f} GiB are free")
    src, dst = build_device_side(w, device, workloads.SEED_BASE + 1)
    mode = {"exit_only": kh.MODE_EXIT_ONLY, "dedup": kh.MODE_DEDUP, "all": kh.MODE_ALL_PLANES}[w.extra.get("mode", args.mode)]
    sv, dv = kh.PoolView.from_cache(src), kh.PoolView.from_cache(dst)
    status = kh.new_status(device)

    def make_batch():
        return kh.HandoffBatch(w.src_tables, w.dst_tables, w.ranges, block_size=w.shape.block_size,
                               exit_planes=w.exit_planes, src_blocks=w.src_blocks, dst_blocks=w.dst_blocks, device=device)

    batch = make_batch()
    stream = torch.cuda.current_stream()

    def step():
        kh.kv_handoff(sv, dv, batch, mode=mode, status=status, variant=args.variant)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    kh.raise_for_status(status)

    sampler = ClockSampler(visible_device_index(0))
    sampler.start()
    time.sleep(0.3)
    launches0 = kh.kernel_launches()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    torch.cuda.synchronize()
    t_begin = torch.cuda.Event(enable_timing=True)
    t_end = torch.cuda.Event(enable_timing=True)
    t_begin.record(stream)
    for a, b in events:
        a.record(stream)
        step()
        b.record(stream)
    t_end.record(stream)
    torch.cuda.synchronize()
    launches = kh.kernel_launches() - launches0
    total_ms = t_begin.elapsed_time(t_end)
    kernel_ms = [a.elapsed_time(b) for a, b in events]
    clocks = sampler.stop()
    kh.raise_for_status(status)
    verified = spot_check(w, src, dst)

    ms_per_step = total_ms / args.steps
    value = w.payload_bytes / (ms_per_step * 1e-3) / 1e9
    peak, peak_note = measured_peaks()
    avg_kernel_ms = statistics.mean(kernel_ms)
    # bytes the algorithm must move: every destination row is written once; a source row is read once per
    # distinct (token, plane) it feeds - in dedup mode the planes beyond a token's exit plane re-use one row
    read_bytes = w.payload_bytes
    if w.extra.get("mode") == "dedup":
        distinct = sum(int(np.minimum(np.asarray(e[lo:hi]) + 1, w.dst_planes).sum()) for e, (lo, hi) in zip(w.exit_planes, w.ranges))
        read_bytes = distinct * w.shape.token_plane_bytes
    algorithmic = read_bytes + w.payload_bytes
    achieved = algorithmic / (avg_kernel_ms * 1e-3) / 1e9

    # end to end through the public API: host tables -> pinned -> device, launch, status read back
    e2e_times = []
    for i in range(args.warmup + args.steps):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        b = make_batch()
        kh.kv_handoff(sv, dv, b, mode=mode, status=status, variant=args.variant)
        kh.raise_for_status(status)  # device -> host read of the status words; synchronises
        if i >= args.warmup:
            e2e_times.append(time.perf_counter() - t0)
    e2e_value = w.payload_bytes / statistics.mean(e2e_times) / 1e9

    # per-request latency: one launch per request, device timed
    lat = []
    for r in range(len(w.lengths)):
        one = workloads.subset(w, [r])
        b = kh.HandoffBatch(one.src_tables, one.dst_tables, one.ranges, block_size=w.shape.block_size,
                            exit_planes=one.exit_planes, device=device)
        kh.kv_handoff(sv, dv, b, mode=mode, status=status, variant=args.variant)  # warm
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        kh.kv_handoff(sv, dv, b, mode=mode, status=status, variant=args.variant)
        z.record(stream)
        torch.cuda.synchronize()
        lat.append(a.elapsed_time(z))
    kh.raise_for_status(status)

    # the streaming tail of one request: what is left to send after its last layer (one layer slice)
    tail = []
    one = workloads.subset(w, [0])
    b = kh.HandoffBatch(one.src_tables, one.dst_tables, one.ranges, block_size=w.shape.block_size,
                        exit_planes=one.exit_planes, device=device)
    last = w.shape.num_layers - 1
    for _ in range(12):
        a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(stream)
        kh.kv_handoff(sv, dv, b, mode=mode, layer_begin=last, layer_end=last + 1, status=status, variant=args.variant)
        z.record(stream)
        torch.cuda.synchronize()
        tail.append(a.elapsed_time(z))
    kh.raise_for_status(status)

    cpu = None if args.no_cpu_baseline else cpu_baseline_sample(w, max_tokens=args.cpu_tokens)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8", "data": "synthetic", "config": config_of(w, args, {"variant": args.variant}),
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": TRAFFIC_PER_ALGORITHMIC_BYTE * algorithmic, "peak_source": peak_note,
                     "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum of a 2-request capture of the same "
                                       "kernel (traffic / algorithmic = 0.98), scaled by tokens",
                     "kernel": "table_fan_kernel" if w.extra.get("mode") == "dedup" and args.variant & 0xf not in (3, 4, 6) else "table_copy_kernel",
                     "algorithmic_bytes_per_launch": algorithmic, "kernel_ms": avg_kernel_ms},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": batch.metadata_bytes,
                "d2h_bytes_per_step": 16, "ms_per_step": statistics.mean(e2e_times) * 1e3,
                "note": "KV pools are device-resident by the API's nature; host inputs are tables, ranges and exit planes"},
        "latency_ms": {"p50": statistics.median(lat), "max": max(lat), "min": min(lat),
                       "what": "one launch per request, CUDA events, intra-device",
                       "last_layer_slice_p50": statistics.median(tail),
                       "tokens_p50": statistics.median(w.lengths)},
        "gpu_launches": launches, "clocks": clocks, "verified": verified,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--mode", default="exit_only", choices=["exit_only", "dedup", "all"])
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--cpu-tokens", type=int, default=1024)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--prefill", type=int, default=0, help="prefill ranks at N >= 2 (default N/2)")
    ap.add_argument("--workload", default="ouro1p4b",
                    choices=["ouro1p4b", "ouro2p6b", "ouro2p6b_fp8_shared", "huginn", "huginn_recurrent", "ouro2p6b_chunk", "ouro2p6b_4k",
                             "ouro2p6b_fp8_4k"])
    ap.add_argument("--streaming", action="store_true", help="also replay a layer-by-layer prefill and stream behind it")
    ap.add_argument("--layer-us", type=float, default=200.0, help="simulated prefill time per layer and depth")
    ap.add_argument("--layers-per-slice", type=int, default=4)
    ap.add_argument("--direction", default="pull", choices=["push", "pull"],
                    help="N >= 2, direct path: the prefill GPU writes into the decode pool, or the decode GPU reads the prefill pool")
    ap.add_argument("--path", default="direct", choices=["direct", "staged"],
                    help="N >= 2: one kernel that writes destination blocks over NVLink, or pack into peer staging + scatter")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world == 1 and args.gpus == 1:
        run_single(args)
    else:
        if args.path == "staged":
            from vllm_rlt_b200.pd import staged

            staged.run_staged(args, rank, world)
        elif args.direction == "pull" and not args.streaming:
            from vllm_rlt_b200.pd import pull_harness

            pull_harness.run_pull(args, rank, world)
        else:
            from vllm_rlt_b200.pd import harness

            harness.run_multi(args, rank, world)


if __name__ == "__main__":
    main()
