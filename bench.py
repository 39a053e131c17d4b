"""KV-handoff benchmark: GB/s of the prefill->decode KV handoff on B200, with roofline and CPU baseline.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One JSON line on stdout (rank 0). A step is one pass of the handoff over the
whole synthetic batch. At N=1 the workload is the intra-device pool-to-pool
handoff of a LAST_EXITED Ouro-1.4B-shaped source (64 requests, per-token exit
planes, exit-only into a single-plane pool). Inputs are synthetic and larger
than L2, so no cache flush is needed between iterations.

Other measurements share the workloads and helpers of this file and print their own JSON lines; they are
not the benchmark line:

    python bench.py --suite kernels [--requests 8]      every other kernel of the library on one GPU
    python bench.py --suite peer [--pull] [--mode ...] [--workload huginn]   one process, two GPUs: the kernel over NVLink
    python bench.py --suite deployment [...]            a vllm-rlt 1P:1D deployment with this connector swapped in
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
# NVLink 5, one direction, per GPU. The nominal figure is what the fractions are quoted against; the other is one
# builder-run peer-to-peer memcpy on a B200 pair, kept for context only (it is not a driver-written peak).
NVLINK_NOMINAL_GBS = 900.0
NVLINK_PEER_MEMCPY_GBS = 770.0
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
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, an earlier STREAM-style copy measurement on B200)"


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


def reference_checkout():
    """A vllm-rlt source tree that travelled with this repository, or None.

    ``$VLLM_RLT_REFERENCE`` if set (and nothing else then), else ``baseline/_ref/src`` under this file (a
    git-ignored, unmodified copy). Only its planner is imported (plain Python, no NIXL, no GPU).
    """
    candidate = os.environ.get("VLLM_RLT_REFERENCE") or str(ROOT / "baseline" / "_ref" / "src")
    if (Path(candidate) / "vllm_rlt" / "pd" / "transport.py").is_file():
        return Path(candidate)
    return None


def cpu_planner():
    """(kv_segments, partition_segments, kind, what): the reference's own planner when a checkout is present
    (vllm_rlt/pd/transport.py:29-112), else the restatement of it under ``oracle/``."""
    checkout = reference_checkout()
    if checkout is not None:
        sys.path.insert(0, str(checkout))
        try:
            from vllm_rlt.pd.transport import kv_segments, partition_segments

            return kv_segments, partition_segments, "reference", "the reference's kv_segments / partition_segments (imported from its source tree)"
        except Exception as exc:  # a broken checkout must not take the baseline down with it
            note = f"reference checkout found but not importable ({type(exc).__name__}); "
        finally:
            sys.path.remove(str(checkout))
    else:
        note = ""
    from oracle import handoff_oracle as ho

    return ho.kv_segments, ho.partition_segments, "port", note + "the restatement of kv_segments / partition_segments under oracle/"


class CpuSample:
    """The reference's CPU path on a bounded slice of the workload.

    The reference always sends every plane of a prompt (it has no exit-plane selection), so the
    sample is the all-planes handoff of the workload's first requests, cut off at ``max_tokens``
    tokens in total: the Python planner as the reference runs it (kv_segments on both sides +
    partition_segments at the reference's limits of 256 MiB and 256 descriptors) and a threaded
    memcpy of the resulting descriptors, which stands in for the NIXL WRITE (third-party, absent).
    Pools are touched once at set-up so that first-touch page faults stay out of the timing.
    """

    def __init__(self, w, max_tokens=1024):
        import random

        from oracle import handoff_oracle as ho

        self.ho = ho
        self.kv_segments, self.partition_segments, self.kind, self.planner_note = cpu_planner()
        s = w.shape
        self.shape = s
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

        P, D = self.P, self.D
        t0 = time.perf_counter()
        triples = []
        for i, n in enumerate(self.lengths):
            src = self.kv_segments(P.info(), P.plane_block_tables(f"r{i}"), 0, n)
            dst = self.kv_segments(D.info(), D.plane_block_tables(f"r{i}"), 0, n)
            for local, remote, _ in self.partition_segments(src, dst, 256 * 1024**2, 256):
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

    def description(self) -> str:
        return (f"all planes (the reference carries every plane), the first {len(self.lengths)} request(s) of the workload "
                f"cut at {sum(self.lengths)} tokens")

    def config(self, w) -> dict:
        """What this arm really moved per step, with the full workload it was cut from beside it."""
        return {
            "workload": w.description,
            "sample": self.description(),
            "requests": len(self.lengths),
            "tokens": sum(self.lengths),
            "payload_bytes": self.payload,
            "mode": "all",
            "l2": "sample larger than the host caches",
            "cut_from": {"requests": len(w.lengths), "tokens": w.tokens, "payload_bytes": w.payload_bytes,
                         "mode": w.extra.get("mode")},
        }

    def result(self):
        import numpy as np

        first_src = self.P.plane_block_tables("r0")[0][0]
        first_dst = self.D.plane_block_tables("r0")[0][0]
        ok = all(np.array_equal(a.data[first_src], b.data[first_dst]) for a, b in zip(self.P.tensors(), self.D.tensors()))
        total = self.plan_s + self.apply_s
        single = None if self.single_s is None else self.payload / self.single_s / 1e9
        return {
            "value": self.payload * self.reps / total / 1e9,
            "unit": UNIT,
            "cores": self.cores,
            "kind": self.kind,
            "planner": self.planner_note,
            "sample_bytes": self.payload,
            "single_thread_value": single,
            "reference_worker_setting": "single_thread_value: a stage worker of the reference runs with "
                                        "torch.set_num_threads(1) (vllm_rlt/engine/worker.py:38); `value` gives the CPU "
                                        f"every host core ({self.cores} copy threads), which the reference never does, so "
                                        "ratios against `value` are a floor",
            "sample": (f"{self.description()} ({self.payload / 1e9:.2f} GB payload), {self.reps} repetitions; Python planner "
                       f"{self.plan_s / self.reps * 1e3:.1f} ms + {self.cores}-thread memcpy {self.apply_s / self.reps * 1e3:.1f} ms "
                       f"per repetition; the memcpy stands in for the NIXL WRITE; pools pre-touched; byte-exact: {ok}"),
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
        "config": sample.config(w), "cpu_baseline": last,
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
        "p50_latency_ms": statistics.median(lat),
        "latency_ms": {"p50": statistics.median(lat), "max": max(lat), "min": min(lat),
                       "what": "one launch per request, CUDA events, intra-device",
                       "last_layer_slice_p50": statistics.median(tail),
                       "tokens_p50": statistics.median(w.lengths)},
        "gpu_launches": launches, "clocks": clocks, "verified": verified,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------- other measurements


def _timed(fn, reps=5, warm=2, inner=8):
    """Median device time of one ``fn()`` launch. ``inner`` launches are queued back to back behind a short
    sleep kernel, so the GPU is never waiting for the host: a Python wrapper takes tens of microseconds per call,
    which would otherwise be billed to a kernel that runs for a hundred."""
    import torch

    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(600_000)
        a.record()
        for _ in range(inner):
            fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b) / inner)
    return statistics.median(out)


def suite_kernels(args):
    """Every kernel of the library other than the headline handoff, on one GPU: one JSON line each.

    Bytes are the algorithmic bytes a kernel must move (read + written); ``frac`` is that rate over the HBM
    copy peak. Inputs are far larger than L2; timings are CUDA events around eight back-to-back launches
    (median of 5 such groups after 2 warm-ups).
    """
    import numpy as np
    import torch

    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.worker.tensors import TensorTransfer, copy_tensor

    peak, peak_note = measured_peaks()
    only = set(args.only.split(",")) if args.only else None

    def wanted(tag):
        return only is None or tag in only

    def report(tag, name, nbytes, ms, **extra):
        gbps = nbytes / ms / 1e6
        print(json.dumps(dict(suite="kernels", tag=tag, kernel=name, algorithmic_bytes=int(nbytes), ms=round(ms, 4),
                              gbps=round(gbps, 1), frac=round(gbps / peak, 4), peak=peak, peak_source=peak_note, **extra)),
              flush=True)

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    w = workloads.last_exited_exit_only(requests=args.requests if args.requests != 64 else 8, mode="dedup")
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
        for plane, t in enumerate(r):
            tables[i, plane, : len(t)] = torch.from_numpy(np.asarray(t))
    tables = tables.to(dev)
    rows = torch.from_numpy(np.concatenate([
        np.stack([np.full(len(e), i, np.int32), np.asarray(e, np.int32), np.arange(len(e), dtype=np.int32)], 1)
        for i, e in enumerate(w.exit_planes)])).to(dev)
    copies = int((s.planes - 1 - exits).sum())
    sources = int((exits < s.planes - 1).sum())
    if wanted("finalize"):
        # Finalize writes two to three rows for each one it reads, and HBM takes writes more slowly than the mix of
        # the copy the peak was measured with. The same volume as pure writes (the library memset) is timed first;
        # each finalize line carries its own write rate next to it.
        scratch = dst.key_cache.view(torch.uint8).reshape(-1)
        size = min(scratch.numel(), 3 << 30)
        ms = _timed(lambda: scratch[:size].zero_())
        write_rate = size / ms / 1e6
        report("finalize", "context: Tensor.zero_ of 3 GiB (writes only)", size, ms)

        def finalize_line(name, read_rows, written_rows, ms, **extra):
            written = written_rows * ptb / ms / 1e6
            report("finalize", name, (read_rows + written_rows) * ptb, ms, written_gbps=round(written, 1),
                   memset_write_gbps=round(write_rate, 1), written_over_memset=round(written / write_rate, 3), **extra)

        ms = _timed(lambda: kh.kv_finalize(sv, tables, rows, status=status))
        finalize_line("finalize_fan_kernel", sources, copies, ms, rows=len(rows), source_rows=sources, copied_rows=copies,
                      note="each exit row with deeper planes is read once and written once per deeper plane")
        # the same launch with every token leaving at plane 0: whole pages read from one block and written to three,
        # no holes on any plane - separates the cost of the scattered pattern above from the kernel's own
        dense = rows.clone()
        dense[:, 1] = 0
        ms = _timed(lambda: kh.kv_finalize(sv, tables, dense, status=status))
        finalize_line("finalize_fan_kernel, every token exits at plane 0 (dense pages)", len(rows),
                      len(rows) * (s.planes - 1), ms, rows=len(rows))
        # and with every token leaving at plane 1: the same 1 : 2 mix of reads and writes as the U{0..3} launch, on whole pages
        dense[:, 1] = 1
        ms = _timed(lambda: kh.kv_finalize(sv, tables, dense, status=status))
        finalize_line("finalize_fan_kernel, every token exits at plane 1 (dense pages, 1 read : 2 writes)", len(rows),
                      len(rows) * (s.planes - 2), ms, rows=len(rows))
        kh.kv_finalize(sv, tables, rows, status=status)  # restore the copies the dedup measurements below rely on
        few = rows[:256].contiguous()  # what one decode step finalizes
        ms = _timed(lambda: kh.kv_finalize(sv, tables, few, status=status))
        fe = exits[:256]
        finalize_line("finalize_fan_kernel (256 rows, one decode step)", int((fe < s.planes - 1).sum()),
                      int((s.planes - 1 - fe).sum()), ms, rows=256)
    else:
        kh.kv_finalize(sv, tables, rows, status=status)

    full = kh.packed_bytes(sv, tokens, s.planes)
    packed = torch.empty(full, dtype=torch.uint8, device=dev)
    wire = pairs * ptb
    if wanted("pack"):
        ms = _timed(lambda: kh.kv_pack(sv, batch, packed, status=status))
        report("pack", "table_copy_kernel pack all planes", 2 * full, ms)
        ms = _timed(lambda: kh.kv_scatter(packed, dv, batch, status=status))
        report("pack", "table_copy_kernel scatter all planes", 2 * full, ms)
        ws = kh.dedup_workspace(batch, s.planes, dev)
        ms = _timed(lambda: kh.kv_pack(sv, batch, packed, mode=kh.MODE_DEDUP, status=status, workspace=ws))
        report("pack", "dedup plan (3 kernels) + table_copy_kernel pack dedup", 2 * wire, ms, wire_fraction=round(wire / full, 3))
        ms = _timed(lambda: kh.kv_scatter(packed[:wire], dv, batch, mode=kh.MODE_DEDUP, status=status, workspace=ws))
        report("pack", "dedup plan (3 kernels) + table_fan_kernel scatter dedup", wire + full, ms,
               note="reads the wire image once, writes every plane")
    kh.raise_for_status(status)

    if wanted("segments"):
        block = src.key_cache.stride(0) * 2
        blocks = min(256, w.src_blocks, w.dst_blocks)
        segs = torch.tensor([(src.key_cache.data_ptr() + i * block, dst.key_cache.data_ptr() + (blocks - 1 - i) * block, block)
                             for i in range(blocks)], dtype=torch.int64, device=dev)
        ms = _timed(lambda: kh.kv_copy_segments(segs))
        report("segments", "segment_copy_kernel (256 block-sized ranges)", 2 * blocks * block, ms)
        # the reference planner's mix for a request that ends mid-block: full blocks next to per-layer partial rows
        mixed = []
        for i in range(blocks):
            a, b = src.key_cache.data_ptr() + i * block, dst.key_cache.data_ptr() + (blocks - 1 - i) * block
            if i % 8 == 7:
                layer = block // s.num_layers
                mixed += [(a + l * layer, b + l * layer, 5 * s.num_kv_heads * s.head_dim * 2) for l in range(s.num_layers)]
            else:
                mixed.append((a, b, block))
        mixed = mixed[: kh._lib.MAX_SEGMENTS]
        mseg = torch.tensor(mixed, dtype=torch.int64, device=dev)
        ms = _timed(lambda: kh.kv_copy_segments(mseg))
        report("segments", f"segment_copy_kernel ({len(mixed)} ranges, 1.5 MiB blocks mixed with 20 KiB partial rows)",
               2 * sum(m[2] for m in mixed), ms)
        n = min(1 << 30, src.key_cache.numel() * 2)
        ms = _timed(lambda: kh.kv_push(src.key_cache.data_ptr(), dst.key_cache.data_ptr(), n))
        report("segments", "push_kernel (one range)", 2 * n, ms)
        # context for launches this short: a plain device-to-device copy of the same sizes (the HBM peak in
        # MEASURED_PEAKS.json is the same operation on 2 GiB, where ramp-up and tail weigh less)
        flat_a, flat_b = src.key_cache.view(torch.uint8).reshape(-1), dst.key_cache.view(torch.uint8).reshape(-1)
        for size, label in ((n, "1 GiB"), (blocks * block, "the 256 blocks' bytes")):
            size = min(size, flat_a.numel(), flat_b.numel())
            ms = _timed(lambda: flat_b[:size].copy_(flat_a[:size]))
            report("segments", f"context: Tensor.copy_ of {label}, contiguous", 2 * size, ms)

    if wanted("tensors"):
        ids = torch.randint(0, 2**40, (1 << 26,), dtype=torch.int64, device=dev)
        out32 = torch.empty(1 << 26, dtype=torch.int32, device=dev)
        ms = _timed(lambda: copy_tensor(ids, out32))
        report("tensors", "flat_transfer_kernel int64 -> int32", (8 + 4) << 26, ms)
        h = torch.randn(1 << 28, device=dev, dtype=torch.bfloat16)
        h2 = torch.empty_like(h)
        ms = _timed(lambda: copy_tensor(h, h2))
        report("tensors", "flat_transfer_kernel bf16 -> bf16", 4 << 28, ms)
        hidden = torch.randn(4096, 2048, device=dev, dtype=torch.bfloat16)
        staged = torch.empty(4096, 2048, device=dev, dtype=torch.bfloat16)
        tt = TensorTransfer(64, torch.bfloat16, dev)
        for i in range(64):
            tt.append(hidden[i * 64 : (i + 1) * 64], staged[(63 - i) * 64 : (64 - i) * 64])
        ms = _timed(tt.submit)
        report("tensors", "segmented_transfer_kernel (64 copies of 64 x 2048 bf16)", 2 * hidden.numel() * 2, ms,
               note="metadata-sized: launch latency, not bandwidth")


def suite_peer(args):
    """One process, two GPUs: a small batch from a pool on cuda:0 to a pool on cuda:1 over NVLink.

    The smallest cross-GPU use of the library (peer access enabled inside one process, no IPC, no flags); also the
    program to put under a profiler for the link counters of the handoff kernel, since it has a single rank and
    nothing waits on anything. ``--pull`` runs the kernel on the destination GPU.
    """
    import numpy as np
    import torch

    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.core.kv_pool import KVPool
    from vllm_rlt_b200.kernels import kv_handoff as kh
    from vllm_rlt_b200.pd import peer, verify

    if torch.cuda.device_count() < 2:
        raise SystemExit("needs two GPUs")
    peer.enable_peer_access(0, 1)
    peer.enable_peer_access(1, 0)
    run_on = 1 if args.pull else 0
    torch.cuda.set_device(0)
    requests = args.requests if args.requests != 64 else 2
    if args.workload == "huginn":  # 32 planes, 10,560-byte rows; short prompts keep the pools at a few GB
        w = workloads.recurrent_depth_dedup(lengths=[min(args.tokens, 1024)] * requests)
        args.mode = "dedup"
    else:
        w = workloads.last_exited_exit_only(requests=requests, mode=args.mode)
    s = w.shape
    src = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.src_blocks, s.block_size, s.planes, device="cuda:0")
    dst = KVPool(s.num_layers, s.num_kv_heads, s.head_dim, w.dst_blocks, s.block_size, w.dst_planes, device="cuda:1")
    fill_source(src, s, 3)
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
    for i in range(1 + max(args.steps, 3)):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        kh.kv_handoff(sv, dv, batch, mode=mode, status=status, variant=args.variant)
        b.record()
        torch.cuda.synchronize(run_on)
        if i:
            times.append(a.elapsed_time(b))
    kh.raise_for_status(status)
    # every row of every request: checksums of the selected source rows on cuda:0 against the destination's on cuda:1
    torch.cuda.set_device(0)
    want = verify.source_checksums(src, w, range(len(w.lengths)), args.mode)
    torch.cuda.set_device(1)
    got, clean = verify.destination_checksums(dst, w, range(len(w.lengths)), [w.dst_tables[i] for i in range(len(w.lengths))])
    ok = bool(torch.equal(want.cpu(), got.cpu())) and clean
    ms = statistics.median(times)
    link = w.payload_bytes
    if args.mode == "dedup" and args.pull:
        link = sum(int(np.minimum(np.asarray(x[lo:hi]) + 1, w.dst_planes).sum()) for x, (lo, hi) in zip(w.exit_planes, w.ranges)) * s.token_plane_bytes
    print(json.dumps({"suite": "peer", "workload": w.description, "link_bytes": link,
                      "direction": "pull (kernel on the destination GPU)" if args.pull else "push (kernel on the source GPU)",
                      "payload_bytes": w.payload_bytes, "ms": ms, "gbps": w.payload_bytes / ms / 1e6,
                      "link_gbps": link / ms / 1e6, "frac_of_nominal_900": link / ms / 1e6 / NVLINK_NOMINAL_GBS,
                      "verified": ok, "verified_bytes": verify.checked_bytes(w, range(len(w.lengths)))}), flush=True)


def suite_deployment(args):
    """A real vllm-rlt 1P:1D deployment with this handoff swapped in; reports per-request handoff latency.

    The deployment is the reference's own ``PDEngine`` (coordinator, stage workers, scheduler, model runner, a
    random-initialised Ouro-1.4B-shaped model); only the connector is replaced (``dropin.install()``). The
    vllm-rlt source tree must have travelled with this repository (see ``reference_checkout``); nothing of it is part
    of this repository. Latencies come from the coordinator's timing marks (vllm_rlt/pd/engine.py:198-240):
    tail = ``d_received - prefill_compute_completed``, total = ``d_received - prefill_started``.
    """
    import random

    checkout = reference_checkout()
    if checkout is None:
        print(json.dumps({"suite": "deployment", "unavailable": "no vllm-rlt source tree travelled with the repository"}), flush=True)
        return
    sys.path.insert(0, str(checkout))
    os.environ["PYTHONPATH"] = os.pathsep.join([str(checkout), str(ROOT), os.environ.get("PYTHONPATH", "")])
    os.environ.setdefault("RLT_KV_DIRECTION", args.direction)
    if args.stream:  # the prefill worker reports its KV writes layer by layer (vllm_rlt_b200/pd/layer_watch.py)
        os.environ["RLT_KV_STREAM"] = "alternate" if args.stream == "alternate" else "1"
    from vllm_rlt import CacheConfig, SamplingParams, SchedulerConfig
    from vllm_rlt.models.ouro import OuroConfig
    from vllm_rlt.pd.config import PDConfig

    from vllm_rlt_b200.pd import dropin

    dropin.install()
    from vllm_rlt.pd.engine import PDEngine

    config = OuroConfig()  # the defaults are the Ouro-1.4B shape: 24 layers, 16 KV heads, head_dim 128, 4 loops
    cache = CacheConfig(args.blocks, 16, "last_exited", kv_cache_dtype=args.kv_dtype)
    rng = random.Random(0)
    started = time.monotonic()
    with PDEngine(
        config,
        pd_config=PDConfig(prefill_devices=(0,), decode_devices=(1,), startup_timeout=600, request_timeout=600,
                           max_inflight_bytes=args.inflight_gib << 30),
        prefill_cache_config=cache,
        decode_cache_config=cache,
        prefill_scheduler_config=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=args.chunk, prefill_chunk_size=args.chunk),
        decode_scheduler_config=SchedulerConfig(max_num_seqs=32, max_num_batched_tokens=32),
        attention_backend="triton",
        seed=1,
    ) as engine:
        startup = time.monotonic() - started
        params = SamplingParams(max_tokens=2, ignore_eos=True)

        def drain():
            deadline = time.monotonic() + 600
            while engine.has_unfinished_requests():
                engine.step()
                if time.monotonic() > deadline:
                    raise TimeoutError("deployment did not finish")

        engine.add_request("warm", [rng.randrange(config.vocab_size) for _ in range(args.tokens)], params)
        drain()
        engine.metrics.clear()
        n_req = args.requests if args.requests != 64 else 8
        for at in range(0, n_req, args.concurrency):
            for i in range(at, min(n_req, at + args.concurrency)):
                engine.add_request(f"r{i}", [rng.randrange(config.vocab_size) for _ in range(args.tokens)], params)
            drain()
        marks = [m["timings"] for m in engine.metrics if not m["cancelled"]]
    worker_metrics = engine.worker_metrics
    tail = [(t["d_received"] - t["prefill_compute_completed"]) * 1e3 for t in marks]
    total = [(t["d_received"] - t["prefill_started"]) * 1e3 for t in marks]
    prefill = [(t["prefill_compute_completed"] - t["prefill_started"]) * 1e3 for t in marks]
    halves = None
    if args.stream == "alternate" and args.concurrency == 1:
        # the prefill worker saw "warm" first, so r0, r2, ... streamed and r1, r3, ... did not
        def stats(keep):
            rows = [(tail[i], total[i], prefill[i]) for i in range(len(marks)) if keep(i)]
            return {"requests": len(rows), "handoff_tail_ms_p50": statistics.median(r[0] for r in rows),
                    "handoff_total_ms_p50": statistics.median(r[1] for r in rows),
                    "prefill_ms_p50": statistics.median(r[2] for r in rows)} if rows else None
        halves = {"streamed": stats(lambda i: i % 2 == 0), "not_streamed": stats(lambda i: i % 2 == 1)}
    sent = sum(m.get("bytes_sent", 0) for m in worker_metrics.values())
    seconds = sum(m.get("transfer_seconds", 0.0) for m in worker_metrics.values())
    per_request = args.tokens * config.total_ut_steps * 2 * config.num_hidden_layers * config.num_key_value_heads * config.head_dim * (
        2 if args.kv_dtype == "auto" else 1)
    print(json.dumps({
        "suite": "deployment",
        "deployment": "vllm-rlt PDEngine 1P:1D, Ouro-1.4B shape, random weights, B200 handoff connector, direction "
                      + os.environ["RLT_KV_DIRECTION"],
        "requests": len(marks), "prompt_tokens": args.tokens, "prefill_chunk": args.chunk, "concurrency": args.concurrency,
        "kv_bytes_per_request": per_request,
        "handoff_tail_ms": {"p50": statistics.median(tail), "max": max(tail), "min": min(tail)},
        "handoff_total_ms": {"p50": statistics.median(total)},
        "prefill_ms": {"p50": statistics.median(prefill)},
        "bytes_sent": sent, "transfers": sum(m.get("transfers", 0) for m in worker_metrics.values()),
        "transfer_seconds_sum": seconds,
        "gbps_while_transferring": (sent / seconds / 1e9) if seconds else None, "startup_s": startup,
        "layer_streaming": args.stream or False, "alternate": halves, "streamed_slices": sum(m.get("streamed_slices", 0) for m in worker_metrics.values()),
        "stream_host_ms_per_request": (sum(m.get("stream_host_seconds", 0.0) for m in worker_metrics.values()) * 1e3
                                       / max(1, args.requests + 1)),
        "pulled_bytes": sum(m.get("bytes_received", 0) for m in worker_metrics.values()),
        "pull_device_seconds": sum(m.get("pull_seconds", 0.0) for m in worker_metrics.values()),
        # median over the pull launches of the run (the first one of a process carries the module load)
        "pull_gbps_p50_device_timed": max((m.get("pull_gbps_p50", 0.0) for m in worker_metrics.values()), default=0.0),
        "marks_ms_from_prefill_started": [
            {k: round((v - t["prefill_started"]) * 1e3, 3) for k, v in t.items() if isinstance(v, float)} for t in marks[:4]],
    }), flush=True)


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
    ap.add_argument("--latency-requests", type=int, default=16,
                    help="N >= 2: how many requests (per wave) get their own timed handoff for the latency percentiles")
    ap.add_argument("--waves", type=int, default=1,
                    help="N >= 2, pull: run this many independent draws of the workload one after another and report them as "
                         "one line (for request counts whose pools do not fit the GPUs at once)")
    ap.add_argument("--suite", default=None, choices=["kernels", "peer", "deployment"],
                    help="another measurement instead of the benchmark line (see the module docstring)")
    ap.add_argument("--only", default="", help="--suite kernels: comma-separated groups (finalize,pack,segments,tensors)")
    ap.add_argument("--pull", action="store_true", help="--suite peer: run the kernel on the destination GPU")
    ap.add_argument("--tokens", type=int, default=2048, help="--suite deployment: prompt length")
    ap.add_argument("--blocks", type=int, default=8192, help="--suite deployment: pool blocks per worker")
    ap.add_argument("--concurrency", type=int, default=1, help="--suite deployment: requests submitted at once")
    ap.add_argument("--chunk", type=int, default=2048, help="--suite deployment: prefill chunk size")
    ap.add_argument("--kv-dtype", default="auto", choices=["auto", "fp8_e4m3"], help="--suite deployment")
    ap.add_argument("--inflight-gib", type=int, default=2,
                    help="--suite deployment: PDConfig.max_inflight_bytes in GiB")
    ap.add_argument("--stream", nargs="?", const="all", default=None, choices=["all", "alternate"],
                    help="--suite deployment: stream finished layers behind the prefill (RLT_KV_STREAM in the workers); "
                         "'alternate' streams every second request, so that one process yields both figures")
    args = ap.parse_args()
    if args.suite is not None:
        {"kernels": suite_kernels, "peer": suite_peer, "deployment": suite_deployment}[args.suite](args)
        return
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
