"""Run a real vllm-rlt 1P:1D deployment with this handoff swapped in and report per-request handoff latency.

    PYTHONPATH=<vllm-rlt checkout>:<this repository> python -m vllm_rlt_b200.pd.reference_e2e [--requests 8] [--tokens 2048]

The deployment is the reference's own ``PDEngine`` (coordinator, stage workers, scheduler, model runner,
random-initialised Ouro-1.4B-shaped model); only the connector is replaced (``dropin.install()``). Latencies
come from the coordinator's timing marks (vllm_rlt/pd/engine.py:198-240):

* handoff tail  = ``d_received - prefill_compute_completed``: from the end of the prompt's prefill compute to
  the decode worker having every KV byte (what the reference's commit tail measures, vllm_rlt/pd/config.py:10-15);
* handoff total = ``d_received - prefill_started``.

The vllm-rlt checkout must be importable; nothing of it is part of this repository. A placeholder ``nixl``
package is not needed here because ``NixlConnector`` is never constructed.
"""

from __future__ import annotations

import argparse
import json
import random
import statistics
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=8)
    ap.add_argument("--tokens", type=int, default=2048)
    ap.add_argument("--max-tokens", type=int, default=2)
    ap.add_argument("--blocks", type=int, default=8192)
    ap.add_argument("--concurrency", type=int, default=1, help="requests submitted at once")
    ap.add_argument("--chunk", type=int, default=2048, help="prefill chunk size")
    ap.add_argument("--kv-dtype", default="auto", choices=["auto", "fp8_e4m3"])
    ap.add_argument("--stock", action="store_true", help="leave the reference's own connector in place (needs nixl)")
    args = ap.parse_args()

    from vllm_rlt import CacheConfig, SamplingParams, SchedulerConfig
    from vllm_rlt.models.ouro import OuroConfig
    from vllm_rlt.pd.config import PDConfig

    if not args.stock:
        from vllm_rlt_b200.pd import dropin

        dropin.install()
    from vllm_rlt.pd.engine import PDEngine

    config = OuroConfig()  # the defaults are the Ouro-1.4B shape: 24 layers, 16 KV heads, head_dim 128, 4 loops
    cache = CacheConfig(args.blocks, 16, "last_exited", kv_cache_dtype=args.kv_dtype)
    rng = random.Random(0)
    started = time.monotonic()
    with PDEngine(
        config,
        pd_config=PDConfig(prefill_devices=(0,), decode_devices=(1,), startup_timeout=600, request_timeout=600),
        prefill_cache_config=cache,
        decode_cache_config=cache,
        prefill_scheduler_config=SchedulerConfig(max_num_seqs=8, max_num_batched_tokens=args.chunk, prefill_chunk_size=args.chunk),
        decode_scheduler_config=SchedulerConfig(max_num_seqs=32, max_num_batched_tokens=32),
        attention_backend="triton",
        seed=1,
    ) as engine:
        startup = time.monotonic() - started
        params = SamplingParams(max_tokens=args.max_tokens, ignore_eos=True)
        done = 0

        def drain():
            nonlocal done
            deadline = time.monotonic() + 600
            while engine.has_unfinished_requests():
                for out in engine.step():
                    done += bool(out.finished)
                if time.monotonic() > deadline:
                    raise TimeoutError("deployment did not finish")

        # warm-up request (kernel compilation, first mappings)
        engine.add_request("warm", [rng.randrange(config.vocab_size) for _ in range(args.tokens)], params)
        drain()
        engine.metrics.clear()
        for at in range(0, args.requests, args.concurrency):
            for i in range(at, min(args.requests, at + args.concurrency)):
                engine.add_request(f"r{i}", [rng.randrange(config.vocab_size) for _ in range(args.tokens)], params)
            drain()
        marks = [m["timings"] for m in engine.metrics if not m["cancelled"]]
        worker_metrics = None
    worker_metrics = engine.worker_metrics
    tail = [(t["d_received"] - t["prefill_compute_completed"]) * 1e3 for t in marks]
    total = [(t["d_received"] - t["prefill_started"]) * 1e3 for t in marks]
    prefill = [(t["prefill_compute_completed"] - t["prefill_started"]) * 1e3 for t in marks]
    sent = sum(m.get("bytes_sent", 0) for m in worker_metrics.values())
    seconds = sum(m.get("transfer_seconds", 0.0) for m in worker_metrics.values())
    planes = config.total_ut_steps
    per_request = args.tokens * planes * 2 * config.num_hidden_layers * config.num_key_value_heads * config.head_dim * (
        2 if args.kv_dtype == "auto" else 1)
    print(json.dumps({
        "deployment": "vllm-rlt PDEngine 1P:1D, Ouro-1.4B shape, random weights, " + ("stock connector" if args.stock else "B200 handoff connector"),
        "requests": len(marks), "prompt_tokens": args.tokens, "prefill_chunk": args.chunk, "concurrency": args.concurrency,
        "kv_bytes_per_request": per_request,
        "handoff_tail_ms": {"p50": statistics.median(tail), "max": max(tail), "min": min(tail)},
        "handoff_total_ms": {"p50": statistics.median(total)},
        "prefill_ms": {"p50": statistics.median(prefill)},
        "bytes_sent": sent, "transfers": sum(m.get("transfers", 0) for m in worker_metrics.values()),
        "transfer_seconds_sum": seconds, "startup_s": startup,
    }), flush=True)


if __name__ == "__main__":
    main()
