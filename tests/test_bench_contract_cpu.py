"""The reference arm of ``bench.py`` runs without a GPU: its one JSON line must carry the agreed keys."""

import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_prints_one_json_line_with_the_contract_keys():
    done = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "1", "--warmup", "1",
                           "--cpu-tokens", "128"], cwd=str(ROOT), capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = [x for x in done.stdout.splitlines() if x.strip()]
    assert len(lines) == 1
    line = json.loads(lines[0])
    for key in ("impl", "metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in line, key
    assert line["impl"] == "reference" and line["steps"] == 1 and line["warmup"] == 1
    assert line["vs_baseline"] is None and line["higher_is_better"] is True and "workload" in line["config"]
    base = line["cpu_baseline"]
    assert base["kind"] in ("port", "reference") and base["cores"] >= 1 and base["value"] == line["value"] > 0
    assert "byte-exact: True" in base["sample"] and base["single_thread_value"] > 0
    # the line describes the work this arm did, not the workload it was cut from
    config = line["config"]
    assert config["payload_bytes"] == base["sample_bytes"] == 128 * 4 * 196608
    assert config["tokens"] == 128 and config["requests"] == 1 and config["mode"] == "all"
    assert config["cut_from"]["payload_bytes"] > config["payload_bytes"] and config["cut_from"]["mode"] == "exit_only"
    assert "worker.py:38" in base["reference_worker_setting"]
    assert line["e2e"] == {"value": line["value"], "unit": line["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_reference_arm_uses_the_references_planner_when_a_source_tree_is_present_and_the_port_otherwise(tmp_path):
    import os

    def kind(env):
        done = subprocess.run([sys.executable, "bench.py", "--impl", "reference", "--steps", "1", "--warmup", "0",
                               "--cpu-tokens", "64"], cwd=str(ROOT), capture_output=True, text=True, timeout=600,
                              env={**os.environ, **env})
        assert done.returncode == 0, done.stderr[-2000:]
        return json.loads(done.stdout.strip().splitlines()[-1])["cpu_baseline"]

    port = kind({"VLLM_RLT_REFERENCE": str(tmp_path)})  # set, and holds no source tree: the restatement is used
    assert port["kind"] == "port" and "oracle/" in port["planner"]
    sibling = ROOT.parent / "reference"
    if (sibling / "vllm_rlt" / "pd" / "transport.py").is_file():
        ref = kind({"VLLM_RLT_REFERENCE": str(sibling)})
        assert ref["kind"] == "reference" and "imported" in ref["planner"]
