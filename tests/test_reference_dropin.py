"""Run the reference's own connector tests against this repository's connector.

Needs the reference checkout (read-only) beside this repository; skipped where it is absent.
The reference's tests are run unmodified, in a subprocess, with ``vllm_rlt_b200.pd.dropin`` loaded as
a pytest plugin so that ``vllm_rlt.pd.connector.PDStageConnector`` resolves to this implementation.
"""

import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REFERENCE = Path(os.environ.get("VLLM_RLT_REFERENCE", str(ROOT.parent / "reference")))

pytestmark = pytest.mark.skipif(not (REFERENCE / "tests" / "test_transfer_connector.py").is_file(),
                                reason="reference checkout not present")


def run_reference_tests(*selectors, plugin=True):
    env = dict(os.environ, PYTHONPATH=f"{REFERENCE}{os.pathsep}{ROOT}", PYTHONDONTWRITEBYTECODE="1")
    cmd = [sys.executable, "-m", "pytest", "-q", "-p", "no:cacheprovider", "--rootdir", str(REFERENCE),
           "-c", str(REFERENCE / "pyproject.toml")]
    if plugin:
        cmd += ["-p", "vllm_rlt_b200.pd.dropin"]
    cmd += [str(REFERENCE / s) for s in selectors]
    return subprocess.run(cmd, cwd=REFERENCE, env=env, capture_output=True, text=True, timeout=1500)


def test_reference_transfer_connector_suite_passes_with_this_connector():
    out = run_reference_tests("tests/test_transfer_connector.py")
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    assert " passed" in out.stdout and "failed" not in out.stdout


def test_reference_pd_cpu_cases_pass_with_this_connector():
    # the whole of test_pd.py (its GPU/NIXL-marked cases skip themselves) and the stage-engine suite, which
    # includes a spawned worker process driving the connector over a pipe
    out = run_reference_tests("tests/test_pd.py", "tests/test_stage_engine.py")
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    assert " passed" in out.stdout and "failed" not in out.stdout


def test_plugin_really_swaps_the_class():
    code = ("import vllm_rlt_b200.pd.dropin as d; d.install(); import vllm_rlt.pd.connector as c; "
            "print(c.PDStageConnector.__module__)")
    env = dict(os.environ, PYTHONPATH=f"{REFERENCE}{os.pathsep}{ROOT}", PYTHONDONTWRITEBYTECODE="1")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, cwd="/tmp")
    assert out.stdout.strip() == "vllm_rlt_b200.pd.connector", out.stderr[-2000:]
