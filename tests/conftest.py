"""Shared test plumbing: the ``gpu`` marker, import paths, golden-fixture loaders."""

import json
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden"
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def golden_json(name):
    return json.loads((GOLDEN / name).read_text())


def golden_npz(name):
    with np.load(GOLDEN / f"{name}.npz") as z:
        return {k: z[k] for k in z.files}


KINDS = {
    "f32": dict(element=4),
    "bf16": dict(element=2),
    "fp8": dict(fp8=True),
    "fp8_fixed": dict(fp8=True, fixed_scale=0.5),
}


def oracle_pool(kind, shape, *, device=0, base=1 << 20, recurrent_layers=None):
    from oracle.handoff_oracle import OraclePool

    layers, heads, dim, blocks, page, planes = shape
    return OraclePool(
        layers, heads, dim, blocks, page, planes,
        device=device, base=base, recurrent_layers=recurrent_layers, **KINDS[kind],
    )


def load_pool(pool, arrays, prefix):
    """Fill an OraclePool from the ``<prefix><tensor>`` byte arrays of a fixture."""
    for name in ("key", "value", "key_scale", "value_scale"):
        t = getattr(pool, name)
        if t is not None:
            t.data[...] = arrays[prefix + name].reshape(t.data.shape)


def pool_equal(pool, arrays, prefix):
    for name in ("key", "value", "key_scale", "value_scale"):
        t = getattr(pool, name)
        if t is not None and not np.array_equal(t.data.reshape(-1), arrays[prefix + name].reshape(-1)):
            return False
    return True
