"""Helpers that mirror oracle pools onto the GPU and read them back as bytes."""

import numpy as np
import torch

from vllm_rlt_b200.kernels.kv_handoff import PoolView

_DTYPES = {1: torch.uint8, 2: torch.bfloat16, 4: torch.float32}


class GpuPool:
    """Device copy of an ``OraclePool``: same bytes, shaped like the reference's cache tensors."""

    def __init__(self, oracle, device="cuda"):
        self.oracle = oracle
        o = oracle
        shape = (o.num_blocks, o.num_layers, o.block_size, o.num_kv_heads, o.head_dim)
        dtype = torch.float8_e4m3fn if o.fp8 else _DTYPES[o.element]

        def codes(t):
            return torch.from_numpy(t.data).to(device).view(dtype).reshape(shape)

        self.key_cache, self.value_cache = codes(o.key), codes(o.value)
        self.key_scale = self.value_scale = None
        if o.fp8:
            def scales(t):
                return torch.from_numpy(t.data).to(device).view(torch.float32).reshape(shape[:-1])

            self.key_scale, self.value_scale = scales(o.key_scale), scales(o.value_scale)
        self.fp8_scale = o.fixed_scale
        self.storage_depths = o.planes

    def view(self) -> PoolView:
        return PoolView.from_cache(self)

    def tensors(self):
        out = [self.key_cache, self.value_cache]
        if self.key_scale is not None:
            out += [self.key_scale, self.value_scale]
        return out

    def bytes(self):
        """All pool tensors (fixed-scale tensors included) as flat uint8 numpy arrays."""
        return [t.contiguous().view(torch.uint8).reshape(-1).cpu().numpy() for t in self.tensors()]


def oracle_bytes(oracle):
    return [t.data.reshape(-1) for t in oracle.tensors(travelling_only=False)]


def assert_pools_equal(gpu_pool, oracle):
    for i, (a, b) in enumerate(zip(gpu_pool.bytes(), oracle_bytes(oracle))):
        if not np.array_equal(a, b):
            bad = np.flatnonzero(a != b)
            raise AssertionError(f"pool tensor {i}: {bad.size} bytes differ, first at {bad[0]}")
