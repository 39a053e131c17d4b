"""The whole-transfer checksum check of the multi-GPU harnesses, on CPU tensors.

The check must accept a correct handoff and must notice: one flipped byte, two rows swapped, a row on the wrong
layer, a missing scale row, and a write into a slot of a partially filled block that no token owns.
"""

import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from vllm_rlt_b200 import workloads
from vllm_rlt_b200.pd import verify


def make_pool(shape, blocks, planes, *, fill=None, seed=0):
    g = torch.Generator().manual_seed(seed)
    dims = (blocks, shape.num_layers, shape.block_size, shape.num_kv_heads, shape.head_dim)
    if shape.fp8:
        key = torch.randint(0, 255, dims, dtype=torch.uint8, generator=g)
        value = torch.randint(0, 255, dims, dtype=torch.uint8, generator=g)
        key_scale = torch.rand(dims[:-1], generator=g)
        value_scale = torch.rand(dims[:-1], generator=g)
    else:
        key = torch.randn(dims, generator=g).to(torch.bfloat16)
        value = torch.randn(dims, generator=g).to(torch.bfloat16)
        key_scale = value_scale = None
    pool = SimpleNamespace(key_cache=key, value_cache=value, key_scale=key_scale, value_scale=value_scale, fp8_scale=None)
    if fill is not None:
        for t in (pool.key_cache, pool.value_cache):
            t.view(torch.uint8).fill_(fill)
    return pool


def plain_handoff(src, dst, w, mode, deep=None):
    """The handoff written with loops over tokens: the statement the checksums are compared with."""
    bs = w.shape.block_size
    for i, (lo, hi) in enumerate(w.ranges):
        for plane in range(w.dst_planes):
            layers = list(deep) if (deep and plane > 0) else list(range(w.shape.num_layers))
            for t in range(lo, hi):
                e = plane if w.exit_planes is None or mode == "all" else int(w.exit_planes[i][t])
                sp = plane if mode == "all" else e if mode == "exit_only" else min(plane, e)
                sb, db = int(w.src_tables[i][sp][t // bs]), int(w.dst_tables[i][plane][t // bs])
                for a, b in zip(verify.travelling_tensors(src), verify.travelling_tensors(dst)):
                    b[db, layers, t % bs] = a[sb, layers, t % bs]


def run_check(src, dst, w, mode, deep=None):
    box = []
    everything = list(range(len(w.lengths)))
    verify.exchange_and_compare(src, True, [(1, w, everything, None)], mode=mode, deep=deep,
                                send=lambda t, r: box.append(t.clone()), recv=None)
    return verify.exchange_and_compare(dst, False, [(0, w, everything, [w.dst_tables[i] for i in everything])], mode=mode,
                                       deep=deep, send=None, recv=lambda t, r: t.copy_(box.pop(0)))


SMALL = workloads.KVShape("small", 3, 2, 8, 3, block_size=4)
SMALL_FP8 = workloads.KVShape("small-fp8", 2, 2, 8, 2, block_size=4, fp8=True)


@pytest.mark.parametrize("shape,mode", [(SMALL, "exit_only"), (SMALL, "dedup"), (SMALL, "all"), (SMALL_FP8, "dedup")])
def test_a_correct_handoff_is_accepted_and_every_byte_is_counted(shape, mode):
    w = workloads.last_exited_exit_only(shape, requests=3, min_len=5, max_len=19, partial_fraction=0.7, mode=mode, seed=5)
    src = make_pool(shape, w.src_blocks, shape.planes, seed=1)
    dst = make_pool(shape, w.dst_blocks, w.dst_planes, fill=verify.FILL_BYTE)
    plain_handoff(src, dst, w, mode)
    ok, nbytes = run_check(src, dst, w, mode)
    assert ok and nbytes == w.payload_bytes == verify.checked_bytes(w, range(3))


def test_layer_subsets_on_deeper_planes_are_checked_as_carried():
    w = workloads.recurrent_depth_dedup(workloads.KVShape("rd", 4, 2, 8, 3, block_size=4), requests=2, min_len=6, max_len=13,
                                        min_exit=1, seed=3, deep_layers=(1, 2))
    src = make_pool(w.shape, w.src_blocks, 3, seed=2)
    dst = make_pool(w.shape, w.dst_blocks, 3, fill=verify.FILL_BYTE)
    plain_handoff(src, dst, w, "dedup", deep=(1, 2))
    ok, nbytes = run_check(src, dst, w, "dedup", deep=(1, 2))
    assert ok and nbytes == w.payload_bytes


def damaged(kind):
    shape = SMALL_FP8 if kind == "scale" else SMALL
    w = workloads.last_exited_exit_only(shape, requests=2, min_len=9, max_len=14, partial_fraction=1.0, mode="dedup", seed=11)
    src = make_pool(shape, w.src_blocks, shape.planes, seed=4)
    dst = make_pool(shape, w.dst_blocks, w.dst_planes, fill=verify.FILL_BYTE)
    plain_handoff(src, dst, w, "dedup")
    table = w.dst_tables[1][1]
    bs = shape.block_size
    if kind == "byte":
        dst.value_cache.view(torch.uint8)[int(table[0]), 1, 2, 0, 3] ^= 1
    elif kind == "swap":
        a, b = dst.key_cache[int(table[0]), 0, 1].clone(), dst.key_cache[int(table[0]), 0, 2].clone()
        dst.key_cache[int(table[0]), 0, 1], dst.key_cache[int(table[0]), 0, 2] = b, a
    elif kind == "layer":
        a, b = dst.key_cache[int(table[1]), 0, 0].clone(), dst.key_cache[int(table[1]), 1, 0].clone()
        dst.key_cache[int(table[1]), 0, 0], dst.key_cache[int(table[1]), 1, 0] = b, a
    elif kind == "scale":
        dst.key_scale[int(table[0]), 0, 1, 0] += 0.5
    elif kind == "stray":
        hi = w.ranges[1][1]
        assert hi % bs
        dst.key_cache.view(torch.uint8)[int(table[(hi - 1) // bs]), 0, bs - 1, 0, 0] = 0
    return src, dst, w


@pytest.mark.parametrize("kind", ["byte", "swap", "layer", "scale", "stray"])
def test_damage_of_any_kind_is_noticed(kind):
    src, dst, w = damaged(kind)
    ok, nbytes = run_check(src, dst, w, "dedup")
    assert not ok and nbytes < w.payload_bytes
