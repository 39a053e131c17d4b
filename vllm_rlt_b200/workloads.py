"""Seeded synthetic handoff workloads with the shapes of the benchmark configurations.

No dataset is involved anywhere: prompt lengths, exit planes and block tables are
drawn from seeded generators with the distributions the benchmark names, and KV
values are N(0,1) (bf16) or random non-NaN e4m3 bytes with U[0.01, 0.1] scales.
"""

from __future__ import annotations

import math
import random
from dataclasses import dataclass, field

import numpy as np

SEED_BASE = 20261125


@dataclass(frozen=True)
class KVShape:
    name: str
    num_layers: int
    num_kv_heads: int
    head_dim: int
    planes: int
    block_size: int = 16
    fp8: bool = False

    @property
    def element(self) -> int:
        return 1 if self.fp8 else 2

    @property
    def row_bytes(self) -> int:
        """Bytes of one token row of one layer of one tensor, scales included."""
        return self.num_kv_heads * (self.head_dim * self.element + (4 if self.fp8 else 0))

    @property
    def token_plane_bytes(self) -> int:
        """Payload of one token on one plane: K and V over all layers."""
        return 2 * self.num_layers * self.row_bytes

    @property
    def block_bytes(self) -> int:
        """Device bytes of one physical block (K and V, codes and scales)."""
        return self.token_plane_bytes * self.block_size


OURO_1P4B = KVShape("ouro-1.4b", 24, 16, 128, 4)
OURO_2P6B = KVShape("ouro-2.6b", 48, 16, 128, 4)
OURO_2P6B_FP8 = KVShape("ouro-2.6b-fp8", 48, 16, 128, 4, fp8=True)
HUGINN_3P5B = KVShape("huginn-3.5b", 8, 55, 96, 32)


@dataclass
class Workload:
    """Host-side description of one batch of handoffs between two pools."""

    shape: KVShape
    lengths: list[int]
    ranges: list[tuple[int, int]]
    src_tables: list[list[list[int]]]
    dst_tables: list[list[list[int]]]
    exit_planes: list[list[int]] | None
    src_blocks: int
    dst_blocks: int
    dst_planes: int
    description: str = ""
    extra: dict = field(default_factory=dict)

    @property
    def tokens(self) -> int:
        return sum(e - s for s, e in self.ranges)

    @property
    def payload_bytes(self) -> int:
        """Bytes written into the destination pool. With ``extra["deep_layers"]`` (a recurrent-depth model) planes
        beyond the first carry only those layers."""
        deep = self.extra.get("deep_layers")
        if deep and self.dst_planes > 1:
            per_layer = self.shape.token_plane_bytes // self.shape.num_layers
            return self.tokens * (self.shape.token_plane_bytes + (self.dst_planes - 1) * len(deep) * per_layer)
        return self.tokens * self.dst_planes * self.shape.token_plane_bytes


def _tables(rng: random.Random, lengths, planes, block_size, spare=0):
    """Seeded permutation of a pool's blocks, dealt out plane by plane, request by request."""
    pages = [-(-n // block_size) for n in lengths]
    total = sum(pages) * planes + spare
    order = list(range(total))
    rng.shuffle(order)
    order = np.array(order, np.int32)
    at = 0
    tables = []
    for p in pages:
        req = []
        for _ in range(planes):
            req.append(order[at : at + p])  # host int32 arrays: what a worker would keep its tables in
            at += p
        tables.append(req)
    return tables, total


def draw_lengths(rng, shape, requests, min_len, max_len, partial_fraction):
    """Uniform prompt lengths; ``partial_fraction`` of them end inside a block, the rest on a block edge."""
    lengths = []
    for _ in range(requests):
        n = rng.randint(min_len, max_len)
        if rng.random() >= partial_fraction:
            n = -(-n // shape.block_size) * shape.block_size
        elif n % shape.block_size == 0:
            n -= rng.randint(1, shape.block_size - 1)
        lengths.append(n)
    return lengths


def last_exited_exit_only(
    shape: KVShape = OURO_1P4B,
    *,
    requests: int = 64,
    min_len: int = 512,
    max_len: int = 4096,
    partial_fraction: float = 0.2,
    seed: int = SEED_BASE + 1,
    mode: str = "exit_only",
    lengths: list[int] | None = None,
) -> Workload:
    """Intra-device pool-to-pool handoff of a LAST_EXITED source with per-token exit planes.

    Prompt lengths are uniform in [min_len, max_len]; ``partial_fraction`` of the
    requests keep their drawn length when it ends inside a block (so their last
    block is partially filled), the rest are rounded up to a whole block. Exit
    planes are uniform over the planes. ``mode`` picks what is carried:
    ``exit_only`` (one KV per layer per token into a single-plane pool),
    ``dedup`` or ``all`` (every plane).
    """
    rng = random.Random(seed)
    if lengths is None:
        lengths = draw_lengths(rng, shape, requests, min_len, max_len, partial_fraction)
    else:
        lengths, requests = list(lengths), len(lengths)
    dst_planes = 1 if mode == "exit_only" else shape.planes
    src_tables, src_blocks = _tables(rng, lengths, shape.planes, shape.block_size)
    dst_tables, dst_blocks = _tables(rng, lengths, dst_planes, shape.block_size)
    # per-token exit planes as int32 arrays (a model produces them as a tensor, not as Python lists)
    exits = [np.array([rng.randrange(shape.planes) for _ in range(n)], np.int32) for n in lengths]
    return Workload(
        shape, lengths, [(0, n) for n in lengths], src_tables, dst_tables,
        exits if mode != "all" else None, src_blocks, dst_blocks, dst_planes,
        description=(
            f"{shape.name} LAST_EXITED {mode}: {requests} requests, lengths U[{min_len},{max_len}], "
            f"exit plane U{{0..{shape.planes - 1}}}, block {shape.block_size}, "
            f"{int(partial_fraction * 100)}% of requests end mid-block, seeded random block tables"
        ),
        extra=dict(mode=mode),
    )


def per_depth_all_planes(
    shape: KVShape = OURO_1P4B, *, requests: int = 8, min_len: int = 128, max_len: int = 1024,
    seed: int = SEED_BASE, log_uniform: bool = False, lengths: list[int] | None = None,
    resident_prefix: int = 0, resident_fraction: float = 0.0,
) -> Workload:
    """The reference's own case: every plane of every prompt token is sent.

    ``resident_fraction`` of the requests additionally own ``resident_prefix`` leading tokens that the decode
    side already holds (a prefix-cache hit): their tables cover the prefix but the handoff range starts after it,
    which is the ``start = max(start, cached_tokens)`` skip of the reference (vllm_rlt/pd/connector.py:223).
    """
    rng = random.Random(seed)
    if lengths is not None:
        lengths, requests = list(lengths), len(lengths)
    elif log_uniform:
        lengths = [int(round(math.exp(rng.uniform(math.log(min_len), math.log(max_len))))) for _ in range(requests)]
    else:
        lengths = [rng.randint(min_len, max_len) for _ in range(requests)]
    starts = [resident_prefix if resident_prefix and rng.random() < resident_fraction else 0 for _ in lengths]
    lengths = [s + n for s, n in zip(starts, lengths)]
    src_tables, src_blocks = _tables(rng, lengths, shape.planes, shape.block_size)
    dst_tables, dst_blocks = _tables(rng, lengths, shape.planes, shape.block_size)
    skipped = f", {sum(bool(s) for s in starts)} requests skip a resident {resident_prefix}-token prefix" if resident_prefix else ""
    return Workload(
        shape, lengths, [(s, n) for s, n in zip(starts, lengths)], src_tables, dst_tables, None, src_blocks, dst_blocks,
        shape.planes,
        description=(
            f"{shape.name} per-depth all planes: {requests} requests, lengths "
            f"{'log-' if log_uniform else ''}U[{min_len},{max_len}], block {shape.block_size}, seeded random block tables{skipped}"
        ),
        extra=dict(mode="all"),
    )


def recurrent_depth_dedup(
    shape: KVShape = HUGINN_3P5B, *, requests: int = 2, min_len: int = 1024, max_len: int = 16384,
    min_exit: int = 4, p_exit: float = 0.1, seed: int = SEED_BASE + 3, lengths: list[int] | None = None,
    deep_layers: tuple[int, ...] | None = None,
) -> Workload:
    """Recurrent-depth model: per-token exit recurrence geometric(p) truncated to [min_exit, planes], dedup mode.

    A token that exits at recurrence e holds distinct KV in planes 0..e-1; deeper planes are copies, so
    the dedup handoff reads each distinct row once and rebuilds the copies on the destination.
    """
    rng = random.Random(seed)
    if lengths is None:
        lengths = [rng.randint(min_len, max_len) for _ in range(requests)]
    else:
        lengths, requests = list(lengths), len(lengths)
    src_tables, src_blocks = _tables(rng, lengths, shape.planes, shape.block_size)
    dst_tables, dst_blocks = _tables(rng, lengths, shape.planes, shape.block_size)
    exits = []
    for n in lengths:
        draws = np.array([min(shape.planes, max(min_exit, int(math.log(1.0 - rng.random()) / math.log(1.0 - p_exit)) + 1))
                          for _ in range(n)], np.int32)
        exits.append(draws - 1)  # zero-based exit plane
    return Workload(
        shape, lengths, [(0, n) for n in lengths], src_tables, dst_tables, exits, src_blocks, dst_blocks, shape.planes,
        description=(
            f"{shape.name} recurrent-depth dedup: {requests} requests, lengths U[{min_len},{max_len}], exit recurrence "
            f"geometric(p={p_exit}) truncated to [{min_exit},{shape.planes}], block {shape.block_size}, seeded random block tables"
            + (f", planes >= 1 carry layers {list(deep_layers)} only" if deep_layers else "")
        ),
        extra=dict(mode="dedup", **({"deep_layers": tuple(deep_layers)} if deep_layers else {})),
    )


def subset(w: Workload, indices) -> Workload:
    """The same workload restricted to some of its requests (tables keep their block ids)."""
    idx = list(indices)
    return Workload(
        w.shape, [w.lengths[i] for i in idx], [w.ranges[i] for i in idx], [w.src_tables[i] for i in idx],
        [w.dst_tables[i] for i in idx], None if w.exit_planes is None else [w.exit_planes[i] for i in idx],
        w.src_blocks, w.dst_blocks, w.dst_planes, description=w.description + f" (requests {idx[0]}..{idx[-1]})",
        extra=dict(w.extra),
    )
