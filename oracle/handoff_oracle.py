"""CPU restatement of the vllm-rlt prefill->decode KV handoff. TEST INFRASTRUCTURE ONLY.

This module is the checker for the CUDA kernels: tests, the smoke check and the
CPU-baseline leg of the benchmark are the only things allowed to import it. The
product path never routes through it and has no CPU fallback.

Parity status: PINNED. Every function below is checked against fixtures under
``tests/golden/`` that were produced by importing the reference itself (see
``tests/golden/make_golden.py``) and against the known-answer vectors held by
the reference's own tests (``tests/test_pd.py:56-115``).

Each function cites the reference file:line whose behaviour it restates. Paths
are relative to the reference project root.

Everything is plain numpy over ``uint8`` views: the handoff is a byte mover, so
the element type (bf16, e4m3 codes, float32 scales) never matters here.
"""

from __future__ import annotations

import dataclasses
import random
from typing import Iterable, Iterator, Sequence

import numpy as np

Segment = tuple[int, int, int]  # (address, nbytes, device)

MODE_ALL_PLANES = 0  # every plane is carried (what the reference's PD path does)
MODE_DEDUP = 1  # planes <= exit carried, deeper planes rebuilt from the exit plane
MODE_EXIT_ONLY = 2  # one KV per layer per token, taken at the token's exit plane


# --------------------------------------------------------------------------- geometry


def kv_region(key_ptr: int, value_ptr: int, strides_elems: Sequence[int], element: int) -> dict:
    """Byte geometry of one K/V tensor pair.

    Restates ``_kv_region`` (vllm_rlt/pd/transport.py:18-26): block, layer and
    token strides are the first three tensor strides times the element size.
    """
    block, layer, token = (int(s) * element for s in strides_elems[:3])
    return {
        "key_ptr": int(key_ptr),
        "value_ptr": int(value_ptr),
        "block_bytes": block,
        "layer_bytes": layer,
        "token_bytes": token,
    }


# --------------------------------------------------------------------------- planner


def kv_segments(info: dict, tables, start: int, end: int) -> Iterator[Segment]:
    """Byte segments that hold tokens ``[start, end)`` of every plane.

    Restates ``kv_segments`` (vllm_rlt/pd/transport.py:29-63). Walk order is
    plane, logical block, region (codes then scales), tensor (K then V), layer.
    A block that lies wholly inside the range is one segment per tensor; a block
    cut by either end of the range is one segment per layer per tensor. Errors:
    an empty or negative range, a range past the table, and a physical block id
    outside the pool all raise ``ValueError`` exactly where the reference does
    (lazily, as the walk reaches them).
    """
    page = info["block_size"]
    if start < 0 or end <= start:
        raise ValueError("invalid KV range")
    scales = info.get("scale_region")
    regions = [info] if scales is None else [info, scales]
    first, last = start // page, (end - 1) // page
    for table in tables:
        if len(table) * page < end:
            raise ValueError("KV range exceeds allocation")
        for logical in range(first, last + 1):
            physical = table[logical]
            if physical < 0 or physical >= info["num_blocks"]:
                raise ValueError("physical block outside registered pool")
            lo = max(start, logical * page) - logical * page
            hi = min(end, (logical + 1) * page) - logical * page
            whole = (hi - lo) == page
            for region in regions:
                for base in (region["key_ptr"], region["value_ptr"]):
                    origin = base + physical * region["block_bytes"]
                    if whole:
                        yield (origin, region["block_bytes"], info["device"])
                        continue
                    run = (hi - lo) * region["token_bytes"]
                    for layer in range(info["num_layers"]):
                        yield (
                            origin + layer * region["layer_bytes"] + lo * region["token_bytes"],
                            run,
                            info["device"],
                        )


def coalesce_segments(source: Iterable[Segment], target: Iterable[Segment]):
    """Merge neighbouring (source, target) pairs that are adjacent on both sides.

    Restates ``coalesce_segments`` (vllm_rlt/pd/transport.py:66-92): lists of
    unequal length or a pair with unequal byte counts raise ``ValueError``;
    merging needs address adjacency on both sides and unchanged devices.
    Yields ``(src_address, dst_address, nbytes, src_device, dst_device)``.
    """
    source, target = iter(source), iter(target)
    run = None
    while True:
        s = next(source, None)
        d = next(target, None)
        if s is None and d is None:
            break
        if s is None or d is None or s[1] != d[1]:
            raise ValueError("incompatible source/target KV geometry")
        if (
            run is not None
            and run[0] + run[2] == s[0]
            and run[1] + run[2] == d[0]
            and run[3] == s[2]
            and run[4] == d[2]
        ):
            run[2] += s[1]
        else:
            if run is not None:
                yield tuple(run)
            run = [s[0], d[0], s[1], s[2], d[2]]
    if run is not None:
        yield tuple(run)


def partition_segments(source, target, byte_limit: int, descriptor_limit: int):
    """Cut the coalesced pairs into submissions bounded in bytes and descriptors.

    Restates ``partition_segments`` (vllm_rlt/pd/transport.py:95-112). A pair
    may be split across submissions. Yields ``(local, remote, nbytes)`` with
    ``local``/``remote`` lists of ``(address, nbytes, device)``.
    """
    local: list[Segment] = []
    remote: list[Segment] = []
    filled = 0
    for src, dst, length, src_dev, dst_dev in coalesce_segments(source, target):
        done = 0
        while done < length:
            take = min(length - done, byte_limit - filled)
            local.append((src + done, take, src_dev))
            remote.append((dst + done, take, dst_dev))
            filled += take
            done += take
            if filled == byte_limit or len(local) == descriptor_limit:
                yield local, remote, filled
                local, remote, filled = [], [], 0
    if local:
        yield local, remote, filled


# --------------------------------------------------------------------------- pools


@dataclasses.dataclass
class _Tensor:
    """A pool tensor as bytes: ``[num_blocks, num_layers, block_size, row_bytes]``."""

    data: np.ndarray
    base: int

    @property
    def flat(self) -> np.ndarray:
        return self.data.reshape(-1)


class OraclePool:
    """Paged KV pool with the reference's geometry and allocation order.

    Storage restates ``KVCacheManager.__init__`` (vllm_rlt/core/kv_cache_manager.py:261-271):
    ``key`` and ``value`` are ``[num_blocks, num_layers, block_size, kv_heads, head_dim]``
    in the storage element type, and an FP8 pool adds float32 ``key_scale`` /
    ``value_scale`` of shape ``[num_blocks, num_layers, block_size, kv_heads]``,
    pre-filled with 1.0 or the fixed scale (:265-271). A fixed-scale pool keeps
    its scale tensors but they do not travel (vllm_rlt/pd/transport.py:132-137).

    Allocation restates ``_claim``/``allocate``/``free`` (:339-359, :420-461,
    :501-509) for the case without a prefix cache: the free list starts as
    ``reversed(range(num_blocks))`` and blocks are popped from its end, so ids
    come out ascending; plane ``d`` of a request gets slice ``d`` of the claim.
    """

    def __init__(
        self,
        num_layers: int,
        num_kv_heads: int,
        head_dim: int,
        num_blocks: int,
        block_size: int,
        planes: int,
        *,
        element: int = 2,
        fp8: bool = False,
        fixed_scale: float | None = None,
        device: int = 0,
        base: int = 1 << 20,
        recurrent_layers: Sequence[int] | None = None,
    ):
        if fp8:
            element = 1
        self.num_layers, self.num_kv_heads, self.head_dim = num_layers, num_kv_heads, head_dim
        self.num_blocks, self.block_size, self.planes = num_blocks, block_size, planes
        self.element, self.fp8, self.fixed_scale, self.device = element, fp8, fixed_scale, device
        self.recurrent_layers = (
            tuple(range(num_layers)) if recurrent_layers is None else tuple(recurrent_layers)
        )
        row = num_kv_heads * head_dim * element
        shape = (num_blocks, num_layers, block_size, row)
        size = int(np.prod(shape))
        gap = 4096
        self.key = _Tensor(np.zeros(shape, np.uint8), base)
        self.value = _Tensor(np.zeros(shape, np.uint8), base + size + gap)
        self.key_scale = self.value_scale = None
        if fp8:
            srow = num_kv_heads * 4
            sshape = (num_blocks, num_layers, block_size, srow)
            fill = np.float32(1.0 if fixed_scale is None else fixed_scale)
            sbase = base + 2 * (size + gap)
            ssize = int(np.prod(sshape))
            for i, name in enumerate(("key_scale", "value_scale")):
                arr = np.empty(sshape[:-1] + (num_kv_heads,), np.float32)
                arr[...] = fill
                setattr(self, name, _Tensor(arr.view(np.uint8).reshape(sshape), sbase + i * (ssize + gap)))
        self._free = list(reversed(range(num_blocks)))
        self.tables: dict[str, tuple[tuple[int, ...], ...]] = {}

    # geometry -----------------------------------------------------------------

    @property
    def row_bytes(self) -> int:
        return self.key.data.shape[-1]

    @property
    def scales_travel(self) -> bool:
        return self.fp8 and self.fixed_scale is None

    def tensors(self, *, travelling_only: bool = True) -> list[_Tensor]:
        out = [self.key, self.value]
        if self.fp8 and (self.scales_travel or not travelling_only):
            out += [self.key_scale, self.value_scale]
        return out

    def info(self) -> dict:
        """The geometry fields of ``NixlConnector.info`` (vllm_rlt/pd/transport.py:140-154)."""

        def region(k: _Tensor, v: _Tensor) -> dict:
            s = k.data.strides  # bytes already: dtype is uint8
            return kv_region(k.base, v.base, s, 1)

        return dict(
            **region(self.key, self.value),
            device=self.device,
            num_blocks=self.num_blocks,
            block_size=self.block_size,
            num_layers=self.num_layers,
            depths=self.planes,
            scale_region=region(self.key_scale, self.value_scale) if self.scales_travel else None,
        )

    # allocation ---------------------------------------------------------------

    def shuffle_free_list(self, rng: random.Random) -> None:
        """Seeded permutation of the free list, done before any allocation."""
        rng.shuffle(self._free)

    def allocate(self, request_id: str, tokens: int) -> bool:
        if request_id in self.tables:
            raise ValueError(f"request {request_id!r} already owns KV blocks")
        pages = -(-tokens // self.block_size)
        need = pages * self.planes
        if need > len(self._free):
            return False
        fresh = [self._free.pop() for _ in range(need)]
        self.tables[request_id] = tuple(
            tuple(fresh[d * pages : (d + 1) * pages]) for d in range(self.planes)
        )
        return True

    def free(self, request_id: str) -> None:
        tables = self.tables.pop(request_id, None)
        if tables is not None:
            for table in tables:
                self._free.extend(reversed(table))

    def plane_block_tables(self, request_id: str):
        return self.tables[request_id]

    # contents -----------------------------------------------------------------

    def fill_random(self, rng: np.random.Generator, *, fp8_no_nan: bool = True) -> None:
        """Random payload bytes; FP8 codes avoid the two e4m3fn NaN encodings."""
        for t in (self.key, self.value):
            t.data[...] = rng.integers(0, 256, t.data.shape, dtype=np.uint8)
            if self.fp8 and fp8_no_nan:
                t.data[(t.data & 0x7F) == 0x7F] = 0x3C
        if self.scales_travel:
            for t in (self.key_scale, self.value_scale):
                f = rng.uniform(0.01, 0.1, t.data.shape[:-1] + (self.num_kv_heads,)).astype(np.float32)
                t.data[...] = f.view(np.uint8).reshape(t.data.shape)

    def fill_sentinel(self, byte: int = 0xA5) -> None:
        for t in self.tensors(travelling_only=False):
            t.data[...] = byte

    def finalize_token(self, request_id: str, position: int, exit_plane: int) -> None:
        """Copy the exit plane's row of one token into every deeper plane.

        Restates ``KVCacheManager.finalize_token`` (vllm_rlt/core/kv_cache_manager.py:1053-1076):
        for each plane deeper than ``exit_plane`` and each tensor (K, V and, for
        FP8, both scale tensors, fixed-scale pools included) the token's row is
        copied for the recurrent layers only.
        """
        tables = self.tables[request_id]
        page, offset = divmod(position, self.block_size)
        src = tables[exit_plane][page]
        for plane in range(exit_plane + 1, self.planes):
            dst = tables[plane][page]
            for t in self.tensors(travelling_only=False):
                for layer in self.recurrent_layers:
                    t.data[dst, layer, offset] = t.data[src, layer, offset]

    def snapshot(self) -> list[np.ndarray]:
        return [t.data.copy() for t in self.tensors(travelling_only=False)]


# --------------------------------------------------------------------------- memory model


class AddressSpace:
    """Maps the synthetic addresses of one or more pools onto their byte arrays."""

    def __init__(self, *pools: OraclePool):
        self._spans = []
        for pool in pools:
            for t in pool.tensors(travelling_only=False):
                self._spans.append((t.base, t.base + t.flat.size, t.flat, pool.device))
        self._spans.sort(key=lambda s: s[0])

    def view(self, address: int, nbytes: int, device: int | None = None) -> np.ndarray:
        for lo, hi, flat, dev in self._spans:
            if lo <= address and address + nbytes <= hi and (device is None or dev == device):
                return flat[address - lo : address - lo + nbytes]
        raise ValueError(f"segment [{address}, +{nbytes}) is outside every registered tensor")


def apply_write(space_src: AddressSpace, space_dst: AddressSpace, local, remote) -> int:
    """What a WRITE of one submission does: copy each local range onto its remote range.

    This is the one correct outcome of the reference's
    ``initialize_xfer("WRITE", local, remote)`` (vllm_rlt/pd/transport.py:187-199).
    """
    moved = 0
    for (src, n, sdev), (dst, m, ddev) in zip(local, remote, strict=True):
        if n != m:
            raise ValueError("descriptor length mismatch")
        space_dst.view(dst, n, ddev)[:] = space_src.view(src, n, sdev)
        moved += n
    return moved


# --------------------------------------------------------------------------- handoff


def handoff_reference(
    src: OraclePool,
    dst: OraclePool,
    src_tables,
    dst_tables,
    start: int,
    end: int,
    *,
    byte_limit: int = 256 * 1024**2,
    descriptor_limit: int = 256,
) -> int:
    """The reference handoff of one request's tokens ``[start, end)``, all planes.

    Restates the body of ``PDStageConnector.queue_chunk`` (vllm_rlt/pd/connector.py:220-246)
    without the hidden-state tail: plan the source walk with the source pool's
    geometry and tables, the target walk with the peer's, partition, and write.
    Default limits are ``PDConfig``'s (vllm_rlt/pd/config.py:16-18). Returns bytes moved.
    """
    s_info, d_info = src.info(), dst.info()
    source = kv_segments(s_info, src_tables, start, end)
    target = kv_segments(d_info, dst_tables, start, end)
    s_space, d_space = AddressSpace(src), AddressSpace(dst)
    moved = 0
    for local, remote, size in partition_segments(source, target, byte_limit, descriptor_limit):
        got = apply_write(s_space, d_space, local, remote)
        assert got == size
        moved += size
    return moved


def handoff_blocks(src: OraclePool, dst: OraclePool, src_tables, dst_tables) -> None:
    """Whole-block copy of K and V, plane by plane.

    Restates the reference's own CPU transport simulation (tests/test_stage_engine.py:118-126).
    Used to cross-check ``handoff_reference`` on block-aligned ranges.
    """
    for left, right in zip(src_tables, dst_tables):
        for s, d in zip(left, right):
            for a, b in zip(src.tensors(), dst.tensors()):
                b.data[d] = a.data[s]


def source_plane(mode: int, dst_plane: int, exit_plane: int) -> int:
    """Which source plane feeds ``dst_plane`` of a token that exited at ``exit_plane``.

    ALL_PLANES: the same plane. DEDUP: the same plane up to the exit plane, the
    exit plane beyond it (the copies that ``finalize_token`` made, vllm_rlt/core/kv_cache_manager.py:1053-1076,
    so the result equals ALL_PLANES on a finalized source). EXIT_ONLY: the exit
    plane, into a single-plane destination ("shared selects version e").
    """
    if mode == MODE_ALL_PLANES:
        return dst_plane
    if mode == MODE_DEDUP:
        return min(dst_plane, exit_plane)
    if mode == MODE_EXIT_ONLY:
        return exit_plane
    raise ValueError("unknown plane mode")


def handoff_rows(
    src: OraclePool,
    dst: OraclePool,
    src_tables,
    dst_tables,
    start: int,
    end: int,
    *,
    mode: int = MODE_ALL_PLANES,
    exit_planes: Sequence[int] | None = None,
    layer_begin: int = 0,
    layer_end: int | None = None,
) -> int:
    """Row-by-row statement of the handoff, generalised to per-token exit planes and layer slices.

    For ALL_PLANES over all layers the destination equals ``handoff_reference``'s
    (tested). ``exit_planes[t]`` is indexed by absolute token position. Returns
    payload bytes (bytes written to the destination).
    """
    layer_end = src.num_layers if layer_end is None else layer_end
    page = src.block_size
    moved = 0
    for plane, table in enumerate(dst_tables):
        for t in range(start, end):
            e = src.planes - 1 if exit_planes is None else int(exit_planes[t])
            sp = source_plane(mode, plane, e)
            sb, db = src_tables[sp][t // page], table[t // page]
            for a, b in zip(src.tensors(), dst.tensors()):
                b.data[db, layer_begin:layer_end, t % page] = a.data[sb, layer_begin:layer_end, t % page]
                moved += (layer_end - layer_begin) * a.data.shape[-1]
    return moved


def pack_rows(
    src: OraclePool,
    src_tables,
    start: int,
    end: int,
    *,
    mode: int = MODE_ALL_PLANES,
    wire_planes: int | None = None,
    exit_planes: Sequence[int] | None = None,
    layer_begin: int = 0,
    layer_end: int | None = None,
) -> np.ndarray:
    """The packed wire image of one request: source bytes in the reference walk order.

    Order is that of ``kv_segments`` (vllm_rlt/pd/transport.py:40-63): plane,
    logical block, region (codes, scales), tensor (K, V), layer, token, byte.
    For ALL_PLANES over all layers this is exactly the concatenation of the
    source segments (tested). With DEDUP only rows whose plane is not deeper
    than the token's exit plane are present, in the same order.
    """
    layer_end = src.num_layers if layer_end is None else layer_end
    page = src.block_size
    planes = wire_planes if wire_planes is not None else (1 if mode == MODE_EXIT_ONLY else src.planes)
    chunks = []
    for plane in range(planes):
        for logical in range(start // page, (end - 1) // page + 1):
            toks = range(max(start, logical * page), min(end, (logical + 1) * page))
            picks = []
            for t in toks:
                e = src.planes - 1 if exit_planes is None else int(exit_planes[t])
                if mode == MODE_DEDUP and plane > e:
                    continue
                picks.append((src_tables[source_plane(mode, plane, e)][logical], t % page))
            tensors = src.tensors()
            for region in range(len(tensors) // 2):
                for tensor in tensors[2 * region : 2 * region + 2]:
                    for layer in range(layer_begin, layer_end):
                        for block, offset in picks:
                            chunks.append(tensor.data[block, layer, offset])
    return np.concatenate(chunks) if chunks else np.zeros(0, np.uint8)


def payload_bytes(pool: OraclePool, tokens: int, planes: int, layers: int | None = None) -> int:
    """Algorithmic payload: ``2 x layers x kv_heads x (head_dim x elt + scale)`` per token per plane."""
    layers = pool.num_layers if layers is None else layers
    row = pool.row_bytes + (pool.num_kv_heads * 4 if pool.scales_travel else 0)
    return 2 * layers * row * tokens * planes
