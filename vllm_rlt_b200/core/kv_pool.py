"""Device-resident paged KV pool with the reference's tensor layout and block-table allocator.

Storage follows ``KVCacheManager.__init__`` (vllm_rlt/core/kv_cache_manager.py:261-271):
``key_cache`` / ``value_cache`` are ``[num_blocks, num_layers, block_size, kv_heads, head_dim]``
and an FP8 pool adds float32 ``key_scale`` / ``value_scale`` ``[num_blocks, num_layers,
block_size, kv_heads]`` pre-filled with 1.0 or the fixed scale. The attribute names are the
reference's, so the transport accepts either this class or a ``KVCacheManager``.

The allocator is the decode-side block allocation hook of the handoff
(``Scheduler.reserve_transfer`` -> ``allocate`` + ``pin_transfer``,
vllm_rlt/core/scheduler.py:422-436): free-list pop order (:339-359), plane-major block tables
(:445-448), transfer leases that defer ``free`` (:501-521) and ``mark_imported_prefix``
(:523-534). Prefix caching and incremental growth stay with the reference's manager.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class _Allocation:
    max_tokens: int
    block_tables: tuple[tuple[int, ...], ...]
    imported: int | None = None  # tokens published by mark_imported_prefix
    prefix: int = 0              # tokens already present when the request was reserved
    transfer_leases: set = field(default_factory=set)
    release_requested: bool = False


@dataclass
class KVSnapshot:
    """Host copy of one request's pages; same fields and layout as the reference's ``KVSnapshot``
    (vllm_rlt/core/kv_cache_manager.py:143-166): every page of every plane in block-table order,
    ``[pages * planes, layer, token, kv_head, dim]``, in pinned host memory."""

    max_tokens: int
    pages: int
    written: tuple
    keys: torch.Tensor
    values: torch.Tensor
    key_scales: torch.Tensor | None = None
    value_scales: torch.Tensor | None = None
    fp8_scale: float | None = None


class KVPool:
    def __init__(
        self,
        num_layers: int,
        num_kv_heads: int,
        head_dim: int,
        num_blocks: int,
        block_size: int,
        max_loops: int,
        *,
        device="cuda",
        dtype: torch.dtype = torch.bfloat16,
        layout: str = "last_exited",
        kv_cache_dtype: str = "auto",
        fp8_scale: float | None = None,
    ):
        for name, value in dict(num_layers=num_layers, num_kv_heads=num_kv_heads, head_dim=head_dim,
                                num_blocks=num_blocks, block_size=block_size, max_loops=max_loops).items():
            if type(value) is not int or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
            setattr(self, name, value)
        if layout not in ("last_exited", "shared"):
            raise ValueError("unsupported KV layout")
        if kv_cache_dtype not in ("auto", "fp8_e4m3"):
            raise ValueError("kv_cache_dtype must be one of ('auto', 'fp8_e4m3')")
        if fp8_scale is not None and kv_cache_dtype != "fp8_e4m3":
            raise ValueError("fp8_scale requires kv_cache_dtype='fp8_e4m3'")
        self.layout, self.kv_cache_dtype, self.fp8_scale, self.dtype = layout, kv_cache_dtype, fp8_scale, dtype
        self.storage_depths = max_loops if layout == "last_exited" else 1
        shape = (num_blocks, num_layers, block_size, num_kv_heads, head_dim)
        storage = torch.float8_e4m3fn if kv_cache_dtype == "fp8_e4m3" else dtype
        self.key_cache = torch.empty(shape, device=device, dtype=storage)
        self.value_cache = torch.empty_like(self.key_cache)
        self.key_scale = self.value_scale = None
        if kv_cache_dtype == "fp8_e4m3":
            fill = 1.0 if fp8_scale is None else fp8_scale
            self.key_scale = torch.full(shape[:-1], fill, device=device, dtype=torch.float32)
            self.value_scale = torch.full_like(self.key_scale, fill)
        self.device = self.key_cache.device
        self._free_blocks = list(reversed(range(num_blocks)))
        self._allocations: dict[str, _Allocation] = {}

    # -- allocation hook ----------------------------------------------------------------------

    @property
    def num_free_blocks(self) -> int:
        return len(self._free_blocks)

    @property
    def num_used_blocks(self) -> int:
        return self.num_blocks - len(self._free_blocks)

    def required_blocks(self, max_tokens: int) -> int:
        if type(max_tokens) is not int or max_tokens <= 0:
            raise ValueError("max_tokens must be a positive integer")
        return -(-max_tokens // self.block_size) * self.storage_depths

    def allocate(self, request_id: str, max_tokens: int) -> bool:
        if not isinstance(request_id, str) or not request_id:
            raise ValueError("request_id must be a nonempty string")
        if request_id in self._allocations:
            raise ValueError(f"request {request_id!r} already owns KV blocks")
        need = self.required_blocks(max_tokens)
        if need > self.num_blocks:
            raise ValueError(f"request needs {need} physical KV blocks, but the pool has {self.num_blocks}")
        if need > len(self._free_blocks):
            return False
        fresh = [self._free_blocks.pop() for _ in range(need)]
        pages = need // self.storage_depths
        tables = tuple(tuple(fresh[d * pages : (d + 1) * pages]) for d in range(self.storage_depths))
        self._allocations[request_id] = _Allocation(int(max_tokens), tables)
        return True

    def _get(self, request_id: str) -> _Allocation:
        try:
            return self._allocations[request_id]
        except KeyError:
            raise KeyError(f"request {request_id!r} has no KV allocation") from None

    def has_allocation(self, request_id: str) -> bool:
        return request_id in self._allocations

    def plane_block_tables(self, request_id: str):
        return self._get(request_id).block_tables

    def free(self, request_id: str) -> None:
        a = self._allocations.get(request_id)
        if a is None:
            return
        if a.transfer_leases:
            a.release_requested = True
            return
        del self._allocations[request_id]
        for table in a.block_tables:
            self._free_blocks.extend(reversed(table))

    def pin_transfer(self, request_id: str, transfer_id: str) -> None:
        a = self._get(request_id)
        if a.release_requested:
            raise RuntimeError("cannot transfer KV scheduled for release")
        a.transfer_leases.add(transfer_id)

    def unpin_transfer(self, request_id: str, transfer_id: str) -> None:
        a = self._get(request_id)
        a.transfer_leases.discard(transfer_id)
        if a.release_requested and not a.transfer_leases:
            self.free(request_id)

    def has_transfer_lease(self, request_id: str) -> bool:
        return bool(self._get(request_id).transfer_leases)

    def mark_imported_prefix(self, request_id: str, length: int, *, start: int = 0) -> None:
        a = self._get(request_id)
        if type(length) is not int or not 0 < length <= a.max_tokens:
            raise ValueError("imported prefix exceeds reserved capacity")
        if a.release_requested:
            raise RuntimeError("cannot activate cancelled KV")
        if a.imported is not None or a.prefix != start:
            raise RuntimeError("KV prefix was already initialized")
        a.imported = length

    def reserve_transfer(self, transfer_id: str, tokens: int) -> tuple | None:
        """Decode-side hook: allocate the whole prompt, take the transfer lease, return the tables.

        ``None`` means the pool cannot admit the request now ("rejected" in the protocol).
        """
        if not self.allocate(transfer_id, tokens):
            return None
        self.pin_transfer(transfer_id, transfer_id)
        return self.plane_block_tables(transfer_id)

    def poll_prefixes(self) -> None:  # the connector calls this every progress(); nothing to do here
        return None

    # -- preemption snapshots ------------------------------------------------------------------

    def _block_copies(self, blocks, pairs, to_host: bool):
        """(source address, destination address, bytes) of every (tensor, block) of a snapshot."""
        out = []
        for pool_t, host_t in pairs:
            size = pool_t.stride(0) * pool_t.element_size()
            base, host = pool_t.data_ptr(), host_t.data_ptr()
            for row, block in enumerate(blocks):
                a, b = base + block * size, host + row * size
                out.append((a, b, size) if to_host else (b, a, size))
        return out

    def _run_copies(self, triples) -> None:
        from ..kernels import kv_handoff as kh

        with torch.cuda.device(self.device):
            for at in range(0, len(triples), kh._lib.MAX_SEGMENTS):
                table = torch.tensor(triples[at : at + kh._lib.MAX_SEGMENTS], dtype=torch.int64).pin_memory()
                kh.kv_copy_segments(table.to(self.device, non_blocking=True))

    def snapshot(self, request_id: str) -> KVSnapshot:
        """Copy a request's pages to pinned host memory with one segment-copy launch per 4096 pages.

        Same contract as ``KVCacheManager.snapshot`` (vllm_rlt/core/kv_cache_manager.py:625-656): refused
        while the allocation is leased to a transfer; the kernels write straight into the host tensors, so
        no request-sized temporary is taken on a device that may be full. Synchronises before returning.
        """
        a = self._get(request_id)
        if a.transfer_leases:
            raise RuntimeError("cannot snapshot KV during a transfer")
        blocks = [b for table in a.block_tables for b in table]
        keys = torch.empty((len(blocks), *self.key_cache.shape[1:]), dtype=self.key_cache.dtype, pin_memory=True)
        values = torch.empty_like(keys, pin_memory=True)
        pairs = [(self.key_cache, keys), (self.value_cache, values)]
        key_scales = value_scales = None
        if self.key_scale is not None:
            key_scales = torch.empty((len(blocks), *self.key_scale.shape[1:]), dtype=torch.float32, pin_memory=True)
            value_scales = torch.empty_like(key_scales, pin_memory=True)
            pairs += [(self.key_scale, key_scales), (self.value_scale, value_scales)]
        self._run_copies(self._block_copies(blocks, pairs, to_host=True))
        torch.cuda.synchronize(self.device)
        return KVSnapshot(a.max_tokens, len(a.block_tables[0]), (a.imported, a.prefix), keys, values, key_scales,
                          value_scales, self.fp8_scale)

    def restore(self, request_id: str, snapshot: KVSnapshot) -> None:
        """Load a snapshot into a fresh allocation of the same size, on the current stream
        (``KVCacheManager.restore``, vllm_rlt/core/kv_cache_manager.py:658-681; same checks and messages)."""
        a = self._get(request_id)
        if a.max_tokens != snapshot.max_tokens:
            raise ValueError("snapshot capacity does not match the allocation")
        if len(a.block_tables[0]) != snapshot.pages:
            raise ValueError("snapshot page count does not match the allocation")
        if a.imported is not None or a.prefix:
            raise RuntimeError("cannot restore into an allocation that already holds KV")
        if (self.key_scale is None) != (snapshot.key_scales is None):
            raise ValueError("snapshot KV dtype does not match the pool")
        if self.fp8_scale != snapshot.fp8_scale:
            raise ValueError("snapshot FP8 scale policy does not match the pool")
        blocks = [b for table in a.block_tables for b in table]
        pairs = [(self.key_cache, snapshot.keys), (self.value_cache, snapshot.values)]
        if self.key_scale is not None:
            pairs += [(self.key_scale, snapshot.key_scales), (self.value_scale, snapshot.value_scales)]
        self._run_copies(self._block_copies(blocks, pairs, to_host=False))
        a.imported, a.prefix = snapshot.written
