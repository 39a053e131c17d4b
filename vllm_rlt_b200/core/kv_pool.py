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
