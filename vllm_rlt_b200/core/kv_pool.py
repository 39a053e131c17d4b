"""Device-resident paged KV pool with the reference's tensor layout and block-table allocator.

Storage follows ``KVCacheManager.__init__`` (vllm_rlt/core/kv_cache_manager.py:261-271):
``key_cache`` / ``value_cache`` are ``[num_blocks, num_layers, block_size, kv_heads, head_dim]``
and an FP8 pool adds float32 ``key_scale`` / ``value_scale`` ``[num_blocks, num_layers,
block_size, kv_heads]`` pre-filled with 1.0 or the fixed scale. The attribute names are the
reference's, so the transport accepts either this class or a ``KVCacheManager``.

The allocator is the block-allocation half of the decode-side reservation hook of the handoff
(``Scheduler.reserve_transfer`` -> ``allocate`` + ``pin_transfer``, vllm_rlt/core/scheduler.py:422-447;
the admission half is ``vllm_rlt_b200.core.admission``). What is kept from ``KVCacheManager``, because
block ids and table order are visible on the wire and in the tests:

* free-list pop order: ascending ids from a fresh pool (vllm_rlt/core/kv_cache_manager.py:281, :339-359);
* plane-major tables, plane ``d`` = the reused prefix blocks of plane ``d`` followed by the ``d``-th slice of
  the freshly claimed blocks (:420-461); ``ensure_capacity`` appends to every plane the same way (:463-479);
* a block is shared by reference count: prefix-cache entries hold one reference per block, every request
  that reuses a cached page holds another, and a block returns to the free list when the last one goes;
  cached pages that nothing else uses count as free and are evicted oldest-first, but only when the
  eviction actually satisfies the claim (:339-359);
* transfer leases that defer ``free`` (:501-521) and ``mark_imported_prefix`` (:523-534).

The per-plane, per-layer written-prefix bookkeeping of the reference is reduced to one frontier per
request: here KV enters a pool only through the handoff kernels, which write every layer of every
plane of a range, or through ``restore``.
"""

from __future__ import annotations

import hashlib
from collections import OrderedDict
from dataclasses import dataclass, field

import numpy as np
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
        enable_prefix_caching: bool = False,
        incremental_allocation: bool = False,
        watermark_ratio: float = 0.01,
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
        self._refs = [0] * num_blocks
        self._prefixes: OrderedDict[bytes, tuple[int, ...]] = OrderedDict()  # page key -> that page's block on every plane
        self._awaiting_event: list[tuple] = []
        self._restoring: list[tuple] = []  # (event, snapshot): host tensors a restore kernel may still be reading
        if enable_prefix_caching and layout != "last_exited":
            raise ValueError("prefix caching requires last_exited KV")
        self.enable_prefix_caching = enable_prefix_caching
        self.incremental_allocation = incremental_allocation
        self.watermark_blocks = int(watermark_ratio * num_blocks) if incremental_allocation else 0
        self.prefix_hits = self.prefix_queries = 0

    # -- allocation hook ----------------------------------------------------------------------

    @property
    def num_free_blocks(self) -> int:
        """Blocks a claim could obtain: the free list plus cached pages that only the prefix cache holds."""
        evictable = sum(self._refs[b] == 1 for blocks in self._prefixes.values() for b in blocks)
        return len(self._free_blocks) + evictable

    @property
    def num_used_blocks(self) -> int:
        return self.num_blocks - self.num_free_blocks

    def required_blocks(self, max_tokens: int) -> int:
        if type(max_tokens) is not int or max_tokens <= 0:
            raise ValueError("max_tokens must be a positive integer")
        return -(-max_tokens // self.block_size) * self.storage_depths

    def _release(self, blocks) -> None:
        for b in blocks:
            self._refs[b] -= 1
            if self._refs[b] == 0:
                self._free_blocks.append(b)

    def _claim(self, count: int):
        """``count`` blocks off the free list, evicting cached pages oldest-first only when that gets there.

        A claim that cannot be met even after evicting everything evictable returns ``None`` and evicts nothing,
        so a rejected reservation costs the cache no page (vllm_rlt/core/kv_cache_manager.py:339-359).
        """
        if len(self._free_blocks) < count and self.num_free_blocks < count:
            return None
        while len(self._free_blocks) < count and self._prefixes:
            _, page = self._prefixes.popitem(last=False)
            self._release(page)
        if len(self._free_blocks) < count:
            return None
        taken = [self._free_blocks.pop() for _ in range(count)]
        for b in taken:
            self._refs[b] = 1
        return taken

    def allocate(self, request_id: str, max_tokens: int, *, initial_tokens: int | None = None, prefix=()) -> bool:
        """Reserve ``max_tokens`` of logical capacity and take physical pages for the first ``initial_tokens``.

        ``prefix`` is what ``lookup_prefix`` returned: one tuple per reused page holding that page's block on
        every plane. Those blocks open each plane's table and are shared, not copied; the rest is claimed
        fresh. False (and nothing retained) when the pool cannot supply the fresh blocks.
        """
        if not isinstance(request_id, str) or not request_id:
            raise ValueError("request_id must be a nonempty string")
        if request_id in self._allocations:
            raise ValueError(f"request {request_id!r} already owns KV blocks")
        need = self.required_blocks(max_tokens)
        if need > self.num_blocks:
            raise ValueError(f"request needs {need} physical KV blocks, but the pool has {self.num_blocks}")
        frontier = max_tokens if initial_tokens is None else initial_tokens
        if not 0 < frontier <= max_tokens:
            raise ValueError("invalid initial KV frontier")
        pages = -(-frontier // self.block_size)
        reused = len(prefix)
        if reused > pages:
            raise ValueError("prefix exceeds initial KV frontier")
        shared = [b for page in prefix for b in page]
        for b in shared:
            self._refs[b] += 1
        tail = pages - reused
        fresh = self._claim(tail * self.storage_depths)
        if fresh is None:
            self._release(shared)
            return False
        tables = tuple(
            tuple(page[d] for page in prefix) + tuple(fresh[d * tail : (d + 1) * tail]) for d in range(self.storage_depths)
        )
        self._allocations[request_id] = _Allocation(int(max_tokens), tables, prefix=reused * self.block_size)
        self.prefix_queries += 1
        self.prefix_hits += reused * self.block_size
        return True

    def ensure_capacity(self, request_id: str, tokens: int) -> bool:
        """Grow a request's tables to cover ``tokens`` tokens; False if the pool cannot supply the pages."""
        a = self._get(request_id)
        if not 0 < tokens <= a.max_tokens:
            raise ValueError("KV growth exceeds logical capacity")
        extra = -(-tokens // self.block_size) - len(a.block_tables[0])
        if extra <= 0:
            return True
        fresh = self._claim(extra * self.storage_depths)
        if fresh is None:
            return False
        a.block_tables = tuple(t + tuple(fresh[d * extra : (d + 1) * extra]) for d, t in enumerate(a.block_tables))
        return True

    def allocated_blocks(self, request_id: str) -> int:
        """Physical blocks a request holds, over all planes."""
        return len(self._get(request_id).block_tables[0]) * self.storage_depths

    # -- prefix cache ---------------------------------------------------------------------------

    def _page_keys(self, tokens):
        """One chained digest per whole page of ``tokens``: equal keys mean equal token prefixes."""
        ids = np.asarray(tokens, dtype=np.int64)
        link = b""
        for page in range(len(ids) // self.block_size):
            link = hashlib.blake2b(ids[page * self.block_size : (page + 1) * self.block_size].tobytes(), key=link[:64],
                                   digest_size=32).digest()
            yield link

    def publish_prefix(self, request_id: str, tokens, length: int, event=None) -> None:
        """Offer a request's whole prompt pages, up to ``length`` written tokens, for reuse by later prompts.

        Nothing is copied: the cache takes a reference on the page's blocks. The last prompt token is never
        offered (a hit must leave something to compute, vllm_rlt/core/kv_cache_manager.py:374-398), and a page
        is offered only if the request's written frontier covers it. With ``event`` the offer waits until the
        event has fired (``poll_prefixes``).
        """
        if not self.enable_prefix_caching:
            return
        a = self._get(request_id)
        if event is not None:
            self._awaiting_event.append((request_id, a, tuple(tokens), length, event))
            return
        frontier = a.prefix if a.imported is None else a.imported
        usable = min(length, len(tokens) - 1)
        for index, key in enumerate(self._page_keys(tokens[:usable])):
            if key in self._prefixes:
                continue
            if frontier < (index + 1) * self.block_size:
                break
            page = tuple(t[index] for t in a.block_tables)
            for b in page:
                self._refs[b] += 1
            self._prefixes[key] = page

    def lookup_prefix(self, tokens):
        """The longest run of cached leading pages of ``tokens`` (never the page holding the last token)."""
        if not self.enable_prefix_caching:
            return ()
        self.poll_prefixes()
        found = []
        for key in self._page_keys(tokens[:-1]):
            page = self._prefixes.get(key)
            if page is None:
                break
            self._prefixes.move_to_end(key)
            found.append(page)
        return tuple(found)

    def exclusive_prefix_blocks(self, prefix) -> int:
        """Blocks of a hit that only the cache holds: counted as free, yet about to become non-evictable."""
        return sum(self._refs[b] == 1 for page in prefix for b in page)

    def poll_prefixes(self) -> None:
        """Publish the offers whose event has fired; called by the connector on every ``progress()``."""
        waiting, self._awaiting_event = self._awaiting_event, []
        for request_id, allocation, tokens, length, event in waiting:
            if self._allocations.get(request_id) is not allocation:
                continue
            if not event.query():
                self._awaiting_event.append((request_id, allocation, tokens, length, event))
                continue
            self.publish_prefix(request_id, tokens, length)
        self._release_restored()

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
        self._release(b for table in a.block_tables for b in reversed(table))

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
        """Allocate a whole prompt and take the transfer lease in one step; returns the tables.

        This is the allocation step alone, for callers that do their own admission (the benchmark harnesses).
        The budgeted form with prefix reuse is ``vllm_rlt_b200.core.admission.TransferAdmission``.
        ``None`` means the pool cannot supply the blocks now; nothing is retained then.
        """
        if not self.allocate(transfer_id, tokens):
            return None
        self.pin_transfer(transfer_id, transfer_id)
        return self.plane_block_tables(transfer_id)

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

    def _release_restored(self) -> None:
        self._restoring = [(event, snapshot) for event, snapshot in self._restoring if not event.query()]

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
        (``KVCacheManager.restore``, vllm_rlt/core/kv_cache_manager.py:658-681; same checks and messages).

        Stream-ordered and non-blocking: work queued on the current stream after this call sees the restored KV.
        The pool keeps the snapshot's host tensors alive until the copy has finished, so the caller may drop its
        ``KVSnapshot`` at once."""
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
        # The copy kernel reads the snapshot's pinned tensors through raw addresses, which torch's host allocator
        # knows nothing about: keep them referenced until the kernel has finished, whatever the caller does with
        # its KVSnapshot. They are let go by the next poll_prefixes() / restore() that finds the event fired.
        done = torch.cuda.Event()
        with torch.cuda.device(self.device):
            done.record()
        self._restoring.append((done, snapshot))
        self._release_restored()
        a.imported, a.prefix = snapshot.written
