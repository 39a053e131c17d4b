"""Whole-transfer verification for the multi-GPU harnesses: every transferred row of every tensor, by checksum.

Source and destination pools of a P->D pair live on different GPUs (usually in different processes), so the
rows cannot be compared in place. Instead each side reduces the rows it is responsible for to one 64-bit
wrapping checksum per (request, destination plane, tensor), computed with plain torch indexing - nothing of
the handoff kernels is involved - and only that small table crosses the process boundary:

* the prefill side gathers, for every destination plane, the source rows that plane must receive
  (``source plane = plane``, ``min(plane, exit)`` or ``exit`` depending on the mode) through its own tables;
* the decode side gathers the rows that arrived through the destination tables, and also looks at the
  slots of partially filled last blocks that no token owns: they must still hold the pool's fill byte.

The checksum weights every 32-bit word by its index in the row and every row by its token position and
layer, so rows that arrive permuted, shifted or on the wrong layer change it; K, V and the FP8 scale tensors
are separate columns. Byte-for-byte parity of the kernels themselves is established on one GPU against the
CPU oracle; this is the same statement made across NVLink at full size, where the oracle cannot go.
"""

from __future__ import annotations

import numpy as np
import torch

_TOKEN_WEIGHT = 1000003
_LAYER_WEIGHT = 10007
FILL_BYTE = 0xA5


def travelling_tensors(pool) -> list[torch.Tensor]:
    """K and V codes, plus the scale tensors when they travel (a dynamic-scale FP8 pool)."""
    out = [pool.key_cache, pool.value_cache]
    if pool.key_scale is not None and getattr(pool, "fp8_scale", None) is None:
        out += [pool.key_scale, pool.value_scale]
    return out


def _row_checksum(tensor, blocks, offsets, positions, layers, chunk: int = 256) -> torch.Tensor:
    """Checksum of rows ``tensor[blocks[i], layers, offsets[i]]`` with token positions ``positions[i]``."""
    device = tensor.device
    total = torch.zeros((), dtype=torch.int64, device=device)
    layer_ids = torch.as_tensor(layers, device=device, dtype=torch.int64)
    every_layer = len(layers) == tensor.shape[1]
    for at in range(0, blocks.numel(), chunk):
        rows = tensor[blocks[at : at + chunk], :, offsets[at : at + chunk]]  # [n, layers, ...]
        if not every_layer:
            rows = rows[:, layer_ids]
        n = rows.shape[0]
        words = rows.contiguous().view(torch.uint8).reshape(n, len(layers), -1).view(torch.int32).to(torch.int64)
        column = torch.arange(words.shape[-1], device=device, dtype=torch.int64) * 2 + 1
        per_row = (words * column).sum(-1)  # [n, layers]
        weight = (positions[at : at + chunk, None] + 1) * _TOKEN_WEIGHT + (layer_ids[None, :] + 1) * _LAYER_WEIGHT
        total += (per_row * weight).sum()
    return total


def _layers_of(plane: int, num_layers: int, deep):
    return list(deep) if (deep and plane > 0) else list(range(num_layers))


def source_checksums(pool, w, requests, mode: str, deep=None) -> torch.Tensor:
    """``int64 [requests, destination planes, tensors]``: what each destination plane must receive."""
    tensors = travelling_tensors(pool)
    device = pool.key_cache.device
    bs = w.shape.block_size
    out = torch.zeros((len(list(requests)), w.dst_planes, len(tensors)), dtype=torch.int64, device=device)
    for row, i in enumerate(requests):
        lo, hi = w.ranges[i]
        pos = torch.arange(lo, hi, device=device, dtype=torch.int64)
        table = torch.as_tensor(np.stack([np.asarray(t) for t in w.src_tables[i]]), device=device).long()
        exits = None if w.exit_planes is None else torch.as_tensor(np.asarray(w.exit_planes[i][lo:hi]), device=device).long()
        for plane in range(w.dst_planes):
            if exits is None or mode == "all":
                source_plane = torch.full_like(pos, plane)
            elif mode == "exit_only":
                source_plane = exits
            else:
                source_plane = torch.clamp(exits, max=plane)
            blocks = table[source_plane, pos // bs]
            for column, tensor in enumerate(tensors):
                out[row, plane, column] = _row_checksum(tensor, blocks, pos % bs, pos, _layers_of(plane, w.shape.num_layers, deep))
    return out


def destination_checksums(pool, w, requests, dst_tables, deep=None):
    """``(int64 [requests, planes, tensors], clean)``: what arrived, and whether the unowned slots of partially
    filled last blocks of the K and V pools still hold the fill byte."""
    tensors = travelling_tensors(pool)
    device = pool.key_cache.device
    bs = w.shape.block_size
    out = torch.zeros((len(list(requests)), w.dst_planes, len(tensors)), dtype=torch.int64, device=device)
    clean = True
    for row, (i, tables) in enumerate(zip(requests, dst_tables)):
        lo, hi = w.ranges[i]
        pos = torch.arange(lo, hi, device=device, dtype=torch.int64)
        for plane in range(w.dst_planes):
            table = torch.as_tensor(np.asarray(tables[plane]), device=device).long()
            blocks = table[pos // bs]
            for column, tensor in enumerate(tensors):
                out[row, plane, column] = _row_checksum(tensor, blocks, pos % bs, pos, _layers_of(plane, w.shape.num_layers, deep))
            if hi % bs:
                last = int(table[(hi - 1) // bs])
                for tensor in tensors[:2]:
                    unowned = tensor[last, :, hi % bs :].contiguous().view(torch.uint8)
                    clean = clean and bool((unowned == FILL_BYTE).all())
    return out, clean


def checked_bytes(w, requests, deep=None) -> int:
    """Bytes covered by the checksums of these requests: every row written into the destination pool."""
    s = w.shape
    per_layer = s.token_plane_bytes // s.num_layers
    total = 0
    for i in requests:
        lo, hi = w.ranges[i]
        if deep and w.dst_planes > 1:
            total += (hi - lo) * (s.token_plane_bytes + (w.dst_planes - 1) * len(deep) * per_layer)
        else:
            total += (hi - lo) * w.dst_planes * s.token_plane_bytes
    return total


def exchange_and_compare(pool, is_prefill: bool, edges, *, mode: str, deep=None, send, recv) -> tuple[bool, int]:
    """Run the check over a rank's edges. ``edges`` is a list of ``(peer rank, workload, requests, destination
    tables or None)``; ``send(tensor, rank)`` / ``recv(tensor, rank)`` move the checksum table (NCCL in the
    harnesses, gloo in the CPU tests). Returns ``(ok, verified bytes)`` for this rank (a prefill rank verifies
    nothing itself and returns ``(True, 0)``)."""
    ok, verified = True, 0
    for peer, w, requests, dst_tables in edges:
        requests = list(requests)
        if not requests:
            continue
        if is_prefill:
            send(source_checksums(pool, w, requests, mode, deep), peer)
            continue
        got, clean = destination_checksums(pool, w, requests, dst_tables, deep)
        want = torch.zeros_like(got)
        recv(want, peer)
        same = bool(torch.equal(want, got))
        ok = ok and same and clean
        if same and clean:
            verified += checked_bytes(w, requests, deep)
    return ok, verified


def verify_over_group(pool, is_prefill: bool, edges, *, mode: str, deep=None, device=None) -> tuple[bool, int]:
    """``exchange_and_compare`` over the default process group, reduced over all ranks: ``(every edge equal and
    clean, bytes verified on all decode ranks together)``. Prefill ranks must list their edges in the order in
    which their partners list them (ascending peer rank does)."""
    import torch.distributed as dist

    ok, verified = exchange_and_compare(pool, is_prefill, edges, mode=mode, deep=deep,
                                        send=lambda t, r: dist.send(t, r), recv=lambda t, r: dist.recv(t, r))
    device = pool.key_cache.device if device is None else device
    flags = torch.tensor([1 if ok else 0, verified], dtype=torch.int64, device=device)
    worst = flags[:1].clone()
    dist.all_reduce(worst, op=dist.ReduceOp.MIN)
    total = flags[1:].clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    return bool(worst.item() == 1), int(total.item())
