"""The small metadata exchange between decode and prefill workers, over ``torch.distributed``.

This is the only collective of the handoff: the decode worker's block tables for the requests
it reserved, and the IPC handles of its pools. In a deployment the same data rides on the
control pipe (``reserved`` -> ``prefill``, vllm_rlt/pd/engine.py:197-214); in the multi-GPU
harness it is one all-gather of two small tensors (NCCL on GPUs, gloo in the CPU tests).
KV bytes never pass through here.
"""

from __future__ import annotations

import os

import numpy as np
import torch

HANDLE_ROW = 80  # 64-byte IPC handle + 16-byte little-endian offset


def encode_tables(tables, planes: int, width: int) -> torch.Tensor:
    """Per-request per-plane tables -> zero-padded int32 ``[requests, planes, width]``."""
    out = np.zeros((len(tables), planes, width), np.int32)
    for i, req in enumerate(tables):
        if len(req) != planes:
            raise ValueError("every request must have one table per plane")
        for p, t in enumerate(req):
            if len(t) > width:
                raise ValueError("table wider than the agreed width")
            out[i, p, : len(t)] = t
    return torch.from_numpy(out)


def decode_tables(message: torch.Tensor, lengths, block_size: int):
    """Inverse of ``encode_tables`` given each request's token count."""
    a = message.cpu().numpy()
    return [[a[i, p, : -(-n // block_size)].tolist() for p in range(a.shape[1])] for i, n in enumerate(lengths)]


def encode_handles(exported: list[dict]) -> torch.Tensor:
    rows = [list(bytes.fromhex(e["handle"])) + list(int(e["offset"]).to_bytes(16, "little")) for e in exported]
    return torch.tensor(rows, dtype=torch.uint8).reshape(len(exported), HANDLE_ROW)


def decode_handles(message: torch.Tensor) -> list[dict]:
    out = []
    for row in message.cpu().numpy():
        out.append({"handle": bytes(row[:64].tolist()).hex(), "offset": int.from_bytes(bytes(row[64:80].tolist()), "little")})
    return out


def all_gather_metadata(tables_msg: torch.Tensor, handles_msg: torch.Tensor, *, group=None):
    """All ranks contribute same-shaped messages (prefill ranks send zeros); returns per-rank lists."""
    import torch.distributed as dist

    world = dist.get_world_size(group)
    all_tables = [torch.zeros_like(tables_msg) for _ in range(world)]
    all_handles = [torch.zeros_like(handles_msg) for _ in range(world)]
    dist.all_gather(all_tables, tables_msg, group=group)
    dist.all_gather(all_handles, handles_msg, group=group)
    return all_tables, all_handles


def pairing(rank: int, world: int, prefill: int | None = None):
    """Role and partner of a rank for a ``prefill : world - prefill`` split, requests routed round-robin.

    Returns ``(is_prefill, index_in_role, partners)`` where ``partners`` lists the ranks of the
    other role this rank exchanges KV with. With an even split each prefill rank has exactly one
    decode partner; with an uneven split the larger side wraps around the smaller one.
    """
    if world < 2:
        raise ValueError("a P:D split needs at least two ranks")
    prefill = world // 2 if prefill is None else prefill
    decode = world - prefill
    if not 0 < prefill < world:
        raise ValueError("both roles need at least one rank")
    is_prefill = rank < prefill
    index = rank if is_prefill else rank - prefill
    if is_prefill:
        partners = [prefill + d for d in range(decode) if d % prefill == index] if decode >= prefill else [prefill + index % decode]
    else:
        partners = [p for p in range(prefill) if p % decode == index] if prefill >= decode else [index % prefill]
    return is_prefill, index, partners


def assigned_requests(p_rank: int, d_rank: int, world: int, prefill: int, num_requests: int) -> list[int]:
    """Requests of prefill rank ``p_rank`` that go to decode rank ``d_rank``: round-robin over its partners."""
    partners = pairing(p_rank, world, prefill)[2]
    return [i for i in range(num_requests) if partners[i % len(partners)] == d_rank]


def pull_edges(rank: int, world: int, prefill: int, num_requests: int) -> list[dict]:
    """The P->D edges a rank takes part in when the decode side pulls, with the flag slot each end uses.

    Every rank owns ``max fan`` flag words. A decode rank's word ``ready_slot`` is raised by the prefill
    rank when its KV is written; a prefill rank's word ``done_slot`` is raised by the decode rank when it has
    read the KV. Both ends compute the same ``(ready_slot, done_slot)`` for an edge from the pairing alone:
    ``ready_slot`` = position of the prefill rank among the decode rank's partners, ``done_slot`` = position
    of the decode rank among the prefill rank's partners. Edges without requests are left out.
    """
    is_prefill, _, partners = pairing(rank, world, prefill)
    edges = []
    for peer in partners:
        p_rank, d_rank = (rank, peer) if is_prefill else (peer, rank)
        requests = assigned_requests(p_rank, d_rank, world, prefill, num_requests)
        if not requests:
            continue
        edges.append(dict(prefill=p_rank, decode=d_rank, requests=requests,
                          ready_slot=pairing(d_rank, world, prefill)[2].index(p_rank),
                          done_slot=pairing(p_rank, world, prefill)[2].index(d_rank)))
    return edges


def init_process_group_quietly(device):
    """Create the NCCL group with stdout pointed at stderr for the duration: NCCL prints its version banner to
    stdout when its debug level is VERSION or WARN, and rank 0 must print exactly one JSON line there."""
    import sys

    import torch.distributed as dist

    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    try:
        dist.init_process_group("nccl", device_id=device)
        dist.barrier()
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)
