"""CPU stand-ins used by the host-logic tests: a transport backend without CUDA, and a minimal stage engine."""

import ctypes
from types import SimpleNamespace

import torch

from vllm_rlt_b200.pd.transport import Mailbox


class FakeEvent:
    def __init__(self, done=True):
        self.done = done

    def query(self):
        return self.done


class FakeBackend:
    """Backend of ``B200Transport`` over host memory: memmove for the copy, direct writes for the post."""

    device_ordered = False

    def __init__(self):
        self.events = []
        self.complete_immediately = True
        self.hold_start = False  # True: queued work has not begun (it waits behind a producer's event)
        self.markers = []
        self.copies = []
        self.boxes = {}

    def export(self, tensor):
        return {"ptr": tensor.data_ptr(), "bytes": tensor.numel() * tensor.element_size(), "handle": "", "offset": 0,
                "device": -1}

    def translator(self, peer_info):
        spans = [(e["ptr"], e["ptr"] + e["bytes"]) for e in peer_info["metadata"]["tensors"]]

        def translate(address, nbytes):
            if any(lo <= address and address + nbytes <= hi for lo, hi in spans):
                return address
            raise ValueError("remote descriptor outside the peer's registered memory")

        return translate

    STRIDE = 1 << 24  # fake "device addresses" of mailboxes: index * STRIDE

    def mailbox_pointer(self, name):
        if name not in self.boxes:
            self.boxes[name] = Mailbox(name)
        return self.boxes[name], list(self.boxes).index(name) * self.STRIDE

    def copy_segments(self, triples):
        for src, dst, n in triples:
            ctypes.memmove(dst, src, n)
        self.copies.append(list(triples))
        return ()

    copy_ranges = copy_segments

    def handoff(self, cache, peer_info, translate, requests, *, mode=0, layer_begin=0, layer_end=0,
                plane_begin=0, plane_end=0, exit_planes=None, status=None, pull=False, before_launch=None):
        """Row-by-row statement of the table-driven launch over host tensors (all-planes mode only).
        ``pull``: the peer's memory is the source and the local tensors the destination."""
        assert mode == 0 and exit_planes is None
        if before_launch is not None:
            before_launch()
        page, layers = cache.block_size, cache.num_layers
        layer_end = layer_end or layers
        pairs = [(cache.key_cache, "key_ptr", peer_info), (cache.value_cache, "value_ptr", peer_info)]
        if peer_info.get("scale_region") is not None:
            pairs += [(cache.key_scale, "key_ptr", peer_info["scale_region"]), (cache.value_scale, "value_ptr", peer_info["scale_region"])]
        for source, target, start, end in requests:
            planes = list(zip(source, target, strict=True))
            for src_table, dst_table in planes[plane_begin : plane_end or len(planes)]:
                for t in range(start, end):
                    for tensor, key, region in pairs:
                        row = tensor.stride(2) * tensor.element_size()
                        for layer in range(layer_begin, layer_end):
                            off = layer * region["layer_bytes"] + (t % page) * region["token_bytes"]
                            if pull:
                                src = translate(region[key] + int(src_table[t // page]) * region["block_bytes"] + off, row)
                                dst = tensor.data_ptr() + int(dst_table[t // page]) * region["block_bytes"] + off
                            else:
                                src = tensor.data_ptr() + int(src_table[t // page]) * region["block_bytes"] + off
                                dst = translate(region[key] + int(dst_table[t // page]) * region["block_bytes"] + off, row)
                            ctypes.memmove(dst, src, row)
        self.copies.append(("tables", list(requests)))
        return ()

    def post(self, slot_ptr, body, stamp):
        box = list(self.boxes.values())[slot_ptr // self.STRIDE]
        at = slot_ptr % self.STRIDE
        box.bytes[at + 8 : at + 64] = list(body)
        box.words[at // 8] = stamp

    def event(self):
        ev = FakeEvent(self.complete_immediately)
        self.events.append(ev)
        return ev

    def marker(self):
        ev = FakeEvent(not self.hold_start)
        self.markers.append(ev)
        return ev

    def order_after(self, event):
        pass

    def close(self):
        for box in self.boxes.values():
            box.close()
        self.boxes.clear()


def cpu_cache(num_layers=3, heads=2, dim=8, blocks=24, page=4, planes=4, dtype=torch.bfloat16, fp8=False, fp8_scale=None):
    """A ``KVCacheManager``-shaped namespace with CPU tensors (attribute names of the reference)."""
    shape = (blocks, num_layers, page, heads, dim)
    store = torch.float8_e4m3fn if fp8 else dtype
    ns = SimpleNamespace(
        key_cache=torch.zeros(shape, dtype=torch.uint8 if fp8 else dtype).view(store) if fp8 else torch.zeros(shape, dtype=dtype),
        num_blocks=blocks, block_size=page, num_layers=num_layers, storage_depths=planes, fp8_scale=fp8_scale,
        key_scale=None, value_scale=None,
    )
    ns.value_cache = torch.zeros_like(ns.key_cache)
    if fp8:
        fill = 1.0 if fp8_scale is None else fp8_scale
        ns.key_scale = torch.full(shape[:-1], fill)
        ns.value_scale = torch.full(shape[:-1], fill)
    return ns


class FakeRequest:
    def __init__(self, request_id, tokens, phase):
        self.request_id = request_id
        self.prompt_token_ids = list(tokens)
        self.num_prefilled_tokens = 0
        self.hidden_state = None
        self.phase = phase
        self.compute_released = False


class FakeEngine:
    """The handful of stage-engine hooks the connector calls, over a ``KVPool`` on the CPU.

    Mirrors the contracts of ``StageEngine.reserve_transfer / accept_import / release_transfer_compute /
    release_transfer / suspend_transfer`` (vllm_rlt/engine/stage_engine.py:679-775): identity checks on
    the request object, a lease taken at reservation, KV freed only when the lease is dropped.
    """

    def __init__(self, role, pool, *, max_num_seqs=4, hidden_size=16):
        self.cache_manager = pool
        pool.layout = "last_exited"
        pool.attention_info = {"backend": "torch"}
        self.scheduler = SimpleNamespace(requests={}, config=SimpleNamespace(max_num_seqs=max_num_seqs, wavefront_chunked_prefill=False))
        self.stage_config = SimpleNamespace(role=role, produces_tokens=role != "prefill", accepts_prompt=role != "decode", stage_id=f"{role}-0")
        self.model = SimpleNamespace(config=SimpleNamespace(hidden_size=hidden_size))
        self.imported = {}
        self.suspended = []

    def reserve_transfer(self, tid, tokens, params, *, receiving, trace_id=None):
        if tid in self.scheduler.requests:
            raise ValueError("duplicate request")
        if self.cache_manager.reserve_transfer(tid, len(tokens)) is None:
            return None
        request = FakeRequest(tid, tokens, "RECEIVING" if receiving else "WAITING")
        self.scheduler.requests[tid] = request
        return request

    def accept_import(self, request, hidden, *, cached_tokens=0):
        if self.scheduler.requests.get(request.request_id) is not request:
            return False
        self.cache_manager.mark_imported_prefix(request.request_id, len(request.prompt_token_ids), start=cached_tokens)
        self.imported[request.request_id] = hidden.clone()
        return True

    def admit(self, tid):
        """What the scheduler does when it grants the imported request a compute slot."""
        request = self.scheduler.requests[tid]
        self.cache_manager.unpin_transfer(tid, tid)
        request.phase = "CODA"

    def release_transfer_compute(self, request, *, ready_event=None):
        if self.scheduler.requests.get(request.request_id) is not request:
            return False
        if ready_event is not None and not ready_event.query():
            return False
        request.hidden_state = None
        request.compute_released = True
        return True

    def release_transfer(self, request):
        if self.scheduler.requests.get(request.request_id) is not request:
            return False
        del self.scheduler.requests[request.request_id]
        self.cache_manager.unpin_transfer(request.request_id, request.request_id)
        self.cache_manager.free(request.request_id)
        return True

    def suspend_transfer(self, request):
        self.suspended.append(request.request_id)
        request.phase = "TRANSFERRING"
