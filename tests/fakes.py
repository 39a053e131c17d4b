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

    def __init__(self):
        self.events = []
        self.complete_immediately = True
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

    def handoff(self, *a, **k):
        raise RuntimeError("the table-driven handoff needs a GPU")

    def post(self, slot_ptr, body, stamp):
        box = list(self.boxes.values())[slot_ptr // self.STRIDE]
        at = slot_ptr % self.STRIDE
        box.bytes[at + 8 : at + 64] = list(body)
        box.words[at // 8] = stamp

    def event(self):
        ev = FakeEvent(self.complete_immediately)
        self.events.append(ev)
        return ev

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
