"""Layer-by-layer streaming of a handoff behind the prefill that produces the KV.

The reference queues a chunk for transfer only once the chunk has finished every depth
(``prefill_submitted`` acts on ``progress.chunk_complete``, vllm_rlt/pd/connector.py:188-218), so the
whole chunk's bytes leave after its last layer. Here the producer announces each (depth, layer) as it
is written; the streamer launches the matching slice of the handoff (``layer_begin/layer_end``,
``plane_begin/plane_end``) on its own stream behind an event, so bytes move while later layers are
still computing and only the last slice is left when the prefill ends.
"""

from __future__ import annotations

import torch

from ..kernels import kv_handoff as kh


class LayerStreamer:
    """Launches handoff slices of ``batch`` as the producer reports (plane, layer) groups complete.

    ``layers_per_slice`` trades launch count against how much is left after the last layer.
    All launches go to ``stream`` (created on the source pool's device if not given), each behind an
    event recorded on the producer's stream at the moment ``layer_done`` is called.
    """

    def __init__(self, src: kh.PoolView, dst: kh.PoolView, batch: kh.HandoffBatch, *, mode=kh.MODE_ALL_PLANES,
                 layers_per_slice: int = 1, stream=None, status=None, variant: int = 0):
        if layers_per_slice < 1:
            raise ValueError("layers_per_slice must be positive")
        self.src, self.dst, self.batch, self.mode = src, dst, batch, mode
        self.layers_per_slice = layers_per_slice
        self.device = torch.device("cuda", src.device)
        self.stream = stream if stream is not None else torch.cuda.Stream(self.device)
        self.status, self.variant = status, variant
        self.launched = 0
        self._sent: dict[int, int] = {}  # plane -> layers already handed off

    def layer_done(self, plane: int, layer: int, *, producer_stream=None) -> bool:
        """The producer has issued the write of ``layer`` of ``plane`` (and all earlier layers of that plane).

        Returns True if a slice was launched. ``plane`` is the destination plane; for a single-plane
        (exit-only / SHARED) destination pass 0.
        """
        if not 0 <= layer < self.src.num_layers:
            raise ValueError("layer outside the pool")
        sent = self._sent.get(plane, 0)
        ready = layer + 1
        if ready <= sent:
            raise ValueError("layers of a plane must be reported in increasing order")
        last = ready == self.src.num_layers
        if ready - sent < self.layers_per_slice and not last:
            return False
        producer = producer_stream if producer_stream is not None else torch.cuda.current_stream(self.device)
        event = torch.cuda.Event()
        event.record(producer)
        self.stream.wait_event(event)
        kh.kv_handoff(self.src, self.dst, self.batch, mode=self.mode, layer_begin=sent, layer_end=ready,
                      plane_begin=plane, plane_end=plane + 1, status=self.status, stream=self.stream,
                      variant=self.variant)
        self._sent[plane] = ready
        self.launched += 1
        return True

    def complete(self, planes: int) -> bool:
        return all(self._sent.get(p, 0) == self.src.num_layers for p in range(planes))

    def finish(self, flag_ptr: int | None = None, value: int = 0):
        """Optionally post the completion flag behind the last slice; returns an event on the handoff stream."""
        if flag_ptr is not None:
            kh.kv_signal(flag_ptr, value, stream=self.stream)
        done = torch.cuda.Event(enable_timing=True)
        done.record(self.stream)
        return done
