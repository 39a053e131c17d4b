"""Layer-by-layer streaming: slices launched behind producer events add up to the whole handoff."""

import random

import numpy as np
import pytest
import torch

from oracle import handoff_oracle as ho
from tests.conftest import oracle_pool
from tests.gpu_support import GpuPool, assert_pools_equal
from tests.test_kv_handoff_gpu import sentinel_destination

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind,layers_per_slice", [("bf16", 1), ("fp8", 2), ("bf16", 3)])
def test_streamed_slices_equal_the_full_handoff(kind, layers_per_slice):
    from vllm_rlt_b200.kernels import kv_handoff as k
    from vllm_rlt_b200.pd.streaming import LayerStreamer

    shape = (5, 4, 32, 96, 16, 3)
    rng, nrng = random.Random(8), np.random.default_rng(8)
    P, D = oracle_pool(kind, shape), sentinel_destination(kind, shape)
    P.fill_random(nrng)
    P.shuffle_free_list(rng)
    D.shuffle_free_list(rng)
    reqs = []
    for i, n in enumerate((40, 17, 64)):
        assert P.allocate(f"r{i}", n) and D.allocate(f"r{i}", n)
        reqs.append((f"r{i}", rng.randrange(n // 2), n))
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch([P.plane_block_tables(r) for r, *_ in reqs], [D.plane_block_tables(r) for r, *_ in reqs],
                           [(s, e) for _, s, e in reqs], block_size=16)
    status = k.new_status()
    streamer = LayerStreamer(gp.view(), gd.view(), batch, layers_per_slice=layers_per_slice, status=status)
    compute = torch.cuda.Stream()
    launched = 0
    with torch.cuda.stream(compute):
        for plane in range(3):
            for layer in range(5):
                torch.cuda._sleep(200_000)  # the producer is busy for ~0.1 ms per layer
                launched += streamer.layer_done(plane, layer, producer_stream=compute)
    assert streamer.complete(3)
    per_plane = -(-5 // layers_per_slice)
    assert launched == streamer.launched == 3 * per_plane
    done = streamer.finish()
    done.synchronize()
    k.raise_for_status(status)
    for r, s, e in reqs:
        ho.handoff_reference(P, D, P.plane_block_tables(r), D.plane_block_tables(r), s, e)
    assert_pools_equal(gd, D)
    with pytest.raises(ValueError, match="increasing order"):
        streamer.layer_done(0, 2)
    with pytest.raises(ValueError, match="outside the pool"):
        streamer.layer_done(0, 5)


def test_a_slice_never_runs_ahead_of_its_producer_event():
    """The slice of a layer must not start before the producer's write of that layer: the destination still holds
    the sentinel while the producer stream is blocked, and the data once it is released."""
    from vllm_rlt_b200.kernels import kv_handoff as k
    from vllm_rlt_b200.pd.streaming import LayerStreamer

    shape = (2, 2, 16, 32, 16, 1)
    P, D = oracle_pool("bf16", shape), sentinel_destination("bf16", shape)
    P.fill_random(np.random.default_rng(1))
    assert P.allocate("a", 32) and D.allocate("a", 32)
    gp, gd = GpuPool(P), GpuPool(D)
    batch = k.HandoffBatch([P.plane_block_tables("a")], [D.plane_block_tables("a")], [(0, 32)], block_size=16)
    streamer = LayerStreamer(gp.view(), gd.view(), batch, layers_per_slice=2)
    compute = torch.cuda.Stream()
    with torch.cuda.stream(compute):
        torch.cuda._sleep(int(0.3 * 1.9e9))  # ~300 ms of "prefill" before the layers are written
        streamer.layer_done(0, 1, producer_stream=compute)
    probe = torch.cuda.Stream()
    with torch.cuda.stream(probe):
        early = gd.key_cache.clone()
    probe.synchronize()
    assert (early.view(torch.uint8) == 0xA5).all()  # nothing has moved yet: the slice is waiting on the device
    streamer.finish().synchronize()
    ho.handoff_reference(P, D, P.plane_block_tables("a"), D.plane_block_tables("a"), 0, 32)
    assert_pools_equal(gd, D)
