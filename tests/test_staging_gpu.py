"""Host staging objects on a real device: snapshots read in place by the transfer kernels, rotation, growth,
batched dirty-range writes. Expected values are plain tensor arithmetic; int64 values above 2^53 show that
nothing passes through floating point (the property pinned by tests/test_tensor_transfer.py:28-87 in the reference).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

BIG = 2**54


def staging():
    from vllm_rlt_b200.worker import staging as st

    return st


@pytest.mark.parametrize("use_uva", [True, False])
def test_a_snapshot_is_readable_by_kernels_in_place_or_through_its_device_copy(use_uva):
    st = staging()
    from vllm_rlt_b200.worker.tensors import copy_tensor

    buffer = st.UvaBuffer(8, torch.int64, "cuda", use_uva=use_uva)
    buffer.np[:] = [BIG + i for i in range(8)]
    view = buffer.stage(3)
    assert view.tolist() == [BIG, BIG + 1, BIG + 2]
    assert (view.data_ptr() == buffer.cpu.data_ptr()) == use_uva and view.is_cuda != use_uva
    out = torch.zeros(3, dtype=torch.int64, device="cuda")
    copy_tensor(view, out)  # a kernel of the library reads the view, wherever it lives
    assert out.tolist() == [BIG, BIG + 1, BIG + 2]
    with pytest.raises(ValueError, match="no CPU path"):
        st.UvaBuffer(8, torch.int64, "cpu")
    with pytest.raises(ValueError, match="fallback target must match"):
        st.UvaBuffer(8, torch.int64, "cuda", use_uva=False, target=torch.zeros(4, dtype=torch.int64, device="cuda"))


@pytest.mark.parametrize("use_uva", [True, False])
def test_pool_rotates_slots_and_grows_only_the_slot_that_needs_it(use_uva):
    st = staging()
    pool = st.UvaBufferPool((2, 3), torch.int64, "cuda", use_uva=use_uva)
    untouched = pool.buffers[1]
    values = torch.arange(15, dtype=torch.int64).reshape(5, 3) + BIG
    first = pool.stage(values)
    assert torch.equal(first.cpu(), values) and pool.buffers[0].cpu.shape == (8, 3) and pool.buffers[1] is untouched
    grown = pool.buffers[0]
    with pytest.raises(ValueError, match="trailing"):
        pool.stage(torch.zeros((4, 2), dtype=torch.int64))
    with pytest.raises(ValueError, match="CPU tensor"):
        pool.stage(values.cuda())
    second = pool.stage(values[:1])
    assert torch.equal(second.cpu(), values[:1]) and pool.buffers[1] is untouched
    again = pool.stage(values[:3])
    assert pool.buffers[0] is grown and again.data_ptr() == first.data_ptr() and torch.equal(again.cpu(), values[:3])
    assert pool.stage(values[:0]).shape == (0, 3)
    moved = pool.copy_to_gpu(values)
    assert moved.is_cuda and torch.equal(moved.cpu(), values)
    out = torch.zeros(5, 3, dtype=torch.int64, device="cuda")
    assert pool.copy_to_gpu(values, out=out) is out and torch.equal(out.cpu(), values)
    with pytest.raises(ValueError, match="output must match"):
        pool.copy_to_gpu(values, out=torch.zeros(4, 3, dtype=torch.int64, device="cuda"))
    with pytest.raises(ValueError, match="capacity must be positive"):
        st.UvaBufferPool(1, torch.int64, "cuda", max_concurrency=0)


def test_published_snapshots_survive_later_cpu_updates_while_the_gpu_is_still_busy():
    """The CPU master changes right after ``publish``; the copy that reads the snapshot runs later (behind a sleep on
    its stream) and must still see the published values. Two slots cover two submissions in flight."""
    st = staging()
    from vllm_rlt_b200.worker.tensors import copy_tensor

    state = st.UvaBackedTensor(257, torch.int64, "cuda", max_concurrency=2)
    target = torch.empty(257, dtype=torch.int64, device="cuda")
    stream = torch.cuda.Stream()
    results, events = [], []
    for value in range(5):
        if len(events) >= 2:
            events[-2].synchronize()  # the slot about to be reused has been read
        with torch.cuda.stream(stream):
            torch.cuda._sleep(10_000_000)
            state.cpu.fill_(BIG + value)
            copy_tensor(state.publish(), target)
            state.cpu.fill_(-1)
            results.append(target.clone())
            events.append(torch.cuda.Event())
            events[-1].record(stream)
    stream.synchronize()
    for value, got in enumerate(results):
        assert torch.equal(got.cpu(), torch.full((257,), BIG + value, dtype=torch.int64))
    assert state.publish(4).shape == (4,)


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32, torch.bfloat16])
def test_staged_input_keeps_offsets_through_growth_and_uploads_one_flat_array(dtype):
    st = staging()
    storage = st.StagedInputTensor(dtype, "cuda")
    base = BIG if dtype == torch.int64 else 0
    pieces = [[base + 1, base + 2, base + 3], list(range(40, 40 + 70)), torch.tensor([7, 8], dtype=dtype)]
    slices = [storage.append(p) for p in pieces]
    device = storage.upload()
    flat = [x for p in pieces for x in (p.tolist() if isinstance(p, torch.Tensor) else p)]
    assert device.is_cuda and device.numel() == len(flat)
    assert torch.equal(device.cpu(), torch.tensor(flat, dtype=dtype))
    assert torch.equal(storage.cpu[: storage.count], torch.tensor(flat, dtype=dtype))  # growth kept earlier pieces
    assert slices[-1].tolist() == [7, 8]
    storage.reset()
    storage.append([5])
    again = storage.upload()
    assert again.tolist() == [5] and again.data_ptr() != device.data_ptr()  # the next submission uses the other slot
    with pytest.raises(ValueError, match="CPU-owned"):
        storage.append(torch.ones(2, dtype=dtype, device="cuda"))


def test_staged_writes_move_only_the_dirty_ranges_in_one_launch():
    st = staging()
    from vllm_rlt_b200.kernels import kv_handoff as kh

    target = torch.full((2, 3, 8), -1, dtype=torch.int64, device="cuda")
    writes = st.StagedWriteTensor(target, 3, 8)
    values = [BIG + 11, BIG + 12]
    writes.stage_write((1, 2), 3, values)
    values[:] = [99, 99]  # the caller's list may change after staging
    writes.stage_write((0, 0), 7, torch.tensor([42]))
    writes.stage_write((0, 1), 0, [])
    before = kh.kernel_launches()
    writes.submit()
    assert kh.kernel_launches() == before + 1
    want = torch.full((2, 3, 8), -1, dtype=torch.int64)
    want[1, 2, 3:5] = torch.tensor([BIG + 11, BIG + 12])
    want[0, 0, 7] = 42
    assert torch.equal(target.cpu(), want)
    slot = writes.contents.buffers[0].cpu.data_ptr()
    writes.reset()
    for k in range(5):  # more writes than the batch was sized for: it grows
        writes.stage_write((k % 2, k % 3), k, [k])
        want[k % 2, k % 3, k] = k
    writes.submit()
    assert torch.equal(target.cpu(), want) and writes.contents.buffers[0].cpu.data_ptr() == slot
    with pytest.raises(ValueError, match="outside the target row"):
        writes.stage_write((0, 0), 7, [1, 2])
    with pytest.raises(ValueError, match="CPU-owned"):
        writes.stage_write((0, 0), 0, torch.ones(1, device="cuda"))
    writes.reset()
    writes.submit()  # nothing staged: nothing launched
    assert kh.kernel_launches() == before + 2
