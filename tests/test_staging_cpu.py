"""Host logic of the staging helpers without a GPU: rotation, growth, offsets, batched writes.

The device side is replaced by stand-ins (unpinned host memory for pinned, a CPU tensor for the device mirror, a plain
``copy_`` for the transfer kernel), so what is checked here is the bookkeeping; tests/test_staging_gpu.py runs the same
objects on a device.
"""

import pytest
import torch

BIG = 2**54


@pytest.fixture
def st(monkeypatch):
    from vllm_rlt_b200.worker import staging

    real_empty = torch.empty

    class FakeTorch:
        Tensor = torch.Tensor

        def __getattr__(self, name):
            return getattr(torch, name)

        @staticmethod
        def empty(*args, **kwargs):
            kwargs.pop("pin_memory", None)
            kwargs.pop("device", None)
            return real_empty(*args, **kwargs)

    launches = []

    class FakeTransfer:
        def __init__(self, capacity, dtype, device):
            self.capacity, self.copies = capacity, []

        def reset(self):
            self.copies = []

        def append(self, source, target):
            assert len(self.copies) < self.capacity
            self.copies.append((source, target))

        def submit(self):
            launches.append(len(self.copies))
            for source, target in self.copies:
                target.copy_(source)

    monkeypatch.setattr(staging, "torch", FakeTorch())
    monkeypatch.setattr(staging, "_resolve", lambda device: torch.device("cpu"))
    monkeypatch.setattr(staging, "copy_tensor", lambda source, target: target.copy_(source))
    monkeypatch.setattr(staging, "TensorTransfer", FakeTransfer)
    staging.launches = launches
    return staging


def test_pool_hands_out_its_buffers_in_turn_and_grows_one_at_a_time(st):
    pool = st.UvaBufferPool((2, 3), torch.int64, "cuda")
    assert pool.index == 0 and len(pool.buffers) == st.IN_FLIGHT
    second = pool.buffers[1]
    values = torch.arange(15, dtype=torch.int64).reshape(5, 3) + BIG
    view = pool.stage(values)
    assert torch.equal(view, values) and pool.buffers[0].cpu.shape == (8, 3) and pool.index == 1
    assert pool.buffers[1] is second and second.cpu.shape == (2, 3)
    grown = pool.buffers[0]
    pool.stage(values[:1])
    assert pool.index == 0 and pool.buffers[1] is second
    again = pool.stage(values[:3])
    assert pool.buffers[0] is grown and again.data_ptr() == view.data_ptr()
    with pytest.raises(ValueError, match="trailing"):
        pool.stage(torch.zeros((4, 2), dtype=torch.int64))
    with pytest.raises(ValueError, match="capacity must be positive"):
        st.UvaBufferPool(1, torch.int64, "cuda", max_concurrency=0)


def test_a_mirror_is_refreshed_on_stage_and_a_wrong_target_is_refused(st):
    buffer = st.UvaBuffer(4, torch.int64, "cuda", use_uva=False)
    buffer.np[:] = [1, 2, 3, 4]
    mirror = buffer.stage(2)
    assert mirror.tolist() == [1, 2] and mirror.data_ptr() != buffer.cpu.data_ptr()
    buffer.np[:] = [5, 6, 7, 8]
    assert mirror.tolist() == [1, 2] and buffer.stage().tolist() == [5, 6, 7, 8]
    direct = st.UvaBuffer(4, torch.int64, "cuda")
    assert direct.stage(3).data_ptr() == direct.cpu.data_ptr()
    with pytest.raises(ValueError, match="fallback target must match"):
        st.UvaBuffer(4, torch.int64, "cuda", use_uva=False, target=torch.zeros(3, dtype=torch.int64))


def test_published_values_do_not_follow_later_changes_of_the_master(st):
    state = st.UvaBackedTensor(6, torch.int64, "cuda")
    state.np[:] = 7
    first = state.publish()
    state.np[:] = 8
    second = state.publish(4)
    state.np[:] = 9
    assert first.tolist() == [7] * 6 and second.tolist() == [8] * 4
    third = state.publish()  # the first slot comes round again
    assert third.data_ptr() == first.data_ptr() and first.tolist() == [9] * 6


@pytest.mark.parametrize("dtype", [torch.int64, torch.int32, torch.bfloat16])
def test_appended_pieces_keep_their_places_when_the_array_grows(st, dtype):
    storage = st.StagedInputTensor(dtype, "cuda")
    base = BIG if dtype == torch.int64 else 0
    pieces = [[base + 1, base + 2, base + 3], list(range(40, 110)), torch.tensor([7, 8], dtype=dtype)]
    slices = [storage.append(p) for p in pieces]
    flat = torch.tensor([x for p in pieces for x in (p.tolist() if isinstance(p, torch.Tensor) else p)], dtype=dtype)
    assert storage.count == 75 and torch.equal(storage.cpu[:75], flat) and slices[-1].tolist() == [7, 8]
    sent = storage.upload()
    assert torch.equal(sent, flat)
    storage.reset()
    storage.append([5])
    other = storage.upload()
    assert other.tolist() == [5] and other.data_ptr() != sent.data_ptr() and torch.equal(sent, flat)


def test_staged_writes_are_frozen_when_staged_and_leave_as_one_batch(st):
    target = torch.full((2, 3, 8), -1, dtype=torch.int64)
    writes = st.StagedWriteTensor(target, 2, 4)
    values = [BIG + 1, BIG + 2]
    writes.stage_write((1, 2), 3, values)
    values[:] = [0, 0]
    writes.stage_write((0, 0), 7, torch.tensor([42]))
    writes.stage_write((0, 1), 0, [])
    writes.submit()
    want = torch.full((2, 3, 8), -1, dtype=torch.int64)
    want[1, 2, 3:5] = torch.tensor([BIG + 1, BIG + 2])
    want[0, 0, 7] = 42
    assert torch.equal(target, want) and st.launches == [2]
    writes.reset()
    for k in range(5):  # more writes and more values than the object was sized for
        writes.stage_write((k % 2, k % 3), k, [k])
        want[k % 2, k % 3, k] = k
    writes.submit()
    assert torch.equal(target, want) and st.launches == [2, 5]
    with pytest.raises(ValueError, match="outside the target row"):
        writes.stage_write((0, 0), 7, [1, 2])
    writes.reset()
    writes.submit()
    assert st.launches == [2, 5]
