"""Typed tensor transfer against ``Tensor.copy_`` (the reference's own non-kernel path,
vllm_rlt/worker/tensors.py:77-86, :333-335), in the style of the reference's tests/test_tensor_transfer.py."""

import pytest
import torch

pytestmark = pytest.mark.gpu

TYPES = [torch.int32, torch.int64, torch.float16, torch.bfloat16, torch.float32]


def sample(dtype, n, gen):
    if dtype in (torch.int32, torch.int64):
        hi = 2**31 - 1 if dtype == torch.int32 else 2**62
        x = torch.randint(-hi, hi, (n,), dtype=dtype, generator=gen, device="cuda")
        if dtype == torch.int64 and n > 2:
            x[0], x[1] = 2**53 + 1, -(2**53) - 3  # exact only if int64 never passes through a float
        return x
    return (torch.randn(n, generator=gen, device="cuda") * 1000).to(dtype)


@pytest.mark.parametrize("src_t", TYPES)
@pytest.mark.parametrize("dst_t", TYPES)
def test_flat_copy_converts_like_copy_(src_t, dst_t):
    from vllm_rlt_b200.worker.tensors import copy_tensor

    gen = torch.Generator(device="cuda").manual_seed(1)
    src = sample(src_t, 10_007, gen)
    if src_t in (torch.int32, torch.int64) and dst_t in (torch.float16,):
        src = src % 60000  # keep float16 finite
    if src_t in (torch.float16, torch.bfloat16, torch.float32) and dst_t in (torch.int32, torch.int64):
        src = src.clamp(-30000, 30000)
    dst = torch.zeros(10_007, dtype=dst_t, device="cuda")
    second = torch.zeros(10_007, dtype=torch.int32 if dst_t != torch.int32 else torch.int64, device="cuda")
    copy_tensor(src, dst, secondary=second if src_t in (torch.int32, torch.int64) else None)
    want = torch.zeros_like(dst).copy_(src)
    assert torch.equal(dst.view(torch.uint8), want.view(torch.uint8))
    if src_t in (torch.int32, torch.int64):
        assert torch.equal(second, torch.zeros_like(second).copy_(src))


def test_int64_survives_exactly_and_pinned_host_sources_work():
    from vllm_rlt_b200.worker.tensors import copy_tensor

    host = torch.tensor([2**53 + 1, -(2**53) - 3, 2**62 + 7, 5], dtype=torch.int64).pin_memory()
    dst = torch.zeros(4, dtype=torch.int64, device="cuda")
    narrow = torch.zeros(4, dtype=torch.int32, device="cuda")
    copy_tensor(host, dst, secondary=narrow)
    assert dst.tolist() == host.tolist()
    assert narrow.tolist() == host.to(torch.int32).tolist()
    with pytest.raises(ValueError, match="pinned"):
        copy_tensor(torch.zeros(4, dtype=torch.int64), dst)
    with pytest.raises(ValueError, match="equal-sized contiguous"):
        copy_tensor(host[:3], dst)
    with pytest.raises(ValueError, match="unsupported transfer dtype"):
        copy_tensor(torch.zeros(4, dtype=torch.uint8).pin_memory(), dst)


def test_segmented_batch_of_strided_copies_leaves_everything_else_untouched():
    from vllm_rlt_b200.worker.tensors import TensorTransfer

    gen = torch.Generator(device="cuda").manual_seed(2)
    batch = TensorTransfer(8, torch.bfloat16, "cuda:0", target_dtype=torch.float32)
    big_src = sample(torch.bfloat16, 40 * 70, gen).reshape(40, 70)
    big_dst = torch.full((50, 90), -7.0, device="cuda")
    want = big_dst.clone()
    pieces = [
        (big_src[3:9, 5:60:3], big_dst[10:16, 0:19]),       # strided source columns
        (big_src[20, :33], big_dst[40, 7:40]),              # 1-D row
        (big_src[30:34:2, 1:3], big_dst[1:5:2, 80:82]),     # strided rows on both sides
        (big_src[:0, :0], big_dst[:0, :0]),                 # empty: ignored
    ]
    for s, d in pieces:
        batch.append(s, d)
    assert len(batch.copies) == 3 and (batch.max_rows, batch.max_cols) == (6, 33)
    batch.submit()
    want[10:16, 0:19] = big_src[3:9, 5:60:3].float()
    want[40, 7:40] = big_src[20, :33].float()
    want[1:5:2, 80:82] = big_src[30:34:2, 1:3].float()
    assert torch.equal(big_dst, want)
    host = torch.arange(12, dtype=torch.bfloat16).reshape(3, 4).pin_memory()
    batch.reset()
    batch.append(host, big_dst[20:23, 20:24])
    batch.submit()
    torch.cuda.synchronize()
    assert torch.equal(big_dst[20:23, 20:24], host.float().cuda())
    with pytest.raises(ValueError, match="matching 1D/2D shapes"):
        batch.append(big_src[:2, :2], big_dst[:2, :3])
    with pytest.raises(ValueError, match="dtype does not match"):
        batch.append(big_src[:2, :2].float(), big_dst[:2, :2])
    if torch.cuda.device_count() > 1:
        with pytest.raises(ValueError, match="configured device"):
            batch.append(big_src[:2, :2].to("cuda:1"), big_dst[:2, :2])
