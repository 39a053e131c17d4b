"""GPU parity for the descriptor-list copy, the range push, the completion flags and the torch ops."""

import random

import numpy as np
import pytest
import torch

from oracle import handoff_oracle as ho
from tests.conftest import golden_json, golden_npz, load_pool, oracle_pool
from tests.gpu_support import GpuPool, assert_pools_equal

pytestmark = pytest.mark.gpu


def kh():
    from vllm_rlt_b200.kernels import kv_handoff

    return kv_handoff


def device_address(oracle, gpu, address):
    """Oracle synthetic address -> address of the same byte in the GPU copy of the pool."""
    names = ["key", "value", "key_scale", "value_scale"]
    tensors = dict(zip(["key", "value", "key_scale", "value_scale"], [gpu.key_cache, gpu.value_cache, gpu.key_scale, gpu.value_scale]))
    for name in names:
        t = getattr(oracle, name)
        if t is not None and t.base <= address < t.base + t.flat.size:
            return tensors[name].data_ptr() + (address - t.base)
    raise AssertionError("address outside pool")


@pytest.mark.parametrize("case", golden_json("handoff.json"), ids=lambda c: c["name"])
def test_descriptor_lists_of_the_reference_planner_are_written_exactly(case):
    """Drive the copy with the (local, remote) lists partition_segments yields, like NixlConnector.submit."""
    k = kh()
    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    D = oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40)
    load_pool(P, arrays, "src_")
    load_pool(D, arrays, "dst_before_")
    gp, gd = GpuPool(P), GpuPool(D)
    submissions = 0
    for req in case["requests"]:
        source = ho.kv_segments(P.info(), req["src_tables"], req["start"], req["end"])
        target = ho.kv_segments(D.info(), req["dst_tables"], req["start"], req["end"])
        for local, remote, size in ho.partition_segments(source, target, case["byte_limit"], case["descriptor_limit"]):
            rows = [(device_address(P, gp, a), device_address(D, gd, b), n) for (a, n, _), (b, _, _) in zip(local, remote)]
            assert sum(r[2] for r in rows) == size
            k.kv_copy_segments(torch.tensor(rows, dtype=torch.int64, device="cuda"))
            submissions += 1
    assert submissions >= len(case["requests"])
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)


def test_segments_of_any_alignment_and_size():
    k = kh()
    rng = random.Random(9)
    n = 3 << 20
    src = torch.randint(0, 256, (n,), dtype=torch.uint8, device="cuda")
    dst = torch.full((n,), 0xA5, dtype=torch.uint8, device="cuda")
    want = np.full(n, 0xA5, np.uint8)
    host = src.cpu().numpy()
    rows, at = [], 0
    for size in [1, 3, 15, 16, 17, 64, 100, 4096, 4099, 65536, 65537, 200_000, 0, 1 << 20]:
        s_off = rng.randrange(0, n - size - 1)
        at += rng.choice([0, 1, 4, 16, 3])
        rows.append((src.data_ptr() + s_off, dst.data_ptr() + at, size))
        want[at : at + size] = host[s_off : s_off + size]
        at += size
    k.kv_copy_segments(torch.tensor(rows, dtype=torch.int64, device="cuda"))
    assert np.array_equal(dst.cpu().numpy(), want)


def test_more_segments_than_threads():
    k = kh()
    count, size = 1500, 48
    src = torch.randint(0, 256, (count * size,), dtype=torch.uint8, device="cuda")
    dst = torch.zeros(count * size, dtype=torch.uint8, device="cuda")
    perm = list(range(count))
    random.Random(2).shuffle(perm)
    rows = [(src.data_ptr() + i * size, dst.data_ptr() + j * size, size) for i, j in enumerate(perm)]
    k.kv_copy_segments(torch.tensor(rows, dtype=torch.int64, device="cuda"))
    want = src.cpu().numpy().reshape(count, size)
    got = dst.cpu().numpy().reshape(count, size)
    assert np.array_equal(got[perm], want)


@pytest.mark.parametrize("size", [0, 1, 15, 16, 4099, (1 << 20) + 5, 5 << 20])
@pytest.mark.parametrize("shift", [(0, 0), (1, 0), (0, 4), (16, 16)])
def test_push_copies_exactly_the_range(size, shift):
    k = kh()
    src = torch.randint(0, 256, (size + 64,), dtype=torch.uint8, device="cuda")
    dst = torch.full((size + 64,), 0xA5, dtype=torch.uint8, device="cuda")
    k.kv_push(src.data_ptr() + shift[0], dst.data_ptr() + shift[1], size)
    want = np.full(size + 64, 0xA5, np.uint8)
    want[shift[1] : shift[1] + size] = src.cpu().numpy()[shift[0] : shift[0] + size]
    assert np.array_equal(dst.cpu().numpy(), want)


def test_signal_then_wait_and_a_wait_that_runs_out():
    k = kh()
    flag = torch.zeros(1, dtype=torch.int64, device="cuda")
    status = k.new_status()
    k.kv_signal(flag.data_ptr(), 7)
    k.kv_wait(flag.data_ptr(), 7, 50_000_000, status)
    k.raise_for_status(status)
    assert flag.item() == 7
    # nothing ever sets 8: the wait gives up after 2 ms and reports it; the context stays usable
    k.kv_wait(flag.data_ptr(), 8, 2_000_000, status)
    with pytest.raises(TimeoutError, match="last value 7"):
        k.raise_for_status(status)
    assert torch.ones(4, device="cuda").sum().item() == 4


def test_torch_ops_match_the_c_abi_path():
    from vllm_rlt_b200 import _build

    torch.ops.load_library(str(_build.PACKAGE / _build.OPS_NAME))
    ops = torch.ops.vllm_rlt
    case = golden_json("handoff.json")[1]  # fp8 with travelling scales
    arrays = golden_npz(case["name"])
    P = oracle_pool(case["kind"], case["shape"])
    D = oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40)
    load_pool(P, arrays, "src_")
    load_pool(D, arrays, "dst_before_")
    gp, gd, gd2 = GpuPool(P), GpuPool(D), GpuPool(D)
    reqs = case["requests"]
    width = max(len(t) for r in reqs for t in r["src_tables"])

    def table_tensor(key):
        a = np.zeros((len(reqs), P.planes, width), np.int32)
        for i, r in enumerate(reqs):
            for p, t in enumerate(r[key]):
                a[i, p, : len(t)] = t
        return torch.from_numpy(a).cuda()

    st, dt = table_tensor("src_tables"), table_tensor("dst_tables")
    begin = torch.tensor([r["start"] for r in reqs], dtype=torch.int32, device="cuda")
    end = torch.tensor([r["end"] for r in reqs], dtype=torch.int32, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ops.kv_handoff(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, gd.key_cache, gd.value_cache,
                   gd.key_scale, gd.value_scale, st, dt, begin, end, None, None, 0, 0, 0, status)
    assert status.tolist() == [0, 0, 0, 0]
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)
    packed = torch.zeros(arrays["packed"].size, dtype=torch.uint8, device="cuda")
    ops.kv_pack(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, st, begin, end, None, None, 0, 0, 0, packed, status)
    assert np.array_equal(packed.cpu().numpy(), arrays["packed"])
    ops.kv_scatter(packed, dt, begin, end, 0, 0, gd2.key_cache, gd2.value_cache, gd2.key_scale, gd2.value_scale, status)
    assert_pools_equal(gd2, D)
    # same-device "peer" form: destination given as raw addresses
    gd3 = GpuPool(oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40))
    for t, name in zip(gd3.tensors(), ["key", "value", "key_scale", "value_scale"]):
        t.view(torch.uint8).copy_(torch.from_numpy(arrays["dst_before_" + name].reshape(-1)).cuda().view(t.view(torch.uint8).shape))
    ops.kv_handoff_peer(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, gd3.key_cache.data_ptr(),
                        gd3.value_cache.data_ptr(), gd3.key_scale.data_ptr(), gd3.value_scale.data_ptr(),
                        D.num_blocks, D.planes, st, dt, begin, end, None, None, 0, 0, 0, status)
    assert_pools_equal(gd3, D)
    # host-table form: the same tables as CPU tensors, staged by the library
    gd4 = GpuPool(oracle_pool(case["kind"], case["shape"], device=1, base=1 << 40))
    for t, name in zip(gd4.tensors(), ["key", "value", "key_scale", "value_scale"]):
        t.view(torch.uint8).copy_(torch.from_numpy(arrays["dst_before_" + name].reshape(-1)).cuda().view(t.view(torch.uint8).shape))
    ops.kv_handoff_host(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, gd4.key_cache, gd4.value_cache,
                        gd4.key_scale, gd4.value_scale, st.cpu(), dt.cpu(), begin.cpu(), end.cpu(), 0, 0, status)
    assert status.tolist() == [0, 0, 0, 0]
    assert_pools_equal(gd4, D)
    with pytest.raises(RuntimeError, match="CPU int32"):
        ops.kv_handoff_host(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, gd4.key_cache, gd4.value_cache,
                            gd4.key_scale, gd4.value_scale, st, dt, begin, end, 0, 0, status)
    with pytest.raises(RuntimeError, match="contiguous"):
        ops.kv_handoff(gp.key_cache.transpose(0, 1), gp.value_cache, None, None, gd.key_cache, gd.value_cache,
                       None, None, st, dt, begin, end, None, None, 0, 0, 0, None)


def test_torch_ops_for_slices_dedup_wire_and_finalize():
    """The remaining ops: each must equal its ctypes twin on the same inputs."""
    from vllm_rlt_b200 import _build

    torch.ops.load_library(str(_build.PACKAGE / _build.OPS_NAME))
    ops, k = torch.ops.vllm_rlt, kh()
    case = golden_json("finalize.json")[1]  # fp8 with travelling scales, per-token exit planes
    arrays = golden_npz(case["name"])
    shape = case["shape"]
    P = oracle_pool(case["kind"], shape)
    load_pool(P, arrays, "src_before_")
    gp = GpuPool(P)
    reqs = case["requests"]
    planes, page = shape[5], shape[4]
    width = max(len(t) for r in reqs for t in r["src_tables"])

    def table_tensor(key):
        a = np.zeros((len(reqs), planes, width), np.int32)
        for i, r in enumerate(reqs):
            for p, t in enumerate(r[key]):
                a[i, p, : len(t)] = t
        return torch.from_numpy(a).cuda()

    st, dt = table_tensor("src_tables"), table_tensor("dst_tables")
    begin = torch.zeros(len(reqs), dtype=torch.int32, device="cuda")
    end = torch.tensor([r["tokens"] for r in reqs], dtype=torch.int32, device="cuda")
    exits = torch.tensor([e for r in reqs for e in r["exit_planes"]], dtype=torch.int32, device="cuda")
    offs = torch.tensor(np.cumsum([0] + [r["tokens"] for r in reqs])[:-1], dtype=torch.int64, device="cuda")
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    rows = torch.tensor([(i, e, pos) for i, r in enumerate(reqs) for pos, e in enumerate(r["exit_planes"])],
                        dtype=torch.int32, device="cuda")
    ops.kv_finalize(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, st, rows, 0, status)
    load_pool(P, arrays, "src_after_")
    assert_pools_equal(gp, P)
    # dedup wire through the ops, then the replicating scatter
    batch = k.HandoffBatch([r["src_tables"] for r in reqs], [r["dst_tables"] for r in reqs],
                           [(0, r["tokens"]) for r in reqs], block_size=page, exit_planes=[r["exit_planes"] for r in reqs])
    ws = k.dedup_workspace(batch, planes)
    want = np.concatenate([ho.pack_rows(P, r["src_tables"], 0, r["tokens"], mode=ho.MODE_DEDUP, exit_planes=r["exit_planes"]) for r in reqs])
    packed = torch.zeros(want.size, dtype=torch.uint8, device="cuda")
    ops.kv_pack_dedup(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, st, begin, end, exits, offs, 0, 0, packed, ws, status)
    assert np.array_equal(packed.cpu().numpy(), want)
    D = oracle_pool(case["kind"], shape, device=1, base=1 << 40)
    D.fill_sentinel()
    gd, gd2 = GpuPool(D), GpuPool(D)
    ops.kv_scatter_dedup(packed, dt, begin, end, exits, offs, 0, 0, gd.key_cache, gd.value_cache, gd.key_scale, gd.value_scale, ws, status)
    load_pool(D, arrays, "dst_after_")
    assert_pools_equal(gd, D)
    # plane/layer slices tile the handoff
    layers = shape[0]
    for p0, p1 in ((0, 2), (2, planes)):
        for l0, l1 in ((0, 1), (1, layers)):
            ops.kv_handoff_slice(gp.key_cache, gp.value_cache, gp.key_scale, gp.value_scale, gd2.key_cache, gd2.value_cache,
                                 gd2.key_scale, gd2.value_scale, st, dt, begin, end, None, None, 0, l0, l1, p0, p1, status)
    assert_pools_equal(gd2, D)
    assert status.tolist() == [0, 0, 0, 0]


def test_handoff_op_uses_the_current_stream_and_replays_in_a_cuda_graph():
    """Stream and graph behaviour the reference pins for its native op (tests/test_activation.py:328-367)."""
    from vllm_rlt_b200 import _build

    torch.ops.load_library(str(_build.PACKAGE / _build.OPS_NAME))
    ops = torch.ops.vllm_rlt
    shape = (8, 2, 4, 2, 16)  # blocks, layers, block size, heads, dim
    src_k = torch.randn(shape, device="cuda", dtype=torch.bfloat16)
    src_v = torch.randn(shape, device="cuda", dtype=torch.bfloat16)
    dst_k, dst_v = torch.zeros_like(src_k), torch.zeros_like(src_v)
    st = torch.tensor([[[5, 2]]], dtype=torch.int32, device="cuda")
    dt = torch.tensor([[[1, 6]]], dtype=torch.int32, device="cuda")
    begin = torch.tensor([1], dtype=torch.int32, device="cuda")
    end = torch.tensor([7], dtype=torch.int32, device="cuda")

    def launch():
        ops.kv_handoff(src_k, src_v, None, None, dst_k, dst_v, None, None, st, dt, begin, end, None, None, 0, 0, 0, None)

    def expected():
        k, v = torch.zeros_like(src_k), torch.zeros_like(src_v)
        for t in range(1, 7):
            sb, db = (5, 2)[t // 4], (1, 6)[t // 4]
            k[db, :, t % 4] = src_k[sb, :, t % 4]
            v[db, :, t % 4] = src_v[sb, :, t % 4]
        return k, v

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        launch()  # warm-up on the side stream, as graph capture wants
    side.synchronize()
    k, v = expected()
    assert torch.equal(dst_k, k) and torch.equal(dst_v, v)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        launch()
    for _ in range(2):
        src_k.normal_()
        src_v.normal_()
        dst_k.zero_()
        dst_v.zero_()
        graph.replay()
        torch.cuda.synchronize()
        k, v = expected()
        assert torch.equal(dst_k, k) and torch.equal(dst_v, v)
