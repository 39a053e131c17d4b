"""Host-side accounting of the benchmark workloads: payload and link bytes against the oracle's own counts."""

import numpy as np

from oracle import handoff_oracle as ho
from tests.conftest import oracle_pool


def test_link_bytes_of_a_dedup_pull_equal_the_oracle_wire_image():
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.pd.pull_harness import wire_bytes

    shape = workloads.KVShape("small", 2, 2, 8, 4, block_size=4)
    w = workloads.last_exited_exit_only(shape, requests=5, min_len=3, max_len=30, mode="dedup", seed=11)
    P = oracle_pool("bf16", (shape.num_layers, shape.num_kv_heads, shape.head_dim, w.src_blocks, shape.block_size, shape.planes))
    want = 0
    for tables, (lo, hi), exits in zip(w.src_tables, w.ranges, w.exit_planes):
        want += ho.pack_rows(P, [list(t) for t in tables], lo, hi, mode=ho.MODE_DEDUP, exit_planes=list(exits)).size
    assert wire_bytes(w, range(5), "dedup") == want
    assert wire_bytes(w, range(5), "all") == w.payload_bytes == ho.payload_bytes(P, w.tokens, shape.planes)
    assert wire_bytes(w, [1, 3], "dedup") == sum(
        ho.pack_rows(P, [list(t) for t in w.src_tables[i]], *w.ranges[i], mode=ho.MODE_DEDUP, exit_planes=list(w.exit_planes[i])).size
        for i in (1, 3))


def test_recurrent_depth_link_bytes_count_only_the_deep_layers_beyond_plane_zero():
    from vllm_rlt_b200 import workloads
    from vllm_rlt_b200.pd.pull_harness import wire_bytes

    shape = workloads.KVShape("tiny-recurrent", 8, 1, 8, 6, block_size=4)
    w = workloads.recurrent_depth_dedup(shape, requests=3, seed=5, min_len=5, max_len=40, deep_layers=(2, 3, 4, 5))
    per_layer = shape.token_plane_bytes // shape.num_layers
    want = 0
    for (lo, hi), exits in zip(w.ranges, w.exit_planes):
        for e in np.asarray(exits[lo:hi]):
            want += shape.token_plane_bytes + min(int(e), shape.planes - 1) * 4 * per_layer
    assert wire_bytes(w, range(3), "dedup") == want
    assert w.payload_bytes == w.tokens * (shape.token_plane_bytes + (shape.planes - 1) * 4 * per_layer)
