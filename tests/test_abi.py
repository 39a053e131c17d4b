"""The C-ABI library and the torch op library: they load, export what the header declares, and reject bad arguments.

No kernel is launched here; these run without a GPU.
"""

import ctypes as C
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "rlt_kv_handoff.h"


@pytest.fixture(scope="module")
def lib():
    from vllm_rlt_b200 import _build, _lib

    _build.build_library()
    return _lib.load()


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"RLT_API\s+[\w\s\*]+?\b(rlt_\w+)\s*\(", text)))


def test_header_and_ctypes_agree_on_the_symbol_list(lib):
    from vllm_rlt_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 28
    assert names == sorted(_lib.SIGNATURES)
    for name in names:
        assert getattr(lib, name) is not None


def test_header_compiles_as_plain_c(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "rlt_kv_handoff.h"\nint main(void){RltPool p; RltBatch b; RltOptions o; RltHostBatch h; (void)p;(void)b;(void)o;(void)h; return RLT_OK;}\n')
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", f"-I{HEADER.parent}", "-c", str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_struct_layouts_match_the_compiler(tmp_path):
    from vllm_rlt_b200 import _lib

    src = tmp_path / "s.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "rlt_kv_handoff.h"\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(RltRegion), sizeof(RltPool), sizeof(RltBatch),"
        " sizeof(RltOptions), offsetof(RltPool, num_blocks), offsetof(RltBatch, exit_count), offsetof(RltOptions, status),"
        " sizeof(RltHostBatch), offsetof(RltHostBatch, tok_end));return 0;}\n"
    )
    exe = tmp_path / "s"
    subprocess.run(["gcc", f"-I{HEADER.parent}", str(src), "-o", str(exe)], check=True)
    got = list(map(int, subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()))
    want = [C.sizeof(_lib.RltRegion), C.sizeof(_lib.RltPool), C.sizeof(_lib.RltBatch), C.sizeof(_lib.RltOptions),
            _lib.RltPool.num_blocks.offset, _lib.RltBatch.exit_count.offset, _lib.RltOptions.status.offset,
            C.sizeof(_lib.RltHostBatch), _lib.RltHostBatch.tok_end.offset]
    assert got == want


def test_information_entry_points(lib):
    assert lib.rlt_version() == 1
    assert lib.rlt_error_string(0) == b"ok"
    assert b"geometry" in lib.rlt_error_string(-2)
    assert lib.rlt_kernel_launches() >= 0


def test_argument_errors_are_found_on_the_host_before_any_launch(lib):
    """Null structs, bad modes and non-dense pools are rejected without touching a device."""
    from vllm_rlt_b200 import _lib

    assert lib.rlt_kv_handoff(None, None, None, None, None) == _lib.RLT_E_INVALID
    region = _lib.RltRegion(0x1000, 0x2000, 2 * 4 * 64, 4 * 64, 64)
    none = _lib.RltRegion(None, None, 0, 0, 0)
    pool = _lib.RltPool(region, none, 8, 4, 2, 1)
    batch = _lib.RltBatch(1, 2, 0x3000, 0x4000, 0x5000, 0x6000, None, None)
    opts = _lib.RltOptions(7, 0, 0, 0, None, 0, 0)
    assert lib.rlt_kv_handoff(C.byref(pool), C.byref(pool), C.byref(batch), C.byref(opts), None) == _lib.RLT_E_INVALID
    opts.mode = _lib.MODE_DEDUP  # needs exit planes
    assert lib.rlt_kv_handoff(C.byref(pool), C.byref(pool), C.byref(batch), C.byref(opts), None) == _lib.RLT_E_INVALID
    batch.exit_planes, batch.exit_offsets, batch.exit_count = 0x8000, 0x9000, 0  # an exit array of unknown length
    assert lib.rlt_kv_handoff(C.byref(pool), C.byref(pool), C.byref(batch), C.byref(opts), None) == _lib.RLT_E_INVALID
    batch.exit_planes = batch.exit_offsets = None
    opts.mode = _lib.MODE_ALL_PLANES
    opts.layer_begin, opts.layer_end = 1, 1
    assert lib.rlt_kv_handoff(C.byref(pool), C.byref(pool), C.byref(batch), C.byref(opts), None) == _lib.RLT_E_INVALID
    opts.layer_begin, opts.layer_end = 0, 0
    sparse = _lib.RltPool(_lib.RltRegion(0x1000, 0x2000, 2 * 4 * 64 + 64, 4 * 64, 64), none, 8, 4, 2, 1)
    assert lib.rlt_kv_handoff(C.byref(sparse), C.byref(pool), C.byref(batch), C.byref(opts), None) == _lib.RLT_E_GEOMETRY
    other = _lib.RltPool(_lib.RltRegion(0x1000, 0x2000, 2 * 4 * 128, 4 * 128, 128), none, 8, 4, 2, 1)
    assert lib.rlt_kv_handoff(C.byref(pool), C.byref(other), C.byref(batch), C.byref(opts), None) == _lib.RLT_E_GEOMETRY
    batch.num_requests = _lib.MAX_REQUESTS + 1
    assert lib.rlt_kv_handoff(C.byref(pool), C.byref(pool), C.byref(batch), C.byref(opts), None) == _lib.RLT_E_LIMIT
    batch.num_requests = 1
    assert lib.rlt_kv_pack(C.byref(pool), C.byref(batch), C.byref(opts), 0x7001, 64, None) == _lib.RLT_E_ALIGN
    opts.deep_layer_mask = 0b10  # a per-depth layer subset would leave holes in a packed image: handoff only
    assert lib.rlt_kv_pack(C.byref(pool), C.byref(batch), C.byref(opts), 0x7000, 64, None) == _lib.RLT_E_INVALID
    opts.deep_layer_mask = 0
    assert lib.rlt_kv_packed_bytes(C.byref(pool), 10, 3, 2) == 10 * 3 * 2 * 2 * 64
    # the host-table form: same refusals, all before the staging ring or a device is touched
    assert lib.rlt_kv_host_batch_limit() == 64 * 1024
    assert lib.rlt_kv_handoff_host(None, None, None, None, None) == _lib.RLT_E_INVALID
    tables = (C.c_int32 * 2)(0, 1)
    one = (C.c_int32 * 1)(0)
    host = _lib.RltHostBatch(1, 2, 1, 1, C.addressof(tables), C.addressof(tables), C.addressof(one), C.addressof(one))
    opts.mode = _lib.MODE_DEDUP  # per-token exit planes do not come through this form
    assert lib.rlt_kv_handoff_host(C.byref(pool), C.byref(pool), C.byref(host), C.byref(opts), None) == _lib.RLT_E_INVALID
    opts.mode = _lib.MODE_ALL_PLANES
    host.src_planes = 2  # the pool has one plane
    assert lib.rlt_kv_handoff_host(C.byref(pool), C.byref(pool), C.byref(host), C.byref(opts), None) == _lib.RLT_E_GEOMETRY
    host.src_planes, host.table_width = 1, 64 * 1024  # 2 x 256 KiB of tables: more than a staging slot
    assert lib.rlt_kv_handoff_host(C.byref(pool), C.byref(pool), C.byref(host), C.byref(opts), None) == _lib.RLT_E_LIMIT
    host.table_width, host.tok_end = 2, None
    assert lib.rlt_kv_handoff_host(C.byref(pool), C.byref(pool), C.byref(host), C.byref(opts), None) == _lib.RLT_E_INVALID
    assert lib.rlt_kv_copy_segments(None, 1, None) == _lib.RLT_E_INVALID
    assert lib.rlt_kv_copy_segments(0x1000, _lib.MAX_SEGMENTS + 1, None) == _lib.RLT_E_LIMIT
    assert lib.rlt_kv_copy_segments(None, 0, None) == _lib.RLT_OK
    assert lib.rlt_kv_push(None, None, 0, None) == _lib.RLT_OK
    assert lib.rlt_kv_signal(0x1004, 1, None) == _lib.RLT_E_ALIGN
    assert lib.rlt_kv_wait(0x1000, 1, 0, 0x2000, None) == _lib.RLT_E_LIMIT
    assert lib.rlt_kv_wait(0x1000, 1, _lib.MAX_WAIT_NS + 1, 0x2000, None) == _lib.RLT_E_LIMIT


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from vllm_rlt_b200 import _lib

    _lib.load.cache_clear()
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "absent.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()
    _lib.load.cache_clear()


def test_importing_the_package_creates_no_cuda_context():
    """Same property the reference pins for its native op (tests/test_activation.py:111-128)."""
    code = (
        "import sys, torch; import vllm_rlt_b200, vllm_rlt_b200.kernels.kv_handoff; "
        "assert not torch.cuda.is_initialized(); print('ok')"
    )
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=ROOT)
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr


def test_torch_ops_are_registered_in_the_reference_namespace():
    import torch

    from vllm_rlt_b200 import _build

    _build.build_all()
    torch.ops.load_library(str(_build.PACKAGE / _build.OPS_NAME))
    for name in ("kv_handoff", "kv_handoff_host", "kv_handoff_peer", "kv_pack", "kv_scatter", "kv_push", "kv_copy_segments", "kv_signal", "kv_wait"):
        assert hasattr(torch.ops.vllm_rlt, name)
    schema = str(torch.ops.vllm_rlt.kv_scatter.default._schema)
    assert "Tensor(a!) key" in schema
    # CPU tensors are rejected by dispatch: there is no CPU kernel behind these ops
    k = torch.zeros(2, 1, 4, 1, 8)
    t = torch.zeros(1, 1, 1, dtype=torch.int32)
    r = torch.zeros(1, dtype=torch.int32)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.vllm_rlt.kv_handoff(k, k, None, None, k.clone(), k.clone(), None, None, t, t, r, r, None, None, 0, 0, 0, None)


def test_op_loader_registers_the_ops_once_and_fails_loudly_when_unbuilt(monkeypatch, tmp_path):
    import torch

    from vllm_rlt_b200 import _build, _lib

    _build.build_all()
    _lib.load_ops.cache_clear()
    ops = _lib.load_ops()
    assert ops is torch.ops.vllm_rlt and hasattr(ops, "kv_handoff")
    assert _lib.load_ops() is ops  # remembered
    # never built: a clear error, and the failure is not remembered
    _lib.load_ops.cache_clear()
    monkeypatch.setattr(_lib, "OPS_PATH", tmp_path / "_C.so")
    assert not _lib.ops_built()
    for _ in range(2):
        with pytest.raises(RuntimeError, match="not built"):
            _lib.load_ops()
    # present but not loadable: the loader's own error comes through
    (tmp_path / "_C.so").write_bytes(b"not a shared object")
    with pytest.raises(OSError):
        _lib.load_ops()
    _lib.load_ops.cache_clear()
