"""The C-ABI library loads without a GPU and exports every symbol include/b200fa.h declares; the pure host entry
points (workspace sizes, version, head dims, errors) answer without a CUDA context."""
import ctypes
import re
from pathlib import Path

import pytest

from zigfa._impl import lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200fa.h"


def declared_symbols():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"\b(b200fa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    library = lib.library()
    symbols = declared_symbols()
    assert len(symbols) >= 15
    for name in symbols:
        assert hasattr(library, name), f"{name} is declared in b200fa.h but not exported"
    assert set(symbols) == set(lib.EXPORTS)


def test_version_and_head_dims():
    library = lib.library()
    assert library.b200fa_version() >= 100
    assert library.b200fa_supports_head_dim(128, 0) == 1
    assert library.b200fa_supports_head_dim(64, 1) == 1
    assert library.b200fa_supports_head_dim(80, 0) == 0
    assert library.b200fa_supports_head_dim(96, 1) == 1 and library.b200fa_supports_head_dim(72, 0) == 1
    assert library.b200fa_supports_head_dim(256, 0) == 1 and library.b200fa_supports_head_dim(256, 1) == 1
    assert library.b200fa_supports_head_dim(512, 0) == 1 and library.b200fa_supports_head_dim(512, 1) == 0
    assert library.b200fa_supports_head_dim(384, 0) == 0


def problem(**fields):
    defaults = dict(batch=2, seqlen_q=512, seqlen_k=512, heads_q=8, heads_kv=2, head_dim=128, window_left=-1,
                    window_right=0, softmax_scale=0.088)
    defaults.update(fields)
    return lib.Problem(**defaults)


def test_workspace_sizes_are_shape_functions():
    library = lib.library()
    fixed = problem()
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(fixed)) == 0
    rows = 2 * 512
    stats = 8 * rows * 4
    assert library.b200fa_bwd_workspace_bytes(ctypes.byref(fixed)) == 2 * stats + 8 * rows * 128 * 4
    packed = problem(batch=3, seqlen_q=1000, seqlen_k=900, cu_seqlens_q=8, cu_seqlens_k=8)
    entries = library.b200fa_work_list_entries(1000, 3, 256)
    assert entries == (1000 + 3 * 255) // 256
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(packed)) == entries * 8
    assert library.b200fa_work_list_entries(5, 10, 256) == 5
    assert library.b200fa_work_list_entries(0, 4, 256) == 0


def test_invalid_arguments_report_errors_without_a_gpu():
    library = lib.library()
    args = lib.FwdArgs(problem=problem(heads_q=6, heads_kv=4))
    assert library.b200fa_fwd(ctypes.byref(args), None) == -1
    assert "multiple" in lib.last_error()
    with pytest.raises(ValueError, match="multiple"):
        lib.check(-1)
    args = lib.FwdArgs(problem=problem(window_left=-5))
    assert library.b200fa_fwd(ctypes.byref(args), None) == -1
    assert "window" in lib.last_error()
    bad_stride = lib.FwdArgs(problem=problem(), q_stride=lib.Stride3(1, 3, 5))
    assert library.b200fa_fwd(ctypes.byref(bad_stride), None) == -1
    assert "multiples of 8" in lib.last_error()
