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
    # lse_log2, dpsum, pivot_sum, pivot_key; the FP32 dQ accumulator; the flag block and the FP32 pivot terms of dK
    key_rows = 2 * 512
    assert library.b200fa_bwd_workspace_bytes(ctypes.byref(fixed)) == (
        4 * stats + 8 * rows * 128 * 4 + 256 + 2 * key_rows * 128 * 4)
    # one query head per key head: a work-list entry covers 256 query rows of a sequence
    packed = problem(batch=3, seqlen_q=1000, seqlen_k=900, heads_q=2, heads_kv=2, cu_seqlens_q=8, cu_seqlens_k=8)
    entries = library.b200fa_work_list_entries(1000, 3, 256)
    assert entries == (1000 + 3 * 255) // 256
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(packed)) == entries * 8
    # groups of four query heads are packed into the rows of a work item: an entry covers 64 tokens of all four heads
    grouped = problem(batch=3, seqlen_q=1000, seqlen_k=900, cu_seqlens_q=8, cu_seqlens_k=8)
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(grouped)) == library.b200fa_work_list_entries(1000, 3, 64) * 8
    long_batch = problem(batch=3, seqlen_q=1_000_000, seqlen_k=900, cu_seqlens_q=8, cu_seqlens_k=8)
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(long_batch)) == library.b200fa_work_list_entries(1_000_000, 3, 64) * 8
    # groups that are no power of two and head dims above 128 keep one head per work item
    odd_group = problem(batch=3, seqlen_q=1000, seqlen_k=900, heads_q=6, heads_kv=2, cu_seqlens_q=8, cu_seqlens_k=8)
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(odd_group)) == entries * 8
    wide = problem(batch=3, seqlen_q=1000, seqlen_k=900, head_dim=256, cu_seqlens_q=8, cu_seqlens_k=8)
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(wide)) == library.b200fa_work_list_entries(1000, 3, 128) * 8
    assert library.b200fa_work_list_entries(5, 10, 256) == 5
    assert library.b200fa_work_list_entries(0, 4, 256) == 0


def test_pivot_setting_round_trips():
    library = lib.library()
    before = library.b200fa_set_pivot_ds(-1)
    assert before in (0, 1)
    assert library.b200fa_set_pivot_ds(1) == before
    assert library.b200fa_set_pivot_ds(-1) == 1
    assert library.b200fa_set_pivot_ds(before) == 1
    assert library.b200fa_set_pivot_ds(-1) == before


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


def test_backward_rejects_null_and_misaligned_pointers_without_a_launch():
    """b200fa_bwd reads and writes through raw 16-byte accesses: a null or misaligned tensor pointer must come back as an
    error code from the host checks (no CUDA context is needed to reach them), never as a fault on the device."""
    library = lib.library()
    aligned = 1 << 20  # a pointer value that passes the alignment checks; nothing dereferences it on these paths
    names = ("q", "k", "v", "out", "dout", "softmax_lse", "dq", "dk", "dv")

    def arguments(**overrides):
        fields = {name: aligned for name in names}
        fields.update(overrides)
        return lib.BwdArgs(problem=problem(), **fields)

    for name in names:
        assert library.b200fa_bwd(ctypes.byref(arguments(**{name: None})), None) == -1, name
        assert "null tensor pointer" in lib.last_error()
    for name in ("q", "k", "v", "out", "dout", "dq", "dk", "dv"):
        assert library.b200fa_bwd(ctypes.byref(arguments(**{name: aligned + 8})), None) == -1, name
        assert "16-byte aligned" in lib.last_error()
    assert library.b200fa_bwd(ctypes.byref(arguments(softmax_lse=aligned + 2)), None) == -1
    assert "4-byte aligned" in lib.last_error()


def test_noalloc_forward_checks_sizes_before_anything_else():
    library = lib.library()
    negative = lib.FwdArgs(problem=problem(batch=-1))
    assert library.b200fa_fwd_noalloc(ctypes.byref(negative), None) == -1
    assert "negative sizes" in lib.last_error()
    # 8192 entries are the limit; entries cover 256 query rows up to head_dim 128 and 128 rows above
    too_long = lib.FwdArgs(problem=problem(batch=1, seqlen_q=256 * 8192 + 1, seqlen_k=16, cu_seqlens_q=8, cu_seqlens_k=8))
    assert library.b200fa_fwd_noalloc(ctypes.byref(too_long), None) == -1
    assert "entries of 256 query rows" in lib.last_error()
    too_long_256 = lib.FwdArgs(problem=problem(batch=1, seqlen_q=128 * 8192 + 1, seqlen_k=16, head_dim=256,
                                               cu_seqlens_q=8, cu_seqlens_k=8))
    assert library.b200fa_fwd_noalloc(ctypes.byref(too_long_256), None) == -1
    assert "entries of 128 query rows at head_dim 256" in lib.last_error()
