"""The forward entry point that needs no caller workspace (b200fa_fwd_noalloc), called through the C ABI.

Some users of the library cannot allocate device memory around an attention call: their memory is planned up front,
or their binding owns nothing but the input and output tensors. For them the library keeps the work list of a packed
batch in a small array of its own. These tests check that this path returns exactly what the regular entry point
(b200fa_fwd with a caller workspace) returns, on two different batches in a row -- the second smaller than the first,
so stale entries of the first call are still in the shared array -- and that a batch too large for the array is refused
with a clear message. The file name sorts last so that a run that stops at the first failure has already run every
other test.
"""
import ctypes
import itertools

import pytest
import torch

from zigfa._impl import lib

pytestmark = pytest.mark.gpu


def forward_arguments(q, k, v, cu_q, cu_k, window, workspace, **visibility):
    out = torch.full_like(q, float("nan"))
    lse = torch.full((q.shape[1], q.shape[0]), float("nan"), device=q.device)
    problem = lib.make_problem(q, k, cu_q, cu_k, q.shape[-1] ** -0.5, *window, **visibility)
    args = lib.FwdArgs(
        problem=problem, q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(), softmax_lse=lse.data_ptr(),
        q_stride=lib.strides3(q, True), k_stride=lib.strides3(k, True), v_stride=lib.strides3(v, True),
        out_stride=lib.strides3(out, True), lse_stride=lib.Stride2(0, lse.stride(0)),
        workspace=None if workspace is None else workspace.data_ptr(),
        workspace_bytes=0 if workspace is None else workspace.numel(),
    )
    return args, out, lse


def prepared_visibility(cu, visible):
    """The inter-sequence metadata of a boolean (query sequence, key sequence) matrix, made by the library itself."""
    count = len(visible)
    words = (count + 31) // 32
    rows = [[0] * words for _ in range(count)]
    for i, j in itertools.product(range(count), repeat=2):
        if visible[i][j]:
            rows[i][j // 32] |= 1 << (j % 32)
    bits = torch.tensor(rows, dtype=torch.int64).to(torch.int32).cuda()
    bits_t = torch.empty_like(bits)
    cu_visible_k, cu_visible_q = (torch.empty(count + 1, dtype=torch.int32, device="cuda") for _ in range(2))
    status = lib.library().b200fa_interseq_metadata(
        cu.data_ptr(), cu.data_ptr(), bits.data_ptr(), count, bits_t.data_ptr(), cu_visible_k.data_ptr(),
        cu_visible_q.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert status == 0, lib.last_error()
    return dict(visibility_bits=bits, visibility_bits_t=bits_t, cu_visible_k=cu_visible_k, cu_visible_q=cu_visible_q)


def run_both(lengths, heads_q, heads_kv, head_dim, window, seed, visible=None, same_work_list=True):
    library = lib.library()
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(seed)
    total = sum(lengths)
    q = torch.randn(total, heads_q, head_dim, device="cuda", dtype=torch.bfloat16)
    k, v = (torch.randn(total, heads_kv, head_dim, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device="cuda")
    visibility = {} if visible is None else prepared_visibility(cu, visible)
    problem = lib.make_problem(q, k, cu, cu, head_dim**-0.5, *window, **visibility)
    workspace = torch.empty(max(library.b200fa_fwd_workspace_bytes(ctypes.byref(problem)), 1), dtype=torch.uint8, device="cuda")
    regular, out_regular, lse_regular = forward_arguments(q, k, v, cu, cu, window, workspace, **visibility)
    assert library.b200fa_fwd(ctypes.byref(regular), stream) == 0, lib.last_error()
    # no workspace at all: the pointer is null and the size zero
    bare, out_bare, lse_bare = forward_arguments(q, k, v, cu, cu, window, None, **visibility)
    assert library.b200fa_fwd_noalloc(ctypes.byref(bare), stream) == 0, lib.last_error()
    torch.cuda.synchronize()
    assert not torch.isnan(out_regular).any()
    if same_work_list:
        # same kernels, same work list: the results are identical, not merely close
        assert torch.equal(out_bare, out_regular)
        assert torch.equal(lse_bare, lse_regular)
    else:
        # Other rows share a row's warp. When one of them sets keys aside (a near-zero block maximum, fwd_common.cuh) the
        # whole warp sums the block in the order of that rare path, so a row's sum may round differently in its last
        # bit: the log-sum-exp moves by one FP32 step, and 1 / sum may tip the BF16 rounding of an output element (one
        # element in 138 million in this batch).
        different = out_bare != out_regular
        assert int(different.sum()) <= max(1, out_regular.numel() // 10_000_000)
        step = (out_bare.float() - out_regular.float()).abs()
        assert (step <= 2.0**-7 * out_regular.float().abs()).all()
        finite = torch.isfinite(lse_regular)
        assert torch.equal(torch.isfinite(lse_bare), finite)
        assert ((lse_bare - lse_regular)[finite].abs() <= 2.0**-22 * lse_regular[finite].abs().clamp(min=1.0)).all()


def test_noalloc_forward_matches_the_regular_entry_point_twice_in_a_row():
    run_both([700, 33, 0, 1500, 256, 911], 8, 2, 128, (-1, 0), seed=11)
    run_both([120, 300], 4, 4, 64, (50, 10), seed=12)


def test_noalloc_forward_with_the_smaller_work_items_of_head_dim_256():
    # head_dim 256 draws work items of 128 query rows (twice the entries per token), packed batch, then a shorter one
    run_both([300, 0, 129, 1024, 77], 4, 2, 256, (-1, 0), seed=13)
    run_both([128, 65], 2, 1, 256, (-1, -1), seed=14)


def test_noalloc_forward_with_an_inter_sequence_batch():
    # shared prefixes: the work list is sorted by visible key tokens (cu_visible_k), not by the sequences' own lengths
    lengths = [512, 100, 37, 300, 64, 200]
    prefix_of = [0, 0, 0, 3, 3, 3]
    visible = [[j == i or j == prefix_of[i] for j in range(len(lengths))] for i in range(len(lengths))]
    run_both(lengths, 8, 2, 128, (-1, 0), seed=15, visible=visible)
    run_both(lengths[:3], 4, 4, 256, (-1, 0), seed=16, visible=[row[:3] for row in visible[:3]])


def test_noalloc_forward_runs_unpacked_when_the_finer_work_list_does_not_fit():
    """Groups of four query heads are packed into work items of 64 tokens, whose work list (11 390 entries here) exceeds
    the built-in scratch; the list with one head per work item (5097 entries) fits, so the call runs that way and returns
    what the regular entry point computes with packed heads."""
    library = lib.library()
    lengths = [180] * 3000
    probe = lib.Problem(batch=len(lengths), seqlen_q=sum(lengths), seqlen_k=sum(lengths), heads_q=4, heads_kv=1, head_dim=64,
                        window_left=-1, window_right=0, softmax_scale=0.125, cu_seqlens_q=8, cu_seqlens_k=8)
    assert library.b200fa_fwd_workspace_bytes(ctypes.byref(probe)) > 8192 * 8
    assert library.b200fa_work_list_entries(sum(lengths), len(lengths), 256) <= 8192
    run_both(lengths, 4, 1, 64, (-1, 0), seed=17, same_work_list=False)


def test_noalloc_forward_refuses_batches_beyond_its_scratch():
    library = lib.library()
    # shape-only check on the host: 8193 sequences of one row need 8193 work-list entries, one more than the array holds
    q = torch.empty(8193, 1, 128, device="cuda", dtype=torch.bfloat16)
    cu = torch.arange(8194, dtype=torch.int32, device="cuda")
    args, _, _ = forward_arguments(q, q, q, cu, cu, (-1, -1), None)
    assert library.b200fa_fwd_noalloc(ctypes.byref(args), torch.cuda.current_stream().cuda_stream) == -1
    assert "b200fa_fwd_noalloc" in lib.last_error() and "8192" in lib.last_error()
    torch.cuda.synchronize()
