"""Short queries over long keys (decode and extend shapes): the forward pass deals the key blocks of a tile out to
several work items and merges their partial results (split-KV). The shapes are those of the reference's
tests/test_torch.py:270-291; results are checked against the float32 oracle with the tolerance of the other forward
tests, and against the same problem run unsplit through the entry point that has no room for partial results."""
import ctypes

import pytest
import torch

import parity
import zigfa
from zigfa._impl import lib

pytestmark = pytest.mark.gpu

# (batch, seqlen_q, seqlen_k, heads_q, heads_kv), window
SHAPES = {
    "gqa_decode": ((1, 1, 4096, 8, 2), (-1, 0)),
    "mha_decode": ((2, 1, 2048, 4, 4), (-1, -1)),
    "windowed_extend": ((1, 16, 2048, 8, 2), (512, 0)),
    "uneven_lengths": ((1, 100, 3001, 4, 1), (-1, 0)),
    "two_tiles": ((1, 300, 8192, 2, 1), (-1, -1)),
}


def tensors(shape, head_dim, seed):
    batch, seqlen_q, seqlen_k, heads_q, heads_kv = shape
    torch.manual_seed(seed)
    q = torch.randn(batch, seqlen_q, heads_q, head_dim, device="cuda", dtype=torch.bfloat16)
    k, v = (torch.randn(batch, seqlen_k, heads_kv, head_dim, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    return q, k, v


@pytest.mark.parametrize("head_dim", [64, 72, 96, 128])
@pytest.mark.parametrize("name", SHAPES)
def test_split_kv_matches_the_oracle(head_dim, name):
    shape, window = SHAPES[name]
    q, k, v = tensors(shape, head_dim, head_dim + shape[1])
    problem = lib.make_problem(q, k, None, None, head_dim**-0.5, *window)
    assert lib.library().b200fa_fwd_workspace_bytes(ctypes.byref(problem)) > 0, "the planner must split this shape"
    causal = window[1] == 0
    qg, kg, vg = (x.clone().requires_grad_() for x in (q, k, v))
    out, lse = zigfa.flash_attn_func(qg, kg, vg, causal=causal, window_size=(window[0], -1 if causal else window[1]),
                                     return_attn_probs=True)
    dout = torch.randn_like(out)
    grads = torch.autograd.grad(out, (qg, kg, vg), dout)
    parity.check_fixed((out.detach(), lse, grads), q, k, v, dout, causal, window, notes=f"[split-kv {name} d{head_dim}]")


@pytest.mark.parametrize("name", ["gqa_decode", "uneven_lengths"])
def test_split_and_unsplit_runs_agree(name):
    """The same problem through b200fa_fwd with a workspace (split) and through b200fa_fwd_noalloc, whose 64 KiB of
    scratch are too small for these partial results (unsplit): the two differ only by the order of the summation."""
    shape, window = SHAPES[name]
    head_dim = 128
    q, k, v = tensors(shape, head_dim, 7)
    library = lib.library()
    stream = torch.cuda.current_stream().cuda_stream
    results = []
    for entry in (library.b200fa_fwd, library.b200fa_fwd_noalloc):
        out = torch.full_like(q, float("nan"))
        lse = torch.full((q.shape[0], q.shape[2], q.shape[1]), float("nan"), device="cuda")
        problem = lib.make_problem(q, k, None, None, head_dim**-0.5, *window)
        nbytes = library.b200fa_fwd_workspace_bytes(ctypes.byref(problem))
        assert nbytes > 65536
        workspace = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        args = lib.FwdArgs(problem=problem, q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(),
                           softmax_lse=lse.data_ptr(), q_stride=lib.strides3(q, False), k_stride=lib.strides3(k, False),
                           v_stride=lib.strides3(v, False), out_stride=lib.strides3(out, False),
                           lse_stride=lib.Stride2(lse.stride(0), lse.stride(1)), workspace=workspace.data_ptr(),
                           workspace_bytes=nbytes)
        assert entry(ctypes.byref(args), stream) == 0, lib.last_error()
        torch.cuda.synchronize()
        results.append((out, lse))
    (split_out, split_lse), (plain_out, plain_lse) = results
    assert not torch.isnan(split_out).any() and not torch.isnan(plain_out).any()
    assert (split_out.float() - plain_out.float()).abs().max() <= 2**-7 * plain_out.float().abs().max()
    assert (split_lse - plain_lse).abs().max() < 1e-4
