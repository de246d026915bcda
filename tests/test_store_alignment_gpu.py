"""The kernels write the rows of out, dK and dV with 32-byte stores when base addresses and strides are multiples of
32 bytes and with 16-byte stores otherwise (a thread owns a row, so a 16-byte store fills half a sector). Tensors made
by PyTorch always take the wide path; here the same problems are written into tensors that start 16 bytes into their
buffers, through the C ABI, and must give the same bits."""
import ctypes
import itertools

import pytest
import torch

from zigfa._impl import lib

pytestmark = pytest.mark.gpu


def strides(tensor):
    return lib.strides3(tensor, True)


def shifted_like(tensor):
    """A tensor of the same shape whose first element sits 16 bytes behind a 32-byte boundary, and its buffer."""
    buffer = torch.full((tensor.numel() + 8,), float("nan"), device="cuda", dtype=torch.bfloat16)
    view = buffer[8:].view_as(tensor)
    assert view.data_ptr() % 32 == 16
    return view, buffer


def run(lengths, heads_q, heads_kv, head_dim, backward, shift):
    library = lib.library()
    stream = torch.cuda.current_stream().cuda_stream
    torch.manual_seed(head_dim + heads_q)
    total = sum(lengths)
    q = torch.randn(total, heads_q, head_dim, device="cuda", dtype=torch.bfloat16)
    k, v = (torch.randn(total, heads_kv, head_dim, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    dout = torch.randn_like(q)
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device="cuda")
    problem = lib.make_problem(q, k, cu, cu, head_dim**-0.5, -1, 0)
    make = (lambda t: shifted_like(t)) if shift else (lambda t: (torch.full_like(t, float("nan")), None))
    (out, out_buffer), (dq, _), (dk, dk_buffer), (dv, dv_buffer) = make(q), make(q), make(k), make(v)
    lse = torch.full((heads_q, total), float("nan"), device="cuda")
    workspace = torch.empty(max(library.b200fa_fwd_workspace_bytes(ctypes.byref(problem)), 1), dtype=torch.uint8, device="cuda")
    forward = lib.FwdArgs(problem=problem, q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(),
                          softmax_lse=lse.data_ptr(), q_stride=strides(q), k_stride=strides(k), v_stride=strides(v),
                          out_stride=strides(out), lse_stride=lib.Stride2(0, lse.stride(0)), workspace=workspace.data_ptr(),
                          workspace_bytes=workspace.numel())
    assert library.b200fa_fwd(ctypes.byref(forward), stream) == 0, lib.last_error()
    results = [out, lse]
    if backward:
        scratch = torch.empty(max(library.b200fa_bwd_workspace_bytes(ctypes.byref(problem)), 256), dtype=torch.uint8, device="cuda")
        arguments = lib.BwdArgs(problem=problem, q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(),
                                dout=dout.data_ptr(), softmax_lse=lse.data_ptr(), dq=dq.data_ptr(), dk=dk.data_ptr(),
                                dv=dv.data_ptr(), q_stride=strides(q), k_stride=strides(k), v_stride=strides(v),
                                out_stride=strides(out), dout_stride=strides(dout), dq_stride=strides(dq),
                                dk_stride=strides(dk), dv_stride=strides(dv), lse_stride=lib.Stride2(0, lse.stride(0)),
                                workspace=scratch.data_ptr(), workspace_bytes=scratch.numel())
        assert library.b200fa_bwd(ctypes.byref(arguments), stream) == 0, lib.last_error()
        results += [dk, dv]
    torch.cuda.synchronize()
    for buffer in (out_buffer, dk_buffer, dv_buffer):
        assert buffer is None or torch.isnan(buffer[:8]).all()  # nothing was written in front of the tensor
    return [t.clone() for t in results]


@pytest.mark.parametrize("head_dim, backward", [(64, True), (96, True), (128, True), (256, True), (512, False)])
def test_tensors_on_a_16_byte_boundary_give_the_same_bits(head_dim, backward):
    lengths, heads_q, heads_kv = [300, 129, 64], 4, 2
    aligned = run(lengths, heads_q, heads_kv, head_dim, backward, shift=False)
    shifted = run(lengths, heads_q, heads_kv, head_dim, backward, shift=True)
    assert not any(torch.isnan(t).any() for t in aligned)
    for name, one, other in zip(("out", "lse", "dk", "dv"), aligned, shifted):
        assert torch.equal(one, other), name
