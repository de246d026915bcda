"""PyTorch integration contract of the custom ops (reference tests/test_torch.py:392-489): torch.library.opcheck on
every op, torch.compile(fullgraph=True) without graph breaks, and equality of compiled and eager results."""
import itertools

import pytest
import torch
from torch.library import opcheck

import attention_oracle as oracle
import zigfa
from zigfa._impl import ops

pytestmark = pytest.mark.gpu
OPCHECK = ("test_schema", "test_autograd_registration", "test_faketensor", "test_aot_dispatch_dynamic")


def randn(*shape):
    return torch.randn(*shape, device="cuda", dtype=torch.bfloat16)


def test_attention_ops_pass_opcheck():
    q, k, v = randn(2, 130, 4, 128), randn(2, 130, 2, 128), randn(2, 130, 2, 128)
    scale = 128**-0.5
    opcheck(ops.flash_attn_forward, (q, k, v, None, None, 130, 130, scale, -1, 0), test_utils=OPCHECK)
    out, lse = ops.flash_attn_forward(q, k, v, None, None, 130, 130, scale, -1, 0)
    dout = randn(*out.shape)
    arguments = (dout, q, k, v, out, lse, None, None, 130, 130, scale, -1, 0)
    opcheck(ops.flash_attn_backward, arguments, test_utils=OPCHECK)
    dq, dkv = q.new_empty(q.shape), k.new_empty(2, 130, 2, 2, 128)
    opcheck(ops.flash_attn_backward_packed, (*arguments, dq, dkv), test_utils=OPCHECK)
    # packed (varlen) arguments
    cu = torch.tensor([0, 50, 130], dtype=torch.int32, device="cuda")
    qp, kp, vp = q[0], k[0], v[0]
    opcheck(ops.flash_attn_forward, (qp, kp, vp, cu, cu, 80, 80, scale, 7, 3), test_utils=OPCHECK)


def test_inter_sequence_ops_pass_opcheck():
    lengths = [40, 90, 33]
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device="cuda")
    visible = torch.tensor([[1, 0, 0], [1, 1, 0], [1, 0, 1]], dtype=torch.bool)
    bits = torch.from_numpy(oracle.visibility_bits_of(visible.numpy())).cuda()
    q, k, v = randn(sum(lengths), 4, 128), randn(sum(lengths), 2, 128), randn(sum(lengths), 2, 128)
    opcheck(ops.inter_sequence_metadata, (cu, cu, bits), test_utils=OPCHECK)
    metadata = ops.inter_sequence_metadata(cu, cu, bits)
    layout = (cu, cu, bits, *metadata, None)
    scale = 128**-0.5
    opcheck(ops.inter_sequence_forward, (q, k, v, *layout, scale, -1, 0), test_utils=OPCHECK)
    out, lse = ops.inter_sequence_forward(q, k, v, *layout, scale, -1, 0)
    dout = randn(*out.shape)
    arguments = (dout, q, k, v, out, lse, *layout, scale, -1, 0)
    opcheck(ops.inter_sequence_backward, arguments, test_utils=OPCHECK)
    dq, dkv = q.new_empty(q.shape), k.new_empty(k.shape[0], 2, *k.shape[1:])
    opcheck(ops.inter_sequence_backward_packed, (*arguments, dq, dkv), test_utils=OPCHECK)


def test_compiled_attention_matches_eager():
    torch._dynamo.reset()
    q, k, v = (randn(2, 256, 4, 128).requires_grad_(), randn(2, 256, 2, 128).requires_grad_(),
               randn(2, 256, 2, 128).requires_grad_())

    def attention(q, k, v):
        return zigfa.flash_attn_func(q, k, v, causal=True)

    compiled = torch.compile(attention, fullgraph=True, dynamic=True)
    out = compiled(q, k, v)
    dout = randn(*out.shape)
    gradients = torch.autograd.grad(out, (q, k, v), dout)
    eager = attention(q, k, v)
    eager_gradients = torch.autograd.grad(eager, (q, k, v), dout)
    assert torch.equal(out, eager)
    for compiled_gradient, eager_gradient in zip(gradients, eager_gradients):
        assert (compiled_gradient.float() - eager_gradient.float()).abs().max() < 1e-2
    # a second shape reuses the dynamic graph
    q2, k2, v2 = randn(1, 384, 4, 128), randn(1, 384, 2, 128), randn(1, 384, 2, 128)
    assert torch.equal(compiled(q2, k2, v2), attention(q2, k2, v2))
    torch._dynamo.reset()


def symbolic(fake_mode, shape, dynamic, dtype=torch.bfloat16):
    """A fake CUDA tensor whose dimensions listed in `dynamic` are symbolic sizes of fake_mode's shape environment."""
    from torch.fx.experimental.symbolic_shapes import DimDynamic, StatelessSymbolicContext

    kinds = [DimDynamic.DYNAMIC if index in dynamic else DimDynamic.STATIC for index in range(len(shape))]
    return fake_mode.from_tensor(torch.empty(shape, device="cuda", dtype=dtype),
                                 symbolic_context=StatelessSymbolicContext(dynamic_sizes=kinds))


def test_fake_outputs_keep_symbolic_sizes_and_add_no_guards():
    """Shape functions of the ops under symbolic batch and sequence sizes (reference tests/test_torch.py:427-459): the
    outputs carry the symbols of their inputs, and tracing forward, backward and the packed backward records no guard
    on them, so a compiled graph is not specialised to the sizes it was traced with."""
    from torch._subclasses.fake_tensor import FakeTensorMode
    from torch.fx.experimental.symbolic_shapes import ShapeEnv

    scale = 64**-0.5
    environment = ShapeEnv()
    fake_mode = FakeTensorMode(shape_env=environment)
    q = symbolic(fake_mode, (3, 136, 8, 64), (0, 1))
    k, v = (symbolic(fake_mode, (3, 200, 2, 64), (0, 1)) for _ in range(2))
    before = len(environment.guards)
    with fake_mode:
        out, lse = torch.ops.zigfa.flash_attn_forward(q, k, v, None, None, q.shape[1], k.shape[1], scale, -1, 0)
        dq, dk, dv = torch.ops.zigfa.flash_attn_backward(out, q, k, v, out, lse, None, None, q.shape[1], k.shape[1],
                                                         scale, -1, 0)
        dkv = k.new_empty((*k.shape[:-2], 2, *k.shape[-2:]))
        torch.ops.zigfa.flash_attn_backward_packed(out, q, k, v, out, lse, None, None, q.shape[1], k.shape[1], scale,
                                                   -1, 0, dq, dkv)
    for size in (out.shape[0], out.shape[1], lse.shape[0], lse.shape[2], dq.shape[1], dk.shape[0], dk.shape[1], dv.shape[1]):
        assert isinstance(size, torch.SymInt)
    assert len(environment.guards) == before

    # packed (varlen) layout: the token count is the symbolic size
    environment = ShapeEnv()
    fake_mode = FakeTensorMode(shape_env=environment)
    q = symbolic(fake_mode, (310, 8, 64), (0,))
    k, v = (symbolic(fake_mode, (420, 2, 64), (0,)) for _ in range(2))
    cu = fake_mode.from_tensor(torch.zeros(6, dtype=torch.int32, device="cuda"))
    before = len(environment.guards)
    with fake_mode:
        out, lse = torch.ops.zigfa.flash_attn_forward(q, k, v, cu, cu, 128, 128, scale, -1, 0)
    assert isinstance(out.shape[0], torch.SymInt) and isinstance(lse.shape[1], torch.SymInt)
    assert len(environment.guards) == before
