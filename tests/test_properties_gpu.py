"""Size-independent properties of the attention path at the full size of the headline configuration (batch 4,
seqlen 8192, heads 32/8, head_dim 128, causal). Every property here is exact: the kernels compute out, lse, dK and dV
in a fixed order per tile, so these comparisons are bit for bit. dQ is summed with floating-point reductions whose
order is not fixed (the reference refuses `deterministic=True` for the same reason, reference
src/zigfa/_impl/ops.py:368-371), so dQ is compared with a tolerance of a few FP32 roundings of its largest term."""
import pytest
import torch

import zigfa

pytestmark = pytest.mark.gpu

BATCH, SEQLEN, HEADS_Q, HEADS_KV, D = 4, 8192, 32, 8, 128


def randn(*shape):
    return torch.randn(*shape, device="cuda", dtype=torch.bfloat16)


def run(q, k, v, dout, **options):
    q, k, v = (t.detach().requires_grad_() for t in (q, k, v))
    out, lse = zigfa.flash_attn_func(q, k, v, return_attn_probs=True, **options)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    return out.detach(), lse, dq, dk, dv


@pytest.fixture(scope="module")
def problem():
    torch.manual_seed(11)
    q, k, v = randn(BATCH, SEQLEN, HEADS_Q, D), randn(BATCH, SEQLEN, HEADS_KV, D), randn(BATCH, SEQLEN, HEADS_KV, D)
    dout = randn(BATCH, SEQLEN, HEADS_Q, D)
    return q, k, v, dout, run(q, k, v, dout, causal=True)


def dq_close(ours, theirs):
    # BF16 results of two summation orders: equal up to one BF16 rounding step of the value
    difference = (ours.float() - theirs.float()).abs()
    return bool((difference <= 2**-7 * theirs.float().abs() + 1e-6).all())


def test_batch_entries_are_independent(problem):
    """A batch shard computed alone equals its slice of the whole batch: the multi-GPU split by batch entries changes
    no bit of out, lse, dK, dV."""
    q, k, v, dout, (out, lse, dq, dk, dv) = problem
    for entries in (slice(2, 3), slice(0, 2)):
        part = run(q[entries], k[entries], v[entries], dout[entries], causal=True)
        assert torch.equal(part[0], out[entries]) and torch.equal(part[1], lse[entries])
        assert torch.equal(part[3], dk[entries]) and torch.equal(part[4], dv[entries])
        assert dq_close(part[2], dq[entries])


def test_key_head_groups_are_independent(problem):
    """Permuting the key heads together with their query-head groups permutes the results."""
    q, k, v, dout, (out, lse, dq, dk, dv) = problem
    group = HEADS_Q // HEADS_KV
    order = torch.tensor([3, 0, 7, 1, 6, 2, 5, 4], device="cuda")
    q_order = (order[:, None] * group + torch.arange(group, device="cuda")[None, :]).flatten()
    part = run(q[:, :, q_order].contiguous(), k[:, :, order].contiguous(), v[:, :, order].contiguous(),
               dout[:, :, q_order].contiguous(), causal=True)
    assert torch.equal(part[0], out[:, :, q_order]) and torch.equal(part[1], lse[:, q_order])
    assert torch.equal(part[3], dk[:, :, order]) and torch.equal(part[4], dv[:, :, order])
    assert dq_close(part[2], dq[:, :, q_order])


def test_causal_rows_do_not_depend_on_later_tokens(problem):
    """Under a causal mask the first t rows of out and lse are functions of the first t tokens only."""
    q, k, v, dout, (out, lse, _, _, _) = problem
    t = 5000  # not a multiple of the tile sizes
    q2, k2, v2 = q.clone(), k.clone(), v.clone()
    torch.manual_seed(12)
    q2[:, t:], k2[:, t:], v2[:, t:] = randn(BATCH, SEQLEN - t, HEADS_Q, D), randn(BATCH, SEQLEN - t, HEADS_KV, D), randn(BATCH, SEQLEN - t, HEADS_KV, D)
    out2, lse2 = zigfa.flash_attn_func(q2, k2, v2, causal=True, return_attn_probs=True)
    assert torch.equal(out2[:, :t], out[:, :t]) and torch.equal(lse2[:, :, :t], lse[:, :, :t])
    assert not torch.equal(out2[:, t:], out[:, t:])
    # the same prefix computed as a shorter problem
    out3, lse3 = zigfa.flash_attn_func(q[:, :t], k[:, :t], v[:, :t], causal=True, return_attn_probs=True)
    assert torch.equal(out3, out[:, :t]) and torch.equal(lse3, lse[:, :, :t])


def test_scaling_values_and_gradients_by_two_is_exact(problem):
    """out is linear in V and the gradients are linear in dO; a factor of two commutes with every rounding."""
    q, k, v, dout, (out, lse, dq, dk, dv) = problem
    out2, lse2, dq2, dk2, dv2 = run(q, k, v * 2, dout * 2, causal=True)
    assert torch.equal(out2, out * 2) and torch.equal(lse2, lse)
    # dV = P^T dO doubles with dO; dS = P o (dP - D) has dP = dO V^T and D = sum(O dO), each four times as large
    assert torch.equal(dv2, dv * 2)
    assert torch.equal(dk2, dk * 4)
    assert dq_close(dq2, dq.float() * 4)


def test_window_wider_than_the_sequence_equals_causal(problem):
    q, k, v, dout, (out, lse, dq, dk, dv) = problem
    out2, lse2, dq2, dk2, dv2 = run(q[:1], k[:1], v[:1], dout[:1], window_size=(SEQLEN + 7, 0))
    assert torch.equal(out2, out[:1]) and torch.equal(lse2, lse[:1])
    assert torch.equal(dk2, dk[:1]) and torch.equal(dv2, dv[:1])
    assert dq_close(dq2, dq[:1])
