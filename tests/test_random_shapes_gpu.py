"""Seeded random problems through the public API against the oracle: odd sequence lengths, head counts, windows and
packed batches with empty sequences, at every head dimension, the combinations that the hand-picked cases of the other
test files do not enumerate. The reference tests its kernels the same way over a grid of sequence-length pairs
(reference tests/test_torch.py:57-120); here the grid is drawn from a fixed seed so that a failure reproduces.
Forward and backward up to head_dim 256, forward only at 512 (there is no backward at 512); with and without pivot
gradients."""
import random

import pytest
import torch

import attention_oracle as oracle
import parity
import zigfa

pytestmark = pytest.mark.gpu

SEQLENS = [1, 7, 64, 100, 128, 129, 255, 256, 300, 513, 700, 1024, 1500]


def draw(rng, head_dims):
    d = rng.choice(head_dims)
    heads_kv = rng.choice([1, 2, 3, 5] if d < 512 else [1, 2, 3])
    heads_q = heads_kv * rng.choice([1, 2, 3, 4, 6, 8] if d < 512 else [1, 2, 4])
    batch = rng.choice([1, 2, 3])
    seqlen_q = rng.choice(SEQLENS)
    seqlen_k = rng.choice([seqlen_q, seqlen_q, seqlen_q + rng.randint(0, 300), max(1, seqlen_q - rng.randint(0, 200)),
                           rng.randint(1, 1600)])
    kind = rng.choice(["dense", "causal", "causal", "window"])
    window = {"dense": (-1, -1), "causal": (-1, 0), "window": (rng.randint(0, 300), rng.randint(0, 100))}[kind]
    return d, heads_q, heads_kv, batch, seqlen_q, seqlen_k, kind, window


def tensors(rows_q, rows_k, heads_q, heads_kv, d, leading, scale_q):
    q = (scale_q * torch.randn(*leading, rows_q, heads_q, d, device="cuda")).bfloat16()
    k = torch.randn(*leading, rows_k, heads_kv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(*leading, rows_k, heads_kv, d, device="cuda", dtype=torch.bfloat16)
    dout = torch.randn(*leading, rows_q, heads_q, d, device="cuda", dtype=torch.bfloat16)
    return q, k, v, dout


def run_case(rng, head_dims, with_backward):
    d, heads_q, heads_kv, batch, seqlen_q, seqlen_k, kind, window = draw(rng, head_dims)
    scale_q = rng.choice([1.0, 1.0, 3.0])
    options = dict(causal=kind == "causal", window_size=window if kind == "window" else (-1, -1), return_attn_probs=True)
    name = f"B{batch} Sq{seqlen_q} Sk{seqlen_k} H{heads_q}/{heads_kv} D{d} {kind}{window} q x {scale_q}"
    if rng.random() < 0.5:
        q, k, v, dout = tensors(seqlen_q, seqlen_k, heads_q, heads_kv, d, (batch,), scale_q)
        if with_backward:
            q, k, v = (t.requires_grad_() for t in (q, k, v))
        out, lse = zigfa.flash_attn_func(q, k, v, **options)
        grads = torch.autograd.grad(out, (q, k, v), dout) if with_backward else None
        parity.check_fixed((out.detach(), lse, grads), q.detach(), k.detach(), v.detach(), dout if with_backward else None,
                           kind == "causal", window if kind != "causal" else (-1, -1), notes=name)
        return
    lengths_q = [rng.randint(0, seqlen_q) for _ in range(batch + 2)]
    lengths_k = [max(0, length + rng.randint(-50, 200)) for length in lengths_q]
    cu_q = torch.tensor([0, *torch.tensor(lengths_q).cumsum(0).tolist()], dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0, *torch.tensor(lengths_k).cumsum(0).tolist()], dtype=torch.int32, device="cuda")
    total_q, total_k = int(cu_q[-1]), int(cu_k[-1])
    if total_q == 0 or total_k == 0:
        return
    name += f" packed {lengths_q} / {lengths_k}"
    q, k, v, dout = tensors(total_q, total_k, heads_q, heads_kv, d, (), scale_q)
    if with_backward:
        q, k, v = (t.requires_grad_() for t in (q, k, v))
    out, lse = zigfa.flash_attn_varlen_func(q, k, v, cu_q, cu_k, max(lengths_q), max(lengths_k), **options)
    grads = torch.autograd.grad(out, (q, k, v), dout) if with_backward else None
    mask = oracle.packed_mask(cu_q.tolist(), cu_k.tolist(), window)
    parity.check_masked((out.detach(), lse, grads), q.detach(), k.detach(), v.detach(), dout if with_backward else None, mask,
                        notes=name)


@pytest.mark.parametrize("seed", range(6))
@pytest.mark.parametrize("pivot_gradients", [False, True])
def test_random_problems_forward_and_backward(seed, pivot_gradients):
    rng = random.Random(1000 * pivot_gradients + seed)
    torch.manual_seed(seed)
    before = zigfa.set_pivot_gradients(pivot_gradients)
    try:
        for _ in range(6):
            run_case(rng, [64, 72, 96, 128, 128, 256], with_backward=True)
    finally:
        zigfa.set_pivot_gradients(before)


@pytest.mark.parametrize("seed", range(4))
def test_random_problems_head_dim_512_forward(seed):
    rng = random.Random(5120 + seed)
    torch.manual_seed(seed)
    with torch.no_grad():
        for _ in range(8):
            run_case(rng, [512], with_backward=False)
