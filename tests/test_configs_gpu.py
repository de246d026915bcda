"""The five benchmark configurations at their full sizes on the GPU: the library's outputs and gradients for a subset
of (batch entry, key head group) slices against the float32 oracle evaluated in row chunks, the BF16 flash reference
for the tolerance, and whole-tensor sanity properties (no NaN, rows past the end untouched, checksum against the
BF16 reference). Inputs are seeded BF16 N(0,1) tensors of the configurations' shapes."""
import itertools

import pytest
import torch

import attention_oracle as oracle
import parity
import zigfa
from zigfa._impl import ops

pytestmark = pytest.mark.gpu


def randn(*shape, generator=None):
    return torch.randn(*shape, device="cuda", dtype=torch.bfloat16, generator=generator)


def chunked_reference(q, k, v, dout, window, scale, chunk=4096):
    """Float32 oracle for one sequence and one key head: q, dout (S, G, D), k, v (S, 1, D), same lengths.
    Rows are processed `chunk` at a time against only the keys their band can reach."""
    seqlen = q.shape[0]
    left, right = window
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    lse = torch.empty(q.shape[1], seqlen, dtype=torch.float32, device=q.device)
    dq = torch.empty_like(out)
    dk = torch.zeros(k.shape, dtype=torch.float32, device=q.device)
    dv = torch.zeros_like(dk)
    for r0 in range(0, seqlen, chunk):
        r1 = min(r0 + chunk, seqlen)
        c0 = 0 if left < 0 else max(0, r0 - left)
        c1 = seqlen if right < 0 else min(seqlen, r1 + right)
        rows = torch.arange(r0, r1, device=q.device)[:, None]
        cols = torch.arange(c0, c1, device=q.device)[None, :]
        mask = torch.ones(r1 - r0, c1 - c0, dtype=torch.bool, device=q.device)
        if right >= 0:
            mask &= cols <= rows + right
        if left >= 0:
            mask &= cols >= rows - left
        o, l, gq, gk, gv = oracle.gradients(oracle.masked_attention, q[r0:r1], k[c0:c1], v[c0:c1], dout[r0:r1], mask,
                                            softmax_scale=scale)
        out[r0:r1], lse[:, r0:r1], dq[r0:r1] = o, l, gq
        dk[c0:c1] += gk
        dv[c0:c1] += gv
    return out, lse, dq, dk, dv


def check_slice(name, ours, reference, flash):
    """Full-size configurations are held to the stated rule with nothing added; returns error / bound."""
    error, stated = parity.assert_close(name, ours, reference, flash, f"[{name}]", strict=True)
    return error / max(stated, 1e-30)


def test_config1_fixed_causal_gqa():
    batch, seqlen, heads_q, heads_kv, d = 4, 8192, 32, 8, 128
    torch.manual_seed(1)
    q, k, v = (randn(batch, seqlen, h, d).requires_grad_() for h in (heads_q, heads_kv, heads_kv))
    dout = randn(batch, seqlen, heads_q, d)
    out, lse = zigfa.flash_attn_func(q, k, v, causal=True, return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    for tensor in (out, lse, dq, dk, dv):
        assert torch.isfinite(tensor).all()
    flash = parity.aten_flash(q.detach(), k.detach(), v.detach(), dout, None, None, seqlen, seqlen, (-1, 0), d**-0.5)
    group = heads_q // heads_kv
    for b, kv_head in [(0, 0), (3, 5)]:
        heads = slice(kv_head * group, (kv_head + 1) * group)
        ref = chunked_reference(q.detach()[b, :, heads], k.detach()[b, :, kv_head : kv_head + 1],
                                v.detach()[b, :, kv_head : kv_head + 1], dout[b, :, heads], (-1, 0), d**-0.5)
        pick = lambda t, h: None if t is None else t[b, :, h]
        check_slice("out", out.detach()[b, :, heads], ref[0], pick(flash and flash[0], heads))
        parity.assert_lse(lse[b, heads], ref[1])
        check_slice("dq", dq[b, :, heads], ref[2], pick(flash and flash[1], heads))
        check_slice("dk", dk[b, :, kv_head : kv_head + 1], ref[3], pick(flash and flash[2], slice(kv_head, kv_head + 1)))
        check_slice("dv", dv[b, :, kv_head : kv_head + 1], ref[4], pick(flash and flash[3], slice(kv_head, kv_head + 1)))
    if flash:
        # whole tensors: the two BF16 implementations stay within a few BF16 ulps of each other everywhere
        for ours, theirs in zip((out.detach(), dq, dk, dv), flash):
            assert (ours.float() - theirs.float()).abs().max() <= 2**-6 * theirs.float().abs().max()


def config2_lengths():
    generator = torch.Generator().manual_seed(2)
    lengths, total = [], 0
    while total < 65536:
        length = int(torch.randint(256, 8193, (1,), generator=generator))
        length = min(length, 65536 - total)
        lengths.append(length)
        total += length
    return lengths


def test_config2_varlen_window():
    lengths = config2_lengths()
    heads_q, heads_kv, d, window = 64, 8, 128, (4096, 0)
    total, padding = sum(lengths), 256
    torch.manual_seed(2)
    q = randn(total + padding, heads_q, d).requires_grad_()
    k, v = (randn(total + padding, heads_kv, d).requires_grad_() for _ in range(2))
    dout = randn(total + padding, heads_q, d)
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device="cuda")
    out = torch.full_like(q, float("nan")).detach()
    lse = torch.full((heads_q, total + padding), float("nan"), device="cuda")
    ops.launch_forward(q.detach(), k.detach(), v.detach(), out, lse, cu, cu, d**-0.5, *window)
    assert torch.isnan(out[total:]).all() and torch.isfinite(out[:total]).all() and torch.isfinite(lse[:, :total]).all()
    api_out = zigfa.flash_attn_varlen_func(q, k, v, cu, cu, max(lengths), max(lengths), causal=True, window_size=(4096, -1))
    assert torch.equal(api_out[:total], out[:total])
    dq, dk, dv = torch.autograd.grad(api_out, (q, k, v), dout)
    for tensor in (dq[:total], dk[:total], dv[:total]):
        assert torch.isfinite(tensor).all()
    flash = parity.aten_flash(q.detach(), k.detach(), v.detach(), dout, cu, cu, max(lengths), max(lengths), window, d**-0.5)
    group = heads_q // heads_kv
    order = sorted(range(len(lengths)), key=lambda i: lengths[i])
    for sequence, kv_head in [(order[-1], 3), (order[0], 7), (len(lengths) - 1, 0)]:
        rows = slice(int(cu[sequence]), int(cu[sequence + 1]))
        heads = slice(kv_head * group, (kv_head + 1) * group)
        one = slice(kv_head, kv_head + 1)
        ref = chunked_reference(q.detach()[rows, heads], k.detach()[rows, one], v.detach()[rows, one], dout[rows, heads],
                                window, d**-0.5)
        pick = lambda t, h: None if t is None else t[rows, h]
        check_slice("out", out[rows, heads], ref[0], pick(flash and flash[0], heads))
        parity.assert_lse(lse[heads, rows], ref[1])
        check_slice("dq", dq[rows, heads], ref[2], pick(flash and flash[1], heads))
        check_slice("dk", dk[rows, one], ref[3], pick(flash and flash[2], one))
        check_slice("dv", dv[rows, one], ref[4], pick(flash and flash[3], one))


def shared_prefix_layout(groups, prefix, continuations, continuation_length):
    lengths, visible_rows = [], []
    per_group = 1 + continuations
    count = groups * per_group
    for g in range(groups):
        first = g * per_group
        lengths.append(prefix)
        visible_rows.append([first])
        for c in range(continuations):
            lengths.append(continuation_length)
            visible_rows.append([first, first + 1 + c])
    visible = torch.zeros(count, count, dtype=torch.bool)
    for i, keys in enumerate(visible_rows):
        visible[i, keys] = True
    return lengths, visible


@pytest.mark.parametrize("prefix", [2048, 1024])
def test_config3_inter_sequence_shared_prefix(prefix):
    # 8 groups x (prefix + 7 continuations of 512): 45056 tokens with the stated 2048-token prefix, 36864 with 1024
    lengths, visible = shared_prefix_layout(8, prefix, 7, 512)
    heads_q, heads_kv = 32, 8
    d = 256
    assert d in ops.head_dims(ops.BACKWARD)
    total = sum(lengths)
    torch.manual_seed(3)
    q = randn(total, heads_q, d).requires_grad_()
    k, v = (randn(total, heads_kv, d).requires_grad_() for _ in range(2))
    dout = randn(total, heads_q, d)
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device="cuda")
    bits = torch.from_numpy(oracle.visibility_bits_of(visible.numpy())).cuda()
    assert tuple(bits.shape) == (64, 2)
    out, lse = zigfa.flash_attn_inter_sequence_func(q, k, v, cu, cu, max(lengths), max(lengths), bits, causal=True,
                                                    return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    for tensor in (out, lse, dq, dk, dv):
        assert torch.isfinite(tensor).all()
    # one whole group (prefix + its continuations) and two key heads against the dense-mask oracle
    group_heads = heads_q // heads_kv
    windows = [(-1, 0)] * len(lengths)
    for g, kv_head in [(0, 0), (7, 5)]:
        first = g * 8
        rows = slice(int(cu[first]), int(cu[first + 8]))
        sub_lengths = lengths[first : first + 8]
        sub_cu = [0, *itertools.accumulate(sub_lengths)]
        mask = oracle.inter_sequence_mask(sub_cu, sub_cu, visible[first : first + 8, first : first + 8], windows[:8]).cuda()
        heads = slice(kv_head * group_heads, (kv_head + 1) * group_heads)
        one = slice(kv_head, kv_head + 1)
        ref = oracle.gradients(oracle.masked_attention, q.detach()[rows, heads], k.detach()[rows, one],
                               v.detach()[rows, one], dout[rows, heads], mask, softmax_scale=d**-0.5)
        # the BF16 pass of the reference's oracle for this mask (memory-efficient attention with a -inf bias)
        bf16 = parity.aten_masked(q.detach()[rows, heads], k.detach()[rows, one], v.detach()[rows, one],
                                  dout[rows, heads], mask, d**-0.5) or (None,) * 4
        check_slice("out", out.detach()[rows, heads], ref[0], bf16[0])
        parity.assert_lse(lse[heads, rows], ref[1])
        check_slice("dq", dq[rows, heads], ref[2], bf16[1])
        check_slice("dk", dk[rows, one], ref[3], bf16[2])
        check_slice("dv", dv[rows, one], ref[4], bf16[3])


def test_config3_head_dim_512_forward():
    # the forward-only head_dim of the shared-prefix configuration
    lengths, visible = shared_prefix_layout(8, 2048, 7, 512)
    heads_q, heads_kv, d = 32, 8, 512
    total = sum(lengths)
    torch.manual_seed(3)
    q, k, v = randn(total, heads_q, d), randn(total, heads_kv, d), randn(total, heads_kv, d)
    cu = torch.tensor([0, *itertools.accumulate(lengths)], dtype=torch.int32, device="cuda")
    bits = torch.from_numpy(oracle.visibility_bits_of(visible.numpy())).cuda()
    out, lse = zigfa.flash_attn_inter_sequence_func(q, k, v, cu, cu, max(lengths), max(lengths), bits, causal=True,
                                                    return_attn_probs=True)
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    group_heads = heads_q // heads_kv
    for g, kv_head in [(0, 0), (7, 5)]:
        first = g * 8
        rows = slice(int(cu[first]), int(cu[first + 8]))
        sub_cu = [0, *itertools.accumulate(lengths[first : first + 8])]
        mask = oracle.inter_sequence_mask(sub_cu, sub_cu, visible[first : first + 8, first : first + 8], [(-1, 0)] * 8).cuda()
        heads = slice(kv_head * group_heads, (kv_head + 1) * group_heads)
        one = slice(kv_head, kv_head + 1)
        ref_out, ref_lse = oracle.masked_attention(q[rows, heads], k[rows, one], v[rows, one], mask, d**-0.5)
        bf16 = parity.aten_masked(q[rows, heads], k[rows, one], v[rows, one], None, mask, d**-0.5) or (None,)
        check_slice("out", out[rows, heads], ref_out, bf16[0])
        parity.assert_lse(lse[heads, rows], ref_lse)


def test_config4_long_context_window_shard():
    # one shard of the 8-GPU split: 2 of the 16 batch entries
    batch, seqlen, heads_q, heads_kv, d, window = 2, 32768, 32, 4, 128, (4096, 0)
    torch.manual_seed(4)
    q, k, v = (randn(batch, seqlen, h, d).requires_grad_() for h in (heads_q, heads_kv, heads_kv))
    dout = randn(batch, seqlen, heads_q, d)
    out, lse = zigfa.flash_attn_func(q, k, v, causal=True, window_size=(4096, -1), return_attn_probs=True)
    dq, dk, dv = torch.autograd.grad(out, (q, k, v), dout)
    for tensor in (out, lse, dq, dk, dv):
        assert torch.isfinite(tensor).all()
    flash = parity.aten_flash(q.detach(), k.detach(), v.detach(), dout, None, None, seqlen, seqlen, window, d**-0.5)
    group = heads_q // heads_kv
    b, kv_head = 1, 2
    heads = slice(kv_head * group, (kv_head + 1) * group)
    one = slice(kv_head, kv_head + 1)
    ref = chunked_reference(q.detach()[b, :, heads], k.detach()[b, :, one], v.detach()[b, :, one], dout[b, :, heads],
                            window, d**-0.5, chunk=2048)
    pick = lambda t, h: None if t is None else t[b, :, h]
    check_slice("out", out.detach()[b, :, heads], ref[0], pick(flash and flash[0], heads))
    parity.assert_lse(lse[b, heads], ref[1])
    check_slice("dq", dq[b, :, heads], ref[2], pick(flash and flash[1], heads))
    check_slice("dk", dk[b, :, one], ref[3], pick(flash and flash[2], one))
    check_slice("dv", dv[b, :, one], ref[4], pick(flash and flash[3], one))


def test_config0_against_the_cpu_oracle():
    # the CPU-runnable configuration: batch 2, seqlen 512, heads 8/2, head_dim 128, causal, seed 0
    torch.manual_seed(0)
    q = torch.randn(2, 512, 8, 128, dtype=torch.bfloat16)
    k, v = (torch.randn(2, 512, 2, 128, dtype=torch.bfloat16) for _ in range(2))
    dout = torch.randn(2, 512, 8, 128, dtype=torch.bfloat16)
    reference = oracle.gradients(oracle.attention, q, k, v, dout, causal=True)
    qd, kd, vd = (x.cuda().requires_grad_() for x in (q, k, v))
    out, lse = zigfa.flash_attn_func(qd, kd, vd, causal=True, return_attn_probs=True)
    grads = torch.autograd.grad(out, (qd, kd, vd), dout.cuda())
    flash = parity.aten_flash(qd.detach(), kd.detach(), vd.detach(), dout.cuda(), None, None, 512, 512, (-1, 0), 128**-0.5)
    flash = flash or (None,) * 4
    parity.assert_close("out", out.detach().cpu(), reference[0], None if flash[0] is None else flash[0].cpu(), "[config 0]",
                        strict=True)
    parity.assert_lse(lse.cpu(), reference[1])
    for name, ours, ref, bf16 in zip(("dq", "dk", "dv"), grads, reference[2:], flash[1:]):
        parity.assert_close(name, ours.cpu(), ref, None if bf16 is None else bf16.cpu(), "[config 0]", strict=True)
