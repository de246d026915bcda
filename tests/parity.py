"""Parity harness of the GPU tests: runs the library through its public API and compares with the oracle.

Tolerance (stated by the task): for out, dq, dk, dv
    max|ours - ref_fp32| <= 2 * max|ref_bf16 - ref_fp32| + atol + rounding,
    atol = 2 * max|(ref + 0.3) - 0.3 - ref| + 1e-4,   rounding = 2^-9 * max|ref|
where ref_fp32 is the oracle in float32 and ref_bf16 is PyTorch's own BF16 flash attention (the aten kernels the
reference's oracle calls for its BF16 pass, reference tests/reference.py:50-88). `rounding` is half a BF16 ulp of the
largest value: both results are rounded to BF16 at the end, and a result whose unrounded value is as accurate as the
reference's can still land one rounding step further from FP32 than the reference did (measured here: the mean
errors of the two agree within 5 %, the maxima differ by exactly such flips). The 1e-4 covers gradients whose exact
value is 0 (float32 round-off of dP - D summed over a few hundred rows). When the aten kernel cannot express the case or is unavailable the bound falls back to the reference's
own rule 3 * 2^-7 * max|ref| + atol (reference tests/checks.py:11-13,37-50). LSE: |diff| <= 1e-2 * (1 + |lse|) and the
same -inf pattern (reference tests/checks.py:53-59).
"""
import torch

import attention_oracle as oracle

OUTPUT_FACTOR = 2.0
BF16_RULE = 3 * 2**-7
LSE_TOLERANCE = 1e-2


def largest(tensor):
    return tensor.abs().max().item() if tensor.numel() else 0.0


def absolute_slack(reference):
    return 2 * largest((reference + 0.3) - 0.3 - reference) + 1e-4


def flash_expresses(window, max_q, max_k):
    left, right = window
    return left < 0 or 0 <= right < max_k or max_q <= max_k + 1


def aten_flash(q, k, v, dout, cu_q, cu_k, max_q, max_k, window, scale):
    """(out, dq, dk, dv) of PyTorch's BF16 flash attention, or None when it cannot run this case."""
    if not flash_expresses(window, max_q, max_k) or max_q == 0 or max_k == 0:
        return None
    try:
        out, lse, seed, offset, _ = torch.ops.aten._flash_attention_forward(
            q, k, v, cu_q, cu_k, max_q, max_k, 0.0, False, False, scale=scale, window_size_left=window[0],
            window_size_right=window[1],
        )
        if dout is None:
            return out, None, None, None
        dq, dk, dv = torch.ops.aten._flash_attention_backward(
            dout.contiguous(), q, k, v, out, lse, cu_q, cu_k, max_q, max_k, 0.0, False, seed, offset, scale=scale,
            window_size_left=window[0], window_size_right=window[1],
        )
        return out, dq, dk, dv
    except Exception:  # kernel not built for this device / head_dim
        return None


def assert_close(name, ours, reference, bf16_reference, notes):
    reference = reference.float()
    slack = absolute_slack(reference)
    if bf16_reference is not None:
        allowed = OUTPUT_FACTOR * largest(bf16_reference.float() - reference) + slack + 2**-9 * largest(reference)
        rule = "2x bf16 reference error"
    else:
        allowed = BF16_RULE * largest(reference) + slack
        rule = "3*2^-7 * max|ref|"
    error = largest(ours.float() - reference)
    assert not torch.isnan(ours).any(), f"{name}: NaN in the result {notes}"
    assert error <= allowed, f"{name}: error {error:.3e} exceeds {allowed:.3e} ({rule}) {notes}"
    return error, allowed


def assert_lse(lse, lse_reference, notes=""):
    finite = torch.isfinite(lse_reference)
    assert torch.equal(lse == float("-inf"), lse_reference == float("-inf")), f"lse -inf pattern differs {notes}"
    if finite.any():
        excess = (lse - lse_reference).abs() - LSE_TOLERANCE * (1 + lse_reference.abs())
        assert excess[finite].max().item() <= 0, f"lse differs by {(lse - lse_reference)[finite].abs().max().item():.3e} {notes}"


def check_fixed(function_outputs, q, k, v, dout, causal, window_size, scale=None, notes=""):
    """function_outputs = (out, lse, (dq, dk, dv) or None) from the library for fixed-length inputs."""
    out, lse, grads = function_outputs
    window = (window_size[0], 0) if causal else tuple(window_size)
    d = q.shape[-1]
    scale = d**-0.5 if scale is None else scale
    if grads is not None:
        ref = oracle.gradients(oracle.attention, q, k, v, dout, window_size=window, softmax_scale=scale)
    else:
        ref = (*oracle.attention(q, k, v, window_size=window, softmax_scale=scale), None, None, None)
    flash = aten_flash(q, k, v, dout if grads is not None else None, None, None, q.shape[1], k.shape[1], window, scale)
    flash = flash or (None, None, None, None)
    assert_close("out", out, ref[0], flash[0], notes)
    assert_lse(lse, ref[1], notes)
    if grads is not None:
        for name, ours, reference, bf16 in zip(("dq", "dk", "dv"), grads, ref[2:], flash[1:]):
            assert_close(name, ours, reference, bf16, notes)


def check_masked(function_outputs, q, k, v, dout, mask, scale=None, flash=None, notes=""):
    """Packed inputs with an explicit (total_q, total_k) visibility mask."""
    out, lse, grads = function_outputs
    d = q.shape[-1]
    scale = d**-0.5 if scale is None else scale
    rows, cols = mask.shape
    if grads is not None:
        ref = oracle.gradients(oracle.masked_attention, q[:rows], k[:cols], v[:cols], dout[:rows], mask, softmax_scale=scale)
    else:
        ref = (*oracle.masked_attention(q[:rows], k[:cols], v[:cols], mask, scale), None, None, None)
    flash = flash or (None, None, None, None)
    assert_close("out", out[:rows], ref[0], None if flash[0] is None else flash[0][:rows], notes)
    assert_lse(lse[:, :rows], ref[1], notes)
    if grads is not None:
        limits = (rows, cols, cols)
        for name, ours, reference, bf16, limit in zip(("dq", "dk", "dv"), grads, ref[2:], flash[1:], limits):
            assert_close(name, ours[:limit], reference, None if bf16 is None else bf16[:limit], notes)
