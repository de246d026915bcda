"""Accuracy of peaked rows: the log-sum-exp of rows whose largest score is exactly zero, and the gradients of rows in
which one key holds more than 3/4 of the probability (the pivot), against the float64 oracle with the top key taken
apart (oracle.stable_attention). The families, constants and bounds are those of the reference's suite
(tests/test_softmax_fix.py): zero-maximum rows at margins of 17 to 80 nats (:353-402), peaked rows (:577-590), dq under
a common key shift (:621-637), the threshold of exactly 3/4 (:999-1017), rows without keys (:721-780); the bounds are
its `queue_lse_checks`, `queue_output_checks` and `queue_gradient_checks` (:231-288)."""
import math

import pytest
import torch

import attention_oracle as oracle
import zigfa

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _pivot_gradients():
    """The backward half of these guarantees is a setting of the library (the forward half is always on)."""
    before = zigfa.set_pivot_gradients(True)
    yield
    zigfa.set_pivot_gradients(before)


# Constants of the reference's suite (tests/test_softmax_fix.py:27-66).
EXP2_ERROR = 2.0**-13
PUSH = 8.0
QUERY_SPREAD = 0.25
ZERO_MAXIMUM_MARGINS = (17.0, 80.0)
PEAK_MARGINS = (2.0, 60.0)
PEAKED_FRACTION = 0.75
FLUSH_MARGIN = 84.0
RECOVERABLE_MARGIN = 76.0
FLUSH_LIMIT = 2.0**-126
FLUSHED_TERM = 256 * FLUSH_LIMIT
LSE_UNIT = 2.0**-21
GRADIENT_UNIT = 2.0**-6
KEY_SHIFT = 96.0
OTHER_SCALE = 0.2
GQA_HEADS = (4, 2)
WINDOWS = {"dense": (-1, -1), "causal": (-1, 0), "local": (64, 32)}
HEAD_DIMS = (64, 128, 256)


class Problem:
    """A packed problem: q, dout (Tq, Hq, D), k, v (Tk, Hkv, D) in BF16, its mask and the call that runs it."""

    def __init__(self, q, k, v, dout, mask, attend, softmax_scale=None):
        self.q, self.k, self.v, self.dout = (x.bfloat16() for x in (q, k, v, dout))
        self.mask, self.attend, self.softmax_scale = mask, attend, softmax_scale

    def run(self, gradients=True):
        leaves = [x.detach().clone().requires_grad_(bool(gradients)) for x in (self.q, self.k, self.v)]
        out, lse = self.attend(*leaves)
        if not gradients:
            return out.detach(), lse, None, None, None
        return (out.detach(), lse, *torch.autograd.grad(out, leaves, self.dout))

    def reference(self):
        return oracle.stable_attention(self.q, self.k, self.v, self.dout, self.mask, self.softmax_scale)


def random_tensors(rows_q, rows_k, heads, heads_kv, head_dim, query_scale=1.0):
    q = query_scale * torch.randn(rows_q, heads, head_dim, device="cuda", dtype=torch.float64)
    k, v = (torch.randn(rows_k, heads_kv, head_dim, device="cuda", dtype=torch.float64) for _ in range(2))
    dout = torch.randn(rows_q, heads, head_dim, device="cuda", dtype=torch.float64)
    return q, k, v, dout


def with_zero_maximum(q, k, mask, zero_keys, scale):
    """Every key gets the last coordinate PUSH and every query a last coordinate that puts its scores a random margin
    of 17 to 80 nats (less log of the visible keys) below zero; the keys of `zero_keys` are all zero, so they score
    exactly 0 with every query (reference tests/test_softmax_fix.py:95-103)."""
    visible = mask.sum(-1, keepdim=True).clamp(min=1).double().log()
    low, high = ZERO_MAXIMUM_MARGINS[0], ZERO_MAXIMUM_MARGINS[1] - visible
    targets = low + (high - low) * torch.rand(q.shape[:2], device=q.device, dtype=torch.float64)
    q, k = QUERY_SPREAD * q, k.clone()
    q[..., -1] = -(targets + visible) / (PUSH * scale)
    k[..., -1] = PUSH
    k[zero_keys] = 0.0
    return q, k


def with_peaks(q, k, mask, pivots, scale):
    """Moves 3/4 of the queries along their chosen key until that key leads the log-sum-exp of the others by a random
    margin of 2 to 60 nats, by bisection on the step (reference tests/test_softmax_fix.py:115-137)."""
    low, high = PEAK_MARGINS
    targets = low + (high - low) * torch.rand(pivots.shape, device=q.device, dtype=torch.float64)
    peaked = (torch.rand(pivots.shape, device=q.device) < PEAKED_FRACTION) & mask.gather(1, pivots)
    groups = q.shape[1] // k.shape[1]
    keys = k.repeat_interleave(groups, dim=1)
    direction = keys.gather(0, pivots[..., None].expand(-1, -1, keys.shape[-1]))
    direction = direction / direction.norm(dim=-1, keepdim=True).clamp(min=1e-30)
    base = scale * torch.einsum("qhd,khd->qhk", q, keys)
    slope = scale * torch.einsum("qhd,khd->qhk", direction, keys)
    others = mask[:, None, :] & (torch.arange(keys.shape[0], device=q.device) != pivots[..., None])
    step_low, step_high = torch.zeros_like(targets), torch.full_like(targets, 4096.0)
    for _ in range(64):
        middle = (step_low + step_high) / 2
        z = base + middle[..., None] * slope
        margin = z.gather(-1, pivots[..., None])[..., 0] - z.masked_fill(~others, float("-inf")).logsumexp(-1)
        below = margin < targets
        step_low, step_high = torch.where(below, middle, step_low), torch.where(below, step_high, middle)
    return q + torch.where(peaked, step_high, 0.0)[..., None] * direction


def first_visible_keys(mask, heads):
    return mask.int().argmax(-1, keepdim=True).expand(-1, heads)


def random_visible_keys(mask, heads):
    weights = (mask | ~mask.any(-1, keepdim=True)).double()
    return torch.multinomial(weights, heads, replacement=True)


def fixed_attention(batch, window, softmax_scale=None):
    def attend(q, k, v):
        out, lse = zigfa.flash_attn_func(*(x.unflatten(0, (batch, -1)) for x in (q, k, v)), softmax_scale=softmax_scale,
                                         causal=window[1] == 0, window_size=window, return_attn_probs=True)
        return out.flatten(0, 1), lse.transpose(0, 1).flatten(1)

    return attend


def fixed_mask(batch, seqlen_q, seqlen_k, window):
    cu_q = [i * seqlen_q for i in range(batch + 1)]
    cu_k = [i * seqlen_k for i in range(batch + 1)]
    return oracle.packed_mask(cu_q, cu_k, window).cuda()


def packed_attention(cu_q, cu_k, window, softmax_scale=None):
    lengths_q, lengths_k = cu_q[1:] - cu_q[:-1], cu_k[1:] - cu_k[:-1]
    arguments = (cu_q.int().cuda(), cu_k.int().cuda(), max(int(lengths_q.max()), 1), max(int(lengths_k.max()), 1))

    def attend(q, k, v):
        return zigfa.flash_attn_varlen_func(q, k, v, *arguments, softmax_scale=softmax_scale, causal=window[1] == 0,
                                            window_size=window, return_attn_probs=True)

    return attend


# ------------------------------------------------------------------------------------------------ bounds
def worst(name, ratio, selected, required=False):
    if required:
        assert selected.any(), f"{name}: the inputs do not exercise this check"
    value = float(torch.where(selected, ratio, 0.0).amax()) if selected.numel() else 0.0
    assert value <= 1.0, f"{name}: worst error / allowed error = {value:.3f}"
    return value


def check_lse(lse, ref, zero_maximum):
    error = (lse.double() - ref["lse"]).abs()
    finite = torch.isfinite(ref["lse"])
    margin = ref["margin"].nan_to_num(nan=-1.0)
    rows = (ref["top"] == 0) & (margin >= ZERO_MAXIMUM_MARGINS[0]) & (margin <= FLUSH_MARGIN - ref["visible"].log())
    allowed = ref["lse"] * (LSE_UNIT * (8 + ref["spread"]) + EXP2_ERROR)
    worst("lse of rows with a zero maximum", error / allowed, rows, zero_maximum)
    general = 2 * LSE_UNIT * (1 + ref["top"].abs() + ref["lse"].abs()) + EXP2_ERROR
    worst("lse", error / general, finite)
    assert ((lse == float("-inf")) == ~finite).all(), "lse is -inf exactly on the rows without keys"


def check_out(out, dq, ref):
    empty = ~torch.isfinite(ref["lse"]).T
    ratio = (out.double() - ref["out"]).norm(dim=-1) / (GRADIENT_UNIT * ref["out_scale"] + FLUSHED_TERM * ref["visible"].T)
    worst("out", ratio, ~empty)
    assert (out[empty] == 0).all(), "out is zero on the rows without keys"
    if dq is not None:
        assert (dq[empty] == 0).all(), "dq is zero on the rows without keys"


def flush_allowances(problem):
    """Largest change that flushing to zero below 2^-126 can make to a row of dq and of dk (reference
    tests/test_softmax_fix.py:259-271)."""
    q, k, v, dout = (x.double() for x in (problem.q, problem.k, problem.v, problem.dout))
    groups = q.shape[1] // k.shape[1]
    scale = q.shape[-1] ** -0.5 if problem.softmax_scale is None else problem.softmax_scale
    largest_v = v.norm(dim=-1).amax(0).repeat_interleave(groups)
    ds_limit = FLUSH_LIMIT * scale * (2 * dout.norm(dim=-1) * largest_v).clamp(min=1)
    mask = problem.mask.to(q.device, torch.float64)
    dq_allowance = ds_limit * (mask @ k.norm(dim=-1).repeat_interleave(groups, dim=1))
    dk_allowance = (mask.T @ (ds_limit * q.norm(dim=-1))).unflatten(1, (-1, groups)).sum(2)
    return dq_allowance, dk_allowance


def bf16_spacing(x):
    _, exponent = torch.frexp(x)
    return torch.where(x == 0, 0.0, torch.ldexp(torch.ones_like(x), exponent - 8))


def check_gradients(problem, dq, dk, dv, ref, pivots_required):
    margin = ref["margin"].nan_to_num(nan=math.inf)
    rows = (torch.isfinite(ref["lse"]) & (margin <= RECOVERABLE_MARGIN - ref["visible"].log())).T
    pivot = ref["pivot"].T
    dq_flushed, dk_flushed = flush_allowances(problem)
    seers = problem.mask.sum(0)
    dq_ratio = (dq.double() - ref["dq"]).norm(dim=-1) / (GRADIENT_UNIT * ref["dq_scale"] + dq_flushed)
    report = {"dq_pivot": worst("dq of rows with a pivot", dq_ratio, rows & pivot, pivots_required),
              "dq_other": worst("dq of rows without a pivot", dq_ratio, rows & ~pivot)}
    corrected = ref["corrected_keys"]
    half_units = torch.where(corrected, 0.5 * bf16_spacing(ref["dk"]).norm(dim=-1), 0.0)
    dk_ratio = (dk.double() - ref["dk"]).norm(dim=-1) / (GRADIENT_UNIT * ref["dk_scale"] + half_units + dk_flushed)
    seen = ref["dk_scale"] > 0
    report["dk_pivot"] = worst("dk of pivot keys", dk_ratio, seen & corrected, pivots_required)
    report["dk_other"] = worst("dk of other keys", dk_ratio, seen & ~corrected)
    flushed = FLUSHED_TERM * seers[:, None] * (dq.shape[1] // dk.shape[1])
    dv_ratio = (dv.double() - ref["dv"]).norm(dim=-1) / (GRADIENT_UNIT * ref["dv_scale"] + flushed)
    report["dv"] = worst("dv", dv_ratio, ref["dv_scale"] > 0)
    unseen = seers == 0
    assert (dk[unseen] == 0).all() and (dv[unseen] == 0).all(), "dk and dv are zero for the keys that no row sees"
    return report


def check(problem, gradients=True, zero_maximum=False, pivots_required=False):
    ref = problem.reference()
    out, lse, dq, dk, dv = problem.run(gradients)
    check_lse(lse, ref, zero_maximum)
    check_out(out, dq, ref)
    if gradients == "unchecked":  # rows without keys: only the zeros are required
        unseen = problem.mask.sum(0) == 0
        assert (dk[unseen] == 0).all() and (dv[unseen] == 0).all(), "dk and dv are zero for the keys that no row sees"
    elif gradients:
        check_gradients(problem, dq, dk, dv, ref, pivots_required)
    return ref, (out, lse, dq, dk, dv)


# ------------------------------------------------------------------------------------------------ families
def zero_keys_of_batch(batch, seqlen_q, seqlen_k, heads_kv, window):
    """Keys that score exactly zero: one per sequence (the first, or a late one), or one per window period; one
    sequence and head gets two neighbours, a tie (reference tests/test_softmax_fix.py:327-339)."""
    late = max(64, (seqlen_k - seqlen_q) // 64 * 64) if window[1] == 0 else seqlen_k // 2
    if window[0] >= 0:
        period = window[0] + max(window[1], 0) + 1
        positions = [list(range(0, seqlen_k, period))] * batch
    else:
        positions = [[0] if sequence % 2 == 0 else [min(late, seqlen_k - 1)] for sequence in range(batch)]
    zero_keys = torch.zeros(batch * seqlen_k, heads_kv, dtype=torch.bool)
    for sequence, keys in enumerate(positions):
        for key in keys:
            zero_keys[sequence * seqlen_k + key] = True
    zero_keys[(batch - 1) * seqlen_k + positions[-1][0] + 1, 0] = True
    return zero_keys.cuda()


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
@pytest.mark.parametrize("window_name", WINDOWS)
@pytest.mark.parametrize("seqlen_q, seqlen_k", [(200, 600), (300, 520)])
def test_zero_maximum_rows_keep_their_lse(head_dim, window_name, seqlen_q, seqlen_k):
    window, batch, (heads, heads_kv) = WINDOWS[window_name], 2, GQA_HEADS
    torch.manual_seed(head_dim + seqlen_q)
    mask = fixed_mask(batch, seqlen_q, seqlen_k, window)
    zero_keys = zero_keys_of_batch(batch, seqlen_q, seqlen_k, heads_kv, window)
    q, k, v, dout = random_tensors(batch * seqlen_q, batch * seqlen_k, heads, heads_kv, head_dim)
    q, k = with_zero_maximum(q, k, mask, zero_keys, head_dim**-0.5)
    check(Problem(q, k, v, dout, mask, fixed_attention(batch, window)), zero_maximum=True, pivots_required=True)


SPLIT_KV_SHAPES = {
    "gqa_decode": ((1, 1, 4096, 8, 2), (-1, 0)),
    "mha_decode": ((2, 1, 2048, 4, 4), (-1, -1)),
    "windowed_extend": ((1, 16, 2048, 8, 2), (512, 0)),
    "uneven_lengths": ((1, 100, 3001, 4, 1), (-1, 0)),
}


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
@pytest.mark.parametrize("shape_name", SPLIT_KV_SHAPES)
def test_zero_maximum_rows_keep_their_lse_across_key_splits(head_dim, shape_name):
    (batch, seqlen_q, seqlen_k, heads, heads_kv), window = SPLIT_KV_SHAPES[shape_name]
    torch.manual_seed(head_dim + seqlen_k)
    mask = fixed_mask(batch, seqlen_q, seqlen_k, window)
    zero_keys = torch.zeros(batch * seqlen_k, heads_kv, dtype=torch.bool, device="cuda")
    reach = window[0] // 2 if window[0] >= 0 else seqlen_k // 3
    zero_keys[seqlen_k - seqlen_q - reach :: seqlen_k] = True
    q, k, v, dout = random_tensors(batch * seqlen_q, batch * seqlen_k, heads, heads_kv, head_dim)
    q, k = with_zero_maximum(q, k, mask, zero_keys, head_dim**-0.5)
    check(Problem(q, k, v, dout, mask, fixed_attention(batch, window)), zero_maximum=True, pivots_required=True)


VARLEN_CASES = {"short": ((1, 160), None), "long_scaled": ((1, 700), OTHER_SCALE)}


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
@pytest.mark.parametrize("window_name", ["dense", "causal"])
@pytest.mark.parametrize("case_name", VARLEN_CASES)
def test_zero_maximum_and_peaked_varlen_rows(head_dim, window_name, case_name):
    window, (lengths, softmax_scale) = WINDOWS[window_name], VARLEN_CASES[case_name]
    generator = torch.Generator().manual_seed(head_dim + lengths[1])
    lengths_q = torch.randint(*lengths, (6,), generator=generator)
    lengths_k = lengths_q + torch.randint(0, 64, (6,), generator=generator)
    cu_q = torch.cat([torch.zeros(1, dtype=torch.long), lengths_q.cumsum(0)])
    cu_k = torch.cat([torch.zeros(1, dtype=torch.long), lengths_k.cumsum(0)])
    mask = oracle.packed_mask(cu_q, cu_k, window).cuda()
    attend = packed_attention(cu_q, cu_k, window, softmax_scale)
    heads, heads_kv = GQA_HEADS
    rows_q, rows_k = int(cu_q[-1]), int(cu_k[-1])
    scale = head_dim**-0.5 if softmax_scale is None else softmax_scale
    torch.manual_seed(head_dim)
    zero_keys = torch.zeros(rows_k, heads_kv, dtype=torch.bool, device="cuda")
    zero_keys[cu_k[:-1].cuda()] = True
    q, k, v, dout = random_tensors(rows_q, rows_k, heads, heads_kv, head_dim)
    zq, zk = with_zero_maximum(q, k, mask, zero_keys, scale)
    check(Problem(zq, zk, v, dout, mask, attend, softmax_scale), zero_maximum=True, pivots_required=True)
    for choice in (first_visible_keys, random_visible_keys):  # attention sinks, then peaks on random keys
        peaked_q = with_peaks(q, k, mask, choice(mask, heads), scale)
        check(Problem(peaked_q, k, v, dout, mask, attend, softmax_scale), pivots_required=True)


PEAKED_CASES = {"short": ((3, 128, 128), None), "scaled": ((2, 256, 320), OTHER_SCALE)}


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
@pytest.mark.parametrize("window_name", ["dense", "causal"])
@pytest.mark.parametrize("case_name", PEAKED_CASES)
def test_peaked_rows_keep_accurate_gradients(head_dim, window_name, case_name):
    ((batch, seqlen_q, seqlen_k), softmax_scale), (heads, heads_kv) = PEAKED_CASES[case_name], GQA_HEADS
    window = WINDOWS[window_name]
    scale = head_dim**-0.5 if softmax_scale is None else softmax_scale
    mask = fixed_mask(batch, seqlen_q, seqlen_k, window)
    attend = fixed_attention(batch, window, softmax_scale)
    for name, choice in (("sink", first_visible_keys), ("peaked", random_visible_keys)):
        torch.manual_seed(head_dim + seqlen_q + len(name))
        q, k, v, dout = random_tensors(batch * seqlen_q, batch * seqlen_k, heads, heads_kv, head_dim)
        q = with_peaks(q, k, mask, choice(mask, heads), scale)
        check(Problem(q, k, v, dout, mask, attend, softmax_scale), pivots_required=True)


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
def test_peaked_rows_of_a_shape_whose_row_vectors_are_not_a_multiple_of_four(head_dim):
    """3 x 1999 log-sum-exp elements: the per-row vectors of the backward workspace must stay aligned (reference
    tests/test_softmax_fix.py:607-618)."""
    seqlen, heads, window = 1999, 3, WINDOWS["causal"]
    torch.manual_seed(head_dim)
    mask = fixed_mask(1, seqlen, seqlen, window)
    q, k, v, dout = random_tensors(seqlen, seqlen, heads, heads, head_dim)
    q = with_peaks(q, k, mask, first_visible_keys(mask, heads), head_dim**-0.5)
    check(Problem(q, k, v, dout, mask, fixed_attention(1, window)), pivots_required=True)


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
def test_query_gradient_ignores_a_common_key_shift(head_dim):
    """dq = scale sum_j dS_j k_j, and the dS of a row add up to zero when the pivot takes minus the sum of the others, so
    adding 96 to every coordinate of every key (exact in BF16 for keys on a grid of 1/2) moves the dq of pivot rows by
    at most 2^-7 (|dq| + dq_scale / 8) (reference tests/test_softmax_fix.py:621-637)."""
    batch, seqlen_q, seqlen_k, (heads, heads_kv), window = 2, 192, 256, GQA_HEADS, WINDOWS["causal"]
    torch.manual_seed(head_dim)
    mask = fixed_mask(batch, seqlen_q, seqlen_k, window)
    q, _, v, dout = random_tensors(batch * seqlen_q, batch * seqlen_k, heads, heads_kv, head_dim)
    k = (2 * torch.randn(batch * seqlen_k, heads_kv, head_dim, device="cuda", dtype=torch.float64)).round().clamp(-8, 8) / 2
    q = with_peaks(q, k, mask, first_visible_keys(mask, heads), head_dim**-0.5)
    attend = fixed_attention(batch, window)
    problem = Problem(q, k, v, dout, mask, attend)
    ref, (_, _, dq, _, _) = check(problem, pivots_required=True)
    shifted = Problem(problem.q, problem.k + KEY_SHIFT, problem.v, problem.dout, mask, attend)
    assert (shifted.k.double() == problem.k.double() + KEY_SHIFT).all(), "the shifted keys are exact in bfloat16"
    _, _, shifted_dq, _, _ = shifted.run()
    flushed = flush_allowances(problem)[0] + flush_allowances(shifted)[0]
    allowed = 2.0**-7 * (ref["dq"].norm(dim=-1) + ref["dq_scale"] / 8) + flushed
    ratio = (shifted_dq.double() - dq.double()).norm(dim=-1) / allowed
    margin = ref["margin"].nan_to_num(nan=math.inf)
    rows = (torch.isfinite(ref["lse"]) & (margin <= RECOVERABLE_MARGIN - ref["visible"].log())).T
    worst("dq change under a common key shift, rows with a pivot", ratio, rows & ref["pivot"].T, True)


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
@pytest.mark.parametrize("seqlen_k", [3, 131])
def test_pivot_threshold_is_three_quarters(head_dim, seqlen_k):
    """Rows whose top key holds 0.56-0.74 of the probability next to a cancelling pair of values keep P (dP - D) for the
    top key; rows at 0.76-0.8 take it from the others. Both stay inside the gradient bounds (reference
    tests/test_softmax_fix.py:979-1017)."""
    batch, seqlen_q, (heads, heads_kv) = 2, 64, GQA_HEADS
    scale = head_dim**-0.5
    torch.manual_seed(head_dim + seqlen_k)
    top, pair = seqlen_k - 1, (0, seqlen_k - 2)
    q = torch.randn(batch, seqlen_q, heads, head_dim, device="cuda", dtype=torch.float64)
    k = torch.zeros(batch, seqlen_k, heads_kv, head_dim, device="cuda", dtype=torch.float64)
    v = torch.zeros_like(k)
    dout = torch.randn_like(q)
    for sequence, (low, high) in enumerate([(0.56, 0.74), (0.76, 0.8)]):
        probability = low + (high - low) * torch.rand(seqlen_q, heads, device="cuda", dtype=torch.float64)
        q[sequence, ..., 0] = (2 * probability / (1 - probability)).log() / scale
    q[..., 3], dout[..., 1:3] = 1.0, 1.0
    k[:, top, :, 0], k[:, :, :, 3] = 1.0, -1000.0 / scale
    k[:, [top, *pair], :, 3] = 0.0
    v[:, top, :, 1], v[:, pair[0], :, 2], v[:, pair[1], :, 2] = 1.0, 2.0**12, -(2.0**12)
    mask = fixed_mask(batch, seqlen_q, seqlen_k, WINDOWS["dense"])
    problem = Problem(*(x.flatten(0, 1) for x in (q, k, v, dout)), mask, fixed_attention(batch, WINDOWS["dense"]))
    ref, _ = check(problem, pivots_required=True)
    pivot = ref["pivot"].unflatten(1, (batch, seqlen_q))
    assert not pivot[:, 0].any() and pivot[:, 1].all()


def test_rows_without_keys_keep_an_lse_of_minus_infinity_and_zero_gradients():
    head_dim, (heads, heads_kv) = HEAD_DIMS[0], GQA_HEADS
    torch.manual_seed(5)
    batch, seqlen_q, seqlen_k, window = 2, 300, 160, WINDOWS["causal"]  # the first 140 rows of a sequence see no key
    mask = fixed_mask(batch, seqlen_q, seqlen_k, window)
    q, k, v, dout = random_tensors(batch * seqlen_q, batch * seqlen_k, heads, heads_kv, head_dim)
    q = with_peaks(q, k, mask, first_visible_keys(mask, heads), head_dim**-0.5)
    ref, _ = check(Problem(q, k, v, dout, mask, fixed_attention(batch, window)), gradients="unchecked")
    assert (~torch.isfinite(ref["lse"])).any()
    lengths_q, lengths_k = torch.tensor([40, 7, 0, 90, 33]), torch.tensor([50, 0, 12, 0, 70])  # empty key sequences
    cu_q = torch.cat([torch.zeros(1, dtype=torch.long), lengths_q.cumsum(0)])
    cu_k = torch.cat([torch.zeros(1, dtype=torch.long), lengths_k.cumsum(0)])
    mask = oracle.packed_mask(cu_q, cu_k, WINDOWS["dense"]).cuda()
    q, k, v, dout = random_tensors(int(cu_q[-1]), int(cu_k[-1]), heads, heads_kv, head_dim)
    q = with_peaks(q, k, mask, first_visible_keys(mask, heads), head_dim**-0.5)
    check(Problem(q, k, v, dout, mask, packed_attention(cu_q, cu_k, WINDOWS["dense"])), gradients="unchecked")


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
@pytest.mark.parametrize("query_scale", [1.0, 3.0])
def test_random_rows_keep_their_accuracy(head_dim, query_scale):
    """Ordinary rows (few pivots) inside the same bounds, and every gradient within 2.5 x the BF16 rounding of the exact
    one in norm (reference tests/test_softmax_fix.py:290-297,709-718)."""
    batch, seqlen_q, seqlen_k, (heads, heads_kv), window = 2, 256, 384, GQA_HEADS, WINDOWS["causal"]
    torch.manual_seed(head_dim + int(query_scale))
    mask = fixed_mask(batch, seqlen_q, seqlen_k, window)
    tensors = random_tensors(batch * seqlen_q, batch * seqlen_k, heads, heads_kv, head_dim, query_scale)
    ref, (_, _, dq, dk, dv) = check(Problem(*tensors, mask, fixed_attention(batch, window)))
    for name, gradient in (("dq", dq), ("dk", dk), ("dv", dv)):
        exact = ref[name]
        allowed = 2.5 * (exact.bfloat16().double() - exact).norm()
        if name == "dk":
            allowed = allowed + 0.5 * bf16_spacing(exact)[ref["corrected_keys"]].norm()
        assert float((gradient.double() - exact).norm()) <= float(allowed), name


# ------------------------------------------------------------------------------------------------ inter-sequence batches
def inter_sequence_problem(layout, heads, heads_kv, head_dim):
    cu_q, cu_k, bits, window_sizes = layout.tensors()
    arguments = (cu_q, cu_k, max(layout.lengths_q), max(layout.lengths_k), bits)

    def attend(q, k, v):
        return zigfa.flash_attn_inter_sequence_func(q, k, v, *arguments, window_sizes=window_sizes, return_attn_probs=True)

    mask = oracle.inter_sequence_mask(cu_q.tolist(), cu_k.tolist(), layout.visible, layout.windows).cuda()
    tensors = random_tensors(sum(layout.lengths_q), sum(layout.lengths_k), heads, heads_kv, head_dim)
    return tensors, mask, attend, cu_k.long()


@pytest.mark.parametrize("head_dim", (64, 128, 256, 512))
@pytest.mark.parametrize("layout_name", ["image_then_text", "shared_prefix", "interleaved"])
def test_zero_maximum_and_peaked_inter_sequence_rows(head_dim, layout_name):
    """Visibility-bit batches (reference tests/test_softmax_fix.py:552-572): the first key of every sequence scores zero;
    then attention sinks and random peaks. head_dim 512 has a forward kernel only."""
    from test_inter_sequence_gpu import build_layout

    layout = build_layout(layout_name, 4)
    (heads, heads_kv), gradients = GQA_HEADS, head_dim <= 256
    torch.manual_seed(head_dim)
    (q, k, v, dout), mask, attend, cu_k = inter_sequence_problem(layout, heads, heads_kv, head_dim)
    zero_keys = torch.zeros(k.shape[:2], dtype=torch.bool, device="cuda")
    zero_keys[cu_k[:-1][torch.tensor(layout.lengths_k, device="cuda") > 0]] = True
    zq, zk = with_zero_maximum(q, k, mask, zero_keys, head_dim**-0.5)
    check(Problem(zq, zk, v, dout, mask, attend), gradients, zero_maximum=True, pivots_required=gradients)
    if gradients:
        for choice in (first_visible_keys, random_visible_keys):
            peaked_q = with_peaks(q, k, mask, choice(mask, heads), head_dim**-0.5)
            check(Problem(peaked_q, k, v, dout, mask, attend), pivots_required=True)


# ------------------------------------------------------------------------------------------------ ties at a large shift
# Scores on a grid of 1/8 at a common shift of 2^16 or 2^17, built exactly in BF16 from one-hot queries (reference
# tests/test_softmax_fix.py:742-781,798-815): the FP32 product of such a score and log2(e) rounds by up to 2^-8 or 2^-7, and
# the log-sum-exp must carry that remainder instead of counting a tied key as an exact 1.
TIE_SHIFTS = (2.0**16, 2.0**17)
TIE_SCORES = torch.arange(-64, -7, dtype=torch.float64) / 8
FAR_SCORE = 1000.0
LOG2_SUM_SLACK = 2.0**-17
FAR_ROUNDING = 0.375


def float32(x):
    return float(torch.tensor(x, dtype=torch.float32))


def fp32_spacing(x):
    _, exponent = torch.frexp(x)
    return torch.ldexp(torch.ones_like(x), exponent - 24)


def lse_of_scores(scores, shift, head_dim):
    """Runs a dense forward whose scores are exactly `shift + scores` (heads, rows, keys) with softmax_scale 1."""
    heads, rows, keys = scores.shape
    q = torch.zeros(rows, heads, head_dim, dtype=torch.float64)
    q[torch.arange(rows), :, torch.arange(rows)] = 1.0
    q[..., -1] = 1.0
    k = torch.zeros(keys, heads, head_dim, dtype=torch.float64)
    k[..., :rows] = scores.permute(2, 0, 1)
    k[..., -1] = shift
    v = torch.randn(keys, heads, head_dim, generator=torch.Generator().manual_seed(head_dim), dtype=torch.float64)
    attend = fixed_attention(1, WINDOWS["dense"], 1.0)
    return attend(*(x.cuda().bfloat16() for x in (q, k, v)))[1].double()


def base2_log_sum_exp(scores, shift):
    x = (shift + scores.cuda()) * float32(math.log2(math.e))
    top = x.amax(-1, keepdim=True)
    return (top + (x - top).exp2().sum(-1, keepdim=True).log2())[..., 0]


def check_log2_sum(name, lse, log2_sum, exp2_error=0.0):
    ln2 = float32(math.log(2))
    allowed = ln2 * (fp32_spacing(log2_sum) / 2 + LOG2_SUM_SLACK) + fp32_spacing(lse) / 2 + exp2_error
    worst(name, (lse - log2_sum * ln2).abs() / allowed, torch.ones_like(lse, dtype=torch.bool))


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
def test_rows_tied_at_a_large_shift_keep_their_lse_within_fp32_rounding(head_dim):
    heads, rows, keys, positions = 4, 16, 320, (66, 67, 70, 200)
    ties = TIE_SCORES[torch.arange(heads * rows) % len(TIE_SCORES)].reshape(heads, rows, 1)
    where = torch.tensor(positions).expand(heads, rows, -1)
    scores = torch.full((heads, rows, keys), -FAR_SCORE, dtype=torch.float64).scatter(2, where, ties.expand_as(where))
    for shift in TIE_SHIFTS:
        check_log2_sum("lse of rows tied at the maximum", lse_of_scores(scores, shift, head_dim), base2_log_sum_exp(scores, shift))


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
def test_diffuse_rows_at_a_large_shift_keep_their_lse_within_fp32_rounding(head_dim):
    """One top key, eight keys up to 2 nats below in the same group of 16, two keys 6 and 6.5 nats below elsewhere
    (reference tests/test_softmax_fix.py:947-976)."""
    heads, rows, keys = 4, 32, 320
    near, far, groups, top_offset = (3, 5, 6, 9, 10, 12, 13, 15), {10: 6.0, 300: 6.5}, (64, 192), 2
    generator = torch.Generator().manual_seed(head_dim)
    log2_e = torch.tensor(math.log2(math.e), dtype=torch.float32).double()
    for shift in TIE_SHIFTS:
        exact = (shift + TIE_SCORES) * log2_e
        _, exponent = torch.frexp(exact.float().double())
        units = (exact - exact.float().double()).abs() / torch.ldexp(torch.ones_like(exact), exponent - 24)
        candidates = TIE_SCORES[units >= FAR_ROUNDING]  # scores whose product with log2(e) rounds far in FP32
        tops = candidates[torch.randint(len(candidates), (heads, rows, 1), generator=generator)]
        gaps = torch.randint(1, 17, (heads, rows, len(near)), generator=generator) / 8
        scores = torch.full((heads, rows, keys), -FAR_SCORE, dtype=torch.float64)
        for head in range(heads):
            group = groups[head % len(groups)]
            scores[head, :, group + top_offset] = tops[head, :, 0]
            scores[head, :, [group + offset for offset in near]] = tops[head] - gaps[head]
        for position, gap in far.items():
            scores[..., position] = tops[..., 0] - gap
        check_log2_sum("lse of diffuse rows", lse_of_scores(scores, shift, head_dim), base2_log_sum_exp(scores, shift), EXP2_ERROR)


# ------------------------------------------------------------------------------------------------ subnormal sums
# Two keys with the score -(83 + 7/64) and dP of 1 and -(1 - 2^-7) get BF16 dS whose sum is 2^-127, an FP32 subnormal
# number; a key with the score -(76 + 21/128) carries most of the remaining weight of its row (reference
# tests/test_softmax_fix.py:54-62,640-661).
PAIR_SCORE, PAIR_VALUE, HEAVY_SCORE = (83.0, 7 / 64), -(1 - 2.0**-7), (76.0, 21 / 128)
ORTHOGONAL_SHIFT, ROW_SUM_UNIT = 2.0**40, 2.0**-20


def subnormal_pair_problem(head_dim, shift, q=None, dout=None, seqlen_q=16):
    batch, seqlen_k = 2, 130
    layouts = ({1: (PAIR_SCORE, 1.0), 2: (PAIR_SCORE, PAIR_VALUE)},
               {1: (HEAVY_SCORE, 1.0), 128: (PAIR_SCORE, 1.0), 129: (PAIR_SCORE, PAIR_VALUE)})
    if q is None:
        q = torch.zeros(batch * seqlen_q, 1, head_dim, device="cuda", dtype=torch.float64)
        q[..., :2] = 1.0
    k = torch.zeros(batch * seqlen_k, 1, head_dim, device="cuda", dtype=torch.float64)
    v = torch.zeros_like(k)
    k[..., 0] = -FAR_SCORE
    for sequence, keys in enumerate(layouts):
        first = sequence * seqlen_k
        k[first, :, 0] = 0.0
        for key, ((whole, fraction), value) in keys.items():
            k[first + key, :, 0], k[first + key, :, 1], v[first + key, :, 0] = -whole, -fraction, value
    k[..., 2] = shift
    if dout is None:
        dout = torch.zeros_like(q)
        dout[..., 0] = 1.0
    window = WINDOWS["dense"]
    mask = fixed_mask(batch, q.shape[0] // batch, seqlen_k, window)
    return Problem(q, k, v, dout, mask, fixed_attention(batch, window, 1.0), 1.0)


def exact_ds(problem):
    q, k, v, dout = (x.double()[:, 0] for x in (problem.q, problem.k, problem.v, problem.dout))
    p = (problem.softmax_scale * q @ k.T).masked_fill(~problem.mask, float("-inf")).softmax(-1)
    dp = dout @ v.T
    return p * (dp - (p * dp).sum(-1, keepdim=True))


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
def test_query_gradient_ignores_a_key_shift_on_rows_with_subnormal_ds_sums(head_dim):
    """A shift of 2^40 along an axis that every query ignores multiplies the sum of the dS of a row: the sum of the BF16
    dS of the others, an FP32 subnormal number here, must reach the pivot unflushed (reference
    tests/test_softmax_fix.py:671-690)."""
    problem, shifted = subnormal_pair_problem(head_dim, 0.0), subnormal_pair_problem(head_dim, ORTHOGONAL_SHIFT)
    assert (shifted.k[..., 2] == ORTHOGONAL_SHIFT).all(), "the shifted keys are exact in bfloat16"
    ds = exact_ds(problem)
    pair = ds[0, 1:3].bfloat16().double().sum().abs()
    assert 0 < pair < 2.0**-126, "the BF16 dS of the key pair sum to an FP32 subnormal number"
    _, _, dq, _, _ = problem.run()
    _, _, shifted_dq, _, _ = shifted.run()
    allowed = ROW_SUM_UNIT * ORTHOGONAL_SHIFT * problem.softmax_scale * ds.abs().sum(-1, keepdim=True)
    ratio = (shifted_dq.double() - dq.double()).norm(dim=-1) / allowed
    worst("dq change under a key shift orthogonal to the queries", ratio, torch.ones_like(ratio, dtype=torch.bool))


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
def test_pivot_key_gradient_keeps_subnormal_sums_of_terms(head_dim):
    """Every row of the first sequence gives its pivot key the BF16 dS -2^-127; query columns that every key ignores give
    that key dK terms of -2^-133 and -2^-137 per row, which sum to FP32 subnormal numbers over the 16 rows (reference
    tests/test_softmax_fix.py:693-706)."""
    columns = {3: 2.0**-6, 4: 2.0**-10}
    pair = subnormal_pair_problem(head_dim, 0.0)
    q = pair.q.double().clone()
    q[..., list(columns)] = q.new_tensor(list(columns.values()))
    problem = subnormal_pair_problem(head_dim, 0.0, q=q)
    rows = slice(0, q.shape[0] // 2)
    row_sums = exact_ds(problem)[rows, 1:].bfloat16().double().sum(-1)
    expected = -problem.softmax_scale * (row_sums @ problem.q[rows, 0, list(columns)].double())
    assert (expected.abs() < 2.0**-126).all() and (expected != 0).all(), "the dK terms of the pivot key sum to subnormal numbers"
    _, _, _, dk, _ = problem.run()
    assert (dk[0, 0, list(columns)].double() == expected.bfloat16().double()).all(), (dk[0, 0, list(columns)], expected)


@pytest.mark.parametrize("head_dim", HEAD_DIMS)
def test_pivot_key_gradient_mixes_subnormal_and_large_sums_in_one_word(head_dim):
    """512 rows whose dS sum is 2^-127: one query column gives the pivot key terms of -2^-133 (first half of the rows)
    and -2^-27 (second half) in the same word, another only terms of -2^-137 (reference
    tests/test_softmax_fix.py:1020-1045)."""
    mixed_column, small, large, small_only_column, small_only, seqlen_q = 3, 2.0**-6, 2.0**100, 4, 2.0**-10, 512
    pair = subnormal_pair_problem(head_dim, 0.0)
    q = pair.q[:1].double().expand(2 * seqlen_q, -1, -1).clone()
    half = seqlen_q // 2
    for sequence in range(2):
        first = sequence * seqlen_q
        q[first : first + half, :, mixed_column] = small
        q[first + half : first + seqlen_q, :, mixed_column] = large
        q[first : first + seqlen_q, :, small_only_column] = small_only
    dout = pair.dout[:1].double().expand(2 * seqlen_q, -1, -1).clone()
    problem = subnormal_pair_problem(head_dim, 0.0, q=q, dout=dout)
    rows, columns = slice(0, seqlen_q), [mixed_column, small_only_column]
    row_sums = exact_ds(problem)[rows, 1:].bfloat16().double().sum(-1)
    assert (row_sums == 2.0**-127).all(), "every row of the first sequence has the dS sum 2^-127"
    expected = -problem.softmax_scale * (row_sums @ problem.q[rows, 0, columns].double())
    assert expected[0] == -half * 2.0**-27 and expected[1].abs() < 2.0**-126
    _, _, _, dk, _ = problem.run()
    assert (dk[0, 0, columns].double() == expected.bfloat16().double()).all(), (dk[0, 0, columns], expected)


# ------------------------------------------------------------------------------------------------ ties across key splits
def test_keys_tied_across_key_splits_at_a_large_shift_keep_the_unsplit_output():
    """Four keys tie at the row maximum, each in another share of a split-KV forward; the output must stay within 0.05
    BF16 units (mean) of the unsplit run, and so must a run with the ties gathered in one key block (reference
    tests/test_softmax_fix.py:829-861). The unsplit run is b200fa_fwd without a workspace."""
    import ctypes

    from zigfa._impl import lib

    head_dim, rows, keys, heads, tied = 128, 16, 4096, 2, 4
    spread = torch.arange(tied) * (keys // tied) + 5
    gathered = torch.tensor((2, 3, 6, 13))
    order = torch.arange(keys)
    order[spread], order[gathered] = gathered, spread
    generator = torch.Generator().manual_seed(head_dim)
    log2_e = torch.tensor(math.log2(math.e), dtype=torch.float32).double()
    library, stream = lib.library(), torch.cuda.current_stream().cuda_stream

    def forward(q, k, v, split):
        q, k, v = (x[None].contiguous() for x in (q, k, v))
        out = torch.full_like(q, float("nan"))
        lse = torch.full((1, heads, rows), float("nan"), device="cuda")
        problem = lib.make_problem(q, k, None, None, 1.0, -1, -1)
        nbytes = library.b200fa_fwd_workspace_bytes(ctypes.byref(problem)) if split else 0
        assert not split or nbytes > 0, "the planner must split this shape"
        workspace = torch.empty(max(nbytes, 1), dtype=torch.uint8, device="cuda")
        args = lib.FwdArgs(problem=problem, q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), out=out.data_ptr(),
                           softmax_lse=lse.data_ptr(), q_stride=lib.strides3(q, False), k_stride=lib.strides3(k, False),
                           v_stride=lib.strides3(v, False), out_stride=lib.strides3(out, False),
                           lse_stride=lib.Stride2(lse.stride(0), lse.stride(1)),
                           workspace=workspace.data_ptr() if split else None, workspace_bytes=nbytes)
        assert library.b200fa_fwd(ctypes.byref(args), stream) == 0, lib.last_error()
        torch.cuda.synchronize()
        return out[0]

    def tie_difference(name, out, reference):
        unit = 2.0**-8 * reference.double().abs().amax(-1, keepdim=True)
        difference = float(((out.double() - reference.double()).abs() / unit).mean())
        assert difference <= 0.05, f"{name}: mean |O - unsplit O| = {difference:.3f} bfloat16 units"

    for shift in TIE_SHIFTS:
        exact = (shift + TIE_SCORES) * log2_e
        _, exponent = torch.frexp(exact.float().double())
        units = (exact - exact.float().double()).abs() / torch.ldexp(torch.ones_like(exact), exponent - 24)
        candidates = TIE_SCORES[units >= FAR_ROUNDING]
        scores = []
        for _ in range(heads):
            other = -torch.randint(60, 120, (rows, keys), generator=generator).double() / 2
            ties = candidates[torch.randint(len(candidates), (rows, 1), generator=generator)]
            scores.append(other.scatter(1, spread.expand(rows, -1), ties.expand(-1, tied)))
        scores = torch.stack(scores)
        q = torch.zeros(rows, heads, head_dim, dtype=torch.float64)
        q[torch.arange(rows), :, torch.arange(rows)] = 1.0
        q[..., -1] = 1.0
        k = torch.zeros(keys, heads, head_dim, dtype=torch.float64)
        k[..., :rows] = scores.permute(2, 0, 1)
        k[..., -1] = shift
        v = torch.randn(keys, heads, head_dim, generator=generator, dtype=torch.float64).bfloat16().double()
        q, k, v = (x.cuda().bfloat16() for x in (q, k, v))
        unsplit = forward(q, k, v, split=False)
        tie_difference("split keys", forward(q, k, v, split=True), unsplit)
        tie_difference("tied keys in one key block", forward(q, k[order], v[order], split=False), unsplit)
