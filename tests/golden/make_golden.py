"""Generates the golden fixtures of tests/golden/ from the reference's own oracle code.

Run where a checkout of the reference is available (it is not needed to run the tests):
    python tests/golden/make_golden.py <path to the reference checkout>
It imports the reference's tests/reference.py (pure PyTorch) and stores, for seeded inputs:
  * float64 attention outputs and gradients of `stable_attention_f64` (reference tests/reference.py:192-247), and for
    the sharpened cases of STABLE every field of its result (top, margin, spread, pivot rows, error weights, ...),
  * the masks of `visible_keys`, `varlen_visible`, `inter_sequence_visible` (reference tests/reference.py:10-19,
    148-168, 250-260),
as `attention_golden.npz`. The reference's aten-based entry points need a CUDA device and are not used here.
Inputs are regenerated from the stored seeds by tests (torch.manual_seed + torch.randn in BF16), so the file stays small.
"""
import sys
from pathlib import Path

import numpy as np
import torch

CASES = [
    # name, batch, seqlen_q, seqlen_k, heads_q, heads_kv, head_dim, window
    ("causal_gqa", 2, 48, 48, 4, 2, 64, (-1, 0)),
    ("dense_mha", 1, 33, 57, 2, 2, 32, (-1, -1)),
    ("window_mqa", 1, 70, 90, 4, 1, 64, (11, 5)),
    ("short_keys", 1, 40, 7, 2, 1, 32, (-1, 0)),
    ("left_only", 1, 64, 64, 2, 2, 32, (9, -1)),
]
# name, batch, seqlen_q, seqlen_k, heads_q, heads_kv, head_dim, window, factor on q (sharp rows: pivots, large margins)
STABLE = [
    ("sharp_causal_gqa", 1, 40, 56, 4, 2, 32, (-1, 0), 6.0),
    ("sharp_dense_mqa", 2, 24, 24, 2, 1, 16, (-1, -1), 10.0),
    ("sharp_window", 1, 48, 64, 2, 2, 32, (9, 3), 4.0),
]
STABLE_FIELDS = ("out", "lse", "dq", "dk", "dv", "top", "margin", "spread", "visible", "pivot", "out_scale", "dq_scale",
                 "dk_scale", "dv_scale", "corrected_keys")
VARLEN = [([5, 0, 17, 32], [9, 4, 17, 20], (-1, 0)), ([1, 64, 3], [1, 64, 30], (7, 2))]
INTERSEQ = [
    ([6, 10, 4, 9], [6, 12, 4, 9], [[1, 0, 0, 0], [1, 1, 0, 0], [0, 0, 1, 0], [1, 0, 1, 1]],
     [(-1, 0), (-1, -1), (2, 1), (-1, 0)]),
    ([0, 8, 8], [5, 8, 3], [[1, 0, 0], [1, 1, 0], [1, 1, 1]], [(-1, -1), (-1, 0), (0, 0)]),
]


def inputs(seed, batch, seqlen_q, seqlen_k, heads_q, heads_kv, head_dim):
    torch.manual_seed(seed)
    q = torch.randn(batch, seqlen_q, heads_q, head_dim, dtype=torch.bfloat16)
    k = torch.randn(batch, seqlen_k, heads_kv, head_dim, dtype=torch.bfloat16)
    v = torch.randn(batch, seqlen_k, heads_kv, head_dim, dtype=torch.bfloat16)
    dout = torch.randn(batch, seqlen_q, heads_q, head_dim, dtype=torch.bfloat16)
    return q, k, v, dout


def sharp_inputs(seed, batch, seqlen_q, seqlen_k, heads_q, heads_kv, head_dim, factor):
    q, k, v, dout = inputs(1000 + seed, batch, seqlen_q, seqlen_k, heads_q, heads_kv, head_dim)
    return (factor * q.float()).bfloat16(), k, v, dout


def main(reference_root):
    sys.path.insert(0, str(Path(reference_root) / "tests"))
    import reference

    arrays = {}
    for seed, (name, batch, sq, sk, hq, hkv, d, window) in enumerate(CASES):
        q, k, v, dout = inputs(seed, batch, sq, sk, hq, hkv, d)
        visible = reference.visible_keys(torch.tensor([sq] * batch), torch.tensor([sk] * batch), sq, sk, window)
        result = reference.stable_attention_f64(q, k, v, dout, visible)
        arrays[f"{name}/mask"] = np.packbits(visible.numpy())
        for field in ("out", "lse", "dq", "dk", "dv"):
            arrays[f"{name}/{field}"] = getattr(result, field).numpy().astype(np.float32)
    for seed, (name, batch, sq, sk, hq, hkv, d, window, factor) in enumerate(STABLE):
        q, k, v, dout = sharp_inputs(seed, batch, sq, sk, hq, hkv, d, factor)
        visible = reference.visible_keys(torch.tensor([sq] * batch), torch.tensor([sk] * batch), sq, sk, window)
        result = reference.stable_attention_f64(q, k, v, dout, visible)
        for field in STABLE_FIELDS:
            arrays[f"{name}/{field}"] = getattr(result, field).numpy().astype(np.float64)
    for index, (lengths_q, lengths_k, window) in enumerate(VARLEN):
        cu_q = torch.tensor([0, *np.cumsum(lengths_q)])
        cu_k = torch.tensor([0, *np.cumsum(lengths_k)])
        arrays[f"varlen{index}/mask"] = np.packbits(reference.varlen_visible(cu_q, cu_k, window).numpy())
    for index, (lengths_q, lengths_k, visible, windows) in enumerate(INTERSEQ):
        cu_q = torch.tensor([0, *np.cumsum(lengths_q)])
        cu_k = torch.tensor([0, *np.cumsum(lengths_k)])
        mask = reference.inter_sequence_visible(cu_q, cu_k, torch.tensor(visible, dtype=torch.bool), windows)
        arrays[f"interseq{index}/mask"] = np.packbits(mask.numpy())
    target = Path(__file__).resolve().parent / "attention_golden.npz"
    np.savez_compressed(target, **arrays)
    print(target, target.stat().st_size, "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit(__doc__)
    main(sys.argv[1])
