"""The CPU oracle against the golden fixtures generated from the reference's own oracle code
(tests/golden/make_golden.py): float64 attention, gradients and masks."""
from pathlib import Path

import numpy as np
import pytest
import torch

import attention_oracle as oracle
from golden.make_golden import CASES, INTERSEQ, STABLE, STABLE_FIELDS, VARLEN, inputs, sharp_inputs

GOLDEN = np.load(Path(__file__).parent / "golden" / "attention_golden.npz")


def unpack(bits, shape):
    return torch.from_numpy(np.unpackbits(bits)[: int(np.prod(shape))].reshape(shape).astype(bool))


@pytest.mark.parametrize("seed_case", list(enumerate(CASES)), ids=[case[0] for case in CASES])
def test_attention_matches_reference_float64(seed_case):
    seed, (name, batch, sq, sk, hq, hkv, d, window) = seed_case
    q, k, v, dout = inputs(seed, batch, sq, sk, hq, hkv, d)
    mask = oracle.visible_keys([sq] * batch, [sk] * batch, sq, sk, window)
    assert torch.equal(mask, unpack(GOLDEN[f"{name}/mask"], (batch, sq, sk)))
    out, lse, dq, dk, dv = oracle.gradients(oracle.attention, q, k, v, dout, window_size=window, dtype=torch.float64)
    # the fixtures were stored in float32
    for field, value in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        expected = torch.from_numpy(GOLDEN[f"{name}/{field}"]).double()
        assert value.shape == expected.shape
        assert torch.allclose(value, expected, rtol=1e-5, atol=1e-6), field
    expected_lse = torch.from_numpy(GOLDEN[f"{name}/lse"]).double()
    finite = torch.isfinite(expected_lse)
    assert torch.equal(torch.isfinite(lse), finite)
    assert torch.allclose(lse[finite], expected_lse[finite], rtol=1e-5, atol=1e-6)
    # float32 math (the arithmetic of the CPU baseline) stays within 1e-4 of float64
    out32, lse32, *_ = oracle.gradients(oracle.attention, q, k, v, dout, window_size=window, dtype=torch.float32)
    assert (out32.double() - out).abs().max() < 1e-4


@pytest.mark.parametrize("seed_case", list(enumerate(STABLE)), ids=[case[0] for case in STABLE])
def test_stable_attention_matches_reference_float64(seed_case):
    """Every field of the float64 reference with the top key taken apart (out, lse, gradients, pivot rows, margins, error
    weights) on inputs sharp enough that about half of the rows have a pivot."""
    seed, (name, batch, sq, sk, hq, hkv, d, window, factor) = seed_case
    q, k, v, dout = sharp_inputs(seed, batch, sq, sk, hq, hkv, d, factor)
    mask = oracle.visible_keys([sq], [sk], sq, sk, window)[0]
    for b in range(batch):
        result = oracle.stable_attention(q[b], k[b], v[b], dout[b], mask)
        for field in STABLE_FIELDS:
            expected = torch.from_numpy(GOLDEN[f"{name}/{field}"][b])
            value = result[field]
            assert value.shape == expected.shape, field
            if value.dtype == torch.bool:
                assert torch.equal(value, expected.bool()), field
            else:
                assert torch.allclose(value.double(), expected, rtol=1e-9, atol=1e-12, equal_nan=True), field
    assert 0.3 < float(torch.from_numpy(GOLDEN[f"{name}/pivot"]).mean()) < 0.9


@pytest.mark.parametrize("index", range(len(VARLEN)))
def test_packed_mask_matches_reference(index):
    lengths_q, lengths_k, window = VARLEN[index]
    cu_q, cu_k = np.concatenate([[0], np.cumsum(lengths_q)]), np.concatenate([[0], np.cumsum(lengths_k)])
    mask = oracle.packed_mask(cu_q, cu_k, window)
    assert torch.equal(mask, unpack(GOLDEN[f"varlen{index}/mask"], mask.shape))


@pytest.mark.parametrize("index", range(len(INTERSEQ)))
def test_inter_sequence_mask_matches_reference(index):
    lengths_q, lengths_k, visible, windows = INTERSEQ[index]
    cu_q, cu_k = np.concatenate([[0], np.cumsum(lengths_q)]), np.concatenate([[0], np.cumsum(lengths_k)])
    mask = oracle.inter_sequence_mask(cu_q, cu_k, visible, windows)
    assert torch.equal(mask, unpack(GOLDEN[f"interseq{index}/mask"], mask.shape))


def test_zero_window_returns_values():
    # reference tests/test_reference.py:74-80: a (0, 0) window sees only the diagonal, so out == v and lse == q.k*scale
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 16, 2, 32, dtype=torch.bfloat16) for _ in range(3))
    out, lse = oracle.attention(q, k, v, window_size=(0, 0))
    assert torch.allclose(out, v.float(), atol=1e-6)
    expected = (q.float() * k.float()).sum(-1).transpose(1, 2) * 32**-0.5
    assert torch.allclose(lse, expected, atol=1e-5)


def test_rows_without_keys():
    q, k, v = (torch.randn(1, 8, 1, 16, dtype=torch.bfloat16) for _ in range(3))
    out, lse = oracle.attention(q[:, :8], k[:, :3], v[:, :3], causal=True)  # rows 0..4 see nothing (bottom-right)
    assert (out[0, :5] == 0).all() and (lse[0, :, :5] == float("-inf")).all()
    assert torch.isfinite(lse[0, :, 5:]).all()


def test_integer_definitions():
    assert [oracle.length_class(x) for x in (0, 1, 2, 3, 4, 5, 6, 7, 8, 1 << 20)] == [0, 0, 4, 6, 8, 9, 10, 11, 12, 80]
    visible = np.array([[1, 0, 1], [1, 1, 0], [0, 0, 1]], dtype=bool)
    assert oracle.visibility_bits_of(visible).tolist() == [[5], [3], [4]]
    bits_t, cu_k, cu_q = oracle.metadata_definition([2, 3, 4], [5, 6, 7], visible)
    assert bits_t.tolist() == [[3], [2], [5]]
    assert cu_k.tolist() == [0, 12, 23, 30] and cu_q.tolist() == [0, 5, 8, 14]
    big = np.ones((40, 40), dtype=bool)
    assert oracle.visibility_bits_of(big)[0].tolist() == [-1, 255]
    assert oracle.every_block([3, 0, 5], 2, 7) == [(0, 0), (0, 1), (2, 0), (2, 1), (2, 2), (3, 0), (3, 0)]
    assert oracle.visible_pairs([512], [512], (-1, 0)) == 512 * 513 // 2
