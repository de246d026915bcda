"""Host twins of the integer kernels and cursors (same header code as the device) against the numpy definitions of
the oracle: work lists, inter-sequence metadata, and the key / query block cursors against dense masks. Bit-exact."""
import ctypes

import numpy as np
import pytest
import torch

import attention_oracle as oracle
from zigfa._impl import lib


def cu_of(lengths, offset=0):
    return (np.concatenate([[0], np.cumsum(lengths)]) + offset).astype(np.int32)


def host_work_list(lengths, other, block, descending):
    cu, cu_other = cu_of(lengths, 17), cu_of(other, 17)
    entries = oracle.work_list_entries(int(np.sum(lengths)), len(lengths), block)
    table = np.full((max(entries, 1), 2), -1, dtype=np.int32)
    status = lib.library().b200fa_work_list_host(
        cu.ctypes.data, cu_other.ctypes.data, len(lengths), block, descending, entries, table.ctypes.data
    )
    assert status == 0
    return table[:entries], entries


def lengths_of(kind, batch, block, rng):
    # the three families of reference tests/test_specialization.py:18-26
    if kind == "zero":
        lengths = rng.integers(0, 3, batch) * rng.integers(1, 300, batch)
        lengths[: batch // 2] = 0
        return lengths
    if kind == "tile_multiples":
        return rng.integers(0, 4, batch) * block
    return (rng.random(batch) ** 6 * 4000).astype(np.int64) + 1


@pytest.mark.parametrize("batch", [1, 4, 31, 32, 33, 1023, 1024, 1025, 2049, 3000])
@pytest.mark.parametrize("kind", ["heavy_tail", "zero", "tile_multiples"])
@pytest.mark.parametrize("block,descending", [(256, 1), (128, 0)])
def test_work_list_lists_every_block_once_in_the_defined_order(batch, kind, block, descending):
    rng = np.random.default_rng(batch * 7 + len(kind))
    lengths = lengths_of(kind, batch, block, rng)
    other = rng.integers(0, 5000, batch)
    table, entries = host_work_list(lengths, other, block, descending)
    assert entries == lib.library().b200fa_work_list_entries(int(lengths.sum()), batch, block)
    listed = sorted(map(tuple, table.tolist()))
    assert listed == oracle.every_block(lengths.tolist(), block, entries)
    assert np.array_equal(table, oracle.work_list_definition(lengths, other, block, bool(descending), entries))


def test_work_list_treats_decreasing_prefix_sums_as_empty_sequences():
    """A cu_seqlens array that is not non-decreasing describes no batch. Its negative lengths must count as empty
    sequences, so that no entry lands outside the table (in front of it, with a negative index)."""
    cu = np.array([0, 600, 300, 900, 800, 1300], dtype=np.int32)  # lengths 600, -300, 600, -100, 500
    guard, entries = 8, 12
    table = np.full((guard + entries + guard, 2), -7, dtype=np.int32)
    body = table[guard : guard + entries]
    status = lib.library().b200fa_work_list_host(cu.ctypes.data, cu.ctypes.data, 5, 256, 0, entries, body.ctypes.data)
    assert status == 0
    assert (table[:guard] == -7).all() and (table[guard + entries :] == -7).all()
    listed = [tuple(row) for row in body.tolist() if row[0] < 5]
    assert sorted(listed) == [(0, 0), (0, 1), (0, 2), (2, 0), (2, 1), (2, 2), (4, 0), (4, 1)]
    assert all(tuple(row) == (5, 0) for row in body.tolist()[len(listed) :])


@pytest.mark.parametrize("count", [1, 31, 32, 33, 100])
def test_metadata_matches_its_definition(count):
    rng = np.random.default_rng(count)
    lengths_q = rng.integers(0, 160, count)
    lengths_k = lengths_q + rng.integers(0, 40, count)
    visible = rng.random((count, count)) < 0.4
    bits = oracle.visibility_bits_of(visible)
    cu_q, cu_k = cu_of(lengths_q), cu_of(lengths_k)
    words = (count + 31) // 32
    bits_t = np.empty((count, words), dtype=np.int32)
    cu_visible_k, cu_visible_q = np.empty(count + 1, dtype=np.int32), np.empty(count + 1, dtype=np.int32)
    status = lib.library().b200fa_interseq_metadata_host(
        cu_q.ctypes.data, cu_k.ctypes.data, bits.ctypes.data, count, bits_t.ctypes.data, cu_visible_k.ctypes.data,
        cu_visible_q.ctypes.data,
    )
    assert status == 0
    expected = oracle.metadata_definition(lengths_q, lengths_k, visible)
    assert np.array_equal(bits_t, expected[0])
    assert np.array_equal(cu_visible_k, expected[1])
    assert np.array_equal(cu_visible_q, expected[2])


def blocks_of(function, problem, seq, lo, hi):
    out = np.zeros((4096, 4), dtype=np.int32)
    count = function(ctypes.byref(problem), seq, lo, hi, out.ctypes.data, 4096)
    assert 0 <= count <= 4096
    return out[:count]


def covered_by_key_blocks(blocks, band_mask_of_self, k0_self, total_k, rows):
    """Dense (rows, total_k) mask of what the listed key blocks let the rows see."""
    seen = np.zeros((rows.size, total_k), dtype=bool)
    for row0, col0, limit, banded in blocks:
        width = min(128, limit - col0)
        assert width > 0
        if banded:
            assert row0 - col0 == k0_self
            seen[:, row0 : row0 + width] |= band_mask_of_self[rows][:, col0 : col0 + width]
        else:
            seen[:, row0 : row0 + width] = True
    return seen


WINDOWS = [(-1, -1), (-1, 0), (-1, 7), (5, -1), (9, 3), (0, 0), (300, 0), (100, 200)]


@pytest.mark.parametrize("lq,lk", [(1, 1), (64, 128), (113, 203), (640, 128), (1023, 1024), (700, 3), (0, 50), (50, 0)])
@pytest.mark.parametrize("window", WINDOWS)
def test_key_and_query_cursors_cover_exactly_the_band(lq, lk, window):
    problem = lib.Problem(batch=1, seqlen_q=lq, seqlen_k=lk, heads_q=1, heads_kv=1, head_dim=128,
                          window_left=window[0], window_right=window[1], softmax_scale=1.0)
    library = lib.library()
    mask = oracle.visible_keys([lq], [lk], max(lq, 1), max(lk, 1), window)[0].numpy()[:lq, :lk]
    for m0 in range(0, lq, 256):
        rows = np.arange(m0, min(m0 + 256, lq))
        blocks = blocks_of(library.b200fa_key_blocks_host, problem, 0, m0, m0 + 256)
        seen = covered_by_key_blocks(blocks, mask, 0, lk, rows)
        assert np.array_equal(seen, mask[rows]), (m0, blocks.tolist())
        # tile skipping: every listed block holds at least one visible pair of the tile
        for row0, col0, limit, banded in blocks:
            assert mask[rows][:, col0 : col0 + 128].any()
    for c0 in range(0, lk, 128):
        cols = np.arange(c0, min(c0 + 128, lk))
        blocks = blocks_of(library.b200fa_query_blocks_host, problem, 0, c0, c0 + 128)
        seen = np.zeros((lq, cols.size), dtype=bool)
        for row0, col0, limit, banded in blocks:
            height = min(128, limit - col0)
            assert banded == 1 and row0 == col0 and height > 0
            seen[row0 : row0 + height] |= mask[row0 : row0 + height][:, cols]
            assert mask[row0 : row0 + height][:, cols].any()
        assert np.array_equal(seen, mask[:, cols])


@pytest.mark.parametrize("seed", range(6))
def test_inter_sequence_cursors_cover_exactly_the_mask(seed):
    rng = np.random.default_rng(seed)
    count = [5, 11, 40, 70, 9, 33][seed]
    lengths_q = rng.integers(0, 300, count)
    lengths_k = lengths_q + rng.integers(0, 40, count)
    lengths_q[:: max(1, count // 3)] = 0
    visible = rng.random((count, count)) < 0.4
    if seed == 4:
        visible[:] = False
        visible[:, ::2] = True
        np.fill_diagonal(visible, True)
    windows = [WINDOWS[i] for i in rng.integers(0, 6, count)]
    cu_q, cu_k = cu_of(lengths_q), cu_of(lengths_k)
    bits = oracle.visibility_bits_of(visible)
    bits_t, cu_visible_k, cu_visible_q = oracle.metadata_definition(lengths_q, lengths_k, visible)
    window_sizes = np.ascontiguousarray(np.asarray(windows, dtype=np.int32).T)
    problem = lib.Problem(batch=count, seqlen_q=int(cu_q[-1]), seqlen_k=int(cu_k[-1]), heads_q=1, heads_kv=1, head_dim=128,
                          window_left=-1, window_right=-1, softmax_scale=1.0, cu_seqlens_q=cu_q.ctypes.data,
                          cu_seqlens_k=cu_k.ctypes.data, visibility_bits=bits.ctypes.data,
                          visibility_bits_t=bits_t.ctypes.data, cu_visible_k=cu_visible_k.ctypes.data,
                          cu_visible_q=cu_visible_q.ctypes.data, window_sizes=window_sizes.ctypes.data)
    library = lib.library()
    mask = oracle.inter_sequence_mask(cu_q, cu_k, visible, windows).numpy()
    for i in range(count):
        lq, lk = int(lengths_q[i]), int(lengths_k[i])
        own = oracle.visible_keys([lq], [lk], max(lq, 1), max(lk, 1), windows[i])[0].numpy()
        for m0 in range(0, lq, 256):
            rows = np.arange(m0, min(m0 + 256, lq))
            blocks = blocks_of(library.b200fa_key_blocks_host, problem, i, m0, m0 + 256)
            seen = covered_by_key_blocks(blocks, own, int(cu_k[i]), int(cu_k[-1]), rows)
            assert np.array_equal(seen, mask[cu_q[i] + rows]), (i, m0)
    for j in range(count):
        lq, lk = int(lengths_q[j]), int(lengths_k[j])
        own = oracle.visible_keys([lq], [lk], max(lq, 1), max(lk, 1), windows[j])[0].numpy()
        for c0 in range(0, lk, 128):
            cols = np.arange(c0, min(c0 + 128, lk))
            blocks = blocks_of(library.b200fa_query_blocks_host, problem, j, c0, c0 + 128)
            seen = np.zeros((int(cu_q[-1]), cols.size), dtype=bool)
            for row0, col0, limit, banded in blocks:
                height = min(128, limit - col0)
                if banded:
                    assert row0 - col0 == cu_q[j]
                    seen[row0 : row0 + height] |= own[col0 : col0 + height][:, cols]
                else:
                    seen[row0 : row0 + height] = True
            assert np.array_equal(seen, mask[:, cu_k[j] + cols]), (j, c0)
