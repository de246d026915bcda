"""Partitioning of attention problems over the GPUs of one node. Shards are independent (attention never mixes batch
entries, sequences that cannot see each other, or key-head groups), so the data path needs no collective; a gather of
outputs is only used to verify or to assemble results. The reference has no multi-GPU code; these helpers define the
work split the benchmark reports."""
from __future__ import annotations

import numpy as np


def batch_shard(batch: int, world: int, rank: int) -> range:
    """Contiguous, near-even split of `batch` entries."""
    base, extra = divmod(batch, world)
    start = rank * base + min(rank, extra)
    return range(start, start + base + (1 if rank < extra else 0))


def sequence_cost(length_q: int, length_k: int, window=(-1, -1)) -> int:
    """Visible (query, key) pairs of one sequence: proportional to its attention FLOPs."""
    left, right = window
    rows = np.arange(length_q, dtype=np.int64)
    shift = length_k - length_q
    hi = np.full(length_q, length_k) if right < 0 else np.minimum(length_k, rows + shift + right + 1)
    lo = np.zeros(length_q, dtype=np.int64) if left < 0 else np.maximum(0, rows + shift - left)
    return int(np.maximum(hi - lo, 0).sum())


def varlen_shards(lengths_q, lengths_k, world: int, window=(-1, -1)) -> list[list[int]]:
    """Longest-processing-time assignment of whole sequences to ranks; each rank keeps its sequences in input order."""
    costs = [sequence_cost(lq, lk, window) for lq, lk in zip(lengths_q, lengths_k)]
    loads, shards = [0] * world, [[] for _ in range(world)]
    for sequence in sorted(range(len(costs)), key=lambda i: -costs[i]):
        rank = min(range(world), key=lambda r: (loads[r], r))
        loads[rank] += costs[sequence]
        shards[rank].append(sequence)
    return [sorted(shard) for shard in shards]


def rebase_cu_seqlens(lengths, members) -> np.ndarray:
    return np.concatenate([[0], np.cumsum([lengths[i] for i in members])]).astype(np.int32)


def visibility_components(visible) -> list[list[int]]:
    """Connected components of the visibility graph (query i - key j): sequences of different components never
    interact, so whole components can go to different ranks."""
    visible = np.asarray(visible, dtype=bool)
    count = visible.shape[0]
    linked = visible | visible.T
    label = [-1] * count
    components = []
    for start in range(count):
        if label[start] >= 0:
            continue
        stack, members = [start], []
        label[start] = len(components)
        while stack:
            node = stack.pop()
            members.append(node)
            for other in np.nonzero(linked[node])[0]:
                if label[other] < 0:
                    label[other] = len(components)
                    stack.append(int(other))
        components.append(sorted(members))
    return components
