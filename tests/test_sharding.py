"""Multi-rank path on the CPU (gloo, world size 2): each rank computes its shard with the oracle, results are
gathered, and the assembled tensors equal the unsharded computation. Covers the batch split, the longest-first
assignment of packed sequences and the split of inter-sequence batches by visibility component."""
import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "zig-flash-attn_b200"))
sys.path.insert(0, str(ROOT / "oracle"))

import attention_oracle as oracle  # noqa: E402
import sharding  # noqa: E402


def test_batch_shards_cover_the_batch_evenly():
    for batch, world in [(16, 8), (16, 1), (7, 4), (3, 8)]:
        parts = [list(sharding.batch_shard(batch, world, rank)) for rank in range(world)]
        assert sum(parts, []) == list(range(batch))
        assert max(map(len, parts)) - min(map(len, parts)) <= 1


def test_varlen_shards_balance_and_cover():
    rng = np.random.default_rng(0)
    lengths = rng.integers(256, 8193, 20).tolist()
    shards = sharding.varlen_shards(lengths, lengths, 4, window=(4096, 0))
    assert sorted(sum(shards, [])) == list(range(20))
    loads = [sum(sharding.sequence_cost(lengths[i], lengths[i], (4096, 0)) for i in shard) for shard in shards]
    assert max(loads) <= 1.25 * (sum(loads) / 4)
    assert sharding.sequence_cost(512, 512, (-1, 0)) == 512 * 513 // 2


def test_visibility_components_split_groups():
    visible = np.zeros((6, 6), dtype=bool)
    np.fill_diagonal(visible, True)
    visible[1, 0] = visible[2, 0] = True  # group {0, 1, 2}
    visible[5, 3] = True                  # group {3, 5}; 4 alone
    assert sharding.visibility_components(visible) == [[0, 1, 2], [3, 5], [4]]


def _worker(rank, world, port, result_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    batch, seqlen, heads_q, heads_kv, d = 4, 48, 4, 2, 32
    q = torch.randn(batch, seqlen, heads_q, d, dtype=torch.bfloat16)
    k, v = (torch.randn(batch, seqlen, heads_kv, d, dtype=torch.bfloat16) for _ in range(2))
    mine = sharding.batch_shard(batch, world, rank)
    out, _ = oracle.attention(q[mine.start : mine.stop], k[mine.start : mine.stop], v[mine.start : mine.stop], causal=True)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out.contiguous())
    full, _ = oracle.attention(q, k, v, causal=True)
    same_batch = torch.equal(torch.cat(gathered), full)

    # packed sequences: longest-first assignment, shard-local cu_seqlens, results scattered back by sequence
    lengths = [40, 7, 33, 64, 12, 25]
    shards = sharding.varlen_shards(lengths, lengths, world, window=(-1, 0))
    cu = np.concatenate([[0], np.cumsum(lengths)])
    qp = torch.randn(int(cu[-1]), heads_q, d, dtype=torch.bfloat16)
    kp, vp = (torch.randn(int(cu[-1]), heads_kv, d, dtype=torch.bfloat16) for _ in range(2))
    rows = torch.cat([torch.arange(cu[i], cu[i + 1]) for i in shards[rank]])
    local_cu = sharding.rebase_cu_seqlens(lengths, shards[rank])
    local, _ = oracle.varlen_attention(qp[rows], kp[rows], vp[rows], local_cu, local_cu, causal=True)
    sizes = [sum(lengths[i] for i in shard) for shard in shards]
    padded = torch.zeros(max(sizes), heads_q, d)
    padded[: local.shape[0]] = local
    pieces = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(pieces, padded)
    assembled = torch.empty(int(cu[-1]), heads_q, d)
    for r, shard in enumerate(shards):
        shard_rows = torch.cat([torch.arange(cu[i], cu[i + 1]) for i in shard])
        assembled[shard_rows] = pieces[r][: sizes[r]]
    whole, _ = oracle.varlen_attention(qp, kp, vp, cu, cu, causal=True)
    same_packed = torch.allclose(assembled, whole, atol=1e-6)
    if rank == 0:
        Path(result_path).write_text(f"{same_batch} {same_packed}")
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reassemble_the_unsharded_result(tmp_path):
    result = tmp_path / "result.txt"
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(result)), nprocs=2, join=True)
    assert result.read_text() == "True True"
