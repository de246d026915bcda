// Pieces shared by the forward kernels: kernel parameters, work-item decoding and the host-side set-up of both.
#pragma once
#include "common.h"
#include "ptx.cuh"

namespace b200fa {

struct FwdParams {
  Problem prob;
  float scale_log2;
  __nv_bfloat16* o;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  float* lse;
  int64_t lse_batch_stride, lse_head_stride;
  const int2* work_list;  // packed problems: (sequence, block) per entry; null for fixed length
  int m_blocks;           // fixed length: work items per (batch, head)
  int num_tiles;
  int head_dim;           // columns of the tensors (<= the compiled width; TMA zero-fills the columns in between)
  int* status;            // device status word of the library
  long long* trace;       // optional cycle counters of tuning builds (slots 16-23), null = off
};

struct FwdTile {
  int seq, head, kv_head, m0;
  SeqInfo s;
  bool valid;
};

// `tile_rows` = query rows per work item (256 for the two-stage kernel, 128 for the head_dim 256 kernel).
__device__ __forceinline__ FwdTile decode_tile(const FwdParams& p, int tile, int tile_rows = kFwdTileM) {
  FwdTile t;
  const Problem& pr = p.prob;
  if (p.work_list) {
    int entry = tile / pr.heads_q;
    t.head = tile - entry * pr.heads_q;
    int2 e = p.work_list[entry];
    t.seq = e.x;
    t.m0 = e.y * tile_rows;
    t.valid = e.x < pr.batch;
  } else {
    // Work items that run at the same time share K and V: all query blocks and query heads of one (batch entry, key
    // head) are consecutive, late (heavy under a causal mask) query blocks first, so the K/V stream they read stays
    // in L2 (reference zig/tile_scheduler.zig:516-669 orders tiles in L2-sized sections for the same reason).
    const int group = pr.heads_q / pr.heads_kv;
    const int per_group = p.m_blocks * group;
    const int kv_group = tile / per_group;  // (batch entry, key head)
    const int rem = tile - kv_group * per_group;
    const int mb = rem / group;
    t.seq = kv_group / pr.heads_kv;
    t.head = (kv_group - t.seq * pr.heads_kv) * group + (rem - mb * group);
    t.m0 = (p.m_blocks - 1 - mb) * tile_rows;
    t.valid = true;
  }
  t.kv_head = t.head / (pr.heads_q / pr.heads_kv);
  if (t.valid) t.s = seq_info(pr, t.seq);
  return t;
}

// Fills the kernel parameters, builds the work list of a packed batch and encodes the Q / K / V tensor maps.
// `tile_rows` = query rows per work item, `kv_box_rows` = key rows per TMA box. Sets *nothing_to_do when no kernel is
// needed. Defined in fwd.cu.
int prepare_forward(const b200fa_fwd_args& a, cudaStream_t stream, int head_dim, int tile_rows, int kv_box_rows,
                    FwdParams* p, CUtensorMap* map_q, CUtensorMap* map_k, CUtensorMap* map_v, bool* nothing_to_do);
int launch_fwd_256(const b200fa_fwd_args& a, cudaStream_t stream);
int launch_fwd_512(const b200fa_fwd_args& a, cudaStream_t stream);

}  // namespace b200fa
