// Pieces shared by the two backward main kernels for head_dim 256 (bwd_d256.cu, bwd_d256_pair.cu): the role and tile
// constants and the cursor that walks the query blocks of a key block in 64-row halves.
#pragma once

#include "bwd_common.cuh"

namespace b200fa {
namespace bd256 {

constexpr int kSubM = 64;                   // query rows per iteration
constexpr int kGroups = 4;                   // compute warpgroups: a thread handles one key row and 64 / kGroups query columns
constexpr int kCols = kSubM / kGroups;
constexpr int kComputeWarps = 4 * kGroups;
constexpr int kDrains = 2;                   // dQ drain warpgroups: each takes half of the 64 query rows of an iteration
constexpr int kMmaWarp = kComputeWarps + 4 * kDrains, kLoadWarp = kMmaWarp + 1;
constexpr int kThreads = 32 * (kMmaWarp + 4);
// registers per thread of the compute, drain and MMA/load warpgroups: 4 x 128 x 88 + 2 x 128 x 56 + 128 x 40 = 896 x 72
constexpr int kRegsCompute = 88, kRegsDrain = 56, kRegsMisc = 40;
static_assert(kComputeWarps * 32 * kRegsCompute + kDrains * 128 * kRegsDrain + 128 * kRegsMisc == kThreads * 72,
              "the per-role register budgets must add up to the launch allocation");
constexpr int kKvPanel = 128 * 128;         // 128 key rows x 64 columns BF16
constexpr int kKvBytes = 4 * kKvPanel;      // 64 KB
constexpr int kQPanel = kSubM * 128;        // 64 query rows x 64 columns BF16
constexpr int kQBytes = 4 * kQPanel;        // 32 KB
constexpr int kDsBytes = 128 * 128;         // 128 keys x 64 queries BF16
constexpr int kStageRows = 16;              // query rows per staging buffer
constexpr int kStageBytes = kStageRows * 128 * 4;

// Yields the 128-row query blocks of a QueryCursor as 64-row halves (a half past the end of its run is skipped).
struct HalfBlockCursor {
  QueryCursor cursor;
  OtherBlock block;
  int half;
  __device__ void init(const Problem* problem, int seq, const SeqInfo& s, int c0, int c1) {
    cursor.init(problem, seq, s, c0, c1);
    half = 2;
  }
  __device__ bool next(OtherBlock* out) {
    for (;;) {
      if (half >= 2) {
        if (!cursor.next(&block)) return false;
        half = 0;
      }
      const int h = half++;
      if (block.col0 + h * kSubM >= block.limit) continue;
      *out = block;
      out->row = block.row + h * kSubM;
      out->col0 = block.col0 + h * kSubM;
      return true;
    }
  }
};

}  // namespace bd256

// The same work as launch_bwd_main_d256 with the two CTAs of a key block (the halves of the head dimension) running as
// a cluster that computes the scores once (bwd_d256_pair.cu). Without pivot gradients only.
int launch_bwd_main_d256_pair(const b200fa_bwd_args& a, const BwdParams& p, dim3 grid, float* dq_accum, int64_t stat_rows,
                              cudaStream_t stream);

}  // namespace b200fa
