// Shared pieces of the backward kernels: the parameter block, small shared-memory helpers and the launcher of the
// head_dim 256 main kernel (defined in bwd_d256.cu, called from bwd.cu).
#pragma once

#include "common.h"
#include "ptx.cuh"

namespace b200fa {

constexpr float kLog2e = 1.4426950408889634f;
// The reference's rule (zig/fragments.zig:23-30): a key with a probability above 3/4 is the pivot of its row.
constexpr float kPivotProbability = 0.75f;
// Row sums of BF16 dS are multiples of 2^-133; scaled by 2^7 every nonzero sum is a normal FP32 number, which the
// reductions (red.add.f32 flushes subnormal numbers) keep (reference zig/BackwardParams.zig:52-58).
constexpr float kPivotSumScale = 128.f;
// The pivot terms of dK are summed in FP32 by atomic adds, scaled by 2^40 for the same reason: a term as small as
// 2^-166 stays normal, sums up to 2^87 stay finite.
constexpr float kDkFixScale = 1099511627776.f;

struct BwdParams {
  Problem prob;
  float scale, scale_log2;
  const float* lse_log2;  // (heads_q, rows) : -lse * log2(e)
  const float* dpsum;     // (heads_q, rows) : -sum_d O * dO
  int64_t rows;           // rows of the statistics / dQ accumulator per head (batch * seqlen_q or total_q)
  // Pivot rows (at most one key of a query row holds more than 3/4 of its probability): the main kernel leaves the dS
  // of that key out, records the key in `pivot_key` (tensor row of K, -1 = none) and adds the BF16 dS of the other keys,
  // times kPivotSumScale, into `pivot_sum`; the postprocess kernel takes the dS of the pivot as minus that sum. Both are
  // (heads_q, rows). Null: pivot gradients are off (b200fa_set_pivot_ds).
  float* pivot_sum;
  int* pivot_key;
  int head_dim;           // columns of the tensors (<= the compiled D; TMA zero-fills the columns in between)
  int dkv_wide;           // 1: dK and dV rows may be written with 32-byte stores (alignment of bases and strides)
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  int64_t dk_batch_stride, dk_row_stride, dk_head_stride;
  int64_t dv_batch_stride, dv_row_stride, dv_head_stride;
  const int2* work_list;  // packed problems: (key sequence, key block) per blockIdx.x
  int n_blocks, head_slots, section;  // fixed length: decoding of the linear CTA index, see bwd_cta_of
  int* status;
  long long* trace;  // optional cycle counters, null = off
};

__device__ __forceinline__ void cp_async_4(uint32_t smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}

// Fixed-length problems launch a one-dimensional grid. CTAs start in index order, so the order decides both the tail of
// the launch and what runs together: a section of `section` (batch entry, head slot) pairs is walked key block by key
// block, first (under a causal mask: heaviest) key blocks first, then the next section. The CTAs that run together
// then read the Q, dO and dQ-accumulator rows of a few heads only, which stay in L2, and the light CTAs of a section
// fill the tail of its heavy ones.
struct BwdCta {
  int seq, n_block, head_slot;
};
__device__ __forceinline__ BwdCta bwd_cta_of(const BwdParams& p, int linear) {
  const int groups = p.prob.batch * p.head_slots;
  const int per_section = p.section * p.n_blocks;
  const int s = linear / per_section, r = linear - s * per_section;
  const int n = imin(p.section, groups - s * p.section);
  BwdCta c;
  c.n_block = r / n;
  const int g = s * p.section + (r - c.n_block * n);
  c.seq = g / p.head_slots;
  c.head_slot = g - c.seq * p.head_slots;
  return c;
}

// Main kernel for head_dim in (128, 256]: grid.y = 2 * heads_kv (kv head, half of the head dimension).
int launch_bwd_main_d256(const b200fa_bwd_args& a, const BwdParams& p, dim3 grid, float* dq_accum, int64_t stat_rows,
                         cudaStream_t stream);

}  // namespace b200fa
