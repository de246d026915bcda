// Pieces shared by the forward kernels: kernel parameters, work-item decoding and the host-side set-up of both.
#pragma once
#include "common.h"
#include "ptx.cuh"

namespace b200fa {

// Division of a non-negative 31-bit number by a divisor that is fixed for a launch: quotient = umulhi(n, mul) >> shift
// (mul = ceil(2^(31 + ceil_log2 d) / d)), or n itself for d = 1. The work-item decode runs once per item in every warp of
// the forward kernels; four hardware divisions there are a visible part of the gap between two items.
struct FastDiv {
  uint32_t mul, shift, divisor;
  __host__ __device__ static FastDiv make(uint32_t d) {
    FastDiv f{0u, 0u, d ? d : 1u};
    if (f.divisor > 1u) {
      uint32_t log2 = 0;
      while ((1u << log2) < f.divisor) ++log2;
      const uint64_t power = 1ull << (31 + log2);
      f.mul = static_cast<uint32_t>((power + f.divisor - 1) / f.divisor);
      f.shift = log2 - 1;
    }
    return f;
  }
  __device__ __forceinline__ int div(int n) const {
    return divisor == 1u ? n : static_cast<int>(__umulhi(static_cast<uint32_t>(n), mul) >> shift);
  }
};

struct FwdParams {
  Problem prob;
  float scale_log2;
  __nv_bfloat16* o;
  int64_t o_batch_stride, o_row_stride, o_head_stride;
  float* lse;
  int64_t lse_batch_stride, lse_head_stride;
  int* tile_counter;      // zero at launch; the CTAs draw their work items from it (TileQueue)
  const int2* work_list;  // packed problems: (sequence, block) per entry; null for fixed length
  int m_blocks;           // fixed length: work items per (batch, head)
  // decode_tile: divisors fixed per launch (work items per key head, per query block, key heads, query heads) and the
  // query heads per key head
  FastDiv div_per_group, div_group, div_heads_kv, div_heads_q, div_ratio;
  int ratio;
  int num_tiles;
  int head_dim;           // columns of the tensors (<= the compiled width; TMA zero-fills the columns in between)
  int* status;            // device status word of the library
  long long* trace;       // optional cycle counters of tuning builds (slots 16-23), null = off
  // Split-KV (fwd.cu, short queries over long keys): a work item is (tile, share of the key blocks); every share writes
  // its normalised partial output and its log-sum-exp here and a second kernel merges them. splits == 1: off.
  int splits;
  float* o_partial;       // (splits, rows, heads_q, head_dim) fp32, rows = batch * seqlen_q
  float* lse_partial;     // (splits, heads_q, rows) fp32
  int64_t partial_rows;
  // Packed query heads (fwd.cu, fixed-length problems with a power-of-two number of query heads per key head): the rows
  // of a work item are (token, head of the group) pairs, row = token << pack_shift | head, so a work item covers
  // 256 >> pack_shift tokens of all heads of one key head. 0: a work item is 256 tokens of one head.
  int pack_shift;
  int o_wide;  // 1: the rows of the output may be written with 32-byte stores (alignment of base and strides)
};

// log2(1 + x) for 0 <= x < 1/16 from the series of ln(1 + x) up to x^6 (truncation error below 1e-9 relative).
__device__ __forceinline__ float log2p1_series(float x) {
  float series = -1.f / 6.f;
  series = fmaf(series, x, 1.f / 5.f);
  series = fmaf(series, x, -1.f / 4.f);
  series = fmaf(series, x, 1.f / 3.f);
  series = fmaf(series, x, -1.f / 2.f);
  series = fmaf(series, x, 1.f);
  return 1.4426950408889634f * (x * series);
}

// Per-row state of the keys that the online softmax sets aside (see row_totals below): `ones` keys, all scoring exactly
// `apart`, are kept out of the running sum. (Two registers: the softmax warps have none to spare, and a third one for
// the running maximum of the row cost the masked blocks of causal problems 4 %.)
struct TopApart {
  float apart = -INFINITY, ones = 0.f;
};

// Decides, from the maxima of two disjoint parts of a key block, whether this row sets the largest keys of the block
// aside: the block maximum is not below the score set aside so far, the part without it lies at least 2^3.9 below (necessary
// for a row whose largest term ends up more than 16 times the sum of the others), and that score is so close to zero
// that the sum of the others shows in the log-sum-exp at all (above 2^-7 in log2 units the rounding of m c + log2(sum)
// hides it). The parts are the even and the odd pairs of columns, so that a masked block (a causal diagonal) has visible
// keys in both as soon as the row sees more than two keys: with the lower and upper half of the columns as parts, the
// fully masked upper half of every diagonal block qualified and short causal sequences lost 10 %. Whether the keys
// set aside are the largest of the row needs no bookkeeping: a larger key elsewhere makes the rest exceed their term,
// and row_totals then takes the plain logarithm.
__device__ __forceinline__ bool sets_keys_apart(const TopApart& st, float part_a, float part_b, float scale_log2) {
  const float block_max = fmaxf(part_a, part_b);
  return block_max >= st.apart && fabsf(part_a - part_b) * scale_log2 > 3.9f && fabsf(block_max) * scale_log2 < 0.0078125f;
}

// The rare path of a block in which some row of the warp sets keys aside: sums the exponentials of the kColumns scores at
// TMEM address `t_s` (still intact: P is stored later) a second time, without the keys that score `block_max` when
// `set_apart` is true for this thread, which it counts in st.ones instead. Keys set aside earlier at a lower score are
// folded back into `l` first. A rolled loop over four columns at a time keeps the path small; `mc` is the reference
// maximum times scale_log2 that the block's exponentials use. Returns the sum that replaces the block sum.
template <int kColumns>
__device__ __forceinline__ float sum_without_keys_apart(TopApart& st, float& l, bool set_apart, float block_max,
                                                        uint32_t t_s, bool masked, int lo, int hi, float scale_log2,
                                                        float mc) {
  float apart_here = __int_as_float(0x7fc00000);  // NaN: no score equals it
  if (set_apart) {
    if (block_max > st.apart) {  // the keys set aside earlier are ordinary terms from now on
      if (st.ones > 0.f) l = fmaf(st.ones, ex2_approx(fmaf(st.apart, scale_log2, -mc)), l);
      st.ones = 0.f;
      st.apart = block_max;
    }
    apart_here = block_max;
  }
  const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-mc, -mc);
  float sum_even = 0.f, sum_odd = 0.f, ones = st.ones;
#pragma unroll 1
  for (int c = 0; c < kColumns; c += 4) {  // four columns per step: the path is rare, its code stays small
    float2 again[2];
    tmem_ld4(t_s + c, reinterpret_cast<uint32_t*>(again));
    tc_wait_ld();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float sx = (!masked || (c + 2 * i >= lo && c + 2 * i < hi)) ? again[i].x : -INFINITY;
      const float sy = (!masked || (c + 2 * i + 1 >= lo && c + 2 * i + 1 < hi)) ? again[i].y : -INFINITY;
      const float2 x = __ffma2_rn(make_float2(sx, sy), scale2, shift2);
      const float ex = ex2_approx(x.x), ey = ex2_approx(x.y);
      ones += (sx == apart_here ? 1.f : 0.f) + (sy == apart_here ? 1.f : 0.f);
      const float kept = (sx == apart_here ? 0.f : ex) + (sy == apart_here ? 0.f : ey);
      if (i & 1) sum_odd += kept; else sum_even += kept;
    }
  }
  st.ones = ones;
  return sum_even + sum_odd;
}

// End of a query row of the online softmax: the sum of the exponentials and the natural log-sum-exp.
//   m       lazy reference maximum of the row (-inf: the row saw no key), in score units
//   rest    sum of exp2(s c - m c) over the keys that were not set aside
//   ones    number of keys set aside, all of which score exactly `apart`
// The keys set aside contribute ones * exp2(apart c - m c). When the rest is below 1/16 of their term (they are then
// the largest keys of the row: a larger key would contribute more than the term itself), the logarithm is formed as apart c + log2(ones) + log2(1 + rest / term) with the series
// above: `rest` then keeps its relative accuracy, which the FP32 sum term + rest would round away (a row whose maximum
// score is exactly 0 over keys 17 to 80 nats below gets an LSE of about exp(-17) ... exp(-80), not 0). This is the
// accuracy contract of the reference's tie-counting LSE (zig/flash_fwd_sm100.zig:885-901, zig/fragments.zig:123-140,
// tests/test_softmax_fix.py:353-402); apart c is taken as the FP32 product plus its rounding remainder, as there.
__device__ __forceinline__ void row_totals(float m, float rest, float ones, float apart, float scale_log2,
                                           float* total, float* lse) {
  if (m == -INFINITY) {
    *total = 0.f;
    *lse = -INFINITY;
    return;
  }
  const float mc = m * scale_log2;
  float term = 0.f;
  if (ones > 0.f) term = ones * ex2_approx(fmaf(apart, scale_log2, -mc));
  const float sum = term + rest;
  float lse2 = mc + log2f(sum);
  if (ones > 0.f && rest < 0.0625f * term) {
    const float high = apart * scale_log2;
    const float low = fmaf(apart, scale_log2, -high);
    lse2 = high + (low + (ones > 1.f ? log2f(ones) : 0.f) + log2p1_series(rest / term));
  }
  *total = sum;
  *lse = sum > 0.f ? lse2 * 0.69314718055994531f : -INFINITY;
}

struct FwdTile {
  int seq, head, kv_head, m0;
  SeqInfo s;
  bool valid;
};

// Dynamic work distribution of the persistent kernels. One producer thread (the TMA warp) draws tile indices from a
// global counter and publishes them through a ring in shared memory; every other role pops them in the same order.
// A CTA that finishes a light tile early simply draws the next one, so the tail of a launch is as long as one tile,
// not as long as the imbalance of a static assignment (the reference's persistent kernels fetch tiles from an atomic
// counter as well, zig/tile_scheduler.zig:374-430).
struct TileQueue {
  static constexpr int kSlots = 4;
  static constexpr int kBytes = 4 * kSlots + 16 * kSlots;  // ring of tile indices, full and empty barriers
  uint32_t ring, bar_full, bar_empty;
  __device__ __forceinline__ void place(uint32_t smem) {
    bar_full = smem;
    bar_empty = smem + 8 * kSlots;
    ring = smem + 16 * kSlots;
  }
  // One thread, before the barriers are used; `consumers` = arrivals per pop round (one per consumer warp).
  __device__ __forceinline__ void init(int consumers) const {
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(bar_full + 8 * i, 1);
      mbar_init(bar_empty + 8 * i, consumers);
    }
  }
  // Producer thread: the next tile of this CTA, -1 when the launch has no more tiles, -2 when a wait ran out of time.
  __device__ __forceinline__ int push(uint32_t& n, int* counter, int num_tiles, const WaitCtx& ctx) const {
    const uint32_t slot = n % kSlots, phase = (n / kSlots) & 1;
    if (!mbar_wait(bar_empty + 8 * slot, phase ^ 1, ctx, kWaitTile)) return -2;
    int tile = atomicAdd(counter, 1);
    if (tile >= num_tiles) tile = -1;
    asm volatile("st.shared.b32 [%0], %1;" ::"r"(ring + 4 * slot), "r"(tile) : "memory");
    mbar_arrive(bar_full + 8 * slot);  // release: the store above is visible to whoever sees this phase complete
    ++n;
    return tile;
  }
  // Consumer, a single thread (the MMA issuer).
  __device__ __forceinline__ int pop_thread(uint32_t& n, const WaitCtx& ctx) const {
    const uint32_t slot = n % kSlots, phase = (n / kSlots) & 1;
    if (!mbar_wait(bar_full + 8 * slot, phase, ctx, kWaitTile)) return -2;
    int tile;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tile) : "r"(ring + 4 * slot) : "memory");
    mbar_arrive(bar_empty + 8 * slot);
    ++n;
    return tile;
  }
  // Consumer, all 32 lanes of a warp together (one arrival per warp).
  __device__ __forceinline__ int pop_warp(uint32_t& n, const WaitCtx& ctx) const {
    const uint32_t slot = n % kSlots, phase = (n / kSlots) & 1;
    if (!mbar_wait_warp(bar_full + 8 * slot, phase, ctx, kWaitTile)) return -2;
    int tile;
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(tile) : "r"(ring + 4 * slot) : "memory");
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar_empty + 8 * slot);
    ++n;
    return tile;
  }
};

// `tile_rows` = query rows per work item (256 for the two-stage kernel, 128 for the head_dim 256 kernel).
__device__ __forceinline__ FwdTile decode_tile(const FwdParams& p, int tile, int tile_rows = kFwdTileM) {
  FwdTile t;
  const Problem& pr = p.prob;
  if (p.work_list) {
    int entry = p.div_heads_q.div(tile);  // work items per entry: query heads, or key heads when groups are packed
    t.head = (tile - entry * (pr.heads_q >> p.pack_shift)) << p.pack_shift;  // packed: the first head of the group
    int2 e = p.work_list[entry];
    t.seq = e.x;
    t.m0 = e.y * (tile_rows >> p.pack_shift);
    t.valid = e.x < pr.batch;
  } else {
    // Work items that run at the same time share K and V: all query blocks and query heads of one (batch entry, key
    // head) are consecutive, late (heavy under a causal mask) query blocks first, so the K/V stream they read stays
    // in L2 (reference zig/tile_scheduler.zig:516-669 orders tiles in L2-sized sections for the same reason).
    const int group = p.pack_shift ? 1 : p.ratio;  // work items per query block and key head
    const int per_group = p.m_blocks * group;
    const int kv_group = p.div_per_group.div(tile);  // (batch entry, key head)
    const int rem = tile - kv_group * per_group;
    const int mb = p.div_group.div(rem);
    t.seq = p.div_heads_kv.div(kv_group);
    t.head = (kv_group - t.seq * pr.heads_kv) * p.ratio + (rem - mb * group);  // packed: the first head of the group
    t.m0 = (p.m_blocks - 1 - mb) * (tile_rows >> p.pack_shift);
    t.valid = true;
  }
  t.kv_head = p.div_ratio.div(t.head);
  if (t.valid) t.s = seq_info(pr, t.seq);
  return t;
}

// Fills the kernel parameters, builds the work list of a packed batch and encodes the Q / K / V tensor maps.
// `tile_rows` = query rows per work item, `kv_box_rows` = key rows per TMA box. Sets *nothing_to_do when no kernel is
// needed. Defined in fwd.cu.
int prepare_forward(const b200fa_fwd_args& a, cudaStream_t stream, int head_dim, int tile_rows, int kv_box_rows,
                    FwdParams* p, CUtensorMap* map_q, CUtensorMap* map_k, CUtensorMap* map_v, bool* nothing_to_do,
                    int v_box_rows = 0 /* rows per TMA box of V when they differ from those of K */,
                    int pack_shift = 0 /* log2 of the query heads packed into the rows of a work item */);
// A zeroed work-item counter for one launch on `stream`: the next slot of the device's ring of 4096 counters inside the
// library, reset by a memset node ahead of the kernel. Launches share a slot only 4096 launches apart (or through a
// captured graph, which keeps its slot); see the contract at its definition in fwd.cu.
int acquire_tile_counter(cudaStream_t stream, int** counter);
int launch_fwd_256(const b200fa_fwd_args& a, cudaStream_t stream);
int launch_fwd_256_pair(const b200fa_fwd_args& a, cudaStream_t stream);  // two-CTA variant (fwd_d256_pair.cu)
int launch_fwd_512(const b200fa_fwd_args& a, cudaStream_t stream);

}  // namespace b200fa
