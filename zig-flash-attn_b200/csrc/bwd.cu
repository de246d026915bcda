// Backward attention for sm_100a: preprocess, main dK/dV/dQ kernel, postprocess.
//
// Takes the place of the reference's flash_attn_bwd_preprocess (zig/flash_bwd_preprocess.zig:118-237), its sm_100
// main kernels (zig/flash_bwd_sm100.zig:31-1097) and flash_attn_bwd_postprocess (zig/flash_bwd_postprocess.zig:139-347).
//
// Main kernel: one CTA per (128-key block, kv head, sequence). It keeps the K and V tiles of its block in shared
// memory and walks every (query head of the group, 128-row query block) that can see the block (QueryCursor).
// Scores are computed transposed, keys on the 128 TMEM lanes and queries on the columns:
//   S^T  = K Q^T          SS-MMA  -> TMEM [0,128)            P^T  = exp2(S^T c - lse) (BF16, over S^T)
//   dP^T = V dO^T         SS-MMA  -> TMEM [128,256)          dS^T = P^T o (dP^T - D)  (BF16, to shared memory)
//   dV  += P^T dO         TS-MMA  -> TMEM [256,256+D)
//   dK  += dS^T Q         SS-MMA  -> TMEM [256+D,256+2D)
//   dQ   = dS K           SS-MMA  -> TMEM [128,128+D) (over dP^T), drained by the reduce warps into shared memory
//                                    and added into the FP32 dQ accumulator with TMA reduce-add.
// Warps 0-15 compute P and dS (four groups of four warps, 32 query columns each), warps 16-23 drain dQ (two groups, half
// of the columns each), warp 24 issues MMAs, warp 25 issues TMA loads and the asynchronous copies of the per-row
// statistics.
// Per iteration the MMA warp issues dV, S^T of the next iteration, then dQ before dK (the drain of dQ gates the next
// dP^T, which uses the same TMEM columns), then dP^T of the next iteration. The CTAs of a fixed-length problem are
// ordered by bwd_cta_of (bwd_common.cuh); packed problems take their (sequence, key block) from the work list.
#include <limits.h>

#include "bwd_common.cuh"

namespace b200fa {

#ifndef B200FA_BWD_GROUPS
#define B200FA_BWD_GROUPS 4
#endif
#ifndef B200FA_BWD_DRAINS
#define B200FA_BWD_DRAINS 2
#endif
template <int D>
struct BwdConfig {
  static constexpr int kTileBytes = 128 * D * 2;
  static constexpr int kPanelBytes = 128 * 128;
  static constexpr int kHalves = D / 64;
  static constexpr int kDsBytes = 128 * 128 * 2;
  static constexpr int kStageBytes = 128 * 32 * 4;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kOffK + kTileBytes;
  static constexpr int kOffQ = kOffV + kTileBytes;       // two stages
  static constexpr int kOffDo = kOffQ + 2 * kTileBytes;
  static constexpr int kOffDs = kOffDo + kTileBytes;
  static constexpr int kOffStage = kOffDs + kDsBytes;    // two staging buffers
  static constexpr int kOffStats = kOffStage + 2 * kStageBytes;  // lse[2][128], dpsum[2][128] floats
  static constexpr int kOffBars = kOffStats + 4 * 512;
  static constexpr int kSmemBytes = kOffBars + 128;
  // Compute warpgroups (P, dS): each thread handles one key row and 128 / kGroups query columns.
  // Four groups of 32 columns instead of two of 64 halve the latency of the P and dS phases, which sit on the serial
  // chain of an iteration (989 against 880 TF/s on batch 4, seqlen 8192, heads 32/8, causal).
  static constexpr int kGroups = B200FA_BWD_GROUPS;
  static constexpr int kCols = 128 / kGroups;
  static constexpr int kComputeWarps = 4 * kGroups;
  // Registers of the compute, drain and MMA/load warpgroups (setmaxnreg). They add up to the launch allocation:
  // 2 groups: 512 threads x 128 = 2 x 128 x 168 + 128 x 96 + 128 x 80; 4 groups and 1 drain group: 768 threads x 80 =
  // 4 x 128 x 88 + 128 x 72 + 128 x 56; 4 groups and 2 drain groups: 896 threads x 72 = 4 x 128 x 88 + 2 x 128 x 56 + 128 x 40.
  // dQ-drain warpgroups, each takes D / kDrains columns: with two the accumulator is released after one staging step
  // instead of three (1017 against 969 TF/s).
  static constexpr int kDrains = (kGroups == 4 && D == 128) ? B200FA_BWD_DRAINS : 1;  // head_dim 64 has two chunks only: 645 (one group) against 601 TF/s
  static constexpr int kRegsCompute = kGroups == 2 ? 168 : 88, kRegsDrain = kGroups == 2 ? 96 : (kDrains == 2 ? 56 : 72);
  static constexpr int kRegsMisc = kGroups == 2 ? 80 : (kDrains == 2 ? 40 : 56);
  static_assert(32 * (4 * kGroups + 4 * kDrains + 4) * (kGroups == 2 ? 128 : kDrains == 2 ? 72 : 80) ==
                    128 * (kGroups * kRegsCompute + kDrains * kRegsDrain + kRegsMisc),
                "the setmaxnreg budgets must add up to the launch allocation");
  static_assert(kGroups == 2 || kGroups == 4, "two or four compute warpgroups");
  static constexpr int kThreads = 32 * (kComputeWarps + 4 * kDrains + 4);  // + 1 dQ-drain warpgroup, 1 warpgroup with the MMA and load warps
  static constexpr int kTmemS = 0, kTmemDp = 128, kTmemDv = 256, kTmemDk = 256 + D;
};

template <int D, bool kPivot>
__global__ void __launch_bounds__(BwdConfig<D>::kThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
           const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ BwdParams p) {
  using Cfg = BwdConfig<D>;
  const Problem& pr = p.prob;
  // ---- work item (uniform over the CTA; exits before any barrier or TMEM allocation)
  int seq, n_block, kv_head;
  if (p.work_list) {
    const int2 e = p.work_list[blockIdx.x];
    seq = e.x;
    n_block = e.y;
    kv_head = blockIdx.y;
    if (seq >= pr.batch) return;
  } else {
    const BwdCta cta = bwd_cta_of(p, blockIdx.x);
    seq = cta.seq;
    n_block = cta.n_block;
    kv_head = cta.head_slot;
  }
  const SeqInfo s = seq_info(pr, seq);
  const int n0 = n_block * kBlockN;
  if (n0 >= s.lk) return;
  const int c1 = imin(n0 + kBlockN, s.lk);
  const int group = pr.heads_q / pr.heads_kv;
  const int64_t stat_base = pr.cu_q ? 0 : (int64_t)seq * pr.seqlen_q;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  if (base & 1023u) {  // the swizzled tiles need 1024-byte alignment; report instead of computing garbage
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (kWaitBwdLoad << 16) | 0xffff);
    return;
  }
  const uint32_t smem_k = base + Cfg::kOffK, smem_v = base + Cfg::kOffV, smem_q = base + Cfg::kOffQ;
  const uint32_t smem_do = base + Cfg::kOffDo, smem_ds = base + Cfg::kOffDs, smem_stage = base + Cfg::kOffStage;
  const uint32_t smem_lse = base + Cfg::kOffStats, smem_dpsum = smem_lse + 1024;
  const uint32_t bars = base + Cfg::kOffBars;
  const uint32_t bar_kv_full = bars, bar_q_full = bars + 8 /*[2]*/, bar_q_empty = bars + 24 /*[2]*/;
  const uint32_t bar_do_full = bars + 40, bar_s_full = bars + 56, bar_p_full = bars + 64;
  const uint32_t bar_dp_full = bars + 72, bar_ds_full = bars + 80, bar_dq_full = bars + 88, bar_dq_empty = bars + 96;
  const uint32_t bar_final = bars + 104, bar_ds_free = bars + 120;
  const uint32_t tmem_slot = bars + 112, abort_slot = bars + 116;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (abort_slot - smem_u32(smem_raw)));
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  const WaitCtx wctx{abort_flag, p.status, p.trace};
  int trace_n = 0;
  const bool traced_cta = kTraceBuild && n_block == 8 && kv_head == 0 && seq == 0;  // timeline of one CTA

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv_full, 1);
    mbar_init(bar_q_full, 33);
    mbar_init(bar_q_full + 8, 33);
    mbar_init(bar_q_empty, 1);
    mbar_init(bar_q_empty + 8, 1);
    mbar_init(bar_do_full, 33);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_p_full, 32 * Cfg::kComputeWarps);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_ds_full, 32 * Cfg::kComputeWarps);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_empty, 128 * Cfg::kDrains);
    mbar_init(bar_final, 1);
    mbar_init(bar_ds_free, 128 * Cfg::kDrains);
    fence_barrier_init();
  }
  constexpr int kMmaWarp = Cfg::kComputeWarps + 4 * Cfg::kDrains, kLoadWarp = kMmaWarp + 1;
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  const long long trace_start = trace_clock(WaitCtx{nullptr, nullptr, p.trace});
  // Query blocks per head (the same for every head of the group).
  int blocks_per_head = 0;
  {
    QueryCursor cur;
    cur.init(&pr, seq, s, n0, c1);
    OtherBlock qb;
    while (cur.next(&qb)) ++blocks_per_head;
  }
  const int iterations = blocks_per_head * group;

  // Register split (setmaxnreg, one site per warpgroup): see BwdConfig.
  if (warp >= kMmaWarp) {
   setmaxnreg_dec<Cfg::kRegsMisc>();
   if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ loads
    if (lane == 0) {
      tma_prefetch_descriptor(&map_q);
      tma_prefetch_descriptor(&map_do);
      if (iterations > 0) {
        mbar_expect_tx(bar_kv_full, 2 * Cfg::kTileBytes);
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) {
          tma_load_4d(smem_k + h * Cfg::kPanelBytes, &map_k, bar_kv_full, h * 64, kv_head, s.k0 + n0, s.batch_coord);
          tma_load_4d(smem_v + h * Cfg::kPanelBytes, &map_v, bar_kv_full, h * 64, kv_head, s.k0 + n0, s.batch_coord);
        }
      }
    }
    int it = 0;
    bool ok = true;
    for (int g = 0; ok && g < group; ++g) {
      const int head = kv_head * group + g;
      const float* lse_head = p.lse_log2 + (int64_t)head * p.rows;
      const float* dpsum_head = p.dpsum + (int64_t)head * p.rows;
      QueryCursor cur;
      cur.init(&pr, seq, s, n0, c1);
      OtherBlock qb;
      while (cur.next(&qb)) {
        const int st = it & 1;
        const int64_t row0 = stat_base + qb.row;
        if (!mbar_wait_traced(bar_q_empty + 8 * st, ((it >> 1) & 1) ^ 1, wctx, kWaitBwdLoad, 0, true)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(bar_q_full + 8 * st, Cfg::kTileBytes);
#pragma unroll
          for (int h = 0; h < Cfg::kHalves; ++h)
            tma_load_4d(smem_q + st * Cfg::kTileBytes + h * Cfg::kPanelBytes, &map_q, bar_q_full + 8 * st, h * 64, head,
                        qb.row, s.batch_coord);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int r = lane + 32 * k;
          if (row0 + r < p.rows) cp_async_4(smem_lse + st * 512 + r * 4, lse_head + row0 + r);
        }
        cp_async_arrive_noinc(bar_q_full + 8 * st);
        // The dO tile is free when dV(it - 1) has completed. The commit that announces S^T(it) was issued right after
        // those MMAs and covers them, so no barrier of its own is spent on it (a tcgen05.commit costs the MMA stream
        // about 90 cycles).
        // The wait runs in every iteration, the first included: a parity wait is only valid on a barrier whose earlier
        // completions the waiter has observed, and completion `it` is that of S^T(it), issued after dV(it - 1).
        if (!mbar_wait_traced(bar_s_full, it & 1, wctx, kWaitBwdLoad, 1, true)) { ok = false; break; }
        if (lane == 0) {
          trace_event(wctx, traced_cta && it < 10, 3, trace_n, 1000 + it);  // dO load issued
          mbar_expect_tx(bar_do_full, Cfg::kTileBytes);
#pragma unroll
          for (int h = 0; h < Cfg::kHalves; ++h)
            tma_load_4d(smem_do + h * Cfg::kPanelBytes, &map_do, bar_do_full, h * 64, head, qb.row, s.batch_coord);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int r = lane + 32 * k;
          if (row0 + r < p.rows) cp_async_4(smem_dpsum + st * 512 + r * 4, dpsum_head + row0 + r);
        }
        cp_async_arrive_noinc(bar_do_full);
        ++it;
      }
    }
   } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && iterations > 0) {
      constexpr uint32_t idesc_st = umma_idesc_bf16(128, 128, 0, 0);   // S^T, dP^T
      constexpr uint32_t idesc_dv = umma_idesc_bf16(128, D, 0, 1);     // dV: A in TMEM, B MN-major
      constexpr uint32_t idesc_dk = umma_idesc_bf16(128, D, 0, 1);     // dK: A K-major smem, B MN-major
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, D, 1, 1);     // dQ: A MN-major, B MN-major
      const uint32_t t_s = tmem_base + Cfg::kTmemS, t_dp = tmem_base + Cfg::kTmemDp;
      const uint32_t t_dv = tmem_base + Cfg::kTmemDv, t_dk = tmem_base + Cfg::kTmemDk;
      const int k_steps = (p.head_dim + 15) / 16;  // 16-column steps of the products over head_dim that hold data
      auto mma_kmajor = [&](uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem) {  // D = A B^T over head_dim
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk >= k_steps) break;  // head dims below the compiled width: the remaining columns are zero-filled
          const uint32_t off = (kk >> 2) * Cfg::kPanelBytes + (kk & 3) * 32;
          umma_ss(d_tmem, umma_smem_desc(a_smem + off, 16, 1024), umma_smem_desc(b_smem + off, 16, 1024), idesc_st, kk > 0);
        }
      };
      bool ok = mbar_wait(bar_kv_full, 0, wctx, kWaitBwdMma) && mbar_wait(bar_q_full, 0, wctx, kWaitBwdMma);
      if (ok) {
        tc_fence_after();
        mma_kmajor(t_s, smem_k, smem_q);
        tc_commit(bar_s_full);
        ok = mbar_wait(bar_do_full, 0, wctx, kWaitBwdMma);
      }
      if (ok) {
        tc_fence_after();
        mma_kmajor(t_dp, smem_v, smem_do);
        tc_commit(bar_dp_full);
      }
      for (int it = 0; ok && it < iterations; ++it) {
        const int st = it & 1;
        const uint32_t q_tile = smem_q + st * Cfg::kTileBytes;
        const bool more = it + 1 < iterations;
        // dV += P^T dO
        if (!mbar_wait_traced(bar_p_full, it & 1, wctx, kWaitBwdMma, 2, false)) { ok = false; break; }
        tc_fence_after();
        trace_event(wctx, traced_cta && it < 10, 0, trace_n, 50 + it);  // P(it) complete
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ts(t_dv, t_s + (Cfg::kGroups == 2 ? (kk >> 2) * 64 + (kk & 3) * 8 : (kk >> 1) * 32 + (kk & 1) * 8),
                  umma_smem_desc(smem_do + kk * 2048, Cfg::kPanelBytes, 1024), idesc_dv, it > 0 || kk > 0);
        trace_event(wctx, traced_cta && it < 10, 0, trace_n, 100 + it);  // dV issued
        // S^T of the next iteration
        if (more) {
          if (!mbar_wait_traced(bar_q_full + 8 * (st ^ 1), ((it + 1) >> 1) & 1, wctx, kWaitBwdMma, 3, false)) { ok = false; break; }
          tc_fence_after();
          mma_kmajor(t_s, smem_k, smem_q + (st ^ 1) * Cfg::kTileBytes);
          tc_commit(bar_s_full);
          trace_event(wctx, traced_cta && it < 10, 0, trace_n, 200 + it);  // S(it+1) issued
        }
        // dK += dS^T Q ; dQ = dS K
        if (!mbar_wait_traced(bar_ds_full, it & 1, wctx, kWaitBwdMma, 4, false)) { ok = false; break; }
        tc_fence_after();
        trace_event(wctx, traced_cta && it < 10, 0, trace_n, 250 + it);  // dS(it) complete
        auto issue_dq = [&]() {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(t_dp, umma_smem_desc(smem_ds + kk * 2048, Cfg::kPanelBytes, 1024),
                    umma_smem_desc(smem_k + kk * 2048, Cfg::kPanelBytes, 1024), idesc_dq, kk > 0);
          tc_commit(bar_dq_full);
        };
        auto issue_dk = [&]() {
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {
            const uint32_t a_off = (kk >> 2) * Cfg::kPanelBytes + (kk & 3) * 32;
            umma_ss(t_dk, umma_smem_desc(smem_ds + a_off, 16, 1024), umma_smem_desc(q_tile + kk * 2048, Cfg::kPanelBytes, 1024),
                    idesc_dk, it > 0 || kk > 0);
          }
          tc_commit(bar_q_empty + 8 * st);
        };
        // dQ first: its drain is on the chain to the next dP^T (same TMEM columns); dK runs while the drain does.
        issue_dq();
        issue_dk();
        trace_event(wctx, traced_cta && it < 10, 0, trace_n, 300 + it);  // dK, dQ issued
        // dP^T of the next iteration (its TMEM columns hold dQ until the reduce warps have drained it)
        if (more) {
          if (!mbar_wait_traced(bar_do_full, (it + 1) & 1, wctx, kWaitBwdMma, 5, false) ||
              !mbar_wait_traced(bar_dq_empty, it & 1, wctx, kWaitBwdMma, 6, false)) { ok = false; break; }
          tc_fence_after();
          trace_event(wctx, traced_cta && it < 10, 0, trace_n, 350 + it);  // dO(it+1) and dQ drain ready
          mma_kmajor(t_dp, smem_v, smem_do);
          tc_commit(bar_dp_full);
          trace_event(wctx, traced_cta && it < 10, 0, trace_n, 400 + it);  // dP(it+1) issued
        }
      }
      if (ok) tc_commit(bar_final);
    }
   }
  } else if (warp < Cfg::kComputeWarps) {
    setmaxnreg_inc<Cfg::kRegsCompute>();
    constexpr int C = Cfg::kCols;
    // ------------------------------------------------------------------ P and dS (thread = key row)
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int cb = wg * C;  // first query column of this group
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + Cfg::kTmemS, t_dp = tmem_base + lane_addr + Cfg::kTmemDp;
    const int c = n0 + r;  // key column within its sequence
    const bool key_valid = c < s.lk;
    int left, right;
    window_of(pr, seq, &left, &right);
    const int off = s.lk - s.lq;
    const uint32_t ds_row = smem_ds + (cb >> 6) * Cfg::kPanelBytes + r * 128;  // panel of 64 query columns
    const int ds_chunk0 = (cb & 63) >> 3;                                      // first 16-byte chunk within the row
    int it = 0;
    bool ok = true;
    for (int g = 0; ok && g < group; ++g) {
      QueryCursor cur;
      cur.init(&pr, seq, s, n0, c1);
      OtherBlock qb;
      while (cur.next(&qb)) {
        const int st = it & 1;
        int qlo = 0, qhi = qb.limit - qb.col0;
        if (qb.banded) {
          if (right >= 0) qlo = imax(0, c - off - right - qb.col0);
          if (left >= 0) qhi = imin(qhi, c - off + left + 1 - qb.col0);
        }
        if (!key_valid) qhi = 0;
        const bool masked = __any_sync(0xffffffffu, qlo > cb || qhi < cb + C);
        // ---- P^T (kept in FP32 registers for dS, stored to TMEM as BF16 for the dV MMA)
        if (!mbar_wait_traced(bar_s_full, it & 1, wctx, kWaitBwdCompute, 7, true)) { ok = false; break; }
        tc_fence_after();
        const long long t_p = trace_clock(wctx);
        trace_event(wctx, traced_cta && threadIdx.x == 0 && it < 10, 1, trace_n, 500 + it);  // S ready
        trace_event(wctx, traced_cta && threadIdx.x == 32 * Cfg::kComputeWarps - 32 && it < 10, 4, trace_n, 1500 + it);  // the same from the last compute warp
        float pf[C];
        tmem_ld32(t_s + cb, reinterpret_cast<uint32_t*>(pf));
        if constexpr (C == 64) tmem_ld32(t_s + cb + 32, reinterpret_cast<uint32_t*>(pf) + 32);
        tc_wait_ld();
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int j = 0; j < C / 4; ++j) {
          const float4 l4 = ld_shared_f4(smem_lse + st * 512 + (cb + 4 * j) * 4);  // -lse * log2(e)
          const float2 x01 = __ffma2_rn(make_float2(pf[4 * j + 0], pf[4 * j + 1]), scale2, make_float2(l4.x, l4.y));
          const float2 x23 = __ffma2_rn(make_float2(pf[4 * j + 2], pf[4 * j + 3]), scale2, make_float2(l4.z, l4.w));
          float p0 = ex2_approx(x01.x), p1 = ex2_approx(x01.y), p2 = ex2_approx(x23.x), p3 = ex2_approx(x23.y);
          if (masked) {
            const int q = cb + 4 * j;
            p0 = (q + 0 >= qlo && q + 0 < qhi) ? p0 : 0.f;
            p1 = (q + 1 >= qlo && q + 1 < qhi) ? p1 : 0.f;
            p2 = (q + 2 >= qlo && q + 2 < qhi) ? p2 : 0.f;
            p3 = (q + 3 >= qlo && q + 3 < qhi) ? p3 : 0.f;
          }
          pf[4 * j + 0] = p0;
          pf[4 * j + 1] = p1;
          pf[4 * j + 2] = p2;
          pf[4 * j + 3] = p3;
        }
        // P^T of a group goes over the first half of the group's own S^T columns.
#pragma unroll
        for (int h = 0; h < C / 32; ++h) {
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(pf[32 * h + 2 * i], pf[32 * h + 2 * i + 1]);
          tmem_st16(t_s + cb + 16 * h, pk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_full);
        // A probability above 3/4 is the pivot of its query row: dV keeps it (P^T is stored above), dS leaves it out
        // and the postprocess kernel forms it from the sum of the others. The branch is uniform over the warp and
        // almost never taken.
        if constexpr (kPivot) {
          // Necessary for a probability above 3/4 among the thread's C: their sum is above 3/4 (packed adds).
          float2 total = make_float2(pf[0], pf[1]);
#pragma unroll
          for (int j = 2; j < C; j += 2) total = __fadd2_rn(total, make_float2(pf[j], pf[j + 1]));
          if (__any_sync(0xffffffffu, total.x + total.y > kPivotProbability)) {
            const int head = kv_head * group + g;
            int* keys = p.pivot_key + (int64_t)head * p.rows + stat_base + qb.row + cb;
#pragma unroll
            for (int j = 0; j < C; ++j) {
              if (pf[j] > kPivotProbability) {
                keys[j] = s.k0 + c;
                pf[j] = 0.f;
              }
            }
          }
        }
        trace_add(wctx, 13, trace_clock(wctx) - t_p);
        trace_event(wctx, traced_cta && threadIdx.x == 0 && it < 10, 1, trace_n, 600 + it);  // P stored
        trace_event(wctx, traced_cta && threadIdx.x == 32 * Cfg::kComputeWarps - 32 && it < 10, 4, trace_n, 1600 + it);  // the same from the last compute warp
        // ---- dS^T = P^T o (dP^T - D), written to shared memory as BF16
        if (!mbar_wait_traced(bar_dp_full, it & 1, wctx, kWaitBwdCompute, 8, true)) { ok = false; break; }
        // The dS tile of the previous iteration must have been consumed by its dK and dQ MMAs.
        if (it > 0 && !mbar_wait_traced(bar_q_empty + 8 * ((it - 1) & 1), ((it - 1) >> 1) & 1, wctx, kWaitBwdCompute, 9, true)) { ok = false; break; }
        // ... and summed over its keys by the drain warps (pivot rows).
        if (kPivot && it > 0 && !mbar_wait_traced(bar_ds_free, (it - 1) & 1, wctx, kWaitBwdCompute, 16, true)) { ok = false; break; }
        tc_fence_after();
        const long long t_ds = trace_clock(wctx);
        trace_event(wctx, traced_cta && threadIdx.x == 0 && it < 10, 1, trace_n, 700 + it);  // dP ready
        trace_event(wctx, traced_cta && threadIdx.x == 32 * Cfg::kComputeWarps - 32 && it < 10, 4, trace_n, 1700 + it);  // the same from the last compute warp
#pragma unroll
        for (int h = 0; h < C / 32; ++h) {
          float dp[32];
          tmem_ld32(t_dp + cb + 32 * h, reinterpret_cast<uint32_t*>(dp));
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // 8 queries = one 16-byte chunk
            uint32_t packed[4];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int i = 8 * j + 4 * e;  // column within this half
              const float4 d4 = ld_shared_f4(smem_dpsum + st * 512 + (cb + 32 * h + i) * 4);  // -sum_d O dO
              const float2 s01 = __fmul2_rn(make_float2(pf[32 * h + i + 0], pf[32 * h + i + 1]),
                                            __fadd2_rn(make_float2(dp[i + 0], dp[i + 1]), make_float2(d4.x, d4.y)));
              const float2 s23 = __fmul2_rn(make_float2(pf[32 * h + i + 2], pf[32 * h + i + 3]),
                                            __fadd2_rn(make_float2(dp[i + 2], dp[i + 3]), make_float2(d4.z, d4.w)));
              float s0 = s01.x, s1 = s01.y, s2 = s23.x, s3 = s23.y;
              if (masked) {
                const int q = cb + 32 * h + i;
                s0 = (q + 0 >= qlo && q + 0 < qhi) ? s0 : 0.f;
                s1 = (q + 1 >= qlo && q + 1 < qhi) ? s1 : 0.f;
                s2 = (q + 2 >= qlo && q + 2 < qhi) ? s2 : 0.f;
                s3 = (q + 3 >= qlo && q + 3 < qhi) ? s3 : 0.f;
              }
              packed[2 * e] = pack_bf16x2(s0, s1);
              packed[2 * e + 1] = pack_bf16x2(s2, s3);
            }
            st_shared_v4(ds_row + (((ds_chunk0 + 4 * h + j) ^ (r & 7)) << 4), packed[0], packed[1], packed[2], packed[3]);
          }
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(bar_ds_full);
        trace_add(wctx, 14, trace_clock(wctx) - t_ds);
        trace_event(wctx, traced_cta && threadIdx.x == 0 && it < 10, 1, trace_n, 800 + it);  // dS stored
        trace_event(wctx, traced_cta && threadIdx.x == 32 * Cfg::kComputeWarps - 32 && it < 10, 4, trace_n, 1800 + it);  // the same from the last compute warp
        ++it;
      }
    }
    // ---- epilogue: group 0 writes dV, group 1 writes dK * scale
    if (ok) {
      const bool have = iterations > 0;
      if (have) ok = mbar_wait_warp(bar_final, 0, wctx, kWaitEpilogue);
      if (ok) {
        tc_fence_after();
        // The first half of the groups writes dV, the second half dK * scale; a group writes D / kParts columns.
        constexpr int kParts = Cfg::kGroups / 2;
        const bool is_dv = wg < kParts;
        const int part = is_dv ? wg : wg - kParts;
        __nv_bfloat16* out = is_dv ? p.dv : p.dk;
        const int64_t bs = is_dv ? p.dv_batch_stride : p.dk_batch_stride;
        const int64_t rs = is_dv ? p.dv_row_stride : p.dk_row_stride;
        const int64_t hs = is_dv ? p.dv_head_stride : p.dk_head_stride;
        const float mul = is_dv ? 1.f : p.scale;
        const uint32_t t_acc = tmem_base + lane_addr + (is_dv ? Cfg::kTmemDv : Cfg::kTmemDk);
        uint4* dst = reinterpret_cast<uint4*>(out + s.batch_coord * bs + (int64_t)(s.k0 + c) * rs + (int64_t)kv_head * hs);
#pragma unroll
        for (int ch0 = 0; ch0 < D / 32 / kParts; ++ch0) {
          const int ch = part * (D / 32 / kParts) + ch0;
          uint32_t acc[32];
          if (have) {
            tmem_ld32(t_acc + 32 * ch, acc);
            tc_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0;
          }
          if (key_valid && p.dkv_wide) {  // 32-byte stores: a lane writes whole sectors of its row
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                w[j] = pack_bf16x2(__uint_as_float(acc[16 * i + 2 * j]) * mul, __uint_as_float(acc[16 * i + 2 * j + 1]) * mul);
              if (32 * ch + 16 * i < p.head_dim) st_global_v8(dst + 4 * ch + 2 * i, w);
            }
          } else if (key_valid) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(acc[8 * i + 0]) * mul, __uint_as_float(acc[8 * i + 1]) * mul);
              v.y = pack_bf16x2(__uint_as_float(acc[8 * i + 2]) * mul, __uint_as_float(acc[8 * i + 3]) * mul);
              v.z = pack_bf16x2(__uint_as_float(acc[8 * i + 4]) * mul, __uint_as_float(acc[8 * i + 5]) * mul);
              v.w = pack_bf16x2(__uint_as_float(acc[8 * i + 6]) * mul, __uint_as_float(acc[8 * i + 7]) * mul);
              if (32 * ch + 8 * i < p.head_dim) dst[4 * ch + i] = v;
            }
          }
        }
        tc_fence_before();
      }
    }
  } else {
    setmaxnreg_dec<Cfg::kRegsDrain>();
    // ------------------------------------------------------------------ dQ drain (one warpgroup, thread = query row)
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_dq = tmem_base + lane_addr + Cfg::kTmemDp;
    // Drain warpgroup `dg` takes the columns [dg * D / kDrains, (dg + 1) * D / kDrains) of dQ; with two groups each has one
    // staging buffer of its own and the accumulator is released after one staging step instead of three.
    const int dg = (warp - Cfg::kComputeWarps) >> 2;
    const bool leader = (threadIdx.x & 127) == 0;
    constexpr int kChunks = D / 32 / Cfg::kDrains;
    int it = 0;
    uint32_t chunks = 0;
    bool ok = true;
    for (int g = 0; ok && g < group; ++g) {
      const int head = kv_head * group + g;
      QueryCursor cur;
      cur.init(&pr, seq, s, n0, c1);
      OtherBlock qb;
      while (cur.next(&qb)) {
        const int row0 = (int)(stat_base + qb.row);
        if (!mbar_wait_traced(bar_dq_full, it & 1, wctx, kWaitBwdReduce, 10, true)) { ok = false; break; }
        tc_fence_after();
        trace_event(wctx, traced_cta && leader && dg == 0 && it < 10, 2, trace_n, 9100 + it);  // dQ ready
#pragma unroll
        for (int c0 = 0; c0 < kChunks; ++c0) {
          const int ch = dg * kChunks + c0;
          uint32_t acc[32];
          tmem_ld32(t_dq + 32 * ch, acc);
          tc_wait_ld();
          if (c0 == kChunks - 1) {
            tc_fence_before();
            mbar_arrive(bar_dq_empty);
            trace_event(wctx, traced_cta && leader && dg == 0 && it < 10, 2, trace_n, 900 + it);  // dQ drained
          }
          const uint32_t stage = smem_stage + (Cfg::kDrains == 2 ? dg : (chunks & 1)) * Cfg::kStageBytes;
          if (leader) {  // the copy that last read this buffer is done with it
            if (Cfg::kDrains == 2) bulk_wait_group_read<0>(); else bulk_wait_group_read<1>();
          }
          named_barrier_sync(1 + dg, 128);
          trace_event(wctx, traced_cta && leader && dg == 0 && it < 10 && c0 == 0, 2, trace_n, 9400 + it);  // staging buffer free
          const uint32_t row_addr = stage + r * 128;
#pragma unroll
          for (int j = 0; j < 8; ++j)
            st_shared_v4(row_addr + ((j ^ (r & 7)) << 4), acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
          trace_event(wctx, traced_cta && leader && dg == 0 && it < 10 && c0 == 0, 2, trace_n, 9500 + it);  // stores issued
          fence_proxy_async_smem();
          named_barrier_sync(1 + dg, 128);
          if (leader) {
            tma_reduce_add_4d(&map_dq, stage, 32 * ch, head, row0, 0);
            bulk_commit_group();
            trace_event(wctx, traced_cta && dg == 0 && it < 10 && c0 == 0, 2, trace_n, 9300 + it);  // first chunk handed to the reduce-add
          }
          ++chunks;
        }
        // Sums of the BF16 dS over the 128 keys of the block, per query row, after the drain, off the chain dS -> dQ ->
        // drain -> next dP^T (placed before the drain they cost the kernel 10 %). Drain warp w takes
        // the 16-byte chunks (8 queries) c0 and c0 + 1 of the [key][query] tile: lane = (key row mod 16, chunk), eight
        // loads cover the 128 rows (a warp-wide load reads 16 rows x 32 bytes, 4 wavefronts of 128 bytes: no excess bank
        // conflicts under the tile's swizzle), FP32 adds in packed pairs, then a halving exchange over the 16 row lanes
        // leaves one query's sum per lane. (A warp-level mma.sync with an all-ones A costs 10 % of the kernel: it
        // costs the same.) The compute warps overwrite the tile only after bar_ds_free, which the drain warps arrive at below.
        if (kPivot && !mbar_wait_traced(bar_ds_full, it & 1, wctx, kWaitBwdReduce, 15, true)) { ok = false; break; }
        if constexpr (kPivot) {
          constexpr int kRounds = 8 / (4 * Cfg::kDrains);  // pairs of chunks per drain warp (16 chunks in all)
          const int drain_warp = warp - Cfg::kComputeWarps;
          const int sel = lane & 1, row_lane = lane >> 1;
          float sums[kRounds];
#pragma unroll
          for (int round = 0; round < kRounds; ++round) {
            const int chunk = 2 * (drain_warp * kRounds + round) + sel;  // queries [8 chunk, 8 chunk + 8)
            const uint32_t panel = smem_ds + (chunk >> 3) * Cfg::kPanelBytes;
            float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int key = 16 * i + row_lane;
              const float4 w = ld_shared_f4(panel + key * 128 + (((chunk & 7) ^ (key & 7)) << 4));
              const uint32_t words[4] = {__float_as_uint(w.x), __float_as_uint(w.y), __float_as_uint(w.z), __float_as_uint(w.w)};
#pragma unroll
              for (int j = 0; j < 4; ++j)
                acc[j] = __fadd2_rn(acc[j], make_float2(__uint_as_float(words[j] << 16), __uint_as_float(words[j] & 0xffff0000u)));
            }
            // Halving exchange over lane bits 4, 3, 2 (each step keeps one half of the values and adds the partner's),
            // then a plain exchange over bit 1: the lane ends with the sum of query 4 b4 + 2 b3 + b2 of its chunk.
            float v[8] = {acc[0].x, acc[0].y, acc[1].x, acc[1].y, acc[2].x, acc[2].y, acc[3].x, acc[3].y};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const bool upper = lane & 16;
              const float send = upper ? v[k] : v[k + 4], keep = upper ? v[k + 4] : v[k];
              v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
            }
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              const bool upper = lane & 8;
              const float send = upper ? v[k] : v[k + 2], keep = upper ? v[k + 2] : v[k];
              v[k] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
            }
            {
              const bool upper = lane & 4;
              const float send = upper ? v[0] : v[1], keep = upper ? v[1] : v[0];
              v[0] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
            }
            v[0] += __shfl_xor_sync(0xffffffffu, v[0], 2);
            sums[round] = v[0];
          }
          // The tile may be overwritten from here on. The arrive comes before the reductions: it has release
          // semantics, and behind them it would wait for their round trip to L2 (measured: 12 % of the kernel).
          mbar_arrive(bar_ds_free);
#pragma unroll
          for (int round = 0; round < kRounds; ++round) {
            const int chunk = 2 * (drain_warp * kRounds + round) + sel;
            const int q = 8 * chunk + ((lane >> 2) & 7);  // 4 b4 + 2 b3 + b2
            if ((lane & 2) == 0 && sums[round] != 0.f && row0 + q < p.rows)
              red_add_f32(p.pivot_sum + (int64_t)head * p.rows + row0 + q, sums[round] * kPivotSumScale);
          }
        }
        ++it;
      }
    }
    if (leader) bulk_wait_group<0>();
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, 512);
  if (kTraceBuild && threadIdx.x == 0) {
    trace_add(wctx, 11, trace_clock(wctx) - trace_start);
    trace_add(wctx, 12, iterations);
  }
}

// ---------------------------------------------------------------------------------------------- pre / post process
struct RowMap {
  const int32_t* cu_q;  // null = fixed length
  int batch, seqlen_q;
  int64_t rows;  // batch * seqlen_q or total_q
  int head_dim;  // columns of the tensors (the kernels are compiled for head_dim rounded up to 64 or 128)
};
// Maps a statistics row to (sequence, row within the sequence, batch coordinate, packed row).
__device__ __forceinline__ bool locate_row(const RowMap& m, int64_t row, int* batch_coord, int64_t* tensor_row) {
  if (m.cu_q) {
    if (row >= m.cu_q[m.batch]) return false;  // rows past the last sequence stay untouched
    *batch_coord = 0;
    *tensor_row = row;
  } else {
    *batch_coord = (int)(row / m.seqlen_q);
    *tensor_row = row - (int64_t)(*batch_coord) * m.seqlen_q;
  }
  return true;
}

// Both kernels below are HBM-bound streams. A lane handles 8 columns (16 bytes of BF16, 32 bytes of FP32), so a row of
// D columns takes D / 8 lanes and a warp handles 256 / D rows at once; a block of 256 threads covers kPrePostRows rows.
template <int D>
struct PrePost {
  static constexpr int kLanesPerRow = D / 8;
  static constexpr int kRowsPerWarp = 32 / kLanesPerRow;
  static constexpr int kRowsPerBlock = 8 * kRowsPerWarp;
};

// dpsum = -sum_d O dO, lse_log2 = -lse log2(e), dq_accum row = 0, no pivot yet (reference
// zig/flash_bwd_preprocess.zig:118-237).
template <int D>
__global__ void __launch_bounds__(256) bwd_preprocess_kernel(
    const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout, const float* __restrict__ lse,
    int64_t o_bs, int64_t o_rs, int64_t o_hs, int64_t do_bs, int64_t do_rs, int64_t do_hs, int64_t lse_bs, int64_t lse_hs,
    RowMap map, int heads, float* __restrict__ lse_log2, float* __restrict__ dpsum, float* __restrict__ dq_accum,
    float* __restrict__ pivot_sum, int* __restrict__ pivot_key) {
  using P = PrePost<D>;
  const int lane = threadIdx.x & 31;
  const int sub = lane % P::kLanesPerRow;  // 8-column group of the row
  const int64_t row = (int64_t)blockIdx.x * P::kRowsPerBlock + (threadIdx.x >> 5) * P::kRowsPerWarp + lane / P::kLanesPerRow;
  const int head = blockIdx.y;
  int batch_coord = 0;
  int64_t tensor_row = 0;
  const bool active = row < map.rows && locate_row(map, row, &batch_coord, &tensor_row);
  float sum = 0.f;
  if (active && sub * 8 < map.head_dim) {  // columns at and above head_dim are padding of the compiled width
    const uint4 a = *reinterpret_cast<const uint4*>(o + batch_coord * o_bs + tensor_row * o_rs + (int64_t)head * o_hs + sub * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(dout + batch_coord * do_bs + tensor_row * do_rs + (int64_t)head * do_hs + sub * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i)
      sum += __uint_as_float(aw[i] << 16) * __uint_as_float(bw[i] << 16) +
             __uint_as_float(aw[i] & 0xffff0000u) * __uint_as_float(bw[i] & 0xffff0000u);
  }
#pragma unroll
  for (int d = P::kLanesPerRow / 2; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
  if (!active) return;
  const int64_t stat = (int64_t)head * map.rows + row;
  if (sub == 0) {
    const float value = lse[batch_coord * lse_bs + (int64_t)head * lse_hs + tensor_row];
    lse_log2[stat] = value == -INFINITY ? -INFINITY : -value * kLog2e;  // rows without keys: exp2(x + -inf) = 0
    dpsum[stat] = -sum;
    pivot_sum[stat] = 0.f;
    pivot_key[stat] = -1;
  }
  float4* acc = reinterpret_cast<float4*>(dq_accum + stat * D + sub * 8);
  acc[0] = make_float4(0.f, 0.f, 0.f, 0.f);
  acc[1] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// The pivot terms that the postprocess kernel adds (all null / zero: none).
struct PivotFix {
  const float* pivot_sum;        // (heads_q, rows): kPivotSumScale x the sum of the BF16 dS of the other keys of the row
  const int* pivot_key;          // (heads_q, rows): tensor row of the pivot key, -1 = the row has none
  const __nv_bfloat16* q;        // query and key tensors, for the two products with the dS of the pivot
  const __nv_bfloat16* k;
  int64_t q_bs, q_rs, q_hs, k_bs, k_rs, k_hs;
  float* dk_fix;                 // (heads_kv, key rows, D) FP32, kDkFixScale x the pivot terms of dK, zeroed beforehand
  int* any_pivot;                // set to 1 when some row has a pivot
  int64_t key_rows;              // key rows per batch entry (seqlen_k), or of the packed tensor
  int group;                     // query heads per key head
};

// dq = bf16(scale * (dq_accum + dS_pivot * K[pivot])) for valid rows, and the pivot term dS_pivot * scale * Q[row] of
// dK into the FP32 side buffer (reference zig/flash_bwd_postprocess.zig:139-347). dS_pivot = -pivot_sum / kPivotSumScale:
// the dS of a row add up to zero, so the one the main kernel left out is minus the sum of the others, without the
// cancellation of P (dP - D) for P near 1 (reference zig/fragments.zig:23-30).
template <int D>
__global__ void __launch_bounds__(256) bwd_postprocess_kernel(const float* __restrict__ dq_accum, RowMap map, float scale,
                                                              __nv_bfloat16* __restrict__ dq, int64_t dq_bs,
                                                              int64_t dq_rs, int64_t dq_hs, PivotFix fix) {
  using P = PrePost<D>;
  const int lane = threadIdx.x & 31;
  const int sub = lane % P::kLanesPerRow;
  const int64_t row = (int64_t)blockIdx.x * P::kRowsPerBlock + (threadIdx.x >> 5) * P::kRowsPerWarp + lane / P::kLanesPerRow;
  const int head = blockIdx.y;
  if (row >= map.rows || sub * 8 >= map.head_dim) return;
  int batch_coord;
  int64_t tensor_row;
  if (!locate_row(map, row, &batch_coord, &tensor_row)) return;
  const int64_t stat = (int64_t)head * map.rows + row;
  const float4* acc = reinterpret_cast<const float4*>(dq_accum + stat * D + sub * 8);
  float4 v = acc[0], w = acc[1];
  const int key = fix.pivot_key ? fix.pivot_key[stat] : -1;
  if (key >= 0) {
    const float ds = fix.pivot_sum[stat] * (-1.f / kPivotSumScale);
    const int kv_head = head / fix.group;
    const uint4 kw = *reinterpret_cast<const uint4*>(fix.k + batch_coord * fix.k_bs + (int64_t)key * fix.k_rs +
                                                     (int64_t)kv_head * fix.k_hs + sub * 8);
    const uint4 qw = *reinterpret_cast<const uint4*>(fix.q + batch_coord * fix.q_bs + tensor_row * fix.q_rs +
                                                     (int64_t)head * fix.q_hs + sub * 8);
    const uint32_t kk[4] = {kw.x, kw.y, kw.z, kw.w}, qq[4] = {qw.x, qw.y, qw.z, qw.w};
    float dqv[8] = {v.x, v.y, v.z, v.w, w.x, w.y, w.z, w.w};
    float* side = fix.dk_fix + (((int64_t)kv_head * (map.cu_q ? 1 : map.batch) + batch_coord) * fix.key_rows + key) * D + sub * 8;
    const float ds_scaled = ds * kDkFixScale;  // exact: a power of two, and the product stays normal
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float k_lo = __uint_as_float(kk[i] << 16), k_hi = __uint_as_float(kk[i] & 0xffff0000u);
      const float q_lo = __uint_as_float(qq[i] << 16), q_hi = __uint_as_float(qq[i] & 0xffff0000u);
      dqv[2 * i] = fmaf(ds, k_lo, dqv[2 * i]);
      dqv[2 * i + 1] = fmaf(ds, k_hi, dqv[2 * i + 1]);
      const float t_lo = ds_scaled * (scale * q_lo), t_hi = ds_scaled * (scale * q_hi);
      if (t_lo != 0.f) red_add_f32(side + 2 * i, t_lo);
      if (t_hi != 0.f) red_add_f32(side + 2 * i + 1, t_hi);
    }
    v = make_float4(dqv[0], dqv[1], dqv[2], dqv[3]);
    w = make_float4(dqv[4], dqv[5], dqv[6], dqv[7]);
    if (sub == 0) *fix.any_pivot = 1;
  }
  uint4 packed;
  packed.x = pack_bf16x2(v.x * scale, v.y * scale);
  packed.y = pack_bf16x2(v.z * scale, v.w * scale);
  packed.z = pack_bf16x2(w.x * scale, w.y * scale);
  packed.w = pack_bf16x2(w.z * scale, w.w * scale);
  *reinterpret_cast<uint4*>(dq + batch_coord * dq_bs + tensor_row * dq_rs + (int64_t)head * dq_hs + sub * 8) = packed;
}

// dk += the pivot terms gathered by the postprocess kernel (reference zig/flash_bwd_postprocess.zig:349-397): the main
// kernel wrote dk without them, rounded to BF16; keys without a term stay untouched. The whole kernel is a no-op when
// no row had a pivot.
template <int D>
__global__ void __launch_bounds__(256) bwd_fix_dk_kernel(const float* __restrict__ dk_fix, const int* __restrict__ any_pivot,
                                                         int64_t rows, int64_t key_rows, int heads_kv, int head_dim,
                                                         __nv_bfloat16* __restrict__ dk, int64_t dk_bs, int64_t dk_rs,
                                                         int64_t dk_hs) {
  if (*any_pivot == 0) return;
  constexpr int kLanes = D / 8;
  const int64_t items = rows * heads_kv * kLanes;  // rows = key rows of all batch entries
  for (int64_t item = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; item < items; item += (int64_t)gridDim.x * blockDim.x) {
    const int sub = (int)(item % kLanes);
    const int64_t flat = item / kLanes;  // kv_head * rows + row
    const int kv_head = (int)(flat / rows);
    const int64_t row = flat - (int64_t)kv_head * rows;
    if (sub * 8 >= head_dim) continue;
    const float4* src = reinterpret_cast<const float4*>(dk_fix + flat * D + sub * 8);
    const float4 a = src[0], b = src[1];
    if (a.x == 0.f && a.y == 0.f && a.z == 0.f && a.w == 0.f && b.x == 0.f && b.y == 0.f && b.z == 0.f && b.w == 0.f) continue;
    const int64_t batch_coord = row / key_rows, key = row - batch_coord * key_rows;
    uint4* dst = reinterpret_cast<uint4*>(dk + batch_coord * dk_bs + key * dk_rs + (int64_t)kv_head * dk_hs + sub * 8);
    const uint4 old = *dst;
    const float unscale = 1.f / kDkFixScale;
    uint4 packed;
    packed.x = pack_bf16x2(__uint_as_float(old.x << 16) + a.x * unscale, __uint_as_float(old.x & 0xffff0000u) + a.y * unscale);
    packed.y = pack_bf16x2(__uint_as_float(old.y << 16) + a.z * unscale, __uint_as_float(old.y & 0xffff0000u) + a.w * unscale);
    packed.z = pack_bf16x2(__uint_as_float(old.z << 16) + b.x * unscale, __uint_as_float(old.z & 0xffff0000u) + b.y * unscale);
    packed.w = pack_bf16x2(__uint_as_float(old.w << 16) + b.z * unscale, __uint_as_float(old.w & 0xffff0000u) + b.w * unscale);
    *dst = packed;
  }
}

// ---------------------------------------------------------------------------------------------- host side
static thread_local cudaEvent_t g_timing_events[4];
static thread_local bool g_timing_armed = false;

void arm_bwd_timing(void* const* events) {
  g_timing_armed = events != nullptr;
  for (int i = 0; i < 4 && events; ++i) g_timing_events[i] = static_cast<cudaEvent_t>(events[i]);
}
static void mark(int index, cudaStream_t stream) {
  if (g_timing_armed) cudaEventRecord(g_timing_events[index], stream);
}

struct BwdWorkspace {
  size_t lse_log2, dpsum, pivot_sum, pivot_key, dq_accum, dk_fix, dk_fix_bytes, work_list, total;
  int64_t rows, key_rows, entries;
};

static BwdWorkspace plan_workspace(const b200fa_problem& p) {
  BwdWorkspace w;
  const bool packed = p.cu_seqlens_q != nullptr;
  w.rows = packed ? (int64_t)p.seqlen_q : (int64_t)p.batch * p.seqlen_q;
  const size_t stat_bytes = ((size_t)p.heads_q * w.rows * 4 + 255) & ~size_t(255);
  w.lse_log2 = 0;
  w.dpsum = stat_bytes;
  w.pivot_sum = 2 * stat_bytes;
  w.pivot_key = 3 * stat_bytes;
  w.dq_accum = 4 * stat_bytes;
  const int compiled_dim = p.head_dim <= 64 ? 64 : p.head_dim <= 128 ? 128 : 256;  // the accumulator has the compiled width
  const size_t acc_bytes = ((size_t)p.heads_q * w.rows * compiled_dim * 4 + 255) & ~size_t(255);
  // Pivot terms of dK: 256 bytes that hold the "some row has a pivot" flag, then (heads_kv, key rows, compiled width)
  // FP32; one memset zeroes both.
  w.key_rows = packed ? (int64_t)p.seqlen_k : (int64_t)p.batch * p.seqlen_k;
  w.dk_fix = w.dq_accum + acc_bytes;
  w.dk_fix_bytes = 256 + (((size_t)p.heads_kv * w.key_rows * compiled_dim * 4 + 255) & ~size_t(255));
  w.work_list = w.dk_fix + w.dk_fix_bytes;
  w.entries = packed ? work_list_entries(p.seqlen_k, p.batch, kBlockN) : 0;
  w.total = w.work_list + (size_t)w.entries * 8;
  return w;
}

size_t bwd_workspace_bytes(const b200fa_problem& p) { return plan_workspace(p).total; }

template <int D>
static int launch_main(const b200fa_bwd_args& a, const BwdParams& p, dim3 grid, float* dq_accum, int64_t stat_rows,
                       cudaStream_t stream) {
  using Cfg = BwdConfig<D>;
  const b200fa_problem& bp = a.problem;
  const bool packed = bp.cu_seqlens_q != nullptr;
  const int64_t rows_q = bp.seqlen_q, rows_k = bp.seqlen_k;
  const int64_t tensor_batch = packed ? 1 : bp.batch;
  // A problem without query rows has nothing to load; its dK and dV are zero.
  const bool no_queries = rows_q == 0 || stat_rows == 0;
  CUtensorMap map_q, map_k, map_v, map_do, map_dq;
  int status;
  const void* q_base = no_queries ? a.k : a.q;
  const void* do_base = no_queries ? a.k : a.dout;
  const int64_t q_rows = no_queries ? 1 : rows_q;
  const int64_t qh = no_queries ? 1 : bp.heads_q;
  status = encode_tensor_map(&map_q, q_base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, bp.head_dim, qh, q_rows, tensor_batch,
                             no_queries ? D : a.q_stride[2], no_queries ? D : a.q_stride[1],
                             no_queries ? D : (packed ? q_rows * a.q_stride[1] : a.q_stride[0]), 64, kBlockM);
  if (status != B200FA_OK) return status;
  status = encode_tensor_map(&map_do, do_base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, bp.head_dim, qh, q_rows, tensor_batch,
                             no_queries ? D : a.dout_stride[2], no_queries ? D : a.dout_stride[1],
                             no_queries ? D : (packed ? q_rows * a.dout_stride[1] : a.dout_stride[0]), 64, kBlockM);
  if (status != B200FA_OK) return status;
  status = encode_tensor_map(&map_k, a.k, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, bp.head_dim, bp.heads_kv, rows_k, tensor_batch,
                             a.k_stride[2], a.k_stride[1], packed ? rows_k * a.k_stride[1] : a.k_stride[0], 64, kBlockN);
  if (status != B200FA_OK) return status;
  status = encode_tensor_map(&map_v, a.v, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, bp.head_dim, bp.heads_kv, rows_k, tensor_batch,
                             a.v_stride[2], a.v_stride[1], packed ? rows_k * a.v_stride[1] : a.v_stride[0], 64, kBlockN);
  if (status != B200FA_OK) return status;
  if (no_queries) {
    map_dq = map_q;
  } else {
    status = encode_tensor_map(&map_dq, dq_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, D, bp.heads_q, stat_rows, 1,
                               stat_rows * D, D, (int64_t)bp.heads_q * stat_rows * D, 32, kBlockM);
    if (status != B200FA_OK) return status;
  }

  if (p.pivot_key) {
    static bool attribute_set[64] = {false};
    status = set_dynamic_smem_once(reinterpret_cast<const void*>(&bwd_kernel<D, true>), Cfg::kSmemBytes, attribute_set);
    if (status != B200FA_OK) return status;
    bwd_kernel<D, true><<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map_q, map_k, map_v, map_do, map_dq, p);
  } else {
    static bool attribute_set[64] = {false};
    status = set_dynamic_smem_once(reinterpret_cast<const void*>(&bwd_kernel<D, false>), Cfg::kSmemBytes, attribute_set);
    if (status != B200FA_OK) return status;
    bwd_kernel<D, false><<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map_q, map_k, map_v, map_do, map_dq, p);
  }
  B200FA_CUDA_CHECK(cudaGetLastError());

  return B200FA_OK;
}

template <int D>
static int launch_bwd_d(const b200fa_bwd_args& a, cudaStream_t stream) {
  const b200fa_problem& bp = a.problem;
  const bool packed = bp.cu_seqlens_q != nullptr;
  const BwdWorkspace w = plan_workspace(bp);
  B200FA_REQUIRE(a.workspace_bytes >= w.total && (w.total == 0 || a.workspace), "backward workspace is too small: need %zu bytes",
                 w.total);
  B200FA_REQUIRE(reinterpret_cast<uintptr_t>(a.workspace) % 256 == 0, "backward workspace must be 256-byte aligned");
  if (bp.batch == 0) return B200FA_OK;
  const bool no_keys = bp.seqlen_k == 0;
  uint8_t* ws = static_cast<uint8_t*>(a.workspace);
  float* lse_log2 = reinterpret_cast<float*>(ws + w.lse_log2);
  float* dpsum = reinterpret_cast<float*>(ws + w.dpsum);
  float* dq_accum = reinterpret_cast<float*>(ws + w.dq_accum);
  float* pivot_sum = reinterpret_cast<float*>(ws + w.pivot_sum);
  int* pivot_key = reinterpret_cast<int*>(ws + w.pivot_key);
  // Pivot gradients: on request (b200fa_set_pivot_ds).
  const bool pivots = pivot_ds_enabled() && w.dk_fix_bytes > 0 && w.rows > 0 && w.key_rows > 0;
  int* any_pivot = reinterpret_cast<int*>(ws + w.dk_fix);
  float* dk_fix = reinterpret_cast<float*>(ws + w.dk_fix + 256);

  RowMap map{bp.cu_seqlens_q, bp.batch, bp.seqlen_q, w.rows, bp.head_dim};
  mark(0, stream);
  if (w.rows > 0) {
    dim3 grid((unsigned)((w.rows + PrePost<D>::kRowsPerBlock - 1) / PrePost<D>::kRowsPerBlock), (unsigned)bp.heads_q);
    bwd_preprocess_kernel<D><<<grid, 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(a.out), static_cast<const __nv_bfloat16*>(a.dout), a.softmax_lse,
        packed ? 0 : a.out_stride[0], a.out_stride[1], a.out_stride[2], packed ? 0 : a.dout_stride[0], a.dout_stride[1],
        a.dout_stride[2], packed ? 0 : a.lse_stride[0], a.lse_stride[1], map, bp.heads_q, lse_log2, dpsum, dq_accum,
        pivot_sum, pivot_key);
    B200FA_CUDA_CHECK(cudaGetLastError());
  }
  if (pivots) B200FA_CUDA_CHECK(cudaMemsetAsync(ws + w.dk_fix, 0, w.dk_fix_bytes, stream));

  BwdParams p;
  p.prob = to_problem(bp);
  p.scale = bp.softmax_scale;
  p.scale_log2 = bp.softmax_scale * kLog2e;
  p.lse_log2 = lse_log2;
  p.dpsum = dpsum;
  p.rows = w.rows;
  p.pivot_sum = pivots ? pivot_sum : nullptr;
  p.pivot_key = pivots ? pivot_key : nullptr;
  p.head_dim = bp.head_dim;
  p.dk = static_cast<__nv_bfloat16*>(a.dk);
  p.dv = static_cast<__nv_bfloat16*>(a.dv);
  p.dk_batch_stride = packed ? 0 : a.dk_stride[0];
  p.dk_row_stride = a.dk_stride[1];
  p.dk_head_stride = a.dk_stride[2];
  p.dv_batch_stride = packed ? 0 : a.dv_stride[0];
  p.dv_row_stride = a.dv_stride[1];
  p.dv_head_stride = a.dv_stride[2];
  // every dK and dV row starts on a 32-byte boundary and holds a whole number of 32-byte pieces
  p.dkv_wide = (reinterpret_cast<uintptr_t>(a.dk) & 31) == 0 && (reinterpret_cast<uintptr_t>(a.dv) & 31) == 0 &&
               (packed || (a.dk_stride[0] % 16 == 0 && a.dv_stride[0] % 16 == 0)) && a.dk_stride[1] % 16 == 0 &&
               a.dk_stride[2] % 16 == 0 && a.dv_stride[1] % 16 == 0 && a.dv_stride[2] % 16 == 0 && bp.head_dim % 16 == 0;
  p.work_list = nullptr;
  p.n_blocks = p.head_slots = p.section = 1;
  p.status = device_status_word();
  if (!p.status) return B200FA_ERR_CUDA;
  p.trace = trace_buffer();

  constexpr int kBwdSection = 4;  // (batch entry, head slot) pairs per section of the launch order
  constexpr unsigned kHeadSplit = D == 256 ? 2 : 1;  // the 256-column kernel runs one CTA per half of the head dimension
  dim3 grid;
  bool run_main = !no_keys;
  if (packed) {
    if (w.entries == 0) run_main = false;
  }
  if (run_main && packed) {
    const int32_t* other = bp.cu_visible_q ? bp.cu_visible_q : bp.cu_seqlens_q;
    int status = b200fa_work_list(bp.cu_seqlens_k, other, bp.batch, kBlockN, 0, (int32_t)w.entries,
                                  reinterpret_cast<int32_t*>(ws + w.work_list), stream);
    if (status != B200FA_OK) return status;
    p.work_list = reinterpret_cast<const int2*>(ws + w.work_list);
    grid = dim3((unsigned)w.entries, (unsigned)bp.heads_kv * kHeadSplit, 1);
  } else if (run_main) {
    p.n_blocks = ceil_div(bp.seqlen_k, kBlockN);
    p.head_slots = bp.heads_kv * kHeadSplit;
    const int64_t groups = (int64_t)p.head_slots * bp.batch;
    // Interleaving sections pays when the key blocks differ in weight (causal: the first block sees every query
    // block, the last one sees one): it shortens the tail of the launch by up to 20 %. When the weights are about
    // equal (no mask, a narrow window over a long sequence) there is no tail to fix and the CTAs of one head slot
    // sharing Q and dO tiles in L2 is worth more (measured: 6-15 % either way), so those launch head slot by head slot.
    const Band band = make_band(bp.seqlen_q, bp.seqlen_k, bp.window_left, bp.window_right);
    int64_t total_weight = 0, heaviest = 0;
    for (int nb = 0; nb < p.n_blocks; ++nb) {
      int first = 0, last = 0;
      const int c0 = nb * kBlockN, c1 = c0 + kBlockN < bp.seqlen_k ? c0 + kBlockN : bp.seqlen_k;
      band_query_block_range(band, bp.seqlen_q, c0, c1, &first, &last);
      const int64_t weight = last > first ? last - first : 0;
      total_weight += weight;
      heaviest = weight > heaviest ? weight : heaviest;
    }
    const bool uneven = 2 * heaviest * p.n_blocks >= 3 * total_weight;  // heaviest block >= 1.5 x the mean
    // Short sequences have few key blocks per (batch entry, head slot) pair, so a section of four pairs is a small
    // share of a wave and the launch ends in a long tail: wider sections there (measured on 16 384 causal tokens, heads
    // 16/4: seqlen 1024 502 -> 568 TF/s with 16 pairs, seqlen 2048 666 -> 758 with 8; from seqlen 4096 on four is best).
    const int64_t wide = p.n_blocks <= 8 ? 16 : p.n_blocks <= 16 ? 8 : kBwdSection;
    const int64_t wanted = uneven ? wide : 1;
    p.section = (int)(groups < wanted ? groups : wanted);
    B200FA_REQUIRE(groups * p.n_blocks < INT_MAX, "too many key blocks for one backward launch");
    grid = dim3((unsigned)(groups * p.n_blocks), 1, 1);
  }
  mark(1, stream);
  if (run_main) {
    int status;
    if constexpr (D == 256) {
      status = launch_bwd_main_d256(a, p, grid, dq_accum, w.rows, stream);
    } else {
      status = launch_main<D>(a, p, grid, dq_accum, w.rows, stream);
    }
    if (status != B200FA_OK) return status;
  }
  mark(2, stream);

  if (w.rows > 0) {
    dim3 post((unsigned)((w.rows + PrePost<D>::kRowsPerBlock - 1) / PrePost<D>::kRowsPerBlock), (unsigned)bp.heads_q);
    PivotFix fix{};
    if (pivots && run_main) {
      fix.pivot_sum = pivot_sum;
      fix.pivot_key = pivot_key;
      fix.q = static_cast<const __nv_bfloat16*>(a.q);
      fix.k = static_cast<const __nv_bfloat16*>(a.k);
      fix.q_bs = packed ? 0 : a.q_stride[0], fix.q_rs = a.q_stride[1], fix.q_hs = a.q_stride[2];
      fix.k_bs = packed ? 0 : a.k_stride[0], fix.k_rs = a.k_stride[1], fix.k_hs = a.k_stride[2];
      fix.dk_fix = dk_fix;
      fix.any_pivot = any_pivot;
      fix.key_rows = bp.seqlen_k;
      fix.group = bp.heads_q / bp.heads_kv;
    }
    bwd_postprocess_kernel<D><<<post, 256, 0, stream>>>(dq_accum, map, bp.softmax_scale, static_cast<__nv_bfloat16*>(a.dq),
                                                        packed ? 0 : a.dq_stride[0], a.dq_stride[1], a.dq_stride[2], fix);
    B200FA_CUDA_CHECK(cudaGetLastError());
    if (pivots && run_main) {
      const int64_t items = w.key_rows * bp.heads_kv * (D / 8);
      const unsigned blocks = (unsigned)(items / 256 + 1 < 148 * 8 ? items / 256 + 1 : 148 * 8);
      bwd_fix_dk_kernel<D><<<blocks, 256, 0, stream>>>(dk_fix, any_pivot, w.key_rows, bp.seqlen_k, bp.heads_kv, bp.head_dim,
                                                       p.dk, p.dk_batch_stride, p.dk_row_stride, p.dk_head_stride);
      B200FA_CUDA_CHECK(cudaGetLastError());
    }
  }
  mark(3, stream);
  g_timing_armed = false;
  return B200FA_OK;
}

int launch_bwd(const b200fa_bwd_args& a, cudaStream_t stream) {
  switch (a.problem.head_dim) {
    case 64:
      return launch_bwd_d<64>(a, stream);
    case 72:   // compiled for 128 columns; TMA zero-fills the missing ones and the epilogues skip them
    case 96:
    case 128:
      return launch_bwd_d<128>(a, stream);
    case 256:
      return launch_bwd_d<256>(a, stream);
    default:
      set_error("head_dim %d is not supported by the backward kernels (supported: 64, 72, 96, 128, 256)", a.problem.head_dim);
      return B200FA_ERR_UNSUPPORTED;
  }
}

}  // namespace b200fa
