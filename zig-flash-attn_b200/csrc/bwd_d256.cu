// Backward main kernel for head dimensions above 128 (compiled for 256 columns) on sm_100a.
//
// Covers the head_dim 256 case that the reference serves with two passes, flash_attn_bwd_sm100_dq
// (zig/flash_bwd_sm100_dq.zig:25-600) and flash_attn_bwd_sm100_dkdv (zig/flash_bwd_sm100_dkdv.zig:23-666). Here it is one
// pass: the accumulators of a 128-key block at 256 columns (dV and dK, 256 TMEM columns each) would fill the tensor
// memory on their own, so a CTA owns one HALF of the head dimension of its key block: it computes the full scores
// (reduction over all 256 columns) but accumulates only dV[:, half], dK[:, half] and dQ[:, half]. The two halves of
// a key block are separate CTAs (head slot = 2 * kv_head + half).
//
// Per iteration a CTA takes 64 query rows of one head (a 128-row block of the QueryCursor in two halves):
//   S^T  = K Q^T            SS-MMA 128x64x256   -> TMEM [0,64)        P^T  = exp2(S^T c - lse)  (BF16, over S^T)
//   dP^T = V dO^T           TS-MMA 128x64x256   -> TMEM [64,128)      dS^T = P^T o (dP^T - D)   (BF16, shared memory)
//   dV_h += P^T dO_h        TS-MMA 128x128x64   -> TMEM [128,256)
//   dK_h += dS^T Q_h        SS-MMA 128x128x64   -> TMEM [256,384)
//   dQ_h^T = K_h^T dS^T     SS-MMA 128x64x128   -> TMEM [64,128) (over dP^T): head-dim columns on the lanes, queries on
//                           the columns; the drain warps transpose it through shared memory and add it into the FP32
//                           dQ accumulator with TMA reduce-add.
// V of the key block lives in TMEM (128 columns of BF16 pairs, copied there once): dP^T = V dO^T then reads only dO from
// shared memory (a 128 x 64 x 16 MMA with both operands in shared memory needs 6 KB per 32 tensor cycles, more than
// the SM delivers), and the 64 KB that V would take hold a second Q / dO stage, so the loads of the next iteration
// and its S^T MMA overlap the current one.
// Shared memory: K of the block (64 KB), two stages of a Q and a dO tile (32 KB each), the dS tile, two 8 KB staging
// buffers.
// Warps 0-15 compute P and dS (four groups, 16 query columns each), warps 16-23 drain dQ (two groups, 32 query rows
// each), warp 24 issues MMAs, warp 25 issues the loads.
#include "bwd_d256_common.cuh"

#include <cstdlib>

namespace b200fa {
namespace bd256 {

constexpr int kOffK = 0;
constexpr int kOffQ = kOffK + kKvBytes;     // two stages of (Q tile, dO tile): Q0 dO0 Q1 dO1
constexpr int kStageStride = 2 * kQBytes;
constexpr int kOffVTemp = kOffQ + kStageStride;  // V lands in the second stage before it moves to TMEM
constexpr int kOffDs = kOffQ + 2 * kStageStride;
constexpr int kOffStage = kOffDs + kDsBytes;
constexpr int kOffStats = kOffStage + 2 * kStageBytes;  // lse[2][64], dpsum[2][64] floats
constexpr int kOffBars = kOffStats + 4 * 256;
constexpr int kSmemBytes = kOffBars + 192;
constexpr int kTmemS = 0, kTmemDp = 64, kTmemDv = 128, kTmemDk = 256, kTmemV = 384;
static_assert(kSmemBytes <= 232448, "shared memory of the head_dim 256 backward kernel exceeds the per-CTA limit");

template <bool kPivot>
__global__ void __launch_bounds__(kThreads, 1)
bwd_d256_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ BwdParams p) {
  const Problem& pr = p.prob;
  // ---- work item (uniform over the CTA; exits before any barrier or TMEM allocation)
  int seq, n_block, head_slot;
  if (p.work_list) {
    const int2 e = p.work_list[blockIdx.x];
    seq = e.x;
    n_block = e.y;
    head_slot = blockIdx.y;
    if (seq >= pr.batch) return;
  } else {
    const BwdCta cta = bwd_cta_of(p, blockIdx.x);
    seq = cta.seq;
    n_block = cta.n_block;
    head_slot = cta.head_slot;
  }
  const int kv_head = head_slot >> 1;
  const int dh = head_slot & 1;  // half of the head dimension owned by this CTA
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
  const uint32_t smem_k = base + kOffK, smem_v = base + kOffVTemp, smem_q = base + kOffQ, smem_do = base + kOffQ + kQBytes;
  const uint32_t smem_ds = base + kOffDs, smem_stage = base + kOffStage;
  const uint32_t smem_lse = base + kOffStats, smem_dpsum = smem_lse + 512;
  const uint32_t bars = base + kOffBars;
  const uint32_t bar_kv_full = bars, bar_s_full = bars + 8, bar_p_full = bars + 16, bar_dp_full = bars + 24;
  const uint32_t bar_ds_full = bars + 32, bar_dq_full = bars + 48, bar_dq_empty = bars + 56;
  const uint32_t bar_final = bars + 64, bar_v_ready = bars + 72;
  const uint32_t bar_q_full = bars + 80 /*[2]*/, bar_q_empty = bars + 96 /*[2]*/, bar_do_full = bars + 112 /*[2]*/;
  const uint32_t tmem_slot = bars + 144, abort_slot = bars + 148, bar_ds_free = bars + 152;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (abort_slot - base));
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - base));
  const WaitCtx wctx{abort_flag, p.status, nullptr};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_q_full + 8 * i, 33);
      mbar_init(bar_q_empty + 8 * i, 1);
      mbar_init(bar_do_full + 8 * i, 1);
    }
    mbar_init(bar_v_ready, 32 * kComputeWarps);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_p_full, 32 * kComputeWarps);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_ds_full, 32 * kComputeWarps);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq_empty, 128 * kDrains);
    mbar_init(bar_final, 1);
    mbar_init(bar_ds_free, 128 * kDrains);
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;

  // 64-row query blocks per head (the same for every head of the group).
  int blocks_per_head = 0;
  {
    HalfBlockCursor cur;
    cur.init(&pr, seq, s, n0, c1);
    OtherBlock qb;
    while (cur.next(&qb)) ++blocks_per_head;
  }
  const int iterations = blocks_per_head * group;

  // Register split (setmaxnreg, one site per warpgroup): see kRegsCompute.
  if (warp >= kMmaWarp) {
   setmaxnreg_dec<kRegsMisc>();
   if (warp == kLoadWarp) {
    // ------------------------------------------------------------------ loads
    if (lane == 0) {
      tma_prefetch_descriptor(&map_q);
      tma_prefetch_descriptor(&map_do);
      if (iterations > 0) {
        mbar_expect_tx(bar_kv_full, 2 * kKvBytes);
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          tma_load_4d(smem_k + h * kKvPanel, &map_k, bar_kv_full, h * 64, kv_head, s.k0 + n0, s.batch_coord);
          tma_load_4d(smem_v + h * kKvPanel, &map_v, bar_kv_full, h * 64, kv_head, s.k0 + n0, s.batch_coord);
        }
      }
    }
    int it = 0;
    bool ok = true;
    for (int g = 0; ok && g < group; ++g) {
      const int head = kv_head * group + g;
      const float* lse_head = p.lse_log2 + (int64_t)head * p.rows;
      const float* dpsum_head = p.dpsum + (int64_t)head * p.rows;
      HalfBlockCursor cur;
      cur.init(&pr, seq, s, n0, c1);
      OtherBlock qb;
      while (cur.next(&qb)) {
        const int st = it & 1;
        const uint32_t phase = (it >> 1) & 1;
        const int64_t row0 = stat_base + qb.row;
        // The second stage holds V until the compute warps have moved it to TMEM.
        if (it == 1 && !mbar_wait(bar_v_ready, 0, wctx, kWaitBwdLoad)) { ok = false; break; }
        if (!mbar_wait(bar_q_empty + 8 * st, phase ^ 1, wctx, kWaitBwdLoad)) { ok = false; break; }
        if (lane == 0) {
          mbar_expect_tx(bar_q_full + 8 * st, kQBytes);
#pragma unroll
          for (int h = 0; h < 4; ++h)
            tma_load_4d(smem_q + st * kStageStride + h * kQPanel, &map_q, bar_q_full + 8 * st, h * 64, head, qb.row, s.batch_coord);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int r = lane + 32 * k;
          if (row0 + r < p.rows) {
            // Both row statistics travel with the Q tile: its stage is released by the dK MMA, which comes after the
            // dS phase has read them.
            cp_async_4(smem_lse + st * 256 + r * 4, lse_head + row0 + r);
            cp_async_4(smem_dpsum + st * 256 + r * 4, dpsum_head + row0 + r);
          }
        }
        cp_async_arrive_noinc(bar_q_full + 8 * st);
        // The dO tile of the stage is released with its Q tile (bar_q_empty, waited for above): one commit for both,
        // because every tcgen05.commit takes a slot of the MMA stream that bounds this kernel (one commit less per
        // iteration measured +4.5 %).
        if (lane == 0) {
          mbar_expect_tx(bar_do_full + 8 * st, kQBytes);
#pragma unroll
          for (int h = 0; h < 4; ++h)
            tma_load_4d(smem_do + st * kStageStride + h * kQPanel, &map_do, bar_do_full + 8 * st, h * 64, head, qb.row, s.batch_coord);
        }
        ++it;
      }
    }
   } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && iterations > 0) {
      constexpr uint32_t idesc_st = umma_idesc_bf16(128, kSubM, 0, 0);  // S^T, dP^T: both operands K-major
      constexpr uint32_t idesc_dv = umma_idesc_bf16(128, 128, 0, 1);    // dV: A in TMEM, B MN-major
      constexpr uint32_t idesc_dk = umma_idesc_bf16(128, 128, 0, 1);    // dK: A K-major, B MN-major
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, kSubM, 1, 1);  // dQ^T: A and B MN-major
      const uint32_t t_s = tmem_base + kTmemS, t_dp = tmem_base + kTmemDp;
      const uint32_t t_dv = tmem_base + kTmemDv, t_dk = tmem_base + kTmemDk;
      const uint32_t t_v = tmem_base + kTmemV;  // V of the key block as BF16, the A operand of dP^T
      const uint32_t k_half = smem_k + 2 * dh * kKvPanel;
      // S^T = K Q^T over all 256 columns (both operands in shared memory)
      auto issue_s = [&](uint32_t q_tile) {
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * kKvPanel + (kk & 3) * 32;
          const uint32_t b_off = (kk >> 2) * kQPanel + (kk & 3) * 32;
          umma_ss(t_s, umma_smem_desc(smem_k + a_off, 16, 1024), umma_smem_desc(q_tile + b_off, 16, 1024), idesc_st, kk > 0);
        }
        tc_commit(bar_s_full);
      };
      // dP^T = V dO^T with V read from TMEM: only dO comes from shared memory (2 KB per 32 tensor cycles)
      auto issue_dp = [&](uint32_t do_tile) {
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          const uint32_t b_off = (kk >> 2) * kQPanel + (kk & 3) * 32;
          umma_ts(t_dp, t_v + kk * 8, umma_smem_desc(do_tile + b_off, 16, 1024), idesc_st, kk > 0);
        }
        tc_commit(bar_dp_full);
      };
      bool ok = mbar_wait(bar_kv_full, 0, wctx, kWaitBwdMma) && mbar_wait(bar_q_full, 0, wctx, kWaitBwdMma);
      if (ok) {
        tc_fence_after();
        issue_s(smem_q);
        ok = mbar_wait(bar_do_full, 0, wctx, kWaitBwdMma) && mbar_wait(bar_v_ready, 0, wctx, kWaitBwdMma);
      }
      if (ok) {
        tc_fence_after();
        issue_dp(smem_do);
      }
      for (int it = 0; ok && it < iterations; ++it) {
        const int st = it & 1;
        const uint32_t phase = (it >> 1) & 1;
        const uint32_t q_tile = smem_q + st * kStageStride, do_tile = smem_do + st * kStageStride;
        const uint32_t q_half = q_tile + 2 * dh * kQPanel, do_half = do_tile + 2 * dh * kQPanel;
        const bool more = it + 1 < iterations;
        // dV_h += P^T dO_h
        if (!mbar_wait(bar_p_full, it & 1, wctx, kWaitBwdMma)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ts(t_dv, t_s + kk * kCols, umma_smem_desc(do_half + kk * 2048, kQPanel, 1024), idesc_dv,
                  it > 0 || kk > 0);
        // S^T of the next iteration (P^T of this one has been consumed by the MMAs above, which run first)
        if (more) {
          if (!mbar_wait(bar_q_full + 8 * (st ^ 1), ((it + 1) >> 1) & 1, wctx, kWaitBwdMma)) { ok = false; break; }
          tc_fence_after();
          issue_s(smem_q + (st ^ 1) * kStageStride);
        }
        // dQ_h^T = K_h^T dS^T first (its drain gates the next dP^T), then dK_h += dS^T Q_h
        if (!mbar_wait(bar_ds_full, it & 1, wctx, kWaitBwdMma)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma_ss(t_dp, umma_smem_desc(k_half + kk * 2048, kKvPanel, 1024), umma_smem_desc(smem_ds + kk * 2048, kDsBytes, 1024),
                  idesc_dq, kk > 0);
        tc_commit(bar_dq_full);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_ss(t_dk, umma_smem_desc(smem_ds + kk * 32, 16, 1024), umma_smem_desc(q_half + kk * 2048, kQPanel, 1024), idesc_dk,
                  it > 0 || kk > 0);
        tc_commit(bar_q_empty + 8 * st);
        (void)phase;
        // dP^T of the next iteration (its TMEM columns hold dQ^T until the drain warps have read it)
        if (more) {
          if (!mbar_wait(bar_do_full + 8 * (st ^ 1), ((it + 1) >> 1) & 1, wctx, kWaitBwdMma) ||
              !mbar_wait(bar_dq_empty, it & 1, wctx, kWaitBwdMma)) { ok = false; break; }
          tc_fence_after();
          issue_dp(smem_do + (st ^ 1) * kStageStride);
        }
      }
      if (ok) tc_commit(bar_final);
    }
   }
  } else if (warp < kComputeWarps) {
    setmaxnreg_inc<kRegsCompute>();
    // ------------------------------------------------------------------ P and dS (thread = key row)
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int cb = wg * kCols;  // first query column of this group (16 columns = one k-step of the dV MMA)
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + kTmemS, t_dp = tmem_base + lane_addr + kTmemDp;
    const int c = n0 + r;  // key column within its sequence
    const bool key_valid = c < s.lk;
    int left, right;
    window_of(pr, seq, &left, &right);
    const int off = s.lk - s.lq;
    const uint32_t ds_row = smem_ds + r * 128;
    int it = 0;
    bool ok = true;
    if (iterations > 0) {
      // V of the key block moves from its landing place in shared memory to TMEM (BF16 pairs, key row on the lane), where
      // it is the A operand of every dP^T MMA; the shared memory becomes the second Q / dO stage. Group wg copies the
      // 64 columns of panel wg: eight 16-byte chunks per row, stored with the 128-byte swizzle of the TMA box.
      ok = mbar_wait_warp(bar_kv_full, 0, wctx, kWaitBwdCompute);
      if (ok) {
        uint32_t words[32];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const float4 chunk = ld_shared_f4(smem_v + wg * kKvPanel + r * 128 + ((ch ^ (r & 7)) << 4));
          words[4 * ch + 0] = __float_as_uint(chunk.x);
          words[4 * ch + 1] = __float_as_uint(chunk.y);
          words[4 * ch + 2] = __float_as_uint(chunk.z);
          words[4 * ch + 3] = __float_as_uint(chunk.w);
        }
        tmem_st32(tmem_base + lane_addr + kTmemV + 32 * wg, words);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_v_ready);
      }
    }
    for (int g = 0; ok && g < group; ++g) {
      HalfBlockCursor cur;
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
        const bool masked = __any_sync(0xffffffffu, qlo > cb || qhi < cb + kCols);
        // ---- P^T (kept in FP32 registers for dS, stored to TMEM as BF16 for the dV MMA)
        if (!mbar_wait(bar_s_full, it & 1, wctx, kWaitBwdCompute)) { ok = false; break; }
        tc_fence_after();
        float pf[kCols];
        tmem_ld16(t_s + cb, reinterpret_cast<uint32_t*>(pf));
        tc_wait_ld();
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int j = 0; j < kCols / 4; ++j) {
          const float4 l4 = ld_shared_f4(smem_lse + st * 256 + (cb + 4 * j) * 4);  // -lse * log2(e)
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
        {  // P^T of a group goes over the first half of the group's own S^T columns
          uint32_t pk[kCols / 2];
#pragma unroll
          for (int i = 0; i < kCols / 2; ++i) pk[i] = pack_bf16x2(pf[2 * i], pf[2 * i + 1]);
          tmem_st8(t_s + cb, pk);
        }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_full);
        // A probability above 3/4 is the pivot of its query row (see bwd.cu): dV keeps it, dS leaves it out. Both CTAs
        // of a key block (the two halves of the head dimension) compute the same scores; the first one records the key.
        if constexpr (kPivot) {
          float2 total = make_float2(pf[0], pf[1]);
#pragma unroll
          for (int j = 2; j < kCols; j += 2) total = __fadd2_rn(total, make_float2(pf[j], pf[j + 1]));
          if (__any_sync(0xffffffffu, total.x + total.y > kPivotProbability)) {
            const int head = kv_head * group + g;
            int* keys = p.pivot_key + (int64_t)head * p.rows + stat_base + qb.row + cb;
#pragma unroll
            for (int j = 0; j < kCols; ++j) {
              if (pf[j] > kPivotProbability) {
                if (dh == 0) keys[j] = s.k0 + c;
                pf[j] = 0.f;
              }
            }
          }
        }
        // ---- dS^T = P^T o (dP^T - D), written to shared memory as BF16
        if (!mbar_wait(bar_dp_full, it & 1, wctx, kWaitBwdCompute)) { ok = false; break; }
        // The dS tile of the previous iteration must have been consumed by its dK and dQ MMAs.
        // (announced by the commit that releases the Q stage of that iteration, issued after the same MMAs)
        if (it > 0 && !mbar_wait(bar_q_empty + 8 * ((it - 1) & 1), ((it - 1) >> 1) & 1, wctx, kWaitBwdCompute)) { ok = false; break; }
        // ... and summed over its keys by the drain warps (pivot rows).
        if (kPivot && it > 0 && !mbar_wait(bar_ds_free, (it - 1) & 1, wctx, kWaitBwdCompute)) { ok = false; break; }
        tc_fence_after();
        float dp[kCols];
        tmem_ld16(t_dp + cb, reinterpret_cast<uint32_t*>(dp));
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < kCols / 8; ++j) {  // 8 queries = one 16-byte chunk
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int i = 8 * j + 4 * e;
            const float4 d4 = ld_shared_f4(smem_dpsum + st * 256 + (cb + i) * 4);  // -sum_d O dO
            const float2 s01 = __fmul2_rn(make_float2(pf[i + 0], pf[i + 1]),
                                          __fadd2_rn(make_float2(dp[i + 0], dp[i + 1]), make_float2(d4.x, d4.y)));
            const float2 s23 = __fmul2_rn(make_float2(pf[i + 2], pf[i + 3]),
                                          __fadd2_rn(make_float2(dp[i + 2], dp[i + 3]), make_float2(d4.z, d4.w)));
            float s0 = s01.x, s1 = s01.y, s2 = s23.x, s3 = s23.y;
            if (masked) {
              const int q = cb + i;
              s0 = (q + 0 >= qlo && q + 0 < qhi) ? s0 : 0.f;
              s1 = (q + 1 >= qlo && q + 1 < qhi) ? s1 : 0.f;
              s2 = (q + 2 >= qlo && q + 2 < qhi) ? s2 : 0.f;
              s3 = (q + 3 >= qlo && q + 3 < qhi) ? s3 : 0.f;
            }
            packed[2 * e] = pack_bf16x2(s0, s1);
            packed[2 * e + 1] = pack_bf16x2(s2, s3);
          }
          st_shared_v4(ds_row + ((((cb >> 3) + j) ^ (r & 7)) << 4), packed[0], packed[1], packed[2], packed[3]);
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(bar_ds_full);
        ++it;
      }
    }
    // ---- epilogue
    if (ok) {
      const bool have = iterations > 0;
      if (have) ok = mbar_wait_warp(bar_final, 0, wctx, kWaitEpilogue);
      if (ok) {
        tc_fence_after();
        // groups 0 and 1 write the two 64-column halves of dV, groups 2 and 3 those of dK * scale
        const bool is_dv = wg < kGroups / 2;
        const int part = wg & 1;
        __nv_bfloat16* out = is_dv ? p.dv : p.dk;
        const int64_t bs = is_dv ? p.dv_batch_stride : p.dk_batch_stride;
        const int64_t rs = is_dv ? p.dv_row_stride : p.dk_row_stride;
        const int64_t hs = is_dv ? p.dv_head_stride : p.dk_head_stride;
        const float mul = is_dv ? 1.f : p.scale;
        const uint32_t t_acc = tmem_base + lane_addr + (is_dv ? kTmemDv : kTmemDk);
        uint4* dst = reinterpret_cast<uint4*>(out + s.batch_coord * bs + (int64_t)(s.k0 + c) * rs + (int64_t)kv_head * hs + dh * 128);
#pragma unroll
        for (int ch0 = 0; ch0 < 2; ++ch0) {
          const int ch = 2 * part + ch0;
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
              if (dh * 128 + 32 * ch + 16 * i < p.head_dim) st_global_v8(dst + 4 * ch + 2 * i, w);
            }
          } else if (key_valid) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack_bf16x2(__uint_as_float(acc[8 * i + 0]) * mul, __uint_as_float(acc[8 * i + 1]) * mul);
              v.y = pack_bf16x2(__uint_as_float(acc[8 * i + 2]) * mul, __uint_as_float(acc[8 * i + 3]) * mul);
              v.z = pack_bf16x2(__uint_as_float(acc[8 * i + 4]) * mul, __uint_as_float(acc[8 * i + 5]) * mul);
              v.w = pack_bf16x2(__uint_as_float(acc[8 * i + 6]) * mul, __uint_as_float(acc[8 * i + 7]) * mul);
              if (dh * 128 + 32 * ch + 8 * i < p.head_dim) dst[4 * ch + i] = v;
            }
          }
        }
        tc_fence_before();
      }
    }
  } else {
    setmaxnreg_dec<kRegsDrain>();
    // ------------------------------------------------------------------ dQ drain (two warpgroups, thread = head-dim column)
    // Drain group dg takes query rows [32 dg, 32 dg + 32) of every iteration in two chunks of 16 through its own
    // staging buffer.
    const int dg = (warp - kComputeWarps) >> 2;
    const int d = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_dq = tmem_base + lane_addr + kTmemDp + 2 * kStageRows * dg;
    const uint32_t stage = smem_stage + dg * kStageBytes;
    const bool leader = (warp & 3) == 0 && lane == 0;
    constexpr int kChunks = kSubM / kStageRows / kDrains;
    int it = 0;
    bool ok = true;
    for (int g = 0; ok && g < group; ++g) {
      const int head = kv_head * group + g;
      HalfBlockCursor cur;
      cur.init(&pr, seq, s, n0, c1);
      OtherBlock qb;
      while (cur.next(&qb)) {
        const int row0 = (int)(stat_base + qb.row) + 2 * kStageRows * dg;
        if (!mbar_wait(bar_dq_full, it & 1, wctx, kWaitBwdReduce)) { ok = false; break; }
        tc_fence_after();
        // All 32 query columns of this group leave TMEM at once, so the next dP^T MMA can start while they are staged.
        uint32_t acc[kChunks * kStageRows];
        static_assert(kChunks * kStageRows == 32, "the drain reads its TMEM columns with one 32-column load");
        tmem_ld32(t_dq, acc);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(bar_dq_empty);
#pragma unroll
        for (int ch = 0; ch < kChunks; ++ch) {
          if (leader) bulk_wait_group_read<0>();  // the copy that read the staging buffer last is done with it
          named_barrier_sync(1 + dg, 128);
          // Transpose: this thread holds column d of 16 query rows; the staging buffer is (query row, column) row-major.
#pragma unroll
          for (int i = 0; i < kStageRows; ++i)
            st_shared_f32(stage + i * 512 + d * 4, __uint_as_float(acc[kStageRows * ch + i]));
          fence_proxy_async_smem();
          named_barrier_sync(1 + dg, 128);
          if (leader) {
            tma_reduce_add_4d(&map_dq, stage, dh * 128, head, row0 + kStageRows * ch, 0);
            bulk_commit_group();
          }
        }
        // Sums of the BF16 dS over the 128 keys of the block for the 64 queries of the iteration, as in bwd.cu: the first
        // four drain warps take two 16-byte chunks (8 queries) each, lane = (key row mod 16, chunk). Only the CTA of the
        // first half of the head dimension adds them to pivot_sum (the other half holds the same scores).
        if constexpr (kPivot) {
          if (!mbar_wait(bar_ds_full, it & 1, wctx, kWaitBwdReduce)) { ok = false; break; }
          const int drain_warp = warp - kComputeWarps;
          float sum = 0.f;
          const int sel = lane & 1, row_lane = lane >> 1;
          const int chunk = 2 * (drain_warp & 3) + sel;  // queries [8 chunk, 8 chunk + 8)
          if (drain_warp < 4 && dh == 0) {
            float2 acc[4] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int key = 16 * i + row_lane;
              const float4 w = ld_shared_f4(smem_ds + key * 128 + ((chunk ^ (key & 7)) << 4));
              const uint32_t words[4] = {__float_as_uint(w.x), __float_as_uint(w.y), __float_as_uint(w.z), __float_as_uint(w.w)};
#pragma unroll
              for (int j = 0; j < 4; ++j)
                acc[j] = __fadd2_rn(acc[j], make_float2(__uint_as_float(words[j] << 16), __uint_as_float(words[j] & 0xffff0000u)));
            }
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
            sum = v[0] + __shfl_xor_sync(0xffffffffu, v[0], 2);
          }
          mbar_arrive(bar_ds_free);  // before the reductions: the arrive has release semantics
          const int64_t row = stat_base + qb.row + 8 * chunk + ((lane >> 2) & 7);
          if (drain_warp < 4 && dh == 0 && (lane & 2) == 0 && sum != 0.f && row < p.rows)
            red_add_f32(p.pivot_sum + (int64_t)head * p.rows + row, sum * kPivotSumScale);
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
}

}  // namespace bd256

int launch_bwd_main_d256(const b200fa_bwd_args& a, const BwdParams& p, dim3 grid, float* dq_accum, int64_t stat_rows,
                         cudaStream_t stream) {
  using namespace bd256;
  constexpr int D = 256;
  // B200FA_BWD_D256_PAIR=1 (read at the first call) runs the two halves of a key block as a cluster that computes the
  // scores once (bwd_d256_pair.cu), without pivot gradients. It measured 7-9 % slower than the independent CTAs of this
  // file on full-size problems, so it is not the default.
  static const bool paired = [] {
    const char* setting = std::getenv("B200FA_BWD_D256_PAIR");
    return setting != nullptr && setting[0] == '1';
  }();
  if (paired && !p.pivot_key) return launch_bwd_main_d256_pair(a, p, grid, dq_accum, stat_rows, stream);
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
                             no_queries ? D : (packed ? q_rows * a.q_stride[1] : a.q_stride[0]), 64, kSubM);
  if (status != B200FA_OK) return status;
  status = encode_tensor_map(&map_do, do_base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, bp.head_dim, qh, q_rows, tensor_batch,
                             no_queries ? D : a.dout_stride[2], no_queries ? D : a.dout_stride[1],
                             no_queries ? D : (packed ? q_rows * a.dout_stride[1] : a.dout_stride[0]), 64, kSubM);
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
    // Box of 128 columns x 16 rows without swizzle: the staging buffers are plain row-major.
    status = encode_tensor_map(&map_dq, dq_accum, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, D, bp.heads_q, stat_rows, 1,
                               stat_rows * D, D, (int64_t)bp.heads_q * stat_rows * D, 128, kStageRows);
    if (status != B200FA_OK) return status;
  }
  if (p.pivot_key) {  // pivot gradients requested (b200fa_set_pivot_ds)
    static bool attribute_set[64] = {false};
    status = set_dynamic_smem_once(reinterpret_cast<const void*>(&bwd_d256_kernel<true>), kSmemBytes, attribute_set);
    if (status != B200FA_OK) return status;
    bwd_d256_kernel<true><<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, map_do, map_dq, p);
  } else {
    static bool attribute_set[64] = {false};
    status = set_dynamic_smem_once(reinterpret_cast<const void*>(&bwd_d256_kernel<false>), kSmemBytes, attribute_set);
    if (status != B200FA_OK) return status;
    bwd_d256_kernel<false><<<grid, kThreads, kSmemBytes, stream>>>(map_q, map_k, map_v, map_do, map_dq, p);
  }
  B200FA_CUDA_CHECK(cudaGetLastError());
  return B200FA_OK;
}

}  // namespace b200fa
