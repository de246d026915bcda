// Backward main kernel for head_dim 256 on sm_100a as a cluster of two CTAs that computes the scores of a key block once.
//
// bwd_d256_kernel (bwd_d256.cu) gives each half of the head dimension of a 128-key block a CTA of its own, and both
// compute the full S^T and dP^T: 1.4 x the MMA work of the problem. Here the two CTAs form a cluster and take turns:
// iteration `it` (64 query rows of one head) is OWNED by the CTA of rank it & 1, which computes
//   S^T  = K Q^T            SS-MMA 128x64x256   -> TMEM [0,64)        P^T  = exp2(S^T c - lse)   (BF16)
//   dP^T = V dO^T           TS-MMA 128x64x256   -> TMEM [64,128)      dS^T = P^T o (dP^T - D)    (BF16)
// keeps P^T in TMEM and writes dS^T and P^T as BF16 tiles Y and X into its shared memory, from where bulk copies
// (cp.async.bulk shared::cta -> shared::cluster, completing on a barrier of the other CTA) put them into the tiles Yr
// and X of the other CTA. Every iteration both CTAs add their half:
//   dV_h += P^T dO_h        128x128x64 (the owner reads P^T from TMEM, the other CTA from its tile X)
//   dK_h += dS^T Q_h        128x128x64 (the owner reads dS^T from its tile Y, the other CTA from its tile Yr)
// and the owner alone computes dQ^T for BOTH halves of the head dimension (it holds all of K):
//   dQ_0^T = K_0^T dS^T -> TMEM [64,128) (over dP^T),   dQ_1^T = K_1^T dS^T -> TMEM [0,64) (over S^T / P^T)
// which its drain warps transpose through shared memory and add into the FP32 dQ accumulator with TMA reduce-add.
// The score regions of a CTA are used every other iteration only, so the chain S^T -> P^T -> dS^T -> dQ^T -> drain of one
// CTA runs beside that of the other, and a non-owned iteration needs only Q_h and dO_h (half of the loads).
// The reference serves head_dim 256 with two passes (zig/flash_bwd_sm100_dq.zig:25-600,
// zig/flash_bwd_sm100_dkdv.zig:23-666), both as clusters of two; this is one pass.
//
// Tile X of a CTA holds its own P^T on its iterations (only as the source of the copy) and the received one on the other
// CTA's iterations; dS^T has a tile for each direction, because the owner's dS^T write is on the chain that bounds an
// iteration and must not wait for the other CTA's tile to be consumed. A CTA copies into the other CTA's tiles only
// after it has received that CTA's previous tiles (their copy out is complete) and that CTA's MMAs have read what it
// received before (announced by a tcgen05.commit onto a barrier of this CTA). Scattered 16-byte stores into the other
// CTA's shared memory were measured first: 32 KB of them take about 3800 cycles and slow the MMAs of the receiving
// SM several times over.
//
// Shared memory: K (64 KB), stage A = Q and dO tiles of the owned iteration (64 KB; V lands here first and moves to
// TMEM), stage B = Q_h and dO_h of the other CTA's iteration (32 KB), X, Y and Yr (16 KB each), two 8 KB staging
// buffers.
// Warps 0-15 compute P and dS on owned iterations (four groups, 16 query columns each), warps 16-23 drain dQ (two
// groups, 32 query rows each), warp 24 issues MMAs, warp 25 issues the loads, warp 26 the copies between the CTAs.
// Every TMA load goes to the shared memory of the CTA that issues it; the only traffic between the CTAs is those bulk
// copies from shared memory to shared memory and one tcgen05.commit per iteration onto
// a barrier of the other CTA.
//
// Selected by B200FA_BWD_D256_PAIR=1 and not the default: with a third fewer MMA instructions per iteration it runs
// 7-9 % slower than bwd_d256_kernel on full-size problems (B4 S8192 heads 16/4 causal: 559 against 600-613 TF/s). Both
// kernels are bound by the rate at which one thread gets tcgen05 instructions through the tensor pipe (about 95-105
// cycles per MMA or commit of any N <= 128 inside these kernels); what the pair saves in instructions it gives back in
// the waits of the MMA thread between the two CTAs' phases and in the copies.
#include "bwd_d256_common.cuh"

namespace b200fa {
namespace bd256p {

using namespace bd256;

constexpr int kOffK = 0;
constexpr int kOffA = kOffK + kKvBytes;        // Q tile (32 KB), dO tile (32 KB) of the owned iteration; V at the start
constexpr int kOffB = kOffA + 2 * kQBytes;     // Q_h (16 KB), dO_h (16 KB) of the other CTA's iteration
constexpr int kHalfBytes = 2 * kQPanel;        // 64 query rows x 128 columns BF16
constexpr int kOffX = kOffB + 2 * kHalfBytes;  // P^T tile (own on owned iterations, received otherwise)
constexpr int kOffY = kOffX + kDsBytes;        // own dS^T tile
constexpr int kOffYr = kOffY + kDsBytes;       // received dS^T tile
constexpr int kOffStage = kOffYr + kDsBytes;
constexpr int kOffStats = kOffStage + 2 * kStageBytes;  // lse[64], dpsum[64] floats of the owned iteration
constexpr int kOffBars = kOffStats + 512;
constexpr int kSmemBytes = kOffBars + 192;
constexpr int kXferWarp = kLoadWarp + 1;
constexpr int kTmemS = 0, kTmemDp = 64, kTmemDv = 128, kTmemDk = 256, kTmemV = 384;
static_assert(kSmemBytes <= 232448, "shared memory of the paired head_dim 256 backward kernel exceeds the per-CTA limit");
static_assert(kOffB - kOffA == kKvBytes, "V lands in stage A before it moves to TMEM");

__global__ void __launch_bounds__(kThreads, 1)
bwd_d256_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                     const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                     const __grid_constant__ CUtensorMap map_dq, const __grid_constant__ BwdParams p) {
  const Problem& pr = p.prob;
  // ---- work item: the two CTAs of a cluster decode the same key block and key head and differ in the half of the head
  // dimension, so every early exit below is taken by both or by neither.
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
  const int dh = head_slot & 1;  // half of the head dimension owned by this CTA = its rank in the cluster
  const uint32_t rank = cluster_rank();
  const SeqInfo s = seq_info(pr, seq);
  const int n0 = n_block * kBlockN;
  if (n0 >= s.lk) return;
  const int c1 = imin(n0 + kBlockN, s.lk);
  const int group = pr.heads_q / pr.heads_kv;
  const int64_t stat_base = pr.cu_q ? 0 : (int64_t)seq * pr.seqlen_q;

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t smem_k = base + kOffK, smem_v = base + kOffA;
  const uint32_t smem_qa = base + kOffA, smem_doa = base + kOffA + kQBytes;
  const uint32_t smem_qb = base + kOffB, smem_dob = base + kOffB + kHalfBytes;
  const uint32_t smem_x = base + kOffX, smem_y = base + kOffY, smem_yr = base + kOffYr, smem_stage = base + kOffStage;
  const uint32_t smem_lse = base + kOffStats, smem_dpsum = smem_lse + 256;
  const uint32_t bars = base + kOffBars;
  const uint32_t bar_kv_full = bars, bar_v_ready = bars + 8;
  const uint32_t bar_qa_full = bars + 16, bar_qa_empty = bars + 24, bar_doa_full = bars + 32, bar_doa_empty = bars + 40;
  const uint32_t bar_qb_full = bars + 48, bar_qb_empty = bars + 56, bar_dob_full = bars + 64, bar_dob_empty = bars + 72;
  const uint32_t bar_s_full = bars + 80, bar_p_full = bars + 88, bar_dp_full = bars + 96, bar_ds_full = bars + 104;
  const uint32_t bar_dq_full = bars + 112 /* half 0 */, bar_dq1_full = bars + 176, bar_dq1_empty = bars + 120, bar_dq0_empty = bars + 128;
  const uint32_t bar_recv_full = bars + 136;   // the other CTA's P^T and dS^T have landed in this CTA's X and Y (32 KB)
  const uint32_t bar_may_send = bars + 144;    // the other CTA's MMAs have read its own dS^T: its tiles may be overwritten
  const uint32_t bar_final = bars + 152, bar_x_full = bars + 160;
  const uint32_t tmem_slot = bars + 168, abort_slot = bars + 172;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (abort_slot - base));
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - base));
  const WaitCtx wctx{abort_flag, p.status, p.trace};

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // The swizzled tiles need 1024-byte alignment and the rank must be the half of the head dimension. Both conditions are
  // the same in the two CTAs (same kernel, same launch), so a CTA that leaves here leaves with its partner.
  const bool usable = (base & 1023u) == 0 && rank == (uint32_t)dh;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_kv_full, 1);
    mbar_init(bar_v_ready, 32 * kComputeWarps);
    mbar_init(bar_qa_full, 33);
    mbar_init(bar_qa_empty, 1);
    mbar_init(bar_doa_full, 1);
    mbar_init(bar_doa_empty, 1);
    mbar_init(bar_qb_full, 1);
    mbar_init(bar_qb_empty, 1);
    mbar_init(bar_dob_full, 1);
    mbar_init(bar_dob_empty, 1);
    mbar_init(bar_s_full, 1);
    mbar_init(bar_p_full, 32 * kComputeWarps);
    mbar_init(bar_dp_full, 1);
    mbar_init(bar_ds_full, 32 * kComputeWarps);
    mbar_init(bar_dq_full, 1);
    mbar_init(bar_dq1_full, 1);
    mbar_init(bar_dq1_empty, 128 * kDrains);
    mbar_init(bar_dq0_empty, 128 * kDrains);
    mbar_init(bar_recv_full, 1);
    mbar_init(bar_may_send, 1);
    mbar_init(bar_x_full, 32 * kComputeWarps);
    mbar_init(bar_final, 1);
    fence_barrier_init();
  }
  if (warp == kMmaWarp && usable) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();  // the barriers of both CTAs exist before anything crosses between them
  if (!usable) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, (kWaitBwdLoad << 16) | 0xffff);
    return;
  }
  const uint32_t tmem_base = *tmem_ptr_smem;
  const uint32_t peer = rank ^ 1u;
  // Tuning builds: timeline of the first cluster (roles 0-2: MMA thread, first compute thread and a drain leader of rank
  // 0; roles 3-4: MMA thread and first compute thread of rank 1).
  const bool traced = blockIdx.x < 2 && blockIdx.y < 2 && (threadIdx.x & 127) == 0;
  int trace_n = 0;

  // 64-row query blocks per head (the same for every head of the group).
  int blocks_per_head = 0;
  {
    HalfBlockCursor cur;
    cur.init(&pr, seq, s, n0, c1);
    OtherBlock qb;
    while (cur.next(&qb)) ++blocks_per_head;
  }
  const int iterations = blocks_per_head * group;
  // Iteration `it` is owned by rank it & 1; k = it >> 1 counts the owned and the other iterations of a CTA alike, so
  // every barrier completes once per k and its phase parity is k & 1.

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
        const uint32_t phase = (it >> 1) & 1;
        if ((it & 1) == dh) {
          const int64_t row0 = stat_base + qb.row;
          // Stage A holds V until the compute warps have moved it to TMEM.
          if (it < 2 && !mbar_wait(bar_v_ready, 0, wctx, kWaitBwdLoad)) { ok = false; break; }
          if (!mbar_wait(bar_qa_empty, phase ^ 1, wctx, kWaitBwdLoad)) { ok = false; break; }
          if (lane == 0) {
            mbar_expect_tx(bar_qa_full, kQBytes);
#pragma unroll
            for (int h = 0; h < 4; ++h)
              tma_load_4d(smem_qa + h * kQPanel, &map_q, bar_qa_full, h * 64, head, qb.row, s.batch_coord);
          }
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const int r = lane + 32 * k;
            if (row0 + r < p.rows) {
              // Both row statistics travel with the Q tile: its stage is released by the dK MMA, which comes after the
              // dS phase has read them (the dO stage is released earlier, by the dV MMA).
              cp_async_4(smem_lse + r * 4, lse_head + row0 + r);
              cp_async_4(smem_dpsum + r * 4, dpsum_head + row0 + r);
            }
          }
          cp_async_arrive_noinc(bar_qa_full);
          if (!mbar_wait(bar_doa_empty, phase ^ 1, wctx, kWaitBwdLoad)) { ok = false; break; }
          if (lane == 0) {
            mbar_expect_tx(bar_doa_full, kQBytes);
#pragma unroll
            for (int h = 0; h < 4; ++h)
              tma_load_4d(smem_doa + h * kQPanel, &map_do, bar_doa_full, h * 64, head, qb.row, s.batch_coord);
          }
        } else {
          // The other CTA's iteration: only this CTA's half of the head dimension of Q and dO.
          if (!mbar_wait(bar_qb_empty, phase ^ 1, wctx, kWaitBwdLoad)) { ok = false; break; }
          if (lane == 0) {
            mbar_expect_tx(bar_qb_full, kHalfBytes);
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_4d(smem_qb + h * kQPanel, &map_q, bar_qb_full, (2 * dh + h) * 64, head, qb.row, s.batch_coord);
          }
          if (!mbar_wait(bar_dob_empty, phase ^ 1, wctx, kWaitBwdLoad)) { ok = false; break; }
          if (lane == 0) {
            mbar_expect_tx(bar_dob_full, kHalfBytes);
#pragma unroll
            for (int h = 0; h < 2; ++h)
              tma_load_4d(smem_dob + h * kQPanel, &map_do, bar_dob_full, (2 * dh + h) * 64, head, qb.row, s.batch_coord);
          }
        }
        ++it;
      }
    }
   } else if (warp == kXferWarp) {
    // ------------------------------------------------------------------ copies of X and Y into the other CTA
    if (lane == 0) {
      const uint32_t peer_x = map_to_rank(smem_x, peer), peer_yr = map_to_rank(smem_yr, peer);
      const uint32_t peer_recv_full = map_to_rank(bar_recv_full, peer);
      for (int it = dh; it < iterations; it += 2) {
        const uint32_t phase = (it >> 1) & 1;
        if (!mbar_wait(bar_ds_full, phase, wctx, kWaitBwdLoad)) break;
        if (it > 0) {
          // The other CTA's tiles are free: its copy of iteration it - 1 has arrived here (so it has been read there)
          // and its MMAs have read what this CTA sent for iteration it - 2.
          const uint32_t before = ((it - 1) >> 1) & 1;
          if (!mbar_wait(bar_recv_full, before, wctx, kWaitBwdLoad) || !mbar_wait(bar_may_send, before, wctx, kWaitBwdLoad)) break;
        }
        bulk_copy_to_cluster(peer_yr, smem_y, kDsBytes, peer_recv_full);
        if (!mbar_wait(bar_x_full, phase, wctx, kWaitBwdLoad)) break;
        bulk_copy_to_cluster(peer_x, smem_x, kDsBytes, peer_recv_full);
      }
    }
   } else if (warp == kMmaWarp) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && iterations > 0) {
      constexpr uint32_t idesc_st = umma_idesc_bf16(128, kSubM, 0, 0);  // S^T, dP^T: both operands K-major
      constexpr uint32_t idesc_acc = umma_idesc_bf16(128, 128, 0, 1);   // dV, dK: A K-major (or TMEM), B MN-major
      constexpr uint32_t idesc_dq = umma_idesc_bf16(128, kSubM, 1, 1);  // dQ^T: A and B MN-major
      const uint32_t t_s = tmem_base + kTmemS, t_dp = tmem_base + kTmemDp;
      const uint32_t t_dv = tmem_base + kTmemDv, t_dk = tmem_base + kTmemDk;
      const uint32_t t_v = tmem_base + kTmemV;  // V of the key block as BF16, the A operand of dP^T
      const uint32_t q_half = smem_qa + 2 * dh * kQPanel, do_half = smem_doa + 2 * dh * kQPanel;
      const uint32_t peer_may_send = map_to_rank(bar_may_send, peer);
      auto issue_s = [&]() {
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          const uint32_t a_off = (kk >> 2) * kKvPanel + (kk & 3) * 32;
          const uint32_t b_off = (kk >> 2) * kQPanel + (kk & 3) * 32;
          umma_ss(t_s, umma_smem_desc(smem_k + a_off, 16, 1024), umma_smem_desc(smem_qa + b_off, 16, 1024), idesc_st, kk > 0);
        }
        tc_commit(bar_s_full);
      };
      auto issue_dp = [&]() {
#pragma unroll
        for (int kk = 0; kk < 16; ++kk) {
          const uint32_t b_off = (kk >> 2) * kQPanel + (kk & 3) * 32;
          umma_ts(t_dp, t_v + kk * 8, umma_smem_desc(smem_doa + b_off, 16, 1024), idesc_st, kk > 0);
        }
        tc_commit(bar_dp_full);
      };
      // The copies of the other CTA complete on bar_recv_full: one arrival and 32 KB per iteration of the other CTA.
      if ((dh ^ 1) < iterations) mbar_expect_tx(bar_recv_full, 2 * kDsBytes);
      bool ok = mbar_wait(bar_kv_full, 0, wctx, kWaitBwdMma);
      if (ok && dh < iterations) {  // this CTA owns at least one iteration: its scores are issued ahead of the loop
        ok = mbar_wait(bar_qa_full, 0, wctx, kWaitBwdMma);
        if (ok) {
          tc_fence_after();
          issue_s();
          ok = mbar_wait(bar_doa_full, 0, wctx, kWaitBwdMma) && mbar_wait(bar_v_ready, 0, wctx, kWaitBwdMma);
        }
        if (ok) {
          tc_fence_after();
          issue_dp();
        }
      }
      for (int it = 0; ok && it < iterations; ++it) {
        const uint32_t phase = (it >> 1) & 1;
        if ((it & 1) == dh) {
          // ---- owned iteration. dV_h += P^T dO_h with P^T in TMEM
          trace_event(wctx, traced, 3 * dh, trace_n, 100);
          if (!mbar_wait(bar_p_full, phase, wctx, kWaitBwdMma)) { ok = false; break; }
          trace_event(wctx, traced, 3 * dh, trace_n, 101);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ts(t_dv, t_s + kk * kCols, umma_smem_desc(do_half + kk * 2048, kQPanel, 1024), idesc_acc, it > 0 || kk > 0);
          tc_commit(bar_doa_empty);  // dP^T and dV_h of this iteration have read the dO tile
          // dK_h += dS^T Q_h first (it releases the Q tile, whose reload gates the next S^T), then dQ^T of both halves:
          // half 1 over S^T / P^T (consumed by the dV MMAs above, which run first), half 0 over dP^T
          if (!mbar_wait(bar_ds_full, phase, wctx, kWaitBwdMma)) { ok = false; break; }
          trace_event(wctx, traced, 3 * dh, trace_n, 102);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(t_dk, umma_smem_desc(smem_y + kk * 32, 16, 1024), umma_smem_desc(q_half + kk * 2048, kQPanel, 1024), idesc_acc,
                    it > 0 || kk > 0);
          tc_commit(bar_qa_empty);
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(t_s, umma_smem_desc(smem_k + 2 * kKvPanel + kk * 2048, kKvPanel, 1024),
                    umma_smem_desc(smem_y + kk * 2048, kDsBytes, 1024), idesc_dq, kk > 0);
          tc_commit(bar_dq1_full);  // the drain of this half frees the S^T region while the other half is computed
#pragma unroll
          for (int kk = 0; kk < 8; ++kk)
            umma_ss(t_dp, umma_smem_desc(smem_k + kk * 2048, kKvPanel, 1024), umma_smem_desc(smem_y + kk * 2048, kDsBytes, 1024),
                    idesc_dq, kk > 0);
          tc_commit(bar_dq_full);
          // The other CTA may copy its next tiles over this CTA's (announced only if it has an iteration that waits for
          // it, so that no arrive is in flight towards a CTA that has left).
          if (it + 1 < iterations) tc_commit(peer_may_send);
          trace_event(wctx, traced, 3 * dh, trace_n, 103);
          // Scores of the next owned iteration: each region is free once the drain warps have read its dQ^T
          if (it + 2 < iterations) {
            if (!mbar_wait(bar_qa_full, phase ^ 1, wctx, kWaitBwdMma) || !mbar_wait(bar_dq1_empty, phase, wctx, kWaitBwdMma)) { ok = false; break; }
            trace_event(wctx, traced, 3 * dh, trace_n, 104);
            tc_fence_after();
            issue_s();
            if (!mbar_wait(bar_doa_full, phase ^ 1, wctx, kWaitBwdMma) || !mbar_wait(bar_dq0_empty, phase, wctx, kWaitBwdMma)) { ok = false; break; }
            trace_event(wctx, traced, 3 * dh, trace_n, 105);
            tc_fence_after();
            issue_dp();
          }
        } else {
          trace_event(wctx, traced, 3 * dh, trace_n, 200);
          // ---- the other CTA's iteration: its P^T and dS^T have arrived in this CTA's tiles
          if (!mbar_wait(bar_dob_full, phase, wctx, kWaitBwdMma) || !mbar_wait(bar_qb_full, phase, wctx, kWaitBwdMma) ||
              !mbar_wait(bar_recv_full, phase, wctx, kWaitBwdMma)) { ok = false; break; }
          trace_event(wctx, traced, 3 * dh, trace_n, 201);
          if (it + 2 < iterations) mbar_expect_tx(bar_recv_full, 2 * kDsBytes);
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(t_dv, umma_smem_desc(smem_x + kk * 32, 16, 1024), umma_smem_desc(smem_dob + kk * 2048, kQPanel, 1024),
                    idesc_acc, it > 0 || kk > 0);
          tc_commit(bar_dob_empty);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_ss(t_dk, umma_smem_desc(smem_yr + kk * 32, 16, 1024), umma_smem_desc(smem_qb + kk * 2048, kQPanel, 1024),
                    idesc_acc, it > 0 || kk > 0);
          tc_commit(bar_qb_empty);
          trace_event(wctx, traced, 3 * dh, trace_n, 202);
        }
      }
      if (ok) tc_commit(bar_final);
    }
   }
  } else if (warp < kComputeWarps) {
    setmaxnreg_inc<kRegsCompute>();
    // ------------------------------------------------------------------ P and dS on owned iterations (thread = key row)
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
    // This thread's two 16-byte chunks (8 queries each) of row r in the three tiles with the layout of the dS tile.
    const uint32_t chunk0 = (((cb >> 3) + 0) ^ (r & 7)) << 4, chunk1 = (((cb >> 3) + 1) ^ (r & 7)) << 4;
    const uint32_t x_row = smem_x + r * 128, y_row = smem_y + r * 128;
    int it = 0;
    bool ok = true;
    if (iterations > 0) {
      // V of the key block moves from its landing place in shared memory to TMEM (BF16 pairs, key row on the lane), where
      // it is the A operand of every dP^T MMA. Group wg copies the 64 columns of panel wg: eight 16-byte chunks per row,
      // stored with the 128-byte swizzle of the TMA box.
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
        if ((it & 1) != dh) {  // the other CTA's iteration: its compute warps do this work
          ++it;
          continue;
        }
        const uint32_t phase = (it >> 1) & 1;
        int qlo = 0, qhi = qb.limit - qb.col0;
        if (qb.banded) {
          if (right >= 0) qlo = imax(0, c - off - right - qb.col0);
          if (left >= 0) qhi = imin(qhi, c - off + left + 1 - qb.col0);
        }
        if (!key_valid) qhi = 0;
        const bool masked = __any_sync(0xffffffffu, qlo > cb || qhi < cb + kCols);
        // ---- P^T (kept in FP32 registers for dS, stored to TMEM as BF16 for the dV MMA)
        trace_event(wctx, traced && warp == 0, 1 + 3 * dh, trace_n, 300);
        if (!mbar_wait(bar_s_full, phase, wctx, kWaitBwdCompute)) { ok = false; break; }
        trace_event(wctx, traced && warp == 0, 1 + 3 * dh, trace_n, 301);
        tc_fence_after();
        float pf[kCols];
        tmem_ld16(t_s + cb, reinterpret_cast<uint32_t*>(pf));
        tc_wait_ld();
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int j = 0; j < kCols / 4; ++j) {
          const float4 l4 = ld_shared_f4(smem_lse + (cb + 4 * j) * 4);  // -lse * log2(e)
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
        const uint32_t before = ((it - 1) >> 1) & 1;
        trace_event(wctx, traced && warp == 0, 1 + 3 * dh, trace_n, 302);
        // ---- dS^T = P^T o (dP^T - D), written to shared memory as BF16
        if (!mbar_wait(bar_dp_full, phase, wctx, kWaitBwdCompute)) { ok = false; break; }
        // Tile Y held this CTA's dS^T of two iterations ago: its MMAs were issued ahead of the scores of this iteration,
        // and its copy out is complete once the other CTA's tiles of the previous iteration, sent after it, are here.
        if (it > 0 && !mbar_wait(bar_recv_full, before, wctx, kWaitBwdCompute)) { ok = false; break; }
        trace_event(wctx, traced && warp == 0, 1 + 3 * dh, trace_n, 303);
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
            const float4 d4 = ld_shared_f4(smem_dpsum + (cb + i) * 4);  // -sum_d O dO
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
          st_shared_v4(y_row + (j == 0 ? chunk0 : chunk1), packed[0], packed[1], packed[2], packed[3]);
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(bar_ds_full);
        trace_event(wctx, traced && warp == 0, 1 + 3 * dh, trace_n, 304);
        // The copy of P^T for the other CTA, off the chain: tile X holds what that CTA sent for the previous iteration
        // until this CTA's dV MMAs of that iteration have read it.
        if (it > 0 && !mbar_wait(bar_dob_empty, before, wctx, kWaitBwdCompute)) { ok = false; break; }
        {
          uint32_t pk[kCols / 2];
#pragma unroll
          for (int i = 0; i < kCols / 2; ++i) pk[i] = pack_bf16x2(pf[2 * i], pf[2 * i + 1]);
          st_shared_v4(x_row + chunk0, pk[0], pk[1], pk[2], pk[3]);
          st_shared_v4(x_row + chunk1, pk[4], pk[5], pk[6], pk[7]);
        }
        fence_proxy_async_smem();
        mbar_arrive(bar_x_full);
        trace_event(wctx, traced && warp == 0, 1 + 3 * dh, trace_n, 305);
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
    // On owned iterations drain group dg takes query rows [32 dg, 32 dg + 32) of both halves of the head dimension, the
    // half over S^T first (the next S^T is issued before the next dP^T), 16 rows at a time through its staging buffer.
    const int dg = (warp - kComputeWarps) >> 2;
    const int d = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_col = tmem_base + lane_addr + 2 * kStageRows * dg;
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
        if ((it & 1) != dh) {
          ++it;
          continue;
        }
        const uint32_t phase = (it >> 1) & 1;
        const int row0 = (int)(stat_base + qb.row) + 2 * kStageRows * dg;
        trace_event(wctx, traced && dh == 0 && dg == 0, 2, trace_n, 400);
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
          const int half = 1 - pass;  // half of the head dimension: 1 lies over S^T, 0 over dP^T
          if (!mbar_wait(half ? bar_dq1_full : bar_dq_full, phase, wctx, kWaitBwdReduce)) { ok = false; break; }
          trace_event(wctx, traced && dh == 0 && dg == 0, 2, trace_n, 401);
          tc_fence_after();
          uint32_t acc[kChunks * kStageRows];
          static_assert(kChunks * kStageRows == 32, "the drain reads its TMEM columns with one 32-column load");
          tmem_ld32(t_col + (half ? kTmemS : kTmemDp), acc);
          tc_wait_ld();
          tc_fence_before();
          mbar_arrive(half ? bar_dq1_empty : bar_dq0_empty);
          trace_event(wctx, traced && dh == 0 && dg == 0, 2, trace_n, 402 + pass);
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
              tma_reduce_add_4d(&map_dq, stage, half * 128, head, row0 + kStageRows * ch, 0);
              bulk_commit_group();
            }
          }
        }
        if (!ok) break;
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
  cluster_sync_all();  // the other CTA stores into this CTA's shared memory and arrives on its barriers until here
  if (warp == kMmaWarp) tmem_dealloc(tmem_base, 512);
}

}  // namespace bd256p

int launch_bwd_main_d256_pair(const b200fa_bwd_args& a, const BwdParams& params, dim3 grid, float* dq_accum,
                              int64_t stat_rows, cudaStream_t stream) {
  using namespace bd256p;
  constexpr int D = 256;
  const b200fa_problem& bp = a.problem;
  const bool packed = bp.cu_seqlens_q != nullptr;
  const int64_t rows_q = bp.seqlen_q, rows_k = bp.seqlen_k;
  const int64_t tensor_batch = packed ? 1 : bp.batch;
  BwdParams p = params;
  // The two halves of the head dimension of a key block must be neighbours in the launch order: consecutive head slots
  // of one key block, which the decoding of the linear index gives when a section holds an even number of slots.
  if (!p.work_list && (p.section & 1)) p.section = 2;
  B200FA_REQUIRE(p.work_list ? grid.y % 2 == 0 : grid.x % 2 == 0, "the paired head_dim 256 backward needs an even grid");
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
  static bool attribute_set[64] = {false};
  status = set_dynamic_smem_once(reinterpret_cast<const void*>(&bwd_d256_pair_kernel), kSmemBytes, attribute_set);
  if (status != B200FA_OK) return status;
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(kThreads, 1, 1);
  config.dynamicSmemBytes = kSmemBytes;
  config.stream = stream;
  cudaLaunchAttribute attribute;
  attribute.id = cudaLaunchAttributeClusterDimension;
  attribute.val.clusterDim.x = p.work_list ? 1 : 2;
  attribute.val.clusterDim.y = p.work_list ? 2 : 1;
  attribute.val.clusterDim.z = 1;
  config.attrs = &attribute;
  config.numAttrs = 1;
  B200FA_CUDA_CHECK(cudaLaunchKernelEx(&config, bwd_d256_pair_kernel, map_q, map_k, map_v, map_do, map_dq, p));
  return B200FA_OK;
}

}  // namespace b200fa
