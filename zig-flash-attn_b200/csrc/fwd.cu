// Forward attention kernel for sm_100a: O = softmax(scale Q K^T + mask) V and the row log-sum-exp.
//
// Takes the place of the reference's flash_attn_fwd for sm_100 (zig/flash_fwd_sm100.zig:41-1380) and of its
// persistent inter-sequence forward (zig/inter_sequence_forward_sm100.zig:40-1274); one kernel serves fixed-length,
// packed (varlen) and inter-sequence problems because key blocks come from the KeyCursor of attn_index.h.
//
// One persistent CTA per SM; the CTAs draw work items from a global counter (TileQueue). A work item is 256 query rows
// of one head (two 128-row MMA tiles, "stages"), or, with packed query heads (fixed-length problems whose key heads
// serve a power-of-two group of G query heads; the reference packs the same way, zig/m_block_work.zig:17-35), 256 / G
// tokens of all G heads of one key head: the Q box of the TMA load then spans (128 / G tokens, G heads), which lands
// in shared memory as rows ordered token-major, and a softmax thread derives its (token, head) from its row. Packed
// items read each key block once for the whole group and, under a causal mask, see fewer masked blocks.
// Warp roles: warps 0-3 softmax of stage 0, warps 4-7 softmax of stage 1 (one thread per query row, TMEM lane =
// row), warp 8 issues tcgen05 MMAs, warp 9 issues TMA loads.
//   S_i = Q_i K_j^T   SS-MMA 128x128xD  into TMEM columns [128 i, 128 i + 128)
//   P_i               BF16, written by the softmax warps over columns [64,128) of S_i (whose scores they hold in registers)
//   O_i += P_i V_j    TS-MMA 128xDx128 (A from TMEM) into TMEM columns [256 + D i, 256 + D i + D), issued in two key
//                     halves: keys [64,128) as soon as their probabilities are stored, keys [0,64) after the rest
// Q tiles, and a ring of K/V tiles, are TMA-loaded into 128-byte swizzled shared memory and tracked by mbarriers.
// Softmax runs in the log2 domain with a lazy rescale: the running reference maximum only moves when the block
// maximum exceeds it by more than 8 (in log2 units), so O is almost never rescaled (reference
// zig/flash_fwd_sm100.zig:963-976).
#include <atomic>
#include <cstdlib>

#include "fwd_common.cuh"

namespace b200fa {

template <int D>
struct FwdConfig {
  static constexpr int kStages = D <= 64 ? 8 : 4;             // K/V ring slots
  static constexpr int kTileBytes = kBlockM * D * 2;           // one 128 x D BF16 tile
  static constexpr int kHalves = D / 64;                       // 64-column (128-byte) swizzle panels per tile
  static constexpr int kPanelBytes = kBlockM * 128;
  static constexpr int kSmemQ = 2 * kTileBytes;
  static constexpr int kSmemKv = kStages * kTileBytes;
  static constexpr int kSmemBytes = kSmemQ + kSmemKv + 1024 /*alignment slack*/ + 512 /*barriers, tile queue*/;
  static constexpr int kThreads = 384;  // 2 softmax warpgroups + 1 warpgroup holding the MMA and TMA warps
  static constexpr int kTmemS = 0;
  static constexpr int kTmemO = 256;
  // head_dim 64 leaves 128 TMEM columns free (S 2 x 128, O 2 x 64): P gets columns of its own there instead of going
  // over the upper half of S, so the scores of block j + 1 of a stage can be computed as soon as the softmax warps have
  // read those of block j (bar_s_free), not only after the PV product of block j has been issued. That takes the S
  // product and two barrier hand-overs off the chain softmax -> PV -> S -> softmax of a stage; measured it is worth
  // 0.6 % at seqlen 8192 and 2.5 % at seqlen 2048 (causal), so that chain is not what bounds this kernel.
  static constexpr bool kOwnP = D <= 64;
  static constexpr int kTmemP = kOwnP ? 384 : kTmemS + 64;  // first P column of stage 0
  static constexpr int kPStride = kOwnP ? 64 : 128;          // columns between the P of the two stages
};

template <int D, bool kSplit, bool kBits>
__global__ void __launch_bounds__(FwdConfig<D>::kThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
           const __grid_constant__ CUtensorMap map_v, const __grid_constant__ FwdParams p) {
  using Cfg = FwdConfig<D>;
  constexpr int NS = Cfg::kStages;
  // head_dim 64 (24 MMAs and 6 commits per pair of blocks) is bound by the rate of tcgen05 instructions, and handing the
  // K/V slots back from a softmax thread instead of by a commit gains 1.5-3 % there; at head_dim 128 it changes nothing.
  constexpr bool kSimtRelease = Cfg::kOwnP;
  // Shares of the key blocks per tile (split-KV). The unsplit instance folds the divisions by it and the partial-result
  // epilogue away: with both in one kernel, problems of 512-2048 tokens lost 4-8 % to the code they never run.
  const int splits = kSplit ? p.splits : 1;
  // Register split between the warpgroups: 2 x 128 x 200 + 128 x 104 = 64512, the 384 x 168 registers the CTA is
  // launched with (setmaxnreg only moves registers inside that pool). With 208 / 88 the MMA and TMA warps spilled.
  constexpr int kRegsSoftmax = 200, kRegsOther = 104;
  // Of every kPolyPeriod pairs of scores, kPolyCount take the polynomial exp2 and the rest the MUFU.
  constexpr int kPolyPeriod = 4, kPolyCount = 0;
  // Keep all 128 scores of a row in registers (true) or read the lower half from TMEM a second time (false).
  constexpr bool kSinglePass = false;
  // The PV product of a block is issued in two halves: keys [64,128) as soon as their probabilities are stored, keys
  // [0,64) after the rest, so the first half runs while the softmax warps still work on the second.
#ifndef B200FA_SPLIT_PV
#define B200FA_SPLIT_PV 1
#endif
  constexpr bool kSplitPv = B200FA_SPLIT_PV && !kSinglePass;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_q = smem_base;
  const uint32_t smem_kv = smem_base + Cfg::kSmemQ;
  const uint32_t bar_base = smem_kv + Cfg::kSmemKv;
  // barrier layout (8 bytes each)
  const uint32_t bar_q_full = bar_base;            // [2]
  const uint32_t bar_q_empty = bar_base + 16;      // [1]
  const uint32_t bar_kv_full = bar_base + 24;      // [NS]
  const uint32_t bar_kv_empty = bar_kv_full + 8 * NS;
  const uint32_t bar_s_full = bar_kv_empty + 8 * NS;   // [2]
  const uint32_t bar_p_full = bar_s_full + 16;         // [2]
  const uint32_t bar_pv_done = bar_p_full + 16;        // [2]
  const uint32_t bar_p_half = bar_pv_done + 16;        // [2]
  const uint32_t tmem_slot = bar_p_half + 16;          // 4 bytes
  const uint32_t abort_slot = tmem_slot + 4;           // 4 bytes
  const uint32_t bar_s_free = abort_slot + 4;          // [2] (kOwnP) the softmax warps have read the scores of a block
  TileQueue tiles;
  tiles.place(bar_base + 384);                         // the barriers above end below byte 256
  volatile int* abort_flag =
      reinterpret_cast<volatile int*>(smem_raw + (abort_slot - smem_u32(smem_raw)));
  volatile uint32_t* tmem_ptr_smem =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  const WaitCtx wctx{abort_flag, p.status, p.trace};
  int trace_n = 0;  // timeline of the first work item of CTA 0 (tuning builds; see trace_event)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_full + 8, 1);
    mbar_init(bar_q_empty, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(bar_kv_full + 8 * i, 1);
      mbar_init(bar_kv_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_p_full + 8 * i, 128);
      mbar_init(bar_p_half + 8 * i, 128);
      mbar_init(bar_pv_done + 8 * i, 1);
      mbar_init(bar_s_free + 8 * i, 128);
    }
    tiles.init(1 + 8);  // the MMA thread and the eight softmax warps
    fence_barrier_init();
  }
  if (warp == 8) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (warp == 9 && lane == 0) {
    tma_prefetch_descriptor(&map_q);
    tma_prefetch_descriptor(&map_k);
    tma_prefetch_descriptor(&map_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const Problem& pr = p.prob;

  // setmaxnreg is executed once per warpgroup, by all four of its warps at the same instruction.
  if (warp >= 8) {
   setmaxnreg_dec<kRegsOther>();
   if (warp == 9) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t ring = 0;      // K/V slots issued so far
      uint32_t q_count = 0;   // tiles with at least one key block
      bool ok = true;
      auto load_tile = [&](const CUtensorMap* map, uint32_t dst, uint32_t bar, int head, int row, int batch_coord) {
        mbar_expect_tx(bar, Cfg::kTileBytes);
#pragma unroll
        for (int h = 0; h < Cfg::kHalves; ++h) tma_load_4d(dst + h * Cfg::kPanelBytes, map, bar, h * 64, head, row, batch_coord);
      };
      auto load_kv = [&](const CUtensorMap* map, int head, int row, int batch_coord) -> bool {
        uint32_t slot = ring % NS, phase = (ring / NS) & 1;
        if (!mbar_wait(bar_kv_empty + 8 * slot, phase ^ 1, wctx, kWaitKvEmpty)) return false;
        load_tile(map, smem_kv + slot * Cfg::kTileBytes, bar_kv_full + 8 * slot, head, row, batch_coord);
        ++ring;
        return true;
      };
      uint32_t drawn = 0;
      for (int tile; ok && (tile = tiles.push(drawn, p.tile_counter, p.num_tiles, wctx)) >= 0;) {
        FwdTile t = decode_tile(p, tile / splits);
        if (!t.valid) continue;
        KeyCursorT<kBits> cur;
        cur.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + (kFwdTileM >> p.pack_shift), t.s.lq));
        if (kSplit) cur.restrict_to_share(tile % splits, splits);
        OtherBlock kb;
        if (!cur.next(&kb)) continue;
        if (!mbar_wait(bar_q_empty, (q_count & 1) ^ 1, wctx, kWaitQEmpty)) { ok = false; break; }
        ++q_count;
        load_tile(&map_q, smem_q, bar_q_full, t.head, t.s.q0 + t.m0, t.s.batch_coord);
        if (!load_kv(&map_k, t.kv_head, kb.row, t.s.batch_coord)) { ok = false; break; }
        load_tile(&map_q, smem_q + Cfg::kTileBytes, bar_q_full + 8, t.head, t.s.q0 + t.m0 + (kBlockM >> p.pack_shift),
                  t.s.batch_coord);
        for (;;) {
          if (!load_kv(&map_v, t.kv_head, kb.row, t.s.batch_coord)) { ok = false; break; }
          if (!cur.next(&kb)) break;
          if (!load_kv(&map_k, t.kv_head, kb.row, t.s.batch_coord)) { ok = false; break; }
        }
      }
    }
   } else if (warp == 8) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kBlockM, D, 0, 1);
      uint32_t ring = 0, q_count = 0, blocks = 0;
      bool ok = true;
      const int k_steps = (p.head_dim + 15) / 16;  // 16-column steps of the score product that hold data
      auto issue_s = [&](int stage, uint32_t k_smem) {
        const uint32_t q_addr = smem_q + stage * Cfg::kTileBytes;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk >= k_steps) break;  // head dims below the compiled width: the remaining columns are zero-filled
          const uint32_t off = (kk >> 2) * Cfg::kPanelBytes + (kk & 3) * 32;
          umma_ss(tmem_base + Cfg::kTmemS + stage * 128, umma_smem_desc(q_addr + off, 16, 1024),
                  umma_smem_desc(k_smem + off, 16, 1024), idesc_s, kk > 0);
        }
      };
      // O += P V over the key steps [first, first + count) of the block (16 keys per step).
      auto issue_pv_steps = [&](int stage, uint32_t v_smem, int first, int count, bool accumulate) {
#pragma unroll
        for (int kk = first; kk < first + count; ++kk) {
          umma_ts(tmem_base + Cfg::kTmemO + stage * D, tmem_base + Cfg::kTmemP + stage * Cfg::kPStride + kk * 8,
                  umma_smem_desc(v_smem + kk * 2048, Cfg::kPanelBytes, 1024), idesc_pv, accumulate || kk > first);
        }
      };
      // The whole product of a stage: with kSplitPv the upper key half goes first, behind its own barrier.
      auto issue_pv = [&](int stage, uint32_t v_smem, bool accumulate, uint32_t phase) -> bool {
        constexpr int kSteps = kBlockN / 16;
        if (kSplitPv) {
          if (!mbar_wait(bar_p_half + 8 * stage, phase, wctx, kWaitPFull)) return false;
          tc_fence_after();
          trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 300 + 1000 * stage + (blocks % 100));  // first half of P present
          issue_pv_steps(stage, v_smem, kSteps / 2, kSteps / 2, accumulate);
        }
        if (!mbar_wait_traced(bar_p_full + 8 * stage, phase, wctx, kWaitPFull, 17 + stage, false)) return false;
        tc_fence_after();
        trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 500 + 1000 * stage + (blocks % 100));  // all of P present
        if (kSplitPv) {
          issue_pv_steps(stage, v_smem, 0, kSteps / 2, true);
        } else {
          issue_pv_steps(stage, v_smem, 0, kSteps, accumulate);
        }
        return true;
      };
      auto wait_kv = [&](uint32_t index) -> bool {
        return mbar_wait_traced(bar_kv_full + 8 * (index % NS), (index / NS) & 1, wctx, kWaitKvFull, 16, false);
      };
      uint32_t popped = 0;
      for (int tile; ok && (tile = tiles.pop_thread(popped, wctx)) >= 0;) {
        FwdTile t = decode_tile(p, tile / splits);
        if (!t.valid) continue;
        KeyCursorT<kBits> cur;
        cur.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + (kFwdTileM >> p.pack_shift), t.s.lq));
        if (kSplit) cur.restrict_to_share(tile % splits, splits);
        OtherBlock kb;
        if (!cur.next(&kb)) continue;
        const uint32_t q_phase = q_count & 1;
        ++q_count;
        uint32_t k_index = ring++;
        if (!mbar_wait(bar_q_full, q_phase, wctx, kWaitQFull) || !wait_kv(k_index)) { ok = false; break; }
        tc_fence_after();
        issue_s(0, smem_kv + (k_index % NS) * Cfg::kTileBytes);
        tc_commit(bar_s_full);
        if (!mbar_wait(bar_q_full + 8, q_phase, wctx, kWaitQFull)) { ok = false; break; }
        tc_fence_after();
        issue_s(1, smem_kv + (k_index % NS) * Cfg::kTileBytes);
        tc_commit(bar_s_full + 8);
        if (!kSimtRelease) tc_commit(bar_kv_empty + 8 * (k_index % NS));
        bool first = true;
        for (;;) {
          const bool more = cur.next(&kb);
          const uint32_t v_index = ring++;
          if (!wait_kv(v_index)) { ok = false; break; }
          if (more) {
            k_index = ring++;
            if (!wait_kv(k_index)) { ok = false; break; }
          }
          const uint32_t v_smem = smem_kv + (v_index % NS) * Cfg::kTileBytes;
          const uint32_t k_smem = smem_kv + (k_index % NS) * Cfg::kTileBytes;
          const uint32_t phase = blocks & 1;
          if (Cfg::kOwnP) {
            // P has TMEM columns of its own: the scores of the next block are issued as soon as the softmax warps of
            // the stage have read the current ones, ahead of the stage's PV product.
            if (more) {
              if (!mbar_wait(bar_s_free, phase, wctx, kWaitPFull)) { ok = false; break; }
              tc_fence_after();
              issue_s(0, k_smem);
              tc_commit(bar_s_full);
            }
            if (!issue_pv(0, v_smem, !first, phase)) { ok = false; break; }
            // Announced for every block here: the scores of block j + 1 no longer prove PV(j) complete, and the softmax
            // warps must know it before they rescale O or overwrite P.
            tc_commit(bar_pv_done);
            if (more) {
              if (!mbar_wait(bar_s_free + 8, phase, wctx, kWaitPFull)) { ok = false; break; }
              tc_fence_after();
              issue_s(1, k_smem);
              tc_commit(bar_s_full + 8);
              if (!kSimtRelease) tc_commit(bar_kv_empty + 8 * (k_index % NS));
            }
            if (!issue_pv(1, v_smem, !first, phase)) { ok = false; break; }
            tc_commit(bar_pv_done + 8);
            if (!kSimtRelease) tc_commit(bar_kv_empty + 8 * (v_index % NS));
            if (!more) tc_commit(bar_q_empty);
          } else {
            if (!issue_pv(0, v_smem, !first, phase)) { ok = false; break; }
            // PV done is announced for the last block of a tile only (the epilogue waits for it). In between, the scores of
            // block j + 1 being present already proves PV(j) complete: a commit covers every MMA issued before it, and a
            // tcgen05.commit costs a 128 x 128 x 16 MMA stream about 90 cycles.
            if (!more) tc_commit(bar_pv_done);
            trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 600 + (blocks % 100));  // PV of stage 0 issued
            if (more) {
              issue_s(0, k_smem);
              tc_commit(bar_s_full);
              trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 100 + (blocks % 100));  // S of stage 0 issued
            }
            if (!issue_pv(1, v_smem, !first, phase)) { ok = false; break; }
            if (!more) tc_commit(bar_pv_done + 8);
            trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 1600 + (blocks % 100));  // PV of stage 1 issued
            if (!kSimtRelease) tc_commit(bar_kv_empty + 8 * (v_index % NS));
            if (more) {
              issue_s(1, k_smem);
              tc_commit(bar_s_full + 8);
              trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 1100 + (blocks % 100));  // S of stage 1 issued
              if (!kSimtRelease) tc_commit(bar_kv_empty + 8 * (k_index % NS));
            } else {
              tc_commit(bar_q_empty);
            }
          }
          ++blocks;
          first = false;
          if (!more) break;
        }
      }
      // The last commit of this thread must land before the CTA may exit.
      if (ok && q_count > 0) mbar_wait(bar_q_empty, (q_count - 1) & 1, wctx, kWaitQEmpty);
    }
   }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue (one thread per row)
    setmaxnreg_inc<kRegsSoftmax>();
    const int stage = warp >> 2;
    const int row_in_stage = (warp & 3) * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + lane_addr + Cfg::kTmemS + stage * 128;
    const uint32_t t_o = tmem_base + lane_addr + Cfg::kTmemO + stage * D;
    const uint32_t t_p = tmem_base + lane_addr + Cfg::kTmemP + stage * Cfg::kPStride;
    const uint32_t my_s_full = bar_s_full + 8 * stage;
    const uint32_t my_p_full = bar_p_full + 8 * stage;
    const uint32_t my_pv_done = bar_pv_done + 8 * stage;
    const float scale_log2 = p.scale_log2;
    uint32_t blocks = 0, tiles_done = 0;  // key blocks and work items with key blocks so far
    // K/V slots are handed back to the load warp by one softmax thread of stage 1 instead of a tcgen05.commit of the MMA
    // thread: a commit takes a slot in the MMA stream like an MMA does. The scores of block j of stage 1 being present
    // proves that every MMA issued before them is complete: those on K_j and, for j > 0, those on V_(j-1). The ring
    // indices mirror the MMA thread's: a work item with n key blocks takes K_0 V_0 K_1 V_1 ... V_(n-1).
    const bool releaser = kSimtRelease && stage == 1 && (warp & 3) == 0 && lane == 0;
    uint32_t ring = 0;
    bool ok = true;
    uint32_t popped = 0;
    for (int tile; ok && (tile = tiles.pop_warp(popped, wctx)) >= 0;) {
      FwdTile t = decode_tile(p, tile / splits);
      if (!t.valid) continue;
      // Row within the sequence and head of this thread (packed heads: tile row = token << pack_shift | head of group).
      const int tile_row = stage * kBlockM + row_in_stage;
      const int row = t.m0 + (tile_row >> p.pack_shift);
      const int head = t.head + (tile_row & ((1 << p.pack_shift) - 1));
      KeyCursorT<kBits> cur;
      cur.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + (kFwdTileM >> p.pack_shift), t.s.lq));
      const int split = kSplit ? tile % splits : 0;
      if (kSplit) cur.restrict_to_share(split, splits);
      const int band_lo = cur.band.lo(row), band_hi = cur.band.hi(row);
      // Row state: `m` is the lazy reference maximum, `l` the sum of the exponentials relative to it of every key except
      // the keys set aside (TopApart, fwd_common.cuh: the tie-counting LSE of the reference,
      // zig/flash_fwd_sm100.zig:885-901, with the counting done only in the blocks where it can matter).
      float m = -INFINITY, l = 0.f;
      TopApart top;
      int tile_blocks = 0;
      OtherBlock kb;
      while (cur.next(&kb)) {
        if (!mbar_wait_traced(my_s_full, blocks & 1, wctx, kWaitSFull, 19, true)) { ok = false; break; }
        if (releaser) mbar_arrive(bar_kv_empty + 8 * ((ring + 2 * tile_blocks) % NS));
        const long long t_soft = trace_clock(wctx);
        tc_fence_after();
        const bool traced = blockIdx.x == 0 && (threadIdx.x & 127) == 0 && popped == 1;
        trace_event(wctx, traced, 1 + stage, trace_n, 2000 + 1000 * stage + (tile_blocks % 100));  // scores present
        // Column limits of this row inside the block; `masked` is uniform over the warp.
        int lo, hi;
        if (kb.banded) {
          lo = band_lo - kb.col0;
          hi = band_hi - kb.col0;
        } else {
          lo = 0;
          hi = kb.limit - kb.col0;
        }
        const bool masked = __any_sync(0xffffffffu, lo > 0 || hi < kBlockN);
        auto apply_mask = [&](float2* values, int first_column) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int c = first_column + 2 * i;
            values[i].x = (c >= lo && c < hi) ? values[i].x : -INFINITY;
            values[i].y = (c + 1 >= lo && c + 1 < hi) ? values[i].y : -INFINITY;
          }
        };
        auto max_of = [&](const float2* values) {
          float a = fmaxf(values[0].x, values[0].y), b = fmaxf(values[1].x, values[1].y);
          float c = fmaxf(values[2].x, values[2].y), d = fmaxf(values[3].x, values[3].y);
#pragma unroll
          for (int i = 4; i < 32; i += 4) {
            a = fmaxf(a, fmaxf(values[i].x, values[i].y));
            b = fmaxf(b, fmaxf(values[i + 1].x, values[i + 1].y));
            c = fmaxf(c, fmaxf(values[i + 2].x, values[i + 2].y));
            d = fmaxf(d, fmaxf(values[i + 3].x, values[i + 3].y));
          }
          return make_float2(fmaxf(a, c), fmaxf(b, d));  // maxima over the even and over the odd pairs of columns
        };
        // Pass 1: row maximum. Columns [0,64) are read for the maximum only and read again in pass 2; columns
        // [64,128) stay in registers. P (BF16) goes over columns [64,128) of S, upper half first, so nothing that is
        // still to be read gets overwritten.
        float2 low[32], high[32];
        tmem_ld32(t_s, reinterpret_cast<uint32_t*>(low));
        tmem_ld32(t_s + 32, reinterpret_cast<uint32_t*>(low) + 32);
        tc_wait_ld();
        if (masked) apply_mask(low, 0);
        const float2 max_low = max_of(low);
        tmem_ld32(t_s + 64, reinterpret_cast<uint32_t*>(high));
        tmem_ld32(t_s + 96, reinterpret_cast<uint32_t*>(high) + 32);
        tc_wait_ld();
        if (masked) apply_mask(high, 64);
        const float2 max_high = max_of(high);
        // Maxima over two interleaved halves of the block (even and odd pairs of columns): under a causal or window mask
        // both halves hold visible keys as soon as the row sees more than two keys of the block.
        const float max_even = fmaxf(max_low.x, max_high.x), max_odd = fmaxf(max_low.y, max_high.y);
        const float block_max = fmaxf(max_even, max_odd);
        const float m_new = fmaxf(m, block_max);
        const bool set_apart = sets_keys_apart(top, max_even, max_odd, scale_log2);
        trace_event(wctx, traced, 1 + stage, trace_n, 4000 + 1000 * stage + (tile_blocks % 100));  // row maximum known
        const bool grow = (m_new - m) * scale_log2 > 8.f;  // also true when m is -inf and m_new is finite
        // With P in columns of its own the scores of this block may be present before the PV product of the previous one
        // has read its P (and accumulated into O): wait for it before O is rescaled or P overwritten. Every completion
        // of the barrier is observed here or, for the last block of a work item, in the epilogue.
        if (Cfg::kOwnP && tile_blocks > 0 && !mbar_wait_traced(my_pv_done, (blocks - 1) & 1, wctx, kWaitPvDone, 26, true)) { ok = false; break; }
        if (Cfg::kOwnP && tile_blocks > 0) tc_fence_after();
        if (releaser && tile_blocks > 0) mbar_arrive(bar_kv_empty + 8 * ((ring + 2 * tile_blocks - 1) % NS));
        // One rarely taken branch, behind one vote, holds both the rescale and the second summation of blocks with keys
        // set aside, so the common path has a single vote and branch between the maximum and the exponentials.
        float sum_counted = 0.f;
        bool counting = false;
        if (__any_sync(0xffffffffu, grow || set_apart)) {
          const bool any_grow = __any_sync(0xffffffffu, grow);
          if (any_grow) {
            float alpha = 1.f;
            if (grow) {
              alpha = (m == -INFINITY) ? 0.f : ex2_approx((m - m_new) * scale_log2);
              l *= alpha;
              m = m_new;
            }
            if (tile_blocks > 0) {
              // The scores of this block are present, so the PV product of the previous block has completed.
              const float2 alpha2 = make_float2(alpha, alpha);
#pragma unroll
              for (int c = 0; c < D / 32; ++c) {
                float2 o[16];
                tmem_ld32(t_o + 32 * c, reinterpret_cast<uint32_t*>(o));
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) o[i] = __fmul2_rn(o[i], alpha2);
                tmem_st32(t_o + 32 * c, reinterpret_cast<uint32_t*>(o));
              }
            }
          }
          // Blocks in which some row of the warp sets keys aside (rare) sum their exponentials a second time, without
          // those keys, here, where the rescale branch already splits the instruction stream: the common path below
          // carries no compare per score.
          counting = __any_sync(0xffffffffu, set_apart);
          if (__builtin_expect(counting, 0))
            sum_counted = sum_without_keys_apart<kBlockN>(top, l, set_apart, block_max, t_s, masked, lo, hi, scale_log2,
                                                          (m == -INFINITY) ? 0.f : m * scale_log2);
        }
        const float mc = (m == -INFINITY) ? 0.f : m * scale_log2;
        const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-mc, -mc);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
        // 64 scores -> 64 probabilities (BF16) stored at P columns [first_p_column, first_p_column + 32)
        auto exponentiate = [&](const float2* values, uint32_t first_p_column) {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 x = __ffma2_rn(values[16 * c + i], scale2, shift2);
              float2 e;
              if ((i % kPolyPeriod) < kPolyCount) {  // this share of the pairs is exponentiated on the FMA pipe
                e = ex2_poly2(x);
              } else {
                e.x = ex2_approx(x.x);
                e.y = ex2_approx(x.y);
              }
              if (i & 1) sum_b = __fadd2_rn(sum_b, e); else sum_a = __fadd2_rn(sum_a, e);
              packed[i] = pack_bf16x2(e.x, e.y);
            }
            tmem_st16(t_p + first_p_column + 16 * c, packed);
          }
        };
        if (kSinglePass) {
          exponentiate(high, 32);
          exponentiate(low, 0);
        } else {
          // Pass 2 for columns [0,64): the loads are in flight while the upper half is exponentiated.
          tmem_ld32(t_s, reinterpret_cast<uint32_t*>(low));
          tmem_ld32(t_s + 32, reinterpret_cast<uint32_t*>(low) + 32);
          exponentiate(high, 32);
          if (kSplitPv) {  // the probabilities of keys [64,128) are in TMEM: their half of the PV product may start
            tc_wait_st();
            tc_fence_before();
            mbar_arrive(bar_p_half + 8 * stage);
          }
          trace_event(wctx, traced, 1 + stage, trace_n, 6000 + 1000 * stage + (tile_blocks % 100));  // first half of P stored
          tc_wait_ld();
          if (Cfg::kOwnP) {  // the scores of this block have left TMEM: the next block's may be computed
            tc_fence_before();
            mbar_arrive(bar_s_free + 8 * stage);
          }
          if (masked) apply_mask(low, 0);
          exponentiate(low, 0);
        }
        l += counting ? sum_counted : (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(my_p_full);
        trace_event(wctx, traced, 1 + stage, trace_n, 8000 + 1000 * stage + (tile_blocks % 100));  // all of P stored
        trace_add(wctx, 20, trace_clock(wctx) - t_soft);
        trace_add(wctx, 21, 1);
        ++blocks;
        ++tile_blocks;
      }
      if (!ok) break;
      // ---- epilogue: O / l -> BF16 -> global, lse
      const bool row_valid = row < t.s.lq;
      __nv_bfloat16* o_row = p.o + t.s.batch_coord * p.o_batch_stride + (int64_t)(t.s.q0 + row) * p.o_row_stride +
                             (int64_t)head * p.o_head_stride;
      float* lse_ptr = p.lse + t.s.batch_coord * p.lse_batch_stride + (int64_t)head * p.lse_head_stride + t.s.q0 + row;
      // Split-KV: this share's normalised output (fp32) and log-sum-exp go to the partial buffers instead.
      float* o_part = nullptr;
      if (kSplit) {
        const int64_t global_row = (int64_t)t.s.batch_coord * pr.seqlen_q + row;
        o_part = p.o_partial + (((int64_t)split * p.partial_rows + global_row) * pr.heads_q + head) * p.head_dim;
        lse_ptr = p.lse_partial + ((int64_t)split * pr.heads_q + head) * p.partial_rows + global_row;
      }
      if (tile_blocks == 0) {
        if (row_valid) {
          const uint4 zero = make_uint4(0, 0, 0, 0);
          if (o_part) {
#pragma unroll
            for (int c = 0; c < D / 4; ++c)
              if (4 * c < p.head_dim) reinterpret_cast<uint4*>(o_part)[c] = zero;
          } else {
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
              if (8 * c < p.head_dim) reinterpret_cast<uint4*>(o_row)[c] = zero;
          }
          *lse_ptr = -INFINITY;
        }
        continue;
      }
      if (!mbar_wait_traced(my_pv_done, (Cfg::kOwnP ? blocks - 1 : tiles_done) & 1, wctx, kWaitEpilogue, 22, true)) { ok = false; break; }
      ++tiles_done;
      if (releaser) mbar_arrive(bar_kv_empty + 8 * ((ring + 2 * tile_blocks - 1) % NS));
      ring += 2 * tile_blocks;
      const long long t_epi = trace_clock(wctx);
      tc_fence_after();
      float total, lse_row;
      row_totals(m, l, top.ones, top.apart, scale_log2, &total, &lse_row);
      const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(t_o + 32 * c, o);
        tc_wait_ld();
        if (row_valid && o_part) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 v = make_float4(__uint_as_float(o[4 * i + 0]) * inv, __uint_as_float(o[4 * i + 1]) * inv,
                                         __uint_as_float(o[4 * i + 2]) * inv, __uint_as_float(o[4 * i + 3]) * inv);
            if (32 * c + 4 * i < p.head_dim) reinterpret_cast<float4*>(o_part)[8 * c + i] = v;
          }
        } else if (row_valid && p.o_wide) {
          // 32-byte stores: a lane writes whole sectors of its row (with 16-byte stores a warp instruction touches 32
          // sectors and fills half of each)
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              w[j] = pack_bf16x2(__uint_as_float(o[16 * i + 2 * j]) * inv, __uint_as_float(o[16 * i + 2 * j + 1]) * inv);
            if (32 * c + 16 * i < p.head_dim) st_global_v8(o_row + 32 * c + 16 * i, w);
          }
        } else if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            if (32 * c + 8 * i < p.head_dim) reinterpret_cast<uint4*>(o_row)[4 * c + i] = v;
          }
        }
      }
      if (row_valid) *lse_ptr = lse_row;
      tc_fence_before();
      trace_add(wctx, 23, trace_clock(wctx) - t_epi);
      trace_add(wctx, 24, 1);
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    // A wait ran out: give copies in flight time to land before the shared memory is released.
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 8) tmem_dealloc(tmem_base, 512);
}

// -------------------------------------------------------------------------------------------------- host side

// Work-item counters of the persistent kernels: a ring of counters per device inside the library (the library
// allocates no device memory). Every launch takes the next slot of its device's ring and zeroes it with a memset node
// on its own stream ahead of the kernel. Two launches use the same slot when kTileCounters other forward launches were
// issued on that device in between, or when one of them is a replay of a captured graph (a graph keeps the slot it was
// captured with). Sharing is harmless while the two are ordered on the GPU; two kernels that share a slot and overlap
// in time (different streams, no ordering) would draw from one counter and skip or repeat work items. The contract
// is therefore: per device, at most kTileCounters forward launches may be in flight or held in captured graphs that
// can run concurrently with later launches.
constexpr unsigned kTileCounters = 4096;
static __device__ int g_tile_counters[kTileCounters];

int acquire_tile_counter(cudaStream_t stream, int** counter) {
  static int* base[64] = {nullptr};
  static unsigned next[64] = {0};
  int device = 0;
  B200FA_CUDA_CHECK(cudaGetDevice(&device));
  B200FA_REQUIRE(device >= 0 && device < 64, "device ordinal %d is out of range", device);
  int* slot = nullptr;
  {
    std::lock_guard<std::mutex> lock(cache_mutex());
    if (!base[device]) {
      void* address = nullptr;
      B200FA_CUDA_CHECK(cudaGetSymbolAddress(&address, g_tile_counters));
      base[device] = static_cast<int*>(address);
    }
    slot = base[device] + next[device]++ % kTileCounters;
  }
  B200FA_CUDA_CHECK(cudaMemsetAsync(slot, 0, sizeof(int), stream));
  *counter = slot;
  return B200FA_OK;
}

// ---- split-KV (short queries over long keys; reference src/zigfa/_impl/forward.py:51-69)
// With few query tiles and many key blocks most SMs would idle while a few walk long key ranges: the key blocks of a
// tile are then dealt out in `splits` equal shares to as many work items, and split_combine_kernel merges the shares.
// The plan is a pure function of the shapes (it assumes the 148 SMs of a B200), so the workspace size it implies can be
// computed without a device.
constexpr int kPlanSms = 148;
// Entries of the work list that b200fa_fwd_noalloc keeps in device memory: (sequence, block) pairs; one entry covers 256
// query rows (128 at head_dim 256 and 512; 256 >> shift tokens of every head of a group when query heads are packed).
constexpr int kStaticWorkListEntries = 8192;

// log2 of the query heads packed into the rows of a work item of fwd_kernel (0 = no packing): problems whose query heads
// per key head are a power of two between 2 and 128 (fixed-length, packed and inter-sequence batches alike). B200FA_PACK_GQA=0 in the
// environment turns it off (tuning comparisons). A pure function of the shapes, like the split plan and the work-list
// size that build on it. The work list of a packed (varlen) batch then has entries of 256 >> shift tokens; a call whose
// workspace holds only the coarser list (the built-in scratch of b200fa_fwd_noalloc for a large batch) runs with one
// head per work item instead (prepare_forward).
static int pack_shift_of(const b200fa_problem& bp) {
  static const bool disabled = [] {
    const char* value = getenv("B200FA_PACK_GQA");
    return value && value[0] == '0';
  }();
  if (disabled || bp.head_dim > 128 || bp.heads_kv <= 0) return 0;
  if (bp.heads_q % bp.heads_kv) return 0;
  const int group = bp.heads_q / bp.heads_kv;
  if (group < 2 || group > kBlockM || (group & (group - 1))) return 0;
  int shift = 0;
  while ((1 << shift) < group) ++shift;
  // The work list is written one sequence per thread: entries of fewer than 16 tokens would make that loop long.
  if (bp.cu_seqlens_q && shift > 4) return 0;
  return shift;
}
int fwd_pack_shift(const b200fa_problem& bp) { return pack_shift_of(bp); }

struct SplitPlan {
  int splits;
  size_t o_bytes, lse_bytes;
};
static SplitPlan plan_split(const b200fa_problem& bp) {
  SplitPlan plan{1, 0, 0};
  if (bp.cu_seqlens_q || bp.visibility_bits || bp.head_dim > 128 || bp.batch <= 0 || bp.seqlen_q <= 0) return plan;
  const int tile_tokens = kFwdTileM >> pack_shift_of(bp);
  const int64_t tiles = (int64_t)bp.batch * (bp.heads_q >> pack_shift_of(bp)) * ceil_div(bp.seqlen_q, tile_tokens);
  int64_t keys = bp.seqlen_k;
  if (bp.window_left >= 0) {
    const int64_t reach = (int64_t)bp.window_left + imin(bp.seqlen_q, tile_tokens) + imax(bp.window_right, 0);
    keys = keys < reach ? keys : reach;
  }
  const int64_t blocks = (keys + kBlockN - 1) / kBlockN;
  // The reference's rule (src/zigfa/_impl/forward.py:23-25,60-62): keys >= 4 x queries, at least 256 keys per share.
  if (2 * tiles > kPlanSms || blocks < 4 || keys < 4 * (int64_t)bp.seqlen_q) return plan;
  int64_t splits = kPlanSms / tiles;
  if (splits > blocks / 2) splits = blocks / 2;  // at least two key blocks per share
  if (splits > 32) splits = 32;
  if (splits < 2) return plan;
  plan.splits = (int)splits;
  const size_t rows = (size_t)bp.batch * bp.seqlen_q;
  plan.o_bytes = ((size_t)splits * rows * bp.heads_q * bp.head_dim * 4 + 255) & ~size_t(255);
  plan.lse_bytes = ((size_t)splits * rows * bp.heads_q * 4 + 255) & ~size_t(255);
  return plan;
}
size_t fwd_split_workspace_bytes(const b200fa_problem& bp) {
  const SplitPlan plan = plan_split(bp);
  return plan.o_bytes + plan.lse_bytes;
}

// out = sum_i w_i O_i / sum_i w_i with w_i = exp(lse_i - max lse), lse = max + log(sum w_i); a row no share saw keeps
// zeros and -inf. One thread per (row, head, group of 4 columns).
__global__ void __launch_bounds__(256) split_combine_kernel(const float* __restrict__ o_partial,
                                                            const float* __restrict__ lse_partial, int splits,
                                                            int64_t rows, int seqlen_q, int heads, int head_dim,
                                                            __nv_bfloat16* __restrict__ out, int64_t o_bs, int64_t o_rs,
                                                            int64_t o_hs, float* __restrict__ lse, int64_t lse_bs,
                                                            int64_t lse_hs) {
  const int groups = head_dim / 4;
  const int64_t index = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= rows * heads * groups) return;
  const int g = (int)(index % groups);
  const int head = (int)((index / groups) % heads);
  const int64_t row = index / groups / heads;
  // The share with the largest log-sum-exp has the weight 1 exactly; the weights of the others are summed apart from
  // it and enter the logarithm as log1p(rest), so a row whose log-sum-exp is close to zero keeps its relative accuracy
  // across the shares (reference tests/test_softmax_fix.py:381-399).
  float top = -INFINITY;
  int top_share = 0;
  for (int i = 0; i < splits; ++i) {
    const float value = lse_partial[((int64_t)i * heads + head) * rows + row];
    if (value > top) {
      top = value;
      top_share = i;
    }
  }
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float rest = 0.f;
  if (top != -INFINITY) {
    for (int i = 0; i < splits; ++i) {
      const float w = i == top_share ? 1.f : __expf(lse_partial[((int64_t)i * heads + head) * rows + row] - top);
      const float4 o = *reinterpret_cast<const float4*>(o_partial + (((int64_t)i * rows + row) * heads + head) * head_dim + 4 * g);
      acc.x += w * o.x;
      acc.y += w * o.y;
      acc.z += w * o.z;
      acc.w += w * o.w;
      if (i != top_share) rest += w;
    }
  }
  const float total = top != -INFINITY ? 1.f + rest : 0.f;
  const float inv = total > 0.f ? 1.f / total : 0.f;
  const int64_t b = row / seqlen_q, r = row - b * seqlen_q;
  uint2 packed;
  packed.x = pack_bf16x2(acc.x * inv, acc.y * inv);
  packed.y = pack_bf16x2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(out + b * o_bs + r * o_rs + (int64_t)head * o_hs + 4 * g) = packed;
  if (g == 0) lse[b * lse_bs + (int64_t)head * lse_hs + r] = total > 0.f ? top + log1pf(rest) : -INFINITY;
}

int prepare_forward(const b200fa_fwd_args& a, cudaStream_t stream, int head_dim, int tile_rows, int kv_box_rows,
                    FwdParams* params, CUtensorMap* map_q, CUtensorMap* map_k, CUtensorMap* map_v, bool* nothing_to_do,
                    int v_box_rows, int pack_shift) {
  const b200fa_problem& bp = a.problem;
  const int D = bp.head_dim;  // columns of the tensors; `head_dim` is the width the kernel is compiled for
  (void)head_dim;
  const bool packed = bp.cu_seqlens_q != nullptr;
  FwdParams& p = *params;
  *nothing_to_do = true;
  p.prob = to_problem(bp);
  p.scale_log2 = bp.softmax_scale * 1.4426950408889634f;
  p.o = static_cast<__nv_bfloat16*>(a.out);
  p.o_batch_stride = packed ? 0 : a.out_stride[0];
  p.o_row_stride = a.out_stride[1];
  p.o_head_stride = a.out_stride[2];
  p.lse = a.softmax_lse;
  p.lse_batch_stride = packed ? 0 : a.lse_stride[0];
  p.lse_head_stride = a.lse_stride[1];
  // every output row starts on a 32-byte boundary and holds a whole number of 32-byte pieces
  p.o_wide = (reinterpret_cast<uintptr_t>(a.out) & 31) == 0 && (packed || a.out_stride[0] % 16 == 0) &&
             a.out_stride[1] % 16 == 0 && a.out_stride[2] % 16 == 0 && bp.head_dim % 16 == 0;
  p.work_list = nullptr;
  p.splits = 1;
  p.o_partial = nullptr;
  p.lse_partial = nullptr;
  p.partial_rows = 0;
  p.pack_shift = pack_shift;
  p.tile_counter = nullptr;
  p.m_blocks = 0;
  p.head_dim = bp.head_dim;
  p.status = device_status_word();
  if (!p.status) return B200FA_ERR_CUDA;
  p.trace = trace_buffer();

  const int64_t rows_q = bp.seqlen_q, rows_k = bp.seqlen_k;
  const int64_t tensor_batch = packed ? 1 : bp.batch;
  if (packed) {
    int64_t entries = work_list_entries(rows_q, bp.batch, tile_rows >> p.pack_shift);
    if (p.pack_shift > 0 && a.workspace_bytes < static_cast<size_t>(entries) * 8) {
      // The finer work list of packed query heads does not fit what the caller has: one head per work item (same
      // results; b200fa_fwd_workspace_bytes asks for the finer list).
      p.pack_shift = 0;
      entries = work_list_entries(rows_q, bp.batch, tile_rows);
    }
    const int entry_rows = tile_rows >> p.pack_shift;  // tokens per work-list entry
    B200FA_REQUIRE(a.workspace_bytes >= static_cast<size_t>(entries) * 8 && (entries == 0 || a.workspace),
                   "forward workspace is too small: need %zu bytes (%zu recommended)", static_cast<size_t>(entries) * 8,
                   b200fa_fwd_workspace_bytes(&bp));
    if (entries == 0) return B200FA_OK;
    const int32_t* other = bp.cu_visible_k ? bp.cu_visible_k : bp.cu_seqlens_k;
    int status = b200fa_work_list(bp.cu_seqlens_q, other, bp.batch, entry_rows, 1, (int32_t)entries,
                                  static_cast<int32_t*>(a.workspace), stream);
    if (status != B200FA_OK) return status;
    p.work_list = static_cast<const int2*>(a.workspace);
    p.num_tiles = (int)(entries * (bp.heads_q >> p.pack_shift));
  } else {
    p.m_blocks = ceil_div(bp.seqlen_q, tile_rows >> p.pack_shift);
    p.num_tiles = p.m_blocks * bp.batch * (bp.heads_q >> p.pack_shift);
  }
  p.ratio = bp.heads_kv > 0 ? bp.heads_q / bp.heads_kv : 1;
  {
    const int group = p.pack_shift ? 1 : p.ratio;
    p.div_per_group = FastDiv::make((uint32_t)(p.m_blocks * group));
    p.div_group = FastDiv::make((uint32_t)group);
    p.div_heads_kv = FastDiv::make((uint32_t)bp.heads_kv);
    p.div_heads_q = FastDiv::make((uint32_t)(bp.heads_q >> p.pack_shift));  // work items per work-list entry
    p.div_ratio = FastDiv::make((uint32_t)p.ratio);
  }
  if (p.num_tiles <= 0 || rows_q == 0) return B200FA_OK;

  int status = encode_tensor_map(map_q, a.q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, bp.heads_q, rows_q, tensor_batch,
                                 a.q_stride[2], a.q_stride[1], packed ? rows_q * a.q_stride[1] : a.q_stride[0], 64,
                                 kBlockM >> p.pack_shift, 1 << p.pack_shift);
  if (status != B200FA_OK) return status;
  // An empty key tensor still needs valid maps: give them one row of the query tensor (never read, no key blocks).
  const bool no_keys = rows_k == 0;
  const void* k_base = no_keys ? a.q : a.k;
  const void* v_base = no_keys ? a.q : a.v;
  const int64_t k_rows = no_keys ? 1 : rows_k;
  status = encode_tensor_map(map_k, k_base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, no_keys ? 1 : bp.heads_kv, k_rows,
                             tensor_batch, no_keys ? D : a.k_stride[2], no_keys ? D : a.k_stride[1],
                             no_keys ? D : (packed ? k_rows * a.k_stride[1] : a.k_stride[0]), 64, kv_box_rows);
  if (status != B200FA_OK) return status;
  status = encode_tensor_map(map_v, v_base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, D, no_keys ? 1 : bp.heads_kv, k_rows,
                             tensor_batch, no_keys ? D : a.v_stride[2], no_keys ? D : a.v_stride[1],
                             no_keys ? D : (packed ? k_rows * a.v_stride[1] : a.v_stride[0]), 64,
                             v_box_rows > 0 ? v_box_rows : kv_box_rows);
  if (status != B200FA_OK) return status;
  status = acquire_tile_counter(stream, &p.tile_counter);
  if (status != B200FA_OK) return status;
  *nothing_to_do = false;
  return B200FA_OK;
}

template <int D>
static int launch_fwd_d(const b200fa_fwd_args& a, cudaStream_t stream) {
  using Cfg = FwdConfig<D>;
  FwdParams p;
  CUtensorMap map_q, map_k, map_v;
  bool nothing_to_do = false;
  int status = prepare_forward(a, stream, D, kFwdTileM, kBlockN, &p, &map_q, &map_k, &map_v, &nothing_to_do, 0,
                               pack_shift_of(a.problem));
  if (status != B200FA_OK || nothing_to_do) return status;
  int sms = 0;
  status = device_sm_count(&sms);
  if (status != B200FA_OK) return status;
  // Split-KV when the plan asks for it and the caller's workspace has room for the partial results (an entry point
  // that brings its own small scratch runs the same problem unsplit).
  const b200fa_problem& bp = a.problem;
  const SplitPlan plan = plan_split(bp);
  const bool split = plan.splits > 1 && a.workspace && a.workspace_bytes >= plan.o_bytes + plan.lse_bytes &&
                     reinterpret_cast<uintptr_t>(a.workspace) % 16 == 0;
  if (split) {
    p.splits = plan.splits;
    p.o_partial = static_cast<float*>(a.workspace);
    p.lse_partial = reinterpret_cast<float*>(static_cast<uint8_t*>(a.workspace) + plan.o_bytes);
    p.partial_rows = (int64_t)bp.batch * bp.seqlen_q;
    p.num_tiles *= plan.splits;
  }
  const int grid = p.num_tiles < sms ? p.num_tiles : sms;
  // Three instances: split-KV, problems with visibility bits (inter-sequence batches), and the plain one.
  auto launch = [&](auto kernel, bool (&attribute_set)[64]) -> int {
    const int set = set_dynamic_smem_once(reinterpret_cast<const void*>(kernel), Cfg::kSmemBytes, attribute_set);
    if (set != B200FA_OK) return set;
    kernel<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
    return B200FA_OK;
  };
  static bool set_split[64] = {false}, set_bits[64] = {false}, set_plain[64] = {false};
  if (split) {
    status = launch(&fwd_kernel<D, true, false>, set_split);
  } else if (bp.visibility_bits) {
    status = launch(&fwd_kernel<D, false, true>, set_bits);
  } else {
    status = launch(&fwd_kernel<D, false, false>, set_plain);
  }
  if (status != B200FA_OK) return status;
  B200FA_CUDA_CHECK(cudaGetLastError());
  if (split) {
    const int64_t threads = p.partial_rows * bp.heads_q * (bp.head_dim / 4);
    split_combine_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
        p.o_partial, p.lse_partial, plan.splits, p.partial_rows, bp.seqlen_q, bp.heads_q, bp.head_dim,
        static_cast<__nv_bfloat16*>(a.out), a.out_stride[0], a.out_stride[1], a.out_stride[2], a.softmax_lse,
        a.lse_stride[0], a.lse_stride[1]);
    B200FA_CUDA_CHECK(cudaGetLastError());
  }
  return B200FA_OK;
}

int launch_fwd(const b200fa_fwd_args& a, cudaStream_t stream) {
  switch (a.problem.head_dim) {
    case 64:
      return launch_fwd_d<64>(a, stream);
    case 72:   // compiled for 128 columns; TMA zero-fills the missing ones and the epilogue skips them
    case 96:
    case 128:
      return launch_fwd_d<128>(a, stream);
    case 256: {
      // B200FA_FWD_D256_PAIR=1 in the environment selects the two-CTA variant (same results bit for bit, measured
      // slower: kept for tuning work on `cta_group::2` tiles).
      static const bool pair_kernel = [] {
        const char* value = getenv("B200FA_FWD_D256_PAIR");
        return value && value[0] == '1';
      }();
      return pair_kernel ? launch_fwd_256_pair(a, stream) : launch_fwd_256(a, stream);
    }
    case 512:
      return launch_fwd_512(a, stream);
    default:
      set_error("head_dim %d is not supported by the forward kernel (supported: 64, 72, 96, 128, 256, 512)", a.problem.head_dim);
      return B200FA_ERR_UNSUPPORTED;
  }
}

}  // namespace b200fa

// -------------------------------------------------------------------------------------------------- no-allocation entry
// Forward attention for callers that cannot hand the library a workspace. The only scratch the forward pass needs is
// the work list of a packed (varlen / inter-sequence) batch; here it lives in a fixed array in device memory that
// belongs to the library. Every GPU that loads the library holds these 64 KiB until the process exits.
namespace b200fa {
static __device__ __align__(256) int32_t g_static_work_list[2 * kStaticWorkListEntries];

// Device address of the array on the current device. `g_static_work_list` as written in host code is only a host-side
// handle for the symbol, so the address a kernel can use has to be asked for, once per device, with that device current.
static int static_work_list(int32_t** address) {
  static int32_t* cached[64] = {nullptr};
  int device = 0;
  B200FA_CUDA_CHECK(cudaGetDevice(&device));
  B200FA_REQUIRE(device >= 0 && device < 64, "device index %d is out of range", device);
  std::lock_guard<std::mutex> lock(cache_mutex());
  if (!cached[device]) {
    int32_t* pointer = nullptr;
    B200FA_CUDA_CHECK(cudaGetSymbolAddress(reinterpret_cast<void**>(&pointer), g_static_work_list));
    cached[device] = pointer;
  }
  *address = cached[device];
  return B200FA_OK;
}
}  // namespace b200fa

extern "C" int b200fa_fwd_noalloc(const b200fa_fwd_args* args, void* stream) {
  using namespace b200fa;
  B200FA_REQUIRE(args != nullptr, "null arguments");
  const b200fa_problem& problem = args->problem;
  B200FA_REQUIRE(problem.batch >= 0 && problem.seqlen_q >= 0 && problem.seqlen_k >= 0, "negative sizes");
  // Only the work list of a packed batch is scratch this entry point must provide; the partial results the split-KV path
  // of a fixed-length problem would like are optional (without room for them the problem runs unsplit).
  // (the list with one head per work item: where b200fa_fwd_workspace_bytes asks for the finer list of packed query
  // heads and that does not fit, the batch runs unpacked)
  const int tile_rows = problem.head_dim >= 256 ? kBlockM : kFwdTileM;
  const size_t needed =
      problem.cu_seqlens_q ? static_cast<size_t>(work_list_entries(problem.seqlen_q, problem.batch, tile_rows)) * 8 : 0;
  B200FA_REQUIRE(needed <= sizeof(int32_t) * 2 * kStaticWorkListEntries,
                 "b200fa_fwd_noalloc: the batch needs a work list of %zu bytes (%zu entries of %d query rows at "
                 "head_dim %d) but the built-in scratch holds %zu bytes (%d entries); use b200fa_fwd with a "
                 "caller-provided workspace",
                 needed, needed / 8, tile_rows, problem.head_dim, sizeof(int32_t) * 2 * kStaticWorkListEntries,
                 kStaticWorkListEntries);
  int32_t* scratch = nullptr;
  const int status = static_work_list(&scratch);
  if (status != B200FA_OK) return status;
  b200fa_fwd_args with_scratch = *args;
  with_scratch.workspace = scratch;
  with_scratch.workspace_bytes = sizeof(int32_t) * 2 * kStaticWorkListEntries;
  return b200fa_fwd(&with_scratch, stream);
}
