// Forward attention kernel for head_dim 256 on sm_100a with 128-key blocks (the reference builds head_dim 256 forward
// as a 2-CTA variant of zig/flash_fwd_sm100.zig, zig/configurations.zig:1567-1574; this is a single-CTA design).
//
// A key block has 128 keys, so the score MMA is 128 x 128 x 16 (8 KB of operands for 64 cycles of tensor work) like in
// the head_dim 128 kernel; with 64-key blocks (the kernel of fwd_d512.cu, which served head_dim 256 before) a
// 128 x 64 x 16 MMA reads 6 KB for 32 cycles and the score product is bound by shared-memory bandwidth (1010 against
// 1290 TF/s on batch 4, seqlen 8192, heads 16/4, causal):
//   S(n)   = Q K_n^T     SS-MMA 128x128x256 -> TMEM buffer n & 1, columns [128 b, 128 b + 128)
//   P(n)                 BF16, over columns [64,128) of the same buffer (whose scores the softmax warps hold in registers)
//   O     += P(n) V_n    TS-MMA 128x256x128 -> TMEM columns [256, 512), issued in two key halves
// One 128-row query stage with the score tile double-buffered: the MMA warp issues S(n + 2) right after O += P(n) V_n, so
// the softmax of block n + 1 overlaps the PV product of block n and the scores of block n + 2.
// Shared memory: Q 64 KB, one K slot of 64 KB (128 keys x 256 columns; the next K block is loaded as soon as the score
// MMA of the current one has completed, which the loader learns from the barrier of the score buffer) and a ring of three V slots of 32 KB (64 keys x 256 columns each).
// Warps 0-3: softmax and epilogue (thread = query row), warp 4: MMA issue, warp 5: TMA loads, warps 6-7: spare.
#include "fwd_common.cuh"

namespace b200fa {

namespace d256 {
constexpr int D = 256;
constexpr int kVSlots = 3;                        // ring of V half-blocks
constexpr int kQBytes = kBlockM * D * 2;          // 64 KB
constexpr int kKBytes = kBlockN * D * 2;          // 64 KB
constexpr int kVBytes = 64 * D * 2;               // 32 KB: 64 keys
constexpr int kQPanel = kBlockM * 128;            // 64-column panel of Q (128 rows)
constexpr int kKPanel = kBlockN * 128;            // 64-column panel of K (128 rows)
constexpr int kVPanel = 64 * 128;                 // 64-column panel of a V half-block (64 rows)
constexpr int kSmemBytes = kQBytes + kKBytes + kVSlots * kVBytes + 1024 + 512;
constexpr int kThreads = 256;
constexpr int kTmemO = 256;
static_assert(kSmemBytes <= 232448, "shared memory exceeds the per-CTA limit");
}  // namespace d256

template <bool kBits>  // false: no visibility bits, the scan of the key cursor is compiled out (see KeyCursorT)
__global__ void __launch_bounds__(d256::kThreads, 1)
fwd_d256_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const __grid_constant__ FwdParams p) {
  using namespace d256;
  constexpr int NV = kVSlots;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_q = smem_base;
  const uint32_t smem_k = smem_q + kQBytes;
  const uint32_t smem_v = smem_k + kKBytes;
  const uint32_t bars = smem_v + NV * kVBytes;
  const uint32_t bar_q_full = bars, bar_q_empty = bars + 8, bar_k_full = bars + 16;
  const uint32_t bar_v_full = bars + 32, bar_v_empty = bar_v_full + 8 * NV;  // [NV] each
  const uint32_t bar_s_full = bar_v_empty + 8 * NV;                          // [2]
  const uint32_t bar_p_half = bar_s_full + 16;                               // [2]
  const uint32_t bar_p_full = bar_p_half + 16;                               // [2]
  const uint32_t bar_pv_done = bar_p_full + 16;
  const uint32_t tmem_slot = bar_pv_done + 8, abort_slot = tmem_slot + 4;
  TileQueue tiles;
  tiles.place(bars + 256);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (abort_slot - smem_u32(smem_raw)));
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  const WaitCtx wctx{abort_flag, p.status, p.trace};
  int trace_n = 0;  // timeline of the first work item of CTA 0 (tuning builds)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    mbar_init(bar_k_full, 1);
    for (int i = 0; i < NV; ++i) {
      mbar_init(bar_v_full + 8 * i, 1);
      mbar_init(bar_v_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full + 8 * i, 1);
      mbar_init(bar_p_half + 8 * i, 128);
      mbar_init(bar_p_full + 8 * i, 128);
    }
    mbar_init(bar_pv_done, 1);
    tiles.init(1 + 4);  // the MMA thread and the four softmax warps
    fence_barrier_init();
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_smem;
  const Problem& pr = p.prob;

  // Number of key blocks of a work item (every role needs it to know where the pipeline ends).
  auto count_blocks = [&](const FwdTile& t) {
    KeyCursorT<kBits> cur;
    cur.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
    OtherBlock kb;
    int n = 0;
    while (cur.next(&kb)) ++n;
    return n;
  };

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer
    // Load order = consumption order of the MMA warp: K0, K1, then V_hi(n), V_lo(n), K(n + 2) for n = 0, 1, ...
    if (lane == 0) {
      uint32_t k_count = 0, v_count = 0, q_count = 0, drawn = 0;
      bool ok = true;
      // The K slot is free when the score MMAs of the block before have completed, which is what the barrier of their
      // score buffer announces: the loader follows those barriers (every completion of both, in order) instead of a
      // barrier of its own, which saves the MMA stream one tcgen05.commit per key block.
      uint32_t s_issued[2] = {0, 0};  // score products issued into each buffer so far
      int prev_buffer = -1;
      uint32_t prev_phase = 0;
      auto load_k = [&](int head, int row, int batch_coord, int buffer) -> bool {
        if (prev_buffer >= 0 && !mbar_wait(bar_s_full + 8 * prev_buffer, prev_phase, wctx, kWaitKvEmpty)) return false;
        prev_buffer = buffer;
        prev_phase = s_issued[buffer] & 1;
        ++s_issued[buffer];
        mbar_expect_tx(bar_k_full, kKBytes);
#pragma unroll
        for (int h = 0; h < 4; ++h) tma_load_4d(smem_k + h * kKPanel, &map_k, bar_k_full, h * 64, head, row, batch_coord);
        trace_event(wctx, blockIdx.x == 0 && q_count == 1, 3, trace_n, 1000 + (k_count % 100));  // K load issued
        ++k_count;
        return true;
      };
      auto load_v_half = [&](int head, int row, int batch_coord) -> bool {  // 64 keys starting at `row`
        const uint32_t slot = v_count % NV, phase = (v_count / NV) & 1;
        if (!mbar_wait(bar_v_empty + 8 * slot, phase ^ 1, wctx, kWaitKvEmpty)) return false;
        const uint32_t bar = bar_v_full + 8 * slot;
        mbar_expect_tx(bar, kVBytes);
#pragma unroll
        for (int h = 0; h < 4; ++h) tma_load_4d(smem_v + slot * kVBytes + h * kVPanel, &map_v, bar, h * 64, head, row, batch_coord);
        trace_event(wctx, blockIdx.x == 0 && q_count == 1, 3, trace_n, 1100 + (v_count % 100));  // V half load issued
        ++v_count;
        return true;
      };
      for (int tile; ok && (tile = tiles.push(drawn, p.tile_counter, p.num_tiles, wctx)) >= 0;) {
        FwdTile t = decode_tile(p, tile, kBlockM);
        if (!t.valid) continue;
        const int n_blocks = count_blocks(t);
        if (n_blocks == 0) continue;
        KeyCursorT<kBits> cur_k, cur_v;
        cur_k.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
        cur_v.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
        OtherBlock kb;
        if (!mbar_wait(bar_q_empty, (q_count & 1) ^ 1, wctx, kWaitQEmpty)) { ok = false; break; }
        ++q_count;
        mbar_expect_tx(bar_q_full, kQBytes);
#pragma unroll
        for (int h = 0; h < 4; ++h)
          tma_load_4d(smem_q + h * kQPanel, &map_q, bar_q_full, h * 64, t.head, t.s.q0 + t.m0, t.s.batch_coord);
        for (int i = 0; ok && i < imin(2, n_blocks); ++i) {
          cur_k.next(&kb);
          ok = load_k(t.kv_head, kb.row, t.s.batch_coord, i);
        }
        for (int n = 0; ok && n < n_blocks; ++n) {
          cur_v.next(&kb);
          ok = load_v_half(t.kv_head, kb.row + 64, t.s.batch_coord) && load_v_half(t.kv_head, kb.row, t.s.batch_coord);
          if (ok && n + 2 < n_blocks) {
            cur_k.next(&kb);
            ok = load_k(t.kv_head, kb.row, t.s.batch_coord, n & 1);
          }
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(kBlockM, kBlockN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kBlockM, D, 0, 1);
      uint32_t k_count = 0, v_count = 0, q_count = 0, popped = 0;
      uint32_t p_phase[2] = {0, 0};
      bool ok = true;
      // S = Q K^T into score buffer `buffer`; the K slot is released when these MMAs have completed.
      auto issue_s = [&](int buffer) -> bool {
        if (!mbar_wait(bar_k_full, k_count & 1, wctx, kWaitKvFull)) return false;
        trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 200 + (k_count % 100));  // K present
        ++k_count;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          umma_ss(tmem_base + buffer * 128, umma_smem_desc(smem_q + (kk >> 2) * kQPanel + (kk & 3) * 32, 16, 1024),
                  umma_smem_desc(smem_k + (kk >> 2) * kKPanel + (kk & 3) * 32, 16, 1024), idesc_s, kk > 0);
        }
        tc_commit(bar_s_full + 8 * buffer);
        trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 100 + ((k_count - 1) % 100));  // S issued
        return true;
      };
      // O += P[:, 64 h .. 64 h + 64) V_half: the next V slot of the ring holds those 64 keys.
      auto issue_pv_half = [&](int buffer, int half, bool accumulate) -> bool {
        const uint32_t slot = v_count % NV, phase = (v_count / NV) & 1;
        if (!mbar_wait(bar_v_full + 8 * slot, phase, wctx, kWaitKvFull)) return false;
        ++v_count;
        tc_fence_after();
        const uint32_t v_smem = smem_v + slot * kVBytes;
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
          umma_ts(tmem_base + kTmemO, tmem_base + buffer * 128 + 64 + (4 * half + kk) * 8,
                  umma_smem_desc(v_smem + kk * 2048, kVPanel, 1024), idesc_pv, accumulate || kk > 0);
        }
        tc_commit(bar_v_empty + 8 * slot);
        return true;
      };
      for (int tile; ok && (tile = tiles.pop_thread(popped, wctx)) >= 0;) {
        FwdTile t = decode_tile(p, tile, kBlockM);
        if (!t.valid) continue;
        const int n_blocks = count_blocks(t);
        if (n_blocks == 0) continue;
        const uint32_t q_phase = q_count & 1;
        ++q_count;
        if (!mbar_wait(bar_q_full, q_phase, wctx, kWaitQFull)) { ok = false; break; }
        for (int i = 0; ok && i < imin(2, n_blocks); ++i) ok = issue_s(i);
        for (int n = 0; ok && n < n_blocks; ++n) {
          const int buffer = n & 1;
          // keys [64,128) first: their probabilities are stored first
          if (!mbar_wait(bar_p_half + 8 * buffer, p_phase[buffer], wctx, kWaitPFull)) { ok = false; break; }
          trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 300 + (n % 100));  // first half of P present
          if (!issue_pv_half(buffer, 1, n > 0)) { ok = false; break; }
          trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 400 + (n % 100));  // PV of the first half issued
          if (!mbar_wait(bar_p_full + 8 * buffer, p_phase[buffer], wctx, kWaitPFull)) { ok = false; break; }
          trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 500 + (n % 100));  // all of P present
          p_phase[buffer] ^= 1;
          if (!issue_pv_half(buffer, 0, true)) { ok = false; break; }
          tc_commit(bar_pv_done);
          trace_event(wctx, blockIdx.x == 0 && q_count == 1, 0, trace_n, 600 + (n % 100));  // PV of the second half issued
          if (n + 2 < n_blocks) ok = issue_s(buffer);
        }
        if (ok) tc_commit(bar_q_empty);
      }
      if (ok && q_count > 0) mbar_wait(bar_q_empty, (q_count - 1) & 1, wctx, kWaitQEmpty);
    }
  } else if (warp < 4) {
    // ------------------------------------------------------------------ softmax + epilogue (thread = query row)
    const int row_in_tile = warp * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
    const uint32_t t_o = tmem_base + lane_addr + kTmemO;
    const float scale_log2 = p.scale_log2;
    uint32_t blocks = 0, popped = 0;
    uint32_t s_phase[2] = {0, 0};
    bool ok = true;
    for (int tile; ok && (tile = tiles.pop_warp(popped, wctx)) >= 0;) {
      FwdTile t = decode_tile(p, tile, kBlockM);
      if (!t.valid) continue;
      const int row = t.m0 + row_in_tile;
      KeyCursorT<kBits> cur;
      cur.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
      const int band_lo = cur.band.lo(row), band_hi = cur.band.hi(row);
      float m = -INFINITY, l = 0.f;
      TopApart top;  // keys set aside for the log-sum-exp of rows with a near-zero maximum (fwd_common.cuh)
      int tile_blocks = 0;
      OtherBlock kb;
      while (cur.next(&kb)) {
        const int buffer = tile_blocks & 1;
        const uint32_t t_s = tmem_base + lane_addr + buffer * 128;
        if (!mbar_wait_warp(bar_s_full + 8 * buffer, s_phase[buffer], wctx, kWaitSFull)) { ok = false; break; }
        s_phase[buffer] ^= 1;
        tc_fence_after();
        const bool traced = blockIdx.x == 0 && threadIdx.x == 0 && popped == 1;
        trace_event(wctx, traced, 1, trace_n, 2000 + (tile_blocks % 100));  // scores present
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
        // [64,128) stay in registers, because P goes over them.
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
        const bool counting = __any_sync(0xffffffffu, set_apart);
        trace_event(wctx, traced, 1, trace_n, 2100 + (tile_blocks % 100));  // row maximum known
        const bool grow = (m_new - m) * scale_log2 > 8.f;  // also true when m is -inf and m_new is finite
        if (__any_sync(0xffffffffu, grow)) {
          float alpha = 1.f;
          if (grow) {
            alpha = (m == -INFINITY) ? 0.f : ex2_approx((m - m_new) * scale_log2);
            l *= alpha;
            m = m_new;
          }
          if (tile_blocks > 0) {
            if (!mbar_wait_warp(bar_pv_done, (blocks - 1) & 1, wctx, kWaitPvDone)) { ok = false; break; }
            tc_fence_after();
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
        const float mc = (m == -INFINITY) ? 0.f : m * scale_log2;
        const float2 scale2 = make_float2(scale_log2, scale_log2), shift2 = make_float2(-mc, -mc);
        float sum_counted = 0.f;
        if (counting)  // rare: the block sum without the keys set aside, from the scores still in TMEM
          sum_counted = sum_without_keys_apart<kBlockN>(top, l, set_apart, block_max, t_s, masked, lo, hi, scale_log2, mc);
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
              e.x = ex2_approx(x.x);
              e.y = ex2_approx(x.y);
              if (i & 1) sum_b = __fadd2_rn(sum_b, e); else sum_a = __fadd2_rn(sum_a, e);
              packed[i] = pack_bf16x2(e.x, e.y);
            }
            tmem_st16(t_s + 64 + first_p_column + 16 * c, packed);
          }
        };
        // Pass 2 for columns [0,64): the loads are in flight while the upper half is exponentiated.
        tmem_ld32(t_s, reinterpret_cast<uint32_t*>(low));
        tmem_ld32(t_s + 32, reinterpret_cast<uint32_t*>(low) + 32);
        exponentiate(high, 32);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_half + 8 * buffer);  // keys [64,128): their half of the PV product may start
        trace_event(wctx, traced, 1, trace_n, 2200 + (tile_blocks % 100));  // first half of P stored
        tc_wait_ld();
        if (masked) apply_mask(low, 0);
        exponentiate(low, 0);
        l += counting ? sum_counted : (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        trace_event(wctx, traced, 1, trace_n, 2300 + (tile_blocks % 100));  // second half exponentiated
        // Observe the PV product of the previous block before releasing this one: the scores of block n only prove that
        // PV(n - 2) has completed, and a parity wait cannot tell a barrier that is two completions behind from one that
        // is done.
        if (tile_blocks > 0 && !mbar_wait_warp(bar_pv_done, (blocks - 1) & 1, wctx, kWaitPvDone)) { ok = false; break; }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_full + 8 * buffer);
        trace_event(wctx, traced, 1, trace_n, 2400 + (tile_blocks % 100));  // all of P stored
        ++blocks;
        ++tile_blocks;
      }
      if (!ok) break;
      // ---- epilogue
      const bool row_valid = row < t.s.lq;
      __nv_bfloat16* o_row = p.o + t.s.batch_coord * p.o_batch_stride + (int64_t)(t.s.q0 + row) * p.o_row_stride +
                             (int64_t)t.head * p.o_head_stride;
      float* lse_ptr = p.lse + t.s.batch_coord * p.lse_batch_stride + (int64_t)t.head * p.lse_head_stride + t.s.q0 + row;
      if (tile_blocks == 0) {
        if (row_valid) {
          const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(o_row)[c] = zero;
          *lse_ptr = -INFINITY;
        }
        continue;
      }
      if (!mbar_wait_warp(bar_pv_done, (blocks - 1) & 1, wctx, kWaitEpilogue)) { ok = false; break; }
      tc_fence_after();
      float total, lse_row;
      row_totals(m, l, top.ones, top.apart, scale_log2, &total, &lse_row);
      const float inv = total > 0.f ? 1.f / total : 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(t_o + 32 * c, o);
        tc_wait_ld();
        if (row_valid && p.o_wide) {  // 32-byte stores: a lane writes whole sectors of its row
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              w[j] = pack_bf16x2(__uint_as_float(o[16 * i + 2 * j]) * inv, __uint_as_float(o[16 * i + 2 * j + 1]) * inv);
            st_global_v8(o_row + 32 * c + 16 * i, w);
          }
        } else if (row_valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack_bf16x2(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            v.y = pack_bf16x2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            v.z = pack_bf16x2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            v.w = pack_bf16x2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
            reinterpret_cast<uint4*>(o_row)[4 * c + i] = v;
          }
        }
      }
      if (row_valid) *lse_ptr = lse_row;
      tc_fence_before();
    }
  }

  // ------------------------------------------------------------------ teardown
  if (*abort_flag) {
    for (int i = 0; i < 50; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 4) tmem_dealloc(tmem_base, 512);
}

int launch_fwd_256(const b200fa_fwd_args& a, cudaStream_t stream) {
  FwdParams p;
  CUtensorMap map_q, map_k, map_v;
  bool nothing_to_do = false;
  int status = prepare_forward(a, stream, d256::D, kBlockM, kBlockN, &p, &map_q, &map_k, &map_v, &nothing_to_do, 64);
  if (status != B200FA_OK || nothing_to_do) return status;
  int sms = 0;
  status = device_sm_count(&sms);
  if (status != B200FA_OK) return status;
  const int grid = p.num_tiles < sms ? p.num_tiles : sms;
  if (a.problem.visibility_bits) {
    static bool attribute_set[64] = {false};
    status = set_dynamic_smem_once(reinterpret_cast<const void*>(&fwd_d256_kernel<true>), d256::kSmemBytes, attribute_set);
    if (status != B200FA_OK) return status;
    fwd_d256_kernel<true><<<grid, d256::kThreads, d256::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
  } else {
    static bool attribute_set[64] = {false};
    status = set_dynamic_smem_once(reinterpret_cast<const void*>(&fwd_d256_kernel<false>), d256::kSmemBytes, attribute_set);
    if (status != B200FA_OK) return status;
    fwd_d256_kernel<false><<<grid, d256::kThreads, d256::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
  }
  B200FA_CUDA_CHECK(cudaGetLastError());
  return B200FA_OK;
}

}  // namespace b200fa
