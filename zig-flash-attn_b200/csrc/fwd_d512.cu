// Forward attention kernel for head_dim 512 on sm_100a, built on a head_dim 256 kernel with 64-key blocks (kSplit = 1,
// kept as the base case of the template; head_dim 256 itself is served by the 128-key kernel of fwd_d256.cu).
//
// With 256 output columns the FP32 accumulator O takes half of TMEM, so there is one query stage: a work item is 128
// query rows of one head. Keys are taken 64 at a time, and the score tile S (128 x 64) is double-buffered instead:
//   S(n)   = Q K_n^T     SS-MMA 128x64x256  -> TMEM buffer n & 1, columns [128 b, 128 b + 64)
//   P(n)                 BF16, columns [128 b + 64, 128 b + 96) of the same buffer (no aliasing with S)
//   O     += P(n) V_n    TS-MMA 128x256x64  -> TMEM columns [256, 512)
// The MMA warp issues S(n + 2) right after O += P(n) V_n, so while the softmax warps work on block n + 1 the tensor pipe
// runs the PV product of block n and the scores of block n + 2. Per block the tensor work (2 x 512 cycles) about equals
// the softmax work of one warpgroup, which is why one softmax warpgroup is enough here.
// Warps 0-3: softmax and epilogue (thread = query row), warp 4: MMA issue, warp 5: TMA loads, warps 6-7: spare.
//
// head_dim 512 (kSplit = 2) runs the same kernel: an accumulator of 512 columns would take all of TMEM, so a work
// item is split in two, one per 256 output columns (tile index = 2 * item + half). Both halves compute the full
// scores (reduction over 512 columns: a key block is two ring slots) and their own half of P V. The query tile takes
// 128 KB of shared memory, which leaves three ring slots.
#include "fwd_common.cuh"

namespace b200fa {

namespace wide {
constexpr int D = 256;                            // output columns of a CTA; the reduction runs over kSplit * D columns
constexpr int kSubN = 64;                         // keys per block
constexpr int kKvBytes = kSubN * D * 2;           // 32 KB: one ring slot (64 keys x 256 columns)
constexpr int kQPanel = kBlockM * 128;            // 64-column panel of Q
constexpr int kKvPanel = kSubN * 128;             // 64-column panel of K / V
constexpr int kThreads = 256;
constexpr int kTmemO = 256;
template <int kSplit>
struct Config {
  static constexpr int kStages = kSplit == 1 ? 5 : 3;            // K/V ring slots
  static constexpr int kQBytes = kBlockM * D * kSplit * 2;       // 64 KB or 128 KB
  static constexpr int kSmemBytes = kQBytes + kStages * kKvBytes + 1024 + 256;
  static_assert(kSmemBytes <= 232448, "shared memory exceeds the per-CTA limit");
};
}  // namespace wide

// Yields the key blocks of a KeyCursor as 64-key halves.
struct SubBlockCursor {
  KeyCursor cursor;
  OtherBlock block;
  int half;
  __device__ void init(const Problem* problem, int seq, const SeqInfo& s, int m0, int m1) {
    cursor.init(problem, seq, s, m0, m1);
    half = 2;
  }
  __device__ bool next(OtherBlock* out) {
    if (half >= 2) {
      if (!cursor.next(&block)) return false;
      half = 0;
    }
    *out = block;
    out->row = block.row + half * wide::kSubN;
    out->col0 = block.col0 + half * wide::kSubN;
    ++half;
    return true;
  }
};

template <int kSplit>
__global__ void __launch_bounds__(wide::kThreads, 1)
fwd_wide_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ FwdParams p) {
  using namespace wide;
  constexpr int NS = Config<kSplit>::kStages;
  constexpr int kQBytes = Config<kSplit>::kQBytes;
  const int num_tiles = p.num_tiles * kSplit;  // tile = kSplit * work item + half of the output columns
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_q = smem_base;
  const uint32_t smem_kv = smem_base + kQBytes;
  const uint32_t bars = smem_kv + NS * kKvBytes;
  const uint32_t bar_q_full = bars, bar_q_empty = bars + 8;
  const uint32_t bar_kv_full = bars + 16, bar_kv_empty = bar_kv_full + 8 * NS;
  const uint32_t bar_s_full = bar_kv_empty + 8 * NS;  // [2]
  const uint32_t bar_p_full = bar_s_full + 16;        // [2]
  const uint32_t bar_pv_done = bar_p_full + 16;
  const uint32_t tmem_slot = bar_pv_done + 8, abort_slot = tmem_slot + 4;
  TileQueue tiles;
  tiles.place(bars + 160);  // the barriers above end at byte 144 with five ring slots
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + (abort_slot - smem_u32(smem_raw)));
  volatile uint32_t* tmem_ptr_smem = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  const WaitCtx wctx{abort_flag, p.status, nullptr};
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(bar_q_full, 1);
    mbar_init(bar_q_empty, 1);
    for (int i = 0; i < NS; ++i) {
      mbar_init(bar_kv_full + 8 * i, 1);
      mbar_init(bar_kv_empty + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_s_full + 8 * i, 1);
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

  // Number of 64-key blocks of a work item (every role needs it to know where the pipeline ends).
  auto count_blocks = [&](const FwdTile& t) {
    SubBlockCursor cur;
    cur.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
    OtherBlock kb;
    int n = 0;
    while (cur.next(&kb)) ++n;
    return n;
  };

  if (warp == 5) {
    // ------------------------------------------------------------------ TMA producer
    // Load order = consumption order of the MMA warp: K0, K1, then V(n), K(n + 2) for n = 0, 1, ...
    if (lane == 0) {
      uint32_t ring = 0, q_count = 0;
      bool ok = true;
      // One ring slot: 64 rows x 256 columns starting at column col0.
      auto load_slot = [&](const CUtensorMap* map, int col0, int head, int row, int batch_coord) -> bool {
        const uint32_t slot = ring % NS, phase = (ring / NS) & 1;
        if (!mbar_wait(bar_kv_empty + 8 * slot, phase ^ 1, wctx, kWaitKvEmpty)) return false;
        const uint32_t bar = bar_kv_full + 8 * slot;
        mbar_expect_tx(bar, kKvBytes);
#pragma unroll
        for (int h = 0; h < 4; ++h)
          tma_load_4d(smem_kv + slot * kKvBytes + h * kKvPanel, map, bar, col0 + h * 64, head, row, batch_coord);
        ++ring;
        return true;
      };
      auto load_k = [&](int head, int row, int batch_coord) -> bool {  // all reduction columns: kSplit slots
        for (int part = 0; part < kSplit; ++part)
          if (!load_slot(&map_k, part * D, head, row, batch_coord)) return false;
        return true;
      };
      uint32_t drawn = 0;
      for (int tile; ok && (tile = tiles.push(drawn, p.tile_counter, num_tiles, wctx)) >= 0;) {
        FwdTile t = decode_tile(p, tile / kSplit, kBlockM);
        const int dh = tile % kSplit;
        if (!t.valid) continue;
        const int n_blocks = count_blocks(t);
        if (n_blocks == 0) continue;
        SubBlockCursor cur_k, cur_v;
        cur_k.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
        cur_v.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
        OtherBlock kb;
        if (!mbar_wait(bar_q_empty, (q_count & 1) ^ 1, wctx, kWaitQEmpty)) { ok = false; break; }
        ++q_count;
        mbar_expect_tx(bar_q_full, kQBytes);
#pragma unroll
        for (int h = 0; h < 4 * kSplit; ++h)
          tma_load_4d(smem_q + h * kQPanel, &map_q, bar_q_full, h * 64, t.head, t.s.q0 + t.m0, t.s.batch_coord);
        for (int i = 0; ok && i < imin(2, n_blocks); ++i) {
          cur_k.next(&kb);
          ok = load_k(t.kv_head, kb.row, t.s.batch_coord);
        }
        for (int n = 0; ok && n < n_blocks; ++n) {
          cur_v.next(&kb);
          ok = load_slot(&map_v, dh * D, t.kv_head, kb.row, t.s.batch_coord);
          if (ok && n + 2 < n_blocks) {
            cur_k.next(&kb);
            ok = load_k(t.kv_head, kb.row, t.s.batch_coord);
          }
        }
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_s = umma_idesc_bf16(kBlockM, kSubN, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(kBlockM, D, 0, 1);
      uint32_t ring = 0, q_count = 0, blocks = 0;  // blocks: PV products issued so far (all work items)
      uint32_t p_phase[2] = {0, 0};
      bool ok = true;
      auto wait_kv = [&](uint32_t index) -> bool {
        return mbar_wait(bar_kv_full + 8 * (index % NS), (index / NS) & 1, wctx, kWaitKvFull);
      };
      // S = Q K^T over the kSplit ring slots of a key block; each slot is released as soon as its MMAs are issued.
      auto issue_s = [&](int buffer) -> bool {
        for (int part = 0; part < kSplit; ++part) {
          const uint32_t k_index = ring++;
          if (!wait_kv(k_index)) return false;
          tc_fence_after();
          const uint32_t k_smem = smem_kv + (k_index % NS) * kKvBytes;
          const uint32_t q_smem = smem_q + part * 4 * kQPanel;
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            umma_ss(tmem_base + buffer * 128, umma_smem_desc(q_smem + (kk >> 2) * kQPanel + (kk & 3) * 32, 16, 1024),
                    umma_smem_desc(k_smem + (kk >> 2) * kKvPanel + (kk & 3) * 32, 16, 1024), idesc_s, part > 0 || kk > 0);
          }
          tc_commit(bar_kv_empty + 8 * (k_index % NS));
        }
        tc_commit(bar_s_full + 8 * buffer);
        return true;
      };
      uint32_t popped = 0;
      for (int tile; ok && (tile = tiles.pop_thread(popped, wctx)) >= 0;) {
        FwdTile t = decode_tile(p, tile / kSplit, kBlockM);
        const int dh = tile % kSplit;
        if (!t.valid) continue;
        const int n_blocks = count_blocks(t);
        if (n_blocks == 0) continue;
        const uint32_t q_phase = q_count & 1;
        ++q_count;
        if (!mbar_wait(bar_q_full, q_phase, wctx, kWaitQFull)) { ok = false; break; }
        // The S buffers alternate with the block index of the work item; their barrier phases count per buffer.
        for (int i = 0; ok && i < imin(2, n_blocks); ++i) ok = issue_s(i);
        for (int n = 0; ok && n < n_blocks; ++n) {
          const int buffer = n & 1;
          const uint32_t v_index = ring++;
          if (!wait_kv(v_index)) { ok = false; break; }
          // phase of p_full[buffer]: number of earlier blocks that used this buffer
          if (!mbar_wait(bar_p_full + 8 * buffer, p_phase[buffer], wctx, kWaitPFull)) { ok = false; break; }
          p_phase[buffer] ^= 1;
          tc_fence_after();
          const uint32_t v_smem = smem_kv + (v_index % NS) * kKvBytes;
#pragma unroll
          for (int kk = 0; kk < kSubN / 16; ++kk) {
            umma_ts(tmem_base + kTmemO, tmem_base + buffer * 128 + 64 + kk * 8,
                    umma_smem_desc(v_smem + kk * 2048, kKvPanel, 1024), idesc_pv, n > 0 || kk > 0);
          }
          tc_commit(bar_pv_done);
          tc_commit(bar_kv_empty + 8 * (v_index % NS));
          ++blocks;
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
    uint32_t blocks = 0;
    uint32_t s_phase[2] = {0, 0};
    bool ok = true;
    uint32_t popped = 0;
    for (int tile; ok && (tile = tiles.pop_warp(popped, wctx)) >= 0;) {
      FwdTile t = decode_tile(p, tile / kSplit, kBlockM);
      const int dh = tile % kSplit;
      if (!t.valid) continue;
      const int row = t.m0 + row_in_tile;
      SubBlockCursor cur;
      cur.init(&pr, t.seq, t.s, t.m0, imin(t.m0 + kBlockM, t.s.lq));
      const int band_lo = cur.cursor.band.lo(row), band_hi = cur.cursor.band.hi(row);
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
        float2 s[32];  // 64 scores
        tmem_ld32(t_s, reinterpret_cast<uint32_t*>(s));
        tmem_ld32(t_s + 32, reinterpret_cast<uint32_t*>(s) + 32);
        tc_wait_ld();
        int lo, hi;
        if (kb.banded) {
          lo = band_lo - kb.col0;
          hi = band_hi - kb.col0;
        } else {
          lo = 0;
          hi = kb.limit - kb.col0;
        }
        const bool masked_block = __any_sync(0xffffffffu, lo > 0 || hi < kSubN);
        if (masked_block) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            s[i].x = (2 * i >= lo && 2 * i < hi) ? s[i].x : -INFINITY;
            s[i].y = (2 * i + 1 >= lo && 2 * i + 1 < hi) ? s[i].y : -INFINITY;
          }
        }
        float bm0 = fmaxf(s[0].x, s[0].y), bm1 = fmaxf(s[1].x, s[1].y);
        float bm2 = fmaxf(s[2].x, s[2].y), bm3 = fmaxf(s[3].x, s[3].y);
#pragma unroll
        for (int i = 4; i < 32; i += 4) {
          bm0 = fmaxf(bm0, fmaxf(s[i].x, s[i].y));
          bm1 = fmaxf(bm1, fmaxf(s[i + 1].x, s[i + 1].y));
          bm2 = fmaxf(bm2, fmaxf(s[i + 2].x, s[i + 2].y));
          bm3 = fmaxf(bm3, fmaxf(s[i + 3].x, s[i + 3].y));
        }
        const float part_a = fmaxf(bm0, bm2), part_b = fmaxf(bm1, bm3);  // even and odd pairs of columns
        const float block_max = fmaxf(part_a, part_b);
        const float m_new = fmaxf(m, block_max);
        const bool set_apart = sets_keys_apart(top, part_a, part_b, scale_log2);
        const bool counting = __any_sync(0xffffffffu, set_apart);
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
          sum_counted = sum_without_keys_apart<kSubN>(top, l, set_apart, block_max, t_s, masked_block, lo, hi, scale_log2, mc);
        float2 sum_a = make_float2(0.f, 0.f), sum_b = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 x = __ffma2_rn(s[16 * c + i], scale2, shift2);
            float2 e;
            e.x = ex2_approx(x.x);
            e.y = ex2_approx(x.y);
            if (i & 1) sum_b = __fadd2_rn(sum_b, e); else sum_a = __fadd2_rn(sum_a, e);
            packed[i] = pack_bf16x2(e.x, e.y);
          }
          tmem_st16(t_s + 64 + 16 * c, packed);
        }
        l += counting ? sum_counted : (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
        // Observe the PV product of the previous block before releasing this one. The scores of block n only prove
        // that PV(n - 2) has completed, so without this wait the barrier could be two completions away from the one
        // the epilogue waits for, which a parity wait cannot tell apart from "done".
        if (tile_blocks > 0 && !mbar_wait_warp(bar_pv_done, (blocks - 1) & 1, wctx, kWaitPvDone)) { ok = false; break; }
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_p_full + 8 * buffer);
        ++blocks;
        ++tile_blocks;
      }
      if (!ok) break;
      // ---- epilogue
      const bool row_valid = row < t.s.lq;
      __nv_bfloat16* o_row = p.o + t.s.batch_coord * p.o_batch_stride + (int64_t)(t.s.q0 + row) * p.o_row_stride +
                             (int64_t)t.head * p.o_head_stride + dh * D;
      float* lse_ptr = p.lse + t.s.batch_coord * p.lse_batch_stride + (int64_t)t.head * p.lse_head_stride + t.s.q0 + row;
      if (tile_blocks == 0) {
        if (row_valid) {
          const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll
          for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(o_row)[c] = zero;
          if (dh == 0) *lse_ptr = -INFINITY;
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
        if (row_valid) {
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
      if (row_valid && dh == 0) *lse_ptr = lse_row;  // both halves hold the same statistics
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

template <int kSplit>
static int launch_fwd_wide(const b200fa_fwd_args& a, cudaStream_t stream) {
  using Cfg = wide::Config<kSplit>;
  FwdParams p;
  CUtensorMap map_q, map_k, map_v;
  bool nothing_to_do = false;
  int status = prepare_forward(a, stream, wide::D * kSplit, kBlockM, wide::kSubN, &p, &map_q, &map_k, &map_v, &nothing_to_do);
  if (status != B200FA_OK || nothing_to_do) return status;
  static bool attribute_set[64] = {false};
  status = set_dynamic_smem_once(reinterpret_cast<const void*>(&fwd_wide_kernel<kSplit>), Cfg::kSmemBytes, attribute_set);
  if (status != B200FA_OK) return status;
  int sms = 0;
  status = device_sm_count(&sms);
  if (status != B200FA_OK) return status;
  const int tiles = p.num_tiles * kSplit;
  const int grid = tiles < sms ? tiles : sms;
  fwd_wide_kernel<kSplit><<<grid, wide::kThreads, Cfg::kSmemBytes, stream>>>(map_q, map_k, map_v, p);
  B200FA_CUDA_CHECK(cudaGetLastError());
  return B200FA_OK;
}

int launch_fwd_512(const b200fa_fwd_args& a, cudaStream_t stream) { return launch_fwd_wide<2>(a, stream); }

}  // namespace b200fa
