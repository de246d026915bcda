// Inline-PTX wrappers for the sm_100a primitives the attention kernels use: mbarrier (with bounded waits),
// TMA tiled loads / reduce-adds, tcgen05 MMA / TMEM allocation / TMEM loads and stores, and UMMA descriptors.
//
// Every wait in this file is bounded. When a wait runs out it records an error code in a global status word,
// raises a CTA-wide abort flag in shared memory and returns false; callers leave their loops, the CTA waits for
// its copies in flight, frees its TMEM and returns. Nothing here traps or spins without a limit.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200fa {

// Where a wait that ran out of time reports: a CTA-wide abort flag in shared memory and the library's device-side
// status word (0 = no error, else code << 16 | low bits of the CTA index of the first failed wait; read by
// b200fa_device_status()).
struct WaitCtx {
  volatile int* abort_flag;
  int* status;
  long long* trace;  // optional cycle counters (null = off): see b200fa_set_trace
};

enum WaitCode : int {
  kWaitQFull = 1,
  kWaitQEmpty = 2,
  kWaitKvFull = 3,
  kWaitKvEmpty = 4,
  kWaitSFull = 5,
  kWaitPFull = 6,
  kWaitPvDone = 7,
  kWaitBwdLoad = 8,
  kWaitBwdMma = 9,
  kWaitBwdCompute = 10,
  kWaitBwdReduce = 11,
  kWaitEpilogue = 12,
  kWaitTile = 13,
};

// Time a single wait may take before it gives up: 2 s, far above anything a healthy launch needs. A test build can
// shorten it (-DB200FA_WAIT_BUDGET_NS=...) to watch a wait run out.
#ifndef B200FA_WAIT_BUDGET_NS
#define B200FA_WAIT_BUDGET_NS 2000000000ull
#endif
constexpr unsigned long long kWaitBudgetNs = B200FA_WAIT_BUDGET_NS;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait on the phase with the given parity.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, WaitCtx ctx, int code) {
  const unsigned long long start = global_timer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*ctx.abort_flag) return false;
    if (global_timer_ns() - start > kWaitBudgetNs) {
      *ctx.abort_flag = 1;
      atomicCAS(ctx.status, 0, (code << 16) | (int)(blockIdx.x & 0xffff));
      return false;
    }
  }
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ctx, code);
}
// Tuning builds (-DB200FA_TRACE) add the cycles spent in each wait to trace[slot] (lane 0 of a warp only); regular
// builds compile the traced calls down to the plain waits.
#ifdef B200FA_TRACE
constexpr bool kTraceBuild = true;
#else
constexpr bool kTraceBuild = false;
#endif
// -DB200FA_TRACE_SUMS=0 leaves the per-wait sums out of a tuning build: their atomics (every warp of every CTA on a few
// addresses) stretch the iterations, which a per-role timeline (trace_event) must not see.
#ifndef B200FA_TRACE_SUMS
#define B200FA_TRACE_SUMS 1
#endif
constexpr bool kTraceSums = B200FA_TRACE_SUMS != 0;
__device__ __forceinline__ bool mbar_wait_traced(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code, int slot,
                                                 bool warp_uniform) {
  if (!kTraceBuild || !kTraceSums || ctx.trace == nullptr) {
    const bool done = mbar_wait(bar, parity, ctx, code);
    return warp_uniform ? __all_sync(0xffffffffu, done) : done;
  }
  const long long start = clock64();
  bool done = mbar_wait(bar, parity, ctx, code);
  if (warp_uniform) done = __all_sync(0xffffffffu, done);
  if ((threadIdx.x & 31) == 0 || !warp_uniform)
    atomicAdd(reinterpret_cast<unsigned long long*>(ctx.trace + slot), static_cast<unsigned long long>(clock64() - start));
  return done;
}
__device__ __forceinline__ long long trace_clock(const WaitCtx& ctx) {
  return (kTraceBuild && ctx.trace != nullptr) ? clock64() : 0;
}
// Timeline events of one CTA (tuning builds): each role writes id << 48 | cycle counter into its own region
// trace[64 + 720 * role + n]; plain stores, so the logging thread does not wait on memory.
__device__ __forceinline__ void trace_event(const WaitCtx& ctx, bool selected, int role, int& n, int id) {
  if (kTraceBuild && ctx.trace != nullptr && selected && n < 720) {
    ctx.trace[64 + 720 * role + n] = (static_cast<long long>(id) << 48) | (clock64() & 0xffffffffffffll);
    ++n;
  }
}
__device__ __forceinline__ void trace_add(const WaitCtx& ctx, int slot, long long cycles) {
  if (kTraceBuild && kTraceSums && ctx.trace != nullptr && (threadIdx.x & 31) == 0)
    atomicAdd(reinterpret_cast<unsigned long long*>(ctx.trace + slot), static_cast<unsigned long long>(cycles));
}
// Same, with a warp-uniform result (for code that goes on to execute .sync.aligned instructions).
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, const WaitCtx& ctx, int code) {
  return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, code));
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_descriptor(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}
// 4-D tiled load: coordinates are (c0 = innermost column, c1, c2, c3).
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], "
      "[%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 4-D tiled reduce-add (shared -> global), completion tracked by the bulk async-group of the issuing thread.
__device__ __forceinline__ void tma_reduce_add_4d(const void* tmap, uint32_t smem_src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// 1-D bulk copy global -> shared (size and both addresses multiples of 16 bytes).
__device__ __forceinline__ void bulk_load_1d(uint32_t smem_dst, const void* gmem_src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gmem_src)), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------- TMEM allocation (one full warp executes these)
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}

// ---------------------------------------------------------------- tcgen05 fences / commit / waits
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Arrives once on `bar` when every MMA this thread issued before has completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---------------------------------------------------------------- clusters of two CTAs
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of `addr` (a shared-memory address of this CTA) in CTA `rank` of the cluster, in the shared::cluster window.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  // default semantics (release at CTA scope): what is published is TMEM content, ordered by the tcgen05 fences; a
  // release at cluster scope costs the arriving warp about 1300 cycles
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Bulk copy of `bytes` (a multiple of 16) from this CTA's shared memory into the shared memory of a CTA of the cluster;
// the bytes complete on a barrier of that CTA (both given as shared::cluster addresses).
__device__ __forceinline__ void bulk_copy_to_cluster(uint32_t dst_cluster, uint32_t src, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_cluster),
               "r"(src), "r"(bytes), "r"(bar_cluster)
               : "memory");
}

// ---------------------------------------------------------------- UMMA descriptors
// Shared-memory matrix descriptor, 128-byte swizzle. Offsets in bytes.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t leading_bytes, uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;  // descriptor version for sm_100
  d |= 2ull << 61;  // SWIZZLE_128B
  return d;
}
// Instruction descriptor: BF16 x BF16 -> FP32, dense. a_mn / b_mn: 1 when the operand is MN-major in shared memory.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a_mn) << 15) |
         (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---------------------------------------------------------------- TMEM loads / stores (32 lanes x 32 bit, N columns)
#define B200FA_R4(a, i) "=r"(a[i]), "=r"(a[i + 1]), "=r"(a[i + 2]), "=r"(a[i + 3])
#define B200FA_R16(a, i) B200FA_R4(a, i), B200FA_R4(a, i + 4), B200FA_R4(a, i + 8), B200FA_R4(a, i + 12)
#define B200FA_I4(a, i) "r"(a[i]), "r"(a[i + 1]), "r"(a[i + 2]), "r"(a[i + 3])
#define B200FA_I16(a, i) B200FA_I4(a, i), B200FA_I4(a, i + 4), B200FA_I4(a, i + 8), B200FA_I4(a, i + 12)

__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : B200FA_R16(r, 0)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : B200FA_R16(r, 0), B200FA_R16(r, 16)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               :
               : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
               : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      :
      : "r"(taddr), B200FA_I16(r, 0)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      :
      : "r"(taddr), B200FA_I16(r, 0), B200FA_I16(r, 16)
      : "memory");
}

// ---------------------------------------------------------------- register reallocation between warpgroups
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ---------------------------------------------------------------- named barriers and scalar shared-memory access
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void st_shared_f32(uint32_t addr, float value) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(addr), "f"(value) : "memory");
}
__device__ __forceinline__ float ld_shared_f32(uint32_t addr) {
  float value;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(value) : "r"(addr) : "memory");
  return value;
}

// ---------------------------------------------------------------- small math helpers
__device__ __forceinline__ void red_add_f32(float* address, float value) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(address), "f"(value) : "memory");
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for two values on the FMA pipe instead of the special-function unit: floor(x) through a round-down add of
// 1.5 * 2^23, a degree-3 minimax polynomial for 2^frac on [0, 1) (relative error 8.6e-5, far below the BF16 rounding
// of the result) and the integer part added into the exponent bits. Inputs below -127 are clamped (result ~ 0).
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
  const float2 magic = make_float2(12582912.f, 12582912.f);
  x.x = fmaxf(x.x, -127.f);
  x.y = fmaxf(x.y, -127.f);
  const float2 shifted = __fadd2_rd(x, magic);
  const float2 whole = __fadd2_rn(shifted, make_float2(-12582912.f, -12582912.f));
  const float2 frac = __ffma2_rn(whole, make_float2(-1.f, -1.f), x);
  float2 poly = __ffma2_rn(make_float2(0.07706566154956818f, 0.07706566154956818f), frac,
                           make_float2(0.22764649987220764f, 0.22764649987220764f));
  poly = __ffma2_rn(poly, frac, make_float2(0.6951164603233337f, 0.6951164603233337f));
  poly = __ffma2_rn(poly, frac, make_float2(1.f, 1.f));
  float2 result;
  result.x = __int_as_float(__float_as_int(poly.x) + (__float_as_int(shifted.x) << 23));
  result.y = __int_as_float(__float_as_int(poly.y) + (__float_as_int(shifted.y) << 23));
  // Exactly zero for masked scores (-inf) and anything else at the clamp: rows without keys must sum to zero.
  result.x = x.x > -127.f ? result.x : 0.f;
  result.y = x.y > -127.f ? result.y : 0.f;
  return result;
}
// 32-byte store to global memory (the address must be 32-byte aligned).
__device__ __forceinline__ void st_global_v8(void* address, const uint32_t* w) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(address), "r"(w[0]), "r"(w[1]), "r"(w[2]),
               "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));
  return d;
}

}  // namespace b200fa
