// Tuning microbenchmark (not part of the library): cycles per tcgen05.mma (kind::f16, BF16 -> FP32, cta_group::1,
// M = 128, K = 16) for several N, operand sources, operand majorness and accumulator patterns. One CTA on each of
// `ctas` SMs; thread 0 issues `count` MMAs back to back on zeroed operands, commits, and waits (bounded) for the commit.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate zig-flash-attn_b200/csrc/tuning/mma_rate.cu
//   ./mma_rate
#include <cstdio>
#include <cuda_runtime.h>
#include "../ptx.cuh"
using namespace b200fa;

__device__ __forceinline__ float4 ld_shared_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < 4000000; ++i) if (mbar_try_wait(bar, parity)) return true;
  return false;
}

template <int N, int MODE>  // MODE 0: SS, both operands K-major, one accumulator; 1: the same with two accumulators in turn; 2: TS (A in TMEM);
                             // 3: SS with B MN-major; 4: SS with A and B MN-major; 5: as 0 with a tcgen05.commit after every eighth MMA
__global__ void __launch_bounds__(384, 1) rate_kernel(long long* out, int count, int fill, int load) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const uint32_t base = smem_u32(smem);
  const uint32_t bar = base + 200 * 1024, slot = bar + 16;
  // Operands: zeros, or (fill != 0) BF16 values in (-2, -1] and [1, 2) with random mantissas, which toggle the datapath
  // the way real data does (the MMA rate under load depends on it).
  for (int i = threadIdx.x; i < 200 * 1024 / 4; i += blockDim.x) {
    uint32_t h = (i + 1) * 2654435761u + blockIdx.x * 40503u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    reinterpret_cast<uint32_t*>(smem)[i] = fill ? ((h & 0x807f807fu) | 0x3f803f80u) : 0u;
  }
  if (threadIdx.x == 0) { mbar_init(bar, 1); mbar_init(bar + 8, 1 << 20); fence_barrier_init(); }
  if (threadIdx.x < 32) { tmem_alloc(slot, 512); tmem_relinquish(); }
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + 200 * 1024 + 16);
  volatile int* stop = reinterpret_cast<volatile int*>(smem + 200 * 1024 + 32);
  if (threadIdx.x == 0) *stop = 0;
  __syncthreads();
  if (threadIdx.x >= 128 && load != 0) {
    // Background work of the kind the attention kernels run next to their MMAs, on warps 4-11 until thread 0 is done:
    // load 1 = exp2 and FMA arithmetic, 2 = TMEM loads and stores (columns 384-511), 3 = shared-memory copies.
    float x = 0.001f * threadIdx.x, y = 1.f;
    uint32_t regs[32];
    for (int i = 0; i < 32; ++i) regs[i] = threadIdx.x + i;
    const uint32_t taddr = tmem + (static_cast<uint32_t>((threadIdx.x >> 5) & 3) * 32 << 16) + 384 + 32 * (((threadIdx.x >> 7) - 1) & 1);
    const uint32_t saddr = base + 128 * 1024 + (threadIdx.x - 128) * 16;
    while (!*stop) {
      for (int it = 0; it < 64; ++it) {
        if (load == 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) { x = ex2_approx(-x * 0.5f); y = fmaf(y, 0.999f, x); }
        } else if (load == 2) {
          tmem_ld32(taddr, regs);
          tc_wait_ld();
          tmem_st32(taddr, regs);
          tc_wait_st();
        } else {
          float4 v = ld_shared_f4(saddr + (it & 15) * 4096);
          st_shared_v4(saddr + 65536 - 4096 * (it & 7), __float_as_uint(v.x), __float_as_uint(v.y), __float_as_uint(v.z), __float_as_uint(v.w));
        }
      }
    }
    if (x + y == 12345.f && regs[3] == 77) out[15] = 1;
  }
  if (threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(128, N, MODE == 4 ? 1 : 0, MODE >= 3 ? 1 : 0);
    const uint32_t a = base, b = base + 64 * 1024;
    for (int rep = 0; rep < 3; ++rep) {
      const long long t0 = clock64();
      for (int i = 0; i < count; ++i) {
        const uint32_t off = (i & 3) * 32 + ((i >> 2) & 1) * 16384;
        const uint32_t d = tmem + ((MODE == 1 && (i & 1)) ? 256 : 0);
        if (MODE == 2) umma_ts(d, tmem + 256 + (i & 7) * 8, umma_smem_desc(b + off, 16, 1024), idesc, i > 1);
        else if (MODE == 4) umma_ss(d, umma_smem_desc(a + (i & 7) * 2048, 16384, 1024), umma_smem_desc(b + (i & 7) * 2048, 16384, 1024), idesc, i > 1);
        else if (MODE == 3) umma_ss(d, umma_smem_desc(a + off, 16, 1024), umma_smem_desc(b + (i & 7) * 2048, 16384, 1024), idesc, i > 1);
        else umma_ss(d, umma_smem_desc(a + off, 16, 1024), umma_smem_desc(b + off, 16, 1024), idesc, i > 1);
        if (MODE == 5 && (i & 7) == 7) tc_commit(bar + 8);  // a commit after every eighth MMA, to a barrier nobody waits on
      }
      const long long t1 = clock64();
      tc_commit(bar);
      const bool ok = wait_bar(bar, rep & 1);
      const long long t2 = clock64();
      if (blockIdx.x == 0) { out[3 * rep] = t1 - t0; out[3 * rep + 1] = t2 - t0; out[3 * rep + 2] = ok; }
      if (!ok) break;
    }
    *stop = 1;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x < 32) tmem_dealloc(tmem, 512);
}

template <int N, int MODE>
void run(const char* name, int ctas, int count, int fill = 0, int load = 0) {
  long long* out; cudaMalloc(&out, 128); cudaMemset(out, 0, 128);
  const int smem = 200 * 1024 + 64;
  cudaFuncSetAttribute(rate_kernel<N, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  rate_kernel<N, MODE><<<ctas, 384, smem>>>(out, count, fill, load);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[9]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
  printf("%-34s %s ctas %3d: issue %6.1f  total %6.1f cycles per MMA (ok %lld) %s\n", name, load == 0 ? (fill ? "random" : "zeros ") : load == 1 ? "rnd+alu" : load == 2 ? "rnd+tmem" : "rnd+smem", ctas, double(h[6]) / count, double(h[7]) / count,
         h[8], e == cudaSuccess ? "" : cudaGetErrorString(e));
  cudaFree(out);
}

int main() {
  const int count = 512;
  for (int ctas : {1, 148}) {
    run<64, 0>("SS N=64 one accumulator", ctas, count);
    run<128, 0>("SS N=128 one accumulator", ctas, count);
    run<256, 0>("SS N=256 one accumulator", ctas, count);
    run<128, 1>("SS N=128 two accumulators", ctas, count);
    run<64, 1>("SS N=64 two accumulators", ctas, count);
    run<64, 2>("TS N=64", ctas, count);
    run<128, 2>("TS N=128", ctas, count);
    run<256, 2>("TS N=256 (acc over A: timing only)", ctas, count);
    run<64, 3>("SS N=64 B MN-major", ctas, count);
    run<128, 3>("SS N=128 B MN-major", ctas, count);
    run<256, 3>("SS N=256 B MN-major", ctas, count);
    run<64, 4>("SS N=64 A and B MN-major", ctas, count);
    run<128, 4>("SS N=128 A and B MN-major", ctas, count);
  }
  // The same instructions on random operands, long enough for the power management to react (each run about 40 ms).
  for (int ctas : {1, 148}) {
    run<128, 0>("SS N=128 one accumulator", ctas, 1 << 20, 1);
    run<256, 0>("SS N=256 one accumulator", ctas, 1 << 19, 1);
    run<128, 3>("SS N=128 B MN-major", ctas, 1 << 20, 1);
    run<128, 0>("SS N=128 one accumulator", ctas, 1 << 20, 0);
    run<128, 5>("SS N=128, commit every 8 MMAs", ctas, 1 << 16, 1);
    run<256, 5>("SS N=256, commit every 8 MMAs", ctas, 1 << 16, 1);
    for (int load = 1; load <= 3; ++load) {
      run<128, 0>("SS N=128 one accumulator", ctas, 1 << 18, 1, load);
      run<256, 0>("SS N=256 one accumulator", ctas, 1 << 17, 1, load);
    }
  }
  return 0;
}
