// Tuning microbenchmark (not part of the library): cycles per tcgen05.mma with cta_group::2 (kind::f16, BF16 -> FP32,
// M = 256 over the two CTAs of a cluster, K = 16) for N = 128 and 256, both operands K-major in shared memory. Each CTA
// holds its 128 rows of A and its N / 2 rows of B at the same shared-memory offsets; thread 0 of the leader CTA (rank 0)
// issues `count` MMAs back to back on zeroed operands, commits to its own barrier and waits (bounded). Every wait in
// here has an iteration limit; the TMEM of both CTAs is freed by both after a cluster barrier.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate_2cta zig-flash-attn_b200/csrc/tuning/mma_rate_2cta.cu
//   ./mma_rate_2cta
#include <cstdio>
#include <cuda_runtime.h>
#include <cooperative_groups.h>
#include "../ptx.cuh"
using namespace b200fa;
namespace cg = cooperative_groups;

__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
  for (int i = 0; i < 4000000; ++i) if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void umma_ss_2cta(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <int N>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) rate_kernel(long long* out, int count) {
  extern __shared__ __align__(1024) uint8_t smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const bool leader = cluster.block_rank() == 0;
  const uint32_t base = smem_u32(smem);
  const uint32_t bar = base + 200 * 1024, slot = bar + 16;
  for (int i = threadIdx.x; i < 200 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(bar, 1); fence_barrier_init(); }
  if (threadIdx.x < 32) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(512) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  fence_proxy_async_smem();
  tc_fence_before();
  cluster.sync();
  tc_fence_after();
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + 200 * 1024 + 16);
  if (leader && threadIdx.x == 0) {
    constexpr uint32_t idesc = umma_idesc_bf16(256, N, 0, 0);
    const uint32_t a = base, b = base + 64 * 1024;
    for (int rep = 0; rep < 3; ++rep) {
      const long long t0 = clock64();
      for (int i = 0; i < count; ++i) {
        const uint32_t off = (i & 3) * 32 + ((i >> 2) & 1) * 16384;
        umma_ss_2cta(tmem, umma_smem_desc(a + off, 16, 1024), umma_smem_desc(b + off, 16, 1024), idesc, i > 0);
      }
      const long long t1 = clock64();
      asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
      const bool ok = wait_bar(bar, rep & 1);
      const long long t2 = clock64();
      if (blockIdx.x == 0) { out[3 * rep] = t1 - t0; out[3 * rep + 1] = t2 - t0; out[3 * rep + 2] = ok; }
      if (!ok) break;
    }
  }
  tc_fence_before();
  cluster.sync();  // the peer's shared memory and TMEM stay in place until the leader has seen its MMAs complete
  tc_fence_after();
  if (threadIdx.x < 32)
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
}

template <int N>
void run(const char* name, int ctas, int count) {
  long long* out; cudaMalloc(&out, 128); cudaMemset(out, 0, 128);
  const int smem = 200 * 1024 + 64;
  cudaFuncSetAttribute(rate_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  rate_kernel<N><<<ctas, 128, smem>>>(out, count);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[9]; cudaMemcpy(h, out, sizeof(h), cudaMemcpyDeviceToHost);
  printf("%-30s ctas %3d: issue %6.1f  total %6.1f cycles per MMA (ok %lld) %s\n", name, ctas, double(h[6]) / count, double(h[7]) / count,
         h[8], e == cudaSuccess ? "" : cudaGetErrorString(e));
  cudaFree(out);
}

int main() {
  const int count = 512;
  for (int ctas : {2, 148}) {
    run<128>("2-CTA SS M=256 N=128", ctas, count);
    run<256>("2-CTA SS M=256 N=256", ctas, count);
    run<64>("2-CTA SS M=256 N=64", ctas, count);
  }
  return 0;
}
