// Tuning microbenchmark (not part of the library): throughput of ex2.approx on f32, f16x2 and bf16x2 operands, in
// lane operations and results per cycle and SM, for 4 to 32 warps per SM.
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o ex2_rate zig-flash-attn_b200/csrc/tuning/ex2_rate.cu
//   ./ex2_rate
#include <cstdio>
#include <cuda_runtime.h>
#include <cstdint>
template <int MODE>
__global__ void k(float* out, int iters, long long* cyc) {
  uint32_t a[8];
  for (int i = 0; i < 8; ++i) a[i] = 0x3c003c00u + threadIdx.x + i;  // packed values near 1.0 (f16) / small bf16
  float f[8];
  for (int i = 0; i < 8; ++i) f[i] = -0.001f * (threadIdx.x + i);
  __syncthreads();
  long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (MODE == 0) asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(f[i]));
      if (MODE == 1) asm volatile("ex2.approx.f16x2 %0, %0;" : "+r"(a[i]));
      if (MODE == 2) asm volatile("ex2.approx.ftz.bf16x2 %0, %0;" : "+r"(a[i]));
    }
  }
  long long t1 = clock64();
  float s = 0;
  for (int i = 0; i < 8; ++i) s += f[i] + __uint_as_float(a[i]);
  out[blockIdx.x * blockDim.x + threadIdx.x] = s;
  if (threadIdx.x == 0 && blockIdx.x == 0) *cyc = t1 - t0;
}
int main() {
  float* out; long long* cyc; cudaMalloc(&out, 148 * 1024 * 4); cudaMalloc(&cyc, 8);
  const int iters = 2000;
  for (int threads : {128, 256, 512, 1024}) {
    long long h[3];
    k<0><<<148, threads>>>(out, iters, cyc); cudaMemcpy(&h[0], cyc, 8, cudaMemcpyDeviceToHost);
    k<1><<<148, threads>>>(out, iters, cyc); cudaMemcpy(&h[1], cyc, 8, cudaMemcpyDeviceToHost);
    k<2><<<148, threads>>>(out, iters, cyc); cudaMemcpy(&h[2], cyc, 8, cudaMemcpyDeviceToHost);
    const double n = double(iters) * 8 * threads;  // instructions (lane-ops) per SM
    printf("threads %4d: f32 %.2f lane-ops/clk/SM, f16x2 %.2f (%.2f results), bf16x2 %.2f (%.2f results)  %s\n", threads, n / h[0], n / h[1],
           2 * n / h[1], n / h[2], 2 * n / h[2], cudaGetErrorString(cudaGetLastError()));
  }
  return 0;
}
