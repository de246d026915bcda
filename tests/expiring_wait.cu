// Test-only kernel: a wait of the library's own bounded-wait primitive (csrc/ptx.cuh) on an mbarrier that nobody ever
// arrives at, built with a budget of one millisecond instead of two seconds. It follows the shape of the attention
// kernels: TMEM allocated up front, the roles wait, the wait gives up, raises the CTA's abort flag and records
// code << 16 | CTA in the status word, the other warps see the flag in their own waits, everybody meets at the
// final barrier, TMEM is freed and the kernel returns. Nothing traps and no loop is unbounded.
#define B200FA_WAIT_BUDGET_NS 1000000ull
#include "ptx.cuh"

#include <cuda_runtime.h>

using namespace b200fa;

__global__ void __launch_bounds__(128, 1) expiring_wait_kernel(int* status, int* passed) {
  __shared__ __align__(8) unsigned long long barrier_storage;
  __shared__ int abort_storage;
  __shared__ uint32_t tmem_slot;
  const uint32_t bar = smem_u32(&barrier_storage);
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    abort_storage = 0;
    mbar_init(bar, 1);
    fence_barrier_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&tmem_slot), 32);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(&tmem_slot);
  const WaitCtx ctx{&abort_storage, status, nullptr};
  // Every warp waits for phase 0 of a barrier with one expected arrival that never comes.
  const bool done = mbar_wait_warp(bar, 0, ctx, kWaitSFull);
  if (abort_storage) {
    for (int i = 0; i < 5; ++i) __nanosleep(20000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 0) tmem_dealloc(tmem_base, 32);
  if (done && (threadIdx.x & 31) == 0) atomicAdd(passed, 1);
}

// Launches `blocks` CTAs, waits for them and reports the status word, how many warps saw the barrier complete (must be
// zero) and the kernel's duration. Returns the CUDA error code of the first failing call (0 = none).
extern "C" int run_expiring_wait(int blocks, int* status_out, int* passed_out, float* milliseconds_out) {
  int* device_words = nullptr;
  cudaError_t error = cudaMalloc(&device_words, 2 * sizeof(int));
  if (error != cudaSuccess) return static_cast<int>(error);
  cudaMemset(device_words, 0, 2 * sizeof(int));
  cudaEvent_t start, stop;
  cudaEventCreate(&start);
  cudaEventCreate(&stop);
  cudaEventRecord(start);
  expiring_wait_kernel<<<blocks, 128>>>(device_words, device_words + 1);
  cudaEventRecord(stop);
  error = cudaDeviceSynchronize();
  int words[2] = {0, 0};
  if (error == cudaSuccess) error = cudaMemcpy(words, device_words, sizeof(words), cudaMemcpyDeviceToHost);
  if (error == cudaSuccess) cudaEventElapsedTime(milliseconds_out, start, stop);
  *status_out = words[0];
  *passed_out = words[1];
  cudaEventDestroy(start);
  cudaEventDestroy(stop);
  cudaFree(device_words);
  return static_cast<int>(error);
}
