// Host-side helpers shared by the C-ABI translation units: thread-local error text, CUDA error checks and the
// TMA tensor-map encoder (driver entry point fetched at run time, so the library has no link dependency on libcuda
// and loads on machines without a GPU).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/b200fa.h"
#include "attn_index.h"

namespace b200fa {

void set_error(const char* format, ...);

#define B200FA_CUDA_CHECK(call)                                                             \
  do {                                                                                      \
    cudaError_t status_ = (call);                                                           \
    if (status_ != cudaSuccess) {                                                           \
      ::b200fa::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(status_), __FILE__, __LINE__); \
      return B200FA_ERR_CUDA;                                                               \
    }                                                                                       \
  } while (0)

#define B200FA_REQUIRE(condition, ...)      \
  do {                                      \
    if (!(condition)) {                     \
      ::b200fa::set_error(__VA_ARGS__);     \
      return B200FA_ERR_INVALID;            \
    }                                       \
  } while (0)

// 4-D tensor map over a (batch, row, head, column) tensor of `element_bytes`-wide elements with strides in elements.
// Box = (box_cols, box_heads, box_rows, 1 batch); swizzle 128 B when box_cols * element_bytes == 128. In shared memory
// a box is laid out row-major as [row][head][column].
int encode_tensor_map(CUtensorMap* map, const void* base, CUtensorMapDataType type, int element_bytes, int64_t cols,
                      int64_t heads, int64_t rows, int64_t batch, int64_t head_stride, int64_t row_stride,
                      int64_t batch_stride, int box_cols, int box_rows, int box_heads = 1);

Problem to_problem(const b200fa_problem& in);

// Guards every per-device cache of the library (see api.cu).
std::mutex& cache_mutex();

int device_sm_count(int* count);
// Bytes of partial results the split-KV forward path wants for this problem (0 = the problem is not split). Defined in
// fwd.cu; a pure function of the shapes.
size_t fwd_split_workspace_bytes(const b200fa_problem& problem);
// log2 of the query heads that the forward kernel packs into the rows of a work item for this problem (fwd.cu).
int fwd_pack_shift(const b200fa_problem& problem);
// Raises the dynamic shared-memory limit of `kernel` once per device (function attributes are per device; `done` is
// the caller's per-kernel record, indexed by device ordinal).
int set_dynamic_smem_once(const void* kernel, int bytes, bool (&done)[64]);

// Device address of the library's status word on the current device (null + error text on failure).
int* device_status_word();

// The process-wide pivot-gradient setting (b200fa_set_pivot_ds).
bool pivot_ds_enabled();
// Device buffer of 32 cycle counters set with b200fa_set_trace (null = tracing off).
long long* trace_buffer();

}  // namespace b200fa
