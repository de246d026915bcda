// C-ABI entry points (include/b200fa.h): argument validation, workspace sizing and dispatch to the launchers.
#include <atomic>
#include <cstdlib>
#include <mutex>

#include "common.h"

namespace b200fa {

__device__ int g_device_status = 0;

static thread_local char g_error[512] = "";

void set_error(const char* format, ...) {
  va_list arguments;
  va_start(arguments, format);
  vsnprintf(g_error, sizeof(g_error), format, arguments);
  va_end(arguments);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_entry() {
  static EncodeTiledFn entry = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* function = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &function, cudaEnableDefault, &result) == cudaSuccess &&
        result == cudaDriverEntryPointSuccess) {
      entry = reinterpret_cast<EncodeTiledFn>(function);
    }
  });
  return entry;
}

int encode_tensor_map(CUtensorMap* map, const void* base, CUtensorMapDataType type, int element_bytes, int64_t cols,
                      int64_t heads, int64_t rows, int64_t batch, int64_t head_stride, int64_t row_stride,
                      int64_t batch_stride, int box_cols, int box_rows, int box_heads) {
  EncodeTiledFn encode = encode_tiled_entry();
  if (!encode) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return B200FA_ERR_CUDA;
  }
  B200FA_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, "tensor base pointer must be 16-byte aligned");
  B200FA_REQUIRE((head_stride * element_bytes) % 16 == 0 && (row_stride * element_bytes) % 16 == 0 &&
                     (batch_stride * element_bytes) % 16 == 0,
                 "tensor strides must be multiples of 16 bytes");
  cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)batch};
  cuuint64_t strides[3] = {(cuuint64_t)(head_stride * element_bytes), (cuuint64_t)(row_stride * element_bytes),
                           (cuuint64_t)(batch_stride * element_bytes)};
  // Size-1 dimensions may carry any stride; give them a harmless one.
  if (heads == 1) strides[0] = (cuuint64_t)cols * element_bytes;
  if (batch == 1) strides[2] = strides[1] * (cuuint64_t)rows > strides[0] * (cuuint64_t)heads
                                   ? strides[1] * (cuuint64_t)rows
                                   : strides[0] * (cuuint64_t)heads;
  cuuint32_t box[4] = {(cuuint32_t)box_cols, (cuuint32_t)box_heads, (cuuint32_t)box_rows, 1u};
  cuuint32_t element_strides[4] = {1, 1, 1, 1};
  const CUtensorMapSwizzle swizzle =
      box_cols * element_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult result = encode(map, type, 4, const_cast<void*>(base), dims, strides, box, element_strides,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (result != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with %d (dims %lld x %lld x %lld x %lld, strides %lld/%lld/%lld bytes)",
              (int)result, (long long)cols, (long long)heads, (long long)rows, (long long)batch, (long long)strides[0],
              (long long)strides[1], (long long)strides[2]);
    return B200FA_ERR_INVALID;
  }
  return B200FA_OK;
}

// The per-device caches of the library (SM counts, symbol addresses, "attribute already set" records) are read and
// filled under this one mutex: the entry points may be called from several host threads at once. It is held for a
// few loads on the launch path and for one CUDA query the first time a device is seen.
std::mutex& cache_mutex() {
  static std::mutex mutex;
  return mutex;
}

int device_sm_count(int* count) {
  static int cached[64] = {0};
  int device = 0;
  B200FA_CUDA_CHECK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(cache_mutex());
  if (device >= 0 && device < 64 && cached[device] > 0) {
    *count = cached[device];
    return B200FA_OK;
  }
  int value = 0;
  B200FA_CUDA_CHECK(cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device));
  if (device >= 0 && device < 64) cached[device] = value;
  *count = value;
  return B200FA_OK;
}

int set_dynamic_smem_once(const void* kernel, int bytes, bool (&done)[64]) {
  int device = 0;
  B200FA_CUDA_CHECK(cudaGetDevice(&device));
  std::lock_guard<std::mutex> lock(cache_mutex());
  if (device >= 0 && device < 64 && done[device]) return B200FA_OK;
  B200FA_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (device >= 0 && device < 64) done[device] = true;
  return B200FA_OK;
}

int* device_status_word() {
  static int* cached[64] = {nullptr};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) {
    set_error("cudaGetDevice failed");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(cache_mutex());
  if (device >= 0 && device < 64 && cached[device]) return cached[device];
  void* address = nullptr;
  cudaError_t status = cudaGetSymbolAddress(&address, g_device_status);
  if (status != cudaSuccess) {
    set_error("cudaGetSymbolAddress failed: %s", cudaGetErrorString(status));
    return nullptr;
  }
  if (device >= 0 && device < 64) cached[device] = static_cast<int*>(address);
  return static_cast<int*>(address);
}

static std::atomic<long long*> g_trace{nullptr};
long long* trace_buffer() { return g_trace.load(std::memory_order_relaxed); }

int launch_fwd(const b200fa_fwd_args& args, cudaStream_t stream);
int launch_bwd(const b200fa_bwd_args& args, cudaStream_t stream);
size_t bwd_workspace_bytes(const b200fa_problem& problem);
void arm_bwd_timing(void* const* events);

static int validate_problem(const b200fa_problem& p) {
  B200FA_REQUIRE(p.batch >= 0 && p.seqlen_q >= 0 && p.seqlen_k >= 0, "negative sizes");
  B200FA_REQUIRE(p.heads_q > 0 && p.heads_kv > 0 && p.heads_q % p.heads_kv == 0,
                 "the query head count must be a positive multiple of the key head count");
  B200FA_REQUIRE(p.window_left >= -1 && p.window_right >= -1, "window bounds must each be -1 or non-negative");
  B200FA_REQUIRE((p.cu_seqlens_q == nullptr) == (p.cu_seqlens_k == nullptr),
                 "cu_seqlens_q and cu_seqlens_k must be given together");
  if (p.visibility_bits) {
    B200FA_REQUIRE(p.cu_seqlens_q && p.visibility_bits_t && p.cu_visible_k && p.cu_visible_q,
                   "inter-sequence attention needs cu_seqlens and the prepared metadata");
  }
  return B200FA_OK;
}

static bool strides_ok(const int64_t* stride) { return stride[0] % 8 == 0 && stride[1] % 8 == 0 && stride[2] % 8 == 0; }

std::atomic<int>& pivot_setting() {
  static std::atomic<int> value([] {
    const char* env = getenv("B200FA_PIVOT_DS");
    return env && env[0] == '1' ? 1 : 0;
  }());
  return value;
}
bool pivot_ds_enabled() { return pivot_setting().load(std::memory_order_relaxed) != 0; }

}  // namespace b200fa

using namespace b200fa;

extern "C" {

const char* b200fa_last_error(void) { return g_error; }
int b200fa_version(void) { return 100; }

int b200fa_supports_head_dim(int32_t head_dim, int32_t direction) {
  if (head_dim == 64 || head_dim == 72 || head_dim == 96 || head_dim == 128 || head_dim == 256) return 1;
  return head_dim == 512 && direction == 0;  // head_dim 512: forward only
}

int b200fa_device_status(void) {
  int status = 0, zero = 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -1;
  if (cudaMemcpyFromSymbol(&status, g_device_status, sizeof(int)) != cudaSuccess) return -1;
  if (status != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  return status;
}

size_t b200fa_fwd_workspace_bytes(const b200fa_problem* p) {
  if (!p->cu_seqlens_q) return fwd_split_workspace_bytes(*p);  // partial results of the split-KV path, usually 0
  // work-list entries cover 256 query rows, 128 at head_dim 256 and 512, 256 >> shift tokens where query heads are packed
  const int tile_rows = p->head_dim >= 256 ? kBlockM : kFwdTileM >> fwd_pack_shift(*p);
  return static_cast<size_t>(work_list_entries(p->seqlen_q, p->batch, tile_rows)) * 8;
}

int b200fa_fwd(const b200fa_fwd_args* args, void* stream) {
  if (!args) {
    set_error("null arguments");
    return B200FA_ERR_INVALID;
  }
  const b200fa_problem& p = args->problem;
  int status = validate_problem(p);
  if (status != B200FA_OK) return status;
  B200FA_REQUIRE(strides_ok(args->q_stride) && strides_ok(args->k_stride) && strides_ok(args->v_stride) &&
                     strides_ok(args->out_stride),
                 "tensor strides must be multiples of 8 elements");
  B200FA_REQUIRE(reinterpret_cast<uintptr_t>(args->out) % 16 == 0, "out must be 16-byte aligned");
  if (p.batch == 0 || p.seqlen_q == 0) return B200FA_OK;
  B200FA_REQUIRE(args->q && args->out && args->softmax_lse, "null tensor pointer");
  B200FA_REQUIRE(p.seqlen_k == 0 || (args->k && args->v), "null tensor pointer");
  return launch_fwd(*args, static_cast<cudaStream_t>(stream));
}

int b200fa_set_trace(void* counters) {
  g_trace.store(static_cast<long long*>(counters), std::memory_order_relaxed);
  return B200FA_OK;
}

int b200fa_set_pivot_ds(int enabled) {
  if (enabled < 0) return pivot_setting().load(std::memory_order_relaxed);
  return pivot_setting().exchange(enabled ? 1 : 0, std::memory_order_relaxed);
}

int b200fa_bwd_timing_events(void* const* events) {
  arm_bwd_timing(events);
  return B200FA_OK;
}

size_t b200fa_bwd_workspace_bytes(const b200fa_problem* p) { return bwd_workspace_bytes(*p); }

int b200fa_bwd(const b200fa_bwd_args* args, void* stream) {
  if (!args) {
    set_error("null arguments");
    return B200FA_ERR_INVALID;
  }
  const b200fa_problem& p = args->problem;
  int status = validate_problem(p);
  if (status != B200FA_OK) return status;
  B200FA_REQUIRE(strides_ok(args->q_stride) && strides_ok(args->k_stride) && strides_ok(args->v_stride) &&
                     strides_ok(args->out_stride) && strides_ok(args->dout_stride) && strides_ok(args->dq_stride) &&
                     strides_ok(args->dk_stride) && strides_ok(args->dv_stride),
                 "tensor strides must be multiples of 8 elements");
  if (p.batch == 0) return B200FA_OK;
  // The kernels read and write these tensors with 16-byte accesses and no further checks: refuse here what would
  // otherwise fault on the device. (q, k, v, dout go through tensor maps, whose encoder checks them once more.)
  const bool have_q = p.seqlen_q > 0, have_k = p.seqlen_k > 0;
  B200FA_REQUIRE(!have_q || (args->q && args->out && args->dout && args->softmax_lse && args->dq),
                 "null tensor pointer (q, out, dout, softmax_lse and dq are required when there are query rows)");
  B200FA_REQUIRE(!have_k || (args->k && args->v && args->dk && args->dv),
                 "null tensor pointer (k, v, dk and dv are required when there are key rows)");
  const void* aligned16[] = {args->q, args->k, args->v, args->out, args->dout, args->dq, args->dk, args->dv};
  for (const void* pointer : aligned16)
    B200FA_REQUIRE(reinterpret_cast<uintptr_t>(pointer) % 16 == 0, "tensor pointers must be 16-byte aligned");
  B200FA_REQUIRE(reinterpret_cast<uintptr_t>(args->softmax_lse) % 4 == 0, "softmax_lse must be 4-byte aligned");
  return launch_bwd(*args, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
