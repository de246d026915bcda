// Integer kernels of the attention path and their host twins:
//   * the sorted work list of a packed batch (takes the place of the reference's *_prepare_varlen_num_blocks kernels,
//     zig/prepare_scheduler.zig:101-170),
//   * inter-sequence metadata: bit-matrix transpose and visible-token prefix sums (zig/inter_sequence.zig:225-249,
//     682-726).
// The host twins run the same definitions on the CPU; CPU unit tests compare them with the numpy oracle and GPU tests
// compare the kernels with both, bit for bit.
#include <algorithm>
#include <vector>

#include "common.h"

namespace b200fa {

constexpr int kListThreads = 1024;
constexpr uint32_t kClasses = 128;

// ------------------------------------------------------------------------------------------------ work list
__global__ void __launch_bounds__(kListThreads, 1)
work_list_kernel(const int32_t* __restrict__ cu, const int32_t* __restrict__ cu_other, int batch, int block_rows,
                 int descending, int num_entries, int2* __restrict__ table) {
  __shared__ uint32_t keys[kListThreads];
  __shared__ int order[kListThreads];
  __shared__ int count[kListThreads];
  __shared__ int scan[kListThreads];
  __shared__ int written_shared;
  const int tid = threadIdx.x;
  if (tid == 0) written_shared = 0;
  __syncthreads();
  for (int first = 0; first < batch; first += kListThreads) {
    const int i = first + tid;
    const bool valid = i < batch;
    uint32_t key = 2 * kClasses;  // invalid entries sort last
    int blocks = 0;
    if (valid) {
      const uint32_t other = static_cast<uint32_t>(cu_other[i + 1] - cu_other[i]);
      key = kClasses - 1 - length_class(other);
      // A prefix-sum array that is not non-decreasing describes no batch; its negative lengths count as empty
      // sequences, so that no entry index can become negative (the kernels that read the list then skip them).
      blocks = ceil_div(imax(cu[i + 1] - cu[i], 0), block_rows);
    }
    keys[tid] = key;
    __syncthreads();
    int rank = 0;
    for (int j = 0; j < kListThreads; ++j) {
      const uint32_t other_key = keys[j];
      rank += (other_key < key || (other_key == key && j < tid)) ? 1 : 0;
    }
    order[rank] = i;
    count[rank] = blocks;
    __syncthreads();
    // inclusive scan of count[] (Hillis-Steele, double buffered through `scan`)
    int value = count[tid];
    scan[tid] = value;
    __syncthreads();
    for (int distance = 1; distance < kListThreads; distance <<= 1) {
      const int add = tid >= distance ? scan[tid - distance] : 0;
      __syncthreads();
      value += add;
      scan[tid] = value;
      __syncthreads();
    }
    const int base = written_shared;
    const int my_blocks = count[tid];
    const int start = base + value - my_blocks;
    const int sequence = order[tid];
    for (int b = 0; b < my_blocks; ++b) {
      const int entry = start + b;
      if (entry >= 0 && entry < num_entries) table[entry] = make_int2(sequence, descending ? my_blocks - 1 - b : b);
    }
    __syncthreads();
    if (tid == kListThreads - 1) written_shared = base + value;
    __syncthreads();
  }
  for (int entry = written_shared + tid; entry < num_entries; entry += kListThreads) table[entry] = make_int2(batch, 0);
}

// ------------------------------------------------------------------------------------------------ metadata
__global__ void transpose_bits_kernel(const int32_t* __restrict__ bits, int n, int words, int32_t* __restrict__ bits_t) {
  const int index = blockIdx.x * blockDim.x + threadIdx.x;
  if (index >= n * words) return;
  const int j = index / words, w = index - j * words;
  uint32_t out = 0;
  for (int b = 0; b < 32; ++b) {
    const int i = 32 * w + b;
    if (i < n) out |= ((static_cast<uint32_t>(bits[i * words + (j >> 5)]) >> (j & 31)) & 1u) << b;
  }
  bits_t[index] = static_cast<int32_t>(out);
}

// out_k[i + 1] = tokens of the key sequences that query sequence i sees; out_q[i + 1] = tokens of the query sequences
// that see key sequence i (both clamped to INT32_MAX); element 0 = 0.
__global__ void visible_tokens_kernel(const int32_t* __restrict__ cu_q, const int32_t* __restrict__ cu_k,
                                      const int32_t* __restrict__ bits, int n, int words, int32_t* __restrict__ out_k,
                                      int32_t* __restrict__ out_q) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i == 0) {
    out_k[0] = 0;
    out_q[0] = 0;
  }
  if (i >= n) return;
  long long sum_k = 0, sum_q = 0;
  for (int j = 0; j < n; ++j) {
    if ((static_cast<uint32_t>(bits[i * words + (j >> 5)]) >> (j & 31)) & 1u) sum_k += cu_k[j + 1] - cu_k[j];
    if ((static_cast<uint32_t>(bits[j * words + (i >> 5)]) >> (i & 31)) & 1u) sum_q += cu_q[j + 1] - cu_q[j];
  }
  out_k[i + 1] = static_cast<int32_t>(sum_k > INT32_MAX ? INT32_MAX : sum_k);
  out_q[i + 1] = static_cast<int32_t>(sum_q > INT32_MAX ? INT32_MAX : sum_q);
}

// In-place saturating inclusive prefix sums of two arrays of n + 1 entries (entry 0 stays 0). One CTA.
__global__ void __launch_bounds__(kListThreads, 1) saturating_scan_kernel(int32_t* a, int32_t* b, int n) {
  __shared__ long long warp_sums[2][32];
  __shared__ long long carry[2];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < 2) carry[tid] = 0;
  __syncthreads();
  for (int first = 1; first <= n; first += kListThreads) {
    const int i = first + tid;
    long long v[2] = {i <= n ? a[i] : 0, i <= n ? b[i] : 0};
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      long long x = v[which];
      for (int d = 1; d < 32; d <<= 1) {
        long long y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      if (lane == 31) warp_sums[which][warp] = x;
      v[which] = x;
    }
    __syncthreads();
    if (warp < 2) {
      long long x = warp_sums[warp][lane];
      for (int d = 1; d < 32; d <<= 1) {
        long long y = __shfl_up_sync(0xffffffffu, x, d);
        if (lane >= d) x += y;
      }
      warp_sums[warp][lane] = x;
    }
    __syncthreads();
    long long total[2];
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      total[which] = carry[which] + v[which] + (warp > 0 ? warp_sums[which][warp - 1] : 0);
    }
    if (i <= n) {
      a[i] = static_cast<int32_t>(total[0] > INT32_MAX ? INT32_MAX : total[0]);
      b[i] = static_cast<int32_t>(total[1] > INT32_MAX ? INT32_MAX : total[1]);
    }
    __syncthreads();
    if (tid < 2) carry[tid] += warp_sums[tid][31];
    __syncthreads();
  }
}

Problem to_problem(const b200fa_problem& in) {
  Problem p;
  p.batch = in.batch;
  p.seqlen_q = in.seqlen_q;
  p.seqlen_k = in.seqlen_k;
  p.heads_q = in.heads_q;
  p.heads_kv = in.heads_kv;
  p.window_left = in.window_left;
  p.window_right = in.window_right;
  p.cu_q = in.cu_seqlens_q;
  p.cu_k = in.cu_seqlens_k;
  p.bits = in.visibility_bits;
  p.bits_t = in.visibility_bits_t;
  p.window_sizes = in.window_sizes;
  p.words = (in.batch + 31) / 32;
  return p;
}

}  // namespace b200fa

using namespace b200fa;

extern "C" {

int64_t b200fa_work_list_entries(int64_t rows, int64_t batch, int64_t block_rows) {
  return work_list_entries(rows, batch, block_rows);
}

int b200fa_work_list(const int32_t* cu_seqlens, const int32_t* cu_seqlens_other, int32_t batch, int32_t block_rows,
                     int32_t descending, int32_t num_entries, int32_t* table, void* stream) {
  B200FA_REQUIRE(batch >= 0 && block_rows > 0 && num_entries >= 0, "work list: bad sizes");
  if (num_entries == 0) return B200FA_OK;
  B200FA_REQUIRE(cu_seqlens && cu_seqlens_other && table, "work list: null pointer");
  B200FA_REQUIRE(reinterpret_cast<uintptr_t>(table) % 8 == 0, "work list: table must be 8-byte aligned");
  work_list_kernel<<<1, kListThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      cu_seqlens, cu_seqlens_other, batch, block_rows, descending, num_entries, reinterpret_cast<int2*>(table));
  B200FA_CUDA_CHECK(cudaGetLastError());
  return B200FA_OK;
}

int b200fa_work_list_host(const int32_t* cu_seqlens, const int32_t* cu_seqlens_other, int32_t batch, int32_t block_rows,
                          int32_t descending, int32_t num_entries, int32_t* table) {
  B200FA_REQUIRE(batch >= 0 && block_rows > 0 && num_entries >= 0, "work list: bad sizes");
  int written = 0;
  for (int first = 0; first < batch; first += kListThreads) {
    const int last = std::min(batch, first + kListThreads);
    std::vector<int> order;
    for (int i = first; i < last; ++i) order.push_back(i);
    std::stable_sort(order.begin(), order.end(), [&](int x, int y) {
      return length_class(static_cast<uint32_t>(cu_seqlens_other[x + 1] - cu_seqlens_other[x])) >
             length_class(static_cast<uint32_t>(cu_seqlens_other[y + 1] - cu_seqlens_other[y]));
    });
    for (int sequence : order) {
      const int blocks = ceil_div(imax(cu_seqlens[sequence + 1] - cu_seqlens[sequence], 0), block_rows);  // as the kernel
      for (int b = 0; b < blocks; ++b, ++written) {
        if (written < num_entries) {
          table[2 * written] = sequence;
          table[2 * written + 1] = descending ? blocks - 1 - b : b;
        }
      }
    }
  }
  for (; written < num_entries; ++written) {
    table[2 * written] = batch;
    table[2 * written + 1] = 0;
  }
  return B200FA_OK;
}

int b200fa_interseq_metadata(const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* visibility_bits,
                             int32_t n, int32_t* bits_t, int32_t* cu_visible_k, int32_t* cu_visible_q, void* stream_) {
  B200FA_REQUIRE(n >= 1, "inter-sequence metadata needs at least one sequence");
  B200FA_REQUIRE(cu_seqlens_q && cu_seqlens_k && visibility_bits && bits_t && cu_visible_k && cu_visible_q,
                 "inter-sequence metadata: null pointer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int words = (n + 31) / 32;
  transpose_bits_kernel<<<ceil_div(n * words, 256), 256, 0, stream>>>(visibility_bits, n, words, bits_t);
  visible_tokens_kernel<<<ceil_div(n, 128), 128, 0, stream>>>(cu_seqlens_q, cu_seqlens_k, visibility_bits, n, words,
                                                              cu_visible_k, cu_visible_q);
  saturating_scan_kernel<<<1, kListThreads, 0, stream>>>(cu_visible_k, cu_visible_q, n);
  B200FA_CUDA_CHECK(cudaGetLastError());
  return B200FA_OK;
}

int b200fa_interseq_metadata_host(const int32_t* cu_q, const int32_t* cu_k, const int32_t* bits, int32_t n,
                                  int32_t* bits_t, int32_t* cu_visible_k, int32_t* cu_visible_q) {
  B200FA_REQUIRE(n >= 1, "inter-sequence metadata needs at least one sequence");
  const int words = (n + 31) / 32;
  auto bit = [&](int i, int j) { return (static_cast<uint32_t>(bits[i * words + (j >> 5)]) >> (j & 31)) & 1u; };
  for (int j = 0; j < n; ++j)
    for (int w = 0; w < words; ++w) {
      uint32_t out = 0;
      for (int b = 0; b < 32; ++b)
        if (32 * w + b < n) out |= bit(32 * w + b, j) << b;
      bits_t[j * words + w] = static_cast<int32_t>(out);
    }
  long long sum_k = 0, sum_q = 0;
  cu_visible_k[0] = 0;
  cu_visible_q[0] = 0;
  for (int i = 0; i < n; ++i) {
    for (int j = 0; j < n; ++j) {
      if (bit(i, j)) sum_k += cu_k[j + 1] - cu_k[j];
      if (bit(j, i)) sum_q += cu_q[j + 1] - cu_q[j];
    }
    cu_visible_k[i + 1] = static_cast<int32_t>(std::min<long long>(sum_k, INT32_MAX));
    cu_visible_q[i + 1] = static_cast<int32_t>(std::min<long long>(sum_q, INT32_MAX));
  }
  return B200FA_OK;
}

int b200fa_key_blocks_host(const b200fa_problem* problem, int32_t seq, int32_t m0, int32_t m1, int32_t* out,
                           int32_t max_blocks) {
  Problem p = to_problem(*problem);
  SeqInfo s = seq_info(p, seq);
  KeyCursor cursor;
  cursor.init(&p, seq, s, m0, imin(m1, s.lq));
  OtherBlock block;
  int count = 0;
  while (cursor.next(&block)) {
    if (count < max_blocks) {
      out[4 * count] = block.row;
      out[4 * count + 1] = block.col0;
      out[4 * count + 2] = block.limit;
      out[4 * count + 3] = block.banded;
    }
    ++count;
  }
  return count;
}

int b200fa_query_blocks_host(const b200fa_problem* problem, int32_t seq, int32_t c0, int32_t c1, int32_t* out,
                             int32_t max_blocks) {
  Problem p = to_problem(*problem);
  SeqInfo s = seq_info(p, seq);
  QueryCursor cursor;
  cursor.init(&p, seq, s, c0, imin(c1, s.lk));
  OtherBlock block;
  int count = 0;
  while (cursor.next(&block)) {
    if (count < max_blocks) {
      out[4 * count] = block.row;
      out[4 * count + 1] = block.col0;
      out[4 * count + 2] = block.limit;
      out[4 * count + 3] = block.banded;
    }
    ++count;
  }
  return count;
}

}  // extern "C"
