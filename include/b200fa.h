/* b200fa -- C ABI of the B200 (sm_100a) FlashAttention library.
 *
 * This is the boundary a host binding (ctypes, cgo, JNI ...) calls. It replaces the launch interface of the
 * reference, `runtime.run(kernel, grid, threads, smem, signature, values, stream, ...)`
 * (reference src/zigfa/_impl/runtime.py:233-259), together with the launch planners that feed it
 * (src/zigfa/_impl/forward.py:118-265, backward.py:314-551, inter_sequence.py:223-562).
 *
 * Rules common to every entry point:
 *  - all tensor pointers are device pointers owned by the caller; unless an entry point says otherwise the
 *    library allocates and frees no device memory;
 *  - a call only enqueues work on `stream` (a cudaStream_t passed as void*) and returns; it never synchronises;
 *  - return value 0 = success, negative = error; b200fa_last_error() returns the message of the calling thread;
 *  - tensors are BF16 with a contiguous last dimension, 16-byte aligned base pointers and strides (in elements)
 *    that are multiples of 8 (reference src/zigfa/_impl/tensors.py:114-127);
 *  - `*_workspace_bytes` functions are pure host functions of the shapes and run without a GPU.
 */
#ifndef B200FA_H_
#define B200FA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200FA_OK 0
#define B200FA_ERR_INVALID (-1)   /* bad argument (shape, alignment, head_dim, workspace too small) */
#define B200FA_ERR_CUDA (-2)      /* a CUDA call failed */
#define B200FA_ERR_UNSUPPORTED (-3)

/* Attention problem shared by forward and backward.
 * Fixed length: q (batch, seqlen_q, heads_q, head_dim), k/v (batch, seqlen_k, heads_kv, head_dim), cu_seqlens NULL.
 * Packed (varlen / inter-sequence): q (total_q, heads_q, head_dim), k/v (total_k, heads_kv, head_dim),
 * cu_seqlens_q/k int32 prefix sums of length batch + 1; seqlen_q / seqlen_k are then the row counts of the packed
 * tensors (their shape[0]) and stride[0] is unused.
 * window_left / window_right: -1 = unbounded; causal = (left, 0). Bottom-right aligned
 * (reference tests/reference.py:10-19).
 * Inter-sequence (reference src/zigfa/_impl/ops.py:701-742): visibility_bits (batch, ceil(batch/32)) int32, bit j of
 * row i set = query sequence i sees key sequence j; visibility_bits_t is its transpose, cu_visible_k the prefix sums
 * of visible key tokens per query sequence (both from b200fa_interseq_metadata); window_sizes (2, batch) int32 or NULL.
 * All three NULL = ordinary attention. */
typedef struct b200fa_problem {
  int32_t batch;
  int32_t seqlen_q, seqlen_k;
  int32_t heads_q, heads_kv, head_dim;
  int32_t window_left, window_right;
  float softmax_scale;
  const int32_t* cu_seqlens_q;
  const int32_t* cu_seqlens_k;
  const int32_t* visibility_bits;
  const int32_t* visibility_bits_t;
  const int32_t* cu_visible_k;
  const int32_t* cu_visible_q;
  const int32_t* window_sizes;
} b200fa_problem;

/* Strides in elements: [0] batch, [1] row, [2] head. */
typedef struct b200fa_fwd_args {
  b200fa_problem problem;
  const void* q;
  const void* k;
  const void* v;
  void* out;           /* bf16, shape of q */
  float* softmax_lse;  /* fp32 (batch, heads_q, seqlen_q) or packed (heads_q, total_q); natural log; -inf = no keys */
  int64_t q_stride[3], k_stride[3], v_stride[3], out_stride[3];
  int64_t lse_stride[2]; /* [0] batch (0 when packed), [1] head; rows are contiguous */
  void* workspace;
  size_t workspace_bytes;
} b200fa_fwd_args;

/* Replaces forward.compute_scratch_shapes (reference src/zigfa/_impl/forward.py:105-115). */
size_t b200fa_fwd_workspace_bytes(const b200fa_problem* problem);
/* Replaces forward.forward (reference src/zigfa/_impl/forward.py:118-265): out = softmax(scale q k^T + mask) v. */
int b200fa_fwd(const b200fa_fwd_args* args, void* stream);

/* Forward attention without a caller workspace (no counterpart in the reference, whose forward always takes the
 * scratch tensors its op layer allocates). Meant for callers that must not allocate device memory around the call:
 * code running under a fixed device-memory plan where every byte is assigned up front, or a host-language binding
 * that owns only the input and output buffers and has no allocator to ask for a workspace. Same arguments and results as b200fa_fwd; `workspace` and
 * `workspace_bytes` are ignored. The work list of a packed batch is kept in a 64 KiB array in device memory owned by
 * the library (held by every GPU that loads it until the process exits). The limit is
 * b200fa_fwd_workspace_bytes(problem) <= 65536, i.e. at most 8192 work-list entries: one entry covers 256 query rows
 * of a sequence at head_dim <= 128 ((total_q + 255 * batch) / 256 <= 8192) and 128 rows at head_dim 256 and 512
 * ((total_q + 127 * batch) / 128 <= 8192); larger batches are rejected with B200FA_ERR_INVALID and a
 * message. (Where the query heads of a group are packed into the rows of a work item -- a power-of-two number of query
 * heads per key head, at most 16 in a packed batch, head_dim <= 128 -- an entry covers 256 / group tokens and
 * b200fa_fwd_workspace_bytes asks for that finer list; a call whose workspace holds only the list with one head per
 * work item, as this entry point's scratch may, runs unpacked (a row's sum of exponentials may then round differently
 * in its last bit; nothing else changes), so the limit above decides.) Fixed-length problems need no scratch and have no such limit. The call itself allocates and frees nothing.
 * The first call on each device looks up the array's device address (a synchronous CUDA runtime query), so make that
 * first call before any stream capture begins. All calls on a device share the one array: each call rewrites every
 * entry it uses before its kernel reads them, nothing needs clearing, but two calls whose kernels can overlap on the
 * GPU (different streams without ordering) race on it -- keep calls to this entry point stream-ordered per device. */
int b200fa_fwd_noalloc(const b200fa_fwd_args* args, void* stream);

typedef struct b200fa_bwd_args {
  b200fa_problem problem;
  const void* q;
  const void* k;
  const void* v;
  const void* out;
  const void* dout;
  const float* softmax_lse;
  void* dq;
  void* dk;
  void* dv;
  int64_t q_stride[3], k_stride[3], v_stride[3], out_stride[3], dout_stride[3];
  int64_t dq_stride[3], dk_stride[3], dv_stride[3];
  int64_t lse_stride[2];
  void* workspace;
  size_t workspace_bytes;
} b200fa_bwd_args;

/* Replaces backward.compute_scratch_shapes (reference src/zigfa/_impl/backward.py:141-180). */
size_t b200fa_bwd_workspace_bytes(const b200fa_problem* problem);
/* Replaces backward.backward (reference src/zigfa/_impl/backward.py:314-551): preprocess, dK/dV/dQ main kernel,
 * postprocess. dQ accumulates with floating-point atomics (not deterministic), as in the reference. */
int b200fa_bwd(const b200fa_bwd_args* args, void* stream);

/* Pivot gradients (the backward half of the reference's "softmax fix": zig/fragments.zig:23-30,
 * zig/flash_bwd_sm100.zig:635-645,984-997, zig/flash_bwd_postprocess.zig:150-397). With the setting on, b200fa_bwd
 * treats a key that holds more than 3/4 of the probability of a query row as the pivot of that row: its dS is not formed
 * as P (dP - D), which cancels for P near 1, but as minus the sum of the BF16 dS of the other keys of the row, and the
 * pivot terms of dQ and dK are added by the postprocess kernels. The results of rows without a pivot do not change.
 * The setting is process-wide, read at every b200fa_bwd call; it starts as 1 when the environment variable
 * B200FA_PIVOT_DS is "1" and as 0 otherwise (the pivot path costs the backward main kernel about 16 %; without it the
 * gradients stay within the stated tolerance of the BF16 reference). Returns the previous value; a negative `enabled`
 * only queries. */
int b200fa_set_pivot_ds(int enabled);

/* Measurement hook (no counterpart in the reference): the next b200fa_bwd call of the calling thread records the four
 * cudaEvent_t handles events[0..3] on its stream -- before the preprocess kernel, before the main kernel, after the
 * main kernel, after the postprocess kernel -- so a benchmark can time the main kernel by itself. NULL clears it. */
int b200fa_bwd_timing_events(void* const* events);

/* Tuning hook (no counterpart in the reference): `counters` is a device buffer of 32 int64 that the backward main
 * kernel adds cycle counts to -- slots 0-10 = cycles its warps spent in each of its waits, 11 = cycles per CTA,
 * 12 = iterations. NULL (the default) turns tracing off. Only libraries built with -DB200FA_TRACE count; the regular
 * build accepts the call and records nothing. */
int b200fa_set_trace(void* counters);

/* Replaces inter_sequence.prepare_metadata (reference src/zigfa/_impl/inter_sequence.py:223-254).
 * Outputs: bits_t (n, ceil(n/32)) int32, cu_visible_k (n + 1) int32, cu_visible_q (n + 1) int32 (saturating). */
int b200fa_interseq_metadata(const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k, const int32_t* visibility_bits,
                             int32_t num_sequences, int32_t* bits_t, int32_t* cu_visible_k, int32_t* cu_visible_q,
                             void* stream);

/* Builds the sorted work list of a packed batch on the device: entry e = (sequence, block), sequences ordered by
 * descending length class of `cu_seqlens_other` within windows of 1024 sequences, padding entries (batch, 0).
 * Replaces tensors.build_scheduler_metadata (reference src/zigfa/_impl/tensors.py:87-107,
 * zig/prepare_scheduler.zig:101-170). `descending` orders the blocks of a sequence last-to-first. */
int b200fa_work_list(const int32_t* cu_seqlens, const int32_t* cu_seqlens_other, int32_t batch, int32_t block_rows,
                     int32_t descending, int32_t num_entries, int32_t* table, void* stream);
/* Host twins of the integer kernels (same code path compiled for the CPU; used by the CPU unit tests). */
int64_t b200fa_work_list_entries(int64_t rows, int64_t batch, int64_t block_rows);
int b200fa_work_list_host(const int32_t* cu_seqlens, const int32_t* cu_seqlens_other, int32_t batch, int32_t block_rows,
                          int32_t descending, int32_t num_entries, int32_t* table);
int b200fa_interseq_metadata_host(const int32_t* cu_seqlens_q, const int32_t* cu_seqlens_k,
                                  const int32_t* visibility_bits, int32_t num_sequences, int32_t* bits_t,
                                  int32_t* cu_visible_k, int32_t* cu_visible_q);
/* Lists, for query rows [m0, m1) of sequence `seq`, the key blocks the forward kernel visits:
 * out[4*i..4*i+3] = (first key row in the packed tensor, first column relative to its run, run length, banded).
 * Returns the number of blocks (at most max_blocks are written). Host twin of the device cursor. */
int b200fa_key_blocks_host(const b200fa_problem* problem, int32_t seq, int32_t m0, int32_t m1, int32_t* out,
                           int32_t max_blocks);
/* Same for the backward pass: query blocks that see key columns [c0, c1) of key sequence `seq`. */
int b200fa_query_blocks_host(const b200fa_problem* problem, int32_t seq, int32_t c0, int32_t c1, int32_t* out,
                             int32_t max_blocks);

/* Reads and clears the device-side status word (synchronises the device). 0 = no kernel wait ran out of time. */
int b200fa_device_status(void);
const char* b200fa_last_error(void);
int b200fa_version(void);
/* 1 when head_dim is supported by the forward (direction 0) / backward (direction 1) kernels. */
int b200fa_supports_head_dim(int32_t head_dim, int32_t direction);

#ifdef __cplusplus
}
#endif
#endif /* B200FA_H_ */
