// Integer side of the attention path, shared by the CUDA kernels and the host (CPU unit tests call the same code
// through the host entry points of the library): sequence offsets, the bottom-right aligned causal / sliding-window
// band, tile-skip ranges, the key-block cursor over visible key runs (fixed length, varlen and inter-sequence
// visibility bits), the mirrored query-block cursor of the backward pass, and the length classes of the work list.
//
// Semantics follow the reference's definitions:
//   band            zig/BlockInfo.zig:12-27, tests/reference.py:10-19  (col <= row + (Lk-Lq) + right, >= ... - left)
//   tile skipping   zig/BlockInfo.zig:42-67
//   key runs        zig/inter_sequence.zig:27-97 (maximal runs of set bits; only the query's own sequence is banded)
//   length class    zig/prepare_scheduler.zig:18-24
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define B200FA_HD __host__ __device__ __forceinline__
#else
#define B200FA_HD inline
#endif

namespace b200fa {

constexpr int kBlockN = 128;     // keys per block
constexpr int kBlockM = 128;     // query rows per MMA tile
constexpr int kFwdTileM = 256;   // query rows per forward work item (two MMA tiles)

B200FA_HD int imin(int a, int b) { return a < b ? a : b; }
B200FA_HD int imax(int a, int b) { return a > b ? a : b; }
B200FA_HD int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ceil(log2)-style class used to order sequences by work: exponent << 2 | next two mantissa bits.
B200FA_HD uint32_t length_class(uint32_t length) {
  if (length == 0) return 0;
  uint32_t exponent = 31;
  while (!((length >> exponent) & 1u)) --exponent;
  uint32_t mantissa = static_cast<uint32_t>(((static_cast<uint64_t>(length) << 2) >> exponent) & 3u);
  return (exponent << 2) | mantissa;
}

// Visible columns of query row `row` (relative to its sequence) are [lo(row), hi(row)) within a key sequence of
// length lk, when the query sequence has length lq. left/right = -1 means unbounded on that side.
struct Band {
  int off;  // lk - lq
  int lk;
  int left, right;
  B200FA_HD bool unbounded() const { return left < 0 && right < 0; }
  B200FA_HD int lo(int row) const { return left < 0 ? 0 : imax(0, row + off - left); }
  B200FA_HD int hi(int row) const { return right < 0 ? lk : imin(lk, row + off + right + 1); }
  // Rows [row_lo(c0), row_hi(c1)) are the only ones that can see a column in [c0, c1).
  B200FA_HD int row_lo(int c0) const { return right < 0 ? 0 : imax(0, c0 - off - right); }
  B200FA_HD int row_hi(int c1, int lq) const { return left < 0 ? lq : imin(lq, c1 - off + left); }
};

B200FA_HD Band make_band(int lq, int lk, int left, int right) {
  Band b;
  b.off = lk - lq;
  b.lk = lk;
  b.left = left;
  b.right = right;
  return b;
}

// Key blocks [first, last) of a banded key sequence that rows [m0, m1) can see (m1 > m0).
B200FA_HD void band_key_block_range(const Band& band, int m0, int m1, int* first, int* last) {
  int lo = band.lo(m0);
  int hi = band.hi(m1 - 1);
  if (hi <= lo || hi <= 0 || lo >= band.lk) {
    *first = 0;
    *last = 0;
    return;
  }
  *first = lo / kBlockN;
  *last = ceil_div(hi, kBlockN);
}
// Query blocks [first, last) (of kBlockM rows) of a banded query sequence that can see key columns [c0, c1).
B200FA_HD void band_query_block_range(const Band& band, int lq, int c0, int c1, int* first, int* last) {
  int lo = band.row_lo(c0);
  int hi = band.row_hi(c1, lq);
  if (hi <= lo || hi <= 0 || lo >= lq) {
    *first = 0;
    *last = 0;
    return;
  }
  *first = lo / kBlockM;
  *last = ceil_div(hi, kBlockM);
}

// Problem description common to forward and backward kernels (plain data; passed by value to kernels).
struct Problem {
  int batch;        // batch entries (fixed length) or sequences (varlen / inter-sequence)
  int seqlen_q;     // fixed length only
  int seqlen_k;     // fixed length only
  int heads_q, heads_kv;
  int window_left, window_right;
  const int32_t* cu_q;  // null = fixed length
  const int32_t* cu_k;
  // inter-sequence visibility (null = every sequence sees only itself)
  const int32_t* bits;          // (n, words): bit j of row i set = query sequence i sees key sequence j
  const int32_t* bits_t;        // transpose
  const int32_t* window_sizes;  // (2, n) or null
  int words;
};

struct SeqInfo {
  int q0, k0;  // first row of the sequence in the packed q / k tensors (0 for fixed length)
  int lq, lk;
  int batch_coord;  // batch coordinate for tensor maps (0 for packed layouts)
};

B200FA_HD SeqInfo seq_info(const Problem& p, int seq) {
  SeqInfo s;
  if (p.cu_q) {
    s.q0 = p.cu_q[seq];
    s.k0 = p.cu_k[seq];
    s.lq = p.cu_q[seq + 1] - s.q0;
    s.lk = p.cu_k[seq + 1] - s.k0;
    s.batch_coord = 0;
  } else {
    s.q0 = 0;
    s.k0 = 0;
    s.lq = p.seqlen_q;
    s.lk = p.seqlen_k;
    s.batch_coord = seq;
  }
  return s;
}

B200FA_HD void window_of(const Problem& p, int seq, int* left, int* right) {
  if (p.window_sizes) {
    *left = p.window_sizes[seq];
    *right = p.window_sizes[p.batch + seq];
  } else {
    *left = p.window_left;
    *right = p.window_right;
  }
}

// One block of the "other" side handed out by a cursor.
struct OtherBlock {
  int row;      // first row of the block in the packed tensor of the other side (tensor-map row coordinate)
  int col0;     // first column (key cursor) / row (query cursor) of the block relative to its sequence or run
  int limit;    // length of the sequence or run: entries at col0 + i >= limit are out of range
  int banded;   // 1: the band of `band` applies (block of the sequence itself); 0: dense
};

// Walks the key blocks that the query rows [m0, m1) of sequence `seq` can see, in increasing key order.
// Fixed length / varlen: one banded run (the sequence's own keys). Inter-sequence: every maximal run of visible key
// sequences is a dense run of contiguous key rows, except that the query's own key sequence is a banded run of its
// own when a window or causal bound applies to it.
// kBits = false compiles the visibility-bit scan out (problems without bits: fixed length and plain packed batches);
// the forward kernel at head_dim <= 128 has an instance of its own for them, because the scan code inlined into its
// three roles costs short sequences a few percent even when it never runs.
template <bool kBits>
struct KeyCursorT {
  const Problem* p;
  int seq, m0, m1;
  Band band;       // band of the sequence itself
  int self_banded;
  // current run
  int run_row0, run_len, run_banded;
  int blk, blk_end;
  // scan position over key sequences (inter-sequence only); -1 = finished
  int scan;

  B200FA_HD void init(const Problem* problem, int sequence, const SeqInfo& s, int row0, int row1) {
    p = problem;
    seq = sequence;
    m0 = row0;
    m1 = row1;
    int left, right;
    window_of(*p, seq, &left, &right);
    band = make_band(s.lq, s.lk, left, right);
    blk = 0;
    blk_end = 0;
    if (m1 <= m0) {
      scan = -1;
      return;
    }
    if (!kBits || !p->bits) {
      scan = -1;
      run_row0 = s.k0;
      run_len = s.lk;
      run_banded = 1;
      band_key_block_range(band, m0, m1, &blk, &blk_end);
    } else {
      self_banded = !band.unbounded();
      scan = 0;
    }
  }

  B200FA_HD bool bit(int j) const { return (static_cast<uint32_t>(p->bits[seq * p->words + (j >> 5)]) >> (j & 31)) & 1u; }

  // Split-KV: keeps share `split` of `splits` equal shares of the key blocks (call right after init; problems with
  // one key run only, i.e. without visibility bits). Shares of a run shorter than `splits` blocks may be empty.
  B200FA_HD void restrict_to_share(int split, int splits) {
    // 32-bit arithmetic on purpose (a run has far fewer than 2^26 blocks and there are at most 32 shares): a 64-bit
    // division is a subroutine call, which the warp-specialised kernels avoid.
    const unsigned n = static_cast<unsigned>(blk_end - blk), first = static_cast<unsigned>(blk);
    blk = static_cast<int>(first + n * static_cast<unsigned>(split) / static_cast<unsigned>(splits));
    blk_end = static_cast<int>(first + n * static_cast<unsigned>(split + 1) / static_cast<unsigned>(splits));
  }

  // Finds the next non-empty run at or after `scan`. Returns false when there is none.
  B200FA_HD bool next_run() {
    const int n = p->batch;
    while (scan >= 0 && scan < n) {
      int j = scan;
      // skip to the next set bit
      while (j < n) {
        uint32_t word = static_cast<uint32_t>(p->bits[seq * p->words + (j >> 5)]) >> (j & 31);
        if (word == 0) {
          j = ((j >> 5) + 1) << 5;
        } else {
          while (!(word & 1u)) {
            word >>= 1;
            ++j;
          }
          break;
        }
      }
      if (j >= n) break;
      if (j == seq && self_banded) {
        scan = j + 1;
        run_row0 = p->cu_k[j];
        run_len = p->cu_k[j + 1] - run_row0;
        run_banded = 1;
        band_key_block_range(band, m0, m1, &blk, &blk_end);
        if (blk_end > blk) return true;
        continue;
      }
      int e = j + 1;
      while (e < n && bit(e) && !(e == seq && self_banded)) ++e;
      scan = e;
      run_row0 = p->cu_k[j];
      run_len = p->cu_k[e] - run_row0;
      run_banded = 0;
      blk = 0;
      blk_end = ceil_div(run_len, kBlockN);
      if (blk_end > blk) return true;
    }
    scan = -1;
    return false;
  }

  B200FA_HD bool next(OtherBlock* out) {
    if (blk >= blk_end) {
      if (!kBits || scan < 0 || !next_run()) return false;
    }
    out->row = run_row0 + blk * kBlockN;
    out->col0 = blk * kBlockN;
    out->limit = run_len;
    out->banded = run_banded;
    ++blk;
    return true;
  }
};

using KeyCursor = KeyCursorT<true>;

// Mirror of KeyCursor for the backward pass: walks the query blocks (kBlockM rows) that can see the key columns
// [c0, c1) of key sequence `seq`, in increasing query order. Uses the transposed visibility bits.
// kBits = false compiles the scan of the transposed visibility bits out. The backward kernels use the full cursor:
// an instance without the scan measured 1-3 % slower there, unlike in the forward kernel.
template <bool kBits>
struct QueryCursorT {
  const Problem* p;
  int seq, c0, c1;
  Band band;
  int self_banded;
  int self_lq;
  int run_row0, run_len, run_banded;
  int blk, blk_end;
  int scan;

  B200FA_HD void init(const Problem* problem, int sequence, const SeqInfo& s, int col0, int col1) {
    p = problem;
    seq = sequence;
    c0 = col0;
    c1 = col1;
    int left, right;
    window_of(*p, seq, &left, &right);
    band = make_band(s.lq, s.lk, left, right);
    self_lq = s.lq;
    blk = 0;
    blk_end = 0;
    if (c1 <= c0) {
      scan = -1;
      return;
    }
    if (!kBits || !p->bits_t) {
      scan = -1;
      run_row0 = s.q0;
      run_len = s.lq;
      run_banded = 1;
      band_query_block_range(band, s.lq, c0, c1, &blk, &blk_end);
    } else {
      self_banded = !band.unbounded();
      scan = 0;
    }
  }

  B200FA_HD bool bit(int i) const {
    return (static_cast<uint32_t>(p->bits_t[seq * p->words + (i >> 5)]) >> (i & 31)) & 1u;
  }

  B200FA_HD bool next_run() {
    const int n = p->batch;
    while (scan >= 0 && scan < n) {
      int i = scan;
      while (i < n) {
        uint32_t word = static_cast<uint32_t>(p->bits_t[seq * p->words + (i >> 5)]) >> (i & 31);
        if (word == 0) {
          i = ((i >> 5) + 1) << 5;
        } else {
          while (!(word & 1u)) {
            word >>= 1;
            ++i;
          }
          break;
        }
      }
      if (i >= n) break;
      if (i == seq && self_banded) {
        scan = i + 1;
        run_row0 = p->cu_q[i];
        run_len = self_lq;
        run_banded = 1;
        band_query_block_range(band, self_lq, c0, c1, &blk, &blk_end);
        if (blk_end > blk) return true;
        continue;
      }
      int e = i + 1;
      while (e < n && bit(e) && !(e == seq && self_banded)) ++e;
      scan = e;
      run_row0 = p->cu_q[i];
      run_len = p->cu_q[e] - run_row0;
      run_banded = 0;
      blk = 0;
      blk_end = ceil_div(run_len, kBlockM);
      if (blk_end > blk) return true;
    }
    scan = -1;
    return false;
  }

  B200FA_HD bool next(OtherBlock* out) {
    if (blk >= blk_end) {
      if (!kBits || scan < 0 || !next_run()) return false;
    }
    out->row = run_row0 + blk * kBlockM;
    out->col0 = blk * kBlockM;
    out->limit = run_len;
    out->banded = run_banded;
    ++blk;
    return true;
  }
};
using QueryCursor = QueryCursorT<true>;

// Number of entries of a work list over `rows` packed rows in `batch` sequences with `block` rows per entry
// (upper bound that needs no knowledge of the individual lengths): reference src/zigfa/_impl/tensors.py:79-84.
B200FA_HD int64_t work_list_entries(int64_t rows, int64_t batch, int64_t block) {
  if (batch == 0) return rows;
  int64_t blocks = (rows + batch * (block - 1)) / block;
  return blocks < rows ? blocks : rows;
}

}  // namespace b200fa
