// Work list of one (sequence, kv head, split) of the sparse decode-attention
// kernels.  The list is the concatenation of
//   * the physical pages of the selected blocks that fall into the block range,
//   * (hybrid mode) tiles of 16 consecutive blocks whose unselected members
//     contribute their representative (z, v_bar),
//   * the pages of the generated suffix [prefix_len, seq_len).
// Split s of n owns the items [N s / n, N (s + 1) / n).  Descriptors are
// resolved (selection list -> block table -> physical page) by all threads at
// once and parked in shared memory, so that the load pipeline never waits on a
// dependent global load.
#pragma once

#include "ia_common.cuh"

namespace ia {

struct DecodeParams {
  const void* q;
  const void* k_pool;
  const void* v_pool;
  const int32_t* block_table;
  const int32_t* prefix_lens;
  const int32_t* seq_lens;
  const int32_t* sel_idx;
  const int32_t* sel_count;
  const void* v_bar;  // hybrid only
  const float* z;     // hybrid only: [batch, rows, max_blocks]
  float* o_partial;
  float* lse_partial;
  // optional fused finalize: the CTA that completes a (sequence, kv head) last merges
  // its n_splits partials and writes the output rows [batch, rows, D] itself
  void* final_out;      // null: partials only
  int* split_counters;  // [batch * kv heads], zero at launch; reset by the merging CTA
  int final_dtype;      // ia_dtype of final_out
  // optional exchange with peer GPUs (split-KV across GPUs): instead of o_partial / lse_partial every
  // partial is stored into the gather buffer of every rank - this one's included - over peer pointers,
  // and the last CTA of the grid publishes this rank's step number on every rank
  ia_peer_exchange px;  // n_ranks == 0: no exchange
  int64_t page_stride, head_stride;
  int n_kv_heads, group_size, page_size, block_size, max_pages, max_blocks, max_sel;
  int rep_mode, n_splits, block_lo, block_hi, with_suffix;
  // Guards for caller-supplied indices: a selected block outside [0, max_blocks), or a block-table
  // entry outside [0, n_pool_pages) (n_pool_pages 0: the pool size is unknown, entries are trusted),
  // makes its item empty - nothing is read through it - and sets DEV_STATUS_BAD_INDEX in *status.
  int n_pool_pages;
  int* status;  // device status word
  // Equal-share grid (sparse_decode_mma.cu, flat kernel): partials of the (CTA, pair) segments,
  // [slot][G][D] and [slot][G] with slot = cta + pair.
  float* flat_o;
  float* flat_lse;
  int n_pairs;
#ifdef IA_DECODE_TRACE
  float* trace;  // profiling build: 16 floats per CTA, time stamps of the kernel's phases
#endif
};

// Profiling build (-DIA_DECODE_TRACE): thread 0 of every CTA leaves time stamps (microseconds since the
// CTA started, from the nanosecond global timer) in a buffer whose address the environment variable
// IA_TRACE_PTR gives - a timeline of the attention kernel's phases without a profiler.  Slot 15 holds the
// CTA's start (low 24 bits of the timer, ns), slot 14 the SM it ran on.
#ifdef IA_DECODE_TRACE
__device__ __forceinline__ unsigned long long decode_trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define IA_DTRACE_BEGIN()                                                                           \
  const unsigned long long dtrace_t0 = decode_trace_now();                                           \
  if (threadIdx.x == 0 && p.trace != nullptr) {                                                      \
    unsigned dtrace_sm;                                                                              \
    asm volatile("mov.u32 %0, %%smid;" : "=r"(dtrace_sm));                                           \
    p.trace[(int64_t)blockIdx.x * 16 + 15] = (float)(dtrace_t0 & 0xffffffull);                       \
    p.trace[(int64_t)blockIdx.x * 16 + 14] = (float)dtrace_sm;                                       \
  }                                                                                                  \
  do { } while (0)
#define IA_DTRACE(i)                                                                                 \
  do {                                                                                               \
    if (threadIdx.x == 0 && p.trace != nullptr)                                                      \
      p.trace[(int64_t)blockIdx.x * 16 + (i)] = (float)(decode_trace_now() - dtrace_t0) * 1e-3f;     \
  } while (0)
#else
#define IA_DTRACE_BEGIN() do { } while (0)
#define IA_DTRACE(i) do { } while (0)
#endif

enum : int { ITEM_PAGE = 0, ITEM_REP_TILE = 1 };
constexpr int kRepTile = 16;     // blocks per representative tile (= page_size rows of v_bar)
constexpr int kItemChunk = 512;  // descriptors resident in shared memory at a time

// kind, first: physical page (ITEM_PAGE) or first block (ITEM_REP_TILE),
// lo/hi: valid rows [lo, hi) of the page / tile
struct __align__(16) Item { int kind, first, lo, hi; };

struct ItemRange {
  int prefix, seq_len, nb_eff, lo_b, hi_b;
  int sel_first, n_sel_items, n_rep, n_suf, suf_first_page;
  int begin, end;  // this split's items
};

// Called by every thread of the CTA.  scratch: 2 ints of shared memory.
__device__ __forceinline__ ItemRange item_range(const DecodeParams& p, int seq, int head, int split,
                                                int* scratch) {
  ItemRange r;
  // lengths come from device memory: never index the block table past its row
  const int capacity = p.max_pages * p.page_size;
  r.prefix = min(max(p.prefix_lens[seq], 0), capacity);
  r.seq_len = min(p.seq_lens[seq], capacity);
  r.nb_eff = min((r.prefix + p.block_size - 1) / p.block_size, p.max_blocks);
  r.lo_b = max(p.block_lo, 0);
  r.hi_b = min(p.block_hi, r.nb_eff);
  const int pair = seq * p.n_kv_heads + head;
  const int count = min(p.sel_count[pair], p.max_sel);
  const int32_t* idx = p.sel_idx + (int64_t)pair * p.max_sel;
  int n_sel;
  if (r.lo_b == 0 && r.hi_b >= r.nb_eff) {
    // every block is in range: the whole list, no counting pass (and none of its barriers); entries
    // out of range or out of order are caught where they are resolved
    r.sel_first = 0;
    n_sel = max(count, 0);
  } else {
    if (threadIdx.x < 2) scratch[threadIdx.x] = 0;
    __syncthreads();
    // The list is ascending (ia_select writes it so; the header asks it of callers): the entries of the
    // block range are then the run [#(b < lo), #(b < hi)).  A list out of order - an entry that follows
    // a larger one - or an entry outside [0, max_blocks) is reported in the status word; the result is
    // then unspecified but every access stays guarded.
    int below_lo = 0, below_hi = 0, disorder = 0;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
      const int b = idx[i];
      below_lo += (b < r.lo_b);
      below_hi += (b < r.hi_b);
      disorder |= (i > 0 && idx[i - 1] >= b) || b < 0 || b >= p.max_blocks;  // out of range: dropped by the range below
    }
    if (below_lo) atomicAdd(&scratch[0], below_lo);
    if (below_hi) atomicAdd(&scratch[1], below_hi);
    if (disorder && p.status != nullptr) atomicOr(p.status, DEV_STATUS_BAD_INDEX);
    __syncthreads();
    r.sel_first = scratch[0];
    n_sel = max(scratch[1] - scratch[0], 0);
    __syncthreads();
  }
  const int ppb = p.block_size / p.page_size;
  r.n_sel_items = n_sel * ppb;
  r.n_rep = (p.rep_mode == IA_REP_HYBRID && r.hi_b > r.lo_b) ? (r.hi_b - r.lo_b + kRepTile - 1) / kRepTile : 0;
  r.n_suf = 0;
  r.suf_first_page = r.prefix / p.page_size;
  if (p.with_suffix && r.seq_len > r.prefix)
    r.n_suf = (r.seq_len - 1) / p.page_size - r.suf_first_page + 1;
  const int64_t n = (int64_t)r.n_sel_items + r.n_rep + r.n_suf;
  r.begin = (int)(n * split / p.n_splits);
  r.end = (int)(n * (split + 1) / p.n_splits);
  return r;
}

// Physical page of logical page `lpage` of a sequence, or -1 (and DEV_STATUS_BAD_INDEX) when the
// logical page lies outside the table row or the entry outside the pool: the caller then makes the
// item empty, so a bad index or table entry is never dereferenced.
__device__ __forceinline__ int guarded_page(const DecodeParams& p, const int32_t* table, int lpage) {
  bool ok = lpage >= 0 && lpage < p.max_pages;
  int page = 0;
  if (ok) {
    page = table[lpage];
    ok = page >= 0 && (p.n_pool_pages <= 0 || page < p.n_pool_pages);
  }
  if (!ok) {
    if (p.status != nullptr) atomicOr(p.status, DEV_STATUS_BAD_INDEX);
    return -1;
  }
  return page;
}

// Item i of a (sequence, kv head) whose list starts with n_sel_items selected pages (from entry
// sel_first of its index list), then n_rep representative tiles from block lo_b, then the suffix.
struct ResolvedItem { int kind, first, lo, hi; };
__device__ __forceinline__ ResolvedItem resolve_one(const DecodeParams& p, const int32_t* idx, const int32_t* table,
                                                    int i, int sel_first, int n_sel_items, int n_rep, int lo_b,
                                                    int hi_b, int suf_first_page, int prefix, int seq_len) {
  const int ppb = p.block_size / p.page_size;
  ResolvedItem it;
  // The index entry is fetched before `i < n_sel_items` is known (the position is clamped into the
  // list): when the caller has not waited for the count yet, the two loads overlap instead of chaining.
  const int blk_spec = idx[min(max(sel_first + i / ppb, 0), p.max_sel - 1)];
  if (i < n_sel_items) {
    const int blk = blk_spec;
    it.kind = ITEM_PAGE;
    it.lo = 0;
    it.hi = 0;
    it.first = 0;
    const int at = sel_first + i / ppb;
    const bool disorder = i % ppb == 0 && at > 0 && idx[at - 1] >= blk;  // checked once per block
    if (blk < 0 || blk >= p.max_blocks || disorder) {
      if (p.status != nullptr) atomicOr(p.status, DEV_STATUS_BAD_INDEX);
    }
    if (blk >= 0 && blk < p.max_blocks) {
      const int lpage = blk * ppb + i % ppb;
      const int tok0 = lpage * p.page_size;
      it.hi = max(min(p.page_size, prefix - tok0), 0);
      if (it.hi > 0) {
        it.first = guarded_page(p, table, lpage);
        if (it.first < 0) { it.first = 0; it.hi = 0; }
      }
    }
  } else if (i < n_sel_items + n_rep) {
    const int b0 = lo_b + (i - n_sel_items) * kRepTile;
    it.kind = ITEM_REP_TILE;
    it.first = b0;
    it.lo = 0;
    it.hi = min(kRepTile, hi_b - b0);
  } else {
    const int lpage = suf_first_page + (i - n_sel_items - n_rep);
    const int tok0 = lpage * p.page_size;
    it.kind = ITEM_PAGE;
    it.lo = max(prefix - tok0, 0);
    it.hi = min(p.page_size, seq_len - tok0);
    it.first = guarded_page(p, table, lpage);
    if (it.first < 0) { it.first = 0; it.hi = it.lo; }
  }
  return it;
}

// Resolve items [chunk_begin, chunk_end) into items_s[0 ..).  All threads; ends with a barrier.
__device__ __forceinline__ void resolve_items(const DecodeParams& p, const ItemRange& r, int seq, int head,
                                              int chunk_begin, int chunk_end, Item* items_s) {
  const int pair = seq * p.n_kv_heads + head;
  const int32_t* idx = p.sel_idx + (int64_t)pair * p.max_sel;
  const int32_t* table = p.block_table + (int64_t)seq * p.max_pages;
  for (int i = chunk_begin + threadIdx.x; i < chunk_end; i += blockDim.x) {
    const ResolvedItem ri = resolve_one(p, idx, table, i, r.sel_first, r.n_sel_items, r.n_rep, r.lo_b, r.hi_b,
                                        r.suf_first_page, r.prefix, r.seq_len);
    items_s[i - chunk_begin] = Item{ri.kind, ri.first, ri.lo, ri.hi};
  }
  __syncthreads();
}

// ---- equal shares of the flattened item list -----------------------------------------
// The items of all (sequence, kv head) pairs, pair after pair, form one list of N items; CTA c of
// n_ctas owns the contiguous slice [N c / n_ctas, N (c + 1) / n_ctas), which may end inside a pair
// and start the next.  A (CTA, pair) intersection is a segment and yields one partial.  As c and
// pair only ever step by one from a segment to the next, c + pair numbers the segments without
// collisions: slot = c + pair.
struct PairItems {
  int prefix, seq_len, nb_eff, n_sel_items, n_rep, n_suf, suf_first_page;
  __device__ __forceinline__ int total() const { return n_sel_items + n_rep + n_suf; }
};
__device__ __forceinline__ PairItems pair_items(const DecodeParams& p, int pair) {
  PairItems r;
  const int seq = pair / p.n_kv_heads;
  const int capacity = p.max_pages * p.page_size;
  r.prefix = min(max(p.prefix_lens[seq], 0), capacity);
  r.seq_len = min(p.seq_lens[seq], capacity);
  r.nb_eff = min((r.prefix + p.block_size - 1) / p.block_size, p.max_blocks);
  const int count = max(min(p.sel_count[pair], p.max_sel), 0);
  r.n_sel_items = count * (p.block_size / p.page_size);
  r.n_rep = (p.rep_mode == IA_REP_HYBRID) ? (r.nb_eff + kRepTile - 1) / kRepTile : 0;
  r.suf_first_page = r.prefix / p.page_size;
  r.n_suf = (p.with_suffix && r.seq_len > r.prefix) ? (r.seq_len - 1) / p.page_size - r.suf_first_page + 1 : 0;
  return r;
}
// first item of CTA c's slice, and the CTA that owns item i (the inverse)
__device__ __host__ __forceinline__ int64_t flat_slice_begin(int64_t n_items, int c, int n_ctas) {
  return n_items * c / n_ctas;
}
__device__ __host__ __forceinline__ int flat_cta_of(int64_t n_items, int64_t i, int n_ctas) {
  return (int)(((i + 1) * n_ctas + n_items - 1) / n_items) - 1;
}
// kind and pair in one word, valid rows and kv head in another; `mask` (representative tiles): bit t
// set = block first + t is selected and contributes its tokens, not its representative
struct __align__(16) FlatItem { int kind_pair, first, lohi_head, mask; };

// ---- exchange of the partials with peer GPUs ---------------------------------------
// Gather buffer of a rank: [2 (step parity)][n_ranks][chunk_floats]; a chunk is o [rows, n_splits, D]
// followed by lse [rows, n_splits].  Flags of a rank: [2][n_ranks] step numbers.  Two parities are
// enough: a rank can run at most one step ahead of a peer, because its next merge needs that peer's
// next partials.
struct ExchangeView {
  int step, parity;
};
__device__ __forceinline__ ExchangeView exchange_view(const DecodeParams& p) {
  ExchangeView v;
  v.step = *p.px.step_counter + 1;  // changed only by the last CTA of this kernel, after every CTA has read it
  v.parity = v.step & 1;
  return v;
}
// one float of this rank's chunk (element offset inside the chunk), stored on every rank
__device__ __forceinline__ void exchange_store(const DecodeParams& p, const ExchangeView& v, int64_t offset,
                                               float value) {
  const int64_t at = ((int64_t)v.parity * p.px.n_ranks + p.px.my_rank) * p.px.chunk_floats + offset;
  for (int w = 0; w < p.px.n_ranks; ++w) p.px.gather[w][at] = value;
}
// Called by every thread of a CTA after its exchange_store calls.  `flag`: one int of shared memory.
__device__ __forceinline__ void exchange_publish(const DecodeParams& p, const ExchangeView& v) {
  __syncthreads();  // every thread's peer stores are issued
  if (threadIdx.x == 0) {
    __threadfence_system();  // cumulative: the CTA's stores are visible system-wide before the count
    const unsigned done = atomicAdd(reinterpret_cast<unsigned*>(p.px.grid_counter), 1u);
    if (done == gridDim.x - 1) {  // every CTA of this rank has stored and fenced
      *p.px.grid_counter = 0;
      __threadfence_system();
      for (int w = 0; w < p.px.n_ranks; ++w) {
        volatile int32_t* f = p.px.flags[w] + v.parity * p.px.n_ranks + p.px.my_rank;
        *f = v.step;
      }
      *p.px.step_counter = v.step;
    }
  }
}

// Fused split-KV finalize (same arithmetic as condition_block_stage2_reduce_kernel).
// Called by every thread of a CTA right after it wrote its partial.  `flag` is one
// int of shared memory.
template <int D>
__device__ __forceinline__ void finish_pair(const DecodeParams& p, int seq, int head, int G, int* flag) {
  if (p.final_out == nullptr) return;
  const int pair = seq * p.n_kv_heads + head;
  const int rows = p.n_kv_heads * G;
  if (p.n_splits > 1) {
    // The barrier orders every thread's partial stores before thread 0; its fence is
    // cumulative, so they are visible device-wide before the count is.
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const int old = atomicAdd(&p.split_counters[pair], 1);
      const int is_last = old == p.n_splits - 1;
      if (is_last) {
        p.split_counters[pair] = 0;  // ready for the next launch
        __threadfence();             // the other splits' partials, before this CTA reads them
      }
      *flag = is_last;
    }
    __syncthreads();
    if (*flag == 0) return;
  } else {
    __syncthreads();
  }
  // Four output elements per thread; the parts' (lse, o) loads are independent of one another and are
  // issued eight parts at a time, so the merge costs one or two L2 round trips, not one per part.
  // The arithmetic (maximum over all parts first, then weights and sums in part order) is that of the
  // stand-alone finalize kernel, value for value.
  constexpr int kBatch = 8;
  constexpr int VPR = D / 4;
  const int n = p.n_splits;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int e = threadIdx.x; e < G * VPR; e += blockDim.x) {
    const int g = e / VPR, d = (e - g * VPR) * 4;
    const int64_t row = (int64_t)seq * rows + head * G + g;
    const float* lse = p.lse_partial + row * n;
    const float* o = p.o_partial + row * n * D + d;
    float l[kBatch];
    float4 v[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      l[j] = j < n ? __ldcg(lse + j) : -INFINITY;
      v[j] = j < n ? __ldcg(reinterpret_cast<const float4*>(o + (int64_t)j * D)) : zero4;
    }
    float top = -INFINITY;
#pragma unroll
    for (int j = 0; j < kBatch; ++j) top = fmaxf(top, l[j]);
    for (int s0 = kBatch; s0 < n; s0 += kBatch) {  // more than eight parts: the rest of the maximum
      float more[kBatch];
#pragma unroll
      for (int j = 0; j < kBatch; ++j) more[j] = s0 + j < n ? __ldcg(lse + s0 + j) : -INFINITY;
#pragma unroll
      for (int j = 0; j < kBatch; ++j) top = fmaxf(top, more[j]);
    }
    const float ref = top == -INFINITY ? 0.f : top;
    float4 num = zero4;
    float den = 0.f;
    for (int s0 = 0;;) {
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        if (s0 + j < n) {
          const float w = expf(l[j] - ref);  // exp(-inf) = 0 for an empty part
          num.x = fmaf(w, v[j].x, num.x); num.y = fmaf(w, v[j].y, num.y);
          num.z = fmaf(w, v[j].z, num.z); num.w = fmaf(w, v[j].w, num.w);
          den += w;
        }
      }
      s0 += kBatch;
      if (s0 >= n) break;
#pragma unroll
      for (int j = 0; j < kBatch; ++j) {
        l[j] = s0 + j < n ? __ldcg(lse + s0 + j) : -INFINITY;
        v[j] = s0 + j < n ? __ldcg(reinterpret_cast<const float4*>(o + (int64_t)(s0 + j) * D)) : zero4;
      }
    }
    const float inv = 1.f / fmaxf(den, 1e-30f);  // same rounding as the stand-alone finalize kernel
    const int64_t at = row * D + d;
    if (p.final_dtype == IA_BF16) {
      __nv_bfloat162 a = __floats2bfloat162_rn(num.x * inv, num.y * inv);
      __nv_bfloat162 b = __floats2bfloat162_rn(num.z * inv, num.w * inv);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&a);
      packed.y = *reinterpret_cast<uint32_t*>(&b);
      *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p.final_out) + at) = packed;
    } else {
      *reinterpret_cast<float4*>(static_cast<float*>(p.final_out) + at) =
          make_float4(num.x * inv, num.y * inv, num.z * inv, num.w * inv);
    }
  }
}

}  // namespace ia
