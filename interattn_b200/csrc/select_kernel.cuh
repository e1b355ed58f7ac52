// Condition-block selection: block scores + top-k (or epsilon) routing, fused.
//
// Reference arithmetic (paths relative to the reference project,
// IMPL = llama/script/analysis/condition_block_gen/methods/condition_block_triton_impl):
//   score definition ........ _select_prompt_blocks_eager, IMPL/core.py:509-546
//   GPU pass of the same .... _condition_block_selection_stats_kernel, IMPL/core.py:751-814
//                             and the routing half of the fused finalize kernel,
//                             IMPL/page_attention.py:84-171
// The reference spreads this over two launches and parks s / delta / four
// online-softmax partials in HBM in between.  Here one CTA owns one
// (sequence, kv head): it streams the three summary vectors of every block
// once through a TMA (cp.async.bulk.tensor) + mbarrier shared-memory ring,
// keeps z = s + log(count) and the range bound delta of all
// G x n_blocks (row, block) pairs in shared memory, forms the global
// normalisers on the fly, the GQA-mean score and then routes - a radix select
// for the k best blocks (higher score first, lower block index first among
// equal scores) or the reference's score > eps rule - without the score
// vector leaving the SM.
//
// Roofline: HBM.  Algorithmic bytes per block and kv head:
//   D*4 (k_bar f32; D*2 with the bf16 k_bar option) + 2*D*sizeof(T) (k_max, k_min) + 4 (v_norm_max).
//
// A ring stage is 32 blocks: every summary vector arrives as TMA boxes of
// 128 bytes x 32 rows written with the 128-byte swizzle, so both access
// patterns below are bank-conflict free without padding.
//   * bf16 pools, G <= 8: tensor cores.  Blocks are the M side, query rows the
//     N side, head_dim is K; two warps take 16 blocks each of a stage.
//   * otherwise: CUDA cores.  Lane <-> block; a stage is consumed by a group of
//     four warps, each taking a quarter of head_dim; their partial sums meet in
//     shared memory and warp w of the group finishes rows g = w, w + 4, ...
#pragma once
#include <string.h>

#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through the runtime)

#include "ia_common.cuh"

namespace ia {

// The kernels are instantiated in several translation units (one per dtype / head_dim / bound, see
// select_inst_*.cu) so that they compile side by side; these two structs cross between them.
struct SelectParams {
  // TMA descriptors of the three summary arrays viewed as [rows, D] matrices
  // (rows = batch * kv heads * max_blocks); box = 128 bytes x 32 rows, 128-byte swizzle
  CUtensorMap tm_kbar, tm_kmax, tm_kmin;
  const void* q;
  const void* k_bar;  // f32, or bf16 with IA_GEOM_KBAR_BF16
  const void* k_max;
  const void* k_min;
  const float* v_norm_max;
  const float* rho;  // diag_ell bound only: [pairs, max_blocks]; tm_kmax then describes w
  const int32_t* prefix_lens;
  int n_kv_heads, max_blocks, block_size;
  int mode, top_k, max_sel;
  int mass_exp;  // score variant: first term 2 b_all softmax(z + delta) (IA_SELECT_TERM1_MASS_EXP)
  float eps;
  int32_t* sel_idx;
  int32_t* sel_count;
  int* split_counters;  // may be null
  ia_select_aux aux;
  int n_stages, nb_cap;
  int longest_first;  // CTAs take the sequences in order of descending prefix length (grids of several waves)
  int cluster;     // CTAs per (sequence, kv head): a thread-block cluster splits the blocks
  int nb_loc_cap;  // row stride of the per-CTA (row, block) arrays
  // Split-KV across GPUs: this rank scores the blocks [block_lo, block_hi) only and exchanges the row
  // normalisers and its top-k candidates with the other ranks (xch.n_ranks == 0: one GPU, all blocks).
  ia_select_exchange xch;
  int block_lo, block_hi;
  int n_pairs;
  int* status;  // the device status word (bounded waits that ran out, indices out of range)
  unsigned long long* stamps;  // may be null: the first CTA of the one-kernel step leaves three time stamps
  // One-kernel layer step (att.on): the CTA that routed a (sequence, kv head) attends over what it picked.
  struct Attend {
    // the K and V pools as 4-D tensors [page, kv head, token, head_dim]; box = 128 bytes x one page of tokens
    CUtensorMap tm_k, tm_v;
    CUtensorMap tm_vbar;  // hybrid: the mean values [pairs * max_blocks, head_dim], box = 128 bytes x 16 blocks
    int hybrid;           // IA_REP_HYBRID: every block that was not picked attends through (z, v_bar)
    int heads_outer;      // the pools' tensor maps are [kv head, page, token, head_dim] (head stride > page stride)
    const int32_t* block_table;
    const int32_t* seq_lens;
    void* out;
    int max_pages, n_pool_pages;
    int ring_bytes;  // shared memory of the ring (the selection's stages), reused for the pages
    int on;
  } att;
};

// What launch_select was asked to fuse; resolved into SelectParams::att once the launch shape is known.
struct AttendRequest {
  SelectAttend* req;
  const ia_geom* geom;
  const void* vbar;
};

// One entry per translation unit of instantiations: launch for this dtype / head_dim / k_bar type / bound.
int launch_select_bf16_d128_range(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_bf16_d128_diag(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_bf16_d64(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_f32_d128(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_f32_d64(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_kbar16_d128(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_kbar16_d64(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
// the same with the coordinate range in the packed layout (IA_GEOM_PACKED_BOUNDS)
int launch_select_bf16_d128_packed(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_bf16_d64_packed(const SelectParams&, const AttendRequest&, int n_pairs, int group, cudaStream_t);
int launch_select_f32_packed(const SelectParams&, const AttendRequest&, int n_pairs, int group, int head_dim, cudaStream_t);
int launch_select_kbar16_packed(const SelectParams&, const AttendRequest&, int n_pairs, int group, int head_dim, cudaStream_t);

namespace {

// Profiling build (-DIA_SELECT_TRACE): thread 0 of every CTA leaves time stamps (microseconds since the
// CTA started, from the nanosecond global timer) in the first floats of its pair's aux.score row instead
// of the scores - a timeline of the kernel's phases without a profiler.  Expands to nothing otherwise.
#ifdef IA_SELECT_TRACE
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define IA_TRACE_BEGIN()                                                                              \
  const unsigned long long trace_t0 = trace_now();                                                     \
  if (threadIdx.x == 0 && p.aux.delta != nullptr) /* start time modulo 2^24 ns: exact in a float */      \
    p.aux.delta[(int64_t)blockIdx.x * 16 + 15] = (float)(trace_t0 & 0xffffffull)
#define IA_TRACE(i)                                                                                   \
  do {                                                                                                \
    if (threadIdx.x == 0 && p.aux.delta != nullptr)                                                    \
      p.aux.delta[(int64_t)blockIdx.x * 16 + (i)] = (float)(trace_now() - trace_t0) * 1e-3f;           \
  } while (0)
#define IA_TRACE_T0 trace_t0
#else
#define IA_TRACE_BEGIN() do { } while (0)
#define IA_TRACE(i) do { } while (0)
#define IA_TRACE_T0 0ull
#endif

// CTA shape: NG warp groups of four warps (one ring stage each at a time) plus one
// TMA producer warp.  The wide shape (3 groups, 416 threads, one CTA per SM) gives a
// single (sequence, kv head) pair the whole SM; the narrow shape (1 group, 160
// threads, two or three CTAs per SM) is for batches with more pairs than SMs, where
// the serial phases of one pair overlap the streaming of its neighbours.
constexpr int kGroupWarps = 4;     // warps per group: each takes head_dim / 4
template <int NG> struct Shape {
  static constexpr int groups = NG;
  static constexpr int consumer_warps = NG * kGroupWarps;
  static constexpr int warps = consumer_warps + 1;
  static constexpr int threads = warps * 32;
  static constexpr int min_ctas = NG >= 3 ? 1 : 3;
};
constexpr int kWideGroups = 3, kNarrowGroups = 1;
constexpr int kTileBlocks = 32;
constexpr int kMaxStages = 8;
constexpr uint32_t kWaitPolls = 1u << 20;  // bounded mbarrier wait, then give up


__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false when the phase did not complete in time; the
// caller records that in the device status word and carries on (the results
// are then garbage, but the GPU is not left spinning).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  // try_wait parks the thread for a hardware-defined time before it reports "not yet"
  for (uint32_t i = 0; i < kWaitPolls; ++i)
    if (mbar_test(bar, parity)) return true;
  return false;
}
// one 2-D tile (box) global -> shared, completing on an mbarrier; x = element column, y = row
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D(16x8, f32) += A(16x8, tf32, row-major) * B(8x8, tf32, col-major)
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// D(16x8, f32) += A(16x16, bf16, row-major) * B(16x8, bf16, col-major)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// one box of a 4-D tensor (c0 = element column .. c3 = outermost coordinate) global -> shared
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::
          "r"(smem_u32(dst)),
      "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// transpose of an 8 x 8 matrix of 16-bit elements held one row pair per thread (fragment layout)
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

// Running softmax normalisers of one query row: m = max z, l = sum e^{z - m},
// d = sum e^{z - m} cosh(delta).  Blocks are absorbed as they are scored and the
// per-lane / per-warp states are merged afterwards, so no extra pass over the
// blocks is needed for the normalisers.
struct RowNorm { float m, l, d; };
__device__ __forceinline__ void norm_absorb(RowNorm& a, float z, float ch) {
  const float m = fmaxf(a.m, z);
  const float sa = expf(a.m - m);  // a.m = -inf on first use: 0
  const float w = expf(z - m);
  a.l = fmaf(a.l, sa, w);
  a.d = fmaf(a.d, sa, w * ch);
  a.m = m;
}
// Merge of the states held by the lanes whose indices differ in the bits of `xor_mask` (a set of
// power-of-two strides below 32): one max-reduction, one rescale of every lane's sums to the
// common maximum, one sum-reduction - two exponentials on the dependent path instead of two per level.
template <int kFirst, int kEnd> __device__ __forceinline__ void norm_reduce_lanes(RowNorm& a) {
  float top = a.m;
#pragma unroll
  for (int o = kFirst; o < kEnd; o <<= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
  const float f = (a.m == -INFINITY) ? 0.f : expf(a.m - top);  // top is finite whenever a.m is
  float l = a.l * f, d = a.d * f;
#pragma unroll
  for (int o = kFirst; o < kEnd; o <<= 1) {
    l += __shfl_xor_sync(0xffffffffu, l, o);
    d += __shfl_xor_sync(0xffffffffu, d, o);
  }
  a.m = top; a.l = l; a.d = d;
}
__device__ __forceinline__ void norm_merge(RowNorm& a, float bm, float bl, float bd) {
  const float m = fmaxf(a.m, bm);
  if (m == -INFINITY) return;  // both empty
  const float sa = expf(a.m - m), sb = expf(bm - m);
  a.l = a.l * sa + bl * sb;
  a.d = a.d * sa + bd * sb;
  a.m = m;
}
// What the score needs from delta, and the block's contribution to the normalisers:
//   A = cosh(delta) - 1,  th = tanh(delta / 2)
// With mass_exp the first term is 2 b_all softmax(z + delta) (IMPL/core.py:798-803, 893-896):
// e^delta takes the place of cosh(delta) in the normaliser and of cosh(delta) - 1 in the term.
__device__ __forceinline__ void delta_terms(float delta, int mass_exp, float& ch, float& a_term, float& th) {
  const float e = expf(delta);
  ch = mass_exp ? e : 0.5f * (e + 1.f / e);
  a_term = mass_exp ? e : ch - 1.f;
  th = 1.f - 2.f / (e + 1.f);
}

// The tensor-core form of phase 1 needs exact operands: bf16 summaries / query
// (exact in tf32 and bf16) and at most eight query rows per kv head.
template <typename T, int G> constexpr bool kUseMma = (sizeof(T) == 2) && (G <= 8);

// ---- thread-block cluster: distributed shared memory and the cluster barrier --------
__device__ __forceinline__ uint32_t map_to_rank(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void st_cluster_s32(uint32_t addr, int v) {
  asm volatile("st.shared::cluster.s32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// every thread of every CTA of the cluster; orders the remote stores before it against the loads after it
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// ---- exchange with peer GPUs (plain peer stores and flags; no multicast) -----------------
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *flag reaches `want` (about a second); false when it did not.
__device__ __forceinline__ bool wait_flag(const int* flag, int want) {
  for (uint32_t i = 0; i < (1u << 22); ++i) {
    if (ld_acquire_sys(flag) - want >= 0) return true;
    __nanosleep(200);
  }
  return false;
}

// barrier among the 128 threads of one warp group (ids 1..kGroups; 0 is __syncthreads)
__device__ __forceinline__ void group_sync(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(kGroupWarps * 32) : "memory");
}

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// eight consecutive elements from 16-byte aligned shared memory, as floats
__device__ __forceinline__ void load8(const float* p, float (&o)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load4(const float* p, float* o) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  o[0] = bf16lo(a.x); o[1] = bf16hi(a.x); o[2] = bf16lo(a.y); o[3] = bf16hi(a.y);
  o[4] = bf16lo(a.z); o[5] = bf16hi(a.z); o[6] = bf16lo(a.w); o[7] = bf16hi(a.w);
}

// One ring stage = 32 blocks.  Every summary vector arrives as boxes of
// 128 bytes x 32 rows (4 KB, 1024-byte aligned) written by TMA with the
// 128-byte swizzle: the 16-byte chunk c of row r lands at chunk c ^ (r & 7).
// Lane r walking its own row therefore hits eight different bank groups per
// quarter-warp - no padding, no conflicts.
// DIAG: the stage holds k_bar and w (the diagonal-ellipsoid bound) instead of k_bar, k_max and k_min.
template <typename T, int D, typename KB = float, bool DIAG = false> struct TileLayout {
  static constexpr int box_bytes = 128 * kTileBlocks;
  static constexpr int kbar_boxes = D * (int)sizeof(KB) / 128;
  static constexpr int bnd_boxes = D * (int)sizeof(T) / 128;
  static constexpr int kbar_bytes = kbar_boxes * box_bytes;
  static constexpr int bnd_bytes = bnd_boxes * box_bytes;
  static constexpr int bytes = kbar_bytes + (DIAG ? 1 : 2) * bnd_bytes;
  static constexpr int kbar_box_cols = 128 / (int)sizeof(KB);  // k_bar elements per 128 bytes
  static constexpr int bnd_box_cols = 128 / (int)sizeof(T);
};

// 16 bytes at element offset `elem` (a multiple of 16 / sizeof(E)) of row `row` of a swizzled vector
template <typename E>
__device__ __forceinline__ const E* swz(const unsigned char* vec_base, int row, int elem) {
  const int byte = elem * (int)sizeof(E);
  const int box = byte >> 7, chunk = (byte >> 4) & 7;
  return reinterpret_cast<const E*>(vec_base + box * (128 * kTileBlocks) + row * 128 + ((chunk ^ (row & 7)) << 4));
}

// Fixed shared-memory carve-up (bytes), shared by the kernel and the launcher.
template <int D, int G, bool MMA, int NG> struct SmemPlan {
  static constexpr int kWarps = Shape<NG>::warps, kConsumerWarps = Shape<NG>::consumer_warps;
  static constexpr size_t bars = 4 * kMaxStages * 8;  // full / empty of the ring, and of the second pass's ring
  static constexpr size_t hist = 3 * 256 * 4;
  static constexpr size_t scan = 32 * 4;
  static constexpr size_t red = (size_t)kWarps * 16 * 3 * 4 + (size_t)kWarps * 4 + 12;  // [warp][row][m,l,d] + b_max per warp
  static constexpr size_t norm = 4 * 16 * 4;
  static constexpr size_t state = 8 * 4;
  static constexpr size_t qrows = 2 * (size_t)G * D * 4;
  static constexpr size_t part = MMA ? 0 : (size_t)kConsumerWarps * 3 * G * 32 * 4;
  static constexpr size_t xch = 8 * 16 * 3 * 4;  // [cluster rank][row][m, l, d]
  static constexpr size_t xst = 16 * 4 * 4;      // [row][m, l, d, b_all] of this GPU, on its way to the peers
  static constexpr size_t fixed = bars + hist + scan + red + norm + state + qrows + part + xch + xst;
  static size_t per_blocks(int nb_cap, int nb_loc_cap, int n_candidates = 0) {
    return (size_t)nb_cap * 4 * 3 + (size_t)nb_loc_cap * 4 * 2 * G + (size_t)n_candidates * 8;
  }
};

// ---- the attention phase of the one-kernel layer step ---------------------------------------
// Warp-level attention of up to eight query rows over 16-token pages with the operands swapped: the
// page's tokens are the M side of both products, the query rows the N side (padded to 8) -
//   S^T[token, row] = K[token, :] . Q[row, :]          (A = K tile as stored, B = Q)
//   O^T[d, row]    += V^T[d, token] P^T[token, row]    (A = V tile through ldmatrix.trans, B = P^T)
// so that a thread holds 32 output accumulators (head_dim 128) instead of the 64 of the row-major
// form, and the whole phase fits the register budget of the selection kernel it is appended to.  A
// thread's two S columns are its two query rows: the running maximum and sum of a row live in the
// four threads of a quad column and are combined across the eight token rows with three shuffles.
// P^T reaches the B-fragment layout through one 8 x 8 transpose (movmatrix) per eight tokens.
template <int D, int G> struct PageAttention {
  static constexpr int KSTEPS = D / 16, MT = D / 16;
  static constexpr int kBox = 16 * 128;            // one TMA box: 16 token rows x 128 bytes, 128-byte swizzle
  static constexpr int kTile = 16 * D * 2;         // the K (or V) rows of one page and kv head
  uint32_t qb[KSTEPS][2];
  float o[MT][4];
  float m0, m1, l0, l1;  // query rows 2 qlane and 2 qlane + 1, log2 domain; l: this thread's share
  int lane, quad, qlane;
  float sc_qk;

  __device__ __forceinline__ void init(int lane_, const float* q_s) {
    lane = lane_; quad = lane_ >> 2; qlane = lane_ & 3;
    sc_qk = kLog2e / sqrtf((float)D);
#pragma unroll
    for (int j = 0; j < MT; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
    m0 = -INFINITY; m1 = -INFINITY; l0 = 0.f; l1 = 0.f;
    // B fragments of Q^T: (k = head_dim 2 qlane, +1 (+8), n = query row quad); rows past G are zero
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d0 = kk * 16 + qlane * 2;
      qb[kk][0] = quad < G ? pack_bf16(q_s[quad * D + d0], q_s[quad * D + d0 + 1]) : 0u;
      qb[kk][1] = quad < G ? pack_bf16(q_s[quad * D + d0 + 8], q_s[quad * D + d0 + 9]) : 0u;
    }
  }

  // One page (K tile at `stage`, V tile behind it; token rows [lo, hi) are live) into the running state.
  __device__ __forceinline__ void consume(uint32_t stage, int lo, int hi) {
    const uint32_t ktile = stage;
    const int mat = lane >> 3, rr = lane & 7;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const int row = (mat & 1) * 8 + rr;  // token row of this lane's ldmatrix address
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int ch = kk * 2 + (mat >> 1);
        uint32_t a[4];
        ldmatrix_x4(ktile + (ch >> 3) * kBox + row * 128 + (((ch & 7) ^ (row & 7)) << 4), a);
        mma_bf16(s, a, qb[kk]);
      }
    }
    // s[0], s[1]: token quad, rows 2 qlane, 2 qlane + 1;  s[2], s[3]: token quad + 8
    const bool oka = quad >= lo && quad < hi, okb = quad + 8 >= lo && quad + 8 < hi;
    s[0] = oka ? s[0] * sc_qk : -INFINITY;
    s[1] = oka ? s[1] * sc_qk : -INFINITY;
    s[2] = okb ? s[2] * sc_qk : -INFINITY;
    s[3] = okb ? s[3] * sc_qk : -INFINITY;
    accumulate(s, stage + kTile);
  }

  // A tile of 16 representatives: the mean values of blocks [first, first + n) are in the V half of the
  // stage, their logits z = s + log count (natural log, from the selection pass) in shared memory as
  // z[row * z_stride + block]; bit t of `skip` drops block first + t (it was picked and is attended
  // token by token).
  __device__ __forceinline__ void consume_reps(uint32_t stage, const float* z, int z_stride, int n, uint32_t skip) {
    const int r0 = 2 * qlane, r1 = r0 + 1;
    const bool oka = quad < n && ((skip >> quad) & 1u) == 0u;
    const bool okb = quad + 8 < n && ((skip >> (quad + 8)) & 1u) == 0u;
    float s[4];
    s[0] = oka && r0 < G ? z[r0 * z_stride + quad] * kLog2e : -INFINITY;
    s[1] = oka && r1 < G ? z[r1 * z_stride + quad] * kLog2e : -INFINITY;
    s[2] = okb && r0 < G ? z[r0 * z_stride + quad + 8] * kLog2e : -INFINITY;
    s[3] = okb && r1 < G ? z[r1 * z_stride + quad + 8] * kLog2e : -INFINITY;
    accumulate(s, stage + kTile);
  }

  // online softmax over the 16 columns of S^T held as s[] (log2 domain, -inf = masked), then O^T += V^T P^T
  __device__ __forceinline__ void accumulate(float (&s)[4], uint32_t vtile) {
    const int mat = lane >> 3, rr = lane & 7;
    float t0 = fmaxf(s[0], s[2]), t1 = fmaxf(s[1], s[3]);
#pragma unroll
    for (int x = 4; x < 32; x <<= 1) {
      t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, x));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, x));
    }
    const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);
    const float ref0 = n0 == -INFINITY ? 0.f : n0, ref1 = n1 == -INFINITY ? 0.f : n1;
    const float a0 = exp2f(m0 - ref0), a1 = exp2f(m1 - ref1);
    m0 = n0; m1 = n1;
    const float p0 = exp2f(s[0] - ref0), p1 = exp2f(s[1] - ref1);
    const float p2 = exp2f(s[2] - ref0), p3 = exp2f(s[3] - ref1);
    l0 = l0 * a0 + (p0 + p2);
    l1 = l1 * a1 + (p1 + p3);
    uint32_t pb[2];
    pb[0] = movmatrix_trans(pack_bf16(p0, p1));  // (tokens 2 qlane, +1; row quad)
    pb[1] = movmatrix_trans(pack_bf16(p2, p3));  // tokens + 8
#pragma unroll
    for (int j = 0; j < MT; ++j) { o[j][0] *= a0; o[j][1] *= a1; o[j][2] *= a0; o[j][3] *= a1; }
    const int row = (mat >> 1) * 8 + rr;  // token row
#pragma unroll
    for (int j = 0; j < MT; ++j) {
      const int ch = j * 2 + (mat & 1);
      uint32_t a[4];
      ldmatrix_x4_trans(vtile + (ch >> 3) * kBox + row * 128 + (((ch & 7) ^ (row & 7)) << 4), a);
      mma_bf16(o[j], a, pb);
    }
  }
};

// Warps that attend: the consumer warps of the selection; in the narrow shape the idle producer warp
// joins them (five warps, ten page stages in the shared memory a narrow CTA has, instead of four and eight).
template <int NG> constexpr int kAttendWarps = NG == 1 ? Shape<NG>::warps : Shape<NG>::consumer_warps;

// Every thread of the CTA that routed `pair` calls this after the routing: sel_list[0..count) are the
// picked blocks, ascending.  All threads resolve the pages through the block table into page_list;
// the CW consumer warps then take the pages round robin, each through a ring of its own carved from
// the selection's stages (the stage count is a multiple of CW) that it fills itself with four TMA
// boxes per page, and are merged through the idle ring at the end.  All waits are bounded.
template <int D, int G, int CW>
__device__ __forceinline__ void attend_selected_pages(const SelectParams& p, int pair, int seq, int prefix_raw,
                                                      int crank, int C, const int* sel_list, int count,
                                                      const float* q_s, const float* z_s, int z_stride, int b_lo,
                                                      int b_hi, uint32_t* sel_bits, int nb_cap,
                                                      int* page_list, int page_cap, unsigned char* ring,
                                                      unsigned char* bar_area, unsigned long long trace_t0) {
  (void)trace_t0;  // read by the stamps of the profiling build only
  using PA = PageAttention<D, G>;
  constexpr int kPage = 16;
  constexpr int kTile = PA::kTile, kStage = 2 * kTile, kBoxes = D * 2 / 128, kBox = PA::kBox;
  constexpr int kMaxRing = 32;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint64_t* full_b = reinterpret_cast<uint64_t*>(bar_area);
  // A cluster keeps the end of rank 0's ring free of pages: the ranks' partial results are stored there.
  constexpr int kShare = G * D + 2 * G;  // floats: [G][D] sums relative to top[g], then top[G], den[G]
  const int share_bytes = C > 1 ? C * kShare * 4 : 0;
  int nsb = min((p.att.ring_bytes - share_bytes) / kStage, kMaxRing);
  nsb -= nsb % CW;  // the launcher made sure that at least CW stages fit
  const int ppb = p.block_size / kPage;
  const int cap = p.att.max_pages * kPage;
  const int prefix = min(prefix_raw, cap);
  const int seq_len = min(max(p.att.seq_lens[seq], prefix), cap);
  const int n_sel_items = count * ppb;
  const int suf_first = prefix / kPage;
  const int n_suf = seq_len > prefix ? (seq_len - 1) / kPage - suf_first + 1 : 0;
  // a cluster of C CTAs shares the pair: rank r takes the pages r, r + C, ... (item i of this CTA is page
  // i * C + crank of the pair) and the ranks' partial results are merged by rank 0 at the end
  const int n_pair_items = n_sel_items + n_suf;
  // Hybrid: the blocks this CTA scored, [b_lo, b_hi), also attend through their representatives, 16 blocks
  // (one tile of mean values) per item; their logits are still in this CTA's shared memory.  These items
  // come first: they need no table look-up.
  const int n_rep = p.att.hybrid ? (max(b_hi - b_lo, 0) + 15) / 16 : 0;
  const int n_items = n_rep + (n_pair_items - crank + C - 1) / C;
  const int head = pair - seq * p.n_kv_heads;

  if (tid == 0) {
    for (int s = 0; s < nsb; ++s) mbar_init(&full_b[s], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (n_rep > 0)
    for (int i = tid; i < (nb_cap + 31) / 32; i += blockDim.x) sel_bits[i] = 0u;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the ring was read through ldmatrix; TMA writes it next
  __syncthreads();
  IA_TRACE(11);  // profiling build: stamps 11 - 14 are the attention phase (11, 12 replace the late radix passes)
  if (n_rep > 0)  // which blocks were picked: their representatives are dropped (visible past the barrier below)
    for (int i = tid; i < count; i += blockDim.x) {
      const int b = sel_list[i];
      if (b >= 0 && b < nb_cap) atomicOr(&sel_bits[b >> 5], 1u << (b & 31));
    }

  // item i >= n_rep: page i % ppb of picked block i / ppb, then the pages that hold the suffix [prefix, seq_len)
  auto describe = [&](int item, int& lpage, int& lo, int& hi) {
    if (item < n_rep) {  // representatives of blocks [b_lo + 16 item, + hi)
      lpage = -1;
      lo = 0;
      hi = min(b_hi - (b_lo + item * 16), 16);
      return;
    }
    const int i = (item - n_rep) * C + crank;
    if (i < n_sel_items) {
      lpage = sel_list[i / ppb] * ppb + i % ppb;
      lo = 0;
      hi = max(min(prefix - lpage * kPage, kPage), 0);
    } else {
      lpage = suf_first + (i - n_sel_items);
      lo = max(prefix - lpage * kPage, 0);
      hi = max(min(seq_len - lpage * kPage, kPage), lo);
    }
  };
  const int32_t* table = p.att.block_table + (int64_t)seq * p.att.max_pages;
  PA w;
  if (warp < CW) w.init(lane, q_s);
  // Items go through in chunks of page_cap (one chunk unless the epsilon rule kept nearly every block).
  // Item i always uses stage i % nsb, so the ring carries over from chunk to chunk.
  for (int c0 = 0; c0 < n_items; c0 += page_cap) {
    const int c1 = min(c0 + page_cap, n_items);
    // every thread: the chunk's physical pages, one round trip to the block table for all of them;
    // -1 = nothing to fetch (no live row, or an entry outside the table or the pool - reported, never read)
    for (int i = c0 + tid; i < c1; i += blockDim.x) {
      int lpage, lo, hi, page = -1;
      describe(i, lpage, lo, hi);
      if (i < n_rep) {
        page = 0;  // nothing to look up
      } else if (hi > lo) {
        if (lpage >= 0 && lpage < p.att.max_pages) page = table[lpage];
        if (page < 0 || page >= p.att.n_pool_pages) {
          atomicOr(p.status, DEV_STATUS_BAD_INDEX);
          page = -1;
        }
      }
      page_list[i - c0] = page;
    }
    __syncthreads();
    if (warp < CW) {
      // Warp w takes the items w, w + CW, ... of the chunk; they cycle through its own nsb / CW stages.
      // It fills those stages itself: lane 0 issues the page of item i + nsb into the stage that item
      // i has just been consumed from - no producer warp, no "empty" barriers, and the issue cost of
      // the TMA instructions (four per page) is spread over all consumer warps.
      auto issue = [&](int i) {  // one lane
        int lpage, lo, hi;
        describe(i, lpage, lo, hi);
        const int page = page_list[i - c0];
        const int stage = i % nsb;
        unsigned char* st = ring + (size_t)stage * kStage;
        if (i < n_rep) {  // 16 rows of mean values into the V half; rows past the pair's last block are masked
          const int y = pair * p.max_blocks + b_lo + i * 16;
          mbar_arrive_expect_tx(&full_b[stage], (uint32_t)kTile);
#pragma unroll
          for (int j = 0; j < kBoxes; ++j) tma_load_2d(st + kTile + j * kBox, &p.att.tm_vbar, j * 64, y, &full_b[stage]);
        } else if (page >= 0 && hi > lo) {
          const int c_inner = p.att.heads_outer ? page : head, c_outer = p.att.heads_outer ? head : page;
          mbar_arrive_expect_tx(&full_b[stage], (uint32_t)kStage);
#pragma unroll
          for (int j = 0; j < kBoxes; ++j) {
            tma_load_4d(st + j * kBox, &p.att.tm_k, j * 64, 0, c_inner, c_outer, &full_b[stage]);
            tma_load_4d(st + kTile + j * kBox, &p.att.tm_v, j * 64, 0, c_inner, c_outer, &full_b[stage]);
          }
        } else {
          mbar_arrive(&full_b[stage]);  // nothing to fetch: the phase completes at once
        }
      };
      const int first = c0 + (warp - c0 % CW + CW) % CW;
      if (lane == 0)
        for (int i = first, k = 0; k < nsb / CW && i < c1; ++k, i += CW) issue(i);
      bool alive = true;
      for (int i = first; i < c1; i += CW) {
        const int stage = i % nsb, use = i / nsb;
        if (alive && !mbar_wait(&full_b[stage], (uint32_t)(use & 1))) {
          alive = false;
          if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
        }
        int lpage, lo, hi;
        describe(i, lpage, lo, hi);
        if (page_list[i - c0] >= 0 && hi > lo) {
          const uint32_t st = smem_u32(ring + (size_t)stage * kStage);
          if (lo > 0 || hi < kPage) {
            // A partly live tile: the dead rows of V hold whatever the pool (or the next pair's
            // summaries) holds there, and 0 x NaN would poison the product - zero them first.
            for (int x = lane; x < kPage * (D * 2 / 16); x += 32) {
              const int row = x / (D * 2 / 16), ch = x % (D * 2 / 16);
              if (row < lo || row >= hi)
                *reinterpret_cast<uint4*>(ring + (size_t)stage * kStage + kTile + (ch >> 3) * kBox + row * 128 +
                                          ((ch & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // before TMA refills the stage
            __syncwarp();
          }
          if (i < n_rep) {
            const int first = b_lo + i * 16;
            const uint32_t skip = (sel_bits[first >> 5] >> (first & 31)) & 0xffffu;
            w.consume_reps(st, z_s + (first - b_lo), z_stride, hi, skip);
          } else {
            w.consume(st, lo, hi);
          }
        }
        if (i == warp) IA_TRACE(13);
        __syncwarp();  // every lane has read the stage: it may be refilled
        if (lane == 0 && i + nsb < c1) issue(i + nsb);
      }
    }
    if (c1 < n_items) __syncthreads();  // the page list is rewritten for the next chunk
  }
  __syncthreads();  // every page is consumed, nothing is in flight: the ring is scratch now
  IA_TRACE(12);

  // ---- merge the consumer warps: [warp][G rows][D + 4] partial outputs, then m[8], l[8] ----------
  constexpr int kRow = D + 4;
  constexpr int kPerWarp = 8 * kRow + 16;
  float* mbuf = reinterpret_cast<float*>(ring);
  if (warp < CW) {
    w.l0 += __shfl_xor_sync(0xffffffffu, w.l0, 4);
    w.l0 += __shfl_xor_sync(0xffffffffu, w.l0, 8);
    w.l0 += __shfl_xor_sync(0xffffffffu, w.l0, 16);
    w.l1 += __shfl_xor_sync(0xffffffffu, w.l1, 4);
    w.l1 += __shfl_xor_sync(0xffffffffu, w.l1, 8);
    w.l1 += __shfl_xor_sync(0xffffffffu, w.l1, 16);
    float* mo = mbuf + (size_t)warp * kPerWarp;
    const int r0 = 2 * w.qlane, r1 = r0 + 1;
#pragma unroll
    for (int j = 0; j < PA::MT; ++j) {
      const int d = j * 16 + w.quad;
      if (r0 < G) { mo[r0 * kRow + d] = w.o[j][0]; mo[r0 * kRow + d + 8] = w.o[j][2]; }
      if (r1 < G) { mo[r1 * kRow + d] = w.o[j][1]; mo[r1 * kRow + d + 8] = w.o[j][3]; }
    }
    if (w.quad == 0) {
      mo[8 * kRow + r0] = w.m0; mo[8 * kRow + 8 + r0] = w.l0;
      mo[8 * kRow + r1] = w.m1; mo[8 * kRow + 8 + r1] = w.l1;
    }
  }
  __syncthreads();
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.att.out) + (int64_t)pair * G * D;
  // C > 1: this CTA's share of the pair goes into slot `crank` of the shares at the end of rank 0's ring
  float* shares = reinterpret_cast<float*>(ring + p.att.ring_bytes - share_bytes);
  const uint32_t my_share = C > 1 ? map_to_rank(shares + crank * kShare, 0u) : 0u;
  for (int e = tid; e < G * D; e += blockDim.x) {
    const int g = e / D, d = e - g * D;
    float top = -INFINITY;
#pragma unroll
    for (int ww = 0; ww < CW; ++ww) top = fmaxf(top, mbuf[(size_t)ww * kPerWarp + 8 * kRow + g]);
    float num = 0.f, den = 0.f;
    if (top > -INFINITY) {
#pragma unroll
      for (int ww = 0; ww < CW; ++ww) {
        const float* mo = mbuf + (size_t)ww * kPerWarp;
        const float a = exp2f(mo[8 * kRow + g] - top);
        num = fmaf(a, mo[g * kRow + d], num);
        den = fmaf(a, mo[8 * kRow + 8 + g], den);
      }
    }
    if (C == 1) {
      out[e] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
    } else {
      st_cluster_f32(my_share + (uint32_t)e * 4u, num);
      if (d == 0) {
        st_cluster_f32(my_share + (uint32_t)(G * D + g) * 4u, top);
        st_cluster_f32(my_share + (uint32_t)(G * D + G + g) * 4u, den);
      }
    }
  }
  if (C > 1) {
    cluster_sync_all();  // every rank's share has landed in rank 0; the other ranks are done
    if (crank == 0) {
      for (int e = tid; e < G * D; e += blockDim.x) {
        const int g = e / D;
        float top = -INFINITY;
        for (int r = 0; r < C; ++r) top = fmaxf(top, shares[r * kShare + G * D + g]);
        float num = 0.f, den = 0.f;
        if (top > -INFINITY) {
          for (int r = 0; r < C; ++r) {  // rank order: the same sum on every run
            const float a = exp2f(shares[r * kShare + G * D + g] - top);
            num = fmaf(a, shares[r * kShare + e], num);
            den = fmaf(a, shares[r * kShare + G * D + G + g], den);
          }
        }
        out[e] = __float2bfloat16_rn(den > 0.f ? num / den : 0.f);
      }
    }
  }
  IA_TRACE(14);
}

template <typename T, int D, int G, int NG, typename KB, int BOUND, bool FUSE, bool TWOPASS = false>
__device__ __forceinline__ void select_body(const SelectParams& p) {
  // TWOPASS: no per-(row, block) state.  The first pass over the summaries only forms the row normalisers;
  // a second pass over the same tiles (out of L2) scores every block again and turns it into its condition
  // score at once.  The CTA then needs a few KB per thousand blocks instead of 8 G bytes per block, so that
  // long sequences with eight query rows per kv head still fit two narrow CTAs per SM.
  static_assert(!TWOPASS || (kUseMma<T, G> && BOUND == 0 && !FUSE && NG == kNarrowGroups),
                "the two-pass form is built for the narrow tensor-core shape and the range bound");
  // BOUND: 0 = coordinate range from two arrays, 1 = diagonal ellipsoid (w, rho), 2 = coordinate range from the
  // packed array of (k_max[d], k_min[d]) pairs (same stage layout as 0: the pairs fill the two bound vectors' space)
  constexpr bool DIAG = BOUND == 1, PACKED = BOUND == 2;
  using L = TileLayout<T, D, KB, DIAG>;
  using P = SmemPlan<D, G, kUseMma<T, G>, NG>;
  constexpr int kGroups = NG, kConsumerWarps = Shape<NG>::consumer_warps, kWarps = Shape<NG>::warps,
                kThreads = Shape<NG>::threads;
  constexpr int DQ = D / kGroupWarps;  // head_dim slice of one warp of a group
  static_assert(kWarps <= 16, "a scratch row of the compaction holds 16 warps");
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int C = p.cluster;
  int pair = blockIdx.x / C;  // (sequence, kv head); re-mapped below when the grid runs in several waves
  const int crank = blockIdx.x - pair * C;  // rank inside the cluster that shares this pair
  // Launched with programmatic dependent launch: nothing in global memory may be read
  // before the predecessor on the stream has completed (it may have produced the
  // lengths or the query, and the attention kernel of the previous step may still be
  // reading the selection this kernel overwrites).  Then let this step's attention
  // kernel start occupying free SMs.
  IA_TRACE_BEGIN();
  if (tid == Shape<NG>::consumer_warps * 32) {  // the producer lane: descriptors are kernel parameters, fetch them early
    asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_kbar) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_kmax) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&p.tm_kmin) : "memory");
    if constexpr (FUSE) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.att.tm_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&p.att.tm_v) : "memory");
      if (p.att.hybrid) asm volatile("prefetch.tensormap [%0];" ::"l"(&p.att.tm_vbar) : "memory");
    }
  }
  grid_dependency_wait();
  grid_launch_dependents();
  IA_TRACE(0);
  if constexpr (FUSE) {
    if (blockIdx.x == 0 && tid == 0 && p.stamps != nullptr) p.stamps[0] = global_timer_ns();
  }
  if (p.longest_first) {
    // More CTAs than the GPU holds at once: the hardware hands out CTAs in index order, so the CTAs take
    // the sequences longest first - a long sequence that starts in the last wave would run alone at the
    // end.  Every CTA ranks the batch by prefix length for itself (ties by index): a few hundred
    // cached loads per thread.
    int& seq_of_rank = reinterpret_cast<int*>(smem_raw + P::bars + P::hist)[30];  // a free word of the scan scratch
    const int n_seq = p.n_pairs / p.n_kv_heads;
    const int want = pair / p.n_kv_heads, head = pair - want * p.n_kv_heads;
    for (int t = tid; t < n_seq; t += kThreads) {
      const int len = p.prefix_lens[t];
      int rank = 0;
      for (int j = 0; j < n_seq; ++j) {
        const int lj = p.prefix_lens[j];
        rank += (lj > len || (lj == len && j < t)) ? 1 : 0;
      }
      if (rank == want) seq_of_rank = t;
    }
    __syncthreads();
    pair = seq_of_rank * p.n_kv_heads + head;
  }
  const int seq = pair / p.n_kv_heads;
  const int prefix = p.prefix_lens[seq];
  const int nb = min((prefix + p.block_size - 1) / p.block_size, p.max_blocks);
  const int nb_cap = p.nb_cap;
  // Blocks of this GPU: all of them, or the rank's range [block_lo, block_hi) in split-KV (tile
  // aligned).  This CTA scores the tiles [t_lo, t_hi) = blocks [b_lo, b_hi) of them; cluster rank 0
  // routes for the pair.
  const bool xch_on = p.xch.n_ranks > 0;
  const int r_lo = xch_on ? min(p.block_lo, nb) : 0, r_hi = xch_on ? min(p.block_hi, nb) : nb;
  const int rt_lo = r_lo / kTileBlocks;
  const int n_tiles = max((r_hi + kTileBlocks - 1) / kTileBlocks - rt_lo, 0);
  const int t_lo = rt_lo + n_tiles * crank / C, t_hi = rt_lo + n_tiles * (crank + 1) / C;
  const int n_my_tiles = t_hi - t_lo;
  const int b_lo = t_lo * kTileBlocks, b_hi = min(t_hi * kTileBlocks, r_hi);
  const int nbl = p.nb_loc_cap;
  const int xstep = xch_on ? *p.xch.step_counter + 1 : 0;  // advanced by the last CTA to leave
  const int xpar = xstep & 1;
  // Ring geometry.  The consumers of a stage are "slots" (two tensor-core warps, or a group of four
  // CUDA-core warps) that walk the tiles round robin.  A parity wait can only tell a phase from its
  // neighbour, so the slot that waits for use u of a stage must know that use u - 1 has completed:
  // the stage count is cut to a multiple of the slot count, which makes every stage the property of
  // one slot - the slot that consumed use u - 1 is the one that waits for use u.  (With 8 stages
  // and 6 slots the owners rotated; a wait then passed on the previous phase, the ring lost step
  // and a bounded wait ran out.)
  constexpr int kSlotUnits = kUseMma<T, G> ? kConsumerWarps / 2 : kGroups;
  const int n_slots = min(kSlotUnits, p.n_stages);
  const int n_stages = p.n_stages - p.n_stages % n_slots;

  // ---- shared memory carve-up -------------------------------------------------
  unsigned char* sp = smem_raw;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sp);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* full_bar2 = empty_bar + kMaxStages;        // second pass (TWOPASS)
  uint64_t* empty_bar2 = full_bar2 + kMaxStages;       sp += P::bars;
  int* hist = reinterpret_cast<int*>(sp);              sp += P::hist;   // three rotating 256-bin histograms
  int* scan_scratch = reinterpret_cast<int*>(sp);      sp += P::scan;
  float* red_s = reinterpret_cast<float*>(sp);                          // [kWarps][16][3] row normalisers
  float* redb_s = red_s + kWarps * 16 * 3;             sp += P::red;    // [kWarps] max value norm
  float* norm_s = reinterpret_cast<float*>(sp);        sp += P::norm;   // z_m[16], 1/z_l[16], 2 b_all/denom[16]
  sp += P::state;
  float* q_s = reinterpret_cast<float*>(sp);                            // [G][D]
  float* aq_s = q_s + G * D;                           sp += P::qrows;  // |q|
  float* part_s = reinterpret_cast<float*>(sp);        sp += P::part;   // [consumer warp][3G][32]
  float* xch_s = reinterpret_cast<float*>(sp);         sp += P::xch;    // [cluster rank][16][3], written by peers
  float* xst_s = reinterpret_cast<float*>(sp);         sp += P::xst;    // [16][4] this GPU's row normalisers
  float* vn_s = reinterpret_cast<float*>(sp);                           // [nb_cap]
  float* score_s = vn_s + nb_cap;                                       // [nb_cap]
  float* rho_s = score_s + nb_cap;                                      // [nb_cap] (diag_ell bound only)
  float* z_s = rho_s + nb_cap;                                          // [G][nbl]: z = s + log count (own blocks)
  float* d_s = z_s + (TWOPASS ? 0 : (size_t)G * nbl);                   // [G][nbl]: delta (range bound)
  // split-KV: the ranks' top-k candidates, gathered: [n_ranks * max_sel] scores and block indices
  float* cand_s = d_s + (TWOPASS ? 0 : (size_t)G * nbl);
  int* candb_s = reinterpret_cast<int*>(cand_s + (xch_on ? p.xch.n_ranks * p.max_sel : 0));
  unsigned char* stage_base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(candb_s + (xch_on ? p.xch.n_ranks * p.max_sel : 0)) + 1023) & ~uintptr_t(1023));

  const int64_t sum_row0 = (int64_t)pair * p.max_blocks;  // first summary row of this pair
  // one ring stage: the TMA box copies of 32 blocks' summaries, completing on the stage's barrier
  auto issue_tile_on = [&](int lt, uint64_t* full_bar) {
    const int stage = lt % n_stages;
    unsigned char* st = stage_base + (size_t)stage * L::bytes;
    const int y = (int)sum_row0 + (t_lo + lt) * kTileBlocks;  // rows past the array are zero-filled by the TMA unit
    mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)L::bytes);
#pragma unroll
    for (int j = 0; j < L::kbar_boxes; ++j)
      tma_load_2d(st + j * L::box_bytes, &p.tm_kbar, j * L::kbar_box_cols, y, &full_bar[stage]);
    if constexpr (PACKED) {  // rows of 2 D elements: twice the boxes of one vector, into the two vectors' space
#pragma unroll
      for (int j = 0; j < 2 * L::bnd_boxes; ++j)
        tma_load_2d(st + L::kbar_bytes + j * L::box_bytes, &p.tm_kmax, j * L::bnd_box_cols, y, &full_bar[stage]);
    } else {
#pragma unroll
      for (int j = 0; j < L::bnd_boxes; ++j) {
        tma_load_2d(st + L::kbar_bytes + j * L::box_bytes, &p.tm_kmax, j * L::bnd_box_cols, y, &full_bar[stage]);
        if constexpr (!DIAG)
          tma_load_2d(st + L::kbar_bytes + L::bnd_bytes + j * L::box_bytes, &p.tm_kmin, j * L::bnd_box_cols, y,
                      &full_bar[stage]);
      }
    }
  };
  auto issue_tile = [&](int lt) { issue_tile_on(lt, full_bar); };
  // The producer lane owns the barriers: it initialises them and fills the ring's first uses while
  // the other warps still fetch the query and the value norms - the summaries are on their way
  // before the CTA's set-up barrier.  The consumers touch the barriers only after that barrier.
  // With the pair to itself (C == 1) the CTA does not even wait for the sequence length: it primes
  // the ring with the first tiles of the pair's rows of the summary arrays (they exist up to
  // max_blocks whatever the length; a tile past the sequence's last block is awaited and skipped),
  // so the length's load latency is off the path to the first data.
  const int n_primed = (C == 1 && !xch_on) ? min(n_stages, nb_cap / kTileBlocks) : min(n_stages, n_my_tiles);
  if (warp == kConsumerWarps) {
    if (lane == 0) {
      for (int s = 0; s < n_stages; ++s) {
        mbar_init(&full_bar[s], 1);
        mbar_init(&empty_bar[s], kUseMma<T, G> ? 2 : kGroupWarps);
        if constexpr (TWOPASS) {
          mbar_init(&full_bar2[s], 1);
          mbar_init(&empty_bar2[s], 2);
        }
      }
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
      for (int lt = 0; lt < n_primed; ++lt) issue_tile(lt);
    }
    __syncwarp();
  } else {
    const T* qrow = static_cast<const T*>(p.q) + (int64_t)pair * G * D;
    for (int i = tid; i < G * D; i += kConsumerWarps * 32) {
      const float v = to_f32(qrow[i]);
      q_s[i] = v;
      aq_s[i] = DIAG ? v * v : fabsf(v);  // what the CUDA-core form multiplies the bound vector with
    }
  }
  const float* vn_g = p.v_norm_max + (int64_t)pair * p.max_blocks;
  {
    // value norms of every block the arrays hold, four loads in flight per thread before the first
    // use of the sequence length (entries past the last block are parked but never read)
    float bmax = 0.f;  // b_all = max_b v_norm_max[b]
    if (warp != kConsumerWarps) {
      constexpr int kStride = kConsumerWarps * 32;
      for (int base = tid; base < p.max_blocks; base += 4 * kStride) {
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = base + j * kStride < p.max_blocks ? vn_g[base + j * kStride] : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int b = base + j * kStride;
          if (b < p.max_blocks) vn_s[b] = v[j];
          if (b >= r_lo && b < r_hi) bmax = fmaxf(bmax, v[j]);
        }
        if constexpr (DIAG) {
          const float* rho_g = p.rho + (int64_t)pair * p.max_blocks;
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (base + j * kStride < p.max_blocks) rho_s[base + j * kStride] = rho_g[base + j * kStride];
        }
      }
      bmax = warp_max(bmax);
    }
    if (lane == 0) redb_s[warp] = bmax;
  }
  __syncthreads();
  IA_TRACE(1);

  const float root = sqrtf((float)D);
  const float log_full = logf((float)p.block_size);

  // ---- phase 1: stream the summaries, s / delta per (row, block) -----------------
  if (warp == kConsumerWarps) {
    // producer: one elected lane issues the TMA box copies of each stage
    bool alive = true;
    for (int lt = n_primed; lt < n_my_tiles; ++lt) {  // the first use of every stage was issued above
      const int stage = lt % n_stages;
      const int use = lt / n_stages;
      if (alive && !mbar_wait(&empty_bar[stage], (uint32_t)((use - 1) & 1))) {
        alive = false;
        if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
      }
      if (lane == 0) issue_tile(lt);
      __syncwarp();
    }
  } else if constexpr (kUseMma<T, G>) {
    // Tensor-core consumers.  A stage holds 32 blocks; the two warps of a slot
    // take 16 blocks each as the M side of the MMAs, the query rows are the N
    // side (padded to 8), head_dim is K.  All operands are exact: k_bar is cut
    // into three tf32 pieces (11 + 11 + 2 bits), the bounds and the query are
    // bf16; q+ = max(q, 0) and q- = min(q, 0) turn the reference's
    // sum_d max(q k_max, q k_min) into k_max . q+ + k_min . q- (IMPL/core.py:520-530).
    const int mh = warp & 1, slot = warp >> 1;
    constexpr int kSlots = kConsumerWarps / 2;
    const int n = lane >> 2, kq = lane & 3;
    uint32_t bq[D / 8][2], bp[D / 16][2], bm[D / 16][2];
#pragma unroll
    for (int kk = 0; kk < D / 8; ++kk) {
      bq[kk][0] = n < G ? __float_as_uint(q_s[n * D + kk * 8 + kq]) : 0u;
      bq[kk][1] = n < G ? __float_as_uint(q_s[n * D + kk * 8 + kq + 4]) : 0u;
    }
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float x0 = n < G ? q_s[n * D + kk * 16 + h * 8 + kq * 2] : 0.f;
        const float x1 = n < G ? q_s[n * D + kk * 16 + h * 8 + kq * 2 + 1] : 0.f;
        bp[kk][h] = pack_bf16(fmaxf(x0, 0.f), fmaxf(x1, 0.f));
        bm[kk][h] = pack_bf16(fminf(x0, 0.f), fminf(x1, 0.f));
      }
    }
    // diag_ell bound: sum_d q_d^2 w_d^2 on the tensor cores with exact operands - the square of a
    // bf16 value has 16 significant bits and splits exactly into two bf16 pieces, for q^2 (here, once)
    // and for w^2 (below, per tile); the four partial products are accumulated in fp32.
    uint32_t bq2h[D / 16][2], bq2l[D / 16][2];
    if constexpr (DIAG) {
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float x0 = n < G ? q_s[n * D + kk * 16 + h * 8 + kq * 2] : 0.f;
          const float x1 = n < G ? q_s[n * D + kk * 16 + h * 8 + kq * 2 + 1] : 0.f;
          const float s0 = x0 * x0, s1 = x1 * x1;
          const float h0 = __bfloat162float(__float2bfloat16_rn(s0)), h1 = __bfloat162float(__float2bfloat16_rn(s1));
          bq2h[kk][h] = pack_bf16(h0, h1);
          bq2l[kk][h] = pack_bf16(s0 - h0, s1 - h1);
        }
      }
    }
    // ldmatrix row addressing: matrix m of the x4 = (rows 8 (m & 1) .., 16-byte chunk (m >> 1))
    const int lm = lane >> 3, lr = lane & 7;
    const int arow = mh * 16 + (lm & 1) * 8 + lr;
    const uint32_t row_off = (uint32_t)(arow * 128);
    const uint32_t row_xor = (uint32_t)(arow & 7);
    RowNorm rn[2] = {{-INFINITY, 0.f, 0.f}, {-INFINITY, 0.f, 0.f}};
    bool alive = true;
    int lt = slot;
    for (; slot < n_slots && lt < n_my_tiles; lt += n_slots) {
      const int t = t_lo + lt;
      const int stage = lt % n_stages;
      const int use = lt / n_stages;
      if (alive && !mbar_wait(&full_bar[stage], (uint32_t)(use & 1))) {
        alive = false;
        if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
      }
      if (lt == slot) IA_TRACE(2);
      const uint32_t st = smem_u32(stage_base + (size_t)stage * L::bytes);
      float cd[4] = {0.f, 0.f, 0.f, 0.f};
      float xp[4] = {0.f, 0.f, 0.f, 0.f}, xm[4] = {0.f, 0.f, 0.f, 0.f};  // k_max . q+, k_max . q-
      float np_[4] = {0.f, 0.f, 0.f, 0.f}, nm[4] = {0.f, 0.f, 0.f, 0.f};  // k_min . q+, k_min . q-
      if constexpr (sizeof(KB) == 4) {
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk) {
          const int byte = (kk * 8 + (lm >> 1) * 4) * 4;
          uint32_t a[4], hi[4], md[4], lo[4];
          ldmatrix_x4(st + (byte >> 7) * L::box_bytes + row_off + ((((byte >> 4) & 7) ^ row_xor) << 4), a);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            hi[i] = a[i] & 0xffffe000u;
            const float r1 = __uint_as_float(a[i]) - __uint_as_float(hi[i]);
            md[i] = __float_as_uint(r1) & 0xffffe000u;
            lo[i] = __float_as_uint(r1 - __uint_as_float(md[i]));
          }
          mma_tf32(cd, hi, bq[kk]);
          mma_tf32(cd, md, bq[kk]);
          mma_tf32(cd, lo, bq[kk]);
        }
      } else {
        // bf16 k_bar: the same exact bf16 products as the bounds, q = q+ + q-
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int byte = (kk * 16 + (lm >> 1) * 8) * 2;
          uint32_t a[4];
          ldmatrix_x4(st + (byte >> 7) * L::box_bytes + row_off + ((((byte >> 4) & 7) ^ row_xor) << 4), a);
          mma_bf16(cd, a, bp[kk]);
          mma_bf16(cd, a, bm[kk]);
        }
      }
      if constexpr (PACKED) {
        // Rows of (k_max[d], k_min[d]) pairs: a k-step of 16 packed elements is eight coordinates, and
        //   sum_d max(q k_max, q k_min) = row . (q+_0, q-_0, q+_1, q-_1, ...),
        //   sum_d min(q k_max, q k_min) = row . (q-_0, q+_0, q-_1, q+_1, ...):
        // two contractions of length 2 D with the query's signed parts interleaved - the B fragments are
        // put together from the query row in shared memory at every step, the accumulators are xp and np_.
#pragma unroll
        for (int kk = 0; kk < D / 8; ++kk) {
          const int byte = (kk * 16 + (lm >> 1) * 8) * 2;
          const uint32_t off = (byte >> 7) * L::box_bytes + row_off + ((((byte >> 4) & 7) ^ row_xor) << 4);
          uint32_t a[4];
          ldmatrix_x4(st + L::kbar_bytes + off, a);
          const float x0 = n < G ? q_s[n * D + kk * 8 + kq] : 0.f;      // fragment k = 2 kq, 2 kq + 1: coordinate kq
          const float x1 = n < G ? q_s[n * D + kk * 8 + kq + 4] : 0.f;  // k + 8: coordinate kq + 4
          const uint32_t bu[2] = {pack_bf16(fmaxf(x0, 0.f), fminf(x0, 0.f)), pack_bf16(fmaxf(x1, 0.f), fminf(x1, 0.f))};
          const uint32_t bl[2] = {pack_bf16(fminf(x0, 0.f), fmaxf(x0, 0.f)), pack_bf16(fminf(x1, 0.f), fmaxf(x1, 0.f))};
          mma_bf16(xp, a, bu);
          mma_bf16(np_, a, bl);
        }
      }
#pragma unroll
      for (int kk = 0; kk < (PACKED ? 0 : D / 16); ++kk) {
        const int byte = (kk * 16 + (lm >> 1) * 8) * 2;
        const uint32_t off = (byte >> 7) * L::box_bytes + row_off + ((((byte >> 4) & 7) ^ row_xor) << 4);
        uint32_t a[4];
        ldmatrix_x4(st + L::kbar_bytes + off, a);
        if constexpr (DIAG) {
          // a = 16 x 16 fragment of w; square it in registers and split each square into two bf16 pieces
          uint32_t ah[4], al[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float w0 = bf16lo(a[i]), w1 = bf16hi(a[i]);
            const float s0 = w0 * w0, s1 = w1 * w1;
            const float h0 = __bfloat162float(__float2bfloat16_rn(s0)), h1 = __bfloat162float(__float2bfloat16_rn(s1));
            ah[i] = pack_bf16(h0, h1);
            al[i] = pack_bf16(s0 - h0, s1 - h1);
          }
          mma_bf16(xp, ah, bq2h[kk]);
          mma_bf16(xp, ah, bq2l[kk]);
          mma_bf16(xp, al, bq2h[kk]);
          mma_bf16(xp, al, bq2l[kk]);
        } else {
          mma_bf16(xp, a, bp[kk]);
          mma_bf16(xm, a, bm[kk]);
          ldmatrix_x4(st + L::kbar_bytes + L::bnd_bytes + off, a);
          mma_bf16(np_, a, bp[kk]);
          mma_bf16(nm, a, bm[kk]);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp is done with the stage
      // Accumulator element e of this lane = (block row n + 8 (e >> 1), query row 2 kq + (e & 1)).
      // With G <= 4 only the lanes kq < 2 hold real rows: they hand their e = 2, 3
      // to the idle lanes kq + 2, so every lane finishes two (block, row) entries.
      auto finish = [&](int g, int b, float dotv, float up, float lw, RowNorm& acc) {
        if (g < G && b < nb) {
          const int count = min(p.block_size, prefix - b * p.block_size);
          const float s = dotv / root;
          float delta;
          if constexpr (DIAG) {  // up = sum_d q_d^2 w_d^2 (condition_block_ball/gen_selection.py:82-87)
            delta = rho_s[b] * sqrtf(fmaxf(up, 0.f)) / root;
          } else {
            const float upper = up / root;  // sum_d max(q k_max, q k_min)
            const float lower = lw / root;  // sum_d min(q k_max, q k_min)
            delta = fmaxf(fabsf(upper - s), fabsf(lower - s));
          }
          const float z = (count == p.block_size ? log_full : logf((float)count)) + s;
          float ch, a_term, th;
          delta_terms(delta, p.mass_exp, ch, a_term, th);
          norm_absorb(acc, z, ch);
          if constexpr (!TWOPASS) {
            z_s[g * nbl + b - b_lo] = z;
            d_s[g * nbl + b - b_lo] = delta;  // the score phase recomputes cosh - 1 and tanh from it
          }
          const int64_t o = ((int64_t)pair * G + g) * p.max_blocks + b;
          if (p.aux.s != nullptr) p.aux.s[o] = s;
          if (p.aux.z != nullptr) p.aux.z[o] = z;
#ifndef IA_SELECT_TRACE
          if (p.aux.delta != nullptr) p.aux.delta[o] = delta;
#endif
        }
      };
      const int b0 = t * kTileBlocks + mh * 16 + n;
      if constexpr (G <= 4) {
        float dv[2], up[2], lw[2];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const float d2 = __shfl_xor_sync(0xffffffffu, cd[2 + j], 2);
          const float u2 = __shfl_xor_sync(0xffffffffu, xp[2 + j] + nm[2 + j], 2);
          const float l2 = __shfl_xor_sync(0xffffffffu, np_[2 + j] + xm[2 + j], 2);
          dv[j] = kq < 2 ? cd[j] : d2;
          up[j] = kq < 2 ? xp[j] + nm[j] : u2;
          lw[j] = kq < 2 ? np_[j] + xm[j] : l2;
        }
        const int b = b0 + (kq >> 1) * 8;
#pragma unroll
        for (int j = 0; j < 2; ++j) finish((kq & 1) * 2 + j, b, dv[j], up[j], lw[j], rn[j]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          finish(kq * 2 + (e & 1), b0 + (e >> 1) * 8, cd[e], xp[e] + nm[e], np_[e] + xm[e], rn[e & 1]);
      }
    }
    // primed tiles past the sequence's last one: nothing to score, but their copies must have landed
    // before this CTA's shared memory can go away
    for (; slot < n_slots && lt < n_primed; lt += n_slots)
      if (alive && !mbar_wait(&full_bar[lt % n_stages], 0u)) {
        alive = false;
        if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
      }
    // rows held by this lane: G <= 4: 2 (kq & 1) + {0, 1}, shared by the 16 lanes with the same
    // kq & 1; else 2 kq + {0, 1}, shared by 8 lanes.  Merge them; one lane per row reports.
    IA_TRACE(3);
    constexpr int kFirstXor = G <= 4 ? 2 : 4;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      norm_reduce_lanes<kFirstXor, 32>(rn[r]);
      const int g = (G <= 4 ? (kq & 1) : kq) * 2 + r;
      const bool reporter = (G <= 4) ? (lane < 2) : (n == 0);
      if (reporter && g < G) {
        red_s[(warp * 16 + g) * 3 + 0] = rn[r].m;
        red_s[(warp * 16 + g) * 3 + 1] = rn[r].l;
        red_s[(warp * 16 + g) * 3 + 2] = rn[r].d;
      }
    }
  } else {
    const int group = warp / kGroupWarps, wq = warp % kGroupWarps;
    float* my_part = part_s + (size_t)warp * 3 * G * 32;
    const float* grp_part = part_s + (size_t)group * kGroupWarps * 3 * G * 32;
    constexpr int kRowsPerWarp = (G + kGroupWarps - 1) / kGroupWarps;
    RowNorm rn[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) rn[r] = RowNorm{-INFINITY, 0.f, 0.f};
    const int n_groups = n_slots;  // see the note on the ring geometry above
    bool alive = true;
    int lt = group;
    for (; group < n_groups && lt < n_my_tiles; lt += n_groups) {
      const int t = t_lo + lt;
      const int stage = lt % n_stages;
      const int use = lt / n_stages;
      if (alive && !mbar_wait(&full_bar[stage], (uint32_t)(use & 1))) {
        alive = false;
        if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
      }
      const unsigned char* st = stage_base + (size_t)stage * L::bytes;
      const unsigned char* kbar_v = st;
      const unsigned char* kmax_v = st + L::kbar_bytes;
      const unsigned char* kmin_v = st + L::kbar_bytes + L::bnd_bytes;
      const float* q_r = q_s + wq * DQ;
      const float* aq_r = aq_s + wq * DQ;
      float dot[G], mid[G], wid[G];
#pragma unroll
      for (int g = 0; g < G; ++g) { dot[g] = 0.f; mid[g] = 0.f; wid[g] = 0.f; }
#pragma unroll
      for (int c = 0; c < DQ; c += 8) {
        const int e0 = wq * DQ + c;  // first of eight head_dim elements
        float kb[8], hi[8], lo[8];
        if constexpr (sizeof(KB) == 4) {
          load4(swz<float>(kbar_v, lane, e0), kb);
          load4(swz<float>(kbar_v, lane, e0 + 4), kb + 4);
        } else {
          load8(swz<__nv_bfloat16>(kbar_v, lane, e0), kb);
        }
        if constexpr (PACKED) {
          // sixteen packed elements = the (k_max, k_min) pairs of the eight coordinates e0 .. e0 + 7
          float both[16];
          if constexpr (sizeof(T) == 2) {
            float a8[8], b8[8];
            load8(swz<T>(kmax_v, lane, 2 * e0), a8);
            load8(swz<T>(kmax_v, lane, 2 * e0 + 8), b8);
#pragma unroll
            for (int i = 0; i < 8; ++i) { both[i] = a8[i]; both[8 + i] = b8[i]; }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) load4(swz<float>(kmax_v, lane, 2 * e0 + 4 * i), both + 4 * i);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) { hi[i] = both[2 * i]; lo[i] = both[2 * i + 1]; }
        } else if constexpr (sizeof(T) == 2) {
          load8(swz<T>(kmax_v, lane, e0), hi);
          if constexpr (!DIAG) load8(swz<T>(kmin_v, lane, e0), lo);
        } else {
          load4(swz<float>(kmax_v, lane, e0), hi);
          load4(swz<float>(kmax_v, lane, e0 + 4), hi + 4);
          if constexpr (!DIAG) {
            load4(swz<float>(kmin_v, lane, e0), lo);
            load4(swz<float>(kmin_v, lane, e0 + 4), lo + 4);
          }
        }
        // range bound: centre and span of [k_min, k_max]; diag_ell bound: hi holds w, span = w^2 meets q^2
        float ctr[8], span[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if constexpr (DIAG) { ctr[i] = 0.f; span[i] = hi[i] * hi[i]; }
          else { ctr[i] = hi[i] + lo[i]; span[i] = hi[i] - lo[i]; }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float qv[8], av[8];
          load8(q_r + g * D + c, qv);   // warp-uniform address: a broadcast
          load8(aq_r + g * D + c, av);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dot[g] = fmaf(qv[i], kb[i], dot[g]);
            mid[g] = fmaf(qv[i], ctr[i], mid[g]);
            wid[g] = fmaf(av[i], span[i], wid[g]);
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);  // this warp is done with the stage
#pragma unroll
      for (int g = 0; g < G; ++g) {
        my_part[(g * 3 + 0) * 32 + lane] = dot[g];
        my_part[(g * 3 + 1) * 32 + lane] = mid[g];
        my_part[(g * 3 + 2) * 32 + lane] = wid[g];
      }
      group_sync(group);
      const int b = t * kTileBlocks + lane;
      if (b < nb) {
        const int count = min(p.block_size, prefix - b * p.block_size);
        const float logc = count == p.block_size ? log_full : logf((float)count);
        for (int g = wq; g < G; g += kGroupWarps) {
          float v[3];
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < kGroupWarps; ++w) acc += grp_part[((size_t)w * 3 * G + g * 3 + j) * 32 + lane];
            v[j] = acc;
          }
          const float s = v[0] / root;
          float delta;
          if constexpr (DIAG) {  // v[2] = sum_d q_d^2 w_d^2
            delta = rho_s[b] * sqrtf(fmaxf(v[2], 0.f)) / root;
          } else {
            // sum_d max(q k_max, q k_min) = (mid + wid) / 2, sum_d min(...) = (mid - wid) / 2
            const float upper = (0.5f * (v[1] + v[2])) / root;
            const float lower = (0.5f * (v[1] - v[2])) / root;
            delta = fmaxf(fabsf(upper - s), fabsf(lower - s));
          }
          const float z = logc + s;
          float ch, a_term, th;
          delta_terms(delta, p.mass_exp, ch, a_term, th);
          norm_absorb(rn[g / kGroupWarps], z, ch);
          z_s[g * nbl + b - b_lo] = z;
          d_s[g * nbl + b - b_lo] = delta;  // the score phase recomputes cosh - 1 and tanh from it
          const int64_t o = ((int64_t)pair * G + g) * p.max_blocks + b;
          if (p.aux.s != nullptr) p.aux.s[o] = s;
          if (p.aux.z != nullptr) p.aux.z[o] = z;
#ifndef IA_SELECT_TRACE
          if (p.aux.delta != nullptr) p.aux.delta[o] = delta;
#endif
        }
      }
      group_sync(group);  // partial sums may be overwritten from here on
    }
    for (; group < n_groups && lt < n_primed; lt += n_groups)  // primed tiles past the last one: see above
      if (alive && !mbar_wait(&full_bar[lt % n_stages], 0u)) {
        alive = false;
        if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
      }
    // this warp scored rows wq, wq + 4, ...: merge its 32 lanes, lane 0 reports
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      norm_reduce_lanes<1, 32>(rn[r]);
      const int g = wq + r * kGroupWarps;
      if (lane == 0 && g < G) {
        red_s[(warp * 16 + g) * 3 + 0] = rn[r].m;
        red_s[(warp * 16 + g) * 3 + 1] = rn[r].l;
        red_s[(warp * 16 + g) * 3 + 2] = rn[r].d;
      }
    }
  }
  __syncthreads();
  IA_TRACE(4);

  // ---- phase 2: merge the warps' row normalisers (warp g merges row g as a tree) ---------
  for (int g = warp; g < G; g += kWarps) {
    // which warps scored row g: every tensor-core consumer warp, or the warps with
    // w mod 4 = g mod 4 (fma form); the others left nothing
    const bool has = lane < kConsumerWarps && (kUseMma<T, G> ? true : (lane % kGroupWarps == g % kGroupWarps));
    RowNorm tot{-INFINITY, 0.f, 0.f};
    if (has) tot = RowNorm{red_s[(lane * 16 + g) * 3], red_s[(lane * 16 + g) * 3 + 1], red_s[(lane * 16 + g) * 3 + 2]};
    norm_reduce_lanes<1, 16>(tot);
    // this CTA's share of row g goes to every CTA of the cluster (slot = own rank); a CTA that has
    // the pair to itself keeps it where the next loop looks for it, without the cluster round trip
    if (C == 1) {
      if (lane == 0) {
        xch_s[g * 3] = tot.m; xch_s[g * 3 + 1] = tot.l; xch_s[g * 3 + 2] = tot.d;
      }
    } else if (lane < C) {
      const uint32_t dst = map_to_rank(xch_s + (crank * 16 + g) * 3, (uint32_t)lane);
      st_cluster_f32(dst, tot.m);
      st_cluster_f32(dst + 4, tot.l);
      st_cluster_f32(dst + 8, tot.d);
    }
  }
  if (C > 1) cluster_sync_all();
  else __syncwarp();  // row g was parked by this very warp
  for (int g = warp; g < G; g += kWarps) {
    RowNorm tot{-INFINITY, 0.f, 0.f};
    if (lane < C) tot = RowNorm{xch_s[(lane * 16 + g) * 3], xch_s[(lane * 16 + g) * 3 + 1], xch_s[(lane * 16 + g) * 3 + 2]};
    if (C > 1) norm_reduce_lanes<1, 8>(tot);
    float b_all = lane < kWarps ? redb_s[lane] : 0.f;
    b_all = warp_max(b_all);
    if (xch_on) {  // this GPU's share of row g: parked for the exchange below
      if (lane == 0) { xst_s[g * 4] = tot.m; xst_s[g * 4 + 1] = tot.l; xst_s[g * 4 + 2] = tot.d; xst_s[g * 4 + 3] = b_all; }
      continue;
    }
    if (lane == 0) {
      const float denom = fmaxf(tot.d / tot.l, 1e-30f);  // sum_b softmax(z)_b cosh(delta_b)
      norm_s[g] = tot.m;
      norm_s[16 + g] = 1.f / tot.l;
      norm_s[32 + g] = 2.f * b_all / denom;
      if (p.aux.globals != nullptr && crank == 0) {
        // [batch, 4, rows]: (z_m, z_l) and a normaliser pair (c_m, c_l) with
        // c_l e^{c_m} = sum_b e^{z_b} cosh(delta_b); here c_m = z_m.
        const int rows = p.n_kv_heads * G;
        const int head = pair - seq * p.n_kv_heads;
        float* gl = p.aux.globals + (int64_t)seq * 4 * rows + head * G + g;
        gl[0 * rows] = tot.m;
        gl[1 * rows] = tot.l;
        gl[2 * rows] = tot.m;
        gl[3 * rows] = tot.d;
      }
    }
  }
  if (xch_on) {
    // Exchange of the row normalisers between the GPUs of a split-KV group.  Cluster rank 0 stores
    // this GPU's (m, l, d, b_all) of every row into the buffer of every GPU (plain peer stores), fences
    // at system scope and raises its flag there; every CTA of the pair then waits - bounded - for the
    // flags of all GPUs in its own memory and merges the W shares, in rank order on every GPU.
    const int W = p.xch.n_ranks, me = p.xch.my_rank;
    const int64_t slot0 = ((int64_t)xpar * p.n_pairs + pair) * W;
    __syncthreads();
    if (crank == 0) {
      for (int i = tid; i < G * W; i += kThreads) {
        const int g = i % G, w = i / G;
        const float4 v = *reinterpret_cast<const float4*>(xst_s + g * 4);
        *reinterpret_cast<float4*>(p.xch.norm[w] + ((slot0 + me) * 16 + g) * 4) = v;
      }
      __syncthreads();
      if (tid == 0) {
        __threadfence_system();
        for (int w = 0; w < W; ++w) {
          volatile int32_t* f = p.xch.flags[w] + ((int64_t)(xpar * 2 + 0) * p.n_pairs + pair) * W + me;
          *f = xstep;
        }
      }
    }
    if (tid < W && !wait_flag(p.xch.flags[me] + ((int64_t)(xpar * 2 + 0) * p.n_pairs + pair) * W + tid, xstep))
      atomicOr(p.status, DEV_STATUS_PEER_WAIT_TIMEOUT);
    __syncthreads();
    for (int g = warp; g < G; g += kWarps) {
      RowNorm tot{-INFINITY, 0.f, 0.f};
      float b_all = 0.f;
      if (lane < W) {
        const float4 v = __ldcg(reinterpret_cast<const float4*>(p.xch.norm[me] + ((slot0 + lane) * 16 + g) * 4));
        tot = RowNorm{v.x, v.y, v.z};
        b_all = v.w;
      }
      norm_reduce_lanes<1, 8>(tot);
      b_all = warp_max(b_all);
      if (lane == 0) {
        const float denom = fmaxf(tot.d / tot.l, 1e-30f);
        norm_s[g] = tot.m;
        norm_s[16 + g] = 1.f / tot.l;
        norm_s[32 + g] = 2.f * b_all / denom;
        if (p.aux.globals != nullptr && crank == 0) {
          const int rows = p.n_kv_heads * G;
          const int head = pair - seq * p.n_kv_heads;
          float* gl = p.aux.globals + (int64_t)seq * 4 * rows + head * G + g;
          gl[0 * rows] = tot.m;
          gl[1 * rows] = tot.l;
          gl[2 * rows] = tot.m;
          gl[3 * rows] = tot.d;
        }
      }
    }
  }
  __syncthreads();
  IA_TRACE(5);

  // ---- phase 3: GQA-mean condition score -------------------------------------------
  // cond = softmax(z) (2 b_all (cosh d - 1) / denom + 2 b_c tanh(d / 2))   (IMPL/core.py:535-544)
  // Each CTA scores its own blocks and delivers the scores to rank 0 of the cluster,
  // which routes for the whole (sequence, kv head).
  if constexpr (TWOPASS) {
    // Second pass (C == 1, no exchange): the tiles come through the ring once more - out of L2, this CTA has
    // just streamed them - on a second pair of barriers; s, delta and z are formed again, value for value,
    // and go straight into the block's score.  The four lanes of a quad hold the rows of a block; the
    // terms are gathered and added in row order, which is the order of the one-pass form.
    if (warp == kConsumerWarps) {
      const int n_first = min(n_stages, n_my_tiles);
      if (lane == 0)
        for (int lt = 0; lt < n_first; ++lt) issue_tile_on(lt, full_bar2);
      __syncwarp();
      bool alive = true;
      for (int lt = n_first; lt < n_my_tiles; ++lt) {
        const int stage = lt % n_stages, use = lt / n_stages;
        if (alive && !mbar_wait(&empty_bar2[stage], (uint32_t)((use - 1) & 1))) {
          alive = false;
          if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
        }
        if (lane == 0) issue_tile_on(lt, full_bar2);
        __syncwarp();
      }
    } else {
      const int mh = warp & 1, slot = warp >> 1;
      const int n = lane >> 2, kq = lane & 3;
      uint32_t bq[D / 8][2], bp[D / 16][2], bm[D / 16][2];
#pragma unroll
      for (int kk = 0; kk < D / 8; ++kk) {
        bq[kk][0] = n < G ? __float_as_uint(q_s[n * D + kk * 8 + kq]) : 0u;
        bq[kk][1] = n < G ? __float_as_uint(q_s[n * D + kk * 8 + kq + 4]) : 0u;
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const float x0 = n < G ? q_s[n * D + kk * 16 + h * 8 + kq * 2] : 0.f;
          const float x1 = n < G ? q_s[n * D + kk * 16 + h * 8 + kq * 2 + 1] : 0.f;
          bp[kk][h] = pack_bf16(fmaxf(x0, 0.f), fmaxf(x1, 0.f));
          bm[kk][h] = pack_bf16(fminf(x0, 0.f), fminf(x1, 0.f));
        }
      }
      const int lm = lane >> 3, lr = lane & 7;
      const int arow = mh * 16 + (lm & 1) * 8 + lr;
      const uint32_t row_off = (uint32_t)(arow * 128);
      const uint32_t row_xor = (uint32_t)(arow & 7);
      const unsigned quad_base = (unsigned)(lane & ~3);
      bool alive = true;
      for (int lt = slot; slot < n_slots && lt < n_my_tiles; lt += n_slots) {
        const int t = t_lo + lt;
        const int stage = lt % n_stages, use = lt / n_stages;
        if (alive && !mbar_wait(&full_bar2[stage], (uint32_t)(use & 1))) {
          alive = false;
          if (lane == 0) atomicOr(p.status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
        }
        const uint32_t st = smem_u32(stage_base + (size_t)stage * L::bytes);
        float cd[4] = {0.f, 0.f, 0.f, 0.f};
        float xp[4] = {0.f, 0.f, 0.f, 0.f}, xm[4] = {0.f, 0.f, 0.f, 0.f};
        float np_[4] = {0.f, 0.f, 0.f, 0.f}, nm[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (sizeof(KB) == 4) {
#pragma unroll
          for (int kk = 0; kk < D / 8; ++kk) {
            const int byte = (kk * 8 + (lm >> 1) * 4) * 4;
            uint32_t a[4], hi[4], md[4], lo[4];
            ldmatrix_x4(st + (byte >> 7) * L::box_bytes + row_off + ((((byte >> 4) & 7) ^ row_xor) << 4), a);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              hi[i] = a[i] & 0xffffe000u;
              const float r1 = __uint_as_float(a[i]) - __uint_as_float(hi[i]);
              md[i] = __float_as_uint(r1) & 0xffffe000u;
              lo[i] = __float_as_uint(r1 - __uint_as_float(md[i]));
            }
            mma_tf32(cd, hi, bq[kk]);
            mma_tf32(cd, md, bq[kk]);
            mma_tf32(cd, lo, bq[kk]);
          }
        } else {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const int byte = (kk * 16 + (lm >> 1) * 8) * 2;
            uint32_t a[4];
            ldmatrix_x4(st + (byte >> 7) * L::box_bytes + row_off + ((((byte >> 4) & 7) ^ row_xor) << 4), a);
            mma_bf16(cd, a, bp[kk]);
            mma_bf16(cd, a, bm[kk]);
          }
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int byte = (kk * 16 + (lm >> 1) * 8) * 2;
          const uint32_t off = (byte >> 7) * L::box_bytes + row_off + ((((byte >> 4) & 7) ^ row_xor) << 4);
          uint32_t a[4];
          ldmatrix_x4(st + L::kbar_bytes + off, a);
          mma_bf16(xp, a, bp[kk]);
          mma_bf16(xm, a, bm[kk]);
          ldmatrix_x4(st + L::kbar_bytes + L::bnd_bytes + off, a);
          mma_bf16(np_, a, bp[kk]);
          mma_bf16(nm, a, bm[kk]);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar2[stage]);
        // one (row, block) entry -> its term of the block's score (0 where there is no such row or block)
        auto term = [&](int g, int b, float dotv, float up, float lw) -> float2 {
          if (g >= G || b >= nb) return make_float2(0.f, 0.f);
          const int count = min(p.block_size, prefix - b * p.block_size);
          const float s = dotv / root;
          const float upper = up / root, lower = lw / root;
          const float delta = fmaxf(fabsf(upper - s), fabsf(lower - s));
          const float z = (count == p.block_size ? log_full : logf((float)count)) + s;
          const float pm = expf(z - norm_s[g]) * norm_s[16 + g];
          float ch, a_term, th;
          delta_terms(delta, p.mass_exp, ch, a_term, th);
          const float two_bc = 2.f * vn_s[b];
          return make_float2(pm, fmaf(norm_s[32 + g], a_term, two_bc * th));  // the row adds pm * (...) to the score
        };
        const int b0 = t * kTileBlocks + mh * 16 + n;
        if constexpr (G <= 4) {
          // as in the first pass: lane kq finishes rows 2 (kq & 1) + {0, 1} of block b0 + 8 (kq >> 1)
          float2 tv[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const float d2 = __shfl_xor_sync(0xffffffffu, cd[2 + j], 2);
            const float u2 = __shfl_xor_sync(0xffffffffu, xp[2 + j] + nm[2 + j], 2);
            const float l2 = __shfl_xor_sync(0xffffffffu, np_[2 + j] + xm[2 + j], 2);
            const float dv = kq < 2 ? cd[j] : d2;
            const float up = kq < 2 ? xp[j] + nm[j] : u2;
            const float lw = kq < 2 ? np_[j] + xm[j] : l2;
            tv[j] = term((kq & 1) * 2 + j, b0 + (kq >> 1) * 8, dv, up, lw);
          }
          // rows 0, 1 sit in lane 2 h, rows 2, 3 in lane 2 h + 1 of the quad (h = block half)
          const unsigned src = quad_base + (unsigned)(kq & 2);
          float sum = 0.f;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float pm = __shfl_sync(0xffffffffu, tv[j].x, src + r), f = __shfl_sync(0xffffffffu, tv[j].y, src + r);
              if (2 * r + j < G) sum = fmaf(pm, f, sum);
            }
          }
          const int b = b0 + (kq >> 1) * 8;
          if ((kq & 1) == 0 && b < nb) {
            const float sc = sum / (float)G;
            score_s[b] = sc;
            if (p.aux.score != nullptr) p.aux.score[(int64_t)pair * p.max_blocks + b] = sc;
          }
        } else {
          // lane kq holds rows 2 kq, 2 kq + 1 of the blocks b0 and b0 + 8
          float2 tv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e)
            tv[e] = term(kq * 2 + (e & 1), b0 + (e >> 1) * 8, cd[e], xp[e] + nm[e], np_[e] + xm[e]);
          float sum[2] = {0.f, 0.f};
#pragma unroll
          for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                const float pm = __shfl_sync(0xffffffffu, tv[2 * h + j].x, quad_base + r);
                const float f = __shfl_sync(0xffffffffu, tv[2 * h + j].y, quad_base + r);
                if (2 * r + j < G) sum[h] = fmaf(pm, f, sum[h]);
              }
            }
          }
          if (kq == 0) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int b = b0 + h * 8;
              if (b < nb) {
                const float sc = sum[h] / (float)G;
                score_s[b] = sc;
                if (p.aux.score != nullptr) p.aux.score[(int64_t)pair * p.max_blocks + b] = sc;
              }
            }
          }
        }
      }
    }
  } else {
    const uint32_t score_r0 = map_to_rank(score_s, 0u);
    for (int b = b_lo + tid; b < b_hi; b += kThreads) {
      const float two_bc = 2.f * vn_s[b];
      float sum = 0.f;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pm = expf(z_s[g * nbl + b - b_lo] - norm_s[g]) * norm_s[16 + g];
        float ch, a_term, th;
        delta_terms(d_s[g * nbl + b - b_lo], p.mass_exp, ch, a_term, th);
        sum = fmaf(pm, fmaf(norm_s[32 + g], a_term, two_bc * th), sum);  // written out: the two-pass form adds the same way
      }
      const float sc = sum / (float)G;
      if (C == 1) score_s[b] = sc;
      else st_cluster_f32(score_r0 + (uint32_t)b * 4u, sc);
      if (p.aux.score != nullptr) p.aux.score[(int64_t)pair * p.max_blocks + b] = sc;
    }
  }
  if (C > 1) cluster_sync_all();
  else __syncthreads();
  IA_TRACE(6);
  // Split-KV bookkeeping: the CTA that leaves last advances this GPU's step number (every CTA has
  // read it by then), so that the next launch - also a replay of a captured graph - uses the next one.
  auto leave = [&]() {
    if (xch_on && tid == 0) {
      const unsigned done = atomicAdd(reinterpret_cast<unsigned*>(p.xch.grid_counter), 1u);
      if (done == gridDim.x - 1) {
        *p.xch.grid_counter = 0;
        *p.xch.step_counter = xstep;
      }
    }
  };
  // One-kernel step: the picked blocks also stay in shared memory (the value norms are not needed any more).
  int* sel_list = reinterpret_cast<int*>(vn_s);
  int count = 0;
  if (crank != 0) {
    leave();
    // nobody reads this CTA's shared memory any more - unless it goes on to attend its share of the pages
    if constexpr (!FUSE) return;
  } else {
    // ---- phase 4: routing ----------------------------------------------------------------
    // route(sc, n, emit): among the n scores sc[0..n) pick the top_k best (higher score first, lower
    // position first among equal scores) or, in epsilon mode, every score above eps; emit(slot, j) is
    // called once per picked position j with its output slot - slots ascend with j.  Returns how
    // many were picked.  Every thread of the CTA calls it (it contains CTA barriers).
    auto route = [&](const float* sc, int n, auto emit) -> int {
      uint32_t thr_key = 0, thr_mask = 0xffffffffu;  // keys are compared on the digits resolved so far
      int take_equal = 0;
      const int k_eff = (p.mode == IA_SELECT_TOPK) ? min(min(p.top_k, n), p.max_sel) : 0;
      if (k_eff > 0 && k_eff < n) {
        // Radix select of the k_eff-th largest key, 8 bits per pass.  Three
        // histograms rotate: pass p fills hist[p % 3] and clears hist[(p + 1) % 3]
        // (last read two passes ago), and every warp resolves the digit for itself
        // from the finished histogram - so a pass needs one barrier.
        uint32_t fixed = 0, fixed_mask = 0;
        int remaining = k_eff;
        for (int i = tid; i < 256; i += kThreads) hist[i] = 0;
        __syncthreads();
#pragma unroll 1  // executed once per launch: keep the cold code short (it is fetched from L2)
        for (int pass = 0; pass < 4; ++pass) {
          const int shift = 24 - 8 * pass;
          int* h = hist + (pass % 3) * 256;
          int* h_next = hist + ((pass + 1) % 3) * 256;
          for (int i = tid; i < 256; i += kThreads) h_next[i] = 0;
          for (int base = 0; base < n; base += kThreads) {
            const int b = base + tid;
            const uint32_t key = b < n ? order_key(sc[b]) : 0u;
            const bool live = b < n && (key & fixed_mask) == fixed;
            const uint32_t digit = (key >> shift) & 255u;
            // Bin d lives at word (d & 7) * 32 + (d >> 3): the eight bins a lane scans below are then in
            // eight different rows of 32 consecutive words, so the scan's loads are free of bank conflicts
            // (a [256] array read as h[8 lane + i] is an 8-way conflict, paid by every warp in every pass).
            // The leading digit (sign and high exponent bits) is shared by most keys: there the lanes of
            // a warp that share a digit send one atomic together; the later digits are spread, and finding
            // equal ones costs more than the few conflicts it would save.
            if (pass == 0) {
              const uint32_t peers = __match_any_sync(0xffffffffu, live ? digit : 0xffffffffu);
              if (live && lane == __ffs(peers) - 1) atomicAdd(&h[(digit & 7u) * 32u + (digit >> 3)], __popc(peers));
            } else if (live) {
              atomicAdd(&h[(digit & 7u) * 32u + (digit >> 3)], 1);
            }
          }
#ifdef IA_SELECT_TRACE_FINE
          if (pass < 2) IA_TRACE(9 + 3 * pass);
#endif
          __syncthreads();
#ifdef IA_SELECT_TRACE_FINE
          if (pass < 2) IA_TRACE(10 + 3 * pass);
#endif
          // lane owns bins [8 lane, 8 lane + 8); `above` = keys in the bins of higher lanes
          int c[8], mine = 0;
#pragma unroll
          for (int i = 0; i < 8; ++i) { c[i] = h[i * 32 + lane]; mine += c[i]; }
          int incl = mine;  // inclusive suffix sum over lanes
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const int v = __shfl_down_sync(0xffffffffu, incl, o);
            if (lane + o < 32) incl += v;
          }
          const int above = incl - mine;
          const bool owner = (above < remaining) && (incl >= remaining);
          int digit = 0, left = 0, in_bin = 0;
          if (owner) {
            int acc = above;
#pragma unroll
            for (int i = 7; i >= 0; --i) {
              if (acc + c[i] >= remaining) { digit = lane * 8 + i; in_bin = c[i]; break; }
              acc += c[i];
            }
            left = remaining - acc;
          }
          const int src = max(__ffs(__ballot_sync(0xffffffffu, owner)) - 1, 0);  // exactly one owner lane
          digit = __shfl_sync(0xffffffffu, digit, src);
          remaining = __shfl_sync(0xffffffffu, left, src);
          in_bin = __shfl_sync(0xffffffffu, in_bin, src);
          fixed |= (uint32_t)digit << shift;
          fixed_mask |= 255u << shift;
#ifdef IA_SELECT_TRACE_FINE
          if (pass < 2) IA_TRACE(11 + 3 * pass);
#else
          IA_TRACE(9 + pass);
#endif
          // every key of the threshold bin is wanted: the remaining digits cannot change the outcome
          if (in_bin == remaining) break;
        }
        thr_key = fixed;
        thr_mask = fixed_mask;
        take_equal = remaining;
      }
      IA_TRACE(7);

      // Ordered compaction.  Selected = key above the threshold, plus the first
      // `take_equal` keys equal to it in index order; one block scan of the packed
      // counts (greater: low 16 bits, equal: high 16 bits) gives every output slot.
      int n_written = 0;
      const bool any = (p.mode == IA_SELECT_EPS) ? (n > 0) : (k_eff > 0);
      if (any) {
        const bool everything = (p.mode == IA_SELECT_TOPK) && (k_eff >= n);
        int gt_seen = 0, eq_seen = 0;
        for (int base = 0; base < n; base += kThreads) {
          const int b = base + tid;
          const bool in = b < n;
          const float v = in ? sc[b] : 0.f;
          bool gt, eq = false;
          if (p.mode == IA_SELECT_EPS) {
            gt = in && (v > p.eps);
          } else if (everything) {
            gt = in;
          } else {
            const uint32_t key = order_key(v) & thr_mask;
            gt = in && key > thr_key;
            eq = in && key == thr_key;
          }
          // exclusive scan of (gt, eq) over the block
          const uint32_t bg = __ballot_sync(0xffffffffu, gt), be = __ballot_sync(0xffffffffu, eq);
          const uint32_t below = (1u << lane) - 1u;
          // two scratch rows used alternately: the row of this iteration is not rewritten before every
          // warp has passed the barrier of the next one, so one barrier per iteration is enough
          int* scan_row = scan_scratch + ((base / kThreads) & 1) * 16;
          if (lane == 0) scan_row[warp] = __popc(bg) | (__popc(be) << 16);
          __syncthreads();
          int packed_before = 0, packed_total = 0;
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const int c = scan_row[w];
            if (w < warp) packed_before += c;
            packed_total += c;
          }
          const int gt_before = gt_seen + (packed_before & 0xffff) + __popc(bg & below);
          const int eq_before = eq_seen + (packed_before >> 16) + __popc(be & below);
          const bool take = gt || (eq && eq_before < take_equal);
          const int pos = gt_before + min(eq_before, take_equal);
          if (take && pos >= 0 && pos < p.max_sel) emit(pos, b);
          gt_seen += packed_total & 0xffff;
          eq_seen += packed_total >> 16;
        }
        n_written = gt_seen + min(eq_seen, take_equal);
      }
      return max(min(n_written, p.max_sel), 0);
    };

    int32_t* out_idx = p.sel_idx + (int64_t)pair * p.max_sel;
    int n_written;
    if (!xch_on) {
      n_written = route(score_s, nb, [&](int slot, int b) {
        out_idx[slot] = b;
        if constexpr (FUSE) {
          // the picked blocks stay on chip, in the shared memory of every CTA that will attend over them
          if (C == 1) sel_list[slot] = b;
          else
            for (int r = 0; r < C; ++r) st_cluster_s32(map_to_rank(sel_list + slot, (uint32_t)r), b);
        }
      });
    } else {
      // Split-KV: the k best of this GPU's blocks are candidates - (score, block index) in block order -
      // and go to every GPU; the k best of all candidates, taken in rank order (= block order, the
      // ranks own ascending ranges), are the selection, identical on every GPU.
      const int W = p.xch.n_ranks, me = p.xch.my_rank, kc = p.max_sel;
      const int64_t slot0 = ((int64_t)xpar * p.n_pairs + pair) * W;
      const int n_mine = route(score_s + r_lo, max(r_hi - r_lo, 0), [&](int slot, int j) {
        const float2 c = make_float2(score_s[r_lo + j], __int_as_float(r_lo + j));
        for (int w = 0; w < W; ++w) reinterpret_cast<float2*>(p.xch.cand[w])[(slot0 + me) * (kc + 1) + slot] = c;
      });
      if (tid == 0)
        for (int w = 0; w < W; ++w)
          reinterpret_cast<float2*>(p.xch.cand[w])[(slot0 + me) * (kc + 1) + kc] = make_float2(__int_as_float(n_mine), 0.f);
      __syncthreads();
      if (tid == 0) {
        __threadfence_system();
        for (int w = 0; w < W; ++w) {
          volatile int32_t* f = p.xch.flags[w] + ((int64_t)(xpar * 2 + 1) * p.n_pairs + pair) * W + me;
          *f = xstep;
        }
      }
      if (tid < W && !wait_flag(p.xch.flags[me] + ((int64_t)(xpar * 2 + 1) * p.n_pairs + pair) * W + tid, xstep))
        atomicOr(p.status, DEV_STATUS_PEER_WAIT_TIMEOUT);
      __syncthreads();
      const float2* mine = reinterpret_cast<const float2*>(p.xch.cand[me]);
      int n_all = 0;
      for (int w = 0; w < W; ++w) {  // rank order; every thread walks the W counts
        const int n_w = min(max(__float_as_int(__ldcg(&mine[(slot0 + w) * (kc + 1) + kc]).x), 0), kc);
        for (int i = tid; i < n_w; i += kThreads) {
          const float2 c = __ldcg(&mine[(slot0 + w) * (kc + 1) + i]);
          cand_s[n_all + i] = c.x;
          candb_s[n_all + i] = __float_as_int(c.y);
        }
        n_all += n_w;
      }
      __syncthreads();
      n_written = route(cand_s, n_all, [&](int slot, int j) { out_idx[slot] = candb_s[j]; });
    }
    IA_TRACE(8);
    count = n_written;
    for (int i = count + tid; i < p.max_sel; i += kThreads) out_idx[i] = -1;
    if (tid == 0) {
      p.sel_count[pair] = count;
      if (p.split_counters != nullptr) p.split_counters[pair] = 0;
    }
    leave();
  }
  if constexpr (FUSE) {
    if (C > 1) {
      // The cluster shares the attention too: rank 0 has stored what it picked into every rank's shared
      // memory (above) and adds the count; past the barrier every rank takes every C-th page.
      int* count_slot = scan_scratch + 31;  // the compaction's scratch rows end at [28]
      if (crank == 0 && tid == 0)
        for (int r = 0; r < C; ++r) st_cluster_s32(map_to_rank(count_slot, (uint32_t)r), count);
      cluster_sync_all();
      count = *count_slot;
    }
    // The histograms are idle: their 3 KB hold the page ring's barriers and descriptors.
    static_assert(P::hist >= 32 * 8, "the page ring's barriers live in the histogram area");
    if (blockIdx.x == 0 && tid == 0 && p.stamps != nullptr) p.stamps[1] = global_timer_ns();
    // delta per (row, block) is dead too: the resolved page numbers go there; the scores' array holds the
    // bitmap of the picked blocks (hybrid); z stays - the representatives' logits
    attend_selected_pages<D, G, kAttendWarps<NG>>(p, pair, seq, prefix, crank, C, sel_list, count, q_s, z_s, nbl,
                                                b_lo, b_hi, reinterpret_cast<uint32_t*>(score_s), nb_cap,
                                                reinterpret_cast<int*>(d_s), G * nbl, stage_base,
                                                reinterpret_cast<unsigned char*>(hist), IA_TRACE_T0);
    if (blockIdx.x == 0 && tid == 0 && p.stamps != nullptr) p.stamps[2] = global_timer_ns();
  }
}

template <typename T, int D, int G, int NG, typename KB, int BOUND>
__global__ void __launch_bounds__(Shape<NG>::threads, Shape<NG>::min_ctas)
condition_block_select_kernel(const __grid_constant__ SelectParams p) {
  select_body<T, D, G, NG, KB, BOUND, false>(p);
}

// The one-kernel layer step: selection, then - in the same CTA, with the picked blocks still in shared
// memory - paged attention over them and the suffix, and the output rows.  bf16 pools, at most eight
// query rows per kv head, one CTA per (sequence, kv head).
template <int D, int G, int NG, typename KB, int BOUND>
__global__ void __launch_bounds__(Shape<NG>::threads, Shape<NG>::min_ctas)
condition_block_select_attend_kernel(const __grid_constant__ SelectParams p) {
  select_body<__nv_bfloat16, D, G, NG, KB, BOUND, true>(p);
}

// The selection without per-(row, block) state (see TWOPASS in select_body): narrow CTAs for sequences whose
// (z, delta) arrays would not leave room for two CTAs per SM.  bf16 pools, at most eight query rows per kv
// head, the range bound from two arrays.
template <int D, int G, typename KB>
__global__ void __launch_bounds__(Shape<kNarrowGroups>::threads, 2)
condition_block_select_twopass_kernel(const __grid_constant__ SelectParams p) {
  select_body<__nv_bfloat16, D, G, kNarrowGroups, KB, 0, false, true>(p);
}


// cuTensorMapEncodeTiled lives in the driver library; fetch it through the
// runtime so that the shared library links against cudart only.
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn tensor_map_encoder() {
  static EncodeTiledFn fn = nullptr;  // every thread would store the same pointer
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &found) == cudaSuccess &&
        found == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// a [rows, D] row-major matrix cut into boxes of 128 bytes x 32 rows with the 128-byte swizzle.
// The descriptor depends only on (base, rows, D, element type); a decode loop asks for the same few
// every step, so the last ones encoded on this thread are kept.
struct CachedMap { const void* base; int64_t rows; int D; bool is_bf16; int box_rows; CUtensorMap map; };
static int encode_rows(CUtensorMap* tm, const void* base, bool is_bf16, int64_t rows, int D,
                       int box_rows = kTileBlocks) {
  constexpr int kSlots = 16;
  static thread_local CachedMap cache[kSlots];
  static thread_local int next_slot = 0;
  for (int i = 0; i < kSlots; ++i)
    if (cache[i].base == base && cache[i].rows == rows && cache[i].D == D && cache[i].is_bf16 == is_bf16 &&
        cache[i].box_rows == box_rows && base != nullptr) {
      *tm = cache[i].map;
      return IA_OK;
    }
  EncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return fail(IA_ERR_LAUNCH, "select: cuTensorMapEncodeTiled is not available from this driver");
  const int esz = is_bf16 ? 2 : 4;
  const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)D * esz};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / esz), (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(IA_ERR_LAUNCH, "select: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  cache[next_slot] = CachedMap{base, rows, D, is_bf16, box_rows, *tm};
  next_slot = (next_slot + 1) % kSlots;
  return IA_OK;
}

// A bf16 KV pool as the 4-D tensor [page, kv head, token, head_dim] with its own page and head strides
// (elements); box = 64 elements x 16 tokens of one (page, kv head), 128-byte swizzle.  Pages past
// n_pages are out of the tensor: the TMA unit fills them with zeros instead of reading.  The two outer
// dimensions are ordered by stride (a cache laid out [batch, kv head, token, head_dim] and addressed in
// place as pages has the larger stride on the head): *heads_outer tells the kernel which coordinate is which.
struct CachedPool { const void* base; int D, heads, pages; int64_t hs, ps; CUtensorMap map; };
static int encode_pool(CUtensorMap* tm, const void* base, int D, int heads, int pages, int64_t head_stride,
                       int64_t page_stride, int* heads_outer) {
  *heads_outer = head_stride > page_stride;
  constexpr int kSlots = 16;
  static thread_local CachedPool cache[kSlots];
  static thread_local int next_slot = 0;
  for (int i = 0; i < kSlots; ++i)
    if (cache[i].base == base && cache[i].D == D && cache[i].heads == heads && cache[i].pages == pages &&
        cache[i].hs == head_stride && cache[i].ps == page_stride && base != nullptr) {
      *tm = cache[i].map;
      return IA_OK;
    }
  EncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return fail(IA_ERR_LAUNCH, "select: cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[4] = {(cuuint64_t)D, 16, (cuuint64_t)heads, (cuuint64_t)pages};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)head_stride * 2, (cuuint64_t)page_stride * 2};
  if (*heads_outer) {
    dims[2] = (cuuint64_t)pages; dims[3] = (cuuint64_t)heads;
    strides[1] = (cuuint64_t)page_stride * 2; strides[2] = (cuuint64_t)head_stride * 2;
  }
  const cuuint32_t box[4] = {64, 16, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return IA_ERR_UNSUPPORTED;  // strides the TMA unit cannot express: the caller keeps two kernels
  cache[next_slot] = CachedPool{base, D, heads, pages, head_stride, page_stride, *tm};
  next_slot = (next_slot + 1) % kSlots;
  return IA_OK;
}


template <typename Kern>
static int launch_kernel(Kern kern, const char* name, const SelectParams& p, int n_pairs, unsigned threads, size_t smem,
                         cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "select: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  e = launch_overlapped(kern, (unsigned)(n_pairs * p.cluster), threads, smem, stream, p, p.cluster);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "%s: %s", name, cudaGetErrorString(e));
  return check_launch(name);
}

// The fused form applies to bf16 pools with head_dim 128, at most eight query rows per kv head, a
// grid that is resident at once, no exchange with other GPUs, and a ring that holds at least one page
// per attending warp.  INTERATTN_B200_FUSED=0 / ia_set_fused_step(0) keep the two kernels;
// INTERATTN_B200_FUSED_WAVES=any lifts the single-wave rule (an experiment switch: measured slower).
template <typename T, int D, int G, int NG, typename KB, int BOUND>
static bool try_launch_fused(SelectParams& p, const AttendRequest& ar, int n_pairs, size_t smem, size_t ring_bytes,
                             int resident_ctas, cudaStream_t stream, int* status) {
  if constexpr (sizeof(T) == 2 && D == 128 && G <= 8) {
    // One wave only: with more CTAs than resident slots a CTA would hold its SM through the serial
    // phases of the selection while the attention of other pairs waits for a slot (measured: the ragged
    // 70B batch, 512 pairs, 255 us fused against 240 us as two kernels).
    static const bool any_waves = [] {
      const char* v = getenv("INTERATTN_B200_FUSED_WAVES");
      return v != nullptr && strcmp(v, "any") == 0;
    }();
    if (ar.req == nullptr || p.xch.n_ranks > 0 || (n_pairs * p.cluster > resident_ctas && !any_waves)) return false;
    const bool off = !fused_step_enabled();
    const ia_geom& g = *ar.geom;
    constexpr size_t kStage = 2 * 16 * D * 2;
    // at the end the start of the ring holds the warps' partial results, and the end of rank 0's ring
    // (kept free of pages) the shares of the CTAs of a cluster
    constexpr size_t kMerge = (size_t)kAttendWarps<NG> * (8 * (D + 4) + 16) * 4;
    const size_t shares = p.cluster > 1 ? (size_t)p.cluster * (G * D + 2 * G) * 4 : 0;
    if (off || g.page_size != 16 || g.block_size % 16 != 0 || g.n_pool_pages <= 0 ||
        ring_bytes < (size_t)kAttendWarps<NG> * kStage + shares || ring_bytes < kMerge + shares)
      return false;
    if (encode_pool(&p.att.tm_k, ar.req->k_pool, D, g.n_kv_heads, g.n_pool_pages, g.pool_head_stride,
                    g.pool_page_stride, &p.att.heads_outer) != IA_OK ||
        encode_pool(&p.att.tm_v, ar.req->v_pool, D, g.n_kv_heads, g.n_pool_pages, g.pool_head_stride,
                    g.pool_page_stride, &p.att.heads_outer) != IA_OK)
      return false;
    p.att.hybrid = ar.req->hybrid;
    if (ar.req->hybrid) {
      const int64_t rows = (int64_t)n_pairs * p.max_blocks;
      if (ar.vbar == nullptr || encode_rows(&p.att.tm_vbar, ar.vbar, true, rows, D, 16) != IA_OK) return false;
      if (ar.req->z_scratch) p.aux.z = nullptr;  // the logits stay in shared memory
    }
    p.att.block_table = ar.req->block_table;
    p.att.seq_lens = ar.req->seq_lens;
    p.att.out = ar.req->out;
    p.att.max_pages = g.max_pages;
    p.att.n_pool_pages = g.n_pool_pages;
    p.att.ring_bytes = (int)ring_bytes;
    p.att.on = 1;
    *status = launch_kernel(condition_block_select_attend_kernel<D, G, NG, KB, BOUND>, "condition_block_select_attend_kernel",
                            p, n_pairs, (unsigned)Shape<NG>::threads, smem, stream);
    ar.req->used = 1;
    return true;
  } else {
    return false;
  }
}

static bool select_in_index_order() {
  static const bool in_order = [] {
    const char* v = getenv("INTERATTN_B200_SELECT_ORDER");
    return v != nullptr && strcmp(v, "index") == 0;
  }();
  return in_order;
}

template <typename T, int D, int G, int NG, typename KB, int BOUND>
static int launch_shaped(SelectParams& p, const AttendRequest& ar, int n_pairs, size_t smem, size_t ring_bytes,
                         int resident_ctas, cudaStream_t stream) {
  int status = IA_OK;
  p.longest_first = !select_in_index_order() && n_pairs * p.cluster > resident_ctas && n_pairs / p.n_kv_heads <= 4096;
  if (try_launch_fused<T, D, G, NG, KB, BOUND>(p, ar, n_pairs, smem, ring_bytes, resident_ctas, stream, &status))
    return status;
  return launch_kernel(condition_block_select_kernel<T, D, G, NG, KB, BOUND>, "condition_block_select_kernel", p,
                       n_pairs, (unsigned)Shape<NG>::threads, smem, stream);
}


template <typename T, int D, int G, typename KB, int BOUND>
static int launch_typed(const SelectParams& base, const AttendRequest& ar, int n_pairs, cudaStream_t stream) {
  constexpr bool DIAG = BOUND == 1, PACKED = BOUND == 2;
  using L = TileLayout<T, D, KB, DIAG>;
  using PW = SmemPlan<D, G, kUseMma<T, G>, kWideGroups>;
  using PN = SmemPlan<D, G, kUseMma<T, G>, kNarrowGroups>;
  SelectParams p = base;
  p.nb_cap = (p.max_blocks + 31) & ~31;
  int dev = 0, max_smem = 0, sm_smem = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  cudaDeviceGetAttribute(&sm_smem, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (max_smem <= 0) max_smem = 227 * 1024;
  if (sm_smem <= 0) sm_smem = 228 * 1024;
  if (sms <= 0) sms = 148;
  // Wide shape: one CTA per SM (shared memory).  With few (sequence, kv head) pairs a
  // thread-block cluster shares each pair: double the cluster while the grid still fits
  // the SMs and every CTA keeps at least two 32-block tiles.
  // INTERATTN_B200_SELECT_CLUSTER pins it.
  // tiles of a pair that this GPU scores: all of them, or those of its block range (split-KV)
  const bool xch_on = p.xch.n_ranks > 0;
  const int max_tiles = xch_on ? (min(p.block_hi, p.nb_cap) - p.block_lo + kTileBlocks - 1) / kTileBlocks
                               : p.nb_cap / kTileBlocks;
  const int n_cand = xch_on ? p.xch.n_ranks * p.max_sel : 0;
  int cluster = 1;
  while (cluster < 8 && n_pairs * cluster * 2 <= sms && max_tiles / (cluster * 2) >= 2) cluster *= 2;
  if (const char* force = getenv("INTERATTN_B200_SELECT_CLUSTER")) {
    const int c = atoi(force);
    if (c == 1 || c == 2 || c == 4 || c == 8) cluster = c;
  }
  p.cluster = cluster;
  p.nb_loc_cap = (max_tiles / cluster + 1) * kTileBlocks;
  const int64_t rows = (int64_t)n_pairs * p.max_blocks;
  if (rows > 0x7fffffff) return fail(IA_ERR_UNSUPPORTED, "select: %lld summary rows exceed the TMA coordinate range", (long long)rows);
  if (int s = encode_rows(&p.tm_kbar, p.k_bar, sizeof(KB) == 2, rows, D)) return s;
  // diag_ell: k_max is w; packed range: k_max is the array of (k_max, k_min) pairs, rows of 2 D elements
  if (int s = encode_rows(&p.tm_kmax, p.k_max, sizeof(T) == 2, rows, PACKED ? 2 * D : D)) return s;
  if constexpr (DIAG || PACKED) p.tm_kmin = p.tm_kmax;  // not read
  else if (int s = encode_rows(&p.tm_kmin, p.k_min, sizeof(T) == 2, rows, D)) return s;

  // Narrow shape: more pairs than SMs and room for two or three CTAs per SM (each CTA pays 1 KB of
  // reserved shared memory) with a ring of at least two stages.  A cluster of narrow CTAs per pair
  // (every CTA keeps only its slice of the (row, block) arrays) is built too but never chosen:
  // on B200 it measured slower than one wide CTA per pair wherever the narrow shape does not fit a
  // whole pair (ragged 70B batch: 162 / 181 us with clusters of 2 / 4 against 119 us) - the
  // cluster barriers and the score hand-over cost more than the overlap of the tails returns.
  // INTERATTN_B200_SELECT_SHAPE=wide|narrow (+ INTERATTN_B200_SELECT_CLUSTER) pin the choice where it fits.
  const char* shape = getenv("INTERATTN_B200_SELECT_SHAPE");
  const bool want_narrow = shape != nullptr ? strcmp(shape, "narrow") == 0 : n_pairs > sms;
  const char* tp = getenv("INTERATTN_B200_SELECT_TWOPASS");
  const int twopass = tp == nullptr ? 0 : atoi(tp);  // 1: the two-pass form wherever the narrow shape is wanted
  if (xch_on && (want_narrow || n_pairs * cluster > sms))
    // the CTAs of a split-KV selection wait for their peers on the other GPUs: all of them must be
    // resident at once (one wide CTA per SM), or a CTA could wait for one that is not scheduled yet
    return fail(IA_ERR_UNSUPPORTED, "select (split-KV): %d (sequence, kv head) pairs x cluster %d exceed the %d SMs",
                n_pairs, cluster, sms);
  if (want_narrow) {
    for (int c = cluster; c <= 8 && twopass != 1; c *= 2) {
      p.cluster = c;
      p.nb_loc_cap = (max_tiles / c + 1) * kTileBlocks;
      const size_t fixed = PN::fixed + PN::per_blocks(p.nb_cap, p.nb_loc_cap) + 1024;
      int ctas = (n_pairs * c + sms - 1) / sms;
      ctas = ctas < 2 ? 2 : (ctas > 3 ? 3 : ctas);
      for (; ctas >= 2; --ctas) {
        const size_t budget = (size_t)sm_smem / ctas - 1024;
        if (budget < fixed + 2 * (size_t)L::bytes) continue;
        int stages = (int)((budget - fixed) / L::bytes);
        const int my_tiles = (max_tiles + c - 1) / c;
        if (stages > my_tiles) stages = my_tiles < 2 ? 2 : my_tiles;
        if (stages > kMaxStages) stages = kMaxStages;
        p.n_stages = stages;
        // the one-kernel step turns the rest of the CTA's share of shared memory into page stages
        const size_t ring = ar.req != nullptr ? ((budget - fixed) & ~(size_t)1023) : (size_t)stages * L::bytes;
        return launch_shaped<T, D, G, kNarrowGroups, KB, BOUND>(p, ar, n_pairs, fixed + ring, ring, sms * ctas, stream);
      }
      break;  // the narrow shape is only ever tried with the cluster chosen above (1 unless pinned)
    }
    // The two-pass form keeps no (z, delta) arrays and so fits two narrow CTAs per SM where the one-pass
    // narrow shape does not (long sequences, eight query rows per kv head).  Measured on the ragged 70B
    // batch it loses to the wide shape all the same (135.8 against 113.5 us: four consumer warps and a
    // two-stage ring per CTA, every summary through the tensor cores twice), so it is taken on request
    // only: INTERATTN_B200_SELECT_TWOPASS=1 (also where the one-pass narrow shape fits - A/B runs, tests).
    if constexpr (kUseMma<T, G> && BOUND == 0 && sizeof(T) == 2) {
      if (twopass == 1 && cluster == 1 && !xch_on) {
        p.cluster = 1;
        p.nb_loc_cap = (max_tiles + 1) * kTileBlocks;
        const size_t fixed = PN::fixed + (size_t)p.nb_cap * 4 * 3 + 1024;
        const int ctas = 2;
        const size_t budget = (size_t)sm_smem / ctas - 1024;
        if (budget >= fixed + 2 * (size_t)L::bytes) {
          int stages = (int)((budget - fixed) / L::bytes);
          if (stages > max_tiles) stages = max_tiles < 2 ? 2 : max_tiles;
          if (stages > kMaxStages) stages = kMaxStages;
          p.n_stages = stages;
          p.longest_first = !select_in_index_order() && n_pairs > sms * ctas && n_pairs / p.n_kv_heads <= 4096;
          return launch_kernel(condition_block_select_twopass_kernel<D, G, KB>, "condition_block_select_twopass_kernel",
                               p, n_pairs, (unsigned)Shape<kNarrowGroups>::threads, fixed + (size_t)stages * L::bytes,
                               stream);
        }
      }
    }
    p.cluster = cluster;  // no narrow form fits: the wide shape with the cluster chosen above
    p.nb_loc_cap = (max_tiles / cluster + 1) * kTileBlocks;
  }
  const size_t fixed = PW::fixed + PW::per_blocks(p.nb_cap, p.nb_loc_cap, n_cand) + 1024;
  if ((size_t)max_smem < fixed + 2 * (size_t)L::bytes)
    return fail(IA_ERR_UNSUPPORTED, "select: %d blocks x %d query rows per kv head do not fit in shared memory",
                p.max_blocks, G);
  int stages = (int)(((size_t)max_smem - fixed) / L::bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.n_stages = stages;
  const size_t ring = ar.req != nullptr ? (((size_t)max_smem - fixed) & ~(size_t)1023) : (size_t)stages * L::bytes;
  return launch_shaped<T, D, G, kWideGroups, KB, BOUND>(p, ar, n_pairs, fixed + ring, ring, sms, stream);
}

template <typename T, int D, typename KB, int BOUND>
static int launch_group_bound(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group,
                              cudaStream_t stream) {
  switch (group) {
    case 1: return launch_typed<T, D, 1, KB, BOUND>(p, ar, n_pairs, stream);
    case 2: return launch_typed<T, D, 2, KB, BOUND>(p, ar, n_pairs, stream);
    case 4: return launch_typed<T, D, 4, KB, BOUND>(p, ar, n_pairs, stream);
    case 8: return launch_typed<T, D, 8, KB, BOUND>(p, ar, n_pairs, stream);
    case 16: return launch_typed<T, D, 16, KB, BOUND>(p, ar, n_pairs, stream);
    default: return fail(IA_ERR_UNSUPPORTED, "select: group_size %d not built (1, 2, 4, 8, 16)", group);
  }
}
template <typename T, int D, typename KB = float>
static int launch_group_packed(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group,
                               cudaStream_t stream) {
  return launch_group_bound<T, D, KB, 2>(p, ar, n_pairs, group, stream);
}
template <typename T, int D, typename KB = float>
static int launch_group(const SelectParams& p, const AttendRequest& ar, int n_pairs, int group, cudaStream_t stream) {
  return p.rho != nullptr ? launch_group_bound<T, D, KB, 1>(p, ar, n_pairs, group, stream)
                          : launch_group_bound<T, D, KB, 0>(p, ar, n_pairs, group, stream);
}

}  // namespace

}  // namespace ia
