// Block summaries of a paged KV prefix: one pass over K and V.
//
// Follows the rule of the reference's _build_prompt_blocks
// (llama/script/analysis/condition_block_gen/methods/condition_block_triton_impl/core.py:449-500):
// per (kv head, block) the fp32 mean of K and of V over the block's valid
// tokens, the per-coordinate max / min of K, and the largest token |v|_2.
// Optionally also the diagonal-ellipsoid pair (w, rho) of the reference's
// condition_block_ball study (a second walk over the block's keys).
// The reference runs this as a chain of PyTorch ops over a padded
// [Hkv, nb, B, D] view; here one warp owns one (sequence, kv head, block),
// walks the block's physical pages through the block table and keeps every
// running statistic in registers.  HBM-bound: each K/V byte of the prefix is
// read exactly once (2 * D * sizeof(T) bytes per token per kv head).
#include <stdlib.h>
#include <string.h>

#include "ia_common.cuh"

namespace ia {

// k_max / k_min of a lane's VEC coordinates: two arrays, or - IA_GEOM_PACKED_BOUNDS - one array of
// (k_max[d], k_min[d]) pairs (the reference's packed k_bounds, IMPL/core.py:490-499)
template <typename T, int VEC>
__device__ __forceinline__ void store_bounds(const ia_geom& g, const ia_summaries& out, int64_t row,
                                             const float (&kmax)[VEC], const float (&kmin)[VEC]) {
  if (g.reserved & IA_GEOM_PACKED_BOUNDS) {
    float both[2 * VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) { both[2 * i] = kmax[i]; both[2 * i + 1] = kmin[i]; }
    T* dst = reinterpret_cast<T*>(out.k_max) + 2 * row;
    if constexpr (VEC == 4) {
      float lo[4] = {both[0], both[1], both[2], both[3]}, hi[4] = {both[4], both[5], both[6], both[7]};
      store_vec<4>(dst, lo);
      store_vec<4>(dst + 4, hi);
    } else {
      store_vec<2 * VEC>(dst, both);
    }
  } else {
    store_vec<VEC>(reinterpret_cast<T*>(out.k_max) + row, kmax);
    store_vec<VEC>(reinterpret_cast<T*>(out.k_min) + row, kmin);
  }
}

template <typename T, int D>
__global__ void __launch_bounds__(128)
condition_block_build_summaries_direct_kernel(const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                       const int32_t* __restrict__ block_table,
                                       const int32_t* __restrict__ prefix_lens,
                                       const int32_t* __restrict__ first_blocks, ia_geom g,
                                       ia_summaries out) {
  constexpr int VEC = D / 32;  // elements of a token row per lane
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t n_units = (int64_t)g.batch * g.n_kv_heads * g.max_blocks;
  if (unit >= n_units) return;
  const int blk = (int)(unit % g.max_blocks);
  const int head = (int)((unit / g.max_blocks) % g.n_kv_heads);
  const int seq = (int)(unit / ((int64_t)g.max_blocks * g.n_kv_heads));
  // lengths come from device memory: never index the block table past its row
  const int prefix = min(prefix_lens[seq], g.max_pages * g.page_size);
  const int first = blk * g.block_size;
  if (first >= prefix) return;  // block holds no token: its summary is never read
  // incremental update: blocks below first_blocks[seq] keep the summary they already have
  if (first_blocks != nullptr && blk < first_blocks[seq]) return;
  const int count = min(g.block_size, prefix - first);

  float ksum[VEC], vsum[VEC], kmax[VEC], kmin[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    ksum[i] = 0.f; vsum[i] = 0.f; kmax[i] = -INFINITY; kmin[i] = INFINITY;
  }
  float vn2max = 0.f;

  const int32_t* table = block_table + (int64_t)seq * g.max_pages;
  const int64_t head_off = (int64_t)head * g.pool_head_stride + lane * VEC;
  const int n_pages = (count + g.page_size - 1) / g.page_size;
  for (int p = 0; p < n_pages; ++p) {
    const int page = table[first / g.page_size + p];
    const int64_t base = (int64_t)page * g.pool_page_stride + head_off;
    const int rows = min(g.page_size, count - p * g.page_size);
    // tokens in ascending order: the fp32 sums are accumulated in token order
#pragma unroll 4
    for (int t = 0; t < rows; ++t) {
      float kv[VEC], vv[VEC];
      load_vec<VEC>(k_pool + base + (int64_t)t * D, kv);
      load_vec<VEC>(v_pool + base + (int64_t)t * D, vv);
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        ksum[i] += kv[i];
        vsum[i] += vv[i];
        kmax[i] = fmaxf(kmax[i], kv[i]);
        kmin[i] = fminf(kmin[i], kv[i]);
        sq = fmaf(vv[i], vv[i], sq);
      }
      vn2max = fmaxf(vn2max, warp_sum(sq));
    }
  }

  const float denom = (float)count;
  const int64_t row = unit * D + lane * VEC;
  float kb[VEC], vb[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    kb[i] = ksum[i] / denom;
    vb[i] = vsum[i] / denom;
  }
  if (g.reserved & IA_GEOM_KBAR_BF16)  // the reference's bf16 k_bar option: the fp32 mean, rounded once
    store_vec<VEC>(reinterpret_cast<__nv_bfloat16*>(out.k_bar) + row, kb);
  else
    store_vec<VEC>(out.k_bar + row, kb);
  store_vec<VEC>(reinterpret_cast<T*>(out.v_bar) + row, vb);
  store_bounds<T, VEC>(g, out, row, kmax, kmin);
  if (lane == 0) out.v_norm_max[unit] = sqrtf(vn2max);
  if (out.w == nullptr || out.rho == nullptr) return;

  // Diagonal-ellipsoid pair (condition_block_ball/gen_selection.py:53-73): w from the stored mean and
  // the range, rounded up before a bf16 cast; rho = max_t |(k_t - k_bar) / w| from the stored w, which
  // needs the finished mean and therefore a second walk over the block's keys (they are in L2 now).
  float kc[VEC], inv_w2[VEC], wv[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    kc[i] = kb[i];
    if (g.reserved & IA_GEOM_KBAR_BF16) kc[i] = __bfloat162float(__float2bfloat16_rn(kb[i]));  // the stored mean
    float wi = fmaxf(fmaxf(kmax[i] - kc[i], kc[i] - kmin[i]), 1e-6f);
    if (sizeof(T) == 2) wi = __bfloat162float(__float2bfloat16_rn(wi * (1.f + 0.0078125f)));
    wv[i] = wi;
    inv_w2[i] = 1.f / (wi * wi);
  }
  store_vec<VEC>(reinterpret_cast<T*>(out.w) + row, wv);
  float d2max = 0.f;
  for (int p = 0; p < n_pages; ++p) {
    const int page = table[first / g.page_size + p];
    const int64_t base = (int64_t)page * g.pool_page_stride + head_off;
    const int rows = min(g.page_size, count - p * g.page_size);
#pragma unroll 4
    for (int t = 0; t < rows; ++t) {
      float kv[VEC];
      load_vec<VEC>(k_pool + base + (int64_t)t * D, kv);
      float sq = 0.f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float c = kv[i] - kc[i];
        sq = fmaf(c * c, inv_w2[i], sq);
      }
      d2max = fmaxf(d2max, warp_sum(sq));
    }
  }
  if (lane == 0) out.rho[unit] = sqrtf(d2max);
}

template <typename T, int D>
static int launch_direct(const void* k_pool, const void* v_pool, const int32_t* block_table,
                        const int32_t* prefix_lens, const int32_t* first_blocks, const ia_geom& g,
                        const ia_summaries& out, cudaStream_t stream) {
  const int64_t n_units = (int64_t)g.batch * g.n_kv_heads * g.max_blocks;
  const int warps = 4;
  const int64_t grid = ceil_div64(n_units, warps);
  if (grid <= 0) return IA_OK;
  if (grid > 0x7fffffff) return fail(IA_ERR_UNSUPPORTED, "build_summaries: grid too large");
  condition_block_build_summaries_direct_kernel<T, D><<<(unsigned)grid, warps * 32, 0, stream>>>(
      static_cast<const T*>(k_pool), static_cast<const T*>(v_pool), block_table, prefix_lens, first_blocks, g, out);
  return check_launch("condition_block_build_summaries_direct_kernel");
}

// ---- the streaming form: every page through a per-warp ring of bulk copies ----------------------
// The kernel above keeps a warp's loads in flight only between two rounds of arithmetic.  Here a warp owns
// a ring of page stages in shared memory (the K run and the V run of one (page, kv head): 2 x 16 x D
// elements, each one contiguous piece of the pool) and keeps the ring full with cp.async.bulk copies that
// complete on the stage's mbarrier: the copy of page i + stages is issued the moment page i has been
// consumed, across block and unit boundaries, so HBM never waits for the arithmetic.  The grid is
// persistent (CTAs x 4 warps stride over the (sequence, kv head, block) units); the per-token arithmetic
// and its order are those of the kernel above, value for value.
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void ring_bar_init(uint64_t* bar) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bar)));
}
__device__ __forceinline__ void ring_expect(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ring_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void ring_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_addr(dst)),
               "l"(src), "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
// bounded: false when the phase did not complete (the caller reports it and carries on)
__device__ __forceinline__ bool ring_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < (1u << 20); ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

constexpr int kMaxStreamWarps = 16;

template <typename T, int D>
__global__ void __launch_bounds__(kMaxStreamWarps * 32)
condition_block_build_summaries_kernel(const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                                       const int32_t* __restrict__ block_table,
                                       const int32_t* __restrict__ prefix_lens,
                                       const int32_t* __restrict__ first_blocks, ia_geom g, ia_summaries out,
                                       int n_stages, int* status) {
  constexpr int VEC = D / 32;
  constexpr int kPage = 16;
  constexpr int kRun = kPage * D;                       // elements of one (page, kv head) run
  constexpr uint32_t kRunBytes = kRun * sizeof(T);
  extern __shared__ __align__(128) unsigned char smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int kStreamWarps = (int)(blockDim.x >> 5);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem) + warp * 16;  // up to 16 stages per warp
  T* ring = reinterpret_cast<T*>(smem + kStreamWarps * 16 * 8) + (size_t)warp * n_stages * 2 * kRun;
  int* live = reinterpret_cast<int*>(smem + kStreamWarps * 16 * 8 + (size_t)kStreamWarps * n_stages * 2 * kRunBytes) +
              warp * 16;  // 1: the stage holds a page; 0: its table entry was out of range, nothing was copied
  if (lane == 0) {
    for (int s = 0; s < n_stages; ++s) ring_bar_init(&full[s]);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  const int n_rows = g.batch * g.n_kv_heads;  // (sequence, kv head) rows of max_blocks units each
  const int stride = (int)gridDim.x * kStreamWarps;
  const int cap = g.max_pages * g.page_size;
  // A cursor walks the pages this warp handles: the units w, w + stride, ... (unit = row * max_blocks +
  // block) that hold tokens and are not below first_blocks, page by page.  Two cursors run over the same
  // sequence, the one that issues copies n_stages pages ahead of the one that consumes them.  Runs of
  // units that hold nothing (past a sequence's last block, below first_blocks) are stepped over at once.
  struct Cursor {
    int row, blk;  // blk may exceed max_blocks between steps: normalised in open_unit
    int seq, head, first, count, page, n_pages;
    int page_id;   // issuing cursor: lane j holds the table entry of the unit's page j, fetched when the unit is
                   // opened and first needed a page of arithmetic later, so its latency stays off the warp's path
  };
  auto open_unit = [&](Cursor& c) -> bool {  // (c.row, c.blk) -> the next unit with tokens, or false
    for (;;) {
      if (c.blk >= g.max_blocks) {
        c.row += c.blk / g.max_blocks;
        c.blk %= g.max_blocks;
      }
      if (c.row >= n_rows) return false;
      c.seq = c.row / g.n_kv_heads;
      c.head = c.row - c.seq * g.n_kv_heads;
      const int prefix = min(prefix_lens[c.seq], cap);
      const int nb = min((prefix + g.block_size - 1) / g.block_size, g.max_blocks);
      const int lo = first_blocks != nullptr ? max(first_blocks[c.seq], 0) : 0;
      if (c.blk >= nb) {  // nothing more in this row: the first of this warp's units in a later row
        c.blk += (g.max_blocks - c.blk + stride - 1) / stride * stride;
        continue;
      }
      if (c.blk < lo) {   // summaries below lo are kept: the first of this warp's units at or past it
        c.blk += (lo - c.blk + stride - 1) / stride * stride;
        continue;
      }
      c.first = c.blk * g.block_size;
      c.count = min(g.block_size, prefix - c.first);
      c.n_pages = (c.count + kPage - 1) / kPage;
      c.page = 0;
      return true;
    }
  };
  auto fetch_table = [&](Cursor& c) {
    c.page_id = lane < c.n_pages ? block_table[(int64_t)c.seq * g.max_pages + c.first / kPage + lane] : -1;
  };
  auto next_page = [&](Cursor& c, bool issuing) -> bool {  // advance by one page
    if (++c.page < c.n_pages) return true;
    c.blk += stride;
    const bool ok = open_unit(c);
    if (ok && issuing) fetch_table(c);
    return ok;
  };
  auto issue = [&](const Cursor& c, int stage) {  // every lane computes, lane 0 copies
    const int page = __shfl_sync(0xffffffffu, c.page_id, c.page);
    const bool ok = page >= 0 && (g.n_pool_pages <= 0 || page < g.n_pool_pages);
    if (lane == 0) {
      live[stage] = ok ? 1 : 0;
      if (ok) {
        const int64_t at = (int64_t)page * g.pool_page_stride + (int64_t)c.head * g.pool_head_stride;
        T* dst = ring + (size_t)stage * 2 * kRun;
        ring_expect(&full[stage], 2 * kRunBytes);
        ring_copy(dst, k_pool + at, kRunBytes, &full[stage]);
        ring_copy(dst + kRun, v_pool + at, kRunBytes, &full[stage]);
      } else {
        atomicOr(status, DEV_STATUS_BAD_INDEX);  // never dereferenced: the page's tokens are left out
        ring_arrive(&full[stage]);
      }
    }
  };

  Cursor ic{};
  ic.blk = (int)blockIdx.x * kStreamWarps + warp;
  bool more = open_unit(ic);
  if (more) fetch_table(ic);
  for (int s = 0; s < n_stages && more; ++s) {
    issue(ic, s);
    more = next_page(ic, true);
  }
  Cursor cc{};
  cc.blk = (int)blockIdx.x * kStreamWarps + warp;
  bool alive = true;
  uint32_t n_done = 0;  // pages consumed so far: page n sits in stage n % n_stages, use n / n_stages
  for (bool have = open_unit(cc); have;) {
    float ksum[VEC], vsum[VEC], kmax[VEC], kmin[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) { ksum[i] = 0.f; vsum[i] = 0.f; kmax[i] = -INFINITY; kmin[i] = INFINITY; }
    float vn2max = 0.f;
    const int64_t unit = (int64_t)cc.row * g.max_blocks + cc.blk;
    const int count = cc.count, first = cc.first, seq = cc.seq, head = cc.head, n_pages = cc.n_pages;
    for (int pg = 0; pg < n_pages; ++pg) {
      const int stage = (int)(n_done % (uint32_t)n_stages);
      if (alive && !ring_wait(&full[stage], (n_done / (uint32_t)n_stages) & 1u)) {
        alive = false;
        if (lane == 0) atomicOr(status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
      }
      const T* kt = ring + (size_t)stage * 2 * kRun + lane * VEC;
      const T* vt = kt + kRun;
      const int rows = live[stage] ? min(kPage, count - pg * kPage) : 0;
      // tokens in ascending order: the fp32 sums are accumulated in token order
      float sq[kPage];  // this lane's share of |v_t|^2, one per token of the page
#pragma unroll
      for (int t = 0; t < kPage; ++t) {
        sq[t] = 0.f;
        if (t < rows) {
          float kv[VEC], vv[VEC];
          load_vec<VEC>(kt + t * D, kv);
          load_vec<VEC>(vt + t * D, vv);
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            ksum[i] += kv[i];
            vsum[i] += vv[i];
            kmax[i] = fmaxf(kmax[i], kv[i]);
            kmin[i] = fminf(kmin[i], kv[i]);
            sq[t] = fmaf(vv[i], vv[i], sq[t]);
          }
        }
      }
      // The sixteen sums over the 32 lanes at once: at every halving step a lane passes on the half of its
      // values that its partner keeps - 8 + 4 + 2 + 1 + 1 shuffles for the page instead of 5 per token.
      // Every lane ends up with the complete |v_t|^2 of one token (each token in two lanes).
#pragma unroll
      for (int n = kPage / 2, x = 16; n >= 1; n >>= 1, x >>= 1) {
        const bool upper = (lane & x) != 0;
#pragma unroll
        for (int i = 0; i < n; ++i) {
          const float keep = upper ? sq[i + n] : sq[i];
          const float give = upper ? sq[i] : sq[i + n];
          sq[i] = keep + __shfl_xor_sync(0xffffffffu, give, x);
        }
      }
      sq[0] += __shfl_xor_sync(0xffffffffu, sq[0], 1);
      vn2max = fmaxf(vn2max, sq[0]);  // per lane; the warp's maximum is taken once per block
      __syncwarp();  // every lane has read the stage: it may be refilled
      if (more) {
        issue(ic, stage);
        more = next_page(ic, true);
      }
      ++n_done;
    }
    cc.page = n_pages - 1;  // the unit is done: on to this warp's next one
    have = next_page(cc, false);

    const float denom = (float)count;
    const int64_t row = unit * D + lane * VEC;
    float kb[VEC], vb[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      kb[i] = ksum[i] / denom;
      vb[i] = vsum[i] / denom;
    }
    if (g.reserved & IA_GEOM_KBAR_BF16)  // the reference's bf16 k_bar option: the fp32 mean, rounded once
      store_vec<VEC>(reinterpret_cast<__nv_bfloat16*>(out.k_bar) + row, kb);
    else
      store_vec<VEC>(out.k_bar + row, kb);
    store_vec<VEC>(reinterpret_cast<T*>(out.v_bar) + row, vb);
    store_bounds<T, VEC>(g, out, row, kmax, kmin);
    vn2max = warp_max(vn2max);
    if (lane == 0) out.v_norm_max[unit] = sqrtf(vn2max);
    if (out.w == nullptr || out.rho == nullptr) continue;

    // The diagonal-ellipsoid pair as in the kernel above: a second walk over the block's keys, straight
    // from L2 (the ring has moved on).
    float kc[VEC], inv_w2[VEC], wv[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      kc[i] = kb[i];
      if (g.reserved & IA_GEOM_KBAR_BF16) kc[i] = __bfloat162float(__float2bfloat16_rn(kb[i]));
      float wi = fmaxf(fmaxf(kmax[i] - kc[i], kc[i] - kmin[i]), 1e-6f);
      if (sizeof(T) == 2) wi = __bfloat162float(__float2bfloat16_rn(wi * (1.f + 0.0078125f)));
      wv[i] = wi;
      inv_w2[i] = 1.f / (wi * wi);
    }
    store_vec<VEC>(reinterpret_cast<T*>(out.w) + row, wv);
    float d2max = 0.f;
    const int32_t* table = block_table + (int64_t)seq * g.max_pages;
    const int64_t head_off = (int64_t)head * g.pool_head_stride + lane * VEC;
    for (int pg = 0; pg < n_pages; ++pg) {
      const int page = table[first / kPage + pg];
      if (page < 0 || (g.n_pool_pages > 0 && page >= g.n_pool_pages)) continue;
      const int64_t base = (int64_t)page * g.pool_page_stride + head_off;
      const int rows = min(kPage, count - pg * kPage);
#pragma unroll 4
      for (int t = 0; t < rows; ++t) {
        float kv[VEC];
        load_vec<VEC>(k_pool + base + (int64_t)t * D, kv);
        float sq = 0.f;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          const float c = kv[i] - kc[i];
          sq = fmaf(c * c, inv_w2[i], sq);
        }
        d2max = fmaxf(d2max, warp_sum(sq));
      }
    }
    if (lane == 0) out.rho[unit] = sqrtf(d2max);
  }
}

template <typename T, int D>
static int launch_typed(const void* k_pool, const void* v_pool, const int32_t* block_table,
                        const int32_t* prefix_lens, const int32_t* first_blocks, const ia_geom& g,
                        const ia_summaries& out, cudaStream_t stream) {
  // read on every call (once per prompt): A/B runs and tests switch forms inside one process
  const char* form = getenv("INTERATTN_B200_SUMMARIES");
  const bool direct = form != nullptr && strcmp(form, "direct") == 0;
  // The diagonal-ellipsoid pair needs the block's keys a second time, after the mean is known; the ring has
  // moved on by then, and 14 warps re-reading them from L2 are slower than the direct kernel's 40 (measured
  // 884 vs 703 us at the 32k geometry): builds that keep the pair take the direct kernel.
  if (direct || g.page_size != 16 || (out.w != nullptr && out.rho != nullptr))
    return launch_direct<T, D>(k_pool, v_pool, block_table, prefix_lens, first_blocks, g, out, stream);
  const int64_t n_units = (int64_t)g.batch * g.n_kv_heads * g.max_blocks;
  if (n_units <= 0) return IA_OK;
  int dev = 0, sms = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (sms <= 0) sms = 148;
  if (max_smem <= 0) max_smem = 227 * 1024;
  // One CTA per SM.  The per-token arithmetic (about thirty instructions per warp and token) needs a dozen
  // warps per SM to hide its latencies, so the shared memory goes to as many warps as it holds with a
  // double-buffered ring each (2 x 8 KB at head_dim 128 bf16: 14 warps, 112 KB of copies in flight per SM);
  // with four warps and seven stages each the same kernel ran at 2.7 TB/s.
  const size_t stage_bytes = 2 * 16 * (size_t)D * sizeof(T);
  const size_t per_warp_fixed = 16 * 8 + 16 * 4;
  int stages = 2;
  int warps = (int)((size_t)max_smem / (stages * stage_bytes + per_warp_fixed));
  if (warps > kMaxStreamWarps) {
    warps = kMaxStreamWarps;
    stages = (int)(((size_t)max_smem / warps - per_warp_fixed) / stage_bytes);
    if (stages > 16) stages = 16;
  }
  if (warps < 4) return launch_direct<T, D>(k_pool, v_pool, block_table, prefix_lens, first_blocks, g, out, stream);
  const int kStreamWarps = warps;
  const size_t fixed = (size_t)warps * per_warp_fixed;
  const size_t smem = fixed + (size_t)warps * stages * stage_bytes;
  int* status = device_status_address();
  if (status == nullptr) return IA_ERR_LAUNCH;
  auto kern = condition_block_build_summaries_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "build_summaries: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  const int64_t want = (n_units + kStreamWarps - 1) / kStreamWarps;
  const unsigned grid = (unsigned)(want < sms ? want : sms);
  kern<<<grid, kStreamWarps * 32, smem, stream>>>(static_cast<const T*>(k_pool), static_cast<const T*>(v_pool),
                                                   block_table, prefix_lens, first_blocks, g, out, stages, status);
  return check_launch("condition_block_build_summaries_kernel");
}

int launch_build_summaries(const void* k_pool, const void* v_pool, const int32_t* block_table,
                           const int32_t* prefix_lens, const int32_t* first_blocks, const ia_geom& g,
                           const ia_summaries& out, cudaStream_t stream) {
  if (g.dtype == IA_BF16) {
    if (g.head_dim == 128)
      return launch_typed<__nv_bfloat16, 128>(k_pool, v_pool, block_table, prefix_lens, first_blocks, g, out, stream);
    if (g.head_dim == 64)
      return launch_typed<__nv_bfloat16, 64>(k_pool, v_pool, block_table, prefix_lens, first_blocks, g, out, stream);
  } else if (g.dtype == IA_F32) {
    if (g.head_dim == 128)
      return launch_typed<float, 128>(k_pool, v_pool, block_table, prefix_lens, first_blocks, g, out, stream);
    if (g.head_dim == 64)
      return launch_typed<float, 64>(k_pool, v_pool, block_table, prefix_lens, first_blocks, g, out, stream);
  }
  return fail(IA_ERR_UNSUPPORTED, "build_summaries: head_dim %d / dtype %d not built", g.head_dim, g.dtype);
}

}  // namespace ia
