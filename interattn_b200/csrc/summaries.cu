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
#include "ia_common.cuh"

namespace ia {

template <typename T, int D>
__global__ void __launch_bounds__(128)
condition_block_build_summaries_kernel(const T* __restrict__ k_pool, const T* __restrict__ v_pool,
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
  store_vec<VEC>(reinterpret_cast<T*>(out.k_max) + row, kmax);
  store_vec<VEC>(reinterpret_cast<T*>(out.k_min) + row, kmin);
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
static int launch_typed(const void* k_pool, const void* v_pool, const int32_t* block_table,
                        const int32_t* prefix_lens, const int32_t* first_blocks, const ia_geom& g,
                        const ia_summaries& out, cudaStream_t stream) {
  const int64_t n_units = (int64_t)g.batch * g.n_kv_heads * g.max_blocks;
  const int warps = 4;
  const int64_t grid = ceil_div64(n_units, warps);
  if (grid <= 0) return IA_OK;
  if (grid > 0x7fffffff) return fail(IA_ERR_UNSUPPORTED, "build_summaries: grid too large");
  condition_block_build_summaries_kernel<T, D><<<(unsigned)grid, warps * 32, 0, stream>>>(
      static_cast<const T*>(k_pool), static_cast<const T*>(v_pool), block_table, prefix_lens, first_blocks, g, out);
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
