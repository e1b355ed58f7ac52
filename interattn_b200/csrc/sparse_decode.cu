// Paged sparse / hybrid decode attention - portable fp32-FMA kernel.
//
// Attention half of the reference's fused finalize kernel
// (llama/script/analysis/condition_block_gen/methods/condition_block_triton_impl/page_attention.py:173-309):
// a joint online softmax over the tokens of the selected blocks, the
// representatives (z, v_bar) of the unselected blocks (hybrid mode) and the
// generated suffix, for the G query rows that share one kv head.  This
// translation unit holds the all-fp32 CUDA-core version: it serves fp32 KV
// pools (1e-5 parity against the fp32 reference) and any geometry the
// tensor-core kernel is not built for.  One warp walks whole pages, lanes
// split head_dim, dot products are reduced with shuffles.
#include "decode_items.cuh"

namespace ia {

int launch_sparse_decode_mma(const DecodeParams& p, const ia_geom& g, bool flat, cudaStream_t stream);  // bf16 tensor-core path

namespace {

constexpr int kWarps = 4;

template <typename T, int D, int G>
__global__ void __launch_bounds__(kWarps * 32)
condition_block_finalize_attention_fma_kernel(DecodeParams p) {
  constexpr int VEC = D / 32;
  __shared__ Item items_s[kItemChunk];
  __shared__ int scratch[2];
  __shared__ float merge_m[kWarps][G], merge_l[kWarps][G];
  __shared__ float merge_o[kWarps][G][D];
  extern __shared__ uint32_t sel_bits[];  // hybrid: one bit per block

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int split = blockIdx.x % p.n_splits;
  const int pair = blockIdx.x / p.n_splits;
  const int head = pair % p.n_kv_heads, seq = pair / p.n_kv_heads;
  const int rows = p.n_kv_heads * G;

  ExchangeView xv{};
  if (p.px.n_ranks > 0) xv = exchange_view(p);
  const ItemRange r = item_range(p, seq, head, split, scratch);
  if (p.rep_mode == IA_REP_HYBRID) {
    const int words = (p.max_blocks + 31) / 32;
    for (int i = threadIdx.x; i < words; i += blockDim.x) sel_bits[i] = 0u;
    __syncthreads();
    const int count = min(p.sel_count[pair], p.max_sel);
    const int32_t* idx = p.sel_idx + (int64_t)pair * p.max_sel;
    for (int i = threadIdx.x; i < count; i += blockDim.x) {
      const int b = idx[i];
      if (b >= 0 && b < p.max_blocks) atomicOr(&sel_bits[b >> 5], 1u << (b & 31));
    }
    __syncthreads();
  }

  float q[G][VEC], acc[G][VEC], m[G], l[G];
  const T* qp = static_cast<const T*>(p.q) + ((int64_t)seq * rows + head * G) * D + lane * VEC;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    load_vec<VEC>(qp + g * D, q[g]);
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[g][i] = 0.f;
  }
  const float root = sqrtf((float)D);
  const T* kp = static_cast<const T*>(p.k_pool) + (int64_t)head * p.head_stride + lane * VEC;
  const T* vp = static_cast<const T*>(p.v_pool) + (int64_t)head * p.head_stride + lane * VEC;
  const T* vbar = static_cast<const T*>(p.v_bar) + ((int64_t)pair * p.max_blocks) * D + lane * VEC;
  const float* zrow = p.z + ((int64_t)seq * rows + head * G) * p.max_blocks;

  auto absorb = [&](const float (&logit)[G], const float (&v)[VEC]) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float top = fmaxf(m[g], logit[g]);
      const float a = expf(m[g] - top);  // m = -inf on first use: exp(-inf) = 0
      const float w = expf(logit[g] - top);
      l[g] = l[g] * a + w;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[g][i] = fmaf(acc[g][i], a, w * v[i]);
      m[g] = top;
    }
  };

  for (int chunk = r.begin; chunk < r.end; chunk += kItemChunk) {
    const int chunk_end = min(chunk + kItemChunk, r.end);
    __syncthreads();  // previous chunk fully consumed
    resolve_items(p, r, seq, head, chunk, chunk_end, items_s);
    for (int i = chunk + warp; i < chunk_end; i += kWarps) {
      const Item it = items_s[i - chunk];
      if (it.kind == ITEM_PAGE) {
        const int64_t base = (int64_t)it.first * p.page_stride;
        for (int t = it.lo; t < it.hi; ++t) {
          float kv[VEC], vv[VEC], logit[G];
          load_vec<VEC>(kp + base + (int64_t)t * D, kv);
          load_vec<VEC>(vp + base + (int64_t)t * D, vv);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            float part = 0.f;
#pragma unroll
            for (int j = 0; j < VEC; ++j) part = fmaf(q[g][j], kv[j], part);
            logit[g] = warp_sum(part) / root;
          }
          absorb(logit, vv);
        }
      } else {
        for (int t = it.lo; t < it.hi; ++t) {
          const int b = it.first + t;
          if ((sel_bits[b >> 5] >> (b & 31)) & 1u) continue;  // selected: its tokens are attended exactly
          float vv[VEC], logit[G];
          load_vec<VEC>(vbar + (int64_t)b * D, vv);
#pragma unroll
          for (int g = 0; g < G; ++g) logit[g] = zrow[(int64_t)g * p.max_blocks + b];
          absorb(logit, vv);
        }
      }
    }
  }

  // ---- merge the four warps, emit (o, lse) ------------------------------------
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) { merge_m[warp][g] = m[g]; merge_l[warp][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < VEC; ++i) merge_o[warp][g][lane * VEC + i] = acc[g][i];
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
    const int g = e / D, d = e - g * D;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) top = fmaxf(top, merge_m[w][g]);
    float num = 0.f, den = 0.f;
    if (top > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float a = expf(merge_m[w][g] - top);
        num = fmaf(a, merge_o[w][g][d], num);
        den = fmaf(a, merge_l[w][g], den);
      }
    }
    const int64_t orow = ((int64_t)seq * rows + head * G + g) * p.n_splits + split;
    const float ov = den > 0.f ? num / den : 0.f;
    const float lv = den > 0.f ? top + logf(den) : -INFINITY;
    if (p.px.n_ranks > 0) {
      exchange_store(p, xv, orow * D + d, ov);
      if (d == 0) exchange_store(p, xv, p.px.lse_offset + orow, lv);
    } else {
      p.o_partial[orow * D + d] = ov;
      if (d == 0) p.lse_partial[orow] = lv;
    }
  }
  if (p.px.n_ranks > 0) {
    exchange_publish(p, xv);
    return;
  }
  finish_pair<D>(p, seq, head, G, scratch);
}

template <typename T, int D, int G>
int launch_fma(const DecodeParams& p, const ia_geom& g, cudaStream_t stream) {
  const int64_t grid = (int64_t)g.batch * g.n_kv_heads * p.n_splits;
  if (grid <= 0) return IA_OK;
  const size_t dyn = p.rep_mode == IA_REP_HYBRID ? (size_t)((g.max_blocks + 31) / 32) * 4 : 0;
  condition_block_finalize_attention_fma_kernel<T, D, G><<<(unsigned)grid, kWarps * 32, dyn, stream>>>(p);
  return check_launch("condition_block_finalize_attention_fma_kernel");
}

template <typename T, int D>
int launch_fma_group(const DecodeParams& p, const ia_geom& g, cudaStream_t stream) {
  switch (g.group_size) {
    case 1: return launch_fma<T, D, 1>(p, g, stream);
    case 2: return launch_fma<T, D, 2>(p, g, stream);
    case 4: return launch_fma<T, D, 4>(p, g, stream);
    case 8: return launch_fma<T, D, 8>(p, g, stream);
    default: return fail(IA_ERR_UNSUPPORTED, "sparse_decode (fma): group_size %d not built (1, 2, 4, 8)", g.group_size);
  }
}

}  // namespace

int launch_sparse_decode(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_table, const int32_t* prefix_lens,
                         const int32_t* seq_lens, const int32_t* sel_idx, const int32_t* sel_count,
                         int max_sel, const ia_summaries* summaries, const float* z, const ia_geom& g,
                         int rep_mode, int n_splits, int block_lo, int block_hi, int with_suffix,
                         float* o_partial, float* lse_partial, const FusedFinalize* fused, cudaStream_t stream,
                         const ia_peer_exchange* exchange) {
  DecodeParams p{};
  if (exchange != nullptr) p.px = *exchange;
  if (fused != nullptr) {
    p.final_out = fused->out;
    p.split_counters = fused->split_counters;
    p.final_dtype = fused->out_dtype;
    p.flat_o = fused->flat_o;
    p.flat_lse = fused->flat_lse;
  }
  p.n_pool_pages = g.n_pool_pages;
  p.status = device_status_address();
  p.n_pairs = g.batch * g.n_kv_heads;
#ifdef IA_DECODE_TRACE
  p.trace = getenv("IA_TRACE_PTR") ? reinterpret_cast<float*>(strtoull(getenv("IA_TRACE_PTR"), nullptr, 16)) : nullptr;
#endif
  p.q = q; p.k_pool = k_pool; p.v_pool = v_pool; p.block_table = block_table;
  p.prefix_lens = prefix_lens; p.seq_lens = seq_lens; p.sel_idx = sel_idx; p.sel_count = sel_count;
  p.v_bar = summaries ? summaries->v_bar : nullptr;
  p.z = z;
  p.o_partial = o_partial; p.lse_partial = lse_partial;
  p.page_stride = g.pool_page_stride; p.head_stride = g.pool_head_stride;
  p.n_kv_heads = g.n_kv_heads; p.group_size = g.group_size; p.page_size = g.page_size;
  p.block_size = g.block_size; p.max_pages = g.max_pages; p.max_blocks = g.max_blocks; p.max_sel = max_sel;
  p.rep_mode = rep_mode; p.n_splits = n_splits; p.block_lo = block_lo; p.block_hi = block_hi;
  p.with_suffix = with_suffix;

  const char* force = getenv("INTERATTN_B200_DECODE_KERNEL");  // "fma" pins the portable kernel (profiling aid)
  const bool want_fma = force != nullptr && force[0] == 'f';
  if (g.dtype == IA_BF16 && g.page_size == 16 && g.group_size <= 16 && !want_fma &&
      (g.head_dim == 128 || g.head_dim == 64)) {
    const bool flat = p.flat_o != nullptr &&
                      decode_flat_grid_applies(g, fused != nullptr, block_lo <= 0 && block_hi >= g.max_blocks,
                                               exchange != nullptr);
    return launch_sparse_decode_mma(p, g, flat, stream);
  }
  if (g.dtype == IA_BF16) {
    if (g.head_dim == 128) return launch_fma_group<__nv_bfloat16, 128>(p, g, stream);
    if (g.head_dim == 64) return launch_fma_group<__nv_bfloat16, 64>(p, g, stream);
  } else if (g.dtype == IA_F32) {
    if (g.head_dim == 128) return launch_fma_group<float, 128>(p, g, stream);
    if (g.head_dim == 64) return launch_fma_group<float, 64>(p, g, stream);
  }
  return fail(IA_ERR_UNSUPPORTED, "sparse_decode: head_dim %d / dtype %d not built", g.head_dim, g.dtype);
}

}  // namespace ia
