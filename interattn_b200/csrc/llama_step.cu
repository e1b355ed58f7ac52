// The element-wise part of one batched Llama decode step around the sparse
// attention layer-step: residual add + RMSNorm, rotary embedding fused with the
// KV-cache append, SiLU(gate) * up, and the greedy arg-max over the vocabulary.
//
// In the reference these run as the Hugging Face model's own PyTorch ops inside
// the captured decode step (condition_block_triton_impl/core.py:190-316): about
// forty small kernels per layer.  Here each group is one launch.  Every kernel
// reproduces the bf16 rounding points of the PyTorch expression it replaces
// (transformers/models/llama/modeling_llama.py: LlamaRMSNorm.forward,
// apply_rotary_pos_emb, LlamaMLP.forward), so the fused step and the module-by-module
// step agree to the last bit except for the order of the fp32 sum of squares.
//
// All tensors are bf16, rows are contiguous.
#include "ia_common.cuh"

namespace ia {
namespace {

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// 8 bf16 values <-> 8 floats through one 16-byte access
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 w = *reinterpret_cast<const uint4*>(p);
  v[0] = bf16lo(w.x); v[1] = bf16hi(w.x); v[2] = bf16lo(w.y); v[3] = bf16hi(w.y);
  v[4] = bf16lo(w.z); v[5] = bf16hi(w.z); v[6] = bf16lo(w.w); v[7] = bf16hi(w.w);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 w;
  w.x = pack2(v[0], v[1]); w.y = pack2(v[2], v[3]); w.z = pack2(v[4], v[5]); w.w = pack2(v[6], v[7]);
  *reinterpret_cast<uint4*>(p) = w;
}

// ---- residual add + RMSNorm ------------------------------------------------------
// x = residual (+ delta, rounded to bf16 and written back); out = weight * bf16(x * rsqrt(mean(x^2) + eps)).
// One CTA per row; kChunks * 8 * blockDim >= hidden, the row stays in registers.
constexpr int kNormThreads = 256;
template <int kChunks>
__global__ void __launch_bounds__(kNormThreads)
llama_add_rmsnorm_kernel(__nv_bfloat16* __restrict__ residual, const __nv_bfloat16* __restrict__ delta,
                         const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out, int hidden,
                         float eps) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int64_t row = (int64_t)blockIdx.x * hidden;
  float x[kChunks][8];
  float sq = 0.f;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int i = (c * kNormThreads + threadIdx.x) * 8;
    if (i < hidden) {
      load8(residual + row + i, x[c]);
      if (delta != nullptr) {
        float d[8];
        load8(delta + row + i, d);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[c][j] = round_bf16(x[c][j] + d[j]);
        store8(residual + row + i, x[c]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sq = fmaf(x[c][j], x[c][j], sq);
    }
  }
  __shared__ float part[kNormThreads / 32];
  __shared__ float scale_s;
  sq = warp_sum(sq);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < kNormThreads / 32 ? part[threadIdx.x] : 0.f;
    v = warp_sum(v);
    if (threadIdx.x == 0) scale_s = rsqrtf(v / (float)hidden + eps);
  }
  __syncthreads();
  const float scale = scale_s;
#pragma unroll
  for (int c = 0; c < kChunks; ++c) {
    const int i = (c * kNormThreads + threadIdx.x) * 8;
    if (i < hidden) {
      float w[8], y[8];
      load8(weight + i, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = w[j] * round_bf16(x[c][j] * scale);
      store8(out + row + i, y);
    }
  }
}

// ---- rotary embedding + cache append ---------------------------------------------
// qkv row of a sequence: [Hq * D | Hkv * D | Hkv * D].  One CTA per (sequence, head of
// the fused row), D / 2 threads; thread d owns the pair (d, d + D/2):
//   out[d]       = bf16( bf16(x[d] * cos[d])             + bf16(-x[d + D/2] * sin[d]) )
//   out[d + D/2] = bf16( bf16(x[d + D/2] * cos[d + D/2]) + bf16( x[d]       * sin[d + D/2]) )
// q goes to q_out [B, Hq, D]; k (rotated) and v (as is) go to the cache row of position
// seq_lens[b] - 1.  A position outside [0, max_pos) or the cache leaves the row untouched.
__global__ void llama_rope_append_kernel(const __nv_bfloat16* __restrict__ qkv, const __nv_bfloat16* __restrict__ cos_t,
                                         const __nv_bfloat16* __restrict__ sin_t, int max_pos,
                                         const int32_t* __restrict__ seq_lens, __nv_bfloat16* __restrict__ k_cache,
                                         __nv_bfloat16* __restrict__ v_cache, int64_t seq_stride, int64_t head_stride,
                                         int cache_len, __nv_bfloat16* __restrict__ q_out, int n_q_heads,
                                         int n_kv_heads, int D) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int b = blockIdx.x, head = blockIdx.y, d = threadIdx.x, half = D >> 1;
  const int pos = seq_lens[b] - 1;
  if (pos < 0 || pos >= max_pos || pos >= cache_len) return;
  const int row_elems = (n_q_heads + 2 * n_kv_heads) * D;
  const __nv_bfloat16* src = qkv + (int64_t)b * row_elems + (int64_t)head * D;
  if (head >= n_q_heads + n_kv_heads) {  // value head: plain copy
    const int h = head - n_q_heads - n_kv_heads;
    __nv_bfloat16* dst = v_cache + b * seq_stride + h * head_stride + (int64_t)pos * D;
    dst[d] = src[d];
    dst[d + half] = src[d + half];
    return;
  }
  const float x1 = __bfloat162float(src[d]), x2 = __bfloat162float(src[d + half]);
  const __nv_bfloat16* c = cos_t + (int64_t)pos * D;
  const __nv_bfloat16* s = sin_t + (int64_t)pos * D;
  const float lo = round_bf16(x1 * __bfloat162float(c[d])) + round_bf16(-x2 * __bfloat162float(s[d]));
  const float hi = round_bf16(x2 * __bfloat162float(c[d + half])) + round_bf16(x1 * __bfloat162float(s[d + half]));
  __nv_bfloat16* dst = head < n_q_heads
                           ? q_out + ((int64_t)b * n_q_heads + head) * D
                           : k_cache + b * seq_stride + (head - n_q_heads) * head_stride + (int64_t)pos * D;
  dst[d] = __float2bfloat16_rn(lo);
  dst[d + half] = __float2bfloat16_rn(hi);
}

// ---- SiLU(gate) * up ----------------------------------------------------------------
// gate_up row: [I gate | I up]; out = bf16( bf16(g / (1 + exp(-g))) * u )
__global__ void llama_silu_mul_kernel(const __nv_bfloat16* __restrict__ gate_up, __nv_bfloat16* __restrict__ out,
                                      int n_rows, int inter) {
  grid_launch_dependents();
  grid_dependency_wait();
  const int per_row = inter >> 3;
  const int64_t unit = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (unit >= (int64_t)n_rows * per_row) return;
  const int64_t r = unit / per_row;
  const int i = (int)(unit - r * per_row) * 8;
  float g[8], u[8], y[8];
  load8(gate_up + r * 2 * inter + i, g);
  load8(gate_up + r * 2 * inter + inter + i, u);
#pragma unroll
  for (int j = 0; j < 8; ++j) y[j] = round_bf16(g[j] / (1.f + expf(-g[j]))) * u[j];
  store8(out + r * inter + i, y);
}

// ---- arg-max over the vocabulary --------------------------------------------------
// One CTA per row; the lowest index among equal maxima wins.  NaN never wins.
constexpr int kArgmaxThreads = 1024;
__global__ void __launch_bounds__(kArgmaxThreads)
llama_argmax_kernel(const __nv_bfloat16* __restrict__ logits, int64_t row_stride, int vocab,
                    int64_t* __restrict__ out) {
  grid_launch_dependents();
  grid_dependency_wait();
  const __nv_bfloat16* row = logits + (int64_t)blockIdx.x * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  const int vec_end = ((reinterpret_cast<uintptr_t>(row) & 15u) == 0) ? (vocab & ~7) : 0;
  for (int i = threadIdx.x * 8; i < vec_end; i += kArgmaxThreads * 8) {
    float v[8];
    load8(row + i, v);
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (v[j] > best) { best = v[j]; best_i = i + j; }  // ascending i: the first maximum stays
  }
  for (int i = vec_end + threadIdx.x; i < vocab; i += kArgmaxThreads) {
    const float v = __bfloat162float(row[i]);
    if (v > best || (v == best && i < best_i)) { best = v; best_i = i; }
  }
  __shared__ float best_s[kArgmaxThreads / 32];
  __shared__ int idx_s[kArgmaxThreads / 32];
  auto merge = [](float& a, int& ai, float b, int bi) {
    if (b > a || (b == a && bi < ai)) { a = b; ai = bi; }
  };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1)
    merge(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
  if ((threadIdx.x & 31) == 0) { best_s[threadIdx.x >> 5] = best; idx_s[threadIdx.x >> 5] = best_i; }
  __syncthreads();
  if (threadIdx.x < 32) {
    best = best_s[threadIdx.x];
    best_i = idx_s[threadIdx.x];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
      merge(best, best_i, __shfl_xor_sync(0xffffffffu, best, o), __shfl_xor_sync(0xffffffffu, best_i, o));
    if (threadIdx.x == 0) out[blockIdx.x] = best_i == 0x7fffffff ? 0 : best_i;
  }
}

template <typename Kern, typename... Args>
int launch(const char* what, Kern kern, dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  int n = 0;
  if (overlapped_launch_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)n;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, args...);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return check_launch(what);
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace
}  // namespace ia

using namespace ia;

extern "C" {

int ia_llama_add_rmsnorm(void* residual, const void* delta, const void* weight, void* out, int n_rows, int hidden,
                         float eps, ia_stream_t stream) {
  if (!residual || !weight || !out) return fail(IA_ERR_BAD_ARG, "add_rmsnorm: null pointer");
  if (n_rows < 0 || hidden <= 0 || hidden % 8 != 0)
    return fail(IA_ERR_BAD_ARG, "add_rmsnorm: %d rows of %d (a multiple of 8)", n_rows, hidden);
  if (!aligned16(residual) || !aligned16(weight) || !aligned16(out) || (delta && !aligned16(delta)))
    return fail(IA_ERR_BAD_ARG, "add_rmsnorm: pointers must be 16-byte aligned");
  if (n_rows == 0) return IA_OK;
  auto* r = static_cast<__nv_bfloat16*>(residual);
  auto* d = static_cast<const __nv_bfloat16*>(delta);
  auto* w = static_cast<const __nv_bfloat16*>(weight);
  auto* o = static_cast<__nv_bfloat16*>(out);
  const int chunks = (hidden + kNormThreads * 8 - 1) / (kNormThreads * 8);
  const dim3 grid((unsigned)n_rows), block(kNormThreads);
  cudaStream_t st = (cudaStream_t)stream;
  switch (chunks) {
    case 1: return launch("llama_add_rmsnorm_kernel", llama_add_rmsnorm_kernel<1>, grid, block, st, r, d, w, o, hidden, eps);
    case 2: return launch("llama_add_rmsnorm_kernel", llama_add_rmsnorm_kernel<2>, grid, block, st, r, d, w, o, hidden, eps);
    case 3:
    case 4: return launch("llama_add_rmsnorm_kernel", llama_add_rmsnorm_kernel<4>, grid, block, st, r, d, w, o, hidden, eps);
    case 5: case 6: case 7:
    case 8: return launch("llama_add_rmsnorm_kernel", llama_add_rmsnorm_kernel<8>, grid, block, st, r, d, w, o, hidden, eps);
    default: return fail(IA_ERR_UNSUPPORTED, "add_rmsnorm: hidden size %d above %d", hidden, kNormThreads * 64);
  }
}

int ia_llama_rope_append(const void* qkv, const void* cos_table, const void* sin_table, int max_pos,
                         const int32_t* seq_lens, void* k_cache, void* v_cache, int64_t cache_seq_stride,
                         int64_t cache_head_stride, int cache_len, void* q_out, int batch, int n_q_heads,
                         int n_kv_heads, int head_dim, ia_stream_t stream) {
  if (!qkv || !cos_table || !sin_table || !seq_lens || !k_cache || !v_cache || !q_out)
    return fail(IA_ERR_BAD_ARG, "rope_append: null pointer");
  if (batch < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || max_pos <= 0 || cache_len <= 0)
    return fail(IA_ERR_BAD_ARG, "rope_append: batch %d, heads %d/%d, %d positions, cache of %d", batch, n_q_heads,
                n_kv_heads, max_pos, cache_len);
  if (head_dim <= 0 || head_dim % 2 != 0 || head_dim > 2048)
    return fail(IA_ERR_UNSUPPORTED, "rope_append: head_dim %d (even, at most 2048)", head_dim);
  if (cache_head_stride < (int64_t)cache_len * head_dim)
    return fail(IA_ERR_BAD_ARG, "rope_append: head stride %lld below %d rows of %d", (long long)cache_head_stride,
                cache_len, head_dim);
  if (batch == 0) return IA_OK;
  const dim3 grid((unsigned)batch, (unsigned)(n_q_heads + 2 * n_kv_heads)), block((unsigned)(head_dim / 2));
  return launch("llama_rope_append_kernel", llama_rope_append_kernel, grid, block, (cudaStream_t)stream,
                static_cast<const __nv_bfloat16*>(qkv), static_cast<const __nv_bfloat16*>(cos_table),
                static_cast<const __nv_bfloat16*>(sin_table), max_pos, seq_lens, static_cast<__nv_bfloat16*>(k_cache),
                static_cast<__nv_bfloat16*>(v_cache), cache_seq_stride, cache_head_stride, cache_len,
                static_cast<__nv_bfloat16*>(q_out), n_q_heads, n_kv_heads, head_dim);
}

int ia_llama_silu_mul(const void* gate_up, void* out, int n_rows, int intermediate, ia_stream_t stream) {
  if (!gate_up || !out) return fail(IA_ERR_BAD_ARG, "silu_mul: null pointer");
  if (n_rows < 0 || intermediate <= 0 || intermediate % 8 != 0)
    return fail(IA_ERR_BAD_ARG, "silu_mul: %d rows of %d (a multiple of 8)", n_rows, intermediate);
  if (!aligned16(gate_up) || !aligned16(out)) return fail(IA_ERR_BAD_ARG, "silu_mul: pointers must be 16-byte aligned");
  if (n_rows == 0) return IA_OK;
  const int64_t units = (int64_t)n_rows * (intermediate / 8);
  const dim3 grid((unsigned)ceil_div64(units, 256)), block(256);
  return launch("llama_silu_mul_kernel", llama_silu_mul_kernel, grid, block, (cudaStream_t)stream,
                static_cast<const __nv_bfloat16*>(gate_up), static_cast<__nv_bfloat16*>(out), n_rows, intermediate);
}

int ia_llama_argmax(const void* logits, int64_t row_stride, int n_rows, int vocab, int64_t* out, ia_stream_t stream) {
  if (!logits || !out) return fail(IA_ERR_BAD_ARG, "argmax: null pointer");
  if (n_rows < 0 || vocab <= 0 || row_stride < vocab)
    return fail(IA_ERR_BAD_ARG, "argmax: %d rows of %d, row stride %lld", n_rows, vocab, (long long)row_stride);
  if (n_rows == 0) return IA_OK;
  // rows that start off a 16-byte boundary take the scalar loop
  const dim3 grid((unsigned)n_rows), block(kArgmaxThreads);
  return launch("llama_argmax_kernel", llama_argmax_kernel, grid, block, (cudaStream_t)stream,
                static_cast<const __nv_bfloat16*>(logits), row_stride, vocab, out);
}

}  // extern "C"
