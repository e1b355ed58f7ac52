// Split-KV finalize: log-sum-exp merge of partial attention outputs.
//
// Same arithmetic as the reference's _condition_block_stage2_reduce_kernel
// (llama/script/analysis/condition_block_gen/methods/condition_block_triton_impl/legacy.py:765-794),
// written for normalised partials: with o_s = acc_s / l_s and
// lse_s = m_s + log l_s,  out = sum_s o_s e^{lse_s - M} / sum_s e^{lse_s - M},
// M = max_s lse_s.  A part with lse = -inf carries nothing; a row whose parts
// are all empty gives 0 (the reference clamps the denominator to 1e-30).
// One warp per output row; the partials are a few hundred bytes per row, so
// this kernel is launch-latency bound.
//
// The partials may come in n_groups chunks of the same shape, group_stride
// floats apart (one chunk per GPU after an all-gather of the split-KV
// partials): part (w, s) of a row is then chunk w's part s.
#include "ia_common.cuh"

namespace ia {

template <typename TOut, int D>
__global__ void __launch_bounds__(128)
condition_block_stage2_reduce_kernel(const float* __restrict__ o_partial,
                                     const float* __restrict__ lse_partial, int n_rows, int n_parts,
                                     int n_groups, int64_t group_stride, TOut* __restrict__ out,
                                     float* __restrict__ out_lse) {
  constexpr int VEC = D / 32;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const float* lse = lse_partial + (int64_t)row * n_parts;
  float top = -INFINITY;
  for (int w = 0; w < n_groups; ++w)
    for (int s = lane; s < n_parts; s += 32) top = fmaxf(top, lse[w * group_stride + s]);
  top = warp_max(top);
  const float ref = (top == -INFINITY) ? 0.f : top;

  float acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  float den = 0.f;
  const float* o = o_partial + (int64_t)row * n_parts * D + lane * VEC;
  for (int g = 0; g < n_groups; ++g)
    for (int s = 0; s < n_parts; ++s) {
      const float w = expf(lse[g * group_stride + s] - ref);  // exp(-inf) = 0 for an empty part
      float v[VEC];
      load_vec<VEC>(o + g * group_stride + (int64_t)s * D, v);
      den += w;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = fmaf(w, v[i], acc[i]);
    }
  const float inv = 1.f / fmaxf(den, 1e-30f);
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] *= inv;
  store_vec<VEC>(out + (int64_t)row * D + lane * VEC, acc);
  if (out_lse != nullptr && lane == 0) out_lse[row] = den > 0.f ? ref + logf(den) : -INFINITY;
}

// The merge of a split-KV step whose partials the ranks stored into this rank's gather buffer
// through peer pointers.  Each CTA first waits until the flag of every rank carries this step
// - polling its own memory, with a limit of about a second, after which it records the fact in
// the device status word and carries on - then merges the chunks with L2 loads (the lines may
// sit in L1 from the step two before).
constexpr uint32_t kPeerPolls = 1u << 20;
__device__ __forceinline__ int ld_acquire_sys(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
template <typename TOut, int D>
__global__ void __launch_bounds__(128)
condition_block_stage2_reduce_exchange_kernel(const ia_peer_exchange px, int n_rows, int n_parts,
                                              TOut* __restrict__ out, int* __restrict__ status) {
  constexpr int VEC = D / 32;
  const int step = *px.step_counter;  // set by this rank's attention kernel, which has completed
  const int parity = step & 1;
  if (threadIdx.x < px.n_ranks) {
    const int32_t* flag = px.flags[px.my_rank] + parity * px.n_ranks + threadIdx.x;
    bool arrived = false;
    for (uint32_t i = 0; i < kPeerPolls; ++i) {
      if (ld_acquire_sys(flag) >= step) {
        arrived = true;
        break;
      }
      __nanosleep(256);
    }
    if (!arrived) atomicOr(status, DEV_STATUS_PEER_WAIT_TIMEOUT);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const float* base = px.gather[px.my_rank] + (int64_t)parity * px.n_ranks * px.chunk_floats;
  const float* lse = base + px.lse_offset + (int64_t)row * n_parts;
  float top = -INFINITY;
  for (int w = 0; w < px.n_ranks; ++w)
    for (int s = lane; s < n_parts; s += 32) top = fmaxf(top, __ldcg(lse + w * px.chunk_floats + s));
  top = warp_max(top);
  const float ref = (top == -INFINITY) ? 0.f : top;
  float acc[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
  float den = 0.f;
  const float* o = base + (int64_t)row * n_parts * D + lane * VEC;
  for (int g = 0; g < px.n_ranks; ++g)
    for (int s = 0; s < n_parts; ++s) {
      const float w = expf(__ldcg(lse + g * px.chunk_floats + s) - ref);  // exp(-inf) = 0 for an empty part
      const float* src = o + g * px.chunk_floats + (int64_t)s * D;
      den += w;
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = fmaf(w, __ldcg(src + i), acc[i]);
    }
  const float inv = 1.f / fmaxf(den, 1e-30f);
#pragma unroll
  for (int i = 0; i < VEC; ++i) acc[i] *= inv;
  store_vec<VEC>(out + (int64_t)row * D + lane * VEC, acc);
}

template <typename TOut, int D>
static int launch_exchange_typed(const ia_peer_exchange& px, int n_rows, int n_parts, void* out, int* status,
                                 cudaStream_t stream) {
  const int warps = 4;
  const int grid = (n_rows + warps - 1) / warps;
  condition_block_stage2_reduce_exchange_kernel<TOut, D><<<grid, warps * 32, 0, stream>>>(
      px, n_rows, n_parts, static_cast<TOut*>(out), status);
  return check_launch("condition_block_stage2_reduce_exchange_kernel");
}

int launch_finalize_exchange(const ia_peer_exchange& px, int n_rows, int n_parts, int head_dim, void* out,
                             int out_dtype, int* status, cudaStream_t stream) {
  if (n_rows <= 0) return IA_OK;
  if (out_dtype == IA_BF16) {
    if (head_dim == 128) return launch_exchange_typed<__nv_bfloat16, 128>(px, n_rows, n_parts, out, status, stream);
    if (head_dim == 64) return launch_exchange_typed<__nv_bfloat16, 64>(px, n_rows, n_parts, out, status, stream);
  } else if (out_dtype == IA_F32) {
    if (head_dim == 128) return launch_exchange_typed<float, 128>(px, n_rows, n_parts, out, status, stream);
    if (head_dim == 64) return launch_exchange_typed<float, 64>(px, n_rows, n_parts, out, status, stream);
  }
  return fail(IA_ERR_UNSUPPORTED, "finalize: head_dim %d / out dtype %d not built", head_dim, out_dtype);
}

template <typename TOut, int D>
static int launch_typed(const float* o_partial, const float* lse_partial, int n_rows, int n_parts, int n_groups,
                        int64_t group_stride, void* out, float* out_lse, cudaStream_t stream) {
  const int warps = 4;
  const int grid = (n_rows + warps - 1) / warps;
  condition_block_stage2_reduce_kernel<TOut, D><<<grid, warps * 32, 0, stream>>>(
      o_partial, lse_partial, n_rows, n_parts, n_groups, group_stride, static_cast<TOut*>(out), out_lse);
  return check_launch("condition_block_stage2_reduce_kernel");
}

int launch_finalize(const float* o_partial, const float* lse_partial, int n_rows, int n_parts,
                    int head_dim, void* out, int out_dtype, float* out_lse, cudaStream_t stream) {
  return launch_finalize_groups(o_partial, lse_partial, n_rows, n_parts, 1, 0, head_dim, out, out_dtype, out_lse,
                                stream);
}

int launch_finalize_groups(const float* o_partial, const float* lse_partial, int n_rows, int n_parts, int n_groups,
                           int64_t group_stride, int head_dim, void* out, int out_dtype, float* out_lse,
                           cudaStream_t stream) {
  if (n_rows <= 0) return IA_OK;
  if (out_dtype == IA_BF16) {
    if (head_dim == 128) return launch_typed<__nv_bfloat16, 128>(o_partial, lse_partial, n_rows, n_parts, n_groups, group_stride, out, out_lse, stream);
    if (head_dim == 64) return launch_typed<__nv_bfloat16, 64>(o_partial, lse_partial, n_rows, n_parts, n_groups, group_stride, out, out_lse, stream);
  } else if (out_dtype == IA_F32) {
    if (head_dim == 128) return launch_typed<float, 128>(o_partial, lse_partial, n_rows, n_parts, n_groups, group_stride, out, out_lse, stream);
    if (head_dim == 64) return launch_typed<float, 64>(o_partial, lse_partial, n_rows, n_parts, n_groups, group_stride, out, out_lse, stream);
  }
  return fail(IA_ERR_UNSUPPORTED, "finalize: head_dim %d / out dtype %d not built", head_dim, out_dtype);
}

}  // namespace ia
