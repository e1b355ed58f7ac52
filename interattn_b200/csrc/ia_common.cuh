// Shared helpers of the interattn_b200 kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/interattn_b200.h"

namespace ia {

// ---- host-side status plumbing -------------------------------------------------
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);
int check_launch(const char* what);
int check_geom(const ia_geom* g);

inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---- device status word --------------------------------------------------------
// Bit set by a kernel whose bounded wait (mbarrier) ran out; read with
// ia_read_device_status().  Waiting is always bounded so that a programming
// error shows up as a status bit instead of a hung GPU.
enum : int {
  DEV_STATUS_SELECT_WAIT_TIMEOUT = IA_DEV_STATUS_SELECT_WAIT,
  DEV_STATUS_GEMM_WAIT_TIMEOUT = IA_DEV_STATUS_GEMM_WAIT,
  DEV_STATUS_PEER_WAIT_TIMEOUT = IA_DEV_STATUS_PEER_WAIT,
  DEV_STATUS_BAD_INDEX = IA_DEV_STATUS_BAD_INDEX
};
int* device_status_address();  // device address of the status word on the current device
int read_and_clear_device_status(int* out);  // defined next to the kernel that owns the word
int read_step_phases(double* selection_us, double* attention_us);  // of the last one-kernel step's first CTA

// ---- dtype traits ---------------------------------------------------------------
template <typename T> struct DType;
template <> struct DType<float> { static constexpr int id = IA_F32; };
template <> struct DType<__nv_bfloat16> { static constexpr int id = IA_BF16; };

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ void from_f32(float& dst, float x) { dst = x; }
__device__ __forceinline__ void from_f32(__nv_bfloat16& dst, float x) { dst = __float2bfloat16_rn(x); }

// bf16 pair packed in a 32-bit word -> two floats (exact: a shift and a mask)
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Load N consecutive elements (N * sizeof(T) in {4, 8, 16} bytes, aligned) as floats.
template <int N> __device__ __forceinline__ void load_vec(const float* p, float (&out)[N]) {
  if constexpr (N == 4) {
    float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
  } else if constexpr (N == 2) {
    float2 v = *reinterpret_cast<const float2*>(p);
    out[0] = v.x; out[1] = v.y;
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = p[i];
  }
}
template <int N> __device__ __forceinline__ void load_vec(const __nv_bfloat16* p, float (&out)[N]) {
  if constexpr (N == 4) {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    out[0] = bf16lo(v.x); out[1] = bf16hi(v.x); out[2] = bf16lo(v.y); out[3] = bf16hi(v.y);
  } else if constexpr (N == 2) {
    uint32_t v = *reinterpret_cast<const uint32_t*>(p);
    out[0] = bf16lo(v); out[1] = bf16hi(v);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) out[i] = __bfloat162float(p[i]);
  }
}
template <int N> __device__ __forceinline__ void store_vec(float* p, const float (&v)[N]) {
  if constexpr (N == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  } else if constexpr (N == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) p[i] = v[i];
  }
}
template <int N> __device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[N]) {
  if constexpr (N == 4) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&a);
    w.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = w;
  } else if constexpr (N == 2) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]);
    *reinterpret_cast<__nv_bfloat162*>(p) = a;
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) p[i] = __float2bfloat16_rn(v[i]);
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- programmatic dependent launch ----------------------------------------------
// The layer-step is a chain of short kernels on one stream; between two of them the
// GPU would idle for a launch latency and a drain.  A kernel launched through
// launch_overlapped() may be scheduled while its predecessor is still running: its
// CTAs take whatever SM resources become free and park in grid_dependency_wait(),
// which returns once the predecessor grid has completed and its writes are visible.
// Rule for kernels launched this way: call grid_dependency_wait() before the first
// access to memory the predecessor writes - or still reads, if this kernel overwrites it.
// INTERATTN_B200_NO_PDL=1 falls back to ordinary stream order.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
bool overlapped_launch_enabled();
// the one-kernel layer step may be used (INTERATTN_B200_FUSED, ia_set_fused_step)
bool fused_step_enabled();
template <typename Kern, typename Params>
inline cudaError_t launch_overlapped(Kern kern, unsigned grid, unsigned block, size_t smem, cudaStream_t stream,
                                     const Params& params, int cluster = 1) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (cluster > 1) {  // grid is a multiple of the cluster size; CTAs of a cluster are co-scheduled
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (overlapped_launch_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)n;
  return cudaLaunchKernelEx(&cfg, kern, params);
}

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

// ---- kernel launchers (one per translation unit) -------------------------------
int launch_build_summaries(const void* k_pool, const void* v_pool, const int32_t* block_table,
                           const int32_t* prefix_lens, const int32_t* first_blocks, const ia_geom& g,
                           const ia_summaries& out, cudaStream_t stream);
// split_counters (may be null): one int per (sequence, kv head), cleared by the selection
// kernel for the attention kernel's fused finalize
// exchange (may be null) + block range: split-KV across GPUs, this rank scores blocks [block_lo, block_hi)
// attend (may be null): the one-kernel layer step.  Where the launch shape gives every (sequence, kv head)
// to one CTA, that CTA goes on to attend over the pages of the blocks it has just picked (and the
// suffix) and writes the output rows - `used` tells the caller whether it did, i.e. whether the
// attention kernel is still to be launched.
struct SelectAttend {
  const void* k_pool;
  const void* v_pool;
  const int32_t* block_table;
  const int32_t* seq_lens;
  void* out;      // [batch, kv heads * group, head_dim] in the KV dtype
  int hybrid;     // blocks that are not picked attend through their representatives (z, v_bar)
  int z_scratch;  // aux.z only feeds the attention kernel: the fused kernel need not write it
  int used;       // out: 1 when the fused kernel was launched
};
int launch_select(const void* q, const ia_summaries& s, const int32_t* prefix_lens, const ia_geom& g,
                  int mode, int top_k, float eps, int max_sel, int32_t* sel_idx, int32_t* sel_count,
                  const ia_select_aux& aux, int* split_counters, cudaStream_t stream,
                  const ia_select_exchange* exchange = nullptr, int block_lo = 0, int block_hi = 0,
                  SelectAttend* attend = nullptr);
// Fused finalize of the attention kernel: the last CTA of a (sequence, kv head) merges the splits.
struct FusedFinalize {
  void* out;            // [batch, rows, D]
  int out_dtype;        // ia_dtype
  int* split_counters;  // [batch * kv heads], zero at launch
  float* flat_o;        // partials of the equal-share grid, decode_flat_partial_floats() floats (o, then lse)
  float* flat_lse;
};
// The one-call layer-step cuts the items of all (sequence, kv head) pairs into equal shares for
// decode_flat_ctas() CTAs where decode_flat_grid_applies(); its partials need this many floats.
int decode_flat_ctas();
bool decode_flat_grid_applies(const ia_geom& g, bool fused_finalize, bool full_range, bool exchange);
bool decode_flat_grid_possible(const ia_geom& g);  // the same without the environment switch: sizes the workspace
inline int64_t decode_flat_slots(const ia_geom& g) {
  return (int64_t)decode_flat_ctas() + (int64_t)g.batch * g.n_kv_heads;  // one per (CTA, pair) segment
}
int launch_sparse_decode(const void* q, const void* k_pool, const void* v_pool,
                         const int32_t* block_table, const int32_t* prefix_lens,
                         const int32_t* seq_lens, const int32_t* sel_idx, const int32_t* sel_count,
                         int max_sel, const ia_summaries* summaries, const float* z, const ia_geom& g,
                         int rep_mode, int n_splits, int block_lo, int block_hi, int with_suffix,
                         float* o_partial, float* lse_partial, const FusedFinalize* fused, cudaStream_t stream,
                         const ia_peer_exchange* exchange = nullptr);
// merge of the partials the ranks stored into this rank's gather buffer, after a bounded wait for their flags
int launch_finalize_exchange(const ia_peer_exchange& px, int n_rows, int n_parts, int head_dim, void* out,
                             int out_dtype, int* status, cudaStream_t stream);
int launch_finalize(const float* o_partial, const float* lse_partial, int n_rows, int n_parts,
                    int head_dim, void* out, int out_dtype, float* out_lse, cudaStream_t stream);
// the same merge over n_groups chunks of partials, group_stride floats apart (one chunk per GPU)
int launch_finalize_groups(const float* o_partial, const float* lse_partial, int n_rows, int n_parts, int n_groups,
                           int64_t group_stride, int head_dim, void* out, int out_dtype, float* out_lse,
                           cudaStream_t stream);

}  // namespace ia
