// Condition-block selection: host entry point.  The kernels live in select_kernel.cuh and are
// instantiated in select_inst_*.cu; this file owns the device status word and picks the instantiation.
#include "select_kernel.cuh"

namespace ia {

// Set by a kernel whose bounded mbarrier wait ran out (see mbar_wait below).
__device__ int g_device_status = 0;

// device address of the status word on the current device, for kernels of other translation units
int* device_status_address() {
  constexpr int kMaxDevices = 64;
  static int* cached[kMaxDevices] = {};  // every thread would store the same pointer
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    fail(IA_ERR_LAUNCH, "device status: no current device");
    return nullptr;
  }
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_device_status);
    if (e != cudaSuccess) {
      fail(IA_ERR_LAUNCH, "device status: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cached[dev] = static_cast<int*>(ptr);
  }
  return cached[dev];
}

// Time stamps of the one-kernel step's first CTA (nanosecond global timer): kernel entry, start of the
// attention phase, end.  A reporting aid: benchmarks split the fused kernel's time into its two phases.
__device__ unsigned long long g_step_stamps[4] = {0, 0, 0, 0};

unsigned long long* step_stamps_address() {
  constexpr int kMaxDevices = 64;
  static unsigned long long* cached[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_step_stamps) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<unsigned long long*>(ptr);
  }
  return cached[dev];
}

int read_step_phases(double* selection_us, double* attention_us) {
  unsigned long long v[4] = {0, 0, 0, 0};
  const cudaError_t e = cudaMemcpyFromSymbol(v, g_step_stamps, sizeof(v));
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "step phases: %s", cudaGetErrorString(e));
  *selection_us = v[1] >= v[0] ? (double)(v[1] - v[0]) * 1e-3 : 0.0;
  *attention_us = v[2] >= v[1] ? (double)(v[2] - v[1]) * 1e-3 : 0.0;
  return IA_OK;
}

int read_and_clear_device_status(int* out) {
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "device status: %s", cudaGetErrorString(e));
  *out = v;
  return IA_OK;
}

int launch_select(const void* q, const ia_summaries& s, const int32_t* prefix_lens, const ia_geom& g,
                  int mode, int top_k, float eps, int max_sel, int32_t* sel_idx, int32_t* sel_count,
                  const ia_select_aux& aux, int* split_counters, cudaStream_t stream,
                  const ia_select_exchange* exchange, int block_lo, int block_hi, SelectAttend* attend) {
  SelectParams p{};
  if (attend != nullptr) attend->used = 0;
  const AttendRequest ar{attend, &g, s.v_bar};
  if (exchange != nullptr) {
    p.xch = *exchange;
    p.block_lo = block_lo;
    p.block_hi = block_hi < g.max_blocks ? block_hi : g.max_blocks;
  }
  p.n_pairs = g.batch * g.n_kv_heads;
  p.status = device_status_address();
  if (p.status == nullptr) return IA_ERR_LAUNCH;
  p.stamps = step_stamps_address();
  p.q = q; p.k_bar = s.k_bar; p.k_max = s.k_max; p.k_min = s.k_min; p.v_norm_max = s.v_norm_max;
  if (g.reserved & IA_GEOM_DIAG_ELL) {  // the diagonal-ellipsoid bound: w takes the place of k_max, k_min is not read
    p.k_max = s.w;
    p.k_min = s.w;
    p.rho = s.rho;
  }
  p.prefix_lens = prefix_lens;
  p.n_kv_heads = g.n_kv_heads; p.max_blocks = g.max_blocks; p.block_size = g.block_size;
  p.mode = mode & 0xff; p.mass_exp = (mode & IA_SELECT_TERM1_MASS_EXP) != 0;
  p.top_k = top_k; p.max_sel = max_sel; p.eps = eps;
  p.sel_idx = sel_idx; p.sel_count = sel_count; p.aux = aux; p.split_counters = split_counters;
  const int n_pairs = g.batch * g.n_kv_heads;
  if (n_pairs <= 0) return IA_OK;
  if (g.reserved & IA_GEOM_PACKED_BOUNDS) {  // k_max holds the (k_max, k_min) pairs; k_min is not read
    p.k_min = p.k_max;
    if (g.head_dim != 128 && g.head_dim != 64)
      return fail(IA_ERR_UNSUPPORTED, "select: head_dim %d / dtype %d not built", g.head_dim, g.dtype);
    if (g.reserved & IA_GEOM_KBAR_BF16) {
      if (g.dtype != IA_BF16) return fail(IA_ERR_UNSUPPORTED, "select: bf16 k_bar needs bf16 pools");
      return launch_select_kbar16_packed(p, ar, n_pairs, g.group_size, g.head_dim, stream);
    }
    if (g.dtype == IA_BF16)
      return g.head_dim == 128 ? launch_select_bf16_d128_packed(p, ar, n_pairs, g.group_size, stream)
                               : launch_select_bf16_d64_packed(p, ar, n_pairs, g.group_size, stream);
    return launch_select_f32_packed(p, ar, n_pairs, g.group_size, g.head_dim, stream);
  }
  if (g.reserved & IA_GEOM_KBAR_BF16) {  // k_bar stored in bf16: only next to bf16 pools ("mixed" storage)
    if (g.dtype != IA_BF16) return fail(IA_ERR_UNSUPPORTED, "select: bf16 k_bar needs bf16 pools");
    if (g.head_dim == 128) return launch_select_kbar16_d128(p, ar, n_pairs, g.group_size, stream);
    if (g.head_dim == 64) return launch_select_kbar16_d64(p, ar, n_pairs, g.group_size, stream);
  } else if (g.dtype == IA_BF16) {
    if (g.head_dim == 128)
      return p.rho != nullptr ? launch_select_bf16_d128_diag(p, ar, n_pairs, g.group_size, stream)
                              : launch_select_bf16_d128_range(p, ar, n_pairs, g.group_size, stream);
    if (g.head_dim == 64) return launch_select_bf16_d64(p, ar, n_pairs, g.group_size, stream);
  } else if (g.dtype == IA_F32) {
    if (g.head_dim == 128) return launch_select_f32_d128(p, ar, n_pairs, g.group_size, stream);
    if (g.head_dim == 64) return launch_select_f32_d64(p, ar, n_pairs, g.group_size, stream);
  }
  return fail(IA_ERR_UNSUPPORTED, "select: head_dim %d / dtype %d not built", g.head_dim, g.dtype);
}

}  // namespace ia
