// extern "C" surface of libinterattn_b200.so: argument checks, status
// plumbing and the one-call layer-step.  Declarations and the reference
// interfaces they replace: include/interattn_b200.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "ia_common.cuh"

namespace ia {

static thread_local char tls_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tls_error, sizeof(tls_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return IA_OK;
  return fail(IA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

bool overlapped_launch_enabled() {
  static const bool on = [] {
    const char* v = getenv("INTERATTN_B200_NO_PDL");
    return !(v != nullptr && v[0] == '1');
  }();
  return on;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_geom(const ia_geom* g) {
  if (g == nullptr) return fail(IA_ERR_BAD_ARG, "geom is null");
  if (g->batch < 0 || g->n_kv_heads <= 0 || g->group_size <= 0)
    return fail(IA_ERR_BAD_ARG, "geom: batch %d, n_kv_heads %d, group_size %d", g->batch, g->n_kv_heads, g->group_size);
  if (g->head_dim != 64 && g->head_dim != 128)
    return fail(IA_ERR_UNSUPPORTED, "geom: head_dim %d (built: 64, 128)", g->head_dim);
  if (g->page_size != 16) return fail(IA_ERR_UNSUPPORTED, "geom: page_size %d (built: 16)", g->page_size);
  if (g->block_size <= 0 || g->block_size % g->page_size != 0 || g->block_size > 128)
    return fail(IA_ERR_BAD_ARG, "geom: block_size %d must be a multiple of page_size %d, at most 128", g->block_size,
                g->page_size);
  if (g->group_size > 16) return fail(IA_ERR_UNSUPPORTED, "geom: group_size %d (built: up to 16)", g->group_size);
  if (g->max_pages <= 0 || g->max_blocks <= 0)
    return fail(IA_ERR_BAD_ARG, "geom: max_pages %d, max_blocks %d", g->max_pages, g->max_blocks);
  if (g->dtype != IA_F32 && g->dtype != IA_BF16) return fail(IA_ERR_BAD_ARG, "geom: dtype %d", g->dtype);
  const int64_t run = (int64_t)g->page_size * g->head_dim;
  if (g->pool_head_stride < run || g->pool_page_stride < run)
    return fail(IA_ERR_BAD_ARG, "geom: pool strides (%lld, %lld) smaller than one page run %lld",
                (long long)g->pool_page_stride, (long long)g->pool_head_stride, (long long)run);
  const int64_t esz = g->dtype == IA_BF16 ? 2 : 4;
  if ((g->pool_head_stride * esz) % 16 != 0 || (g->pool_page_stride * esz) % 16 != 0)
    return fail(IA_ERR_BAD_ARG, "geom: pool strides must be multiples of 16 bytes");
  if (g->reserved & ~(IA_GEOM_KBAR_BF16 | IA_GEOM_DIAG_ELL | IA_GEOM_PACKED_BOUNDS))
    return fail(IA_ERR_BAD_ARG, "geom: unknown flag bits in reserved (%d)", g->reserved);
  if ((g->reserved & IA_GEOM_DIAG_ELL) && (g->reserved & IA_GEOM_PACKED_BOUNDS))
    return fail(IA_ERR_BAD_ARG, "geom: the packed range layout and the diag_ell bound exclude one another");
  if (g->n_pool_pages < 0 || g->reserved2 != 0)
    return fail(IA_ERR_BAD_ARG, "geom: n_pool_pages %d (0 = unknown), reserved2 %d (must be 0)", g->n_pool_pages,
                g->reserved2);
  return IA_OK;
}

// diag_ell: the selection reads (k_bar, w, rho) and k_max / k_min may be absent; building summaries
// always needs k_max / k_min as outputs (w is derived from them)
static int check_summaries(const ia_summaries* s, const ia_geom* g = nullptr, bool building = false) {
  if (s == nullptr) return fail(IA_ERR_BAD_ARG, "summaries is null");
  const bool diag = g != nullptr && (g->reserved & IA_GEOM_DIAG_ELL) != 0;
  const bool packed = g != nullptr && (g->reserved & IA_GEOM_PACKED_BOUNDS) != 0;  // k_max holds both, k_min unused
  if (!s->k_bar || !s->v_bar || !s->v_norm_max) return fail(IA_ERR_BAD_ARG, "summaries: null member");
  if ((!diag || building) && (!s->k_max || (!packed && !s->k_min)))
    return fail(IA_ERR_BAD_ARG, "summaries: null k_max / k_min");
  if (packed && building && (s->w || s->rho))
    return fail(IA_ERR_BAD_ARG, "summaries: the packed range layout does not carry the diagonal-ellipsoid pair");
  if ((diag || s->w || s->rho) && (!s->w || !s->rho))
    return fail(IA_ERR_BAD_ARG, "summaries: the diagonal-ellipsoid bound needs both w and rho");
  if (!aligned16(s->k_bar) || !aligned16(s->k_max) || !aligned16(s->k_min) || !aligned16(s->v_bar) || !aligned16(s->w))
    return fail(IA_ERR_BAD_ARG, "summaries: arrays must be 16-byte aligned");
  return IA_OK;
}

struct Workspace {
  int32_t* sel_idx;
  int32_t* sel_count;
  float* z;
  float* o_partial;
  float* lse_partial;
  int* split_counters;
  float* flat_o;    // partials of the equal-share attention grid (bf16 pools), else null
  float* flat_lse;
  int64_t bytes;
};

static int64_t align256(int64_t x) { return (x + 255) & ~int64_t(255); }

static Workspace carve(const ia_geom& g, int max_sel, int n_splits, int rep_mode, void* base) {
  Workspace w{};
  const int64_t pairs = (int64_t)g.batch * g.n_kv_heads;
  const int64_t rows = pairs * g.group_size;
  char* p = static_cast<char*>(base);
  int64_t off = 0;
  auto take = [&](int64_t bytes) {
    char* r = p ? p + off : nullptr;
    off += align256(bytes);
    return r;
  };
  w.sel_idx = reinterpret_cast<int32_t*>(take(pairs * max_sel * 4));
  w.sel_count = reinterpret_cast<int32_t*>(take(pairs * 4));
  w.z = reinterpret_cast<float*>(take(rep_mode == IA_REP_HYBRID ? rows * g.max_blocks * 4 : 0));
  w.o_partial = reinterpret_cast<float*>(take(rows * n_splits * g.head_dim * 4));
  w.lse_partial = reinterpret_cast<float*>(take(rows * n_splits * 4));
  w.split_counters = reinterpret_cast<int*>(take(pairs * 4));
  if (decode_flat_grid_possible(g)) {
    const int64_t slots = decode_flat_slots(g);
    w.flat_o = reinterpret_cast<float*>(take(slots * g.group_size * g.head_dim * 4));
    w.flat_lse = reinterpret_cast<float*>(take(slots * g.group_size * 4));
  }
  w.bytes = off;
  return w;
}

}  // namespace ia

using namespace ia;

// -1: not set by the caller, the environment decides (INTERATTN_B200_FUSED=0 turns the one-kernel step off)
static std::atomic<int> g_fused_step{-1};

namespace ia {
bool fused_step_enabled() {
  const int v = g_fused_step.load(std::memory_order_relaxed);
  if (v >= 0) return v != 0;
  static const bool env_on = [] {
    const char* e = getenv("INTERATTN_B200_FUSED");
    return !(e != nullptr && e[0] == '0');
  }();
  return env_on;
}
}  // namespace ia

extern "C" {

int ia_abi_version(void) { return 3; }

const char* ia_last_error_string(void) { return tls_error; }

// Reads and clears the device status word (IA_DEV_STATUS_* masks).  Synchronises
// the device, so it is not part of the step.
int ia_read_device_status(int* out) {
  if (out == nullptr) return fail(IA_ERR_BAD_ARG, "out is null");
  return read_and_clear_device_status(out);
}

int ia_build_summaries(const void* k_pool, const void* v_pool, const int32_t* block_table,
                       const int32_t* prefix_lens, const ia_geom* geom, const ia_summaries* out,
                       ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (int s = check_summaries(out, geom, true)) return s;
  if (!k_pool || !v_pool || !block_table || !prefix_lens) return fail(IA_ERR_BAD_ARG, "build_summaries: null argument");
  if (!aligned16(k_pool) || !aligned16(v_pool)) return fail(IA_ERR_BAD_ARG, "build_summaries: pools must be 16-byte aligned");
  return launch_build_summaries(k_pool, v_pool, block_table, prefix_lens, nullptr, *geom, *out, (cudaStream_t)stream);
}

int ia_update_summaries(const void* k_pool, const void* v_pool, const int32_t* block_table,
                        const int32_t* prefix_lens, const int32_t* first_blocks, const ia_geom* geom,
                        const ia_summaries* out, ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (int s = check_summaries(out, geom, true)) return s;
  if (!k_pool || !v_pool || !block_table || !prefix_lens || !first_blocks)
    return fail(IA_ERR_BAD_ARG, "update_summaries: null argument");
  if (!aligned16(k_pool) || !aligned16(v_pool)) return fail(IA_ERR_BAD_ARG, "update_summaries: pools must be 16-byte aligned");
  return launch_build_summaries(k_pool, v_pool, block_table, prefix_lens, first_blocks, *geom, *out,
                                (cudaStream_t)stream);
}

int ia_select(const void* q, const ia_summaries* summaries, const int32_t* prefix_lens,
              const ia_geom* geom, int mode, int top_k, float eps, int max_sel, int32_t* sel_idx,
              int32_t* sel_count, const ia_select_aux* aux, ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (int s = check_summaries(summaries, geom)) return s;
  if (!q || !prefix_lens || !sel_idx || !sel_count) return fail(IA_ERR_BAD_ARG, "select: null argument");
  const int full_mode = mode;
  mode &= 0xff;  // the high bits carry the score variant (IA_SELECT_TERM1_MASS_EXP)
  if ((mode != IA_SELECT_TOPK && mode != IA_SELECT_EPS) || (full_mode & ~(0xff | IA_SELECT_TERM1_MASS_EXP)))
    return fail(IA_ERR_BAD_ARG, "select: mode %d", full_mode);
  if (max_sel <= 0) return fail(IA_ERR_BAD_ARG, "select: max_sel %d", max_sel);
  if (mode == IA_SELECT_TOPK && (top_k < 0 || top_k > max_sel))
    return fail(IA_ERR_BAD_ARG, "select: top_k %d outside [0, max_sel %d]", top_k, max_sel);
  if (mode == IA_SELECT_EPS && max_sel < geom->max_blocks)
    return fail(IA_ERR_BAD_ARG, "select: epsilon mode may keep every block: max_sel %d < max_blocks %d", max_sel,
                geom->max_blocks);
  ia_select_aux none{};
  return launch_select(q, *summaries, prefix_lens, *geom, full_mode, top_k, eps, max_sel, sel_idx, sel_count,
                       aux ? *aux : none, nullptr, (cudaStream_t)stream);
}

int ia_select_split(const void* q, const ia_summaries* summaries, const int32_t* prefix_lens, const ia_geom* geom,
                    int top_k, int max_sel, int block_lo, int block_hi, int32_t* sel_idx, int32_t* sel_count,
                    const ia_select_aux* aux, const ia_select_exchange* x, ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (int s = check_summaries(summaries, geom)) return s;
  if (!q || !prefix_lens || !sel_idx || !sel_count || !x) return fail(IA_ERR_BAD_ARG, "select_split: null argument");
  if (max_sel <= 0 || top_k < 0 || top_k > max_sel)
    return fail(IA_ERR_BAD_ARG, "select_split: top_k %d outside [0, max_sel %d]", top_k, max_sel);
  if (x->n_ranks < 1 || x->n_ranks > 8 || x->my_rank < 0 || x->my_rank >= x->n_ranks)
    return fail(IA_ERR_BAD_ARG, "select_split: rank %d of %d (at most 8)", x->my_rank, x->n_ranks);
  for (int w = 0; w < x->n_ranks; ++w)
    if (!x->norm[w] || !x->cand[w] || !x->flags[w] || (reinterpret_cast<uintptr_t>(x->norm[w]) & 15u) != 0 ||
        (reinterpret_cast<uintptr_t>(x->cand[w]) & 7u) != 0)
      return fail(IA_ERR_BAD_ARG, "select_split: null or misaligned buffer of rank %d", w);
  if (!x->step_counter || !x->grid_counter) return fail(IA_ERR_BAD_ARG, "select_split: null counter");
  if (block_lo < 0 || block_hi < block_lo || block_lo % 32 != 0 || (block_hi % 32 != 0 && block_hi < geom->max_blocks))
    return fail(IA_ERR_BAD_ARG, "select_split: block range [%d, %d) must start on a multiple of 32 and end on one "
                "(or at max_blocks %d)", block_lo, block_hi, geom->max_blocks);
  if ((int64_t)x->n_ranks * max_sel > 4096)
    return fail(IA_ERR_UNSUPPORTED, "select_split: %d ranks x max_sel %d candidates (at most 4096)", x->n_ranks, max_sel);
  ia_select_aux none{};
  return launch_select(q, *summaries, prefix_lens, *geom, IA_SELECT_TOPK, top_k, 0.f, max_sel, sel_idx, sel_count,
                       aux ? *aux : none, nullptr, (cudaStream_t)stream, x, block_lo, block_hi);
}

static int check_exchange(const ia_peer_exchange* px, int64_t n_rows, int n_parts, int head_dim) {
  if (!px) return fail(IA_ERR_BAD_ARG, "exchange: null argument");
  if (px->n_ranks < 1 || px->n_ranks > 8 || px->my_rank < 0 || px->my_rank >= px->n_ranks)
    return fail(IA_ERR_BAD_ARG, "exchange: rank %d of %d (at most 8)", px->my_rank, px->n_ranks);
  for (int w = 0; w < px->n_ranks; ++w)
    if (!px->gather[w] || !px->flags[w]) return fail(IA_ERR_BAD_ARG, "exchange: null buffer of rank %d", w);
  if (!px->step_counter || !px->grid_counter) return fail(IA_ERR_BAD_ARG, "exchange: null counter");
  const int64_t n_o = n_rows * n_parts * head_dim;
  if (px->lse_offset < n_o || px->chunk_floats < px->lse_offset + n_rows * n_parts)
    return fail(IA_ERR_BAD_ARG, "exchange: chunk of %lld floats, lse at %lld, need %lld + %lld",
                (long long)px->chunk_floats, (long long)px->lse_offset, (long long)n_o, (long long)(n_rows * n_parts));
  return IA_OK;
}

static int sparse_decode_impl(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                              const int32_t* prefix_lens, const int32_t* seq_lens, const int32_t* sel_idx,
                              const int32_t* sel_count, int max_sel, const ia_summaries* summaries, const float* z,
                              const ia_geom* geom, int rep_mode, int n_splits, int block_lo, int block_hi,
                              int with_suffix, float* o_partial, float* lse_partial,
                              const ia_peer_exchange* exchange, ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (!q || !k_pool || !v_pool || !block_table || !prefix_lens || !seq_lens || !sel_idx || !sel_count ||
      (exchange == nullptr && (!o_partial || !lse_partial)))
    return fail(IA_ERR_BAD_ARG, "sparse_decode: null argument");
  if (exchange != nullptr) {
    const int64_t rows = (int64_t)geom->batch * geom->n_kv_heads * geom->group_size;
    if (int s = check_exchange(exchange, rows, n_splits, geom->head_dim)) return s;
  }
  if (!aligned16(k_pool) || !aligned16(v_pool) || !aligned16(q))
    return fail(IA_ERR_BAD_ARG, "sparse_decode: q and pools must be 16-byte aligned");
  if (rep_mode != IA_REP_SPARSE_ONLY && rep_mode != IA_REP_HYBRID)
    return fail(IA_ERR_BAD_ARG, "sparse_decode: rep_mode %d", rep_mode);
  if (rep_mode == IA_REP_HYBRID) {
    if (!summaries || !summaries->v_bar || !z)
      return fail(IA_ERR_BAD_ARG, "sparse_decode: hybrid mode needs summaries->v_bar and z");
    if (!aligned16(summaries->v_bar)) return fail(IA_ERR_BAD_ARG, "sparse_decode: v_bar must be 16-byte aligned");
  }
  if (n_splits <= 0 || n_splits > 64) return fail(IA_ERR_BAD_ARG, "sparse_decode: n_splits %d outside [1, 64]", n_splits);
  if (max_sel <= 0) return fail(IA_ERR_BAD_ARG, "sparse_decode: max_sel %d", max_sel);
  if (block_lo < 0 || block_hi < block_lo) return fail(IA_ERR_BAD_ARG, "sparse_decode: block range [%d, %d)", block_lo, block_hi);
  return launch_sparse_decode(q, k_pool, v_pool, block_table, prefix_lens, seq_lens, sel_idx, sel_count, max_sel,
                              summaries, z, *geom, rep_mode, n_splits, block_lo, block_hi, with_suffix, o_partial,
                              lse_partial, nullptr, (cudaStream_t)stream, exchange);
}

int ia_sparse_decode(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                     const int32_t* prefix_lens, const int32_t* seq_lens, const int32_t* sel_idx,
                     const int32_t* sel_count, int max_sel, const ia_summaries* summaries, const float* z,
                     const ia_geom* geom, int rep_mode, int n_splits, int block_lo, int block_hi,
                     int with_suffix, float* o_partial, float* lse_partial, ia_stream_t stream) {
  return sparse_decode_impl(q, k_pool, v_pool, block_table, prefix_lens, seq_lens, sel_idx, sel_count, max_sel,
                            summaries, z, geom, rep_mode, n_splits, block_lo, block_hi, with_suffix, o_partial,
                            lse_partial, nullptr, stream);
}

int ia_sparse_decode_exchange(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                              const int32_t* prefix_lens, const int32_t* seq_lens, const int32_t* sel_idx,
                              const int32_t* sel_count, int max_sel, const ia_summaries* summaries, const float* z,
                              const ia_geom* geom, int rep_mode, int n_splits, int block_lo, int block_hi,
                              int with_suffix, const ia_peer_exchange* exchange, ia_stream_t stream) {
  if (!exchange) return fail(IA_ERR_BAD_ARG, "sparse_decode_exchange: null exchange");
  return sparse_decode_impl(q, k_pool, v_pool, block_table, prefix_lens, seq_lens, sel_idx, sel_count, max_sel,
                            summaries, z, geom, rep_mode, n_splits, block_lo, block_hi, with_suffix, nullptr, nullptr,
                            exchange, stream);
}

int ia_finalize_exchange(const ia_peer_exchange* exchange, int n_rows, int n_parts, int head_dim, void* out,
                         int out_dtype, ia_stream_t stream) {
  if (!out) return fail(IA_ERR_BAD_ARG, "finalize_exchange: null out");
  if (n_rows < 0 || n_parts <= 0 || head_dim <= 0)
    return fail(IA_ERR_BAD_ARG, "finalize_exchange: %d rows, %d parts", n_rows, n_parts);
  if (int s = check_exchange(exchange, n_rows, n_parts, head_dim)) return s;
  int* status = device_status_address();
  if (status == nullptr) return IA_ERR_LAUNCH;
  return launch_finalize_exchange(*exchange, n_rows, n_parts, head_dim, out, out_dtype, status, (cudaStream_t)stream);
}

int ia_finalize(const float* o_partial, const float* lse_partial, int n_rows, int n_parts, int head_dim,
                void* out, int out_dtype, float* out_lse, ia_stream_t stream) {
  if (!o_partial || !lse_partial || !out) return fail(IA_ERR_BAD_ARG, "finalize: null argument");
  if (n_rows < 0 || n_parts <= 0) return fail(IA_ERR_BAD_ARG, "finalize: n_rows %d, n_parts %d", n_rows, n_parts);
  return launch_finalize(o_partial, lse_partial, n_rows, n_parts, head_dim, out, out_dtype, out_lse,
                         (cudaStream_t)stream);
}

int ia_finalize_gathered(const float* gathered, int n_ranks, int64_t rank_stride, int n_rows, int n_parts,
                         int head_dim, void* out, int out_dtype, ia_stream_t stream) {
  if (!gathered || !out) return fail(IA_ERR_BAD_ARG, "finalize_gathered: null argument");
  if (n_ranks <= 0 || n_rows < 0 || n_parts <= 0 || head_dim <= 0)
    return fail(IA_ERR_BAD_ARG, "finalize_gathered: %d ranks, %d rows, %d parts", n_ranks, n_rows, n_parts);
  const int64_t chunk = (int64_t)n_rows * n_parts * (head_dim + 1);
  if (rank_stride < chunk || rank_stride % 4 != 0)
    return fail(IA_ERR_BAD_ARG, "finalize_gathered: rank stride %lld floats (at least %lld, a multiple of 4)",
                (long long)rank_stride, (long long)chunk);
  if (!aligned16(gathered)) return fail(IA_ERR_BAD_ARG, "finalize_gathered: the buffer must be 16-byte aligned");
  return launch_finalize_groups(gathered, gathered + (int64_t)n_rows * n_parts * head_dim, n_rows, n_parts, n_ranks,
                                rank_stride, head_dim, out, out_dtype, nullptr, (cudaStream_t)stream);
}

int64_t ia_workspace_bytes(const ia_geom* geom, int max_sel, int n_splits, int rep_mode) {
  if (check_geom(geom) != IA_OK || max_sel <= 0 || n_splits <= 0) return -1;
  return carve(*geom, max_sel, n_splits, rep_mode, nullptr).bytes;
}

// Split-KV parts per (sequence, kv head) for ia_sparse_decode.  The attention
// kernel keeps two CTAs per SM resident; a grid that is not a whole number of
// such waves leaves SMs idle in its last wave, and a lone CTA cannot pull much
// more than its fair share of HBM (its loads in flight are bounded by its
// shared-memory ring).  The estimate below is that model, fitted on B200:
//   time(S) = sum over waves of max(bytes per CTA / r_cta, bytes of the wave / B) + c
// with r_cta = 26 GB/s, B = 5.4 TB/s, c = 3 us.
int ia_suggest_splits(const ia_geom* geom, int expected_blocks) {
  if (check_geom(geom) != IA_OK || expected_blocks <= 0) return 1;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const double slots = 2.0 * sms;
  const double pairs = (double)geom->batch * geom->n_kv_heads;
  const double esz = geom->dtype == IA_BF16 ? 2.0 : 4.0;
  const double pair_bytes = (double)expected_blocks * geom->block_size * geom->head_dim * 2.0 * esz;
  const double r_cta = 26e9, hbm = 5.4e12, fixed = 3e-6;
  const int pages = expected_blocks * (geom->block_size / geom->page_size);
  int best = 1;
  double best_t = 1e30;
  for (int s = 1; s <= 16; ++s) {
    if (s > 1 && pages / s < 8) break;  // keep at least two pages per warp
    const double cta_bytes = pair_bytes / s;
    double left = pairs * s, t = 0.0;
    while (left > 0.0) {
      const double n = left < slots ? left : slots;
      const double a = cta_bytes / r_cta, b = n * cta_bytes / hbm;
      t += (a > b ? a : b) + fixed;
      left -= n;
    }
    if (t < best_t * 0.98) { best_t = t; best = s; }
  }
  return best;
}

static thread_local int t_last_decode_fused = 0;

static int decode_attention_impl(const void* q, const void* k_pool, const void* v_pool,
                                 const int32_t* block_table, const int32_t* prefix_lens,
                                 const int32_t* seq_lens, const ia_summaries* summaries, const ia_geom* geom,
                                 int mode, int top_k, float eps, int max_sel, int rep_mode, int n_splits,
                                 void* workspace, int64_t workspace_bytes, int32_t* sel_idx, int32_t* sel_count,
                                 void* out, void* const* events, ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (!workspace || !out) return fail(IA_ERR_BAD_ARG, "decode_attention: null workspace or out");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0)
    return fail(IA_ERR_BAD_ARG, "decode_attention: workspace must be 256-byte aligned");
  if (max_sel <= 0 || n_splits <= 0) return fail(IA_ERR_BAD_ARG, "decode_attention: max_sel %d, n_splits %d", max_sel, n_splits);
  Workspace w = carve(*geom, max_sel, n_splits, rep_mode, workspace);
  if (workspace_bytes < w.bytes)
    return fail(IA_ERR_BAD_ARG, "decode_attention: workspace %lld bytes, need %lld", (long long)workspace_bytes,
                (long long)w.bytes);
  cudaStream_t st = (cudaStream_t)stream;
  auto mark = [&](int i) {
    if (events != nullptr && events[i] != nullptr) cudaEventRecord((cudaEvent_t)events[i], st);
  };
  int32_t* idx = sel_idx ? sel_idx : w.sel_idx;
  int32_t* cnt = sel_count ? sel_count : w.sel_count;
  ia_select_aux aux{};
  if (rep_mode == IA_REP_HYBRID) aux.z = w.z;
#ifdef IA_SELECT_TRACE
  // profiling build: the selection kernel's time stamps go where IA_STEP_TRACE_PTR says (16 floats per CTA)
  if (const char* at = getenv("IA_STEP_TRACE_PTR")) aux.delta = reinterpret_cast<float*>(strtoull(at, nullptr, 16));
#endif
  // Argument checks of the public entry points, then two launches: the selection
  // kernel (which also clears the per-pair split counters) and the attention kernel
  // with the fused finalize - the CTA that finishes a (sequence, kv head) last merges
  // its splits and writes `out`, so no third kernel is needed.
  if (int s = check_summaries(summaries, geom)) return s;
  if (!q || !k_pool || !v_pool || !block_table || !prefix_lens || !seq_lens)
    return fail(IA_ERR_BAD_ARG, "decode_attention: null argument");
  if (!aligned16(k_pool) || !aligned16(v_pool) || !aligned16(q) || !aligned16(out))
    return fail(IA_ERR_BAD_ARG, "decode_attention: q, out and pools must be 16-byte aligned");
  const int full_mode = mode;
  mode &= 0xff;  // the high bits carry the score variant (IA_SELECT_TERM1_MASS_EXP)
  if ((mode != IA_SELECT_TOPK && mode != IA_SELECT_EPS) || (full_mode & ~(0xff | IA_SELECT_TERM1_MASS_EXP)))
    return fail(IA_ERR_BAD_ARG, "decode_attention: mode %d", full_mode);
  if (mode == IA_SELECT_TOPK && (top_k < 0 || top_k > max_sel))
    return fail(IA_ERR_BAD_ARG, "decode_attention: top_k %d outside [0, max_sel %d]", top_k, max_sel);
  if (mode == IA_SELECT_EPS && max_sel < geom->max_blocks)
    return fail(IA_ERR_BAD_ARG, "decode_attention: epsilon mode may keep every block: max_sel %d < max_blocks %d",
                max_sel, geom->max_blocks);
  if (rep_mode != IA_REP_SPARSE_ONLY && rep_mode != IA_REP_HYBRID)
    return fail(IA_ERR_BAD_ARG, "decode_attention: rep_mode %d", rep_mode);
  if (n_splits > 64) return fail(IA_ERR_BAD_ARG, "decode_attention: n_splits %d outside [1, 64]", n_splits);
  mark(0);
  // The selection kernel can go on to attend over what it picked - one launch; it says whether its
  // launch shape allowed that (the whole grid resident at once, bf16, head_dim 128, <= 8 rows per kv head).
  ia::SelectAttend attend{k_pool, v_pool, block_table, seq_lens, out, rep_mode == IA_REP_HYBRID, 1, 0};
  if (int s = launch_select(q, *summaries, prefix_lens, *geom, full_mode, top_k, eps, max_sel, idx, cnt, aux,
                            w.split_counters, st, nullptr, 0, 0, &attend))
    return s;
  mark(1);
  t_last_decode_fused = attend.used;
  if (attend.used) {
    mark(2);
    mark(3);
    return IA_OK;
  }
  FusedFinalize fused{out, geom->dtype, w.split_counters, w.flat_o, w.flat_lse};
  const int s = launch_sparse_decode(q, k_pool, v_pool, block_table, prefix_lens, seq_lens, idx, cnt, max_sel,
                                     summaries, w.z, *geom, rep_mode, n_splits, 0, geom->max_blocks, 1, w.o_partial,
                                     w.lse_partial, &fused, st);
  mark(2);
  mark(3);  // the finalize is part of the attention kernel: events 2 and 3 coincide
  return s;
}

int ia_decode_attention(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                        const int32_t* prefix_lens, const int32_t* seq_lens, const ia_summaries* summaries,
                        const ia_geom* geom, int mode, int top_k, float eps, int max_sel, int rep_mode,
                        int n_splits, void* workspace, int64_t workspace_bytes, int32_t* sel_idx,
                        int32_t* sel_count, void* out, ia_stream_t stream) {
  return decode_attention_impl(q, k_pool, v_pool, block_table, prefix_lens, seq_lens, summaries, geom, mode, top_k,
                               eps, max_sel, rep_mode, n_splits, workspace, workspace_bytes, sel_idx, sel_count, out,
                               nullptr, stream);
}

int ia_last_decode_fused(void) { return t_last_decode_fused; }

int ia_last_step_phases(double* selection_us, double* attention_us) {
  if (!selection_us || !attention_us) return fail(IA_ERR_BAD_ARG, "last_step_phases: null argument");
  return read_step_phases(selection_us, attention_us);
}

int ia_set_fused_step(int enabled) {
  const int before = ia::fused_step_enabled() ? 1 : 0;
  g_fused_step.store(enabled ? 1 : 0, std::memory_order_relaxed);
  return before;
}

int ia_decode_attention_timed(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                              const int32_t* prefix_lens, const int32_t* seq_lens, const ia_summaries* summaries,
                              const ia_geom* geom, int mode, int top_k, float eps, int max_sel, int rep_mode,
                              int n_splits, void* workspace, int64_t workspace_bytes, int32_t* sel_idx,
                              int32_t* sel_count, void* out, void* const* events, ia_stream_t stream) {
  if (events == nullptr) return fail(IA_ERR_BAD_ARG, "decode_attention_timed: events is null");
  return decode_attention_impl(q, k_pool, v_pool, block_table, prefix_lens, seq_lens, summaries, geom, mode, top_k,
                               eps, max_sel, rep_mode, n_splits, workspace, workspace_bytes, sel_idx, sel_count, out,
                               events, stream);
}

// Device alias of a host buffer the GPU can address directly (pinned, mapped host memory under
// unified addressing), or null.  INTERATTN_B200_HOST_STAGING=1 turns the direct path off (A/B runs).
static void* device_alias_of_host(const void* host) {
  static const bool off = [] {
    const char* v = getenv("INTERATTN_B200_HOST_STAGING");
    return v != nullptr && v[0] == '1';
  }();
  if (off) return nullptr;
  cudaPointerAttributes a{};
  if (cudaPointerGetAttributes(&a, host) != cudaSuccess) {
    cudaGetLastError();  // pageable memory the runtime has never seen: not an error of this call
    return nullptr;
  }
  if (a.type != cudaMemoryTypeHost || a.devicePointer == nullptr) return nullptr;
  return (reinterpret_cast<uintptr_t>(a.devicePointer) & 15u) == 0 ? a.devicePointer : nullptr;
}

int ia_decode_attention_host(const void* q_host, void* q_dev, const void* k_pool, const void* v_pool,
                             const int32_t* block_table, const int32_t* prefix_lens, const int32_t* seq_lens,
                             const ia_summaries* summaries, const ia_geom* geom, int mode, int top_k, float eps,
                             int max_sel, int rep_mode, int n_splits, void* workspace, int64_t workspace_bytes,
                             void* out_dev, void* out_host, ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (!q_host || !q_dev || !out_dev || !out_host) return fail(IA_ERR_BAD_ARG, "decode_attention_host: null buffer");
  const size_t esz = geom->dtype == IA_BF16 ? 2 : 4;
  const size_t bytes = (size_t)geom->batch * geom->n_kv_heads * geom->group_size * geom->head_dim * esz;
  cudaStream_t st = (cudaStream_t)stream;
  // Pinned host buffers are addressable from the device: the kernels then read the query rows and
  // write the output rows across PCIe themselves (a kilobyte per (sequence, kv head), fetched while
  // the first summaries and pages are in flight), which spares the two copy operations and their
  // latency on the stream.  Pageable buffers go through the caller's staging buffers instead.
  void* q_direct = device_alias_of_host(q_host);
  void* out_direct = device_alias_of_host(out_host);
  cudaError_t e = cudaSuccess;
  if (q_direct == nullptr) {
    e = cudaMemcpyAsync(q_dev, q_host, bytes, cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "decode_attention_host: h2d: %s", cudaGetErrorString(e));
  }
  if (int s = ia_decode_attention(q_direct ? q_direct : q_dev, k_pool, v_pool, block_table, prefix_lens, seq_lens,
                                  summaries, geom, mode, top_k, eps, max_sel, rep_mode, n_splits, workspace,
                                  workspace_bytes, nullptr, nullptr, out_direct ? out_direct : out_dev, stream))
    return s;
  if (out_direct == nullptr) e = cudaMemcpyAsync(out_host, out_dev, bytes, cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "decode_attention_host: d2h: %s", cudaGetErrorString(e));
  return IA_OK;
}

}  // extern "C"

// ---- the layer-step for callers that cannot allocate device memory ---------------------
//
// Some hosts of this library never get to call cudaMalloc: an inference server
// that hands (nearly) all of HBM to its KV-cache pool at start-up, so that a
// later allocation by a plug-in fails or fragments the pool; a runtime whose
// hot loop is audited to be allocation-free.  For them the scratch of the
// layer-step (selection list, split-KV partials, hybrid-mode logits) lives in
// the array below, which is part of the library image: every GPU that loads
// the library holds these IA_NOALLOC_SCRATCH_BYTES until the process exits.
namespace ia {

static __device__ __align__(256) unsigned char g_noalloc_scratch[IA_NOALLOC_SCRATCH_BYTES];

// In host code `g_noalloc_scratch` only names the symbol; it is not a device
// address and must never be handed to a kernel.  The device address is looked
// up once per device (with that device current) and cached here.
constexpr int kMaxDevices = 64;
static void* g_noalloc_addr[kMaxDevices] = {};

static int noalloc_scratch(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(IA_ERR_NO_DEVICE, "decode_attention_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(IA_ERR_UNSUPPORTED, "decode_attention_noalloc: device ordinal %d", dev);
  void* p = __atomic_load_n(&g_noalloc_addr[dev], __ATOMIC_ACQUIRE);
  if (p == nullptr) {
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(IA_ERR_LAUNCH, "decode_attention_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    __atomic_store_n(&g_noalloc_addr[dev], p, __ATOMIC_RELEASE);  // every thread would store the same address
  }
  *out = p;
  return IA_OK;
}

}  // namespace ia

extern "C" {

int64_t ia_noalloc_scratch_bytes(void) { return (int64_t)IA_NOALLOC_SCRATCH_BYTES; }

int ia_decode_attention_noalloc(const void* q, const void* k_pool, const void* v_pool,
                                const int32_t* block_table, const int32_t* prefix_lens,
                                const int32_t* seq_lens, const ia_summaries* summaries, const ia_geom* geom,
                                int mode, int top_k, float eps, int max_sel, int rep_mode, int n_splits, void* out,
                                ia_stream_t stream) {
  if (int s = check_geom(geom)) return s;
  if (max_sel <= 0 || n_splits <= 0)
    return fail(IA_ERR_BAD_ARG, "decode_attention_noalloc: max_sel %d, n_splits %d", max_sel, n_splits);
  const int64_t need = carve(*geom, max_sel, n_splits, rep_mode, nullptr).bytes;
  if (need > (int64_t)IA_NOALLOC_SCRATCH_BYTES)
    return fail(IA_ERR_UNSUPPORTED,
                "decode_attention_noalloc: this step needs %lld bytes of scratch, the built-in array holds %lld; "
                "use ia_decode_attention with a caller-owned workspace, or fewer sequences / splits per call",
                (long long)need, (long long)IA_NOALLOC_SCRATCH_BYTES);
  void* scratch = nullptr;
  if (int s = noalloc_scratch(&scratch)) return s;
  // Nothing in the scratch has to start at zero: the selection kernel writes the
  // whole index list and every count and clears the per-pair arrival counters, the
  // attention kernel writes every partial it later merges, and hybrid-mode logits
  // are read only where the selection wrote them.
  return decode_attention_impl(q, k_pool, v_pool, block_table, prefix_lens, seq_lens, summaries, geom, mode, top_k,
                               eps, max_sel, rep_mode, n_splits, scratch, need, nullptr, nullptr, out, nullptr,
                               stream);
}

}  // extern "C"
