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
// once through a TMA (cp.async.bulk) + mbarrier shared-memory ring, keeps
// z = s + log(count) and the range bound delta of all G x n_blocks
// (row, block) pairs in shared memory, forms the two global normalisers, the
// GQA-mean score and then routes - a radix select for the k best blocks
// (higher score first, lower block index first among equal scores) or the
// reference's score > eps rule - without the score vector leaving the SM.
//
// Roofline: HBM.  Algorithmic bytes per block and kv head:
//   D*4 (k_bar f32) + 2*D*sizeof(T) (k_max, k_min) + 4 (v_norm_max).
//
// Layout of one ring stage (32 blocks, lane <-> block): rows are padded by 16
// bytes so that the 32 lanes, each walking its own row with 16-byte loads, hit
// distinct banks; the query rows are read as warp-uniform broadcasts.  A stage
// is consumed by a group of four warps, each taking a quarter of head_dim;
// their partial sums meet in shared memory, and each warp of the group then
// finishes the rows g = warp, warp + 4, ... (s, delta, z) - so sixteen compute
// warps stay busy on four stages while the producer fills the others.
#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through the runtime)

#include "ia_common.cuh"

namespace ia {

// Set by a kernel whose bounded mbarrier wait ran out (see mbar_wait below).
__device__ int g_device_status = 0;

int read_and_clear_device_status(int* out) {
  int v = 0, zero = 0;
  cudaError_t e = cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "device status: %s", cudaGetErrorString(e));
  *out = v;
  return IA_OK;
}

namespace {

constexpr int kGroups = 4;         // warp groups, one ring stage each at a time
constexpr int kGroupWarps = 4;     // warps per group: each takes head_dim / 4
constexpr int kConsumerWarps = kGroups * kGroupWarps;
constexpr int kWarps = kConsumerWarps + 1;  // + one TMA producer warp
constexpr int kThreads = kWarps * 32;
constexpr int kTileBlocks = 32;
constexpr int kMaxStages = 8;
constexpr uint32_t kWaitPolls = 4u << 20;  // bounded mbarrier wait (~0.3 s), then give up

struct SelectParams {
  // TMA descriptors of the three summary arrays viewed as [rows, D] matrices
  // (rows = batch * kv heads * max_blocks); box = 128 bytes x 32 rows, 128-byte swizzle
  CUtensorMap tm_kbar, tm_kmax, tm_kmin;
  const void* q;
  const float* k_bar;
  const void* k_max;
  const void* k_min;
  const float* v_norm_max;
  const int32_t* prefix_lens;
  int n_kv_heads, max_blocks, block_size;
  int mode, top_k, max_sel;
  float eps;
  int32_t* sel_idx;
  int32_t* sel_count;
  ia_select_aux aux;
  int n_stages, nb_cap;
};

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
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
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
  for (uint32_t i = 0; i < kWaitPolls; ++i) {
    if (mbar_test(bar, parity)) return true;
    if (i > 64) __nanosleep(32);
  }
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
template <typename T, int D> struct TileLayout {
  static constexpr int box_bytes = 128 * kTileBlocks;
  static constexpr int kbar_boxes = D * 4 / 128;
  static constexpr int bnd_boxes = D * (int)sizeof(T) / 128;
  static constexpr int kbar_bytes = kbar_boxes * box_bytes;
  static constexpr int bnd_bytes = bnd_boxes * box_bytes;
  static constexpr int bytes = kbar_bytes + 2 * bnd_bytes;
  static constexpr int kbar_box_cols = 32;                    // floats per 128 bytes
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
template <int D, int G> struct SmemPlan {
  static constexpr size_t bars = 2 * kMaxStages * 8;
  static constexpr size_t hist = 256 * 4;
  static constexpr size_t scan = 32 * 4;
  static constexpr size_t red = (size_t)kWarps * 32 * 4;
  static constexpr size_t norm = 4 * 16 * 4;
  static constexpr size_t state = 8 * 4;
  static constexpr size_t qrows = 2 * (size_t)G * D * 4;
  static constexpr size_t part = (size_t)kConsumerWarps * 3 * G * 32 * 4;
  static constexpr size_t fixed = bars + hist + scan + red + norm + state + qrows + part;
  static size_t per_blocks(int nb_cap) { return (size_t)nb_cap * 4 * (2 + 2 * G); }
};

// exclusive block-wide scan of a 0/1 flag; returns this thread's prefix and the
// block total.  scratch: kWarps ints.  Contains two __syncthreads().
__device__ __forceinline__ int block_scan_flag(bool flag, int* scratch, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t bal = __ballot_sync(0xffffffffu, flag);
  const int within = __popc(bal & ((1u << lane) - 1u));
  if (lane == 0) scratch[warp] = __popc(bal);
  __syncthreads();
  int before = 0, sum = 0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    const int c = scratch[w];
    if (w < warp) before += c;
    sum += c;
  }
  __syncthreads();
  total = sum;
  return before + within;
}

template <typename T, int D, int G>
__global__ void __launch_bounds__(kThreads, 1)
condition_block_select_kernel(const __grid_constant__ SelectParams p) {
  using L = TileLayout<T, D>;
  using P = SmemPlan<D, G>;
  constexpr int DQ = D / kGroupWarps;  // head_dim slice of one warp of a group
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pair = blockIdx.x;  // (sequence, kv head)
  const int seq = pair / p.n_kv_heads;
  const int prefix = p.prefix_lens[seq];
  const int nb = min((prefix + p.block_size - 1) / p.block_size, p.max_blocks);
  const int n_tiles = (nb + kTileBlocks - 1) / kTileBlocks;
  const int nb_cap = p.nb_cap;

  // ---- shared memory carve-up -------------------------------------------------
  unsigned char* sp = smem_raw;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(sp);
  uint64_t* empty_bar = full_bar + kMaxStages;         sp += P::bars;
  int* hist = reinterpret_cast<int*>(sp);              sp += P::hist;
  int* scan_scratch = reinterpret_cast<int*>(sp);      sp += P::scan;
  float* red_s = reinterpret_cast<float*>(sp);         sp += P::red;    // [kWarps][32]
  float* norm_s = reinterpret_cast<float*>(sp);        sp += P::norm;   // z_m[16], z_l[16], denom[16], b_all
  int* sel_state = reinterpret_cast<int*>(sp);         sp += P::state;
  float* q_s = reinterpret_cast<float*>(sp);                            // [G][D]
  float* aq_s = q_s + G * D;                           sp += P::qrows;  // |q|
  float* part_s = reinterpret_cast<float*>(sp);        sp += P::part;   // [consumer warp][3G][32]
  float* vn_s = reinterpret_cast<float*>(sp);                           // [nb_cap]
  float* score_s = vn_s + nb_cap;                                       // [nb_cap]
  float* z_s = score_s + nb_cap;                                        // [G][nb_cap]: z, later exp(z - z_m)
  float* d_s = z_s + (size_t)G * nb_cap;                                // [G][nb_cap]: delta, later exp(delta)
  unsigned char* stage_base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(d_s + (size_t)G * nb_cap) + 1023) & ~uintptr_t(1023));

  if (tid == 0) {
    for (int s = 0; s < p.n_stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], kGroupWarps);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  const T* qrow = static_cast<const T*>(p.q) + (int64_t)pair * G * D;
  for (int i = tid; i < G * D; i += kThreads) {
    const float v = to_f32(qrow[i]);
    q_s[i] = v;
    aq_s[i] = fabsf(v);
  }
  const float* vn_g = p.v_norm_max + (int64_t)pair * p.max_blocks;
  for (int b = tid; b < nb; b += kThreads) vn_s[b] = vn_g[b];
  __syncthreads();

  const float root = sqrtf((float)D);
  const int64_t sum_row0 = (int64_t)pair * p.max_blocks;  // first summary row of this pair

  // ---- phase 1: stream the summaries, s / delta per (row, block) -----------------
  if (warp == kConsumerWarps) {
    // producer: one elected lane issues the TMA box copies of each stage
    bool alive = true;
    const int row0 = (int)sum_row0;
    for (int t = 0; t < n_tiles; ++t) {
      const int stage = t % p.n_stages;
      const int use = t / p.n_stages;
      if (use > 0 && alive) {
        if (!mbar_wait(&empty_bar[stage], (uint32_t)((use - 1) & 1))) {
          alive = false;
          if (lane == 0) atomicOr(&g_device_status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
        }
      }
      if (lane == 0) {
        unsigned char* st = stage_base + (size_t)stage * L::bytes;
        const int y = row0 + t * kTileBlocks;  // rows past the array are zero-filled by the TMA unit
        mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)L::bytes);
#pragma unroll
        for (int j = 0; j < L::kbar_boxes; ++j)
          tma_load_2d(st + j * L::box_bytes, &p.tm_kbar, j * L::kbar_box_cols, y, &full_bar[stage]);
#pragma unroll
        for (int j = 0; j < L::bnd_boxes; ++j) {
          tma_load_2d(st + L::kbar_bytes + j * L::box_bytes, &p.tm_kmax, j * L::bnd_box_cols, y, &full_bar[stage]);
          tma_load_2d(st + L::kbar_bytes + L::bnd_bytes + j * L::box_bytes, &p.tm_kmin, j * L::bnd_box_cols, y,
                      &full_bar[stage]);
        }
      }
      __syncwarp();
    }
  } else {
    const int group = warp / kGroupWarps, wq = warp % kGroupWarps;
    float* my_part = part_s + (size_t)warp * 3 * G * 32;
    const float* grp_part = part_s + (size_t)group * kGroupWarps * 3 * G * 32;
    bool alive = true;
    for (int t = group; t < n_tiles; t += kGroups) {
      const int stage = t % p.n_stages;
      const int use = t / p.n_stages;
      if (alive && !mbar_wait(&full_bar[stage], (uint32_t)(use & 1))) {
        alive = false;
        if (lane == 0) atomicOr(&g_device_status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
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
        load4(swz<float>(kbar_v, lane, e0), kb);
        load4(swz<float>(kbar_v, lane, e0 + 4), kb + 4);
        if constexpr (sizeof(T) == 2) {
          load8(swz<T>(kmax_v, lane, e0), hi);
          load8(swz<T>(kmin_v, lane, e0), lo);
        } else {
          load4(swz<float>(kmax_v, lane, e0), hi);
          load4(swz<float>(kmax_v, lane, e0 + 4), hi + 4);
          load4(swz<float>(kmin_v, lane, e0), lo);
          load4(swz<float>(kmin_v, lane, e0 + 4), lo + 4);
        }
        float ctr[8], span[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { ctr[i] = hi[i] + lo[i]; span[i] = hi[i] - lo[i]; }
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
        const float logc = logf((float)count);
        for (int g = wq; g < G; g += kGroupWarps) {
          float v[3];
#pragma unroll
          for (int j = 0; j < 3; ++j) {
            float acc = 0.f;
#pragma unroll
            for (int w = 0; w < kGroupWarps; ++w) acc += grp_part[((size_t)w * 3 * G + g * 3 + j) * 32 + lane];
            v[j] = acc;
          }
          // sum_d max(q k_max, q k_min) = (mid + wid) / 2, sum_d min(...) = (mid - wid) / 2
          const float s = v[0] / root;
          const float upper = (0.5f * (v[1] + v[2])) / root;
          const float lower = (0.5f * (v[1] - v[2])) / root;
          const float delta = fmaxf(fabsf(upper - s), fabsf(lower - s));
          const float z = logc + s;
          z_s[g * nb_cap + b] = z;
          d_s[g * nb_cap + b] = delta;
          const int64_t o = ((int64_t)pair * G + g) * p.max_blocks + b;
          if (p.aux.s != nullptr) p.aux.s[o] = s;
          if (p.aux.z != nullptr) p.aux.z[o] = z;
          if (p.aux.delta != nullptr) p.aux.delta[o] = delta;
        }
      }
      group_sync(group);  // partial sums may be overwritten from here on
    }
  }
  __syncthreads();

  // ---- phase 2: per-row normalisers (all threads) ----------------------------------
  {
    float zmax[G];
#pragma unroll
    for (int g = 0; g < G; ++g) zmax[g] = -INFINITY;
    float bmax = 0.f;
    for (int b = tid; b < nb; b += kThreads) {
      bmax = fmaxf(bmax, vn_s[b]);
#pragma unroll
      for (int g = 0; g < G; ++g) zmax[g] = fmaxf(zmax[g], z_s[g * nb_cap + b]);
    }
    bmax = warp_max(bmax);
#pragma unroll
    for (int g = 0; g < G; ++g) zmax[g] = warp_max(zmax[g]);
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) red_s[warp * 32 + g] = zmax[g];
      red_s[warp * 32 + 31] = bmax;
    }
  }
  __syncthreads();
  if (tid < G) {
    float m = -INFINITY;
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, red_s[w * 32 + tid]);
    norm_s[tid] = m;
  } else if (tid == 31) {
    float m = 0.f;
    for (int w = 0; w < kWarps; ++w) m = fmaxf(m, red_s[w * 32 + 31]);
    norm_s[48] = m;
  }
  __syncthreads();
  {
    // z_l = sum_b exp(z - z_m);  dn = sum_b exp(z - z_m) cosh(delta).  The arrays are
    // rewritten in place with exp(z - z_m) and exp(delta) for the scoring pass.
    float zl[G], dn[G];
#pragma unroll
    for (int g = 0; g < G; ++g) { zl[g] = 0.f; dn[g] = 0.f; }
    for (int b = tid; b < nb; b += kThreads) {
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float ez = expf(z_s[g * nb_cap + b] - norm_s[g]);
        const float e = expf(d_s[g * nb_cap + b]);
        const float ch = 0.5f * (e + 1.f / e);
        zl[g] += ez;
        dn[g] = fmaf(ez, ch, dn[g]);
        z_s[g * nb_cap + b] = ez;
        d_s[g * nb_cap + b] = e;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) { zl[g] = warp_sum(zl[g]); dn[g] = warp_sum(dn[g]); }
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < G; ++g) { red_s[warp * 32 + g] = zl[g]; red_s[warp * 32 + 16 + g] = dn[g]; }
    }
  }
  __syncthreads();
  if (tid < G) {
    float zl = 0.f, dn = 0.f;
    for (int w = 0; w < kWarps; ++w) { zl += red_s[w * 32 + tid]; dn += red_s[w * 32 + 16 + tid]; }
    norm_s[16 + tid] = zl;
    norm_s[32 + tid] = fmaxf(dn / zl, 1e-30f);  // sum_b softmax(z)_b cosh(delta_b)
    if (p.aux.globals != nullptr) {
      // [batch, 4, rows]: (z_m, z_l) and a normaliser pair (c_m, c_l) with
      // c_l e^{c_m} = sum_b e^{z_b} cosh(delta_b); here c_m = z_m.
      const int rows = p.n_kv_heads * G;
      const int head = pair - seq * p.n_kv_heads;
      float* gl = p.aux.globals + (int64_t)seq * 4 * rows + head * G + tid;
      gl[0 * rows] = norm_s[tid];
      gl[1 * rows] = zl;
      gl[2 * rows] = norm_s[tid];
      gl[3 * rows] = dn;
    }
  }
  __syncthreads();

  // ---- phase 3: GQA-mean condition score -------------------------------------------
  {
    const float b_all = norm_s[48];
    for (int b = tid; b < nb; b += kThreads) {
      const float b_c = vn_s[b];
      float sum = 0.f;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pm = z_s[g * nb_cap + b] / norm_s[16 + g];
        const float e = d_s[g * nb_cap + b];
        const float ch = 0.5f * (e + 1.f / e);
        const float th = 1.f - 2.f / (e + 1.f);  // tanh(delta / 2)
        sum += pm * (2.f * b_all * (ch - 1.f) / norm_s[32 + g] + 2.f * b_c * th);
      }
      const float sc = sum / (float)G;
      score_s[b] = sc;
      if (p.aux.score != nullptr) p.aux.score[(int64_t)pair * p.max_blocks + b] = sc;
    }
  }
  __syncthreads();

  // ---- phase 4: routing ----------------------------------------------------------------
  int32_t* out_idx = p.sel_idx + (int64_t)pair * p.max_sel;
  uint32_t thr_key = 0;
  int take_equal = 0;
  const int k_eff = (p.mode == IA_SELECT_TOPK) ? min(min(p.top_k, nb), p.max_sel) : 0;
  if (k_eff > 0 && k_eff < nb) {
    uint32_t fixed = 0, fixed_mask = 0;
    int remaining = k_eff;
    for (int pass = 0; pass < 4; ++pass) {
      const int shift = 24 - 8 * pass;
      for (int i = tid; i < 256; i += kThreads) hist[i] = 0;
      __syncthreads();
      for (int b = tid; b < nb; b += kThreads) {
        const uint32_t key = order_key(score_s[b]);
        if ((key & fixed_mask) == fixed) atomicAdd(&hist[(key >> shift) & 255u], 1);
      }
      __syncthreads();
      if (warp == 0) {
        // lane owns bins [8*lane, 8*lane+8); walk from the top digit down
        int mine = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) mine += hist[lane * 8 + i];
        int above = 0;  // keys in the bins owned by higher lanes
        for (int l = 31; l >= 0; --l) {
          const int v = __shfl_sync(0xffffffffu, mine, l);
          if (l > lane) above += v;
        }
        if ((above < remaining) && (above + mine >= remaining)) {
          int acc = above, digit = 0;
          for (int i = 7; i >= 0; --i) {
            const int c = hist[lane * 8 + i];
            if (acc + c >= remaining) { digit = lane * 8 + i; break; }
            acc += c;
          }
          sel_state[0] = (int)(fixed | ((uint32_t)digit << shift));
          sel_state[1] = remaining - acc;
        }
      }
      __syncthreads();
      fixed = (uint32_t)sel_state[0];
      remaining = sel_state[1];
      fixed_mask |= 255u << shift;
      __syncthreads();
    }
    thr_key = fixed;
    take_equal = remaining;
  }

  int n_written = 0, n_equal_seen = 0;
  const bool any = (p.mode == IA_SELECT_EPS) ? (nb > 0) : (k_eff > 0);
  if (any) {
    const bool everything = (p.mode == IA_SELECT_TOPK) && (k_eff >= nb);
    for (int base = 0; base < nb; base += kThreads) {
      const int b = base + tid;
      const bool in = b < nb;
      const float sc = in ? score_s[b] : 0.f;
      bool take;
      if (p.mode == IA_SELECT_EPS) {
        take = in && (sc > p.eps);
      } else if (everything) {
        take = in;
      } else {
        const uint32_t key = order_key(sc);
        const bool eq = in && key == thr_key;
        int eq_total;
        const int eq_before = block_scan_flag(eq, scan_scratch, eq_total);
        take = in && (key > thr_key || (eq && n_equal_seen + eq_before < take_equal));
        n_equal_seen += eq_total;
      }
      int total;
      const int pos = block_scan_flag(take, scan_scratch, total);
      if (take && n_written + pos < p.max_sel) out_idx[n_written + pos] = b;
      n_written += total;
    }
  }
  const int count = min(n_written, p.max_sel);
  for (int i = count + tid; i < p.max_sel; i += kThreads) out_idx[i] = -1;
  if (tid == 0) p.sel_count[pair] = count;
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

// a [rows, D] row-major matrix cut into boxes of 128 bytes x 32 rows with the 128-byte swizzle
static int encode_rows(CUtensorMap* tm, const void* base, bool is_bf16, int64_t rows, int D) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return fail(IA_ERR_LAUNCH, "select: cuTensorMapEncodeTiled is not available from this driver");
  const int esz = is_bf16 ? 2 : 4;
  const cuuint64_t dims[2] = {(cuuint64_t)D, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)D * esz};
  const cuuint32_t box[2] = {(cuuint32_t)(128 / esz), (cuuint32_t)kTileBlocks};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                         const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(IA_ERR_LAUNCH, "select: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return IA_OK;
}

template <typename T, int D, int G>
static int launch_typed(const SelectParams& base, int n_pairs, cudaStream_t stream) {
  using L = TileLayout<T, D>;
  using P = SmemPlan<D, G>;
  SelectParams p = base;
  p.nb_cap = (p.max_blocks + 31) & ~31;
  const size_t fixed = P::fixed + P::per_blocks(p.nb_cap) + 1024;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (max_smem <= 0) max_smem = 227 * 1024;
  if ((size_t)max_smem < fixed + 2 * (size_t)L::bytes)
    return fail(IA_ERR_UNSUPPORTED, "select: %d blocks x %d query rows per kv head do not fit in shared memory",
                p.max_blocks, G);
  int stages = (int)(((size_t)max_smem - fixed) / L::bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p.n_stages = stages;
  const int64_t rows = (int64_t)n_pairs * p.max_blocks;
  if (rows > 0x7fffffff) return fail(IA_ERR_UNSUPPORTED, "select: %lld summary rows exceed the TMA coordinate range", (long long)rows);
  if (int s = encode_rows(&p.tm_kbar, p.k_bar, false, rows, D)) return s;
  if (int s = encode_rows(&p.tm_kmax, p.k_max, sizeof(T) == 2, rows, D)) return s;
  if (int s = encode_rows(&p.tm_kmin, p.k_min, sizeof(T) == 2, rows, D)) return s;
  const size_t smem = fixed + (size_t)stages * L::bytes;
  auto kern = condition_block_select_kernel<T, D, G>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "select: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  kern<<<n_pairs, kThreads, smem, stream>>>(p);
  return check_launch("condition_block_select_kernel");
}

template <typename T, int D>
static int launch_group(const SelectParams& p, int n_pairs, int group, cudaStream_t stream) {
  switch (group) {
    case 1: return launch_typed<T, D, 1>(p, n_pairs, stream);
    case 2: return launch_typed<T, D, 2>(p, n_pairs, stream);
    case 4: return launch_typed<T, D, 4>(p, n_pairs, stream);
    case 8: return launch_typed<T, D, 8>(p, n_pairs, stream);
    case 16: return launch_typed<T, D, 16>(p, n_pairs, stream);
    default: return fail(IA_ERR_UNSUPPORTED, "select: group_size %d not built (1, 2, 4, 8, 16)", group);
  }
}

}  // namespace

int launch_select(const void* q, const ia_summaries& s, const int32_t* prefix_lens, const ia_geom& g,
                  int mode, int top_k, float eps, int max_sel, int32_t* sel_idx, int32_t* sel_count,
                  const ia_select_aux& aux, cudaStream_t stream) {
  SelectParams p{};
  p.q = q; p.k_bar = s.k_bar; p.k_max = s.k_max; p.k_min = s.k_min; p.v_norm_max = s.v_norm_max;
  p.prefix_lens = prefix_lens;
  p.n_kv_heads = g.n_kv_heads; p.max_blocks = g.max_blocks; p.block_size = g.block_size;
  p.mode = mode; p.top_k = top_k; p.max_sel = max_sel; p.eps = eps;
  p.sel_idx = sel_idx; p.sel_count = sel_count; p.aux = aux;
  const int n_pairs = g.batch * g.n_kv_heads;
  if (n_pairs <= 0) return IA_OK;
  if (g.dtype == IA_BF16) {
    if (g.head_dim == 128) return launch_group<__nv_bfloat16, 128>(p, n_pairs, g.group_size, stream);
    if (g.head_dim == 64) return launch_group<__nv_bfloat16, 64>(p, n_pairs, g.group_size, stream);
  } else if (g.dtype == IA_F32) {
    if (g.head_dim == 128) return launch_group<float, 128>(p, n_pairs, g.group_size, stream);
    if (g.head_dim == 64) return launch_group<float, 64>(p, n_pairs, g.group_size, stream);
  }
  return fail(IA_ERR_UNSUPPORTED, "select: head_dim %d / dtype %d not built", g.head_dim, g.dtype);
}

}  // namespace ia
