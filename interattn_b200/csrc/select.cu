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
// Layout of one ring stage (32 blocks = one warp tile, lane <-> block): rows
// are padded by 16 bytes so that the 32 lanes, each walking its own row with
// 16-byte loads, hit distinct banks; the query rows are read as warp-uniform
// broadcasts.
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

constexpr int kConsumerWarps = 4;
constexpr int kThreads = (kConsumerWarps + 1) * 32;  // + one TMA producer warp
constexpr int kTileBlocks = 32;
constexpr int kMaxStages = 8;
constexpr uint32_t kWaitPolls = 4u << 20;  // bounded mbarrier wait (~0.3 s), then give up

struct SelectParams {
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
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
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
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&o)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  o[0] = bf16lo(a.x); o[1] = bf16hi(a.x); o[2] = bf16lo(a.y); o[3] = bf16hi(a.y);
  o[4] = bf16lo(a.z); o[5] = bf16hi(a.z); o[6] = bf16lo(a.w); o[7] = bf16hi(a.w);
}

template <typename T, int D> struct TileLayout {
  static constexpr int kbar_row = D * 4 + 16;
  static constexpr int bnd_row = D * (int)sizeof(T) + 16;
  static constexpr int kbar_bytes = kTileBlocks * kbar_row;
  static constexpr int bnd_bytes = kTileBlocks * bnd_row;
  static constexpr int bytes = kbar_bytes + 2 * bnd_bytes;
  static constexpr int row_payload = D * 4 + 2 * D * (int)sizeof(T);
};

// exclusive block-wide scan of a 0/1 flag; returns this thread's prefix and the
// block total.  scratch: kThreads / 32 ints.  Contains two __syncthreads().
__device__ __forceinline__ int block_scan_flag(bool flag, int* scratch, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t bal = __ballot_sync(0xffffffffu, flag);
  const int within = __popc(bal & ((1u << lane) - 1u));
  if (lane == 0) scratch[warp] = __popc(bal);
  __syncthreads();
  int before = 0, sum = 0;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) {
    const int c = scratch[w];
    if (w < warp) before += c;
    sum += c;
  }
  __syncthreads();
  total = sum;
  return before + within;
}

template <typename T, int D, int G>
__global__ void __launch_bounds__(kThreads, 1) condition_block_select_kernel(SelectParams p) {
  using L = TileLayout<T, D>;
  extern __shared__ __align__(128) unsigned char smem_raw[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pair = blockIdx.x;  // (sequence, kv head)
  const int seq = pair / p.n_kv_heads;
  const int prefix = p.prefix_lens[seq];
  const int nb = min((prefix + p.block_size - 1) / p.block_size, p.max_blocks);
  const int n_tiles = (nb + kTileBlocks - 1) / kTileBlocks;
  const int nb_cap = p.nb_cap;

  // ---- shared memory carve-up -------------------------------------------------
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem_raw);
  uint64_t* empty_bar = full_bar + kMaxStages;
  int* hist = reinterpret_cast<int*>(empty_bar + kMaxStages);  // 256
  int* scan_scratch = hist + 256;                                // 8
  float* red_scratch = reinterpret_cast<float*>(scan_scratch + 8);  // 8
  float* norm_s = red_scratch + 8;   // z_m[G], z_l[G], denom[G], c_m[G], c_l[G]
  int* sel_state = reinterpret_cast<int*>(norm_s + 5 * 16);  // threshold key, take-equal, ...
  float* q_s = reinterpret_cast<float*>(sel_state + 8);  // [G][D]
  float* aq_s = q_s + G * D;                              // |q|
  float* vn_s = aq_s + G * D;                             // [nb_cap]
  float* score_s = vn_s + nb_cap;                         // [nb_cap]
  float* z_s = score_s + nb_cap;                          // [G][nb_cap]
  float* d_s = z_s + (size_t)G * nb_cap;                  // [G][nb_cap]
  unsigned char* stage_base = reinterpret_cast<unsigned char*>(
      (reinterpret_cast<uintptr_t>(d_s + (size_t)G * nb_cap) + 127) & ~uintptr_t(127));

  if (tid == 0) {
    for (int s = 0; s < p.n_stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
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
    // producer: one bulk copy per (block, vector); rows land padded
    const float* kbar_g = p.k_bar + sum_row0 * D;
    const T* kmax_g = static_cast<const T*>(p.k_max) + sum_row0 * D;
    const T* kmin_g = static_cast<const T*>(p.k_min) + sum_row0 * D;
    bool alive = true;
    for (int t = 0; t < n_tiles; ++t) {
      const int stage = t % p.n_stages;
      const int use = t / p.n_stages;
      if (use > 0 && alive) {
        if (!mbar_wait(&empty_bar[stage], (uint32_t)((use - 1) & 1))) {
          alive = false;
          if (lane == 0) atomicOr(&g_device_status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
        }
      }
      const int b0 = t * kTileBlocks;
      const int n_valid = min(kTileBlocks, nb - b0);
      unsigned char* st = stage_base + (size_t)stage * L::bytes;
      if (lane == 0) mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)(n_valid * L::row_payload));
      __syncwarp();
      if (lane < n_valid) {
        const int64_t r = (int64_t)(b0 + lane) * D;
        bulk_g2s(st + lane * L::kbar_row, kbar_g + r, D * 4, &full_bar[stage]);
        bulk_g2s(st + L::kbar_bytes + lane * L::bnd_row, kmax_g + r, D * (int)sizeof(T), &full_bar[stage]);
        bulk_g2s(st + L::kbar_bytes + L::bnd_bytes + lane * L::bnd_row, kmin_g + r, D * (int)sizeof(T),
                 &full_bar[stage]);
      }
    }
  } else {
    bool alive = true;
    for (int t = warp; t < n_tiles; t += kConsumerWarps) {
      const int stage = t % p.n_stages;
      const int use = t / p.n_stages;
      if (alive && !mbar_wait(&full_bar[stage], (uint32_t)(use & 1))) {
        alive = false;
        if (lane == 0) atomicOr(&g_device_status, DEV_STATUS_SELECT_WAIT_TIMEOUT);
      }
      const unsigned char* st = stage_base + (size_t)stage * L::bytes;
      const float* kbar_r = reinterpret_cast<const float*>(st + lane * L::kbar_row);
      const T* kmax_r = reinterpret_cast<const T*>(st + L::kbar_bytes + lane * L::bnd_row);
      const T* kmin_r = reinterpret_cast<const T*>(st + L::kbar_bytes + L::bnd_bytes + lane * L::bnd_row);
      float dot[G], mid[G], wid[G];
#pragma unroll
      for (int g = 0; g < G; ++g) { dot[g] = 0.f; mid[g] = 0.f; wid[g] = 0.f; }
#pragma unroll 2
      for (int c = 0; c < D; c += 8) {
        float kb[8], hi[8], lo[8];
        load8(kbar_r + c, kb);
        load8(kmax_r + c, hi);
        load8(kmin_r + c, lo);
        float ctr[8], span[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { ctr[i] = hi[i] + lo[i]; span[i] = hi[i] - lo[i]; }
#pragma unroll
        for (int g = 0; g < G; ++g) {
          float qv[8], av[8];
          load8(q_s + g * D + c, qv);   // warp-uniform address: a broadcast
          load8(aq_s + g * D + c, av);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dot[g] = fmaf(qv[i], kb[i], dot[g]);
            mid[g] = fmaf(qv[i], ctr[i], mid[g]);
            wid[g] = fmaf(av[i], span[i], wid[g]);
          }
        }
      }
      const int b = t * kTileBlocks + lane;
      if (b < nb) {
        const int count = min(p.block_size, prefix - b * p.block_size);
        const float logc = logf((float)count);
#pragma unroll
        for (int g = 0; g < G; ++g) {
          // sum_d max(q k_max, q k_min) = (mid + wid) / 2, sum_d min(...) = (mid - wid) / 2
          const float s = dot[g] / root;
          const float upper = (0.5f * (mid[g] + wid[g])) / root;
          const float lower = (0.5f * (mid[g] - wid[g])) / root;
          const float delta = fmaxf(fabsf(upper - s), fabsf(lower - s));
          z_s[g * nb_cap + b] = logc + s;
          d_s[g * nb_cap + b] = delta;
          if (p.aux.s != nullptr) p.aux.s[((int64_t)pair * G + g) * p.max_blocks + b] = s;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
  }
  __syncthreads();

  // ---- phase 2: per-row normalisers ---------------------------------------------
  // b_all = max_b v_norm_max[b]
  {
    float m = 0.f;
    for (int b = tid; b < nb; b += kThreads) m = fmaxf(m, vn_s[b]);
    m = warp_max(m);
    if (lane == 0) red_scratch[warp] = m;
  }
  __syncthreads();
  float b_all = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) b_all = fmaxf(b_all, red_scratch[w]);

  for (int g = warp; g < G; g += kThreads / 32) {
    const float* zr = z_s + g * nb_cap;
    const float* dr = d_s + g * nb_cap;
    float zm = -INFINITY, cm = -INFINITY;
    for (int b = lane; b < nb; b += 32) {
      zm = fmaxf(zm, zr[b]);
      const float dl = dr[b];
      const float lc = dl < 80.f ? logf(coshf(dl)) : dl - kLn2;
      cm = fmaxf(cm, zr[b] + lc);
    }
    zm = warp_max(zm);
    cm = warp_max(cm);
    float zl = 0.f, cl = 0.f;
    for (int b = lane; b < nb; b += 32) {
      zl += expf(zr[b] - zm);
      const float dl = dr[b];
      const float lc = dl < 80.f ? logf(coshf(dl)) : dl - kLn2;
      cl += expf(zr[b] + lc - cm);
    }
    zl = warp_sum(zl);
    cl = warp_sum(cl);
    // denom = sum_b softmax(z)_b cosh(delta_b), the way the eager reference forms it
    float dn = 0.f;
    for (int b = lane; b < nb; b += 32) dn += (expf(zr[b] - zm) / zl) * coshf(dr[b]);
    dn = fmaxf(warp_sum(dn), 1e-30f);
    if (lane == 0) {
      norm_s[0 * 16 + g] = zm; norm_s[1 * 16 + g] = zl; norm_s[2 * 16 + g] = dn;
      norm_s[3 * 16 + g] = cm; norm_s[4 * 16 + g] = cl;
    }
  }
  __syncthreads();

  // ---- phase 3: GQA-mean condition score -------------------------------------------
  for (int b = tid; b < nb; b += kThreads) {
    const float b_c = vn_s[b];
    float sum = 0.f;
#pragma unroll
    for (int g = 0; g < G; ++g) {
      const float z = z_s[g * nb_cap + b];
      const float dl = d_s[g * nb_cap + b];
      const float pm = expf(z - norm_s[g]) / norm_s[16 + g];
      const float ch = coshf(dl);
      const float cond = pm * (2.f * b_all * (ch - 1.f) / norm_s[32 + g] + 2.f * b_c * tanhf(dl * 0.5f));
      sum += cond;
    }
    score_s[b] = sum / (float)G;
  }
  __syncthreads();

  // optional diagnostics
  if (p.aux.score != nullptr)
    for (int b = tid; b < nb; b += kThreads) p.aux.score[(int64_t)pair * p.max_blocks + b] = score_s[b];
  if (p.aux.z != nullptr || p.aux.delta != nullptr) {
    for (int i = tid; i < G * nb; i += kThreads) {
      const int g = i / nb, b = i - g * nb;
      const int64_t o = ((int64_t)pair * G + g) * p.max_blocks + b;
      if (p.aux.z != nullptr) p.aux.z[o] = z_s[g * nb_cap + b];
      if (p.aux.delta != nullptr) p.aux.delta[o] = d_s[g * nb_cap + b];
    }
  }
  if (p.aux.globals != nullptr && tid < G) {
    // [batch, 4, rows]: z_m, z_l, c_m, c_l
    const int rows = p.n_kv_heads * G;
    const int head = pair - seq * p.n_kv_heads;
    float* gl = p.aux.globals + (int64_t)seq * 4 * rows + head * G + tid;
    gl[0 * rows] = norm_s[0 * 16 + tid];
    gl[1 * rows] = norm_s[1 * 16 + tid];
    gl[2 * rows] = norm_s[3 * 16 + tid];
    gl[3 * rows] = norm_s[4 * 16 + tid];
  }

  // ---- phase 4: routing ----------------------------------------------------------------
  int32_t* out_idx = p.sel_idx + (int64_t)pair * p.max_sel;
  uint32_t thr_key = 0;
  int take_equal = 0;
  if (p.mode == IA_SELECT_TOPK) {
    const int k_eff = min(min(p.top_k, nb), p.max_sel);
    if (k_eff > 0) {
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
          const bool here = (above < remaining) && (above + mine >= remaining);
          if (here) {
            int acc = above;
            int digit = 0;
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
  }

  int n_written = 0, n_equal_seen = 0;
  const bool any = (p.mode == IA_SELECT_EPS) ? (nb > 0) : (min(min(p.top_k, nb), p.max_sel) > 0);
  if (any) {
    for (int base = 0; base < nb; base += kThreads) {
      const int b = base + tid;
      const bool in = b < nb;
      const float sc = in ? score_s[b] : 0.f;
      bool take;
      if (p.mode == IA_SELECT_EPS) {
        take = in && (sc > p.eps);
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

template <typename T, int D, int G>
static int launch_typed(const SelectParams& base, int n_pairs, cudaStream_t stream) {
  using L = TileLayout<T, D>;
  SelectParams p = base;
  p.nb_cap = (p.max_blocks + 31) & ~31;
  const size_t fixed = 2 * kMaxStages * 8 + 256 * 4 + 8 * 4 + 8 * 4 + 5 * 16 * 4 + 8 * 4 +
                       2 * (size_t)G * D * 4 + (size_t)p.nb_cap * 4 * (2 + 2 * G) + 128;
  int dev = 0, max_smem = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  if (max_smem <= 0) max_smem = 227 * 1024;
  int stages = (int)(((size_t)max_smem - fixed) / L::bytes);
  if ((size_t)max_smem < fixed + 2 * (size_t)L::bytes)
    return fail(IA_ERR_UNSUPPORTED, "select: %d blocks x %d rows do not fit in shared memory", p.max_blocks, G);
  if (stages > kMaxStages) stages = kMaxStages;
  p.n_stages = stages;
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
