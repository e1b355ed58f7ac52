// Paged sparse / hybrid decode attention - bf16 tensor-core kernels (sm_100a).
//
// Attention half of the reference's fused finalize kernel
// (llama/script/analysis/condition_block_gen/methods/condition_block_triton_impl/page_attention.py:173-309).
// Like the reference kernel it feeds bf16 q / K / V / probabilities to the
// tensor cores and keeps the softmax and the accumulators in fp32; unlike it,
// the pages to visit are known up front (an index list through a block
// table), so nothing in the load path depends on a computed value:
//
//   * item descriptors (physical page, valid rows) are resolved by all
//     threads of a CTA at once and parked in shared memory;
//   * each of the four warps runs its own ring of NS stages: a stage holds
//     one 16-token K page and V page (2 * 16 * D * 2 bytes), filled with
//     16-byte cp.async copies into an XOR-swizzled layout (zero-filled for
//     rows outside the valid range), so up to 4 * (NS - 1) pages per CTA are
//     in flight and ldmatrix reads are bank-conflict free;
//   * per page: S = Q K^T as 2 x (D/16) m16n8k16 MMAs (the G <= 16 query rows
//     of the kv head padded to 16), online softmax on the accumulator
//     fragments, O += P V as D/8 MMAs with P re-used straight from the S
//     fragments.
//
// Two grids share that warp-level code:
//   * pair grid - one CTA per (sequence, kv head, split); the four warps'
//     (m, l, O) are merged through shared memory into one normalised partial
//     (o, lse) per split.  The public ia_sparse_decode (partials out), block
//     ranges and the peer exchange use it.
//   * flat grid - the one-call layer-step.  The items of all pairs form one
//     list and each of 2 x SMs CTAs owns an equal contiguous slice of it, so
//     every resident CTA slot streams the same number of pages whatever the
//     batch, the top-k or how ragged the lengths are; a slice may end inside
//     one pair and start the next.  The warps' rings never drain at a pair
//     boundary: at the end of a (CTA, pair) segment the four warps merge
//     through the one ring stage each of them has free at that moment, the
//     CTA writes one partial, and the CTA that completes a pair last merges
//     the pair's partials and writes the output rows.
//
// Roofline: HBM.  Algorithmic bytes: 2 * D * 2 bytes per attended token
// (K and V row), D * 2 per representative.  Arithmetic intensity is 2 G / 2
// flop per byte, far below the ridge, so the tensor cores idle most of the time;
// they are used because fp32 FMAs alone would cap the kernel near half of HBM
// speed at G = 4 and below it at G = 8.
#include <stdlib.h>
#include <string.h>

#include "decode_items.cuh"

namespace ia {

namespace {

constexpr int kWarps = 4;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D(16x8, f32) += A(16x16, bf16 row-major) * B(16x8, bf16 col-major)
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// barrier among `threads` threads of the CTA (ids 1..15; 0 is __syncthreads)
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// What one warp holds while it walks its items: the query fragments of the current (sequence, kv
// head), the running softmax state and the output accumulators, plus the two operations on a ring
// stage.  Both grids inline these; nothing here is shared between warps.
template <int D, int NS, bool HI_ROWS> struct WarpAttention {
  using bf16 = __nv_bfloat16;
  static constexpr int ROW_BYTES = D * 2;               // one token row of a tile
  static constexpr int CHUNKS = ROW_BYTES / 16;         // 16-byte chunks per row
  static constexpr int TILE_BYTES = 16 * ROW_BYTES;     // one K or V page
  static constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  static constexpr int KSTEPS = D / 16;
  static constexpr int NT_O = D / 8;
  static constexpr int COPIES = 16 * CHUNKS / 32;       // 16-byte copies per lane per tile

  uint32_t qa[KSTEPS][4];
  float o[NT_O][4];
  float m0, m1, l0, l1;  // log2 domain; l: this thread's share
  int lane, quad, qlane, G;
  float sc_qk;
  unsigned char* ring;  // this warp's NS stages
  uint32_t ring_u32;

  __device__ __forceinline__ void init(int lane_, int G_, unsigned char* my_ring) {
    lane = lane_; quad = lane_ >> 2; qlane = lane_ & 3; G = G_;
    sc_qk = kLog2e / sqrtf((float)D);
    ring = my_ring;
    ring_u32 = smem_u32(my_ring);
    reset();
  }
  __device__ __forceinline__ void reset() {
#pragma unroll
    for (int j = 0; j < NT_O; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
    m0 = -INFINITY; m1 = -INFINITY; l0 = 0.f; l1 = 0.f;
  }
  // Q rows [G, D] of one (sequence, kv head) as A fragments (rows >= G are zero)
  __device__ __forceinline__ void load_q(const bf16* qp) {
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d0 = kk * 16 + qlane * 2;
      qa[kk][0] = quad < G ? *reinterpret_cast<const uint32_t*>(qp + quad * D + d0) : 0u;
      qa[kk][1] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(qp + (quad + 8) * D + d0) : 0u;
      qa[kk][2] = quad < G ? *reinterpret_cast<const uint32_t*>(qp + quad * D + d0 + 8) : 0u;
      qa[kk][3] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(qp + (quad + 8) * D + d0 + 8) : 0u;
    }
  }

  // Fill one stage: K tile then V tile, swizzled, rows outside [lo, hi) zero-filled.  ksrc null:
  // a tile of representatives - vsrc is then 16 v_bar rows and zsrc / z_stride give their logits
  // z[row][block], which ride in the unused K half of the stage as [16 rows][16 blocks] floats, so
  // that consume() does not wait on global loads.
  __device__ __forceinline__ void issue(int stage, int lo, int hi, const bf16* ksrc, const bf16* vsrc,
                                        const float* zsrc, int64_t z_stride) {
    if (hi <= lo) return;
    const uint32_t kdst = ring_u32 + stage * STAGE_BYTES;
    const uint32_t vdst = kdst + TILE_BYTES;
#pragma unroll
    for (int c = 0; c < COPIES; ++c) {
      const int id = c * 32 + lane;
      const int row = id / CHUNKS, ch = id % CHUNKS;
      const bool live = row >= lo && row < hi;
      const int srow = live ? row : lo;  // keep the address in bounds; nothing is read when !live
      const uint32_t off = row * ROW_BYTES + ((ch ^ (row & 7)) << 4);
      if (ksrc != nullptr) cp_async16(kdst + off, ksrc + srow * D + ch * 8, live ? 16u : 0u);
      cp_async16(vdst + off, vsrc + srow * D + ch * 8, live ? 16u : 0u);
    }
    if (ksrc == nullptr) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int id = c * 32 + lane;
        const int row = id >> 4, tok = id & 15;
        if (row < G && tok < hi) cp_async4(kdst + id * 4, zsrc + (int64_t)row * z_stride + tok);
      }
    }
  }

  // One stage into the running state.  is_page: S = Q K^T; else the logits staged by issue(), where
  // bit t of rep_skip drops representative t (its block is selected and attended token by token).
  __device__ __forceinline__ void consume(int stage, int lo, int hi, bool is_page, uint32_t rep_skip) {
    if (hi <= lo) return;
    const uint32_t ktile = ring_u32 + stage * STAGE_BYTES;
    const uint32_t vtile = ktile + TILE_BYTES;
    float s[2][4];
    if (is_page) {
#pragma unroll
      for (int t = 0; t < 2; ++t) { s[t][0] = 0.f; s[t][1] = 0.f; s[t][2] = 0.f; s[t][3] = 0.f; }
      const int mat = lane >> 3, rr = lane & 7;
      const int token = (mat >> 1) * 8 + rr;
#pragma unroll
      for (int kk = 0; kk < KSTEPS; ++kk) {
        const int ch = kk * 2 + (mat & 1);
        uint32_t b[4];
        ldmatrix_x4(ktile + token * ROW_BYTES + ((ch ^ (token & 7)) << 4), b);
        mma_bf16(s[0], qa[kk], b[0], b[1]);
        mma_bf16(s[1], qa[kk], b[2], b[3]);
      }
#pragma unroll
      for (int t = 0; t < 2; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = t * 8 + qlane * 2 + (e & 1);
          const bool ok = tok >= lo && tok < hi;
          s[t][e] = ok ? s[t][e] * sc_qk : -INFINITY;
        }
      }
    } else {
      // representatives: logits come from the selection pass (z = s + log count)
      const float* zt = reinterpret_cast<const float*>(ring + (size_t)stage * STAGE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = t * 8 + qlane * 2 + (e & 1);
          const int row = quad + (e >> 1) * 8;
          const bool ok = tok < hi && row < G && ((rep_skip >> tok) & 1u) == 0u;
          s[t][e] = ok ? zt[row * 16 + tok] * kLog2e : -INFINITY;
        }
      }
    }
    // online softmax, row `quad` (and quad + 8 when G > 8)
    float t0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
    t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
    const float n0 = fmaxf(m0, t0);
    const float ref0 = n0 == -INFINITY ? 0.f : n0;
    const float a0 = exp2f(m0 - ref0);
    m0 = n0;
    float p00 = exp2f(s[0][0] - ref0), p01 = exp2f(s[0][1] - ref0);
    float p10 = exp2f(s[1][0] - ref0), p11 = exp2f(s[1][1] - ref0);
    l0 = l0 * a0 + (p00 + p01 + p10 + p11);
    uint32_t pa[4];
    pa[0] = pack_bf16(p00, p01);
    pa[2] = pack_bf16(p10, p11);
    float a1 = 1.f;
    if constexpr (HI_ROWS) {
      float t1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
      t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
      const float n1 = fmaxf(m1, t1);
      const float ref1 = n1 == -INFINITY ? 0.f : n1;
      a1 = exp2f(m1 - ref1);
      m1 = n1;
      float p02 = exp2f(s[0][2] - ref1), p03 = exp2f(s[0][3] - ref1);
      float p12 = exp2f(s[1][2] - ref1), p13 = exp2f(s[1][3] - ref1);
      l1 = l1 * a1 + (p02 + p03 + p12 + p13);
      pa[1] = pack_bf16(p02, p03);
      pa[3] = pack_bf16(p12, p13);
    } else {
      pa[1] = 0u;
      pa[3] = 0u;
    }
#pragma unroll
    for (int j = 0; j < NT_O; ++j) {
      o[j][0] *= a0; o[j][1] *= a0;
      if constexpr (HI_ROWS) { o[j][2] *= a1; o[j][3] *= a1; }
    }
    // O += P V
    {
      const int mat = lane >> 3, rr = lane & 7;
      const int token = (mat & 1) * 8 + rr;
#pragma unroll
      for (int j = 0; j < NT_O; j += 2) {
        const int ch = j + (mat >> 1);
        uint32_t b[4];
        ldmatrix_x4_trans(vtile + token * ROW_BYTES + ((ch ^ (token & 7)) << 4), b);
        mma_bf16(o[j], pa, b[0], b[1]);
        mma_bf16(o[j + 1], pa, b[2], b[3]);
      }
    }
  }

  // the quad's shares of l into every lane of the quad
  __device__ __forceinline__ void reduce_l() {
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  }
};

// ---- pair grid: one CTA per (sequence, kv head, split) ---------------------------------
template <int D, int NS, bool HI_ROWS>
__global__ void __launch_bounds__(kWarps * 32, 2)
condition_block_finalize_attention_kernel(DecodeParams p) {
  using W = WarpAttention<D, NS, HI_ROWS>;
  using bf16 = __nv_bfloat16;
  constexpr int STAGE_BYTES = W::STAGE_BYTES, NT_O = W::NT_O;

  extern __shared__ __align__(128) unsigned char smem[];
  Item* items_s = reinterpret_cast<Item*>(smem);
  unsigned char* ring = smem + kItemChunk * sizeof(Item);
  uint32_t* sel_bits = reinterpret_cast<uint32_t*>(ring + (size_t)kWarps * NS * STAGE_BYTES);
  __shared__ int scratch[2];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int quad = lane >> 2, qlane = lane & 3;
  const int split = blockIdx.x % p.n_splits;
  const int pair = blockIdx.x / p.n_splits;
  const int head = pair % p.n_kv_heads, seq = pair / p.n_kv_heads;
  const int G = p.group_size;
  const int rows = p.n_kv_heads * G;

  // Let the next kernel on the stream start filling SMs as this grid drains, then wait
  // for the selection kernel: everything below reads what it wrote.
  IA_DTRACE_BEGIN();
  grid_launch_dependents();
  grid_dependency_wait();
  IA_DTRACE(0);
  ExchangeView xv{};
  if (p.px.n_ranks > 0) xv = exchange_view(p);
  const ItemRange r = item_range(p, seq, head, split, scratch);
  IA_DTRACE(1);
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

  W w;
  w.init(lane, G, ring + (size_t)warp * NS * STAGE_BYTES);
  w.load_q(static_cast<const bf16*>(p.q) + ((int64_t)seq * rows + head * G) * D);

  const bf16* kbase = static_cast<const bf16*>(p.k_pool) + (int64_t)head * p.head_stride;
  const bf16* vbase = static_cast<const bf16*>(p.v_pool) + (int64_t)head * p.head_stride;
  const bf16* vbar = static_cast<const bf16*>(p.v_bar) + (int64_t)pair * p.max_blocks * D;
  const float* zrow = p.z + ((int64_t)seq * rows + head * G) * p.max_blocks;

  auto issue = [&](const Item& it, int stage) {
    if (it.kind == ITEM_PAGE)
      w.issue(stage, it.lo, it.hi, kbase + (int64_t)it.first * p.page_stride, vbase + (int64_t)it.first * p.page_stride,
              nullptr, 0);
    else
      w.issue(stage, it.lo, it.hi, nullptr, vbar + (int64_t)it.first * D, zrow + it.first, p.max_blocks);
  };
  auto consume = [&](const Item& it, int stage) {
    uint32_t skip = 0u;
    if (it.kind != ITEM_PAGE) {
      // selected members of the tile: 16 consecutive bits of the pair's bitmap (first is a multiple of 16)
      skip = (sel_bits[it.first >> 5] >> (it.first & 31)) & 0xffffu;
    }
    w.consume(stage, it.lo, it.hi, it.kind == ITEM_PAGE, skip);
  };

  for (int chunk = r.begin; chunk < r.end; chunk += kItemChunk) {
    const int chunk_end = min(chunk + kItemChunk, r.end);
    __syncthreads();  // every warp is done with the previous descriptors
    resolve_items(p, r, seq, head, chunk, chunk_end, items_s);
    IA_DTRACE(2);
    const int n_mine = (chunk_end - chunk - warp + kWarps - 1) / kWarps;  // items warp, warp+4, ...
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {
      if (s < n_mine) issue(items_s[warp + s * kWarps], s);
      cp_async_commit();
    }
    for (int n = 0; n < n_mine; ++n) {
      const int ahead = n + NS - 1;
      if (ahead < n_mine) issue(items_s[warp + ahead * kWarps], ahead % NS);
      cp_async_commit();
      cp_async_wait<NS - 1>();
      __syncwarp();
      if (n == 0) IA_DTRACE(3);
      consume(items_s[warp + n * kWarps], n % NS);
      __syncwarp();
    }
    cp_async_wait<0>();
  }
  IA_DTRACE(4);

  // ---- merge the four warps ------------------------------------------------------------
  __syncthreads();  // all rings idle: reuse them as merge buffers
  IA_DTRACE(5);
  float* mo = reinterpret_cast<float*>(w.ring);               // [16][D]
  float* mm = reinterpret_cast<float*>(w.ring + 16 * D * 4);  // m[16], l[16]
  w.reduce_l();
#pragma unroll
  for (int j = 0; j < NT_O; ++j) {
    const int d = j * 8 + qlane * 2;
    *reinterpret_cast<float2*>(mo + quad * D + d) = make_float2(w.o[j][0], w.o[j][1]);
    if constexpr (HI_ROWS) *reinterpret_cast<float2*>(mo + (quad + 8) * D + d) = make_float2(w.o[j][2], w.o[j][3]);
  }
  if (qlane == 0) {
    mm[quad] = w.m0; mm[16 + quad] = w.l0;
    if constexpr (HI_ROWS) { mm[quad + 8] = w.m1; mm[16 + quad + 8] = w.l1; }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
    const int g = e / D, d = e - g * D;
    float top = -INFINITY;
#pragma unroll
    for (int ww = 0; ww < kWarps; ++ww)
      top = fmaxf(top, reinterpret_cast<const float*>(ring + (size_t)ww * NS * STAGE_BYTES + 16 * D * 4)[g]);
    float num = 0.f, den = 0.f;
    if (top > -INFINITY) {
#pragma unroll
      for (int ww = 0; ww < kWarps; ++ww) {
        const float* wo = reinterpret_cast<const float*>(ring + (size_t)ww * NS * STAGE_BYTES);
        const float* wm = wo + 16 * D;
        const float a = exp2f(wm[g] - top);
        num = fmaf(a, wo[g * D + d], num);
        den = fmaf(a, wm[16 + g], den);
      }
    }
    const int64_t orow = ((int64_t)seq * rows + head * G + g) * p.n_splits + split;
    const float ov = den > 0.f ? num / den : 0.f;
    const float lv = den > 0.f ? (top + log2f(den)) * kLn2 : -INFINITY;
    if (p.px.n_ranks > 0) {
      exchange_store(p, xv, orow * D + d, ov);
      if (d == 0) exchange_store(p, xv, p.px.lse_offset + orow, lv);
    } else if (p.final_out != nullptr && p.n_splits == 1) {
      // the pair's only part, inside the one-call step: this is the output row - same value, same
      // rounding as the merge of a single part (weight e^0 = 1, denominator 1), without the round
      // trip of the partial through global memory
      const int64_t at = ((int64_t)seq * rows + head * G + g) * D + d;
      if (p.final_dtype == IA_BF16) static_cast<bf16*>(p.final_out)[at] = __float2bfloat16_rn(ov);
      else static_cast<float*>(p.final_out)[at] = ov;
    } else {
      p.o_partial[orow * D + d] = ov;
      if (d == 0) p.lse_partial[orow] = lv;
    }
  }
  IA_DTRACE(6);
  if (p.px.n_ranks > 0) {
    exchange_publish(p, xv);
    return;
  }
  if (p.n_splits > 1) finish_pair<D>(p, seq, head, G, scratch);
  IA_DTRACE(7);
}

// ---- flat grid: equal contiguous shares of all pairs' items -------------------------------
// Shared memory: item descriptors, the rings, and the exclusive prefix sums of the pairs' item
// counts (n_pairs + 1 ints), which every CTA computes for itself from the selection counts and the
// lengths - a few loads per thread, so that no planning launch sits between selection and
// attention.
template <int D, int NS, bool HI_ROWS>
__global__ void __launch_bounds__(kWarps * 32, 2)
condition_block_finalize_attention_flat_kernel(DecodeParams p) {
  using W = WarpAttention<D, NS, HI_ROWS>;
  using bf16 = __nv_bfloat16;
  constexpr int STAGE_BYTES = W::STAGE_BYTES, NT_O = W::NT_O;
  constexpr int kThreads = kWarps * 32;

  extern __shared__ __align__(128) unsigned char smem[];
  FlatItem* items_s = reinterpret_cast<FlatItem*>(smem);
  unsigned char* ring = smem + kItemChunk * sizeof(FlatItem);
  int* pre_s = reinterpret_cast<int*>(ring + (size_t)kWarps * NS * STAGE_BYTES);  // [n_pairs + 1]
  __shared__ int warp_tot[kWarps];
  __shared__ int carry_s;
  __shared__ float seg_lse[kWarps][16];  // the warps' log-sum-exps of the segment being closed
  __shared__ int seg_stage[kWarps];      // ring stage in which each warp parked its partial

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = lane >> 2, qlane = lane & 3;
  const int G = p.group_size;
  const int n_pairs = p.n_pairs;
  const int cta = (int)blockIdx.x;
  const int ppb = p.block_size / p.page_size;

  grid_launch_dependents();
  grid_dependency_wait();

  // ---- exclusive prefix sums of the item counts -------------------------------------------
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < n_pairs; base += kThreads) {
    const int pr = base + tid;
    const int n = pr < n_pairs ? pair_items(p, pr).total() : 0;
    int incl = n;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = carry_s;
#pragma unroll
    for (int ww = 0; ww < kWarps; ++ww)
      if (ww < warp) before += warp_tot[ww];
    if (pr < n_pairs) pre_s[pr] = before + incl - n;
    __syncthreads();
    if (tid == kThreads - 1) carry_s = before + incl;
    __syncthreads();
  }
  if (tid == 0) pre_s[n_pairs] = carry_s;
  __syncthreads();
  const int64_t n_items = pre_s[n_pairs];

  // pairs with nothing to attend to have no segment anywhere: their output rows are zero
  for (int pr = cta; pr < n_pairs; pr += (int)gridDim.x) {
    if (pre_s[pr + 1] != pre_s[pr]) continue;
    for (int e = tid; e < G * D; e += kThreads) {
      const int64_t at = (int64_t)pr * G * D + e;
      if (p.final_dtype == IA_BF16) static_cast<bf16*>(p.final_out)[at] = __float2bfloat16_rn(0.f);
      else static_cast<float*>(p.final_out)[at] = 0.f;
    }
  }
  // With fewer items than CTAs only the first n_items CTAs work (one item each), so that every
  // CTA counted between the first and the last CTA of a pair really holds a segment of it.
  const int n_ctas = (int)min((int64_t)gridDim.x, n_items);
  if (cta >= n_ctas) return;
  const int s0 = (int)flat_slice_begin(n_items, cta, n_ctas), s1 = (int)flat_slice_begin(n_items, cta + 1, n_ctas);

  // pair that holds item i: the last pair whose prefix sum is <= i
  auto pair_of = [&](int i) {
    int lo = 0, hi = n_pairs;  // pre_s[lo] <= i < pre_s[hi]
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (pre_s[mid] <= i) lo = mid; else hi = mid;
    }
    return lo;
  };
  const int pair_first = pair_of(s0), pair_last = pair_of(s1 - 1);

  W w;
  w.init(lane, G, ring + (size_t)warp * NS * STAGE_BYTES);
  int cur_pair = pair_first;
  w.load_q(static_cast<const bf16*>(p.q) + (int64_t)cur_pair * G * D);

  const bf16* kpool = static_cast<const bf16*>(p.k_pool);
  const bf16* vpool = static_cast<const bf16*>(p.v_pool);

  auto issue = [&](const FlatItem& it, int stage) {
    const int lo = it.lohi_head & 0xff, hi = (it.lohi_head >> 8) & 0xff;
    if (it.kind_pair & 1) {
      const int pr = it.kind_pair >> 1;
      const bf16* vbar = static_cast<const bf16*>(p.v_bar) + ((int64_t)pr * p.max_blocks + it.first) * D;
      w.issue(stage, lo, hi, nullptr, vbar, p.z + (int64_t)pr * G * p.max_blocks + it.first, p.max_blocks);
    } else {
      const int64_t off = (int64_t)(it.lohi_head >> 16) * p.head_stride + (int64_t)it.first * p.page_stride;
      w.issue(stage, lo, hi, kpool + off, vpool + off, nullptr, 0);
    }
  };

  // End of the segment (cta, pair).  All four warps come here, in the same order for every pair of
  // the slice.  Each parks its normalised partial in the ring stage it is not using at that moment
  // (`free_stage`: consumed, not yet refilled) and they meet at a named barrier; each warp then merges
  // a quarter of the output elements over the four partials and writes it into the CTA's slot
  // (cta + pair) in global memory; after a second barrier (the stages may be refilled from here on)
  // warp 0 counts the CTA in at the pair, and the CTA that arrives last merges the pair's CTA
  // partials - in slot order, so the result does not depend on who that is - and writes the
  // output rows.
  auto flush_pair = [&](int pr, int free_stage) {
    w.reduce_l();
    {
      float* so = reinterpret_cast<float*>(w.ring + (size_t)free_stage * STAGE_BYTES);  // [G][D] of this warp
      const float inv0 = w.l0 > 0.f ? 1.f / w.l0 : 0.f;
      if (quad < G) {
#pragma unroll
        for (int j = 0; j < NT_O; ++j)
          *reinterpret_cast<float2*>(so + quad * D + j * 8 + qlane * 2) = make_float2(w.o[j][0] * inv0, w.o[j][1] * inv0);
        if (qlane == 0) seg_lse[warp][quad] = w.l0 > 0.f ? (w.m0 + log2f(w.l0)) * kLn2 : -INFINITY;
      }
      if constexpr (HI_ROWS) {
        const float inv1 = w.l1 > 0.f ? 1.f / w.l1 : 0.f;
        if (quad + 8 < G) {
#pragma unroll
          for (int j = 0; j < NT_O; ++j)
            *reinterpret_cast<float2*>(so + (quad + 8) * D + j * 8 + qlane * 2) =
                make_float2(w.o[j][2] * inv1, w.o[j][3] * inv1);
          if (qlane == 0) seg_lse[warp][quad + 8] = w.l1 > 0.f ? (w.m1 + log2f(w.l1)) * kLn2 : -INFINITY;
        }
      }
      if (lane == 0) seg_stage[warp] = free_stage;
    }
    w.reset();
    named_barrier(1, kThreads);
    const int64_t slot = (int64_t)cta + pr;
    {
      // elements [warp, warp + 1) * G * D / 4 of the segment's partial, four at a time
      const int per_warp = G * D / kWarps;
      for (int e = lane * 4; e < per_warp; e += 128) {
        const int at = warp * per_warp + e;
        const int g = at / D;
        float top = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < kWarps; ++ww) top = fmaxf(top, seg_lse[ww][g]);
        const float ref = top == -INFINITY ? 0.f : top;
        float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
        float den = 0.f;
#pragma unroll
        for (int ww = 0; ww < kWarps; ++ww) {
          const float wgt = expf(seg_lse[ww][g] - ref);  // exp(-inf) = 0 for a warp without items
          const float4 v = *reinterpret_cast<const float4*>(
              ring + ((size_t)ww * NS + seg_stage[ww]) * STAGE_BYTES + (size_t)at * 4);
          num.x = fmaf(wgt, v.x, num.x); num.y = fmaf(wgt, v.y, num.y);
          num.z = fmaf(wgt, v.z, num.z); num.w = fmaf(wgt, v.w, num.w);
          den += wgt;
        }
        const float inv = den > 0.f ? 1.f / den : 0.f;
        *reinterpret_cast<float4*>(p.flat_o + slot * G * D + at) =
            make_float4(num.x * inv, num.y * inv, num.z * inv, num.w * inv);
        if (at - g * D == 0) p.flat_lse[slot * G + g] = den > 0.f ? ref + logf(den) : -INFINITY;
      }
    }
    __threadfence();  // this thread's part of the CTA partial is visible device-wide ...
    named_barrier(2, kThreads);  // ... for every thread, before the CTA is counted in; stages are free again
    if (warp != 0) return;
    const int c_lo = flat_cta_of(n_items, pre_s[pr], n_ctas), c_hi = flat_cta_of(n_items, pre_s[pr + 1] - 1, n_ctas);
    const int n_parts = c_hi - c_lo + 1;
    int last = 0;
    if (lane == 0) {
      const int old = atomicAdd(&p.split_counters[pr], 1);
      last = old == n_parts - 1;
      if (last) p.split_counters[pr] = 0;  // ready for the next launch
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (!last) return;
    __threadfence();  // the other CTAs' partials, before this warp reads them (L2 loads below)
    const int64_t first_slot = (int64_t)c_lo + pr;  // consecutive slots c_lo + pr .. c_hi + pr
    for (int e = lane * 4; e < G * D; e += 128) {
      const int g = e / D;
      const float* lse = p.flat_lse + first_slot * G + g;
      const float* src = p.flat_o + first_slot * G * D + e;
      // one pass with a running maximum: the loads do not depend on it, so several parts are in flight
      float top = -INFINITY, den = 0.f;
      float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
      for (int s = 0; s < n_parts; ++s) {
        const float l = __ldcg(lse + (int64_t)s * G);
        const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (int64_t)s * G * D));
        const float nt = fmaxf(top, l);
        const float ref = nt == -INFINITY ? 0.f : nt;
        const float keep = expf(top - ref), wgt = expf(l - ref);  // exp(-inf) = 0 for an empty part
        num.x = fmaf(num.x, keep, wgt * v.x); num.y = fmaf(num.y, keep, wgt * v.y);
        num.z = fmaf(num.z, keep, wgt * v.z); num.w = fmaf(num.w, keep, wgt * v.w);
        den = fmaf(den, keep, wgt);
        top = nt;
      }
      const float inv = 1.f / fmaxf(den, 1e-30f);
      const int64_t at = (int64_t)pr * G * D + e;
      if (p.final_dtype == IA_BF16) {
        __nv_bfloat162 a = __floats2bfloat162_rn(num.x * inv, num.y * inv);
        __nv_bfloat162 b = __floats2bfloat162_rn(num.z * inv, num.w * inv);
        uint2 packed;
        packed.x = *reinterpret_cast<uint32_t*>(&a);
        packed.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(static_cast<bf16*>(p.final_out) + at) = packed;
      } else {
        *reinterpret_cast<float4*>(static_cast<float*>(p.final_out) + at) =
            make_float4(num.x * inv, num.y * inv, num.z * inv, num.w * inv);
      }
    }
  };
  // leave cur_pair (and any pair of this CTA's slice between it and `target`) behind
  auto advance_to = [&](int target, int free_stage) {
    while (cur_pair < target) {
      if (pre_s[cur_pair + 1] != pre_s[cur_pair]) flush_pair(cur_pair, free_stage);
      ++cur_pair;
    }
    if (cur_pair <= pair_last) w.load_q(static_cast<const bf16*>(p.q) + (int64_t)cur_pair * G * D);
  };

  for (int chunk = s0; chunk < s1; chunk += kItemChunk) {
    const int chunk_end = min(chunk + kItemChunk, s1);
    __syncthreads();  // every warp is done with the previous descriptors
    for (int i = chunk + tid; i < chunk_end; i += kThreads) {
      const int pr = pair_of(i);
      const int seq = pr / p.n_kv_heads, head = pr - seq * p.n_kv_heads;
      const PairItems pi = pair_items(p, pr);
      const int32_t* idx = p.sel_idx + (int64_t)pr * p.max_sel;
      const ResolvedItem ri = resolve_one(p, idx, p.block_table + (int64_t)seq * p.max_pages, i - pre_s[pr], 0,
                                          pi.n_sel_items, pi.n_rep, 0, pi.nb_eff, pi.suf_first_page, pi.prefix,
                                          pi.seq_len);
      FlatItem it;
      it.kind_pair = (ri.kind == ITEM_REP_TILE ? 1 : 0) | (pr << 1);
      it.first = ri.first;
      it.lohi_head = ri.lo | (ri.hi << 8) | (head << 16);
      it.mask = 0;
      if (ri.kind == ITEM_REP_TILE) {
        // selected members of the tile, from the ascending index list: first entry >= ri.first, then on
        const int count = pi.n_sel_items / ppb;
        int lo = 0, hi = count;
        while (lo < hi) {
          const int mid = (lo + hi) >> 1;
          if (idx[mid] < ri.first) lo = mid + 1; else hi = mid;
        }
        for (int j = lo; j < count; ++j) {
          const int b = idx[j] - ri.first;
          if (b < 0 || b >= kRepTile) break;
          it.mask |= 1 << b;
        }
      }
      items_s[i - chunk] = it;
    }
    __syncthreads();
    const int n_mine = (chunk_end - chunk - warp + kWarps - 1) / kWarps;  // items warp, warp+4, ...
#pragma unroll
    for (int s = 0; s < NS - 1; ++s) {
      if (s < n_mine) issue(items_s[warp + s * kWarps], s);
      cp_async_commit();
    }
    for (int n = 0; n < n_mine; ++n) {
      const FlatItem it = items_s[warp + n * kWarps];
      const int pr = it.kind_pair >> 1;
      // items n .. n + NS - 2 are in flight: stage (n + NS - 1) % NS is consumed and not yet refilled
      if (pr != cur_pair) advance_to(pr, (n + NS - 1) % NS);
      const int ahead = n + NS - 1;
      if (ahead < n_mine) issue(items_s[warp + ahead * kWarps], ahead % NS);
      cp_async_commit();
      cp_async_wait<NS - 1>();
      __syncwarp();
      w.consume(n % NS, it.lohi_head & 0xff, (it.lohi_head >> 8) & 0xff, (it.kind_pair & 1) == 0, (uint32_t)it.mask);
      __syncwarp();
    }
    cp_async_wait<0>();
    // Every warp leaves the chunk at the pair of the chunk's last item, so that all four have gone
    // through the same segment ends (and their barriers) before they meet at the next chunk's barrier.
    advance_to(items_s[chunk_end - chunk - 1].kind_pair >> 1, 0);
  }
  advance_to(pair_last + 1, 0);
}

size_t pair_grid_smem(int D, int NS, int rep_mode, int max_blocks) {
  return kItemChunk * sizeof(Item) + (size_t)kWarps * NS * (2 * 16 * D * 2) +
         (rep_mode == IA_REP_HYBRID ? (size_t)((max_blocks + 31) / 32) * 4 : 0);
}
size_t flat_grid_smem(int D, int NS, int n_pairs) {
  return kItemChunk * sizeof(FlatItem) + (size_t)kWarps * NS * (2 * 16 * D * 2) + ((size_t)n_pairs + 1) * 4;
}
constexpr size_t kTwoCtaSmem = (228 * 1024) / 2 - 1024;  // what one of two resident CTAs may take

template <typename Kern>
int launch_kernel(Kern kern, const char* name, int64_t grid, size_t smem, const DecodeParams& p, cudaStream_t stream) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "sparse_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  e = launch_overlapped(kern, (unsigned)grid, (unsigned)(kWarps * 32), smem, stream, p);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "%s: %s", name, cudaGetErrorString(e));
  return check_launch(name);
}

template <int D, int NS>
int launch_typed(const DecodeParams& p, const ia_geom& g, bool flat, cudaStream_t stream) {
  if (flat) {
    const size_t smem = flat_grid_smem(D, NS, p.n_pairs);
    const int64_t grid = decode_flat_ctas();
    const char* name = "condition_block_finalize_attention_flat_kernel";
    if (g.group_size > 8)
      return launch_kernel(condition_block_finalize_attention_flat_kernel<D, NS, true>, name, grid, smem, p, stream);
    return launch_kernel(condition_block_finalize_attention_flat_kernel<D, NS, false>, name, grid, smem, p, stream);
  }
  const int64_t grid = (int64_t)g.batch * g.n_kv_heads * p.n_splits;
  if (grid <= 0) return IA_OK;
  const size_t smem = pair_grid_smem(D, NS, p.rep_mode, g.max_blocks);
  const char* name = "condition_block_finalize_attention_kernel";
  if (g.group_size > 8)
    return launch_kernel(condition_block_finalize_attention_kernel<D, NS, true>, name, grid, smem, p, stream);
  return launch_kernel(condition_block_finalize_attention_kernel<D, NS, false>, name, grid, smem, p, stream);
}

}  // namespace

// CTAs of the flat grid: two resident CTAs per SM of the current device.
int decode_flat_ctas() {
  constexpr int kMaxDevices = 64;
  static int cached[kMaxDevices] = {};  // every thread would store the same value
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 2 * 148;
  if (cached[dev] == 0) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
    cached[dev] = 2 * sms;
  }
  return cached[dev];
}

// Whether the one-call layer-step may take the flat grid: bf16 tensor-core geometry, the fused
// finalize, every block in range, no peer exchange, and a prefix-sum array that still leaves two
// CTAs per SM.  The pair grid is the default: on B200 the step is bound by HBM and by its fixed
// start-up and tail latency, not by how evenly the pages are spread over the CTAs - a second,
// smaller wave of pair CTAs still saturates HBM - and the flat grid pays for its segment ends
// (measured: 61 vs 58 us at batch 16 x 32k, 156 vs 144 us on the ragged 70B batch).
// INTERATTN_B200_DECODE_GRID=flat selects it.
bool decode_flat_grid_possible(const ia_geom& g) {
  if (g.dtype != IA_BF16 || g.page_size != 16 || g.group_size > 16) return false;
  if (g.head_dim != 128 && g.head_dim != 64) return false;
  const int64_t n_pairs = (int64_t)g.batch * g.n_kv_heads;
  if (n_pairs <= 0 || n_pairs >= (1 << 26)) return false;
  const int ns = g.head_dim == 128 ? 3 : 4;
  return flat_grid_smem(g.head_dim, ns, (int)n_pairs) <= kTwoCtaSmem;
}
bool decode_flat_grid_applies(const ia_geom& g, bool fused_finalize, bool full_range, bool exchange) {
  if (!fused_finalize || !full_range || exchange || !decode_flat_grid_possible(g)) return false;
  const char* force = getenv("INTERATTN_B200_DECODE_GRID");
  return force != nullptr && strcmp(force, "flat") == 0;
}

int launch_sparse_decode_mma(const DecodeParams& p, const ia_geom& g, bool flat, cudaStream_t stream) {
  if (g.head_dim == 128) return launch_typed<128, 3>(p, g, flat, stream);
  if (g.head_dim == 64) return launch_typed<64, 4>(p, g, flat, stream);
  return fail(IA_ERR_UNSUPPORTED, "sparse_decode (mma): head_dim %d not built", g.head_dim);
}

}  // namespace ia
