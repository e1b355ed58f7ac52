// Paged sparse / hybrid decode attention - bf16 tensor-core kernel (sm_100a).
//
// Attention half of the reference's fused finalize kernel
// (llama/script/analysis/condition_block_gen/methods/condition_block_triton_impl/page_attention.py:173-309).
// Like the reference kernel it feeds bf16 q / K / V / probabilities to the
// tensor cores and keeps the softmax and the accumulators in fp32; unlike it,
// the pages to visit are known up front (an index list through a block
// table), so nothing in the load path depends on a computed value:
//
//   * a CTA owns one (sequence, kv head, split); its item descriptors
//     (physical page, valid rows) are resolved by all threads at once;
//   * each of the four warps runs its own ring of NS stages: a stage holds
//     one 16-token K page and V page (2 * 16 * D * 2 bytes), filled with
//     16-byte cp.async copies into an XOR-swizzled layout (zero-filled for
//     rows outside the valid range), so up to 4 * (NS - 1) pages per CTA are
//     in flight and ldmatrix reads are bank-conflict free;
//   * per page: S = Q K^T as 2 x (D/16) m16n8k16 MMAs (the G <= 16 query rows
//     of the kv head padded to 16), online softmax on the accumulator
//     fragments, O += P V as D/8 MMAs with P re-used straight from the S
//     fragments;
//   * the four warps' (m, l, O) are merged through shared memory and written
//     as a normalised partial (o, lse).
//
// Roofline: HBM.  Algorithmic bytes: 2 * D * 2 bytes per attended token
// (K and V row), D * 2 per representative.  Arithmetic intensity is 2 G / 2
// flop per byte, far below the ridge, so the tensor cores idle most of the time;
// they are used because fp32 FMAs alone would cap the kernel near half of HBM
// speed at G = 4 and below it at G = 8.
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
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, int NS, bool HI_ROWS>
__global__ void __launch_bounds__(kWarps * 32, 2)
condition_block_finalize_attention_kernel(DecodeParams p) {
  constexpr int ROW_BYTES = D * 2;               // one token row of a tile
  constexpr int CHUNKS = ROW_BYTES / 16;         // 16-byte chunks per row
  constexpr int TILE_BYTES = 16 * ROW_BYTES;     // one K or V page
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;
  constexpr int KSTEPS = D / 16;
  constexpr int NT_O = D / 8;
  constexpr int COPIES = 16 * CHUNKS / 32;       // 16-byte copies per lane per tile
  using bf16 = __nv_bfloat16;

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
  grid_launch_dependents();
  grid_dependency_wait();
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

  // ---- Q as A fragments (rows >= G are zero) --------------------------------------
  uint32_t qa[KSTEPS][4];
  {
    const bf16* qp = static_cast<const bf16*>(p.q) + ((int64_t)seq * rows + head * G) * D;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      const int d0 = kk * 16 + qlane * 2;
      qa[kk][0] = quad < G ? *reinterpret_cast<const uint32_t*>(qp + quad * D + d0) : 0u;
      qa[kk][1] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(qp + (quad + 8) * D + d0) : 0u;
      qa[kk][2] = quad < G ? *reinterpret_cast<const uint32_t*>(qp + quad * D + d0 + 8) : 0u;
      qa[kk][3] = quad + 8 < G ? *reinterpret_cast<const uint32_t*>(qp + (quad + 8) * D + d0 + 8) : 0u;
    }
  }

  float o[NT_O][4];
#pragma unroll
  for (int j = 0; j < NT_O; ++j) { o[j][0] = 0.f; o[j][1] = 0.f; o[j][2] = 0.f; o[j][3] = 0.f; }
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;  // log2 domain; l: this thread's share

  const float sc_qk = kLog2e / sqrtf((float)D);
  const bf16* kbase = static_cast<const bf16*>(p.k_pool) + (int64_t)head * p.head_stride;
  const bf16* vbase = static_cast<const bf16*>(p.v_pool) + (int64_t)head * p.head_stride;
  const bf16* vbar = static_cast<const bf16*>(p.v_bar) + (int64_t)pair * p.max_blocks * D;
  const float* zrow = p.z + ((int64_t)seq * rows + head * G) * p.max_blocks;
  unsigned char* my_ring = ring + (size_t)warp * NS * STAGE_BYTES;
  const uint32_t my_ring_u32 = smem_u32(my_ring);

  // fill one stage: K tile then V tile, swizzled, rows outside [lo, hi) zero-filled
  auto issue = [&](const Item& it, int stage) {
    if (it.hi <= it.lo) return;
    const uint32_t kdst = my_ring_u32 + stage * STAGE_BYTES;
    const uint32_t vdst = kdst + TILE_BYTES;
    const bf16* ksrc;
    const bf16* vsrc;
    if (it.kind == ITEM_PAGE) {
      ksrc = kbase + (int64_t)it.first * p.page_stride;
      vsrc = vbase + (int64_t)it.first * p.page_stride;
    } else {
      ksrc = nullptr;
      vsrc = vbar + (int64_t)it.first * D;
    }
#pragma unroll
    for (int c = 0; c < COPIES; ++c) {
      const int id = c * 32 + lane;
      const int row = id / CHUNKS, ch = id % CHUNKS;
      const bool live = row >= it.lo && row < it.hi;
      const int srow = live ? row : it.lo;  // keep the address in bounds; nothing is read when !live
      const uint32_t off = row * ROW_BYTES + ((ch ^ (row & 7)) << 4);
      if (ksrc != nullptr) cp_async16(kdst + off, ksrc + srow * D + ch * 8, live ? 16u : 0u);
      cp_async16(vdst + off, vsrc + srow * D + ch * 8, live ? 16u : 0u);
    }
    if (ksrc == nullptr) {
      // representatives: their logits z[row][block] ride in the unused K half of the stage as
      // [16 rows][16 blocks] floats, so that consume() does not wait on global loads
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int id = c * 32 + lane;
        const int row = id >> 4, tok = id & 15;
        if (row < G && tok < it.hi)
          cp_async4(kdst + id * 4, zrow + (int64_t)row * p.max_blocks + it.first + tok);
      }
    }
  };

  auto consume = [&](const Item& it, int stage) {
    if (it.hi <= it.lo) return;
    const uint32_t ktile = my_ring_u32 + stage * STAGE_BYTES;
    const uint32_t vtile = ktile + TILE_BYTES;
    float s[2][4];
    if (it.kind == ITEM_PAGE) {
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
          const bool ok = tok >= it.lo && tok < it.hi;
          s[t][e] = ok ? s[t][e] * sc_qk : -INFINITY;
        }
      }
    } else {
      // representatives: logits come from the selection pass (z = s + log count), staged by issue()
      const float* zt = reinterpret_cast<const float*>(my_ring + (size_t)stage * STAGE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = t * 8 + qlane * 2 + (e & 1);
          const int row = quad + (e >> 1) * 8;
          const int b = it.first + tok;
          bool ok = tok < it.hi && row < G;
          if (ok) ok = ((sel_bits[b >> 5] >> (b & 31)) & 1u) == 0u;
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
  };

  for (int chunk = r.begin; chunk < r.end; chunk += kItemChunk) {
    const int chunk_end = min(chunk + kItemChunk, r.end);
    __syncthreads();  // every warp is done with the previous descriptors
    resolve_items(p, r, seq, head, chunk, chunk_end, items_s);
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
      consume(items_s[warp + n * kWarps], n % NS);
      __syncwarp();
    }
    cp_async_wait<0>();
  }

  // ---- merge the four warps ------------------------------------------------------------
  __syncthreads();  // all rings idle: reuse them as merge buffers
  float* mo = reinterpret_cast<float*>(my_ring);            // [16][D]
  float* mm = reinterpret_cast<float*>(my_ring + 16 * D * 4);  // m[16], l[16]
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
  l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
  for (int j = 0; j < NT_O; ++j) {
    const int d = j * 8 + qlane * 2;
    *reinterpret_cast<float2*>(mo + quad * D + d) = make_float2(o[j][0], o[j][1]);
    if constexpr (HI_ROWS) *reinterpret_cast<float2*>(mo + (quad + 8) * D + d) = make_float2(o[j][2], o[j][3]);
  }
  if (qlane == 0) {
    mm[quad] = m0; mm[16 + quad] = l0;
    if constexpr (HI_ROWS) { mm[quad + 8] = m1; mm[16 + quad + 8] = l1; }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < G * D; e += blockDim.x) {
    const int g = e / D, d = e - g * D;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w)
      top = fmaxf(top, reinterpret_cast<const float*>(ring + (size_t)w * NS * STAGE_BYTES + 16 * D * 4)[g]);
    float num = 0.f, den = 0.f;
    if (top > -INFINITY) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float* wo = reinterpret_cast<const float*>(ring + (size_t)w * NS * STAGE_BYTES);
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

template <int D, int NS>
int launch_typed(const DecodeParams& p, const ia_geom& g, cudaStream_t stream) {
  const int64_t grid = (int64_t)g.batch * g.n_kv_heads * p.n_splits;
  if (grid <= 0) return IA_OK;
  const size_t smem = kItemChunk * sizeof(Item) + (size_t)kWarps * NS * (2 * 16 * D * 2) +
                      (p.rep_mode == IA_REP_HYBRID ? (size_t)((g.max_blocks + 31) / 32) * 4 : 0);
  if (g.group_size > 8) {
    auto kern = condition_block_finalize_attention_kernel<D, NS, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "sparse_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    e = launch_overlapped(kern, (unsigned)grid, (unsigned)(kWarps * 32), smem, stream, p);
    if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "condition_block_finalize_attention_kernel: %s", cudaGetErrorString(e));
  } else {
    auto kern = condition_block_finalize_attention_kernel<D, NS, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "sparse_decode: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    e = launch_overlapped(kern, (unsigned)grid, (unsigned)(kWarps * 32), smem, stream, p);
    if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "condition_block_finalize_attention_kernel: %s", cudaGetErrorString(e));
  }
  return check_launch("condition_block_finalize_attention_kernel");
}

}  // namespace

int launch_sparse_decode_mma(const DecodeParams& p, const ia_geom& g, cudaStream_t stream) {
  if (g.head_dim == 128) return launch_typed<128, 3>(p, g, stream);
  if (g.head_dim == 64) return launch_typed<64, 4>(p, g, stream);
  return fail(IA_ERR_UNSUPPORTED, "sparse_decode (mma): head_dim %d not built", g.head_dim);
}

}  // namespace ia
