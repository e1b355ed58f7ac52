// out[M, N] = x[M, K] * W[N, K]^T for a decode batch (M <= 32 rows), bf16 in, fp32
// accumulate, bf16 out - the projection GEMMs of a Llama decode step, where the
// whole cost is reading W once.  The reference leaves these to the Hugging Face
// model's nn.Linear (cuBLAS) inside its captured step
// (condition_block_triton_impl/core.py:190-316); at 32 rows the library kernels
// reach 40-85 % of the HBM rate depending on the shape, which is what this
// kernel is for.
//
// Work = chunks of (128 rows of W) x (64 columns of K), 16 KB each, ordered K-fastest.
// W is static, so it is packed once (ia_llama_gemm_pack) into exactly that order, each
// chunk stored as the shared-memory image the tensor core wants (rows of 128 bytes,
// 128-byte swizzle).  The grid is one CTA per SM and CTA i streams the chunk range
// [i T / P, (i + 1) T / P): one contiguous run of HBM, the same number of bytes on
// every SM whatever N and K are.  A producer thread issues one bulk copy per ring
// stage (up to four chunks, 64 KB) plus a TMA box for the matching 4 KB of x per
// chunk; an MMA thread issues tcgen05.mma (M = 128 rows of W, N = 32 tokens, K = 16)
// straight from the ring with the fp32 accumulator in tensor memory; four epilogue
// warps read the accumulator back and write bf16.
// A tile of 128 output columns whose K range is split over several CTAs is finished
// by the last of them to arrive: every contributor parks its fp32 partial in its own
// slot, and the last one adds the slots in CTA order - no atomics on data, the result
// does not depend on timing.
//
// The weights do not depend on the previous kernel of the stream, so the ring is
// primed with W before the programmatic-dependent-launch wait; only the x boxes
// are issued after it.
#include <stdlib.h>
#include <string.h>

#include <cuda.h>  // CUtensorMap (types only; the encoder is fetched through the runtime)

#include "ia_common.cuh"

namespace ia {
namespace {

constexpr int kBM = 32, kBN = 128, kBK = 64;
constexpr int kWBytes = kBN * kBK * 2, kXBytes = kBM * kBK * 2, kStageBytes = kWBytes + kXBytes;
constexpr int kSlotFloats = kBM * kBN;  // one fp32 partial tile
constexpr uint32_t kWaitPolls = 1u << 22;  // polls of a few tens of cycles: some tens of milliseconds

struct GemmParams {
  CUtensorMap tm_x;
  const unsigned char* w_packed;  // chunk c (K-fastest) = the 16 KB shared-memory image at c * 16 KB
  __nv_bfloat16* out;
  float* slots;        // [grid][2][kSlotFloats]
  int* tile_counters;  // [n_tiles], zero between launches
  int* status;
  int M, N, K;
  int k_chunks;  // ceil(K / 64)
  int total_chunks;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
// Bounded: false when the phase did not complete in time (the caller sets the status bit and
// carries on).  The poll is test_wait, which returns at once: try_wait parks the thread, and
// with one waiting thread per role its wake-up delay was paid once per ring stage - 16 KB
// stages reached 3.0 TB/s with try_wait.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kWaitPolls; ++i)
    if (mbar_test(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}
// contiguous global -> shared, completing on an mbarrier (addresses and size multiples of 16 bytes)
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// CTA that streams chunk x when P CTAs split T chunks as [i T / P, (i + 1) T / P)
__device__ __forceinline__ int owner_of(int x, int T, int P) { return (int)((((int64_t)x + 1) * P + T - 1) / T) - 1; }

// ---- the 5th-generation tensor core ---------------------------------------------------
// One thread issues tcgen05.mma (M = 128 rows of W, N = 32 tokens, K = 16 per instruction,
// four per chunk) with both operands read straight from the 128-byte-swizzled images in
// shared memory and the fp32 accumulator in tensor memory; nothing but the epilogue
// touches registers.  Warp roles: 0 = TMA producer, 1 = MMA issuer (and owner of the
// tensor-memory allocation), 2..5 = epilogue (warp w may read TMEM lanes 32 (w % 4) ..).
// Two accumulator buffers of 32 columns alternate between consecutive tiles of a CTA, so
// the epilogue of one tile overlaps the MMAs of the next.
constexpr int kTcThreads = 6 * 32;
constexpr int kTmemCols = 64;  // two fp32 accumulators of 32 columns (power of two, at least 32)

// shared-memory matrix descriptor: K-major operand, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart (bits 0-13 address >> 4, 32-45 stride >> 4, 46-47 version 1, 61-63 layout 2)
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3ffffu) >> 4) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// instruction descriptor of kind::f16: fp32 accumulate (bit 4), bf16 A and B (bits 7, 10), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24
constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kBM >> 3) << 17) | ((uint32_t)(kBN >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate)
      : "memory");
}
// the mbarrier gets one arrival when every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// 32 lanes x 32 columns of fp32: thread t of the warp gets lane (base lane + t), columns [col, col + 32)
__device__ __forceinline__ void tmem_load_32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }

// CPS = chunks per ring stage.  A stage holds up to CPS consecutive chunks of one tile: one
// bulk copy of W (the chunks are adjacent in the packed stream) and one x box per chunk.
// Stages are cut at multiples of CPS chunks from the tile's start, at the tile's end and
// at the end of the CTA's range; producer and MMA issuer walk the same cuts.  The walk is
// 32-bit and incremental: the two single-thread loops are the serial part of the kernel,
// and a 64-bit division per stage in them cost more than the copy it issued.
template <int CPS> struct TcRing {
  static constexpr int stage_bytes = CPS * kStageBytes;  // W chunks first, then the x boxes
  static constexpr int stages = (200 * 1024) / stage_bytes;
  static constexpr size_t smem = (size_t)stages * stage_bytes + 1024;
};
struct StageWalk {
  int s0, c1, kc, KC;  // next chunk, end of the range, s0's chunk index inside its tile, chunks per tile
  __device__ StageWalk(int c0, int c1_, int KC_) : s0(c0), c1(c1_), kc(c0 % KC_), KC(KC_) {}
  __device__ bool done() const { return s0 >= c1; }
  template <int CPS> __device__ int len() const { return min(min(CPS - (kc & (CPS - 1)), KC - kc), c1 - s0); }
  __device__ bool starts_tile_or_range(int c0) const { return kc == 0 || s0 == c0; }
  __device__ void advance(int n) {
    s0 += n;
    kc += n;
    if (kc == KC) kc = 0;
  }
};

template <int CPS>
__global__ void __launch_bounds__(kTcThreads, 1) llama_skinny_gemm_tc_kernel(const __grid_constant__ GemmParams p) {
  using R = TcRing<CPS>;
  static_assert((CPS & (CPS - 1)) == 0, "chunks per stage: a power of two");
  constexpr int kStages = R::stages;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* stage_base =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[kStages], empty_bar[kStages], acc_full[2], acc_empty[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int last_flag;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int P = gridDim.x, cta = blockIdx.x;
  const int T = p.total_chunks, KC = p.k_chunks;
  const int c0 = (int)((int64_t)T * cta / P), c1 = (int)((int64_t)T * (cta + 1) / P);

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);  // one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);   // one tcgen05.commit
      mbar_init(&acc_empty[b], 4);  // one lane of each epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the whole warp allocates; the base address lands in shared memory
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_s;
  grid_launch_dependents();

  if (warp == 0) {
    // ---- TMA producer ---------------------------------------------------------------
    if (lane == 0) {
      // W of the first stages does not depend on the predecessor: prime the ring before the wait
      StageWalk w(c0, c1, KC);
      int primed = 0;
      for (; primed < kStages && !w.done(); ++primed) {
        const int n = w.template len<CPS>();
        mbar_expect_tx(&full_bar[primed], (uint32_t)n * kWBytes);
        bulk_load(stage_base + (size_t)primed * R::stage_bytes, p.w_packed + (size_t)w.s0 * kWBytes,
                  (uint32_t)n * kWBytes, &full_bar[primed]);
        w.advance(n);
      }
      grid_dependency_wait();
      StageWalk x(c0, c1, KC);
      for (int st_i = 0; st_i < primed; ++st_i) {
        const int n = x.template len<CPS>();
        unsigned char* xs = stage_base + (size_t)st_i * R::stage_bytes + CPS * kWBytes;
        mbar_arrive_expect_tx(&full_bar[st_i], (uint32_t)n * kXBytes);
        for (int j = 0; j < n; ++j) tma_load_2d(xs + j * kXBytes, &p.tm_x, (x.kc + j) * kBK, 0, &full_bar[st_i]);
        x.advance(n);
      }
      bool alive = true;
      for (int it = primed; !w.done(); ++it) {
        const int stage = it % kStages, use = it / kStages;
        if (alive && !mbar_wait(&empty_bar[stage], (uint32_t)((use - 1) & 1))) {
          alive = false;
          atomicOr(p.status, DEV_STATUS_GEMM_WAIT_TIMEOUT);
        }
        const int n = w.template len<CPS>();
        unsigned char* st = stage_base + (size_t)stage * R::stage_bytes;
        mbar_arrive_expect_tx(&full_bar[stage], (uint32_t)n * kStageBytes);
        bulk_load(st, p.w_packed + (size_t)w.s0 * kWBytes, (uint32_t)n * kWBytes, &full_bar[stage]);
        for (int j = 0; j < n; ++j)
          tma_load_2d(st + CPS * kWBytes + j * kXBytes, &p.tm_x, (w.kc + j) * kBK, 0, &full_bar[stage]);
        w.advance(n);
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -------------------------------------------------------------------
    if (lane == 0) {
      bool alive = true;
      int seg = 0;  // tiles this CTA has started
      StageWalk w(c0, c1, KC);
      for (int it = 0; !w.done(); ++it) {
        const int n = w.template len<CPS>();
        const bool first = w.starts_tile_or_range(c0);
        if (first) {
          const int buf = seg & 1, use = seg >> 1;
          // the epilogue must have drained this buffer's previous tile
          if (use > 0 && alive && !mbar_wait(&acc_empty[buf], (uint32_t)((use - 1) & 1))) {
            alive = false;
            atomicOr(p.status, DEV_STATUS_GEMM_WAIT_TIMEOUT);
          }
          ++seg;
        }
        const int buf = (seg - 1) & 1;
        const int stage = it % kStages, use = it / kStages;
        if (alive && !mbar_wait(&full_bar[stage], (uint32_t)(use & 1))) {
          alive = false;
          atomicOr(p.status, DEV_STATUS_GEMM_WAIT_TIMEOUT);
        }
        tc_fence_after();
        const uint32_t st = smem_u32(stage_base + (size_t)stage * R::stage_bytes);
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * kBM);
        uint64_t a_desc = umma_desc(st), b_desc = umma_desc(st + CPS * kWBytes);
        for (int j = 0; j < n; ++j) {
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk)  // 16 columns = 32 bytes further along K inside the swizzled row
            umma_bf16(d_tmem, a_desc + (uint64_t)(kk * 2), b_desc + (uint64_t)(kk * 2),
                      (first && j == 0 && kk == 0) ? 0u : 1u);
          a_desc += kWBytes >> 4;
          b_desc += kXBytes >> 4;
        }
        umma_commit(&empty_bar[stage]);  // the stage is free once these MMAs have read it
        w.advance(n);
        if (w.kc == 0 || w.done()) umma_commit(&acc_full[buf]);  // that was the tile's last stage here
      }
    }
  } else {
    // ---- epilogue -----------------------------------------------------------------------
    grid_dependency_wait();  // the output and the slots may still be read by earlier kernels
    const int q = warp & 3;       // TMEM lane quarter this warp may read
    const int r = q * 32 + lane;  // row of the tile (= row of W) held by this thread
    // CTA c parks the partial of the tile its range starts in at slot 0, of the tile it ends in at slot 1
    auto slot_at = [&](int c, int which) -> float* {
      return p.slots + ((size_t)c * 2 + which) * kSlotFloats + (size_t)r * 32;
    };
    auto store_row = [&](int tile, const float (&v)[32]) {
      const int n = tile * kBN + r;
      if (n >= p.N) return;
#pragma unroll
      for (int m = 0; m < kBM; ++m)
        if (m < p.M) p.out[(int64_t)m * p.N + n] = __float2bfloat16_rn(v[m]);
    };
    bool alive = true;
    int seg = 0;
    int from = c0;
    int tile = c0 / KC;
    while (from < c1) {
      const int t_lo = tile * KC, t_hi = t_lo + KC;
      const int to = t_hi < c1 ? t_hi : c1;
      const int buf = seg & 1, use = seg >> 1;
      if (alive && !mbar_wait(&acc_full[buf], (uint32_t)(use & 1))) {
        alive = false;
        if (lane == 0) atomicOr(p.status, DEV_STATUS_GEMM_WAIT_TIMEOUT);
      }
      tc_fence_after();
      float v[32];
      tmem_load_32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * kBM), v);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);  // the MMA warp may overwrite this buffer
      if (from == t_lo && to == t_hi) {
        store_row(tile, v);
      } else {
        float4* mine = reinterpret_cast<float4*>(slot_at(cta, from == c0 ? 0 : 1));
#pragma unroll
        for (int i = 0; i < 8; ++i) mine[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
        const int c_first = owner_of(t_lo, T, P), c_last = owner_of(t_hi - 1, T, P);
        epilogue_sync();  // every partial row is written
        if (tid == 64) {
          __threadfence();
          const int old = atomicAdd(&p.tile_counters[tile], 1);
          const int is_last = old == c_last - c_first;
          if (is_last) {
            p.tile_counters[tile] = 0;  // ready for the next launch
            __threadfence();
          }
          last_flag = is_last;
        }
        epilogue_sync();
        const bool last = last_flag != 0;
        epilogue_sync();  // last_flag may be rewritten by the next tile
        if (last) {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
          // Only the first contributor can have started before this tile (its slot 1); all others
          // start inside it (slot 0).  Contributors are read four at a time with every load of the
          // group in flight together - one L2 round trip per group instead of one per contributor -
          // and added in CTA order, so the sum does not depend on who arrived last.
          const int first_which = (int)((int64_t)T * c_first / P) >= t_lo ? 0 : 1;
          for (int cb = c_first; cb <= c_last; cb += 4) {
            float4 part[4][8];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int c = min(cb + u, c_last);  // past the end: a valid slot, not added below
              const float4* src = reinterpret_cast<const float4*>(slot_at(c, c == c_first ? first_which : 0));
#pragma unroll
              for (int i = 0; i < 8; ++i) part[u][i] = __ldcg(src + i);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
              if (cb + u <= c_last) {
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                  v[4 * i] += part[u][i].x; v[4 * i + 1] += part[u][i].y;
                  v[4 * i + 2] += part[u][i].z; v[4 * i + 3] += part[u][i].w;
                }
              }
          }
          store_row(tile, v);
        }
      }
      from = to;
      ++tile;
      ++seg;
    }
  }
  // everyone meets here; then the allocating warp returns the tensor memory
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}

// Row-major W [N, K] -> the stream the GEMM reads: for every (128-row tile, 64-column chunk), K fastest, the
// 16 KB shared-memory image of that chunk (rows of 128 bytes, 16-byte piece c of row r at c ^ (r & 7), rows and
// columns past the matrix zero).  One thread per 16-byte piece of the output.
__global__ void llama_gemm_pack_kernel(const __nv_bfloat16* __restrict__ w, uint4* __restrict__ packed, int N, int K,
                                       int k_chunks, int64_t n_pieces) {
  const int64_t o = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (o >= n_pieces) return;
  const int64_t chunk = o >> 10;  // 1024 pieces per chunk
  const int within = (int)(o & 1023);
  const int r = within >> 3, c = (within & 7) ^ (r & 7);
  const int64_t n = (chunk / k_chunks) * kBN + r;
  const int k = (int)(chunk % k_chunks) * kBK + c * 8;
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  if (n < N && k < K) v = *reinterpret_cast<const uint4*>(w + n * K + k);
  packed[o] = v;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn tensor_map_encoder() {
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

// a row-major bf16 [rows, K] matrix cut into boxes of 64 columns x box_rows rows, 128-byte swizzle
int encode_bf16(CUtensorMap* tm, const void* base, int64_t rows, int64_t K, int box_rows, CUtensorMapL2promotion l2) {
  EncodeTiledFn enc = tensor_map_encoder();
  if (enc == nullptr) return fail(IA_ERR_LAUNCH, "gemm: cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
  const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, l2,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(IA_ERR_LAUNCH, "gemm: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return IA_OK;
}

template <int CPS> int launch_tc(const GemmParams& p, int grid, cudaStream_t stream) {
  auto kern = llama_skinny_gemm_tc_kernel<CPS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TcRing<CPS>::smem);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "gemm: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
  e = launch_overlapped(kern, (unsigned)grid, (unsigned)kTcThreads, TcRing<CPS>::smem, stream, p);
  if (e != cudaSuccess) return fail(IA_ERR_LAUNCH, "llama_skinny_gemm_tc_kernel: %s", cudaGetErrorString(e));
  return check_launch("llama_skinny_gemm_tc_kernel");
}

int grid_for(int64_t total_chunks) {
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  return (int)(total_chunks < sms ? total_chunks : sms);
}

}  // namespace
}  // namespace ia

using namespace ia;

extern "C" {

int64_t ia_llama_gemm_workspace_bytes(int n) {
  if (n <= 0) return 0;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    sms = 148;
  const int64_t n_tiles = ((int64_t)n + kBN - 1) / kBN;
  return (int64_t)sms * 2 * kSlotFloats * 4 + ((n_tiles * 4 + 255) / 256) * 256;
}

int64_t ia_llama_gemm_packed_bytes(int n, int k) {
  if (n <= 0 || k <= 0) return 0;
  return (((int64_t)n + kBN - 1) / kBN) * (((int64_t)k + kBK - 1) / kBK) * kWBytes;
}

int ia_llama_gemm_pack(const void* w, int n, int k, void* packed, ia_stream_t stream) {
  if (!w || !packed) return fail(IA_ERR_BAD_ARG, "gemm_pack: null pointer");
  if (n <= 0 || k <= 0 || k % 8 != 0) return fail(IA_ERR_BAD_ARG, "gemm_pack: n %d, k %d (a multiple of 8)", n, k);
  if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(packed)) & 15u)
    return fail(IA_ERR_BAD_ARG, "gemm_pack: pointers must be 16-byte aligned");
  const int k_chunks = (k + kBK - 1) / kBK;
  const int64_t n_pieces = ia_llama_gemm_packed_bytes(n, k) / 16;
  llama_gemm_pack_kernel<<<(unsigned)ceil_div64(n_pieces, 256), 256, 0, (cudaStream_t)stream>>>(
      static_cast<const __nv_bfloat16*>(w), static_cast<uint4*>(packed), n, k, k_chunks, n_pieces);
  return check_launch("llama_gemm_pack_kernel");
}

int ia_llama_gemm(const void* x, const void* w, void* out, int m, int n, int k, void* workspace,
                  int64_t workspace_bytes, ia_stream_t stream) {
  if (!x || !w || !out || !workspace) return fail(IA_ERR_BAD_ARG, "gemm: null pointer");
  if (m < 0 || m > kBM) return fail(IA_ERR_UNSUPPORTED, "gemm: %d rows (at most %d)", m, kBM);
  if (n <= 0 || k <= 0 || k % 8 != 0) return fail(IA_ERR_BAD_ARG, "gemm: n %d, k %d (a multiple of 8)", n, k);
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(workspace)) & 15u)
    return fail(IA_ERR_BAD_ARG, "gemm: x, w and the workspace must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(out) & 3u) return fail(IA_ERR_BAD_ARG, "gemm: out must be 4-byte aligned");
  if (workspace_bytes < ia_llama_gemm_workspace_bytes(n))
    return fail(IA_ERR_BAD_ARG, "gemm: workspace %lld bytes, need %lld", (long long)workspace_bytes,
                (long long)ia_llama_gemm_workspace_bytes(n));
  if (m == 0) return IA_OK;
  GemmParams p{};
  p.out = static_cast<__nv_bfloat16*>(out);
  p.M = m; p.N = n; p.K = k;
  p.k_chunks = (k + kBK - 1) / kBK;
  const int64_t n_tiles = ((int64_t)n + kBN - 1) / kBN;
  if (n_tiles * p.k_chunks > 0x3fffffff) return fail(IA_ERR_UNSUPPORTED, "gemm: %d x %d is too large", n, k);
  p.total_chunks = (int)(n_tiles * p.k_chunks);
  const int grid = grid_for(p.total_chunks);
  p.tile_counters = static_cast<int*>(workspace);
  p.slots = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + ((n_tiles * 4 + 255) / 256) * 256);
  p.status = device_status_address();
  if (p.status == nullptr) return IA_ERR_LAUNCH;
  p.w_packed = static_cast<const unsigned char*>(w);
  if (int s = encode_bf16(&p.tm_x, x, m, k, kBM, CU_TENSOR_MAP_L2_PROMOTION_L2_128B)) return s;
  // chunks per ring stage: 4 (two stages of 80 KB) measured best - 6.6 TB/s on a 1 GB weight against
  // 6.5 with 2 and 4.6 with 1; INTERATTN_B200_GEMM_CPS=1|2|4 picks another
  int cps = 4;
  if (const char* c = getenv("INTERATTN_B200_GEMM_CPS")) cps = atoi(c);
  switch (cps) {
    case 1: return launch_tc<1>(p, grid, (cudaStream_t)stream);
    case 2: return launch_tc<2>(p, grid, (cudaStream_t)stream);
    default: return launch_tc<4>(p, grid, (cudaStream_t)stream);
  }
}

}  // extern "C"
