/*
 * interattn_b200 - C ABI of the B200 (sm_100a) condition-block sparse
 * decode-attention path.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes,
 * enqueues its kernels on the given CUDA stream and returns immediately with
 * an `ia_status`.  Unless an entry point's comment says otherwise it allocates
 * nothing, synchronises nothing and keeps no state; all device memory,
 * including scratch, belongs to the caller.  Calls are CUDA-graph capturable:
 * per-step quantities (sequence lengths, selection results) are read from
 * device memory.
 *
 * Reference interfaces these entry points stand behind (paths relative to the
 * reference project; IMPL = llama/script/analysis/condition_block_gen/methods/
 * condition_block_triton_impl):
 *   ia_build_summaries  <- _build_prompt_blocks                 IMPL/core.py:449-500
 *   ia_select           <- _run_condition_block_selection_stats IMPL/core.py:573-698
 *                          + the routing half of the fused finalize kernel
 *                            IMPL/page_attention.py:84-171, and the eager rule
 *                            _select_prompt_blocks_eager        IMPL/core.py:509-555
 *   ia_sparse_decode    <- _condition_block_finalize_attention_kernel
 *                            IMPL/page_attention.py:173-309 (attention half)
 *   ia_finalize         <- _condition_block_stage2_reduce_kernel IMPL/legacy.py:765-794
 *   ia_decode_attention <- _condition_block_decode_output_fused_triton
 *                            IMPL/core.py:1035-1155 (the launches of one layer-step)
 *   ia_update_summaries <- no counterpart (the reference never re-blocks its suffix)
 *   ia_select_split, ia_sparse_decode_exchange, ia_finalize_exchange, ia_finalize_gathered
 *                       <- no counterpart (split-KV across GPUs; the reference has one GPU)
 *   ia_llama_*          <- the Hugging Face modules the reference replays around its hook in
 *                          the captured decode step, IMPL/core.py:190-316
 *
 * Tensor conventions
 *   q            [batch, n_kv_heads * group_size, head_dim]   dtype; query head = kv * G + g
 *   k_pool/v_pool physical KV pages; element (page p, kv head h, token t, dim d) lives at
 *                p * pool_page_stride + h * pool_head_stride + t * head_dim + d   (dtype)
 *                so one (page, kv head) is a contiguous page_size x head_dim run.
 *   block_table  int32 [batch, max_pages]; entry j = physical page of logical tokens
 *                [j * page_size, (j + 1) * page_size)
 *   prefix_lens  int32 [batch]; tokens covered by block summaries (the prompt)
 *   seq_lens     int32 [batch]; all visible tokens (prefix + generated suffix)
 *   summaries    per (sequence, kv head, logical block): see ia_summaries
 *   sel_idx      int32 [batch, n_kv_heads, max_sel] ascending block indices
 *   sel_count    int32 [batch, n_kv_heads]
 */
#ifndef INTERATTN_B200_H_
#define INTERATTN_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* ia_stream_t; /* same type as cudaStream_t */

typedef enum ia_status {
  IA_OK = 0,
  IA_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, inconsistent geometry */
  IA_ERR_UNSUPPORTED = -2,  /* geometry outside what the kernels are built for */
  IA_ERR_LAUNCH = -3,       /* CUDA reported an error at launch */
  IA_ERR_NO_DEVICE = -4
} ia_status;

typedef enum ia_dtype { IA_F32 = 0, IA_BF16 = 1 } ia_dtype;
typedef enum ia_select_mode { IA_SELECT_TOPK = 0, IA_SELECT_EPS = 1 } ia_select_mode;
/* Score variant, OR-ed into the mode argument: the first term of the block score becomes
 * 2 b_all softmax(z + delta) instead of 2 b_all softmax(z) (cosh(delta) - 1) / sum(softmax(z) cosh(delta)) -
 * the reference's term1_mass_exp (IMPL/core.py:798-803 and 893-896;
 * GEN/methods/condition_block_triton_term1_softmax.py). */
#define IA_SELECT_TERM1_MASS_EXP 0x100
typedef enum ia_rep_mode {
  IA_REP_SPARSE_ONLY = 0, /* selected blocks + suffix */
  IA_REP_HYBRID = 1       /* + one (z, v_bar) representative per unselected block */
} ia_rep_mode;

typedef struct ia_geom {
  int32_t batch;
  int32_t n_kv_heads;
  int32_t group_size;   /* query heads per kv head (1..16) */
  int32_t head_dim;     /* 64 or 128 */
  int32_t page_size;    /* tokens per physical page: 16 */
  int32_t block_size;   /* tokens per selection block: multiple of page_size, <= 128 */
  int32_t max_pages;    /* row length of block_table */
  int32_t max_blocks;   /* blocks per (sequence, kv head) in the summary arrays */
  int32_t dtype;        /* ia_dtype of q, pools, k_max/k_min/v_bar */
  int32_t reserved;     /* flags: IA_GEOM_KBAR_BF16 | IA_GEOM_DIAG_ELL | IA_GEOM_PACKED_BOUNDS, else 0 */
  int32_t n_pool_pages; /* physical pages in k_pool / v_pool; block-table entries are checked against
                           it before they are used.  0: unknown, entries are trusted. */
  int32_t reserved2;    /* 0 */
  int64_t pool_page_stride; /* in elements */
  int64_t pool_head_stride; /* in elements */
} ia_geom;

/* ia_geom.reserved flag: ia_summaries.k_bar holds bf16 values (same shape) instead of fp32 - the
 * reference's CONDITION_BLOCK_K_BAR_DTYPE=bfloat16 option (IMPL/core.py:428-446, 482; only with
 * bf16 pools).  The mean is accumulated in fp32 and rounded once; scores computed from it are
 * approximate with respect to the fp32 k_bar and may rank near-equal blocks differently.  768
 * instead of 1024 summary bytes per block and kv head at head_dim 128. */
#define IA_GEOM_KBAR_BF16 1
/* ia_geom.reserved flag: the selection bounds |q . (k - k_bar)| with the diagonal-ellipsoid summaries
 * (ia_summaries.w, .rho) instead of the coordinate range (k_max, k_min) - the "diag_ell" bound of the
 * reference's condition_block_ball study (condition_block_ball/gen_selection.py:21-87, conclusions in
 * condition_block_ball/README.md:228-241): w = max(k_max - k_bar, k_bar - k_min) clamped at 1e-6,
 * rho = max_t |(k_t - k_bar) / w|, delta = rho |q * w| / sqrt(D).  Two vectors and a scalar per block
 * instead of three vectors; k_max / k_min are then not read by ia_select (and may be null there). */
#define IA_GEOM_DIAG_ELL 2
/* ia_geom.reserved flag: the coordinate range is stored packed, as the reference does with
 * CONDITION_BLOCK_TMA_BOUNDS=1 (IMPL/core.py:490-499: torch.stack((k_max, k_min), dim=-1).flatten(2)):
 * ia_summaries.k_max points to one array [batch, kv heads, max_blocks, 2 * head_dim] in the KV dtype whose
 * element 2 d is k_max[d] and element 2 d + 1 is k_min[d]; ia_summaries.k_min is not read.  ia_build_summaries
 * writes that layout, ia_select / ia_decode_attention read it (same bytes per block as the two arrays).
 * Not together with IA_GEOM_DIAG_ELL. */
#define IA_GEOM_PACKED_BOUNDS 4

/* Block summaries, "mixed" storage of the reference (IMPL/core.py:411-446):
 * means accumulated in fp32, k_bar kept in fp32, the rest in the KV dtype
 * (the coordinate bounds are copies of K values, so that is lossless). */
typedef struct ia_summaries {
  float* k_bar;      /* [batch, n_kv_heads, max_blocks, head_dim] f32 */
  void* k_max;       /* same shape, dtype */
  void* k_min;       /* same shape, dtype */
  void* v_bar;       /* same shape, dtype */
  float* v_norm_max; /* [batch, n_kv_heads, max_blocks] f32: max token |v|_2 in the block */
  /* Optional (null: not kept): the diagonal-ellipsoid pair of IA_GEOM_DIAG_ELL.  w in the KV dtype -
   * with bf16 pools rounded up by 1 + 2^-7 before the cast, the reference's
   * CONDITION_BLOCK_BALL_W_DTYPE=bfloat16 option, so that the bound stays strict - and rho computed
   * from the stored w.  ia_build_summaries / ia_update_summaries fill them when both are given. */
  void* w;           /* [batch, n_kv_heads, max_blocks, head_dim] dtype */
  float* rho;        /* [batch, n_kv_heads, max_blocks] f32 */
} ia_summaries;

/* Optional diagnostics of ia_select; any pointer may be null. */
typedef struct ia_select_aux {
  float* score;   /* [batch, n_kv_heads, max_blocks]  GQA-mean condition score */
  float* z;       /* [batch, rows, max_blocks]  s + log(count); needed by IA_REP_HYBRID */
  float* s;       /* [batch, rows, max_blocks]  q.k_bar / sqrt(D) */
  float* delta;   /* [batch, rows, max_blocks]  range bound */
  float* globals; /* [batch, 4, rows]  z_m, z_l, c_m, c_l (online-softmax normalisers) */
} ia_select_aux;

/* Version of this ABI; bumped on any incompatible change (2: ia_geom carries n_pool_pages; 3: ia_summaries
 * carries the optional diagonal-ellipsoid pair w, rho). */
int ia_abi_version(void);

/* Message for the last non-OK status returned on the calling thread. */
const char* ia_last_error_string(void);

/* The device status word: kernels never trap and never wait without a limit; what goes wrong on
 * the device is recorded here instead, as an OR of these masks.
 *   IA_DEV_STATUS_SELECT_WAIT  a bounded shared-memory barrier wait inside the selection kernel ran
 *                              out: that launch's selection is invalid
 *   IA_DEV_STATUS_GEMM_WAIT    the same inside ia_llama_gemm: that product is invalid
 *   IA_DEV_STATUS_PEER_WAIT    a bounded wait for another GPU's flag ran out (ia_finalize_exchange,
 *                              ia_select_split): that step's output is invalid
 *   IA_DEV_STATUS_BAD_INDEX    a selected block index outside [0, max_blocks), a block-table entry
 *                              outside [0, n_pool_pages), a logical page outside the table row, or an
 *                              index list that is not ascending was met.  The access was skipped
 *                              (the page contributes nothing), so no memory outside the arrays the
 *                              geometry declares is touched; the output lacks those tokens.
 * ia_read_device_status reads and clears the word.  It synchronises the device, so call it where
 * the host waits anyway. */
#define IA_DEV_STATUS_SELECT_WAIT 1
#define IA_DEV_STATUS_GEMM_WAIT 2
#define IA_DEV_STATUS_PEER_WAIT 4
#define IA_DEV_STATUS_BAD_INDEX 8
int ia_read_device_status(int* out);

/* Replaces _build_prompt_blocks (IMPL/core.py:449-500): one pass over the K/V
 * pages of every sequence's prefix through the block table. */
int ia_build_summaries(const void* k_pool, const void* v_pool, const int32_t* block_table,
                       const int32_t* prefix_lens, const ia_geom* geom, const ia_summaries* out,
                       ia_stream_t stream);

/* Summary maintenance during decode: recompute only the blocks
 * b >= first_blocks[sequence] (int32 [batch], device) for the prefix lengths
 * given - e.g. after 64 more generated tokens, raise prefix_lens by one block
 * and call this with first_blocks = the old block count.  The reference never
 * re-blocks the generated suffix (GEN/CONDITION_BLOCK_TRITON_README.md:244-246):
 * its suffix is always attended in full and grows linearly; with this call a
 * long generation keeps a bounded suffix.  Same kernel as ia_build_summaries. */
int ia_update_summaries(const void* k_pool, const void* v_pool, const int32_t* block_table,
                        const int32_t* prefix_lens, const int32_t* first_blocks, const ia_geom* geom,
                        const ia_summaries* out, ia_stream_t stream);

/* Replaces the selection stats kernel plus the routing decision
 * (IMPL/core.py:751-814, IMPL/page_attention.py:84-171): condition score of
 * every block, then either the top_k best blocks per (sequence, kv head) -
 * higher score first, lower block index first among equal scores - or every
 * block whose score exceeds eps (the reference rule, IMPL/core.py:546).
 * Indices are written in ascending order; entries past sel_count are -1.
 * The score vector stays on chip unless aux asks for it. */
int ia_select(const void* q, const ia_summaries* summaries, const int32_t* prefix_lens,
              const ia_geom* geom, int mode, int top_k, float eps, int max_sel,
              int32_t* sel_idx, int32_t* sel_count, const ia_select_aux* aux, ia_stream_t stream);

/* Replaces the attention half of the fused finalize kernel
 * (IMPL/page_attention.py:173-309): online-softmax attention of the G query
 * rows of each kv head over the tokens of the selected blocks (gathered page
 * by page through the block table), the generated suffix
 * [prefix_len, seq_len) and, in IA_REP_HYBRID, the representatives of the
 * unselected blocks (logit z from ia_select, value v_bar).  The work of one
 * (sequence, kv head) is cut into n_splits parts; part s writes a normalised
 * partial output and its log-sum-exp:
 *   o_partial   f32 [batch, rows, n_splits, head_dim]
 *   lse_partial f32 [batch, rows, n_splits]       (-inf for an empty part)
 * block_lo/block_hi (blocks, hi exclusive; pass 0 / max_blocks for all) and
 * with_suffix restrict the call to one rank's share in multi-GPU split-KV.
 * sel_idx must be ascending per (sequence, kv head), as ia_select writes it.  Indices and table
 * entries are checked against max_blocks, max_pages and n_pool_pages before use: a bad one is
 * skipped and reported as IA_DEV_STATUS_BAD_INDEX, never dereferenced. */
int ia_sparse_decode(const void* q, const void* k_pool, const void* v_pool,
                     const int32_t* block_table, const int32_t* prefix_lens,
                     const int32_t* seq_lens, const int32_t* sel_idx, const int32_t* sel_count,
                     int max_sel, const ia_summaries* summaries, const float* z,
                     const ia_geom* geom, int rep_mode, int n_splits, int block_lo, int block_hi,
                     int with_suffix, float* o_partial, float* lse_partial, ia_stream_t stream);

/* Replaces _condition_block_stage2_reduce_kernel (IMPL/legacy.py:765-794),
 * written for (o, lse) partials: out = sum_s o_s e^{lse_s - M} / sum_s
 * e^{lse_s - M}.  n_rows = batch * rows.  out_dtype is an ia_dtype; out_lse
 * (f32 [n_rows], may be null) receives the merged log-sum-exp so that the
 * result can itself be merged again (across GPUs). */
int ia_finalize(const float* o_partial, const float* lse_partial, int n_rows, int n_parts,
                int head_dim, void* out, int out_dtype, float* out_lse, ia_stream_t stream);

/* ---- split-KV across GPUs with the exchange inside the kernels -------------------------
 * No counterpart in the reference (one GPU).  Instead of an all-gather after the attention
 * kernel, the kernel stores every partial into the gather buffer of every rank through
 * peer pointers (NVLink stores), and its last CTA publishes the rank's step number in a
 * flag on every rank; the merge kernel of a rank waits - bounded - until the flags of all
 * ranks carry the step, then merges the chunks in place.
 *   gather[w]  rank w's buffer, float [2][n_ranks][chunk_floats] (two step parities; a chunk
 *              is o [n_rows, n_parts, head_dim] followed, lse_offset floats in, by lse
 *              [n_rows, n_parts]); flags[w]  rank w's int32 [2][n_ranks], zero at start.
 *              Entry my_rank is this rank's own memory, the others are peer mappings of
 *              the same allocations (CUDA IPC or symmetric memory).
 *   step_counter, grid_counter  this rank's own int32 words, zero at start.
 * A wait that runs out sets IA_DEV_STATUS_PEER_WAIT in the device status word and the kernel
 * carries on (the output of that step is then invalid); nothing spins without a limit. */
typedef struct ia_peer_exchange {
  int32_t n_ranks, my_rank;
  float* gather[8];
  int32_t* flags[8];
  int64_t chunk_floats, lse_offset;
  int32_t* step_counter;
  int32_t* grid_counter;
} ia_peer_exchange;
/* Split-KV selection: every rank owns a contiguous range [block_lo, block_hi) of the logical blocks of
 * every sequence (block_lo a multiple of 32; block_hi a multiple of 32 or >= max_blocks) and only its
 * own range of the summary arrays needs to be valid.  No counterpart in the reference (one GPU; its
 * building blocks are the chunk partials of IMPL/core.py:806-814 and their re-reduction in
 * IMPL/page_attention.py:106-124).  The kernel streams the rank's summaries, exchanges the per-row
 * softmax normalisers with the other ranks, scores its blocks with the global normalisers, exchanges
 * its top_k best (score, block) candidates and takes the top_k of all candidates: sel_idx / sel_count
 * receive the global selection, identical on every rank and - up to the rounding of the normalisers'
 * merge order - the one ia_select computes from all blocks.  Both exchanges are plain peer stores
 * into the buffers below plus flags polled in the rank's own memory (bounded waits:
 * IA_DEV_STATUS_PEER_WAIT); no collective call, no multicast.  IA_SELECT_TOPK only.  The grid
 * (pairs x cluster) must fit the SMs at once.
 *   norm[w]   rank w's float [2][n_pairs][n_ranks][16][4]          (two step parities)
 *   cand[w]   rank w's float [2][n_pairs][n_ranks][max_sel + 1][2]
 *   flags[w]  rank w's int32 [2][2][n_pairs][n_ranks], zero at start
 *             n_pairs = batch * n_kv_heads; entry my_rank is this rank's own memory, the others are
 *             peer mappings of the same allocations
 *   step_counter, grid_counter  this rank's own int32 words, zero at start */
typedef struct ia_select_exchange {
  int32_t n_ranks, my_rank;
  float* norm[8];
  float* cand[8];
  int32_t* flags[8];
  int32_t* step_counter;
  int32_t* grid_counter;
} ia_select_exchange;
int ia_select_split(const void* q, const ia_summaries* summaries, const int32_t* prefix_lens,
                    const ia_geom* geom, int top_k, int max_sel, int block_lo, int block_hi,
                    int32_t* sel_idx, int32_t* sel_count, const ia_select_aux* aux,
                    const ia_select_exchange* exchange, ia_stream_t stream);

int ia_sparse_decode_exchange(const void* q, const void* k_pool, const void* v_pool, const int32_t* block_table,
                              const int32_t* prefix_lens, const int32_t* seq_lens, const int32_t* sel_idx,
                              const int32_t* sel_count, int max_sel, const ia_summaries* summaries, const float* z,
                              const ia_geom* geom, int rep_mode, int n_splits, int block_lo, int block_hi,
                              int with_suffix, const ia_peer_exchange* exchange, ia_stream_t stream);
int ia_finalize_exchange(const ia_peer_exchange* exchange, int n_rows, int n_parts, int head_dim, void* out,
                         int out_dtype, ia_stream_t stream);

/* The merge after an all-gather of split-KV partials across GPUs (the reference runs on one
 * GPU; its merge of chunk partials is the same arithmetic, IMPL/legacy.py:781-793).
 * `gathered` holds n_ranks chunks, rank_stride floats apart; a chunk is what one rank's
 * ia_sparse_decode wrote when its o_partial [n_rows, n_parts, head_dim] and lse_partial
 * [n_rows, n_parts] are adjacent in one buffer (o first).  out [n_rows, head_dim]. */
int ia_finalize_gathered(const float* gathered, int n_ranks, int64_t rank_stride, int n_rows, int n_parts,
                         int head_dim, void* out, int out_dtype, ia_stream_t stream);

/* Scratch needed by ia_decode_attention (and its _timed / _host forms), in bytes, on the current
 * device: the selection list, the split-KV partials of both attention grids and, in hybrid mode,
 * the representatives' logits. */
int64_t ia_workspace_bytes(const ia_geom* geom, int max_sel, int n_splits, int rep_mode);

/* A good n_splits for ia_sparse_decode / ia_decode_attention on the current
 * device, given how many blocks a (sequence, kv head) is expected to attend
 * (top_k, or a typical count in epsilon mode): picks the split count whose
 * grid fills whole waves of resident CTAs.  Host arithmetic only. */
int ia_suggest_splits(const ia_geom* geom, int expected_blocks);

/* One decode-attention layer-step, replacing
 * _condition_block_decode_output_fused_triton (IMPL/core.py:1035-1155): the
 * selection kernel, then the attention kernel with the split-KV finalize fused
 * in (the CTA that completes a (sequence, kv head) last merges its parts and
 * writes out) - two launches on one stream instead of the reference's three.
 * Every pair is cut into n_splits parts (ia_suggest_splits).  INTERATTN_B200_DECODE_GRID=flat in the
 * environment switches bf16 pools to a fixed grid of two CTAs per SM, each taking an equal share of
 * all pairs' pages whatever n_splits says (slower on B200 as measured; kept for comparison).
 * One launch instead of two where it applies - bf16 pools of 16-token pages with head_dim 128 and a
 * known size (geom->n_pool_pages > 0), at most eight query rows per kv head, the range bound, and a
 * batch whose selection grid is resident at once ((sequence, kv head) pairs x cluster size <= SMs x
 * CTAs per SM): the CTA (or cluster) that picked a pair's blocks then attends over their pages, which
 * it still has in shared memory - in hybrid mode also over the representatives, whose logits never
 * leave shared memory - and writes the output rows (condition_block_select_attend_kernel; n_splits
 * is not used).
 * INTERATTN_B200_FUSED=0 in the environment keeps the two launches.
 * workspace: ia_workspace_bytes() bytes, 256-byte aligned.  out [batch, rows, head_dim] in
 * geom->dtype, 16-byte aligned.  sel_idx/sel_count may be null (the selection then lives in the
 * workspace). */
int ia_decode_attention(const void* q, const void* k_pool, const void* v_pool,
                        const int32_t* block_table, const int32_t* prefix_lens,
                        const int32_t* seq_lens, const ia_summaries* summaries,
                        const ia_geom* geom, int mode, int top_k, float eps, int max_sel,
                        int rep_mode, int n_splits, void* workspace, int64_t workspace_bytes,
                        int32_t* sel_idx, int32_t* sel_count, void* out, ia_stream_t stream);

/* 1 when the calling thread's last ia_decode_attention (any form) ran as the single fused launch, else 0.
 * No reference counterpart: a reporting aid for benchmarks, which attribute time and bytes per kernel. */
int ia_last_decode_fused(void);

/* How the last completed one-kernel step on the current device split its time, in microseconds, as seen by
 * its first CTA: from kernel entry to the end of the routing (selection_us) and from there to the written
 * output rows (attention_us).  Reads device memory with a synchronous copy: call it where the host waits
 * anyway.  No reference counterpart: benchmarks report the two phases of the fused kernel separately. */
int ia_last_step_phases(double* selection_us, double* attention_us);

/* Process-wide switch of the one-kernel form (1 = allowed where it applies, the default unless
 * INTERATTN_B200_FUSED=0 is in the environment; 0 = always two launches).  Returns the previous setting.
 * No reference counterpart: for A/B measurements and for profiling the two kernels separately. */
int ia_set_fused_step(int enabled);

/* ia_decode_attention that also records four caller-created CUDA events
 * (cudaEvent_t, timing enabled) on the stream: events[0] before the selection
 * kernel, [1] between selection and attention, [2] and [3] after the
 * attention kernel (the finalize is fused into it) - per-kernel device times
 * of a live step without a profiler.  A null entry is skipped. */
int ia_decode_attention_timed(const void* q, const void* k_pool, const void* v_pool,
                              const int32_t* block_table, const int32_t* prefix_lens,
                              const int32_t* seq_lens, const ia_summaries* summaries,
                              const ia_geom* geom, int mode, int top_k, float eps, int max_sel,
                              int rep_mode, int n_splits, void* workspace, int64_t workspace_bytes,
                              int32_t* sel_idx, int32_t* sel_count, void* out, void* const* events,
                              ia_stream_t stream);

/* The same layer-step with HOST buffers, for callers that keep only the KV
 * pool and the summaries on the device: copies q_host -> device (async on
 * stream), runs ia_decode_attention, copies the output back into out_host and
 * waits for the stream.  q_dev/out_dev are caller-owned device staging
 * buffers of the same sizes; q_host/out_host should be pinned.  Pinned, 16-byte
 * aligned host buffers that the device can address are read and written by the
 * kernels directly (the query rows and the output rows cross PCIe without a copy
 * operation on the stream); anything else is staged through q_dev / out_dev. */
int ia_decode_attention_host(const void* q_host, void* q_dev, const void* k_pool,
                             const void* v_pool, const int32_t* block_table,
                             const int32_t* prefix_lens, const int32_t* seq_lens,
                             const ia_summaries* summaries, const ia_geom* geom, int mode,
                             int top_k, float eps, int max_sel, int rep_mode, int n_splits,
                             void* workspace, int64_t workspace_bytes, void* out_dev,
                             void* out_host, ia_stream_t stream);

/* ia_decode_attention for callers that cannot allocate device memory at all -
 * for example a plug-in inside an inference server that gave all of HBM to its
 * KV-cache pool at start-up, where a cudaMalloc made afterwards fails or
 * fragments that pool.  No counterpart in the reference (its scratch is a dict
 * of torch tensors, IMPL/core.py:558-570).
 *
 * Same step, same results, but the scratch (selection list, split-KV partials,
 * hybrid-mode logits) is a fixed IA_NOALLOC_SCRATCH_BYTES array inside the
 * library image instead of a caller workspace; every GPU that loads the
 * library holds that array until the process exits.  The caller still passes q,
 * the KV pool, the summaries and out [batch, rows, head_dim] (geom->dtype).
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine.
 *  - A step whose ia_workspace_bytes() exceeds IA_NOALLOC_SCRATCH_BYTES is
 *    refused with IA_ERR_UNSUPPORTED (at the Llama-3-8B geometry, batch 16,
 *    top-64, 2 splits the step needs about 4 MB on a 148-SM GPU; hybrid mode
 *    at 32k context about 5 MB).
 *  - The first call on each device looks up the array's device address (with
 *    that device current); make that first call before any stream capture.
 *  - All calls share the one array and it keeps the previous call's contents.
 *    Nothing in it needs clearing between calls, but two calls that overlap on
 *    the GPU (different streams, or different host threads) race on it: keep
 *    the calls of one device on one stream, or order them with events. */
#define IA_NOALLOC_SCRATCH_BYTES (8 * 1024 * 1024)
int64_t ia_noalloc_scratch_bytes(void);
int ia_decode_attention_noalloc(const void* q, const void* k_pool, const void* v_pool,
                                const int32_t* block_table, const int32_t* prefix_lens,
                                const int32_t* seq_lens, const ia_summaries* summaries,
                                const ia_geom* geom, int mode, int top_k, float eps, int max_sel,
                                int rep_mode, int n_splits, void* out, ia_stream_t stream);

/* ---- the element-wise part of a batched Llama decode step -----------------------
 * The reference replays the Hugging Face model's own PyTorch ops around its
 * attention hook inside one captured decode step (IMPL/core.py:190-316,
 * _generate_condition_block_cuda_graph); each entry point below replaces one
 * group of those ops by a single launch and keeps their bf16 rounding points
 * (transformers 5.5.0, models/llama/modeling_llama.py).  All tensors are bf16
 * device memory, rows contiguous, pointers 16-byte aligned.
 *
 * ia_llama_add_rmsnorm - LlamaDecoderLayer's `residual + hidden_states` followed
 *   by LlamaRMSNorm.forward (modeling_llama.py:62-67).  residual [n_rows, hidden]
 *   is updated in place with bf16(residual + delta) when delta is not null;
 *   out = weight * bf16(x * rsqrt(mean(x^2) + eps)).
 * ia_llama_rope_append - apply_rotary_pos_emb (modeling_llama.py:146-168) on the
 *   q and k heads of the fused projection row qkv [batch, (Hq + 2 Hkv) * D],
 *   with cos/sin rows [max_pos, D] as LlamaRotaryEmbedding.forward returns them,
 *   fused with the static cache's update (one index_copy_ per tensor in
 *   transformers/cache_utils.py StaticLayer.update): sequence b's token sits at
 *   position seq_lens[b] - 1; k (rotated) and v go to
 *   cache + b * cache_seq_stride + h * cache_head_stride + position * D (element
 *   strides), q (rotated) to q_out [batch, Hq, D].
 * ia_llama_silu_mul - LlamaMLP.forward's act_fn(gate) * up on the fused
 *   projection row gate_up [n_rows, 2 * intermediate] -> out [n_rows, intermediate].
 * ia_llama_argmax - the greedy `logits.argmax(-1)` of the generation loop
 *   (IMPL/core.py:136, 178, 281); lowest index among equal maxima; out int64 [n_rows]. */
int ia_llama_add_rmsnorm(void* residual, const void* delta, const void* weight, void* out, int n_rows,
                         int hidden, float eps, ia_stream_t stream);
int ia_llama_rope_append(const void* qkv, const void* cos_table, const void* sin_table, int max_pos,
                         const int32_t* seq_lens, void* k_cache, void* v_cache, int64_t cache_seq_stride,
                         int64_t cache_head_stride, int cache_len, void* q_out, int batch, int n_q_heads,
                         int n_kv_heads, int head_dim, ia_stream_t stream);
int ia_llama_silu_mul(const void* gate_up, void* out, int n_rows, int intermediate, ia_stream_t stream);
int ia_llama_argmax(const void* logits, int64_t row_stride, int n_rows, int vocab, int64_t* out,
                    ia_stream_t stream);

/* out[m, n] = x[m, k] * w[n, k]^T - nn.Linear without bias as the Llama modules
 * call it (modeling_llama.py: q/k/v/o_proj, gate/up/down_proj, lm_head) for a
 * decode batch of m <= 32 rows; bf16 in and out, fp32 accumulation, rows
 * contiguous, k a multiple of 8.  The kernel is bound by reading the weights once;
 * several projections of the same input run as one call on their row-concatenated
 * weights.
 * The weights are static, so they are packed once: ia_llama_gemm_pack turns the
 * row-major w [n, k] into ia_llama_gemm_packed_bytes(n, k) bytes (tiles of 128 rows
 * x 64 columns in the order and shared-memory layout the kernel streams them;
 * ragged edges zero-filled), and ia_llama_gemm takes that packed buffer.
 * workspace: ia_llama_gemm_workspace_bytes(n) bytes, 16-byte aligned, zero before
 * its first use and left zero where it has to be by every call; calls that
 * overlap on the GPU need workspaces of their own. */
int64_t ia_llama_gemm_packed_bytes(int n, int k);
int ia_llama_gemm_pack(const void* w, int n, int k, void* packed, ia_stream_t stream);
int64_t ia_llama_gemm_workspace_bytes(int n);
int ia_llama_gemm(const void* x, const void* w_packed, void* out, int m, int n, int k, void* workspace,
                  int64_t workspace_bytes, ia_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* INTERATTN_B200_H_ */
