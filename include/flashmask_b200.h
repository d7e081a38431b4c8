/*
 * flashmask_b200.h — C ABI of libflashmask_b200.so (sm_100a only).
 *
 * Every entry point is `extern "C"`, takes plain pointers / integers, enqueues
 * its work on the CUDA stream it is given and returns an int status
 * (FM_OK == 0).  On failure nothing is launched (argument errors) or the CUDA
 * error is captured; `fm_last_error()` returns a thread-local message.
 * Nothing here allocates device memory unless its comment says so: outputs and
 * workspaces are owned by the caller, and `*_workspace_bytes` says how large
 * a workspace must be.
 *
 * Reference interfaces replaced (paths inside PaddlePaddle/FlashMask):
 *   flashmask/cute/flashmask_utils.py  (prepare_block_maxmin, reduce_block_count)
 *   flashmask/cute/ops/fwd.py          (_flash_attn_fwd)
 *   flashmask/cute/ops/bwd.py          (_flash_attn_bwd)
 *   flashmask/cp_balance/csrc/cp_balance_bridge.cu (fm_cpb_* C ABI)
 */
#ifndef FLASHMASK_B200_H_
#define FLASHMASK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Exported symbol marker (the library is built with hidden visibility). */
#if defined(__GNUC__)
#define FM_API __attribute__((visibility("default")))
#else
#define FM_API
#endif

#define FM_OK 0
#define FM_ERR_INVALID_ARGUMENT 1
#define FM_ERR_UNSUPPORTED 2
#define FM_ERR_CUDA 3
#define FM_ERR_WORKSPACE 4
#define FM_ERR_TIMEOUT 5

#define FM_DTYPE_BF16 0
#define FM_DTYPE_FP16 1

/* Tile classes written by fm_mask_prepare (one int8 per (Q tile, K tile)). */
#define FM_TILE_SKIP 0    /* fully masked: never computed */
#define FM_TILE_PARTIAL 1 /* element-wise mask applied from the column bounds */
#define FM_TILE_FULL 2    /* unmasked */

/* Order of the eight per-K-tile reductions inside the `minmax` buffer:
 * minmax[(which * BHm + bh) * nblk_pad + n], which in
 * {LTSmax, LTSmin, LTEmax, LTEmin, UTSmax, UTSmin, UTEmax, UTEmin}.
 * Reductions of bounds the mask does not carry are left untouched. */
#define FM_MM_LTS_MAX 0
#define FM_MM_LTS_MIN 1
#define FM_MM_LTE_MAX 2
#define FM_MM_LTE_MIN 3
#define FM_MM_UTS_MAX 4
#define FM_MM_UTS_MIN 5
#define FM_MM_UTE_MAX 6
#define FM_MM_UTE_MIN 7

/* Library / build information: returns "flashmask_b200 <version> sm_100a". */
FM_API const char* fm_version(void);
/* Message of the last failure on the calling thread ("" when none). */
FM_API const char* fm_last_error(void);

/* Padded number of K tiles per (batch, mask head) row of `minmax`:
 * ((ceil(Sk / tile_n) + 3) & ~3).
 * Replaces _compute_nblock_seqlen, flashmask/cute/flashmask_utils.py:96-103. */
FM_API int fm_mask_nblk_pad(int Sk, int tile_n);

/*
 * Mask preprocessing + tile classification.
 *
 *   mask       [B, Hm, Sk, ncols] int32, contiguous.  Column meaning:
 *              ncols=1 [LTS]; causal ncols=2 [LTS,LTE]; non-causal ncols=2
 *              [LTS,UTE]; ncols=4 [LTS,LTE,UTS,UTE].
 *   minmax     out, int32 [8, B*Hm, nblk_pad] (see FM_MM_*); max is reduced
 *              from 0 and min from INT_MAX; pad entries are written as 0.
 *   valid_cnt  out (may be NULL), int32 [B, Hm, ceil(Sq/tile_m)]: number of K
 *              tiles below the causal limit that are not fully masked.
 *   tile_class out (may be NULL), int8 [B, Hm, ceil(Sq/tile_m), ceil(Sk/tile_n)]
 *              FM_TILE_* including causal / ragged-edge geometry.
 *
 * Replaces prepare_block_maxmin + scan_max_min_kernel
 * (flashmask/cute/flashmask_utils.py:106-190,227-282), reduce_block_count
 * (:357-424,472-548) and the classification predicates of
 * compute_flashmask_block_lists (:567-708) /
 * flash_fwd_sm100.py:2297-2427 (generate_block).
 */
FM_API int fm_mask_prepare(const int32_t* mask, int B, int Hm, int Sq, int Sk, int ncols,
                    int causal, int tile_m, int tile_n, int32_t* minmax,
                    int32_t* valid_cnt, int8_t* tile_class, void* stream);

/*
 * Exact number of unmasked (query, key) pairs per (batch, mask head), from the
 * bounds alone (element exact, O(Sk) per row).  out: int64 [B, Hm].
 * No counterpart kernel in the reference; it is the work measure of the
 * unmasked-FLOP throughput metric (tests/common/bench_utils.py:21-29 uses a
 * 128x128 block density instead).
 */
FM_API int fm_mask_count_visible(const int32_t* mask, int B, int Hm, int Sq, int Sk,
                          int ncols, int causal, int64_t* out, void* stream);

/* dQ of several backward calls over the same queries (context parallel: own
 * shard, pulled shards) can be summed inside the fp32 accumulator of the
 * one-kernel backward instead of being rounded per call and added afterwards:
 * the first call sets FM_BWD_DQ_LEAVE (dq is not written, the accumulator keeps
 * the sums), later calls pass the SAME workspace and set FM_BWD_DQ_CARRY (the
 * accumulator is not cleared), the last one leaves FM_BWD_DQ_LEAVE off and
 * writes dq once.  Ignored by the other backward variants; fm_bwd_accumulates()
 * says whether the variant a call would take honours them. */
#define FM_BWD_DQ_CARRY 1
#define FM_BWD_DQ_LEAVE 2

/* Arguments shared by forward and backward.  Strides are in ELEMENTS; the
 * innermost (head-dim) stride is 1.  Layouts follow the reference:
 * q/o/do/dq [B,Sq,Hq,*], k/dk [B,Sk,Hkv,d], v/dv [B,Sk,Hkv,dv],
 * lse [B,Hq,Sq] fp32 natural log (flashmask/cute/ops/fwd.py:52-110). */
typedef struct fm_attn_args {
  int32_t B, Sq, Sk, Hq, Hkv, Hm;
  int32_t d, dv;      /* head dims of q/k and of v/o                        */
  int32_t ncols;      /* 0 = no mask tensor, else 1 | 2 | 4                  */
  int32_t causal;     /* bottom-right aligned causal triangle               */
  int32_t dtype;      /* FM_DTYPE_*                                          */
  int32_t mask_B;     /* batch of the mask tensor: B or 1 (broadcast)        */
  int32_t tile_m, tile_n; /* tile shape `minmax` was prepared for            */
  int32_t deterministic;  /* backward only: 1 = fixed summation order, bitwise
                             reproducible gradients (two tcgen05 kernels, one
                             owner per output element); 0 = the one-kernel
                             backward may be used (d = dv = 64 or 128), whose dQ
                             is summed by reductions in an order that is not
                             fixed                                            */
  int32_t bwd_flags;      /* backward only, one-kernel variant: FM_BWD_* bits below, 0 = a
                             self-contained call                               */
  float softmax_scale;
  float reserved1;
  const void* q; const void* k; const void* v;
  void* o; float* lse;
  const int32_t* mask;   /* [mask_B,Hm,Sk,ncols] or NULL                    */
  const int32_t* minmax; /* from fm_mask_prepare or NULL when ncols == 0    */
  const float* sink;     /* [Hq] fp32 or NULL                                */
  /* backward */
  const void* d_o; void* dq; void* dk; void* dv_out; float* dsink;
  void* workspace; size_t workspace_bytes;
  int64_t q_stride[3];  /* batch, seq, head */
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int64_t do_stride[3];
  int64_t dq_stride[3];
  int64_t dk_stride[3];
  int64_t dv_stride[3];
  /* Optional launch orders from fm_launch_order (NULL: tiles in index order).
   * The entries are only read, but the 4 counters at the end of a backward table
   * are advanced and rewound by every fm_bwd launch that walks it: a table must not
   * be shared by two backward launches that can overlap on the GPU (two streams
   * without an ordering between them); build one table per stream instead. */
  const int32_t* fwd_order;  /* FM_ORDER_FWD, read by fm_fwd                     */
  const int32_t* dq_order;   /* FM_ORDER_BWD_DQ, walked by fm_bwd                */
  const int32_t* dkdv_order; /* FM_ORDER_BWD_DKDV, walked by fm_bwd              */
} fm_attn_args;

/* Tile shape (rows of Q, columns of K per tile) the forward / backward kernel
 * variant for (d, dv) classifies and skips on; `minmax` must be prepared with
 * the matching tile_n.  Returns FM_ERR_UNSUPPORTED for head dims outside
 * {<=64, <=128, 192/128, 256/256, 512/512, 576/512}
 * (flashmask/cute/ops/_common.py:95-132). */
FM_API int fm_fwd_tile_shape(int d, int dv, int* tile_m, int* tile_n);
FM_API int fm_bwd_tile_shape(int d, int dv, int* tile_m, int* tile_n);

/* The library reads its A/B switches from the environment once, when it is loaded
 * (FLASHMASK_B200_FWD=mma / FLASHMASK_B200_BWD=mma: warp-MMA kernels for every head
 * dim; FLASHMASK_B200_BWD=split: the two-kernel tcgen05 backward even when
 * args->deterministic is 0; FLASHMASK_B200_PERSIST=0: one unit per CTA in that
 * backward; FLASHMASK_B200_CLASSES=n: work classes of the launch tables).  A host
 * that changes them afterwards calls fm_reload_options() to have them read again;
 * no other entry point touches the environment.  No counterpart in the reference,
 * which reads its switches per call in Python. */
FM_API int fm_reload_options(void);

/* Number of kernels this library has launched in this process so far (all
 * entry points, all streams).  A benchmark reads it before and after its timed
 * region to state how many launches that region made.  No counterpart in the
 * reference. */
FM_API unsigned long long fm_launch_count(void);

/* Forward: O = softmax(QK^T*scale + M [, sink]) V and LSE.
 * Replaces _flash_attn_fwd (flashmask/cute/ops/fwd.py:52-882) +
 * FlashAttentionForwardSm100 (flashmask/cute/flash_fwd_sm100.py:1485-2104).
 * Uses no workspace. */
FM_API int fm_fwd(const fm_attn_args* args, void* stream);

/* fm_fwd with the fused block-score side output: besides O and LSE, for every
 * query row and every block of `block_size` key columns the maximum of the
 * masked, scaled scores softmax_scale * q.k (the values softmax is fed) goes to
 *   block_logit[((b * Hq + head) * Sq + row) * block_ld + block]   (fp32).
 * Masked columns count as -inf.  Only the K tiles the attention loop visits are
 * written, so the caller fills block_logit with -inf first; a block that lies
 * inside one K tile is stored as it is, a block that straddles two tiles (only
 * possible with block_bos) is merged into the entry with fmax.
 * With block_bos ([B, Sq] int32, first key column of the row's document) block
 * ids are relative to that column: block j of a row covers the columns
 * [bos + j * block_size, bos + (j + 1) * block_size); NULL means bos = 0.
 * block_size is 32, 64 or 128; block_ld >= ceil(Sk / block_size); O and LSE
 * are bitwise those of fm_fwd.  Every head dim fm_fwd takes is served.
 * Replaces the block_logit / block_size / block_bos arguments of
 * _flash_attn_fwd (flashmask/cute/ops/fwd.py:75-77,605-658) and the fused
 * epilogue of flashmask/cute/flash_fwd_sm100.py:4256-4371. */
FM_API int fm_fwd_block_score(const fm_attn_args* args, float* block_logit, int block_size, int block_ld,
                              const int32_t* block_bos, void* stream);

/*
 * Longest-work-first launch order for sparse masks.  A kernel's CTAs are handed
 * to the SMs in launch order, so starting the heaviest tiles first keeps the
 * tail of the launch short when tiles differ widely in the number of K tiles
 * (or query tiles) the mask leaves them.  `which` selects the kernel:
 * FM_ORDER_FWD (units of 256 query rows), FM_ORDER_BWD_DQ (128 query rows),
 * FM_ORDER_BWD_DKDV (one 128-column K tile; work = 64-row query blocks kept).
 * Units are dealt into 8 work classes relative to the heaviest unit; the launch
 * runs class by class, heaviest first, and inside a class head by head with
 * the units in index order, so neighbouring CTAs still share operands in L2.
 * Only the problem geometry of `args` is read (B, Hq, Hkv, mask_B, Hm, Sq, Sk,
 * ncols, causal, d, dv, minmax, tile_n).  With E = mask_B*Hm*units and
 * N = E * (heads/Hm) * (B/mask_B) = the number of CTAs of the kernel:
 *   fm_launch_order_ints  number of int32 `out` must hold, 2*N + 2*E + 4, or 0
 *                         when the kernel variant for (d, dv) takes no order,
 *                         there is no mask tensor, or E > 4096.
 *   fm_launch_order       out[2L], out[2L+1] = (unit, b*heads + head) of the
 *                         L-th CTA in dispatch order; then E ints of work per
 *                         unit (mask_b, mask_h, unit flattened) and E ints of
 *                         the units by (class, index), then 4 ints of counters
 *                         that the backward kernels, which walk their table
 *                         persistently (one CTA per SM fetching entries through
 *                         a counter), advance and rewind on every launch: one
 *                         table serves one stream at a time.  `out` is 8-byte
 *                         aligned.  Pass it as the matching *_order field of
 *                         later fm_fwd / fm_bwd calls with the same mask and
 *                         the same B, Hq, Hkv.
 * Plays the role of the reference's longest-processing-time tile schedulers
 * (flashmask/cute/tile_scheduler.py:400-539, 542-660), which order by causal
 * geometry only; here the order follows the mask itself.
 */
#define FM_ORDER_FWD 0
#define FM_ORDER_BWD_DQ 1
#define FM_ORDER_BWD_DKDV 2
FM_API int64_t fm_launch_order_ints(const fm_attn_args* args, int which);
FM_API int fm_launch_order(const fm_attn_args* args, int which, int32_t* out, void* stream);
/* The same for up to three kernels in ONE launch (a NULL pointer skips that kernel's table). */
FM_API int fm_launch_orders(const fm_attn_args* args, int32_t* out_fwd, int32_t* out_dq, int32_t* out_dkdv,
                            void* stream);

/* Device-side status of the kernels that wait on barriers (the tcgen05
 * variants): every wait is bounded, and a wait that ran out makes its CTA
 * unwind and record FM_ERR_TIMEOUT here instead of hanging.  Synchronises the
 * device (debug / test use; not called on the hot path).  `reset` != 0 clears
 * the word.  The reference instead traps the GPU from its spin watchdog
 * (flashmask/cute/barrier.py:95-148). */
FM_API int fm_kernel_status(int* status, int reset);

/* Launches one CTA that waits, with a budget of `budget_us` microseconds, on a
 * barrier nothing arrives on: the wait gives up, the kernel returns normally
 * and fm_kernel_status reports FM_ERR_TIMEOUT.  Failure-detection self test of
 * the bounded-wait machinery every tcgen05 kernel uses; no GPU fault, trap or
 * hang is involved.  (The reference's watchdog traps instead,
 * flashmask/cute/barrier.py:95-148.) */
FM_API int fm_selftest_bounded_wait(int budget_us, void* stream);

/* Backward: dQ, dK, dV (and dsink when sink != NULL).
 * Replaces _flash_attn_bwd (flashmask/cute/ops/bwd.py:56-1261): preprocess
 * (flash_bwd_preprocess.py:184-342), main (flash_bwd_sm100.py:1435-),
 * postprocess (flash_bwd_postprocess.py:309-) and dsink
 * (flash_bwd_sink.py:67-114).  `workspace` must hold
 * fm_bwd_workspace_bytes(args) bytes; its contents need no initialisation.
 * The size depends on args->deterministic: the one-kernel backward
 * (flash_bwd_sm100.py:129-140: S, dP, dV, dK and dQ of a tile pair computed once)
 * adds an fp32 dQ accumulator [B, Hq, roundup(Sq,128), 64|128] behind the row
 * statistics, the role of the reference's dq_accum (ops/bwd.py:366-383), which it
 * clears itself and rounds into dq with one more small kernel (the reference's
 * postprocess, flash_bwd_postprocess.py).  Ask for the size with the same
 * args->deterministic the call will carry. */
FM_API size_t fm_bwd_workspace_bytes(const fm_attn_args* args);
/* 1 when fm_bwd(args) would run the one-kernel variant (and so honours
 * args->bwd_flags), else 0. */
FM_API int fm_bwd_accumulates(const fm_attn_args* args);
FM_API int fm_bwd(const fm_attn_args* args, void* stream);

/* ------------------------------------------------------------------------
 * Context parallel (sequence sharded over ranks)
 * ------------------------------------------------------------------------ */

/* Workload per balance chunk: out[h, c] = {sum over batch and over the 128-row
 * blocks of chunk c of valid_cnt, c}; out is int32 [Hm, ceil(Tq/blocks_per_chunk), 2].
 * `valid_cnt` comes from fm_mask_prepare(causal=0, tile 128x128).
 * Replaces get_q_workload + reduce_workload_kernel
 * (flashmask/cp_balance/cp_balance.py:11-93, csrc/cp_balance_bridge.cu:74-151);
 * only real K blocks are counted (the reference also walks the uninitialised
 * pad entries of its scan output, which is only well defined when S % 512 == 0,
 * where both agree). */
FM_API int fm_cp_chunk_workload(const int32_t* valid_cnt, int B, int Hm, int Tq, int blocks_per_chunk,
                                int32_t* out, void* stream);

/* LPT heap partition of n weighted tasks into n_buckets buckets of capacity
 * n / n_buckets (HOST pointers).  bucket_of[t] = bucket of task t.
 * Replaces assign_tasks_heap (flashmask/cp_balance/cp_balance.py:96-174). */
FM_API int fm_cp_partition_heap(const int32_t* weights, int n, int n_buckets, int32_t* bucket_of);

/* Iterative pairwise / triple optimal repartition of n weighted tasks into
 * n_buckets buckets of exactly n / n_buckets tasks each (HOST pointers):
 * assign[j * (n / n_buckets) + t] = index of the t-th task of bucket j, in the
 * solver's order; *max_load (may be NULL) = the heaviest bucket.  Requires
 * n % n_buckets == 0, n <= 512, n_buckets <= 32 (FM_ERR_UNSUPPORTED beyond: the
 * caller falls back to the heap partition, as assign_tasks_ipo does).
 * Replaces CpBalanceSolver::solve_to (flashmask/cp_balance/csrc/cp_balance_fast.hpp:86-100,
 * core :416-581) behind cp_balance_ipo_solve (cp_balance_cuda_kernels.py) and
 * assign_tasks_ipo (flashmask/cp_balance/cp_balance.py:177-228). */
FM_API int fm_cp_partition_ipo(const int32_t* weights, int n, int n_buckets, int32_t* assign,
                               int64_t* max_load);

/* Gather the key axis of the mask into chunk order `chunk_idx`:
 * out[b,h,c*C + r,:] = mask[b,h,chunk_idx[c]*C + r,:].
 * Replaces indices_rerank_kernel (csrc/cp_balance_bridge.cu:185-216). */
FM_API int fm_cp_rerank(const int32_t* mask, const int32_t* chunk_idx, int32_t* out, int B, int H, int S,
                        int D, int n_chunks, int chunk_size, void* stream);

/* Map global row bounds into the row space of the rank that owns chunks
 * `local_chunk_idx` (n elements of `mask`, any shape).
 * Replaces indices_to_chunks_kernel (csrc/cp_balance_bridge.cu:153-183). */
FM_API int fm_cp_localize(const int32_t* mask, const int32_t* local_chunk_idx, int32_t* out, int64_t n,
                          int n_local, int chunk_size, void* stream);

/* out[(b*Hm+h), s] = unmasked pairs between the Sq local rows and key shard s
 * (Sk / n_shards columns each): a rank needs shard s iff the sum over (b,h) is
 * non-zero.  Plays the role of ChunkMaskKernel
 * (flashmask/overlap/csrc/distributed/remote_get_kernel.cuh:45-71). */
FM_API int fm_cp_shard_visible(const int32_t* mask, int B, int Hm, int Sq, int Sk, int ncols, int causal,
                               int n_shards, int64_t* out, void* stream);

/* Running log-sum-exp merge of forward partials (acc fp32 [B,S,H,dv],
 * lse_run fp32 [B,H,S]) with (o_s 16-bit [B,S,H,dv], lse_s): first != 0
 * initialises.  fm_cp_cast rounds the accumulator to the 16-bit output.
 * No reference counterpart: the reference gathers K/V and runs one kernel
 * (tests/torch/distributed/all_gather_flashmask.py:29-111). */
FM_API int fm_cp_merge_partial(float* acc, float* lse_run, const void* o_s, const float* lse_s, int B, int S,
                               int H, int dv, int dtype, int first, void* stream);
/* The same merge for exactly two partials, written straight to the 16-bit output
 * (out [B,S,H,dv], lse_out [B,H,S]) with one rounding: what the context-parallel
 * forward needs (own shard + pulled shards).  May run in place (out == o_a). */
FM_API int fm_cp_merge_two(const void* o_a, const float* lse_a, const void* o_b, const float* lse_b, void* out,
                           float* lse_out, int B, int S, int H, int dv, int dtype, void* stream);
FM_API int fm_cp_accumulate(float* acc, const void* x, int64_t n, int dtype, int first, void* stream);
FM_API int fm_cp_cast(const float* acc, void* out, int64_t n, int dtype, void* stream);

/* out = round(sum_i fp32(parts[i])) in index order (deterministic); parts is
 * a HOST array of n_parts <= 64 device pointers to 16-bit arrays of n elements.
 * Replaces ReducedKdVKernel (flashmask/overlap/csrc/distributed/dk_dv_reduce_bf16.cuh:58-168). */
FM_API int fm_cp_reduce_partials(const void* const* parts, int n_parts, void* out, int64_t n, int dtype,
                                 void* stream);

/*
 * Backward without any allocation, for callers that cannot provide device
 * memory of their own at call time: code running under a memory pool that is
 * frozen (an inference / training runtime that sized its arena at start-up),
 * a host thread that is not allowed to touch the CUDA allocator, or a plug-in
 * boundary where the caller only owns the tensors it passes.  It has no
 * counterpart in the reference, whose backward always allocates its own
 * workspaces (flashmask/cute/ops/bwd.py:358-499).
 *
 * Same arguments and results as fm_bwd, except that args->workspace is
 * ignored: the per-row scratch lives in a fixed 8 MiB array inside the library
 * image on every GPU that loads it.  Limit: B * Hq * roundup(Sq, 128) must not
 * exceed 1,048,576 rows (e.g. B=2, Hq=32, Sq=8192 uses half of it); larger
 * problems are rejected with FM_ERR_WORKSPACE before anything is launched.
 * The call makes no cudaMalloc / cudaFree and uses no allocating library
 * routine.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress with that device current), so make that first call
 * outside of any stream capture.  All calls on a device share the one array:
 * two calls whose kernels may overlap on the GPU (different streams without an
 * ordering between them) race on it; calls on one stream are safe, and a call
 * never depends on what an earlier call left in the array.
 */
FM_API int fm_bwd_static_scratch(const fm_attn_args* args, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FLASHMASK_B200_H_ */
