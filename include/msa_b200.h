/*
 * msa_b200.h -- C ABI of libmsa_b200.so, the sm_100a implementation of the
 * MiniMax-Sparse-Attention hot path (paged / sparse FMHA forward, page top-k
 * selection, split-KV LSE merge).
 *
 * Every entry point replaces one native export of the upstream msa_for_sail
 * package (paths below are relative to the upstream project root).  All
 * functions take plain pointers and sizes, enqueue work on the given CUDA
 * stream, never synchronise, and return 0 or a negative MSA_ERR_* code.
 * Unless stated otherwise they allocate nothing: every buffer is owned by the
 * caller (upstream: "every tensor is allocated by Python", api.py:1374-1389).
 */
#ifndef MSA_B200_H_
#define MSA_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MSA_OK               0
#define MSA_ERR_BAD_ARG     -1   /* NULL / inconsistent argument                    */
#define MSA_ERR_UNSUPPORTED -2   /* combination the library does not implement     */
#define MSA_ERR_LAUNCH      -3   /* cudaGetLastError() after the launch was not OK */
#define MSA_ERR_TOO_LARGE   -4   /* size beyond a documented maximum               */

/* element types */
#define MSA_DT_BF16 0
#define MSA_DT_E4M3 1
#define MSA_DT_F32  2

/* msa_fmha_fwd mode bits (upstream SparseAttnMode, csrc/include/fmha_fusion.hpp:42-54) */
#define MSA_FLAG_OUT_O      1   /* compute P.V and write O                      */
#define MSA_FLAG_OUT_SCORE  2   /* write per-128-key-tile row max of raw q.k    */
#define MSA_FLAG_SPARSE     4   /* iterate kv_block_indexes instead of all keys */

/* device status word values (written only when MsaFmhaParams.status != NULL) */
#define MSA_STATUS_OK        0
#define MSA_STATUS_TIMEOUT   1   /* a bounded wait inside a kernel gave up       */
#define MSA_STATUS_BOUNDS    2   /* bounds-checked build only (-DMSA_BOUNDS_CHECK): an index read from a
                                    caller's table (work item, page table, token -> batch map) was out of
                                    range; it was clamped into range before use                            */

typedef void* msa_stream_t;      /* a cudaStream_t */

/* One unit of dense work: BLOCK_M packed rows of one (batch item, head group)
 * against KV tiles [kv_tile_begin, kv_tile_end) of 128 keys.  Replaces the
 * upstream 64-bit packed work item + kv_tile_begin/end/split arrays
 * (csrc/include/fmha_tile_scheduler.hpp:49-55, api.py:841-845). */
typedef struct MsaWorkItem {
  int32_t batch;          /* batch item                                            */
  int32_t head0;          /* first query head covered by this item                 */
  int32_t row0;           /* first packed row (row = token_in_seq * pack + head_in_pack) */
  int32_t kv_tile_begin;  /* first 128-key tile                                    */
  int32_t kv_tile_end;    /* one past the last tile                                */
  int32_t split;          /* split index for the partial workspace (0 if unsplit)  */
  int32_t num_rows;       /* packed rows of this item (<= block_m)                  */
  int32_t reserved;
} MsaWorkItem;

/* Arguments of the FMHA forward.  Field-for-field successor of the upstream
 * FMHACutlassSailParams (csrc/fmha_sail_params.h:10-77) minus the PPU-only
 * members.  Strides are in elements. */
typedef struct MsaFmhaParams {
  const void*    q;                /* [total_q, Hq, 128] bf16 | e4m3                         */
  const void*    k;                /* ragged [sum_kv, Hkv, 128] or paged 4-D, bf16 | e4m3   */
  const void*    v;                /* same layout as k (may be NULL without MSA_FLAG_OUT_O)  */
  void*          out;              /* [total_q, Hq, 128] bf16 or NULL                        */
  float*         lse;              /* [total_q, Hq] natural-log LSE or NULL                  */
  void*          max_score;        /* [Hq, max_k_tiles, total_q] f32 | bf16 or NULL          */
  float*         partial_o;        /* split workspace [S, total_q, Hq, 128] f32 or NULL      */
  float*         partial_lse;      /* split workspace [S, total_q, Hq] f32 or NULL           */
  const int32_t* qo_start;         /* [B+1] first token of each batch item                   */
  const int32_t* kv_start;         /* [B+1] first key of each item (ragged only)             */
  const int32_t* kv_len;           /* [B]                                                    */
  const int32_t* qo_offset;        /* [B] row i sees key j iff i + qo_offset >= j            */
  const int32_t* kv_page_indptr;   /* [B+1] (paged)                                          */
  const int32_t* kv_indices;       /* flat physical page table (paged)                       */
  const int32_t* kv_block_indexes; /* [total_q, Hkv, kv_block_num] logical pages (sparse)    */
  const int32_t* token_batch;      /* [total_q] batch item of each token (sparse)            */
  const MsaWorkItem* work;         /* [num_work] (dense)                                     */
  const float*   k_scale_head;     /* optional [Hkv] de-quantisation scale of K             */
  const float*   v_scale_head;     /* optional [Hkv] de-quantisation scale of V             */
  int32_t*       status;           /* optional device status word                            */
  const int32_t* page_batch;       /* optional [num_logical_pages] batch item owning each entry of kv_indices */
  void*          sparse_ws;        /* optional workspace of msa_sparse_workspace_bytes() bytes: enables the
                                      page-major (KV-outer) sparse prefill path                             */
  int64_t        sparse_ws_bytes;
  int64_t q_stride_tok, q_stride_head;
  int64_t k_stride_page, k_stride_head, k_stride_tok;   /* ragged: page stride unused       */
  int64_t v_stride_page, v_stride_head, v_stride_tok;
  int64_t out_stride_tok, out_stride_head;
  int64_t kbi_stride_tok, kbi_stride_head;
  int64_t kv_extent;       /* outermost extent of k / v: total keys (ragged) or pages in the pool */
  int32_t total_q, num_qo_heads, num_kv_heads, batch;
  int32_t num_work;        /* dense: work items; sparse: ignored                             */
  int32_t block_m;         /* 16, 64, 128 packed rows per item; 256 selects the tcgen05 kernel */
  int32_t pack;            /* query heads folded into the row dimension (1 or Hq/Hkv)        */
  int32_t page_size;       /* 0 = ragged K/V                                                 */
  int32_t kv_block_num;    /* sparse: entries per (token, kv head)                           */
  int32_t num_splits;      /* size of the S dimension of the partial workspace (1 = unsplit) */
  int32_t max_k_tiles;     /* second dimension of max_score                                  */
  int32_t num_logical_pages; /* length of kv_indices (sparse page-major path)                        */
  int32_t decode_rows;     /* > 0: every item has at most this many packed rows (<= 128) and may run on the
                              tcgen05 decode kernel; 0: do not use it                                 */
  int32_t q_dtype, kv_dtype, max_score_dtype;
  int32_t flags;           /* MSA_FLAG_*                                                     */
  float   sm_scale;        /* q_scale * k_scale * softmax scale                              */
  float   out_scale;       /* v_scale * o_scale                                              */
} MsaFmhaParams;

/* FMHA forward: dense ragged / dense paged / sparse, optional split-KV partials.
 * Replaces the per-variant export `run` (csrc/fmha_sail_variant_run.cu.jinja:17-43,261
 * -> run_fmha_fwd, csrc/include/fmha_cutlass_sm80.cuh:185-486).  With
 * partial_o != NULL the kernel writes normalised partial O and LSE per split
 * and the caller runs msa_lse_merge afterwards. */
int msa_fmha_fwd(const MsaFmhaParams* params, msa_stream_t stream);

/* Bytes of MsaFmhaParams.sparse_ws needed by the page-major sparse prefill path (reverse
 * index page -> tokens, per-slot partial O in bf16 and LSE).  No upstream counterpart: there
 * sparse attention always runs token by token (csrc/include/prepare_plan_metadata.cuh:90-112). */
int64_t msa_sparse_workspace_bytes(int64_t total_q, int32_t num_qo_heads, int32_t num_kv_heads,
                                   int32_t kv_block_num, int64_t num_logical_pages);

/* Split-KV merge: out[t,h,:] = sum_s w_s * partial_o[s,t,h,:] / sum_s w_s with
 * w_s = exp(partial_lse[s,t,h] - max_s); a -inf LSE gives weight 0 and its
 * partial is ignored.  splits_per_row ([total_q] or NULL = num_splits for all)
 * bounds s per token.  Replaces `reduction` (csrc/fmha_sm80_reduction.cu:42-104,
 * csrc/include/sm80_fmha_reduction.hpp:74-216). */
int msa_lse_merge(const void* partial_o, int32_t partial_dtype /* MSA_DT_F32 | MSA_DT_BF16 */,
                  const float* partial_lse,
                  const int32_t* splits_per_row, void* out, float* lse_out,
                  int32_t num_splits, int32_t total_q, int32_t num_heads,
                  int64_t out_stride_tok, int64_t out_stride_head,
                  float out_scale, msa_stream_t stream);

/* The same merge with two more degrees of freedom, for partials that do not sit in the dense
 * [S, total_q, H, ...] arrangement and for callers that want the result unrounded:
 *  - o_split_stride / lse_split_stride: elements between split s and split s + 1 of partial_o /
 *    partial_lse (<= 0: the dense default total_q*H*128 / total_q*H).  Lets one buffer hold
 *    several ranks' packed (O, LSE) blocks as an all-gather delivers them;
 *  - out_dtype: MSA_DT_BF16 or MSA_DT_F32 (the fp32 result of a local merge is what a rank
 *    contributes to a cross-GPU merge).
 * No upstream counterpart beyond `reduction` itself (upstream is single-device). */
int msa_lse_merge_ex(const void* partial_o, int32_t partial_dtype, const float* partial_lse,
                     const int32_t* splits_per_row, void* out, int32_t out_dtype, float* lse_out,
                     int32_t num_splits, int32_t total_q, int32_t num_heads,
                     int64_t o_split_stride, int64_t lse_split_stride,
                     int64_t out_stride_tok, int64_t out_stride_head,
                     float out_scale, msa_stream_t stream);

/* Page top-k: per (head, token) row of scores[H, K, T] pick the `topk` best
 * pages of [0, num_valid_pages) by (score desc, index asc), emit them
 * ascending into out[T, H, topk] (int32), pad with -1.  Pages [0, force_begin)
 * and [nvp - force_end, nvp) rank as FLT_MAX.  topk in {4, 8, 16, 32}.
 * Replaces `sparse_topk_select` (csrc/sparse_topk_select.cu:19-88,
 * csrc/include/sparse_topk_select.cuh:1410-1459).  Needs no workspace. */
int msa_topk_select(const void* scores, int32_t score_dtype, int32_t* out,
                    int32_t num_heads, int32_t max_k_tiles, int32_t total_q,
                    int32_t topk, int32_t num_valid_pages,
                    int32_t force_begin, int32_t force_end, msa_stream_t stream);

/* Host-side planner for the dense path: enumerates (batch, head group, row
 * tile) items, cuts long KV ranges into splits, orders items longest first.
 * Host arrays in, host arrays out (the caller uploads `work`).  Replaces
 * `prepare_plan_metadata` + `plan` (csrc/prepare_plan_metadata.cu:19-37,
 * csrc/fmha_sm80_plan.cu:20-37; behaviour spec: tests/integration/
 * test_plan_correctness.py:58-190 -- every tile exactly once, split ranges
 * contiguous from 0).  Returns the number of items written, or a negative
 * error (MSA_ERR_TOO_LARGE if `capacity` is too small). */
typedef struct MsaPlanArgs {
  const int32_t* qo_len;      /* [B] host */
  const int32_t* kv_len;      /* [B] host */
  const int32_t* qo_offset;   /* [B] host */
  int32_t batch;
  int32_t num_qo_heads, num_kv_heads;
  int32_t block_m;            /* 16 / 64 / 128 / 256 */
  int32_t pack;               /* 1 or Hq/Hkv   */
  int32_t num_splits;         /* >=1 fixed; <=0 adaptive with -num_splits as the ceiling */
  int32_t num_sms;            /* device SM count (adaptive mode target)  */
  int32_t reserved;
} MsaPlanArgs;
int msa_plan_dense(const MsaPlanArgs* args, MsaWorkItem* work, int32_t capacity,
                   int32_t* splits_per_row /* [total_q] host */,
                   int32_t* max_splits_out);

/* Planning on the device, for callers that capture plan + run into one CUDA graph and only
 * update the length tensors between replays (upstream: `graph_safe=True`, the
 * prepare_plan_metadata + plan kernels, api.py:916-941, 1040-1048, 1196-1203).
 * Everything that sizes a launch is fixed when the graph is built: batch, the number of
 * row tiles per batch item (`row_tiles` >= ceil(max qo_len * pack / block_m)), the split count.
 * One kernel launch on `stream`; reads no device memory on the host, allocates nothing.
 * Fills, for i in [0, batch):  qo_start / kv_start (exclusive prefix sums, [batch + 1]),
 * kv_len_out, qo_offset_out (causal: kv_len - qo_len where qo_offset_in is NULL or
 * negative; non-causal: `noncausal_offset`), kv_page_indptr ([batch + 1], pages of
 * `page_size` keys, NULL for ragged K/V), token_batch ([max_total_q], NULL when unused),
 * splits_per_row ([max_total_q]: num_splits for real tokens, 0 for the padding past the last
 * one, so that a merge over max_total_q rows writes zeros there) and the work list: exactly
 * batch * row_tiles * (num_qo_heads / pack) * num_splits items, item
 * (((b * row_tiles + r) * groups) + g) * S + s = row tile (row_tiles - 1 - r) of batch item b
 * (later rows first: under a causal mask they see more keys), head group g, the s-th of S
 * equal chunks of the key tiles those rows can see.  A row tile past the item's rows, or a
 * chunk past its tiles, is an item with num_rows = 0 / an empty tile range.  NULL outputs
 * are skipped. */
typedef struct MsaPlanDeviceArgs {
  const int32_t* qo_len;       /* [B] device */
  const int32_t* kv_len;       /* [B] device */
  const int32_t* qo_offset_in; /* [B] device or NULL */
  int32_t* qo_start;
  int32_t* kv_start;
  int32_t* kv_len_out;
  int32_t* qo_offset_out;
  int32_t* kv_page_indptr;
  int32_t* token_batch;
  int32_t* splits_per_row;
  MsaWorkItem* work;
  int32_t batch;
  int32_t num_qo_heads, num_kv_heads;
  int32_t block_m, pack, num_splits;
  int32_t page_size;           /* <= 0: ragged */
  int32_t causal;
  int32_t noncausal_offset;
  int32_t max_total_q;
  int32_t row_tiles;           /* >= 1 */
} MsaPlanDeviceArgs;
int msa_plan_device(const MsaPlanDeviceArgs* args, msa_stream_t stream);

/* Split-KV forward + merge with the partial-result scratch held inside the library.
 * No counterpart in the upstream project (there the caller always owns the split
 * workspace, api.py:141-167).  It exists for embedders that may not allocate device
 * memory at call time -- an engine whose memory pool owns the whole device after
 * start-up, a sandboxed plugin host that passes tensors but no allocator.  Same
 * arguments and the same argument checks as msa_fmha_fwd (dense or sparse, MSA_FLAG_OUT_O
 * only, block_m 16/64/128) with partial_o / partial_lse left NULL and num_splits = the S of
 * the work list; the result goes to params->out (and params->lse).  `splits_per_row`
 * ([total_q] device int32, or NULL) has the meaning it has in msa_lse_merge: how many of
 * the S slots of a token the merge looks at; NULL = all S.  Either way a slot that no work
 * item of this call wrote counts as empty: the call first marks every slot as empty (LSE
 * -inf), so a short or empty work list gives zeros / -inf LSE, never a value left behind by
 * an earlier call.  The call performs no cudaMalloc / cudaFree and calls no allocating
 * routine.
 *  - Limit: num_splits * total_q * num_qo_heads <= MSA_STATIC_SCRATCH_MAX_ROWS,
 *    otherwise MSA_ERR_TOO_LARGE.  The array (about 8.5 MB) is resident on every GPU
 *    that loads the library, until the process exits.
 *  - The first call on a device resolves the array's device address; make that first
 *    call before any stream capture on that device.
 *  - All calls on a device share the one array: two calls whose kernels overlap on the
 *    GPU (different streams) race on it.  Serialise them on one stream. */
#define MSA_STATIC_SCRATCH_MAX_ROWS 16384
int msa_fmha_fwd_split_static(const MsaFmhaParams* params, const int32_t* splits_per_row,
                              msa_stream_t stream);

/* Human-readable text of an MSA_ERR_* code. */
const char* msa_status_string(int code);

/* Library build info: returns the SM architecture the kernels were built for (100). */
int msa_build_arch(void);

/* sizeof() of the ABI structs as the library was compiled: 0 = MsaFmhaParams,
 * 1 = MsaWorkItem, 2 = MsaPlanArgs, 3 = MsaPlanDeviceArgs.  Lets a foreign-language binding verify its
 * own struct declaration at load time. */
int msa_sizeof(int which);

#ifdef __cplusplus
}
#endif
#endif /* MSA_B200_H_ */
