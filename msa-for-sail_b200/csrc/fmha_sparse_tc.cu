// Sparse (selected-pages) attention for long query batches on tcgen05, iterating KV-outer.
//
// Upstream walks sparse attention token by token: every token becomes its own batch item with
// Hq/Hkv rows and re-reads its pages (csrc/include/prepare_plan_metadata.cuh:90-112,
// csrc/include/sm80_fmha_sparse_fwd_mainloop.hpp:249-601).  With tens of thousands of query
// tokens that is an 8-row MMA and hundreds of GB of page re-reads.  Here the loop is turned
// inside out (the MSA paper's KV-outer schedule): a reverse index page -> (token, slot) is built
// from kv_block_indexes on the device, and one CTA keeps ONE page of K and V resident in shared
// memory while it streams chunks of 128/G query tokens (G = Hq/Hkv rows each) that selected it:
//
//   S = Q_chunk K_page^T  (tcgen05, TMEM)  ->  mask on original positions, softmax of the one
//   tile  ->  O = P V_page  ->  normalised partial O (bf16) + LSE, stored in the order of the
//   sorted selection list (a chunk's 128 rows are one contiguous 32 KB block: two TMA stores)
//
// and a merge kernel combines the `kv_block_num` partials of every row through the inverse map
// (token, kv head, slot) -> position in the sorted list.  Every (token, page) pair is computed
// exactly once regardless of how the selections overlap.
//
// Kernels in this file: count / scan / scatter (counting sort of the selections by page), the merge and the
// attention kernel.  Roles of the attention kernel (20 warps): warps 0-3 / 4-7 softmax of even / odd
// chunks (152 registers each: a whole row of S is held at once); warps 8-11 / 12-15 epilogue of
// head_dim [0, 64) / [64, 128) (O out of TMEM, bf16, shared memory, one TMA tensor store per chunk
// and half, overlapping the softmax of later chunks); warps 16-18 loaders (the page by TMA, once;
// the Q rows of a chunk gathered with one TMA box per 8 rows, the boxes spread over the lanes of
// three warps because a warp issues its lanes' boxes one after another); warp 19 MMA issuer.
// All waits are bounded (see tc_ptx.cuh).
#include "tc_ptx.cuh"

namespace msa {
int make_tma_map_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box);

namespace sparse_tc {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 128;
constexpr int SUB_BYTES = BM * 64 * 2;
constexpr int TILE_BYTES = 2 * SUB_BYTES;
constexpr int OFF_Q = 0;                        // two Q chunk buffers
constexpr int OFF_K = 2 * TILE_BYTES;
constexpr int OFF_V = 3 * TILE_BYTES;
constexpr int OFF_STAGE = 4 * TILE_BYTES;       // two buffers of 128 rows x 256 B of bf16 O on their way out
// what the softmax warpgroups hand to the epilogue warpgroup, per row, for the 4 chunks in flight
struct RowMeta { float inv; float lse; };
constexpr int OFF_META = OFF_STAGE + 2 * TILE_BYTES;    // [4][128] RowMeta
constexpr int OFF_BAR = OFF_META + 4 * BM * 8;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int NTHREADS = 640;
constexpr int EPI_WARP0 = 8, GATHER_WARP0 = 16, GATHER_WARPS = 3, MMA_WARP = 19;
constexpr int GATHER_THREADS = GATHER_WARPS * 32;
constexpr int ITEM_CHUNKS = 32;                 // chunks of 128 rows per work item
constexpr uint32_t kEmuMask = 0x5252;

// TMEM: three S buffers (chunk c uses c % 3; P_c overwrites the front of S_c) and one O, drained by
// two warpgroups (64 columns each).  With only two S buffers Q_{c+2} K^T would have to wait for P_c V, which puts the softmax of a
// warpgroup, that MMA and the next Q K^T on one serial chain.
constexpr int NSBUF = 3;
constexpr uint32_t O_COL = NSBUF * BN;
// META_FULL has one barrier per chunk in flight (c & 3): the softmax warpgroups run ahead of the
// epilogue, and a barrier that completed twice since the waiter last looked reads as "not yet".
enum Bar { K_FULL = 0, V_FULL = 1, V_FIX = 2, Q_FULL = 3, Q_EMPTY = 5, S_FULL = 7, P_FULL = 10, O_FULL = 13,
           O_FREE = 14, META_FULL = 15, NUM_BARS = 19 };

// test hook: take the global-atomics index kernels even when the histogram fits shared memory
bool g_force_global_index = false;

// optional clock trace of one CTA (debugging aid): [6 roles][512 chunks][8 tags]; roles: softmax 0/1,
// MMA 2, loaders 3, epilogue 4
__device__ unsigned long long g_trace[6 * 512 * 8];
__device__ int g_trace_cta = -1;

struct Ws {                 // device workspace carved by carve()
  int32_t* bin_count;       // [NB + 1]
  int32_t* bin_offset;      // [NB + 1]  start of a bin in `entries`, a multiple of the tokens per chunk
  int32_t* bin_cursor;      // [NB]
  int32_t* part_start;      // [Hkv + 1]  first work item of every kv head, then the item count
  int4* items;              // [max_items] {bin, entry_begin, entry_end, 0}
  int32_t* entries;         // [cap]  token << 5 | slot, sorted by (kv head, page); gaps between bins are padding
  int32_t* inv;             // [T, Hkv, kbn]  position of a selection in `entries`, -1 if it selects nothing
  float* partial_lse;       // [cap * G]   row = position * G + head in group
  __nv_bfloat16* partial_o; // [cap * G, 128]
  int64_t cap;              // entries incl. padding
  int64_t max_items;
  int64_t total_bytes;
};

inline int64_t align256(int64_t x) { return (x + 255) & ~int64_t(255); }

Ws carve(void* base, int64_t T, int Hq, int Hkv, int kbn, int64_t NP) {
  Ws w;
  const int64_t NB = static_cast<int64_t>(Hkv) * NP;
  const int G = Hq / Hkv;
  const int64_t tpc = BM / G;
  w.cap = T * Hkv * kbn + NB * tpc;
  w.max_items = (T * Hkv * kbn) / (tpc * ITEM_CHUNKS) + NB + 1;
  char* p = static_cast<char*>(base);
  int64_t off = 0;
  auto take = [&](int64_t bytes) { char* r = p ? p + off : nullptr; off = align256(off + bytes); return r; };
  w.bin_count = reinterpret_cast<int32_t*>(take((NB + 1) * 4));
  w.part_start = reinterpret_cast<int32_t*>(take((Hkv + 1) * 4));
  // everything above is zeroed before each run
  w.bin_offset = reinterpret_cast<int32_t*>(take((NB + 1) * 4));
  w.bin_cursor = reinterpret_cast<int32_t*>(take(NB * 4));
  w.items = reinterpret_cast<int4*>(take(w.max_items * 16));
  w.entries = reinterpret_cast<int32_t*>(take(w.cap * 4));
  w.inv = reinterpret_cast<int32_t*>(take(T * Hkv * kbn * 4));
  w.partial_lse = reinterpret_cast<float*>(take(w.cap * G * 4));
  w.partial_o = reinterpret_cast<__nv_bfloat16*>(take(w.cap * G * kHeadDim * 2));
  w.total_bytes = off;
  return w;
}

// ------------------------------------------------------------------------------------------
// reverse index: counting sort of the valid (token, kv head, slot) selections by (kv head, page)
// ------------------------------------------------------------------------------------------
struct IndexArgs {
  const int32_t* kbi; int64_t kbi_stride_tok, kbi_stride_head;
  const int32_t* token_batch; const int32_t* qo_start; const int32_t* kv_len; const int32_t* qo_offset;
  const int32_t* kv_page_indptr;
  int32_t total_q, num_kv_heads, num_qo_heads, kbn, num_pages;
};

__device__ __forceinline__ bool entry_valid(const IndexArgs& a, int t, int b, int blk) {
  if (blk < 0) return false;
  const int pos0 = blk * BN;
  if (pos0 >= a.kv_len[b]) return false;
  const int i = t - a.qo_start[b];
  return pos0 <= i + a.qo_offset[b];            // at least the page's first key is visible
}

template <bool SCATTER>
__global__ void __launch_bounds__(256)
sparse_index_kernel(const IndexArgs a, int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_cursor,
                    int32_t* __restrict__ entries, int32_t* __restrict__ inv) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // kvh-major, token fastest
  const int64_t n = static_cast<int64_t>(a.total_q) * a.num_kv_heads;
  if (gid >= n) return;
  const int kvh = static_cast<int>(gid / a.total_q), t = static_cast<int>(gid % a.total_q);
  const int b = a.token_batch[t];
  const int page_base = a.kv_page_indptr[b];
  const int32_t* row = a.kbi + static_cast<int64_t>(t) * a.kbi_stride_tok + static_cast<int64_t>(kvh) * a.kbi_stride_head;
  int32_t* inv_row = inv + (static_cast<int64_t>(t) * a.num_kv_heads + kvh) * a.kbn;
  for (int s = 0; s < a.kbn; ++s) {
    const int blk = row[s];
    if (entry_valid(a, t, b, blk)) {
      const int bin = kvh * a.num_pages + page_base + blk;
      if (SCATTER) {
        const int pos = atomicAdd(&bin_cursor[bin], 1);
        entries[pos] = (t << 5) | s;
        inv_row[s] = pos;
      } else {
        atomicAdd(&bin_count[bin], 1);
      }
    } else if (SCATTER) {
      inv_row[s] = -1;                                       // this slot contributes nothing to the merge
    }
  }
}

// The same two passes with a shared-memory histogram: a CTA owns 256 consecutive tokens of one kv
// head, counts (or ranks) its selections per page in shared memory and touches global memory once
// per (CTA, page) -- the global atomics drop from one per selection to one per distinct page of a
// CTA.  Needs num_pages * 4 bytes of shared memory; larger page counts use the kernel above.
template <bool SCATTER, int KBN>
__global__ void __launch_bounds__(256)
sparse_index_smem_kernel(const IndexArgs a, int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_cursor,
                         int32_t* __restrict__ entries, int32_t* __restrict__ inv) {
  extern __shared__ int32_t s_hist[];                      // [num_pages] count, then (scatter) next position
  const int blocks_per_head = (a.total_q + 255) / 256;
  const int kvh = blockIdx.x / blocks_per_head;
  const int t = (blockIdx.x % blocks_per_head) * 256 + threadIdx.x;
  for (int i = threadIdx.x; i < a.num_pages; i += 256) s_hist[i] = 0;
  __syncthreads();
  int gpage[KBN];                                           // global page of each valid selection, -1 otherwise
#pragma unroll
  for (int s = 0; s < KBN; ++s) gpage[s] = -1;
  if (t < a.total_q) {
    const int b = a.token_batch[t];
    const int page_base = a.kv_page_indptr[b];
    const int32_t* row = a.kbi + static_cast<int64_t>(t) * a.kbi_stride_tok + static_cast<int64_t>(kvh) * a.kbi_stride_head;
#pragma unroll
    for (int s = 0; s < KBN; ++s) {
      if (s < a.kbn) {
        const int blk = row[s];
        if (entry_valid(a, t, b, blk)) { gpage[s] = page_base + blk; atomicAdd(&s_hist[gpage[s]], 1); }
      }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < a.num_pages; i += 256) {
    const int c = s_hist[i];
    if (c > 0) {
      if (SCATTER) s_hist[i] = atomicAdd(&bin_cursor[kvh * a.num_pages + i], c);   // reserve c consecutive positions
      else atomicAdd(&bin_count[kvh * a.num_pages + i], c);
    }
  }
  if (!SCATTER) return;
  __syncthreads();
  if (t < a.total_q) {
    int32_t* inv_row = inv + (static_cast<int64_t>(t) * a.num_kv_heads + kvh) * a.kbn;
#pragma unroll
    for (int s = 0; s < KBN; ++s) {
      if (s < a.kbn) {
        int pos = -1;
        if (gpage[s] >= 0) {
          pos = atomicAdd(&s_hist[gpage[s]], 1);
          entries[pos] = (t << 5) | s;
        }
        inv_row[s] = pos;
      }
    }
  }
}

// exclusive scan of the bin counts + work items (one CTA; NB is a few thousand to ~1e5)
__global__ void __launch_bounds__(1024)
sparse_scan_kernel(const int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_offset,
                   int32_t* __restrict__ bin_cursor, int4* __restrict__ items, int32_t* __restrict__ part_start,
                   int num_bins, int rows_per_item, int max_items, int tpc, int bins_per_head) {
  __shared__ int s_ent[1024], s_itm[1024];
  __shared__ int carry_ent, carry_itm;
  if (threadIdx.x == 0) { carry_ent = 0; carry_itm = 0; }
  __syncthreads();
  for (int base = 0; base < num_bins; base += 1024) {
    const int bin = base + threadIdx.x;
    const int cnt = bin < num_bins ? bin_count[bin] : 0;
    const int cnt_pad = (cnt + tpc - 1) / tpc * tpc;        // a bin starts on a chunk boundary
    const int nit = (cnt + rows_per_item - 1) / rows_per_item;
    s_ent[threadIdx.x] = cnt_pad; s_itm[threadIdx.x] = nit;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {                   // Hillis-Steele inclusive scan
      const int e = threadIdx.x >= d ? s_ent[threadIdx.x - d] : 0;
      const int i2 = threadIdx.x >= d ? s_itm[threadIdx.x - d] : 0;
      __syncthreads();
      s_ent[threadIdx.x] += e; s_itm[threadIdx.x] += i2;
      __syncthreads();
    }
    const int ent0 = carry_ent + s_ent[threadIdx.x] - cnt_pad;
    const int itm0 = carry_itm + s_itm[threadIdx.x] - nit;
    if (bin < num_bins) {
      if (bin % bins_per_head == 0) part_start[bin / bins_per_head] = min(itm0, max_items);
      bin_offset[bin] = ent0;
      bin_cursor[bin] = ent0;
      for (int k = 0; k < nit; ++k)
        if (itm0 + k < max_items)
          items[itm0 + k] = make_int4(bin, ent0 + k * rows_per_item, min(ent0 + cnt, ent0 + (k + 1) * rows_per_item), 0);
    }
    __syncthreads();
    if (threadIdx.x == 1023) { carry_ent += s_ent[1023]; carry_itm += s_itm[1023]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { bin_offset[num_bins] = carry_ent; part_start[num_bins / bins_per_head] = min(carry_itm, max_items); }
}

// ------------------------------------------------------------------------------------------
// merge: out[t, h] = sum_s w_s O_s / sum_s w_s over the selections of (t, kv head), w_s = exp(lse_s - max)
// Half a warp per (token, head) row, lane l of the half owns columns 8l..8l+7; the partial rows are
// found through `inv`.  All loads of a row are issued before any is used.
// ------------------------------------------------------------------------------------------
template <int KBN>
__global__ void __launch_bounds__(256)
sparse_merge_kernel(const __nv_bfloat16* __restrict__ po, const float* __restrict__ pl, const int32_t* __restrict__ inv,
                    __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, int kbn, int total_q, int num_heads,
                    int num_kv_heads, int64_t out_stride_tok, int64_t out_stride_head, float out_scale, int kvh0, int nkvh) {
  const int l16 = threadIdx.x & 15;
  // rows are walked kv-head-major: the partials of one kv head are one contiguous eighth (1 / Hkv) of
  // the buffer, which keeps the randomly gathered 2 KB reads of a pass within reach of the TLB.
  // This launch covers kv heads [kvh0, kvh0 + nkvh); a small grid strides over them (used while the
  // attention kernel of the next kv head runs on the other SMs).
  const int G = num_heads / num_kv_heads;
  const int64_t n_idx = static_cast<int64_t>(total_q) * G * nkvh;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4); idx < n_idx;
       idx += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 4)) {
  const int g = static_cast<int>(idx % G);
  const int64_t tg = idx / G;
  const int kvh = kvh0 + static_cast<int>(tg / total_q), t = static_cast<int>(tg % total_q);
  const int h = kvh * G + g;
  const int64_t row = static_cast<int64_t>(t) * num_heads + h;
  const int32_t* iv = inv + (static_cast<int64_t>(t) * num_kv_heads + kvh) * kbn;
  float lse[KBN];
  uint4 raw[KBN];
  float mx = -INFINITY;
#pragma unroll
  for (int s = 0; s < KBN; ++s) {
    const int pos = s < kbn ? iv[s] : -1;
    const int64_t prow = static_cast<int64_t>(max(pos, 0)) * G + g;             // clamped: always a readable row
    raw[s] = *reinterpret_cast<const uint4*>(po + prow * kHeadDim + l16 * 8);
    const float l = __ldg(pl + prow);
    lse[s] = pos >= 0 ? l : -INFINITY;
    mx = fmaxf(mx, lse[s]);
  }
  const float mxs = (mx == -INFINITY) ? 0.f : mx;
  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  float sw = 0.f;
#pragma unroll
  for (int s = 0; s < KBN; ++s) {
    const float w = lse[s] != -INFINITY ? __expf(lse[s] - mxs) : 0.f;
    if (w != 0.f) {                                          // value select after an unconditional load
      sw += w;
      const uint32_t* r4 = reinterpret_cast<const uint32_t*>(&raw[s]);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        acc[2 * c] = fmaf(w, bf16_bits_to_float(r4[c] & 0xffff), acc[2 * c]);
        acc[2 * c + 1] = fmaf(w, bf16_bits_to_float(r4[c] >> 16), acc[2 * c + 1]);
      }
    }
  }
  const float sc = sw > 0.f ? out_scale / sw : 0.f;
  __nv_bfloat16* dst = out + static_cast<int64_t>(t) * out_stride_tok + static_cast<int64_t>(h) * out_stride_head + l16 * 8;
  uint4 pk;
  pk.x = pack2<false>(acc[0] * sc, acc[1] * sc);
  pk.y = pack2<false>(acc[2] * sc, acc[3] * sc);
  pk.z = pack2<false>(acc[4] * sc, acc[5] * sc);
  pk.w = pack2<false>(acc[6] * sc, acc[7] * sc);
  *reinterpret_cast<uint4*>(dst) = pk;
  if (lse_out && l16 == 0) lse_out[row] = sw > 0.f ? mxs + __logf(sw) : -INFINITY;
  }
}

// ------------------------------------------------------------------------------------------
// attention kernel
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS, 1)
sparse_tc_kernel(const __grid_constant__ MsaFmhaParams p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const __grid_constant__ CUtensorMap tm_o, const int4* __restrict__ items, const int32_t* __restrict__ part_start,
                 const int part,
                 const int32_t* __restrict__ entries, float* __restrict__ partial_lse) {
  // this launch covers the work items of kv head `part`, or all of them (part < 0)
  const int item_idx = (part >= 0 ? part_start[part] : 0) + static_cast<int>(blockIdx.x);
  if (item_idx >= part_start[part >= 0 ? part + 1 : p.num_kv_heads]) return;   // uniform: before any barrier / TMEM use
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + OFF_BAR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 8);
  volatile int* skip_flag = abort_flag + 1;      // set when the status word already reports a timeout
  auto bar = [&](int i) -> uint32_t { return bars + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool tracing = static_cast<int>(blockIdx.x) == g_trace_cta;
  auto trace = [&](int role, int c, int tag) {
    if (tracing && c < 512) g_trace[(role * 512 + c) * 8 + tag] = clock64();
  };

  // ---------------- work item ----------------
  const int4 item = items[item_idx];
  const int NP = p.num_logical_pages;
  const int kvh = item.x / NP, gp = item.x % NP;
  const int b = p.page_batch[gp];
  const int lpage = gp - p.kv_page_indptr[b];
  const int phys = p.kv_indices[gp];
  const int G = p.num_qo_heads / p.num_kv_heads;
  const int tpc = BM / G;                                  // tokens per chunk
  const int n_ent = item.z - item.y;
  const int n_chunks = (n_ent + tpc - 1) / tpc;
  const int qo_base = p.qo_start[b];
  const int kv_len = p.kv_len[b];
  const int off = p.qo_offset[b];
  const int pos0 = lpage * BN;
  const int valid_rows = min(BN, kv_len - pos0);

  // a timeout reported earlier on this device (status word not cleared yet): do not start.  Read by
  // another thread than the one that sets up the barriers, so the load overlaps that work.
  if (threadIdx.x == blockDim.x - 1)
    *skip_flag = (p.status != nullptr && *reinterpret_cast<const volatile int32_t*>(p.status) != 0) ? 1 : 0;
  if (threadIdx.x == 0) {
    mbar_init(bar(K_FULL), 1); mbar_init(bar(V_FULL), 1); mbar_init(bar(V_FIX), 1);
    for (int s = 0; s < 2; ++s) { mbar_init(bar(Q_FULL + s), 1);  mbar_init(bar(Q_EMPTY + s), 1); }
    for (int s = 0; s < NSBUF; ++s) { mbar_init(bar(S_FULL + s), 1);  mbar_init(bar(P_FULL + s), BM); }
    for (int s = 0; s < 4; ++s) mbar_init(bar(META_FULL + s), BM);
    mbar_init(bar(O_FULL), 1);  mbar_init(bar(O_FREE), 2 * BM);       // both epilogue warpgroups drain O
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  const bool run = *skip_flag == 0;
  if (!run) {
    // nothing: fall through to the teardown
  } else if (warp >= GATHER_WARP0 && warp < GATHER_WARP0 + GATHER_WARPS) {
    // =========================== loaders: page and Q chunks by TMA ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    const int gt = threadIdx.x - GATHER_WARP0 * 32;
    bool alive = true;
    if (warp == GATHER_WARP0) {
      if (lane == 0) { tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
      const bool fix = valid_rows < BN;
      if (elect_one()) {
        mbar_arrive_expect_tx(bar(K_FULL), TILE_BYTES);
        const uint32_t vbar = fix ? bar(V_FIX) : bar(V_FULL);
        mbar_arrive_expect_tx(vbar, TILE_BYTES);
#pragma unroll
        for (int hlf = 0; hlf < 2; ++hlf) {
          tma_load_4d(smem_base + OFF_K + hlf * SUB_BYTES, &tm_k, bar(K_FULL), hlf * 64, 0, kvh, phys);
          tma_load_4d(smem_base + OFF_V + hlf * SUB_BYTES, &tm_v, vbar, hlf * 64, 0, kvh, phys);
        }
      }
      __syncwarp();
      if (fix) {
        alive = mbar_wait(bar(V_FIX), 0, abort_flag);
        alive = __all_sync(0xffffffffu, alive);
        if (alive) {
          unsigned char* vt = smem_gen + OFF_V;
          for (int c = lane; c < (BN - valid_rows) * 16; c += 32) {
            const int r = valid_rows + (c >> 4), ch = c & 15;
            *reinterpret_cast<uint4*>(vt + (ch >> 3) * SUB_BYTES + r * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(V_FULL));
        }
      }
    }
    // Q gather: one TMA box per 8 consecutive rows (the 8 heads of a token, or of half a token when
    // G = 16, ...) holding BOTH 64-element halves of head_dim: box {64, 8, 2, 1} of the 4-D view
    // [token][half][head][64].  It lands as two 1 KB swizzle atoms, half 0 then half 1, so unit n of
    // a chunk sits at n * 2 KB and the MMA descriptor steps 2 KB between 8-row groups.  That is
    // 16 boxes per chunk, issued by 16 different lanes spread over the three loader warps (a
    // warp issues the boxes of its lanes one after another).  G < 8: one {64, G, 1} box per token and
    // half in the plain layout.
    const bool unit8 = (G & 7) == 0;
    const int unit = (warp - GATHER_WARP0) + GATHER_WARPS * lane;      // unit n -> warp n % 3, lane n / 3
    const int upt = unit8 ? G / 8 : 1;                      // units per token
    auto entry_of = [&](int c) -> int {                      // entry of the token this lane loads in chunk c (unit8)
      const int e = item.y + c * tpc + unit / upt;
      return (c < n_chunks && unit8 && unit < BM / 8 && e < item.z) ? entries[e] : -1;
    };
    int ent = entry_of(0);
    for (int c = 0; c < n_chunks && alive; ++c) {
      const int x = c & 1, u = c >> 1;
      if (gt == 0) trace(3, c, 0);
      alive = mbar_wait(bar(Q_EMPTY + x), (u & 1) ^ 1, abort_flag);   // Q K^T of chunk c - 2 has read the buffer
      if (!alive) break;
      const int e0 = item.y + c * tpc;
      const int ntok = min(tpc, item.z - e0);
      if (gt == 0) {
        trace(3, c, 1);
        mbar_arrive_expect_tx(bar(Q_FULL + x), ntok * G * 256);
      }
      if (unit8) {
        if (ent >= 0)
          tma_load_4d(smem_base + OFF_Q + x * TILE_BYTES + unit * 2048, &tm_q, bar(Q_FULL + x), 0, kvh * G + (unit % upt) * 8, 0,
                      ent >> 5);
        ent = entry_of(c + 1);
      } else {
        for (int ti = unit; ti < ntok; ti += GATHER_THREADS) {
          const int tok = entries[e0 + ti] >> 5;
          const uint32_t dst = smem_base + OFF_Q + x * TILE_BYTES + ti * G * 128;
          tma_load_3d(dst, &tm_q, bar(Q_FULL + x), 0, kvh * G, tok);
          tma_load_3d(dst + SUB_BYTES, &tm_q, bar(Q_FULL + x), 64, kvh * G, tok);
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    constexpr uint32_t IDESC_QK = idesc_bf16(BM, BN, false, false);
    constexpr uint32_t IDESC_PV = idesc_bf16(BM, kHeadDim, false, true);
    const uint64_t dk_hi = smem_desc(0, 16, 1024) & 0xFFFFFFFFFFFF0000ull;
    const uint64_t dv_hi = smem_desc(0, SUB_BYTES, 1024) & 0xFFFFFFFFFFFF0000ull;
    // Q: 8-row groups 2 KB apart with the second head_dim half 1 KB after the first (G % 8 == 0),
    // else the plain two-sub-tile layout
    const bool unit8 = (G & 7) == 0;
    const uint64_t dq_hi = unit8 ? (smem_desc(0, 16, 2048) & 0xFFFFFFFFFFFF0000ull) : dk_hi;
    const uint32_t q_half = unit8 ? 1024u : static_cast<uint32_t>(SUB_BYTES);
    auto issue_qk = [&](int x, int sb) {
      const uint32_t qa = (smem_base + OFF_Q + x * TILE_BYTES) >> 4, ka = (smem_base + OFF_K) >> 4;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t o = ((k >> 2) * SUB_BYTES + (k & 3) * 32) >> 4;
        const uint32_t oq = ((k >> 2) * q_half + (k & 3) * 32) >> 4;
        mma_ss(tmem + sb * BN, dq_hi | ((qa + oq) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
      }
    };
    auto issue_pv = [&](int sb) {
      const uint32_t va = (smem_base + OFF_V) >> 4;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_ts(tmem + O_COL, tmem + sb * BN + k * 8, dv_hi | ((va + k * (2048 >> 4)) & 0x3FFF), IDESC_PV, k > 0 ? 1u : 0u);
    };
    bool alive = mbar_wait(bar(K_FULL), 0, abort_flag);
    // S[c % 3] = Q_c K^T.  Issued three chunks ahead of the P V stream: S_{c+3} reuses the buffer
    // of chunk c, so it may follow P_c V directly and is ready long before its warpgroup asks.
    auto do_qk = [&](int c) {
      const int x = c & 1, u = c >> 1;
      if (lane == 0) trace(2, c, 0);
      alive = mbar_wait(bar(Q_FULL + x), u & 1, abort_flag);
      if (lane == 0) trace(2, c, 2);
      if (!alive) return;
      tc_fence_after();
      if (elect_one()) {
        issue_qk(x, c % NSBUF);
        mma_commit(bar(S_FULL + c % NSBUF));
        mma_commit(bar(Q_EMPTY + x));
      }
      __syncwarp();
    };
    for (int c = 0; c < NSBUF && c < n_chunks && alive; ++c) do_qk(c);
    for (int d = 0; d < n_chunks && alive; ++d) {           // O = P_d V, once the epilogue has drained O of chunk d - 1
      if (d == 0) alive = mbar_wait(bar(V_FULL), 0, abort_flag);
      if (lane == 0) trace(2, d, 3);
      if (alive) alive = mbar_wait(bar(P_FULL + d % NSBUF), (d / NSBUF) & 1, abort_flag);
      if (lane == 0) trace(2, d, 4);
      if (alive && d > 0) alive = mbar_wait(bar(O_FREE), (d - 1) & 1, abort_flag);
      if (!alive) break;
      tc_fence_after();
      if (elect_one()) {
        issue_pv(d % NSBUF);
        mma_commit(bar(O_FULL));
      }
      __syncwarp();
      if (lane == 0) trace(2, d, 5);
      if (d + NSBUF < n_chunks) do_qk(d + NSBUF);
    }
  } else if (warp >= EPI_WARP0) {
    // =========================== epilogue: one 64-column half of O of every chunk -> bf16 partial rows ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 64;");
    const int w4 = warp & 3;
    const int hlf = (warp - EPI_WARP0) >> 2;
    const int r = (w4 << 5) | lane;
    const uint32_t lane_addr = static_cast<uint32_t>(w4 << 5) << 16;
    const uint32_t tO = tmem + O_COL + hlf * 64 + lane_addr;
    const bool issuer = (threadIdx.x & 127) == 0;             // first thread of this half's warpgroup
    if (issuer) tma_prefetch_desc(&tm_o);
    bool alive = true;
    for (int c = 0; c < n_chunks; ++c) {
      const RowMeta* meta = reinterpret_cast<const RowMeta*>(smem_gen + OFF_META) + (c & 3) * BM;
      // staging: a 128-byte-swizzled [128 rows][128 B] tile per half, the layout a TMA tensor store
      // reads (and conflict-free to write); two buffers, chunk parity
      unsigned char* my_stage = smem_gen + OFF_STAGE + (c & 1) * TILE_BYTES + hlf * SUB_BYTES + r * 128;
      if (r == 0) trace(4 + hlf, c, 0);
      bool ok = mbar_wait(bar(META_FULL + (c & 3)), (c >> 2) & 1, abort_flag);
      RowMeta mine = {0.f, 0.f};
      if (ok) mine = meta[r];
      if (ok) ok = mbar_wait(bar(O_FULL), c & 1, abort_flag);
      if (ok) {
        tc_fence_after();
        if (r == 0) trace(4 + hlf, c, 1);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {                     // 32 columns at a time
          uint32_t v[32];
          tmem_ld32(tO + cc * 32, v);
          tmem_wait_ld();
          if (cc == 1) {                                      // this half of the TMEM buffer has been read
            tc_fence_before();
            mbar_arrive(bar(O_FREE));
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {                      // 16-byte pieces
            uint4 o4;
            o4.x = pack2<false>(__uint_as_float(v[q * 8]) * mine.inv, __uint_as_float(v[q * 8 + 1]) * mine.inv);
            o4.y = pack2<false>(__uint_as_float(v[q * 8 + 2]) * mine.inv, __uint_as_float(v[q * 8 + 3]) * mine.inv);
            o4.z = pack2<false>(__uint_as_float(v[q * 8 + 4]) * mine.inv, __uint_as_float(v[q * 8 + 5]) * mine.inv);
            o4.w = pack2<false>(__uint_as_float(v[q * 8 + 6]) * mine.inv, __uint_as_float(v[q * 8 + 7]) * mine.inv);
            *reinterpret_cast<uint4*>(my_stage + (((cc * 4 + q) ^ (r & 7)) << 4)) = o4;
          }
        }
      }
      if (r == 0) trace(4 + hlf, c, 2);
      const int64_t row0 = (static_cast<int64_t>(item.y) + static_cast<int64_t>(c) * tpc) * G;   // a multiple of 128
      if (ok && hlf == 0) partial_lse[row0 + r] = mine.lse;
      fence_proxy_async_smem();                               // generic-proxy writes -> read by the TMA store
      // the store of chunk c - 1 has read its buffer before anybody passes this barrier, so chunk c + 1
      // may overwrite it; the barrier also ANDs `ok`: nobody is left waiting at it after a timeout
      if (issuer) tma_store_wait_read();
      {
        uint32_t out;
        asm volatile("{\n\t.reg .pred pi, po;\n\tsetp.ne.u32 pi, %1, 0;\n\t"
                     "bar.red.and.pred po, %2, 128, pi;\n\tselp.u32 %0, 1, 0, po;\n\t}"
                     : "=r"(out) : "r"(static_cast<uint32_t>(ok)), "r"(1 + hlf) : "memory");
        alive = out != 0;
      }
      if (!alive) break;
      if (issuer) {
        tma_store_2d(&tm_o, smem_base + OFF_STAGE + (c & 1) * TILE_BYTES + hlf * SUB_BYTES, hlf * 64, static_cast<int>(row0));
        tma_store_commit();
      }
      if (r == 0) trace(4 + hlf, c, 3);
    }
    if (issuer) tma_store_wait_all();                         // shared memory stays valid until the stores are done
  } else {
    // =========================== softmax ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
    const int x = warp >> 2;
    const int r = ((warp & 3) << 5) | lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const float scale_log2 = p.sm_scale * kLog2e * (p.k_scale_head ? p.k_scale_head[kvh] : 1.f);
    const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;
    bool alive = true;
    int entry_next = (x < n_chunks && item.y + x * tpc + r / G < item.z) ? entries[item.y + x * tpc + r / G] : 0;
    for (int c = x; c < n_chunks && alive; c += 2) {
      const int e_idx = item.y + c * tpc + r / G;
      const bool row_ok = e_idx < item.z;
      const int entry = entry_next;
      {                                                       // prefetch the entry of this warpgroup's next chunk
        const int e_nx = e_idx + 2 * tpc;
        entry_next = (c + 2 < n_chunks && e_nx < item.z) ? entries[e_nx] : 0;
      }
      const int tok = entry >> 5;
      const int lim = row_ok ? min(tok - qo_base + off, kv_len - 1) : -1;
      if (r == 0) trace(x, c, 0);
      const int sb = c % NSBUF;
      const uint32_t tS = tmem + sb * BN + lane_addr;
      alive = mbar_wait(bar(S_FULL + sb), (c / NSBUF) & 1, abort_flag);
      if (!alive) break;
      tc_fence_after();
      if (r == 0) trace(x, c, 1);
      uint32_t sv[4][32];
      tmem_ld32(tS, sv[0]);
      tmem_ld32(tS + 32, sv[1]);
      tmem_ld32(tS + 64, sv[2]);
      tmem_ld32(tS + 96, sv[3]);
      tmem_wait_ld();
      if (pos0 + BN - 1 > lim) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (pos0 + cc * 32 + e > lim) sv[cc][e] = 0xff800000u;
      }
      float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int cc = 0; cc < 4; ++cc)
#pragma unroll
        for (int e = 0; e < 32; e += 2)
          mxs[(e >> 1) & 3] = max3(mxs[(e >> 1) & 3], __uint_as_float(sv[cc][e]), __uint_as_float(sv[cc][e + 1]));
      const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3])) * scale_log2;
      const float msafe = (mx == -INFINITY) ? 0.f : mx;
      const uint64_t scale2 = f2_pack(scale_log2, scale_log2);
      const uint64_t negm2 = f2_pack(-msafe, -msafe);
      uint64_t lsum2 = f2_pack(0.f, 0.f);
      if (r == 0) trace(x, c, 3);
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(sv[cc][e]), __uint_as_float(sv[cc][e + 1])), scale2, negm2);
          float p0, p1, x0, x1;
          f2_unpack(x2, x0, x1);
          if ((kEmuMask >> ((e >> 1) & 15)) & 1) {
            const uint64_t xc = f2_pack(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
            const uint64_t t2 = f2_add(xc, f2_pack(12582912.f, 12582912.f));
            const uint64_t n2 = f2_add(t2, f2_pack(-12582912.f, -12582912.f));
            const uint64_t fr = f2_fma(n2, f2_pack(-1.f, -1.f), xc);
            uint64_t pl = f2_fma(fr, f2_pack(0.055171650f, 0.055171650f), f2_pack(0.24261113f, 0.24261113f));
            pl = f2_fma(pl, fr, f2_pack(0.69326097f, 0.69326097f));
            pl = f2_fma(pl, fr, f2_pack(0.99992806f, 0.99992806f));
            float q0, q1, t0, t1;
            f2_unpack(pl, q0, q1);
            f2_unpack(t2, t0, t1);
            p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
            p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
          } else {
            p0 = exp2_fast(x0);
            p1 = exp2_fast(x1);
          }
          lsum2 = f2_add(lsum2, f2_pack(p0, p1));
          pk[e >> 1] = pack2<false>(p0, p1);
        }
        tmem_st16(tS + cc * 16, pk);
      }
      float l0, l1;
      f2_unpack(lsum2, l0, l1);
      const float l_sum = l0 + l1;
      if (r == 0) trace(x, c, 4);
      // what the epilogue warpgroup needs for this row (4 buffers: chunk c + 4 cannot get this far
      // before the epilogue of chunk c has read its entry)
      RowMeta* meta = reinterpret_cast<RowMeta*>(smem_gen + OFF_META) + (c & 3) * BM;
      RowMeta mine;
      mine.inv = l_sum > 0.f ? vsh / l_sum : 0.f;
      mine.lse = l_sum > 0.f ? msafe * kLn2 + __logf(l_sum) : -INFINITY;
      meta[r] = mine;
      mbar_arrive(bar(META_FULL + (c & 3)));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + sb));
      if (r == 0) trace(x, c, 2);
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0 && p.status) atomicExch(p.status, MSA_STATUS_TIMEOUT);
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace
}  // namespace sparse_tc

int64_t fmha_sparse_tc_workspace_bytes(int64_t total_q, int num_qo_heads, int num_kv_heads, int kbn, int64_t num_pages) {
  return sparse_tc::carve(nullptr, total_q, num_qo_heads, num_kv_heads, kbn, num_pages).total_bytes;
}

int fmha_sparse_tc_supported(const MsaFmhaParams& p) {
  if (!(p.flags & MSA_FLAG_SPARSE) || !(p.flags & MSA_FLAG_OUT_O) || (p.flags & MSA_FLAG_OUT_SCORE)) return 0;
  if (!p.sparse_ws || !p.page_batch || p.num_logical_pages <= 0) return 0;
  if (p.q_dtype != MSA_DT_BF16 || p.kv_dtype != MSA_DT_BF16 || p.page_size != sparse_tc::BN) return 0;
  const int G = p.num_qo_heads / p.num_kv_heads;
  if (G < 1 || G > 128 || (128 % G) != 0 || p.kv_block_num > 32 || p.total_q >= (1 << 26)) return 0;
  // row indices of the partial buffer are int32 TMA coordinates
  if ((static_cast<int64_t>(p.total_q) * p.kv_block_num + 128LL * p.num_logical_pages) * p.num_qo_heads > 0x7fffffffLL) return 0;
  if (p.sparse_ws_bytes < fmha_sparse_tc_workspace_bytes(p.total_q, p.num_qo_heads, p.num_kv_heads, p.kv_block_num,
                                                         p.num_logical_pages))
    return 0;
  return 1;
}

int fmha_sparse_tc_launch(const MsaFmhaParams& p, cudaStream_t stream) {
  using namespace sparse_tc;
  if (!p.out) return MSA_ERR_BAD_ARG;
  const int G = p.num_qo_heads / p.num_kv_heads;
  const int64_t NP = p.num_logical_pages;
  const int64_t NB = NP * p.num_kv_heads;
  if (NB > 0x7fffffffLL / 2) return MSA_ERR_TOO_LARGE;
  Ws w = carve(p.sparse_ws, p.total_q, p.num_qo_heads, p.num_kv_heads, p.kv_block_num, NP);
  if (w.max_items > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;

  // 1. reverse index
  const int64_t zero_bytes = reinterpret_cast<char*>(w.bin_offset) - reinterpret_cast<char*>(w.bin_count);
  if (cudaMemsetAsync(w.bin_count, 0, zero_bytes, stream) != cudaSuccess) return MSA_ERR_LAUNCH;
  IndexArgs ia;
  ia.kbi = p.kv_block_indexes; ia.kbi_stride_tok = p.kbi_stride_tok; ia.kbi_stride_head = p.kbi_stride_head;
  ia.token_batch = p.token_batch; ia.qo_start = p.qo_start; ia.kv_len = p.kv_len; ia.qo_offset = p.qo_offset;
  ia.kv_page_indptr = p.kv_page_indptr;
  ia.total_q = p.total_q; ia.num_kv_heads = p.num_kv_heads; ia.num_qo_heads = p.num_qo_heads;
  ia.kbn = p.kv_block_num; ia.num_pages = static_cast<int32_t>(NP);
  const int64_t n_thr = static_cast<int64_t>(p.total_q) * p.num_kv_heads;
  const unsigned n_blk = static_cast<unsigned>((n_thr + 255) / 256);
  const int tpc = BM / G;
  const int rows_per_item = tpc * ITEM_CHUNKS;
  const size_t hist_bytes = static_cast<size_t>(NP) * 4;
  const bool smem_hist = hist_bytes <= 48 * 1024 && !g_force_global_index;
  const unsigned n_blk_s = static_cast<unsigned>((p.total_q + 255) / 256) * p.num_kv_heads;
  auto index_pass = [&](bool scatter) {
    if (!smem_hist) {
      if (scatter) sparse_index_kernel<true><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.inv);
      else sparse_index_kernel<false><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.inv);
    } else if (p.kv_block_num <= 16) {
      if (scatter) sparse_index_smem_kernel<true, 16><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.inv);
      else sparse_index_smem_kernel<false, 16><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.inv);
    } else {
      if (scatter) sparse_index_smem_kernel<true, 32><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.inv);
      else sparse_index_smem_kernel<false, 32><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.inv);
    }
  };
  index_pass(false);
  sparse_scan_kernel<<<1, 1024, 0, stream>>>(w.bin_count, w.bin_offset, w.bin_cursor, w.items, w.part_start,
                                             static_cast<int>(NB), rows_per_item, static_cast<int>(w.max_items), tpc,
                                             static_cast<int>(NP));
  index_pass(true);
  if (cudaGetLastError() != cudaSuccess) return MSA_ERR_LAUNCH;

  // 2. attention over (page, token chunk) items
  CUtensorMap tq, tk, tv, to;
  {
    if ((G & 7) == 0) {       // [token][half][head][64]: one box carries both halves of 8 rows
      const uint64_t dims[4] = {64, static_cast<uint64_t>(p.num_qo_heads), 2, static_cast<uint64_t>(p.total_q)};
      const uint64_t str[3] = {static_cast<uint64_t>(p.q_stride_head) * 2, 128, static_cast<uint64_t>(p.q_stride_tok) * 2};
      const uint32_t box[4] = {64, 8, 2, 1};
      if (make_tma_map_bf16(&tq, p.q, 4, dims, str, box) != MSA_OK) return MSA_ERR_LAUNCH;
    } else {
      const uint64_t dims[3] = {128, static_cast<uint64_t>(p.num_qo_heads), static_cast<uint64_t>(p.total_q)};
      const uint64_t str[2] = {static_cast<uint64_t>(p.q_stride_head) * 2, static_cast<uint64_t>(p.q_stride_tok) * 2};
      const uint32_t box[3] = {64, static_cast<uint32_t>(G), 1};
      if (make_tma_map_bf16(&tq, p.q, 3, dims, str, box) != MSA_OK) return MSA_ERR_LAUNCH;
    }
    // the partial rows: [cap * G][128], stored one 128-row chunk and 64-column half at a time
    const uint64_t odims[2] = {128, static_cast<uint64_t>(w.cap) * G};
    const uint64_t ostr[1] = {256};
    const uint32_t obox[2] = {64, BM};
    if (make_tma_map_bf16(&to, w.partial_o, 2, odims, ostr, obox) != MSA_OK) return MSA_ERR_LAUNCH;
    const uint64_t kd[4] = {128, BN, static_cast<uint64_t>(p.num_kv_heads), static_cast<uint64_t>(p.kv_extent)};
    const uint64_t ks[3] = {static_cast<uint64_t>(p.k_stride_tok) * 2, static_cast<uint64_t>(p.k_stride_head) * 2,
                            static_cast<uint64_t>(p.k_stride_page) * 2};
    const uint64_t vs[3] = {static_cast<uint64_t>(p.v_stride_tok) * 2, static_cast<uint64_t>(p.v_stride_head) * 2,
                            static_cast<uint64_t>(p.v_stride_page) * 2};
    const uint32_t kbox[4] = {64, BN, 1, 1};
    if (make_tma_map_bf16(&tk, p.k, 4, kd, ks, kbox) != MSA_OK || make_tma_map_bf16(&tv, p.v, 4, kd, vs, kbox) != MSA_OK)
      return MSA_ERR_LAUNCH;
  }
  static bool attr_done[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 16 || !attr_done[dev]) {
    if (cudaFuncSetAttribute(sparse_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return MSA_ERR_LAUNCH;
    if (dev < 16) attr_done[dev] = true;
  }
  sparse_tc_kernel<<<static_cast<unsigned>(w.max_items), NTHREADS, SMEM_BYTES, stream>>>(p, tq, tk, tv, to, w.items, w.part_start,
                                                                                     -1, w.entries, w.partial_lse);
  if (cudaGetLastError() != cudaSuccess) return MSA_ERR_LAUNCH;

  // 3. merge the kv_block_num partials of every (token, head).  (Running the merge of kv head k on a
  // second stream with a small grid while the attention kernel works on head k + 1 was tried: an SM
  // sustains ~60 GB/s of gathered reads with its registers as the only landing space, so the merge
  // needs a third of the SMs to keep up and the attention kernel loses more than the merge gains.)
  const int64_t rows = static_cast<int64_t>(p.total_q) * p.num_qo_heads;
  const int64_t blocks = (rows + 15) / 16;
  if (blocks > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  __nv_bfloat16* outp = static_cast<__nv_bfloat16*>(p.out);
#define MSA_MERGE(KK)                                                                                             \
  sparse_merge_kernel<KK><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(                                    \
      w.partial_o, w.partial_lse, w.inv, outp, p.lse, p.kv_block_num, p.total_q, p.num_qo_heads, p.num_kv_heads, \
      p.out_stride_tok, p.out_stride_head, p.out_scale, 0, p.num_kv_heads)
  if (p.kv_block_num <= 8) MSA_MERGE(8);
  else if (p.kv_block_num <= 16) MSA_MERGE(16);
  else MSA_MERGE(32);
#undef MSA_MERGE
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

}  // namespace msa

// Test hook (not part of the documented ABI): exercise the index kernels that large page counts use.
extern "C" void msa_debug_sparse_force_global_index(int on) { msa::sparse_tc::g_force_global_index = on != 0; }

// Debug aid: choose the CTA whose phase clocks are recorded (-1 = none) / read the record back.
extern "C" void msa_debug_sparse_trace_cta(int cta) {
  cudaMemcpyToSymbol(msa::sparse_tc::g_trace_cta, &cta, sizeof(int));
}
extern "C" void msa_debug_sparse_trace_read(unsigned long long* host_buf) {
  cudaMemcpyFromSymbol(host_buf, msa::sparse_tc::g_trace, sizeof(unsigned long long) * 6 * 512 * 8);
}
