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
//   tile  ->  O = P V_page  ->  normalised partial O (bf16) + LSE, stored token-major at
//   [token][kv head][slot][head in group] (one TMA box per 8 rows: the heads of a token)
//
// and a merge kernel streams that buffer once: the `kv_block_num` partials of a (token, kv head)
// are one contiguous block, a bit mask per (token, kv head) says which slots were computed.
// Every (token, page) pair is computed exactly once regardless of how the selections overlap.
//
// Kernels in this file: count / scan / scatter (counting sort of the selections by page), the merge and the
// attention kernel.  Roles of the attention kernel (16 warps): warpgroups 0-2 (warps 0-11, 152 registers
// each) own every third chunk from S to the stored partial -- softmax of the chunk (a whole row of S is
// held at once), then, once P V is done, O out of TMEM, normalised, bf16, staged in shared memory and
// stored with one bulk copy per token; warps 12-14 loaders (the page by TMA, once; the Q rows of a chunk
// gathered with one TMA box per 8 rows, the boxes spread over the lanes of three warps because a warp
// issues its lanes' boxes one after another); warp 15 MMA issuer.
// All waits are bounded (see tc_ptx.cuh).
#include "tc_ptx.cuh"

namespace msa {
int make_tma_map_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box);
int make_tma_map_u8(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box);

namespace sparse_tc {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 128;
constexpr int SUB_BYTES = BM * 128;             // one [128 rows][128 bytes] swizzled sub-tile: 64 bf16 or 128 e4m3 per row
constexpr int STAGE_BYTES = BM * 256;           // bf16 O of one chunk on its way out
constexpr int NWG = 3;                          // softmax + epilogue warpgroups; warpgroup x owns chunks c % 3 == x
constexpr int NSBUF = NWG;                      // S / P buffers in TMEM, one per warpgroup
// F8: Q, K, V (and P) are e4m3 and the MMAs are kind::f8f6f4; otherwise bf16 and kind::f16.  The tiles are
// half as large in e4m3 and the shared memory that frees holds two more Q chunk buffers.
template <bool F8>
struct Cfg {
  static constexpr int NSUB = F8 ? 1 : 2;                 // sub-tiles per [128][head_dim] tile
  static constexpr int ROW_BYTES = F8 ? 128 : 256;        // one row of Q
  static constexpr int TILE_BYTES = NSUB * SUB_BYTES;
  static constexpr int NQBUF = F8 ? 4 : 2;                // Q chunk buffers
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = NQBUF * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + TILE_BYTES;
  // bf16 O on its way out: [128 rows][256 B] per warpgroup, the 16-byte pieces of a row XOR-ed with
  // (head & 7).  (Two buffers shared by the three warpgroups would leave room for a third bf16 Q buffer,
  // but a warpgroup then waits for another one's bulk copies to be read, ~1 000 clocks: slower.)
  static constexpr int OFF_STAGE = OFF_V + TILE_BYTES;
  static constexpr int OFF_BAR = OFF_STAGE + NWG * STAGE_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // P = 2^(s - m + offset) with m the exact maximum of the one tile: at most 2^8 in e4m3 (upstream's
  // offset, csrc/include/sm80_fmha_sparse_fwd_mainloop.hpp:409), which keeps small probabilities normal
  static constexpr float kPOffset = F8 ? 8.0f : 0.0f;
};
// 512 threads start with 128 registers each (65 536 in all); setmaxnreg then moves them between the
// roles.  The sum after the moves must stay within what the launch allocated, or the increase
// never completes: the launcher checks the compiled register count before it launches.
constexpr int NTHREADS = 512;
constexpr int GATHER_WARP0 = 4 * NWG, GATHER_WARPS = 3, MMA_WARP = GATHER_WARP0 + GATHER_WARPS;
constexpr int GATHER_THREADS = GATHER_WARPS * 32;
constexpr int REGS_SOFTMAX = 152, REGS_OTHER = 40;
constexpr int REGS_NEEDED = NWG * 128 * REGS_SOFTMAX + (GATHER_WARPS + 1) * 32 * REGS_OTHER;
static_assert(NTHREADS == (MMA_WARP + 1) * 32, "warp roles");
static_assert(REGS_NEEDED <= 65536, "setmaxnreg budget");
constexpr int ITEM_CHUNKS = 32;                 // chunks of 128 rows per work item
constexpr uint32_t kEmuMask = 0x5252;

// TMEM: three S buffers (P_c overwrites the front of S_c) and one O.  Q_{c+3} K^T reuses the buffer of
// chunk c, so it follows P_c V directly in the MMA warp's program and is ready long before its
// warpgroup asks.
constexpr uint32_t O_COL = NSBUF * BN;
// O_FULL has one barrier per warpgroup: a warpgroup that finished P_c may come to wait for O_c while
// O_{c-2} is the latest completion, and a single barrier would read as "done" (same parity).
enum Bar { K_FULL = 0, V_FULL = 1, V_FIX = 2, Q_FULL = 3, Q_EMPTY = 7, S_FULL = 11, P_FULL = 14, O_FULL = 17,
           O_FREE = 20, NUM_BARS = 21 };

#ifdef MSA_DEBUG_HOOKS
// optional clock trace of one CTA (debugging aid): [6 roles][512 chunks][8 tags]; roles: warpgroups 0-2,
// MMA 3, loaders 4
__device__ unsigned long long g_trace[6 * 512 * 8];
__device__ int g_trace_cta = -1;
#endif

struct Ws {                 // device workspace carved by carve()
  int32_t* bin_count;       // [NB + 1]
  int32_t* bin_offset;      // [NB + 1]  start of a bin in `entries`, a multiple of the tokens per chunk
  int32_t* bin_cursor;      // [NB]
  int32_t* part_start;      // [Hkv + 1]  first work item of every kv head, then the item count
  int4* items;              // [max_items] {bin, entry_begin, entry_end, 0}
  int32_t* entries;         // [cap]  token << 5 | slot, sorted by (kv head, page); gaps between bins are padding
  int32_t* vmask;           // [T, Hkv]  bit s: slot s of this (token, kv head) selects a visible page
  float* partial_lse;       // [T, Hkv, kbn, G]
  __nv_bfloat16* partial_o; // [T, Hkv, kbn, G, 128]
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
  w.vmask = reinterpret_cast<int32_t*>(take(T * Hkv * 4));
  w.partial_lse = reinterpret_cast<float*>(take(T * Hkv * kbn * G * 4));
  w.partial_o = reinterpret_cast<__nv_bfloat16*>(take(T * Hkv * kbn * G * kHeadDim * 2));
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
  int32_t* status; int32_t batch;
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
                    int32_t* __restrict__ entries, int32_t* __restrict__ vmask) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // kvh-major, token fastest
  const int64_t n = static_cast<int64_t>(a.total_q) * a.num_kv_heads;
  if (gid >= n) return;
  const int kvh = static_cast<int>(gid / a.total_q), t = static_cast<int>(gid % a.total_q);
  const int b = chk(a.token_batch[t], 0, a.batch, a.status);
  const int page_base = a.kv_page_indptr[b];
  const int32_t* row = a.kbi + static_cast<int64_t>(t) * a.kbi_stride_tok + static_cast<int64_t>(kvh) * a.kbi_stride_head;
  uint32_t mask = 0;
  for (int s = 0; s < a.kbn; ++s) {
    const int blk = row[s];
    if (entry_valid(a, t, b, blk)) {
      const int bin = kvh * a.num_pages + page_base + blk;
      mask |= 1u << s;
      if (SCATTER) entries[atomicAdd(&bin_cursor[bin], 1)] = (t << 5) | s;
      else atomicAdd(&bin_count[bin], 1);
    }
  }
  if (SCATTER) vmask[static_cast<int64_t>(t) * a.num_kv_heads + kvh] = static_cast<int32_t>(mask);
}

// The same two passes with a shared-memory histogram: a CTA owns 256 consecutive tokens of one kv
// head, counts (or ranks) its selections per page in shared memory and touches global memory once
// per (CTA, page) -- the global atomics drop from one per selection to one per distinct page of a
// CTA.  Needs num_pages * 4 bytes of shared memory; larger page counts use the kernel above.
template <bool SCATTER, int KBN>
__global__ void __launch_bounds__(256)
sparse_index_smem_kernel(const IndexArgs a, int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_cursor,
                         int32_t* __restrict__ entries, int32_t* __restrict__ vmask) {
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
    const int b = chk(a.token_batch[t], 0, a.batch, a.status);
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
    uint32_t mask = 0;
#pragma unroll
    for (int s = 0; s < KBN; ++s) {
      if (s < a.kbn && gpage[s] >= 0) {
        entries[atomicAdd(&s_hist[gpage[s]], 1)] = (t << 5) | s;
        mask |= 1u << s;
      }
    }
    vmask[static_cast<int64_t>(t) * a.num_kv_heads + kvh] = static_cast<int32_t>(mask);
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
// Half a warp per (token, head) row, lane l of the half owns columns 8l..8l+7.  Rows are walked in
// output order, which is also the order of the partial buffer: the kbn x G partial rows of a
// (token, kv head) are one contiguous block, so the pass streams.  All loads of a row are issued
// before any is used.
// ------------------------------------------------------------------------------------------
template <int KBN>
__global__ void __launch_bounds__(256)
sparse_merge_kernel(const __nv_bfloat16* __restrict__ po, const float* __restrict__ pl, const int32_t* __restrict__ vmask,
                    __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, int kbn, int total_q, int num_heads,
                    int num_kv_heads, int64_t out_stride_tok, int64_t out_stride_head, float out_scale) {
  const int l16 = threadIdx.x & 15;
  const int G = num_heads / num_kv_heads;
  const int64_t n_idx = static_cast<int64_t>(total_q) * num_heads;
  for (int64_t idx = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4); idx < n_idx;
       idx += static_cast<int64_t>(gridDim.x) * (blockDim.x >> 4)) {
  const int t = static_cast<int>(idx / num_heads), h = static_cast<int>(idx % num_heads);
  const int kvh = h / G, g = h % G;
  const int64_t row = idx;
  const int64_t tk = static_cast<int64_t>(t) * num_kv_heads + kvh;
  const uint32_t mask = static_cast<uint32_t>(__ldg(vmask + tk));
  const int64_t prow0 = tk * kbn * G + g;                   // slot s of this row: prow0 + s * G
  const int piece = l16 ^ (g & 7);                          // the attention kernel stores a row's 16-byte pieces XOR-ed with (head & 7)
  float lse[KBN];
  uint4 raw[KBN];
  float mx = -INFINITY;
#pragma unroll
  for (int s = 0; s < KBN; ++s) {
    const bool have = s < kbn && ((mask >> s) & 1u);
    const int64_t prow = prow0 + static_cast<int64_t>(s < kbn ? s : 0) * G;   // always a readable row; unused if !have
    raw[s] = *reinterpret_cast<const uint4*>(po + prow * kHeadDim + piece * 8);
    const float l = __ldg(pl + prow);
    lse[s] = have ? l : -INFINITY;
    mx = fmaxf(mx, lse[s]);
  }
  const float mxs = (mx == -INFINITY) ? 0.f : mx;
  // two columns per packed FMA; a bf16 pair widens with one shift and one mask
  uint64_t acc2[4];
#pragma unroll
  for (int c = 0; c < 4; ++c) acc2[c] = f2_pack(0.f, 0.f);
  float sw = 0.f;
#pragma unroll
  for (int s = 0; s < KBN; ++s) {
    const float w = lse[s] != -INFINITY ? __expf(lse[s] - mxs) : 0.f;
    if (w != 0.f) {                                          // value select after an unconditional load
      sw += w;
      const uint64_t w2 = f2_pack(w, w);
      const uint32_t* r4 = reinterpret_cast<const uint32_t*>(&raw[s]);
#pragma unroll
      for (int c = 0; c < 4; ++c)
        acc2[c] = f2_fma(f2_pack(__uint_as_float(r4[c] << 16), __uint_as_float(r4[c] & 0xffff0000u)), w2, acc2[c]);
    }
  }
  float acc[8];
#pragma unroll
  for (int c = 0; c < 4; ++c) f2_unpack(acc2[c], acc[2 * c], acc[2 * c + 1]);
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
template <bool F8>
__global__ void __launch_bounds__(NTHREADS, 1)
sparse_tc_kernel(const __grid_constant__ MsaFmhaParams p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const int4* __restrict__ items, const int32_t* __restrict__ part_start, const int part,
                 const int32_t* __restrict__ entries, float* __restrict__ partial_lse,
                 __nv_bfloat16* __restrict__ partial_o) {
  // this launch covers the work items of kv head `part`, or all of them (part < 0)
  const int item_idx = (part >= 0 ? part_start[part] : 0) + static_cast<int>(blockIdx.x);
  if (item_idx >= part_start[part >= 0 ? part + 1 : p.num_kv_heads]) return;   // uniform: before any barrier / TMEM use
  using C = Cfg<F8>;
  constexpr int TILE_BYTES = C::TILE_BYTES, NSUB = C::NSUB, NQBUF = C::NQBUF, ROW_BYTES = C::ROW_BYTES;
  constexpr int OFF_Q = C::OFF_Q, OFF_K = C::OFF_K, OFF_V = C::OFF_V, OFF_STAGE = C::OFF_STAGE, OFF_BAR = C::OFF_BAR;
  constexpr int SUB_ELEMS = F8 ? 128 : 64;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + OFF_BAR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 8);
  volatile int* skip_flag = abort_flag + 1;      // set when the status word already reports a timeout
  auto bar = [&](int i) -> uint32_t { return bars + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef MSA_DEBUG_HOOKS
  const bool tracing = static_cast<int>(blockIdx.x) == g_trace_cta;
  auto trace = [&](int role, int c, int tag) {
    if (tracing && c < 512) g_trace[(role * 512 + c) * 8 + tag] = clock64();
  };
#else
  auto trace = [](int, int, int) {};              // compiles to nothing
#endif

  // ---------------- work item ----------------
  const int4 item = items[item_idx];
  const int NP = p.num_logical_pages;
  const int kvh = item.x / NP, gp = item.x % NP;
  const int b = chk(p.page_batch[gp], 0, p.batch, p.status);
  const int lpage = gp - p.kv_page_indptr[b];
  const int phys = chk(p.kv_indices[gp], 0, static_cast<int>(p.kv_extent), p.status);
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
    for (int s = 0; s < NQBUF; ++s) { mbar_init(bar(Q_FULL + s), 1);  mbar_init(bar(Q_EMPTY + s), 1); }
    for (int s = 0; s < NSBUF; ++s) {
      mbar_init(bar(S_FULL + s), 1);  mbar_init(bar(P_FULL + s), BM);  mbar_init(bar(O_FULL + s), 1);
    }
    mbar_init(bar(O_FREE), BM);                                      // the warpgroup of the chunk drains O
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
        for (int hlf = 0; hlf < NSUB; ++hlf) {
          tma_load_4d(smem_base + OFF_K + hlf * SUB_BYTES, &tm_k, bar(K_FULL), hlf * SUB_ELEMS, 0, kvh, phys);
          tma_load_4d(smem_base + OFF_V + hlf * SUB_BYTES, &tm_v, vbar, hlf * SUB_ELEMS, 0, kvh, phys);
        }
      }
      __syncwarp();
      if (fix) {
        alive = mbar_wait(bar(V_FIX), 0, abort_flag);
        alive = __all_sync(0xffffffffu, alive);
        if (alive) {
          unsigned char* vt = smem_gen + OFF_V;
          for (int c = lane; c < (BN - valid_rows) * (NSUB * 8); c += 32) {
            const int r = valid_rows + c / (NSUB * 8), ch = c % (NSUB * 8);
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
    // half in the plain layout.  e4m3: a row is 128 bytes, so the box {128, 8, 1} of [token][head][128]
    // is one swizzle atom and unit n sits at n * 1 KB, which is the plain layout.
    const bool unit8 = (G & 7) == 0;
    const int unit = (warp - GATHER_WARP0) + GATHER_WARPS * lane;      // unit n -> warp n % 3, lane n / 3
    const int upt = unit8 ? G / 8 : 1;                      // units per token
    auto entry_of = [&](int c) -> int {                      // entry of the token this lane loads in chunk c (unit8)
      const int e = item.y + c * tpc + unit / upt;
      return (c < n_chunks && unit8 && unit < BM / 8 && e < item.z) ? entries[e] : -1;
    };
    // (Prefetching the boxes of the next chunk into L2 was tried: the loaders' time goes into issuing
    // boxes, ~150 clocks each within a warp, and twice as many made the gather later, not earlier.)
    int ent = entry_of(0);
    for (int c = 0; c < n_chunks && alive; ++c) {
      const int x = c % NQBUF, u = c / NQBUF;
      if (gt == 0) trace(4, c, 0);
      alive = mbar_wait(bar(Q_EMPTY + x), (u & 1) ^ 1, abort_flag);   // Q K^T of chunk c - 3 has read the buffer
      if (!alive) break;
      const int e0 = item.y + c * tpc;
      const int ntok = min(tpc, item.z - e0);
      if (gt == 0) {
        trace(4, c, 1);
        mbar_arrive_expect_tx(bar(Q_FULL + x), ntok * G * ROW_BYTES);
      }
      if (unit8) {
        if (ent >= 0) {
          if constexpr (F8)
            tma_load_3d(smem_base + OFF_Q + x * TILE_BYTES + unit * 1024, &tm_q, bar(Q_FULL + x), 0, kvh * G + (unit % upt) * 8,
                        ent >> 5);
          else
            tma_load_4d(smem_base + OFF_Q + x * TILE_BYTES + unit * 2048, &tm_q, bar(Q_FULL + x), 0, kvh * G + (unit % upt) * 8, 0,
                        ent >> 5);
        }
        ent = entry_of(c + 1);
      } else {
        for (int ti = unit; ti < ntok; ti += GATHER_THREADS) {
          const int tok = entries[e0 + ti] >> 5;
          const uint32_t dst = smem_base + OFF_Q + x * TILE_BYTES + ti * G * 128;
          tma_load_3d(dst, &tm_q, bar(Q_FULL + x), 0, kvh * G, tok);
          if constexpr (!F8) tma_load_3d(dst + SUB_BYTES, &tm_q, bar(Q_FULL + x), 64, kvh * G, tok);
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    constexpr uint32_t IDESC_QK = F8 ? idesc_e4m3(BM, BN, false, false) : idesc_bf16(BM, BN, false, false);
    constexpr uint32_t IDESC_PV = F8 ? idesc_e4m3(BM, kHeadDim, false, true) : idesc_bf16(BM, kHeadDim, false, true);
    constexpr int KSTEPS = F8 ? 4 : 8;              // MMAs per 128-deep contraction (32 bytes of K extent each)
    constexpr int V_KSTEP = (F8 ? 32 : 16) * 128;   // bytes between the key slices of consecutive P V MMAs
    const uint64_t dk_hi = smem_desc(0, 16, 1024) & 0xFFFFFFFFFFFF0000ull;
    const uint64_t dv_hi = smem_desc(0, SUB_BYTES, 1024) & 0xFFFFFFFFFFFF0000ull;
    // Q: 8-row groups 2 KB apart with the second head_dim half 1 KB after the first (G % 8 == 0),
    // else the plain two-sub-tile layout
    // (bf16; an e4m3 chunk is a single plain sub-tile)
    const bool unit8 = !F8 && (G & 7) == 0;
    const uint64_t dq_hi = unit8 ? (smem_desc(0, 16, 2048) & 0xFFFFFFFFFFFF0000ull) : dk_hi;
    const uint32_t q_half = unit8 ? 1024u : static_cast<uint32_t>(SUB_BYTES);
    auto issue_qk = [&](int x, int sb) {
      const uint32_t qa = (smem_base + OFF_Q + x * TILE_BYTES) >> 4, ka = (smem_base + OFF_K) >> 4;
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        const uint32_t o = ((k >> 2) * SUB_BYTES + (k & 3) * 32) >> 4;
        const uint32_t oq = ((k >> 2) * q_half + (k & 3) * 32) >> 4;
        if constexpr (F8) mma_ss_f8(tmem + sb * BN, dq_hi | ((qa + oq) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
        else mma_ss(tmem + sb * BN, dq_hi | ((qa + oq) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
      }
    };
    auto issue_pv = [&](int sb) {
      const uint32_t va = (smem_base + OFF_V) >> 4;
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {              // P: 8 TMEM columns per MMA in both formats
        const uint64_t vd = dv_hi | ((va + k * (V_KSTEP >> 4)) & 0x3FFF);
        if constexpr (F8) mma_ts_f8(tmem + O_COL, tmem + sb * BN + k * 8, vd, IDESC_PV, k > 0 ? 1u : 0u);
        else mma_ts(tmem + O_COL, tmem + sb * BN + k * 8, vd, IDESC_PV, k > 0 ? 1u : 0u);
      }
    };
    // Two streams share this warp: S_c = Q_c K^T (c may run three chunks ahead of the other stream:
    // S_{c+3} reuses the buffer of P_c, so it must follow P_c V in issue order) and O_d = P_d V (needs P_d
    // from its warpgroup and O of chunk d - 1 drained).  Each has waits of its own -- the Q gather on
    // one side, the drain of O on the other -- so the warp polls both and issues whichever is ready
    // instead of blocking on one in a fixed order.
    bool alive = mbar_wait(bar(K_FULL), 0, abort_flag);
    int pv = 0, qk = 0;
    uint32_t idle = 0;
    bool v_ready = false;
    while (alive && pv < n_chunks) {
      bool did = false;
      if (qk > pv) {                                          // S_pv has been issued
        bool rdy = mbar_test(bar(P_FULL + pv % NSBUF), (pv / NSBUF) & 1);
        if (rdy && pv > 0) rdy = mbar_test(bar(O_FREE), (pv - 1) & 1);
        if (__any_sync(0xffffffffu, rdy)) {
          if (!v_ready) { alive = mbar_wait(bar(V_FULL), 0, abort_flag); v_ready = true; if (!alive) break; }
          // every lane observes the completed phases itself (returns at once): the issuing lane may
          // not be one that saw them
          alive = mbar_wait(bar(P_FULL + pv % NSBUF), (pv / NSBUF) & 1, abort_flag);
          if (alive && pv > 0) alive = mbar_wait(bar(O_FREE), (pv - 1) & 1, abort_flag);
          if (!alive) break;
          tc_fence_after();
          if (lane == 0) trace(3, pv, 4);
          if (elect_one()) {
            issue_pv(pv % NSBUF);
            mma_commit(bar(O_FULL + pv % NSBUF));
          }
          __syncwarp();
          if (lane == 0) trace(3, pv, 5);
          ++pv;
          did = true;
        }
      }
      if (qk < n_chunks && qk < pv + NSBUF) {
        const int x = qk % NQBUF;
        if (__any_sync(0xffffffffu, mbar_test(bar(Q_FULL + x), (qk / NQBUF) & 1))) {
          alive = mbar_wait(bar(Q_FULL + x), (qk / NQBUF) & 1, abort_flag);
          if (!alive) break;
          tc_fence_after();
          if (lane == 0) trace(3, qk, 2);
          if (elect_one()) {
            issue_qk(x, qk % NSBUF);
            mma_commit(bar(S_FULL + qk % NSBUF));
            mma_commit(bar(Q_EMPTY + x));
          }
          __syncwarp();
          ++qk;
          did = true;
        }
      }
      if (did) {
        idle = 0;
      } else if (++idle >= kSpinLimit) {
        *abort_flag = 1;
        alive = false;
      } else if ((idle & 255u) == 255u && *abort_flag) {
        alive = false;
      }
    }
  } else {
    // =========================== softmax + epilogue: warpgroup x owns chunks c % 3 == x ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
    const int x = warp >> 2;
    const int r = ((warp & 3) << 5) | lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tS = tmem + x * BN + lane_addr;
    const uint32_t tO = tmem + O_COL + lane_addr;
    const float scale_log2 = p.sm_scale * kLog2e * (p.k_scale_head ? p.k_scale_head[kvh] : 1.f);
    const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;
    // The partial rows of a token (its G heads, for one slot) are contiguous in the token-major buffer
    // and in this warpgroup's staging tile: the first lane of every unit (G rows, at most the 32 rows
    // of a warp) stores it with one bulk copy.  Everything after the TMEM reads is local to a warp --
    // its 32 staging rows are written by its own lanes and stored by its own unit leaders -- so
    // __syncwarp is all the ordering the epilogue needs.
    const int unit_rows = G < 32 ? G : 32;
    const bool issuer = (r & (unit_rows - 1)) == 0;
    const int g = r & (G - 1);                                // head within the group
    bool alive = true;
    unsigned char* my_stage = smem_gen + OFF_STAGE + x * STAGE_BYTES + r * 256;
    int entry_next = (x < n_chunks && item.y + x * tpc + r / G < item.z) ? entries[item.y + x * tpc + r / G] : 0;
    for (int c = x; c < n_chunks && alive; c += NWG) {
      const int u = c / NWG;
      const int e_idx = item.y + c * tpc + r / G;
      const bool row_ok = e_idx < item.z;
      const int entry = entry_next;
      {                                                       // prefetch the entry of this warpgroup's next chunk
        const int e_nx = e_idx + NWG * tpc;
        entry_next = (c + NWG < n_chunks && e_nx < item.z) ? entries[e_nx] : 0;
      }
      const int tok = entry >> 5;
      const int lim = row_ok ? min(tok - qo_base + off, kv_len - 1) : -1;
      if (r == 0) trace(x, c, 0);
      alive = mbar_wait(bar(S_FULL + x), u & 1, abort_flag);
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
      const float msafe = ((mx == -INFINITY) ? 0.f : mx) - C::kPOffset;
      const uint64_t scale2 = f2_pack(scale_log2, scale_log2);
      const uint64_t negm2 = f2_pack(-msafe, -msafe);
      uint64_t lsum2 = f2_pack(0.f, 0.f);
      if (r == 0) trace(x, c, 3);
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t pk[F8 ? 8 : 16];
        uint16_t held = 0;
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
          if constexpr (F8) {
            const uint16_t pr = __nv_cvt_float2_to_fp8x2(make_float2(p0, p1), __NV_SATFINITE, __NV_E4M3);
            if (e & 2) pk[e >> 2] = static_cast<uint32_t>(held) | (static_cast<uint32_t>(pr) << 16);
            else held = pr;
          } else {
            pk[e >> 1] = pack2<false>(p0, p1);
          }
        }
        if constexpr (F8) tmem_st8(tS + cc * 8, pk);
        else tmem_st16(tS + cc * 16, pk);
      }
      float l0, l1;
      f2_unpack(lsum2, l0, l1);
      const float l_sum = l0 + l1;
      if (r == 0) trace(x, c, 4);
      const float inv = l_sum > 0.f ? vsh / l_sum : 0.f;
      const float lse = l_sum > 0.f ? msafe * kLn2 + __logf(l_sum) : -INFINITY;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + x));
      if (r == 0) trace(x, c, 2);

      // ---- epilogue of the same chunk: O = P V (issued once P is in place and O of chunk c - 1 is drained) ----
      // row of the partial buffer: [token][kv head][slot][head in group]
      const int64_t prow = ((static_cast<int64_t>(tok) * p.num_kv_heads + kvh) * p.kv_block_num + (entry & 31)) * G + g;
      if (row_ok) partial_lse[prow] = lse;
      // the bulk copies of chunk c - 3 have left this warp's staging rows
      if (issuer) tma_store_wait_read();
      __syncwarp();
      alive = mbar_wait(bar(O_FULL + x), u & 1, abort_flag);
      if (!__all_sync(0xffffffffu, alive)) { alive = false; break; }
      tc_fence_after();
      if (r == 0) trace(x, c, 5);
      tmem_ld32(tO, sv[0]);
      tmem_ld32(tO + 32, sv[1]);
      tmem_ld32(tO + 64, sv[2]);
      tmem_ld32(tO + 96, sv[3]);
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(bar(O_FREE));                               // P_{c+1} V may overwrite O
      if (r == 0) trace(x, c, 6);
      const uint64_t inv2 = f2_pack(inv, inv), zero2 = f2_pack(0.f, 0.f);
#pragma unroll
      for (int cc = 0; cc < 4; ++cc)
#pragma unroll
        for (int q = 0; q < 4; ++q) {                        // 16-byte pieces, XOR-swizzled by the head index
          uint32_t o[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {                       // two columns per packed multiply
            float a, b;
            f2_unpack(f2_fma(f2_pack(__uint_as_float(sv[cc][q * 8 + 2 * k]), __uint_as_float(sv[cc][q * 8 + 2 * k + 1])), inv2, zero2), a, b);
            o[k] = pack2<false>(a, b);
          }
          const uint4 o4 = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(my_stage + (((cc * 4 + q) ^ (g & 7)) << 4)) = o4;
        }
      fence_proxy_async_smem();                               // generic-proxy writes -> read by the bulk copy
      __syncwarp();
      if (issuer && row_ok) {
        bulk_store(partial_o + prow * kHeadDim, smem_base + OFF_STAGE + x * STAGE_BYTES + r * 256, unit_rows * 256);
        tma_store_commit();
      }
      if (r == 0) trace(x, c, 7);
    }
    if (issuer) tma_store_wait_all();                         // shared memory stays valid until the copies are done
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
  if (p.q_dtype != p.kv_dtype || (p.kv_dtype != MSA_DT_BF16 && p.kv_dtype != MSA_DT_E4M3)) return 0;
  if (p.page_size != sparse_tc::BN) return 0;
  const int G = p.num_qo_heads / p.num_kv_heads;
  if (G < 1 || G > 128 || (128 % G) != 0 || p.kv_block_num > 32 || p.total_q >= (1 << 26)) return 0;
  // row indices of the partial buffer are int32 TMA coordinates
  if (static_cast<int64_t>(p.total_q) * p.kv_block_num * p.num_qo_heads > 0x7fffffffLL) return 0;
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
  ia.kv_page_indptr = p.kv_page_indptr; ia.status = p.status; ia.batch = p.batch;
  ia.total_q = p.total_q; ia.num_kv_heads = p.num_kv_heads; ia.num_qo_heads = p.num_qo_heads;
  ia.kbn = p.kv_block_num; ia.num_pages = static_cast<int32_t>(NP);
  const int64_t n_thr = static_cast<int64_t>(p.total_q) * p.num_kv_heads;
  const unsigned n_blk = static_cast<unsigned>((n_thr + 255) / 256);
  const int tpc = BM / G;
  const int rows_per_item = tpc * ITEM_CHUNKS;
  const size_t hist_bytes = static_cast<size_t>(NP) * 4;
  const bool smem_hist = hist_bytes <= 48 * 1024;
  const unsigned n_blk_s = static_cast<unsigned>((p.total_q + 255) / 256) * p.num_kv_heads;
  auto index_pass = [&](bool scatter) {
    if (!smem_hist) {
      if (scatter) sparse_index_kernel<true><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
      else sparse_index_kernel<false><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
    } else if (p.kv_block_num <= 16) {
      if (scatter) sparse_index_smem_kernel<true, 16><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
      else sparse_index_smem_kernel<false, 16><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
    } else {
      if (scatter) sparse_index_smem_kernel<true, 32><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
      else sparse_index_smem_kernel<false, 32><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
    }
  };
  index_pass(false);
  sparse_scan_kernel<<<1, 1024, 0, stream>>>(w.bin_count, w.bin_offset, w.bin_cursor, w.items, w.part_start,
                                             static_cast<int>(NB), rows_per_item, static_cast<int>(w.max_items), tpc,
                                             static_cast<int>(NP));
  index_pass(true);
  if (cudaGetLastError() != cudaSuccess) return MSA_ERR_LAUNCH;

  // 2. attention over (page, token chunk) items
  CUtensorMap tq, tk, tv;
  const bool f8 = p.kv_dtype == MSA_DT_E4M3;
  const uint64_t es = f8 ? 1 : 2;                              // bytes per element
  const uint32_t sub = f8 ? 128 : 64;                          // elements per 128-byte row of a sub-tile
  auto make_map = f8 ? make_tma_map_u8 : make_tma_map_bf16;
  {
    if ((G & 7) == 0 && !f8) {       // [token][half][head][64]: one box carries both halves of 8 rows
      const uint64_t dims[4] = {64, static_cast<uint64_t>(p.num_qo_heads), 2, static_cast<uint64_t>(p.total_q)};
      const uint64_t str[3] = {static_cast<uint64_t>(p.q_stride_head) * 2, 128, static_cast<uint64_t>(p.q_stride_tok) * 2};
      const uint32_t box[4] = {64, 8, 2, 1};
      if (make_tma_map_bf16(&tq, p.q, 4, dims, str, box) != MSA_OK) return MSA_ERR_LAUNCH;
    } else {
      const uint64_t dims[3] = {128, static_cast<uint64_t>(p.num_qo_heads), static_cast<uint64_t>(p.total_q)};
      const uint64_t str[2] = {static_cast<uint64_t>(p.q_stride_head) * es, static_cast<uint64_t>(p.q_stride_tok) * es};
      const uint32_t box[3] = {sub, static_cast<uint32_t>((G & 7) == 0 ? 8 : G), 1};
      if (make_map(&tq, p.q, 3, dims, str, box) != MSA_OK) return MSA_ERR_LAUNCH;
    }
    const uint64_t kd[4] = {128, BN, static_cast<uint64_t>(p.num_kv_heads), static_cast<uint64_t>(p.kv_extent)};
    const uint64_t ks[3] = {static_cast<uint64_t>(p.k_stride_tok) * es, static_cast<uint64_t>(p.k_stride_head) * es,
                            static_cast<uint64_t>(p.k_stride_page) * es};
    const uint64_t vs[3] = {static_cast<uint64_t>(p.v_stride_tok) * es, static_cast<uint64_t>(p.v_stride_head) * es,
                            static_cast<uint64_t>(p.v_stride_page) * es};
    const uint32_t kbox[4] = {sub, BN, 1, 1};
    if (make_map(&tk, p.k, 4, kd, ks, kbox) != MSA_OK || make_map(&tv, p.v, 4, kd, vs, kbox) != MSA_OK)
      return MSA_ERR_LAUNCH;
  }
  static bool attr_done[2][16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int smem_bytes = f8 ? Cfg<true>::SMEM_BYTES : Cfg<false>::SMEM_BYTES;
  if (dev >= 16 || !attr_done[f8][dev]) {
    // setmaxnreg can only hand out what the launch allocated: threads x compiled registers
    cudaFuncAttributes fa;
    const cudaError_t e1 = f8 ? cudaFuncGetAttributes(&fa, sparse_tc_kernel<true>) : cudaFuncGetAttributes(&fa, sparse_tc_kernel<false>);
    if (e1 != cudaSuccess || fa.numRegs * NTHREADS < REGS_NEEDED) return MSA_ERR_LAUNCH;
    const cudaError_t e2 = f8 ? cudaFuncSetAttribute(sparse_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes)
                              : cudaFuncSetAttribute(sparse_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e2 != cudaSuccess) return MSA_ERR_LAUNCH;
    if (dev < 16) attr_done[f8][dev] = true;
  }
  if (f8)
    sparse_tc_kernel<true><<<static_cast<unsigned>(w.max_items), NTHREADS, smem_bytes, stream>>>(
        p, tq, tk, tv, w.items, w.part_start, -1, w.entries, w.partial_lse, w.partial_o);
  else
    sparse_tc_kernel<false><<<static_cast<unsigned>(w.max_items), NTHREADS, smem_bytes, stream>>>(
        p, tq, tk, tv, w.items, w.part_start, -1, w.entries, w.partial_lse, w.partial_o);
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
      w.partial_o, w.partial_lse, w.vmask, outp, p.lse, p.kv_block_num, p.total_q, p.num_qo_heads, p.num_kv_heads, \
      p.out_stride_tok, p.out_stride_head, p.out_scale)
  if (p.kv_block_num <= 8) MSA_MERGE(8);
  else if (p.kv_block_num <= 16) MSA_MERGE(16);
  else MSA_MERGE(32);
#undef MSA_MERGE
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

}  // namespace msa

#ifdef MSA_DEBUG_HOOKS
// Debug aid (builds with -DMSA_DEBUG_HOOKS only): choose the CTA whose phase clocks are recorded
// (-1 = none) / read the record back.
extern "C" void msa_debug_sparse_trace_cta(int cta) {
  cudaMemcpyToSymbol(msa::sparse_tc::g_trace_cta, &cta, sizeof(int));
}
extern "C" void msa_debug_sparse_trace_read(unsigned long long* host_buf) {
  cudaMemcpyFromSymbol(host_buf, msa::sparse_tc::g_trace, sizeof(unsigned long long) * 6 * 512 * 8);
}
#endif
