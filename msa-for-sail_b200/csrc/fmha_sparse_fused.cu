// Sparse (selected-pages) attention for long query batches: KV-outer attention and the merge of its
// per-page partials in ONE persistent kernel, scheduled so that the partials never leave the L2.
//
// The page-major schedule (fmha_sparse_tc.cu) computes every (token, selected page) pair once, as
// 128-row MMAs of the tokens that selected a page against that page -- and pays for it with one
// partial (O, LSE) row per (token, head, selected page): kv_block_num x the size of the output,
// written to HBM by the attention kernel and read back by a merge kernel.  On the MSA prefill
// shape that is 2 x 17 GB around 4.4 TFLOP of attention.  Here the same work is cut into BANDS of
// consecutive tokens of one KV head, small enough that a band's partials (tokens x kv_block_num x
// group heads x 256 B, about 32 MB) stay in the 126 MB L2 between being written and being merged:
//
//   stream of work items:  ATT(band 0) ATT(band 1) MRG(band 0) ATT(band 2) MRG(band 1) ...
//     ATT item = up to 32 chunks (of 128 / G tokens) of the tokens of one band that selected one page
//     MRG item = 32 tokens of a band: their kv_block_num partials -> the final O (and LSE)
//
// 148 persistent CTAs take items from the stream with an atomic ticket counter, in stream order.
// A MRG item waits (bounded) until every ATT item of its band has signalled that its partial rows
// are written; those items have lower tickets, so they are finished or running on another CTA, and
// an ATT item never waits for anything: no deadlock whatever the number of resident CTAs.
//
// Roles of a CTA (16 warps): warpgroups 0-2 (warps 0-11, 152 registers) own every third chunk from
// S to the stored partial (softmax, then O out of TMEM, normalised, bf16, staged, one bulk copy per
// token) and run the MRG items; warps 12-14 fetch tickets and gather the Q rows of a chunk (one TMA
// box per 8 rows); warp 15 issues the MMAs and the TMA loads of the page (K when the last Q K^T of
// the previous item has completed, V when its last P V has).  TMEM, barriers and the tensor maps
// are set up once per CTA.  All waits are bounded (tc_ptx.cuh).
//
// Upstream walks sparse attention token by token (csrc/include/prepare_plan_metadata.cuh:90-112,
// csrc/include/sm80_fmha_sparse_fwd_mainloop.hpp:249-601); the split-KV merge semantics are those
// of csrc/include/sm80_fmha_reduction.hpp:133-215.
#include "tc_ptx.cuh"

namespace msa {
int make_tma_map_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box);

namespace sparse_fused {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 128;
constexpr int SUB_BYTES = BM * 64 * 2;
constexpr int TILE_BYTES = 2 * SUB_BYTES;
constexpr int NWG = 3;                          // softmax + epilogue warpgroups; warpgroup x owns chunks r % 3 == x
constexpr int NSBUF = NWG;                      // S / P buffers in TMEM, one per warpgroup
constexpr int NQBUF = 2;                        // Q chunk buffers
constexpr int RING = 16;                        // work items a CTA holds descriptors of
constexpr int TICKETS = 4;                      // consecutive items taken per atomic
constexpr int OFF_Q = 0;
constexpr int OFF_K = NQBUF * TILE_BYTES;
constexpr int OFF_V = OFF_K + TILE_BYTES;
constexpr int OFF_STAGE = OFF_V + TILE_BYTES;   // bf16 O on its way out: [128 rows][256 B] per warpgroup
constexpr int OFF_BAR = OFF_STAGE + NWG * TILE_BYTES;
constexpr int OFF_RING = OFF_BAR + 512;
constexpr int ITEM_INTS = 12;
constexpr int SMEM_BYTES = OFF_RING + RING * ITEM_INTS * 4 + 64 + 1024;
constexpr int NTHREADS = 512;
constexpr int GATHER_WARP0 = 4 * NWG, GATHER_WARPS = 3, MMA_WARP = GATHER_WARP0 + GATHER_WARPS;
constexpr int GATHER_THREADS = GATHER_WARPS * 32;
constexpr int REGS_SOFTMAX = 152, REGS_OTHER = 40;
constexpr int REGS_NEEDED = NWG * 128 * REGS_SOFTMAX + (GATHER_WARPS + 1) * 32 * REGS_OTHER;
static_assert(NTHREADS == (MMA_WARP + 1) * 32, "warp roles");
static_assert(REGS_NEEDED <= 65536, "setmaxnreg budget");
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory");
constexpr int ITEM_CHUNKS = 32;                 // chunks of 128 rows per ATT item
constexpr int MERGE_TOKENS = 32;                // tokens per MRG item
constexpr int64_t BAND_BYTES = 32ll << 20;      // partial bytes of one band
constexpr int64_t MAX_BINS = 1ll << 22;         // bands get longer rather than the histogram larger
constexpr uint32_t kEmuMask = 0x5252;
constexpr uint32_t O_COL = NSBUF * BN;
constexpr uint32_t kFlagSpin = 1u << 22;        // polls (with back-off) of a band's completion count

enum Bar { K_FULL = 0, V_FULL = 1, V_FIX = 2, K_EMPTY = 3, V_EMPTY = 4, Q_FULL = 5, Q_EMPTY = 7, S_FULL = 9, P_FULL = 12,
           O_FULL = 15, O_FREE = 18, ITEM_FULL = 19, ITEM_EMPTY = ITEM_FULL + RING, NUM_BARS = ITEM_EMPTY + RING };
static_assert(NUM_BARS * 8 <= 512 - 32, "barrier area");

// work item: 12 ints.  [0] kind: 0 ATT, 1 MRG, 2 END
//   ATT: [1] kv head [2] physical page [3] first key position of the page [4] entry_begin [5] entry_end
//        [6] band group [7] first token of the batch item [8] kv_len [9] qo_offset [10] valid rows of the page
//   MRG: [1] kv head [2] token_begin [3] token_end [6] band group [7] completion count to wait for
enum { KIND_ATT = 0, KIND_MRG = 1, KIND_END = 2 };

struct Ws {                 // device workspace carved by carve()
  int32_t* bin_count;       // [NB]   selections per (kv head, band, page)                       } zeroed
  int32_t* band_done;       // [NG]   warps that finished their part of an ATT item of the band   } before
  int32_t* ticket;          // [1]                                                                  } each run
  int32_t* bin_cursor;      // [NB]
  int32_t* bin_ent;         // [NB]   start of the bin within its group's entries (chunk aligned)
  int32_t* bin_item;        // [NB]   first ATT item of the bin within its group
  int32_t* grp_ent;         // [NG]   entries (padded) of the group
  int32_t* grp_att;         // [NG]   ATT items of the group
  int32_t* grp_sig;         // [NG]   completion signals its ATT items send
  int32_t* grp_ent_base;    // [NG]
  int32_t* grp_att_pos;     // [NG]   stream position of the group's first ATT item
  int32_t* grp_mrg_pos;     // [NG]   ... of its first MRG item
  int32_t* n_stream;        // [1]    items in the stream
  int32_t* items;           // [max_items][12]
  int32_t* entries;         // [cap]  token << 5 | slot, sorted by (group, page); gaps between bins are padding
  int32_t* vmask;           // [T, Hkv]  bit s: slot s of this (token, kv head) selects a visible page
  float* partial_lse;       // [T, Hkv, kbn, G]
  __nv_bfloat16* partial_o; // [T, Hkv, kbn, G, 128]
  int64_t cap, max_items, total_bytes, zero_bytes;
  int32_t band_tokens, num_bands, num_groups;
  int64_t num_bins;
};

inline int64_t align256(int64_t x) { return (x + 255) & ~int64_t(255); }

Ws carve(void* base, int64_t T, int Hq, int Hkv, int kbn, int64_t NP) {
  Ws w;
  const int G = Hq / Hkv;
  const int64_t tpc = BM / G;
  // band length: a power of two of at least 256 tokens whose partials fill BAND_BYTES; longer when the
  // (kv head, band, page) histogram would otherwise grow past MAX_BINS
  int64_t bt = 256;
  while (bt * kbn * G * 256 * 2 <= BAND_BYTES) bt *= 2;
  while (((T + bt - 1) / bt) * Hkv * NP > MAX_BINS && bt < (int64_t(1) << 30)) bt *= 2;
  w.band_tokens = static_cast<int32_t>(bt);
  w.num_bands = static_cast<int32_t>(T > 0 ? (T + bt - 1) / bt : 1);
  w.num_groups = w.num_bands * Hkv;
  w.num_bins = static_cast<int64_t>(w.num_groups) * NP;
  const int64_t sel = T * Hkv * kbn;
  const int64_t nonempty = sel < w.num_bins ? sel : w.num_bins;
  w.cap = sel + nonempty * (tpc - 1) + tpc;
  const int64_t mrg = static_cast<int64_t>(Hkv) * ((T + MERGE_TOKENS - 1) / MERGE_TOKENS + w.num_bands);
  w.max_items = sel / (tpc * ITEM_CHUNKS) + nonempty + mrg + 16;
  char* p = static_cast<char*>(base);
  int64_t off = 0;
  auto take = [&](int64_t bytes) { char* r = p ? p + off : nullptr; off = align256(off + bytes); return r; };
  w.bin_count = reinterpret_cast<int32_t*>(take(w.num_bins * 4));
  w.band_done = reinterpret_cast<int32_t*>(take(w.num_groups * 4));
  w.ticket = reinterpret_cast<int32_t*>(take(4));
  w.zero_bytes = off;                                            // everything above is zeroed before each run
  w.bin_cursor = reinterpret_cast<int32_t*>(take(w.num_bins * 4));
  w.bin_ent = reinterpret_cast<int32_t*>(take(w.num_bins * 4));
  w.bin_item = reinterpret_cast<int32_t*>(take(w.num_bins * 4));
  w.grp_ent = reinterpret_cast<int32_t*>(take(w.num_groups * 4));
  w.grp_att = reinterpret_cast<int32_t*>(take(w.num_groups * 4));
  w.grp_sig = reinterpret_cast<int32_t*>(take(w.num_groups * 4));
  w.grp_ent_base = reinterpret_cast<int32_t*>(take(w.num_groups * 4));
  w.grp_att_pos = reinterpret_cast<int32_t*>(take(w.num_groups * 4));
  w.grp_mrg_pos = reinterpret_cast<int32_t*>(take(w.num_groups * 4));
  w.n_stream = reinterpret_cast<int32_t*>(take(4));
  w.items = reinterpret_cast<int32_t*>(take(w.max_items * ITEM_INTS * 4));
  w.entries = reinterpret_cast<int32_t*>(take(w.cap * 4));
  w.vmask = reinterpret_cast<int32_t*>(take(T * Hkv * 4));
  w.partial_lse = reinterpret_cast<float*>(take(T * Hkv * kbn * G * 4));
  w.partial_o = reinterpret_cast<__nv_bfloat16*>(take(T * Hkv * kbn * G * kHeadDim * 2));
  w.total_bytes = off;
  return w;
}

// ------------------------------------------------------------------------------------------
// reverse index: counting sort of the valid (token, kv head, slot) selections by (kv head, band, page)
// ------------------------------------------------------------------------------------------
struct IndexArgs {
  const int32_t* kbi; int64_t kbi_stride_tok, kbi_stride_head;
  const int32_t* token_batch; const int32_t* qo_start; const int32_t* kv_len; const int32_t* qo_offset;
  const int32_t* kv_page_indptr;
  int32_t* status; int32_t batch;
  int32_t total_q, num_kv_heads, kbn, num_pages, band_tokens, num_bands;
};

__device__ __forceinline__ bool entry_valid(const IndexArgs& a, int t, int b, int blk) {
  if (blk < 0) return false;
  const int pos0 = blk * BN;
  if (pos0 >= a.kv_len[b]) return false;
  const int i = t - a.qo_start[b];
  return pos0 <= i + a.qo_offset[b];            // at least the page's first key is visible
}

// one thread per (kv head, token); global atomics (any page count)
template <bool SCATTER>
__global__ void __launch_bounds__(256)
index_kernel(const IndexArgs a, int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_cursor,
             int32_t* __restrict__ entries, int32_t* __restrict__ vmask) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // kvh-major, token fastest
  const int64_t n = static_cast<int64_t>(a.total_q) * a.num_kv_heads;
  if (gid >= n) return;
  const int kvh = static_cast<int>(gid / a.total_q), t = static_cast<int>(gid % a.total_q);
  const int b = chk(a.token_batch[t], 0, a.batch, a.status);
  const int page_base = a.kv_page_indptr[b];
  const int64_t bin0 = (static_cast<int64_t>(kvh) * a.num_bands + t / a.band_tokens) * a.num_pages;
  const int32_t* row = a.kbi + static_cast<int64_t>(t) * a.kbi_stride_tok + static_cast<int64_t>(kvh) * a.kbi_stride_head;
  uint32_t mask = 0;
  for (int s = 0; s < a.kbn; ++s) {
    const int blk = row[s];
    if (entry_valid(a, t, b, blk)) {
      const int64_t bin = bin0 + page_base + blk;
      mask |= 1u << s;
      if (SCATTER) entries[atomicAdd(&bin_cursor[bin], 1)] = (t << 5) | s;
      else atomicAdd(&bin_count[bin], 1);
    }
  }
  if (SCATTER) vmask[static_cast<int64_t>(t) * a.num_kv_heads + kvh] = static_cast<int32_t>(mask);
}

// The same two passes with a shared-memory histogram: a CTA owns 256 consecutive tokens of one kv head
// (one band: bands are multiples of 256 tokens), counts (or ranks) its selections per page in shared
// memory and touches global memory once per (CTA, page).  Needs num_pages * 4 bytes of shared memory.
template <bool SCATTER, int KBN>
__global__ void __launch_bounds__(256)
index_smem_kernel(const IndexArgs a, int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_cursor,
                  int32_t* __restrict__ entries, int32_t* __restrict__ vmask) {
  extern __shared__ int32_t s_hist[];                      // [num_pages] count, then (scatter) next position
  const int blocks_per_head = (a.total_q + 255) / 256;
  const int kvh = blockIdx.x / blocks_per_head;
  const int tb = (blockIdx.x % blocks_per_head) * 256;
  const int t = tb + threadIdx.x;
  const int64_t bin0 = (static_cast<int64_t>(kvh) * a.num_bands + tb / a.band_tokens) * a.num_pages;
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
      if (SCATTER) s_hist[i] = atomicAdd(&bin_cursor[bin0 + i], c);   // reserve c consecutive positions
      else atomicAdd(&bin_count[bin0 + i], c);
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

__device__ __forceinline__ int block_exclusive_scan_256(int v, int* s_warp, int& total) {
  // exclusive prefix of v over the 256 threads of the CTA; total = the CTA's sum
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int x = v;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int y = __shfl_up_sync(0xffffffffu, x, d);
    if (lane >= d) x += y;
  }
  __syncthreads();                                          // s_warp may still be read from the previous call
  if (lane == 31) s_warp[warp] = x;
  __syncthreads();
  int base = 0, tot = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) { const int sw = s_warp[i]; if (i < warp) base += sw; tot += sw; }
  total = tot;
  return base + x - v;
}

// pass 1 of the layout: one CTA per (kv head, band) group scans the group's page bins
__global__ void __launch_bounds__(256)
group_scan_kernel(const int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_ent, int32_t* __restrict__ bin_item,
                  int32_t* __restrict__ grp_ent, int32_t* __restrict__ grp_att, int32_t* __restrict__ grp_sig, int num_pages,
                  int tpc, int rows_per_item) {
  __shared__ int s_warp[8];
  const int g = blockIdx.x;
  const int64_t bin0 = static_cast<int64_t>(g) * num_pages;
  int carry_ent = 0, carry_itm = 0, sig = 0;
  for (int base = 0; base < num_pages; base += 256) {
    const int i = base + threadIdx.x;
    const int cnt = i < num_pages ? bin_count[bin0 + i] : 0;
    const int pad = (cnt + tpc - 1) / tpc * tpc;            // a bin starts on a chunk boundary
    const int nit = (cnt + rows_per_item - 1) / rows_per_item;
    int tot_e, tot_i;
    const int pe = block_exclusive_scan_256(pad, s_warp, tot_e);
    const int pi = block_exclusive_scan_256(nit, s_warp, tot_i);
    if (i < num_pages) { bin_ent[bin0 + i] = carry_ent + pe; bin_item[bin0 + i] = carry_itm + pi; }
    // completion signals of the bin's items: one per warp of every warpgroup that gets a chunk
    for (int k = 0; k < nit; ++k) {
      const int rows = min(rows_per_item, cnt - k * rows_per_item);
      sig += 4 * min(NWG, (rows + tpc - 1) / tpc);
    }
    carry_ent += tot_e; carry_itm += tot_i;
  }
  // sum of sig over the CTA
  int tot_s;
  block_exclusive_scan_256(sig, s_warp, tot_s);
  if (threadIdx.x == 0) { grp_ent[g] = carry_ent; grp_att[g] = carry_itm; grp_sig[g] = tot_s; }
}

// pass 2: one CTA walks the groups: entry bases and stream positions
//   stream: ATT(0) ATT(1) MRG(0) ATT(2) MRG(1) ... ATT(NG-1) MRG(NG-2) MRG(NG-1)
__global__ void __launch_bounds__(256)
stream_scan_kernel(const int32_t* __restrict__ grp_ent, const int32_t* __restrict__ grp_att, int32_t* __restrict__ grp_ent_base,
                   int32_t* __restrict__ grp_att_pos, int32_t* __restrict__ grp_mrg_pos, int32_t* __restrict__ n_stream,
                   int num_groups, int num_bands, int band_tokens, int total_q) {
  __shared__ int s_warp[8];
  auto mrg_units = [&](int g) {                              // MRG items of a group = its band's tokens / 32
    const int band = g % num_bands;
    const int tok = min(band_tokens, total_q - band * band_tokens);
    return (max(tok, 0) + MERGE_TOKENS - 1) / MERGE_TOKENS;
  };
  int carry_ent = 0, carry_pos = 0;
  for (int base = 0; base < num_groups; base += 256) {
    const int g = base + threadIdx.x;
    const int e = g < num_groups ? grp_ent[g] : 0;
    // what group g adds to the stream before ATT(g + 1): its own ATT items and MRG(g - 1)
    const int adv = g < num_groups ? grp_att[g] + (g >= 1 ? mrg_units(g - 1) : 0) : 0;
    int tot_e, tot_p;
    const int pe = block_exclusive_scan_256(e, s_warp, tot_e);
    const int pp = block_exclusive_scan_256(adv, s_warp, tot_p);
    if (g < num_groups) {
      grp_ent_base[g] = carry_ent + pe;
      grp_att_pos[g] = carry_pos + pp;
      if (g >= 1) grp_mrg_pos[g - 1] = carry_pos + pp + grp_att[g];
    }
    carry_ent += tot_e; carry_pos += tot_p;
  }
  if (threadIdx.x == 0) {
    grp_mrg_pos[num_groups - 1] = carry_pos;
    *n_stream = carry_pos + mrg_units(num_groups - 1);
  }
}

// pass 3: one CTA per group writes its ATT items, its MRG items and the scatter cursors of its bins
struct ItemArgs {
  const int32_t* bin_count; const int32_t* bin_ent; const int32_t* bin_item; const int32_t* grp_ent_base;
  const int32_t* grp_att_pos; const int32_t* grp_mrg_pos; const int32_t* grp_sig;
  int32_t* bin_cursor; int32_t* items;
  const int32_t* page_batch; const int32_t* kv_page_indptr; const int32_t* kv_indices; const int32_t* qo_start;
  const int32_t* kv_len; const int32_t* qo_offset;
  int32_t num_pages, num_bands, band_tokens, total_q, rows_per_item, max_items;
  int32_t* status; int32_t batch; int32_t kv_extent;
};

__global__ void __launch_bounds__(256) item_kernel(const ItemArgs a) {
  const int g = blockIdx.x;
  const int kvh = g / a.num_bands, band = g % a.num_bands;
  const int64_t bin0 = static_cast<int64_t>(g) * a.num_pages;
  const int ent_base = a.grp_ent_base[g], att_pos = a.grp_att_pos[g];
  for (int i = threadIdx.x; i < a.num_pages; i += 256) {
    const int cnt = a.bin_count[bin0 + i];
    const int ent0 = ent_base + a.bin_ent[bin0 + i];
    a.bin_cursor[bin0 + i] = ent0;
    if (cnt == 0) continue;
    const int b = chk(a.page_batch[i], 0, a.batch, a.status);
    const int lpage = i - a.kv_page_indptr[b];
    const int kvl = a.kv_len[b];
    const int nit = (cnt + a.rows_per_item - 1) / a.rows_per_item;
    for (int k = 0; k < nit; ++k) {
      const int pos = att_pos + a.bin_item[bin0 + i] + k;
      if (pos >= a.max_items) break;
      int32_t* it = a.items + static_cast<int64_t>(pos) * ITEM_INTS;
      it[0] = KIND_ATT; it[1] = kvh; it[2] = chk(a.kv_indices[i], 0, a.kv_extent, a.status); it[3] = lpage * BN;
      it[4] = ent0 + k * a.rows_per_item; it[5] = min(ent0 + cnt, ent0 + (k + 1) * a.rows_per_item);
      it[6] = g; it[7] = a.qo_start[b]; it[8] = kvl; it[9] = a.qo_offset[b]; it[10] = min(BN, kvl - lpage * BN); it[11] = 0;
    }
  }
  const int t0 = band * a.band_tokens, t1 = min(a.total_q, t0 + a.band_tokens);
  const int units = (max(t1 - t0, 0) + MERGE_TOKENS - 1) / MERGE_TOKENS;
  const int mrg_pos = a.grp_mrg_pos[g], sig = a.grp_sig[g];
  for (int u = threadIdx.x; u < units; u += 256) {
    const int pos = mrg_pos + u;
    if (pos >= a.max_items) break;
    int32_t* it = a.items + static_cast<int64_t>(pos) * ITEM_INTS;
    it[0] = KIND_MRG; it[1] = kvh; it[2] = t0 + u * MERGE_TOKENS; it[3] = min(t1, t0 + (u + 1) * MERGE_TOKENS);
    it[4] = 0; it[5] = 0; it[6] = g; it[7] = sig; it[8] = 0; it[9] = 0; it[10] = 0; it[11] = 0;
  }
}

__device__ __forceinline__ int ld_acquire(const int32_t* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ------------------------------------------------------------------------------------------
// the persistent kernel
// ------------------------------------------------------------------------------------------
struct RunArgs {
  const int32_t* items; const int32_t* n_stream; int32_t* ticket; int32_t* band_done;
  const int32_t* entries; const int32_t* vmask; float* partial_lse; __nv_bfloat16* partial_o;
};

template <int KBN>
__global__ void __launch_bounds__(NTHREADS, 1)
sparse_fused_kernel(const __grid_constant__ MsaFmhaParams p, const __grid_constant__ CUtensorMap tm_q,
                    const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                    const RunArgs ra) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + OFF_BAR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 8);
  volatile int* skip_flag = abort_flag + 1;      // set when the status word already reports a timeout
  volatile int32_t* ring = reinterpret_cast<volatile int32_t*>(smem_gen + OFF_RING);      // [RING][ITEM_INTS]
  auto bar = [&](int i) -> uint32_t { return bars + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int G = p.num_qo_heads / p.num_kv_heads;
  const int tpc = BM / G;                                  // tokens per chunk

  if (threadIdx.x == blockDim.x - 1)
    *skip_flag = (p.status != nullptr && *reinterpret_cast<const volatile int32_t*>(p.status) != 0) ? 1 : 0;
  if (threadIdx.x == 0) {
    mbar_init(bar(K_FULL), 1); mbar_init(bar(V_FULL), 1); mbar_init(bar(V_FIX), 1);
    mbar_init(bar(K_EMPTY), 1); mbar_init(bar(V_EMPTY), 1);
    for (int s = 0; s < NQBUF; ++s) { mbar_init(bar(Q_FULL + s), 1);  mbar_init(bar(Q_EMPTY + s), 1); }
    for (int s = 0; s < NSBUF; ++s) {
      mbar_init(bar(S_FULL + s), 1);  mbar_init(bar(P_FULL + s), BM);  mbar_init(bar(O_FULL + s), 1);
    }
    mbar_init(bar(O_FREE), BM);                                      // the warpgroup of the chunk drains O
    for (int s = 0; s < RING; ++s) {
      mbar_init(bar(ITEM_FULL + s), 1);
      mbar_init(bar(ITEM_EMPTY + s), GATHER_WARPS + 1 + 4 * NWG);    // every consumer warp releases the slot
    }
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

  // the work item at stream position s of THIS CTA (its s-th item), once ITEM_FULL of the slot has completed
  auto item_field = [&](int s, int f) -> int { return ring[(s % RING) * ITEM_INTS + f]; };

  if (!run) {
    // nothing: fall through to the teardown
  } else if (warp >= GATHER_WARP0 && warp < GATHER_WARP0 + GATHER_WARPS) {
    // =========================== ticket fetch + Q gather ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    const int gw = warp - GATHER_WARP0;
    const int gt = threadIdx.x - GATHER_WARP0 * 32;
    if (gw == 0 && lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
    const bool unit8 = (G & 7) == 0;
    const int unit = gw + GATHER_WARPS * lane;              // unit n -> warp n % 3, lane n / 3
    const int upt = unit8 ? G / 8 : 1;                      // units per token
    bool alive = true;
    int fetched = 0;                                        // items written to the ring (warp 0 only)
    bool ended = false;
    int r = 0;                                              // real chunks so far (Q buffer ring)
    const int n_stream = *ra.n_stream;
    for (int s = 0; alive; ++s) {
      // ---- warp 0: keep the ring ahead of this position (a batch of TICKETS items per atomic) ----
      if (gw == 0) {
        while (!ended && fetched < s + 2 && alive) {           // fewer than two items ahead: take the next batch
          int first = 0;
          if (lane == 0) first = atomicAdd(ra.ticket, TICKETS);
          first = __shfl_sync(0xffffffffu, first, 0);
          for (int k = 0; k < TICKETS && alive; ++k) {
            const int slot = fetched % RING;
            if (fetched >= RING) alive = mbar_wait(bar(ITEM_EMPTY + slot), ((fetched / RING) - 1) & 1, abort_flag);
            if (!alive) break;
            const int tk = first + k;
            if (lane < ITEM_INTS) {
              int v = lane == 0 ? KIND_END : 0;
              if (tk < n_stream) v = ra.items[static_cast<int64_t>(tk) * ITEM_INTS + lane];
              ring[slot * ITEM_INTS + lane] = v;
            }
            __syncwarp();
            if (lane == 0) { __threadfence_block(); mbar_arrive(bar(ITEM_FULL + slot)); }
            ++fetched;
            if (tk >= n_stream) { ended = true; break; }    // the END marker is the last thing written
          }
        }
      }
      if (!alive) break;
      alive = mbar_wait(bar(ITEM_FULL + s % RING), (s / RING) & 1, abort_flag);
      if (!alive) break;
      const int kind = item_field(s, 0);
      if (kind == KIND_ATT) {
        const int kvh = item_field(s, 1), e_begin = item_field(s, 4), e_end = item_field(s, 5);
        const int n_chunks = (e_end - e_begin + tpc - 1) / tpc;
        auto entry_of = [&](int c) -> int {
          const int e = e_begin + c * tpc + unit / upt;
          return (c < n_chunks && unit8 && unit < BM / 8 && e < e_end) ? ra.entries[e] : -1;
        };
        int ent = entry_of(0);
        for (int c = 0; c < n_chunks && alive; ++c, ++r) {
          const int x = r % NQBUF, u = r / NQBUF;
          alive = mbar_wait(bar(Q_EMPTY + x), (u & 1) ^ 1, abort_flag);   // Q K^T of chunk r - 2 has read the buffer
          if (!alive) break;
          const int e0 = e_begin + c * tpc;
          const int ntok = min(tpc, e_end - e0);
          if (gt == 0) mbar_arrive_expect_tx(bar(Q_FULL + x), ntok * G * 256);
          if (unit8) {
            if (ent >= 0)
              tma_load_4d(smem_base + OFF_Q + x * TILE_BYTES + unit * 2048, &tm_q, bar(Q_FULL + x), 0, kvh * G + (unit % upt) * 8, 0,
                          ent >> 5);
            ent = entry_of(c + 1);
          } else {
            for (int ti = unit; ti < ntok; ti += GATHER_THREADS) {
              const int tok = ra.entries[e0 + ti] >> 5;
              const uint32_t dst = smem_base + OFF_Q + x * TILE_BYTES + ti * G * 128;
              tma_load_3d(dst, &tm_q, bar(Q_FULL + x), 0, kvh * G, tok);
              tma_load_3d(dst + SUB_BYTES, &tm_q, bar(Q_FULL + x), 64, kvh * G, tok);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(ITEM_EMPTY + s % RING));
      if (kind == KIND_END) break;
    }
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer + page loads ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");
    constexpr uint32_t IDESC_QK = idesc_bf16(BM, BN, false, false);
    constexpr uint32_t IDESC_PV = idesc_bf16(BM, kHeadDim, false, true);
    const uint64_t dk_hi = smem_desc(0, 16, 1024) & 0xFFFFFFFFFFFF0000ull;
    const uint64_t dv_hi = smem_desc(0, SUB_BYTES, 1024) & 0xFFFFFFFFFFFF0000ull;
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
    // Two cursors walk this CTA's items: the Q K^T stream (up to three chunks ahead: S_{r+3} reuses the buffer
    // of P_r, so it follows P_r V in issue order) and the P V stream.  Each loads its operand page when it
    // enters an item -- K once the last Q K^T of the previous item has completed, V once its last P V has --
    // and the warp polls everything it could do next instead of blocking on one thing in a fixed order.
    bool alive = true;
    int s_qk = 0, s_pv = 0;            // item positions of the cursors
    int n_qk = -1, n_pv = -1;          // chunks of the item under the cursor; -1: descriptor not read yet
    int c_qk = 0, c_pv = 0;
    int a_qk = 0, a_pv = 0;            // ATT items entered so far (phase of the page barriers)
    int qk = 0, pv = 0;                // real chunks issued so far
    bool k_issued = false, k_ready = false, v_issued = false, v_ready = false, end_qk = false, end_pv = false;
    int n_fix = 0;                     // pages whose tail rows were zeroed so far (phase of V_FIX)
    uint32_t idle = 0;
    while (alive && !end_pv) {
      bool did = false;
      // ---------------- P V cursor ----------------
      if (n_pv < 0) {
        if (mbar_test(bar(ITEM_FULL + s_pv % RING), (s_pv / RING) & 1)) {
          alive = mbar_wait(bar(ITEM_FULL + s_pv % RING), (s_pv / RING) & 1, abort_flag);   // every lane observes it
          if (!alive) break;
          const int kind = item_field(s_pv, 0);
          if (kind == KIND_ATT) {
            n_pv = (item_field(s_pv, 5) - item_field(s_pv, 4) + tpc - 1) / tpc;
            c_pv = 0; v_issued = false; v_ready = false;
          } else {
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ITEM_EMPTY + s_pv % RING));
            if (kind == KIND_END) end_pv = true; else ++s_pv;
          }
          did = true;
        }
      } else {
        if (!v_issued && (a_pv == 0 || mbar_test(bar(V_EMPTY), (a_pv - 1) & 1))) {
          if (a_pv > 0) { alive = mbar_wait(bar(V_EMPTY), (a_pv - 1) & 1, abort_flag); if (!alive) break; }
          const int valid_rows = item_field(s_pv, 10);
          const bool fix = valid_rows < BN;
          const uint32_t vbar = fix ? bar(V_FIX) : bar(V_FULL);
          if (elect_one()) {
            mbar_arrive_expect_tx(vbar, TILE_BYTES);
            tma_load_4d(smem_base + OFF_V, &tm_v, vbar, 0, 0, item_field(s_pv, 1), item_field(s_pv, 2));
            tma_load_4d(smem_base + OFF_V + SUB_BYTES, &tm_v, vbar, 64, 0, item_field(s_pv, 1), item_field(s_pv, 2));
          }
          __syncwarp();
          if (fix) {                                       // rows past the sequence's last key may hold anything: zero them
            alive = mbar_wait(bar(V_FIX), n_fix & 1, abort_flag);
            ++n_fix;
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            unsigned char* vt = smem_gen + OFF_V;
            for (int c = lane; c < (BN - valid_rows) * 16; c += 32) {
              const int rr = valid_rows + (c >> 4), ch = c & 15;
              *reinterpret_cast<uint4*>(vt + (ch >> 3) * SUB_BYTES + rr * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(V_FULL));
          }
          v_issued = true; did = true;
        }
        if (c_pv == n_pv) {                                  // the item's last P V has been issued
          if (elect_one()) mma_commit(bar(V_EMPTY));       // ... V may be overwritten once it has completed
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(ITEM_EMPTY + s_pv % RING));
          ++s_pv; ++a_pv; n_pv = -1; did = true;
        } else if (qk > pv && v_issued) {                    // S_pv has been issued
          bool rdy = mbar_test(bar(P_FULL + pv % NSBUF), (pv / NSBUF) & 1);
          if (rdy && pv > 0) rdy = mbar_test(bar(O_FREE), (pv - 1) & 1);
          if (rdy && !v_ready) rdy = mbar_test(bar(V_FULL), a_pv & 1);
          if (__any_sync(0xffffffffu, rdy)) {
            // every lane observes the completed phases itself (returns at once): the issuing lane may
            // not be one that saw them
            alive = mbar_wait(bar(P_FULL + pv % NSBUF), (pv / NSBUF) & 1, abort_flag);
            if (alive && pv > 0) alive = mbar_wait(bar(O_FREE), (pv - 1) & 1, abort_flag);
            if (alive && !v_ready) alive = mbar_wait(bar(V_FULL), a_pv & 1, abort_flag);
            if (!alive) break;
            v_ready = true;
            tc_fence_after();
            if (elect_one()) {
              issue_pv(pv % NSBUF);
              mma_commit(bar(O_FULL + pv % NSBUF));
            }
            __syncwarp();
            ++pv; ++c_pv;
            did = true;
          }
        }
      }
      // ---------------- Q K^T cursor ----------------
      if (!end_qk) {
        if (n_qk < 0) {
          if (mbar_test(bar(ITEM_FULL + s_qk % RING), (s_qk / RING) & 1)) {
            alive = mbar_wait(bar(ITEM_FULL + s_qk % RING), (s_qk / RING) & 1, abort_flag);
            if (!alive) break;
            const int kind = item_field(s_qk, 0);
            if (kind == KIND_ATT) {
              n_qk = (item_field(s_qk, 5) - item_field(s_qk, 4) + tpc - 1) / tpc;
              c_qk = 0; k_issued = false; k_ready = false;
            } else if (kind == KIND_END) {
              end_qk = true;
            } else {
              ++s_qk;                                        // MRG: nothing to issue (the P V cursor releases the slot)
            }
            did = true;
          }
        } else {
          if (!k_issued && (a_qk == 0 || mbar_test(bar(K_EMPTY), (a_qk - 1) & 1))) {
            if (a_qk > 0) { alive = mbar_wait(bar(K_EMPTY), (a_qk - 1) & 1, abort_flag); if (!alive) break; }
            if (elect_one()) {
              mbar_arrive_expect_tx(bar(K_FULL), TILE_BYTES);
              tma_load_4d(smem_base + OFF_K, &tm_k, bar(K_FULL), 0, 0, item_field(s_qk, 1), item_field(s_qk, 2));
              tma_load_4d(smem_base + OFF_K + SUB_BYTES, &tm_k, bar(K_FULL), 64, 0, item_field(s_qk, 1), item_field(s_qk, 2));
            }
            __syncwarp();
            k_issued = true; did = true;
          }
          if (c_qk == n_qk) {                                // the item's last Q K^T has been issued
            if (elect_one()) mma_commit(bar(K_EMPTY));
            __syncwarp();
            ++s_qk; ++a_qk; n_qk = -1; did = true;
          } else if (k_issued && qk < pv + NSBUF) {
            const int x = qk % NQBUF;
            bool rdy = mbar_test(bar(Q_FULL + x), (qk / NQBUF) & 1);
            if (rdy && !k_ready) rdy = mbar_test(bar(K_FULL), a_qk & 1);
            if (__any_sync(0xffffffffu, rdy)) {
              alive = mbar_wait(bar(Q_FULL + x), (qk / NQBUF) & 1, abort_flag);
              if (alive && !k_ready) alive = mbar_wait(bar(K_FULL), a_qk & 1, abort_flag);
              if (!alive) break;
              k_ready = true;
              tc_fence_after();
              if (elect_one()) {
                issue_qk(x, qk % NSBUF);
                mma_commit(bar(S_FULL + qk % NSBUF));
                mma_commit(bar(Q_EMPTY + x));
              }
              __syncwarp();
              ++qk; ++c_qk;
              did = true;
            }
          }
        }
      }
      if (did) {
        idle = 0;
      } else if (++idle >= kSpinLimit * 4u) {                // a MRG item may keep the warpgroups busy for a while
        *abort_flag = 1;
        alive = false;
      } else if ((idle & 255u) == 255u && *abort_flag) {
        alive = false;
      }
    }
  } else {
    // =========================== softmax + epilogue + merge: warpgroup x owns chunks r % 3 == x ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 152;");
    const int x = warp >> 2;
    const int r = ((warp & 3) << 5) | lane;                   // row of the chunk = TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tS = tmem + x * BN + lane_addr;
    const uint32_t tO = tmem + O_COL + lane_addr;
    const int unit_rows = G < 32 ? G : 32;
    const bool issuer = (r & (unit_rows - 1)) == 0;
    const int g = r & (G - 1);                                // head within the group
    bool alive = true;
    unsigned char* my_stage = smem_gen + OFF_STAGE + x * TILE_BYTES + r * 256;
    int rc = 0;                                               // real chunks so far, all warpgroups
    // completion signal of the last ATT item this warp wrote partial rows for: sent once those rows have
    // left the SM (the bulk copies of the warp's NEXT chunk are committed and all older ones completed)
    int pend_band = -1;
    auto flush_signal = [&](bool all) {
      if (pend_band < 0) return;
      if (issuer) { if (all) tma_store_wait_all(); else asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); }
      __syncwarp();
      if (lane == 0) { __threadfence(); atomicAdd(ra.band_done + pend_band, 1); }
      pend_band = -1;
    };
    for (int s = 0; alive; ++s) {
      alive = mbar_wait(bar(ITEM_FULL + s % RING), (s / RING) & 1, abort_flag);
      if (!alive) break;
      const int kind = item_field(s, 0);
      if (kind == KIND_ATT) {
        const int kvh = item_field(s, 1), pos0 = item_field(s, 3), e_begin = item_field(s, 4), e_end = item_field(s, 5);
        const int band = item_field(s, 6), qo_base = item_field(s, 7), kv_len = item_field(s, 8), off = item_field(s, 9);
        const int n_chunks = (e_end - e_begin + tpc - 1) / tpc;
        const float scale_log2 = p.sm_scale * kLog2e * (p.k_scale_head ? p.k_scale_head[kvh] : 1.f);
        const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;
        bool wrote = false;
        // first chunk of this item that belongs to this warpgroup
        int c = ((x - rc) % NWG + NWG) % NWG;
        int entry_next = (c < n_chunks && e_begin + c * tpc + r / G < e_end) ? ra.entries[e_begin + c * tpc + r / G] : 0;
        for (; c < n_chunks && alive; c += NWG) {
          const int rr = rc + c;                              // global chunk number: buffer phases
          const int u = rr / NWG;
          const int e_idx = e_begin + c * tpc + r / G;
          const bool row_ok = e_idx < e_end;
          const int entry = entry_next;
          {                                                   // the entry of this warpgroup's next chunk of the item
            const int e_nx = e_idx + NWG * tpc;
            entry_next = (c + NWG < n_chunks && e_nx < e_end) ? ra.entries[e_nx] : 0;
          }
          const int tok = entry >> 5;
          const int lim = row_ok ? min(tok - qo_base + off, kv_len - 1) : -1;
          alive = mbar_wait(bar(S_FULL + x), u & 1, abort_flag);
          if (!alive) break;
          tc_fence_after();
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
          const float inv = l_sum > 0.f ? vsh / l_sum : 0.f;
          const float lse = l_sum > 0.f ? msafe * kLn2 + __logf(l_sum) : -INFINITY;
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(bar(P_FULL + x));

          // ---- epilogue of the same chunk: O = P V (issued once P is in place and O of the chunk before is drained) ----
          // row of the partial buffer: [token][kv head][slot][head in group]
          const int64_t prow = ((static_cast<int64_t>(tok) * p.num_kv_heads + kvh) * p.kv_block_num + (entry & 31)) * G + g;
          if (row_ok) ra.partial_lse[prow] = lse;
          // the bulk copies of this warp's previous chunk have left its staging rows; if that chunk closed an
          // item, its band can be told now
          if (issuer) tma_store_wait_read();
          __syncwarp();
          alive = mbar_wait(bar(O_FULL + x), u & 1, abort_flag);
          if (!__all_sync(0xffffffffu, alive)) { alive = false; break; }
          tc_fence_after();
          tmem_ld32(tO, sv[0]);
          tmem_ld32(tO + 32, sv[1]);
          tmem_ld32(tO + 64, sv[2]);
          tmem_ld32(tO + 96, sv[3]);
          tmem_wait_ld();
          tc_fence_before();
          mbar_arrive(bar(O_FREE));                               // the next P V may overwrite O
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
          if (issuer) {                                           // every issuer commits a group per chunk: equal counts
            if (row_ok) bulk_store(ra.partial_o + prow * kHeadDim, smem_base + OFF_STAGE + x * TILE_BYTES + r * 256, unit_rows * 256);
            tma_store_commit();
          }
          flush_signal(false);                                    // the chunk before this one (if it closed an item)
          wrote = true;
        }
        if (wrote) pend_band = band;                              // signalled after this warp's next chunk, or at the next MRG / END
        rc += n_chunks;
      } else if (kind == KIND_MRG) {
        // ---- merge 32 tokens of a band: out[t, h] = sum_s w_s O_s / sum_s w_s, w_s = exp(lse_s - max) ----
        flush_signal(true);                                       // the band may be waiting for this warp's own rows
        const int kvh = item_field(s, 1), t_begin = item_field(s, 2), t_end = item_field(s, 3);
        const int band = item_field(s, 6), target = item_field(s, 7);
        bool ok = true;
        if (lane == 0) {
          uint32_t spins = 0;
          while (ld_acquire(ra.band_done + band) < target) {
            if (++spins >= kFlagSpin || ((spins & 255u) == 255u && *abort_flag)) { ok = false; break; }
            __nanosleep(64);
          }
          if (!ok) *abort_flag = 1;
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) { alive = false; break; }
        const int hw = (x * 128 + r) >> 4, l16 = r & 15;          // 24 half-warps, one (token, head) row each per pass
        const int n_rows = (t_end - t_begin) * G;
        const int kbn = p.kv_block_num;
        __nv_bfloat16* outp = static_cast<__nv_bfloat16*>(p.out);
        for (int row = hw; row < n_rows; row += NWG * 8) {
          const int t = t_begin + row / G, gh = row % G, h = kvh * G + gh;
          const int64_t tk = static_cast<int64_t>(t) * p.num_kv_heads + kvh;
          const uint32_t mask = static_cast<uint32_t>(ra.vmask[tk]);
          const int64_t prow0 = tk * kbn * G + gh;                // slot s of this row: prow0 + s * G
          const int piece = l16 ^ (gh & 7);                       // the 16-byte pieces of a stored row are XOR-ed with (head & 7)
          float lse[KBN];
          uint4 raw[KBN];
          float mx = -INFINITY;
#pragma unroll
          for (int s2 = 0; s2 < KBN; ++s2) {
            const bool have = s2 < kbn && ((mask >> s2) & 1u);
            const int64_t prow = prow0 + static_cast<int64_t>(s2 < kbn ? s2 : 0) * G;   // always a readable row; unused if !have
            raw[s2] = __ldcg(reinterpret_cast<const uint4*>(ra.partial_o + prow * kHeadDim + piece * 8));
            const float l = __ldcg(ra.partial_lse + prow);
            lse[s2] = have ? l : -INFINITY;
            mx = fmaxf(mx, lse[s2]);
          }
          const float mxs = (mx == -INFINITY) ? 0.f : mx;
          float acc[8];
#pragma unroll
          for (int cc = 0; cc < 8; ++cc) acc[cc] = 0.f;
          float sw = 0.f;
#pragma unroll
          for (int s2 = 0; s2 < KBN; ++s2) {
            const float wgt = lse[s2] != -INFINITY ? __expf(lse[s2] - mxs) : 0.f;
            if (wgt != 0.f) {                                      // value select after an unconditional load
              sw += wgt;
              const uint32_t* r4 = reinterpret_cast<const uint32_t*>(&raw[s2]);
#pragma unroll
              for (int cc = 0; cc < 4; ++cc) {
                acc[2 * cc] = fmaf(wgt, __uint_as_float(r4[cc] << 16), acc[2 * cc]);
                acc[2 * cc + 1] = fmaf(wgt, __uint_as_float(r4[cc] & 0xffff0000u), acc[2 * cc + 1]);
              }
            }
          }
          const float sc = sw > 0.f ? p.out_scale / sw : 0.f;
          __nv_bfloat16* dst = outp + static_cast<int64_t>(t) * p.out_stride_tok + static_cast<int64_t>(h) * p.out_stride_head + l16 * 8;
          uint4 pk;
          pk.x = pack2<false>(acc[0] * sc, acc[1] * sc);
          pk.y = pack2<false>(acc[2] * sc, acc[3] * sc);
          pk.z = pack2<false>(acc[4] * sc, acc[5] * sc);
          pk.w = pack2<false>(acc[6] * sc, acc[7] * sc);
          *reinterpret_cast<uint4*>(dst) = pk;
          if (p.lse && l16 == 0) p.lse[static_cast<int64_t>(t) * p.num_qo_heads + h] = sw > 0.f ? mxs + __logf(sw) : -INFINITY;
        }
      }
      // release the ring slot (one arrival per warp; no CTA-level barrier, so that a warp that gave up on a
      // wait never leaves another one waiting)
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(ITEM_EMPTY + s % RING));
      if (kind == KIND_END) break;
    }
    flush_signal(true);
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
}  // namespace sparse_fused

int64_t fmha_sparse_fused_workspace_bytes(int64_t total_q, int num_qo_heads, int num_kv_heads, int kbn, int64_t num_pages) {
  return sparse_fused::carve(nullptr, total_q, num_qo_heads, num_kv_heads, kbn, num_pages).total_bytes;
}

int fmha_sparse_fused_launch(const MsaFmhaParams& p, cudaStream_t stream) {
  using namespace sparse_fused;
  if (!p.out) return MSA_ERR_BAD_ARG;
  const int G = p.num_qo_heads / p.num_kv_heads;
  const int64_t NP = p.num_logical_pages;
  Ws w = carve(p.sparse_ws, p.total_q, p.num_qo_heads, p.num_kv_heads, p.kv_block_num, NP);
  if (w.max_items > 0x7fffffffLL / ITEM_INTS || w.num_bins > 0x7fffffffLL || w.cap > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  if (w.total_bytes > p.sparse_ws_bytes) return MSA_ERR_BAD_ARG;

  // 1. reverse index and the work stream
  if (cudaMemsetAsync(w.bin_count, 0, w.zero_bytes, stream) != cudaSuccess) return MSA_ERR_LAUNCH;
  IndexArgs ia;
  ia.kbi = p.kv_block_indexes; ia.kbi_stride_tok = p.kbi_stride_tok; ia.kbi_stride_head = p.kbi_stride_head;
  ia.token_batch = p.token_batch; ia.qo_start = p.qo_start; ia.kv_len = p.kv_len; ia.qo_offset = p.qo_offset;
  ia.kv_page_indptr = p.kv_page_indptr; ia.status = p.status; ia.batch = p.batch;
  ia.total_q = p.total_q; ia.num_kv_heads = p.num_kv_heads; ia.kbn = p.kv_block_num;
  ia.num_pages = static_cast<int32_t>(NP); ia.band_tokens = w.band_tokens; ia.num_bands = w.num_bands;
  const int64_t n_thr = static_cast<int64_t>(p.total_q) * p.num_kv_heads;
  const unsigned n_blk = static_cast<unsigned>((n_thr + 255) / 256);
  const int tpc = BM / G;
  const int rows_per_item = tpc * ITEM_CHUNKS;
  const size_t hist_bytes = static_cast<size_t>(NP) * 4;
  const bool smem_hist = hist_bytes <= 48 * 1024;
  const unsigned n_blk_s = static_cast<unsigned>((p.total_q + 255) / 256) * p.num_kv_heads;
  auto index_pass = [&](bool scatter) {
    if (!smem_hist) {
      if (scatter) index_kernel<true><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
      else index_kernel<false><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
    } else if (p.kv_block_num <= 16) {
      if (scatter) index_smem_kernel<true, 16><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
      else index_smem_kernel<false, 16><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
    } else {
      if (scatter) index_smem_kernel<true, 32><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
      else index_smem_kernel<false, 32><<<n_blk_s, 256, hist_bytes, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.vmask);
    }
  };
  index_pass(false);
  group_scan_kernel<<<w.num_groups, 256, 0, stream>>>(w.bin_count, w.bin_ent, w.bin_item, w.grp_ent, w.grp_att, w.grp_sig,
                                                       static_cast<int>(NP), tpc, rows_per_item);
  stream_scan_kernel<<<1, 256, 0, stream>>>(w.grp_ent, w.grp_att, w.grp_ent_base, w.grp_att_pos, w.grp_mrg_pos, w.n_stream,
                                            w.num_groups, w.num_bands, w.band_tokens, p.total_q);
  ItemArgs it;
  it.bin_count = w.bin_count; it.bin_ent = w.bin_ent; it.bin_item = w.bin_item; it.grp_ent_base = w.grp_ent_base;
  it.grp_att_pos = w.grp_att_pos; it.grp_mrg_pos = w.grp_mrg_pos; it.grp_sig = w.grp_sig;
  it.bin_cursor = w.bin_cursor; it.items = w.items;
  it.page_batch = p.page_batch; it.kv_page_indptr = p.kv_page_indptr; it.kv_indices = p.kv_indices; it.qo_start = p.qo_start;
  it.kv_len = p.kv_len; it.qo_offset = p.qo_offset;
  it.num_pages = static_cast<int32_t>(NP); it.num_bands = w.num_bands; it.band_tokens = w.band_tokens; it.total_q = p.total_q;
  it.rows_per_item = rows_per_item; it.max_items = static_cast<int32_t>(w.max_items);
  it.status = p.status; it.batch = p.batch; it.kv_extent = static_cast<int32_t>(p.kv_extent);
  item_kernel<<<w.num_groups, 256, 0, stream>>>(it);
  index_pass(true);
  if (cudaGetLastError() != cudaSuccess) return MSA_ERR_LAUNCH;

  // 2. attention + merge over the work stream
  CUtensorMap tq, tk, tv;
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
    const uint64_t kd[4] = {128, BN, static_cast<uint64_t>(p.num_kv_heads), static_cast<uint64_t>(p.kv_extent)};
    const uint64_t ks[3] = {static_cast<uint64_t>(p.k_stride_tok) * 2, static_cast<uint64_t>(p.k_stride_head) * 2,
                            static_cast<uint64_t>(p.k_stride_page) * 2};
    const uint64_t vs[3] = {static_cast<uint64_t>(p.v_stride_tok) * 2, static_cast<uint64_t>(p.v_stride_head) * 2,
                            static_cast<uint64_t>(p.v_stride_page) * 2};
    const uint32_t kbox[4] = {64, BN, 1, 1};
    if (make_tma_map_bf16(&tk, p.k, 4, kd, ks, kbox) != MSA_OK || make_tma_map_bf16(&tv, p.v, 4, kd, vs, kbox) != MSA_OK)
      return MSA_ERR_LAUNCH;
  }
  RunArgs ra;
  ra.items = w.items; ra.n_stream = w.n_stream; ra.ticket = w.ticket; ra.band_done = w.band_done;
  ra.entries = w.entries; ra.vmask = w.vmask; ra.partial_lse = w.partial_lse; ra.partial_o = w.partial_o;
  static int num_sms[16] = {};
  static bool attr_done[16][3] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  const int di = dev < 16 ? dev : 0;
  const int ki = p.kv_block_num <= 8 ? 0 : (p.kv_block_num <= 16 ? 1 : 2);
  auto setup = [&](auto kern) -> int {
    if (dev >= 16 || !attr_done[di][ki]) {
      // setmaxnreg can only hand out what the launch allocated: threads x compiled registers
      cudaFuncAttributes fa;
      if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess || fa.numRegs * NTHREADS < REGS_NEEDED) return MSA_ERR_LAUNCH;
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return MSA_ERR_LAUNCH;
      if (cudaDeviceGetAttribute(&num_sms[di], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return MSA_ERR_LAUNCH;
      if (dev < 16) attr_done[di][ki] = true;
    }
    return MSA_OK;
  };
#define MSA_FUSED(KK)                                                                                   \
  do {                                                                                                  \
    if (setup(sparse_fused_kernel<KK>) != MSA_OK) return MSA_ERR_LAUNCH;                                \
    sparse_fused_kernel<KK><<<num_sms[di], NTHREADS, SMEM_BYTES, stream>>>(p, tq, tk, tv, ra);          \
  } while (0)
  if (ki == 0) MSA_FUSED(8);
  else if (ki == 1) MSA_FUSED(16);
  else MSA_FUSED(32);
#undef MSA_FUSED
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

}  // namespace msa
