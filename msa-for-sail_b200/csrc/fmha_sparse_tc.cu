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
//   tile  ->  O = P V_page  ->  normalised partial O (bf16) + LSE per (slot, token, head)
//
// and the split-KV merge kernel combines the `kv_block_num` partials of every row.  Every
// (token, page) pair is computed exactly once regardless of how the selections overlap.
//
// Kernels in this file: count / scan / scatter (counting sort of the selections by page) and the
// attention kernel.  Roles of the attention kernel: warps 0-3 / 4-7 softmax + epilogue of even /
// odd chunks, warp 8 TMA producer (page once, Q rows of a chunk gathered per token), warp 9 MMA
// issuer.  All waits are bounded (see tc_ptx.cuh).
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
constexpr int OFF_STAGE = 4 * TILE_BYTES;       // per softmax warpgroup: 128 rows x 256 B of bf16 O
constexpr int OFF_ROWID = OFF_STAGE + 2 * TILE_BYTES;   // per warpgroup: 128 x int64 destination rows
constexpr int OFF_BAR = OFF_ROWID + 2 * BM * 8;
constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
constexpr int NTHREADS = 384;
constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;
constexpr int ITEM_CHUNKS = 32;                 // chunks of 128 rows per work item
constexpr uint32_t kEmuMask = 0x5252;

enum Bar { K_FULL = 0, V_FULL = 1, V_FIX = 2, Q_FULL = 3, Q_EMPTY = 5, S_FULL = 7, P_FULL = 9, O_FULL = 11,
           O_FREE = 13, NUM_BARS = 15 };

// optional clock trace of one CTA (debugging aid): [4 roles][512 chunks][8 tags]
__device__ unsigned long long g_trace[4 * 512 * 8];
__device__ int g_trace_cta = -1;

struct Ws {                 // device workspace carved by carve()
  int32_t* bin_count;       // [NB + 1]
  int32_t* bin_offset;      // [NB + 1]
  int32_t* bin_cursor;      // [NB]
  int32_t* item_count;      // [1]
  int4* items;              // [max_items] {bin, entry_begin, entry_end, 0}
  int32_t* entries;         // [T * Hkv * kbn]  token << 5 | slot
  float* partial_lse;       // [kbn, T, Hq]
  __nv_bfloat16* partial_o; // [kbn, T, Hq, 128]
  int64_t max_items;
  int64_t total_bytes;
};

inline int64_t align256(int64_t x) { return (x + 255) & ~int64_t(255); }

Ws carve(void* base, int64_t T, int Hq, int Hkv, int kbn, int64_t NP) {
  Ws w;
  const int64_t NB = static_cast<int64_t>(Hkv) * NP;
  const int G = Hq / Hkv;
  const int64_t tpc = BM / G;
  w.max_items = (T * Hkv * kbn) / (tpc * ITEM_CHUNKS) + NB + 1;
  char* p = static_cast<char*>(base);
  int64_t off = 0;
  auto take = [&](int64_t bytes) { char* r = p ? p + off : nullptr; off = align256(off + bytes); return r; };
  w.bin_count = reinterpret_cast<int32_t*>(take((NB + 1) * 4));
  w.item_count = reinterpret_cast<int32_t*>(take(256));
  const int64_t zero_bytes = off;   // everything above is zeroed before each run
  (void)zero_bytes;
  w.bin_offset = reinterpret_cast<int32_t*>(take((NB + 1) * 4));
  w.bin_cursor = reinterpret_cast<int32_t*>(take(NB * 4));
  w.items = reinterpret_cast<int4*>(take(w.max_items * 16));
  w.entries = reinterpret_cast<int32_t*>(take(T * Hkv * kbn * 4));
  w.partial_lse = reinterpret_cast<float*>(take(static_cast<int64_t>(kbn) * T * Hq * 4));
  w.partial_o = reinterpret_cast<__nv_bfloat16*>(take(static_cast<int64_t>(kbn) * T * Hq * kHeadDim * 2));
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
                    int32_t* __restrict__ entries, float* __restrict__ partial_lse) {
  const int64_t gid = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;   // kvh-major, token fastest
  const int64_t n = static_cast<int64_t>(a.total_q) * a.num_kv_heads;
  if (gid >= n) return;
  const int kvh = static_cast<int>(gid / a.total_q), t = static_cast<int>(gid % a.total_q);
  const int b = a.token_batch[t];
  const int page_base = a.kv_page_indptr[b];
  const int32_t* row = a.kbi + static_cast<int64_t>(t) * a.kbi_stride_tok + static_cast<int64_t>(kvh) * a.kbi_stride_head;
  const int G = a.num_qo_heads / a.num_kv_heads;
  for (int s = 0; s < a.kbn; ++s) {
    const int blk = row[s];
    if (entry_valid(a, t, b, blk)) {
      const int bin = kvh * a.num_pages + page_base + blk;
      if (SCATTER) entries[atomicAdd(&bin_cursor[bin], 1)] = (t << 5) | s;
      else atomicAdd(&bin_count[bin], 1);
    } else if (!SCATTER) {
      // this slot contributes nothing: its LSE reads as -inf in the merge
      float* l = partial_lse + (static_cast<int64_t>(s) * a.total_q + t) * a.num_qo_heads + kvh * G;
      for (int h = 0; h < G; ++h) l[h] = -INFINITY;
    }
  }
}

// exclusive scan of the bin counts + work items (one CTA; NB is a few thousand to ~1e5)
__global__ void __launch_bounds__(1024)
sparse_scan_kernel(const int32_t* __restrict__ bin_count, int32_t* __restrict__ bin_offset,
                   int32_t* __restrict__ bin_cursor, int4* __restrict__ items, int32_t* __restrict__ item_count,
                   int num_bins, int rows_per_item, int max_items) {
  __shared__ int s_ent[1024], s_itm[1024];
  __shared__ int carry_ent, carry_itm;
  if (threadIdx.x == 0) { carry_ent = 0; carry_itm = 0; }
  __syncthreads();
  for (int base = 0; base < num_bins; base += 1024) {
    const int bin = base + threadIdx.x;
    const int cnt = bin < num_bins ? bin_count[bin] : 0;
    const int nit = (cnt + rows_per_item - 1) / rows_per_item;
    s_ent[threadIdx.x] = cnt; s_itm[threadIdx.x] = nit;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {                   // Hillis-Steele inclusive scan
      const int e = threadIdx.x >= d ? s_ent[threadIdx.x - d] : 0;
      const int i2 = threadIdx.x >= d ? s_itm[threadIdx.x - d] : 0;
      __syncthreads();
      s_ent[threadIdx.x] += e; s_itm[threadIdx.x] += i2;
      __syncthreads();
    }
    const int ent0 = carry_ent + s_ent[threadIdx.x] - cnt;
    const int itm0 = carry_itm + s_itm[threadIdx.x] - nit;
    if (bin < num_bins) {
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
  if (threadIdx.x == 0) { bin_offset[num_bins] = carry_ent; *item_count = min(carry_itm, max_items); }
}

// ------------------------------------------------------------------------------------------
// attention kernel
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(NTHREADS, 1)
sparse_tc_kernel(const __grid_constant__ MsaFmhaParams p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                 const int4* __restrict__ items, const int32_t* __restrict__ item_count,
                 const int32_t* __restrict__ entries, __nv_bfloat16* __restrict__ partial_o,
                 float* __restrict__ partial_lse) {
  if (static_cast<int>(blockIdx.x) >= *item_count) return;       // uniform: before any barrier / TMEM use
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + OFF_BAR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return bars + 8u * i; };
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool tracing = static_cast<int>(blockIdx.x) == g_trace_cta;
  auto trace = [&](int role, int c, int tag) {
    if (tracing && c < 512) g_trace[(role * 512 + c) * 8 + tag] = clock64();
  };

  // ---------------- work item ----------------
  const int4 item = items[blockIdx.x];
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

  if (threadIdx.x == 0) {
    mbar_init(bar(K_FULL), 1); mbar_init(bar(V_FULL), 1); mbar_init(bar(V_FIX), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(Q_FULL + s), 1);  mbar_init(bar(Q_EMPTY + s), 1);
      mbar_init(bar(S_FULL + s), 1);  mbar_init(bar(P_FULL + s), BM);
      mbar_init(bar(O_FULL + s), 1);  mbar_init(bar(O_FREE + s), BM);
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

  if (warp == PRODUCER_WARP) {
    // =========================== TMA producer ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
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
    bool alive = true;
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
    for (int c = 0; c < n_chunks && alive; ++c) {
      const int x = c & 1, u = c >> 1;
      if (lane == 0) trace(3, c, 0);
      alive = mbar_wait(bar(Q_EMPTY + x), (u & 1) ^ 1, abort_flag);
      if (lane == 0) trace(3, c, 1);
      if (!alive) break;
      const int e0 = item.y + c * tpc;
      const int ntok = min(tpc, item.z - e0);
      if (lane == 0) mbar_arrive_expect_tx(bar(Q_FULL + x), ntok * G * 256);
      __syncwarp();
      for (int ti = lane; ti < ntok; ti += 32) {            // every lane gathers the rows of its own tokens
        const int tok = entries[e0 + ti] >> 5;
        const uint32_t dst = smem_base + OFF_Q + x * TILE_BYTES + ti * G * 128;
        tma_load_3d(dst, &tm_q, bar(Q_FULL + x), 0, kvh * G, tok);
        tma_load_3d(dst + SUB_BYTES, &tm_q, bar(Q_FULL + x), 64, kvh * G, tok);
      }
      __syncwarp();
    }
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    constexpr uint32_t IDESC_QK = idesc_bf16(BM, BN, false, false);
    constexpr uint32_t IDESC_PV = idesc_bf16(BM, kHeadDim, false, true);
    const uint64_t dk_hi = smem_desc(0, 16, 1024) & 0xFFFFFFFFFFFF0000ull;
    const uint64_t dv_hi = smem_desc(0, SUB_BYTES, 1024) & 0xFFFFFFFFFFFF0000ull;
    auto issue_qk = [&](int x) {
      const uint32_t qa = (smem_base + OFF_Q + x * TILE_BYTES) >> 4, ka = (smem_base + OFF_K) >> 4;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t o = ((k >> 2) * SUB_BYTES + (k & 3) * 32) >> 4;
        mma_ss(tmem + x * BN, dk_hi | ((qa + o) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
      }
    };
    auto issue_pv = [&](int x) {
      const uint32_t va = (smem_base + OFF_V) >> 4;
#pragma unroll
      for (int k = 0; k < 8; ++k)
        mma_ts(tmem + 256 + x * kHeadDim, tmem + x * BN + k * 8, dv_hi | ((va + k * (2048 >> 4)) & 0x3FFF), IDESC_PV,
               k > 0 ? 1u : 0u);
    };
    bool alive = mbar_wait(bar(K_FULL), 0, abort_flag);
    for (int c = 0; c <= n_chunks && alive; ++c) {
      if (c < n_chunks) {                                   // S[x] = Q_c K^T
        const int x = c & 1, u = c >> 1;
        if (lane == 0) trace(2, c, 0);
        alive = mbar_wait(bar(O_FREE + x), (u & 1) ^ 1, abort_flag);
        if (lane == 0) trace(2, c, 1);
        if (alive) alive = mbar_wait(bar(Q_FULL + x), u & 1, abort_flag);
        if (lane == 0) trace(2, c, 2);
        if (!alive) break;
        tc_fence_after();
        if (elect_one()) {
          issue_qk(x);
          mma_commit(bar(S_FULL + x));
          mma_commit(bar(Q_EMPTY + x));
        }
        __syncwarp();
      }
      if (c > 0) {                                          // O[y] = P_{c-1} V
        const int y = (c - 1) & 1, u = (c - 1) >> 1;
        if (c == 1) alive = mbar_wait(bar(V_FULL), 0, abort_flag);
        if (lane == 0) trace(2, c, 3);
        if (alive) alive = mbar_wait(bar(P_FULL + y), u & 1, abort_flag);
        if (lane == 0) trace(2, c, 4);
        if (!alive) break;
        tc_fence_after();
        if (elect_one()) {
          issue_pv(y);
          mma_commit(bar(O_FULL + y));
        }
        __syncwarp();
        if (lane == 0) trace(2, c, 5);
      }
    }
  } else if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  } else {
    // =========================== softmax + epilogue ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int x = warp >> 2;
    const int r = ((warp & 3) << 5) | lane;
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tS = tmem + x * BN + lane_addr;
    const uint32_t tO = tmem + 256 + x * kHeadDim + lane_addr;
    const int head = kvh * G + r % G;
    const float scale_log2 = p.sm_scale * kLog2e * (p.k_scale_head ? p.k_scale_head[kvh] : 1.f);
    const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;
    bool alive = true;
    int entry_next = (x < n_chunks && item.y + x * tpc + r / G < item.z) ? entries[item.y + x * tpc + r / G] : 0;
    for (int c = x; c < n_chunks && alive; c += 2) {
      const int u = c >> 1;
      const int e_idx = item.y + c * tpc + r / G;
      const bool row_ok = e_idx < item.z;
      const int entry = entry_next;
      {                                                       // prefetch the entry of this warpgroup's next chunk
        const int e_nx = e_idx + 2 * tpc;
        entry_next = (c + 2 < n_chunks && e_nx < item.z) ? entries[e_nx] : 0;
      }
      const int tok = entry >> 5, slot = entry & 31;
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
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + x));
      if (r == 0) trace(x, c, 2);

      // ---- epilogue of this chunk: normalised partial O (bf16) + LSE ----
      alive = mbar_wait(bar(O_FULL + x), u & 1, abort_flag);
      if (!alive) break;
      tc_fence_after();
      if (r == 0) trace(x, c, 3);
      const float inv = l_sum > 0.f ? vsh / l_sum : 0.f;
      const int64_t row_id = (static_cast<int64_t>(slot) * p.total_q + tok) * p.num_qo_heads + head;
      // stage the bf16 row in shared memory (16-byte chunks XOR-swizzled by row) so that the global
      // stores below are whole 256-byte rows instead of 16-byte pieces of 32 different rows
      unsigned char* stage = smem_gen + OFF_STAGE + x * TILE_BYTES;
      int64_t* rowids = reinterpret_cast<int64_t*>(smem_gen + OFF_ROWID) + x * BM;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t v[32];
        tmem_ld32(tO + cc * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 o4;
          o4.x = pack2<false>(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
          o4.y = pack2<false>(__uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
          o4.z = pack2<false>(__uint_as_float(v[e + 4]) * inv, __uint_as_float(v[e + 5]) * inv);
          o4.w = pack2<false>(__uint_as_float(v[e + 6]) * inv, __uint_as_float(v[e + 7]) * inv);
          const int chunk = cc * 4 + (e >> 3);
          *reinterpret_cast<uint4*>(stage + r * 256 + ((chunk ^ (r & 15)) << 4)) = o4;
        }
      }
      rowids[r] = row_ok ? row_id : -1;
      if (row_ok) partial_lse[row_id] = l_sum > 0.f ? msafe * kLn2 + __logf(l_sum) : -INFINITY;
      tc_fence_before();
      mbar_arrive(bar(O_FREE + x));                           // TMEM slot is free again
      if (r == 0) trace(x, c, 4);
      asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");
      {
        const int w4 = warp & 3;
#pragma unroll 4
        for (int it = 0; it < 16; ++it) {
          const int rr = w4 * 32 + it * 2 + (lane >> 4), chunk = lane & 15;
          const int64_t rid = rowids[rr];
          const uint4 val = *reinterpret_cast<const uint4*>(stage + rr * 256 + ((chunk ^ (rr & 15)) << 4));
          if (rid >= 0) __stcs(reinterpret_cast<uint4*>(partial_o + rid * kHeadDim + chunk * 8), val);   // streamed: keep L2 for Q / K / V
        }
      }
      asm volatile("bar.sync %0, 128;" ::"r"(1 + x) : "memory");
      if (r == 0) trace(x, c, 5);
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
  sparse_index_kernel<false><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.partial_lse);
  const int rows_per_item = (BM / G) * ITEM_CHUNKS;
  sparse_scan_kernel<<<1, 1024, 0, stream>>>(w.bin_count, w.bin_offset, w.bin_cursor, w.items, w.item_count,
                                             static_cast<int>(NB), rows_per_item, static_cast<int>(w.max_items));
  sparse_index_kernel<true><<<n_blk, 256, 0, stream>>>(ia, w.bin_count, w.bin_cursor, w.entries, w.partial_lse);
  if (cudaGetLastError() != cudaSuccess) return MSA_ERR_LAUNCH;

  // 2. attention over (page, token chunk) items
  CUtensorMap tq, tk, tv;
  {
    const uint64_t dims[3] = {128, static_cast<uint64_t>(p.num_qo_heads), static_cast<uint64_t>(p.total_q)};
    const uint64_t str[2] = {static_cast<uint64_t>(p.q_stride_head) * 2, static_cast<uint64_t>(p.q_stride_tok) * 2};
    const uint32_t box[3] = {64, static_cast<uint32_t>(G), 1};
    if (make_tma_map_bf16(&tq, p.q, 3, dims, str, box) != MSA_OK) return MSA_ERR_LAUNCH;
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
  sparse_tc_kernel<<<static_cast<unsigned>(w.max_items), NTHREADS, SMEM_BYTES, stream>>>(
      p, tq, tk, tv, w.items, w.item_count, w.entries, w.partial_o, w.partial_lse);
  if (cudaGetLastError() != cudaSuccess) return MSA_ERR_LAUNCH;

  // 3. merge the kv_block_num partials of every (token, head)
  return msa_lse_merge(w.partial_o, MSA_DT_BF16, w.partial_lse, nullptr, p.out, p.lse, p.kv_block_num, p.total_q,
                       p.num_qo_heads, p.out_stride_tok, p.out_stride_head, p.out_scale, stream);
}

}  // namespace msa

// Debug aid: choose the CTA whose phase clocks are recorded (-1 = none) / read the record back.
extern "C" void msa_debug_sparse_trace_cta(int cta) {
  cudaMemcpyToSymbol(msa::sparse_tc::g_trace_cta, &cta, sizeof(int));
}
extern "C" void msa_debug_sparse_trace_read(unsigned long long* host_buf) {
  cudaMemcpyFromSymbol(host_buf, msa::sparse_tc::g_trace, sizeof(unsigned long long) * 4 * 512 * 8);
}
