// Decode / short-query attention on tcgen05, sized for HBM bandwidth.
//
// Serves the q_len * (Hq/Hkv) <= 128 shapes of `fmha_sail` over a bf16 or e4m3 paged cache with
// 128-key pages (e4m3: kind::f8f6f4 MMAs, Q and P converted to e4m3, P offset by 2^4): dense paged decode with split-KV (upstream dense mainloop + pack-GQA,
// csrc/include/sm80_fmha_fwd_mainloop.hpp:262-636, api.py:308-318) and per-token sparse decode
// over kv_block_indexes (csrc/include/sm80_fmha_sparse_fwd_mainloop.hpp:249-601).
//
// A decode step reads every selected K/V byte once and does ~16 FLOP per byte, so what matters
// is keeping loads in flight.  One CTA = one (batch item | token, KV head, split).  Its rows are
// the packed (token, head-in-group) pairs; they occupy the first lanes of a 128-row MMA tile (the
// idle rows cost tensor time that is not on the critical path).  K and V pages stream through TMA
// rings of their own (3 tiles deep for bf16, 6 half-page tiles for e4m3); no thread ever computes
// a load address.
//
//   warps 0-3   softmax: thread r owns row r; with at most 16 rows (QUAD) the rows are replicated
//               into the four 32-lane quadrants and warp w handles key columns [32 w, 32 w + 32)
//   warp 4      TMA producer of K (page id read from the page table / the selected-page list)
//   warp 5      MMA issuer: S[j & 1] = Q K_j^T, O += P_j V_j; S is double-buffered in TMEM so
//               QK of tile j + 1 overlaps the softmax of tile j
//   warp 6      TMA producer of V (its own ring, so a full V ring never delays the next K tile)
//
// Output: normalised partial O (fp32) + natural-log LSE per split, or the final bf16 O when the
// work item is unsplit.  Every wait is bounded (tc_ptx.cuh).
#include <cstdio>

#include "tc_ptx.cuh"

namespace msa {
int make_tma_map_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box);
int make_tma_map_u8(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box);

namespace decode_tc {
namespace {

using namespace tc;

// The row sum is taken over the probabilities AS THE MMA SEES THEM (rounded to e4m3 / bf16), so that the
// weights of a row add up to its normaliser exactly: a row dominated by one key then reproduces that key's V
// whatever the rounding of its probability (with the unrounded sum the rounding error of the largest
// probability, up to 2^-4 in e4m3, goes straight into O).
__device__ __forceinline__ float2 e4m3x2_as_float2(uint16_t x) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(x), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

constexpr int BM = 128, BN = 128;
constexpr int SUB_BYTES = BM * 128;             // one [128 rows][128 bytes] swizzled sub-tile
constexpr int NTHREADS = 224;
constexpr int PRODUCER_WARP = 4, MMA_WARP = 5, V_PRODUCER_WARP = 6;
constexpr int MAX_SPARSE_TILES = 64;            // selected pages per work item
constexpr int MAX_STAGES = 6;
constexpr int QUAD_MAX_ROWS = 16;               // rows of a work item the 4-way column split accepts
constexpr int STAGE_LD = kHeadDim + 4;          // floats per staged O row (padding spreads the banks)

// PV_DONE completes once per tile (a warp that rescales O at tile j waits for P_{j-1} V: at that point the
// barrier is at most one phase behind, so the parity wait is unambiguous).  The epilogue must NOT wait on it: a
// softmax warp can finish its last tile while P_{n-2} V is still waiting for its V tile, i.e. two phases ahead
// of the barrier, where a parity wait for phase n - 1 reads phase n - 3 as "done".  O_DONE completes once, after
// the last P V.
enum Bar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 7, V_FULL = 13, V_EMPTY = 19, S_FULL = 25, P_FULL = 27, PV_DONE = 29,
           V_FIX = 30, O_DONE = 31, NUM_BARS = 32 };

#ifdef MSA_DEBUG_HOOKS
// diagnostic timeline: when set, every CTA records 16 words (see msa_debug_decode_trace)
__device__ unsigned long long* g_trace = nullptr;
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#endif

// Shared / tensor memory plan of one instantiation.
//   F8    K/V (and Q, P) are e4m3 and the MMAs are kind::f8f6f4; otherwise bf16 and kind::f16.
//   QUAD  work items of <= 16 rows: the rows are replicated into the four 32-lane quadrants of
//         the MMA tile and quadrant w runs an independent online softmax over key columns
//         [32 w, 32 w + 32) of every tile (its P is zero elsewhere), so all four softmax warps
//         work on a tile instead of the first lanes of one; the four partial (O, m, l) of a row
//         are combined in shared memory at the end.
//   F8 && QUAD ("dual"): half the shared memory and 256 TMEM columns, two CTAs per SM, so the
//         prologue and epilogue of short work items overlap with another item's loads.  Tiles are
//         half pages (64 keys): two 64-column S buffers and O fit the 256 columns, so Q K^T of tile
//         j + 1 still overlaps the softmax of tile j.  The barriers live in rows 16-31 of the Q
//         tile, which no real row uses.
template <bool F8, bool QUAD>
struct Cfg {
  static constexpr bool DUAL = F8 && QUAD;
  static constexpr int TK = DUAL ? 64 : 128;              // keys per tile
  static constexpr int NSUB = F8 ? 1 : 2;                 // 128-byte-wide sub-tiles per tile
  static constexpr int TILE_BYTES = NSUB * TK * 128;
  static constexpr int RING_BYTES = DUAL ? 48 * 1024 : 96 * 1024;
  static constexpr int STAGES = RING_BYTES / TILE_BYTES;  // bf16 3, e4m3 6 (dual: 6 half pages)
  static constexpr int OFF_Q = 0;
  // dual: rows 112-127 of the Q tile are never real rows, the K ring may start there
  static constexpr int OFF_K = DUAL ? SUB_BYTES - 2048 : 2 * SUB_BYTES;
  static constexpr int OFF_V = OFF_K + RING_BYTES;
  static constexpr int END = OFF_V + RING_BYTES;
  static constexpr int OFF_BAR = DUAL ? 2048 : END;
  static constexpr int SMEM_BYTES = (DUAL ? END : END + 1024) + 1024;   // + slack to align the base to 1 KB
  static constexpr int NBUF = 2;                          // S buffers in TMEM
  static constexpr int TMEM_COLS = DUAL ? 256 : 512;
  static constexpr int O_COL = NBUF * TK;
  static constexpr int MIN_CTAS = DUAL ? 2 : 1;
  static_assert(STAGES <= MAX_STAGES, "barrier table");
  static_assert(4 * QUAD_MAX_ROWS * STAGE_LD * 4 <= RING_BYTES, "O staging fits the K ring");
};

template <bool F8, bool QUAD>
__global__ void __launch_bounds__(NTHREADS, (Cfg<F8, QUAD>::MIN_CTAS))
decode_tc_kernel(const __grid_constant__ MsaFmhaParams p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  using C = Cfg<F8, QUAD>;
  constexpr int NSUB = C::NSUB, TILE_BYTES = C::TILE_BYTES, STAGES = C::STAGES, NBUF = C::NBUF, TK = C::TK;
  constexpr int UPP = BN / TK;                      // tiles per page
  constexpr int OFF_Q = C::OFF_Q, OFF_K = C::OFF_K, OFF_V = C::OFF_V, OFF_BAR = C::OFF_BAR;
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + OFF_BAR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 8);
  volatile int* skip_flag = abort_flag + 1;      // set when the status word already reports a timeout
  int* s_tiles = reinterpret_cast<int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 16);      // sparse: first key / TK of every tile, in order
  int* s_phys = s_tiles + MAX_SPARSE_TILES * UPP;                                      // ... and the physical id of its page
  int* s_ntiles = s_phys + MAX_SPARSE_TILES * UPP;
  auto bar = [&](int i) -> uint32_t { return bars + 8u * i; };
  constexpr int SUB_ELEMS = F8 ? 128 : 64;          // elements of head_dim per sub-tile
  constexpr int KSTEPS = F8 ? 4 : 8;                // MMAs per 128-deep contraction
  // e4m3 P (3 mantissa bits, largest finite value 448): written as 2^(x - m + 4) with m the running
  // max, which is raised (and O rescaled) only when it lags the true max by more than 4: P stays
  // within (0, 2^8], and what falls below e4m3's smallest subnormal (2^-9) is a weight under 2^-13
  // of the row's largest.  (Upstream uses the exact max and a 2^8 offset, fmha_common.hpp:567-570;
  // with the exact max nearly every tile of a short work item triggers an O rescale.)
  constexpr float kRescaleThreshold = F8 ? 4.0f : 8.0f;
  constexpr float kPOffset = F8 ? 4.0f : 0.0f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef MSA_DEBUG_HOOKS
  unsigned long long* trace = (threadIdx.x == 0 && g_trace) ? g_trace + 16ull * blockIdx.x : nullptr;
  const long long clk0 = clock64();
  if (trace) { trace[0] = global_ns(); unsigned id; asm("mov.u32 %0, %%smid;" : "=r"(id)); trace[2] = id; }
#else
  constexpr unsigned long long* trace = nullptr;   // the `if (trace)` records below compile to nothing
  constexpr long long clk0 = 0;
#endif
  const bool sparse = (p.flags & MSA_FLAG_SPARSE) != 0;
  const bool has_o = (p.flags & MSA_FLAG_OUT_O) != 0;   // false: score-only pass (no V, no P, no O)
  const int G = p.pack;
  const int h_r = p.num_qo_heads / p.num_kv_heads;

  // ---------------- work item ----------------
  int b, head0, tb, te, split, i_base, ntok;
  int blk_first = -1;                       // sparse: this lane's entry of the selected-page list, fetched early
  const int32_t* blocks = nullptr;
  if (!sparse) {
    const MsaWorkItem w = p.work[blockIdx.x];
    b = chk(w.batch, 0, p.batch, p.status); head0 = chk(w.head0, 0, p.num_qo_heads, p.status);
    tb = w.kv_tile_begin; te = w.kv_tile_end; split = chk(w.split, 0, p.num_splits, p.status);
    i_base = 0;
    ntok = p.qo_start[b + 1] - p.qo_start[b];
  } else {
    const int S = p.num_splits;
    int idx = blockIdx.x;
    split = idx % S; idx /= S;
    const int kvh_s = idx % p.num_kv_heads;
    const int t = idx / p.num_kv_heads;
    blocks = p.kv_block_indexes + static_cast<int64_t>(t) * p.kbi_stride_tok + static_cast<int64_t>(kvh_s) * p.kbi_stride_head;
    const int per = (p.kv_block_num + S - 1) / S;
    tb = split * per;
    te = min(p.kv_block_num, tb + per);
    // independent of the batch item: in flight together with the loads below that depend on it
    if (warp == PRODUCER_WARP && tb + lane < te) blk_first = blocks[tb + lane];
    b = chk(p.token_batch[t], 0, p.batch, p.status);
    head0 = kvh_s * h_r;
    i_base = t - p.qo_start[b];
    ntok = 1;
  }
  const int kvh = head0 / h_r;
  const int nrows = ntok * G;                                  // real rows of the 128-row tile
  const int qo_base = p.qo_start[b];
  const int kv_len = p.kv_len[b];
  const int off = p.qo_offset[b];
  const int page_base = p.kv_page_indptr[b];
  const int n_active_warps = QUAD ? 4 : (nrows + 31) / 32;

  // a timeout reported earlier on this device (status word not cleared yet): do not start.  Read by
  // another thread than the one that sets up the barriers, so the load overlaps that work.
  if (threadIdx.x == blockDim.x - 1)
    *skip_flag = (p.status != nullptr && *reinterpret_cast<const volatile int32_t*>(p.status) != 0) ? 1 : 0;
  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), F8 ? 32 * n_active_warps : 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(K_FULL + s), 1);  mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);  mbar_init(bar(V_EMPTY + s), 1);
    }
    for (int s = 0; s < NBUF; ++s) { mbar_init(bar(S_FULL + s), 1); mbar_init(bar(P_FULL + s), 32 * n_active_warps); }
    mbar_init(bar(PV_DONE), 1);
    mbar_init(bar(O_DONE), 1);
    mbar_init(bar(V_FIX), 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == PRODUCER_WARP) {
    // tile list: dense = [tb, te) of the sequence; sparse = the valid selected pages of this
    // split in list order, compacted by the whole warp, with their page-table entries
    if (sparse) {
      int n = 0;
      for (int j0 = tb; j0 < te; j0 += 32) {
        const int j = j0 + lane;
        const int blk = j0 == tb ? blk_first : (j < te ? blocks[j] : -1);
        // tiles of this page that hold a key this token may see
        int nu = 0;
        if (blk >= 0) {
          const int vis = min(kv_len, i_base + off + 1) - blk * BN;          // visible keys from the page start on
          nu = vis <= 0 ? 0 : min(UPP, (vis + TK - 1) / TK);
        }
        int incl = nu;                                         // inclusive scan over the warp
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += v;
        }
        const int pos = n + incl - nu;
        if (nu > 0 && pos + nu <= MAX_SPARSE_TILES * UPP) {
          const int ph = chk(p.kv_indices[page_base + blk], 0, static_cast<int>(p.kv_extent), p.status);
          for (int u = 0; u < nu; ++u) { s_tiles[pos + u] = blk * UPP + u; s_phys[pos + u] = ph; }
        }
        n += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) *s_ntiles = min(n, MAX_SPARSE_TILES * UPP);
    } else if (lane == 0) {
      // [tb, te) pages of the sequence, up to the last tile that holds a key
      const int keys = min(te * BN, kv_len) - tb * BN;
      *s_ntiles = keys <= 0 ? 0 : (keys + TK - 1) / TK;
    }
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_tiles = *s_ntiles;
  if (trace) trace[3] = clock64() - clk0;
  auto tile_key0 = [&](int j) -> int { return (sparse ? s_tiles[j] : tb * UPP + j) * TK; };   // position of the first key of tile j

  const bool run = *skip_flag == 0;
  if (!run) {
    // nothing: fall through to the teardown
  } else if (warp == PRODUCER_WARP || warp == V_PRODUCER_WARP) {
    // =========================== TMA producers ===========================
    // Sparse items (a few pages each): one warp for Q and K, one for V -- a single producer waits for a
    // free V stage before it may issue the next K tile, and with so few tiles that wait is exposed.
    // Long dense streams: one warp issues both (measured 4 % faster there than two warps).
    const bool do_k = warp == PRODUCER_WARP;
    const bool do_v = has_o && (sparse ? warp == V_PRODUCER_WARP : warp == PRODUCER_WARP);
    if (lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
    if (do_k && n_tiles > 0 && !F8) {                                 // e4m3: the softmax warps convert and place Q
      constexpr int COPIES = QUAD ? 4 : 1;
      if (lane == 0) mbar_arrive_expect_tx(bar(Q_FULL), COPIES * nrows * 256);
      __syncwarp();
      for (int c = lane; c < ntok * COPIES; c += 32) {       // G rows of one token per box
        const int ti = c / COPIES, quad = c % COPIES;
        const uint32_t dst = smem_base + OFF_Q + (quad * 32 + ti * G) * 128;
        tma_load_3d(dst, &tm_q, bar(Q_FULL), 0, head0, qo_base + i_base + ti);
        tma_load_3d(dst + SUB_BYTES, &tm_q, bar(Q_FULL), 64, head0, qo_base + i_base + ti);
      }
      __syncwarp();
    }
    // page-table entries: one per lane, 32 pages at a time, the next batch already in flight
    int phys_cur = 0, phys_next = 0;
    const int n_pages = (n_tiles + UPP - 1) / UPP;
    if (!sparse) {
      phys_cur = lane < n_pages ? chk(p.kv_indices[page_base + tb + lane], 0, static_cast<int>(p.kv_extent), p.status) : 0;
      phys_next = 32 + lane < n_pages ? chk(p.kv_indices[page_base + tb + 32 + lane], 0, static_cast<int>(p.kv_extent), p.status) : 0;
    }
    uint32_t fix_phase = 0;
    bool alive = do_k || do_v;
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int st = j % STAGES;
      const int key0 = tile_key0(j);
      const int row_in_page = key0 % BN;
      const int pg = j / UPP;                                // dense: page index within this item
      if (!sparse && j > 0 && (j % (32 * UPP)) == 0) {
        phys_cur = phys_next;
        phys_next = pg + 32 + lane < n_pages ? chk(p.kv_indices[page_base + tb + pg + 32 + lane], 0, static_cast<int>(p.kv_extent), p.status) : 0;
      }
      const int phys = sparse ? s_phys[j] : __shfl_sync(0xffffffffu, phys_cur, pg & 31);
      const int valid_rows = min(TK, kv_len - key0);
      const bool fix = valid_rows < TK;
      if (do_k) {
        alive = mbar_wait(bar(K_EMPTY + st), ((j / STAGES) & 1) ^ 1, abort_flag);
        if (!alive) break;
        if (elect_one()) {
          mbar_arrive_expect_tx(bar(K_FULL + st), TILE_BYTES);
#pragma unroll
          for (int hlf = 0; hlf < NSUB; ++hlf)
            tma_load_4d(smem_base + OFF_K + st * TILE_BYTES + hlf * SUB_BYTES, &tm_k, bar(K_FULL + st), hlf * SUB_ELEMS,
                        row_in_page, kvh, phys);
        }
        __syncwarp();
      }
      if (!do_v) continue;
      alive = mbar_wait(bar(V_EMPTY + st), ((j / STAGES) & 1) ^ 1, abort_flag);
      if (!alive) break;
      if (elect_one()) {
        const uint32_t vbar = fix ? bar(V_FIX) : bar(V_FULL + st);
        mbar_arrive_expect_tx(vbar, TILE_BYTES);
#pragma unroll
        for (int hlf = 0; hlf < NSUB; ++hlf)
          tma_load_4d(smem_base + OFF_V + st * TILE_BYTES + hlf * SUB_BYTES, &tm_v, vbar, hlf * SUB_ELEMS, row_in_page, kvh, phys);
      }
      __syncwarp();
      if (fix) {                                             // rows past kv_len must read as 0 in V
        alive = mbar_wait(bar(V_FIX), fix_phase, abort_flag);
        alive = __all_sync(0xffffffffu, alive);
        fix_phase ^= 1;
        if (alive) {
          unsigned char* vt = smem_gen + OFF_V + st * TILE_BYTES;
          for (int c = lane; c < (TK - valid_rows) * 8 * NSUB; c += 32) {
            const int r = valid_rows + c / (8 * NSUB), ch = c % (8 * NSUB);
            *reinterpret_cast<uint4*>(vt + (ch >> 3) * SUB_BYTES + r * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(V_FULL + st));
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer ===========================
    constexpr uint32_t IDESC_QK = F8 ? idesc_e4m3(BM, TK, false, false) : idesc_bf16(BM, TK, false, false);
    constexpr uint32_t IDESC_PV = F8 ? idesc_e4m3(BM, kHeadDim, false, true) : idesc_bf16(BM, kHeadDim, false, true);
    const uint64_t dk_hi = smem_desc(0, 16, 1024) & 0xFFFFFFFFFFFF0000ull;
    const uint64_t dv_hi = smem_desc(0, SUB_BYTES, 1024) & 0xFFFFFFFFFFFF0000ull;
    constexpr int KEYS_PER_PV = F8 ? 32 : 16;        // keys one P.V MMA contracts over
    constexpr int PV_STEPS = TK / KEYS_PER_PV;
    constexpr int V_KSTEP = KEYS_PER_PV * 128;       // bytes between the key slices of consecutive P.V MMAs
    auto sbuf = [&](int j) -> uint32_t { return tmem + (j % NBUF) * TK; };
    auto issue_qk = [&](int j) {
      const uint32_t qa = (smem_base + OFF_Q) >> 4, ka = (smem_base + OFF_K + (j % STAGES) * TILE_BYTES) >> 4;
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        const uint32_t o = ((k >> 2) * SUB_BYTES + (k & 3) * 32) >> 4;      // 32 bytes of head_dim per MMA
        if constexpr (F8) mma_ss_f8(sbuf(j), dk_hi | ((qa + o) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
        else mma_ss(sbuf(j), dk_hi | ((qa + o) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
      }
    };
    auto issue_pv = [&](int j) {
      const uint32_t va = (smem_base + OFF_V + (j % STAGES) * TILE_BYTES) >> 4;
#pragma unroll
      for (int k = 0; k < PV_STEPS; ++k) {              // P: 8 TMEM columns per MMA in both formats
        const uint64_t vd = dv_hi | ((va + k * (V_KSTEP >> 4)) & 0x3FFF);
        if constexpr (F8) mma_ts_f8(tmem + C::O_COL, sbuf(j) + k * 8, vd, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        else mma_ts(tmem + C::O_COL, sbuf(j) + k * 8, vd, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
      }
    };
    // S[j + 1] = Q K_{j+1}^T.  Two S buffers: issued before P_j V_j so it overlaps the softmax of
    // tile j.  One buffer (dual): issued after P_j V_j, which is what frees the buffer.
    auto next_qk = [&](int j, bool& alive) {
      const int st = (j + 1) % STAGES;
      alive = mbar_wait(bar(K_FULL + st), ((j + 1) / STAGES) & 1, abort_flag);
      // score-only pass: no P.V orders the reuse of the S buffer, wait for its reader instead
      if (alive && !has_o && j + 1 >= NBUF)
        alive = mbar_wait(bar(P_FULL + (j + 1) % NBUF), ((j + 1 - NBUF) / NBUF) & 1, abort_flag);
      if (!alive) return;
      tc_fence_after();
      if (elect_one()) { issue_qk(j + 1); mma_commit(bar(S_FULL + (j + 1) % NBUF)); mma_commit(bar(K_EMPTY + st)); }
      __syncwarp();
    };
    bool alive = n_tiles > 0 ? mbar_wait(bar(Q_FULL), 0, abort_flag) : true;
    if (alive && n_tiles > 0) alive = mbar_wait(bar(K_FULL + 0), 0, abort_flag);
    if (alive && n_tiles > 0) {
      tc_fence_after();
      if (elect_one()) { issue_qk(0); mma_commit(bar(S_FULL + 0)); mma_commit(bar(K_EMPTY + 0)); }
      __syncwarp();
    }
    for (int j = 0; j < n_tiles && alive; ++j) {
      if (NBUF == 2 && j + 1 < n_tiles) { next_qk(j, alive); if (!alive) break; }
      if (has_o) {
        alive = mbar_wait(bar(V_FULL + j % STAGES), (j / STAGES) & 1, abort_flag);
        if (alive) alive = mbar_wait(bar(P_FULL + j % NBUF), (j / NBUF) & 1, abort_flag);
        if (!alive) break;
        tc_fence_after();
        if (elect_one()) {
          issue_pv(j); mma_commit(bar(V_EMPTY + j % STAGES)); mma_commit(bar(PV_DONE));
          if (j == n_tiles - 1) mma_commit(bar(O_DONE));
        }
        __syncwarp();
      }
      if (NBUF == 1 && j + 1 < n_tiles) { next_qk(j, alive); if (!alive) break; }
    }
  } else if (warp < n_active_warps) {
    // =========================== softmax / epilogue ===========================
    const int trow = (warp << 5) | lane;                     // row of the MMA tile == TMEM lane
    const int r = QUAD ? lane : trow;                        // logical row of the work item
    const uint32_t lane_addr = static_cast<uint32_t>(warp << 5) << 16;
    const uint32_t tO = tmem + C::O_COL + lane_addr;
    const bool row_ok = r < nrows;
    const int i = i_base + (row_ok ? r / G : 0);
    const int head = head0 + (row_ok ? r % G : 0);
    const int gtok = qo_base + i;
    const int lim = row_ok ? min(i + off, kv_len - 1) : -1;
    const float scale_log2 = p.sm_scale * kLog2e * (p.k_scale_head ? p.k_scale_head[kvh] : 1.f);
    const bool want_score = (p.flags & MSA_FLAG_OUT_SCORE) != 0 && p.max_score != nullptr;
    float m_used = -INFINITY, l_sum = 0.f;
    bool alive = true;

    if constexpr (F8) {
      // place this row of Q in shared memory as e4m3, in the 128-byte-swizzled K-major layout
      if (n_tiles > 0) {
        uint4 chunks[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) chunks[c] = make_uint4(0, 0, 0, 0);
        if (row_ok) {
          if (p.q_dtype == MSA_DT_E4M3) {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.q) +
                                   static_cast<int64_t>(gtok) * p.q_stride_tok + static_cast<int64_t>(head) * p.q_stride_head);
#pragma unroll
            for (int c = 0; c < 8; ++c) chunks[c] = src[c];
          } else {
            const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.q) +
                                   static_cast<int64_t>(gtok) * p.q_stride_tok + static_cast<int64_t>(head) * p.q_stride_head);
#pragma unroll
            for (int c = 0; c < 8; ++c) {                     // 16 bf16 -> 16 e4m3 bytes
              const uint4 lo = src[2 * c], hi = src[2 * c + 1];
              const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
              uint32_t o[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const uint32_t a = w[2 * e], bq = w[2 * e + 1];
                const uint16_t p01 = __nv_cvt_float2_to_fp8x2(
                    make_float2(bf16_bits_to_float(a & 0xffff), bf16_bits_to_float(a >> 16)), __NV_SATFINITE, __NV_E4M3);
                const uint16_t p23 = __nv_cvt_float2_to_fp8x2(
                    make_float2(bf16_bits_to_float(bq & 0xffff), bf16_bits_to_float(bq >> 16)), __NV_SATFINITE, __NV_E4M3);
                o[e] = static_cast<uint32_t>(p01) | (static_cast<uint32_t>(p23) << 16);
              }
              chunks[c] = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
        // QUAD: only the real rows are written (rows 16-31 of the first quadrant hold the
        // barriers; what the MMA reads from unused rows only reaches unused TMEM lanes)
        if (!QUAD || row_ok) {
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(smem_gen + OFF_Q + trow * 128 + ((c ^ (trow & 7)) << 4)) = chunks[c];
        }
        fence_proxy_async_smem();
        mbar_arrive(bar(Q_FULL));
      }
    }

    if constexpr (QUAD) {
      // quadrant `warp` owns key columns [32 warp, 32 warp + 32) of every tile
      for (int j = 0; j < n_tiles && alive; ++j) {
        const uint32_t tS = tmem + (j % NBUF) * TK + lane_addr;
        alive = mbar_wait(bar(S_FULL + j % NBUF), (j / NBUF) & 1, abort_flag);
        if (!alive) break;
        if (trace && j == 12) trace[4] = clock64() - clk0;       // S of tile 12 ready
        if (trace && j == 13) trace[14] = clock64() - clk0;
        tc_fence_after();
        constexpr int CW = TK / 4;                           // key columns of a tile per quadrant
        const int pos0 = tile_key0(j) + warp * CW;
        uint32_t sv[CW];
        if constexpr (CW == 32) tmem_ld32(tS + warp * CW, sv);
        else tmem_ld16(tS + warp * CW, sv);
        tmem_wait_ld();
        if (trace && j == 12) trace[5] = clock64() - clk0;       // ... loaded
        if (pos0 + CW - 1 > lim) {
#pragma unroll
          for (int e = 0; e < CW; ++e)
            if (pos0 + e > lim) sv[e] = 0xff800000u;
        }
        float mxs[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int e = 0; e < CW; e += 2)
          mxs[(e >> 1) & 1] = max3(mxs[(e >> 1) & 1], __uint_as_float(sv[e]), __uint_as_float(sv[e + 1]));
        const float mx = fmaxf(mxs[0], mxs[1]);
        const float m_cand = fmaxf(m_used, mx * scale_log2);
        const bool bump = (m_cand - m_used) > kRescaleThreshold;
        float factor = 1.f;
        if (bump) { factor = exp2_fast(m_used - m_cand); m_used = m_cand; l_sum *= factor; }
        if (j > 0 && __any_sync(0xffffffffu, bump)) {
          alive = mbar_wait(bar(PV_DONE), (j - 1) & 1, abort_flag);
          if (!alive) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(tO + c * 32, v);
            tmem_wait_ld();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
            tmem_st32(tO + c * 32, v);
          }
        }
        const float msafe = ((m_used == -INFINITY) ? 0.f : m_used) - kPOffset;
        float l0 = 0.f, l1 = 0.f;
        if (trace && j == 12) trace[6] = clock64() - clk0;       // ... max / rescale done
        constexpr int PCOLS = F8 ? CW / 4 : CW / 2;          // TMEM columns of this quadrant's P
        uint32_t pk[PCOLS];
        if constexpr (F8) {
#pragma unroll
          for (int e = 0; e < CW; e += 4) {
            const float p0 = exp2_fast(fmaf(__uint_as_float(sv[e]), scale_log2, -msafe));
            const float p1 = exp2_fast(fmaf(__uint_as_float(sv[e + 1]), scale_log2, -msafe));
            const float p2 = exp2_fast(fmaf(__uint_as_float(sv[e + 2]), scale_log2, -msafe));
            const float p3 = exp2_fast(fmaf(__uint_as_float(sv[e + 3]), scale_log2, -msafe));
            const uint16_t lo = __nv_cvt_float2_to_fp8x2(make_float2(p0, p1), __NV_SATFINITE, __NV_E4M3);
            const uint16_t hi = __nv_cvt_float2_to_fp8x2(make_float2(p2, p3), __NV_SATFINITE, __NV_E4M3);
            const float2 ra = e4m3x2_as_float2(lo), rb = e4m3x2_as_float2(hi);
            l0 += ra.x + rb.x; l1 += ra.y + rb.y;
            pk[e >> 2] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
          }
        } else {
#pragma unroll
          for (int e = 0; e < CW; e += 2) {
            const float p0 = exp2_fast(fmaf(__uint_as_float(sv[e]), scale_log2, -msafe));
            const float p1 = exp2_fast(fmaf(__uint_as_float(sv[e + 1]), scale_log2, -msafe));
            const uint32_t pr = pack2<false>(p0, p1);
            l0 += __uint_as_float(pr << 16); l1 += __uint_as_float(pr & 0xffff0000u);
            pk[e >> 1] = pr;
          }
        }
        // P of this quadrant's rows: own keys, zero for the other three quarters of the tile
        if constexpr (PCOLS == 4) {                           // 16 columns in all: one store
          uint32_t all[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) all[c] = (c >> 2) == warp ? pk[c & 3] : 0u;
          tmem_st16(tS, all);
        } else {
          uint32_t zero[PCOLS];
#pragma unroll
          for (int e = 0; e < PCOLS; ++e) zero[e] = 0u;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            if constexpr (PCOLS == 8) { if (q == warp) tmem_st8(tS + q * PCOLS, pk); else tmem_st8(tS + q * PCOLS, zero); }
            else { if (q == warp) tmem_st16(tS + q * PCOLS, pk); else tmem_st16(tS + q * PCOLS, zero); }
          }
        }
        l_sum += l0 + l1;
        if (trace && j == 12) trace[7] = clock64() - clk0;       // ... P stored (before the wait)
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(bar(P_FULL + j % NBUF));
        if (trace && j == 12) trace[15] = clock64() - clk0;      // ... P_FULL arrived
        if (trace && j == n_tiles - 1) trace[8] = clock64() - clk0;
      }
    } else {
    for (int j = 0; j < n_tiles && alive; ++j) {
      const uint32_t tS = tmem + (j % NBUF) * TK + lane_addr;
      alive = mbar_wait(bar(S_FULL + j % NBUF), (j / NBUF) & 1, abort_flag);
      if (!alive) break;
      tc_fence_after();
      const int pos0 = tile_key0(j);
      uint32_t sv[4][32];
      tmem_ld32(tS, sv[0]);
      tmem_ld32(tS + 32, sv[1]);
      tmem_ld32(tS + 64, sv[2]);
      tmem_ld32(tS + 96, sv[3]);
      tmem_wait_ld();
      if (pos0 + BN - 1 > lim) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (pos0 + c * 32 + e > lim) sv[c][e] = 0xff800000u;
      }
      float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int e = 0; e < 32; e += 2)
          mxs[(e >> 1) & 3] = max3(mxs[(e >> 1) & 3], __uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1]));
      const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
      if (want_score && row_ok) {
        const int tile_idx = pos0 / BN;
        if (tile_idx < p.max_k_tiles) {
          const int64_t o = (static_cast<int64_t>(head) * p.max_k_tiles + tile_idx) * p.total_q + gtok;
          if (p.max_score_dtype == MSA_DT_BF16) static_cast<__nv_bfloat16*>(p.max_score)[o] = __float2bfloat16_rn(mx);
          else static_cast<float*>(p.max_score)[o] = mx;
        }
      }
      if (!has_o) {                      // score-only pass: S is consumed, hand the buffer back
        tc_fence_before();
        mbar_arrive(bar(P_FULL + j % NBUF));
        continue;
      }
      const float m_cand = fmaxf(m_used, mx * scale_log2);
      const bool bump = (m_cand - m_used) > kRescaleThreshold;
      float factor = 1.f;
      if (bump) { factor = exp2_fast(m_used - m_cand); m_used = m_cand; l_sum *= factor; }
      if (j > 0 && __any_sync(0xffffffffu, bump)) {
        // O may still be the target of P_{j-1} V_{j-1}: wait for that MMA before touching it
        alive = mbar_wait(bar(PV_DONE), (j - 1) & 1, abort_flag);
        if (!alive) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld32(tO + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * factor);
          tmem_st32(tO + c * 32, v);
        }
      }
      const float msafe = ((m_used == -INFINITY) ? 0.f : m_used) - kPOffset;
      float l0 = 0.f, l1 = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if constexpr (F8) {
          uint32_t pk[8];                                   // four e4m3 per TMEM column
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            const float p0 = exp2_fast(fmaf(__uint_as_float(sv[c][e]), scale_log2, -msafe));
            const float p1 = exp2_fast(fmaf(__uint_as_float(sv[c][e + 1]), scale_log2, -msafe));
            const float p2 = exp2_fast(fmaf(__uint_as_float(sv[c][e + 2]), scale_log2, -msafe));
            const float p3 = exp2_fast(fmaf(__uint_as_float(sv[c][e + 3]), scale_log2, -msafe));
            const uint16_t lo = __nv_cvt_float2_to_fp8x2(make_float2(p0, p1), __NV_SATFINITE, __NV_E4M3);
            const uint16_t hi = __nv_cvt_float2_to_fp8x2(make_float2(p2, p3), __NV_SATFINITE, __NV_E4M3);
            const float2 ra = e4m3x2_as_float2(lo), rb = e4m3x2_as_float2(hi);
            l0 += ra.x + rb.x; l1 += ra.y + rb.y;
            pk[e >> 2] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
          }
          tmem_st8(tS + c * 8, pk);
        } else {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = exp2_fast(fmaf(__uint_as_float(sv[c][e]), scale_log2, -msafe));
            const float p1 = exp2_fast(fmaf(__uint_as_float(sv[c][e + 1]), scale_log2, -msafe));
            const uint32_t pr = pack2<false>(p0, p1);
            l0 += __uint_as_float(pr << 16); l1 += __uint_as_float(pr & 0xffff0000u);
            pk[e >> 1] = pr;
          }
          tmem_st16(tS + c * 16, pk);
        }
      }
      l_sum += l0 + l1;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + j % NBUF));
    }

    }

    // ---- epilogue ----
    if (alive && n_tiles > 0 && has_o) alive = mbar_wait(bar(O_DONE), 0, abort_flag);
    if (trace) trace[9] = clock64() - clk0;
    if constexpr (QUAD) {
      // every MMA and every TMA load of this CTA has completed: the K ring is free to stage the
      // four partial results of each row; thread t then combines column t of every row
      float* stage = reinterpret_cast<float*>(smem_gen + OFF_K);              // [4][nrows][STAGE_LD]
      float* st_m = reinterpret_cast<float*>(smem_gen + OFF_V);               // [4][QUAD_MAX_ROWS]
      float* st_l = st_m + 4 * QUAD_MAX_ROWS;
      alive = __all_sync(0xffffffffu, alive);
      if (alive && has_o) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          if (n_tiles > 0) {
            tmem_ld32(tO + c * 32, v);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = 0u;
          }
          if (row_ok) {
            float* dst = stage + (warp * nrows + r) * STAGE_LD + c * 32;
#pragma unroll
            for (int e = 0; e < 32; e += 4)
              *reinterpret_cast<float4*>(dst + e) = make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]),
                                                                __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
          }
        }
        if (row_ok) { st_m[warp * QUAD_MAX_ROWS + r] = m_used; st_l[warp * QUAD_MAX_ROWS + r] = l_sum; }
      }
      if (trace) trace[10] = clock64() - clk0;
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (trace) trace[11] = clock64() - clk0;
      if (*abort_flag == 0 && has_o) {
        // thread -> (row, 8 columns): 16 threads per row, 8 rows per pass; the weights of a row
        // are computed once per thread
        const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;
        const bool to_partial = p.partial_o != nullptr;
        const int c8 = (trow & 15) * 8;
        for (int rr = trow >> 4; rr < nrows; rr += 8) {
          float mq[4], wq[4], M = -INFINITY, L = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) { mq[q] = st_m[q * QUAD_MAX_ROWS + rr]; M = fmaxf(M, mq[q]); }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            wq[q] = (mq[q] == -INFINITY) ? 0.f : exp2_fast(mq[q] - M);
            L += st_l[q * QUAD_MAX_ROWS + rr] * wq[q];
          }
          const float inv = L > 0.f ? __fdividef(to_partial ? vsh : p.out_scale * vsh, L) : 0.f;
          float acc[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 a0 = *reinterpret_cast<const float4*>(stage + (q * nrows + rr) * STAGE_LD + c8);
            const float4 a1 = *reinterpret_cast<const float4*>(stage + (q * nrows + rr) * STAGE_LD + c8 + 4);
            const float w = wq[q] * inv;                      // a quadrant that saw no key has weight 0 and O == 0
            acc[0] = fmaf(a0.x, w, acc[0]); acc[1] = fmaf(a0.y, w, acc[1]); acc[2] = fmaf(a0.z, w, acc[2]); acc[3] = fmaf(a0.w, w, acc[3]);
            acc[4] = fmaf(a1.x, w, acc[4]); acc[5] = fmaf(a1.y, w, acc[5]); acc[6] = fmaf(a1.z, w, acc[6]); acc[7] = fmaf(a1.w, w, acc[7]);
          }
          const int gt = qo_base + i_base + rr / G, hd = head0 + rr % G;
          const float lse = L > 0.f ? (M - kPOffset) * kLn2 + __logf(L) : -INFINITY;   // l carries 2^kPOffset
          const int64_t prow = (static_cast<int64_t>(split) * p.total_q + gt) * p.num_qo_heads + hd;
          if (to_partial) {
            float* dst = p.partial_o + prow * kHeadDim + c8;
            *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            if (c8 == 0) p.partial_lse[prow] = lse;
          } else {
            if (p.out) {
              uint4 o4;
              o4.x = pack2<false>(acc[0], acc[1]); o4.y = pack2<false>(acc[2], acc[3]);
              o4.z = pack2<false>(acc[4], acc[5]); o4.w = pack2<false>(acc[6], acc[7]);
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(gt) * p.out_stride_tok +
                                        static_cast<int64_t>(hd) * p.out_stride_head + c8) = o4;
            }
            if (c8 == 0 && p.lse) p.lse[static_cast<int64_t>(gt) * p.num_qo_heads + hd] = lse;
          }
        }
      }
      if (trace) trace[12] = clock64() - clk0;
    } else
    if (alive && has_o) {
      tc_fence_after();
      const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;
      const bool to_partial = p.partial_o != nullptr;
      const float inv = l_sum > 0.f ? (to_partial ? vsh : p.out_scale * vsh) / l_sum : 0.f;
      const float lse = l_sum > 0.f ? (m_used - kPOffset) * kLn2 + __logf(l_sum) : -INFINITY;   // l carries 2^kPOffset
      const int64_t prow = (static_cast<int64_t>(split) * p.total_q + gtok) * p.num_qo_heads + head;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (n_tiles > 0) {
          tmem_ld32(tO + c * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (!row_ok) continue;
        if (to_partial) {
          float* dst = p.partial_o + prow * kHeadDim + c * 32;
#pragma unroll
          for (int e = 0; e < 32; e += 4)
            *reinterpret_cast<float4*>(dst + e) = make_float4(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv,
                                                              __uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
        } else if (p.out) {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(gtok) * p.out_stride_tok +
                               static_cast<int64_t>(head) * p.out_stride_head + c * 32;
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 o4;
            o4.x = pack2<false>(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
            o4.y = pack2<false>(__uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
            o4.z = pack2<false>(__uint_as_float(v[e + 4]) * inv, __uint_as_float(v[e + 5]) * inv);
            o4.w = pack2<false>(__uint_as_float(v[e + 6]) * inv, __uint_as_float(v[e + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + e) = o4;
          }
        }
      }
      if (row_ok) {
        if (to_partial) p.partial_lse[prow] = lse;
        else if (p.lse) p.lse[static_cast<int64_t>(gtok) * p.num_qo_heads + head] = lse;
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0 && p.status) atomicExch(p.status, MSA_STATUS_TIMEOUT);
#ifdef MSA_DEBUG_HOOKS
  if (trace) { trace[13] = clock64() - clk0; trace[1] = global_ns(); }
#endif
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, C::TMEM_COLS);
  }
}

}  // namespace
}  // namespace decode_tc

// bf16 or e4m3 cache with 128-key pages; every work item's rows fit one 128-row tile; either O
// (optionally as split partials) or, for the proxy pass, the per-page max score alone
int fmha_decode_tc_supported(const MsaFmhaParams& p) {
  const bool has_o = (p.flags & MSA_FLAG_OUT_O) != 0, has_s = (p.flags & MSA_FLAG_OUT_SCORE) != 0;
  if (has_o == has_s) return 0;                                  // O + score together stays on the generic kernel
  if (p.page_size != decode_tc::BN) return 0;
  if (p.kv_dtype == MSA_DT_BF16) { if (p.q_dtype != MSA_DT_BF16) return 0; }
  else if (p.kv_dtype != MSA_DT_E4M3) return 0;
  if (p.block_m != 16 && p.block_m != 64 && p.block_m != 128) return 0;
  const int h_r = p.num_qo_heads / p.num_kv_heads;
  if (p.pack != h_r || p.pack > 128 || (128 % p.pack) != 0) return 0;
  if (p.decode_rows <= 0 || p.decode_rows > 128) return 0;       // 0: caller does not want this kernel
  if ((p.flags & MSA_FLAG_SPARSE) && p.kv_block_num > decode_tc::MAX_SPARSE_TILES) return 0;
  return 1;
}

int fmha_decode_tc_launch(const MsaFmhaParams& p, cudaStream_t stream) {
  using namespace decode_tc;
  const bool sparse = (p.flags & MSA_FLAG_SPARSE) != 0;
  const bool has_o = (p.flags & MSA_FLAG_OUT_O) != 0;
  const bool f8 = p.kv_dtype == MSA_DT_E4M3;
  const int64_t grid64 = sparse ? static_cast<int64_t>(p.total_q) * p.num_kv_heads * p.num_splits : p.num_work;
  if (grid64 <= 0) return MSA_OK;
  if (grid64 > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  CUtensorMap tq, tk, tv;
  const uint64_t e = f8 ? 1 : 2;
  // the 4-way column split needs O (its quadrants do not share a row max) and <= 16 rows
  const bool quad = has_o && p.decode_rows <= QUAD_MAX_ROWS;
  {
    const uint64_t kd[4] = {128, BN, static_cast<uint64_t>(p.num_kv_heads), static_cast<uint64_t>(p.kv_extent)};
    const uint64_t ks[3] = {static_cast<uint64_t>(p.k_stride_tok) * e, static_cast<uint64_t>(p.k_stride_head) * e,
                            static_cast<uint64_t>(p.k_stride_page) * e};
    const uint64_t vs[3] = {static_cast<uint64_t>(p.v_stride_tok) * e, static_cast<uint64_t>(p.v_stride_head) * e,
                            static_cast<uint64_t>(p.v_stride_page) * e};
    const void* vptr = has_o ? p.v : p.k;
    if (f8) {
      const uint32_t kbox[4] = {128, static_cast<uint32_t>(quad ? Cfg<true, true>::TK : BN), 1, 1};   // dual: half pages
      if (make_tma_map_u8(&tk, p.k, 4, kd, ks, kbox) != MSA_OK ||
          make_tma_map_u8(&tv, vptr, 4, kd, has_o ? vs : ks, kbox) != MSA_OK)
        return MSA_ERR_LAUNCH;
      tq = tk;                                                   // Q is placed by the softmax warps
    } else {
      const uint64_t dims[3] = {128, static_cast<uint64_t>(p.num_qo_heads), static_cast<uint64_t>(p.total_q)};
      const uint64_t str[2] = {static_cast<uint64_t>(p.q_stride_head) * 2, static_cast<uint64_t>(p.q_stride_tok) * 2};
      const uint32_t box[3] = {64, static_cast<uint32_t>(p.pack), 1};
      if (make_tma_map_bf16(&tq, p.q, 3, dims, str, box) != MSA_OK) return MSA_ERR_LAUNCH;
      const uint32_t kbox[4] = {64, BN, 1, 1};
      if (make_tma_map_bf16(&tk, p.k, 4, kd, ks, kbox) != MSA_OK ||
          make_tma_map_bf16(&tv, vptr, 4, kd, has_o ? vs : ks, kbox) != MSA_OK)
        return MSA_ERR_LAUNCH;
    }
  }
  static bool attr_done[16][4] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  using Kern = void (*)(const MsaFmhaParams, const CUtensorMap, const CUtensorMap, const CUtensorMap);
  const int variant = (f8 ? 2 : 0) | (quad ? 1 : 0);
  Kern kern;
  int smem;
  switch (variant) {
    case 0: kern = decode_tc_kernel<false, false>; smem = Cfg<false, false>::SMEM_BYTES; break;
    case 1: kern = decode_tc_kernel<false, true>;  smem = Cfg<false, true>::SMEM_BYTES;  break;
    case 2: kern = decode_tc_kernel<true, false>;  smem = Cfg<true, false>::SMEM_BYTES;  break;
    default: kern = decode_tc_kernel<true, true>;  smem = Cfg<true, true>::SMEM_BYTES;   break;
  }
  if (dev >= 16 || !attr_done[dev][variant]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return MSA_ERR_LAUNCH;
    if (variant == 3)      // two co-resident CTAs need the whole shared-memory carve-out
      cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (dev < 16) attr_done[dev][variant] = true;
  }
  kern<<<static_cast<unsigned>(grid64), NTHREADS, smem, stream>>>(p, tq, tk, tv);
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

// CTAs of one decode-kernel variant that fit an SM (what the occupancy calculator reports).
int fmha_decode_tc_occupancy(int f8, int quad) {
  using namespace decode_tc;
  int n = 0;
  cudaError_t e;
  if (f8 && quad) {
    cudaFuncSetAttribute(decode_tc_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<true, true>::SMEM_BYTES);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_tc_kernel<true, true>, NTHREADS, Cfg<true, true>::SMEM_BYTES);
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, decode_tc_kernel<true, true>) == cudaSuccess)
      fprintf(stderr, "decode_tc_kernel<e4m3, quad>: regs %d static smem %zu dyn smem %d local %zu max threads %d\n", fa.numRegs,
              fa.sharedSizeBytes, Cfg<true, true>::SMEM_BYTES, fa.localSizeBytes, fa.maxThreadsPerBlock);
  } else if (f8) {
    cudaFuncSetAttribute(decode_tc_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<true, false>::SMEM_BYTES);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_tc_kernel<true, false>, NTHREADS, Cfg<true, false>::SMEM_BYTES);
  } else if (quad) {
    cudaFuncSetAttribute(decode_tc_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<false, true>::SMEM_BYTES);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_tc_kernel<false, true>, NTHREADS, Cfg<false, true>::SMEM_BYTES);
  } else {
    cudaFuncSetAttribute(decode_tc_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg<false, false>::SMEM_BYTES);
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, decode_tc_kernel<false, false>, NTHREADS, Cfg<false, false>::SMEM_BYTES);
  }
  return e == cudaSuccess ? n : -1;
}

}  // namespace msa

#ifdef MSA_DEBUG_HOOKS
// Diagnostics of builds with -DMSA_DEBUG_HOOKS only.
// resident CTAs per SM of a decode-kernel variant
extern "C" int msa_debug_decode_occupancy(int f8, int quad) { return msa::fmha_decode_tc_occupancy(f8, quad); }

// device buffer of 16 x uint64 per CTA, or NULL to stop
// [0] start ns  [1] end ns  [2] SM id; clocks since entry: [3] prologue done, [4..7], [14], [15] steps of
// tile 12 / 13 in the softmax (S ready, loaded, max done, P stored, S of 13 ready, P_FULL arrived), [8] last P written, [9] last P.V done, [10] O staged, [11] staging barrier passed,
// [12] rows combined and stored, [13] exit
extern "C" void msa_debug_decode_trace(unsigned long long* device_buf) {
  cudaMemcpyToSymbol(msa::decode_tc::g_trace, &device_buf, sizeof(device_buf));
}
#endif
