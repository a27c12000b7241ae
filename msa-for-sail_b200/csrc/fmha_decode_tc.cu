// Decode / short-query attention on tcgen05, sized for HBM bandwidth.
//
// Serves the q_len * (Hq/Hkv) <= 128 shapes of `fmha_sail` over a bf16 or e4m3 paged cache with
// 128-key pages (e4m3: kind::f8f6f4 MMAs, Q and P converted to e4m3, P offset by 2^8): dense paged decode with split-KV (upstream dense mainloop + pack-GQA,
// csrc/include/sm80_fmha_fwd_mainloop.hpp:262-636, api.py:308-318) and per-token sparse decode
// over kv_block_indexes (csrc/include/sm80_fmha_sparse_fwd_mainloop.hpp:249-601).
//
// A decode step reads every selected K/V byte once and does ~16 FLOP per byte, so what matters
// is keeping loads in flight.  One CTA = one (batch item | token, KV head, split).  Its rows are
// the packed (token, head-in-group) pairs; they occupy the first lanes of a 128-row MMA tile (the
// idle rows cost tensor time that is not on the critical path).  K and V pages stream through
// 3-deep TMA rings (192 KB in flight per SM); no thread ever computes a load address.
//
//   warps 0-3   softmax: only the warps that own real rows take part; thread r owns row r
//   warp 4      TMA producer (page id read from the page table / the selected-page list)
//   warp 5      MMA issuer: S[j & 1] = Q K_j^T, O += P_j V_j; S is double-buffered in TMEM so
//               QK of tile j + 1 overlaps the softmax of tile j
//
// Output: normalised partial O (fp32) + natural-log LSE per split, or the final bf16 O when the
// work item is unsplit.  Every wait is bounded (tc_ptx.cuh).
#include "tc_ptx.cuh"

namespace msa {
int make_tma_map_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box);
int make_tma_map_u8(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box);

namespace decode_tc {
namespace {

using namespace tc;

constexpr int BM = 128, BN = 128;
constexpr int SUB_BYTES = BM * 128;             // one [128 rows][128 bytes] swizzled sub-tile
constexpr int RING_BYTES = 96 * 1024;           // per operand: 3 bf16 tiles or 6 e4m3 tiles
constexpr int OFF_Q = 0;
constexpr int OFF_K = 2 * SUB_BYTES;
constexpr int OFF_V = OFF_K + RING_BYTES;
constexpr int OFF_BAR = OFF_V + RING_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + 1024 + 1024;
constexpr int NTHREADS = 192;
constexpr int PRODUCER_WARP = 4, MMA_WARP = 5;
constexpr int MAX_SPARSE_TILES = 64;
constexpr int MAX_STAGES = 6;

enum Bar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 7, V_FULL = 13, V_EMPTY = 19, S_FULL = 25, P_FULL = 27, PV_DONE = 29,
           V_FIX = 30, NUM_BARS = 31 };

// F8: K/V (and Q, P) are e4m3 and the MMAs are kind::f8f6f4; otherwise bf16 and kind::f16.
template <bool F8>
__global__ void __launch_bounds__(NTHREADS, 1)
decode_tc_kernel(const __grid_constant__ MsaFmhaParams p, const __grid_constant__ CUtensorMap tm_q,
                 const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
  extern __shared__ unsigned char smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  unsigned char* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bars = smem_base + OFF_BAR;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem_gen + OFF_BAR + NUM_BARS * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 8);
  int* s_tiles = reinterpret_cast<int*>(smem_gen + OFF_BAR + NUM_BARS * 8 + 16);      // sparse: valid pages, in order
  int* s_ntiles = s_tiles + MAX_SPARSE_TILES;
  auto bar = [&](int i) -> uint32_t { return bars + 8u * i; };
  constexpr int NSUB = F8 ? 1 : 2;                 // 128-byte-wide sub-tiles per 128 x 128 tile
  constexpr int TILE_BYTES = NSUB * SUB_BYTES;
  constexpr int STAGES = RING_BYTES / TILE_BYTES;
  constexpr int SUB_ELEMS = F8 ? 128 : 64;          // elements of head_dim per sub-tile
  constexpr int KSTEPS = F8 ? 4 : 8;                // MMAs per 128-deep contraction
  // e4m3 P has 3 mantissa bits: keep it in (2^-6, 2^8] by using the exact running max (no lazy
  // rescale) and a 2^8 offset, the same trick as the upstream e4m3 path
  // (csrc/include/fmha_common.hpp:567-570)
  constexpr float kRescaleThreshold = F8 ? 0.0f : 8.0f;
  constexpr float kPOffset = F8 ? 8.0f : 0.0f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool sparse = (p.flags & MSA_FLAG_SPARSE) != 0;
  const bool has_o = (p.flags & MSA_FLAG_OUT_O) != 0;   // false: score-only pass (no V, no P, no O)
  const int G = p.pack;
  const int h_r = p.num_qo_heads / p.num_kv_heads;

  // ---------------- work item ----------------
  int b, head0, tb, te, split, i_base, ntok;
  const int32_t* blocks = nullptr;
  if (!sparse) {
    const MsaWorkItem w = p.work[blockIdx.x];
    b = w.batch; head0 = w.head0; tb = w.kv_tile_begin; te = w.kv_tile_end; split = w.split;
    i_base = 0;
    ntok = p.qo_start[b + 1] - p.qo_start[b];
  } else {
    const int S = p.num_splits;
    int idx = blockIdx.x;
    split = idx % S; idx /= S;
    const int kvh_s = idx % p.num_kv_heads;
    const int t = idx / p.num_kv_heads;
    b = p.token_batch[t];
    head0 = kvh_s * h_r;
    i_base = t - p.qo_start[b];
    ntok = 1;
    blocks = p.kv_block_indexes + static_cast<int64_t>(t) * p.kbi_stride_tok + static_cast<int64_t>(kvh_s) * p.kbi_stride_head;
    const int per = (p.kv_block_num + S - 1) / S;
    tb = split * per;
    te = min(p.kv_block_num, tb + per);
  }
  const int kvh = head0 / h_r;
  const int nrows = ntok * G;                                  // real rows of the 128-row tile
  const int qo_base = p.qo_start[b];
  const int kv_len = p.kv_len[b];
  const int off = p.qo_offset[b];
  const int page_base = p.kv_page_indptr[b];
  const int n_active_warps = (nrows + 31) / 32;

  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), F8 ? 32 * n_active_warps : 1);
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(K_FULL + s), 1);  mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);  mbar_init(bar(V_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) { mbar_init(bar(S_FULL + s), 1); mbar_init(bar(P_FULL + s), 32 * n_active_warps); }
    mbar_init(bar(PV_DONE), 1);
    mbar_init(bar(V_FIX), 1);
    *abort_flag = 0;
    mbar_fence_init();
    // tile list: dense = [tb, te) of the sequence; sparse = the valid selected pages of this split
    if (sparse) {
      int n = 0;
      const int i_tok = i_base;
      for (int j = tb; j < te && n < MAX_SPARSE_TILES; ++j) {
        const int blk = blocks[j];
        if (blk >= 0 && blk * BN < kv_len && blk * BN <= i_tok + off) s_tiles[n++] = blk;
      }
      *s_ntiles = n;
    } else {
      *s_ntiles = max(0, te - tb);
    }
  }
  if (warp == MMA_WARP) {
    tmem_alloc(smem_u32(tmem_slot), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const int n_tiles = *s_ntiles;
  auto tile_page = [&](int j) -> int { return sparse ? s_tiles[j] : tb + j; };     // logical page of tile j

  if (warp == PRODUCER_WARP) {
    // =========================== TMA producer ===========================
    if (lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
    if (n_tiles > 0 && !F8) {                                 // e4m3: the softmax warps convert and place Q
      if (lane == 0) mbar_arrive_expect_tx(bar(Q_FULL), nrows * 256);
      __syncwarp();
      for (int ti = lane; ti < ntok; ti += 32) {             // G rows of one token per box
        const uint32_t dst = smem_base + OFF_Q + ti * G * 128;
        tma_load_3d(dst, &tm_q, bar(Q_FULL), 0, head0, qo_base + i_base + ti);
        tma_load_3d(dst + SUB_BYTES, &tm_q, bar(Q_FULL), 64, head0, qo_base + i_base + ti);
      }
      __syncwarp();
    }
    uint32_t fix_phase = 0;
    bool alive = true;
    for (int j = 0; j < n_tiles && alive; ++j) {
      const int st = j % STAGES;
      const int lp = tile_page(j);
      const int phys = p.kv_indices[page_base + lp];
      const int valid_rows = min(BN, kv_len - lp * BN);
      const bool fix = valid_rows < BN;
      alive = mbar_wait(bar(K_EMPTY + st), ((j / STAGES) & 1) ^ 1, abort_flag);
      if (!alive) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(bar(K_FULL + st), TILE_BYTES);
#pragma unroll
        for (int hlf = 0; hlf < NSUB; ++hlf)
          tma_load_4d(smem_base + OFF_K + st * TILE_BYTES + hlf * SUB_BYTES, &tm_k, bar(K_FULL + st), hlf * SUB_ELEMS, 0,
                      kvh, phys);
      }
      __syncwarp();
      if (!has_o) continue;
      alive = mbar_wait(bar(V_EMPTY + st), ((j / STAGES) & 1) ^ 1, abort_flag);
      if (!alive) break;
      if (elect_one()) {
        const uint32_t vbar = fix ? bar(V_FIX) : bar(V_FULL + st);
        mbar_arrive_expect_tx(vbar, TILE_BYTES);
#pragma unroll
        for (int hlf = 0; hlf < NSUB; ++hlf)
          tma_load_4d(smem_base + OFF_V + st * TILE_BYTES + hlf * SUB_BYTES, &tm_v, vbar, hlf * SUB_ELEMS, 0, kvh, phys);
      }
      __syncwarp();
      if (fix) {                                             // rows past kv_len must read as 0 in V
        alive = mbar_wait(bar(V_FIX), fix_phase, abort_flag);
        alive = __all_sync(0xffffffffu, alive);
        fix_phase ^= 1;
        if (alive) {
          unsigned char* vt = smem_gen + OFF_V + st * TILE_BYTES;
          for (int c = lane; c < (BN - valid_rows) * 8 * NSUB; c += 32) {
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
    constexpr uint32_t IDESC_QK = F8 ? idesc_e4m3(BM, BN, false, false) : idesc_bf16(BM, BN, false, false);
    constexpr uint32_t IDESC_PV = F8 ? idesc_e4m3(BM, kHeadDim, false, true) : idesc_bf16(BM, kHeadDim, false, true);
    const uint64_t dk_hi = smem_desc(0, 16, 1024) & 0xFFFFFFFFFFFF0000ull;
    const uint64_t dv_hi = smem_desc(0, SUB_BYTES, 1024) & 0xFFFFFFFFFFFF0000ull;
    constexpr int V_KSTEP = (BN / KSTEPS) * 128;     // bytes between the key slices of consecutive P.V MMAs
    auto issue_qk = [&](int j) {
      const uint32_t qa = (smem_base + OFF_Q) >> 4, ka = (smem_base + OFF_K + (j % STAGES) * TILE_BYTES) >> 4;
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        const uint32_t o = ((k >> 2) * SUB_BYTES + (k & 3) * 32) >> 4;      // 32 bytes of head_dim per MMA
        if constexpr (F8) mma_ss_f8(tmem + (j & 1) * BN, dk_hi | ((qa + o) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
        else mma_ss(tmem + (j & 1) * BN, dk_hi | ((qa + o) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
      }
    };
    auto issue_pv = [&](int j) {
      const uint32_t va = (smem_base + OFF_V + (j % STAGES) * TILE_BYTES) >> 4;
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {                // P: 8 TMEM columns per MMA in both formats
        const uint64_t vd = dv_hi | ((va + k * (V_KSTEP >> 4)) & 0x3FFF);
        if constexpr (F8) mma_ts_f8(tmem + 256, tmem + (j & 1) * BN + k * 8, vd, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        else mma_ts(tmem + 256, tmem + (j & 1) * BN + k * 8, vd, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
      }
    };
    bool alive = n_tiles > 0 ? mbar_wait(bar(Q_FULL), 0, abort_flag) : true;
    if (alive && n_tiles > 0) alive = mbar_wait(bar(K_FULL + 0), 0, abort_flag);
    if (alive && n_tiles > 0) {
      tc_fence_after();
      if (elect_one()) { issue_qk(0); mma_commit(bar(S_FULL + 0)); mma_commit(bar(K_EMPTY + 0)); }
      __syncwarp();
    }
    for (int j = 0; j < n_tiles && alive; ++j) {
      if (j + 1 < n_tiles) {                                 // S[(j+1)&1] = Q K_{j+1}^T while tile j is in softmax
        const int st = (j + 1) % STAGES;
        alive = mbar_wait(bar(K_FULL + st), ((j + 1) / STAGES) & 1, abort_flag);
        // score-only pass: no P.V orders the reuse of the S buffer, wait for its reader instead
        if (alive && !has_o && j >= 1) alive = mbar_wait(bar(P_FULL + ((j + 1) & 1)), ((j - 1) >> 1) & 1, abort_flag);
        if (!alive) break;
        tc_fence_after();
        if (elect_one()) { issue_qk(j + 1); mma_commit(bar(S_FULL + ((j + 1) & 1))); mma_commit(bar(K_EMPTY + st)); }
        __syncwarp();
      }
      if (!has_o) continue;
      alive = mbar_wait(bar(V_FULL + j % STAGES), (j / STAGES) & 1, abort_flag);
      if (alive) alive = mbar_wait(bar(P_FULL + (j & 1)), (j >> 1) & 1, abort_flag);
      if (!alive) break;
      tc_fence_after();
      if (elect_one()) { issue_pv(j); mma_commit(bar(V_EMPTY + j % STAGES)); mma_commit(bar(PV_DONE)); }
      __syncwarp();
    }
  } else if (warp < n_active_warps) {
    // =========================== softmax / epilogue ===========================
    const int r = (warp << 5) | lane;                        // row == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>(warp << 5) << 16;
    const uint32_t tO = tmem + 256 + lane_addr;
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
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(smem_gen + OFF_Q + r * 128 + ((c ^ (r & 7)) << 4)) = chunks[c];
        fence_proxy_async_smem();
        mbar_arrive(bar(Q_FULL));
      }
    }

    for (int j = 0; j < n_tiles && alive; ++j) {
      const uint32_t tS = tmem + (j & 1) * BN + lane_addr;
      alive = mbar_wait(bar(S_FULL + (j & 1)), (j >> 1) & 1, abort_flag);
      if (!alive) break;
      tc_fence_after();
      const int pos0 = tile_page(j) * BN;
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
        mbar_arrive(bar(P_FULL + (j & 1)));
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
            l0 += p0 + p2; l1 += p1 + p3;
            const uint16_t lo = __nv_cvt_float2_to_fp8x2(make_float2(p0, p1), __NV_SATFINITE, __NV_E4M3);
            const uint16_t hi = __nv_cvt_float2_to_fp8x2(make_float2(p2, p3), __NV_SATFINITE, __NV_E4M3);
            pk[e >> 2] = static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
          }
          tmem_st8(tS + c * 8, pk);
        } else {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float p0 = exp2_fast(fmaf(__uint_as_float(sv[c][e]), scale_log2, -msafe));
            const float p1 = exp2_fast(fmaf(__uint_as_float(sv[c][e + 1]), scale_log2, -msafe));
            l0 += p0; l1 += p1;
            pk[e >> 1] = pack2<false>(p0, p1);
          }
          tmem_st16(tS + c * 16, pk);
        }
      }
      l_sum += l0 + l1;
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + (j & 1)));
    }

    // ---- epilogue ----
    if (alive && n_tiles > 0 && has_o) alive = mbar_wait(bar(PV_DONE), (n_tiles - 1) & 1, abort_flag);
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
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
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
  {
    const uint64_t kd[4] = {128, BN, static_cast<uint64_t>(p.num_kv_heads), static_cast<uint64_t>(p.kv_extent)};
    const uint64_t ks[3] = {static_cast<uint64_t>(p.k_stride_tok) * e, static_cast<uint64_t>(p.k_stride_head) * e,
                            static_cast<uint64_t>(p.k_stride_page) * e};
    const uint64_t vs[3] = {static_cast<uint64_t>(p.v_stride_tok) * e, static_cast<uint64_t>(p.v_stride_head) * e,
                            static_cast<uint64_t>(p.v_stride_page) * e};
    const void* vptr = has_o ? p.v : p.k;
    if (f8) {
      const uint32_t kbox[4] = {128, BN, 1, 1};
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
  static bool attr_done[16][2] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = f8 ? decode_tc_kernel<true> : decode_tc_kernel<false>;
  if (dev >= 16 || !attr_done[dev][f8]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess)
      return MSA_ERR_LAUNCH;
    if (dev < 16) attr_done[dev][f8] = true;
  }
  kern<<<static_cast<unsigned>(grid64), NTHREADS, SMEM_BYTES, stream>>>(p, tq, tk, tv);
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

}  // namespace msa
