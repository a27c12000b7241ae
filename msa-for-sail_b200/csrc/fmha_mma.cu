// Generic FMHA forward for sm_100a built on warp-level mma.sync tiles.
//
// One kernel template covers every mode of the upstream `fmha_sail` run call
// (api.py:1394-1440): dense ragged / dense paged / sparse-by-page-list, O and/or per-tile
// max-score output, bf16 or e4m3 operands, optional split-KV partial output.  It is the
// functional backbone; the tcgen05 kernels take over the shapes they are specialised for.
//
// Work decomposition: one CTA = one work item = BLOCK_M packed rows of one (batch item, head
// group).  A packed row r stands for (token r / pack, head head0 + r % pack) -- with pack =
// Hq/Hkv the query heads that share a KV head fill the MMA M dimension (what upstream calls
// pack-GQA, api.py:308-318).  KV is walked in tiles of 128 keys through a cp.async ring.
//
// Warp layout <MW, NW>: MW warps along rows (16 rows each), NW warps along the keys of a
// tile (128/NW keys each, every warp keeping its own online-softmax state that is merged in
// the epilogue).  <8,1> and <4,1> serve prefill, <1,4> serves decode / per-token sparse.
#include "common.cuh"

namespace msa {
namespace {

struct TileSrc {
  int pos0;     // original position of the tile's first key
  bool valid;   // false: nothing to load, every key masked
  int lpage;    // sparse: logical page
};

template <int MW, int NW, bool HAS_O, bool KV8>
struct Cfg {
  static constexpr int BM = 16 * MW;
  static constexpr int NT = 32 * MW * NW;
  static constexpr int BNW = kKvTile / NW;           // keys per warp per tile
  static constexpr int STAGES = (MW == 1) ? 3 : 2;
  static constexpr int KV_ELT = KV8 ? 1 : 2;
  static constexpr int TILE_BYTES = kKvTile * kHeadDim * KV_ELT;      // raw K (or V) tile
  static constexpr int STAGE_BYTES = TILE_BYTES * (HAS_O ? 2 : 1);
  static constexpr int Q_BYTES = BM * kHeadDim * 2;
  static constexpr int CVT_BYTES = KV8 ? (kKvTile * kHeadDim * 2) * (HAS_O ? 2 : 1) : 0;
  static constexpr int MERGE_BYTES = (NW > 1) ? (NW * 16 * (kHeadDim + 2) * 4) : 0;
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES + CVT_BYTES;
  static constexpr int SMEM = Q_BYTES + (RING_BYTES > MERGE_BYTES ? RING_BYTES : MERGE_BYTES) + 1024;
};

template <int MW, int NW, bool HAS_O, bool KV8>
__global__ void __launch_bounds__(32 * MW * NW, 1)
fmha_mma_kernel(const __grid_constant__ MsaFmhaParams p) {
  using C = Cfg<MW, NW, HAS_O, KV8>;
  constexpr bool HF = KV8;                      // e4m3 K/V are widened to fp16, else bf16 math
  constexpr int BM = C::BM, NT = C::NT, BNW = C::BNW, STAGES = C::STAGES;
  constexpr int NTILE_S = BNW / 8;              // n-tiles of S per warp
  constexpr int KSTEP_PV = BNW / 16;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  unsigned char* sQ = smem;
  unsigned char* sRing = smem + C::Q_BYTES;
  unsigned char* sCvt = sRing + STAGES * C::STAGE_BYTES;   // fp16 copies of the current tile (KV8)
  __shared__ float s_rowmax[NW > 1 ? NW : 1][16];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int wm = warp / NW, wn = warp % NW;
  const bool sparse = (p.flags & MSA_FLAG_SPARSE) != 0;
  const bool want_score = (p.flags & MSA_FLAG_OUT_SCORE) != 0 && p.max_score != nullptr;
  const int G = p.pack;
  const int h_r = p.num_qo_heads / p.num_kv_heads;

  // ---------------- item ----------------
  int b, head0, row0, tb, te, split, i_base, rows_total;   // rows_total: one past the item's last packed row
  const int32_t* blocks = nullptr;
  if (!sparse) {
    if (static_cast<int>(blockIdx.x) >= p.num_work) return;
    const MsaWorkItem w = p.work[blockIdx.x];
    b = chk(w.batch, 0, p.batch, p.status); head0 = chk(w.head0, 0, p.num_qo_heads, p.status); row0 = w.row0;
    tb = w.kv_tile_begin; te = w.kv_tile_end; split = chk(w.split, 0, p.num_splits, p.status);
    i_base = 0;
    rows_total = min((p.qo_start[b + 1] - p.qo_start[b]) * G, w.row0 + w.num_rows);
  } else {
    const int S = p.num_splits;
    int idx = blockIdx.x;
    split = idx % S; idx /= S;
    const int kvh_s = idx % p.num_kv_heads;
    const int t = idx / p.num_kv_heads;
    if (t >= p.total_q) return;
    b = chk(p.token_batch[t], 0, p.batch, p.status);
    head0 = kvh_s * h_r; row0 = 0; rows_total = G;
    i_base = t - p.qo_start[b];
    blocks = p.kv_block_indexes + static_cast<int64_t>(t) * p.kbi_stride_tok + static_cast<int64_t>(kvh_s) * p.kbi_stride_head;
    const int per = (p.kv_block_num + S - 1) / S;
    tb = split * per;
    te = min(p.kv_block_num, tb + per);
  }
  const int kvh = head0 / h_r;
  const int qo_base = p.qo_start[b];
  const int kv_len = p.kv_len[b];
  const int off = p.qo_offset[b];
  const int page_base = p.page_size > 0 ? p.kv_page_indptr[b] : 0;
  const int kv_base = p.page_size > 0 ? 0 : p.kv_start[b];
  const int ps = p.page_size;

  float scale_log2 = p.sm_scale * kLog2e;
  if (p.k_scale_head) scale_log2 *= p.k_scale_head[kvh];

  // ---------------- Q tile -> shared (compute type) ----------------
  {
    const bool q8 = p.q_dtype == MSA_DT_E4M3;
    for (int c = tid; c < BM * 16; c += NT) {
      const int r = c >> 4, ch = c & 15;
      const int pr = row0 + r;
      const bool ok = pr < rows_total;
      const int i = i_base + (ok ? pr / G : 0);
      const int head = head0 + (ok ? pr % G : 0);
      const int64_t base = static_cast<int64_t>(qo_base + i) * p.q_stride_tok + static_cast<int64_t>(head) * p.q_stride_head + ch * 8;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (ok) {
        if (q8) {
          const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(p.q) + base);
          val.x = cvt_e4m3x2<HF>(raw.x & 0xffff); val.y = cvt_e4m3x2<HF>(raw.x >> 16);
          val.z = cvt_e4m3x2<HF>(raw.y & 0xffff); val.w = cvt_e4m3x2<HF>(raw.y >> 16);
        } else {
          val = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.q) + base);
          if constexpr (HF) {   // bf16 -> fp16 for the fp16 MMA used with e4m3 K/V
            uint32_t* w4 = reinterpret_cast<uint32_t*>(&val);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float lo = bf16_bits_to_float(w4[e] & 0xffff), hi = bf16_bits_to_float(w4[e] >> 16);
              w4[e] = pack2<true>(lo, hi);
            }
          }
        }
      }
      *reinterpret_cast<uint4*>(sQ + swz_off(r, ch)) = val;
    }
  }

  // ---------------- tile source + loader ----------------
  auto tile_src = [&](int j) -> TileSrc {
    TileSrc s;
    if (!sparse) { s.pos0 = j * kKvTile; s.valid = true; s.lpage = 0; return s; }
    const int blk = blocks[j];
    s.lpage = blk;
    s.pos0 = blk * kKvTile;
    s.valid = blk >= 0 && s.pos0 < kv_len;
    return s;
  };

  constexpr int CH_PER_ROW = KV8 ? 8 : 16;          // 16-byte chunks per key row
  auto load_tile = [&](int stage, int j) {
    const TileSrc s = tile_src(j);
    unsigned char* dK = sRing + stage * C::STAGE_BYTES;
    unsigned char* dV = dK + C::TILE_BYTES;
    for (int c = tid; c < kKvTile * CH_PER_ROW; c += NT) {
      const int r = c / CH_PER_ROW, ch = c % CH_PER_ROW;
      const int pos = s.pos0 + r;
      const bool ok = s.valid && pos < kv_len;
      int64_t ko = 0, vo = 0;
      if (ok) {
        if (ps > 0) {
          const int lp = sparse ? s.lpage : pos / ps;
          const int in_page = sparse ? r : pos - lp * ps;
          const int64_t pg = chk(p.kv_indices[page_base + lp], 0, static_cast<int>(p.kv_extent), p.status);
          ko = pg * p.k_stride_page + static_cast<int64_t>(kvh) * p.k_stride_head + static_cast<int64_t>(in_page) * p.k_stride_tok;
          vo = pg * p.v_stride_page + static_cast<int64_t>(kvh) * p.v_stride_head + static_cast<int64_t>(in_page) * p.v_stride_tok;
        } else {
          ko = static_cast<int64_t>(kv_base + pos) * p.k_stride_tok + static_cast<int64_t>(kvh) * p.k_stride_head;
          vo = static_cast<int64_t>(kv_base + pos) * p.v_stride_tok + static_cast<int64_t>(kvh) * p.v_stride_head;
        }
      }
      if constexpr (KV8) {
        const uint32_t d = r * 128 + ch * 16;        // raw bytes, converted later
        cp_async16(smem_u32(dK + d), static_cast<const uint8_t*>(p.k) + ko + ch * 16, ok);
        if constexpr (HAS_O) cp_async16(smem_u32(dV + d), static_cast<const uint8_t*>(p.v) + vo + ch * 16, ok);
      } else {
        const uint32_t d = swz_off(r, ch);
        cp_async16(smem_u32(dK + d), static_cast<const __nv_bfloat16*>(p.k) + ko + ch * 8, ok);
        if constexpr (HAS_O) cp_async16(smem_u32(dV + d), static_cast<const __nv_bfloat16*>(p.v) + vo + ch * 8, ok);
      }
    }
  };

  // ---------------- per-thread row bookkeeping ----------------
  const int r_lo = wm * 16 + (lane >> 2), r_hi = r_lo + 8;
  int lim[2], gtok[2], headr[2];
  bool rowok[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const int pr = row0 + (e ? r_hi : r_lo);
    rowok[e] = pr < rows_total;
    const int i = i_base + (rowok[e] ? pr / G : 0);
    headr[e] = head0 + (rowok[e] ? pr % G : 0);
    gtok[e] = qo_base + i;
    lim[e] = rowok[e] ? min(i + off, kv_len - 1) : -1;   // last visible key position
  }
  int warp_min_lim = min(lim[0], lim[1]);
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) warp_min_lim = min(warp_min_lim, __shfl_xor_sync(0xffffffffu, warp_min_lim, o));

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float acc_o[16][4];
#pragma unroll
  for (int n = 0; n < 16; ++n) { acc_o[n][0] = acc_o[n][1] = acc_o[n][2] = acc_o[n][3] = 0.f; }

  // ---------------- prologue ----------------
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (tb + s < te) load_tile(s, tb + s);
    cp_async_commit();
  }
  __syncthreads();                               // Q visible
  uint32_t qf[8][4];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    const int r = wm * 16 + (lane & 15), ch = ks * 2 + (lane >> 4);
    ldmatrix_x4(smem_u32(sQ + swz_off(r, ch)), qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3]);
  }

  // ---------------- main loop ----------------
  for (int j = tb; j < te; ++j) {
    const int it = j - tb;
    cp_async_wait<STAGES - 2>();
    __syncthreads();                             // tile j landed; everyone left tile j-1
    if (j + STAGES - 1 < te) load_tile((it + STAGES - 1) % STAGES, j + STAGES - 1);
    cp_async_commit();

    const TileSrc src = tile_src(j);
    const unsigned char* tK = sRing + (it % STAGES) * C::STAGE_BYTES;
    const unsigned char* tV = tK + C::TILE_BYTES;
    if (!src.valid) continue;                    // whole tile masked (sparse padding / beyond kv_len)
    if constexpr (KV8) {                         // widen e4m3 -> fp16 into swizzled tiles
      unsigned char* cK = sCvt;
      unsigned char* cV = sCvt + kKvTile * kHeadDim * 2;
      for (int c = tid; c < kKvTile * 8; c += NT) {
        const int r = c >> 3, ch8 = c & 7;       // 16 raw bytes -> two 16-byte fp16 chunks
        {
          const uint4 raw = *reinterpret_cast<const uint4*>(tK + r * 128 + ch8 * 16);
          uint4 a, bq;
          a.x = cvt_e4m3x2<true>(raw.x & 0xffff); a.y = cvt_e4m3x2<true>(raw.x >> 16);
          a.z = cvt_e4m3x2<true>(raw.y & 0xffff); a.w = cvt_e4m3x2<true>(raw.y >> 16);
          bq.x = cvt_e4m3x2<true>(raw.z & 0xffff); bq.y = cvt_e4m3x2<true>(raw.z >> 16);
          bq.z = cvt_e4m3x2<true>(raw.w & 0xffff); bq.w = cvt_e4m3x2<true>(raw.w >> 16);
          *reinterpret_cast<uint4*>(cK + swz_off(r, ch8 * 2)) = a;
          *reinterpret_cast<uint4*>(cK + swz_off(r, ch8 * 2 + 1)) = bq;
        }
        if constexpr (HAS_O) {
          const uint4 raw = *reinterpret_cast<const uint4*>(tV + r * 128 + ch8 * 16);
          uint4 a, bq;
          a.x = cvt_e4m3x2<true>(raw.x & 0xffff); a.y = cvt_e4m3x2<true>(raw.x >> 16);
          a.z = cvt_e4m3x2<true>(raw.y & 0xffff); a.w = cvt_e4m3x2<true>(raw.y >> 16);
          bq.x = cvt_e4m3x2<true>(raw.z & 0xffff); bq.y = cvt_e4m3x2<true>(raw.z >> 16);
          bq.z = cvt_e4m3x2<true>(raw.w & 0xffff); bq.w = cvt_e4m3x2<true>(raw.w >> 16);
          *reinterpret_cast<uint4*>(cV + swz_off(r, ch8 * 2)) = a;
          *reinterpret_cast<uint4*>(cV + swz_off(r, ch8 * 2 + 1)) = bq;
        }
      }
      __syncthreads();
      tK = cK; tV = cV;
    }

    // ---- S = Q K^T (raw scores) ----
    float acc_s[NTILE_S][4];
#pragma unroll
    for (int n = 0; n < NTILE_S; ++n) { acc_s[n][0] = acc_s[n][1] = acc_s[n][2] = acc_s[n][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
#pragma unroll
      for (int np = 0; np < NTILE_S / 2; ++np) {
        const int key = wn * BNW + np * 16 + (lane & 7) + ((lane >> 4) << 3);
        const int ch = ks * 2 + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldmatrix_x4(smem_u32(tK + swz_off(key, ch)), b0, b1, b2, b3);
        mma_16816<HF>(acc_s[np * 2], qf[ks], b0, b1);
        mma_16816<HF>(acc_s[np * 2 + 1], qf[ks], b2, b3);
      }
    }

    // ---- mask ----
    const int col0 = src.pos0 + wn * BNW + ((lane & 3) << 1);
    if (src.pos0 + kKvTile - 1 > warp_min_lim) {
#pragma unroll
      for (int n = 0; n < NTILE_S; ++n) {
        const int c = col0 + n * 8;
        if (c > lim[0]) acc_s[n][0] = -INFINITY;
        if (c + 1 > lim[0]) acc_s[n][1] = -INFINITY;
        if (c > lim[1]) acc_s[n][2] = -INFINITY;
        if (c + 1 > lim[1]) acc_s[n][3] = -INFINITY;
      }
    }

    // ---- row max of the raw scores ----
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < NTILE_S; ++n) {
      mx[0] = fmaxf(mx[0], fmaxf(acc_s[n][0], acc_s[n][1]));
      mx[1] = fmaxf(mx[1], fmaxf(acc_s[n][2], acc_s[n][3]));
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 1));
      mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xffffffffu, mx[e], 2));
    }

    if (want_score) {
      float tmx[2] = {mx[0], mx[1]};
      if constexpr (NW > 1) {
        if ((lane & 3) == 0) { s_rowmax[wn][lane >> 2] = mx[0]; s_rowmax[wn][(lane >> 2) + 8] = mx[1]; }
        __syncthreads();
        if (wn == 0) {
#pragma unroll
          for (int w2 = 1; w2 < NW; ++w2) {
            tmx[0] = fmaxf(tmx[0], s_rowmax[w2][lane >> 2]);
            tmx[1] = fmaxf(tmx[1], s_rowmax[w2][(lane >> 2) + 8]);
          }
        }
      }
      if (wn == 0 && (lane & 3) == 0) {
        const int tile_idx = src.pos0 / kKvTile;
        if (tile_idx < p.max_k_tiles) {
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            if (!rowok[e]) continue;
            const int64_t o = (static_cast<int64_t>(headr[e]) * p.max_k_tiles + tile_idx) * p.total_q + gtok[e];
            if (p.max_score_dtype == MSA_DT_BF16) static_cast<__nv_bfloat16*>(p.max_score)[o] = __float2bfloat16_rn(tmx[e]);
            else static_cast<float*>(p.max_score)[o] = tmx[e];
          }
        }
      }
    }

    if constexpr (HAS_O) {
      // ---- online softmax (log2 domain) ----
      float msafe[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float m_new = fmaxf(m_run[e], mx[e] * scale_log2);
        msafe[e] = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = exp2_fast(m_run[e] - msafe[e]);      // m_run = -inf -> 0
        m_run[e] = m_new;
        l_run[e] *= corr;
#pragma unroll
        for (int n = 0; n < 16; ++n) { acc_o[n][e * 2] *= corr; acc_o[n][e * 2 + 1] *= corr; }
      }
      uint32_t pf[KSTEP_PV][4];
#pragma unroll
      for (int n = 0; n < NTILE_S; ++n) {
        const float p0 = exp2_fast(acc_s[n][0] * scale_log2 - msafe[0]);
        const float p1 = exp2_fast(acc_s[n][1] * scale_log2 - msafe[0]);
        const float p2 = exp2_fast(acc_s[n][2] * scale_log2 - msafe[1]);
        const float p3 = exp2_fast(acc_s[n][3] * scale_log2 - msafe[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        pf[n >> 1][(n & 1) * 2] = pack2<HF>(p0, p1);
        pf[n >> 1][(n & 1) * 2 + 1] = pack2<HF>(p2, p3);
      }
      // ---- O += P V ----
#pragma unroll
      for (int kk = 0; kk < KSTEP_PV; ++kk) {
#pragma unroll
        for (int dp = 0; dp < 8; ++dp) {
          const int key = wn * BNW + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
          const int ch = dp * 2 + (lane >> 4);
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4_trans(smem_u32(tV + swz_off(key, ch)), b0, b1, b2, b3);
          mma_16816<HF>(acc_o[dp * 2], pf[kk], b0, b1);
          mma_16816<HF>(acc_o[dp * 2 + 1], pf[kk], b2, b3);
        }
      }
    }
  }
  cp_async_wait<0>();

  if constexpr (!HAS_O) return;

  // ---------------- epilogue ----------------
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 1);
    l_run[e] += __shfl_xor_sync(0xffffffffu, l_run[e], 2);
  }
  const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;   // per-head V de-quantisation
  const float out_scale = p.out_scale * vsh;
  const bool to_partial = p.partial_o != nullptr;

  if constexpr (NW == 1) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      if (!rowok[e]) continue;
      const float inv = l_run[e] > 0.f ? (to_partial ? vsh : 1.f) / l_run[e] : 0.f;
      const float lse = l_run[e] > 0.f ? m_run[e] * kLn2 + __logf(l_run[e]) : -INFINITY;
      if (to_partial) {
        const int64_t row = (static_cast<int64_t>(split) * p.total_q + gtok[e]) * p.num_qo_heads + headr[e];
        float* dst = p.partial_o + row * kHeadDim + ((lane & 3) << 1);
#pragma unroll
        for (int n = 0; n < 16; ++n)
          *reinterpret_cast<float2*>(dst + n * 8) = make_float2(acc_o[n][e * 2] * inv, acc_o[n][e * 2 + 1] * inv);
        if ((lane & 3) == 0) p.partial_lse[row] = lse;
      } else {
        if (p.out) {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(gtok[e]) * p.out_stride_tok +
                               static_cast<int64_t>(headr[e]) * p.out_stride_head + ((lane & 3) << 1);
          const float sc = inv * out_scale;
#pragma unroll
          for (int n = 0; n < 16; ++n)
            *reinterpret_cast<uint32_t*>(dst + n * 8) = pack2<false>(acc_o[n][e * 2] * sc, acc_o[n][e * 2 + 1] * sc);
        }
        if (p.lse && (lane & 3) == 0) p.lse[static_cast<int64_t>(gtok[e]) * p.num_qo_heads + headr[e]] = lse;
      }
    }
  } else {
    // merge the NW per-warp softmax states through shared memory (ring is idle now)
    __syncthreads();
    float* sO = reinterpret_cast<float*>(sRing);                 // [NW][16][130]
    constexpr int LD = kHeadDim + 2;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int r = (lane >> 2) + e * 8;
      float* dst = sO + (wn * 16 + r) * LD;
#pragma unroll
      for (int n = 0; n < 16; ++n) {
        dst[n * 8 + ((lane & 3) << 1)] = acc_o[n][e * 2];
        dst[n * 8 + ((lane & 3) << 1) + 1] = acc_o[n][e * 2 + 1];
      }
      if ((lane & 3) == 0) { dst[kHeadDim] = m_run[e]; dst[kHeadDim + 1] = l_run[e]; }
    }
    __syncthreads();
    // thread -> (row, 16-column chunk); NT = 32*NW threads, 16 rows * 8 chunks = 128 tasks
    for (int task = tid; task < 16 * 8; task += NT) {
      const int r = task >> 3, c0 = (task & 7) * 16;
      const int pr = row0 + r;
      if (pr >= rows_total) continue;
      const int i = i_base + pr / G, head = head0 + pr % G;
      const int gt = qo_base + i;
      float M = -INFINITY;
#pragma unroll
      for (int w2 = 0; w2 < NW; ++w2) M = fmaxf(M, sO[(w2 * 16 + r) * LD + kHeadDim]);
      const float Ms = (M == -INFINITY) ? 0.f : M;
      float L = 0.f, o[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) o[c] = 0.f;
#pragma unroll
      for (int w2 = 0; w2 < NW; ++w2) {
        const float* src = sO + (w2 * 16 + r) * LD;
        const float sc = exp2_fast(src[kHeadDim] - Ms);
        L += sc * src[kHeadDim + 1];
#pragma unroll
        for (int c = 0; c < 16; ++c) o[c] += sc * src[c0 + c];
      }
      const float inv = L > 0.f ? (to_partial ? vsh : 1.f) / L : 0.f;
      const float lse = L > 0.f ? Ms * kLn2 + __logf(L) : -INFINITY;
      if (to_partial) {
        const int64_t row = (static_cast<int64_t>(split) * p.total_q + gt) * p.num_qo_heads + head;
        float* dst = p.partial_o + row * kHeadDim + c0;
#pragma unroll
        for (int c = 0; c < 16; c += 4)
          *reinterpret_cast<float4*>(dst + c) = make_float4(o[c] * inv, o[c + 1] * inv, o[c + 2] * inv, o[c + 3] * inv);
        if (c0 == 0) p.partial_lse[row] = lse;
      } else {
        if (p.out) {
          __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(gt) * p.out_stride_tok +
                               static_cast<int64_t>(head) * p.out_stride_head + c0;
          const float sc = inv * out_scale;
          uint4 v0, v1;
          v0.x = pack2<false>(o[0] * sc, o[1] * sc);   v0.y = pack2<false>(o[2] * sc, o[3] * sc);
          v0.z = pack2<false>(o[4] * sc, o[5] * sc);   v0.w = pack2<false>(o[6] * sc, o[7] * sc);
          v1.x = pack2<false>(o[8] * sc, o[9] * sc);   v1.y = pack2<false>(o[10] * sc, o[11] * sc);
          v1.z = pack2<false>(o[12] * sc, o[13] * sc); v1.w = pack2<false>(o[14] * sc, o[15] * sc);
          *reinterpret_cast<uint4*>(dst) = v0;
          *reinterpret_cast<uint4*>(dst + 8) = v1;
        }
        if (p.lse && c0 == 0) p.lse[static_cast<int64_t>(gt) * p.num_qo_heads + head] = lse;
      }
    }
  }
}

template <int MW, int NW, bool HAS_O, bool KV8>
int launch_cfg(const MsaFmhaParams& p, int grid, cudaStream_t stream) {
  using C = Cfg<MW, NW, HAS_O, KV8>;
  auto kern = fmha_mma_kernel<MW, NW, HAS_O, KV8>;
  static bool attr_done[16] = {};                 // per device
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_done[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM) != cudaSuccess) return MSA_ERR_LAUNCH;
    attr_done[dev] = true;
  } else if (dev >= 16) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM);
  }
  kern<<<grid, C::NT, C::SMEM, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

template <bool HAS_O, bool KV8>
int launch_bm(const MsaFmhaParams& p, int grid, cudaStream_t stream) {
  switch (p.block_m) {
    case 16: return launch_cfg<1, 4, HAS_O, KV8>(p, grid, stream);
    case 64: return launch_cfg<4, 1, HAS_O, KV8>(p, grid, stream);
    case 128: return launch_cfg<8, 1, HAS_O, KV8>(p, grid, stream);
    default: return MSA_ERR_UNSUPPORTED;
  }
}

}  // namespace

int fmha_mma_launch(const MsaFmhaParams& p, cudaStream_t stream) {
  const bool sparse = (p.flags & MSA_FLAG_SPARSE) != 0;
  const bool has_o = (p.flags & MSA_FLAG_OUT_O) != 0;
  const bool kv8 = p.kv_dtype == MSA_DT_E4M3;
  int64_t grid64 = sparse ? static_cast<int64_t>(p.total_q) * p.num_kv_heads * p.num_splits : p.num_work;
  if (grid64 <= 0) return MSA_OK;
  if (grid64 > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  const int grid = static_cast<int>(grid64);
  if (has_o) return kv8 ? launch_bm<true, true>(p, grid, stream) : launch_bm<true, false>(p, grid, stream);
  return kv8 ? launch_bm<false, true>(p, grid, stream) : launch_bm<false, false>(p, grid, stream);
}

}  // namespace msa
