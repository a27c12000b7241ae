// Dense causal FMHA forward on the 5th-generation tensor cores (tcgen05 + TMEM) for sm_100a.
//
// Serves the prefill shapes of `fmha_sail` (upstream dense/paged mainloop,
// csrc/include/sm80_fmha_fwd_mainloop.hpp:262-636): Q/K/V all bf16 or all e4m3, head_dim 128,
// ragged K/V or pages of 128 keys, one query head per row tile, optional per-tile max-score and
// LSE output.  With e4m3 operands both products run as kind::f8f6f4 MMAs and P is rounded to
// e4m3 (upstream feeds e4m3 to the MMA unit only in its score-only pass, same file :62-64, and
// converts the cache to bf16 otherwise).
//
// One CTA = 256 consecutive query rows of one (batch item, head) = two 128-row Q tiles "A" and
// "B" that walk the same KV tiles, so every K/V tile in shared memory feeds two MMAs and the
// softmax of one Q tile overlaps the tensor-core work of the other.
//
//   warps 0-3   softmax of tile A: thread r owns row r (TMEM lane r): one TMEM read of the S
//   warps 4-7   softmax of tile B  row, mask, row max, optional max-score store, exp2, bf16 P
//               written back over S, lazy rescale of O, final normalise + store
//   warp 8      TMA producer: Q once, then K and V tiles (2-deep rings each) by
//               cp.async.bulk.tensor with the physical page as a run-time coordinate
//   warp 9      MMA issuer (one elected lane): S = Q K^T into TMEM, O += P V with P read from
//               TMEM; completion is signalled to mbarriers with tcgen05.commit
//   warps 10-11 idle (they complete the third warpgroup so that setmaxnreg can move their
//               registers to the softmax warpgroups: 224 / 224 / 56 per thread)
//
// TMEM (512 columns): S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512); P aliases the
// first 64 columns of its S (32 in e4m3).  Shared memory: Q 64 KB, K 2x32 KB, V 2x32 KB (e4m3:
// Q 32 KB, K 4x16 KB, V 4x16 KB), all in the 128-byte-swizzled layout that both TMA and the UMMA
// descriptors understand.
//
// Every mbarrier wait is bounded; on a timeout the CTA raises an abort flag, reports
// MSA_STATUS_TIMEOUT in the status word, releases its TMEM and exits.
#include <mutex>
#include <type_traits>

#include "tc_ptx.cuh"

namespace msa {
namespace tc {
namespace {

constexpr int BM = 128;                 // rows per Q tile
constexpr int BN = 128;                 // keys per KV tile
constexpr int SUB_BYTES = BM * 128;     // one [128 rows][128 bytes] swizzled sub-tile: 64 bf16 or 128 e4m3 per row
constexpr int NTHREADS = 384;
constexpr int PRODUCER_WARP = 8, MMA_WARP = 9;
constexpr uint32_t kEmuMask = 0x1111;              // pairs (of 16 per 32 columns) whose exp2 is computed on the FMA pipe

// F8: Q, K, V (and P) are e4m3 and the MMAs are kind::f8f6f4; otherwise bf16 and kind::f16.  A tile is
// half as large in e4m3, so the K and V rings are twice as deep in the same shared memory.
template <bool F8>
struct Cfg {
  static constexpr int NSUB = F8 ? 1 : 2;                  // sub-tiles per [128][head_dim] tile
  static constexpr int SUB_ELEMS = F8 ? 128 : 64;          // elements of head_dim per sub-tile
  static constexpr int TILE_BYTES = NSUB * SUB_BYTES;
  static constexpr int STAGES = F8 ? 4 : 2;                // depth of the K ring and of the V ring
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + STAGES * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + STAGES * TILE_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;  // + alignment slack
  // log2 units.  P = 2^(s - m + offset) stays below 2^(threshold + offset): 2^8 in both formats, and in
  // e4m3 the offset keeps the small probabilities out of the subnormal range.
  static constexpr float kRescaleThreshold = F8 ? 4.0f : 8.0f;
  static constexpr float kPOffset = F8 ? 4.0f : 0.0f;
};

enum Bar { Q_FULL = 0, K_FULL = 1, K_EMPTY = 5, V_FULL = 9, V_EMPTY = 13, S_FULL = 17, P_FULL = 19, O_FULL = 21,
           V_FIX = 23, NUM_BARS = 24 };

__device__ __forceinline__ float2 e4m3x2_to_float2(uint16_t x) {
  const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>(x), __NV_E4M3);
  return __half22float2(*reinterpret_cast<const __half2*>(&h));
}

struct Knobs {            // read only in builds with -DMSA_DEBUG_HOOKS
  unsigned long long* trace;   // per-phase clock trace of one CTA: [4 roles][512 tiles][8 tags] clock64 samples, or null
  int trace_cta;
  int stall_tile;              // >= 0: the producer stops before this K tile and issues nothing after it
  uint32_t spin_limit;         // > 0: polls a bounded wait makes before it gives up (instead of kSpinLimit)
};

// HAS_O = false: score-only pass (no V, no P, no O), compiled on its own so that neither path's code is shaped
// by the other's.
template <bool F8, bool HAS_O>
__global__ void __launch_bounds__(NTHREADS, 1)
fmha_tc_kernel(const __grid_constant__ MsaFmhaParams p, const __grid_constant__ CUtensorMap tm_q,
               const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
               const Knobs kn) {
  using C = Cfg<F8>;
  constexpr int TILE_BYTES = C::TILE_BYTES, NSUB = C::NSUB, SUB_ELEMS = C::SUB_ELEMS;
  constexpr int KSTAGES = C::STAGES, VSTAGES = C::STAGES;
  constexpr int OFF_Q = C::OFF_Q, OFF_K = C::OFF_K, OFF_V = C::OFF_V, OFF_BAR = C::OFF_BAR;
  constexpr float kRescaleThreshold = C::kRescaleThreshold, kPOffset = C::kPOffset;
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
  const bool tracing = kn.trace != nullptr && static_cast<int>(blockIdx.x) == kn.trace_cta;
  const uint32_t spin_limit = kn.spin_limit ? kn.spin_limit : kSpinLimit;
  const int stall_tile = kn.stall_tile;
#else
  constexpr bool tracing = false;                 // the trace calls below compile to nothing
  constexpr uint32_t spin_limit = kSpinLimit;
  constexpr int stall_tile = -1;
#endif
  auto trace = [&](int role, int j, int tag) {
    if (tracing && j < 512) kn.trace[(role * 512 + j) * 8 + tag] = clock64();
  };

  // ---------------- work item ----------------
  const MsaWorkItem w = p.work[blockIdx.x];
  const int b = chk(w.batch, 0, p.batch, p.status), head = chk(w.head0, 0, p.num_qo_heads, p.status), row0 = w.row0;
  const int h_r = p.num_qo_heads / p.num_kv_heads;
  const int kvh = head / h_r;
  const int qo_base = p.qo_start[b];
  const int ql = p.qo_start[b + 1] - qo_base;
  const int kv_len = p.kv_len[b];
  const int off = p.qo_offset[b];
  const bool paged = p.page_size > 0;
  constexpr bool has_o = HAS_O;
  int n_tiles[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int m0 = row0 + x * BM;
    if (m0 >= ql) { n_tiles[x] = 0; continue; }
    const int last = min(m0 + BM, ql) - 1;
    long long vis = min(static_cast<long long>(kv_len), static_cast<long long>(last) + off + 1);
    if (vis < 0) vis = 0;
    n_tiles[x] = min(w.kv_tile_end, static_cast<int>((vis + BN - 1) / BN));
  }
  const int n_total = max(n_tiles[0], n_tiles[1]);

  // a timeout reported earlier on this device (status word not cleared yet): do not start.  Read by
  // another thread than the one that sets up the barriers, so the load overlaps that work.
  if (threadIdx.x == blockDim.x - 1)
    *skip_flag = (p.status != nullptr && *reinterpret_cast<const volatile int32_t*>(p.status) != 0) ? 1 : 0;
  if (threadIdx.x == 0) {
    mbar_init(bar(Q_FULL), 1);
    for (int s = 0; s < KSTAGES; ++s) {
      mbar_init(bar(K_FULL + s), 1);  mbar_init(bar(K_EMPTY + s), 1);
      mbar_init(bar(V_FULL + s), 1);  mbar_init(bar(V_EMPTY + s), 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar(S_FULL + s), 1);  mbar_init(bar(P_FULL + s), BM);
      mbar_init(bar(O_FULL + s), 1);
    }
    mbar_init(bar(V_FIX), 1);
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
  } else if (warp == PRODUCER_WARP) {
    // =========================== TMA producer ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (lane == 0) { tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); }
    if (n_total > 0 && elect_one()) {                   // an item without visible keys loads nothing
      mbar_arrive_expect_tx(bar(Q_FULL), 2 * TILE_BYTES);
#pragma unroll
      for (int x = 0; x < 2; ++x)
#pragma unroll
        for (int hlf = 0; hlf < NSUB; ++hlf)
          tma_load_3d(smem_base + OFF_Q + x * TILE_BYTES + hlf * SUB_BYTES, &tm_q, bar(Q_FULL), hlf * SUB_ELEMS, head,
                      qo_base + row0 + x * BM);
    }
    __syncwarp();
    const int page_base = paged ? p.kv_page_indptr[b] : 0;
    const int kv_base = paged ? 0 : p.kv_start[b];
    uint32_t fix_phase = 0;
    bool alive = true;
    for (int j = 0; j < n_total && alive; ++j) {
      if (j == stall_tile) break;                       // test hook: whoever waits for this tile runs out of polls
      const int ks = j % KSTAGES, vs = j % VSTAGES;
      const int page = paged ? chk(p.kv_indices[page_base + j], 0, static_cast<int>(p.kv_extent), p.status) : 0;
      const int valid_rows = min(BN, kv_len - j * BN);
      const bool fix = valid_rows < BN;                 // tail tile: rows past kv_len must read as 0 in V
      if (lane == 0) trace(3, j, 0);
      alive = mbar_wait(bar(K_EMPTY + ks), ((j / KSTAGES) & 1) ^ 1, abort_flag, spin_limit);
      if (lane == 0) trace(3, j, 1);
      if (!alive) break;
      if (elect_one()) {
        mbar_arrive_expect_tx(bar(K_FULL + ks), TILE_BYTES);
#pragma unroll
        for (int hlf = 0; hlf < NSUB; ++hlf) {
          const uint32_t dst = smem_base + OFF_K + ks * TILE_BYTES + hlf * SUB_BYTES;
          if (paged) tma_load_4d(dst, &tm_k, bar(K_FULL + ks), hlf * SUB_ELEMS, 0, kvh, page);
          else tma_load_3d(dst, &tm_k, bar(K_FULL + ks), hlf * SUB_ELEMS, kvh, kv_base + j * BN);
        }
      }
      __syncwarp();
      if (!has_o) continue;
      alive = mbar_wait(bar(V_EMPTY + vs), ((j / VSTAGES) & 1) ^ 1, abort_flag, spin_limit);
      if (lane == 0) trace(3, j, 2);
      if (!alive) break;
      if (elect_one()) {
        const uint32_t vbar = fix ? bar(V_FIX) : bar(V_FULL + vs);
        mbar_arrive_expect_tx(vbar, TILE_BYTES);
#pragma unroll
        for (int hlf = 0; hlf < NSUB; ++hlf) {
          const uint32_t dst = smem_base + OFF_V + vs * TILE_BYTES + hlf * SUB_BYTES;
          if (paged) tma_load_4d(dst, &tm_v, vbar, hlf * SUB_ELEMS, 0, kvh, page);
          else tma_load_3d(dst, &tm_v, vbar, hlf * SUB_ELEMS, kvh, kv_base + j * BN);
        }
      }
      __syncwarp();
      if (fix && alive && has_o) {
        alive = mbar_wait(bar(V_FIX), fix_phase, abort_flag, spin_limit);
        alive = __all_sync(0xffffffffu, alive);
        fix_phase ^= 1;
        if (alive) {
          // whole 128-byte rows are zeroed, so the swizzle does not matter
          unsigned char* vt = smem_gen + OFF_V + vs * TILE_BYTES;
          for (int c = lane; c < (BN - valid_rows) * (NSUB * 8); c += 32) {
            const int r = valid_rows + c / (NSUB * 8), ch = c % (NSUB * 8);
            *reinterpret_cast<uint4*>(vt + (ch >> 3) * SUB_BYTES + r * 128 + (ch & 7) * 16) = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(V_FULL + vs));
        }
      }
    }
  } else if (warp == MMA_WARP) {
    // =========================== MMA issuer ===========================
    // The whole warp walks the loop (waits are warp-uniform); the tcgen05 instructions are
    // issued by the one lane elect.sync picks, so their operands can live in uniform registers.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    constexpr uint32_t IDESC_QK = F8 ? idesc_e4m3(BM, BN, false, false) : idesc_bf16(BM, BN, false, false);
    constexpr uint32_t IDESC_PV = F8 ? idesc_e4m3(BM, kHeadDim, false, true) : idesc_bf16(BM, kHeadDim, false, true);
    constexpr int KSTEPS = F8 ? 4 : 8;              // MMAs per 128-deep contraction (32 bytes of K extent each)
    constexpr int V_KSTEP = (F8 ? 32 : 16) * 128;   // bytes between the key slices of consecutive P V MMAs
    // descriptor templates: K-major operands (Q, K): LBO unused (16 B), SBO 1024 B;
    // MN-major V: LBO 16384 B (next sub-tile of head_dim), SBO 1024 B (next 8 keys)
    const uint64_t dk_hi = smem_desc(0, 16, 1024) & 0xFFFFFFFFFFFF0000ull;
    const uint64_t dv_hi = smem_desc(0, SUB_BYTES, 1024) & 0xFFFFFFFFFFFF0000ull;
    auto issue_qk = [&](int x, int j) {
      const uint32_t qa = (smem_base + OFF_Q + x * TILE_BYTES) >> 4;
      const uint32_t ka = (smem_base + OFF_K + (j % KSTAGES) * TILE_BYTES) >> 4;
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {
        const uint32_t o = ((k >> 2) * SUB_BYTES + (k & 3) * 32) >> 4;
        if constexpr (F8) mma_ss_f8(tmem + x * BN, dk_hi | ((qa + o) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
        else mma_ss(tmem + x * BN, dk_hi | ((qa + o) & 0x3FFF), dk_hi | ((ka + o) & 0x3FFF), IDESC_QK, k > 0);
      }
    };
    auto issue_pv = [&](int x, int j) {
      const uint32_t va = (smem_base + OFF_V + (j % VSTAGES) * TILE_BYTES) >> 4;
#pragma unroll
      for (int k = 0; k < KSTEPS; ++k) {              // P: 8 TMEM columns per MMA in both formats
        const uint64_t vd = dv_hi | ((va + k * (V_KSTEP >> 4)) & 0x3FFF);
        if constexpr (F8) mma_ts_f8(tmem + 256 + x * kHeadDim, tmem + x * BN + k * 8, vd, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
        else mma_ts(tmem + 256 + x * kHeadDim, tmem + x * BN + k * 8, vd, IDESC_PV, (j > 0 || k > 0) ? 1u : 0u);
      }
    };
    bool alive = n_total > 0 ? mbar_wait(bar(Q_FULL), 0, abort_flag, spin_limit) : true;
    if (alive && n_total > 0) {
      alive = mbar_wait(bar(K_FULL + 0), 0, abort_flag, spin_limit);
      if (alive) {
        tc_fence_after();
        if (elect_one()) {
#pragma unroll
          for (int x = 0; x < 2; ++x)
            if (n_tiles[x] > 0) { issue_qk(x, 0); mma_commit(bar(S_FULL + x)); }
          mma_commit(bar(K_EMPTY + 0));
        }
        __syncwarp();
      }
    }
    for (int j = 0; j < n_total && alive; ++j) {
#pragma unroll
      for (int x = 0; x < 2; ++x) {
        if (j >= n_tiles[x] || !alive) continue;
        if (lane == 0) trace(2, j, x * 4 + 0);
        const bool more = j + 1 < n_tiles[x];
        // the tiles this step reads normally landed long ago: check them before P, and only once per j
        if (x == 0 || j >= n_tiles[0]) {
          if (has_o) alive = mbar_wait(bar(V_FULL + j % VSTAGES), (j / VSTAGES) & 1, abort_flag, spin_limit);
          if (alive && j + 1 < n_total)
            alive = mbar_wait(bar(K_FULL + (j + 1) % KSTAGES), ((j + 1) / KSTAGES) & 1, abort_flag, spin_limit);
        }
        if (lane == 0) trace(2, j, x * 4 + 1);
        if (alive) alive = mbar_wait(bar(P_FULL + x), j & 1, abort_flag, spin_limit);
        if (!alive) break;
        tc_fence_after();
        if (lane == 0) trace(2, j, x * 4 + 2);
        if (elect_one()) {
          if (has_o) issue_pv(x, j);
          if (more) {
            issue_qk(x, j + 1);
            mma_commit(bar(S_FULL + x));
          } else if (has_o) {
            mma_commit(bar(O_FULL + x));
          }
          if (x == 1 || j >= n_tiles[1]) {          // last user of this V stage / next K stage
            if (has_o) mma_commit(bar(V_EMPTY + j % VSTAGES));
            if (j + 1 < n_total) mma_commit(bar(K_EMPTY + (j + 1) % KSTAGES));
          }
        }
        __syncwarp();
        if (lane == 0) trace(2, j, x * 4 + 3);
      }
    }
  } else if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
  } else {
    // =========================== softmax / epilogue ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    const int x = warp >> 2;                             // 0: tile A, 1: tile B
    const int r = ((warp & 3) << 5) | lane;              // row in tile == TMEM lane
    const uint32_t lane_addr = static_cast<uint32_t>((warp & 3) << 5) << 16;
    const uint32_t tS = tmem + x * BN + lane_addr;
    const uint32_t tO = tmem + 256 + x * kHeadDim + lane_addr;
    const int m0 = row0 + x * BM;
    const int i = m0 + r;                                // token index within the sequence
    const bool row_ok = i < ql;
    const int gtok = qo_base + i;
    const int lim = row_ok ? min(i + off, kv_len - 1) : -1;
    const int nx = n_tiles[x];
    const float scale_log2 = p.sm_scale * kLog2e * (p.k_scale_head ? p.k_scale_head[kvh] : 1.f);
    const bool want_score = (p.flags & MSA_FLAG_OUT_SCORE) != 0 && p.max_score != nullptr;
    float m_used = -INFINITY, l_sum = 0.f;
    float l_exact = 0.f;                                 // e4m3 only: sum of the unrounded probabilities, for the LSE
    bool alive = true;

    for (int j = 0; j < nx && alive; ++j) {
      if (r == 0) trace(x, j, 0);
      alive = mbar_wait(bar(S_FULL + x), j & 1, abort_flag, spin_limit);
      if (!alive) break;
      tc_fence_after();
      if (r == 0) trace(x, j, 1);
      const int pos0 = j * BN;
      const bool need_mask = (pos0 + BN - 1 > m0 + off) || (pos0 + BN > kv_len);
      // ---- one read of the whole S row (128 fp32) ----
      uint32_t sv[4][32];
      tmem_ld32(tS, sv[0]);
      tmem_ld32(tS + 32, sv[1]);
      tmem_ld32(tS + 64, sv[2]);
      tmem_ld32(tS + 96, sv[3]);
      tmem_wait_ld();
      if (r == 0) trace(x, j, 2);
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (pos0 + c * 32 + e > lim) sv[c][e] = 0xff800000u;     // -inf
      }
      auto store_score = [&](const float mx) {
        if (want_score && row_ok && j < p.max_k_tiles) {
          const int64_t o = (static_cast<int64_t>(head) * p.max_k_tiles + j) * p.total_q + gtok;
          if (p.max_score_dtype == MSA_DT_BF16) static_cast<__nv_bfloat16*>(p.max_score)[o] = __float2bfloat16_rn(mx);
          else static_cast<float*>(p.max_score)[o] = mx;
        }
      };
      if (!has_o) {                    // score-only pass: the row max of the tile, then S goes back to the MMA warp
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};        // four independent chains
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            m4[(e >> 1) & 3] = max3(m4[(e >> 1) & 3], __uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1]));
        store_score(fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
        tc_fence_before();
        mbar_arrive(bar(P_FULL + x));
        continue;
      }
      // P = exp2(S * scale - m) as bf16 / e4m3, written over the front of S; the row max of the tile (the
      // max_score output, and what decides a rescale) is computed in the same pass.
      // The special-function unit does 16 exp2 per clock per SM, a quarter of what the tensor pipe needs
      // here, so kEmuMask selects pairs whose exp2 runs on the FMA pipe instead: round-to-nearest split
      // x = n + f, degree-3 polynomial for 2^f (rel. error 7.5e-5, far below the rounding of P), n added
      // into the exponent field.  All fp32 arithmetic is done on packed pairs (fma.rn.f32x2 / add.rn.f32x2).
      float mxs[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};     // four independent chains
      auto row_max = [&]() {
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int e = 0; e < 32; e += 2)
            mxs[(e >> 1) & 3] = max3(mxs[(e >> 1) & 3], __uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1]));
      };
      float l_rnd = 0.f, l_raw = 0.f;            // row sum of this tile: of P as stored / before rounding (e4m3)
      auto emit_p = [&](auto with_max, const float m_ref) {
        const uint64_t scale2 = f2_pack(scale_log2, scale_log2);
        const uint64_t negm2 = f2_pack(-m_ref, -m_ref);
        uint64_t lsum2 = f2_pack(0.f, 0.f), lex2 = f2_pack(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[F8 ? 8 : 16];
          [[maybe_unused]] uint16_t held = 0;
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            if constexpr (decltype(with_max)::value)
              mxs[(e >> 1) & 3] = max3(mxs[(e >> 1) & 3], __uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1]));
            const uint64_t x2 = f2_fma(f2_pack(__uint_as_float(sv[c][e]), __uint_as_float(sv[c][e + 1])), scale2, negm2);
            float p0, p1;
            if ((kEmuMask >> ((e >> 1) & 15)) & 1) {
              float x0, x1;
              f2_unpack(x2, x0, x1);
              const uint64_t xc = f2_pack(fmaxf(x0, -126.f), fmaxf(x1, -126.f));     // also maps -inf
              const uint64_t t2 = f2_add(xc, f2_pack(12582912.f, 12582912.f));          // 1.5 * 2^23: n in the low bits
              const uint64_t n2 = f2_add(t2, f2_pack(-12582912.f, -12582912.f));
              const uint64_t fr = f2_fma(n2, f2_pack(-1.f, -1.f), xc);                   // f in [-0.5, 0.5]
              uint64_t pl = f2_fma(fr, f2_pack(0.055171650f, 0.055171650f), f2_pack(0.24261113f, 0.24261113f));
              pl = f2_fma(pl, fr, f2_pack(0.69326097f, 0.69326097f));
              pl = f2_fma(pl, fr, f2_pack(0.99992806f, 0.99992806f));
              float q0, q1, t0, t1;
              f2_unpack(pl, q0, q1);
              f2_unpack(t2, t0, t1);
              p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
              p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
            } else {
              float x0, x1;
              f2_unpack(x2, x0, x1);
              p0 = exp2_fast(x0);
              p1 = exp2_fast(x1);
            }
            if constexpr (F8) {
              // O is normalised by the sum of the probabilities as the MMA sees them (see the decode kernel);
              // the LSE reports the sum before rounding
              lex2 = f2_add(lex2, f2_pack(p0, p1));
              const uint16_t pr = __nv_cvt_float2_to_fp8x2(make_float2(p0, p1), __NV_SATFINITE, __NV_E4M3);
              const float2 rr = e4m3x2_to_float2(pr);
              lsum2 = f2_add(lsum2, f2_pack(rr.x, rr.y));
              if (e & 2) pk[e >> 2] = static_cast<uint32_t>(held) | (static_cast<uint32_t>(pr) << 16);
              else held = pr;
            } else {
              lsum2 = f2_add(lsum2, f2_pack(p0, p1));
              pk[e >> 1] = pack2<false>(p0, p1);
            }
          }
          if constexpr (F8) tmem_st8(tS + c * 8, pk);
          else tmem_st16(tS + c * 16, pk);
        }
        float l0, l1;
        f2_unpack(lsum2, l0, l1);
        l_rnd = l0 + l1;
        if constexpr (F8) { f2_unpack(lex2, l0, l1); l_raw = l0 + l1; }
      };
      // Every tile but the first writes P with the running max while it finds its own max: the max does
      // not sit between the S read and the exponentials, and the guess holds unless the row's max grows
      // by more than the rescale threshold (then P is written again below).
      // (bf16 only: with e4m3 operands the kernel measured 6 % slower this way.)
      const bool guess = !F8 && j > 0;                              // warp-uniform
      const float m_guess = ((m_used == -INFINITY) ? 0.f : m_used) - kPOffset;
      if (guess) emit_p(std::true_type{}, m_guess);
      else row_max();
      const float mx = fmaxf(fmaxf(mxs[0], mxs[1]), fmaxf(mxs[2], mxs[3]));
      store_score(mx);
      // ---- running max with lazy rescale ----
      const float m_cand = fmaxf(m_used, mx * scale_log2);
      // false for (-inf) - (-inf) = NaN; true for a row whose first visible key is in this tile (its guess
      // was made without a max)
      const bool bump = (m_cand - m_used) > kRescaleThreshold;
      if (!guess || __any_sync(0xffffffffu, bump)) {
        float factor = 1.f;
        if (bump) { factor = exp2_fast(m_used - m_cand); m_used = m_cand; l_sum *= factor; l_exact *= factor; }
        if (j > 0 && __any_sync(0xffffffffu, bump)) {
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
        if (r == 0) trace(x, j, 3);
        emit_p(std::false_type{}, ((m_used == -INFINITY) ? 0.f : m_used) - kPOffset);
      }
      l_sum += l_rnd;
      if constexpr (F8) l_exact += l_raw;
      if (r == 0) trace(x, j, 4);
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + x));
      if (r == 0) trace(x, j, 5);
    }

    // ---- epilogue ----
    if (alive && nx > 0 && has_o) alive = mbar_wait(bar(O_FULL + x), 0, abort_flag, spin_limit);
    if (alive && has_o) {
      tc_fence_after();
      const float vsh = p.v_scale_head ? p.v_scale_head[kvh] : 1.f;
      const float inv = l_sum > 0.f ? p.out_scale * vsh / l_sum : 0.f;
      __nv_bfloat16* dst = p.out ? static_cast<__nv_bfloat16*>(p.out) + static_cast<int64_t>(gtok) * p.out_stride_tok +
                                       static_cast<int64_t>(head) * p.out_stride_head
                                 : nullptr;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        if (nx > 0) {
          tmem_ld32(tO + c * 32, v);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) v[e] = 0u;
        }
        if (row_ok && dst) {
#pragma unroll
          for (int e = 0; e < 32; e += 8) {
            uint4 o4;
            o4.x = pack2<false>(__uint_as_float(v[e]) * inv, __uint_as_float(v[e + 1]) * inv);
            o4.y = pack2<false>(__uint_as_float(v[e + 2]) * inv, __uint_as_float(v[e + 3]) * inv);
            o4.z = pack2<false>(__uint_as_float(v[e + 4]) * inv, __uint_as_float(v[e + 5]) * inv);
            o4.w = pack2<false>(__uint_as_float(v[e + 6]) * inv, __uint_as_float(v[e + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + e) = o4;
          }
        }
      }
      if (row_ok && p.lse)
        p.lse[static_cast<int64_t>(gtok) * p.num_qo_heads + head] =
            l_sum > 0.f ? (m_used - kPOffset) * kLn2 + __logf(F8 ? l_exact : l_sum) : -INFINITY;
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

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// rank-n bf16 map with a 128-byte swizzle; dims/strides innermost first, strides in bytes for dims 1..n-1
bool make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
              const uint32_t* box, bool bytes = false) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t gd[5]; cuuint64_t gs[4]; cuuint32_t bx[5]; cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
  return fn(m, bytes ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gd, gs, bx, es,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

Knobs g_knobs = {nullptr, 0, -1, 0};

}  // namespace

}  // namespace tc

// bf16 tensor map with a 128-byte swizzle (shared with the sparse page-major kernel)
int make_tma_map_bf16(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                      const uint32_t* box) {
  return tc::make_map(m, base, rank, dims, strides_bytes, box) ? MSA_OK : MSA_ERR_LAUNCH;
}

// same for 1-byte elements (e4m3 caches)
int make_tma_map_u8(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes,
                    const uint32_t* box) {
  return tc::make_map(m, base, rank, dims, strides_bytes, box, true) ? MSA_OK : MSA_ERR_LAUNCH;
}

// Shapes the tcgen05 kernel takes; everything else runs on the mma.sync kernel.
int fmha_tc_supported(const MsaFmhaParams& p) {
  if (p.block_m != 256) return 0;
  return 1;
}

int fmha_tc_launch(const MsaFmhaParams& p, cudaStream_t stream) {
  using namespace tc;
  const bool f8 = p.kv_dtype == MSA_DT_E4M3;
  if (p.q_dtype != p.kv_dtype || (p.kv_dtype != MSA_DT_BF16 && !f8)) return MSA_ERR_UNSUPPORTED;
  if ((p.flags & MSA_FLAG_SPARSE) || p.partial_o || p.pack != 1) return MSA_ERR_UNSUPPORTED;
  if (p.page_size != 0 && p.page_size != BN) return MSA_ERR_UNSUPPORTED;
  const bool has_o = (p.flags & MSA_FLAG_OUT_O) != 0;
  if (has_o && (!p.out || !p.v)) return MSA_ERR_BAD_ARG;
  if (p.num_work <= 0) return MSA_OK;

  CUtensorMap tq, tk, tv;
  const uint64_t es = f8 ? 1 : 2;                              // bytes per element
  const uint32_t sub = f8 ? 128 : 64;                          // elements per 128-byte row of a sub-tile
  {
    const uint64_t dims[3] = {128, static_cast<uint64_t>(p.num_qo_heads), static_cast<uint64_t>(p.total_q)};
    const uint64_t str[2] = {static_cast<uint64_t>(p.q_stride_head) * es, static_cast<uint64_t>(p.q_stride_tok) * es};
    const uint32_t box[3] = {sub, 1, BM};
    if (!make_map(&tq, p.q, 3, dims, str, box, f8)) return MSA_ERR_LAUNCH;
  }
  if (p.kv_extent <= 0) return MSA_ERR_BAD_ARG;
  const uint64_t big = static_cast<uint64_t>(p.kv_extent);   // rows / pages past it read as zero
  if (p.page_size > 0) {
    const uint64_t dims[4] = {128, BN, static_cast<uint64_t>(p.num_kv_heads), big};
    const uint64_t ks[3] = {static_cast<uint64_t>(p.k_stride_tok) * es, static_cast<uint64_t>(p.k_stride_head) * es,
                            static_cast<uint64_t>(p.k_stride_page) * es};
    const uint64_t vs[3] = {static_cast<uint64_t>(p.v_stride_tok) * es, static_cast<uint64_t>(p.v_stride_head) * es,
                            static_cast<uint64_t>(p.v_stride_page) * es};
    const uint32_t box[4] = {sub, BN, 1, 1};
    if (!make_map(&tk, p.k, 4, dims, ks, box, f8) || !make_map(&tv, has_o ? p.v : p.k, 4, dims, has_o ? vs : ks, box, f8))
      return MSA_ERR_LAUNCH;
  } else {
    const uint64_t dims[3] = {128, static_cast<uint64_t>(p.num_kv_heads), big};
    const uint64_t ks[2] = {static_cast<uint64_t>(p.k_stride_head) * es, static_cast<uint64_t>(p.k_stride_tok) * es};
    const uint64_t vs[2] = {static_cast<uint64_t>(p.v_stride_head) * es, static_cast<uint64_t>(p.v_stride_tok) * es};
    const uint32_t box[3] = {sub, 1, BN};
    if (!make_map(&tk, p.k, 3, dims, ks, box, f8) || !make_map(&tv, has_o ? p.v : p.k, 3, dims, has_o ? vs : ks, box, f8))
      return MSA_ERR_LAUNCH;
  }
  static bool attr_done[4][16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  using KernelFn = void (*)(const MsaFmhaParams, const CUtensorMap, const CUtensorMap, const CUtensorMap, const Knobs);
  const int variant = (f8 ? 2 : 0) | (has_o ? 1 : 0);
  const KernelFn kernels[4] = {fmha_tc_kernel<false, false>, fmha_tc_kernel<false, true>, fmha_tc_kernel<true, false>,
                               fmha_tc_kernel<true, true>};
  const KernelFn kern = kernels[variant];
  const int smem_bytes = f8 ? Cfg<true>::SMEM_BYTES : Cfg<false>::SMEM_BYTES;
  if (dev >= 16 || !attr_done[variant][dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return MSA_ERR_LAUNCH;
    if (dev < 16) attr_done[variant][dev] = true;
  }
  kern<<<p.num_work, NTHREADS, smem_bytes, stream>>>(p, tq, tk, tv, g_knobs);
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

}  // namespace msa

#ifdef MSA_DEBUG_HOOKS
// Debug aid (builds with -DMSA_DEBUG_HOOKS only): record the phase clocks of one CTA into `buf`.
extern "C" void msa_debug_tc_trace(unsigned long long* buf, int cta) {
  msa::tc::g_knobs.trace = buf;
  msa::tc::g_knobs.trace_cta = cta;
}
// Test hook (builds with -DMSA_DEBUG_HOOKS only): make the bounded waits of the dense prefill kernel run out.
// The TMA producer of every CTA stops before K tile `tile` (-1: never) and issues nothing after it -- no copy
// is outstanding when the CTA gives up -- and a wait gives up after `spin_limit` polls (0: the normal limit).
extern "C" void msa_debug_tc_stall(int tile, unsigned spin_limit) {
  msa::tc::g_knobs.stall_tile = tile;
  msa::tc::g_knobs.spin_limit = spin_limit;
}
#endif
