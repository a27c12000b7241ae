// Page top-k selection for sm_100a.
//
// Input scores[H, K, T] (token fastest), output out[T, H, TOPK] int32 ascending, -1 padded.
// The ranking is a strict total order -- (score key desc, page index asc) -- so the result is
// deterministic and bit-exact against a stable sort (the contract the upstream tests pin for
// the bf16 path: tests/smoke/test_sparse_topk_forced.py:266-275).  Score keys follow the
// upstream order-preserving float->uint map (sparse_topk_select.cuh:186-213); pages forced by
// force_begin / force_end rank as FLT_MAX (kForcedOrd there).
//
// Layout of the work: a CTA owns 32 consecutive tokens of one head; its lanes read 32
// consecutive tokens (one coalesced 128-byte line per page row for fp32), its SL warps scan
// interleaved blocks of TOPK pages.  Each thread keeps its TOPK best keys sorted in registers and
// folds in TOPK new keys at a time with bitonic compare-exchange networks (branch-free: rows of a
// warp never diverge).  The SL partial lists are merged through shared memory with the same network.
// HBM traffic is one read of the valid part of the score tensor plus the index write; no
// transpose workspace (upstream needs one, api.py:1818-1821).
#include "common.cuh"
#include "nvtx_range.h"

namespace msa {
namespace {

constexpr uint32_t kForcedOrd = 0xFF7FFFFFu;   // key of FLT_MAX

// Order key of a score: the upstream order-preserving float -> uint map with the two cases folded in
// where bit order and value order differ under the stable-sort contract: -0.0 and +0.0 compare equal
// (v + 0.0f turns -0.0 into +0.0), and every NaN ranks above +inf with all NaNs tying (one key).
__device__ __forceinline__ uint32_t ord_key(float v) {
  v += 0.0f;
  const uint32_t bits = __float_as_uint(v);
  const uint32_t key = bits ^ (static_cast<uint32_t>(static_cast<int32_t>(bits) >> 31) | 0x80000000u);
  return v != v ? 0xFFFFFFFFu : key;
}

// Keys of the thread-per-row kernel.  Keys are unique (the page is part of them), hence a strict total order:
// no tie handling anywhere.
//   Key64  (order key << 32 | ~page) in one 64-bit word: a compare-exchange is one 64-bit compare and two
//          64-bit selects.  (An (order key, page) pair in two 32-bit registers, 3 compares + 4 selects per
//          exchange, measured 116-121 us against 101 us at 65 536 rows x 256 pages of fp32 scores.)
//   Key1   bf16 scores: the upper half of the order key is exact for them, so (key16 << 16 | ~page16) is one
//          32-bit word and an exchange is one max and one min.  Not used with forced pages, which rank as the
//          fp32 maximum -- a score bf16 cannot tell from its own largest finite value -- nor beyond 65 535 pages.
struct Key1 {
  uint32_t k;
  static __device__ __forceinline__ Key1 none() { return {0u}; }
  static __device__ __forceinline__ Key1 make(uint32_t ord, int page) {
    return {(ord & 0xffff0000u) | (0xffffu - static_cast<uint32_t>(page))};
  }
  __device__ __forceinline__ bool is_none() const { return k == 0u; }
  __device__ __forceinline__ uint32_t page() const { return 0xffffu - (k & 0xffffu); }
  static __device__ __forceinline__ void order(Key1& a, Key1& b) {
    const uint32_t hi = max(a.k, b.k), lo = min(a.k, b.k);
    a.k = hi; b.k = lo;
  }
  static __device__ __forceinline__ Key1 best(const Key1& a, const Key1& b) { return {max(a.k, b.k)}; }
};

struct Key64 {
  unsigned long long k;
  static __device__ __forceinline__ Key64 none() { return {0ull}; }
  static __device__ __forceinline__ Key64 make(uint32_t ord, int page) {
    return {(static_cast<unsigned long long>(ord) << 32) | (0xffffffffu - static_cast<uint32_t>(page))};
  }
  __device__ __forceinline__ bool is_none() const { return (k >> 32) == 0ull; }
  __device__ __forceinline__ uint32_t page() const { return 0xffffffffu - static_cast<uint32_t>(k); }
  static __device__ __forceinline__ void order(Key64& a, Key64& b) {
    const bool sw = b.k > a.k;
    const unsigned long long hi = sw ? b.k : a.k, lo = sw ? a.k : b.k;
    a.k = hi; b.k = lo;
  }
  static __device__ __forceinline__ Key64 best(const Key64& a, const Key64& b) { return {b.k > a.k ? b.k : a.k}; }
};

// descending bitonic sort of N keys / merge of a descending list into the sorted top-N list (static
// register indices, no data-dependent branch: the 32 rows a warp owns never diverge)
template <int N, typename K>
__device__ __forceinline__ void net_sort_desc(K (&v)[N]) {
#pragma unroll
  for (int k = 2; k <= N; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll
      for (int i = 0; i < N; ++i) {
        const int l = i ^ j;
        if (l > i) {
          if ((i & k) == 0) K::order(v[i], v[l]); else K::order(v[l], v[i]);
        }
      }
    }
  }
}
template <int N, typename K>
__device__ __forceinline__ void net_merge_desc(K (&key)[N], const K (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) key[i] = K::best(key[i], v[N - 1 - i]);     // bitonic now
#pragma unroll
  for (int j = N >> 1; j > 0; j >>= 1) {
#pragma unroll
    for (int i = 0; i < N; ++i) {
      const int l = i ^ j;
      if (l > i) K::order(key[i], key[l]);
    }
  }
}

template <int TOPK, typename T, typename K>
__global__ void __launch_bounds__(256)
topk_select_kernel(const T* __restrict__ scores, int32_t* __restrict__ out, int num_heads, int max_k_tiles,
                   int total_q, int nvp, int force_begin, int force_end_start, int slices) {
  extern __shared__ __align__(8) unsigned char s_raw[];
  K* s_keys = reinterpret_cast<K*>(s_raw);          // [slices][32][TOPK]
  const int lane = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int tok_blocks = (total_q + 31) / 32;
  const int head = blockIdx.x / tok_blocks;
  const int t = (blockIdx.x % tok_blocks) * 32 + lane;
  const bool live = t < total_q;

  K top[TOPK];
#pragma unroll
  for (int i = 0; i < TOPK; ++i) top[i] = K::none();
  if (live) {
    const T* base = scores + static_cast<size_t>(head) * max_k_tiles * total_q + t;
    // slice sl scans page blocks sl, sl + slices, ... of TOPK consecutive pages each
    for (int k0 = sl * TOPK; k0 < nvp; k0 += slices * TOPK) {
      float v[TOPK];
#pragma unroll
      for (int u = 0; u < TOPK; ++u)
        v[u] = (k0 + u < nvp) ? static_cast<float>(base[static_cast<size_t>(k0 + u) * total_q]) : 0.f;
      K blk[TOPK];
#pragma unroll
      for (int u = 0; u < TOPK; ++u) {
        const int kk = k0 + u;
        const bool forced = kk < force_begin || kk >= force_end_start;
        blk[u] = kk < nvp ? K::make(forced ? kForcedOrd : ord_key(v[u]), kk) : K::none();
      }
      net_sort_desc<TOPK, K>(blk);
      net_merge_desc<TOPK, K>(top, blk);
    }
  }
  if (slices > 1) {
    K* mine = s_keys + (static_cast<size_t>(sl) * 32 + lane) * TOPK;
#pragma unroll
    for (int i = 0; i < TOPK; ++i) mine[i] = top[i];
    __syncthreads();
    if (sl != 0) return;
    for (int s2 = 1; s2 < slices; ++s2) {
      const K* other = s_keys + (static_cast<size_t>(s2) * 32 + lane) * TOPK;
      K o[TOPK];
#pragma unroll
      for (int i = 0; i < TOPK; ++i) o[i] = other[i];
      net_merge_desc<TOPK, K>(top, o);
    }
  }
  if (!live) return;

  // page indices ascending; empty slots (cannot occur when nvp > TOPK) become -1 and sort last
  uint32_t idx[TOPK];
#pragma unroll
  for (int i = 0; i < TOPK; ++i) idx[i] = top[i].is_none() ? 0xffffffffu : top[i].page();
#pragma unroll
  for (int k = 2; k <= TOPK; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
#pragma unroll
      for (int i = 0; i < TOPK; ++i) {
        const int l = i ^ j;
        if (l > i) {
          const uint32_t a = idx[i], b = idx[l];
          const bool up = (i & k) == 0;
          idx[i] = up ? min(a, b) : max(a, b);
          idx[l] = up ? max(a, b) : min(a, b);
        }
      }
    }
  }
  int32_t* dst = out + (static_cast<size_t>(t) * num_heads + head) * TOPK;
#pragma unroll
  for (int i = 0; i < TOPK; i += 4) {
    int4 v;
    v.x = static_cast<int32_t>(idx[i]); v.y = static_cast<int32_t>(idx[i + 1]);
    v.z = static_cast<int32_t>(idx[i + 2]); v.w = static_cast<int32_t>(idx[i + 3]);
    *reinterpret_cast<int4*>(dst + i) = v;                  // 0xffffffff == -1
  }
}

// Few rows (decode): one CTA per (token, head) row, its 256 threads share the row's pages, NK
// per thread, kept in registers as order keys.  Two levels of the same selection loop, neither
// with a CTA-wide barrier inside: every warp extracts its own TOPK best (each round the lanes offer
// their best key below the previous winner, redux.sync picks the winner, lane r keeps winner r),
// the 8 x TOPK survivors go through shared memory, and warp 0 extracts the final TOPK from them.
// The order is the same strict total order (key desc, page asc), so the result is identical to the
// thread-per-row kernel above.
template <int NKEYS>
__device__ __forceinline__ void warp_select_round(const uint32_t (&ord)[NKEYS], const uint32_t (&page)[NKEYS],
                                                  uint32_t& last_ord, uint32_t& last_page, uint32_t& win_ord,
                                                  uint32_t& win_page) {
  uint32_t bo = 0u, bp = 0xffffffffu;
#pragma unroll
  for (int i = 0; i < NKEYS; ++i) {
    // below the previous winner in (key desc, page asc) order; last_page starts at "before page 0"
    const bool below = ord[i] < last_ord || (ord[i] == last_ord && static_cast<int32_t>(page[i]) > static_cast<int32_t>(last_page));
    const bool better = ord[i] > bo || (ord[i] == bo && page[i] < bp);
    if (below && ord[i] != 0u && better) { bo = ord[i]; bp = page[i]; }
  }
  win_ord = __reduce_max_sync(0xffffffffu, bo);
  win_page = __reduce_min_sync(0xffffffffu, (bo == win_ord && bo != 0u) ? bp : 0xffffffffu);
  if (win_ord != 0u) { last_ord = win_ord; last_page = win_page; }
  else { last_ord = 0u; last_page = 0x7fffffffu; }            // nothing left: later rounds find nothing either
}

template <int TOPK, int NK, typename T>
__global__ void __launch_bounds__(256)
topk_row_kernel(const T* __restrict__ scores, int32_t* __restrict__ out, int num_heads, int max_k_tiles, int total_q,
                int nvp, int force_begin, int force_end_start) {
  static_assert(TOPK <= 32, "one winner per lane");
  __shared__ uint32_t s_ord[8 * TOPK], s_page[8 * TOPK];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = blockIdx.x % total_q, head = blockIdx.x / total_q;
  const T* base = scores + static_cast<size_t>(head) * max_k_tiles * total_q + t;
  uint32_t ord[NK], page[NK];
#pragma unroll
  for (int i = 0; i < NK; ++i) {
    const int pg = tid + 256 * i;
    page[i] = static_cast<uint32_t>(pg);
    ord[i] = 0u;                                             // 0: not a candidate
    if (pg < nvp) {
      const bool forced = pg < force_begin || pg >= force_end_start;
      ord[i] = forced ? kForcedOrd : ord_key(static_cast<float>(base[static_cast<size_t>(pg) * total_q]));
    }
  }
  // level 1: this warp's TOPK best, winner r in lane r
  uint32_t last_ord = 0xffffffffu, last_page = 0xffffffffu;   // (int32) -1: before page 0
  uint32_t my_ord = 0u, my_page = 0xffffffffu;
#pragma unroll
  for (int r = 0; r < TOPK; ++r) {
    uint32_t wo, wp;
    warp_select_round<NK>(ord, page, last_ord, last_page, wo, wp);
    if (lane == r) { my_ord = wo; my_page = wp; }
  }
  if (lane < TOPK) { s_ord[warp * TOPK + lane] = my_ord; s_page[warp * TOPK + lane] = my_page; }
  __syncthreads();
  if (warp != 0) return;
  // level 2: the final TOPK among the 8 * TOPK survivors
  constexpr int NC = 8 * TOPK / 32;
  uint32_t cord[NC], cpage[NC];
#pragma unroll
  for (int i = 0; i < NC; ++i) { cord[i] = s_ord[lane + 32 * i]; cpage[i] = s_page[lane + 32 * i]; }
  last_ord = 0xffffffffu; last_page = 0xffffffffu;
  uint32_t sel = 0xffffffffu;                                 // lane r: the r-th best page, or -1
#pragma unroll
  for (int r = 0; r < TOPK; ++r) {
    uint32_t wo, wp;
    warp_select_round<NC>(cord, cpage, last_ord, last_page, wo, wp);
    if (lane == r) sel = wo != 0u ? wp : 0xffffffffu;
  }
  // ascending page order, -1 (0xffffffff) last: rank = number of smaller entries (ties by lane)
  int rank = 0;
#pragma unroll
  for (int j = 0; j < TOPK; ++j) {
    const uint32_t o = __shfl_sync(0xffffffffu, sel, j);
    rank += (o < sel || (o == sel && j < lane)) ? 1 : 0;
  }
  if (lane < TOPK) out[(static_cast<size_t>(t) * num_heads + head) * TOPK + rank] = static_cast<int32_t>(sel);
}

template <int TOPK>
__global__ void topk_identity_kernel(int32_t* __restrict__ out, size_t rows, int nvp) {
  const size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= rows * TOPK) return;
  const int c = static_cast<int>(i % TOPK);
  out[i] = c < nvp ? c : -1;
}

template <int TOPK, typename T>
int launch(const T* scores, int32_t* out, int H, int K, int T_, int nvp, int fb, int fe, cudaStream_t stream) {
  const size_t rows = static_cast<size_t>(H) * T_;
  if (rows == 0) return MSA_OK;
  if (nvp <= TOPK) {
    const size_t n = rows * TOPK;
    topk_identity_kernel<TOPK><<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(out, rows, nvp);
    return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
  }
  const int fe_start = fe <= nvp ? nvp - fe : 0;
  if (rows <= 2048 && nvp <= 256 * 32) {                     // decode-sized: a CTA per row
    if (nvp <= 256 * 4)
      topk_row_kernel<TOPK, 4, T><<<static_cast<unsigned>(rows), 256, 0, stream>>>(scores, out, H, K, T_, nvp, fb, fe_start);
    else if (nvp <= 256 * 8)
      topk_row_kernel<TOPK, 8, T><<<static_cast<unsigned>(rows), 256, 0, stream>>>(scores, out, H, K, T_, nvp, fb, fe_start);
    else
      topk_row_kernel<TOPK, 32, T><<<static_cast<unsigned>(rows), 256, 0, stream>>>(scores, out, H, K, T_, nvp, fb, fe_start);
    return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
  }
  const int tok_blocks = (T_ + 31) / 32;
  const long long ctas = static_cast<long long>(tok_blocks) * H;
  // enough slices to put ~16 warps on every SM, bounded by the pages there are to scan
  int slices = 1;
  while (slices < 8 && ctas * slices < 148LL * 16 && nvp / (slices * 2) >= 2 * TOPK) slices *= 2;
  if (ctas > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  const bool one_word = sizeof(T) == 2 && fb == 0 && fe == 0 && nvp <= 65535;      // bf16 scores, nothing forced
  const size_t smem = slices > 1 ? static_cast<size_t>(slices) * 32 * TOPK * (one_word ? sizeof(Key1) : sizeof(Key64)) : 0;
  const unsigned grid = static_cast<unsigned>(ctas);
  if (one_word) {
    auto kern = topk_select_kernel<TOPK, T, Key1>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, 32 * slices, smem, stream>>>(scores, out, H, K, T_, nvp, fb, fe_start, slices);
  } else {
    auto kern = topk_select_kernel<TOPK, T, Key64>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, 32 * slices, smem, stream>>>(scores, out, H, K, T_, nvp, fb, fe_start, slices);
  }
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

}  // namespace
}  // namespace msa

extern "C" int msa_topk_select(const void* scores, int32_t score_dtype, int32_t* out, int32_t num_heads,
                               int32_t max_k_tiles, int32_t total_q, int32_t topk, int32_t num_valid_pages,
                               int32_t force_begin, int32_t force_end, msa_stream_t stream_) {
  using namespace msa;
  if (!scores || !out || num_heads < 0 || total_q < 0 || max_k_tiles <= 0) return MSA_ERR_BAD_ARG;
  if (num_valid_pages <= 0 || num_valid_pages > max_k_tiles) return MSA_ERR_BAD_ARG;
  if (force_begin < 0 || force_end < 0 || force_begin + force_end > topk) return MSA_ERR_BAD_ARG;
  msa::NvtxRange range("msa_topk_select");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
#define MSA_TOPK_CASE(KK)                                                                                          \
  case KK:                                                                                                         \
    if (score_dtype == MSA_DT_F32)                                                                                 \
      return launch<KK, float>(static_cast<const float*>(scores), out, num_heads, max_k_tiles, total_q,           \
                               num_valid_pages, force_begin, force_end, stream);                                  \
    if (score_dtype == MSA_DT_BF16)                                                                                \
      return launch<KK, __nv_bfloat16>(static_cast<const __nv_bfloat16*>(scores), out, num_heads, max_k_tiles,    \
                                       total_q, num_valid_pages, force_begin, force_end, stream);                 \
    return MSA_ERR_UNSUPPORTED;
  switch (topk) {
    MSA_TOPK_CASE(4)
    MSA_TOPK_CASE(8)
    MSA_TOPK_CASE(16)
    MSA_TOPK_CASE(32)
    default: return MSA_ERR_UNSUPPORTED;
  }
#undef MSA_TOPK_CASE
}
