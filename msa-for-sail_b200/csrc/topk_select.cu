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
// interleaved page slices, each thread keeping TOPK 64-bit keys (ord << 32 | ~page) in
// registers with min-replacement.  The SL partial lists are merged through shared memory.
// HBM traffic is one read of the valid part of the score tensor plus the index write; no
// transpose workspace (upstream needs one, api.py:1818-1821).
#include "common.cuh"

namespace msa {
namespace {

constexpr uint32_t kForcedOrd = 0xFF7FFFFFu;   // key of FLT_MAX

__device__ __forceinline__ uint32_t ord_key(float v) {
  const uint32_t bits = __float_as_uint(v);
  return (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
}

template <int TOPK>
struct TopList {
  unsigned long long key[TOPK];
  unsigned long long min_key;
  int min_slot;
  __device__ __forceinline__ void init() {
#pragma unroll
    for (int i = 0; i < TOPK; ++i) key[i] = 0ull;   // below every real key (ord >= 1 for real scores, and ~page != 0)
    min_key = 0ull; min_slot = 0;
  }
  __device__ __forceinline__ void find_min() {
    min_key = key[0]; min_slot = 0;
#pragma unroll
    for (int i = 1; i < TOPK; ++i) if (key[i] < min_key) { min_key = key[i]; min_slot = i; }
  }
  __device__ __forceinline__ void offer(unsigned long long k) {
    if (k > min_key) {
#pragma unroll
      for (int i = 0; i < TOPK; ++i) if (i == min_slot) key[i] = k;
      find_min();
    }
  }
};

template <int TOPK, typename T>
__global__ void __launch_bounds__(256)
topk_select_kernel(const T* __restrict__ scores, int32_t* __restrict__ out, int num_heads, int max_k_tiles,
                   int total_q, int nvp, int force_begin, int force_end_start, int slices) {
  extern __shared__ unsigned long long s_keys[];   // [slices][32][TOPK]
  const int lane = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int tok_blocks = (total_q + 31) / 32;
  const int head = blockIdx.x / tok_blocks;
  const int t = (blockIdx.x % tok_blocks) * 32 + lane;
  const bool live = t < total_q;

  TopList<TOPK> top;
  top.init();
  if (live) {
    const T* base = scores + static_cast<size_t>(head) * max_k_tiles * total_q + t;
    constexpr int UNROLL = 8;
    int k = sl;
    const int step = slices;
    // pages scanned by this slice: sl, sl + slices, ...
    for (; k + (UNROLL - 1) * step < nvp; k += UNROLL * step) {
      float v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = static_cast<float>(base[static_cast<size_t>(k + u * step) * total_q]);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const int kk = k + u * step;
        const bool forced = kk < force_begin || kk >= force_end_start;
        const uint32_t o = forced ? kForcedOrd : ord_key(v[u]);
        top.offer((static_cast<unsigned long long>(o) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(kk)));
      }
    }
    for (; k < nvp; k += step) {
      const float v = static_cast<float>(base[static_cast<size_t>(k) * total_q]);
      const bool forced = k < force_begin || k >= force_end_start;
      const uint32_t o = forced ? kForcedOrd : ord_key(v);
      top.offer((static_cast<unsigned long long>(o) << 32) | static_cast<uint32_t>(~static_cast<uint32_t>(k)));
    }
  }
  if (slices > 1) {
    unsigned long long* mine = s_keys + (static_cast<size_t>(sl) * 32 + lane) * TOPK;
#pragma unroll
    for (int i = 0; i < TOPK; ++i) mine[i] = top.key[i];
    __syncthreads();
    if (sl != 0) return;
    for (int s2 = 1; s2 < slices; ++s2) {
      const unsigned long long* other = s_keys + (static_cast<size_t>(s2) * 32 + lane) * TOPK;
#pragma unroll
      for (int i = 0; i < TOPK; ++i) top.offer(other[i]);
    }
  }
  if (!live) return;

  // page indices; empty slots (never happens when nvp > TOPK) become -1 and sort last
  uint32_t idx[TOPK];
#pragma unroll
  for (int i = 0; i < TOPK; ++i) idx[i] = top.key[i] == 0ull ? 0xffffffffu : ~static_cast<uint32_t>(top.key[i]);
  // ascending odd-even transposition sort (fully unrolled, static register indices)
#pragma unroll
  for (int pass = 0; pass < TOPK; ++pass) {
#pragma unroll
    for (int i = (pass & 1); i + 1 < TOPK; i += 2) {
      const uint32_t a = idx[i], b = idx[i + 1];
      idx[i] = min(a, b); idx[i + 1] = max(a, b);
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
  const int tok_blocks = (T_ + 31) / 32;
  const long long ctas = static_cast<long long>(tok_blocks) * H;
  // enough slices to put ~16 warps on every SM, bounded by the pages there are to scan
  int slices = 1;
  while (slices < 8 && ctas * slices < 148LL * 16 && nvp / (slices * 2) >= TOPK) slices *= 2;
  if (ctas > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  const size_t smem = slices > 1 ? static_cast<size_t>(slices) * 32 * TOPK * sizeof(unsigned long long) : 0;
  auto kern = topk_select_kernel<TOPK, T>;
  if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  kern<<<static_cast<unsigned>(ctas), 32 * slices, smem, stream>>>(scores, out, H, K, T_, nvp, fb, fe_start, slices);
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
