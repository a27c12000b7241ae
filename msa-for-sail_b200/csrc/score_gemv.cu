// Per-page max score for work items of at most four rows (the proxy pass of MSA decode:
// one query token against a one-head index cache, upstream sm80_fmha_fwd_mainloop.hpp:427-470
// with output_o = false).
//
// With so few rows the pass is a matrix-vector product per page: 2 FLOP per K byte (e4m3), far
// below what keeps a tensor-core pipeline fed, and every page's result is independent of every
// other page's.  So there is no pipeline to synchronise at all: one warp owns one 128-key page
// at a time, streams it with 16-byte loads (sixteen in flight per lane, up to 24 resident warps per SM),
// multiplies on the FMA pipe with fp32 accumulation (fma.rn.f32.f16 / .bf16: no conversion of
// the products, e4m3 is widened to f16 exactly), reduces the lanes that share a key with
// shuffles and keeps a running max.  The page table entry is the only dependent load.
//
//   grid = (chunks, work items); warp `blockIdx.x * 8 + warp` of an item takes its tiles
//   round-robin.  Lane l holds head_dim [c * E, c * E + E) of key (l / L) of each 4- or 2-key
//   group, E = 16 elements per 16 bytes (e4m3) or 8 (bf16), L = lanes per key (8 or 16).
#include <algorithm>

#include "common.cuh"

namespace msa {
namespace score_gemv {
namespace {

constexpr int BN = 128;
constexpr int NWARPS = 8;

__device__ __forceinline__ uint4 ld_stream(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}
// acc += a.lo * b.lo + a.hi * b.hi, operands packed f16x2 / bf16x2, fp32 accumulate
template <bool BF>
__device__ __forceinline__ void fma2(float& acc, uint32_t a, uint32_t b) {
  if constexpr (BF) {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
        "fma.rn.f32.bf16 %0, al, bl, %0;\n\tfma.rn.f32.bf16 %0, ah, bh, %0;\n\t}"
        : "+f"(acc) : "r"(a), "r"(b));
  } else {
    asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t"
        "mov.b32 {al, ah}, %1;\n\tmov.b32 {bl, bh}, %2;\n\t"
        "fma.rn.f32.f16 %0, al, bl, %0;\n\tfma.rn.f32.f16 %0, ah, bh, %0;\n\t}"
        : "+f"(acc) : "r"(a), "r"(b));
  }
}
__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint32_t two_bytes) {
  uint32_t r;
  const unsigned short h = static_cast<unsigned short>(two_bytes);
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(h));
  return r;
}

// F8: e4m3 cache (q e4m3 or bf16, multiplied as f16); otherwise bf16 cache and bf16 q.
constexpr int kCtasPerSm = 3;                    // register budget: 85 per thread
template <bool F8, int R>
__global__ void __launch_bounds__(NWARPS * 32, kCtasPerSm)
score_gemv_kernel(const __grid_constant__ MsaFmhaParams p) {
  constexpr int QW = F8 ? 8 : 4;                 // 32-bit words of q per lane per row
  constexpr int L = F8 ? 8 : 16;                 // lanes that share one key
  constexpr int KPL = 32 / L;                    // keys per warp-wide load
  constexpr int NLOAD = BN / KPL;                // loads per lane per tile
  constexpr int UNROLL = R == 4 ? 8 : 16;        // 16-byte loads in flight per lane
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const MsaWorkItem w = p.work[blockIdx.y];
  const int b = chk(w.batch, 0, p.batch, p.status), head0 = chk(w.head0, 0, p.num_qo_heads, p.status);
  const int h_r = p.num_qo_heads / p.num_kv_heads;
  const int kvh = head0 / h_r, G = p.pack;
  // (all of the item's metadata is requested before the first use: one round trip, not two)
  const int qo_base = p.qo_start[b], qo_end = p.qo_start[b + 1];
  const int kv_len = p.kv_len[b], off = p.qo_offset[b], page_base = p.kv_page_indptr[b];
  // rows of this item; a batch slot without query tokens (graph-safe padding) is an empty item: it loads the
  // (clamped, hence valid) first row of Q and walks no tile.  (An early return instead measured 3 % slower
  // on the whole pass.)
  const int nrows = min((qo_end - qo_base) * G, w.num_rows);
  const int c = lane % L, ksub = lane / L;

  // this lane's slice of every row of Q
  uint32_t q[R][QW];
  int lim[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int rr = max(0, min(r, nrows - 1));
    const int gtok = max(0, min(qo_base + rr / G, p.total_q - 1)), head = head0 + rr % G;
    lim[r] = r < nrows ? min(rr / G + off, kv_len - 1) : -1;
    if (p.q_dtype == MSA_DT_E4M3) {
      const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.q) +
          static_cast<int64_t>(gtok) * p.q_stride_tok + static_cast<int64_t>(head) * p.q_stride_head + c * 16);
      const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
      if constexpr (F8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) { q[r][2 * i] = e4m3x2_to_f16x2(wv[i] & 0xffffu); q[r][2 * i + 1] = e4m3x2_to_f16x2(wv[i] >> 16); }
      }
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.q) +
          static_cast<int64_t>(gtok) * p.q_stride_tok + static_cast<int64_t>(head) * p.q_stride_head + c * (F8 ? 16 : 8));
      if constexpr (F8) {                          // bf16 q against an e4m3 cache: multiply as f16
        const uint4 v0 = src[0], v1 = src[1];
        const uint32_t wv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const __half2 h = __floats2half2_rn(bf16_bits_to_float(wv[i] & 0xffffu), bf16_bits_to_float(wv[i] >> 16));
          q[r][i] = *reinterpret_cast<const uint32_t*>(&h);
        }
      } else {
        const uint4 v = src[0];
        q[r][0] = v.x; q[r][1] = v.y; q[r][2] = v.z; q[r][3] = v.w;
      }
    }
  }

  const int e = F8 ? 1 : 2;
  const unsigned char* kbase = static_cast<const unsigned char*>(p.k) + static_cast<int64_t>(kvh) * p.k_stride_head * e +
                               static_cast<int64_t>(ksub) * p.k_stride_tok * e + c * 16;
  const int64_t load_step = static_cast<int64_t>(KPL) * p.k_stride_tok * e;     // bytes between a lane's loads
  const int stride = gridDim.x * NWARPS;
  const int t_end = nrows > 0 ? w.kv_tile_end : w.kv_tile_begin;
  for (int t = w.kv_tile_begin + blockIdx.x * NWARPS + warp; t < t_end; t += stride) {
    const int phys = chk(p.kv_indices[page_base + t], 0, static_cast<int>(p.kv_extent), p.status);
    const unsigned char* kp = kbase + static_cast<int64_t>(phys) * p.k_stride_page * e;
    float mx[R];
#pragma unroll
    for (int r = 0; r < R; ++r) mx[r] = -INFINITY;
    const int pos0 = t * BN + ksub;
#pragma unroll 1
    for (int i0 = 0; i0 < NLOAD; i0 += UNROLL) {
      uint4 v[UNROLL];
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) v[u] = ld_stream(kp + (i0 + u) * load_step);
#pragma unroll
      for (int u = 0; u < UNROLL; ++u) {
        const uint32_t wv[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if constexpr (F8) {
            const uint32_t lo = e4m3x2_to_f16x2(wv[i] & 0xffffu), hi = e4m3x2_to_f16x2(wv[i] >> 16);
#pragma unroll
            for (int r = 0; r < R; ++r) { fma2<false>(acc[r], q[r][2 * i], lo); fma2<false>(acc[r], q[r][2 * i + 1], hi); }
          } else {
#pragma unroll
            for (int r = 0; r < R; ++r) fma2<true>(acc[r], q[r][i], wv[i]);
          }
        }
        const int pos = pos0 + (i0 + u) * KPL;
#pragma unroll
        for (int r = 0; r < R; ++r) {
#pragma unroll
          for (int s = 1; s < L; s <<= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], s);
          mx[r] = fmaxf(mx[r], pos <= lim[r] ? acc[r] : -INFINITY);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
#pragma unroll
      for (int s = L; s < 32; s <<= 1) mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], s));
      if (lane == 0 && r < nrows && t < p.max_k_tiles) {
        const int gtok = qo_base + r / G, head = head0 + r % G;
        const int64_t o = (static_cast<int64_t>(head) * p.max_k_tiles + t) * p.total_q + gtok;
        if (p.max_score_dtype == MSA_DT_BF16) static_cast<__nv_bfloat16*>(p.max_score)[o] = __float2bfloat16_rn(mx[r]);
        else static_cast<float*>(p.max_score)[o] = mx[r];
      }
    }
  }
}

}  // namespace
}  // namespace score_gemv

// score-only, dense page list, <= 4 rows per work item, 128-key pages with contiguous keys
int score_gemv_supported(const MsaFmhaParams& p) {
  if ((p.flags & (MSA_FLAG_OUT_O | MSA_FLAG_OUT_SCORE | MSA_FLAG_SPARSE)) != MSA_FLAG_OUT_SCORE) return 0;
  if (p.page_size != score_gemv::BN || p.decode_rows <= 0 || p.decode_rows > 4) return 0;
  if (p.kv_dtype == MSA_DT_BF16 && p.q_dtype != MSA_DT_BF16) return 0;
  if (p.kv_dtype != MSA_DT_BF16 && p.kv_dtype != MSA_DT_E4M3) return 0;
  const int h_r = p.num_qo_heads / p.num_kv_heads;
  if (p.pack != h_r) return 0;
  return 1;
}

int score_gemv_launch(const MsaFmhaParams& p, cudaStream_t stream) {
  using namespace score_gemv;
  if (p.num_work <= 0) return MSA_OK;
  if (p.num_work > 65535) return MSA_ERR_TOO_LARGE;
  static int sms[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int nsm = dev < 16 ? sms[dev] : 0;
  if (nsm == 0) {
    cudaDeviceGetAttribute(&nsm, cudaDevAttrMultiProcessorCount, dev);
    if (dev < 16) sms[dev] = nsm;
  }
  // the whole grid resident at once (a second, partial wave costs more than idle warp slots), never
  // more warps per item than it has tiles
  const int want = (nsm * kCtasPerSm) / p.num_work;
  const int cap = (p.max_k_tiles + NWARPS - 1) / NWARPS;
  const int chunks = std::max(1, std::min(want, cap));
  const dim3 grid(chunks, p.num_work);
  const bool f8 = p.kv_dtype == MSA_DT_E4M3;
  const int R = p.decode_rows <= 1 ? 1 : (p.decode_rows <= 2 ? 2 : 4);
#define MSA_GEMV(F8_, R_) score_gemv_kernel<F8_, R_><<<grid, NWARPS * 32, 0, stream>>>(p)
  if (f8) { if (R == 1) MSA_GEMV(true, 1); else if (R == 2) MSA_GEMV(true, 2); else MSA_GEMV(true, 4); }
  else    { if (R == 1) MSA_GEMV(false, 1); else if (R == 2) MSA_GEMV(false, 2); else MSA_GEMV(false, 4); }
#undef MSA_GEMV
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

}  // namespace msa
