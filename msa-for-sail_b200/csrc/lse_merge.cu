// Split-KV merge for sm_100a: combines normalised partial outputs with their LSEs.
//
//   out[t,h,:] = sum_s w_s * partial_o[s,t,h,:] / sum_s w_s,   w_s = exp(lse_s - max_s lse_s)
//
// A split whose LSE is -inf contributes nothing and its partial is never multiplied in (it may
// hold NaN or stale bytes).  Same contract as the upstream reduction
// (csrc/include/sm80_fmha_reduction.hpp:133-215); partials here are fp32 or bf16 and the LSE
// is a natural logarithm.  Half a warp handles one (token, head).
#include "common.cuh"
#include "nvtx_range.h"

namespace msa {
namespace {

// Half a warp per (token, head) row: lane l of the half owns columns 8l..8l+7.  Loads of up to
// eight splits are issued back to back before they are consumed.
template <bool PBF16, bool OF32>
__global__ void __launch_bounds__(256)
lse_merge_kernel(const void* __restrict__ po_, const float* __restrict__ pl, const int32_t* __restrict__ spr,
                 void* __restrict__ out_, float* __restrict__ lse_out, int num_splits, int total_q,
                 int num_heads, int64_t o_split_stride, int64_t l_split_stride, int64_t out_stride_tok,
                 int64_t out_stride_head, float out_scale) {
  const int l16 = threadIdx.x & 15;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 4) + (threadIdx.x >> 4);   // t * H + h
  const int64_t rows = static_cast<int64_t>(total_q) * num_heads;
  if (row >= rows) return;
  const int t = static_cast<int>(row / num_heads), h = static_cast<int>(row % num_heads);
  const int S = spr ? min(spr[t], num_splits) : num_splits;

  float mx = -INFINITY;
  for (int s = 0; s < S; ++s) mx = fmaxf(mx, __ldg(pl + static_cast<int64_t>(s) * l_split_stride + row));
  const float mxs = (mx == -INFINITY) ? 0.f : mx;

  float acc[8];
#pragma unroll
  for (int c = 0; c < 8; ++c) acc[c] = 0.f;
  float sw = 0.f;
  constexpr int U = 8;
  for (int s0 = 0; s0 < S; s0 += U) {
    float w[U];
    uint4 raw[U][PBF16 ? 1 : 2];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = min(s0 + u, S - 1);                         // clamped: always a readable slot
      const int64_t base = static_cast<int64_t>(s) * o_split_stride + row * kHeadDim + l16 * 8;
      if constexpr (PBF16) {
        raw[u][0] = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(po_) + base);
      } else {
        raw[u][0] = *reinterpret_cast<const uint4*>(static_cast<const float*>(po_) + base);
        raw[u][1] = *reinterpret_cast<const uint4*>(static_cast<const float*>(po_) + base + 4);
      }
      const float l = __ldg(pl + static_cast<int64_t>(s) * l_split_stride + row);
      w[u] = (s0 + u < S && l != -INFINITY) ? __expf(l - mxs) : 0.f;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (w[u] != 0.f) {                                        // value select after an unconditional load
        sw += w[u];
        if constexpr (PBF16) {
          const uint32_t* r4 = reinterpret_cast<const uint32_t*>(&raw[u][0]);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            acc[2 * c] = fmaf(w[u], bf16_bits_to_float(r4[c] & 0xffff), acc[2 * c]);
            acc[2 * c + 1] = fmaf(w[u], bf16_bits_to_float(r4[c] >> 16), acc[2 * c + 1]);
          }
        } else {
          const float* f = reinterpret_cast<const float*>(&raw[u][0]);
#pragma unroll
          for (int c = 0; c < 8; ++c) acc[c] = fmaf(w[u], f[c], acc[c]);
        }
      }
    }
  }
  const float inv = sw > 0.f ? out_scale / sw : 0.f;
  if (out_ && OF32) {
    float* dst = static_cast<float*>(out_) + static_cast<int64_t>(t) * out_stride_tok + static_cast<int64_t>(h) * out_stride_head + l16 * 8;
    *reinterpret_cast<float4*>(dst) = make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
  } else if (out_) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(out_) + static_cast<int64_t>(t) * out_stride_tok + static_cast<int64_t>(h) * out_stride_head + l16 * 8;
    uint4 pk;
    pk.x = pack2<false>(acc[0] * inv, acc[1] * inv);
    pk.y = pack2<false>(acc[2] * inv, acc[3] * inv);
    pk.z = pack2<false>(acc[4] * inv, acc[5] * inv);
    pk.w = pack2<false>(acc[6] * inv, acc[7] * inv);
    *reinterpret_cast<uint4*>(dst) = pk;
  }
  if (lse_out && l16 == 0) lse_out[row] = sw > 0.f ? mxs + __logf(sw) : -INFINITY;
}

}  // namespace
}  // namespace msa

extern "C" int msa_lse_merge_ex(const void* partial_o, int32_t partial_dtype, const float* partial_lse,
                                const int32_t* splits_per_row, void* out, int32_t out_dtype, float* lse_out,
                                int32_t num_splits, int32_t total_q, int32_t num_heads, int64_t o_split_stride,
                                int64_t lse_split_stride, int64_t out_stride_tok, int64_t out_stride_head,
                                float out_scale, msa_stream_t stream) {
  if (!partial_o || !partial_lse || (!out && !lse_out) || num_splits < 1 || total_q < 0 || num_heads <= 0)
    return MSA_ERR_BAD_ARG;
  msa::NvtxRange range("msa_lse_merge");
  const int64_t rows = static_cast<int64_t>(total_q) * num_heads;
  if (rows == 0) return MSA_OK;
  const int64_t blocks = (rows + 15) / 16;
  if (blocks > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  if (partial_dtype != MSA_DT_F32 && partial_dtype != MSA_DT_BF16) return MSA_ERR_UNSUPPORTED;
  if (out_dtype != MSA_DT_F32 && out_dtype != MSA_DT_BF16) return MSA_ERR_UNSUPPORTED;
  if (o_split_stride <= 0) o_split_stride = rows * msa::kHeadDim;
  if (lse_split_stride <= 0) lse_split_stride = rows;
  // rows are read and written 16 bytes at a time
  const int pe = partial_dtype == MSA_DT_BF16 ? 2 : 4, oe = out_dtype == MSA_DT_BF16 ? 2 : 4;
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  if (!al(partial_o) || (o_split_stride * pe) % 16 || (out && (!al(out) || (out_stride_tok * oe) % 16 ||
                                                                (out_stride_head * oe) % 16)))
    return MSA_ERR_BAD_ARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned nb = static_cast<unsigned>(blocks);
#define MSA_MERGE_CASE(PB, OF)                                                                                       \
  msa::lse_merge_kernel<PB, OF><<<nb, 256, 0, st>>>(partial_o, partial_lse, splits_per_row, out, lse_out, num_splits, \
                                                    total_q, num_heads, o_split_stride, lse_split_stride,           \
                                                    out_stride_tok, out_stride_head, out_scale)
  if (partial_dtype == MSA_DT_BF16) { if (out_dtype == MSA_DT_F32) MSA_MERGE_CASE(true, true); else MSA_MERGE_CASE(true, false); }
  else { if (out_dtype == MSA_DT_F32) MSA_MERGE_CASE(false, true); else MSA_MERGE_CASE(false, false); }
#undef MSA_MERGE_CASE
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}

extern "C" int msa_lse_merge(const void* partial_o, int32_t partial_dtype, const float* partial_lse,
                             const int32_t* splits_per_row, void* out, float* lse_out, int32_t num_splits,
                             int32_t total_q, int32_t num_heads, int64_t out_stride_tok, int64_t out_stride_head,
                             float out_scale, msa_stream_t stream) {
  return msa_lse_merge_ex(partial_o, partial_dtype, partial_lse, splits_per_row, out, MSA_DT_BF16, lse_out, num_splits,
                          total_q, num_heads, 0, 0, out_stride_tok, out_stride_head, out_scale, stream);
}
