// Split-KV merge for sm_100a: combines normalised partial outputs with their LSEs.
//
//   out[t,h,:] = sum_s w_s * partial_o[s,t,h,:] / sum_s w_s,   w_s = exp(lse_s - max_s lse_s)
//
// A split whose LSE is -inf contributes nothing and its partial is never multiplied in (it may
// hold NaN or stale bytes).  Same contract as the upstream reduction
// (csrc/include/sm80_fmha_reduction.hpp:133-215); partials here are fp32 or bf16 and the LSE
// is a natural logarithm.  One warp handles one (token, head): lane l owns columns 4l..4l+3.
#include "common.cuh"

namespace msa {
namespace {

template <bool PBF16>
__global__ void __launch_bounds__(256)
lse_merge_kernel(const void* __restrict__ po_, const float* __restrict__ pl, const int32_t* __restrict__ spr,
                 __nv_bfloat16* __restrict__ out, float* __restrict__ lse_out, int num_splits, int total_q,
                 int num_heads, int64_t out_stride_tok, int64_t out_stride_head, float out_scale) {
  const int lane = threadIdx.x & 31;
  const int64_t row = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);   // t * H + h
  const int64_t rows = static_cast<int64_t>(total_q) * num_heads;
  if (row >= rows) return;
  const int t = static_cast<int>(row / num_heads), h = static_cast<int>(row % num_heads);
  const int S = spr ? min(spr[t], num_splits) : num_splits;

  float mx = -INFINITY;
  for (int s = lane; s < S; s += 32) mx = fmaxf(mx, pl[static_cast<int64_t>(s) * rows + row]);
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  const float mxs = (mx == -INFINITY) ? 0.f : mx;

  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float sw = 0.f;
  for (int s = 0; s < S; ++s) {
    const float l = pl[static_cast<int64_t>(s) * rows + row];
    float4 v;
    if constexpr (PBF16) {
      const uint2 raw = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(po_) +
                                                        (static_cast<int64_t>(s) * rows + row) * kHeadDim + lane * 4);
      v = make_float4(bf16_bits_to_float(raw.x & 0xffff), bf16_bits_to_float(raw.x >> 16),
                      bf16_bits_to_float(raw.y & 0xffff), bf16_bits_to_float(raw.y >> 16));
    } else {
      v = *reinterpret_cast<const float4*>(static_cast<const float*>(po_) +
                                           (static_cast<int64_t>(s) * rows + row) * kHeadDim + lane * 4);
    }
    if (l != -INFINITY) {                      // value select after an unconditional load
      const float w = __expf(l - mxs);
      sw += w;
      acc.x = fmaf(w, v.x, acc.x); acc.y = fmaf(w, v.y, acc.y);
      acc.z = fmaf(w, v.z, acc.z); acc.w = fmaf(w, v.w, acc.w);
    }
  }
  const float inv = sw > 0.f ? out_scale / sw : 0.f;
  if (out) {
    __nv_bfloat16* dst = out + static_cast<int64_t>(t) * out_stride_tok + static_cast<int64_t>(h) * out_stride_head + lane * 4;
    uint2 pk;
    pk.x = pack2<false>(acc.x * inv, acc.y * inv);
    pk.y = pack2<false>(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(dst) = pk;
  }
  if (lse_out && lane == 0) lse_out[row] = sw > 0.f ? mxs + __logf(sw) : -INFINITY;
}

}  // namespace
}  // namespace msa

extern "C" int msa_lse_merge(const void* partial_o, int32_t partial_dtype, const float* partial_lse,
                             const int32_t* splits_per_row, void* out, float* lse_out, int32_t num_splits,
                             int32_t total_q, int32_t num_heads, int64_t out_stride_tok, int64_t out_stride_head,
                             float out_scale, msa_stream_t stream) {
  if (!partial_o || !partial_lse || (!out && !lse_out) || num_splits < 1 || total_q < 0 || num_heads <= 0)
    return MSA_ERR_BAD_ARG;
  const int64_t rows = static_cast<int64_t>(total_q) * num_heads;
  if (rows == 0) return MSA_OK;
  const int64_t blocks = (rows + 7) / 8;
  if (blocks > 0x7fffffffLL) return MSA_ERR_TOO_LARGE;
  if (partial_dtype != MSA_DT_F32 && partial_dtype != MSA_DT_BF16) return MSA_ERR_UNSUPPORTED;
  if (partial_dtype == MSA_DT_BF16)
    msa::lse_merge_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        partial_o, partial_lse, splits_per_row, static_cast<__nv_bfloat16*>(out), lse_out, num_splits, total_q,
        num_heads, out_stride_tok, out_stride_head, out_scale);
  else
    msa::lse_merge_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        partial_o, partial_lse, splits_per_row, static_cast<__nv_bfloat16*>(out), lse_out, num_splits, total_q,
        num_heads, out_stride_tok, out_stride_head, out_scale);
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}
