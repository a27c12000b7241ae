// Split-KV attention forward whose partial-result scratch lives inside the library image.
//
// Some hosts embed this library where device allocation is off the table: an inference engine
// that has already handed the whole device heap to its own pool and forbids cudaMalloc after
// start-up, or a plugin sandbox that is given tensors but no allocator.  The regular split path
// (msa_fmha_fwd with a partial workspace, then msa_lse_merge) needs a caller-allocated buffer
// for the per-split partial outputs.  msa_fmha_fwd_split_static runs the same two kernels but
// points them at a fixed array in device global memory that is part of this module, so the call
// itself allocates nothing.
#include "common.cuh"
#include "nvtx_range.h"

namespace msa {
int fmha_mma_launch(const MsaFmhaParams& p, cudaStream_t stream);
int validate_fmha(const MsaFmhaParams& p, bool own_scratch);

namespace {

// rows = splits * tokens * query heads; each row holds 128 fp32 of partial O plus one fp32 LSE
constexpr long long kMaxRows = MSA_STATIC_SCRATCH_MAX_ROWS;
constexpr long long kFloatsPerRow = kHeadDim + 1;

static __device__ __align__(256) float g_split_scratch[kMaxRows * kFloatsPerRow];

// Marks every (split, token, head) slot as "not computed": the merge gives a slot whose LSE is -inf
// the weight 0 and never reads its partial O.
__global__ void __launch_bounds__(256) clear_lse_kernel(float* __restrict__ lse, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) lse[i] = -INFINITY;
}

// Device address of g_split_scratch on the given device, resolved on first use there.  In host
// code the symbol's name is only a handle, never a pointer a kernel could use.  The cache is
// written without a lock: two threads that race on a device's first call both store the same
// address (the lookup is idempotent), so the worst case is one redundant lookup.
float* scratch_address(int device, cudaError_t* err) {
  static float* addr[64] = {};
  *err = cudaSuccess;
  if (device < 0 || device >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
  if (!addr[device]) {
    float* ptr = nullptr;
    *err = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_split_scratch);
    if (*err != cudaSuccess) return nullptr;
    addr[device] = ptr;
  }
  return addr[device];
}

}  // namespace
}  // namespace msa

extern "C" int msa_fmha_fwd_split_static(const MsaFmhaParams* pp, const int32_t* splits_per_row,
                                         msa_stream_t stream_) {
  using namespace msa;
  if (!pp) return MSA_ERR_BAD_ARG;
  MsaFmhaParams p = *pp;
  // the same argument checks as msa_fmha_fwd, before anything touches the device
  if (!(p.flags & MSA_FLAG_OUT_O) || (p.flags & MSA_FLAG_OUT_SCORE) || !p.out) return MSA_ERR_BAD_ARG;
  if (const int rc = validate_fmha(p, true)) return rc;
  if (p.block_m == 256) return MSA_ERR_UNSUPPORTED;              // 256-row items belong to the unsplit prefill kernel
  const long long rows = static_cast<long long>(p.num_splits) * p.total_q * p.num_qo_heads;
  if (rows > kMaxRows) return MSA_ERR_TOO_LARGE;
  if (rows == 0) return MSA_OK;
  msa::NvtxRange range("msa_fmha_fwd_split_static");

  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess) return MSA_ERR_LAUNCH;
  cudaError_t err;
  float* scratch = scratch_address(device, &err);
  if (!scratch) return MSA_ERR_LAUNCH;

  // The array keeps what the previous call left in it, and a work list need not cover every slot
  // (an empty list; a row tile whose keys gave fewer than num_splits items when splits_per_row is
  // NULL).  So every LSE slot of this call starts at -inf: a slot that no work item writes merges
  // with weight 0 instead of with a stale partial.
  float* user_lse = p.lse;
  p.partial_o = scratch;
  p.partial_lse = scratch + rows * kHeadDim;
  p.lse = nullptr;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int n_lse = static_cast<int>(rows);
  clear_lse_kernel<<<(n_lse + 255) / 256, 256, 0, stream>>>(p.partial_lse, n_lse);
  if (cudaGetLastError() != cudaSuccess) return MSA_ERR_LAUNCH;
  const int rc = fmha_mma_launch(p, stream);
  if (rc != MSA_OK) return rc;
  return msa_lse_merge(p.partial_o, MSA_DT_F32, p.partial_lse, splits_per_row, p.out, user_lse, p.num_splits, p.total_q,
                       p.num_qo_heads, p.out_stride_tok, p.out_stride_head, p.out_scale, stream_);
}
