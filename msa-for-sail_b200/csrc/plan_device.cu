// Planning on the device: the metadata and the work list of a decode-sized batch, produced by one
// small kernel from length tensors that live on the GPU, so that plan + run can sit in one CUDA
// graph whose replays see new lengths (upstream graph_safe mode: prepare_plan_metadata.cuh,
// plan.cuh; api.py:916-941).  Everything that sizes a launch is fixed by the caller: batch, the row
// tiles per batch item, the split count -- hence the work list has a fixed number of items; a row
// tile past a sequence's rows and a chunk past its key tiles are empty items.
#include "common.cuh"
#include "nvtx_range.h"

namespace msa {
namespace {

__global__ void __launch_bounds__(256) plan_device_kernel(const MsaPlanDeviceArgs a) {
  __shared__ int s_total_q;
  const int G = a.pack;
  const int groups = a.num_qo_heads / G;
  const int S = a.num_splits;
  // prefix sums: batches are small (decode), one thread walks them
  if (threadIdx.x == 0) {
    int q = 0, k = 0, pg = 0;
    for (int b = 0; b < a.batch; ++b) {
      const int ql = a.qo_len[b], kl = a.kv_len[b];
      if (a.qo_start) a.qo_start[b] = q;
      if (a.kv_start) a.kv_start[b] = k;
      if (a.kv_page_indptr) a.kv_page_indptr[b] = pg;
      if (a.kv_len_out) a.kv_len_out[b] = kl;
      if (a.qo_offset_out) {
        int off;
        if (!a.causal) off = a.noncausal_offset;
        else {
          off = a.qo_offset_in ? a.qo_offset_in[b] : -1;
          if (off < 0) off = kl - ql;
        }
        a.qo_offset_out[b] = off;
      }
      q += ql; k += kl;
      if (a.page_size > 0) pg += (kl + a.page_size - 1) / a.page_size;
    }
    if (a.qo_start) a.qo_start[a.batch] = q;
    if (a.kv_start) a.kv_start[a.batch] = k;
    if (a.kv_page_indptr) a.kv_page_indptr[a.batch] = pg;
    s_total_q = q;
    __threadfence_block();
  }
  __syncthreads();
  // work items: (((b * RT + r) * groups) + g) * S + s, row tiles in descending order
  if (a.work) {
    const int RT = a.row_tiles;
    const int n_items = a.batch * RT * groups * S;
    const int bm_eff = (a.block_m / G) * G;
    for (int idx = threadIdx.x; idx < n_items; idx += blockDim.x) {
      const int s = idx % S, g = (idx / S) % groups, rr = (idx / (S * groups)) % RT, b = idx / (S * groups * RT);
      const int ql = a.qo_len[b], kl = a.kv_len[b];
      int off;
      if (!a.causal) off = a.noncausal_offset;
      else {
        off = a.qo_offset_in ? a.qo_offset_in[b] : -1;
        if (off < 0) off = kl - ql;
      }
      const int row0 = (RT - 1 - rr) * bm_eff;
      const int nrows = max(0, min(bm_eff, ql * G - row0));
      long long vis = nrows > 0 ? min(static_cast<long long>(kl), static_cast<long long>((row0 + nrows - 1) / G) + off + 1) : 0;
      if (vis < 0) vis = 0;
      const int nt = static_cast<int>((vis + kKvTile - 1) / kKvTile);
      const int chunk = max(1, (nt + S - 1) / S);
      MsaWorkItem w;
      w.batch = b; w.head0 = g * G; w.row0 = row0;
      w.kv_tile_begin = min(nt, s * chunk);
      w.kv_tile_end = min(nt, (s + 1) * chunk);
      w.split = s; w.num_rows = nrows; w.reserved = 0;
      a.work[idx] = w;
    }
  }
  // per-token arrays
  const int total_q = s_total_q;
  for (int t = threadIdx.x; t < a.max_total_q; t += blockDim.x) {
    if (a.splits_per_row) a.splits_per_row[t] = t < total_q ? S : 0;   // padded rows merge to 0 / LSE -inf
    if (a.token_batch) {
      int b = 0;
      if (t < total_q && a.qo_start) {                     // last b with qo_start[b] <= t (binary search)
        int lo = 0, hi = a.batch;                           // invariant: qo_start[lo] <= t < qo_start[hi]
        while (hi - lo > 1) {
          const int mid = (lo + hi) >> 1;
          if (a.qo_start[mid] <= t) lo = mid; else hi = mid;
        }
        b = lo;
      }
      a.token_batch[t] = b;
    }
  }
}

}  // namespace
}  // namespace msa

extern "C" int msa_plan_device(const MsaPlanDeviceArgs* a, msa_stream_t stream) {
  if (!a || !a->qo_len || !a->kv_len || a->batch < 0) return MSA_ERR_BAD_ARG;
  if (a->num_qo_heads <= 0 || a->num_kv_heads <= 0 || a->num_qo_heads % a->num_kv_heads) return MSA_ERR_BAD_ARG;
  if (a->pack < 1 || (a->num_qo_heads / a->num_kv_heads) % a->pack || a->pack > a->block_m) return MSA_ERR_BAD_ARG;
  if (a->num_splits < 1 || a->max_total_q < 0 || a->row_tiles < 1) return MSA_ERR_BAD_ARG;
  if (a->token_batch && !a->qo_start) return MSA_ERR_BAD_ARG;
  if (a->batch == 0) return MSA_OK;
  msa::NvtxRange range("msa_plan_device");
  msa::plan_device_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(*a);
  return cudaGetLastError() == cudaSuccess ? MSA_OK : MSA_ERR_LAUNCH;
}
