// C ABI front end: argument checks, kernel selection, the host-side dense planner.
#include <algorithm>
#include <vector>

#include "common.cuh"
#include "nvtx_range.h"

namespace msa {
int fmha_mma_launch(const MsaFmhaParams& p, cudaStream_t stream);
int fmha_tc_supported(const MsaFmhaParams& p);
int fmha_tc_launch(const MsaFmhaParams& p, cudaStream_t stream);
int score_gemv_supported(const MsaFmhaParams& p);
int score_gemv_launch(const MsaFmhaParams& p, cudaStream_t stream);
int fmha_decode_tc_supported(const MsaFmhaParams& p);
int fmha_decode_tc_launch(const MsaFmhaParams& p, cudaStream_t stream);
int fmha_sparse_tc_supported(const MsaFmhaParams& p);
int fmha_sparse_tc_launch(const MsaFmhaParams& p, cudaStream_t stream);
int64_t fmha_sparse_tc_workspace_bytes(int64_t total_q, int num_qo_heads, int num_kv_heads, int kbn, int64_t num_pages);
}  // namespace msa

namespace msa {
// Argument checks shared by every entry point that takes MsaFmhaParams.  Nothing here touches the
// device.  `own_scratch`: the split workspace is supplied by the library after this check
// (msa_fmha_fwd_split_static), so partial_o / partial_lse are expected to be NULL.
int validate_fmha(const MsaFmhaParams& p, bool own_scratch) {
  const bool sparse = (p.flags & MSA_FLAG_SPARSE) != 0;
  const bool has_o = (p.flags & MSA_FLAG_OUT_O) != 0;
  const bool has_s = (p.flags & MSA_FLAG_OUT_SCORE) != 0;
  if (!has_o && !has_s) return MSA_ERR_BAD_ARG;
  if (!p.q || !p.k || !p.qo_start || !p.kv_len || !p.qo_offset) return MSA_ERR_BAD_ARG;
  if (p.total_q < 0 || p.batch < 0) return MSA_ERR_BAD_ARG;
  if (has_o && (!p.v || (!p.out && !p.partial_o))) return MSA_ERR_BAD_ARG;
  if (has_s && (!p.max_score || p.max_k_tiles <= 0)) return MSA_ERR_BAD_ARG;
  if (own_scratch) {
    if (p.partial_o || p.partial_lse || p.num_splits < 1) return MSA_ERR_BAD_ARG;
  } else {
    if (p.partial_o && (!p.partial_lse || p.num_splits < 1)) return MSA_ERR_BAD_ARG;
    if (!p.partial_o && p.num_splits != 1) return MSA_ERR_BAD_ARG;
  }
  if (p.num_qo_heads <= 0 || p.num_kv_heads <= 0 || p.num_qo_heads % p.num_kv_heads) return MSA_ERR_BAD_ARG;
  const int h_r = p.num_qo_heads / p.num_kv_heads;
  if (p.pack < 1 || h_r % p.pack) return MSA_ERR_BAD_ARG;
  if (p.block_m != 16 && p.block_m != 64 && p.block_m != 128 && p.block_m != 256) return MSA_ERR_BAD_ARG;
  if (p.pack > p.block_m) return MSA_ERR_BAD_ARG;                 // rows of one token never straddle two items
  if (p.page_size > 0 && (!p.kv_page_indptr || !p.kv_indices)) return MSA_ERR_BAD_ARG;
  if (p.page_size <= 0 && !p.kv_start) return MSA_ERR_BAD_ARG;
  if (p.q_dtype != MSA_DT_BF16 && p.q_dtype != MSA_DT_E4M3) return MSA_ERR_UNSUPPORTED;
  if (p.kv_dtype != MSA_DT_BF16 && p.kv_dtype != MSA_DT_E4M3) return MSA_ERR_UNSUPPORTED;
  if (has_s && p.max_score_dtype != MSA_DT_F32 && p.max_score_dtype != MSA_DT_BF16) return MSA_ERR_UNSUPPORTED;
  if (sparse) {
    if (!p.kv_block_indexes || !p.token_batch || p.kv_block_num <= 0) return MSA_ERR_BAD_ARG;
    if (p.page_size != msa::kKvTile) return MSA_ERR_UNSUPPORTED;   // a selected block is one 128-key page
    if (has_s) return MSA_ERR_UNSUPPORTED;
    if (p.pack != h_r) return MSA_ERR_BAD_ARG;
  } else {
    if (p.num_work < 0 || (p.num_work > 0 && !p.work)) return MSA_ERR_BAD_ARG;
  }
  // 16-byte alignment of every row the kernels touch with vector accesses
  const int qe = p.q_dtype == MSA_DT_E4M3 ? 1 : 2, ke = p.kv_dtype == MSA_DT_E4M3 ? 1 : 2;
  auto al = [](const void* ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15) == 0; };
  if (!al(p.q) || !al(p.k) || (p.v && !al(p.v)) || (p.out && !al(p.out))) return MSA_ERR_BAD_ARG;
  if ((p.q_stride_tok * qe) % 16 || (p.q_stride_head * qe) % 16) return MSA_ERR_BAD_ARG;
  if ((p.k_stride_tok * ke) % 16 || (p.k_stride_head * ke) % 16 || (p.k_stride_page * ke) % 16) return MSA_ERR_BAD_ARG;
  if (has_o && ((p.v_stride_tok * ke) % 16 || (p.v_stride_head * ke) % 16 || (p.v_stride_page * ke) % 16)) return MSA_ERR_BAD_ARG;
  if (p.out && ((p.out_stride_tok * 2) % 16 || (p.out_stride_head * 2) % 16)) return MSA_ERR_BAD_ARG;
  return MSA_OK;
}
}  // namespace msa

extern "C" int msa_fmha_fwd(const MsaFmhaParams* pp, msa_stream_t stream_) {
  if (!pp) return MSA_ERR_BAD_ARG;
  msa::NvtxRange range("msa_fmha_fwd");
  const MsaFmhaParams& p = *pp;
  if (const int rc = msa::validate_fmha(p, false)) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (msa::fmha_sparse_tc_supported(p)) return msa::fmha_sparse_tc_launch(p, stream);
  if (msa::score_gemv_supported(p)) return msa::score_gemv_launch(p, stream);
  if (msa::fmha_decode_tc_supported(p)) return msa::fmha_decode_tc_launch(p, stream);
  if (msa::fmha_tc_supported(p)) return msa::fmha_tc_launch(p, stream);
  return msa::fmha_mma_launch(p, stream);
}

extern "C" int msa_plan_dense(const MsaPlanArgs* a, MsaWorkItem* work, int32_t capacity, int32_t* splits_per_row,
                              int32_t* max_splits_out) {
  if (!a || !a->qo_len || !a->kv_len || !a->qo_offset || (!work && capacity > 0)) return MSA_ERR_BAD_ARG;
  msa::NvtxRange range("msa_plan_dense");
  if (a->block_m != 16 && a->block_m != 64 && a->block_m != 128 && a->block_m != 256) return MSA_ERR_BAD_ARG;
  if (a->num_qo_heads <= 0 || a->num_kv_heads <= 0 || a->num_qo_heads % a->num_kv_heads) return MSA_ERR_BAD_ARG;
  const int G = a->pack;
  if (G < 1 || (a->num_qo_heads / a->num_kv_heads) % G || G > a->block_m) return MSA_ERR_BAD_ARG;
  const int groups = a->num_qo_heads / G;
  const int bm_eff = (a->block_m / G) * G;       // a token's heads never straddle two items

  struct Proto { int b, row0, nrows, ntiles; };
  std::vector<Proto> protos;
  int max_tiles = 0;
  for (int b = 0; b < a->batch; ++b) {
    const int rows = a->qo_len[b] * G;
    for (int r0 = 0; r0 < rows; r0 += bm_eff) {
      const int nrows = std::min(bm_eff, rows - r0);
      const long long i_max = (r0 + nrows - 1) / G;
      long long vis = std::min<long long>(a->kv_len[b], i_max + a->qo_offset[b] + 1);
      if (vis < 0) vis = 0;
      const int nt = static_cast<int>((vis + msa::kKvTile - 1) / msa::kKvTile);
      protos.push_back({b, r0, nrows, nt});
      max_tiles = std::max(max_tiles, nt);
    }
  }
  // one chunk size (tiles per split) for the whole plan
  int chunk;
  if (a->num_splits >= 1) {
    chunk = std::max(1, (max_tiles + a->num_splits - 1) / a->num_splits);
  } else {
    const long long items = static_cast<long long>(protos.size()) * groups;
    const int ceiling = a->num_splits < 0 ? -a->num_splits : 128;
    const int sms = a->num_sms > 0 ? a->num_sms : 148;
    if (items == 0 || items >= 2LL * sms) {
      chunk = std::max(1, max_tiles);
    } else {
      int want = static_cast<int>((2LL * sms + items - 1) / items);
      want = std::min(want, ceiling);
      chunk = std::max(4, (max_tiles + want - 1) / want);      // at least 512 keys per split
    }
  }
  std::vector<MsaWorkItem> items;
  int max_splits = 1;
  std::vector<int> tok_base(a->batch + 1, 0);
  for (int b = 0; b < a->batch; ++b) tok_base[b + 1] = tok_base[b] + a->qo_len[b];
  for (const Proto& pr : protos) {
    const int ns = std::max(1, (pr.ntiles + chunk - 1) / chunk);
    max_splits = std::max(max_splits, ns);
    if (splits_per_row) {
      const int i0 = pr.row0 / G, i1 = (pr.row0 + pr.nrows - 1) / G;
      for (int i = i0; i <= i1; ++i) splits_per_row[tok_base[pr.b] + i] = ns;
    }
    for (int g = 0; g < groups; ++g)
      for (int s = 0; s < ns; ++s) {
        MsaWorkItem w;
        w.batch = pr.b; w.head0 = g * G; w.row0 = pr.row0;
        w.kv_tile_begin = std::min(pr.ntiles, s * chunk);
        w.kv_tile_end = std::min(pr.ntiles, (s + 1) * chunk);
        w.split = s; w.num_rows = pr.nrows; w.reserved = 0;
        items.push_back(w);
      }
  }
  std::stable_sort(items.begin(), items.end(), [](const MsaWorkItem& x, const MsaWorkItem& y) {
    return (x.kv_tile_end - x.kv_tile_begin) > (y.kv_tile_end - y.kv_tile_begin);
  });
  if (max_splits_out) *max_splits_out = max_splits;
  if (static_cast<long long>(items.size()) > capacity) return MSA_ERR_TOO_LARGE;
  std::copy(items.begin(), items.end(), work);
  return static_cast<int>(items.size());
}

extern "C" int64_t msa_sparse_workspace_bytes(int64_t total_q, int32_t num_qo_heads, int32_t num_kv_heads,
                                              int32_t kv_block_num, int64_t num_logical_pages) {
  if (total_q < 0 || num_qo_heads <= 0 || num_kv_heads <= 0 || num_qo_heads % num_kv_heads || kv_block_num <= 0 ||
      num_logical_pages < 0)
    return MSA_ERR_BAD_ARG;
  return msa::fmha_sparse_tc_workspace_bytes(total_q, num_qo_heads, num_kv_heads, kv_block_num, num_logical_pages);
}

extern "C" const char* msa_status_string(int code) {
  switch (code) {
    case MSA_OK: return "ok";
    case MSA_ERR_BAD_ARG: return "bad argument (null pointer, misaligned or inconsistent sizes)";
    case MSA_ERR_UNSUPPORTED: return "unsupported combination of dtypes / modes / sizes";
    case MSA_ERR_LAUNCH: return "CUDA launch failed";
    case MSA_ERR_TOO_LARGE: return "size beyond a documented maximum";
    default: return "unknown status";
  }
}

extern "C" int msa_build_arch(void) { return 100; }

extern "C" int msa_sizeof(int which) {
  switch (which) {
    case 0: return static_cast<int>(sizeof(MsaFmhaParams));
    case 1: return static_cast<int>(sizeof(MsaWorkItem));
    case 2: return static_cast<int>(sizeof(MsaPlanArgs));
    case 3: return static_cast<int>(sizeof(MsaPlanDeviceArgs));
    default: return -1;
  }
}
