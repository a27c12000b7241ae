// tcgen05 / TMEM FMHA forward (placeholder selection hook until the kernel lands).
#include "common.cuh"

namespace msa {
int fmha_tc_supported(const MsaFmhaParams&) { return 0; }
int fmha_tc_launch(const MsaFmhaParams&, cudaStream_t) { return MSA_ERR_UNSUPPORTED; }
}  // namespace msa
