// The many-token tcgen05 matrix product, one block per tile of 128 tokens: which file holds
// which tile widths (three files, so that the template instances compile side by side).
#include "gemm_tcgen05.cuh"

namespace tigemm {
int launch_walk_wide(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream);
int launch_walk_mid(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream);
int launch_walk_narrow(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream);

int launch_walk_single(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream) {
    if (bn >= 224) return launch_walk_wide(bn, am, bm, g, sms, stream);
    if (bn >= 176) return launch_walk_mid(bn, am, bm, g, sms, stream);
    return launch_walk_narrow(bn, am, bm, g, sms, stream);
}
}  // namespace tigemm
