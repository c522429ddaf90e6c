// The many-token tcgen05 matrix product on two SMs per tile of 256 tokens x 256 weight rows.
#include "gemm_tcgen05_walk.cuh"

namespace tigemm {
int launch_walk_pair(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream) {
    TI_REQUIRE(bn == 256, "linear (tcgen05, two SMs per tile): tiles are 256 weight rows wide, not %d", bn);
    return launch_walk<256, true>(am, bm, g, sms, stream);
}
}  // namespace tigemm
