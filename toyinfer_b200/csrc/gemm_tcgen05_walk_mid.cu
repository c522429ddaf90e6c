// The many-token tcgen05 matrix product, one block per tile of 128 tokens, tiles of 176 to 208 weight rows.
#include "gemm_tcgen05_walk.cuh"

namespace tigemm {
int launch_walk_mid(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream) {
    switch (bn) {
        case 192: return launch_walk<192, false>(am, bm, g, sms, stream);
        case 176: return launch_walk<176, false>(am, bm, g, sms, stream);
        default: return launch_walk<208, false>(am, bm, g, sms, stream);
    }
}
}  // namespace tigemm
