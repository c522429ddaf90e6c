// The many-token tcgen05 matrix product, one block per tile of 128 tokens, tiles of 128 to 160 weight rows.
#include "gemm_tcgen05_walk.cuh"

namespace tigemm {
int launch_walk_narrow(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream) {
    switch (bn) {
        case 144: return launch_walk<144, false>(am, bm, g, sms, stream);
        case 128: return launch_walk<128, false>(am, bm, g, sms, stream);
        default: return launch_walk<160, false>(am, bm, g, sms, stream);
    }
}
}  // namespace tigemm
