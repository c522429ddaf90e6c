// The many-token tcgen05 matrix product, one block per tile of 128 tokens, tiles of 224 to 256 weight rows.
#include "gemm_tcgen05_walk.cuh"

namespace tigemm {
int launch_walk_wide(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream) {
    switch (bn) {
        case 240: return launch_walk<240, false>(am, bm, g, sms, stream);
        case 224: return launch_walk<224, false>(am, bm, g, sms, stream);
        default: return launch_walk<256, false>(am, bm, g, sms, stream);
    }
}
}  // namespace tigemm
