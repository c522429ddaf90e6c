// The many-token tcgen05 matrix product on two SMs per tile of 256 tokens: 256 weight rows, or a
// wider tile with one accumulator (see gemm_tcgen05_walk.cuh).
#include "gemm_tcgen05_walk.cuh"

namespace tigemm {
int launch_walk_pair(int bn, const CUtensorMap& am, const CUtensorMap& bm, const GemmArgs& g, int sms, cudaStream_t stream) {
    switch (bn) {
        case 256: return launch_walk<256, true>(am, bm, g, sms, stream);
        case 288: return launch_walk<288, true>(am, bm, g, sms, stream);
        case 320: return launch_walk<320, true>(am, bm, g, sms, stream);
        case 384: return launch_walk<384, true>(am, bm, g, sms, stream);
        case 512: return launch_walk<512, true>(am, bm, g, sms, stream);
        default: break;
    }
    TI_FAIL("linear (tcgen05, two SMs per tile): no kernel for tiles of %d weight rows", bn);
}
}  // namespace tigemm
