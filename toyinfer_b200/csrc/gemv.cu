// out[M, N] = x[M, K] w[N, K]^T for one or two tokens, bfloat16 operands, 32-bit sums.
//
// With so few rows the product is a read of the weights and nothing else: every weight is
// used M times, the tensor cores have nothing to do, and what decides the time is how many
// loads are in flight.  So there is no shared memory, no barrier and no split contraction to
// add up afterwards: a warp owns R rows of w, its lanes stride over K in pieces of 8
// elements (16 bytes), U pieces ahead, and a shuffle tree adds the lanes at the end.  Where
// the matrix has too few rows to give every SM its warps, 2, 4 or 8 warps of a block share
// the rows and each takes a part of K; their sums meet in shared memory.  The
// pieces of x are the same for every warp and come from L1.  The first weights are requested
// before the wait for the kernel before this one, which produces x.
//
// Launched early like every kernel here, except `late_start` (without the programmatic
// attribute) where it follows a kernel with large shared memory: see gemm_skinny.cu.
//
// The reference decodes one token through products of this kind, one block per output row
// and two elements per load (src/decode.cu:201-298: gemv_bf16_kernel and its float-output
// twin for the logits); the gated form applies its SwiGLU (src/decode.cu:746-764) to
// (gate, up) row pairs as they are finished.
#include "common.cuh"

namespace {
constexpr int WARPS = 8;

__device__ __forceinline__ uint4 load_stream(const bf16* p) {     // read once: no L1 allocation
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// two bfloat16 in a word -> two floats (a bfloat16 is the upper half of a float)
__device__ __forceinline__ float lo_f32(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float hi_f32(uint32_t u) { return __uint_as_float(u & 0xFFFF0000u); }

template <int M>
__device__ __forceinline__ void fma_piece(float (&acc)[M], const uint4& wv, const uint4 (&xv)[M]) {
    const float w0 = lo_f32(wv.x), w1 = hi_f32(wv.x), w2 = lo_f32(wv.y), w3 = hi_f32(wv.y);
    const float w4 = lo_f32(wv.z), w5 = hi_f32(wv.z), w6 = lo_f32(wv.w), w7 = hi_f32(wv.w);
#pragma unroll
    for (int m = 0; m < M; m++) {
        float a = acc[m];
        a = fmaf(w0, lo_f32(xv[m].x), a); a = fmaf(w1, hi_f32(xv[m].x), a);
        a = fmaf(w2, lo_f32(xv[m].y), a); a = fmaf(w3, hi_f32(xv[m].y), a);
        a = fmaf(w4, lo_f32(xv[m].z), a); a = fmaf(w5, hi_f32(xv[m].z), a);
        a = fmaf(w6, lo_f32(xv[m].w), a); a = fmaf(w7, hi_f32(xv[m].w), a);
        acc[m] = a;
    }
}

template <int M, int R, int U, int WPR, bool GATED, typename OutT>
__global__ void __launch_bounds__(WARPS * 32)
gemv_kernel(const bf16* x, const bf16* __restrict__ w, OutT* __restrict__ out, int N, int K,
            long long ldx, long long ldw, long long ldo) {
    ti_pdl_trigger();
    __shared__ float part_sum[WPR > 1 ? WARPS * R * M : 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = warp / WPR, part = warp % WPR;          // WPR warps share a group of R rows, each a part of K
    const long long row0 = ((long long)blockIdx.x * (WARPS / WPR) + group) * R;
    const int pieces = K >> 3;
    const bf16* wr[R];
#pragma unroll
    for (int r = 0; r < R; r++) wr[r] = w + (size_t)min(row0 + r, (long long)N - 1) * ldw;   // rows past the end repeat the last, unused
    float acc[R][M];
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < M; m++) acc[r][m] = 0.f;

    constexpr int STEP = 32 * WPR;
    bool waited = false;
    for (int c = part * 32 + lane; c < pieces; c += STEP * U) {
        uint4 wv[U][R];
#pragma unroll
        for (int u = 0; u < U; u++)
#pragma unroll
            for (int r = 0; r < R; r++)
                wv[u][r] = (c + STEP * u < pieces) ? load_stream(wr[r] + (size_t)(c + STEP * u) * 8) : make_uint4(0, 0, 0, 0);
        if (!waited) { ti_pdl_sync(); x = ti_dependent(x); waited = true; }      // x is the work of the kernel before this one
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int cc = min(c + STEP * u, pieces - 1);
            uint4 xv[M];
#pragma unroll
            for (int m = 0; m < M; m++) xv[m] = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + (size_t)cc * 8);
#pragma unroll
            for (int r = 0; r < R; r++) fma_piece<M>(acc[r], wv[u][r], xv);
        }
    }
    if (!waited) ti_pdl_sync();
#pragma unroll
    for (int r = 0; r < R; r++)
#pragma unroll
        for (int m = 0; m < M; m++) acc[r][m] = warp_sum(acc[r][m]);
    if (WPR > 1) {
        if (lane == 0)
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int m = 0; m < M; m++) part_sum[(warp * R + r) * M + m] = acc[r][m];
        __syncthreads();
        if (part != 0 || lane != 0) return;
#pragma unroll
        for (int p = 1; p < WPR; p++)          // in the order of the parts, whichever warp finished first
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int m = 0; m < M; m++) acc[r][m] += part_sum[((warp + p) * R + r) * M + m];
    } else if (lane != 0) {
        return;
    }
    if (GATED) {
#pragma unroll
        for (int r = 0; r < R; r += 2) {
            if (row0 + r + 1 >= N) break;
#pragma unroll
            for (int m = 0; m < M; m++) {
                const float g = acc[r][m], up = acc[r + 1][m];
                out[(size_t)m * ldo + (size_t)((row0 + r) >> 1)] = from_f32<OutT>(up * (g / (1.f + expf(-g))));
            }
        }
    } else {
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (row0 + r >= N) break;
#pragma unroll
            for (int m = 0; m < M; m++) out[(size_t)m * ldo + (size_t)(row0 + r)] = from_f32<OutT>(acc[r][m]);
        }
    }
}

// The same for one token whose input is not formed yet: x = rmsnorm(round(h + delta)) * g.  Every
// block forms x itself, in shared memory, after it has asked for its first weights: the 5 to 10 KB
// of h and delta come from L2, and the step loses a kernel whose whole work was this.  The sums run
// as in the row-wise kernel (elementwise.cu: rmsnorm_kernel), thread for thread, so both ways
// give the same bits.  Block 0 stores the rounded sum to h_out, the next reader's hidden state.
template <int R, int U, int WPR, bool GATED, typename NW>
__global__ void __launch_bounds__(WARPS * 32)
gemv_normed_kernel(const bf16* h, const bf16* delta, const NW* __restrict__ g, float eps, bf16* __restrict__ h_out,
                   const bf16* __restrict__ w, bf16* __restrict__ out, int N, int K, long long ldw) {
    ti_pdl_trigger();
    extern __shared__ __align__(16) unsigned char xs_raw[];
    bf16* xs = reinterpret_cast<bf16*>(xs_raw);                 // K elements
    __shared__ float red[33];
    __shared__ float part_sum[WPR > 1 ? WARPS * R : 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int group = warp / WPR, part = warp % WPR;
    const long long row0 = ((long long)blockIdx.x * (WARPS / WPR) + group) * R;
    const int pieces = K >> 3;
    const bf16* wr[R];
#pragma unroll
    for (int r = 0; r < R; r++) wr[r] = w + (size_t)min(row0 + r, (long long)N - 1) * ldw;
    float acc[R][1];
#pragma unroll
    for (int r = 0; r < R; r++) acc[r][0] = 0.f;

    constexpr int STEP = 32 * WPR;
    int c = part * 32 + lane;
    uint4 wv[U][R];
#pragma unroll
    for (int u = 0; u < U; u++)
#pragma unroll
        for (int r = 0; r < R; r++)
            wv[u][r] = (c + STEP * u < pieces) ? load_stream(wr[r] + (size_t)(c + STEP * u) * 8) : make_uint4(0, 0, 0, 0);
    ti_pdl_sync();
    h = ti_dependent(h); delta = ti_dependent(delta);

    float ss = 0.f;
    for (int i = threadIdx.x * 8; i < K; i += WARPS * 32 * 8) {
        uint4 hv = *reinterpret_cast<const uint4*>(h + i);
        if (delta) {
            const uint4 dv = *reinterpret_cast<const uint4*>(delta + i);
            const uint32_t* hp = &hv.x;
            const uint32_t* dp = &dv.x;
            uint32_t s4[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const __nv_bfloat162 two = __floats2bfloat162_rn(lo_f32(hp[j]) + lo_f32(dp[j]), hi_f32(hp[j]) + hi_f32(dp[j]));
                s4[j] = *reinterpret_cast<const uint32_t*>(&two);
            }
            hv = make_uint4(s4[0], s4[1], s4[2], s4[3]);
            if (blockIdx.x == 0 && h_out) *reinterpret_cast<uint4*>(h_out + i) = hv;
        }
        *reinterpret_cast<uint4*>(xs + i) = hv;
        const uint32_t* hp = &hv.x;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float a = lo_f32(hp[j]), b = hi_f32(hp[j]);
            ss = fmaf(a, a, ss);
            ss = fmaf(b, b, ss);
        }
    }
    ss = block_sum(ss, red);
    const float rs = rsqrtf(fmaf(ss, 1.0f / (float)K, eps));
    for (int i = threadIdx.x * 8; i < K; i += WARPS * 32 * 8) {
        const uint4 hv = *reinterpret_cast<const uint4*>(xs + i);      // this thread's own store
        const uint32_t* hp = &hv.x;
        uint32_t s4[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float g0 = to_f32(g[i + 2 * j]), g1 = to_f32(g[i + 2 * j + 1]);
            const __nv_bfloat162 two = __floats2bfloat162_rn(lo_f32(hp[j]) * rs * g0, hi_f32(hp[j]) * rs * g1);
            s4[j] = *reinterpret_cast<const uint32_t*>(&two);
        }
        *reinterpret_cast<uint4*>(xs + i) = make_uint4(s4[0], s4[1], s4[2], s4[3]);
    }
    __syncthreads();

    while (c < pieces) {
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int cc = min(c + STEP * u, pieces - 1);
            uint4 xv[1];
            xv[0] = *reinterpret_cast<const uint4*>(xs + (size_t)cc * 8);
#pragma unroll
            for (int r = 0; r < R; r++) fma_piece<1>(acc[r], wv[u][r], xv);
        }
        c += STEP * U;
        if (c < pieces) {
#pragma unroll
            for (int u = 0; u < U; u++)
#pragma unroll
                for (int r = 0; r < R; r++)
                    wv[u][r] = (c + STEP * u < pieces) ? load_stream(wr[r] + (size_t)(c + STEP * u) * 8) : make_uint4(0, 0, 0, 0);
        }
    }
#pragma unroll
    for (int r = 0; r < R; r++) acc[r][0] = warp_sum(acc[r][0]);
    if (WPR > 1) {
        if (lane == 0)
#pragma unroll
            for (int r = 0; r < R; r++) part_sum[warp * R + r] = acc[r][0];
        __syncthreads();
        if (part != 0 || lane != 0) return;
#pragma unroll
        for (int p = 1; p < WPR; p++)
#pragma unroll
            for (int r = 0; r < R; r++) acc[r][0] += part_sum[(warp + p) * R + r];
    } else if (lane != 0) {
        return;
    }
    if (GATED) {
#pragma unroll
        for (int r = 0; r < R; r += 2) {
            if (row0 + r + 1 >= N) break;
            const float gt = acc[r][0], up = acc[r + 1][0];
            out[(size_t)((row0 + r) >> 1)] = __float2bfloat16_rn(up * (gt / (1.f + expf(-gt))));
        }
    } else {
#pragma unroll
        for (int r = 0; r < R; r++) {
            if (row0 + r >= N) break;
            out[(size_t)(row0 + r)] = __float2bfloat16_rn(acc[r][0]);
        }
    }
}

struct Args {
    const bf16* x; const bf16* w; void* out; int N, K; long long ldx, ldw, ldo; cudaStream_t stream;
};

template <int M, int R, int WPR, bool GATED, typename OutT>
int launch(const Args& a, bool late_start) {
    constexpr int U = R == 2 ? 4 : 2;          // 128 bytes of weights in flight per lane either way
    const long long groups = ((long long)a.N + R - 1) / R;
    const long long blocks = (groups + WARPS / WPR - 1) / (WARPS / WPR);
    TI_REQUIRE(blocks <= 0x7FFFFFFFll, "linear (few tokens): %d rows of weights are too many", a.N);
    if (late_start)
        TI_CUDA(ti_launch_after(gemv_kernel<M, R, U, WPR, GATED, OutT>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, a.stream, a.x, a.w,
                                (OutT*)a.out, a.N, a.K, a.ldx, a.ldw, a.ldo));
    else
        TI_CUDA(ti_launch(gemv_kernel<M, R, U, WPR, GATED, OutT>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, a.stream, a.x, a.w,
                          (OutT*)a.out, a.N, a.K, a.ldx, a.ldw, a.ldo));
    TI_CHECK_LAUNCH("linear (few tokens)");
    return 0;
}

template <int M, int R, bool GATED, typename OutT>
int launch_wpr(const Args& a, int wpr, bool late_start) {
    switch (wpr) {
        case 1: return launch<M, R, 1, GATED, OutT>(a, late_start);
        case 2: return launch<M, R, 2, GATED, OutT>(a, late_start);
        case 4: return launch<M, R, 4, GATED, OutT>(a, late_start);
        default: return launch<M, R, 8, GATED, OutT>(a, late_start);
    }
}

template <int M, bool GATED, typename OutT>
int launch_r(const Args& a, int rows, int wpr, bool late_start) {
    return rows == 4 ? launch_wpr<M, 4, GATED, OutT>(a, wpr, late_start) : launch_wpr<M, 2, GATED, OutT>(a, wpr, late_start);
}

template <int M>
int launch_m(const Args& a, int out_f32, int gated, int rows, int wpr, bool late_start) {
    if (gated) return launch_r<M, true, bf16>(a, rows, wpr, late_start);
    if (out_f32) return launch_r<M, false, float>(a, rows, wpr, late_start);
    return launch_r<M, false, bf16>(a, rows, wpr, late_start);
}
// Measured on the shapes of 0.6B- to 32B-sized layers: with at least half of 32 warps per SM
// from two rows per warp, one warp per pair of rows is best.  With fewer rows, several warps
// share a pair so that the device fills, as long as a lane keeps a full round of loads; and
// four rows per warp halve the reads of x when the contraction is still long then, or when a
// lane keeps four loads per row and the warps still fill the device (2,560 x 4,096: 5.7 -> 5.0 us,
// one sequence's decode step on the 4B shape 2.11 -> 2.09 ms).  Alone, small matrices run faster
// with more warps per pair than this gives them (1,024 x 3,072: 4.15 -> 2.5 us with eight), but
// in a decode step they do not: a 0.6B-shaped step 0.75 -> 0.81 ms, whose kernels overlap.
void choose_shape(int M, int N, int K, int sms, int* rows_out, int* wpr_out) {
    const long long target = 32ll * (sms > 0 ? sms : 1);
    const long long pairs = ((long long)N + 1) / 2;
    const int pieces = K >> 3;
    int rows = 2, wpr = 1;
    if (pairs * 2 < target) {
        while (wpr < WARPS && pairs * wpr < target && pieces >= 32 * (wpr * 2) * 4) wpr *= 2;
        if (pieces >= 32 * wpr * 8 || (pieces >= 32 * wpr * 4 && pairs * wpr >= target)) rows = 4;
    } else if (M == 2 && pairs >= 8 * target) {
        rows = 4;
    }
    *rows_out = rows; *wpr_out = wpr;
}

struct NormedArgs {
    const bf16* h; const bf16* delta; const void* g; float eps; bf16* h_out;
    const bf16* w; bf16* out; int N, K; long long ldw; cudaStream_t stream;
};

template <int R, int WPR, bool GATED, typename NW>
int launch_normed(const NormedArgs& a) {
    constexpr int U = R == 2 ? 4 : 2;
    const long long groups = ((long long)a.N + R - 1) / R;
    const long long blocks = (groups + WARPS / WPR - 1) / (WARPS / WPR);
    TI_REQUIRE(blocks <= 0x7FFFFFFFll, "linear (one token, norm inside): %d rows of weights are too many", a.N);
    TI_CUDA(ti_launch(gemv_normed_kernel<R, U, WPR, GATED, NW>, dim3((unsigned)blocks), dim3(WARPS * 32), (size_t)a.K * sizeof(bf16),
                      a.stream, a.h, a.delta, (const NW*)a.g, a.eps, a.h_out, a.w, a.out, a.N, a.K, a.ldw));
    TI_CHECK_LAUNCH("linear (one token, norm inside)");
    return 0;
}
template <int R, bool GATED, typename NW>
int launch_normed_wpr(const NormedArgs& a, int wpr) {
    switch (wpr) {
        case 1: return launch_normed<R, 1, GATED, NW>(a);
        case 2: return launch_normed<R, 2, GATED, NW>(a);
        case 4: return launch_normed<R, 4, GATED, NW>(a);
        default: return launch_normed<R, 8, GATED, NW>(a);
    }
}
template <bool GATED, typename NW>
int launch_normed_r(const NormedArgs& a, int rows, int wpr) {
    return rows == 4 ? launch_normed_wpr<4, GATED, NW>(a, wpr) : launch_normed_wpr<2, GATED, NW>(a, wpr);
}
}  // namespace

// x[M, K] (row stride ldx), w[N, K] (row stride ldw), both bfloat16, M 1 or 2; out[M, N]
// bfloat16 or float32.  With `gated`, w's rows are (gate_0, up_0, gate_1, up_1, ...) and out is
// [M, N / 2] = up * gate / (1 + exp(-gate)) in bfloat16.  K and the strides are multiples of 8
// elements and the operands 16-byte aligned.  `sms`: the device's multiprocessors; the rows
// per warp and the warps per row are chosen so that about 32 warps per SM have work.
extern "C" int ti_linear_gemv(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                              long long ldw, long long ldo, int out_f32, int gated, int sms, int late_start,
                              cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    TI_REQUIRE(M >= 1 && M <= 2 && N > 0 && K > 0, "linear (few tokens): bad sizes M=%d N=%d K=%d", M, N, K);
    TI_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "linear (few tokens): K and the row strides must be multiples of 8 elements");
    TI_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "linear (few tokens): operands must be 16-byte aligned");
    TI_REQUIRE(!gated || (N % 2 == 0 && !out_f32), "linear (few tokens): a gated product needs an even number of weight rows and a bfloat16 result");
    int rows, wpr;
    choose_shape(M, N, K, sms, &rows, &wpr);
    Args a{(const bf16*)x, (const bf16*)w, out, N, K, ldx, ldw, ldo, stream};
    return M == 1 ? launch_m<1>(a, out_f32, gated, rows, wpr, late_start != 0) : launch_m<2>(a, out_f32, gated, rows, wpr, late_start != 0);
}

// One token whose input is still to be formed: out[N] = w[N, K] x with x = rmsnorm(round(h + delta)) * g
// (delta may be null: x = rmsnorm(h) * g); bfloat16 throughout but for g, which may be float32.
// h_out (may be null; unused without delta) receives round(h + delta).  With `gated` as above.
// K is a multiple of 8 and at most 24,576; h, delta, h_out, g and w are 16-byte aligned.
extern "C" int ti_linear_gemv_normed(const void* h, const void* delta, const void* g, int g_is_f32, float eps, void* h_out,
                                     const void* w, void* out, int N, int K, long long ldw, int gated, int sms,
                                     cudaStream_t stream) {
    if (N == 0) return 0;
    TI_REQUIRE(N > 0 && K > 0, "linear (one token, norm inside): bad sizes N=%d K=%d", N, K);
    TI_REQUIRE(K % 8 == 0 && ldw % 8 == 0 && K <= 24576, "linear (one token, norm inside): K must be a multiple of 8 up to 24576, row strides multiples of 8");
    for (const void* p : {h, delta, g, (const void*)h_out, w})
        TI_REQUIRE((reinterpret_cast<uintptr_t>(p) & 15) == 0, "linear (one token, norm inside): operands must be 16-byte aligned");
    TI_REQUIRE(!gated || N % 2 == 0, "linear (one token, norm inside): a gated product needs an even number of weight rows");
    int rows, wpr;
    choose_shape(1, N, K, sms, &rows, &wpr);
    NormedArgs a{(const bf16*)h, (const bf16*)delta, g, eps, (bf16*)h_out, (const bf16*)w, (bf16*)out, N, K, ldw, stream};
    if (g_is_f32) return gated ? launch_normed_r<true, float>(a, rows, wpr) : launch_normed_r<false, float>(a, rows, wpr);
    return gated ? launch_normed_r<true, bf16>(a, rows, wpr) : launch_normed_r<false, bf16>(a, rows, wpr);
}
