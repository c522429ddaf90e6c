// out[M, N] = x[M, K] w[N, K]^T for a handful of tokens (up to 16), bfloat16 operands,
// float32 accumulation on the tensor cores, operands loaded straight from global memory into
// the MMA's registers.
//
// With few tokens the product is a read of the weights; what decides its time is how many
// bytes are in flight and how little happens between a kernel's start and its first load.
// This kernel has no shared-memory pipeline to fill, no tensor memory to allocate and no
// split contraction to add up in a second pass:
//   * a warp owns 16 rows of w and walks K in steps of 64.  Lane (g, t) = (lane / 4, lane % 4)
//     loads 32 bytes (16 consecutive k) of rows g and g + 8 at k offset 16 t, and 32 bytes of
//     token g of x at the same offset: four lanes read one whole 128-byte line of a row.  The
//     contraction does not care in which order k is visited, so each 8 of those elements feed
//     two m16n8k16 MMAs as they lie: the MMA's k index (2t, 2t+1, 2t+8, 2t+9) stands for the
//     lane's elements (0, 1, 2, 3), then (4, 5, 6, 7) — the same renaming on both operands.  No
//     ldmatrix, no transposition, every load 16 bytes;
//   * loads run UNROLL steps (128 bytes of weights per lane) ahead of the MMAs; the first ones
//     are issued before the wait for the kernel before this one, which produces x;
//   * where the matrix has too few rows to occupy the SMs, the warps of a block share a
//     row group and each takes a slice of K; their partial sums meet in shared memory and are
//     added in slice order.
// x is read from L1/L2 by every warp (at most 16 tokens: it stays resident).
//
// Launch: every block reads all of x, and that is cheap only while x sits in L1.  Blocks that
// start while a kernel with large shared memory is still on the SMs (decode attention: 100 KB
// per block) find the SMs configured with next to no L1, and the configuration stays while
// kernels keep overlapping.  So the product that follows such a kernel is launched `late_start`:
// without the programmatic attribute, when its predecessor has finished and the SMs have
// drained; the other products of a layer start early like every kernel here.  Measured in a
// 36-layer decode step at 8 sequences of 8,192: all late 3.78 ms, all early 5.40, early except
// after the attention 3.69; late with the shared-memory carve-out forced to its maximum 4.9 at
// 2,048 positions against 2.8; the tcgen05 kernel in this one's place 3.0 against 2.8.
#include "common.cuh"
#include "mma_utils.cuh"

namespace {
constexpr int UNROLL = 2;

__device__ __forceinline__ uint4 load_stream(const bf16* p) {     // read once: no L1 allocation
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

struct Args {
    const bf16* x; const bf16* w; void* out;
    int M, N, K;
    long long ldx, ldw, ldo;
    int rows;       // weight rows per group, 8 to 16 (even for a gated product): see rows_per_group
};

// NT: token tiles of 8 (1 or 2); WARPS per block; WPR: warps that share a group of 16 rows.
template <int NT, int WARPS, int WPR, bool GATED, typename OutT>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 16 ? 2 : 3) skinny_kernel(Args a) {
    ti_pdl_trigger();
    __shared__ float part[WPR > 1 ? WARPS * NT * 4 * 32 : 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int group = warp / WPR, slice = warp % WPR;
    const int R = a.rows;
    const long long r0 = ((long long)blockIdx.x * (WARPS / WPR) + group) * R;
    const int steps = (a.K + 63) >> 6;
    const int per = (steps + WPR - 1) / WPR;
    const int s0 = slice * per, s1 = min(steps, s0 + per);
    // of the MMA's 16 rows the group has the first R; the others, and rows past the matrix's end, are
    // not loaded (zeros), and their sums are never stored
    const bool lo_ok = g < R && r0 + g < a.N, hi_ok = g + 8 < R && r0 + g + 8 < a.N;
    const bf16* w_lo = a.w + (size_t)min(r0 + g, (long long)a.N - 1) * a.ldw + 16 * t;
    const bf16* w_hi = a.w + (size_t)min(r0 + g + 8, (long long)a.N - 1) * a.ldw + 16 * t;
    const bf16* x = a.x;
    float c[NT][4];
#pragma unroll
    for (int n = 0; n < NT; n++) c[n][0] = c[n][1] = c[n][2] = c[n][3] = 0.f;

    bool waited = false;
    for (int s = s0; s < s1; s += UNROLL) {
        uint4 wl[UNROLL][2], wh[UNROLL][2];
#pragma unroll
        for (int u = 0; u < UNROLL; u++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int k = (s + u) * 64 + 16 * t + 8 * h;
                const bool ok = s + u < s1 && k < a.K;          // K is a multiple of 8: a piece is whole or absent
                wl[u][h] = ok && lo_ok ? load_stream(w_lo + (size_t)(s + u) * 64 + 8 * h) : make_uint4(0, 0, 0, 0);
                wh[u][h] = ok && hi_ok ? load_stream(w_hi + (size_t)(s + u) * 64 + 8 * h) : make_uint4(0, 0, 0, 0);
            }
        if (!waited) { ti_pdl_sync(); x = ti_dependent(x); waited = true; }      // x is the work of the kernel before this one
        // every piece of x of these steps (for one tile of 8 tokens at a time) is asked for before
        // the tile's first MMA: the warp waits for x once per tile, not once per piece
#pragma unroll
        for (int n = 0; n < NT; n++) {
            const int tok = min(n * 8 + g, a.M - 1);        // tokens past the end repeat the last; never stored
            uint4 xv[UNROLL][2];
#pragma unroll
            for (int u = 0; u < UNROLL; u++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int k = (s + u) * 64 + 16 * t + 8 * h;
                    const bool ok = s + u < s1 && k < a.K;
                    xv[u][h] = ok ? *reinterpret_cast<const uint4*>(x + (size_t)tok * a.ldx + k) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
            for (int u = 0; u < UNROLL; u++)
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t a1[4] = {wl[u][h].x, wh[u][h].x, wl[u][h].y, wh[u][h].y};
                    const uint32_t a2[4] = {wl[u][h].z, wh[u][h].z, wl[u][h].w, wh[u][h].w};
                    mma_bf16(c[n], a1, xv[u][h].x, xv[u][h].y);
                    mma_bf16(c[n], a2, xv[u][h].z, xv[u][h].w);
                }
        }
    }
    if (!waited) ti_pdl_sync();

    if (WPR > 1) {
#pragma unroll
        for (int n = 0; n < NT; n++)
#pragma unroll
            for (int e = 0; e < 4; e++) part[((warp * NT + n) * 4 + e) * 32 + lane] = c[n][e];
        __syncthreads();
        if (slice != 0) return;
#pragma unroll
        for (int p = 1; p < WPR; p++)
#pragma unroll
            for (int n = 0; n < NT; n++)
#pragma unroll
                for (int e = 0; e < 4; e++) c[n][e] += part[(((warp + p) * NT + n) * 4 + e) * 32 + lane];
    }
    // c[n][0..1]: row r0 + g, tokens n*8 + 2t, 2t + 1;  c[n][2..3]: row r0 + g + 8, same tokens
    OutT* out = (OutT*)a.out;
#pragma unroll
    for (int n = 0; n < NT; n++) {
        if (GATED) {
            // rows come in (gate, up) pairs: the partner row lives four lanes away
            float other[4];
#pragma unroll
            for (int e = 0; e < 4; e++) other[e] = __shfl_xor_sync(0xffffffffu, c[n][e], 4);
            if ((g & 1) == 0) {
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int in_group = g + (e >> 1) * 8;
                    const long long row = r0 + in_group;
                    const int tok = n * 8 + 2 * t + (e & 1);
                    if (in_group + 1 < R && row + 1 < a.N && tok < a.M) {
                        const float gate = c[n][e], up = other[e];
                        out[(size_t)tok * a.ldo + (size_t)(row >> 1)] = from_f32<OutT>(up * (gate / (1.f + expf(-gate))));
                    }
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int in_group = g + (e >> 1) * 8;
                const long long row = r0 + in_group;
                const int tok = n * 8 + 2 * t + (e & 1);
                if (in_group < R && row < a.N && tok < a.M) out[(size_t)tok * a.ldo + (size_t)row] = from_f32<OutT>(c[n][e]);
            }
        }
    }
}

int rows_per_group(int N, long long places, bool gated);

template <int NT, int WARPS, int WPR, bool GATED, typename OutT>
int launch(Args a, int sms, bool late_start, cudaStream_t stream) {
    // blocks of this kernel that an SM holds at once, as the runtime counts them (asked once)
    static int per_sm = 0;
    if (per_sm == 0) {
        TI_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, skinny_kernel<NT, WARPS, WPR, GATED, OutT>, WARPS * 32, 0));
        if (per_sm < 1) per_sm = 1;
    }
    a.rows = rows_per_group(a.N, (long long)(sms > 0 ? sms : 1) * per_sm * (WARPS / WPR), GATED);
    const long long groups = ((long long)a.N + a.rows - 1) / a.rows;
    const long long blocks = (groups + WARPS / WPR - 1) / (WARPS / WPR);
    TI_REQUIRE(blocks <= 0x7FFFFFFFll, "linear (small batch): %d rows of weights are too many", a.N);
    if (late_start)
        TI_CUDA(ti_launch_after(skinny_kernel<NT, WARPS, WPR, GATED, OutT>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, a));
    else
        TI_CUDA(ti_launch(skinny_kernel<NT, WARPS, WPR, GATED, OutT>, dim3((unsigned)blocks), dim3(WARPS * 32), 0, stream, a));
    TI_CHECK_LAUNCH("linear (small batch)");
    return 0;
}

template <int NT, bool GATED, typename OutT>
int launch_wpr(const Args& a, int wpr, int sms, bool late_start, cudaStream_t stream) {
    switch (wpr) {
        case 1: return launch<NT, 8, 1, GATED, OutT>(a, sms, late_start, stream);
        case 2: return launch<NT, 8, 2, GATED, OutT>(a, sms, late_start, stream);
        case 4: return launch<NT, 8, 4, GATED, OutT>(a, sms, late_start, stream);
        case 8: return launch<NT, 8, 8, GATED, OutT>(a, sms, late_start, stream);
        default: return launch<NT, 16, 16, GATED, OutT>(a, sms, late_start, stream);
    }
}

template <int NT>
int launch_nt(const Args& a, int out_f32, int gated, int wpr, int sms, bool late_start, cudaStream_t stream) {
    if (gated) return launch_wpr<NT, true, bf16>(a, wpr, sms, late_start, stream);
    if (out_f32) return launch_wpr<NT, false, float>(a, wpr, sms, late_start, stream);
    return launch_wpr<NT, false, bf16>(a, wpr, sms, late_start, stream);
}

// Weight rows per group.  What bounds a product whose blocks all fit the SMs at once is the SM that has
// most to read: 2,560 rows in groups of 16 are 160 blocks for 148 SMs, twelve SMs read twice as much as
// the others and the rest wait for them (measured at 8 tokens, contraction 9,728: 148 groups 9.8 us, 149
// groups 11.8, 160 groups 12.0, 296 groups 17.1).  So where groups of 16 rows leave places free, the
// groups shrink (down to 8 rows; the MMA's other rows stay empty) until the blocks fill the places
// that the SMs offer (`places`: groups on the SMs at once): 285 groups of 9 rows for 296 places.
int g_force_rows = 0;       // for tests: every group size on any device
int rows_per_group(int N, long long places, bool gated) {
    if (g_force_rows) return gated && (g_force_rows & 1) ? g_force_rows + 1 : g_force_rows;
    if (((long long)N + 15) / 16 > places) return 16;
    int rows = (int)((N + places - 1) / places);
    if (rows < 8) rows = 8;
    if (gated && (rows & 1)) rows++;
    return rows > 16 ? 16 : rows;
}
}  // namespace

// For tests on the host: the rows per group that a product of N weight rows takes when the SMs hold `places` groups at once.
extern "C" int ti_skinny_rows_per_group(int N, long long places, int gated) { return rows_per_group(N, places, gated != 0); }

// For tests: 8 to 16 weight rows per group whatever the shape (0: chosen by shape and device again).
extern "C" void ti_set_skinny_rows(int rows) { g_force_rows = rows >= 8 && rows <= 16 ? rows : 0; }

// x[M, K] (row stride ldx), w[N, K] (row stride ldw), both bfloat16, M from 1 to 16; out[M, N]
// bfloat16 or float32.  With `gated`, w's rows are (gate_0, up_0, gate_1, up_1, ...) and out is
// [M, N / 2] = up * gate / (1 + exp(-gate)) in bfloat16.  K and the strides are multiples of 8
// elements and the operands 16-byte aligned.  `sms`: the device's multiprocessors.  `late_start`:
// see the note on launching at the top of this file.
extern "C" int ti_linear_skinny(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                                long long ldw, long long ldo, int out_f32, int gated, int sms, int late_start,
                                cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    TI_REQUIRE(M >= 1 && M <= 16 && N > 0 && K > 0, "linear (small batch): bad sizes M=%d N=%d K=%d", M, N, K);
    TI_REQUIRE(K % 8 == 0 && ldx % 8 == 0 && ldw % 8 == 0, "linear (small batch): K and the row strides must be multiples of 8 elements");
    TI_REQUIRE((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0,
               "linear (small batch): operands must be 16-byte aligned");
    TI_REQUIRE(!gated || (N % 2 == 0 && !out_f32), "linear (small batch): a gated product needs an even number of weight rows and a bfloat16 result");
    // Warps per row group, measured on the shapes of 4B- and 32B-sized layers: what counts is
    // how many warps have loads in flight, so a group's contraction is cut into 8 slices
    // whenever each slice keeps two steps, and into 16 (blocks of 16 warps, registers capped
    // so that two fit an SM) when the matrix has too few rows to give every SM 16 warps.
    const long long target = 16ll * (sms > 0 ? sms : 1);
    const long long groups = ((long long)N + 15) / 16;
    const int steps = (K + 63) / 64;
    int wpr = 1;
    while (wpr < 8 && steps >= (wpr * 2) * UNROLL) wpr *= 2;
    if (wpr == 8 && groups * 8 < target && steps >= 16 * UNROLL) wpr = 16;
    Args a{(const bf16*)x, (const bf16*)w, out, M, N, K, ldx, ldw, ldo, 16};
    return M <= 8 ? launch_nt<1>(a, out_f32, gated, wpr, sms, late_start != 0, stream)
                  : launch_nt<2>(a, out_f32, gated, wpr, sms, late_start != 0, stream);
}
