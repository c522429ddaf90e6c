// out[M, N] = x[M, K] * W[N, K]^T on the CUDA cores, 32-bit accumulation.
//
// Two kernels.  `gemm_tile_kernel` (128x128x16 tiles, 8x8 per thread) is the whole
// 32-bit engine's matrix product (FFMA only, no reduced-precision tensor mode) and
// the fallback of the bfloat16 engine for shapes its tensor-core kernel refuses.
// `gemv_rows_kernel` serves a handful of tokens (M <= 16): each warp streams weight
// rows once and multiplies them with all M activation rows, so decode at a small
// batch is bound by the read of W.
//
// Sums of thousands of 32-bit products are kept short: the tiled kernel adds up 128
// consecutive k in one register and then moves that partial sum into a second one, so
// that rounding errors grow with the square root of K/128 + 128 rather than of K (with
// K = 9,728 a plain running sum alone put logits 1.5e-5 off the exact value; the few-row
// kernel's sums are short already: a lane's share of the row, then a tree over the warp).
//
// Same contraction as the reference's src/decode.cu:202-236 (one token) and
// src/prefill.cu:124-161 (one block per output element, W re-read for every token);
// weights are [out, in] row-major, no bias.
#include "common.cuh"

// ---------------------------------------------------------------------------
// tiled kernel
// ---------------------------------------------------------------------------
namespace {
constexpr int BM = 128, BN = 128, BK = 16, PAD = 4, TILE_THREADS = 256;
constexpr int FLUSH_TILES = 8;      // partial sums over FLUSH_TILES * BK = 128 k are moved into the totals

template <typename T, typename OT>
__global__ void __launch_bounds__(TILE_THREADS)
gemm_tile_kernel(const T* __restrict__ X, const T* __restrict__ W, OT* __restrict__ out,
                 int M, int N, int K, long long ldx, long long ldw, long long ldo) {
    ti_pdl_trigger();
    __shared__ float As[BK][BM + PAD];
    __shared__ float Bs[BK][BN + PAD];
    ti_pdl_sync();
    X = ti_dependent(X);
    const int t = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int ty = t / 16, tx = t % 16;
    float acc[8][8], total[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = total[i][j] = 0.f;

    // loader mapping: 256 threads cover 64 rows x 4 groups of 4 k; two passes for 128 rows
    const int lr = t / 4, lk = (t % 4) * 4;
    int since_flush = 0;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int p = 0; p < 2; p++) {
            const int r = lr + p * 64;
            const int gm = m0 + r, gn = n0 + r;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int gk = k0 + lk + j;
                As[lk + j][r] = (gm < M && gk < K) ? to_f32(X[(size_t)gm * ldx + gk]) : 0.f;
                Bs[lk + j][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[8], b[8];
            const float4 a0 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[kk][64 + ty * 4]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&Bs[kk][64 + tx * 4]);
            a[0] = a0.x; a[1] = a0.y; a[2] = a0.z; a[3] = a0.w; a[4] = a1.x; a[5] = a1.y; a[6] = a1.z; a[7] = a1.w;
            b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (++since_flush == FLUSH_TILES) {
            since_flush = 0;
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) { total[i][j] += acc[i][j]; acc[i][j] = 0.f; }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] += total[i][j];
#pragma unroll
    for (int i = 0; i < 8; i++) {
        const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + (i - 4));
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + (j - 4));
            if (gn < N) out[(size_t)gm * ldo + gn] = from_f32<OT>(acc[i][j]);
        }
    }
}

// ---------------------------------------------------------------------------
// few rows: each warp takes weight rows n = warp, warp + total_warps, ...
// ---------------------------------------------------------------------------
constexpr int GV_ROWS = 8;       // activation rows per pass
constexpr int GV_THREADS = 256;

template <typename T, typename OT, int V>
__global__ void __launch_bounds__(GV_THREADS)
gemv_rows_kernel(const T* __restrict__ X, const T* __restrict__ W, OT* __restrict__ out,
                 int M, int N, int K, long long ldx, long long ldw, long long ldo) {
    ti_pdl_trigger();
    ti_pdl_sync();
    X = ti_dependent(X);
    const int lane = threadIdx.x & 31;
    const int warp = (blockIdx.x * GV_THREADS + threadIdx.x) >> 5;
    const int n_warps = (gridDim.x * GV_THREADS) >> 5;
    const int mb = blockIdx.y * GV_ROWS;
    const int rows = min(GV_ROWS, M - mb);
    struct alignas(sizeof(T) * V) Pack { T v[V]; };
    for (int n = warp; n < N; n += n_warps) {
        float acc[GV_ROWS];
#pragma unroll
        for (int r = 0; r < GV_ROWS; r++) acc[r] = 0.f;
        const T* wrow = W + (size_t)n * ldw;
        for (int k = lane * V; k < K; k += 32 * V) {
            float w[V];
            if constexpr (V == 1) {
                w[0] = to_f32(wrow[k]);
            } else {
                const Pack pw = *reinterpret_cast<const Pack*>(wrow + k);
#pragma unroll
                for (int j = 0; j < V; j++) w[j] = to_f32(pw.v[j]);
            }
#pragma unroll
            for (int r = 0; r < GV_ROWS; r++) {
                if (r < rows) {
                    const T* xr = X + (size_t)(mb + r) * ldx + k;
                    if constexpr (V == 1) {
                        acc[r] = fmaf(w[0], to_f32(xr[0]), acc[r]);
                    } else {
                        const Pack px = *reinterpret_cast<const Pack*>(xr);
#pragma unroll
                        for (int j = 0; j < V; j++) acc[r] = fmaf(w[j], to_f32(px.v[j]), acc[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < GV_ROWS; r++) {
            const float s = warp_sum(acc[r]);
            if (lane == 0 && r < rows) out[(size_t)(mb + r) * ldo + n] = from_f32<OT>(s);
        }
    }
}

template <typename T, typename OT>
int launch_simt(const void* x, const void* w, void* out, int M, int N, int K, long long ldx,
                long long ldw, long long ldo, cudaStream_t stream) {
    if (M <= 16) {
        constexpr int V = 16 / sizeof(T);
        const bool vec = K % V == 0 && ldx % V == 0 && ldw % V == 0 &&
                         (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0;
        const int warps_per_block = GV_THREADS / 32;
        int blocks = (N + warps_per_block - 1) / warps_per_block;
        const int cap = 148 * 8;
        if (blocks > cap) blocks = cap;
        dim3 grid(blocks, (M + GV_ROWS - 1) / GV_ROWS);
        if (vec)
            TI_CUDA(ti_launch(gemv_rows_kernel<T, OT, V>, grid, dim3(GV_THREADS), 0, stream, (const T*)x, (const T*)w, (OT*)out, M, N, K, ldx, ldw, ldo));
        else
            TI_CUDA(ti_launch(gemv_rows_kernel<T, OT, 1>, grid, dim3(GV_THREADS), 0, stream, (const T*)x, (const T*)w, (OT*)out, M, N, K, ldx, ldw, ldo));
        TI_CHECK_LAUNCH("linear (few rows)");
        return 0;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    TI_REQUIRE(grid.y <= 65535, "linear: %d rows exceed the tiled kernel's grid", M);
    TI_CUDA(ti_launch(gemm_tile_kernel<T, OT>, grid, dim3(TILE_THREADS), 0, stream, (const T*)x, (const T*)w, (OT*)out, M, N, K, ldx, ldw, ldo));
    TI_CHECK_LAUNCH("linear (tiled)");
    return 0;
}
}  // namespace

// dtype: element type of x and W.  out_f32 != 0: float32 output whatever dtype is.
extern "C" int ti_linear_simt(const void* x, const void* w, void* out, int M, int N, int K,
                              long long ldx, long long ldw, long long ldo, int dtype, int out_f32,
                              cudaStream_t stream) {
    if (M == 0 || N == 0) return 0;
    TI_REQUIRE(M > 0 && N > 0 && K > 0, "linear: bad sizes M=%d N=%d K=%d", M, N, K);
    TI_REQUIRE(ldx >= K && ldw >= K && ldo >= N, "linear: a leading dimension is smaller than its row");
    if (dtype == TI_F32) return launch_simt<float, float>(x, w, out, M, N, K, ldx, ldw, ldo, stream);
    TI_REQUIRE(dtype == TI_BF16, "linear: unknown element type code %d", dtype);
    if (out_f32) return launch_simt<bf16, float>(x, w, out, M, N, K, ldx, ldw, ldo, stream);
    return launch_simt<bf16, bf16>(x, w, out, M, N, K, ldx, ldw, ldo, stream);
}
