// The arithmetic of the per-head RMS norm and the rotation on bfloat16 heads of 64 or 128
// elements, shared by the rotate-and-store kernel (many tokens) and the decode attention kernel
// (which does it for its own new token), so that a position's key is the same bits whichever of
// the two wrote it.  A head is shared by hd / 16 lanes; a lane holds 8 consecutive elements of
// the lower half and the 8 that pair with them in the upper half.
//
// Formulas (reference: norm src/decode.cu:144-187, rounded to the storage type before the
// rotation as its in-place kernel does; rotation src/decode.cu:301-324, pairs i, i + hd/2).
#pragma once

#include "common.cuh"

namespace tirope {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
        f[2 * e] = __uint_as_float(u[e] << 16);
        f[2 * e + 1] = __uint_as_float(u[e] & 0xFFFF0000u);
    }
}

__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint32_t u[4];
#pragma unroll
    for (int e = 0; e < 4; e++) {
        __nv_bfloat162 t = __floats2bfloat162_rn(f[2 * e], f[2 * e + 1]);
        u[e] = *reinterpret_cast<uint32_t*>(&t);
    }
    return make_uint4(u[0], u[1], u[2], u[3]);
}

__device__ __forceinline__ void load8(const void* w, int w_is_f32, int at, float (&f)[8]) {
    if (w_is_f32) {
        const float4* p = reinterpret_cast<const float4*>((const float*)w + at);
        const float4 x0 = p[0], x1 = p[1];
        f[0] = x0.x; f[1] = x0.y; f[2] = x0.z; f[3] = x0.w; f[4] = x1.x; f[5] = x1.y; f[6] = x1.z; f[7] = x1.w;
    } else {
        unpack8(*reinterpret_cast<const uint4*>((const bf16*)w + at), f);
    }
}

// cos and sin of one position for a lane's 8 pairs (tables are float32 [positions, hd / 2])
__device__ __forceinline__ void load_angles(const float* cos_row, const float* sin_row, int i, float (&c)[8], float (&s)[8]) {
    const float4* cp = reinterpret_cast<const float4*>(cos_row + i);
    const float4* sp = reinterpret_cast<const float4*>(sin_row + i);
    const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
    c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
    s[0] = s0.x; s[1] = s0.y; s[2] = s0.z; s[3] = s0.w; s[4] = s1.x; s[5] = s1.y; s[6] = s1.z; s[7] = s1.w;
}

// One lane's share of a head: vlo, vhi are its 8 + 8 elements (zeros for a lane without a head).
// Every lane of the warp must call this (the sum of squares goes round the head's lanes by
// shuffles); `apply` says whether this lane's head is normed and rotated at all (values are not).
// w: norm weight [HD] or null; rotate: whether c, s hold angles.  i = 8 * (lane % (HD / 16)).
template <int HD>
__device__ __forceinline__ void norm_rotate(uint4& vlo, uint4& vhi, bool apply, const void* w, int w_is_f32, float eps,
                                            bool rotate, const float (&c)[8], const float (&s)[8], int i) {
    constexpr int LPH = HD / 16, half = HD / 2;
    float lo[8], hi[8];
    unpack8(vlo, lo);
    unpack8(vhi, hi);
    float ss = 0.f;
#pragma unroll
    for (int e = 0; e < 8; e++) { ss = fmaf(lo[e], lo[e], ss); ss = fmaf(hi[e], hi[e], ss); }
#pragma unroll
    for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (!apply) return;
    if (w) {
        const float r = rsqrtf(fmaf(ss, 1.0f / (float)HD, eps));
        float wl[8], wh[8];
        load8(w, w_is_f32, i, wl);
        load8(w, w_is_f32, i + half, wh);
#pragma unroll
        for (int e = 0; e < 8; e++) {
            lo[e] = __bfloat162float(__float2bfloat16_rn(lo[e] * r * wl[e]));
            hi[e] = __bfloat162float(__float2bfloat16_rn(hi[e] * r * wh[e]));
        }
    }
    if (rotate) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const float nl = lo[e] * c[e] - hi[e] * s[e];
            const float nh = hi[e] * c[e] + lo[e] * s[e];
            lo[e] = nl; hi[e] = nh;
        }
    }
    vlo = pack8(lo);
    vhi = pack8(hi);
}

}  // namespace tirope
