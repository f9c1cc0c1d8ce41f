// Global-memory staging helpers of the preparation kernels: half rows of q / k / v as 16-byte
// loads, conversion to float and to bf16, and the lambda rows of a token.
#pragma once
#include "common.cuh"

namespace lampa {

// A thread loads half a row (D/2 elements) of a [64][D] tile as floats.
template <int D>
__device__ __forceinline__ void load_half_row(const void* base, int dt, size_t elem_off, bool valid, float (&x)[D / 2]) {
    constexpr int NE = D / 2;
    if (!valid) {
#pragma unroll
        for (int i = 0; i < NE; ++i) x[i] = 0.f;
        return;
    }
    if (dt == LAMPA_F32) {
        const float4* p = reinterpret_cast<const float4*>((const float*)base + elem_off);
#pragma unroll
        for (int i = 0; i < NE / 4; ++i) {
            const float4 f = __ldg(p + i);
            x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
        }
    } else {
        const uint4* p = reinterpret_cast<const uint4*>((const uint16_t*)base + elem_off);
#pragma unroll
        for (int i = 0; i < NE / 8; ++i) {
            const uint4 u = __ldg(p + i);
            const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f;
                if (dt == LAMPA_BF16) f = unpack_bf16x2(w[j]);
                else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
                x[8 * i + 2 * j] = f.x; x[8 * i + 2 * j + 1] = f.y;
            }
        }
    }
}

// Raw 16-byte loads of half a row of a 2-byte-element tile (issued early, converted later).
template <int D>
__device__ __forceinline__ void issue_half_row(const void* base, size_t elem_off, bool valid, uint4 (&u)[D / 16]) {
    const uint4* p = reinterpret_cast<const uint4*>((const uint16_t*)base + elem_off);
#pragma unroll
    for (int i = 0; i < D / 16; ++i) u[i] = valid ? __ldg(p + i) : make_uint4(0u, 0u, 0u, 0u);
}
template <int D>
__device__ __forceinline__ void convert_half_row(const uint4 (&u)[D / 16], int dt, float (&x)[D / 2]) {
#pragma unroll
    for (int i = 0; i < D / 16; ++i) {
        const uint32_t w[4] = {u[i].x, u[i].y, u[i].z, u[i].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f;
            if (dt == LAMPA_BF16) f = unpack_bf16x2(w[j]);
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            x[8 * i + 2 * j] = f.x; x[8 * i + 2 * j + 1] = f.y;
        }
    }
}

template <int NE>
__device__ __forceinline__ void store_half_row_bf16(__nv_bfloat16* dst, const float (&x)[NE]) {
#pragma unroll
    for (int i = 0; i < NE / 8; ++i) {
        uint4 u;
        u.x = pack_bf16x2(x[8 * i], x[8 * i + 1]);
        u.y = pack_bf16x2(x[8 * i + 2], x[8 * i + 3]);
        u.z = pack_bf16x2(x[8 * i + 4], x[8 * i + 5]);
        u.w = pack_bf16x2(x[8 * i + 6], x[8 * i + 7]);
        reinterpret_cast<uint4*>(dst)[i] = u;
    }
}

// Half of a token's lambda row (levels half, half + 2, ...) into shared memory: NIT loads in flight, then NIT stores.
template <int NIT>
__device__ __forceinline__ void stage_lambda(const void* lam, int dt, size_t base, int L, int half, bool valid, float* dst) {
    float lv[NIT];
#pragma unroll
    for (int i = 0; i < NIT; ++i) {
        const int l = half + 2 * i;
        lv[i] = (valid && l < L) ? load_as_float(lam, base + l, dt) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NIT; ++i) {
        const int l = half + 2 * i;
        if (l < L) dst[l] = lv[i];
    }
}

}  // namespace lampa
