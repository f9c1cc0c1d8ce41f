// In-place inverse of a unit-lower-triangular 64x64 fp32 tile in shared memory, blockwise like
// the reference's solve_tril (models/hattention/solve_tril.py:221-276), and the split-bf16
// tensor-core fragments it uses.  Shared by the preparation kernels.
#pragma once
#include "common.cuh"

namespace lampa {

template <int N>
__device__ __forceinline__ void zero_acc(float (&acc)[N][4]) {
#pragma unroll
    for (int i = 0; i < N; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
}

// -------------------------------------------------------------------------------------------------
// Split-bf16 fragments for products that must keep fp32 accuracy (the blockwise triangular inverse):
// operands live as fp32 in shared memory and enter the tensor core as bf16 hi + bf16 lo.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void split2(float x, float y, uint32_t& hi, uint32_t& lo) {
    hi = pack_bf16x2(x, y);
    const float2 h = unpack_bf16x2(hi);
    lo = pack_bf16x2(x - h.x, y - h.y);
}
// A fragment (rows r0.., columns c0.. of an fp32 tile in shared memory), split into hi and lo
__device__ __forceinline__ void load_a_f32(const float* s, int pitch, int r0, int c0, int lane,
                                           uint32_t (&hi)[4], uint32_t (&lo)[4]) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float2 v = *reinterpret_cast<const float2*>(s + (r0 + g + (q & 1) * 8) * pitch + c0 + 2 * t + (q >> 1) * 8);
        split2(v.x, v.y, hi[q], lo[q]);
    }
}
// B fragment of the 16 x 8 block B[k][n] = s[(k0 + k) * pitch + n0 + n]
__device__ __forceinline__ void load_b_f32(const float* s, int pitch, int k0, int n0, int lane,
                                           uint32_t (&hi)[2], uint32_t (&lo)[2]) {
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int q = 0; q < 2; ++q)
        split2(s[(k0 + 2 * t + 8 * q) * pitch + n0 + g], s[(k0 + 2 * t + 1 + 8 * q) * pitch + n0 + g], hi[q], lo[q]);
}
__device__ __forceinline__ void mma3(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                     const uint32_t (&bh)[2], const uint32_t (&bl)[2]) {
    mma16816(c, ah, bh[0], bh[1]);
    mma16816(c, al, bh[0], bh[1]);
    mma16816(c, ah, bl[0], bl[1]);
}
// two adjacent accumulator tiles (16 x 16) as the A fragment of the next product
__device__ __forceinline__ void acc_to_a(const float (&c0)[4], const float (&c1)[4], uint32_t (&hi)[4], uint32_t (&lo)[4]) {
    split2(c0[0], c0[1], hi[0], lo[0]);
    split2(c0[2], c0[3], hi[1], lo[1]);
    split2(c1[0], c1[1], hi[2], lo[2]);
    split2(c1[2], c1[3], hi[3], lo[3]);
}
// s[r0 + ..][c0 + 8 nt + ..] = -acc
__device__ __forceinline__ void store_neg_tile(float* s, int pitch, int r0, int c0, int lane, const float (&c)[4]) {
    const int g = lane >> 2, t = lane & 3;
    *reinterpret_cast<float2*>(s + (r0 + g) * pitch + c0 + 2 * t) = make_float2(-c[0], -c[1]);
    *reinterpret_cast<float2*>(s + (r0 + g + 8) * pitch + c0 + 2 * t) = make_float2(-c[2], -c[3]);
}


// s holds A0 (strictly lower triangular; everything on and above the diagonal is ignored and the
// blocks above the diagonal must be zero on return, which they are if they were zero on entry).
// Called by every warp of the CTA: warp `blk` (0..3) of a tile owns rows 16 blk .. 16 blk + 15,
// inverts its own 16x16 diagonal block of I + A0 by fp32 forward substitution (lane = column) and
// the off-diagonal blocks follow as X_ba = -(X_bb A_ba) X_aa, first inside the two 32x32 halves,
// then for the 32x32 corner, in place.  Those products keep fp32 accuracy by splitting each operand
// into bf16 hi + lo and issuing hi*hi + lo*hi + hi*lo (the reference asks for IEEE fp32 dots there).
// Contains CTA-wide barriers: every warp of the CTA calls it; warps that own no block pass active = false.
template <int PA>
__device__ __forceinline__ void tril_inverse_64(float* sA, int blk, int lane, bool active = true) {
    const int m0 = blk * 16;
    if (active) {
        const int cc = lane & 15;
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            float sum = (i == cc) ? 1.f : 0.f, sum2 = 0.f;    // two partial sums: half the dependent chain
#pragma unroll
            for (int q = 0; q < (i + 3) / 4; ++q) {
                const float4 av = *reinterpret_cast<const float4*>(sA + (m0 + i) * PA + m0 + 4 * q);
                const float ae[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (4 * q + e < i) {
                        if (e & 1) sum2 -= ae[e] * x[4 * q + e];
                        else sum -= ae[e] * x[4 * q + e];
                    }
            }
            x[i] = sum + sum2;
        }
        __syncwarp();
        if (lane < 16) {
#pragma unroll
            for (int i = 0; i < 16; ++i) sA[(m0 + i) * PA + m0 + cc] = x[i];
        }
    }
    __syncthreads();
    if (active && (blk & 1)) {   // X_ba of the pair (a, b) = (blk - 1, blk)
        const int ra = m0 - 16, rb = m0;
        float q0[2][4], xo[2][4];
        zero_acc<2>(q0);
        zero_acc<2>(xo);
        uint32_t ah[4], al[4];
        load_a_f32(sA, PA, rb, rb, lane, ah, al);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            uint32_t bh[2], bl[2];
            load_b_f32(sA, PA, rb, ra + 8 * nt, lane, bh, bl);
            mma3(q0[nt], ah, al, bh, bl);
        }
        acc_to_a(q0[0], q0[1], ah, al);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            uint32_t bh[2], bl[2];
            load_b_f32(sA, PA, ra, ra + 8 * nt, lane, bh, bl);
            mma3(xo[nt], ah, al, bh, bl);
        }
        __syncwarp();
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) store_neg_tile(sA, PA, rb, ra + 8 * nt, lane, xo[nt]);
    }
    __syncthreads();
    // the 32x32 corner: warp = (row tile mt, column half nh)
    const int mt = blk >> 1, nh = blk & 1;
    float xc[2][4];
    zero_acc<2>(xc);
    if (active) {
        float qc[4][4];
        zero_acc<4>(qc);
#pragma unroll
        for (int ks = 0; ks < 2; ++ks)
            if (ks <= mt) {                                   // X_b is block lower-triangular
                uint32_t ah[4], al[4];
                load_a_f32(sA, PA, 32 + 16 * mt, 32 + 16 * ks, lane, ah, al);
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) {
                    uint32_t bh[2], bl[2];
                    load_b_f32(sA, PA, 32 + 16 * ks, 8 * nt, lane, bh, bl);
                    mma3(qc[nt], ah, al, bh, bl);
                }
            }
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t ah[4], al[4];
            acc_to_a(qc[2 * ks], qc[2 * ks + 1], ah, al);
#pragma unroll
            for (int n = 0; n < 2; ++n) {
                const int nt = 2 * nh + n;
                if (nt < 2 + 2 * ks) {                        // X_a rows 0..15 are [X_00 | 0]
                    uint32_t bh[2], bl[2];
                    load_b_f32(sA, PA, 16 * ks, 8 * nt, lane, bh, bl);
                    mma3(xc[n], ah, al, bh, bl);
                }
            }
        }
    }
    __syncthreads();                                          // every warp has read A_ba
    if (active) {
#pragma unroll
        for (int n = 0; n < 2; ++n) store_neg_tile(sA, PA, 32 + 16 * mt, 8 * (2 * nh + n), lane, xc[n]);
    }
    __syncthreads();
}

}  // namespace lampa
