// Region (geo) shift of the LSH keys: quantile regions of two detector coordinates, the key range
// that serves as region stride, and the shifted sort keys.
//
// Reference (models/attention/hept.py:78-88, 127-138; models/model_utils/hash_utils.py:14-27,
// 333-340; models/hattention/modeling_gated_deltaproduct.py:1210-1222): every hit gets, per
// (round, head) row r, a region number floor(rank / ceil(N / R_r)) + 1 along eta and along phi,
// where rank is the hit's position in the argsort of that coordinate and R_r the row's (fractional)
// number of regions; the LSH key of the hit is then moved by
//     region_phi * range_r * (ceil(R_eta_r) + 1) + region_eta * range_r
// with range_r = max - min of the row's keys, so that hits of different regions never interleave
// in the sort.  Padded hits (index >= raw_size) get +inf and sort last.
//
// All three kernels are elementwise/reduction passes over [rows][N] fp32 and are bound by HBM;
// every product and sum is rounded separately, in the reference's order, so that the keys are
// bit-identical to the reference's elementwise torch ops on the same projections.
#include "common.cuh"
#include "profile.cuh"
#include <algorithm>

namespace lampa {

constexpr int GEO_THREADS = 256;

// min / max / (max - min) of each row of a (and of b, when given: the reference takes the range
// over queries and keys together).  One CTA per row; rows are few (rounds x heads).
__global__ void __launch_bounds__(1024)
row_range_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t n,
                 float* __restrict__ mn_out, float* __restrict__ mx_out, float* __restrict__ range_out) {
    __shared__ float smn[32], smx[32];
    const int row = blockIdx.x;
    float mn = INFINITY, mx = -INFINITY;
    const float* pa = a + (size_t)row * n;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float x = pa[i];
        mn = fminf(mn, x); mx = fmaxf(mx, x);
    }
    if (b) {
        const float* pb = b + (size_t)row * n;
        for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
            const float x = pb[i];
            mn = fminf(mn, x); mx = fmaxf(mx, x);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) { smn[threadIdx.x >> 5] = mn; smx[threadIdx.x >> 5] = mx; }
    __syncthreads();
    if (threadIdx.x < 32) {
        const int nw = blockDim.x >> 5;
        mn = threadIdx.x < nw ? smn[threadIdx.x] : INFINITY;
        mx = threadIdx.x < nw ? smx[threadIdx.x] : -INFINITY;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (threadIdx.x == 0) {
            if (mn_out) mn_out[row] = mn;
            if (mx_out) mx_out[row] = mx;
            if (range_out) range_out[row] = __fsub_rn(mx, mn);
        }
    }
}

// region number of a hit whose coordinate has rank `rank` among n hits, for a row with
// `num_regions` regions: floor(rank / ceil(n / num_regions)) + 1.  ceil() makes the divisor an
// integer-valued float, so the reference's float floor-division is an exact integer division.
__device__ __forceinline__ float region_of(int64_t rank, int64_t region_size) {
    return (float)(rank / region_size) + 1.f;
}
__device__ __forceinline__ int64_t region_size_of(int64_t n, float num_regions) {
    const float rs = ceilf(__fdiv_rn((float)n, num_regions));
    return rs >= 1.f ? (int64_t)rs : 1;
}

__global__ void __launch_bounds__(GEO_THREADS)
quantile_regions_kernel(const int64_t* __restrict__ rank, const float* __restrict__ num_regions,
                        int rows, int64_t n, float* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * GEO_THREADS + threadIdx.x;
    if (i >= n) return;
    const int64_t rk = rank[i];
    for (int r = 0; r < rows; ++r)
        out[(size_t)r * n + i] = region_of(rk, region_size_of(n, num_regions[r]));
}

// out[r][i] = proj[r][i] (+inf for padded hits, 0 when proj is NULL) + shift[r][i]
__global__ void __launch_bounds__(GEO_THREADS)
geo_keys_kernel(const float* __restrict__ proj, const float* __restrict__ reg_eta,
                const float* __restrict__ reg_phi, const int64_t* __restrict__ rank_eta,
                const int64_t* __restrict__ rank_phi, const float* __restrict__ regions_eta,
                const float* __restrict__ regions_phi, const float* __restrict__ hash_shift,
                int rows, int64_t n, int64_t raw_size, float* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * GEO_THREADS + threadIdx.x;
    if (i >= n) return;
    int64_t re = 0, rp = 0;
    if (!reg_eta) { re = rank_eta[i]; rp = rank_phi[i]; }
    for (int r = 0; r < rows; ++r) {
        const size_t at = (size_t)r * n + i;
        const float hs = hash_shift[r];
        const float e = reg_eta ? reg_eta[at] : region_of(re, region_size_of(n, regions_eta[r]));
        const float p = reg_phi ? reg_phi[at] : region_of(rp, region_size_of(n, regions_phi[r]));
        const float stride = __fadd_rn(ceilf(regions_eta[r]), 1.f);
        const float shift = __fadd_rn(__fmul_rn(__fmul_rn(p, hs), stride), __fmul_rn(e, hs));
        float base = 0.f;
        if (proj) base = i < raw_size ? proj[at] : INFINITY;
        out[at] = proj ? __fadd_rn(base, shift) : shift;
    }
}

}  // namespace lampa

using namespace lampa;

extern "C" int lampa_row_range(const float* a, const float* b, int32_t rows, int64_t n, float* mn,
                               float* mx, float* range, void* stream) {
    if (rows <= 0 || n <= 0 || !a) return LAMPA_ERR_ARG;
    ProfScope prof("row_range", (cudaStream_t)stream);
    row_range_kernel<<<rows, 1024, 0, (cudaStream_t)stream>>>(a, b, n, mn, mx, range);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_quantile_regions(const int64_t* rank, const float* num_regions, int32_t rows,
                                      int64_t n, float* out, void* stream) {
    if (rows <= 0 || n < 0) return LAMPA_ERR_ARG;
    if (n == 0) return LAMPA_OK;
    if (!rank || !num_regions || !out) return LAMPA_ERR_ARG;
    ProfScope prof("quantile_regions", (cudaStream_t)stream);
    const unsigned grid = (unsigned)((n + GEO_THREADS - 1) / GEO_THREADS);
    quantile_regions_kernel<<<grid, GEO_THREADS, 0, (cudaStream_t)stream>>>(rank, num_regions, rows, n, out);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_geo_keys(const float* proj, const float* reg_eta, const float* reg_phi,
                              const int64_t* rank_eta, const int64_t* rank_phi, const float* regions_eta,
                              const float* regions_phi, const float* hash_shift, int32_t rows, int64_t n,
                              int64_t raw_size, float* out, void* stream) {
    if (rows <= 0 || n < 0 || raw_size < 0) return LAMPA_ERR_ARG;
    if (n == 0) return LAMPA_OK;
    if (!regions_eta || !hash_shift || !out) return LAMPA_ERR_ARG;
    const bool from_regions = reg_eta && reg_phi;
    const bool from_ranks = rank_eta && rank_phi && regions_phi;
    if (!from_regions && !from_ranks) return LAMPA_ERR_ARG;
    ProfScope prof("geo_keys", (cudaStream_t)stream);
    const unsigned grid = (unsigned)((n + GEO_THREADS - 1) / GEO_THREADS);
    geo_keys_kernel<<<grid, GEO_THREADS, 0, (cudaStream_t)stream>>>(
        proj, from_regions ? reg_eta : nullptr, from_regions ? reg_phi : nullptr, rank_eta, rank_phi,
        regions_eta, regions_phi, hash_shift, rows, n, raw_size, out);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}
