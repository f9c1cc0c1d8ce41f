// Bucketed RBF-kernel attention of the HEPT layer, with the gather into LSH order and the scatter
// back fused in.
//
// Reference (models/attention/hept.py:22-33 `qkv_res`, 141-152 of HEPTAttention.forward; copies in
// models/baselines/hmamba.py:49-60 and models/attention/flatformer.py:12-23): hits are sorted per
// (round, head) by their shifted LSH key, cut into buckets of `bucket` consecutive hits, and
// inside a bucket every query i sees every key j with weight
//     p_ij = exp(min(0, q_i . k_j - |q_i|^2 / 2 - |k_j|^2 / 2))        ( = exp(-|q_i - k_j|^2 / 2) )
//     denom_i = sum_j p_ij + 1e-20,      so_i = sum_j p_ij v_j
// after which the rows go back to hit order, the rounds are summed and so / denom is the output.
//
// One CTA per (round, head, bucket).  Keys (transposed, [d][j]) and values of the bucket are
// gathered into shared memory once; each warp then takes 4 query rows at a time: it gathers
// them, computes its 4 x 128 slice of p in registers (thread = 4 queries x 4 keys, operands read
// as 16-byte shared loads), keeps the slice in a private shared tile and multiplies it with V
// (thread = 4 queries x 4 value columns x a share of the keys).  Arithmetic is fp32 FMA: the
// exponent is a difference of large terms, which tensor-core input types cannot carry.
//
// HBM traffic per (round, head, hit): the q, k, v rows once and the so row + denom once.
#include "common.cuh"
#include "profile.cuh"
#include <algorithm>

namespace lampa {

constexpr int BA_THREADS = 256;
constexpr int BA_WARPS = BA_THREADS / 32;
constexpr int BA_MAX_BUCKET = 128;      // keys per bucket = one pass of 32 lanes x 4 keys
constexpr int BA_QROWS = 4;             // query rows per warp iteration

struct BucketAttnArgs {
    const float* q; const float* k; const float* v;         // [rounds?][heads][n][d]
    const int64_t* q_pos; const int64_t* k_pos;             // [rounds][heads][n] or NULL (rows already in order)
    float* so; float* denom;                                // [rounds][heads][n][dv], [rounds][heads][n]
    int64_t n;
    int64_t in_round_stride_q, in_round_stride_v;           // 0: q/k/v shared by all rounds (gathered by position)
    int rounds, heads, bucket, dq, dv;
    int dq4, pv, nd;     // dq rounded up to 4; value pitch (floats); value column groups of 4 per key share (power of 2)
    int scatter;         // 1: row i of a bucket is written to hit q_pos[i]; 0: to its sorted place
    int vec_store;       // so rows are 16-byte aligned: dv % 4 == 0 and an aligned base
};

__host__ __device__ inline int ba_pow2_at_least(int x) { int p = 1; while (p < x) p <<= 1; return p; }

// shared memory: sKt [dq4][128] | sV [128][pv] | per warp: sQ [4][dq4] + sP [4][128] | kn [128]
__host__ __device__ inline size_t ba_smem_floats(int dq4, int pv) {
    return (size_t)dq4 * BA_MAX_BUCKET + (size_t)BA_MAX_BUCKET * pv +
           (size_t)BA_WARPS * BA_QROWS * (dq4 + BA_MAX_BUCKET) + BA_MAX_BUCKET;
}

__global__ void __launch_bounds__(BA_THREADS) bucket_rbf_attn_kernel(BucketAttnArgs a) {
    extern __shared__ __align__(16) float ba_smem[];
    const int dq4 = a.dq4, pv = a.pv, bucket = a.bucket;
    float* sKt = ba_smem;                                           // [dq4][128]
    float* sV = sKt + (size_t)dq4 * BA_MAX_BUCKET;                  // [128][pv]
    float* sW = sV + (size_t)BA_MAX_BUCKET * pv;                    // per warp: q rows, p rows
    float* sKn = sW + (size_t)BA_WARPS * BA_QROWS * (dq4 + BA_MAX_BUCKET);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int64_t nb = a.n / bucket;
    const int64_t b = blockIdx.x % nb, rh = blockIdx.x / nb;        // rh = round * heads + head
    const int h = (int)(rh % a.heads), c = (int)(rh / a.heads);
    const int64_t row0 = b * bucket;
    const float* qbase = a.q + c * a.in_round_stride_q + (size_t)h * a.n * a.dq;
    const float* kbase = a.k + c * a.in_round_stride_q + (size_t)h * a.n * a.dq;
    const float* vbase = a.v + c * a.in_round_stride_v + (size_t)h * a.n * a.dv;
    const int64_t* qp = a.q_pos ? a.q_pos + rh * a.n + row0 : nullptr;
    const int64_t* kp = a.k_pos ? a.k_pos + rh * a.n + row0 : nullptr;

    // keys, transposed: thread = one key, every second feature (shared stores run along j)
    {
        const int j = tid & (BA_MAX_BUCKET - 1);
        const bool live = j < bucket;
        const int64_t src = live ? (kp ? kp[j] : row0 + j) : 0;
        const float* krow = kbase + (size_t)src * a.dq;
        for (int d = tid >> 7; d < dq4; d += BA_THREADS / BA_MAX_BUCKET)
            sKt[d * BA_MAX_BUCKET + j] = (live && d < a.dq) ? __ldg(krow + d) : 0.f;
    }
    // values, row-major with zero padding (rows past the bucket meet p = 0 and must be finite)
    for (int idx = tid; idx < BA_MAX_BUCKET * pv; idx += BA_THREADS) {
        const int j = idx / pv, col = idx - j * pv;
        float x = 0.f;
        if (j < bucket && col < a.dv) {
            const int64_t src = kp ? kp[j] : row0 + j;
            x = __ldg(vbase + (size_t)src * a.dv + col);
        }
        sV[idx] = x;
    }
    __syncthreads();
    if (tid < BA_MAX_BUCKET) {
        float ss = 0.f;
        for (int d = 0; d < a.dq; ++d) { const float x = sKt[d * BA_MAX_BUCKET + tid]; ss = fmaf(x, x, ss); }
        sKn[tid] = -0.5f * ss;
    }
    __syncthreads();

    float* sQ = sW + (size_t)warp * BA_QROWS * (dq4 + BA_MAX_BUCKET);   // [4][dq4]
    float* sP = sQ + BA_QROWS * dq4;                                    // [4][128]
    const int nd = a.nd, dl = lane & (nd - 1), jl = lane / nd, js = 32 / nd;
    const int jc_end = (bucket + 3) >> 2;
    const float4 kn = *reinterpret_cast<const float4*>(sKn + 4 * lane);

    for (int i0 = warp * BA_QROWS; i0 < bucket; i0 += BA_WARPS * BA_QROWS) {
        float qn[BA_QROWS];
        int64_t dst[BA_QROWS];
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) {
            const int i = i0 + r;
            const bool live = i < bucket;
            const int64_t src = live ? (qp ? qp[i] : row0 + i) : 0;
            dst[r] = (a.scatter && qp) ? src : row0 + i;
            float ss = 0.f;
            for (int d = lane; d < dq4; d += 32) {
                const float x = (live && d < a.dq) ? __ldg(qbase + (size_t)src * a.dq + d) : 0.f;
                sQ[r * dq4 + d] = x;
                ss = fmaf(x, x, ss);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            qn[r] = -0.5f * ss;
        }
        __syncwarp();

        // p = exp(min(0, q.k - |q|^2/2 - |k|^2/2)) for 4 queries x keys 4*lane .. 4*lane+3
        float acc[BA_QROWS][4];
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }
        for (int d4 = 0; d4 < dq4; d4 += 4) {
            float4 q4[BA_QROWS];
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r) q4[r] = *reinterpret_cast<const float4*>(sQ + r * dq4 + d4);
#pragma unroll
            for (int dd = 0; dd < 4; ++dd) {
                const float4 k4 = *reinterpret_cast<const float4*>(sKt + (d4 + dd) * BA_MAX_BUCKET + 4 * lane);
#pragma unroll
                for (int r = 0; r < BA_QROWS; ++r) {
                    const float qv = dd == 0 ? q4[r].x : dd == 1 ? q4[r].y : dd == 2 ? q4[r].z : q4[r].w;
                    acc[r][0] = fmaf(qv, k4.x, acc[r][0]); acc[r][1] = fmaf(qv, k4.y, acc[r][1]);
                    acc[r][2] = fmaf(qv, k4.z, acc[r][2]); acc[r][3] = fmaf(qv, k4.w, acc[r][3]);
                }
            }
        }
        float rowsum[BA_QROWS];
        const float knv[4] = {kn.x, kn.y, kn.z, kn.w};
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) {
            float p[4], s = 0.f;
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const float e = expf(fminf((acc[r][jj] + qn[r]) + knv[jj], 0.f));
                p[jj] = (4 * lane + jj < bucket) ? e : 0.f;
                s += p[jj];
            }
            *reinterpret_cast<float4*>(sP + r * BA_MAX_BUCKET + 4 * lane) = make_float4(p[0], p[1], p[2], p[3]);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
            rowsum[r] = s;
        }
        __syncwarp();

        // so = p . V for 4 queries x value columns 4*dl .. 4*dl+3, keys shared out over the js lane groups
        float o[BA_QROWS][4];
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) { o[r][0] = o[r][1] = o[r][2] = o[r][3] = 0.f; }
        for (int jc = jl; jc < jc_end; jc += js) {
            float4 p4[BA_QROWS];
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r) p4[r] = *reinterpret_cast<const float4*>(sP + r * BA_MAX_BUCKET + 4 * jc);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                const float4 v4 = *reinterpret_cast<const float4*>(sV + (size_t)(4 * jc + jj) * pv + 4 * dl);
#pragma unroll
                for (int r = 0; r < BA_QROWS; ++r) {
                    const float pj = jj == 0 ? p4[r].x : jj == 1 ? p4[r].y : jj == 2 ? p4[r].z : p4[r].w;
                    o[r][0] = fmaf(pj, v4.x, o[r][0]); o[r][1] = fmaf(pj, v4.y, o[r][1]);
                    o[r][2] = fmaf(pj, v4.z, o[r][2]); o[r][3] = fmaf(pj, v4.w, o[r][3]);
                }
            }
        }
        for (int off = nd; off < 32; off <<= 1)
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r)
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) o[r][cc] += __shfl_xor_sync(0xffffffffu, o[r][cc], off);
        if (jl == 0) {
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r) {
                if (i0 + r >= bucket) continue;
                float* orow = a.so + ((size_t)rh * a.n + dst[r]) * a.dv + 4 * dl;
                if (a.vec_store) {
                    if (4 * dl < a.dv) *reinterpret_cast<float4*>(orow) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
                } else {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                        if (4 * dl + cc < a.dv) orow[cc] = o[r][cc];
                }
                if (lane == 0) a.denom[(size_t)rh * a.n + dst[r]] = rowsum[r] + 1e-20f;
            }
        }
        __syncwarp();
    }
}

// out[row][col] = (sum over rounds of so) / (sum over rounds of denom), rounds added in order
__global__ void __launch_bounds__(256)
bucket_attn_combine_kernel(const float* __restrict__ so, const float* __restrict__ denom, int rounds,
                           int64_t rows, int dv, float* __restrict__ out) {
    const int64_t total = rows * dv;
    for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (int64_t)gridDim.x * 256) {
        const int64_t row = e / dv;
        float s = so[e], d = denom[row];
        for (int c = 1; c < rounds; ++c) { s += so[(size_t)c * total + e]; d += denom[(size_t)c * rows + row]; }
        out[e] = __fdiv_rn(s, d);
    }
}

// q_hat[h][i] = [query[i][h][:], scale[h][:] * coords[i][:]] (k_hat likewise), v_out[h][i] =
// value[i][h][:]; rows i >= raw_size are zero.  Token-major inputs, head-major outputs.
__global__ void __launch_bounds__(256)
hept_prep_qk_kernel(const float* __restrict__ query, const float* __restrict__ key, const float* __restrict__ value,
                    const float* __restrict__ scale, const float* __restrict__ coords, int64_t n, int heads,
                    int d, int cd, int64_t raw_size, float* __restrict__ q_hat, float* __restrict__ k_hat,
                    float* __restrict__ v_out) {
    const int dq = d + cd;
    const int64_t total = (int64_t)heads * n * dq;
    for (int64_t e = (int64_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (int64_t)gridDim.x * 256) {
        const int col = (int)(e % dq);
        const int64_t hi = e / dq, i = hi % n;
        const int h = (int)(hi / n);
        const bool live = i < raw_size;
        const size_t src = ((size_t)i * heads + h) * d + col;
        if (col < d) {
            q_hat[e] = live ? query[src] : 0.f;
            k_hat[e] = live ? key[src] : 0.f;
            if (v_out) v_out[(size_t)hi * d + col] = live ? value[src] : 0.f;
        } else {
            const float r = live ? __fmul_rn(scale[h * cd + col - d], coords[(size_t)i * cd + col - d]) : 0.f;
            q_hat[e] = r;
            k_hat[e] = r;
        }
    }
}

}  // namespace lampa

using namespace lampa;

extern "C" int lampa_bucket_rbf_attn(const float* q, const float* k, const float* v, const int64_t* q_pos,
                                     const int64_t* k_pos, int32_t rounds, int32_t heads, int64_t n,
                                     int32_t bucket, int32_t dq, int32_t dv, int32_t inputs_per_round,
                                     int32_t scatter, float* so, float* denom, void* stream) {
    if (rounds <= 0 || heads <= 0 || n < 0 || bucket <= 0 || dq <= 0 || dv <= 0) return LAMPA_ERR_ARG;
    if (n % bucket != 0) return LAMPA_ERR_ARG;
    if ((q_pos == nullptr) != (k_pos == nullptr)) return LAMPA_ERR_ARG;
    if (!q_pos && !inputs_per_round && rounds > 1) return LAMPA_ERR_ARG;   // nothing would tell the rounds apart
    if (n == 0) return LAMPA_OK;
    if (!q || !k || !v || !so || !denom) return LAMPA_ERR_ARG;
    if (bucket > BA_MAX_BUCKET || dv > 128 || dq > 1024) return LAMPA_ERR_UNSUPPORTED;
    BucketAttnArgs a;
    a.q = q; a.k = k; a.v = v; a.q_pos = q_pos; a.k_pos = k_pos; a.so = so; a.denom = denom;
    a.n = n; a.rounds = rounds; a.heads = heads; a.bucket = bucket; a.dq = dq; a.dv = dv;
    a.in_round_stride_q = inputs_per_round ? (int64_t)heads * n * dq : 0;
    a.in_round_stride_v = inputs_per_round ? (int64_t)heads * n * dv : 0;
    a.dq4 = (dq + 3) & ~3;
    a.nd = ba_pow2_at_least((dv + 3) >> 2);
    a.pv = a.nd >= 8 ? 4 * a.nd : 4 * a.nd + 4;
    a.scatter = scatter ? 1 : 0;
    a.vec_store = (dv % 4 == 0) && (reinterpret_cast<uintptr_t>(so) % 16 == 0);
    const size_t smem = ba_smem_floats(a.dq4, a.pv) * sizeof(float);
    if (smem > 227 * 1024) return LAMPA_ERR_UNSUPPORTED;
    const int64_t units = (int64_t)rounds * heads * (n / bucket);
    if (units > 0x7fffffffLL) return LAMPA_ERR_UNSUPPORTED;
    if (cudaFuncSetAttribute(bucket_rbf_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return LAMPA_ERR_CUDA;
    ProfScope prof("bucket_rbf_attn", (cudaStream_t)stream);
    bucket_rbf_attn_kernel<<<(unsigned)units, BA_THREADS, smem, (cudaStream_t)stream>>>(a);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_bucket_attn_combine(const float* so, const float* denom, int32_t rounds, int64_t rows,
                                         int32_t dv, float* out, void* stream) {
    if (rounds <= 0 || rows < 0 || dv <= 0) return LAMPA_ERR_ARG;
    if (rows == 0) return LAMPA_OK;
    if (!so || !denom || !out) return LAMPA_ERR_ARG;
    ProfScope prof("bucket_attn_combine", (cudaStream_t)stream);
    const int64_t total = rows * dv;
    const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 16);
    bucket_attn_combine_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(so, denom, rounds, rows, dv, out);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_hept_prep_qk(const float* query, const float* key, const float* value, const float* scale,
                                  const float* coords, int64_t n, int32_t heads, int32_t d, int32_t cd,
                                  int64_t raw_size, float* q_hat, float* k_hat, float* v_out, void* stream) {
    if (n < 0 || heads <= 0 || d <= 0 || cd < 0 || raw_size < 0) return LAMPA_ERR_ARG;
    if (n == 0) return LAMPA_OK;
    if (!query || !key || !q_hat || !k_hat || (cd > 0 && (!scale || !coords)) || (v_out && !value)) return LAMPA_ERR_ARG;
    ProfScope prof("hept_prep_qk", (cudaStream_t)stream);
    const int64_t total = (int64_t)heads * n * (d + cd);
    const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 16);
    hept_prep_qk_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(query, key, value, scale, coords, n, heads, d, cd,
                                                                 raw_size, q_hat, k_hat, v_out);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}
