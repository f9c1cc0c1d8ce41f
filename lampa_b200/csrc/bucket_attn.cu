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
// One CTA per (round, head, bucket), CTAs ordered head by head so that the rounds of a head find its
// rows in L2.  Keys, values and queries of the bucket are gathered into shared memory once, by
// position, with asynchronous copies (16-byte pieces when the rows are padded to whole pieces, else
// 4-byte pieces); each warp then takes tiles of 4 query rows: it computes its 4 x 128 slice of p in
// registers (thread = 4 queries x 4 keys, operands read as 16-byte shared loads: 8 loads per 64
// FMAs), keeps the slice in a private shared tile and multiplies it with V (thread = 4 queries x 4
// value columns x a share of the keys).  The CTA has as many warps as finish the bucket's tiles in
// whole rounds (7 for buckets of 100); three CTAs per SM at the layer's usual sizes, so that one
// CTA's gather overlaps the others' arithmetic.  Arithmetic is fp32 FMA: the exponent is a
// difference of large terms, which tensor-core input types cannot carry.
// Measured (60 000 hits, 3 rounds x 8 heads, buckets of 100, 30 + 24 features): the gather is what
// bounds the kernel - with 4-byte pieces the copy instructions alone took 17 k of a CTA's 52 k
// cycles (in-kernel counters), with 16-byte pieces and three CTAs per SM the kernel went from
// 1.40 ms to 0.97 ms.
//
// HBM traffic per (round, head, hit): the q, k, v rows once and the so row + denom once.
#include "common.cuh"
#include "profile.cuh"
#include <algorithm>

namespace lampa {

constexpr int BA_MAX_WARPS = 8;
constexpr int BA_MAX_BUCKET = 128;      // keys per bucket = one pass of 32 lanes x 4 keys

struct BucketAttnArgs {
    const float* q; const float* k; const float* v;         // [rounds?][heads][n][d]
    const int64_t* q_pos; const int64_t* k_pos;             // [rounds][heads][n] or NULL (rows already in order)
    float* so; float* denom;                                // [rounds][heads][n][dv], [rounds][heads][n]
    int64_t n;
    int64_t in_round_stride_q, in_round_stride_v;           // 0: q/k/v shared by all rounds (gathered by position)
    int rounds, heads, bucket, dq, dv;
    int ldq, ldv;        // floats between consecutive rows of q / k and of v
    int vec_qk, vec_v;   // rows can be fetched as 16-byte pieces (aligned base, pitch % 4 == 0, pitch >= width rounded up to 4)
    int dq4, pk, pv, nd; // dq rounded up to 4; key pitch (floats, pk / 4 odd); value pitch; value column groups of 4 per key share (power of 2)
    int qrows;           // bucket rounded up to whole tiles
    int scatter;         // 1: row i of a bucket is written to hit q_pos[i]; 0: to its sorted place
    int vec_store;       // so rows are 16-byte aligned: dv % 4 == 0 and an aligned base
};

__host__ __device__ inline int ba_pow2_at_least(int x) { int p = 1; while (p < x) p <<= 1; return p; }

// shared memory (floats): sK [128][pk] | sV [128][pv] | sQ [qrows][dq4] | per warp sP [4][128]
// | positions: 2 x [128] int64
__host__ __device__ inline size_t ba_smem_floats(int dq4, int pk, int pv, int qrows, int warps, int BA_QROWS) {
    return (size_t)BA_MAX_BUCKET * pk + (size_t)BA_MAX_BUCKET * pv + (size_t)qrows * dq4 +
           (size_t)warps * BA_QROWS * BA_MAX_BUCKET + 4 * BA_MAX_BUCKET;
}

// 4-byte asynchronous copy global -> shared; `live` false writes a zero without reading
__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool live) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = live ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool live) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int bytes = live ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

// BA_QROWS: query rows per warp tile.  4 (80 registers, up to three CTAs per SM) while at least two CTAs'
// shared memory fits an SM; 8 (fewer operand loads per FMA) for wide rows, where one CTA has the SM to itself.
// Measured at 60 000 hits, 3 x 8: dq 54 / dv 48 1.25 ms with 4 rows against 1.62 with 8; dq 102 / dv 96 3.63 against 3.40.
template <int BA_QROWS>
__global__ void __launch_bounds__(BA_MAX_WARPS * 32, BA_QROWS == 4 ? 3 : 2) bucket_rbf_attn_kernel(BucketAttnArgs a) {
    extern __shared__ __align__(16) float ba_smem[];
    const int dq4 = a.dq4, pk = a.pk, pv = a.pv, bucket = a.bucket;
    const int nthr = blockDim.x, nwarps = nthr >> 5;
    float* sK = ba_smem;                                            // [128][pk]
    float* sV = sK + (size_t)BA_MAX_BUCKET * pk;                    // [128][pv]
    float* sQ = sV + (size_t)BA_MAX_BUCKET * pv;                    // [qrows][dq4]
    float* sPall = sQ + (size_t)a.qrows * dq4;                      // per warp [4][128]
    int64_t* sQpos = reinterpret_cast<int64_t*>(sPall + (size_t)nwarps * BA_QROWS * BA_MAX_BUCKET);
    int64_t* sKpos = sQpos + BA_MAX_BUCKET;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    const int64_t nb = a.n / bucket;
    // CTAs run head by head, the rounds of a head back to back: a head's q, k and v rows (tens of MB)
    // are fetched from DRAM by the first round and found in L2 by the others.
    const int64_t b = blockIdx.x % nb, hc = blockIdx.x / nb;
    const int h = (int)(hc / a.rounds), c = (int)(hc % a.rounds);
    const int64_t rh = (int64_t)c * a.heads + h;                    // row of the positions and outputs
    const int64_t row0 = b * bucket;
    const float* qbase = a.q + c * a.in_round_stride_q + (size_t)h * a.n * a.ldq;
    const float* kbase = a.k + c * a.in_round_stride_q + (size_t)h * a.n * a.ldq;
    const float* vbase = a.v + c * a.in_round_stride_v + (size_t)h * a.n * a.ldv;

    for (int j = tid; j < BA_MAX_BUCKET; j += nthr) {
        const bool live = j < bucket;
        sQpos[j] = !live ? 0 : a.q_pos ? a.q_pos[rh * a.n + row0 + j] : row0 + j;
        sKpos[j] = !live ? 0 : a.k_pos ? a.k_pos[rh * a.n + row0 + j] : row0 + j;
    }
    __syncthreads();
    // Gather by position with asynchronous copies, every piece of the bucket in flight at once; a copy
    // of size 0 writes the zero padding (value rows past the bucket meet p = 0 and must be finite, query
    // rows are padded to a whole tile).  16-byte pieces where the rows allow it, else a warp per row with
    // 4-byte pieces along the row.
    if (a.vec_qk) {
        const int c4 = dq4 >> 2;
        for (int idx = tid; idx < BA_MAX_BUCKET * c4; idx += nthr) {
            const int j = idx / c4, ch = idx - j * c4;
            cp_async16(sK + j * pk + 4 * ch, kbase + (size_t)sKpos[j] * a.ldq + 4 * ch, j < bucket);
        }
        for (int idx = tid; idx < a.qrows * c4; idx += nthr) {
            const int i = idx / c4, ch = idx - i * c4;
            cp_async16(sQ + i * dq4 + 4 * ch, qbase + (size_t)sQpos[i < bucket ? i : 0] * a.ldq + 4 * ch, i < bucket);
        }
    } else {
        for (int j = warp; j < BA_MAX_BUCKET; j += nwarps) {
            const float* src = kbase + (size_t)sKpos[j] * a.ldq;
            for (int d = lane; d < dq4; d += 32)
                cp_async4(sK + j * pk + d, src + (d < a.dq ? d : 0), j < bucket && d < a.dq);
        }
        for (int i = warp; i < a.qrows; i += nwarps) {
            const float* src = qbase + (size_t)sQpos[i < bucket ? i : 0] * a.ldq;
            for (int d = lane; d < dq4; d += 32)
                cp_async4(sQ + i * dq4 + d, src + (d < a.dq ? d : 0), i < bucket && d < a.dq);
        }
    }
    if (a.vec_v) {
        const int c4 = pv >> 2, live4 = (a.dv + 3) >> 2;
        for (int idx = tid; idx < BA_MAX_BUCKET * c4; idx += nthr) {
            const int j = idx / c4, ch = idx - j * c4;
            const bool live = j < bucket && ch < live4;
            cp_async16(sV + j * pv + 4 * ch, vbase + (size_t)sKpos[j] * a.ldv + (live ? 4 * ch : 0), live);
        }
    } else {
        for (int j = warp; j < BA_MAX_BUCKET; j += nwarps) {
            const float* src = vbase + (size_t)sKpos[j] * a.ldv;
            for (int col = lane; col < pv; col += 32)
                cp_async4(sV + j * pv + col, src + (col < a.dv ? col : 0), j < bucket && col < a.dv);
        }
    }
    cp_async_wait_all();
    __syncthreads();

    float* sP = sPall + (size_t)warp * BA_QROWS * BA_MAX_BUCKET;    // [4][128]
    const int nd = a.nd, dl = lane & (nd - 1), jl = lane / nd, js = 32 / nd;
    const int jc_end = (bucket + 3) >> 2;
    // this thread's keys: lane, lane + 32, lane + 64, lane + 96 (rows pk apart, pk / 4 odd: 16-byte loads of
    // consecutive rows fall into different bank groups); -|k|^2 / 2 of each
    const float* k0 = sK + lane * pk;
    float knv[4] = {0.f, 0.f, 0.f, 0.f};
    for (int d4 = 0; d4 < dq4; d4 += 4) {
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const float4 x = *reinterpret_cast<const float4*>(k0 + cc * 32 * pk + d4);
            knv[cc] = fmaf(x.x, x.x, knv[cc]); knv[cc] = fmaf(x.y, x.y, knv[cc]);
            knv[cc] = fmaf(x.z, x.z, knv[cc]); knv[cc] = fmaf(x.w, x.w, knv[cc]);
        }
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) knv[cc] *= -0.5f;

    for (int i0 = warp * BA_QROWS; i0 < bucket; i0 += nwarps * BA_QROWS) {
        const float* q0 = sQ + (size_t)i0 * dq4;
        float qn[BA_QROWS];
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) qn[r] = 0.f;
        for (int d = lane; d < dq4; d += 32)
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r) { const float x = q0[r * dq4 + d]; qn[r] = fmaf(x, x, qn[r]); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r) qn[r] += __shfl_xor_sync(0xffffffffu, qn[r], o);
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) qn[r] *= -0.5f;

        // p = exp(min(0, q.k - |q|^2/2 - |k|^2/2)) for 4 queries x 4 keys
        float acc[BA_QROWS][4];
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) { acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f; }
        for (int d4 = 0; d4 < dq4; d4 += 4) {
            float4 q4[BA_QROWS], k4[4];
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r) q4[r] = *reinterpret_cast<const float4*>(q0 + r * dq4 + d4);
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) k4[cc] = *reinterpret_cast<const float4*>(k0 + cc * 32 * pk + d4);
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r)
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    acc[r][cc] = fmaf(q4[r].x, k4[cc].x, acc[r][cc]); acc[r][cc] = fmaf(q4[r].y, k4[cc].y, acc[r][cc]);
                    acc[r][cc] = fmaf(q4[r].z, k4[cc].z, acc[r][cc]); acc[r][cc] = fmaf(q4[r].w, k4[cc].w, acc[r][cc]);
                }
        }
        float rowsum[BA_QROWS];
#pragma unroll
        for (int r = 0; r < BA_QROWS; ++r) {
            float sum = 0.f;
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const float e = __expf(fminf((acc[r][cc] + qn[r]) + knv[cc], 0.f));
                const float pe = (lane + 32 * cc < bucket) ? e : 0.f;
                sP[r * BA_MAX_BUCKET + lane + 32 * cc] = pe;
                sum += pe;
            }
            rowsum[r] = sum;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < BA_QROWS; ++r) rowsum[r] += __shfl_xor_sync(0xffffffffu, rowsum[r], o);
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
                const int i = i0 + r;
                if (i >= bucket) continue;
                const int64_t dst = a.scatter ? sQpos[i] : row0 + i;
                float* orow = a.so + ((size_t)rh * a.n + dst) * a.dv + 4 * dl;
                if (a.vec_store) {
                    if (4 * dl < a.dv) *reinterpret_cast<float4*>(orow) = make_float4(o[r][0], o[r][1], o[r][2], o[r][3]);
                } else {
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc)
                        if (4 * dl + cc < a.dv) orow[cc] = o[r][cc];
                }
                if (lane == 0) a.denom[(size_t)rh * a.n + dst] = rowsum[r] + 1e-20f;
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
                    int d, int cd, int ldq, int64_t raw_size, float* __restrict__ q_hat, float* __restrict__ k_hat,
                    float* __restrict__ v_out) {
    const int dq = ldq;                       // columns d + cd .. ldq - 1 are zero padding
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
            const float r = (live && col < d + cd) ? __fmul_rn(scale[h * cd + col - d], coords[(size_t)i * cd + col - d]) : 0.f;
            q_hat[e] = r;
            k_hat[e] = r;
        }
    }
}

}  // namespace lampa

using namespace lampa;

extern "C" int lampa_bucket_rbf_attn(const float* q, const float* k, const float* v, const int64_t* q_pos,
                                     const int64_t* k_pos, int32_t rounds, int32_t heads, int64_t n,
                                     int32_t bucket, int32_t dq, int32_t dv, int32_t ldq, int32_t ldv,
                                     int32_t inputs_per_round, int32_t scatter, float* so, float* denom,
                                     void* stream) {
    if (rounds <= 0 || heads <= 0 || n < 0 || bucket <= 0 || dq <= 0 || dv <= 0) return LAMPA_ERR_ARG;
    if (n % bucket != 0 || ldq < dq || ldv < dv) return LAMPA_ERR_ARG;
    if ((q_pos == nullptr) != (k_pos == nullptr)) return LAMPA_ERR_ARG;
    if (!q_pos && !inputs_per_round && rounds > 1) return LAMPA_ERR_ARG;   // nothing would tell the rounds apart
    if (n == 0) return LAMPA_OK;
    if (!q || !k || !v || !so || !denom) return LAMPA_ERR_ARG;
    if (bucket > BA_MAX_BUCKET || dv > 128 || dq > 1024) return LAMPA_ERR_UNSUPPORTED;
    BucketAttnArgs a;
    a.q = q; a.k = k; a.v = v; a.q_pos = q_pos; a.k_pos = k_pos; a.so = so; a.denom = denom;
    a.n = n; a.rounds = rounds; a.heads = heads; a.bucket = bucket; a.dq = dq; a.dv = dv;
    a.ldq = ldq; a.ldv = ldv;
    a.in_round_stride_q = inputs_per_round ? (int64_t)heads * n * ldq : 0;
    a.in_round_stride_v = inputs_per_round ? (int64_t)heads * n * ldv : 0;
    a.dq4 = (dq + 3) & ~3;
    a.pk = ((a.dq4 >> 2) & 1) ? a.dq4 : a.dq4 + 4;
    a.nd = ba_pow2_at_least((dv + 3) >> 2);
    a.pv = a.nd >= 8 ? 4 * a.nd : 4 * a.nd + 4;
    a.scatter = scatter ? 1 : 0;
    auto al16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
    a.vec_qk = ldq % 4 == 0 && ldq >= a.dq4 && al16(q) && al16(k);
    a.vec_v = ldv % 4 == 0 && ldv >= ((dv + 3) & ~3) && al16(v);
    a.vec_store = (dv % 4 == 0) && (reinterpret_cast<uintptr_t>(so) % 16 == 0);
    // whole tiles of query rows, spread over as few warps as finish in the same number of rounds
    auto plan = [&](int qr, int& warps, size_t& smem) {
        const int tiles = (bucket + qr - 1) / qr;
        const int tile_rounds = (tiles + BA_MAX_WARPS - 1) / BA_MAX_WARPS;
        warps = (tiles + tile_rounds - 1) / tile_rounds;
        a.qrows = tiles * qr;
        smem = ba_smem_floats(a.dq4, a.pk, a.pv, a.qrows, warps, qr) * sizeof(float);
    };
    int warps; size_t smem;
    plan(4, warps, smem);
    const bool wide = smem > 113 * 1024;                   // not even two CTAs of 4-row tiles fit an SM
    if (wide) plan(8, warps, smem);
    if (smem > 227 * 1024) return LAMPA_ERR_UNSUPPORTED;
    const int64_t units = (int64_t)rounds * heads * (n / bucket);
    if (units > 0x7fffffffLL) return LAMPA_ERR_UNSUPPORTED;
    auto kernel = wide ? bucket_rbf_attn_kernel<8> : bucket_rbf_attn_kernel<4>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
        return LAMPA_ERR_CUDA;
    ProfScope prof("bucket_rbf_attn", (cudaStream_t)stream);
    kernel<<<(unsigned)units, warps * 32, smem, (cudaStream_t)stream>>>(a);
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
                                  int32_t ldq, int64_t raw_size, float* q_hat, float* k_hat, float* v_out,
                                  void* stream) {
    if (n < 0 || heads <= 0 || d <= 0 || cd < 0 || raw_size < 0 || ldq < d + cd) return LAMPA_ERR_ARG;
    if (n == 0) return LAMPA_OK;
    if (!query || !key || !q_hat || !k_hat || (cd > 0 && (!scale || !coords)) || (v_out && !value)) return LAMPA_ERR_ARG;
    ProfScope prof("hept_prep_qk", (cudaStream_t)stream);
    const int64_t total = (int64_t)heads * n * ldq;
    const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 16);
    hept_prep_qk_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(query, key, value, scale, coords, n, heads, d, cd,
                                                                 ldq, raw_size, q_hat, k_hat, v_out);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}
