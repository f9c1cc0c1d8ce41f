// Fenwick-state side of the hierarchical gated-delta rule: the token levels of the final state
// after a chunkwise forward, and the single-token decode step.
//
// The state of one (batch row, head) is L matrices S_l [K][V] with counts[l] tokens each
// (models/hattention/recurrent.py:9-131).  Inserting token t first cascades (level l is merged
// into l + 1 while it is full, capacity 2^l), then applies the token's transition
// e^g (I - beta k k^T) to every level, then puts beta k v^T into level 0.  After T tokens level 0
// holds one token and level l >= 1 holds 2^(l-1) tokens exactly when bit l-1 of T - 1 is set.
#include "gdn.cuh"
#include "profile.cuh"

namespace lampa {

__device__ __forceinline__ float round_like(float x, int dt) {
    if (dt == LAMPA_BF16) return __bfloat162float(__float2bfloat16_rn(x));
    if (dt == LAMPA_F16) return __half2float(__float2half_rn(x));
    return x;
}

// -------------------------------------------------------------------------------------------------
// Token levels 0..6 of the final state: the recurrence itself over the last chunk of each sequence,
// from an empty state, as the reference's postprocess_prefill_hstate_ does
// (models/hattention/kernel.py:377-466).  Inside one chunk the cascade is fixed: before token
// t > 0, levels 0..tz(t) collapse into level tz(t) + 1 (tz = trailing zeros).  Thread (v, kq) owns
// rows kq*K/4 .. of column v of all seven levels in registers.  Also writes counts [N][L].
// A ragged last chunk is completed with null tokens (k = v = 0, beta = 0, g = 0).
// -------------------------------------------------------------------------------------------------
template <int KD, int VD>
__global__ void __launch_bounds__(VD * 4) hgdn_final_low_kernel(GdnArgs a, float* states, int32_t* counts) {
    constexpr int KQ = KD / 4;
    __shared__ float sK[CHUNK][KD + 1];
    __shared__ float sV[CHUNK][VD];
    __shared__ float sEg[CHUNK], sBeta[CHUNK];
    const int seq = blockIdx.x, h = blockIdx.y, H = a.H, L = a.L;
    const int tid = threadIdx.x, nthr = VD * 4;
    const int nch = a.chunk_off[seq + 1] - a.chunk_off[seq];
    const int vv = tid >> 2, kq = tid & 3;
    float* dst = states + ((size_t)seq * H + h) * KD * VD * L;

    if (h == 0 && tid == 0) {
        int64_t rem = (int64_t)nch * CHUNK - 1;
        int32_t* cn = counts + (size_t)seq * L;
        for (int l = L - 1; l >= 1; --l) {
            const int64_t cap = l - 1 < 40 ? (int64_t)1 << (l - 1) : (int64_t)1 << 40;
            if (nch > 0 && rem >= cap) { rem -= cap; cn[l] = (int32_t)cap; }
            else cn[l] = 0;
        }
        cn[0] = nch > 0 ? 1 : 0;
        if (nch > 0 && rem != 0) set_status(a.status, LAMPA_ERR_LEVELS, 30, seq);
    }

    float S[ELL0][KQ];
#pragma unroll
    for (int l = 0; l < ELL0; ++l)
#pragma unroll
        for (int i = 0; i < KQ; ++i) S[l][i] = 0.f;

    if (nch > 0) {
        const int64_t t0 = a.tok_off[seq] + (int64_t)(nch - 1) * CHUNK;
        const int len = (int)min((int64_t)CHUNK, a.tok_off[seq + 1] - t0);
        for (int idx = tid; idx < CHUNK * KD; idx += nthr) {
            const int r = idx / KD, c = idx - r * KD;
            sK[r][c] = r < len ? load_as_float(a.k, ((size_t)(t0 + r) * H + h) * KD + c, a.qkv_dt) : 0.f;
        }
        for (int idx = tid; idx < CHUNK * VD; idx += nthr) {
            const int r = idx / VD, c = idx - r * VD;
            sV[r][c] = r < len ? load_as_float(a.v, ((size_t)(t0 + r) * H + h) * VD + c, a.qkv_dt) : 0.f;
        }
        if (tid < CHUNK) {
            const bool in = tid < len;
            sEg[tid] = in ? __expf(load_as_float(a.g, (size_t)(t0 + tid) * H + h, a.gb_dt)) : 1.f;
            sBeta[tid] = in ? load_as_float(a.beta, (size_t)(t0 + tid) * H + h, a.gb_dt) : 0.f;
        }
        __syncthreads();
        if (a.use_l2norm) {
            if (tid < CHUNK) {
                float ss = 0.f;
                for (int c = 0; c < KD; ++c) ss += sK[tid][c] * sK[tid][c];
                const float rn = rsqrtf(ss + 1e-6f);
                for (int c = 0; c < KD; ++c) sK[tid][c] = round_like(sK[tid][c] * rn, a.qkv_dt);
            }
            __syncthreads();
        }
        for (int t = 0; t < CHUNK; ++t) {
            if (t > 0) {
                const int tz = __ffs(t) - 1;
#pragma unroll
                for (int j = 0; j < ELL0 - 1; ++j)
                    if (j <= tz) {
#pragma unroll
                        for (int i = 0; i < KQ; ++i) { S[j + 1][i] += S[j][i]; S[j][i] = 0.f; }
                    }
            }
            const float eg = sEg[t], bt = sBeta[t];
            float kr[KQ];
#pragma unroll
            for (int i = 0; i < KQ; ++i) kr[i] = sK[t][kq * KQ + i];
#pragma unroll
            for (int l = 1; l < ELL0; ++l) {
                float dot = 0.f;
#pragma unroll
                for (int i = 0; i < KQ; ++i) dot += kr[i] * S[l][i];
                dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                const float c = bt * dot;
#pragma unroll
                for (int i = 0; i < KQ; ++i) S[l][i] = eg * (S[l][i] - kr[i] * c);
            }
            const float bv = bt * sV[t][vv];
#pragma unroll
            for (int i = 0; i < KQ; ++i) S[0][i] = kr[i] * bv;
        }
    }
#pragma unroll
    for (int l = 0; l < ELL0; ++l)
        if (l < L) {
#pragma unroll
            for (int i = 0; i < KQ; ++i) dst[((size_t)(kq * KQ + i) * VD + vv) * L + l] = S[l][i];
        }
}

template <int KD, int VD>
int launch_final_low(const GdnArgs& a, float* states, int32_t* counts, cudaStream_t st) {
    ProfScope prof("hgdn_final_low", st);
    hgdn_final_low_kernel<KD, VD><<<dim3(a.nseq, a.H), VD * 4, 0, st>>>(a, states, counts);
    if (cudaGetLastError() != cudaSuccess) return LAMPA_ERR_CUDA;
    return LAMPA_OK;
}

// -------------------------------------------------------------------------------------------------
// Decode step (hattention_step -> step_state / step_output, models/hattention/kernel.py:570-633,
// recurrent.py:134-166): cascade, transition, insert, then o = q^T sum_l lambda_l S_l.  One CTA per
// (batch row, head), thread (v, kq) as above; the levels of one (k, v) element are contiguous in
// memory, so the cascade is a prefix sum over a thread's own elements.  counts is shared by the
// batch and is advanced by a second, single-thread kernel once every CTA has read it.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ int cascade_depth(const int32_t* counts, int L, int& merged, bool& overflow) {
    // levels 0 .. depth-1 move into level `depth`, which then holds `merged` tokens
    int depth = 0, carry = 0;
    overflow = false;
    merged = 0;
    for (int l = 0; l < L; ++l) {
        const int64_t cap = l < 31 ? (int64_t)1 << l : (int64_t)1 << 31;
        const int64_t cur = (int64_t)counts[l] + carry;
        if (cur == cap) {
            if (l + 1 >= L) { overflow = true; break; }
            carry = (int)cur;
            depth = l + 1;
        } else {
            if (cur > cap) overflow = true;
            merged = (int)cur;
            break;
        }
    }
    return depth;
}

template <int KD, int VD>
__global__ void __launch_bounds__(VD * 4) hgdn_step_kernel(StepArgs s) {
    constexpr int KQ = KD / 4;
    __shared__ float sK[KD], sQ[KD], sLam[64];
    const int b = blockIdx.x, h = blockIdx.y, H = s.H, L = s.L;
    const int tid = threadIdx.x;
    const int vv = tid >> 2, kq = tid & 3;
    const size_t bh = (size_t)b * H + h;
    if (tid < 32) {
        float kx[(KD + 31) / 32], qx[(KD + 31) / 32];
        float sk = 0.f, sq = 0.f;
#pragma unroll
        for (int j = 0; j < (KD + 31) / 32; ++j) {
            const int c = tid + 32 * j;
            kx[j] = c < KD ? load_as_float(s.k, bh * KD + c, s.qkv_dt) : 0.f;
            qx[j] = c < KD ? load_as_float(s.q, bh * KD + c, s.qkv_dt) : 0.f;
            sk += kx[j] * kx[j];
            sq += qx[j] * qx[j];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            sk += __shfl_xor_sync(0xffffffffu, sk, o);
            sq += __shfl_xor_sync(0xffffffffu, sq, o);
        }
        const float rk = s.use_l2norm ? rsqrtf(sk + 1e-6f) : 1.f;
        const float rq = s.use_l2norm ? rsqrtf(sq + 1e-6f) : 1.f;
#pragma unroll
        for (int j = 0; j < (KD + 31) / 32; ++j) {
            const int c = tid + 32 * j;
            if (c < KD) {
                sK[c] = s.use_l2norm ? round_like(kx[j] * rk, s.qkv_dt) : kx[j];
                sQ[c] = qx[j] * rq;
            }
        }
    }
    if (tid < L && tid < 64) sLam[tid] = load_as_float(s.lam, bh * L + tid, s.lam_dt);
    __syncthreads();

    int merged;
    bool overflow;
    const int depth = cascade_depth(s.counts, L, merged, overflow);
    if (overflow) {
        if (tid == 0 && b == 0 && h == 0) set_status(s.status, LAMPA_ERR_LEVELS, 31, depth);
        return;
    }
    const float eg = __expf(load_as_float(s.g, bh, s.gb_dt));
    const float bt = load_as_float(s.beta, bh, s.gb_dt);
    const float vt = load_as_float(s.v, bh * VD + vv, s.qkv_dt);

    float kr[KQ], qr[KQ], acc[KQ];
    float* P[KQ];
#pragma unroll
    for (int i = 0; i < KQ; ++i) {
        kr[i] = sK[kq * KQ + i];
        qr[i] = sQ[kq * KQ + i];
        P[i] = s.states + ((bh * KD + kq * KQ + i) * VD + vv) * (size_t)L;
        acc[i] = 0.f;
    }
    for (int j = 0; j <= depth; ++j)
        if (j == depth ? merged > 0 : true) {
#pragma unroll
            for (int i = 0; i < KQ; ++i) acc[i] += P[i][j];
        }
    float out = 0.f;
    for (int l = L - 1; l >= 1; --l) {
        const int cnt = l < depth ? 0 : (l == depth ? merged : s.counts[l]);
        if (cnt == 0) {
            if (l < depth) {
#pragma unroll
                for (int i = 0; i < KQ; ++i) P[i][l] = 0.f;
            }
            continue;
        }
        float val[KQ];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < KQ; ++i) {
            val[i] = l == depth ? acc[i] : P[i][l];
            dot += kr[i] * val[i];
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        const float c = bt * dot;
        float qs = 0.f;
#pragma unroll
        for (int i = 0; i < KQ; ++i) {
            const float nv = eg * (val[i] - kr[i] * c);
            P[i][l] = nv;
            qs += qr[i] * nv;
        }
        out += sLam[l] * qs;
    }
    {
        const float bv = bt * vt;
        float qs = 0.f;
#pragma unroll
        for (int i = 0; i < KQ; ++i) {
            const float nv = kr[i] * bv;
            P[i][0] = nv;
            qs += qr[i] * nv;
        }
        out += sLam[0] * qs;
    }
    out += __shfl_xor_sync(0xffffffffu, out, 1);
    out += __shfl_xor_sync(0xffffffffu, out, 2);
    if (kq == 0) store_from_float(s.o, bh * VD + vv, out, s.qkv_dt);
}

__global__ void hgdn_step_counts_kernel(int32_t* counts, int L) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int merged;
    bool overflow;
    const int depth = cascade_depth(counts, L, merged, overflow);
    if (overflow) return;
    for (int l = 0; l < depth; ++l) counts[l] = 0;
    if (depth > 0) counts[depth] = merged;
    counts[0] += 1;
}

template <int KD, int VD>
int launch_hgdn_step(const StepArgs& s, cudaStream_t st) {
    {
        ProfScope prof("hgdn_step", st);
        hgdn_step_kernel<KD, VD><<<dim3(s.B, s.H), VD * 4, 0, st>>>(s);
        if (cudaGetLastError() != cudaSuccess) return LAMPA_ERR_CUDA;
    }
    hgdn_step_counts_kernel<<<1, 32, 0, st>>>(s.counts, s.L);
    if (cudaGetLastError() != cudaSuccess) return LAMPA_ERR_CUDA;
    return LAMPA_OK;
}

#define LAMPA_INST(KD, VD)                                                                      \
    template int launch_final_low<KD, VD>(const GdnArgs&, float*, int32_t*, cudaStream_t);      \
    template int launch_hgdn_step<KD, VD>(const StepArgs&, cudaStream_t);
LAMPA_INST(64, 64)
LAMPA_INST(32, 32)
LAMPA_INST(16, 32)
#undef LAMPA_INST

}  // namespace lampa
