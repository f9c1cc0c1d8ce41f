// Elementwise producers and consumers around the gated-delta op inside one mixer layer: the short
// causal depthwise convolution on the q/k/v projections, the gate inputs (g, beta, lambda) and the
// gated RMS norm on the output.  All of them stream their tensors once and are bound by HBM;
// arithmetic is fp32 whatever the storage type.
//
// Reference: models/hattention/short_convolution.py (ShortConvolution.forward / step, kernels at
// 39-112, 203-253, 484-502), models/hattention/modeling_h_gated_deltanet.py:151-166, 429-437,
// models/hattention/fused_norm.py:40-112 (FusedRMSNormGated).
#include "common.cuh"
#include "profile.cuh"
#include <algorithm>

namespace lampa {

constexpr int CONV_MAX_W = 8;       // taps
constexpr int CONV_TOKENS = 16;     // consecutive tokens per thread (window kept in registers)

template <int DT> struct Vec16;     // 16 bytes of channels
template <> struct Vec16<LAMPA_F32> { static constexpr int N = 4; };
template <> struct Vec16<LAMPA_BF16> { static constexpr int N = 8; };
template <> struct Vec16<LAMPA_F16> { static constexpr int N = 8; };

template <int DT>
__device__ __forceinline__ void unpack_vec(const uint4& u, float (&x)[Vec16<DT>::N]) {
    if (DT == LAMPA_F32) {
        x[0] = __uint_as_float(u.x); x[1] = __uint_as_float(u.y); x[2] = __uint_as_float(u.z); x[3] = __uint_as_float(u.w);
    } else {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float2 f;
            if (DT == LAMPA_BF16) f = unpack_bf16x2(w[j]);
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
            x[2 * j] = f.x; x[2 * j + 1] = f.y;
        }
    }
}
template <int DT>
__device__ __forceinline__ void load_vec(const void* p, size_t elem, float (&x)[Vec16<DT>::N]) {
    unpack_vec<DT>(__ldg(reinterpret_cast<const uint4*>((const char*)p + elem * (DT == LAMPA_F32 ? 4 : 2))), x);
}
template <int DT>
__device__ __forceinline__ void store_vec(void* p, size_t elem, const float (&x)[Vec16<DT>::N]) {
    uint4 u;
    if (DT == LAMPA_F32) {
        u = make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
    } else if (DT == LAMPA_BF16) {
        u = make_uint4(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]), pack_bf16x2(x[4], x[5]), pack_bf16x2(x[6], x[7]));
    } else {
        __half2 h[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(x[2 * j], x[2 * j + 1]);
        u = *reinterpret_cast<const uint4*>(h);
    }
    *reinterpret_cast<uint4*>((char*)p + elem * (DT == LAMPA_F32 ? 4 : 2)) = u;
}

__device__ __forceinline__ float sigmoidf_(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
// log(1 + e^x) as max(x, 0) + log1p(e^-|x|); the log1p is the hardware log above 0.01 (absolute
// error 2e-7) and its cubic Taylor polynomial below.  torch switches to x above 20, where the
// two agree to fp32 rounding.
__device__ __forceinline__ float softplusf_(float x) {
    const float e = __expf(-fabsf(x));
    const float l = e > 0.01f ? __logf(1.f + e) : e * (1.f - e * (0.5f - e * (1.f / 3.f)));
    return fmaxf(x, 0.f) + l;
}

// Four channels of one token: 8 bytes of bf16 / fp16, 16 bytes of fp32.
template <int DT> struct Raw4 { using T = uint2; };
template <> struct Raw4<LAMPA_F32> { using T = uint4; };
template <int DT>
__device__ __forceinline__ typename Raw4<DT>::T ldg4(const void* p, size_t elem) {
    return __ldg(reinterpret_cast<const typename Raw4<DT>::T*>((const char*)p + elem * (DT == LAMPA_F32 ? 4 : 2)));
}
__device__ __forceinline__ void unpack4(const uint4& u, float (&x)[4], int) {
    x[0] = __uint_as_float(u.x); x[1] = __uint_as_float(u.y); x[2] = __uint_as_float(u.z); x[3] = __uint_as_float(u.w);
}
__device__ __forceinline__ void unpack4(const uint2& u, float (&x)[4], int dt) {
    float2 a, b;
    if (dt == LAMPA_BF16) { a = unpack_bf16x2(u.x); b = unpack_bf16x2(u.y); }
    else { a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)); b = __half22float2(*reinterpret_cast<const __half2*>(&u.y)); }
    x[0] = a.x; x[1] = a.y; x[2] = b.x; x[3] = b.y;
}
template <int DT>
__device__ __forceinline__ void store4(void* p, size_t elem, const float (&x)[4]) {
    if (DT == LAMPA_F32) {
        *reinterpret_cast<uint4*>((char*)p + elem * 4) =
            make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3]));
    } else if (DT == LAMPA_BF16) {
        *reinterpret_cast<uint2*>((char*)p + elem * 2) = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
    } else {
        const __half2 h0 = __floats2half2_rn(x[0], x[1]), h1 = __floats2half2_rn(x[2], x[3]);
        *reinterpret_cast<uint2*>((char*)p + elem * 2) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1));
    }
}

// -------------------------------------------------------------------------------------------------
// y[t, d] = act(bias[d] + sum_i w[d, i] x[t - (W-1) + i, d]) (+ residual), taps before the start
// of the token's sequence read as zero.  Thread = 4 channels x CONV_TOKENS consecutive
// tokens; the W-1 earlier rows are re-read once per run (from L2), everything else is read once.
// -------------------------------------------------------------------------------------------------
struct ConvArgs {
    const void* x; const void* w; const void* bias; const void* residual; const int64_t* cu;
    void* y;
    int64_t n_tok;      // B * T
    int64_t T;          // tokens per batch row (fixed-length input)
    int nseq;           // > 0: packed input with cu_seqlens
    int D, W, silu, w_dt;
};

template <int DT, int MW, bool EXACT>   // MW: compile-time bound on the number of taps; EXACT: W == MW, known to the compiler
__global__ void __launch_bounds__(128) short_conv_fwd_kernel(ConvArgs a) {
    constexpr int NV = 4;
    using RawT = typename Raw4<DT>::T;
    const int cg = blockIdx.y * blockDim.x + threadIdx.x;          // channel group
    if (cg * NV >= a.D) return;
    const int d0 = cg * NV;
    const int64_t t_begin = ((int64_t)blockIdx.x * blockDim.y + threadIdx.y) * CONV_TOKENS;
    if (t_begin >= a.n_tok) return;
    const int64_t t_end = min(t_begin + CONV_TOKENS, a.n_tok);
    const int W = EXACT ? MW : a.W;

    float wt[MW][NV], bs[NV];
#pragma unroll
    for (int i = 0; i < MW; ++i)
#pragma unroll
        for (int j = 0; j < NV; ++j)
            wt[i][j] = i < W ? load_as_float(a.w, (size_t)(d0 + j) * W + i, a.w_dt) : 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) bs[j] = a.bias ? load_as_float(a.bias, d0 + j, a.w_dt) : 0.f;

    // sequence of the first token
    int seq = 0;
    int64_t bos, eos;
    if (a.nseq > 0) {
        int lo = 0, hi = a.nseq - 1;
        while (lo < hi) {                                  // last seq with cu[seq] <= t_begin
            const int mid = (lo + hi + 1) >> 1;
            if (a.cu[mid] <= t_begin) lo = mid; else hi = mid - 1;
        }
        seq = lo;
        bos = a.cu[seq]; eos = a.cu[seq + 1];
    } else {
        bos = (t_begin / a.T) * a.T; eos = bos + a.T;
    }
    // window: win[i] = x[t - (W-1) + i]; slots 0 .. W-2 hold the history, slot W-1 the current token
    float win[MW][NV];
#pragma unroll
    for (int i = 0; i < MW; ++i)
#pragma unroll
        for (int j = 0; j < NV; ++j) win[i][j] = 0.f;
#pragma unroll
    for (int i = 0; i < MW - 1; ++i)
        if (i < W - 1) {
            const int64_t tt = t_begin - (W - 1) + i;
            if (tt >= bos) unpack4(ldg4<DT>(a.x, (size_t)tt * a.D + d0), win[i], DT);
        }
    // all rows of the run are requested before the first one is used
    RawT raw[CONV_TOKENS];
#pragma unroll
    for (int i = 0; i < CONV_TOKENS; ++i) {
        const int64_t t = min(t_begin + i, t_end - 1);            // rows past the end re-read the last one, unused
        raw[i] = ldg4<DT>(a.x, (size_t)t * a.D + d0);
    }
    // bit i of starts: token t_begin + i opens a sequence (its history is empty)
    uint32_t starts = 0;
    for (int i = 0; i < CONV_TOKENS; ++i) {
        const int64_t t = t_begin + i;
        if (t >= t_end) break;
        if (t >= eos) {
            if (a.nseq > 0) {
                while (seq + 1 < a.nseq && a.cu[seq + 1] <= t) ++seq;
                bos = a.cu[seq]; eos = a.cu[seq + 1];
            } else {
                bos = eos; eos = bos + a.T;
            }
            starts |= 1u << i;
        }
    }
#pragma unroll
    for (int it = 0; it < CONV_TOKENS; ++it) {
        const int64_t t = t_begin + it;
        if (t < t_end) {
        if ((starts >> it) & 1u) {
#pragma unroll
            for (int i = 0; i < MW; ++i)
#pragma unroll
                for (int j = 0; j < NV; ++j) win[i][j] = 0.f;
        }
        float cur[NV];
        unpack4(raw[it], cur, DT);
        float acc[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) acc[j] = 0.f;
#pragma unroll
        for (int i = 0; i < MW - 1; ++i)
            if (i < W - 1) {
#pragma unroll
                for (int j = 0; j < NV; ++j) acc[j] += win[i][j] * wt[i][j];
            }
#pragma unroll
        for (int i = 0; i < MW; ++i)
            if (i == W - 1) {
#pragma unroll
                for (int j = 0; j < NV; ++j) acc[j] += cur[j] * wt[i][j];
            }
        float out[NV];
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            float v = acc[j] + bs[j];
            if (a.silu) v = v * sigmoidf_(v);
            out[j] = v;
        }
        if (a.residual) {
            float r[NV];
            unpack4(ldg4<DT>(a.residual, (size_t)t * a.D + d0), r, DT);
#pragma unroll
            for (int j = 0; j < NV; ++j) out[j] += r[j];
        }
        store4<DT>(a.y, (size_t)t * a.D + d0, out);
        // slide: history slot i takes slot i + 1, the newest history slot takes the current token
#pragma unroll
        for (int i = 0; i < MW - 2; ++i)
            if (i < W - 2) {
#pragma unroll
                for (int j = 0; j < NV; ++j) win[i][j] = win[i + 1][j];
            }
#pragma unroll
        for (int i = 0; i < MW - 1; ++i)
            if (i == W - 2) {
#pragma unroll
                for (int j = 0; j < NV; ++j) win[i][j] = cur[j];
            }
        }
    }
}

// Convolution state after a prefill: cache[n, d, w] = x[eos_n - W + w, d]; slots that would lie
// before the sequence start are zeroed (zero_fill) or left as they are.
__global__ void __launch_bounds__(256)
short_conv_state_kernel(const void* x, const int64_t* cu, int64_t T, int nseq_packed, int N, int D, int W,
                        int dt, int zero_fill, void* cache) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)N * D * W) return;
    const int w = (int)(idx % W);
    const int d = (int)((idx / W) % D);
    const int n = (int)(idx / ((int64_t)W * D));
    const int64_t bos = nseq_packed > 0 ? cu[n] : (int64_t)n * T;
    const int64_t eos = nseq_packed > 0 ? cu[n + 1] : bos + T;
    const int64_t t = eos - W + w;
    if (t >= bos) store_from_float(cache, idx, load_as_float(x, (size_t)t * D + d, dt), dt);
    else if (zero_fill) store_from_float(cache, idx, 0.f, dt);
}

// Decode step: the cache [N, D, W] moves one slot to the left, takes x in its last slot, and
// y = act(bias + sum_w cache[n, d, w] weight[d, w]) (+ residual).
__global__ void __launch_bounds__(256)
short_conv_step_kernel(const void* x, void* cache, const void* w, const void* bias, const void* residual,
                       int N, int D, int W, int dt, int w_dt, int silu, void* y) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)N * D) return;
    const int d = (int)(idx % D);
    float c[CONV_MAX_W];
#pragma unroll
    for (int i = 0; i < CONV_MAX_W; ++i) c[i] = 0.f;
#pragma unroll
    for (int i = 0; i < CONV_MAX_W - 1; ++i)
        if (i < W - 1) c[i] = load_as_float(cache, (size_t)idx * W + i + 1, dt);
    const float xv = load_as_float(x, idx, dt);
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < CONV_MAX_W; ++i)
        if (i < W) {
            const float v = (i == W - 1) ? xv : c[i];
            store_from_float(cache, (size_t)idx * W + i, v, dt);
            acc += v * load_as_float(w, (size_t)d * W + i, w_dt);
        }
    if (bias) acc += load_as_float(bias, d, w_dt);
    if (silu) acc = acc * sigmoidf_(acc);
    if (residual) acc += load_as_float(residual, idx, dt);
    store_from_float(y, idx, acc, dt);
}

// -------------------------------------------------------------------------------------------------
// Gate inputs of the hierarchical layer (modeling_h_gated_deltanet.py:429-450):
//   g = -exp(A_log[h]) softplus(a + dt_bias[h])      beta = sigmoid(b)
//   lambda = softplus(L[h, l] dl)  |  exp(-exp(L) softplus(dl))  |  L dl        (mode 0 | 1 | 2)
// each multiplied by the token's padding mask when one is given.
// -------------------------------------------------------------------------------------------------
struct GateArgs {
    const void* a; const void* b; const void* dl; const float* A_log; const float* dt_bias; const float* Lw;
    const float* mask;
    float* g; void* beta; void* lam;
    int64_t n_tok; int H, L, in_dt, beta_dt, lam_dt, mode;
};

__device__ __forceinline__ float lambda_of(float Lv, float dv, int mode) {
    if (mode == 0) return softplusf_(Lv * dv);
    if (mode == 1) return __expf(-__expf(Lv) * softplusf_(dv));
    return Lv * dv;
}

// g and beta: one (token, head) per thread
__global__ void __launch_bounds__(256) gate_gb_kernel(GateArgs p) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= p.n_tok * p.H) return;
    const int h = (int)(idx % p.H);
    const float m = p.mask ? p.mask[idx / p.H] : 1.f;
    if (p.g) {
        const float av = load_as_float(p.a, idx, p.in_dt);
        p.g[idx] = -__expf(p.A_log[h]) * softplusf_(av + p.dt_bias[h]) * m;
    }
    if (p.beta) store_from_float(p.beta, idx, sigmoidf_(load_as_float(p.b, idx, p.in_dt)) * m, p.beta_dt);
}

// lambda: VEC consecutive (token, head, level) elements per thread, 16-byte loads when VEC == 8
template <int VEC>
__global__ void __launch_bounds__(256) gate_lambda_kernel(GateArgs p) {
    const int64_t HL = (int64_t)p.H * p.L, total = p.n_tok * HL;
    const int64_t j0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (j0 >= total) return;
    float dv[VEC];
    if (VEC == 8) {
        const uint4 u = __ldg(reinterpret_cast<const uint4*>((const uint16_t*)p.dl + j0));
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float2 f;
            if (p.in_dt == LAMPA_BF16) f = unpack_bf16x2(w[q]);
            else f = __half22float2(*reinterpret_cast<const __half2*>(&w[q]));
            dv[2 * q] = f.x; dv[2 * q + 1] = f.y;
        }
    } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) dv[e] = j0 + e < total ? load_as_float(p.dl, j0 + e, p.in_dt) : 0.f;
    }
    int64_t tok = j0 / HL;
    int r = (int)(j0 - tok * HL);                     // position inside the token's H x L block
    float out[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
        const float m = p.mask ? p.mask[min(tok, p.n_tok - 1)] : 1.f;
        out[e] = lambda_of(p.Lw[r], dv[e], p.mode) * m;
        if (++r == HL) { r = 0; ++tok; }
    }
    if (VEC == 8 && p.lam_dt != LAMPA_F32) {
        uint4 u;
        if (p.lam_dt == LAMPA_BF16) {
            u = make_uint4(pack_bf16x2(out[0], out[1]), pack_bf16x2(out[2], out[3]), pack_bf16x2(out[4], out[5]), pack_bf16x2(out[6], out[7]));
        } else {
            __half2 hh[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) hh[q] = __floats2half2_rn(out[2 * q], out[2 * q + 1]);
            u = make_uint4(*reinterpret_cast<uint32_t*>(&hh[0]), *reinterpret_cast<uint32_t*>(&hh[1]),
                           *reinterpret_cast<uint32_t*>(&hh[2]), *reinterpret_cast<uint32_t*>(&hh[3]));
        }
        *reinterpret_cast<uint4*>((uint16_t*)p.lam + j0) = u;
    } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e)
            if (j0 + e < total) store_from_float(p.lam, j0 + e, out[e], p.lam_dt);
    }
}

// -------------------------------------------------------------------------------------------------
// Gated RMS norm over rows of D: y = x rsqrt(mean(x^2) + eps) w * gate, gate = g sigmoid(g)
// (swish / silu) or sigmoid(g).  One warp per row, 16 bytes per lane and step.
// -------------------------------------------------------------------------------------------------
// A row is spread over LPR = min(32, D/16 bytes) lanes (rounded up to a power of two), so a warp
// holds 32/LPR rows at a time; VPL vectors per lane cover rows wider than 32 vectors.  Each lane
// keeps RPI = 4/VPL rows in flight: all their x and g vectors are requested before the first use.
template <int DT, int VPL>
__global__ void __launch_bounds__(256)
rmsnorm_gate_kernel(const void* x, const void* g, const void* w, int w_dt, int64_t rows, int D, int lpr, float eps,
                    int sigmoid_only, void* y) {
    constexpr int NV = Vec16<DT>::N;
    constexpr int RPI = 4 / VPL;
    constexpr int EB = DT == LAMPA_F32 ? 4 : 2;
    const int lane = threadIdx.x & 31;
    const int rpw = 32 / lpr;                              // rows per warp and step
    const int sub = lane / lpr, l = lane - sub * lpr;
    const int nvec = D / NV;
    float wv[VPL][NV];
#pragma unroll
    for (int v = 0; v < VPL; ++v)
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int c = (l + lpr * v) * NV + j;
            wv[v][j] = (w && c < D) ? load_as_float(w, c, w_dt) : 1.f;
        }
    const int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int64_t rows_per_iter = (int64_t)rpw * RPI;
    for (int64_t base = warp_id * rows_per_iter; base < rows; base += n_warps * rows_per_iter) {
        uint4 rx[RPI][VPL], rg[RPI][VPL];
#pragma unroll
        for (int r = 0; r < RPI; ++r) {
            const int64_t row = base + (int64_t)r * rpw + sub;
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int vi = l + lpr * v;
                const bool ok = row < rows && vi < nvec;
                const size_t off = ((size_t)row * D + (size_t)vi * NV) * EB;
                rx[r][v] = ok ? __ldg(reinterpret_cast<const uint4*>((const char*)x + off)) : make_uint4(0u, 0u, 0u, 0u);
                rg[r][v] = ok ? __ldg(reinterpret_cast<const uint4*>((const char*)g + off)) : make_uint4(0u, 0u, 0u, 0u);
            }
        }
#pragma unroll
        for (int r = 0; r < RPI; ++r) {
            const int64_t row = base + (int64_t)r * rpw + sub;
            float xv[VPL][NV];
            float ss = 0.f;
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                unpack_vec<DT>(rx[r][v], xv[v]);
#pragma unroll
                for (int j = 0; j < NV; ++j) ss += xv[v][j] * xv[v][j];
            }
            for (int o = lpr >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rstd = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int vi = l + lpr * v;
                float gv[NV], out[NV];
                unpack_vec<DT>(rg[r][v], gv);
#pragma unroll
                for (int j = 0; j < NV; ++j) {
                    const float yv = xv[v][j] * rstd * wv[v][j];
                    const float sg = sigmoidf_(gv[j]);
                    out[j] = sigmoid_only ? yv * sg : yv * gv[j] * sg;
                }
                if (row < rows && vi < nvec) store_vec<DT>(y, (size_t)row * D + (size_t)vi * NV, out);
            }
        }
    }
}

// -------------------------------------------------------------------------------------------------
// Residual add + RMS norm over rows of D floats, with the row permutation of the ordering layer folded
// in.  For every j in [0, rows): r = s0 + perm[j] (the row's place in the other order; r = j
// without a permutation), v = res[r] (+ delta[delta_at_r ? r : j]); the sum is written back to
// res[r] when there is a delta; y[y_at_r ? r : j] = v / sqrt(mean(v^2) + eps) * weight when y is
// given.  One warp per row, four rows in flight per warp.
// -------------------------------------------------------------------------------------------------
struct AddNormArgs {
    float* res; const void* delta; int delta_dt; const int64_t* perm; const int64_t* seg; int nseg;
    int64_t rows; int D; const float* w; float eps; int delta_at_r, y_at_r; void* y; int y_dt; int32_t* status;
};

__device__ __forceinline__ int find_seg_rows(const int64_t* off, int nseg, int64_t x) {
    int lo = 0, hi = nseg;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (off[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}
__device__ __forceinline__ float4 load4_as_float(const void* p, size_t i, int dt) {   // i a multiple of 4
    if (dt == LAMPA_F32) return __ldg(reinterpret_cast<const float4*>((const float*)p + i));
    const uint2 u = __ldg(reinterpret_cast<const uint2*>((const uint16_t*)p + i));
    float2 a, b;
    if (dt == LAMPA_BF16) { a = unpack_bf16x2(u.x); b = unpack_bf16x2(u.y); }
    else { a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)); b = __half22float2(*reinterpret_cast<const __half2*>(&u.y)); }
    return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4_from_float(void* p, size_t i, int dt, float4 v) {
    if (dt == LAMPA_F32) { *reinterpret_cast<float4*>((float*)p + i) = v; return; }
    uint2 u;
    if (dt == LAMPA_BF16) { u.x = pack_bf16x2(v.x, v.y); u.y = pack_bf16x2(v.z, v.w); }
    else {
        const __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
        u.x = *reinterpret_cast<const uint32_t*>(&a); u.y = *reinterpret_cast<const uint32_t*>(&b);
    }
    *reinterpret_cast<uint2*>((uint16_t*)p + i) = u;
}

template <int VPL>   // float4 vectors per lane: D <= 128 * VPL
__global__ void __launch_bounds__(256) add_rmsnorm_kernel(AddNormArgs p) {
    constexpr int RPI = 4;
    const int lane = threadIdx.x & 31;
    const int64_t warp_id = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t n_warps = (int64_t)gridDim.x * (blockDim.x >> 5);
    const int nvec = p.D >> 2;
    float4 wv[VPL];
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
        const int vi = lane + 32 * v;
        wv[v] = (p.w && vi < nvec) ? __ldg(reinterpret_cast<const float4*>(p.w) + vi) : make_float4(1.f, 1.f, 1.f, 1.f);
    }
    for (int64_t base = warp_id * RPI; base < p.rows; base += n_warps * RPI) {
        int64_t rr[RPI];
        bool ok[RPI];
        float4 x[RPI][VPL];
#pragma unroll
        for (int q = 0; q < RPI; ++q) {
            const int64_t j = base + q;
            ok[q] = j < p.rows;
            rr[q] = j;
            if (ok[q] && p.perm) {
                int64_t s0 = 0, len = p.rows;
                if (p.seg) { const int si = find_seg_rows(p.seg, p.nseg, j); s0 = p.seg[si]; len = p.seg[si + 1] - s0; }
                else if (p.nseg > 1) { len = p.rows / p.nseg; s0 = (j / len) * len; }
                const int64_t pj = p.perm[j];
                if (pj < 0 || pj >= len || s0 < 0 || s0 + len > p.rows) {
                    if (lane == 0) set_status(p.status, LAMPA_ERR_BOUNDS, 13, (int)j);
                    ok[q] = false;
                } else {
                    rr[q] = s0 + pj;
                }
            }
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int vi = lane + 32 * v;
                x[q][v] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok[q] && vi < nvec) {
                    x[q][v] = *reinterpret_cast<const float4*>(p.res + (size_t)rr[q] * p.D + 4 * vi);
                    if (p.delta) {
                        const float4 d = load4_as_float(p.delta, (size_t)(p.delta_at_r ? rr[q] : base + q) * p.D + 4 * vi, p.delta_dt);
                        x[q][v].x += d.x; x[q][v].y += d.y; x[q][v].z += d.z; x[q][v].w += d.w;
                    }
                }
            }
        }
#pragma unroll
        for (int q = 0; q < RPI; ++q) {
            if (!ok[q]) continue;              // warp-uniform
            float ss = 0.f;
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int vi = lane + 32 * v;
                if (vi < nvec) {
                    if (p.delta) *reinterpret_cast<float4*>(p.res + (size_t)rr[q] * p.D + 4 * vi) = x[q][v];
                    ss += x[q][v].x * x[q][v].x + x[q][v].y * x[q][v].y + x[q][v].z * x[q][v].z + x[q][v].w * x[q][v].w;
                }
            }
            if (p.y == nullptr) continue;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float rstd = 1.f / sqrtf(ss / (float)p.D + p.eps);
            const size_t yrow = (size_t)(p.y_at_r ? rr[q] : base + q) * p.D;
#pragma unroll
            for (int v = 0; v < VPL; ++v) {
                const int vi = lane + 32 * v;
                if (vi < nvec)
                    store4_from_float(p.y, yrow + 4 * vi, p.y_dt,
                                      make_float4(x[q][v].x * rstd * wv[v].x, x[q][v].y * rstd * wv[v].y,
                                                  x[q][v].z * rstd * wv[v].z, x[q][v].w * rstd * wv[v].w));
            }
        }
    }
}

}  // namespace lampa

using namespace lampa;

static bool dt_ok(int dt) { return dt == LAMPA_BF16 || dt == LAMPA_F16 || dt == LAMPA_F32; }

extern "C" int lampa_short_conv_fwd(const void* x, const void* weight, const void* bias, const void* residual,
                                    const int64_t* cu_seqlens, int32_t nseq, int64_t B, int64_t T, int32_t D,
                                    int32_t W, int32_t dtype, int32_t w_dtype, int32_t silu, void* y,
                                    void* final_state, int32_t zero_fill, void* stream) {
    if (B <= 0 || T < 0 || D <= 0 || W < 1 || W > CONV_MAX_W || !dt_ok(dtype) || !dt_ok(w_dtype)) return LAMPA_ERR_ARG;
    if (nseq < 0 || (nseq > 0 && (B != 1 || !cu_seqlens))) return LAMPA_ERR_ARG;
    const int nv = 4;
    if (D % nv != 0) return LAMPA_ERR_UNSUPPORTED;
    if (B * T == 0) return LAMPA_OK;
    if (!x || !weight || !y) return LAMPA_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)residual) & (dtype == LAMPA_F32 ? 15 : 7)) return LAMPA_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    ConvArgs a;
    a.x = x; a.w = weight; a.bias = bias; a.residual = residual; a.cu = cu_seqlens; a.y = y;
    a.n_tok = B * T; a.T = T; a.nseq = nseq; a.D = D; a.W = W; a.silu = silu; a.w_dt = w_dtype;
    const int groups = D / nv;
    const int bx = std::min(groups, 128), by = 128 / bx;
    dim3 block(bx, by), grid((unsigned)((a.n_tok + (int64_t)by * CONV_TOKENS - 1) / ((int64_t)by * CONV_TOKENS)), (groups + bx - 1) / bx);
    {
        ProfScope prof("short_conv_fwd", st);
#define LAMPA_CONV(DT)                                                                    \
        do {                                                                              \
            if (W == 4) short_conv_fwd_kernel<DT, 4, true><<<grid, block, 0, st>>>(a);            \
            else if (W == 2) short_conv_fwd_kernel<DT, 2, true><<<grid, block, 0, st>>>(a);       \
            else if (W == 8) short_conv_fwd_kernel<DT, 8, true><<<grid, block, 0, st>>>(a);       \
            else short_conv_fwd_kernel<DT, CONV_MAX_W, false><<<grid, block, 0, st>>>(a);         \
        } while (0)
        if (dtype == LAMPA_BF16) LAMPA_CONV(LAMPA_BF16);
        else if (dtype == LAMPA_F16) LAMPA_CONV(LAMPA_F16);
        else LAMPA_CONV(LAMPA_F32);
#undef LAMPA_CONV
        if (cudaGetLastError() != cudaSuccess) return LAMPA_ERR_CUDA;
    }
    if (final_state) {
        const int N = nseq > 0 ? nseq : (int)B;
        const int64_t tot = (int64_t)N * D * W;
        short_conv_state_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(x, cu_seqlens, T, nseq, N, D, W, dtype,
                                                                            zero_fill, final_state);
        if (cudaGetLastError() != cudaSuccess) return LAMPA_ERR_CUDA;
    }
    return LAMPA_OK;
}

extern "C" int lampa_short_conv_step(const void* x, void* cache, const void* weight, const void* bias,
                                     const void* residual, int64_t N, int32_t D, int32_t W, int32_t dtype,
                                     int32_t w_dtype, int32_t silu, void* y, void* stream) {
    if (N <= 0 || D <= 0 || W < 1 || W > CONV_MAX_W || !dt_ok(dtype) || !dt_ok(w_dtype)) return LAMPA_ERR_ARG;
    if (!x || !cache || !weight || !y) return LAMPA_ERR_ARG;
    const int64_t tot = N * D;
    ProfScope prof("short_conv_step", (cudaStream_t)stream);
    short_conv_step_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
        x, cache, weight, bias, residual, (int)N, D, W, dtype, w_dtype, silu, y);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_gate_inputs(const void* a, const void* b, const void* dl, const float* A_log,
                                 const float* dt_bias, const float* Lw, const float* mask, int64_t n_tok,
                                 int32_t H, int32_t L, int32_t in_dtype, int32_t beta_dtype, int32_t lam_dtype,
                                 int32_t lambda_mode, float* g, void* beta, void* lam, void* stream) {
    if (n_tok < 0 || H <= 0 || L < 0 || !dt_ok(in_dtype) || !dt_ok(beta_dtype) || !dt_ok(lam_dtype)) return LAMPA_ERR_ARG;
    if (lambda_mode < 0 || lambda_mode > 2) return LAMPA_ERR_ARG;
    if (n_tok == 0) return LAMPA_OK;
    if ((g && (!a || !A_log || !dt_bias)) || (beta && !b) || (lam && (!dl || !Lw || L == 0))) return LAMPA_ERR_ARG;
    GateArgs p;
    p.a = a; p.b = b; p.dl = dl; p.A_log = A_log; p.dt_bias = dt_bias; p.Lw = Lw; p.mask = mask;
    p.g = g; p.beta = beta; p.lam = lam;
    p.n_tok = n_tok; p.H = H; p.L = lam ? L : 0; p.in_dt = in_dtype; p.beta_dt = beta_dtype; p.lam_dt = lam_dtype;
    p.mode = lambda_mode;
    cudaStream_t st = (cudaStream_t)stream;
    ProfScope prof("gate_inputs", st);
    if (g || beta) {
        const int64_t tot = n_tok * H;
        gate_gb_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(p);
        if (cudaGetLastError() != cudaSuccess) return LAMPA_ERR_CUDA;
    }
    if (lam) {
        const int64_t tot = n_tok * H * L;
        const bool vec = in_dtype != LAMPA_F32 && tot % 8 == 0 && (((uintptr_t)dl | (uintptr_t)lam) & 15) == 0;
        if (vec) gate_lambda_kernel<8><<<(unsigned)((tot / 8 + 255) / 256), 256, 0, st>>>(p);
        else gate_lambda_kernel<1><<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(p);
        if (cudaGetLastError() != cudaSuccess) return LAMPA_ERR_CUDA;
    }
    return LAMPA_OK;
}

extern "C" int lampa_rmsnorm_gate(const void* x, const void* g, const void* weight, int64_t rows, int32_t D,
                                  int32_t dtype, int32_t w_dtype, float eps, int32_t sigmoid_only, void* y,
                                  void* stream) {
    if (rows < 0 || D <= 0 || !dt_ok(dtype) || !dt_ok(w_dtype)) return LAMPA_ERR_ARG;
    const int nv = dtype == LAMPA_F32 ? 4 : 8;
    if (D % nv != 0 || D > 32 * 4 * nv) return LAMPA_ERR_UNSUPPORTED;
    if (rows == 0) return LAMPA_OK;
    if (!x || !g || !y || (((uintptr_t)x | (uintptr_t)g | (uintptr_t)y) & 15)) return LAMPA_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int nvec = D / nv;
    int lpr = 1;
    while (lpr < nvec && lpr < 32) lpr <<= 1;
    const int vpl = (nvec + lpr - 1) / lpr;                       // 1 .. 4
    const int64_t rows_per_block = (int64_t)8 * (32 / lpr) * (4 / (vpl == 3 ? 4 : vpl));
    const unsigned grid = (unsigned)std::min<int64_t>((rows + rows_per_block - 1) / rows_per_block, 148 * 16);
    ProfScope prof("rmsnorm_gate", st);
#define LAMPA_NORM(DT)                                                                                                   \
    do {                                                                                                                 \
        if (vpl == 1) rmsnorm_gate_kernel<DT, 1><<<grid, 256, 0, st>>>(x, g, weight, w_dtype, rows, D, lpr, eps, sigmoid_only, y); \
        else if (vpl == 2) rmsnorm_gate_kernel<DT, 2><<<grid, 256, 0, st>>>(x, g, weight, w_dtype, rows, D, lpr, eps, sigmoid_only, y); \
        else rmsnorm_gate_kernel<DT, 4><<<grid, 256, 0, st>>>(x, g, weight, w_dtype, rows, D, lpr, eps, sigmoid_only, y); \
    } while (0)
    if (dtype == LAMPA_BF16) LAMPA_NORM(LAMPA_BF16);
    else if (dtype == LAMPA_F16) LAMPA_NORM(LAMPA_F16);
    else LAMPA_NORM(LAMPA_F32);
#undef LAMPA_NORM
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_add_rmsnorm(float* res, const void* delta, int32_t delta_dtype, const int64_t* perm,
                                 const int64_t* seg_offsets, int32_t nseg, int64_t rows, int32_t D,
                                 const float* weight, float eps, int32_t delta_at_r, int32_t y_at_r, void* y,
                                 int32_t y_dtype, int32_t* status, void* stream) {
    if (rows < 0 || D <= 0 || nseg <= 0) return LAMPA_ERR_ARG;
    if (D % 4 != 0 || D > 1024) return LAMPA_ERR_UNSUPPORTED;
    if (rows == 0) return LAMPA_OK;
    if (!res || (!delta && !y)) return LAMPA_ERR_ARG;
    if ((delta && !dt_ok(delta_dtype)) || (y && !dt_ok(y_dtype))) return LAMPA_ERR_ARG;
    if (perm && !seg_offsets && rows % nseg != 0) return LAMPA_ERR_ARG;
    if ((((uintptr_t)res | (uintptr_t)delta | (uintptr_t)y | (uintptr_t)weight) & 15)) return LAMPA_ERR_ARG;
    AddNormArgs p{res, delta, delta_dtype, perm, seg_offsets, nseg, rows, D, weight, eps, delta_at_r, y_at_r, y, y_dtype, status};
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)std::min<int64_t>((rows + 31) / 32, 148 * 16);
    const int vpl = (D / 4 + 31) / 32;
    ProfScope prof("add_rmsnorm", st);
    if (vpl == 1) add_rmsnorm_kernel<1><<<grid, 256, 0, st>>>(p);
    else if (vpl == 2) add_rmsnorm_kernel<2><<<grid, 256, 0, st>>>(p);
    else if (vpl <= 4) add_rmsnorm_kernel<4><<<grid, 256, 0, st>>>(p);
    else add_rmsnorm_kernel<8><<<grid, 256, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}
