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

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }   // torch's threshold

// -------------------------------------------------------------------------------------------------
// y[t, d] = act(bias[d] + sum_i w[d, i] x[t - (W-1) + i, d]) (+ residual), taps before the start
// of the token's sequence read as zero.  Thread = 16 bytes of channels x CONV_TOKENS consecutive
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

template <int DT, int MW>   // MW: compile-time bound on the number of taps (sizes the register window)
__global__ void __launch_bounds__(128) short_conv_fwd_kernel(ConvArgs a) {
    constexpr int NV = Vec16<DT>::N;
    const int cg = blockIdx.y * blockDim.x + threadIdx.x;          // channel group
    if (cg * NV >= a.D) return;
    const int d0 = cg * NV;
    const int64_t t_begin = ((int64_t)blockIdx.x * blockDim.y + threadIdx.y) * CONV_TOKENS;
    if (t_begin >= a.n_tok) return;
    const int64_t t_end = min(t_begin + CONV_TOKENS, a.n_tok);
    const int W = a.W;

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
            if (tt >= bos) load_vec<DT>(a.x, (size_t)tt * a.D + d0, win[i]);
        }
    // all rows of the run are requested before the first one is used
    uint4 raw[CONV_TOKENS];
#pragma unroll
    for (int i = 0; i < CONV_TOKENS; ++i) {
        const int64_t t = t_begin + i;
        raw[i] = t < t_end ? __ldg(reinterpret_cast<const uint4*>((const char*)a.x + ((size_t)t * a.D + d0) * (DT == LAMPA_F32 ? 4 : 2)))
                           : make_uint4(0u, 0u, 0u, 0u);
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
        unpack_vec<DT>(raw[it], cur);
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
            load_vec<DT>(a.residual, (size_t)t * a.D + d0, r);
#pragma unroll
            for (int j = 0; j < NV; ++j) out[j] += r[j];
        }
        store_vec<DT>(a.y, (size_t)t * a.D + d0, out);
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

__global__ void __launch_bounds__(256) gate_inputs_kernel(GateArgs p) {
    const int64_t per_tok = (int64_t)p.H * (p.L + 1);
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= p.n_tok * per_tok) return;
    // the first n_tok * H threads produce g and beta, the rest one lambda each
    const int64_t n_gb = p.n_tok * p.H;
    if (idx < n_gb) {
        const int h = (int)(idx % p.H);
        const float m = p.mask ? p.mask[idx / p.H] : 1.f;
        if (p.g) {
            const float av = load_as_float(p.a, idx, p.in_dt);
            p.g[idx] = -__expf(p.A_log[h]) * softplusf_(av + p.dt_bias[h]) * m;
        }
        if (p.beta) store_from_float(p.beta, idx, sigmoidf_(load_as_float(p.b, idx, p.in_dt)) * m, p.beta_dt);
    } else if (p.lam) {
        const int64_t j = idx - n_gb;
        const int l = (int)(j % p.L);
        const int h = (int)((j / p.L) % p.H);
        const float m = p.mask ? p.mask[j / ((int64_t)p.L * p.H)] : 1.f;
        const float dv = load_as_float(p.dl, j, p.in_dt), Lv = p.Lw[h * p.L + l];
        float v;
        if (p.mode == 0) v = softplusf_(Lv * dv);
        else if (p.mode == 1) v = __expf(-__expf(Lv) * softplusf_(dv));
        else v = Lv * dv;
        store_from_float(p.lam, j, v * m, p.lam_dt);
    }
}

// -------------------------------------------------------------------------------------------------
// Gated RMS norm over rows of D: y = x rsqrt(mean(x^2) + eps) w * gate, gate = g sigmoid(g)
// (swish / silu) or sigmoid(g).  One warp per row, 16 bytes per lane and step.
// -------------------------------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(256)
rmsnorm_gate_kernel(const void* x, const void* g, const void* w, int w_dt, int64_t rows, int D, float eps,
                    int sigmoid_only, void* y) {
    constexpr int NV = Vec16<DT>::N;
    constexpr int MAXV = 4;                                // D <= 32 lanes * 4 * NV
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    float xv[MAXV][NV];
    float ss = 0.f;
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int c0 = (it * 32 + lane) * NV;
        if (c0 < D) {
            load_vec<DT>(x, (size_t)row * D + c0, xv[it]);
#pragma unroll
            for (int j = 0; j < NV; ++j) ss += xv[it][j] * xv[it][j];
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const float rstd = 1.f / sqrtf(ss / (float)D + eps);
#pragma unroll
    for (int it = 0; it < MAXV; ++it) {
        const int c0 = (it * 32 + lane) * NV;
        if (c0 < D) {
            float gv[NV], out[NV];
            load_vec<DT>(g, (size_t)row * D + c0, gv);
#pragma unroll
            for (int j = 0; j < NV; ++j) {
                const float wv = w ? load_as_float(w, c0 + j, w_dt) : 1.f;
                const float yv = xv[it][j] * rstd * wv;
                const float s = sigmoidf_(gv[j]);
                out[j] = sigmoid_only ? yv * s : yv * gv[j] * s;
            }
            store_vec<DT>(y, (size_t)row * D + c0, out);
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
    const int nv = dtype == LAMPA_F32 ? 4 : 8;
    if (D % nv != 0) return LAMPA_ERR_UNSUPPORTED;
    if (B * T == 0) return LAMPA_OK;
    if (!x || !weight || !y) return LAMPA_ERR_ARG;
    if (((uintptr_t)x | (uintptr_t)y | (uintptr_t)residual) & 15) return LAMPA_ERR_ARG;
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
            if (W <= 4) short_conv_fwd_kernel<DT, 4><<<grid, block, 0, st>>>(a);          \
            else short_conv_fwd_kernel<DT, CONV_MAX_W><<<grid, block, 0, st>>>(a);        \
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
    const int64_t tot = n_tok * H * (p.L + 1);
    ProfScope prof("gate_inputs", (cudaStream_t)stream);
    gate_inputs_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, (cudaStream_t)stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
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
    const unsigned grid = (unsigned)((rows + 7) / 8);
    ProfScope prof("rmsnorm_gate", st);
    if (dtype == LAMPA_BF16) rmsnorm_gate_kernel<LAMPA_BF16><<<grid, 256, 0, st>>>(x, g, weight, w_dtype, rows, D, eps, sigmoid_only, y);
    else if (dtype == LAMPA_F16) rmsnorm_gate_kernel<LAMPA_F16><<<grid, 256, 0, st>>>(x, g, weight, w_dtype, rows, D, eps, sigmoid_only, y);
    else rmsnorm_gate_kernel<LAMPA_F32><<<grid, 256, 0, st>>>(x, g, weight, w_dtype, rows, D, eps, sigmoid_only, y);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}
