// Per-chunk preparation of the gated-delta forward: one CTA of 4 warps per (chunk, head) turns
// 64 tokens of q, k, v, g, beta (and lambda) into the record {M, B^T, Q~, O_local, lambda_chunk}.
// Dense 64-wide contractions run on tensor cores (bf16 operands, fp32 accumulation); the
// 64x64 unit-lower-triangular inverse is an fp32 substitution on CUDA cores, as in the reference
// (models/hattention/solve_tril.py:54-61, 175-197), because bf16 there is where parity breaks.
#include "gdn.cuh"
#include "gdn_inv.cuh"
#include "gdn_load.cuh"
#include "profile.cuh"

namespace lampa {

// ---- plan: token / chunk / block offsets per sequence -------------------------------------------
__global__ void plan_kernel(PlanArgs p) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    int32_t c = 0, b = 0;
    p.chunk_off[0] = 0;
    p.block_off[0] = 0;
    for (int s = 0; s < p.nseq; ++s) {
        const int64_t t0 = p.cu ? p.cu[s] : (int64_t)s * p.T;
        const int64_t t1 = p.cu ? p.cu[s + 1] : (int64_t)(s + 1) * p.T;
        p.tok_off[s] = t0;
        int64_t len = t1 - t0;
        if (len < 0 || t0 < 0 || t1 > (int64_t)p.B * p.T) { set_status(p.status, LAMPA_ERR_BOUNDS, 1, s); len = 0; }
        const int nch = (int)((len + CHUNK - 1) / CHUNK);
        if (p.hier && nch > 0 && ELL0 + ceil_log2_int(nch) > p.L) set_status(p.status, LAMPA_ERR_LEVELS, 1, s);
        c += nch;
        b += (nch + BLOCK_CHUNKS - 1) / BLOCK_CHUNKS;
        p.chunk_off[s + 1] = c;
        p.block_off[s + 1] = b;
        if (s == p.nseq - 1) p.tok_off[s + 1] = t0 + len;
    }
}

int launch_plan(const PlanArgs& p, cudaStream_t st) {
    ProfScope prof("gdn_plan", st);
    plan_kernel<<<1, 32, 0, st>>>(p);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

// ---- shared-memory carve-up ---------------------------------------------------------------------
template <int KD, int VD>
struct PrepSmem {
    static constexpr int KP = KD + 8, VP = VD + 8, CP = CHUNK + 8;
    static constexpr int PA = CHUNK + 4;                         // fp32 pitch of the inverse's working tile (over AW and UH)
    static constexpr int Q = 0;                                  // bf16 [64][KP]   q (normalised); later W (rows are warp-private)
    static constexpr int K = Q + CHUNK * KP * 2;                 // bf16 [64][KP]   k (normalised)
    static constexpr int V = K + CHUNK * KP * 2;                 // bf16 [64][VP]   v
    static constexpr int AW = V + CHUNK * VP * 2;                // bf16 [64][CP]   Awb = (I + A0)^-1 diag(beta)
    static constexpr int UH = AW + CHUNK * CP * 2;               // bf16 [64][VP]   diag(e^{Glast-G}) U
    static constexpr int AFTER_UH = UH + CHUNK * VP * 2, AFTER_SA = AW + CHUNK * PA * 4;   // the fp32 tile covers AW and UH
    static constexpr int G = AFTER_UH > AFTER_SA ? AFTER_UH : AFTER_SA;   // fp32 [64] G, [64] beta, [64] e^G, [64] e^{Glast-G}
    static constexpr int LAM = G + 4 * CHUNK * 4;                // fp32 [64][L+1]
    static int bytes(int L) { return LAM + CHUNK * (L + 1) * 4; }
};

// With beta folded into the columns of the inverse (Awb = (I + A0)^-1 diag(beta), Aub = Awb .* E):
//   W  = Awb K                    M   = e^{G_last} (I - K^T W)
//   U^ = diag(e^{G_last-G}) Aub V B^T = U^^T K
//   R  = tril(Q K^T) Awb          Q~  = s diag(e^G) (Q - R K)
//   O_local = s ((R .* E .* lambda[i][level(i,j)]) V)
// (s = scale and lambda = 1 for the plain rule; s = 1 for the hierarchical one).  These equal
// the definitions in gdn.cuh: every e^{G_last-G_tok} e^{G_tok} pair collapses to e^{G_last}.
template <int KD, int VD, bool HIER>
__global__ void __launch_bounds__(128, 4) gdn_prep_kernel(GdnArgs a) {
    using S = PrepSmem<KD, VD>;
    using R = Rec<KD, VD>;
    constexpr int KP = S::KP, VP = S::VP, CP = S::CP;
    extern __shared__ __align__(128) unsigned char smem[];
    __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem + S::Q);
    __nv_bfloat16* sW = sQ;
    __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem + S::K);
    __nv_bfloat16* sV = reinterpret_cast<__nv_bfloat16*>(smem + S::V);
    __nv_bfloat16* sAw = reinterpret_cast<__nv_bfloat16*>(smem + S::AW);
    __nv_bfloat16* sUh = reinterpret_cast<__nv_bfloat16*>(smem + S::UH);
    float* sG = reinterpret_cast<float*>(smem + S::G);
    float* sBeta = sG + CHUNK;
    float* sEG = sG + 2 * CHUNK;
    float* sEGl = sG + 3 * CHUNK;
    float* sLam = reinterpret_cast<float*>(smem + S::LAM);

    // head is the fastest grid index: the H CTAs of one chunk run together and between them read
    // whole contiguous token rows of q, k, v (one head alone touches 128 B out of every H*128 B)
    const int h = blockIdx.x, c = blockIdx.y, H = a.H;
    ChunkLoc loc;
    if (a.plan_inline && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) write_fixed_plan(a);
    if (!locate_chunk(a, c, loc)) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int gq = lane >> 2, tq = lane & 3;
    const int64_t t0 = loc.t0;
    const int len = loc.len;
    const int LP = a.L + 1;
    if (h == 0) check_out_perm(a, t0, len);

    // ---- stage 0: loads, l2norm, cumulative decay -------------------------------------------------
    // Every global load of the chunk is issued before any of them is consumed (one DRAM round trip
    // instead of four), and the rows of a chunk some 600 CTAs ahead are pulled into L2.
    {
        const int r = tid >> 1, half = tid & 1;
        const bool valid = r < len;
        const size_t tok = (size_t)(t0 + r);
        const bool two_byte = a.qkv_dt != LAMPA_F32;
        uint4 rq[KD / 16], rk[KD / 16], rv[VD / 16];
        if (two_byte) {
            issue_half_row<KD>(a.q, (tok * H + h) * KD + half * (KD / 2), valid, rq);
            issue_half_row<KD>(a.k, (tok * H + h) * KD + half * (KD / 2), valid, rk);
            issue_half_row<VD>(a.v, (tok * H + h) * VD + half * (VD / 2), valid, rv);
        }
        float gv = 0.f, bv = 0.f;
        if (tid < len) {   // len <= 64: threads 0..len-1 carry g and beta of token tid
            gv = load_as_float(a.g, (size_t)(t0 + tid) * H + h, a.gb_dt);
            bv = load_as_float(a.beta, (size_t)(t0 + tid) * H + h, a.gb_dt);
        }
        if (HIER) {   // all of the row's loads in flight before the first store; the unrolled length follows L
            const size_t lam_base = (tok * H + h) * a.L;
            if (a.L <= 18) stage_lambda<9>(a.lam, a.lam_dt, lam_base, a.L, half, valid, sLam + r * LP);
            else if (a.L <= 24) stage_lambda<12>(a.lam, a.lam_dt, lam_base, a.L, half, valid, sLam + r * LP);
            else stage_lambda<20>(a.lam, a.lam_dt, lam_base, a.L, half, valid, sLam + r * LP);
        }
        if (h == 0) {   // L2 prefetch of the token rows (all heads) of a chunk ~80 chunks ahead
            ChunkLoc l2;
            if (locate_chunk(a, c + 80, l2) && r < l2.len) {
                const int eb = dtype_bytes(a.qkv_dt);
                const size_t rowq = (size_t)H * KD * eb, rowv = (size_t)H * VD * eb;
                const char* pq = (const char*)a.q + (size_t)(l2.t0 + r) * rowq;
                const char* pk = (const char*)a.k + (size_t)(l2.t0 + r) * rowq;
                const char* pv = (const char*)a.v + (size_t)(l2.t0 + r) * rowv;
                for (size_t off = (size_t)half * 128; off < rowq; off += 256) {
                    asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pq + off));
                    asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pk + off));
                }
                for (size_t off = (size_t)half * 128; off < rowv; off += 256)
                    asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pv + off));
            }
        }
        float x[KD / 2];
        if (two_byte) convert_half_row<KD>(rq, a.qkv_dt, x);
        else load_half_row<KD>(a.q, a.qkv_dt, (tok * H + h) * KD + half * (KD / 2), valid, x);
        if (a.use_l2norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < KD / 2; ++i) ss += x[i] * x[i];
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            const float rn = rsqrtf(ss + 1e-6f);
#pragma unroll
            for (int i = 0; i < KD / 2; ++i) x[i] *= rn;
        }
        store_half_row_bf16<KD / 2>(sQ + r * KP + half * (KD / 2), x);
        if (two_byte) convert_half_row<KD>(rk, a.qkv_dt, x);
        else load_half_row<KD>(a.k, a.qkv_dt, (tok * H + h) * KD + half * (KD / 2), valid, x);
        if (a.use_l2norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < KD / 2; ++i) ss += x[i] * x[i];
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            const float rn = rsqrtf(ss + 1e-6f);
#pragma unroll
            for (int i = 0; i < KD / 2; ++i) x[i] *= rn;
        }
        store_half_row_bf16<KD / 2>(sK + r * KP + half * (KD / 2), x);
        if (a.qkv_dt == LAMPA_BF16) {   // v is used as it is: the raw 16-byte pieces go straight to shared memory
#pragma unroll
            for (int i = 0; i < VD / 16; ++i) reinterpret_cast<uint4*>(sV + r * VP + half * (VD / 2))[i] = rv[i];
        } else {
            float y[VD / 2];
            if (two_byte) convert_half_row<VD>(rv, a.qkv_dt, y);
            else load_half_row<VD>(a.v, a.qkv_dt, (tok * H + h) * VD + half * (VD / 2), valid, y);
            store_half_row_bf16<VD / 2>(sV + r * VP + half * (VD / 2), y);
        }

        if (tid < CHUNK) {
            float cs = gv;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float yy = __shfl_up_sync(0xffffffffu, cs, o);
                if (lane >= o) cs += yy;
            }
            if (tid == 31) sG[CHUNK - 1] = cs;      // one-float mailbox between the two warps
            sBeta[tid] = bv;
            asm volatile("bar.sync 1, 64;\n" ::: "memory");
            const float carry = (warp == 1) ? sG[CHUNK - 1] : 0.f;
            asm volatile("bar.sync 1, 64;\n" ::: "memory");
            sG[tid] = cs + carry;
        }
    }
    __syncthreads();
    if (tid < CHUNK) {
        const float Gi = sG[tid], Gl = sG[CHUNK - 1];
        sEG[tid] = __expf(Gi);
        sEGl[tid] = __expf(Gl - Gi);
    }
    char* rec = a.rec + ((size_t)c * H + h) * a.rec_bytes;
    if (HIER) {   // lambda of the chunk levels, transposed to [level][token] for the scan
        float* lamc = reinterpret_cast<float*>(rec + R::LAM_OFF);
        for (int idx = tid; idx < a.LC * CHUNK; idx += 128) {
            const int l = idx >> 6, r = idx & 63;
            lamc[idx] = (ELL0 + l < a.L) ? sLam[r * LP + ELL0 + l] : 0.f;
        }
    }

    const int m0 = warp * 16;
    // ---- stage 1: Awb = (I + A0)^-1 diag(beta), A0 = tril(diag(beta) K K^T, -1) ---------------------
    // Blockwise, as the reference's solve_tril does (models/hattention/solve_tril.py:221-276): warp w
    // forms rows 16w.. of A0 on the tensor cores and inverts its own 16x16 diagonal block by fp32
    // forward substitution (lane = column); the off-diagonal blocks follow as X_ba = -(X_bb A_ba) X_aa,
    // first inside the two 32x32 halves, then for the 32x32 corner, in place in one fp32 [64][68] tile
    // that lies over the Awb and U^ buffers (both written later).  These products keep fp32 accuracy
    // by splitting each operand into bf16 hi + lo and issuing hi*hi + lo*hi + hi*lo (the reference
    // asks for IEEE fp32 dots there).
    {
        constexpr int PA = S::PA;
        float* sA = reinterpret_cast<float*>(smem + S::AW);
        {
            float acc[8][4];
            zero_acc<8>(acc);
            warp_gemm<8, KD, false, false>(acc, sK, KP, m0, sK, KP, 0, lane, KD, m0 + 16);
            const float b2[2] = {sBeta[m0 + gq], sBeta[m0 + gq + 8]};   // read before the stores below: they may alias for the compiler
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                    const float bb = b2[hh];
                    *reinterpret_cast<float2*>(sA + i * PA + j) =
                        make_float2(i > j ? bb * acc[nt][2 * hh] : 0.f, i > j + 1 ? bb * acc[nt][2 * hh + 1] : 0.f);
                }
        }
        __syncwarp();
        tril_inverse_64<PA>(sA, warp, lane);
        {   // Awb = X diag(beta) as bf16, written over the front of the fp32 tile
            const int r = tid >> 1, half = tid & 1;
            uint32_t w[16];
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                const float4 v = *reinterpret_cast<const float4*>(sA + r * PA + half * 32 + 4 * q);
                const float4 b = *reinterpret_cast<const float4*>(sBeta + half * 32 + 4 * q);
                w[2 * q] = pack_bf16x2(v.x * b.x, v.y * b.y);
                w[2 * q + 1] = pack_bf16x2(v.z * b.z, v.w * b.w);
            }
            __syncthreads();
#pragma unroll
            for (int q = 0; q < 4; ++q)
                reinterpret_cast<uint4*>(sAw + r * CP + half * 32)[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
        }
        __syncthreads();
    }
    const float osc = HIER ? 1.f : a.scale;
    // ---- per-warp part (rows m0..m0+15 of everything; nothing leaves the warp) --------------------
    {
        // tril(Q K^T) as A fragments, straight from its accumulators
        uint32_t ra[4][4];
        float racc[8][4];
        zero_acc<8>(racc);
        warp_gemm<8, KD, false, false>(racc, sQ, KP, m0, sK, KP, 0, lane, KD, m0 + 16);
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
            if (nt >= (m0 >> 3)) {       // only the warp's two diagonal 8-column tiles can hold i < j
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int i = m0 + gq + (e >> 1) * 8, j = nt * 8 + 2 * tq + (e & 1);
                    if (i < j) racc[nt][e] = 0.f;
                }
            }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            ra[kk][0] = pack_bf16x2(racc[2 * kk][0], racc[2 * kk][1]);
            ra[kk][1] = pack_bf16x2(racc[2 * kk][2], racc[2 * kk][3]);
            ra[kk][2] = pack_bf16x2(racc[2 * kk + 1][0], racc[2 * kk + 1][1]);
            ra[kk][3] = pack_bf16x2(racc[2 * kk + 1][2], racc[2 * kk + 1][3]);
        }
        // R = tril(QK^T) Awb, kept as accumulators and re-used as an A operand twice
        zero_acc<8>(racc);
        warp_gemm_ra<8, 4, true>(racc, ra, sAw, CP, 0, lane, m0 + 16, m0 + 16);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            ra[kk][0] = pack_bf16x2(racc[2 * kk][0], racc[2 * kk][1]);
            ra[kk][1] = pack_bf16x2(racc[2 * kk][2], racc[2 * kk][3]);
            ra[kk][2] = pack_bf16x2(racc[2 * kk + 1][0], racc[2 * kk + 1][1]);
            ra[kk][3] = pack_bf16x2(racc[2 * kk + 1][2], racc[2 * kk + 1][3]);
        }
        // Q~ = s e^G (Q - R K)
        {
            float acc[KD / 8][4];
            zero_acc<KD / 8>(acc);
            warp_gemm_ra<KD / 8, 4, true>(acc, ra, sK, KP, 0, lane, m0 + 16, KD);
            __nv_bfloat16* gQ = reinterpret_cast<__nv_bfloat16*>(rec + R::QT_OFF);
            const float fq[2] = {osc * sEG[m0 + gq], osc * sEG[m0 + gq + 8]};
#pragma unroll
            for (int nt = 0; nt < KD / 8; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                    const float f = fq[hh];
                    const float2 qv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(sQ + i * KP + j));
                    *reinterpret_cast<uint32_t*>(gQ + R::T::off(i, j)) =
                        pack_bf16x2(f * (qv.x - acc[nt][2 * hh]), f * (qv.y - acc[nt][2 * hh + 1]));
                }
        }
        // Pm = R .* E .* lambda, as A fragments;  O_local = s Pm V
        {
            // level(i, j) = bit_length(i ^ j).  Off the diagonal 8x8 tile it depends on the tile only
            // (3 + bit_length(i/8 ^ j/8)): one lambda per (row, tile) serves both of the thread's columns.
            const float gi2[2] = {sG[m0 + gq], sG[m0 + gq + 8]};
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float2 gj = *reinterpret_cast<const float2*>(sG + nt * 8 + 2 * tq);
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                    const int it = (m0 >> 3) + hh;                     // the row's 8x8 tile index (warp-uniform)
                    float p0 = 0.f, p1 = 0.f;
                    if (nt <= it) {
                        if (i >= j) p0 = racc[nt][2 * hh] * __expf(gi2[hh] - gj.x);
                        if (i >= j + 1) p1 = racc[nt][2 * hh + 1] * __expf(gi2[hh] - gj.y);
                        if (HIER) {
                            if (nt < it) {
                                const float lt = sLam[i * LP + 3 + (32 - __clz(it ^ nt))];
                                p0 *= lt; p1 *= lt;
                            } else {
                                p0 *= sLam[i * LP + (32 - __clz(i ^ j))];
                                p1 *= sLam[i * LP + (32 - __clz(i ^ (j + 1)))];
                            }
                        }
                    }
                    racc[nt][2 * hh] = p0;
                    racc[nt][2 * hh + 1] = p1;
                }
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                ra[kk][0] = pack_bf16x2(racc[2 * kk][0], racc[2 * kk][1]);
                ra[kk][1] = pack_bf16x2(racc[2 * kk][2], racc[2 * kk][3]);
                ra[kk][2] = pack_bf16x2(racc[2 * kk + 1][0], racc[2 * kk + 1][1]);
                ra[kk][3] = pack_bf16x2(racc[2 * kk + 1][2], racc[2 * kk + 1][3]);
            }
            float acc[VD / 8][4];
            zero_acc<VD / 8>(acc);
            warp_gemm_ra<VD / 8, 4, true>(acc, ra, sV, VP, 0, lane, m0 + 16, VD);
            __nv_bfloat16* gO = reinterpret_cast<__nv_bfloat16*>(rec + R::OL_OFF);
#pragma unroll
            for (int nt = 0; nt < VD / 8; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                    *reinterpret_cast<uint32_t*>(gO + R::TV::off(i, j)) =
                        pack_bf16x2(osc * acc[nt][2 * hh], osc * acc[nt][2 * hh + 1]);
                }
        }
        // U^ = diag(e^{Glast-G}) (Awb .* E) V: the decay is applied to the A fragments in registers
        {
            float acc[VD / 8][4];
            zero_acc<VD / 8>(acc);
            const float g_lo = sG[m0 + gq], g_hi = sG[m0 + gq + 8];
            const float fu[2] = {sEGl[m0 + gq], sEGl[m0 + gq + 8]};   // read before the stores to U^ below
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                if (kk * 16 < m0 + 16) {
                    uint32_t af[4];
                    load_a(af, sAw, CP, m0, kk * 16, lane);
#pragma unroll
                    for (int x = 0; x < 4; ++x) {
                        const int i = m0 + gq + (x & 1) * 8, j = kk * 16 + (x >> 1) * 8 + 2 * tq;
                        const int it = (m0 >> 3) + (x & 1), jt = 2 * kk + (x >> 1);   // 8x8 tile of the row / of the columns
                        if (jt > it) {
                            af[x] = 0u;                                           // above the diagonal
                        } else {
                            const float gi = (x & 1) ? g_hi : g_lo;
                            const float2 gj = *reinterpret_cast<const float2*>(sG + j);
                            const float2 w = unpack_bf16x2(af[x]);
                            const float u0 = (i >= j) ? w.x * __expf(gi - gj.x) : 0.f;
                            const float u1 = (i >= j + 1) ? w.y * __expf(gi - gj.y) : 0.f;
                            af[x] = pack_bf16x2(u0, u1);
                        }
                    }
#pragma unroll
                    for (int nt = 0; nt < VD / 8; nt += 2) {
                        uint32_t b[4];
                        load_b_t(b, sV, VP, nt * 8, kk * 16, lane);
                        mma16816(acc[nt], af, b[0], b[1]);
                        mma16816(acc[nt + 1], af, b[2], b[3]);
                    }
                }
            }
#pragma unroll
            for (int nt = 0; nt < VD / 8; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                    const float f = fu[hh];
                    *reinterpret_cast<uint32_t*>(sUh + i * VP + j) = pack_bf16x2(f * acc[nt][2 * hh], f * acc[nt][2 * hh + 1]);
                }
        }
        // W = Awb K, written over this warp's own rows of Q (no longer needed)
        {
            float acc[KD / 8][4];
            zero_acc<KD / 8>(acc);
            warp_gemm<KD / 8, CHUNK, false, true>(acc, sAw, CP, m0, sK, KP, 0, lane, m0 + 16, KD);
            __syncwarp();
#pragma unroll
            for (int nt = 0; nt < KD / 8; ++nt)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                    *reinterpret_cast<uint32_t*>(sW + i * KP + j) = pack_bf16x2(acc[nt][2 * hh], acc[nt][2 * hh + 1]);
                }
        }
    }
    __syncthreads();

    // ---- stage 4: M[a][b] = e^{G_last} (delta_ab - sum_tok K[tok][a] W[tok][b]);  B^T = U^^T K -----
    // Both tiles are assembled in the record's layout in shared memory (over Awb and V, which are
    // dead by now) and leave as two bulk copies instead of 4-byte stores from every lane.
    __nv_bfloat16* stM = reinterpret_cast<__nv_bfloat16*>(smem + S::AW);
    __nv_bfloat16* stB = reinterpret_cast<__nv_bfloat16*>(smem + S::V);
    static_assert(R::M_BYTES <= CHUNK * CP * 2 && R::BT_BYTES <= CHUNK * VP * 2, "staging tiles must fit");
    if (m0 < KD) {
        float acc[KD / 8][4];
        zero_acc<KD / 8>(acc);
        warp_gemm<KD / 8, CHUNK, true, true>(acc, sK, KP, m0, sW, KP, 0, lane, CHUNK, KD);
        const float egl = sEG[CHUNK - 1];
#pragma unroll
        for (int nt = 0; nt < KD / 8; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                const float m_0 = egl * (((i == j) ? 1.f : 0.f) - acc[nt][2 * hh]);
                const float m_1 = egl * (((i == j + 1) ? 1.f : 0.f) - acc[nt][2 * hh + 1]);
                *reinterpret_cast<uint32_t*>(stM + R::T::off(i, j)) = pack_bf16x2(m_0, m_1);
            }
    }
    if (m0 < VD) {
        float acc[KD / 8][4];
        zero_acc<KD / 8>(acc);
        warp_gemm<KD / 8, CHUNK, true, true>(acc, sUh, VP, m0, sK, KP, 0, lane, CHUNK, KD);
#pragma unroll
        for (int nt = 0; nt < KD / 8; ++nt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int i = m0 + gq + hh * 8, j = nt * 8 + 2 * tq;
                *reinterpret_cast<uint32_t*>(stB + R::T::off(i, j)) = pack_bf16x2(acc[nt][2 * hh], acc[nt][2 * hh + 1]);
            }
    }
    fence_async_shared();
    __syncthreads();
    if (tid == 0) {
        bulk_s2g(rec + R::M_OFF, stM, R::M_BYTES);
        bulk_s2g(rec + R::BT_OFF, stB, R::BT_BYTES);
        bulk_commit();
        bulk_wait_read();
    }
}

template <int KD, int VD>
int launch_prep(const GdnArgs& a, bool hier, cudaStream_t st) {
    using S = PrepSmem<KD, VD>;
    const int smem = S::bytes(hier ? a.L : 0);
    dim3 grid(a.H, a.nc_max);
    cudaError_t e;
    ProfScope prof(hier ? "gdn_prep_hier" : "gdn_prep_plain", st);
    if (hier) {
        e = cudaFuncSetAttribute(gdn_prep_kernel<KD, VD, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return LAMPA_ERR_CUDA;
        gdn_prep_kernel<KD, VD, true><<<grid, 128, smem, st>>>(a);
    } else {
        e = cudaFuncSetAttribute(gdn_prep_kernel<KD, VD, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return LAMPA_ERR_CUDA;
        gdn_prep_kernel<KD, VD, false><<<grid, 128, smem, st>>>(a);
    }
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

template int launch_prep<64, 64>(const GdnArgs&, bool, cudaStream_t);
template int launch_prep<32, 32>(const GdnArgs&, bool, cudaStream_t);
template int launch_prep<16, 32>(const GdnArgs&, bool, cudaStream_t);

}  // namespace lampa
