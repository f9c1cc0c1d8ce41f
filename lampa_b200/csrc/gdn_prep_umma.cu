// Per-chunk preparation of the gated-delta forward on the 5th-generation tensor cores, K = V = 64.
//
// One CTA of 8 warps turns 64 tokens of TWO heads (2p, 2p + 1) into their records
// {M, Q~, B^T, O_local, lambda_chunk}.  Every 64x64x64 contraction is a tcgen05.mma with M = 64:
// such an instruction occupies 16 lanes of each of the four 32-lane quarters of tensor memory, so
// the two heads interleave (head 0 in lanes 0..15 of a quarter, head 1 in lanes 16..31) and one
// tcgen05.ld hands every thread of the CTA one row segment: thread = (head, row, half of the
// columns).  Operands are bf16 tiles in shared memory with 128-byte rows and the 128-byte
// swizzle; the same tile serves as a K-major operand (rows = M/N index) or as an MN-major one
// (rows = K index), which is what lets K, V, W and U^ be used on either side of a product without
// a transpose.  Intermediates that are only ever a left operand (tril(QK^T), R, R.*E.*lambda) go
// from the accumulator through registers straight back into tensor memory as the bf16 A operand
// of the next product.  With Awb = (I + tril(diag(beta) K K^T, -1))^-1 diag(beta):
//   1  KK  = K K^T                (A, B K-major)        ->  A0, inverted in fp32 on CUDA cores
//   2  P   = tril(Q K^T)          (A, B K-major)        ->  A operand in tensor memory
//   3  R   = P Awb                (A tmem, B MN-major)  ->  A operands R and R .* E .* lambda
//   4  W   = Awb K                (A K-major, B MN)     ->  shared memory
//   5  U^  = (Awb diag(e^{Gl-G})) V                     ->  shared memory
//   6  M   = e^{Gl} (I - K^T W)   (A, B MN-major)       ->  record
//   7  B^T = U^^T K               (A, B MN-major)       ->  record
//   8  Q~  = s e^G (Q - R K)      (A tmem, B MN-major)  ->  record
//   9  O_local = s (R .* E .* lambda) V                 ->  record
// (U^ of gdn.cuh is diag(e^{Gl-G}) (Awb .* E) V; the row factor times E_ij is e^{Gl-G_j}, a column
// factor of Awb, so no 64x64 table of decays is needed for it.)
// The unit-lower-triangular inverse stays an fp32 substitution with split-bf16 block merges
// (gdn_inv.cuh), as in the reference (models/hattention/solve_tril.py:54-61, 175-197).
// Replaces the per-chunk Triton kernels of the reference's forward:
// fla_future/chunk_scaled_dot_kkt.py:14-74, solve_tril.py:221-276, fla_future/wy_fast.py:135-198,
// chunkwise_hgdn.py:40-125 (intra-chunk output), fla_future/chunk_delta_h.py:384-462.
#include "gdn.cuh"
#include "gdn_inv.cuh"
#include "gdn_load.cuh"
#include "profile.cuh"
#include "umma.cuh"

namespace lampa {

namespace {

constexpr int PT = 256;                       // threads
constexpr int PA = CHUNK + 4;                 // fp32 pitch of the inverse's working tile
constexpr int TILE = 8192;                    // one bf16 [64][64] operand tile
// shared-memory map (bytes); operand tiles are 1024-byte aligned
constexpr int S_BAR = 0;                      // mbarriers, TMEM slot at +192
constexpr int S_SC = 1024;                    // per head: G, beta, e^G, e^{Gl-G}: [2][4][64] fp32
constexpr int S_Q = 4096;                     // bf16 tiles [2 heads]: q (normalised)
constexpr int S_K = S_Q + 2 * TILE;           //                       k (normalised)
constexpr int S_V = S_K + 2 * TILE;           //                       v
constexpr int S_X = S_V + 2 * TILE;           // fp32 [2][64][PA] while inverting; then Awb -> W and Awb diag(e^{Gl-G}) -> U^
constexpr int S_X_BYTES = 2 * CHUNK * PA * 4;
constexpr int S_LAM = S_X + S_X_BYTES;        // fp32 [2][64][L + 1]
static_assert(4 * TILE <= S_X_BYTES && S_X % 1024 == 0, "operand tiles must fit over the inverse's tile");
constexpr int prep_umma_smem(int L) { return S_LAM + 2 * CHUNK * (L + 1) * 4; }
// tensor-memory columns (256 allocated): three 64-column accumulators and two 32-column A operands
constexpr int T0 = 0, T1 = 64, T2 = 128, TA_P = 192, TA_R = 224;
enum { B_KK = 0, B_QK, B_R, B_W, B_U, B_M, B_B, B_RK, B_PV, B_DRAIN, NBAR };

constexpr uint32_t ID_KK = umma_idesc(64, 64, 0, 0);   // A, B K-major
constexpr uint32_t ID_KN = umma_idesc(64, 64, 0, 1);   // A K-major (shared or tensor memory), B MN-major
constexpr uint32_t ID_NN = umma_idesc(64, 64, 1, 1);   // A, B MN-major

// 32 floats -> 16 packed bf16 words
__device__ __forceinline__ void pack32(const float (&x)[32], uint32_t (&w)[16]) {
#pragma unroll
    for (int c = 0; c < 16; ++c) w[c] = pack_bf16x2(x[2 * c], x[2 * c + 1]);
}
// 32 consecutive columns (chunks c8 .. c8 + 3) of row r of a swizzled bf16 tile <- 16 packed words
__device__ __forceinline__ void store_row_swz(unsigned char* tile, int r, int c8, const uint32_t (&w)[16]) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
        *reinterpret_cast<uint4*>(tile + r * 128 + (((c8 + q) ^ (r & 7)) << 4)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}

template <bool HIER>
__global__ void __launch_bounds__(PT, 2) gdn_prep_umma_kernel(GdnArgs a) {
    using R = Rec<64, 64>;
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S_BAR);
    uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + S_BAR + 192);
    float* sSc = reinterpret_cast<float*>(smem + S_SC);
    float* sLam = reinterpret_cast<float*>(smem + S_LAM);
    auto sG = [&](int sub) { return sSc + sub * 256; };
    auto sBeta = [&](int sub) { return sSc + sub * 256 + 64; };
    auto sEG = [&](int sub) { return sSc + sub * 256 + 128; };
    auto sEGl = [&](int sub) { return sSc + sub * 256 + 192; };

    const int pair = blockIdx.x, c = blockIdx.y, H = a.H;
    ChunkLoc loc;
    if (!locate_chunk(a, c, loc)) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t t0 = loc.t0;
    const int len = loc.len;
    const int LP = a.L + 1;
    const int budget = a.poll_budget;
    bool dead = false;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    stage_tick(a, cta, 0);


    // ---- stage 0: loads, l2norm, cumulative decay -------------------------------------------------
    // thread = (token r, head sub, half of the head's row); every global load of the chunk is issued
    // before any of them is consumed
    {
        const int r = tid >> 2, sub = (tid >> 1) & 1, half = tid & 1;
        const int h = 2 * pair + sub;
        const bool valid = h < H && r < len;
        const size_t tok = (size_t)(t0 + r);
        uint4 rq[4], rk[4], rv[4];
        issue_half_row<64>(a.q, (tok * H + h) * 64 + half * 32, valid, rq);
        issue_half_row<64>(a.k, (tok * H + h) * 64 + half * 32, valid, rk);
        issue_half_row<64>(a.v, (tok * H + h) * 64 + half * 32, valid, rv);
        float gv = 0.f, bv = 0.f;
        const int tk = tid & 63, sb = (tid >> 6) & 1;          // threads 0..127 carry g and beta of (head sb, token tk)
        if (tid < 128 && 2 * pair + sb < H && tk < len) {
            gv = load_as_float(a.g, (size_t)(t0 + tk) * H + 2 * pair + sb, a.gb_dt);
            bv = load_as_float(a.beta, (size_t)(t0 + tk) * H + 2 * pair + sb, a.gb_dt);
        }
        // (the loads above are in flight while the barriers and the tensor memory are set up)
        if (tid == 0) {
#pragma unroll
            for (int b = 0; b < NBAR; ++b) mbar_init(bars + b, 2);   // one arrival per issuing thread (one per head)
            fence_mbar_init();
        }
        if (warp == 0) tmem_alloc(tslot, 256);
        stage_tick(a, cta, 11);
        if (pair == 0) {   // L2 prefetch of everything a chunk ~80 chunks ahead will read (all heads)
            ChunkLoc l2;
            if (locate_chunk(a, c + 80, l2)) {
                const size_t row = (size_t)H * 64 * 2;
                if (tid < 128) {
                    const int rr = tid >> 1, hf = tid & 1;
                    if (rr < l2.len) {
                        const char* pq = (const char*)a.q + (size_t)(l2.t0 + rr) * row;
                        const char* pk = (const char*)a.k + (size_t)(l2.t0 + rr) * row;
                        const char* pv = (const char*)a.v + (size_t)(l2.t0 + rr) * row;
                        for (size_t off = (size_t)hf * 128; off < row; off += 256) {
                            asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pq + off));
                            asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pk + off));
                            asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pv + off));
                        }
                    }
                } else {
                    const int t2 = tid - 128;
                    const size_t gb_bytes = (size_t)l2.len * H * dtype_bytes(a.gb_dt);
                    const char* pg = (const char*)a.g + (size_t)l2.t0 * H * dtype_bytes(a.gb_dt);
                    const char* pb = (const char*)a.beta + (size_t)l2.t0 * H * dtype_bytes(a.gb_dt);
                    for (size_t off = (size_t)t2 * 128; off < gb_bytes; off += 128 * 128) {
                        asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pg + off));
                        asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pb + off));
                    }
                    if (HIER) {
                        const size_t lam_bytes = (size_t)l2.len * H * a.L * dtype_bytes(a.lam_dt);
                        const char* pl = (const char*)a.lam + (size_t)l2.t0 * H * a.L * dtype_bytes(a.lam_dt);
                        for (size_t off = (size_t)t2 * 128; off < lam_bytes; off += 128 * 128)
                            asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pl + off));
                    }
                }
            }
        }
        stage_tick(a, cta, 12);
        float x[32];
        uint32_t w[16];
        convert_half_row<64>(rq, a.qkv_dt, x);
        if (a.use_l2norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) ss += x[i] * x[i];
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            const float rn = rsqrtf(ss + 1e-6f);
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] *= rn;
        }
        pack32(x, w);
        store_row_swz(smem + S_Q + sub * TILE, r, half * 4, w);
        stage_tick(a, cta, 13);
        convert_half_row<64>(rk, a.qkv_dt, x);
        if (a.use_l2norm) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) ss += x[i] * x[i];
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);
            const float rn = rsqrtf(ss + 1e-6f);
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] *= rn;
        }
        pack32(x, w);
        store_row_swz(smem + S_K + sub * TILE, r, half * 4, w);
        if (a.qkv_dt == LAMPA_BF16) {   // v is used as it is
#pragma unroll
            for (int q = 0; q < 4; ++q) { w[4 * q] = rv[q].x; w[4 * q + 1] = rv[q].y; w[4 * q + 2] = rv[q].z; w[4 * q + 3] = rv[q].w; }
        } else {
            convert_half_row<64>(rv, a.qkv_dt, x);
            pack32(x, w);
        }
        store_row_swz(smem + S_V + sub * TILE, r, half * 4, w);
        stage_tick(a, cta, 14);
        if (HIER) {
            const size_t lam_base = (tok * H + h) * a.L;
            float* dst = sLam + (sub * CHUNK + r) * LP;
            if (a.L <= 18) stage_lambda<9>(a.lam, a.lam_dt, lam_base, a.L, half, valid, dst);
            else if (a.L <= 24) stage_lambda<12>(a.lam, a.lam_dt, lam_base, a.L, half, valid, dst);
            else stage_lambda<20>(a.lam, a.lam_dt, lam_base, a.L, half, valid, dst);
        }

        if (tid < 128) {   // inclusive cumsum of g over the 64 tokens of head sb (two warps per head)
            float cs = gv;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float yy = __shfl_up_sync(0xffffffffu, cs, o);
                if (lane >= o) cs += yy;
            }
            if (lane == 31 && !(warp & 1)) sG(sb)[CHUNK - 1] = cs;      // one-float mailbox between the head's two warps
            sBeta(sb)[tk] = bv;
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            const float carry = (warp & 1) ? sG(sb)[CHUNK - 1] : 0.f;
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            sG(sb)[tk] = cs + carry;
        }
        stage_tick(a, cta, 15);
    }
    __syncthreads();
    stage_tick(a, cta, 1);
    if (tid < 128) {
        const int tk = tid & 63, sb = tid >> 6;
        const float Gi = sG(sb)[tk], Gl = sG(sb)[CHUNK - 1];
        sEG(sb)[tk] = __expf(Gi);
        sEGl(sb)[tk] = __expf(Gl - Gi);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t taddr = *tslot;
    const uint32_t sQ = smem_u32(smem + S_Q), sK = smem_u32(smem + S_K), sV = smem_u32(smem + S_V), sX = smem_u32(smem + S_X);

    // ---- products 1, 2 ------------------------------------------------------------------------------
    const bool issuer = (tid & 127) == 0;      // thread 0 issues head 0's products, thread 128 head 1's
    const int isub = tid >> 7;
    if (issuer) {
        {
            const int sub = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ss(taddr + ((uint32_t)(16 * sub) << 16) + T0, umma_desc_k128(sK + sub * TILE + kk * 32),
                            umma_desc_k128(sK + sub * TILE + kk * 32), ID_KK, kk > 0);
        }
        umma_commit(bars + B_KK);
        {
            const int sub = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ss(taddr + ((uint32_t)(16 * sub) << 16) + T1, umma_desc_k128(sQ + sub * TILE + kk * 32),
                            umma_desc_k128(sK + sub * TILE + kk * 32), ID_KK, kk > 0);
        }
        umma_commit(bars + B_QK);
    }
    __syncwarp();

    // epilogue coordinates: this thread owns row i of head sub, columns 32 ch .. 32 ch + 31
    const int sp = warp & 3, ch = warp >> 2;
    const int sub = lane >> 4, i = 16 * sp + (lane & 15);
    const uint32_t tlane = taddr + ((uint32_t)(32 * sp) << 16);
    const int h = 2 * pair + sub;
    const bool head_ok = h < H;
    char* rec = a.rec + ((size_t)c * H + (head_ok ? h : 0)) * a.rec_bytes;
    float x[32];
    uint32_t w[16];

    stage_tick(a, cta, 2);
    // A0 = tril(diag(beta) K K^T, -1) as fp32 into the inverse's tile
    mbar_wait(bars + B_KK, 0u, dead, a.status, 600, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T0 + 32 * ch);
    {
        float* sA = reinterpret_cast<float*>(smem + S_X) + sub * CHUNK * PA + i * PA + 32 * ch;
        const float bi = sBeta(sub)[i];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int j = 32 * ch + 4 * q;
            *reinterpret_cast<float4*>(sA + 4 * q) = make_float4(j < i ? bi * x[4 * q] : 0.f, j + 1 < i ? bi * x[4 * q + 1] : 0.f,
                                                                 j + 2 < i ? bi * x[4 * q + 2] : 0.f, j + 3 < i ? bi * x[4 * q + 3] : 0.f);
        }
    }
    // P = tril(Q K^T) as the bf16 A operand of product 3
    mbar_wait(bars + B_QK, 0u, dead, a.status, 601, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T1 + 32 * ch);
#pragma unroll
    for (int jj = 0; jj < 32; ++jj)
        if (32 * ch + jj > i) x[jj] = 0.f;
    pack32(x, w);
    tmem_st16(tlane + TA_P + 16 * ch, w);
    tc_fence_before();
    __syncthreads();

    stage_tick(a, cta, 3);
    // ---- the inverse: warp = (head, 16-row block) ----------------------------------------------------
    tril_inverse_64<PA>(reinterpret_cast<float*>(smem + S_X) + (warp >> 2) * CHUNK * PA, warp & 3, lane);
    stage_tick(a, cta, 4);
    {   // Awb = X diag(beta) and Awb diag(e^{Gl-G}) as bf16 tiles over the front of the fp32 tiles
        const int sb = tid >> 7, r = (tid & 127) >> 1, half = tid & 1;
        const float* sA = reinterpret_cast<const float*>(smem + S_X) + sb * CHUNK * PA + r * PA + half * 32;
        uint32_t ws[16];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float4 v = *reinterpret_cast<const float4*>(sA + 4 * q);
            const float4 b = *reinterpret_cast<const float4*>(sBeta(sb) + half * 32 + 4 * q);
            const float4 e = *reinterpret_cast<const float4*>(sEGl(sb) + half * 32 + 4 * q);
            const float y0 = v.x * b.x, y1 = v.y * b.y, y2 = v.z * b.z, y3 = v.w * b.w;
            w[2 * q] = pack_bf16x2(y0, y1);
            w[2 * q + 1] = pack_bf16x2(y2, y3);
            ws[2 * q] = pack_bf16x2(y0 * e.x, y1 * e.y);
            ws[2 * q + 1] = pack_bf16x2(y2 * e.z, y3 * e.w);
        }
        __syncthreads();
        store_row_swz(smem + S_X + sb * TILE, r, half * 4, w);
        store_row_swz(smem + S_X + 2 * TILE + sb * TILE, r, half * 4, ws);
    }
    fence_async_smem();
    __syncthreads();

    stage_tick(a, cta, 5);
    // ---- products 3, 4, 5 ---------------------------------------------------------------------------
    if (issuer && !dead) {
        tc_fence_after();
        {
            const int sb = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ts(taddr + ((uint32_t)(16 * sb) << 16) + T0, taddr + ((uint32_t)(16 * sb) << 16) + TA_P + 8 * kk,
                            umma_desc_mn128(sX + sb * TILE + kk * 2048), ID_KN, kk > 0);
        }
        umma_commit(bars + B_R);
        {
            const int sb = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ss(taddr + ((uint32_t)(16 * sb) << 16) + T1, umma_desc_k128(sX + sb * TILE + kk * 32),
                            umma_desc_mn128(sK + sb * TILE + kk * 2048), ID_KN, kk > 0);
        }
        umma_commit(bars + B_W);
        {
            const int sb = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ss(taddr + ((uint32_t)(16 * sb) << 16) + T2, umma_desc_k128(sX + 2 * TILE + sb * TILE + kk * 32),
                            umma_desc_mn128(sV + sb * TILE + kk * 2048), ID_KN, kk > 0);
        }
        umma_commit(bars + B_U);
    }
    __syncwarp();

    // W and U^ back to shared memory (over Awb and its scaled copy: every product that read them is complete)
    mbar_wait(bars + B_W, 0u, dead, a.status, 602, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T1 + 32 * ch);
    pack32(x, w);
    store_row_swz(smem + S_X + sub * TILE, i, 4 * ch, w);
    mbar_wait(bars + B_U, 0u, dead, a.status, 603, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T2 + 32 * ch);
    pack32(x, w);
    store_row_swz(smem + S_X + 2 * TILE + sub * TILE, i, 4 * ch, w);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    stage_tick(a, cta, 6);
    // ---- products 6, 7 ------------------------------------------------------------------------------
    if (issuer && !dead) {
        tc_fence_after();
        {
            const int sb = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ss(taddr + ((uint32_t)(16 * sb) << 16) + T1, umma_desc_mn128(sK + sb * TILE + kk * 2048),
                            umma_desc_mn128(sX + sb * TILE + kk * 2048), ID_NN, kk > 0);
        }
        umma_commit(bars + B_M);
        {
            const int sb = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ss(taddr + ((uint32_t)(16 * sb) << 16) + T2, umma_desc_mn128(sX + 2 * TILE + sb * TILE + kk * 2048),
                            umma_desc_mn128(sK + sb * TILE + kk * 2048), ID_NN, kk > 0);
        }
        umma_commit(bars + B_B);
    }
    __syncwarp();

    // R (product 3 is long complete) -> the two A operands of products 8 and 9
    const float osc = HIER ? 1.f : a.scale;
    tmem_ld32(x, tlane + T0 + 32 * ch);
    pack32(x, w);                                     // R is lower triangular by construction: no mask
    tmem_st16(tlane + TA_R + 16 * ch, w);
    {
        // Pm = R .* E .* lambda[i][level(i, j)], E_ij = e^{G_i - G_j} for j <= i (masked before the exponential).
        // level(i, j) = bit_length(i ^ j): off the diagonal 8x8 tile it depends on the tiles only.
        const int ib = i >> 3;
        const float Gi = sG(sub)[i];
        const float* lrow = sLam + (sub * CHUNK + i) * LP;
#pragma unroll
        for (int b4 = 0; b4 < 4; ++b4) {
            const int jb = 4 * ch + b4;
            if (jb > ib) {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[8 * b4 + e] = 0.f;
            } else {
                const float4 g0 = *reinterpret_cast<const float4*>(sG(sub) + 8 * jb);
                const float4 g1 = *reinterpret_cast<const float4*>(sG(sub) + 8 * jb + 4);
                const float gj[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                if (jb < ib) {
                    const float lt = HIER ? lrow[3 + (32 - __clz(ib ^ jb))] : 1.f;
#pragma unroll
                    for (int e = 0; e < 8; ++e) x[8 * b4 + e] *= __expf(Gi - gj[e]) * lt;
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int j = 8 * jb + e;
                        const float f = (j <= i) ? __expf(Gi - gj[e]) * (HIER ? lrow[32 - __clz(i ^ j)] : 1.f) : 0.f;
                        x[8 * b4 + e] *= f;
                    }
                }
            }
        }
    }
    pack32(x, w);
    tmem_st16(tlane + TA_P + 16 * ch, w);
    tc_fence_before();
    __syncthreads();

    stage_tick(a, cta, 7);
    // ---- product 8 ----------------------------------------------------------------------------------
    if (issuer && !dead) {
        tc_fence_after();
        {
            const int sb = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ts(taddr + ((uint32_t)(16 * sb) << 16) + T0, taddr + ((uint32_t)(16 * sb) << 16) + TA_R + 8 * kk,
                            umma_desc_mn128(sK + sb * TILE + kk * 2048), ID_KN, kk > 0);
        }
        umma_commit(bars + B_RK);
    }
    __syncwarp();

    // M[a][b] = e^{Gl} (delta_ab - (K^T W)[a][b]) -> record
    mbar_wait(bars + B_M, 0u, dead, a.status, 604, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T1 + 32 * ch);
    {
        const float egl = sEG(sub)[CHUNK - 1];
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) x[jj] = egl * ((32 * ch + jj == i ? 1.f : 0.f) - x[jj]);
        pack32(x, w);
        if (head_ok) store_row_swz(reinterpret_cast<unsigned char*>(rec) + R::M_OFF, i, 4 * ch, w);
    }
    tc_fence_before();
    __syncthreads();

    stage_tick(a, cta, 8);
    // ---- product 9 ----------------------------------------------------------------------------------
    if (issuer && !dead) {
        tc_fence_after();
        {
            const int sb = isub;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk)
                umma_f16_ts(taddr + ((uint32_t)(16 * sb) << 16) + T1, taddr + ((uint32_t)(16 * sb) << 16) + TA_P + 8 * kk,
                            umma_desc_mn128(sV + sb * TILE + kk * 2048), ID_KN, kk > 0);
        }
        umma_commit(bars + B_PV);
    }
    __syncwarp();

    // (while product 9 runs)
    if (HIER) {   // lambda of the chunk levels, transposed to [level][token] for the scan
        for (int idx = tid; idx < 2 * a.LC * CHUNK; idx += PT) {
            const int sub = idx / (a.LC * CHUNK), rem = idx - sub * a.LC * CHUNK;
            const int l = rem >> 6, r = rem & 63;
            if (2 * pair + sub < H) {
                float* lamc = reinterpret_cast<float*>(a.rec + ((size_t)c * H + 2 * pair + sub) * a.rec_bytes + R::LAM_OFF);
                lamc[rem] = (ELL0 + l < a.L) ? sLam[(sub * CHUNK + r) * LP + ELL0 + l] : 0.f;
            }
        }
    }
    // B^T -> record
    mbar_wait(bars + B_B, 0u, dead, a.status, 605, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T2 + 32 * ch);
    pack32(x, w);
    if (head_ok) store_row_swz(reinterpret_cast<unsigned char*>(rec) + R::BT_OFF, i, 4 * ch, w);

    // Q~ = s e^{G_i} (Q - R K) -> record
    mbar_wait(bars + B_RK, 0u, dead, a.status, 606, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T0 + 32 * ch);
    {
        const float f = osc * sEG(sub)[i];
        const unsigned char* qt = smem + S_Q + sub * TILE + i * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint4 u = *reinterpret_cast<const uint4*>(qt + (((4 * ch + q) ^ (i & 7)) << 4));
            const uint32_t uw[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 qv = unpack_bf16x2(uw[e]);
                w[4 * q + e] = pack_bf16x2(f * (qv.x - x[8 * q + 2 * e]), f * (qv.y - x[8 * q + 2 * e + 1]));
            }
        }
        if (head_ok) store_row_swz(reinterpret_cast<unsigned char*>(rec) + R::QT_OFF, i, 4 * ch, w);
    }

    // O_local = s Pm V -> record (bf16 [64][64], plain rows)
    mbar_wait(bars + B_PV, 0u, dead, a.status, 607, budget);
    tc_fence_after();
    tmem_ld32(x, tlane + T1 + 32 * ch);
    if (!HIER) {
#pragma unroll
        for (int jj = 0; jj < 32; ++jj) x[jj] *= osc;
    }
    pack32(x, w);
    if (head_ok) {
        uint4* dst = reinterpret_cast<uint4*>(rec + R::OL_OFF + (i * 64 + 32 * ch) * 2);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }

    stage_tick(a, cta, 9);
    // nothing asynchronous may outlive the CTA: one last commit covers every product issued above
    if (issuer) {
        umma_commit(bars + B_DRAIN);
        mbar_drain(bars + B_DRAIN, 0u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, 256);
    stage_tick(a, cta, 10);
}

}  // namespace

int launch_prep_umma(const GdnArgs& a, bool hier, cudaStream_t st) {
    const int smem = prep_umma_smem(hier ? a.L : 0);
    if (smem > 113 * 1024) return LAMPA_ERR_UNSUPPORTED;
    dim3 grid((a.H + 1) / 2, a.nc_max);
    ProfScope prof(hier ? "gdn_prep_hier" : "gdn_prep_plain", st);
    if (hier) {
        if (cudaFuncSetAttribute(gdn_prep_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return LAMPA_ERR_CUDA;
        gdn_prep_umma_kernel<true><<<grid, PT, smem, st>>>(a);
    } else {
        if (cudaFuncSetAttribute(gdn_prep_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return LAMPA_ERR_CUDA;
        gdn_prep_umma_kernel<false><<<grid, PT, smem, st>>>(a);
    }
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

}  // namespace lampa
