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
// The four record tiles are assembled in shared memory in the record's own layout (over operands that are
// dead by then) and leave as bulk stores.
// (U^ of gdn.cuh is diag(e^{Gl-G}) (Awb .* E) V; the row factor times E_ij is e^{Gl-G_j}, a column
// factor of Awb, so no 64x64 table of decays is needed for it.)
// The unit-lower-triangular inverse stays an fp32 substitution with split-bf16 block merges
// (gdn_inv.cuh), as in the reference (models/hattention/solve_tril.py:54-61, 175-197).
// Replaces the per-chunk Triton kernels of the reference's forward:
// fla_future/chunk_scaled_dot_kkt.py:14-74, solve_tril.py:221-276, fla_future/wy_fast.py:135-198,
// chunkwise_hgdn.py:40-125 (intra-chunk output), fla_future/chunk_delta_h.py:384-462.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cstdlib>

#include "gdn.cuh"
#include "gdn_inv.cuh"
#include "gdn_load.cuh"
#include "profile.cuh"
#include "umma.cuh"

namespace lampa {

namespace {

constexpr int PA = CHUNK + 4;                 // fp32 pitch of the inverse's working tile
constexpr int TILE = 8192;                    // one bf16 [64][64] operand tile
// shared-memory map (bytes); operand tiles are 1024-byte aligned
constexpr int S_BAR = 0;                      // mbarriers, TMEM slot at +192
constexpr int S_SC = 1024;                    // per head: G, beta, e^G, e^{Gl-G}, e^{G(end of 8-block)-G}: [2][5][64] fp32
constexpr int S_Q = 4096;                     // bf16 tiles [2 heads]: q (normalised)
constexpr int S_K = S_Q + 2 * TILE;           //                       k (normalised)
constexpr int S_V = S_K + 2 * TILE;           //                       v
constexpr int S_X = S_V + 2 * TILE;           // fp32 [2][64][PA] while inverting; then Awb -> W and Awb diag(e^{Gl-G}) -> U^
constexpr int S_X_BYTES = 2 * CHUNK * PA * 4;
constexpr int S_LAM = S_X + S_X_BYTES;        // fp32 [2][64][L + 1]
static_assert(4 * TILE <= S_X_BYTES && S_X % 1024 == 0, "operand tiles must fit over the inverse's tile");
constexpr int LAM_TMA_MAX = 20 * 1024;       // largest [64][H * L] 2-byte lambda tile taken by TMA
inline int prep_umma_smem(int L, int lam_tma_bytes) {
    const int staged = 2 * CHUNK * (L + 1) * 4;
    return S_LAM + (lam_tma_bytes > staged ? lam_tma_bytes : staged);
}

// 2-D tiled TMA load of one box into shared memory, completion on an mbarrier; x = innermost coordinate
// (elements; x * element size must be a multiple of 16 bytes), y = row.  Single CTA, no multicast.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int32_t x, int32_t y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 :: "r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int32_t x, int32_t y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n"
                 :: "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y) : "memory");
}
// tensor-memory columns (256 allocated): three 64-column accumulators and two 32-column A operands
constexpr int T0 = 0, T1 = 64, T2 = 128, TA_P = 192, TA_R = 224;
// one mbarrier per group of products issued together (commits complete in issue order, so the group's last one covers it)
enum { B_G1 = 0, B_G2, B_G3, B_PV, B_DRAIN, B_IN, NBAR };

constexpr uint32_t ID_KK = umma_idesc(64, 64, 0, 0);   // A, B K-major
constexpr uint32_t ID_KN = umma_idesc(64, 64, 0, 1);   // A K-major (shared or tensor memory), B MN-major
constexpr uint32_t ID_NN = umma_idesc(64, 64, 1, 1);   // A, B MN-major

// N floats -> N / 2 packed bf16 words
template <int N>
__device__ __forceinline__ void pack_n(const float (&x)[N], uint32_t (&w)[N / 2]) {
#pragma unroll
    for (int c = 0; c < N / 2; ++c) w[c] = pack_bf16x2(x[2 * c], x[2 * c + 1]);
}
// N consecutive columns (16-byte chunks c8 .. c8 + N/8 - 1) of row r of a swizzled bf16 tile <- N / 2 packed words
template <int N>
__device__ __forceinline__ void store_cols_swz(unsigned char* tile, int r, int c8, const uint32_t (&w)[N / 2]) {
#pragma unroll
    for (int q = 0; q < N / 8; ++q)
        *reinterpret_cast<uint4*>(tile + r * 128 + (((c8 + q) ^ (r & 7)) << 4)) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
}
template <int N>
__device__ __forceinline__ void load_cols_swz(const unsigned char* tile, int r, int c8, uint4 (&raw)[N / 8]) {
#pragma unroll
    for (int q = 0; q < N / 8; ++q) raw[q] = *reinterpret_cast<const uint4*>(tile + r * 128 + (((c8 + q) ^ (r & 7)) << 4));
}
template <int N> __device__ __forceinline__ void tmem_ld_n(float (&x)[N], uint32_t taddr);
template <> __device__ __forceinline__ void tmem_ld_n<32>(float (&x)[32], uint32_t taddr) { tmem_ld32(x, taddr); }
template <> __device__ __forceinline__ void tmem_ld_n<16>(float (&x)[16], uint32_t taddr) { tmem_ld16(x, taddr); }
template <int W> __device__ __forceinline__ void tmem_st_n(uint32_t taddr, const uint32_t (&w)[W]);
template <> __device__ __forceinline__ void tmem_st_n<16>(uint32_t taddr, const uint32_t (&w)[16]) { tmem_st16(taddr, w); }
template <> __device__ __forceinline__ void tmem_st_n<8>(uint32_t taddr, const uint32_t (&w)[8]) { tmem_st8(taddr, w); }

// descriptor of the same operand `bytes` further on (k-steps): only the start-address field moves
__device__ __forceinline__ uint64_t desc_adv(uint64_t d, uint32_t bytes) { return d + (uint64_t)(bytes >> 4); }

// NC = columns of an accumulator row per thread: 32 (8 warps) or 16 (16 warps, half the registers).
template <bool HIER, int NC>
__global__ void __launch_bounds__(8192 / NC, 2) gdn_prep_umma_kernel(GdnArgs a, const __grid_constant__ CUtensorMap tq,
                                                                     const __grid_constant__ CUtensorMap tk,
                                                                     const __grid_constant__ CUtensorMap tv,
                                                                     const __grid_constant__ CUtensorMap tl, int lam_tma) {
    using R = Rec<64, 64>;
    constexpr int PT = 8192 / NC;                 // threads
    constexpr int PARTS = 64 / NC;                // threads per row of 64
    constexpr int NCH = NC / 8;                   // 16-byte chunks of bf16 per thread and row
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S_BAR);
    uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + S_BAR + 192);
    float* sSc = reinterpret_cast<float*>(smem + S_SC);
    float* sLam = reinterpret_cast<float*>(smem + S_LAM);
    auto sG = [&](int sub) { return sSc + sub * 320; };
    auto sBeta = [&](int sub) { return sSc + sub * 320 + 64; };
    auto sEG = [&](int sub) { return sSc + sub * 320 + 128; };
    auto sEGl = [&](int sub) { return sSc + sub * 320 + 192; };
    auto sCF = [&](int sub) { return sSc + sub * 320 + 256; };      // e^{G_{8 (j / 8) + 7} - G_j}: decay from token j to the end of its 8-block

    const int pair = blockIdx.x, c = blockIdx.y, H = a.H;
    // lambda[token r of the chunk][head 2 pair + sb][level]: from the TMA tile (2-byte rows of all heads) or from the staged fp32 copy
    auto lam_at = [&](int sb, int r, int lev) -> float {
        if (lam_tma) return load_as_float(smem + S_LAM, (size_t)(r * H + 2 * pair + sb) * a.L + lev, a.lam_dt);
        return sLam[(sb * CHUNK + r) * (a.L + 1) + lev];
    };
    ChunkLoc loc;
    if (a.plan_inline && blockIdx.x == 0 && blockIdx.y == 0) write_fixed_plan(a);
    if (!locate_chunk(a, c, loc)) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t t0 = loc.t0;
    const int len = loc.len;
    if (blockIdx.x == 0) check_out_perm(a, t0, len);
    const int LP = a.L + 1;
    const int budget = a.poll_budget;
    bool dead = false;
    const int cta = blockIdx.y * gridDim.x + blockIdx.x;
    stage_tick(a, cta, 0);
    if (a.ticks != nullptr && threadIdx.x == 0 && cta < a.ticks_ctas) {
        unsigned sm_; unsigned long long gt_;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(sm_));
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));
        a.ticks[(size_t)cta * 16 + 11] = sm_; a.ticks[(size_t)cta * 16 + 12] = (long long)gt_;
    }

    // ---- stage 0: TMA loads, l2norm, cumulative decay ---------------------------------------------
    // One thread asks the TMA unit for the six 64 x 64 tiles (q, k, v of both heads): they land in the
    // 128-byte-swizzled operand layout, rows past the end of the tensor or of a missing head as zeros.
    // A 2-byte lambda comes the same way as whole token rows [64][H * L]; g and beta by plain loads.
    if (tid == 0) {
#pragma unroll
        for (int b = 0; b < NBAR; ++b) mbar_init(bars + b, b == B_IN ? 1 : 2);   // products: one arrival per issuing thread (one per head)
        fence_mbar_init();
        const int32_t y = (int32_t)t0;
        const uint32_t lam_bytes = lam_tma ? (uint32_t)(CHUNK * H * a.L * 2) : 0u;
        mbar_expect_tx(bars + B_IN, 6u * TILE + lam_bytes);
#pragma unroll
        for (int sb = 0; sb < 2; ++sb) {
            const int32_t x = (2 * pair + sb) * 64;
            tma_load_2d(smem + S_Q + sb * TILE, &tq, x, y, bars + B_IN);
            tma_load_2d(smem + S_K + sb * TILE, &tk, x, y, bars + B_IN);
            tma_load_2d(smem + S_V + sb * TILE, &tv, x, y, bars + B_IN);
        }
        if (lam_tma) tma_load_2d(smem + S_LAM, &tl, 0, y, bars + B_IN);
    }
    if (warp == 1) tmem_alloc(tslot, 256);
    if (pair == 0 && warp == 2) {   // L2 prefetch of everything a chunk ~80 chunks ahead will read (all heads)
        ChunkLoc l2;
        if (locate_chunk(a, c + 80, l2)) {
            if (lane < H) {
                tma_prefetch_2d(&tq, lane * 64, (int32_t)l2.t0);
                tma_prefetch_2d(&tk, lane * 64, (int32_t)l2.t0);
                tma_prefetch_2d(&tv, lane * 64, (int32_t)l2.t0);
            }
            if (lam_tma && lane == 31) tma_prefetch_2d(&tl, 0, (int32_t)l2.t0);
            const size_t gb_bytes = (size_t)l2.len * H * dtype_bytes(a.gb_dt);
            const char* pg = (const char*)a.g + (size_t)l2.t0 * H * dtype_bytes(a.gb_dt);
            const char* pb = (const char*)a.beta + (size_t)l2.t0 * H * dtype_bytes(a.gb_dt);
            for (size_t off = (size_t)lane * 128; off < gb_bytes; off += 32 * 128) {
                asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pg + off));
                asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pb + off));
            }
            if (HIER && !lam_tma) {
                const size_t lam_b = (size_t)l2.len * H * a.L * dtype_bytes(a.lam_dt);
                const char* pl = (const char*)a.lam + (size_t)l2.t0 * H * a.L * dtype_bytes(a.lam_dt);
                for (size_t off = (size_t)lane * 128; off < lam_b; off += 32 * 128)
                    asm volatile("prefetch.global.L2 [%0];\n" :: "l"(pl + off));
            }
        }
    }
    float x[NC];
    uint32_t w[NC / 2];
    {
        // thread = (token r, head sub, part of the head's row)
        const int r = tid / (2 * PARTS), sub = (tid / PARTS) & 1, part = tid & (PARTS - 1);
        const int h = 2 * pair + sub;
        const bool valid = h < H && r < len;
        float gv = 0.f, bv = 0.f;
        const int tk_ = tid & 63, sb = (tid >> 6) & 1;         // threads 0..127 carry g and beta of (head sb, token tk_)
        if (tid < 128 && 2 * pair + sb < H && tk_ < len) {
            gv = load_as_float(a.g, (size_t)(t0 + tk_) * H + 2 * pair + sb, a.gb_dt);
            bv = load_as_float(a.beta, (size_t)(t0 + tk_) * H + 2 * pair + sb, a.gb_dt);
        }
        if (HIER && !lam_tma && part < 2) {   // 4-byte lambda, or a row pitch the TMA unit cannot take: staged as fp32 [2][64][L + 1]
            const size_t lam_base = ((size_t)(t0 + r) * H + h) * a.L;
            float* dst = sLam + (sub * CHUNK + r) * LP;
            if (a.L <= 18) stage_lambda<9>(a.lam, a.lam_dt, lam_base, a.L, part, valid, dst);
            else if (a.L <= 24) stage_lambda<12>(a.lam, a.lam_dt, lam_base, a.L, part, valid, dst);
            else stage_lambda<20>(a.lam, a.lam_dt, lam_base, a.L, part, valid, dst);
        }
        if (tid < 128) {   // inclusive cumsum of g over the 64 tokens of head sb (two warps per head)
            float cs = gv;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float yy = __shfl_up_sync(0xffffffffu, cs, o);
                if (lane >= o) cs += yy;
            }
            if (lane == 31 && !(warp & 1)) sG(sb)[CHUNK - 1] = cs;      // one-float mailbox between the head's two warps
            sBeta(sb)[tk_] = bv;
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            const float carry = (warp & 1) ? sG(sb)[CHUNK - 1] : 0.f;
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            const float Gi = cs + carry;
            sG(sb)[tk_] = Gi;
            sEG(sb)[tk_] = __expf(Gi);
        }
        // the tiles have landed: normalise q and k in place, clear rows past the chunk's end
        __syncthreads();                                   // barrier initialisation visible to every waiter
        mbar_wait(bars + B_IN, 0u, dead, a.status, 610, budget);
        uint4 raw[NCH];
#pragma unroll
        for (int which = 0; which < 2; ++which) {
            unsigned char* tile = smem + (which == 0 ? S_Q : S_K) + sub * TILE;
            load_cols_swz<NC>(tile, r, part * NCH, raw);
            convert_half_row<2 * NC>(raw, a.qkv_dt, x);
            float rn = 1.f;
            if (a.use_l2norm) {
                float ss = 0.f;
#pragma unroll
                for (int i = 0; i < NC; ++i) ss += x[i] * x[i];
#pragma unroll
                for (int o = 1; o < PARTS; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                rn = rsqrtf(ss + 1e-6f);
            }
#pragma unroll
            for (int i = 0; i < NC; ++i) x[i] = valid ? x[i] * rn : 0.f;      // rows past the chunk's end hold another sequence's data
            pack_n<NC>(x, w);
            store_cols_swz<NC>(tile, r, part * NCH, w);
        }
        if (a.qkv_dt != LAMPA_BF16 || !valid) {   // v is used as it landed unless it is fp16 or lies past the chunk's end
            unsigned char* tile = smem + S_V + sub * TILE;
            load_cols_swz<NC>(tile, r, part * NCH, raw);
            convert_half_row<2 * NC>(raw, a.qkv_dt, x);
#pragma unroll
            for (int i = 0; i < NC; ++i) x[i] = valid ? x[i] : 0.f;
            pack_n<NC>(x, w);
            store_cols_swz<NC>(tile, r, part * NCH, w);
        }
    }
    __syncthreads();
    stage_tick(a, cta, 1);
    if (tid < 128) {
        const int tk2 = tid & 63, sb = tid >> 6;
        sEGl(sb)[tk2] = __expf(sG(sb)[CHUNK - 1] - sG(sb)[tk2]);
        sCF(sb)[tk2] = __expf(sG(sb)[tk2 | 7] - sG(sb)[tk2]);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t taddr = *tslot;
    const uint32_t sQ = smem_u32(smem + S_Q), sK = smem_u32(smem + S_K), sV = smem_u32(smem + S_V), sX = smem_u32(smem + S_X);

    // ---- products 1, 2 ------------------------------------------------------------------------------
    // Two threads issue the products, one per head: lane 0 of the two warps that own rows 0..31 of the last column
    // group.  Everything they own lies above the diagonal, so their share of the triangular epilogues is the
    // smallest and the time they spend issuing hides behind the other warps' work.
    constexpr int IW0 = 4 * (64 / NC - 1);
    const bool issuer = lane == 0 && (warp == IW0 || warp == IW0 + 1);
    const int isub = warp == IW0 + 1 ? 1 : 0;
    const uint32_t dsub = taddr + ((uint32_t)(16 * isub) << 16);   // the issuer's head: lanes 16 isub .. of every quarter
    if (issuer) {
        const uint64_t dK = umma_desc_k128(sK + isub * TILE), dQ = umma_desc_k128(sQ + isub * TILE);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ss(dsub + T0, desc_adv(dK, kk * 32), desc_adv(dK, kk * 32), ID_KK, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ss(dsub + T1, desc_adv(dQ, kk * 32), desc_adv(dK, kk * 32), ID_KK, kk > 0);
        umma_commit(bars + B_G1);
    }
    __syncwarp();

    // epilogue coordinates: this thread owns row i of head sub, columns NC cq .. NC cq + NC - 1
    const int sp = warp & 3, cq = warp >> 2;
    const int sub = lane >> 4, i = 16 * sp + (lane & 15);
    const int col0 = NC * cq;
    const uint32_t tlane = taddr + ((uint32_t)(32 * sp) << 16);

    stage_tick(a, cta, 2);
    // A0 = tril(diag(beta) K K^T, -1) as fp32 into the inverse's tile
    mbar_wait(bars + B_G1, 0u, dead, a.status, 600, budget);
    tc_fence_after();
    tmem_ld_n<NC>(x, tlane + T0 + col0);
    {
        float* sA = reinterpret_cast<float*>(smem + S_X) + sub * CHUNK * PA + i * PA + col0;
        const float bi = sBeta(sub)[i];
#pragma unroll
        for (int q = 0; q < NC / 4; ++q) {
            const int j = col0 + 4 * q;
            *reinterpret_cast<float4*>(sA + 4 * q) = make_float4(j < i ? bi * x[4 * q] : 0.f, j + 1 < i ? bi * x[4 * q + 1] : 0.f,
                                                                 j + 2 < i ? bi * x[4 * q + 2] : 0.f, j + 3 < i ? bi * x[4 * q + 3] : 0.f);
        }
    }
    // P = tril(Q K^T) as the bf16 A operand of product 3
    tmem_ld_n<NC>(x, tlane + T1 + col0);
#pragma unroll
    for (int jj = 0; jj < NC; ++jj)
        if (col0 + jj > i) x[jj] = 0.f;
    pack_n<NC>(x, w);
    tmem_st_n<NC / 2>(tlane + TA_P + col0 / 2, w);
    tc_fence_before();
    __syncthreads();

    stage_tick(a, cta, 3);
    // ---- the inverse: warps 0..7 = (head, 16-row block) ---------------------------------------------
    tril_inverse_64<PA>(reinterpret_cast<float*>(smem + S_X) + ((warp >> 2) & 1) * CHUNK * PA, warp & 3, lane, warp < 8);
    stage_tick(a, cta, 4);
    {   // Awb = X diag(beta) and Awb diag(e^{Gl-G}) as bf16 tiles over the front of the fp32 tiles
        const int sb = tid / (PT / 2), r = (tid % (PT / 2)) / PARTS, part = tid & (PARTS - 1);
        const float* sA = reinterpret_cast<const float*>(smem + S_X) + sb * CHUNK * PA + r * PA + part * NC;
        uint32_t ws[NC / 2];
#pragma unroll
        for (int q = 0; q < NC / 4; ++q) {
            const float4 v = *reinterpret_cast<const float4*>(sA + 4 * q);
            const float4 b = *reinterpret_cast<const float4*>(sBeta(sb) + part * NC + 4 * q);
            const float4 e = *reinterpret_cast<const float4*>(sEGl(sb) + part * NC + 4 * q);
            const float y0 = v.x * b.x, y1 = v.y * b.y, y2 = v.z * b.z, y3 = v.w * b.w;
            w[2 * q] = pack_bf16x2(y0, y1);
            w[2 * q + 1] = pack_bf16x2(y2, y3);
            ws[2 * q] = pack_bf16x2(y0 * e.x, y1 * e.y);
            ws[2 * q + 1] = pack_bf16x2(y2 * e.z, y3 * e.w);
        }
        __syncthreads();
        store_cols_swz<NC>(smem + S_X + sb * TILE, r, part * NCH, w);
        store_cols_swz<NC>(smem + S_X + 2 * TILE + sb * TILE, r, part * NCH, ws);
    }
    fence_async_smem();
    __syncthreads();

    stage_tick(a, cta, 5);
    // ---- products 3, 4, 5 ---------------------------------------------------------------------------
    if (issuer && !dead) {
        tc_fence_after();
        const uint64_t dAwbN = umma_desc_mn128(sX + isub * TILE), dAwbK = umma_desc_k128(sX + isub * TILE);
        const uint64_t dAwsK = umma_desc_k128(sX + 2 * TILE + isub * TILE);
        const uint64_t dKN = umma_desc_mn128(sK + isub * TILE), dVN = umma_desc_mn128(sV + isub * TILE);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ts(dsub + T0, dsub + TA_P + 8 * kk, desc_adv(dAwbN, kk * 2048), ID_KN, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ss(dsub + T1, desc_adv(dAwbK, kk * 32), desc_adv(dKN, kk * 2048), ID_KN, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ss(dsub + T2, desc_adv(dAwsK, kk * 32), desc_adv(dVN, kk * 2048), ID_KN, kk > 0);
        umma_commit(bars + B_G2);
    }
    __syncwarp();

    // W and U^ back to shared memory (over Awb and its scaled copy: every product that read them is complete)
    mbar_wait(bars + B_G2, 0u, dead, a.status, 602, budget);
    tc_fence_after();
    tmem_ld_n<NC>(x, tlane + T1 + col0);
    pack_n<NC>(x, w);
    store_cols_swz<NC>(smem + S_X + sub * TILE, i, col0 / 8, w);
    tmem_ld_n<NC>(x, tlane + T2 + col0);
    pack_n<NC>(x, w);
    store_cols_swz<NC>(smem + S_X + 2 * TILE + sub * TILE, i, col0 / 8, w);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();

    stage_tick(a, cta, 6);
    // ---- products 6, 7 ------------------------------------------------------------------------------
    if (issuer && !dead) {
        tc_fence_after();
        const uint64_t dKN = umma_desc_mn128(sK + isub * TILE), dWN = umma_desc_mn128(sX + isub * TILE);
        const uint64_t dUN = umma_desc_mn128(sX + 2 * TILE + isub * TILE);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ss(dsub + T1, desc_adv(dKN, kk * 2048), desc_adv(dWN, kk * 2048), ID_NN, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ss(dsub + T2, desc_adv(dUN, kk * 2048), desc_adv(dKN, kk * 2048), ID_NN, kk > 0);
        umma_commit(bars + B_G3);
    }
    __syncwarp();

    // R (product 3 is long complete) -> the two A operands of products 8 and 9
    const float osc = HIER ? 1.f : a.scale;
    // Column tiles (8 wide) of this phase: with 16 warps a thread takes tiles cq and 7 - cq instead of the adjacent pair
    // 2 cq, 2 cq + 1 of the other epilogues, so that the two tiles on the diagonal of a row block (the expensive ones:
    // eight exponentials and level look-ups per row) go to two different warps.
    constexpr int NT = NC / 8;
    int tile_of[NT];
#pragma unroll
    for (int b4 = 0; b4 < NT; ++b4) tile_of[b4] = (NC == 16) ? (b4 == 0 ? cq : 7 - cq) : col0 / 8 + b4;
#pragma unroll
    for (int b4 = 0; b4 < NT; ++b4) tmem_ld8(x + 8 * b4, tlane + T0 + 8 * tile_of[b4]);
    pack_n<NC>(x, w);                                 // R is lower triangular by construction: no mask
#pragma unroll
    for (int b4 = 0; b4 < NT; ++b4) tmem_st4(tlane + TA_R + 4 * tile_of[b4], w + 4 * b4);
    {
        // Pm = R .* E .* lambda[i][level(i, j)], E_ij = e^{G_i - G_j} for j <= i.  level(i, j) = bit_length(i ^ j):
        // off the diagonal 8x8 tile it depends on the tiles only, and there E_ij splits into a factor per (row, tile),
        // e^{G_i - G_end(tile)}, times the column's decay to the end of its tile (both <= 1): one exponential per tile.
        const int ib = i >> 3;
        const float Gi = sG(sub)[i];
        // the row's lambda of the seven levels a chunk can hold (bit_length(i ^ j) <= 6), read once
        float lrow[7];
        if (HIER) {
#pragma unroll
            for (int l = 0; l < 7; ++l) lrow[l] = l < a.L ? lam_at(sub, i, l) : 0.f;
        }
#pragma unroll
        for (int b4 = 0; b4 < NT; ++b4) {
            const int jb = tile_of[b4];
            if (jb > ib) {
#pragma unroll
                for (int e = 0; e < 8; ++e) x[8 * b4 + e] = 0.f;
            } else if (jb < ib) {
                const float4 c0 = *reinterpret_cast<const float4*>(sCF(sub) + 8 * jb);
                const float4 c1 = *reinterpret_cast<const float4*>(sCF(sub) + 8 * jb + 4);
                const float cf[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
                float rowf = __expf(Gi - sG(sub)[8 * jb + 7]);
                if (HIER) { const int d = ib ^ jb; rowf *= d < 2 ? lrow[4] : (d < 4 ? lrow[5] : lrow[6]); }
#pragma unroll
                for (int e = 0; e < 8; ++e) x[8 * b4 + e] *= rowf * cf[e];
            } else {
                const float4 g0 = *reinterpret_cast<const float4*>(sG(sub) + 8 * jb);
                const float4 g1 = *reinterpret_cast<const float4*>(sG(sub) + 8 * jb + 4);
                const float gj[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const int j = 8 * jb + e;
                    const int d = i ^ j;          // < 8 inside the diagonal tile
                    const float lam_ij = HIER ? (d == 0 ? lrow[0] : (d < 2 ? lrow[1] : (d < 4 ? lrow[2] : lrow[3]))) : 1.f;
                    const float f = (j <= i) ? __expf(Gi - gj[e]) * lam_ij : 0.f;
                    x[8 * b4 + e] *= f;
                }
            }
        }
    }
    pack_n<NC>(x, w);
#pragma unroll
    for (int b4 = 0; b4 < NT; ++b4) tmem_st4(tlane + TA_P + 4 * tile_of[b4], w + 4 * b4);

    stage_tick(a, cta, 7);
    // M[a][b] = e^{Gl} (delta_ab - (K^T W)[a][b]) -> record (products 6 and 7 ran while R was converted)
    mbar_wait(bars + B_G3, 0u, dead, a.status, 604, budget);
    tc_fence_after();
    tmem_ld_n<NC>(x, tlane + T1 + col0);
    {
        const float egl = sEG(sub)[CHUNK - 1];
#pragma unroll
        for (int jj = 0; jj < NC; ++jj) x[jj] = egl * ((col0 + jj == i ? 1.f : 0.f) - x[jj]);
        pack_n<NC>(x, w);
        store_cols_swz<NC>(smem + S_X + sub * TILE, i, col0 / 8, w);        // staged over W (product 6 is complete)
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    if (tid < 2 && 2 * pair + tid < H) {   // one bulk store per head
        bulk_s2g(a.rec + ((size_t)c * H + 2 * pair + tid) * a.rec_bytes + R::M_OFF, smem + S_X + tid * TILE, TILE);
        bulk_commit();
    }

    stage_tick(a, cta, 8);
    // ---- products 8, 9: their A operands (R, R .* E .* lambda) are in tensor memory, accumulators T0 and T1 are read out
    if (issuer && !dead) {
        tc_fence_after();
        const uint64_t dKN = umma_desc_mn128(sK + isub * TILE), dVN = umma_desc_mn128(sV + isub * TILE);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ts(dsub + T0, dsub + TA_R + 8 * kk, desc_adv(dKN, kk * 2048), ID_KN, kk > 0);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) umma_f16_ts(dsub + T1, dsub + TA_P + 8 * kk, desc_adv(dVN, kk * 2048), ID_KN, kk > 0);
        umma_commit(bars + B_PV);
    }
    __syncwarp();

    // (while products 8 and 9 run)
    if (HIER) {   // lambda of the chunk levels, transposed to [level][token] for the scan: thread = (token, rows 8 apart)
        const int r = tid & 63;
        for (int row = tid >> 6; row < 2 * a.LC; row += PT / 64) {     // row = head of the pair * LC + level
            const int sb = row >= a.LC ? 1 : 0, l = row - sb * a.LC;
            if (2 * pair + sb < H) {
                float* lamc = reinterpret_cast<float*>(a.rec + ((size_t)c * H + 2 * pair + sb) * a.rec_bytes + R::LAM_OFF);
                lamc[l * CHUNK + r] = (ELL0 + l < a.L && r < len) ? lam_at(sb, r, ELL0 + l) : 0.f;
            }
        }
    }
    // B^T -> record (product 7 completed with product 6)
    tmem_ld_n<NC>(x, tlane + T2 + col0);
    pack_n<NC>(x, w);
    store_cols_swz<NC>(smem + S_X + 2 * TILE + sub * TILE, i, col0 / 8, w);   // staged over U^ (product 7 is complete)

    // Q~ = s e^{G_i} (Q - R K) -> record
    mbar_wait(bars + B_PV, 0u, dead, a.status, 606, budget);
    tc_fence_after();
    tmem_ld_n<NC>(x, tlane + T0 + col0);
    {
        const float f = osc * sEG(sub)[i];
        uint4 rawq[NCH];
        load_cols_swz<NC>(smem + S_Q + sub * TILE, i, col0 / 8, rawq);
#pragma unroll
        for (int q = 0; q < NCH; ++q) {
            const uint32_t uw[4] = {rawq[q].x, rawq[q].y, rawq[q].z, rawq[q].w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 qv = unpack_bf16x2(uw[e]);
                w[4 * q + e] = pack_bf16x2(f * (qv.x - x[8 * q + 2 * e]), f * (qv.y - x[8 * q + 2 * e + 1]));
            }
        }
        store_cols_swz<NC>(smem + S_Q + sub * TILE, i, col0 / 8, w);           // staged in place: each thread overwrites what it read
    }

    // O_local = s Pm V -> record (bf16 [64][64], plain rows)
    tmem_ld_n<NC>(x, tlane + T1 + col0);
    if (!HIER) {
#pragma unroll
        for (int jj = 0; jj < NC; ++jj) x[jj] *= osc;
    }
    pack_n<NC>(x, w);
    store_cols_swz<NC>(smem + S_V + sub * TILE, i, col0 / 8, w);               // staged over V (product 9 is complete)
    fence_async_smem();
    __syncthreads();
    if (tid < 2 && 2 * pair + tid < H) {   // the three remaining tiles of each head leave as bulk stores
        char* rh = a.rec + ((size_t)c * H + 2 * pair + tid) * a.rec_bytes;
        bulk_s2g(rh + R::BT_OFF, smem + S_X + 2 * TILE + tid * TILE, TILE);
        bulk_s2g(rh + R::QT_OFF, smem + S_Q + tid * TILE, TILE);
        bulk_s2g(rh + R::OL_OFF, smem + S_V + tid * TILE, TILE);
        bulk_commit();
        bulk_wait_read();                  // shared memory stays ours until the stores have read it
    }

    stage_tick(a, cta, 9);
    // nothing asynchronous may outlive the CTA: one last commit per issuer covers every product issued above
    if (issuer) {
        umma_commit(bars + B_DRAIN);
        mbar_drain(bars + B_DRAIN, 0u);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(taddr, 256);
    stage_tick(a, cta, 10);
    if (a.ticks != nullptr && threadIdx.x == 0 && cta < a.ticks_ctas) {
        unsigned long long gt_;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));
        a.ticks[(size_t)cta * 16 + 13] = (long long)gt_;
    }
}

}  // namespace

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda)
static PFN_cuTensorMapEncodeTiled tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    }();
    return fn;
}

// [rows][cols] 2-byte tensor, row pitch = cols elements, box of 64 rows x box_cols columns
static bool make_map(CUtensorMap* m, const void* base, int dt, uint64_t rows, uint64_t cols, uint32_t box_cols, bool swizzle) {
    PFN_cuTensorMapEncodeTiled enc = tensor_map_encoder();
    if (!enc) return false;
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * 2};
    const cuuint32_t box[2] = {box_cols, (cuuint32_t)CHUNK};
    const cuuint32_t estr[2] = {1, 1};
    return enc(m, dt == LAMPA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base),
               dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int launch_prep_umma(const GdnArgs& a, bool hier, cudaStream_t st) {
    if (a.qkv_dt == LAMPA_F32) return LAMPA_ERR_UNSUPPORTED;
    const uint64_t tokens = a.fixed_T > 0 ? (uint64_t)a.nseq * a.fixed_T : (uint64_t)a.total_tokens;
    // lambda by TMA when it is a 2-byte type, a token row is a multiple of 16 bytes and the tile is small
    const int lam_tile = hier ? CHUNK * a.H * a.L * 2 : 0;
    const int lam_tma = hier && a.lam_dt != LAMPA_F32 && (a.H * a.L) % 8 == 0 && a.H * a.L <= 256 && lam_tile <= LAM_TMA_MAX;
    const int smem = prep_umma_smem(hier ? a.L : 0, lam_tma ? lam_tile : 0);
    if (smem > 113 * 1024) return LAMPA_ERR_UNSUPPORTED;
    CUtensorMap tq, tk, tv, tl;
    if (!make_map(&tq, a.q, a.qkv_dt, tokens, (uint64_t)a.H * 64, 64, true) ||
        !make_map(&tk, a.k, a.qkv_dt, tokens, (uint64_t)a.H * 64, 64, true) ||
        !make_map(&tv, a.v, a.qkv_dt, tokens, (uint64_t)a.H * 64, 64, true))
        return LAMPA_ERR_UNSUPPORTED;
    tl = tq;
    if (lam_tma && !make_map(&tl, a.lam, a.lam_dt, tokens, (uint64_t)a.H * a.L, (uint32_t)(a.H * a.L), false)) return LAMPA_ERR_UNSUPPORTED;
    dim3 grid((a.H + 1) / 2, a.nc_max);
    ProfScope prof(hier ? "gdn_prep_hier" : "gdn_prep_plain", st);
    static const int nc = [] { const char* e = getenv("LAMPA_B200_PREP_COLS"); return (e && atoi(e) == 32) ? 32 : 16; }();
#define LAMPA_LAUNCH_PREP(HIER_, NC_)                                                                                  \
    do {                                                                                                               \
        if (cudaFuncSetAttribute(gdn_prep_umma_kernel<HIER_, NC_>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) \
            return LAMPA_ERR_CUDA;                                                                                     \
        gdn_prep_umma_kernel<HIER_, NC_><<<grid, 8192 / NC_, smem, st>>>(a, tq, tk, tv, tl, HIER_ ? lam_tma : 0);        \
    } while (0)
    if (hier) { if (nc == 32) LAMPA_LAUNCH_PREP(true, 32); else LAMPA_LAUNCH_PREP(true, 16); }
    else { if (nc == 32) LAMPA_LAUNCH_PREP(false, 32); else LAMPA_LAUNCH_PREP(false, 16); }
#undef LAMPA_LAUNCH_PREP
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

}  // namespace lampa
