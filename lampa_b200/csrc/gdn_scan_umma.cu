// Hierarchical output pass on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM)
// for K = V = 64.
//
// Per (block of 32 chunks, head) one CTA of 4 warps keeps every level state the block touches as
// rows of bf16 A operands in shared memory: slot s holds S_l^T (64 rows v x 64 columns k), two slots
// per 128-row operand ("pair").  Slots 0..4 are the chunk levels that live inside the block,
// the following ones the cross-block levels this block reads (seeded from the level pass).
// A chunk is one record {M | Q~ | B^T | O_local | lambda}; its first 16 KB, the M and Q~ tiles back to
// back, are a single 128-row K-major B operand, so ONE accumulating MMA per pair,
//     D[128 x 128] = [S_a^T ; S_b^T] (128 x 64)  x  [M ; Q~]^T (64 x 128),
// yields both the advanced states (columns 0..63: S^T M^T) and the levels' contributions to the
// output (columns 64..127: S^T Q~^T = (Q~ S)^T).  The epilogue, one thread per TMEM lane (= state
// row), scales the contribution by lambda and accumulates it over the pairs, adds B^T where the
// level is collecting, clears it at the end of its period, and writes the bf16 row back into the A
// operand for the next chunk.  Warp-specialised: 16 epilogue warps (two warpgroups advance the states,
// 32 columns each; two read them and also transpose and store the output) and one control warp whose
// first lane streams the records in (bulk async copies, three stages) and issues the MMAs.  A pair's
// MMA for the next chunk is issued as soon as that pair's epilogue has handed its operand back
// (mbarriers only, no block-wide barrier on the state path), so the tensor core runs ahead of the
// epilogues.  MMA completion is tracked by tcgen05.commit on one mbarrier per pair; every wait is bounded.
#include "gdn.cuh"
#include "profile.cuh"

namespace lampa {

namespace {

constexpr int UKD = 64, UVD = 64;
constexpr int UNP = 5;                       // pairs of slots: 5 in-block levels + up to 5 cross-block levels
constexpr int UEPI_WARPS = 16;               // 4 warpgroups: two advance the states (32 columns each), two read them
constexpr int UTHREADS = (UEPI_WARPS + 1) * 32;   // plus one control warp
constexpr int UNST = 3;                      // record stages
using UR = Rec<UKD, UVD>;

// shared-memory map (bytes); everything that tcgen05 reads is 1024-byte aligned
constexpr int SM_BAR = 0;                    // full[UNST], mma[UNP] mbarriers, TMEM slot
constexpr int SM_OT = 1024;                  // fp32 [2][64 tokens][64 v]: output transpose / pair-half sum
// TMEM columns (512 allocated): the states as bf16 A operands, 32 columns per pair, then two
// 128-column accumulator buffers used by the pairs in turn
constexpr int TM_A = 0;
constexpr int TM_D = 192;
constexpr int SM_STAGE = SM_OT + 2 * 64 * 64 * 4;
constexpr int STAGE_TILES = UR::LAM_OFF;     // M | Q~ | B^T | O_local, then the lambda rows: the whole record
__host__ __device__ constexpr int ustage_bytes(int LC) { return (STAGE_TILES + LC * CHUNK * 4 + 1023) / 1024 * 1024; }

__device__ __forceinline__ uint64_t umma_desc_k128(uint32_t saddr) {   // K-major, 128B swizzle, 8-row groups 1024 B apart
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                 // leading byte offset (ignored for swizzled K-major): 16 B
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset
    d |= (uint64_t)1 << 46;                 // descriptor version
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = 128
constexpr uint32_t UMMA_IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 :: "r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// same with the A operand in TMEM (lane = row, packed bf16 pairs, 8 columns per k-step of 16)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
                 :: "r"(d_tmem), "r"(a_tmem), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(float (&x)[32], uint32_t taddr) {
    uint32_t* r = reinterpret_cast<uint32_t*>(x);
#define LAMPA_LD16(o)                                                                                                     \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n" \
                 : "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]),          \
                   "=r"(r[o + 6]), "=r"(r[o + 7]), "=r"(r[o + 8]), "=r"(r[o + 9]), "=r"(r[o + 10]), "=r"(r[o + 11]),       \
                   "=r"(r[o + 12]), "=r"(r[o + 13]), "=r"(r[o + 14]), "=r"(r[o + 15])                                     \
                 : "r"(taddr + o));
    LAMPA_LD16(0) LAMPA_LD16(16)
#undef LAMPA_LD16
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

// write 32 floats as 16 columns of packed bf16 pairs of this thread's TMEM lane (half a row of an A operand)
__device__ __forceinline__ void tmem_st_bf16x32(uint32_t taddr, const float (&x)[32]) {
    uint32_t w[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) w[c] = pack_bf16x2(x[2 * c], x[2 * c + 1]);
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};\n"
                 :: "r"(taddr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]),
                    "r"(w[8]), "r"(w[9]), "r"(w[10]), "r"(w[11]), "r"(w[12]), "r"(w[13]), "r"(w[14]), "r"(w[15]) : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" :: "r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(UTHREADS, 1) gdn_out_hier_umma_kernel(GdnArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM_BAR);      // record landed            (tx count)
    uint64_t* sfree = full + UNST;                                      // stage consumed           (16 warps)
    uint64_t* mdone = sfree + UNST;                                     // pair's MMA complete      (commit)
    uint64_t* aready = mdone + UNP;                                     // pair's operand rewritten (16 warps)
    uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 256);
    float* sOT = reinterpret_cast<float*>(smem + SM_OT);

    const int gb = blockIdx.x, h = blockIdx.y, H = a.H;
    if (gb >= a.block_off[a.nseq]) return;
    const int seq = find_seq(a.block_off, a.nseq, gb);
    const int b = gb - a.block_off[seq];
    const int nch = a.chunk_off[seq + 1] - a.chunk_off[seq];
    const int nlev = nch > 1 ? ceil_log2_int(nch) : 0;
    const int nhigh = max(0, nlev - BLOCK_LOG);
    const int c0 = a.chunk_off[seq] + b * BLOCK_CHUNKS;
    const int nsteps = min(BLOCK_CHUNKS, nch - b * BLOCK_CHUNKS);
    const int64_t tok0 = a.tok_off[seq] + (int64_t)b * BLOCK_CHUNKS * CHUNK, tok_end = a.tok_off[seq + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wg = warp >> 2;                          // 0,1: advance columns 32*wg..; 2,3: read tokens 32*(wg-2)..; 4: control
    const int row = (warp & 3) * 32 + lane;            // TMEM lane = row of the pair's A operand
    const int u = row >> 6, v = row & 63;              // which slot of the pair, which state row
    const int half = wg & 1;
    const int lam_bytes = a.LC * CHUNK * 4;
    const int stage_bytes = ustage_bytes(a.LC);
    unsigned char* stage0 = smem + SM_STAGE;
    const char* rec0 = a.rec + ((size_t)c0 * H + h) * a.rec_bytes;
    const size_t rec_stride = (size_t)H * a.rec_bytes;

    // cross-block levels this block reads, compacted into slots 5, 6, ...
    int nlive = 0;
    uint32_t live_pack = 0;                            // 4 bits per compact slot: the level index
    for (int lh = 0; lh < nhigh; ++lh)
        if ((b >> lh) & 1) { live_pack |= (uint32_t)lh << (4 * nlive); ++nlive; }
    const int nslots = BLOCK_LOG + nlive;
    const int npairs = (nslots + 1) >> 1;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < UNST; ++s) { mbar_init(full + s, 1); mbar_init(sfree + s, UEPI_WARPS); }
#pragma unroll
        for (int p = 0; p < UNP; ++p) { mbar_init(mdone + p, 1); mbar_init(aready + p, UEPI_WARPS); }
        fence_mbar_init();
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" :: "r"(smem_u32(tslot)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t taddr = *tslot;
    const uint32_t tlane = taddr + ((uint32_t)((warp & 3) * 32) << 16);
    // initial states: zero for the in-block levels, the block's entry state for the cross-block ones
    if (wg < 2) {
        for (int p = 0; p < npairs; ++p) {
            const int s = 2 * p + u;
            float x[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) x[i] = 0.f;
            if (s >= BLOCK_LOG && s < nslots) {
                const int lh = (live_pack >> (4 * (s - BLOCK_LOG))) & 15;
                const float4* e = reinterpret_cast<const float4*>(
                    a.entry + (((size_t)gb * a.nhigh_max + lh) * H + h) * UR::STATE_FLOATS + (size_t)v * UKD + 32 * half);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float4 f = e[i];
                    x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
                }
            }
            tmem_st_bf16x32(tlane + TM_A + 32 * p + 16 * half, x);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    bool dead = false;

    if (wg == 4) {
        // ---- control warp: one lane streams records and issues MMAs --------------------------------
        if (lane == 0) {
            auto load_record = [&](int step) {
                uint64_t* fb = full + (step % UNST);
                unsigned char* dst = stage0 + (size_t)(step % UNST) * stage_bytes;
                const char* src = rec0 + (size_t)step * rec_stride;
                mbar_expect_tx(fb, (uint32_t)(STAGE_TILES + lam_bytes));
                bulk_g2s(dst, src, (uint32_t)(STAGE_TILES + lam_bytes), fb);
            };
            for (int s = 0; s < UNST - 1 && s < nsteps; ++s) load_record(s);
            for (int i = 0; i < nsteps; ++i) {
                const unsigned char* st = stage0 + (size_t)(i % UNST) * stage_bytes;
                mbar_wait(full + (i % UNST), (uint32_t)((i / UNST) & 1), dead, a.status, 200 + i);
                for (int p = 0; p < npairs; ++p) {
                    // the pair's operand rewritten by the previous chunk ...
                    if (i > 0) mbar_wait(aready + p, (uint32_t)((i - 1) & 1), dead, a.status, 400 + p);
                    // ... and the accumulator buffer (p & 1) drained by the pair that used it last
                    if (p >= 2) {
                        mbar_wait(aready + (p - 2), (uint32_t)(i & 1), dead, a.status, 410 + p);
                    } else if (i > 0) {
                        const int q = ((npairs - 1) & 1) == p ? npairs - 1 : npairs - 2;
                        if (q > p) mbar_wait(aready + q, (uint32_t)((i - 1) & 1), dead, a.status, 420 + p);
                    }
                    tc_fence_after();
                    const uint32_t b_base = smem_u32(st + UR::M_OFF);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_f16_ts(taddr + (uint32_t)(TM_D + (p & 1) * 128), taddr + (uint32_t)(TM_A + 32 * p + 8 * kk),
                                    umma_desc_k128(b_base + kk * 32), UMMA_IDESC, kk > 0 ? 1u : 0u);
                    umma_commit(mdone + p);
                }
                if (i + UNST - 1 < nsteps) {       // refill the stage chunk i-1 used, once everyone is done with it
                    if (i >= 1) mbar_wait(sfree + ((i - 1) % UNST), (uint32_t)(((i - 1) / UNST) & 1), dead, a.status, 500 + i);
                    load_record(i + UNST - 1);
                }
            }
        }
    } else {
        // ---- epilogue warps ---------------------------------------------------------------------------
        for (int i = 0; i < nsteps; ++i) {
            const unsigned char* st = stage0 + (size_t)(i % UNST) * stage_bytes;
            const float* sLam = reinterpret_cast<const float*>(st + STAGE_TILES);
            const unsigned char* sBt = st + UR::BT_OFF;
            const int n = b * BLOCK_CHUNKS + i;
            const int otid = tid - 256;                       // output thread index of the read warpgroups
            const int64_t t_out = tok0 + (int64_t)i * CHUNK + (otid >> 2);
            const float* sOl = reinterpret_cast<const float*>(st + UR::OL_OFF);
            mbar_wait(full + (i % UNST), (uint32_t)((i / UNST) & 1), dead, a.status, 250 + i);

            float oacc[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) oacc[j] = 0.f;

            for (int p = 0; p < npairs; ++p) {
                mbar_wait(mdone + p, (uint32_t)(i & 1), dead, a.status, 300 + p);
                tc_fence_after();
                const int s = 2 * p + u;
                const bool active = s < nslots;
                bool do_read = false, clear = false, add_b = false;
                int lam_row = 0;
                if (s < BLOCK_LOG) {
                    const int per = 2 << s, pos = n & (per - 1), bit = (n >> s) & 1;
                    do_read = bit != 0;
                    clear = pos == per - 1;
                    add_b = bit == 0;
                    lam_row = s;
                } else if (active) {
                    do_read = true;
                    lam_row = BLOCK_LOG + ((live_pack >> (4 * (s - BLOCK_LOG))) & 15);
                }
                if (lam_row >= a.LC) do_read = false;      // only reachable when the level check already failed
                const uint32_t tcol = tlane + (uint32_t)(TM_D + (p & 1) * 128);
                if (wg >= 2) {
                    if (do_read) {
                        float y[32];
                        tmem_ld32(y, tcol + 64 + 32 * half);
                        const float4* lr = reinterpret_cast<const float4*>(sLam + lam_row * CHUNK + 32 * half);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 l4 = lr[j];
                            oacc[4 * j] += l4.x * y[4 * j]; oacc[4 * j + 1] += l4.y * y[4 * j + 1];
                            oacc[4 * j + 2] += l4.z * y[4 * j + 2]; oacc[4 * j + 3] += l4.w * y[4 * j + 3];
                        }
                    }
                } else if (active && i + 1 < nsteps) {
                    float x[32];
                    if (clear) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) x[j] = 0.f;
                    } else {
                        tmem_ld32(x, tcol + 32 * half);
                        if (add_b) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const uint4 q4 = *reinterpret_cast<const uint4*>(sBt + v * 128 + (((4 * half + c) ^ (v & 7)) << 4));
                                const float2 f0 = unpack_bf16x2(q4.x), f1 = unpack_bf16x2(q4.y), f2 = unpack_bf16x2(q4.z), f3 = unpack_bf16x2(q4.w);
                                x[8 * c] += f0.x; x[8 * c + 1] += f0.y; x[8 * c + 2] += f1.x; x[8 * c + 3] += f1.y;
                                x[8 * c + 4] += f2.x; x[8 * c + 5] += f2.y; x[8 * c + 6] += f3.x; x[8 * c + 7] += f3.y;
                            }
                        }
                    }
                    tmem_st_bf16x32(tlane + TM_A + 32 * p + 16 * half, x);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(aready + p);
            }
            if (wg < 2) {
                __syncwarp();
                if (lane == 0) mbar_arrive(sfree + (i % UNST));
            }
            if (wg >= 2) {
                // output (read warpgroups only): sum the two halves of the pairs, add O_local, transpose
                asm volatile("bar.sync 1, 256;\n" ::: "memory");       // previous chunk's transpose buffer fully read
#pragma unroll
                for (int j = 0; j < 32; ++j) sOT[(u * 64 + 32 * half + j) * 64 + v] = oacc[j];
                asm volatile("bar.sync 1, 256;\n" ::: "memory");
                if (t_out < tok_end) {
                    const int tok = otid >> 2, col = (otid & 3) * 16;
                    const size_t idx = ((size_t)t_out * H + h) * UVD + col;
                    float r[16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 p0 = *reinterpret_cast<const float4*>(sOT + (0 * 64 + tok) * 64 + col + 4 * q);
                        const float4 q0 = *reinterpret_cast<const float4*>(sOT + (1 * 64 + tok) * 64 + col + 4 * q);
                        r[4 * q] = p0.x + q0.x; r[4 * q + 1] = p0.y + q0.y; r[4 * q + 2] = p0.z + q0.z; r[4 * q + 3] = p0.w + q0.w;
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 o4 = *reinterpret_cast<const float4*>(sOl + tok * UR::OP + col + 4 * q);
                        r[4 * q] += o4.x; r[4 * q + 1] += o4.y; r[4 * q + 2] += o4.z; r[4 * q + 3] += o4.w;
                    }
                    if (a.qkv_dt == LAMPA_F32) {
                        float4* o4 = reinterpret_cast<float4*>((float*)a.o + idx);
#pragma unroll
                        for (int q = 0; q < 4; ++q) o4[q] = make_float4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                    } else {
                        uint32_t w[8];
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            if (a.qkv_dt == LAMPA_BF16) w[q] = pack_bf16x2(r[2 * q], r[2 * q + 1]);
                            else { const __half2 hh = __floats2half2_rn(r[2 * q], r[2 * q + 1]); w[q] = *reinterpret_cast<const uint32_t*>(&hh); }
                        }
                        uint4* o4 = reinterpret_cast<uint4*>((uint16_t*)a.o + idx);
                        o4[0] = make_uint4(w[0], w[1], w[2], w[3]);
                        o4[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(sfree + (i % UNST));   // O_local of this stage has been read
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" :: "r"(taddr), "r"(512) : "memory");
}

}  // namespace

int launch_out_hier_umma(const GdnArgs& a, cudaStream_t st) {
    const int smem = SM_STAGE + UNST * ustage_bytes(a.LC);
    if (smem > 227 * 1024 || a.nhigh_max > UNP) return LAMPA_ERR_UNSUPPORTED;
    if (cudaFuncSetAttribute(gdn_out_hier_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return LAMPA_ERR_CUDA;
    ProfScope prof("gdn_out_hier_umma", st);
    gdn_out_hier_umma_kernel<<<dim3(a.nb_max, a.H), UTHREADS, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

}  // namespace lampa
