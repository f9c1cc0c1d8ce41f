// Output passes on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM) for K = V = 64:
// the hierarchical rule first, the plain rule (one state per head) at the end of the file.
//
// Per (block of 32 chunks, head) one CTA keeps every level state the block touches as rows of
// bf16 A operands in tensor memory: slot s holds S_l^T (64 rows v x 64 columns k), two slots
// per 128-row operand ("pair").  Slots 0..4 are the chunk levels that live inside the block,
// the following ones the cross-block levels this block reads (seeded from the level pass).
// A chunk is one record {M | Q~ | B^T | O_local | lambda}; its first 16 KB, the M and Q~ tiles back to
// back, are a single 128-row K-major B operand, so ONE accumulating MMA per pair,
//     D[128 x 128] = [S_a^T ; S_b^T] (128 x 64)  x  [M ; Q~]^T (64 x 128),
// yields both the advanced states (columns 0..63: S^T M^T) and the levels' contributions to the
// output (columns 64..127: S^T Q~^T = (Q~ S)^T).  The epilogue, one thread per TMEM lane (= state
// row) and quarter of the columns, adds B^T where the level is collecting, clears it at the end of
// its period and writes the bf16 row back into the A operand for the next chunk; then it scales
// the level's contribution to its 16 tokens by lambda and accumulates it over the pairs.
// Warp-specialised: 16 epilogue warps (warp = 32 rows x 16 state columns x 16 tokens; together they
// also transpose the chunk's output through shared memory and store it with O_local added) and one
// control warp whose first lane streams the records in (bulk async copies, three stages) and issues
// the MMAs.  The MMAs take the accumulator buffers in turn; one is issued as soon as every epilogue warp has
// handed back the buffer it overwrites, which it does after rewriting the pair's operand and reading the
// pair's contribution (a hardware named barrier per pair that the control warp joins: no block-wide barrier
// and no polling on the state path).  MMA completion is tracked by tcgen05.commit on one mbarrier per
// pair; every mbarrier wait is bounded, and a CTA whose wait ran out stops issuing copies and MMAs, lets
// every warp walk through its remaining barriers in lockstep, waits for the copies and MMAs in flight
// and only then frees its tensor memory.
#include "gdn.cuh"
#include "profile.cuh"
#include "umma.cuh"

namespace lampa {

namespace {

constexpr int UKD = 64, UVD = 64;
constexpr int UNP = 5;                       // pairs of slots: 5 in-block levels + up to 5 cross-block levels
constexpr int UEPI_WARPS = 16;               // 4 warpgroups, each covering 16 state columns and 16 tokens of all 128 rows
constexpr int UTHREADS = (UEPI_WARPS + 2) * 32;   // plus one control warp and one relay warp
// An mbarrier poll costs the polling warp 200 - 300 cycles even when the phase is long complete, a hardware named
// barrier that everybody else has already reached about 30.  So only the relay warp polls the mbarriers the epilogue
// depends on ("record landed", "pair's MMA complete") and passes each completion on through a named barrier that the
// sixteen epilogue warps join (ids 5 + p; ids 1..4 belong to the output transpose), and the epilogue hands a pair's
// accumulator back to the control warp the same way (ids 11 + p: sixteen warps arrive, the control warp waits).
// Nobody can be left waiting at a named barrier: the relay's and the control lane's own waits are bounded and both
// walk through every barrier whether or not a wait ran out, and the epilogue never waits for anything else.  Nobody
// can reach a barrier twice in one phase either: a pair's next MMA is issued only after its hand-back was joined, and
// once a wait has run out (flag in shared memory) relay and epilogue join their barriers synchronously instead of
// arriving and running on.  (The plain-rule kernel below has one MMA group per chunk and hands its operands back
// through an mbarrier: there the named barrier measured slower; its records alternate between ids 10 and 11.)
constexpr int UNB_PAIR = 5, UNB_REC = 10, UNB_DFREE = 11, UNB_COUNT = (UEPI_WARPS + 1) * 32;
__device__ __forceinline__ void named_arrive(int id) { asm volatile("bar.arrive %0, %1;\n" :: "r"(id), "n"(UNB_COUNT) : "memory"); }
__device__ __forceinline__ void named_sync(int id) { asm volatile("bar.sync %0, %1;\n" :: "r"(id), "n"(UNB_COUNT) : "memory"); }
__device__ __forceinline__ void relay_pass(int id, bool dead) { if (dead) named_sync(id); else named_arrive(id); }
constexpr int UNST = 3;                      // record stages
using UR = Rec<UKD, UVD>;

// shared-memory map (bytes); everything that tcgen05 reads is 1024-byte aligned
constexpr int SM_BAR = 0;                    // full[UNST], mma[UNP] mbarriers, TMEM slot
constexpr int SM_OT = 1024;                  // two buffers (chunk parity) of fp32 [2][64 tokens][64 v]: output transpose / pair-half sum
// TMEM columns (512 allocated): the states as bf16 A operands, 32 columns per pair, then the
// 128-column accumulator buffers used by the MMAs in turn (three from column 128 when there are at
// most four pairs, else two from column 192)
constexpr int TM_A = 0;
constexpr int TM_D = 192;
constexpr int SM_STAGE = SM_OT + 2 * 2 * 64 * 64 * 4;
constexpr int STAGE_TILES = UR::LAM_OFF;     // M | Q~ | B^T | O_local, then the lambda rows: the whole record
__host__ __device__ constexpr int ustage_bytes(int LC) { return (STAGE_TILES + LC * CHUNK * 4 + 1023) / 1024 * 1024; }

// instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = 128
constexpr uint32_t UMMA_IDESC = umma_idesc(128, 128);

// Launch order of the (block, head) units.  A unit's time grows with the number of level pairs it
// carries (3 to 5, from the set bits of its block index), and 240 units on 148 SMs leave the second
// round partly empty: handing the long units out first lets the short ones fill the tail.
struct UnitOrder {
    int nbs;                    // blocks per sequence when all sequences are equally long and nbs <= 64, else 0
    unsigned char order[64];    // block indices, most level pairs first
};

__global__ void __launch_bounds__(UTHREADS, 1) gdn_out_hier_umma_kernel(GdnArgs a, UnitOrder uo) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM_BAR);      // record landed            (tx count)
    uint64_t* sfree = full + UNST;                                      // stage consumed           (16 warps)
    uint64_t* mdone = sfree + UNST;                                     // pair's MMA complete      (commit)
    uint64_t* drainb = mdone + UNP;                                     // every MMA issued has completed (commit at the end)
    uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 256);
    volatile uint32_t* sdead = reinterpret_cast<volatile uint32_t*>(smem + SM_BAR + 260);   // set once a bounded wait has run out
    float* sOT = reinterpret_cast<float*>(smem + SM_OT);

    const int H = a.H;
    int gb, h;
    if (uo.nbs > 0) {
        const int per_rank = H * a.nseq, r = blockIdx.x / per_rank, rem = blockIdx.x - r * per_rank;
        h = rem % H;
        gb = (rem / H) * uo.nbs + uo.order[r];
    } else {
        gb = blockIdx.x % a.nb_max;
        h = blockIdx.x / a.nb_max;
    }
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
    const int wg = warp >> 2;                          // 0..3: state columns / tokens 16*wg .. 16*wg+15; 4: control
    const int row = (warp & 3) * 32 + lane;            // TMEM lane = row of the pair's A operand
    const int u = row >> 6, v = row & 63;              // which slot of the pair, which state row
    const int part = wg & 3;
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
    // accumulator buffers of 128 columns behind the operands: three where four pairs or fewer leave room for them
    const int nbuf = npairs <= 4 ? 3 : 2, tm_d = npairs <= 4 ? 128 : TM_D;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < UNST; ++s) { mbar_init(full + s, 1); mbar_init(sfree + s, UEPI_WARPS); }
#pragma unroll
        for (int p = 0; p < UNP; ++p) mbar_init(mdone + p, 1);
        mbar_init(drainb, 1);
        *sdead = 0u;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(tslot, 512);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t taddr = *tslot;
    const uint32_t tlane = taddr + ((uint32_t)((warp & 3) * 32) << 16);
    // initial states: zero for the in-block levels, the block's entry state for the cross-block ones
    if (wg < 4) {
        for (int p = 0; p < npairs; ++p) {
            const int s = 2 * p + u;
            float x[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) x[i] = 0.f;
            if (s >= BLOCK_LOG && s < nslots) {
                const int lh = (live_pack >> (4 * (s - BLOCK_LOG))) & 15;
                const float4* e = reinterpret_cast<const float4*>(
                    a.entry + (((size_t)gb * a.nhigh_max + lh) * H + h) * UR::STATE_FLOATS + (size_t)v * UKD + 16 * part);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float4 f = e[i];
                    x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
                }
            }
            tmem_st_bf16x16(tlane + TM_A + 32 * p + 8 * part, x);
        }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    bool dead = false;
    const int budget = a.poll_budget;

    if (warp == UEPI_WARPS) {
        // ---- control warp: lane 0 streams records and issues MMAs; the whole warp joins the named barriers ----
        int loaded = 0, landed = 0;                  // records requested / records seen in shared memory (lane 0)
        auto load_record = [&](int step) {
            uint64_t* fb = full + (step % UNST);
            unsigned char* dst = stage0 + (size_t)(step % UNST) * stage_bytes;
            const char* src = rec0 + (size_t)step * rec_stride;
            mbar_expect_tx(fb, (uint32_t)(STAGE_TILES + lam_bytes));
            bulk_g2s(dst, src, (uint32_t)(STAGE_TILES + lam_bytes), fb);
            loaded = step + 1;
        };
        if (lane == 0)
            for (int s = 0; s < UNST - 1 && s < nsteps; ++s) load_record(s);
        // The MMAs are numbered through the chunks, m = i * npairs + p, and take the accumulator buffers in turn:
        // MMA m overwrites the buffer MMA m - nbuf filled, once the epilogue has handed that one back.  The epilogue hands
        // a pair's accumulator back after it has rewritten the pair's operand, and it works through chunks and pairs in
        // order, so the same hand-back also covers the operand of pair p rewritten in the previous chunk (npairs >= nbuf).
        // Every hand-back is joined exactly once and in the order it is given, whether or not anything is still issued.
        int bufi = 0;
        for (int i = 0; i < nsteps; ++i) {
            const unsigned char* st = stage0 + (size_t)(i % UNST) * stage_bytes;
            if (lane == 0 && !dead && mbar_wait(full + (i % UNST), (uint32_t)((i / UNST) & 1), dead, a.status, 200 + i, budget)) landed = i + 1;
            for (int p = 0; p < npairs; ++p) {
                __syncwarp();
                if (p >= nbuf) named_sync(UNB_DFREE + p - nbuf);
                else if (i > 0) named_sync(UNB_DFREE + npairs - nbuf + p);
                const uint32_t dcol = (uint32_t)(tm_d + bufi * 128);
                bufi = bufi + 1 == nbuf ? 0 : bufi + 1;
                if (lane == 0 && !dead) {
                    tc_fence_after();
                    const uint32_t b_base = smem_u32(st + UR::M_OFF);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        umma_f16_ts(taddr + dcol, taddr + (uint32_t)(TM_A + 32 * p + 8 * kk),
                                    umma_desc_k128(b_base + kk * 32), UMMA_IDESC, kk > 0 ? 1u : 0u);
                    umma_commit(mdone + p);
                }
            }
            if (lane == 0 && !dead && i + UNST - 1 < nsteps) {       // refill the stage chunk i-1 used, once everyone is done with it
                if (i >= 1) mbar_wait(sfree + ((i - 1) % UNST), (uint32_t)(((i - 1) / UNST) & 1), dead, a.status, 500 + i, budget);
                if (!dead) load_record(i + UNST - 1);
            }
            if (lane == 0 && dead) *sdead = 1u;
        }
        __syncwarp();
        for (int p = npairs - nbuf; p < npairs; ++p) named_sync(UNB_DFREE + p);      // the last chunk's outstanding hand-backs
        if (lane == 0) {
            // nothing asynchronous may outlive the CTA: records still on their way land first, and one
            // last commit covers every MMA issued above
            for (int s = landed; s < loaded; ++s) mbar_drain(full + (s % UNST), (uint32_t)((s / UNST) & 1));
            umma_commit(drainb);
            mbar_drain(drainb, 0u);
        }
    } else if (wg == 4) {
        // ---- relay warp (the second warp of this group): mbarrier completions -> named barriers ----
        // "record landed" travels with the first pair of the chunk.  A pair's barrier cannot be reached a second time
        // before every epilogue warp has left it: the pair's next MMA is only issued after its accumulator came back.
        for (int i = 0; i < nsteps; ++i) {
            mbar_wait(full + (i % UNST), (uint32_t)((i / UNST) & 1), dead, a.status, 250 + i, budget);
            for (int p = 0; p < npairs; ++p) {
                mbar_wait(mdone + p, (uint32_t)(i & 1), dead, a.status, 300 + p, budget);
                if (dead) *sdead = 1u;
                relay_pass(UNB_PAIR + p, dead);
            }
        }
    } else {
        // ---- epilogue warps: every warp advances 16 state columns and reads 16 tokens of its 32 rows ----
        // per pair, the lambda row of this thread's slot, and the slots that exist and have a lambda row
        uint32_t lam_pack = 0, slot_ok = 0;          // 5 bits per pair: the lambda row of slot 2p + u
#pragma unroll
        for (int p = 0; p < UNP; ++p) {
            const int s = 2 * p + u;
            const int row = s < BLOCK_LOG ? s : BLOCK_LOG + (int)((live_pack >> (4 * max(s - BLOCK_LOG, 0))) & 15);
            lam_pack |= (uint32_t)(row & 31) << (5 * p);
        }
        for (int s = 0; s < nslots; ++s) {
            const int row = s < BLOCK_LOG ? s : BLOCK_LOG + (int)((live_pack >> (4 * (s - BLOCK_LOG))) & 15);
            if (row < a.LC) slot_ok |= 1u << s;      // a missing row is only reachable when the level check already failed
        }
        int bufi = 0;                                // accumulator buffer of the next pair, in step with the control warp
        for (int i = 0; i < nsteps; ++i) {
            const unsigned char* st = stage0 + (size_t)(i % UNST) * stage_bytes;
            const float* sLam = reinterpret_cast<const float*>(st + STAGE_TILES);
            const unsigned char* sBt = st + UR::BT_OFF;
            const int n = b * BLOCK_CHUNKS + i;
            const __nv_bfloat16* sOl = reinterpret_cast<const __nv_bfloat16*>(st + UR::OL_OFF);
            // what this chunk does to each slot, as bit masks: in-block level s is read when bit s of n is
            // set and cleared when its period of 2^(s+1) chunks ends (all of bits 0..s set); the cross-block
            // slots are read by every chunk
            const uint32_t low = (uint32_t)n & (BLOCK_CHUNKS - 1);
            const uint32_t read_mask = (low | (~0u << BLOCK_LOG)) & slot_ok;
            const uint32_t clear_mask = low & ~(low + 1u) & (BLOCK_CHUNKS - 1);      // trailing ones of n
            uint4 bq0, bq1;                            // this row's 16 columns of B^T, shared by every level that collects in this chunk

            float oacc[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) oacc[j] = 0.f;

            for (int p = 0; p < npairs; ++p) {
                named_sync(UNB_PAIR + p);              // pair's MMA complete
                tc_fence_after();
                const uint32_t lockstep = *sdead;      // non-zero: a wait ran out somewhere, nobody runs ahead of anybody from here on
                if (p == 0) {                          // the record has landed too
                    bq0 = *reinterpret_cast<const uint4*>(sBt + v * 128 + (((2 * part) ^ (v & 7)) << 4));
                    bq1 = *reinterpret_cast<const uint4*>(sBt + v * 128 + (((2 * part + 1) ^ (v & 7)) << 4));
                }
                const int s = 2 * p + u;
                const bool active = s < nslots;
                const bool do_read = (read_mask >> s) & 1u, clear = (clear_mask >> s) & 1u, add_b = !((n >> s) & 1) && s < BLOCK_LOG;
                const int lam_row = (int)((lam_pack >> (5 * p)) & 31u);
                const uint32_t tcol = tlane + (uint32_t)(tm_d + bufi * 128);
                bufi = bufi + 1 == nbuf ? 0 : bufi + 1;
                // state path first: the next chunk's MMA of this pair waits for it
                if (active && i + 1 < nsteps) {
                    float x[16];
                    if (clear) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) x[j] = 0.f;
                    } else {
                        tmem_ld16(x, tcol + 16 * part);
                        if (add_b) {
                            const uint32_t bw[8] = {bq0.x, bq0.y, bq0.z, bq0.w, bq1.x, bq1.y, bq1.z, bq1.w};
#pragma unroll
                            for (int c = 0; c < 8; ++c) {
                                const float2 f = unpack_bf16x2(bw[c]);
                                x[2 * c] += f.x; x[2 * c + 1] += f.y;
                            }
                        }
                    }
                    tmem_st_bf16x16(tlane + TM_A + 32 * p + 8 * part, x);
                }
                // read path: lambda-weighted contribution of this level to 16 tokens
                if (do_read) {
                    float y[16];
                    tmem_ld16(y, tcol + 64 + 16 * part);
                    const float4* lr = reinterpret_cast<const float4*>(sLam + lam_row * CHUNK + 16 * part);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float4 l4 = lr[j];
                        oacc[4 * j] += l4.x * y[4 * j]; oacc[4 * j + 1] += l4.y * y[4 * j + 1];
                        oacc[4 * j + 2] += l4.z * y[4 * j + 2]; oacc[4 * j + 3] += l4.w * y[4 * j + 3];
                    }
                }
                tc_fence_before();
                // operand rewritten, accumulator read: the control warp may go on
                if (lockstep) named_sync(UNB_DFREE + p); else named_arrive(UNB_DFREE + p);
            }
            // output: sum the two rows (levels) of the pairs through shared memory, add O_local, store.
            // Tokens 16 wg .. 16 wg + 15 of the tile are written and read by warpgroup wg alone, so the barrier is the
            // warpgroup's own.  The buffer alternates with the chunk: a warp that runs ahead writes the other buffer, and
            // it cannot get two chunks ahead of a warp of its group that is still reading without passing that barrier.
            float* sOTc = sOT + (i & 1) * (2 * 64 * 64);
#pragma unroll
            for (int j = 0; j < 16; ++j) sOTc[(u * 64 + 16 * part + j) * 64 + v] = oacc[j];
            switch (wg) {
                case 0: asm volatile("bar.sync 1, 128;\n" ::: "memory"); break;
                case 1: asm volatile("bar.sync 2, 128;\n" ::: "memory"); break;
                case 2: asm volatile("bar.sync 3, 128;\n" ::: "memory"); break;
                default: asm volatile("bar.sync 4, 128;\n" ::: "memory"); break;
            }
            auto emit = [&](auto scat) {
                // thread = (token, 4 + 4 output columns: 4c.. and 32 + 4c..): the eight lanes of a token read 128
                // contiguous bytes of the tile per load, which is what keeps the 16-byte loads free of bank conflicts
                const int tok = tid >> 3, col = (tid & 7) * 4;
                const int64_t t_out = tok0 + (int64_t)i * CHUNK + tok;
                const int64_t orow = t_out < tok_end ? out_row<decltype(scat)::value>(a, t_out) : -1;
                if (orow >= 0) {
                    const size_t idx = ((size_t)orow * H + h) * UVD + col;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const float4 p0 = *reinterpret_cast<const float4*>(sOTc + (0 * 64 + tok) * 64 + col + 32 * q);
                        const float4 q0 = *reinterpret_cast<const float4*>(sOTc + (1 * 64 + tok) * 64 + col + 32 * q);
                        const uint2 ol = *reinterpret_cast<const uint2*>(sOl + UR::TV::off(tok, col + 32 * q));      // 4 bf16 of O_local
                        const float2 oa = unpack_bf16x2(ol.x), ob = unpack_bf16x2(ol.y);
                        const float r0 = p0.x + q0.x + oa.x, r1 = p0.y + q0.y + oa.y, r2 = p0.z + q0.z + ob.x, r3 = p0.w + q0.w + ob.y;
                        if (a.qkv_dt == LAMPA_F32) {
                            *reinterpret_cast<float4*>((float*)a.o + idx + 32 * q) = make_float4(r0, r1, r2, r3);
                        } else {
                            uint2 w;
                            if (a.qkv_dt == LAMPA_BF16) { w.x = pack_bf16x2(r0, r1); w.y = pack_bf16x2(r2, r3); }
                            else {
                                const __half2 ha = __floats2half2_rn(r0, r1), hb = __floats2half2_rn(r2, r3);
                                w.x = *reinterpret_cast<const uint32_t*>(&ha); w.y = *reinterpret_cast<const uint32_t*>(&hb);
                            }
                            *reinterpret_cast<uint2*>((uint16_t*)a.o + idx + 32 * q) = w;
                        }
                    }
                }
            };
            if (a.out_perm_rows > 0) emit(ScatterOn{}); else emit(ScatterOff{});
            __syncwarp();
            if (lane == 0) mbar_arrive(sfree + (i % UNST));   // B^T, lambda and O_local of this stage have been read
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, 512);
}


// -------------------------------------------------------------------------------------------------
// Plain rule, same machinery with one state per head:  O_n = O_local + Q~ S_n ;  S_{n+1} = M S_n + B.
// One CTA per (block of 32 chunks, pair of heads).  A head's state S^T (64 rows v x 64 columns k) is the
// bf16 A operand of an MMA with M = 64, which occupies 16 lanes of each 32-lane quarter of tensor
// memory: the two heads interleave (head 0 in lanes 0..15 of a quarter, head 1 in lanes 16..31), so one
// tcgen05.ld hands every thread of the 16 epilogue warps one row segment, thread = (head, state row,
// 16 columns).  Per chunk and head ONE accumulating MMA  D[64 x 128] = S^T x [M ; Q~]^T  gives the
// advanced state (columns 0..63) and (Q~ S)^T (columns 64..127).  The chain MMA -> + B^T -> bf16
// operand -> next MMA is serial by nature (one state), and the pass is bound by streaming the records.
// O_local is read straight from the record in global memory by the thread that stores the output.
// -------------------------------------------------------------------------------------------------
constexpr int PNST = 3;                      // record stages (two heads each)
constexpr int PSTAGE_HEAD = UR::OL_OFF;      // M | Q~ | B^T of one head
constexpr int PSTAGE = 2 * PSTAGE_HEAD;
constexpr int PSM_OT = 1024;                 // two buffers (chunk parity) of fp32 [2 heads][64 tokens][64 v]
constexpr int PSM_STAGE = PSM_OT + 2 * 2 * 64 * 64 * 4;
constexpr int PTM_A = 0, PTM_D = 64;         // tensor-memory columns (256 allocated)
constexpr uint32_t PMMA_IDESC = umma_idesc(64, 128);

__global__ void __launch_bounds__(UTHREADS, 1) gdn_out_plain_umma_kernel(GdnArgs a) {
    extern __shared__ __align__(1024) unsigned char smem[];
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + SM_BAR);      // records landed            (tx count)
    uint64_t* sfree = full + PNST;                                      // stage consumed            (16 warps)
    uint64_t* mdone = sfree + PNST;                                     // chunk's MMAs complete     (commit)
    uint64_t* aready = mdone + 1;                                       // operands rewritten        (16 warps)
    uint64_t* drainb = aready + 1;
    uint32_t* tslot = reinterpret_cast<uint32_t*>(smem + SM_BAR + 256);
    float* sOT = reinterpret_cast<float*>(smem + PSM_OT);

    const int H = a.H, npair = (H + 1) / 2;
    const int gb = blockIdx.x / npair, h0 = 2 * (blockIdx.x % npair);
    if (gb >= a.block_off[a.nseq]) return;
    const int nheads = min(2, H - h0);
    const int seq = find_seq(a.block_off, a.nseq, gb);
    const int b = gb - a.block_off[seq];
    const int nch = a.chunk_off[seq + 1] - a.chunk_off[seq];
    const int c0 = a.chunk_off[seq] + b * BLOCK_CHUNKS;
    const int nsteps = min(BLOCK_CHUNKS, nch - b * BLOCK_CHUNKS);
    const int64_t tok0 = a.tok_off[seq] + (int64_t)b * BLOCK_CHUNKS * CHUNK, tok_end = a.tok_off[seq + 1];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int sp = warp & 3, cq = (warp >> 2) & 3;     // lane quarter; 16 state columns and 16 tokens
    const int sub = lane >> 4, v = 16 * sp + (lane & 15);   // head of the pair, state row
    unsigned char* stage0 = smem + PSM_STAGE;
    const char* rec0 = a.rec + ((size_t)c0 * H + h0) * a.rec_bytes;
    const size_t rec_stride = (size_t)H * a.rec_bytes;

    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < PNST; ++s) { mbar_init(full + s, 1); mbar_init(sfree + s, UEPI_WARPS); }
        mbar_init(mdone, 1);
        mbar_init(aready, UEPI_WARPS);
        mbar_init(drainb, 1);
        fence_mbar_init();
    }
    if (warp == 0) tmem_alloc(tslot, 256);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t taddr = *tslot;
    const uint32_t tlane = taddr + ((uint32_t)(32 * sp) << 16);
    // the block's entry state
    if (warp < UEPI_WARPS) {
        float x[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) x[i] = 0.f;
        if (sub < nheads) {
            const float4* e = reinterpret_cast<const float4*>(a.entry + ((size_t)gb * H + h0 + sub) * UR::STATE_FLOATS + (size_t)v * UKD + 16 * cq);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float4 f = e[i];
                x[4 * i] = f.x; x[4 * i + 1] = f.y; x[4 * i + 2] = f.z; x[4 * i + 3] = f.w;
            }
        }
        tmem_st_bf16x16(tlane + PTM_A + 8 * cq, x);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    bool dead = false;
    const int budget = a.poll_budget;

    if (warp == UEPI_WARPS) {
        // ---- control warp: one lane streams records and issues MMAs --------------------------------
        if (lane == 0) {
            int loaded = 0, landed = 0;
            auto load_record = [&](int step) {
                uint64_t* fb = full + (step % PNST);
                unsigned char* dst = stage0 + (size_t)(step % PNST) * PSTAGE;
                const char* src = rec0 + (size_t)step * rec_stride;
                mbar_expect_tx(fb, (uint32_t)(nheads * PSTAGE_HEAD));
                for (int hd = 0; hd < nheads; ++hd) bulk_g2s(dst + hd * PSTAGE_HEAD, src + (size_t)hd * a.rec_bytes, (uint32_t)PSTAGE_HEAD, fb);
                loaded = step + 1;
            };
            for (int s = 0; s < PNST - 1 && s < nsteps; ++s) load_record(s);
            for (int i = 0; i < nsteps && !dead; ++i) {
                const unsigned char* st = stage0 + (size_t)(i % PNST) * PSTAGE;
                if (mbar_wait(full + (i % PNST), (uint32_t)((i / PNST) & 1), dead, a.status, 200 + i, budget)) landed = i + 1;
                // the operands rewritten by the previous chunk (which also means its accumulators have been read)
                if (i > 0) mbar_wait(aready, (uint32_t)((i - 1) & 1), dead, a.status, 400, budget);
                if (dead) break;
                tc_fence_after();
                for (int hd = 0; hd < nheads; ++hd) {
                    const uint32_t dsub = taddr + ((uint32_t)(16 * hd) << 16);
                    const uint64_t db = umma_desc_k128(smem_u32(st + hd * PSTAGE_HEAD + UR::M_OFF));
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) umma_f16_ts(dsub + PTM_D, dsub + PTM_A + 8 * kk, db + 2 * kk, PMMA_IDESC, kk > 0 ? 1u : 0u);
                }
                umma_commit(mdone);
                if (i + PNST - 1 < nsteps) {       // refill the stage chunk i-1 used, once everyone is done with it
                    if (i >= 1) mbar_wait(sfree + ((i - 1) % PNST), (uint32_t)(((i - 1) / PNST) & 1), dead, a.status, 500 + i, budget);
                    if (!dead) load_record(i + PNST - 1);
                }
            }
            // nothing asynchronous may outlive the CTA: records still on their way land first, and one
            // last commit covers every MMA issued above
            for (int s = landed; s < loaded; ++s) mbar_drain(full + (s % PNST), (uint32_t)((s / PNST) & 1));
            umma_commit(drainb);
            mbar_drain(drainb, 0u);
        }
    } else if (warp == UEPI_WARPS + 1) {
        // ---- relay warp: mbarrier completions -> named barriers ----
        for (int i = 0; i < nsteps; ++i) {
            // the record barrier alternates between two ids: with a single MMA per chunk nothing keeps this warp from
            // announcing record i + 1 before every epilogue warp has picked up record i
            mbar_wait(full + (i % PNST), (uint32_t)((i / PNST) & 1), dead, a.status, 250 + i, budget);
            relay_pass(UNB_REC + (i & 1), dead);
            mbar_wait(mdone, (uint32_t)(i & 1), dead, a.status, 300, budget);
            relay_pass(UNB_PAIR, dead);
        }
    } else {
        // ---- epilogue warps: thread = (head sub, state row v, 16 state columns / 16 tokens) ----------
        const int lt = tid & 127;                      // position in the warpgroup that shares cq
        const int otok = 16 * cq + (lt >> 3), ocol = (lt & 7) * 8;
        // Columns of the fp32 output tile are permuted so that neither side meets a bank conflict: bit 4 flips with the
        // head (the two half-warps of a store write the two heads' tiles, 16 KB apart, at the same v) and bit 2 with
        // bit 5 (the eight lanes of a token read 16 bytes every 32 bytes).
        const int vsw = v ^ (16 * sub) ^ (4 * ((v >> 5) & 1));
        const int osw = 4 * ((ocol >> 5) & 1);
        for (int i = 0; i < nsteps; ++i) {
            const unsigned char* sBt = stage0 + (size_t)(i % PNST) * PSTAGE + sub * PSTAGE_HEAD + UR::BT_OFF;
            // this thread's 2 x 8 values of O_local (one per head), from the records in global memory
            const int64_t t_out = tok0 + (int64_t)i * CHUNK + otok;
            uint4 ol[2];
#pragma unroll
            for (int hd = 0; hd < 2; ++hd) {
                ol[hd] = make_uint4(0u, 0u, 0u, 0u);
                if (hd < nheads && t_out < tok_end)
                    ol[hd] = __ldg(reinterpret_cast<const uint4*>(rec0 + (size_t)i * rec_stride + (size_t)hd * a.rec_bytes + UR::OL_OFF) + UR::TV::off(otok, ocol) / 8);
            }
            named_sync(UNB_REC + (i & 1));             // records landed
            named_sync(UNB_PAIR);                      // chunk's MMAs complete
            tc_fence_after();
            float x[16], y[16];
            tmem_ld16_issue(y, tlane + PTM_D + 64 + 16 * cq);
            if (i + 1 < nsteps) tmem_ld16_issue(x, tlane + PTM_D + 16 * cq);
            tmem_wait_ld();
            if (i + 1 < nsteps) {                      // S <- M S + B as the next chunk's operand
                tmem_loaded(x);
                const uint4 bq0 = *reinterpret_cast<const uint4*>(sBt + v * 128 + (((2 * cq) ^ (v & 7)) << 4));
                const uint4 bq1 = *reinterpret_cast<const uint4*>(sBt + v * 128 + (((2 * cq + 1) ^ (v & 7)) << 4));
                const uint32_t bw[8] = {bq0.x, bq0.y, bq0.z, bq0.w, bq1.x, bq1.y, bq1.z, bq1.w};
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const float2 f = unpack_bf16x2(bw[c]);
                    x[2 * c] += f.x; x[2 * c + 1] += f.y;
                }
                tmem_st_bf16x16(tlane + PTM_A + 8 * cq, x);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(aready); mbar_arrive(sfree + (i % PNST)); }   // operand rewritten; B^T of this stage read
            // output: (Q~ S)^T of this row goes through shared memory to the thread that stores the token.  Tokens
            // 16 cq .. 16 cq + 15 are written and read by the four warps with this cq alone, so the barrier is theirs;
            // the buffer alternates with the chunk (a warp cannot get two chunks ahead of one that is still reading
            // without passing that barrier).
            tmem_loaded(y);
            float* sOTc = sOT + (i & 1) * (2 * 64 * 64);
#pragma unroll
            for (int j = 0; j < 16; ++j) sOTc[(sub * 64 + 16 * cq + j) * 64 + vsw] = y[j];
            switch (cq) {
                case 0: asm volatile("bar.sync 1, 128;\n" ::: "memory"); break;
                case 1: asm volatile("bar.sync 2, 128;\n" ::: "memory"); break;
                case 2: asm volatile("bar.sync 3, 128;\n" ::: "memory"); break;
                default: asm volatile("bar.sync 4, 128;\n" ::: "memory"); break;
            }
            auto emit = [&](auto scat) {
            const int64_t orow = t_out < tok_end ? out_row<decltype(scat)::value>(a, t_out) : -1;
            if (orow >= 0) {
#pragma unroll
                for (int hd = 0; hd < 2; ++hd) {
                    if (hd >= nheads) break;
                    const size_t idx = ((size_t)orow * H + h0 + hd) * UVD + ocol;
                    const uint32_t olw[4] = {ol[hd].x, ol[hd].y, ol[hd].z, ol[hd].w};
                    float r[8];
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        const float4 p0 = *reinterpret_cast<const float4*>(sOTc + (hd * 64 + otok) * 64 + ((ocol + 4 * q) ^ (16 * hd) ^ osw));
                        const float2 oa = unpack_bf16x2(olw[2 * q]), ob = unpack_bf16x2(olw[2 * q + 1]);
                        r[4 * q] = p0.x + oa.x; r[4 * q + 1] = p0.y + oa.y; r[4 * q + 2] = p0.z + ob.x; r[4 * q + 3] = p0.w + ob.y;
                    }
                    if (a.qkv_dt == LAMPA_F32) {
                        float4* o4 = reinterpret_cast<float4*>((float*)a.o + idx);
                        o4[0] = make_float4(r[0], r[1], r[2], r[3]);
                        o4[1] = make_float4(r[4], r[5], r[6], r[7]);
                    } else {
                        uint32_t w[4];
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (a.qkv_dt == LAMPA_BF16) w[q] = pack_bf16x2(r[2 * q], r[2 * q + 1]);
                            else { const __half2 hh = __floats2half2_rn(r[2 * q], r[2 * q + 1]); w[q] = *reinterpret_cast<const uint32_t*>(&hh); }
                        }
                        *reinterpret_cast<uint4*>((uint16_t*)a.o + idx) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
            };
            if (a.out_perm_rows > 0) emit(ScatterOn{}); else emit(ScatterOff{});
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(taddr, 256);
}

}  // namespace

int launch_out_hier_umma(const GdnArgs& a, cudaStream_t st) {
    const int smem = SM_STAGE + UNST * ustage_bytes(a.LC);
    if (smem > 227 * 1024 || a.nhigh_max > UNP) return LAMPA_ERR_UNSUPPORTED;
    if (cudaFuncSetAttribute(gdn_out_hier_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return LAMPA_ERR_CUDA;
    UnitOrder uo;
    uo.nbs = 0;
    if (a.fixed_T > 0 && a.nseq > 0 && a.nb_max % a.nseq == 0 && a.nb_max / a.nseq <= 64) {
        uo.nbs = a.nb_max / a.nseq;
        int n = 0;
        for (int pairs = UNP; pairs >= 0; --pairs)        // stable: block order kept inside a class
            for (int b = 0; b < uo.nbs; ++b) {
                int live = 0;
                for (int lh = 0; lh < a.nhigh_max; ++lh) live += (b >> lh) & 1;
                if ((BLOCK_LOG + live + 1) / 2 == pairs) uo.order[n++] = (unsigned char)b;
            }
        if (n != uo.nbs) uo.nbs = 0;
    }
    ProfScope prof("gdn_out_hier_umma", st);
    gdn_out_hier_umma_kernel<<<dim3((unsigned)a.nb_max * a.H), UTHREADS, smem, st>>>(a, uo);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

int launch_out_plain_umma(const GdnArgs& a, cudaStream_t st) {
    const int smem = PSM_STAGE + PNST * PSTAGE;
    if (cudaFuncSetAttribute(gdn_out_plain_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
        return LAMPA_ERR_CUDA;
    ProfScope prof("gdn_out_plain_umma", st);
    gdn_out_plain_umma_kernel<<<dim3((unsigned)a.nb_max * ((a.H + 1) / 2)), UTHREADS, smem, st>>>(a);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

}  // namespace lampa
