// Layout of the per-chunk and per-block intermediates of the gated-delta forward, and the
// launchers shared between translation units.
//
// Algebra (per sequence and head, chunk length 64, G = inclusive cumsum of g inside the chunk,
// E_ij = exp(G_i - G_j) for i >= j):
//   Aw = (I + tril(diag(beta) K K^T, -1))^-1          W~ = diag(e^G) Aw diag(beta) K
//   U  = (Aw .* E) diag(beta) V                        K~ = diag(e^{G_last - G}) K
//   M  = e^{G_last} I - K~^T W~     B = K~^T U         Q~ = diag(e^G) Q - (tril(Q K^T) .* E) W~
// so that one chunk acts on the running state as  S <- M S + B  and reads it as  Q~ S.
// The prep kernels write one record {M, Q~, B^T, O_local, lambda} per (chunk, head); the scan
// kernels only ever multiply by those.
#pragma once
#include "common.cuh"

namespace lampa {

constexpr int BLOCK_CHUNKS = 32;     // chunks per block of the block-parallel scan
constexpr int BLOCK_LOG = 5;         // log2(BLOCK_CHUNKS): chunk levels 0..4 live inside a block
constexpr int NLW = 5;               // level states carried per warp in the hierarchical output pass
constexpr int MAX_GROUPS = 3;        // 1 group of in-block levels + up to 2 groups of cross-block levels

// Layout of a K-wide bf16 tile ([rows][KD]) inside a record.  For KD = 64 rows are dense 128-byte
// lines whose eight 16-byte chunks are XOR-swizzled with the row index (the 128B-swizzle pattern
// tcgen05.mma and ldmatrix both read without bank conflicts); other widths use a padded pitch.
template <int KD>
struct Tile {
    static constexpr bool SWZ = (KD == 64);
    static constexpr int PITCH = SWZ ? 64 : KD + 8;
    __host__ __device__ static constexpr int off(int r, int c) {
        return SWZ ? r * 64 + ((((c >> 3) ^ r) & 7) << 3) + (c & 7) : r * PITCH + c;
    }
    __host__ __device__ static constexpr int bytes(int rows) { return rows * PITCH * 2; }
};

template <int KD, int VD>
struct Rec {
    using T = Tile<KD>;
    static constexpr int KP = KD + 8;                 // padded bf16 row pitch (block composites)
    using TV = Tile<VD>;                              // layout of O_local[token][v]: a V-wide bf16 tile
    static constexpr int M_OFF = 0;
    static constexpr int M_BYTES = T::bytes(KD);      // M[k_out][k_in]
    static constexpr int QT_OFF = M_OFF + M_BYTES;    // M and Q~ are adjacent: together they are one 128-row B operand
    static constexpr int QT_BYTES = T::bytes(CHUNK);  // Q~[token][k]
    static constexpr int BT_OFF = QT_OFF + QT_BYTES;
    static constexpr int BT_BYTES = T::bytes(VD);     // B^T[v][k]
    static constexpr int OL_OFF = BT_OFF + BT_BYTES;
    static constexpr int OL_BYTES = TV::bytes(CHUNK); // O_local, bf16 (added once, in fp32, by the output pass)
    static constexpr int LAM_OFF = OL_OFF + OL_BYTES; // lambda of chunk levels: [LC][64] fp32
    static constexpr int PRE_BYTES = OL_OFF;          // M, Q~, B^T: what the compose pass streams
    static constexpr int ALIGN = T::SWZ ? 1024 : 128; // records and shared-memory stages
    __host__ __device__ static constexpr int bytes(int LC) { return LAM_OFF + LC * CHUNK * 4; }
    // block composite: Mblk[k_out][k_in] bf16 (padded pitch), then Bblk^T[v][k] fp32 (pitch KD + 8)
    static constexpr int BP = KD + 8;
    static constexpr int BLK_M_OFF = 0;
    static constexpr int BLK_M_BYTES = KD * KP * 2;
    static constexpr int BLK_B_OFF = BLK_M_BYTES;
    static constexpr int BLK_BYTES = BLK_M_BYTES + VD * BP * 4;
    static constexpr int STATE_FLOATS = VD * KD;      // an S^T[v][k] fp32 state
};

struct GdnArgs {
    const void* q; const void* k; const void* v; const void* g; const void* beta; const void* lam;
    const float* h0; float* ht; void* o;
    const int64_t* out_perm; long long out_perm_rows;   // optional scatter of the output rows (lampa_hgdn_fwd_scatter)
    int qkv_dt, gb_dt, lam_dt;
    int H, L, LC;
    int use_l2norm;
    float scale;
    int nseq;
    int fixed_T;        // tokens per sequence when there is no cu_seqlens (0 otherwise)
    int fixed_cps;      // chunks per sequence in that case: positions follow by arithmetic, no plan loads
    int plan_inline;    // no cu_seqlens: the first preparation CTA writes the offset tables below (no separate launch)
    int nc_max, nb_max, nhigh_max;
    long long total_tokens;  // B * T of the call (rows of the token-major inputs)
    const int64_t* tok_off; const int32_t* chunk_off; const int32_t* block_off;
    char* rec; size_t rec_bytes;          // per (chunk, head) records
    char* blk;                            // per (block, head) composites
    float* entry;                         // entry states: plain [nb][H][V][K]; hier [nb][nhigh][H][V][K]
    int32_t* status;
    int use_umma;                         // tcgen05 kernels where they exist (K = V = 64)
    int poll_budget;                      // polls before a device wait gives up (MBAR_POLLS unless a test lowers it)
    long long* ticks; int ticks_ctas;     // stage clocks for tuning: [ticks_ctas][16] or NULL (lampa_debug_set_tick_buffer)
};

// Stage clock of a preparation CTA: thread 0 of the first `ticks_ctas` CTAs stores clock64() in its slot.
__device__ __forceinline__ void stage_tick(const GdnArgs& a, int cta, int slot) {
    if (a.ticks != nullptr && threadIdx.x == 0 && cta < a.ticks_ctas) a.ticks[(size_t)cta * 16 + slot] = clock64();
}

// Offset tables of equally long sequences, written by the first CTA of the preparation kernel for the passes that
// follow it (the preparation kernel itself locates its chunks by arithmetic in that case).
__device__ __forceinline__ void write_fixed_plan(const GdnArgs& a) {
    const int bps = (a.fixed_cps + BLOCK_CHUNKS - 1) / BLOCK_CHUNKS;
    for (int s = threadIdx.x; s <= a.nseq; s += blockDim.x) {
        const_cast<int64_t*>(a.tok_off)[s] = (int64_t)s * a.fixed_T;
        const_cast<int32_t*>(a.chunk_off)[s] = s * a.fixed_cps;
        const_cast<int32_t*>(a.block_off)[s] = s * bps;
    }
}

struct PlanArgs {
    const int64_t* cu; int nseq; int B; int T; int L; int hier;
    int64_t* tok_off; int32_t* chunk_off; int32_t* block_off; int32_t* status;
};

int launch_plan(const PlanArgs& p, cudaStream_t st);
template <int KD, int VD> int launch_prep(const GdnArgs& a, bool hier, cudaStream_t st);
template <int KD, int VD> int launch_scan_plain(const GdnArgs& a, cudaStream_t st);
template <int KD, int VD> int launch_scan_hier(const GdnArgs& a, cudaStream_t st);

// Where chunk slot c lives: sequence, first token, number of valid tokens.  False for unused slots.
struct ChunkLoc { int seq; int64_t t0; int len; };
__device__ __forceinline__ bool locate_chunk(const GdnArgs& a, int c, ChunkLoc& loc) {
    if (a.fixed_T > 0) {
        if (c >= a.nseq * a.fixed_cps) return false;
        loc.seq = c / a.fixed_cps;
        const int local = c - loc.seq * a.fixed_cps;
        loc.t0 = (int64_t)loc.seq * a.fixed_T + (int64_t)local * CHUNK;
        loc.len = min(CHUNK, a.fixed_T - local * CHUNK);
        return true;
    }
    if (c >= a.chunk_off[a.nseq]) return false;
    loc.seq = find_seq(a.chunk_off, a.nseq, c);
    loc.t0 = a.tok_off[loc.seq] + (int64_t)(c - a.chunk_off[loc.seq]) * CHUNK;
    loc.len = (int)min((int64_t)CHUNK, a.tok_off[loc.seq + 1] - loc.t0);
    return true;
}

// Row of o that token t of the call is written to: its own, or out_perm[t] for the first out_perm_rows tokens
// when the caller asked for the output to be scattered (the un-ordering of a sorted event folded into the store).
// -1 for an index outside the output: that row is not written (the preparation kernel has reported it, see
// check_out_perm; the output passes stay free of the reporting code).
// SCAT is a compile-time flag so that the common, unscattered store keeps its plain address arithmetic: the output
// passes test a.out_perm_rows once per chunk and run one of two copies of their store code.
template <bool SCAT>
__device__ __forceinline__ int64_t out_row(const GdnArgs& a, int64_t t) {
    if (!SCAT || t >= a.out_perm_rows) return t;
    const int64_t r = a.out_perm[t];
    return (unsigned long long)r < (unsigned long long)a.total_tokens ? r : -1;
}
struct ScatterOn { static constexpr bool value = true; };
struct ScatterOff { static constexpr bool value = false; };
// The scatter indices of one chunk's tokens, checked by the first 64 threads of one preparation CTA per chunk.
__device__ __forceinline__ void check_out_perm(const GdnArgs& a, int64_t t0, int len) {
    const int64_t t = t0 + threadIdx.x;
    if (a.out_perm_rows > 0 && (int)threadIdx.x < len && t < a.out_perm_rows &&
        (unsigned long long)a.out_perm[t] >= (unsigned long long)a.total_tokens)
        set_status(a.status, LAMPA_ERR_BOUNDS, 30, (int)t);
}

// Two output values (adjacent state columns) of one token, converted to the output type.
__device__ __forceinline__ void store_out2(void* o, int dt, size_t idx, float x, float y) {
    if (dt == LAMPA_BF16) *reinterpret_cast<uint32_t*>((__nv_bfloat16*)o + idx) = pack_bf16x2(x, y);
    else if (dt == LAMPA_F16) *reinterpret_cast<__half2*>((__half*)o + idx) = __floats2half2_rn(x, y);
    else *reinterpret_cast<float2*>((float*)o + idx) = make_float2(x, y);
}

int launch_out_hier_umma(const GdnArgs& a, cudaStream_t st);
int launch_out_plain_umma(const GdnArgs& a, cudaStream_t st);  // K = V = 64
int launch_prep_umma(const GdnArgs& a, bool hier, cudaStream_t st);   // K = V = 64, 2-byte q/k/v
template <int KD, int VD> int launch_final_high(const GdnArgs& a, float* states, cudaStream_t st);
template <int KD, int VD> int launch_final_low(const GdnArgs& a, float* states, int32_t* counts, cudaStream_t st);

// One decode step of the hierarchical rule on a Fenwick state (gdn_state.cu).
struct StepArgs {
    const void* q; const void* k; const void* v; const void* g; const void* beta; const void* lam;
    float* states; int32_t* counts; void* o;
    int qkv_dt, gb_dt, lam_dt;
    int B, H, L, use_l2norm;
    int32_t* status;
};
template <int KD, int VD> int launch_hgdn_step(const StepArgs& s, cudaStream_t st);

__host__ __device__ inline int ceil_log2_int(int x) {   // smallest e with 2^e >= x (x >= 1)
    int e = 0;
    while ((1 << e) < x) ++e;
    return e;
}

}  // namespace lampa
