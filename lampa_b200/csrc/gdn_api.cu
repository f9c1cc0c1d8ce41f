// C ABI of the gated-delta forward: argument checks, workspace carve-up, kernel dispatch.
#include "gdn.cuh"
#include <cstdlib>

using namespace lampa;

namespace {

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

int g_poll_budget = MBAR_POLLS;   // see lampa_debug_set_poll_budget
int g_force_mma_sync = 0;         // see lampa_debug_force_mma_sync
long long* g_ticks = nullptr;     // see lampa_debug_set_tick_buffer
int g_ticks_ctas = 0;

struct Layout {
    int nseq, nc_max, nb_max, nhigh_max, LC;
    size_t rec_bytes, blk_bytes, state_bytes;
    size_t off_tok, off_chunk, off_block, off_rec, off_blk, off_entry, total;
};

template <int KD, int VD>
void fill_sizes(Layout& l) {
    using R = Rec<KD, VD>;
    l.rec_bytes = align_up((size_t)R::bytes(l.LC), R::ALIGN);
    l.blk_bytes = R::BLK_BYTES;
    l.state_bytes = (size_t)R::STATE_FLOATS * 4;
}

int dims_supported(int K, int V) {
    return (K == 64 && V == 64) || (K == 32 && V == 32) || (K == 16 && V == 32);
}

int make_layout(const lampa_gdn_desc* d, bool hier, Layout& l) {
    if (!d || d->B <= 0 || d->T < 0 || d->H <= 0) return LAMPA_ERR_ARG;
    if (d->nseq < 0 || (d->nseq > 0 && d->B != 1)) return LAMPA_ERR_ARG;
    if (!dims_supported(d->K, d->V)) return LAMPA_ERR_UNSUPPORTED;
    for (int dt : {d->qkv_dtype, d->gb_dtype})
        if (dt != LAMPA_BF16 && dt != LAMPA_F16 && dt != LAMPA_F32) return LAMPA_ERR_ARG;
    if (hier) {
        if (d->L < 1 || d->L > 40) return LAMPA_ERR_ARG;
        if (d->lam_dtype != LAMPA_BF16 && d->lam_dtype != LAMPA_F16 && d->lam_dtype != LAMPA_F32) return LAMPA_ERR_ARG;
    }
    l.nseq = d->nseq > 0 ? d->nseq : d->B;
    const int64_t ttot = (int64_t)d->B * d->T;
    // each sequence adds at most one ragged chunk and one ragged block
    const int64_t ncm = d->nseq > 0 ? ttot / CHUNK + l.nseq : (int64_t)d->B * ((d->T + CHUNK - 1) / CHUNK);
    const int64_t nbm = d->nseq > 0 ? ncm / BLOCK_CHUNKS + l.nseq
                                    : (int64_t)d->B * (((d->T + CHUNK - 1) / CHUNK + BLOCK_CHUNKS - 1) / BLOCK_CHUNKS);
    if (ncm > (1 << 30) || nbm > 65535LL * 1024) return LAMPA_ERR_UNSUPPORTED;
    l.nc_max = (int)(ncm > 0 ? ncm : 1);
    l.nb_max = (int)(nbm > 0 ? nbm : 1);
    // longest possible sequence bounds the number of cross-block levels
    const int64_t longest = d->nseq > 0 ? (ttot + CHUNK - 1) / CHUNK : (d->T + CHUNK - 1) / CHUNK;
    const int nlev = longest > 1 ? ceil_log2_int((int)longest) : 0;
    l.nhigh_max = hier ? (nlev > BLOCK_LOG ? nlev - BLOCK_LOG : 0) : 0;
    if (hier && 1 + (l.nhigh_max + NLW - 1) / NLW > MAX_GROUPS) return LAMPA_ERR_UNSUPPORTED;
    l.LC = hier ? (d->L > ELL0 ? d->L - ELL0 : 1) : 0;
    if (d->K == 64) fill_sizes<64, 64>(l);
    else if (d->K == 32) fill_sizes<32, 32>(l);
    else fill_sizes<16, 32>(l);
    size_t off = 0;
    l.off_tok = off;   off = align_up(off + (size_t)(l.nseq + 1) * 8, 256);
    l.off_chunk = off; off = align_up(off + (size_t)(l.nseq + 1) * 4, 256);
    l.off_block = off; off = align_up(off + (size_t)(l.nseq + 1) * 4, 256);
    off = align_up(off, 1024);
    l.off_rec = off;   off = align_up(off + (size_t)l.nc_max * d->H * l.rec_bytes, 256);
    l.off_blk = off;   off = align_up(off + (size_t)l.nb_max * d->H * l.blk_bytes, 256);
    l.off_entry = off;
    off = align_up(off + (size_t)l.nb_max * (hier ? (l.nhigh_max > 0 ? l.nhigh_max : 1) : 1) * d->H * l.state_bytes, 256);
    l.total = off;
    return LAMPA_OK;
}

void fill_args(const lampa_gdn_desc* d, bool hier, const Layout& l, char* base, const int64_t* cu,
               int32_t* status, GdnArgs& a) {
    a.q = a.k = a.v = a.g = a.beta = a.lam = nullptr; a.h0 = nullptr; a.ht = nullptr; a.o = nullptr;
    a.out_perm = nullptr; a.out_perm_rows = 0;
    a.qkv_dt = d->qkv_dtype; a.gb_dt = d->gb_dtype; a.lam_dt = d->lam_dtype;
    a.H = d->H; a.L = hier ? d->L : 0; a.LC = l.LC;
    a.use_l2norm = d->use_l2norm; a.scale = d->scale;
    a.fixed_T = cu ? 0 : d->T;
    a.fixed_cps = cu ? 0 : (d->T + CHUNK - 1) / CHUNK;
    a.plan_inline = 0;
    a.total_tokens = (long long)d->B * d->T;
    a.nseq = l.nseq; a.nc_max = l.nc_max; a.nb_max = l.nb_max; a.nhigh_max = l.nhigh_max;
    a.tok_off = (int64_t*)(base + l.off_tok);
    a.chunk_off = (int32_t*)(base + l.off_chunk);
    a.block_off = (int32_t*)(base + l.off_block);
    a.rec = base + l.off_rec; a.rec_bytes = l.rec_bytes;
    a.blk = base + l.off_blk;
    a.entry = (float*)(base + l.off_entry);
    a.status = status;
    static const int no_umma = [] { const char* e = getenv("LAMPA_B200_NO_UMMA"); return (e && e[0] == '1') ? 1 : 0; }();
    a.use_umma = (no_umma || g_force_mma_sync) ? 0 : 1;
    a.poll_budget = g_poll_budget;
    a.ticks = g_ticks;
    a.ticks_ctas = g_ticks_ctas;
}

int run(const lampa_gdn_desc* d, bool hier, const void* q, const void* k, const void* v, const void* g,
        const void* beta, const void* lam, const float* h0, const int64_t* cu, void* o, float* ht,
        void* ws, size_t ws_bytes, int32_t* status, void* stream, const int64_t* out_perm = nullptr,
        int64_t out_perm_rows = 0) {
    Layout l;
    int rc = make_layout(d, hier, l);
    if (rc != LAMPA_OK) return rc;
    if ((int64_t)d->B * d->T == 0) return LAMPA_OK;
    if (!q || !k || !v || !g || !beta || !o || !ws || (hier && !lam)) return LAMPA_ERR_ARG;
    if (d->nseq > 0 && !cu) return LAMPA_ERR_ARG;
    if (ws_bytes < l.total || ((uintptr_t)ws & 1023)) return LAMPA_ERR_WORKSPACE;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)o) & 15)) return LAMPA_ERR_ARG;
    if (hier && !cu && d->L < ELL0 + ((d->T + CHUNK - 1) / CHUNK > 1 ? ceil_log2_int((d->T + CHUNK - 1) / CHUNK) : 0))
        return LAMPA_ERR_LEVELS;
    cudaStream_t st = (cudaStream_t)stream;
    char* base = (char*)ws;

    GdnArgs a;
    fill_args(d, hier, l, base, cu, status, a);
    a.q = q; a.k = k; a.v = v; a.g = g; a.beta = beta; a.lam = lam; a.h0 = h0; a.ht = ht; a.o = o;
    a.out_perm = out_perm; a.out_perm_rows = out_perm ? out_perm_rows : 0;

    PlanArgs p;
    p.cu = cu; p.nseq = l.nseq; p.B = d->B; p.T = d->T; p.L = d->L; p.hier = hier ? 1 : 0;
    p.tok_off = (int64_t*)a.tok_off;
    p.chunk_off = (int32_t*)a.chunk_off;
    p.block_off = (int32_t*)a.block_off;
    p.status = status;
    if (cu) {
        rc = launch_plan(p, st);
        if (rc != LAMPA_OK) return rc;
    } else {
        a.plan_inline = 1;         // equally long sequences: the preparation kernel writes the tables itself
    }

#define LAMPA_DISPATCH(KD, VD)                                         \
    do {                                                               \
        rc = launch_prep<KD, VD>(a, hier, st);                         \
        if (rc != LAMPA_OK) return rc;                                 \
        return hier ? launch_scan_hier<KD, VD>(a, st) : launch_scan_plain<KD, VD>(a, st); \
    } while (0)
    if (d->K == 64 && a.use_umma && d->qkv_dtype != LAMPA_F32) {
        rc = launch_prep_umma(a, hier, st);
        if (rc == LAMPA_OK) return hier ? launch_scan_hier<64, 64>(a, st) : launch_scan_plain<64, 64>(a, st);
        if (rc != LAMPA_ERR_UNSUPPORTED) return rc;       // too many lambda levels for its shared memory: the other kernel takes it
    }
    if (d->K == 64) LAMPA_DISPATCH(64, 64);
    if (d->K == 32) LAMPA_DISPATCH(32, 32);
    LAMPA_DISPATCH(16, 32);
#undef LAMPA_DISPATCH
}

}  // namespace

extern "C" int lampa_version(void) { return 200; }

extern "C" int lampa_debug_set_tick_buffer(long long* ticks, int n_ctas) {
    if (n_ctas < 0 || (n_ctas > 0 && !ticks)) return LAMPA_ERR_ARG;
    g_ticks = n_ctas > 0 ? ticks : nullptr;
    g_ticks_ctas = n_ctas;
    return LAMPA_OK;
}

extern "C" int lampa_debug_force_mma_sync(int on) {
    g_force_mma_sync = on ? 1 : 0;
    return LAMPA_OK;
}

extern "C" int lampa_debug_set_poll_budget(int polls) {
    if (polls < 0) return LAMPA_ERR_ARG;
    g_poll_budget = polls > MBAR_POLLS ? MBAR_POLLS : polls;
    return LAMPA_OK;
}

extern "C" const char* lampa_error_string(int code) {
    switch (code) {
        case LAMPA_OK: return "ok";
        case LAMPA_ERR_ARG: return "invalid argument";
        case LAMPA_ERR_UNSUPPORTED: return "unsupported shape (head dims must be 64/64, 32/32 or 16/32; sequence too long)";
        case LAMPA_ERR_WORKSPACE: return "workspace too small or not 1024-byte aligned";
        case LAMPA_ERR_CUDA: return "CUDA runtime error at launch";
        case LAMPA_ERR_TIMEOUT: return "device wait ran out";
        case LAMPA_ERR_LEVELS: return "lambda has fewer levels than 7 + ceil(log2(chunks))";
        case LAMPA_ERR_BOUNDS: return "index outside its extent (bad cu_seqlens?)";
        case LAMPA_ERR_TOO_LARGE: return "input larger than the fixed capacity of this allocation-free entry point";
        default: return "unknown error";
    }
}

extern "C" int lampa_gdn_workspace_bytes(const lampa_gdn_desc* d, size_t* bytes) {
    if (!bytes) return LAMPA_ERR_ARG;
    Layout l;
    const int rc = make_layout(d, d && d->L > 0, l);
    if (rc != LAMPA_OK) return rc;
    *bytes = l.total;
    return LAMPA_OK;
}

extern "C" int lampa_gdn_workspace_layout(const lampa_gdn_desc* d, size_t out[12]) {
    if (!out) return LAMPA_ERR_ARG;
    Layout l;
    const int rc = make_layout(d, d && d->L > 0, l);
    if (rc != LAMPA_OK) return rc;
    size_t m, bt, qt, ol, lam;
    if (d->K == 64) { using R = Rec<64, 64>; m = R::M_OFF; bt = R::BT_OFF; qt = R::QT_OFF; ol = R::OL_OFF; lam = R::LAM_OFF; }
    else if (d->K == 32) { using R = Rec<32, 32>; m = R::M_OFF; bt = R::BT_OFF; qt = R::QT_OFF; ol = R::OL_OFF; lam = R::LAM_OFF; }
    else { using R = Rec<16, 32>; m = R::M_OFF; bt = R::BT_OFF; qt = R::QT_OFF; ol = R::OL_OFF; lam = R::LAM_OFF; }
    out[0] = l.off_rec; out[1] = l.rec_bytes; out[2] = m; out[3] = bt; out[4] = qt; out[5] = ol; out[6] = lam;
    out[7] = (size_t)l.LC; out[8] = (size_t)l.nc_max; out[9] = (size_t)BLOCK_CHUNKS;
    out[10] = l.off_blk; out[11] = l.off_entry;
    return LAMPA_OK;
}

extern "C" int lampa_gdn_fwd(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                             const void* g, const void* beta, const float* h0, const int64_t* cu_seqlens,
                             void* o, float* ht, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
    if (d && d->L != 0) return LAMPA_ERR_ARG;
    return run(d, false, q, k, v, g, beta, nullptr, h0, cu_seqlens, o, ht, ws, ws_bytes, status, stream);
}

extern "C" int lampa_hgdn_fwd(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                              const void* g, const void* beta, const void* lam, const int64_t* cu_seqlens,
                              void* o, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
    return run(d, true, q, k, v, g, beta, lam, nullptr, cu_seqlens, o, nullptr, ws, ws_bytes, status, stream);
}

extern "C" int lampa_hgdn_fwd_scatter(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                                      const void* g, const void* beta, const void* lam, const int64_t* cu_seqlens,
                                      const int64_t* out_perm, int64_t out_perm_rows, void* o, void* ws,
                                      size_t ws_bytes, int32_t* status, void* stream) {
    if (!d || out_perm_rows < 0 || out_perm_rows > (int64_t)d->B * d->T || (out_perm_rows > 0 && !out_perm)) return LAMPA_ERR_ARG;
    return run(d, true, q, k, v, g, beta, lam, nullptr, cu_seqlens, o, nullptr, ws, ws_bytes, status, stream,
               out_perm, out_perm_rows);
}

extern "C" int lampa_hgdn_final_state(const lampa_gdn_desc* d, const void* k, const void* v, const void* g,
                                      const void* beta, const int64_t* cu_seqlens, void* ws, size_t ws_bytes,
                                      float* states, int32_t* counts, int32_t* status, void* stream) {
    Layout l;
    int rc = make_layout(d, true, l);
    if (rc != LAMPA_OK) return rc;
    if (d->L < ELL0) return LAMPA_ERR_LEVELS;
    if ((int64_t)d->B * d->T == 0) return LAMPA_OK;
    if (!k || !v || !g || !beta || !ws || !states || !counts) return LAMPA_ERR_ARG;
    if (d->nseq > 0 && !cu_seqlens) return LAMPA_ERR_ARG;
    if (ws_bytes < l.total || ((uintptr_t)ws & 1023)) return LAMPA_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    GdnArgs a;
    fill_args(d, true, l, (char*)ws, cu_seqlens, status, a);
    a.k = k; a.v = v; a.g = g; a.beta = beta;
#define LAMPA_DISPATCH(KD, VD)                                           \
    do {                                                                 \
        rc = launch_final_low<KD, VD>(a, states, counts, st);            \
        if (rc != LAMPA_OK) return rc;                                   \
        return launch_final_high<KD, VD>(a, states, st);                 \
    } while (0)
    if (d->K == 64) LAMPA_DISPATCH(64, 64);
    if (d->K == 32) LAMPA_DISPATCH(32, 32);
    LAMPA_DISPATCH(16, 32);
#undef LAMPA_DISPATCH
}

extern "C" int lampa_hgdn_step(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                               const void* g, const void* beta, const void* lam, float* states,
                               int32_t* counts, void* o, int32_t* status, void* stream) {
    if (!d || d->B <= 0 || d->H <= 0 || d->T != 1) return LAMPA_ERR_ARG;
    if (!dims_supported(d->K, d->V)) return LAMPA_ERR_UNSUPPORTED;
    if (d->L < 1 || d->L > 40) return LAMPA_ERR_ARG;
    for (int dt : {d->qkv_dtype, d->gb_dtype, d->lam_dtype})
        if (dt != LAMPA_BF16 && dt != LAMPA_F16 && dt != LAMPA_F32) return LAMPA_ERR_ARG;
    if (!q || !k || !v || !g || !beta || !lam || !states || !counts || !o) return LAMPA_ERR_ARG;
    StepArgs s;
    s.q = q; s.k = k; s.v = v; s.g = g; s.beta = beta; s.lam = lam;
    s.states = states; s.counts = counts; s.o = o;
    s.qkv_dt = d->qkv_dtype; s.gb_dt = d->gb_dtype; s.lam_dt = d->lam_dtype;
    s.B = d->B; s.H = d->H; s.L = d->L; s.use_l2norm = d->use_l2norm;
    s.status = status;
    cudaStream_t st = (cudaStream_t)stream;
    if (d->K == 64) return launch_hgdn_step<64, 64>(s, st);
    if (d->K == 32) return launch_hgdn_step<32, 32>(s, st);
    return launch_hgdn_step<16, 32>(s, st);
}
