/*
 * TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's algorithms for the
 * LSH ordering + (hierarchical) gated-delta forward path.  Nothing in the product
 * package may link or call this file; it exists so that tests, the smoke check and
 * the CPU-baseline leg of the benchmark have an independent checker.
 *
 * Parity status: pinned.  The reference ships no golden vectors for this path, so
 * the pin is against outputs of the reference's own pure-PyTorch code
 * (models/hattention/recurrent.py, models/baselines/hmamba.py,
 * models/model_utils/hash_utils.py) executed on seeded inputs; those outputs are
 * committed as fixtures under tests/golden/ with the script that made them.
 *
 * Layouts follow the reference: token-major [T, H, D] row-major fp32, g/beta [T, H],
 * lambda [T, H, L], states [H, K, V] (plain) or [H, K, V, L] (hierarchical).
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC oracle.c -o liblampa_oracle.so -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define MAXD 256

#ifdef _OPENMP
#include <omp.h>
#endif
/* Number of host threads the parallel loops use (0 or less: leave as is); returns the setting. */
int oracle_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

/* l2norm as models/hattention/l2norm.py:99-103: x * rsqrt(sum(x^2) + 1e-6). */
static void l2norm_row(const float* x, float* y, int d) {
    float s = 0.f;
    for (int i = 0; i < d; ++i) s += x[i] * x[i];
    float r = 1.0f / sqrtf(s + 1e-6f);
    for (int i = 0; i < d; ++i) y[i] = x[i] * r;
}

/*
 * One token of the gated delta rule on one K x V state
 * (models/hattention/recurrent.py:134-156, GDELTA branch of step_state, and
 * gated_delta_rule_ori.py:430-453):
 *   S <- a * (I - b k k^T) S        (the "gate" applied by HState.insert)
 */
static void apply_gate(float* S, const float* k, float a, float b, int K, int V) {
    float kS[MAXD];
    for (int v = 0; v < V; ++v) kS[v] = 0.f;
    for (int i = 0; i < K; ++i) {
        const float ki = k[i];
        const float* Si = S + (size_t)i * V;
        for (int v = 0; v < V; ++v) kS[v] += ki * Si[v];
    }
    for (int i = 0; i < K; ++i) {
        const float bk = b * k[i];
        float* Si = S + (size_t)i * V;
        for (int v = 0; v < V; ++v) Si[v] = a * (Si[v] - bk * kS[v]);
    }
}

/*
 * Plain gated delta rule, token recurrence.
 *   S_t = e^{g_t} (I - beta_t k_t k_t^T) S_{t-1} + beta_t k_t v_t^T ;  o_t = scale * S_t^T q_t
 * Equivalent to hattention_recurrent with L = ones (recurrent.py:169-216) and to
 * the decode kernel gated_delta_rule_ori.py:430-453.  h0/ht may be NULL.
 * If use_l2norm, q and k rows are normalised first (gated_delta_rule_ori.py:176-178).
 * Sequences: cu[0..nseq] token offsets (NULL => one sequence of T tokens); state
 * restarts from h0[seq] at each sequence start.
 */
int oracle_gdn_plain(const float* q, const float* k, const float* v, const float* g,
                     const float* beta, const float* h0, const int64_t* cu, int nseq,
                     float* o, float* ht, int T, int H, int K, int V, float scale,
                     int use_l2norm) {
    if (K > MAXD || V > MAXD) return -1;
    int64_t cu_default[2] = {0, T};
    if (!cu) { cu = cu_default; nseq = 1; }
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int s = 0; s < nseq; ++s) {
        for (int h = 0; h < H; ++h) {
            float* S = (float*)malloc(sizeof(float) * K * V);
            float qn[MAXD], kn[MAXD];
            if (h0) memcpy(S, h0 + ((size_t)s * H + h) * K * V, sizeof(float) * K * V);
            else memset(S, 0, sizeof(float) * K * V);
            for (int64_t t = cu[s]; t < cu[s + 1]; ++t) {
                const float* qt = q + ((size_t)t * H + h) * K;
                const float* kt = k + ((size_t)t * H + h) * K;
                const float* vt = v + ((size_t)t * H + h) * V;
                if (use_l2norm) { l2norm_row(qt, qn, K); l2norm_row(kt, kn, K); }
                else { memcpy(qn, qt, sizeof(float) * K); memcpy(kn, kt, sizeof(float) * K); }
                const float a = expf(g[(size_t)t * H + h]);
                const float b = beta[(size_t)t * H + h];
                apply_gate(S, kn, a, b, K, V);
                for (int i = 0; i < K; ++i) {
                    const float bk = b * kn[i];
                    float* Si = S + (size_t)i * V;
                    for (int x = 0; x < V; ++x) Si[x] += bk * vt[x];
                }
                float* ot = o + ((size_t)t * H + h) * V;
                for (int x = 0; x < V; ++x) ot[x] = 0.f;
                for (int i = 0; i < K; ++i) {
                    const float qi = qn[i] * scale;
                    const float* Si = S + (size_t)i * V;
                    for (int x = 0; x < V; ++x) ot[x] += qi * Si[x];
                }
            }
            if (ht) memcpy(ht + ((size_t)s * H + h) * K * V, S, sizeof(float) * K * V);
            free(S);
        }
    }
    return 0;
}

/*
 * Hierarchical (Fenwick-level, "log-linear") gated delta rule, token recurrence:
 * a restatement of hattention_recurrent (recurrent.py:169-216) with HState of
 * htype WEAK, base 2, hstruct GDELTA:
 *   cascade_weak (recurrent.py:42-54): walking levels upward, a level whose count
 *     equals its capacity 2^level is merged into the next level and cleared;
 *   insert (recurrent.py:76-100): every level state is multiplied by the gate
 *     a (I - b k k^T); level 0 is overwritten with b k v^T; counts[0] += 1;
 *   output (recurrent.py:159-166): o_t = q_t^T sum_l lambda[t,l] S_l.
 * The API layer (gated_delta_rule_apis.py:68-70, kernel.py:109-111) feeds
 * Q = l2norm(q)*scale and L = lambda/scale, which cancel; here q is l2-normalised
 * (when use_l2norm) and lambda is used as given.
 * states_out: [H, K, V, L] fp32 (may be NULL); counts_out: [L] int32 (may be NULL).
 * Each sequence (cu offsets) starts from an empty hierarchy.
 */
int oracle_hgdn(const float* q, const float* k, const float* v, const float* g,
                const float* beta, const float* lam, const int64_t* cu, int nseq,
                float* o, float* states_out, int32_t* counts_out,
                int T, int H, int K, int V, int L, int use_l2norm) {
    if (K > MAXD || V > MAXD || L > 40) return -1;
    int64_t cu_default[2] = {0, T};
    if (!cu) { cu = cu_default; nseq = 1; }
    int err = 0;
#pragma omp parallel for collapse(2) schedule(dynamic)
    for (int s = 0; s < nseq; ++s) {
        for (int h = 0; h < H; ++h) {
            const size_t KV = (size_t)K * V;
            float* S = (float*)calloc((size_t)L * KV, sizeof(float)); /* [L][K][V] */
            int64_t counts[40];
            float qn[MAXD], kn[MAXD];
            for (int l = 0; l < L; ++l) counts[l] = 0;
            for (int64_t t = cu[s]; t < cu[s + 1]; ++t) {
                /* cascade_weak */
                for (int l = 0; l < L; ++l) {
                    const int64_t cap = (int64_t)1 << l;
                    if (counts[l] == cap) {
                        if (l + 1 >= L) { err = -2; break; }
                        float* a_ = S + (size_t)(l + 1) * KV;
                        float* b_ = S + (size_t)l * KV;
                        for (size_t i = 0; i < KV; ++i) { a_[i] += b_[i]; b_[i] = 0.f; }
                        counts[l + 1] += counts[l];
                        counts[l] = 0;
                    } else {
                        break;
                    }
                }
                const float* qt = q + ((size_t)t * H + h) * K;
                const float* kt = k + ((size_t)t * H + h) * K;
                const float* vt = v + ((size_t)t * H + h) * V;
                if (use_l2norm) { l2norm_row(qt, qn, K); l2norm_row(kt, kn, K); }
                else { memcpy(qn, qt, sizeof(float) * K); memcpy(kn, kt, sizeof(float) * K); }
                const float a = expf(g[(size_t)t * H + h]);
                const float b = beta[(size_t)t * H + h];
                for (int l = 1; l < L; ++l)
                    if (counts[l] > 0) apply_gate(S + (size_t)l * KV, kn, a, b, K, V);
                float* S0 = S;
                for (int i = 0; i < K; ++i)
                    for (int x = 0; x < V; ++x) S0[(size_t)i * V + x] = b * kn[i] * vt[x];
                counts[0] += 1;
                const float* lt = lam + ((size_t)t * H + h) * L;
                float* ot = o + ((size_t)t * H + h) * V;
                for (int x = 0; x < V; ++x) ot[x] = 0.f;
                for (int l = 0; l < L; ++l) {
                    if (counts[l] == 0) continue;
                    const float* Sl = S + (size_t)l * KV;
                    for (int i = 0; i < K; ++i) {
                        const float w = lt[l] * qn[i];
                        for (int x = 0; x < V; ++x) ot[x] += w * Sl[(size_t)i * V + x];
                    }
                }
            }
            if (states_out && s == nseq - 1) {
                for (int i = 0; i < K; ++i)
                    for (int x = 0; x < V; ++x)
                        for (int l = 0; l < L; ++l)
                            states_out[(((size_t)h * K + i) * V + x) * L + l] =
                                S[(size_t)l * KV + (size_t)i * V + x];
            }
            if (counts_out && s == nseq - 1 && h == 0)
                for (int l = 0; l < L; ++l) counts_out[l] = (int32_t)counts[l];
            free(S);
        }
    }
    return err;
}

/*
 * E2LSH integer bucket ids.  Parameter shapes follow E2LSH.__init__
 * (models/model_utils/hash_utils.py:359-371): alpha [n_heads, dim, n_hashes],
 * beta [n_hashes] (offset, drawn U(0, r)).  The reference stops at the float
 * projection bmm(vecs, alpha); the integer id is the textbook E2LSH quantisation
 * floor((a.x + b) / w) with this frozen fp32 operation order:
 *   acc = x[n,0]*a[h,0,c]; acc = acc + x[n,d]*a[h,d,c] (d = 1..dim-1, multiply and
 *   add rounded separately); acc = acc + beta[c]; id = (int32) floorf(acc / w).
 * x rows are row_stride floats apart (the coordinates are the first dim floats).
 * ids: [n_hashes, n_heads, N] int32; keys (optional): the float projection acc
 * before the offset, same layout (this is what E2LSH.forward returns, permuted).
 */
int oracle_lsh_ids(const float* x, int64_t row_stride, const float* alpha, const float* beta,
                   float w, int64_t N, int heads, int rounds, int dim,
                   int32_t* ids, float* keys) {
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const float* xr = x + n * row_stride;
        for (int c = 0; c < rounds; ++c) {
            for (int h = 0; h < heads; ++h) {
                volatile float acc = xr[0] * alpha[((size_t)h * dim + 0) * rounds + c];
                for (int d = 1; d < dim; ++d) {
                    volatile float p = xr[d] * alpha[((size_t)h * dim + d) * rounds + c];
                    acc = acc + p;
                }
                const size_t oidx = ((size_t)c * heads + h) * N + n;
                if (keys) keys[oidx] = acc;
                if (ids) {
                    volatile float sft = acc + beta[c];
                    volatile float qv = sft / w;
                    ids[oidx] = (int32_t)floorf(qv);
                }
            }
        }
    }
    return 0;
}

/* Stable ascending merge sort of (key, index) pairs; perm[i] = original index of
 * the i-th smallest key, ties by original index (torch.sort(stable=True),
 * models/baselines/hmamba.py:343). */
static void msort_i32(const int32_t* key, int64_t* idx, int64_t* tmp, int64_t n) {
    for (int64_t w = 1; w < n; w *= 2) {
        for (int64_t lo = 0; lo < n; lo += 2 * w) {
            int64_t mid = lo + w < n ? lo + w : n, hi = lo + 2 * w < n ? lo + 2 * w : n;
            int64_t i = lo, j = mid, o = lo;
            while (i < mid && j < hi) tmp[o++] = (key[idx[j]] < key[idx[i]]) ? idx[j++] : idx[i++];
            while (i < mid) tmp[o++] = idx[i++];
            while (j < hi) tmp[o++] = idx[j++];
        }
        memcpy(idx, tmp, sizeof(int64_t) * n);
    }
}
static void msort_f32(const float* key, int64_t* idx, int64_t* tmp, int64_t n) {
    for (int64_t w = 1; w < n; w *= 2) {
        for (int64_t lo = 0; lo < n; lo += 2 * w) {
            int64_t mid = lo + w < n ? lo + w : n, hi = lo + 2 * w < n ? lo + 2 * w : n;
            int64_t i = lo, j = mid, o = lo;
            while (i < mid && j < hi) tmp[o++] = (key[idx[j]] < key[idx[i]]) ? idx[j++] : idx[i++];
            while (i < mid) tmp[o++] = idx[i++];
            while (j < hi) tmp[o++] = idx[j++];
        }
        memcpy(idx, tmp, sizeof(int64_t) * n);
    }
}

/* Segmented stable sort: rows given by seg[0..nseg]; perm entries are indices
 * local to their segment.  init (optional) gives a starting order per segment
 * (local indices): the result is init composed with the stable sort of
 * key[init[.]], which is LSHOrdering's norm_idx[bk_idx] (hmamba.py:337-346). */
int oracle_segsort_i32(const int32_t* keys, const int64_t* seg, int nseg,
                       const int64_t* init, int64_t* perm) {
#pragma omp parallel for schedule(dynamic)
    for (int s = 0; s < nseg; ++s) {
        const int64_t n = seg[s + 1] - seg[s];
        int64_t* idx = perm + seg[s];
        int64_t* tmp = (int64_t*)malloc(sizeof(int64_t) * (n > 0 ? n : 1));
        for (int64_t i = 0; i < n; ++i) idx[i] = init ? init[seg[s] + i] : i;
        msort_i32(keys + seg[s], idx, tmp, n);
        free(tmp);
    }
    return 0;
}
int oracle_segsort_f32(const float* keys, const int64_t* seg, int nseg,
                       const int64_t* init, int64_t* perm) {
#pragma omp parallel for schedule(dynamic)
    for (int s = 0; s < nseg; ++s) {
        const int64_t n = seg[s + 1] - seg[s];
        int64_t* idx = perm + seg[s];
        int64_t* tmp = (int64_t*)malloc(sizeof(int64_t) * (n > 0 ? n : 1));
        for (int64_t i = 0; i < n; ++i) idx[i] = init ? init[seg[s] + i] : i;
        msort_f32(keys + seg[s], idx, tmp, n);
        free(tmp);
    }
    return 0;
}

/* invert_permutation (hash_utils.py:46-57): inv[perm[i]] = i, per segment. */
int oracle_invert_perm(const int64_t* perm, const int64_t* seg, int nseg, int64_t* inv) {
    for (int s = 0; s < nseg; ++s) {
        const int64_t n = seg[s + 1] - seg[s];
        for (int64_t i = 0; i < n; ++i) {
            const int64_t p = perm[seg[s] + i];
            if (p < 0 || p >= n) return -1;
            inv[seg[s] + p] = i;
        }
    }
    return 0;
}

/* Row gather, the data movement of LSHOrdering's points.gather (hmamba.py:348-351)
 * and sort_to_buckets (models/attention/hept.py:9-14): dst[seg+i] = src[seg+perm[seg+i]]. */
int oracle_permute_rows(const void* src, const int64_t* perm, const int64_t* seg, int nseg,
                        void* dst, int64_t row_bytes) {
    for (int s = 0; s < nseg; ++s) {
        const int64_t n = seg[s + 1] - seg[s];
        for (int64_t i = 0; i < n; ++i)
            memcpy((char*)dst + (seg[s] + i) * row_bytes,
                   (const char*)src + (seg[s] + perm[seg[s] + i]) * row_bytes, row_bytes);
    }
    return 0;
}
