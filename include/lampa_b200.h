/*
 * lampa_b200 — C ABI of the B200 (sm_100a) implementation of Lampa's LSH ordering and
 * (hierarchical) chunkwise gated-delta-rule forward.
 *
 * Conventions
 *  - every pointer named q/k/v/.../ws/status is a DEVICE pointer unless stated otherwise;
 *  - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, asynchronously,
 *    and no entry point synchronises the host with the device;
 *  - the library never allocates device memory: scratch comes from the caller (`ws`), sized
 *    by the matching *_workspace_bytes call;
 *  - return value: LAMPA_OK or a negative LAMPA_ERR_* for problems found on the host before
 *    any launch; problems found on the device (a wait that ran out, not enough lambda levels
 *    for a packed sequence) are written to `status` (int32[4]: code, where, detail, unused),
 *    which the caller zeroes once and may read after synchronising the stream;
 *  - inputs are never written; layouts are the reference's token-major contiguous ones.
 *
 * "Reference" below means the Lampa repository; paths are relative to its root.
 */
#ifndef LAMPA_B200_H
#define LAMPA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
#define LAMPA_BF16 0
#define LAMPA_F16 1
#define LAMPA_F32 2
/* key types of the sort */
#define LAMPA_KEY_I32 0
#define LAMPA_KEY_F32 1

#define LAMPA_OK 0
#define LAMPA_ERR_ARG (-1)          /* null pointer, negative size, bad enum */
#define LAMPA_ERR_UNSUPPORTED (-2)  /* head dims / level count outside the built set */
#define LAMPA_ERR_WORKSPACE (-3)    /* ws too small or misaligned */
#define LAMPA_ERR_CUDA (-4)         /* a CUDA runtime call failed (launch error) */
#define LAMPA_ERR_TIMEOUT (-5)      /* device: a bounded wait ran out (status word only) */
#define LAMPA_ERR_LEVELS (-6)       /* device/host: lambda has fewer levels than the sequence needs */
#define LAMPA_ERR_BOUNDS (-7)       /* device: an index fell outside its extent (status word only) */
#define LAMPA_ERR_TOO_LARGE (-8)    /* input exceeds the fixed capacity of an allocation-free entry point */

/* Shape/type descriptor of one gated-delta forward call. */
typedef struct lampa_gdn_desc {
    int32_t B;          /* batch; must be 1 when cu_seqlens is given                         */
    int32_t T;          /* tokens per batch row (total tokens when packed)                   */
    int32_t H;          /* heads                                                             */
    int32_t K;          /* key/query head dim: 16, 32 or 64                                  */
    int32_t V;          /* value head dim:     16, 32 or 64                                  */
    int32_t L;          /* hierarchical only: number of lambda levels, else 0                */
    int32_t nseq;       /* packed input: number of sequences (len(cu_seqlens) - 1), else 0   */
    int32_t qkv_dtype;  /* LAMPA_BF16 / LAMPA_F16 / LAMPA_F32 for q, k, v and o              */
    int32_t gb_dtype;   /* type of g and beta                                                */
    int32_t lam_dtype;  /* type of lambda                                                    */
    int32_t use_l2norm; /* normalise q and k rows: x * rsqrt(sum x^2 + 1e-6)                 */
    float scale;        /* output scale of the plain rule (K^-0.5 by default in the caller)  */
} lampa_gdn_desc;

int lampa_version(void);
const char* lampa_error_string(int code);

/*
 * Bytes of scratch for lampa_gdn_fwd / lampa_hgdn_fwd with this descriptor (1024-byte aligned
 * pointer expected).  Replaces the reference's torch.empty intermediates (A, Ad, w, u, h, v_new:
 * models/hattention/gated_delta_rule_ori.py:29-80, chunkwise_hgdn.py:628-760).
 */
int lampa_gdn_workspace_bytes(const lampa_gdn_desc* d, size_t* bytes);

/*
 * Where the per-chunk intermediates live inside the workspace, for tests that inspect them.
 * One record per (chunk slot, head), chunk-major.  out[0] = byte offset of the first record,
 * out[1] = bytes per record, then byte offsets inside a record of the bf16 tiles out[2] M [K][K],
 * out[3] B^T [V][K], out[4] Q~ [64][K] (row pitch K+8 elements, except K = 64: dense 128-byte rows
 * with the 16-byte chunk index XORed with row%8), out[5] O_local (bf16 [64][V], same row layout as the other tiles),
 * out[6] chunk-level lambda (fp32 [LC][64], hierarchical only); out[7] = LC, out[8] = number of
 * chunk slots, out[9] = chunks per block, out[10] / out[11] = byte offsets of the block composites
 * and of the block entry states.
 */
int lampa_gdn_workspace_layout(const lampa_gdn_desc* d, size_t out[12]);

/*
 * Chunkwise gated-delta-rule forward.
 * Replaces: chunk_gated_delta_rule -> ChunkGatedDeltaRuleFunction.forward ->
 * chunk_gated_delta_rule_fwd (models/hattention/gated_delta_rule_ori.py:235-357, 163-202, 29-80)
 * and the Triton kernels it chains (l2norm.py:138-180, cumsum.py:386-414,
 * chunk_scaled_dot_kkt.py:74-120, solve_tril.py:221-276, wy_fast.py:192-228,
 * chunk_delta_h.py:397-441, chunk_o.py:433-469).
 *   q,k [B,T,H,K]; v,o [B,T,H,V]; g,beta [B,T,H]; h0 [N,H,K,V] fp32 or NULL;
 *   cu_seqlens int64 [nseq+1] (device) or NULL; ht [N,H,K,V] fp32 or NULL, N = nseq or B.
 */
int lampa_gdn_fwd(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                  const void* g, const void* beta, const float* h0, const int64_t* cu_seqlens,
                  void* o, float* ht, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/*
 * Hierarchical (Fenwick-level, log-linear) chunkwise gated-delta-rule forward.
 * Replaces: chunk_h_gated_delta_rule -> hattention_kernel -> HAttentionFunction.forward (GDELTA)
 * -> chunkwise_hgdn.chunkwise_fwd (models/hattention/gated_delta_rule_apis.py:20-134,
 * kernel.py:338-374, 100-120, chunkwise_hgdn.py:565-791) and its per-level re-scans
 * (fla_future/chunk_delta_h.py:34-186, chunkwise.py:473-647).
 *   lam [B,T,H,L]: weight of level(t,s) = bit_length(t XOR s) (0 on the diagonal); a sequence of
 *   NT chunks needs L >= 7 + ceil(log2(NT)).  q and k are l2-normalised when d->use_l2norm;
 *   the result does not depend on d->scale (the reference multiplies q by it and divides lam by it).
 *   Sequences (cu_seqlens) restart the hierarchy; ragged tails behave as tokens with
 *   k = v = 0, beta = 0, g = 0.
 */
int lampa_hgdn_fwd(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                   const void* g, const void* beta, const void* lam, const int64_t* cu_seqlens,
                   void* o, void* ws, size_t ws_bytes, int32_t* status, void* stream);
/*
 * The same forward with the un-ordering of a sorted event folded into the output store.
 * Replaces: the mixer call followed by the gather with the inverse permutation that puts the rows of a sorted event
 * back in hit order (models/baselines/hmamba.py:451-455), without the second pass over o.
 *   Row t of the result is written to o[out_perm[t]] for t < out_perm_rows and to o[t] beyond
 *   (the padding tokens after an event); out_perm must be a permutation of 0 .. out_perm_rows-1 for o to be fully
 *   written.  An index outside [0, B*T) is skipped and reported as LAMPA_ERR_BOUNDS in the status word.
 */
int lampa_hgdn_fwd_scatter(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                           const void* g, const void* beta, const void* lam, const int64_t* cu_seqlens,
                           const int64_t* out_perm, int64_t out_perm_rows, void* o, void* ws,
                           size_t ws_bytes, int32_t* status, void* stream);

/*
 * Fenwick state left by a hierarchical forward: call after lampa_hgdn_fwd with the same
 * descriptor, inputs, cu_seqlens and workspace (the per-chunk records and block entry states it
 * left there are read again; nothing in the workspace is changed).
 * Replaces: hattention_prefill's state half — HAttentionPrefillFunction's per-level `_ht` and
 * postprocess_prefill_hstate_ (models/hattention/kernel.py:377-560, chunkwise_hgdn.py:738-739) —
 * which the reference reaches through chunk_h_gated_delta_rule(output_final_state=True)
 * (gated_delta_rule_apis.py:87-101).
 *   states fp32 [N][H][K][V][L] (N = nseq or B): the HState.states layout of
 *   models/hattention/recurrent.py:9-40; level 0 holds the last token, level l >= 1 holds
 *   2^(l-1) tokens when bit l-1 of T-1 is set and zeros otherwise (every element is written);
 *   counts int32 [N][L]: tokens per level (all rows are equal without cu_seqlens; the reference
 *   keeps a single [L] row).  A sequence whose length is not a multiple of 64 is treated as
 *   completed by null tokens (k = v = 0, beta = 0, g = 0).
 */
int lampa_hgdn_final_state(const lampa_gdn_desc* d, const void* k, const void* v, const void* g,
                           const void* beta, const int64_t* cu_seqlens, void* ws, size_t ws_bytes,
                           float* states, int32_t* counts, int32_t* status, void* stream);
/*
 * One decode step of the hierarchical rule on a Fenwick state, in place.
 * Replaces: hattention_step -> step_state / step_output (models/hattention/kernel.py:570-633,
 * recurrent.py:134-166, HState.cascade_weak / insert / dot: recurrent.py:42-100), reached through
 * chunk_h_gated_delta_rule(initial_state=..., output_final_state=True) with T = 1
 * (gated_delta_rule_apis.py:102-127).
 *   d->T must be 1; q,k [B,H,K]; v,o [B,H,V]; g,beta [B,H]; lam [B,H,L];
 *   states fp32 [B][H][K][V][L] and counts int32 [L] (one row for the whole batch) are updated:
 *   full levels cascade upward (capacity 2^l), every level is multiplied by
 *   e^g (I - beta k k^T), level 0 becomes beta k v^T, counts[0] += 1;
 *   o = q^T sum_l lam_l S_l.  As in lampa_hgdn_fwd q and k are l2-normalised when
 *   d->use_l2norm and the result does not depend on d->scale.  A cascade that would leave the
 *   last level sets LAMPA_ERR_LEVELS in the status word and changes nothing.
 */
int lampa_hgdn_step(const lampa_gdn_desc* d, const void* q, const void* k, const void* v,
                    const void* g, const void* beta, const void* lam, float* states,
                    int32_t* counts, void* o, int32_t* status, void* stream);
/*
 * E2LSH projection and integer bucket ids.
 * Replaces: E2LSH.forward (models/model_utils/hash_utils.py:359-371; copies in
 * models/baselines/hmamba.py:275-285, full_mamba2.py:128-141) — the float projection — and adds
 * the quantisation floor((a.x + b) / w) the reference leaves out.
 *   x: fp32 rows, `row_stride` floats apart, the first `dim` floats of a row are hashed;
 *      head h reads rows at x + h * head_stride (0: all heads share the rows);
 *   alpha [heads, dim, rounds] fp32, beta [rounds] fp32 (device);
 *   ids  int32 [rounds, heads, N] or NULL;  keys fp32 [rounds, heads, N] (a.x, no offset) or NULL;
 *   packed int32 [rounds, N] = sum_h ids[r,h,n] << h or NULL.
 * Operation order (bit-exact contract): acc = x0*a0; acc = acc + xd*ad (d ascending, multiply
 * and add rounded separately); id = (int32) floorf((acc + beta) / w).
 */
int lampa_lsh_hash(const float* x, int64_t row_stride, int64_t head_stride, const float* alpha,
                   const float* beta, float w, int64_t N, int32_t heads, int32_t rounds, int32_t dim,
                   int32_t* ids, float* keys, int32_t* packed, void* stream);

/* Scratch bytes of lampa_segsort_stable for n_total keys. */
int lampa_segsort_workspace_bytes(int64_t n_total, size_t* bytes);

/*
 * Stable ascending sort of each segment's keys; writes the permutation (indices local to the
 * segment, int64 as torch.sort returns).
 * Replaces: the per-event `argsort` / `sort(stable=True)` pair of LSHOrdering.forward
 * (models/baselines/hmamba.py:335-346) and the `argsort(dim=-1)` of HEPT bucketing
 * (models/attention/hept.py:138-143).
 *   keys: int32 or fp32 [n_total]; seg_offsets int64 [nseg+1] (device) or NULL for nseg equal
 *   segments of n_total/nseg keys; init: optional starting order per segment (local indices) —
 *   the result is init composed with the stable sort of keys[init], i.e. norm_idx[bk_idx].
 *   A segment whose offsets leave [0, n_total] is not sorted and sets LAMPA_ERR_BOUNDS in `status`.
 */
int lampa_segsort_stable(const void* keys, int32_t key_type, int64_t n_total,
                         const int64_t* seg_offsets, int32_t nseg, const int64_t* init,
                         int64_t* perm, void* ws, size_t ws_bytes, int32_t* status, void* stream);

/*
 * lampa_segsort_stable for hosts that may not allocate device memory when they call it.
 * No counterpart in the reference (its sorts allocate through torch on every call).
 *
 * Who needs it: an online reconstruction / trigger-style loop that reserves all of its device
 * memory at start-up and forbids cudaMalloc afterwards (it synchronises the device and can fail
 * late), or a host process whose device memory belongs to an allocator this library cannot reach,
 * so that it has no workspace pointer to hand over.  Same arguments and results as
 * lampa_segsort_stable minus `ws`: the ping-pong buffers are a fixed array inside the library
 * image, 16 bytes x LAMPA_SEGSORT_STATIC_MAX_KEYS = 24 MiB, resident on every GPU that loads the
 * library until the process exits.
 *   - n_total > LAMPA_SEGSORT_STATIC_MAX_KEYS returns LAMPA_ERR_TOO_LARGE and launches nothing;
 *   - neither this call nor anything it uses calls cudaMalloc/cudaFree or an allocating routine;
 *   - the first call on a device looks up the array's address there (cudaGetSymbolAddress, with
 *     that device current) and caches it.  Make that first call part of start-up: outside any
 *     stream capture, and because it may also be the call that loads this library's device code
 *     (with the 24 MiB array) onto the GPU when the CUDA runtime loads modules lazily;
 *   - the cached address belongs to the device's current primary context: after a
 *     cudaDeviceReset in the host process it is stale and this entry point must not be used again
 *     in that process;
 *   - all calls on a device share the one array and it keeps the previous call's contents; the
 *     sort never reads what it has not just written, so nothing is cleared, but two calls that
 *     overlap on the GPU (different streams, or threads without ordering) race on it: keep
 *     calls on one stream or order them with events.
 */
#define LAMPA_SEGSORT_STATIC_MAX_KEYS 1572864
int lampa_segsort_stable_static(const void* keys, int32_t key_type, int64_t n_total,
                                const int64_t* seg_offsets, int32_t nseg, const int64_t* init,
                                int64_t* perm, int32_t* status, void* stream);

/*
 * Row gather / scatter by a per-segment permutation.
 * Replaces: points.gather (hmamba.py:348-351), sort_to_buckets / unsort_from_buckets /
 * batched_index_select (models/attention/hept.py:9-19, hash_utils.py:83-93).
 *   scatter == 0: dst[s0+i] = src[s0+perm[s0+i]];  scatter != 0: dst[s0+perm[s0+i]] = src[s0+i].
 *   row_bytes must be a multiple of 4.  An index outside its segment is not followed: that row is
 *   skipped and LAMPA_ERR_BOUNDS goes to `status` (may be NULL).
 */
int lampa_permute_rows(const void* src, const int64_t* perm, const int64_t* seg_offsets, int32_t nseg,
                       int64_t n_rows, int64_t row_bytes, int32_t scatter, void* dst, int32_t* status,
                       void* stream);

/* inv[s0 + perm[s0+i]] = i.  Replaces invert_permutation (hash_utils.py:46-57) and the
 * `perm.argsort(dim=1)` used to undo the ordering (hmamba.py:451, full_mamba2.py:678).  Entries
 * outside their segment are skipped and reported as LAMPA_ERR_BOUNDS in `status` (may be NULL). */
int lampa_invert_perm(const int64_t* perm, const int64_t* seg_offsets, int32_t nseg, int64_t n_total,
                      int64_t* inv, int32_t* status, void* stream);

/*
 * Per-row range of the LSH projections: mn/mx/range [rows] fp32 (any may be NULL) over the n
 * values of each row of a and, when b is given, of b as well; range = max - min.
 * Replaces: the four max/min reductions of lsh_mapping / lsh_mapping1
 * (models/model_utils/hash_utils.py:333-355, copy in models/baselines/hmamba.py:253-272), whose
 * `hash_shift` is the region stride of the geo shift.
 */
int lampa_row_range(const float* a, const float* b, int32_t rows, int64_t n, float* mn, float* mx,
                    float* range, void* stream);
/*
 * Quantile regions of one coordinate.  rank int64 [n]: position of each hit in the ascending
 * order of the coordinate (the inverse of the reference's argsort, lampa_invert_perm of a
 * lampa_segsort_stable result); num_regions fp32 [rows] (fractional region counts per
 * (round, head) row).  out fp32 [rows][n] = floor(rank / ceil(n / num_regions[r])) + 1.
 * Replaces: quantile_partition (models/model_utils/hash_utils.py:14-27) as called by
 * prepare_input (models/hattention/modeling_gated_deltaproduct.py:1214-1219, models/rwkv/RWKV.py:61-66).
 */
int lampa_quantile_regions(const int64_t* rank, const float* num_regions, int32_t rows, int64_t n,
                           float* out, void* stream);
/*
 * Region shift and shifted sort keys, fp32 [rows][n]:
 *   shift = (reg_phi * hash_shift[r]) * (ceil(regions_eta[r]) + 1) + reg_eta * hash_shift[r]
 *   out   = shift                          when proj is NULL   (get_geo_shift)
 *   out   = (i < raw_size ? proj : +inf) + shift   otherwise   (the keys HEPT sorts)
 * every product and sum rounded separately, in this order.  The regions come either from
 * reg_eta / reg_phi (fp32 [rows][n], lampa_quantile_regions output) or, when those are NULL,
 * straight from rank_eta / rank_phi (int64 [n]) and regions_phi, without materialising them.
 * Replaces: get_geo_shift and the `hashed[..., raw_size:] = inf; hashed + shifts` statements of
 * HEPTAttention.forward (models/attention/hept.py:78-88, 127-136; copy in
 * models/baselines/hmamba.py:76-90).
 */
int lampa_geo_keys(const float* proj, const float* reg_eta, const float* reg_phi,
                   const int64_t* rank_eta, const int64_t* rank_phi, const float* regions_eta,
                   const float* regions_phi, const float* hash_shift, int32_t rows, int64_t n,
                   int64_t raw_size, float* out, void* stream);
/*
 * Short causal depthwise convolution with optional SiLU on a projection, token-major.
 * Replaces: ShortConvolution.forward's prefill path -> causal_conv1d_fwd (+ the final-state copies)
 * (models/hattention/short_convolution.py:595-680, 39-112, 256-291, 484-525).
 *   x, y, residual (or NULL): [B, T, D] of `dtype`; weight [D, W] and bias [D] (or NULL) of `w_dtype`;
 *   W <= 8; D a multiple of 4; cu_seqlens int64 [nseq+1] on the device with B == 1, or
 *   NULL / nseq = 0;  y[t, d] = act(bias[d] + sum_i weight[d, i] x[t - (W-1) + i, d]) + residual, taps
 *   before the start of the token's sequence read as zero, accumulated in fp32 oldest tap first.
 *   final_state (or NULL): [N, D, W] of `dtype`, slot w = x[eos - W + w, d]; slots before the
 *   sequence start are zeroed when zero_fill != 0 (the reference's packed path) and left as they
 *   are otherwise (its in-place update of an existing cache).
 */
int lampa_short_conv_fwd(const void* x, const void* weight, const void* bias, const void* residual,
                         const int64_t* cu_seqlens, int32_t nseq, int64_t B, int64_t T, int32_t D,
                         int32_t W, int32_t dtype, int32_t w_dtype, int32_t silu, void* y,
                         void* final_state, int32_t zero_fill, void* stream);
/*
 * Decode step of the same convolution: cache [N, D, W] moves one slot left and takes x [N, D] in
 * its last slot (in place); y = act(bias + sum_w cache[n, d, w] weight[d, w]) + residual.
 * Replaces: ShortConvolution.step -> causal_conv1d_update (short_convolution.py:682-717, 203-253, 357-389).
 */
int lampa_short_conv_step(const void* x, void* cache, const void* weight, const void* bias,
                          const void* residual, int64_t N, int32_t D, int32_t W, int32_t dtype,
                          int32_t w_dtype, int32_t silu, void* y, void* stream);
/*
 * Gate inputs of the hierarchical gated-delta layer from its projections:
 *   g [n_tok, H] fp32 = -exp(A_log[h]) softplus(a + dt_bias[h]);  beta [n_tok, H] = sigmoid(b);
 *   lam [n_tok, H, L] = softplus(Lw[h,l] dl) (lambda_mode 0, "positive"), exp(-exp(Lw) softplus(dl))
 *   (1, "bounded") or Lw dl (2, default); each times mask[n_tok] (fp32 0/1) when mask is given.
 *   a, b [n_tok, H] and dl [n_tok, H, L] of `in_dtype`; A_log, dt_bias [H], Lw [H, L] fp32.
 *   Any of g / beta / lam may be NULL to skip it.
 * Replaces: models/hattention/modeling_h_gated_deltanet.py:429-450 and compute_lambda (151-166).
 */
int lampa_gate_inputs(const void* a, const void* b, const void* dl, const float* A_log,
                      const float* dt_bias, const float* Lw, const float* mask, int64_t n_tok,
                      int32_t H, int32_t L, int32_t in_dtype, int32_t beta_dtype, int32_t lam_dtype,
                      int32_t lambda_mode, float* g, void* beta, void* lam, void* stream);
/*
 * Gated RMS norm over rows of D (the mixer's output norm, one row per token and head):
 *   y = x / sqrt(mean(x^2) + eps) * weight * g * sigmoid(g)     (sigmoid_only: ... * sigmoid(g))
 *   x, g, y [rows, D] of `dtype`, weight [D] of `w_dtype` or NULL; D a multiple of 8 (4 for fp32),
 *   at most 1024 (512 for fp32).
 * Replaces: FusedRMSNormGated.forward -> rms_norm_gated -> layer_norm_gated_fwd_kernel
 * (models/hattention/fused_norm.py:1003-1064, 858-880, 40-112) without residual / prenorm.
 */
int lampa_rmsnorm_gate(const void* x, const void* g, const void* weight, int64_t rows, int32_t D,
                       int32_t dtype, int32_t w_dtype, float eps, int32_t sigmoid_only, void* y,
                       void* stream);
/*
 * Residual add + RMS norm of a block's fp32 residual stream, with the ordering layer's row
 * permutation folded in.  For every j in [0, rows): r = s0 + perm[s0 + j'] (perm: int64 indices
 * local to the row's segment, as lampa_segsort_stable writes them; r = j when perm is NULL);
 *   v = res[r] + delta[delta_at_r ? r : j]   (delta NULL: v = res[r], res is left untouched)
 *   res[r] = v                                (fp32, in place)
 *   y[y_at_r ? r : j] = v / sqrt(mean(v^2) + eps) * weight    (y NULL: the add only)
 * so the un-ordering of a mixer's output (delta in sorted order, delta_at_r = 0, y_at_r = 1) and the
 * ordering of the next mixer's input (delta_at_r = 1, y_at_r = 0) cost no pass of their own.
 * res [rows, D] fp32; delta, y [rows, D] of their dtypes; weight [D] fp32 or NULL; D a multiple of 4,
 * at most 1024.  An index outside its segment skips the row and sets LAMPA_ERR_BOUNDS in `status`.
 * Replaces: RMSNorm.forward(x, residual, prenorm=True) (models/hattention/fused_norm.py:1288-1330,
 * 1413-1425, as used by the block at modeling_gated_deltaproduct.py:1169-1199) together with the
 * gather / un-gather around the mixer (models/baselines/hmamba.py:428-455).
 */
int lampa_add_rmsnorm(float* res, const void* delta, int32_t delta_dtype, const int64_t* perm,
                      const int64_t* seg_offsets, int32_t nseg, int64_t rows, int32_t D,
                      const float* weight, float eps, int32_t delta_at_r, int32_t y_at_r, void* y,
                      int32_t y_dtype, int32_t* status, void* stream);
/*
 * Bucketed RBF-kernel attention of the HEPT layer, fp32.  Per (round, head) the n hits are taken in
 * the order q_pos / k_pos (int64 [rounds][heads][n]; NULL: rows are already in order), cut into
 * buckets of `bucket` consecutive hits (n % bucket == 0, bucket <= 128), and inside a bucket
 *   p_ij = exp(min(0, q_i.k_j - |q_i|^2/2 - |k_j|^2/2)),  denom_i = sum_j p_ij + 1e-20,
 *   so_i = sum_j p_ij v_j.
 * q, k: [heads][n] rows of dq floats, ldq floats apart; v: [heads][n] rows of dv floats, ldv apart;
 * shared by all rounds and gathered by position; with inputs_per_round != 0 they carry a leading
 * [rounds] axis (rows pre-sorted per round).  Rows are fetched as 16-byte pieces when the base is
 * 16-byte aligned and the pitch is a multiple of 4 and at least the width rounded up to 4; the
 * padding columns of such rows are read and must be zero (lampa_hept_prep_qk writes them so).
 * so [rounds][heads][n][dv] and denom [rounds][heads][n]: row i of a bucket is written at its
 * sorted place (scatter == 0: the outputs of qkv_res) or at hit q_pos[i] (scatter != 0: after
 * unsort_from_buckets with the inverse permutation).  dv <= 128; shared memory bounds dq
 * (LAMPA_ERR_UNSUPPORTED beyond).
 * Replaces: qkv_res (models/attention/hept.py:22-33) and, with positions, the sort_to_buckets /
 * unsort_from_buckets calls around it in HEPTAttention.forward (hept.py:141-150).
 */
int lampa_bucket_rbf_attn(const float* q, const float* k, const float* v, const int64_t* q_pos,
                          const int64_t* k_pos, int32_t rounds, int32_t heads, int64_t n, int32_t bucket,
                          int32_t dq, int32_t dv, int32_t ldq, int32_t ldv, int32_t inputs_per_round,
                          int32_t scatter, float* so, float* denom, void* stream);
/*
 * out[row][:] = (sum over rounds of so[r][row][:]) / (sum over rounds of denom[r][row]), rounds added
 * in order.  rows = heads * n.  Replaces: `o.sum(dim=0) / logits.sum(dim=0)` (hept.py:151).
 */
int lampa_bucket_attn_combine(const float* so, const float* denom, int32_t rounds, int64_t rows,
                              int32_t dv, float* out, void* stream);
/*
 * Inputs of the bucket attention from the layer's projections: query, key, value [n][heads][d]
 * (token-major), coords [n][cd], scale [heads][cd] (= sqrt(2 * per-head coordinate weights));
 * q_hat = k_hat's coordinate part = scale * coords, appended to query / key; outputs head-major
 * q_hat, k_hat [heads][n] rows of d + cd floats, ldq >= d + cd floats apart, the padding columns
 * zero; v_out [heads][n][d] (may be NULL); rows >= raw_size zeroed.
 * Replaces: the elementwise part of prep_qk and the rearrange / zero-padding statements of
 * HEPTAttention.forward (hept.py:55-63, 121-126).
 */
int lampa_hept_prep_qk(const float* query, const float* key, const float* value, const float* scale,
                       const float* coords, int64_t n, int32_t heads, int32_t d, int32_t cd,
                       int32_t ldq, int64_t raw_size, float* q_hat, float* k_hat, float* v_out,
                       void* stream);
/*
 * Per-kernel timing for benchmarks (no counterpart in the reference, which has no timing code).
 * lampa_profile_enable(1) makes every later launch of this library record a pair of CUDA events
 * on its stream; lampa_profile_enable(0) stops and clears.  lampa_profile_read synchronises on
 * the recorded events and returns, per kernel name ('\n'-separated in `names`), the summed
 * milliseconds and the number of launches.  Host-side only; not for concurrent use.
 */
int lampa_profile_enable(int on);
int lampa_profile_read(char* names, size_t names_cap, float* total_ms, int32_t* launches,
                       int32_t max_kernels, int32_t* n_kernels);

/*
 * Test hook (no counterpart in the reference): number of polls after which a device-side wait of
 * the gated-delta kernels gives up (default and maximum 2^22).  A test sets it to 0 to see the
 * give-up path without anything hanging: the kernels then return at once, results are undefined
 * and LAMPA_ERR_TIMEOUT is in the status word; copies and MMAs already in flight are still waited
 * for with the full budget before a CTA exits.  Process-wide; not for concurrent use.
 */
int lampa_debug_set_poll_budget(int polls);
/*
 * Test hook (no counterpart in the reference): on = 1 routes the K = V = 64 gated-delta calls that follow to the
 * mma.sync kernels instead of the tcgen05 ones (what LAMPA_B200_NO_UMMA=1 does for a whole process), on = 0 back;
 * lets a test compare the two tensor-core paths on the same input.  Process-wide; not for concurrent use.
 */
int lampa_debug_force_mma_sync(int on);
/*
 * Tuning hook (no counterpart in the reference): with a device buffer of n_ctas x 16 int64, thread 0
 * of the first n_ctas CTAs of the tcgen05 preparation kernel stores clock64() at its stage boundaries
 * (slots 0..10, slot 0 = start), the SM it ran on (slot 11) and the global nanosecond timer at its start
 * and end (slots 12, 13).  n_ctas = 0 switches it off (the default).  Process-wide; the buffer must
 * stay allocated while it is set.
 */
int lampa_debug_set_tick_buffer(long long* ticks, int n_ctas);

#ifdef __cplusplus
}
#endif
#endif /* LAMPA_B200_H */
