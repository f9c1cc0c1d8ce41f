// Shared device/host helpers for the sm_100a kernels of the LSH + gated-delta path.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/lampa_b200.h"

namespace lampa {

constexpr int CHUNK = 64;          // tokens per chunk (the reference's BT, gated_delta_rule_ori.py:41)
constexpr int ELL0 = 7;            // intra-chunk levels 0..6 (get_num_levels(64, 2), base.py:37-38)

// ---- status word (device int32[4]): [0] code, [1] where, [2..3] detail -----------------------
__device__ __forceinline__ void set_status(int32_t* status, int code, int where, int detail) {
    if (status != nullptr && atomicCAS(status, 0, code) == 0) {
        status[1] = where;
        status[2] = detail;
    }
}

// ---- small numeric helpers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);     // .x = lo (low 16 bits), .y = hi
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
}
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// dtype codes of the C ABI
template <int DT> struct Elem;
template <> struct Elem<LAMPA_BF16> {
    using T = __nv_bfloat16;
    static __device__ __forceinline__ float ld(const void* p, size_t i) { return __bfloat162float(((const T*)p)[i]); }
    static __device__ __forceinline__ void st(void* p, size_t i, float v) { ((T*)p)[i] = __float2bfloat16_rn(v); }
};
template <> struct Elem<LAMPA_F16> {
    using T = __half;
    static __device__ __forceinline__ float ld(const void* p, size_t i) { return __half2float(((const T*)p)[i]); }
    static __device__ __forceinline__ void st(void* p, size_t i, float v) { ((T*)p)[i] = __float2half_rn(v); }
};
template <> struct Elem<LAMPA_F32> {
    using T = float;
    static __device__ __forceinline__ float ld(const void* p, size_t i) { return ((const T*)p)[i]; }
    static __device__ __forceinline__ void st(void* p, size_t i, float v) { ((T*)p)[i] = v; }
};
__device__ __forceinline__ float load_as_float(const void* p, size_t i, int dt) {
    if (dt == LAMPA_BF16) return Elem<LAMPA_BF16>::ld(p, i);
    if (dt == LAMPA_F16) return Elem<LAMPA_F16>::ld(p, i);
    return Elem<LAMPA_F32>::ld(p, i);
}
__device__ __forceinline__ void store_from_float(void* p, size_t i, float v, int dt) {
    if (dt == LAMPA_BF16) Elem<LAMPA_BF16>::st(p, i, v);
    else if (dt == LAMPA_F16) Elem<LAMPA_F16>::st(p, i, v);
    else Elem<LAMPA_F32>::st(p, i, v);
}
__host__ __device__ __forceinline__ int dtype_bytes(int dt) { return dt == LAMPA_F32 ? 4 : 2; }

// ---- warp-level tensor-core primitives (bf16 in, fp32 accumulate) ------------------------------
// D(16x8) += A(16x16, row) * B(16x8, col).  Fragment ownership (g = lane/4, t = lane%4):
//   a0:(g, 2t..2t+1) a1:(g+8, 2t..) a2:(g, 2t+8..) a3:(g+8, 2t+8..)
//   b0:(k=2t..2t+1, n=g) b1:(k=2t+8.., n=g)      c0,c1:(g, 2t..2t+1) c2,c3:(g+8, 2t..2t+1)
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr) : "memory");
}

// A fragment (16 rows m0.., 16 k-columns k0..) from row-major smem A[m][k] (pitch lda elements).
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const __nv_bfloat16* s, int lda, int m0, int k0, int lane) {
    const int mi = lane >> 3, r = lane & 7;
    ldsm_x4(a, smem_u32(s + (size_t)(m0 + r + (mi & 1) * 8) * lda + k0 + (mi >> 1) * 8));
}
// A fragment when smem holds A transposed: At[k][m] (pitch lda).
__device__ __forceinline__ void load_a_t(uint32_t (&a)[4], const __nv_bfloat16* s, int lda, int m0, int k0, int lane) {
    const int mi = lane >> 3, r = lane & 7;
    ldsm_x4_t(a, smem_u32(s + (size_t)(k0 + r + (mi >> 1) * 8) * lda + m0 + (mi & 1) * 8));
}
// B fragments for two adjacent n-tiles (n0..n0+15) and one k-step (k0..k0+15), smem holds Bt[n][k]
// (n rows, k contiguous).  b[0],b[1] = (b0,b1) of n-tile n0; b[2],b[3] = n-tile n0+8.
__device__ __forceinline__ void load_b(uint32_t (&b)[4], const __nv_bfloat16* s, int ldb, int n0, int k0, int lane) {
    const int mi = lane >> 3, r = lane & 7;
    ldsm_x4(b, smem_u32(s + (size_t)(n0 + r + (mi >> 1) * 8) * ldb + k0 + (mi & 1) * 8));
}
// Same fragments when smem holds B[k][n] (k rows, n contiguous).
__device__ __forceinline__ void load_b_t(uint32_t (&b)[4], const __nv_bfloat16* s, int ldb, int n0, int k0, int lane) {
    const int mi = lane >> 3, r = lane & 7;
    ldsm_x4_t(b, smem_u32(s + (size_t)(k0 + r + (mi & 1) * 8) * ldb + n0 + (mi >> 1) * 8));
}

// acc[NT8][4] (16 x 8*NT8) += A[m0:m0+16, 0:k_end) * B[0:k_end, n0:n0+n_end)
// k_end / n_end (warp-uniform, multiples of 16) cut the loops short for triangular operands.
template <int NT8, int KDIM, bool A_T, bool B_T>
__device__ __forceinline__ void warp_gemm(float (&acc)[NT8][4], const __nv_bfloat16* sA, int lda, int m0,
                                          const __nv_bfloat16* sB, int ldb, int n0, int lane,
                                          int k_end = KDIM, int n_end = NT8 * 8) {
    static_assert(NT8 % 2 == 0 && KDIM % 16 == 0, "tile shape");
#pragma unroll
    for (int k0 = 0; k0 < KDIM; k0 += 16) {
        if (k0 < k_end) {
            uint32_t a[4];
            if (A_T) load_a_t(a, sA, lda, m0, k0, lane); else load_a(a, sA, lda, m0, k0, lane);
#pragma unroll
            for (int nt = 0; nt < NT8; nt += 2) {
                if (nt * 8 < n_end) {
                    uint32_t b[4];
                    if (B_T) load_b_t(b, sB, ldb, n0 + nt * 8, k0, lane); else load_b(b, sB, ldb, n0 + nt * 8, k0, lane);
                    mma16816(acc[nt], a, b[0], b[1]);
                    mma16816(acc[nt + 1], a, b[2], b[3]);
                }
            }
        }
    }
}

// Same with the A operand already in registers: afrag[kk] is the A fragment of k-step kk (for a
// 16-row tile held as accumulators C[nt][4], afrag[kk] = {pack(C[2kk][0..1]), pack(C[2kk][2..3]),
// pack(C[2kk+1][0..1]), pack(C[2kk+1][2..3])}).
template <int NT8, int KSTEPS, bool B_T>
__device__ __forceinline__ void warp_gemm_ra(float (&acc)[NT8][4], const uint32_t (&afrag)[KSTEPS][4],
                                             const __nv_bfloat16* sB, int ldb, int n0, int lane,
                                             int k_end = KSTEPS * 16, int n_end = NT8 * 8) {
    static_assert(NT8 % 2 == 0, "tile shape");
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
        if (kk * 16 < k_end) {
#pragma unroll
            for (int nt = 0; nt < NT8; nt += 2) {
                if (nt * 8 < n_end) {
                    uint32_t b[4];
                    if (B_T) load_b_t(b, sB, ldb, n0 + nt * 8, kk * 16, lane); else load_b(b, sB, ldb, n0 + nt * 8, kk * 16, lane);
                    mma16816(acc[nt], afrag[kk], b[0], b[1]);
                    mma16816(acc[nt + 1], afrag[kk], b[2], b[3]);
                }
            }
        }
    }
}

// ---- mbarrier + bulk async copy (TMA, untiled form) -------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" :: "r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `budget` polls (each poll may itself block for a while in hardware;
// the default budget is 2^22), records the failure and lets the caller carry on so that no barrier
// is left unbalanced.  A thread that has given up once (`dead`) does not wait again: it runs to the
// end of its loop, issues nothing new and drains what it has in flight with mbar_drain.
constexpr int MBAR_POLLS = 1 << 22;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, bool& dead, int32_t* status, int where,
                                          int budget = MBAR_POLLS) {
    if (dead) return false;
    for (int i = 0; i < budget; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    dead = true;
    set_status(status, LAMPA_ERR_TIMEOUT, where, (int)parity);
    return false;
}
// Wait for an asynchronous operation that was already started (a bulk copy into this CTA's shared
// memory, a committed MMA group) before the CTA gives its shared / tensor memory back; always the
// full budget, whatever made the thread give up earlier.
__device__ __forceinline__ bool mbar_drain(uint64_t* bar, uint32_t parity) {
    for (int i = 0; i < MBAR_POLLS; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// global -> shared bulk copy; dst/src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 :: "r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// shared -> global bulk copy (same alignment rules).  The writer threads make their shared-memory
// stores visible to the async proxy first (fence_async_shared, then a barrier); the issuing thread
// commits the group and, before the buffer is reused or the CTA exits, waits until it has been read.
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;\n"
                 :: "l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;\n" ::: "memory"); }

// ---- sequence plan (device ints, built once per call from cu_seqlens) ---------------------------
struct SeqPlan {
    const int64_t* tok_off;    // [nseq+1] token offsets
    const int32_t* chunk_off;  // [nseq+1] exclusive prefix of ceil(len/64)
    const int32_t* block_off;  // [nseq+1] exclusive prefix of ceil(chunks/BC)
    int nseq;
};
// index of the sequence whose [off[s], off[s+1]) contains x (off non-decreasing; empty ranges skipped)
__device__ __forceinline__ int find_seq(const int32_t* off, int nseq, int x) {
    int lo = 0, hi = nseq;            // invariant: off[lo] <= x < off[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (off[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}

}  // namespace lampa
