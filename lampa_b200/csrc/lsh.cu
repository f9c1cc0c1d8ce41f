// E2LSH hashing, segmented stable radix sort, row permutation: the ordering half of the path.
// All kernels are HBM/L2-bound integer and byte work; no tensor cores here by design.
#include <cooperative_groups.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "profile.cuh"

namespace cg = cooperative_groups;

namespace lampa {

// -------------------------------------------------------------------------------------------------
// Hash: one thread per hit.  Reads dim floats of the hit's row (for the detector rows of this
// workload 24 B of a 96 B row: one 32 B sector) and writes rounds*heads ids, each coalesced across
// the warp.  The operation order is a contract shared with the CPU checker (see the header).
// -------------------------------------------------------------------------------------------------
constexpr int HASH_THREADS = 256;
constexpr int HASH_MAX_PARAMS = 4096;   // heads*dim*rounds floats staged in shared memory

template <int DIMT>   // DIMT > 0: coordinates kept in registers (dim == DIMT, shared rows)
__global__ void __launch_bounds__(HASH_THREADS)
lsh_hash_kernel(const float* __restrict__ x, int64_t row_stride, int64_t head_stride,
                const float* __restrict__ alpha, const float* __restrict__ beta, float w, int64_t N,
                int heads, int rounds, int dim, int32_t* __restrict__ ids, float* __restrict__ keys,
                int32_t* __restrict__ packed) {
    __shared__ float s_alpha[HASH_MAX_PARAMS];
    __shared__ float s_beta[64];
    const int np = heads * dim * rounds;
    for (int i = threadIdx.x; i < np; i += HASH_THREADS) s_alpha[i] = alpha[i];
    for (int i = threadIdx.x; i < rounds; i += HASH_THREADS) s_beta[i] = beta[i];
    __syncthreads();
    const int64_t n = (int64_t)blockIdx.x * HASH_THREADS + threadIdx.x;
    if (n >= N) return;
    float xv[DIMT > 0 ? DIMT : 1];
    if (DIMT > 0) {
#pragma unroll
        for (int d = 0; d < DIMT; ++d) xv[d] = __ldg(x + n * row_stride + d);
    }
    for (int c = 0; c < rounds; ++c) {
        int32_t pk = 0;
        for (int h = 0; h < heads; ++h) {
            const float* a = s_alpha + (size_t)h * dim * rounds + c;   // a[d*rounds]
            float acc;
            if (DIMT > 0) {
                acc = __fmul_rn(xv[0], a[0]);
#pragma unroll
                for (int d = 1; d < DIMT; ++d) acc = __fadd_rn(acc, __fmul_rn(xv[d], a[d * rounds]));
            } else {
                const float* xr = x + h * head_stride + n * row_stride;
                acc = __fmul_rn(__ldg(xr), a[0]);
                for (int d = 1; d < dim; ++d) acc = __fadd_rn(acc, __fmul_rn(__ldg(xr + d), a[d * rounds]));
            }
            const size_t o = ((size_t)c * heads + h) * N + n;
            if (keys) keys[o] = acc;
            if (ids || packed) {
                const int32_t id = (int32_t)floorf(__fdiv_rn(__fadd_rn(acc, s_beta[c]), w));
                if (ids) ids[o] = id;
                pk += (int32_t)((uint32_t)id << h);
            }
        }
        if (packed) packed[(size_t)c * N + n] = pk;
    }
}

// -------------------------------------------------------------------------------------------------
// Segmented stable LSD radix sort.  One thread-block cluster (up to 8 CTAs) per segment: each CTA
// owns a contiguous slice of the segment in its current order, digit histograms are exchanged
// through distributed shared memory, and the passes are separated by the hardware cluster barrier
// (no flag spinning anywhere).  The cluster size is the largest one for which the occupancy
// calculator reports all clusters resident at once: a cluster lives inside one GPC, and a size that
// merely divides the SM count left a third of the clusters waiting for a second wave (103 us
// against 57 us for the 24 x 60 000 keys of the benchmark).  Keys are reduced to (key - min) first,
// so only ceil(bits(range)/8) passes run: two for the ~15-bit bucket ids of this workload.  A CTA
// keeps its slice of the current pass in shared memory when it fits (filled by the histogram sweep,
// read back by the scatter) and walks it in tiles of 4096 keys; a warp takes 128 consecutive keys
// as four rounds of 32, ranking each round with ballots on top of a per-warp digit histogram, so
// the order (round, lane) is the key order and the sort is stable.
// -------------------------------------------------------------------------------------------------
constexpr int SORT_THREADS = 1024;
constexpr int SORT_MAX_CL = 8;
constexpr int SORT_WARPS = SORT_THREADS / 32;
constexpr int SORT_ITEMS = 4;
constexpr int SORT_TILE = SORT_THREADS * SORT_ITEMS;

__device__ __forceinline__ uint32_t key_xform(const void* keys, int key_type, int64_t i) {
    uint32_t u = ((const uint32_t*)keys)[i];
    if (key_type == LAMPA_KEY_I32) return u ^ 0x80000000u;
    // float: order-preserving map; -0.0 and +0.0 compare equal in torch.sort, so fold -0 onto +0
    if (u == 0x80000000u) u = 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__global__ void __launch_bounds__(SORT_THREADS, 1)
segsort_kernel(const void* __restrict__ keys, int key_type, int64_t n_total,
               const int64_t* __restrict__ seg, int nseg, const int64_t* __restrict__ init,
               int64_t* __restrict__ perm, uint32_t* kbuf0, uint32_t* kbuf1, uint32_t* ibuf0,
               uint32_t* ibuf1, int cache_cap, int32_t* status) {
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int ncl = (int)cluster.num_blocks();
    const int s = blockIdx.x / ncl;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    int64_t s0, n;
    if (seg) { s0 = seg[s]; n = seg[s + 1] - s0; }
    else { n = n_total / nseg; s0 = (int64_t)s * n; }
    if (n < 0 || s0 < 0 || s0 + n > n_total) {   // offsets that leave the key array: sort nothing, say so
        if (tid == 0 && rank == 0) set_status(status, LAMPA_ERR_BOUNDS, 12, s);
        n = 0;
    }
    const int64_t per = (n + ncl - 1) / ncl;
    const int64_t lo = min((int64_t)rank * per, n), hi = min(lo + per, n);

    __shared__ uint32_t hist[256];
    __shared__ uint32_t dbase[256];
    __shared__ uint32_t tile_tot[256];
    __shared__ uint32_t wtot[8];
    __shared__ uint32_t red[2];
    __shared__ uint32_t wcount[SORT_WARPS][257];   // +1: a column (one digit across the warps) is conflict-free
    __shared__ uint32_t tstart[256];
    extern __shared__ uint32_t sort_dyn[];         // [SORT_TILE] keys, [SORT_TILE] indices of the tile, grouped by digit
    uint32_t* skey = sort_dyn;
    uint32_t* sidx = sort_dyn + SORT_TILE;
    // the CTA's slice (keys and indices of the current pass) stays in shared memory when it fits:
    // the histogram sweep fills it and the scatter reads it back instead of going to L2 again
    uint32_t* ckey = sort_dyn + 2 * SORT_TILE;
    uint32_t* cidx = ckey + cache_cap;
    const bool cached = (hi - lo) <= (int64_t)cache_cap;

    // ---- key range over the whole segment -------------------------------------------------------
    if (tid == 0) { red[0] = 0xFFFFFFFFu; red[1] = 0u; }
    __syncthreads();
    {
        uint32_t mn = 0xFFFFFFFFu, mx = 0u;
        if (cached) {   // position i holds element init[i]; four independent loads in flight per thread
            for (int64_t i0 = lo + tid; i0 < hi; i0 += 4 * SORT_THREADS) {
                uint32_t ix[4], u[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int64_t i = i0 + (int64_t)q * SORT_THREADS;
                    ix[q] = i < hi ? (init ? (uint32_t)init[s0 + i] : (uint32_t)i) : 0u;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int64_t i = i0 + (int64_t)q * SORT_THREADS;
                    u[q] = i < hi ? key_xform(keys, key_type, s0 + ix[q]) : 0u;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int64_t i = i0 + (int64_t)q * SORT_THREADS;
                    if (i < hi) { ckey[i - lo] = u[q]; cidx[i - lo] = ix[q]; mn = min(mn, u[q]); mx = max(mx, u[q]); }
                }
            }
        } else {
            for (int64_t i = lo + tid; i < hi; i += SORT_THREADS) {
                const uint32_t u = key_xform(keys, key_type, s0 + i);
                mn = min(mn, u); mx = max(mx, u);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
            mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        if (lane == 0) { atomicMin(&red[0], mn); atomicMax(&red[1], mx); }
    }
    __syncthreads();
    cluster.sync();
    uint32_t gmn = 0xFFFFFFFFu, gmx = 0u;
    for (int r = 0; r < ncl; ++r) {
        const uint32_t* rr = cluster.map_shared_rank(red, r);
        gmn = min(gmn, rr[0]); gmx = max(gmx, rr[1]);
    }
    const uint32_t range = (n > 0 && gmx >= gmn) ? (gmx - gmn) : 0u;
    const int bits = range ? (32 - __clz(range)) : 0;
    const int npass = (bits + 7) / 8;

    if (npass == 0) {
        for (int64_t i = lo + tid; i < hi; i += SORT_THREADS) perm[s0 + i] = init ? init[s0 + i] : i;
    }

    for (int p = 0; p < npass; ++p) {
        const int shift = 8 * p;
        const uint32_t* ksrc = (p & 1) ? kbuf0 : kbuf1;   // pass p reads what pass p-1 wrote
        const uint32_t* isrc = (p & 1) ? ibuf0 : ibuf1;
        uint32_t* kdst = (p & 1) ? kbuf1 : kbuf0;
        uint32_t* idst = (p & 1) ? ibuf1 : ibuf0;
        const bool last = (p == npass - 1);

        // (a) digit histogram of this CTA's slice
        for (int d = tid; d < 256; d += SORT_THREADS) hist[d] = 0;
        __syncthreads();
        if (cached) {
            for (int64_t i0 = lo + tid; i0 < hi; i0 += 4 * SORT_THREADS) {
                uint32_t u[4], ix[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int64_t i = i0 + (int64_t)q * SORT_THREADS;
                    u[q] = 0u; ix[q] = 0u;
                    if (i < hi) {
                        if (p == 0) u[q] = ckey[i - lo] - gmn;
                        else { u[q] = ksrc[s0 + i]; ix[q] = isrc[s0 + i]; }
                    }
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const int64_t i = i0 + (int64_t)q * SORT_THREADS;
                    if (i < hi) {
                        ckey[i - lo] = u[q];
                        if (p > 0) cidx[i - lo] = ix[q];
                        atomicAdd(&hist[(u[q] >> shift) & 255u], 1u);
                    }
                }
            }
        } else {
            for (int64_t i = lo + tid; i < hi; i += SORT_THREADS) {
                uint32_t u;
                if (p == 0) u = key_xform(keys, key_type, s0 + (init ? init[s0 + i] : i)) - gmn;   // position i holds element init[i]
                else u = ksrc[s0 + i];
                atomicAdd(&hist[(u >> shift) & 255u], 1u);
            }
        }
        __syncthreads();
        cluster.sync();

        // (b) where each digit of this slice starts in the segment
        uint32_t tot = 0, before = 0, incl = 0;
        if (tid < 256) {
            for (int r = 0; r < ncl; ++r) {
                const uint32_t hv = cluster.map_shared_rank(hist, r)[tid];
                tot += hv;
                if (r < rank) before += hv;
            }
            incl = tot;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += y;
            }
            if (lane == 31) wtot[warp] = incl;
        }
        __syncthreads();
        if (tid < 256) {
            uint32_t off = 0;
            for (int w2 = 0; w2 < warp; ++w2) off += wtot[w2];
            dbase[tid] = off + incl - tot + before;
        }
        __syncthreads();

        // (c) stable scatter, tile by tile in slice order
        for (int64_t t0 = lo; t0 < hi; t0 += SORT_TILE) {
            uint32_t u[SORT_ITEMS], idx[SORT_ITEMS], rnk[SORT_ITEMS], dg[SORT_ITEMS];
#pragma unroll
            for (int it = 0; it < SORT_ITEMS; ++it) {
                const int64_t i = t0 + warp * (32 * SORT_ITEMS) + it * 32 + lane;
                u[it] = 0; idx[it] = 0;
                if (i < hi) {
                    if (cached) {
                        u[it] = ckey[i - lo];
                        idx[it] = cidx[i - lo];
                    } else if (p == 0) {
                        idx[it] = init ? (uint32_t)init[s0 + i] : (uint32_t)i;
                        u[it] = key_xform(keys, key_type, s0 + idx[it]) - gmn;
                    } else {
                        u[it] = ksrc[s0 + i];
                        idx[it] = isrc[s0 + i];
                    }
                    dg[it] = (u[it] >> shift) & 255u;
                } else {
                    dg[it] = 256u;
                }
            }
            for (int z = tid; z < SORT_WARPS * 257; z += SORT_THREADS) (&wcount[0][0])[z] = 0;
            __syncthreads();
#pragma unroll
            for (int it = 0; it < SORT_ITEMS; ++it) {
                // lanes holding the same digit: eight ballots (one per bit) instead of match.any
                uint32_t m = 0xffffffffu;
#pragma unroll
                for (int bit = 0; bit < 9; ++bit) {
                    const uint32_t bal = __ballot_sync(0xffffffffu, (dg[it] >> bit) & 1u);
                    m &= ((dg[it] >> bit) & 1u) ? bal : ~bal;
                }
                const bool valid = dg[it] < 256u;
                const uint32_t basecnt = valid ? wcount[warp][dg[it]] : 0u;
                rnk[it] = basecnt + __popc(m & ((1u << lane) - 1u));
                __syncwarp();
                if (valid && (__ffs(m) - 1) == lane) wcount[warp][dg[it]] = basecnt + __popc(m);
                __syncwarp();
            }
            __syncthreads();
            // exclusive scan over the warps, per digit: warp w takes digits w, w + 32, ...; lane = source warp
#pragma unroll
            for (int q = 0; q < 256 / SORT_WARPS; ++q) {
                const int d = warp + q * SORT_WARPS;
                const uint32_t c = wcount[lane][d];
                uint32_t incl2 = c;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t y = __shfl_up_sync(0xffffffffu, incl2, o);
                    if (lane >= o) incl2 += y;
                }
                wcount[lane][d] = incl2 - c;
                if (lane == 31) tile_tot[d] = incl2;
            }
            __syncthreads();
            // where each digit starts inside the tile (exclusive scan of the tile's digit counts)
            uint32_t tt = 0, ti = 0;
            if (tid < 256) {
                tt = tile_tot[tid];
                ti = tt;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const uint32_t y = __shfl_up_sync(0xffffffffu, ti, o);
                    if (lane >= o) ti += y;
                }
                if (lane == 31) wtot[warp] = ti;
            }
            __syncthreads();
            if (tid < 256) {
                uint32_t off = 0;
                for (int w2 = 0; w2 < warp; ++w2) off += wtot[w2];
                tstart[tid] = off + ti - tt;
            }
            __syncthreads();
            // group the tile by digit in shared memory, so that the global writes below are runs of
            // consecutive addresses (a direct scatter costs one 32-byte sector per key)
#pragma unroll
            for (int it = 0; it < SORT_ITEMS; ++it) {
                if (dg[it] < 256u) {
                    const uint32_t lp = tstart[dg[it]] + wcount[warp][dg[it]] + rnk[it];
                    skey[lp] = u[it];
                    sidx[lp] = idx[it];
                }
            }
            __syncthreads();
            const int ntile = (int)min((int64_t)SORT_TILE, hi - t0);
#pragma unroll
            for (int it = 0; it < SORT_ITEMS; ++it) {
                const int lp = it * SORT_THREADS + tid;
                if (lp < ntile) {
                    const uint32_t ku = skey[lp], ki = sidx[lp];
                    const uint32_t d = (ku >> shift) & 255u;
                    const int64_t pos = (int64_t)dbase[d] + (lp - tstart[d]);
                    if (last) {
                        perm[s0 + pos] = (int64_t)ki;
                    } else {
                        kdst[s0 + pos] = ku;
                        idst[s0 + pos] = ki;
                    }
                }
            }
            __syncthreads();
            if (tid < 256) dbase[tid] += tile_tot[tid];
        }
        cluster.sync();   // release/acquire at cluster scope: scattered keys visible to the peers; histograms free again
    }
    cluster.sync();       // no CTA leaves while a peer may still read its shared memory
}

// Upper bound of the cluster size for nseg segments: SMs / segments, at most 8 (the launcher lowers it until all fit).
static int sort_cluster_size(int nseg) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int cl = sms / (nseg > 0 ? nseg : 1);
    if (cl > SORT_MAX_CL) cl = SORT_MAX_CL;
    if (cl < 1) cl = 1;
    return cl;
}

// cudaOccupancyMaxActiveClusters for this kernel, remembered per (device, cluster size, cache size):
// the answer does not change and the query costs tens of microseconds of host time.
static int clusters_resident(const cudaLaunchConfig_t& cfg, int cl, int cache_cap) {
    static std::mutex mu;
    static std::map<std::tuple<int, int, int>, int> memo;
    int dev = 0;
    cudaGetDevice(&dev);
    const auto key = std::make_tuple(dev, cl, cache_cap);
    std::lock_guard<std::mutex> lk(mu);
    const auto it = memo.find(key);
    if (it != memo.end()) return it->second;
    int resident = 0;
    if (cudaOccupancyMaxActiveClusters(&resident, segsort_kernel, &cfg) != cudaSuccess) resident = 0;
    memo[key] = resident;
    return resident;
}

static int launch_segsort(const void* keys, int key_type, int64_t n_total, const int64_t* seg, int nseg,
                          const int64_t* init, int64_t* perm, uint32_t* k0, uint32_t* k1, uint32_t* i0,
                          uint32_t* i1, int32_t* status, cudaStream_t st) {
    if (cudaFuncSetAttribute(segsort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * SORT_TILE + 2 * 12288) * 4) != cudaSuccess)
        return LAMPA_ERR_CUDA;
    // Cluster size: the largest one for which every segment's cluster is resident at the same time.
    // A cluster has to fit inside one GPC, so the SM count alone does not tell (148 SMs hold 24
    // clusters of 6 only if every GPC has 18 usable SMs): ask the occupancy calculator.
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    int cl = sort_cluster_size(nseg), cache_cap = 0;
    for (;; --cl) {
        // slice cache: the slice of an equal split, or twice the average slice when the segments are ragged
        // (larger slices simply read from global memory), rounded up to 1 K keys, at most 12 K (96 KB)
        const int64_t avg = (n_total / (nseg > 0 ? nseg : 1) + cl - 1) / cl + 1;
        const int64_t want = seg ? 2 * avg : avg;
        cache_cap = (int)std::min<int64_t>(12288, (want + 1023) / 1024 * 1024);
        cfg.gridDim = dim3((unsigned)nseg * cl, 1, 1);
        cfg.blockDim = dim3(SORT_THREADS, 1, 1);
        cfg.dynamicSmemBytes = (2 * SORT_TILE + 2 * (size_t)cache_cap) * sizeof(uint32_t);
        cfg.stream = st;
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = cl;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
        if (cl == 1) break;
        if (clusters_resident(cfg, cl, cache_cap) >= nseg) break;
    }
    const cudaError_t e = cudaLaunchKernelEx(&cfg, segsort_kernel, keys, key_type, n_total, seg, nseg, init, perm,
                                             k0, k1, i0, i1, cache_cap, status);
    return e == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

// -------------------------------------------------------------------------------------------------
// Row gather/scatter and permutation inverse.
// -------------------------------------------------------------------------------------------------
__device__ __forceinline__ int find_seg64(const int64_t* off, int nseg, int64_t x) {
    int lo = 0, hi = nseg;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (off[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}

// An index outside its segment is not followed: the access is skipped and LAMPA_ERR_BOUNDS is
// recorded in the status word (a permutation that came from lampa_segsort_stable never trips it).
template <typename VEC>
__global__ void __launch_bounds__(256)
permute_rows_kernel(const VEC* __restrict__ src, const int64_t* __restrict__ perm,
                    const int64_t* __restrict__ seg, int nseg, int64_t n_rows, int64_t units_per_row,
                    int scatter, VEC* __restrict__ dst, int32_t* status) {
    const int64_t total = n_rows * units_per_row;
    for (int64_t u = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; u < total;
         u += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = u / units_per_row, col = u - row * units_per_row;
        int64_t s0, len;
        if (seg) { const int si = find_seg64(seg, nseg, row); s0 = seg[si]; len = seg[si + 1] - s0; }
        else { len = n_rows / nseg; s0 = (row / len) * len; }
        const int64_t p = perm[row];
        if (p < 0 || p >= len || s0 < 0 || s0 + len > n_rows) {
            if (col == 0) set_status(status, LAMPA_ERR_BOUNDS, 10, (int)row);
            continue;
        }
        const int64_t other = s0 + p;
        if (scatter) dst[other * units_per_row + col] = src[u];
        else dst[u] = src[other * units_per_row + col];
    }
}

__global__ void __launch_bounds__(256)
invert_perm_kernel(const int64_t* __restrict__ perm, const int64_t* __restrict__ seg, int nseg,
                   int64_t n_total, int64_t* __restrict__ inv, int32_t* status) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_total;
         i += (int64_t)gridDim.x * blockDim.x) {
        int64_t s0, len;
        if (seg) { const int si = find_seg64(seg, nseg, i); s0 = seg[si]; len = seg[si + 1] - s0; }
        else { len = n_total / nseg; s0 = (i / len) * len; }
        const int64_t p = perm[i];
        if (p < 0 || p >= len || s0 < 0 || s0 + len > n_total) { set_status(status, LAMPA_ERR_BOUNDS, 11, (int)i); continue; }
        inv[s0 + p] = i - s0;
    }
}

}  // namespace lampa

using namespace lampa;

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

extern "C" int lampa_lsh_hash(const float* x, int64_t row_stride, int64_t head_stride, const float* alpha,
                              const float* beta, float w, int64_t N, int32_t heads, int32_t rounds,
                              int32_t dim, int32_t* ids, float* keys, int32_t* packed, void* stream) {
    if (!x || !alpha || !beta || N < 0 || heads <= 0 || rounds <= 0 || dim <= 0) return LAMPA_ERR_ARG;
    if (!(w > 0.f)) return LAMPA_ERR_ARG;
    if ((int64_t)heads * dim * rounds > HASH_MAX_PARAMS || rounds > 64 || heads > 31) return LAMPA_ERR_UNSUPPORTED;
    if (N == 0) return LAMPA_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)((N + HASH_THREADS - 1) / HASH_THREADS);
    ProfScope prof("lsh_hash", st);
    if (dim == 6 && head_stride == 0)
        lsh_hash_kernel<6><<<grid, HASH_THREADS, 0, st>>>(x, row_stride, head_stride, alpha, beta, w, N, heads, rounds, dim, ids, keys, packed);
    else
        lsh_hash_kernel<0><<<grid, HASH_THREADS, 0, st>>>(x, row_stride, head_stride, alpha, beta, w, N, heads, rounds, dim, ids, keys, packed);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_segsort_workspace_bytes(int64_t n_total, size_t* bytes) {
    if (n_total < 0 || !bytes) return LAMPA_ERR_ARG;
    *bytes = 4 * align_up((size_t)n_total * 4, 256) + 256;
    return LAMPA_OK;
}

extern "C" int lampa_segsort_stable(const void* keys, int32_t key_type, int64_t n_total,
                                    const int64_t* seg_offsets, int32_t nseg, const int64_t* init,
                                    int64_t* perm, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
    if (n_total < 0 || nseg <= 0 || (key_type != LAMPA_KEY_I32 && key_type != LAMPA_KEY_F32)) return LAMPA_ERR_ARG;
    if (n_total == 0) return LAMPA_OK;
    if (!keys || !perm || !ws) return LAMPA_ERR_ARG;
    if (!seg_offsets && n_total % nseg != 0) return LAMPA_ERR_ARG;
    if (n_total >= ((int64_t)1 << 32)) return LAMPA_ERR_UNSUPPORTED;
    size_t need;
    lampa_segsort_workspace_bytes(n_total, &need);
    if (ws_bytes < need || ((uintptr_t)ws & 15)) return LAMPA_ERR_WORKSPACE;
    const size_t stride = align_up((size_t)n_total * 4, 256);
    char* base = (char*)(((uintptr_t)ws + 255) / 256 * 256);
    uint32_t* k0 = (uint32_t*)base;
    uint32_t* k1 = (uint32_t*)(base + stride);
    uint32_t* i0 = (uint32_t*)(base + 2 * stride);
    uint32_t* i1 = (uint32_t*)(base + 3 * stride);
    ProfScope prof("segsort", (cudaStream_t)stream);
    return launch_segsort(keys, key_type, n_total, seg_offsets, nseg, init, perm, k0, k1, i0, i1, status, (cudaStream_t)stream);
}

extern "C" int lampa_permute_rows(const void* src, const int64_t* perm, const int64_t* seg_offsets,
                                  int32_t nseg, int64_t n_rows, int64_t row_bytes, int32_t scatter,
                                  void* dst, int32_t* status, void* stream) {
    if (n_rows < 0 || row_bytes <= 0 || (row_bytes & 3) || nseg <= 0) return LAMPA_ERR_ARG;
    if (n_rows == 0) return LAMPA_OK;
    if (!src || !perm || !dst) return LAMPA_ERR_ARG;
    if (!seg_offsets && n_rows % nseg != 0) return LAMPA_ERR_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const bool v16 = (row_bytes % 16 == 0) && (((uintptr_t)src | (uintptr_t)dst) % 16 == 0);
    const int64_t upr = v16 ? row_bytes / 16 : row_bytes / 4;
    const int64_t total = n_rows * upr;
    const unsigned grid = (unsigned)std::min<int64_t>((total + 255) / 256, 148 * 32);
    ProfScope prof("permute_rows", st);
    if (v16)
        permute_rows_kernel<uint4><<<grid, 256, 0, st>>>((const uint4*)src, perm, seg_offsets, nseg, n_rows, upr, scatter, (uint4*)dst, status);
    else
        permute_rows_kernel<uint32_t><<<grid, 256, 0, st>>>((const uint32_t*)src, perm, seg_offsets, nseg, n_rows, upr, scatter, (uint32_t*)dst, status);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

extern "C" int lampa_invert_perm(const int64_t* perm, const int64_t* seg_offsets, int32_t nseg,
                                 int64_t n_total, int64_t* inv, int32_t* status, void* stream) {
    if (n_total < 0 || nseg <= 0) return LAMPA_ERR_ARG;
    if (n_total == 0) return LAMPA_OK;
    if (!perm || !inv) return LAMPA_ERR_ARG;
    if (!seg_offsets && n_total % nseg != 0) return LAMPA_ERR_ARG;
    const unsigned grid = (unsigned)std::min<int64_t>((n_total + 255) / 256, 148 * 32);
    ProfScope prof("invert_perm", (cudaStream_t)stream);
    invert_perm_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(perm, seg_offsets, nseg, n_total, inv, status);
    return cudaGetLastError() == cudaSuccess ? LAMPA_OK : LAMPA_ERR_CUDA;
}

// -------------------------------------------------------------------------------------------------
// Sort without any caller- or library-side allocation: the four ping-pong buffers live in a
// fixed array that is part of the loaded module (24 MiB per GPU that loads the library, held
// until the process exits).  Host code cannot use the symbol g_sort_scratch as a pointer — on
// the host it is only a handle — so its device address is looked up once per device with
// cudaGetSymbolAddress and cached.
// -------------------------------------------------------------------------------------------------
namespace {
constexpr size_t kStaticSortStride = (size_t)LAMPA_SEGSORT_STATIC_MAX_KEYS * 4;   // bytes per buffer, multiple of 256
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mu;
void* g_scratch_addr[kMaxDevices] = {nullptr};
}  // namespace

static __device__ __align__(256) unsigned char g_sort_scratch[4 * kStaticSortStride];

// Device address of g_sort_scratch on the CURRENT device (looked up on first use there).
static int static_sort_scratch(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return LAMPA_ERR_CUDA;
    if (dev < 0 || dev >= kMaxDevices) return LAMPA_ERR_UNSUPPORTED;
    std::lock_guard<std::mutex> lk(g_scratch_mu);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_sort_scratch) != cudaSuccess || p == nullptr) return LAMPA_ERR_CUDA;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return LAMPA_OK;
}

extern "C" int lampa_segsort_stable_static(const void* keys, int32_t key_type, int64_t n_total,
                                           const int64_t* seg_offsets, int32_t nseg, const int64_t* init,
                                           int64_t* perm, int32_t* status, void* stream) {
    if (n_total < 0 || nseg <= 0 || (key_type != LAMPA_KEY_I32 && key_type != LAMPA_KEY_F32)) return LAMPA_ERR_ARG;
    if (n_total > (int64_t)LAMPA_SEGSORT_STATIC_MAX_KEYS) return LAMPA_ERR_TOO_LARGE;
    if (n_total == 0) return LAMPA_OK;
    if (!keys || !perm) return LAMPA_ERR_ARG;
    if (!seg_offsets && n_total % nseg != 0) return LAMPA_ERR_ARG;
    void* base_v = nullptr;
    const int rc = static_sort_scratch(&base_v);
    if (rc != LAMPA_OK) return rc;
    char* base = (char*)base_v;
    // No buffer needs clearing between calls: every pass writes positions [0, n) of its
    // destination pair before the next pass reads them, and nothing beyond n is ever read.
    ProfScope prof("segsort_static", (cudaStream_t)stream);
    return launch_segsort(keys, key_type, n_total, seg_offsets, nseg, init, perm, (uint32_t*)base,
                          (uint32_t*)(base + kStaticSortStride), (uint32_t*)(base + 2 * kStaticSortStride),
                          (uint32_t*)(base + 3 * kStaticSortStride), status, (cudaStream_t)stream);
}
