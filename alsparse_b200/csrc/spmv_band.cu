// Column-band SpMV for the long rows of a skewed matrix (sm_100a).
//
// Every stored element of a row with unstructured columns gathers one x element from a different
// cache line, and a B200 SM gets roughly one such line per clock out of L2: for a matrix whose
// elements sit mostly in rows of tens of thousands of entries that rate, not HBM, sets the time.
// A long row with ascending columns can do better.  Cut the columns into bands of `width`; the part
// of the row that falls into one band is a contiguous run of its elements (a "segment"), and all of
// its gathers land in the `width` x elements of that band.  So a thread block stages one band of x
// in shared memory with coalesced loads (64 KB), and then runs through the segments that ALL long
// rows have in this band, gathering from shared memory at many elements per clock instead of one.
// The col / val streams are still read exactly once, coalesced, which leaves HBM as the limit.
//
// Each (row, band) segment yields one partial sum; a second kernel adds a row's partials in band
// order and accumulates alpha times the total into y.  No atomics: the result does not depend on
// scheduling.  The analysis decides which rows qualify (band_build) and removes the merge tiles they
// cover from the merge kernel's schedule; what is left of such a row at its two ends (less than a
// tile each) stays with the merge kernel, which also applies beta.
//
// Arithmetic defined by the reference's gemv kernel, src/plain/kernel/level2/mv/gemv/gemv_x_csr_plain.c:4-24
// (same products, another summation order, inside the parity tolerance).  The reference's device
// build has one kernel shape for all rows (src/kernel/dcu/level2/mv/csrmv/dcu_gemv_vector.h:59-182
// picks a sub-wavefront width from nnz/m); it has no counterpart of this path.
#include <algorithm>
#include <numeric>
#include <vector>

#include "internal.h"

namespace asb {

constexpr int kBandThreads = 512;
constexpr int kBandLanes = 8;  // lanes per segment

// Block (b, s): band b, list positions [s*chunk, (s+1)*chunk).  A group of G lanes takes R segments at a time and
// keeps U quads per segment in flight in every lane.  A lane takes whole aligned quads (four consecutive stored
// elements: one int4 of columns, one or two 16-byte loads of values) and masks the elements that fall outside the
// segment, as the vector SpMV kernel does for rows: the bytes in flight per load instruction are what covers the
// latency of HBM in a kernel that streams the matrix once.  Measured on B200 (power-law matrix, 1.9e8 elements in
// 4205 long rows, 1024 bands): 8 lanes x 1 quad x 2 segments and 4 lanes x 2 quads x 1 segment per group, 512
// threads, two blocks per SM, are the fastest shapes; scalar loads (4 bytes per lane) took twice as long, and
// forcing three blocks per SM (40 registers, spills) or 32 KB bands with six smaller blocks were slower too.
template <typename T>
struct BandQuad {
    T v[4];
};
__device__ __forceinline__ BandQuad<float> band_load_val(const float *__restrict__ val, int q) {
    const float4 t = __ldcs(reinterpret_cast<const float4 *>(val) + q);
    return {{t.x, t.y, t.z, t.w}};
}
__device__ __forceinline__ BandQuad<double> band_load_val(const double *__restrict__ val, int q) {
    const double2 a = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q);
    const double2 b = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q + 1);
    return {{a.x, a.y, b.x, b.y}};
}

template <typename T, int G, int U, int R, int NT>
__global__ void __launch_bounds__(NT)
    spmv_band_quad_kernel(int cols, int width, int bands, int nl, int chunk, const int *__restrict__ seg,
                          const int *__restrict__ col, const T *__restrict__ val, const T *__restrict__ x,
                          T *__restrict__ partial, int *__restrict__ status) {
    extern __shared__ __align__(16) unsigned char band_smem[];
    T *sx = reinterpret_cast<T *>(band_smem);
    const int b = blockIdx.x, s = blockIdx.y, tid = threadIdx.x;
    const long long c0l = (long long)b * width;
    const int c0 = (int)c0l;
    const int n = (int)(cols - c0l < width ? cols - c0l : width);
    const T *xb = x + c0l;

    constexpr int NG = NT / G;
    const int g = tid / G, gl = tid % G;
    const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (((tid & 31) / G) * G));
    const int p1 = min(nl, (s + 1) * chunk);
    const int *seg_lo = seg + (size_t)b * nl, *seg_hi = seg_lo + nl;

    // The bounds of the first segments are fetched before the band of x is staged, and those of every later
    // step while the current one is multiplied: the look-up never sits in front of the matrix loads.
    int na[R], ne[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int pp = s * chunk + g + r * NG;
        na[r] = 0, ne[r] = 0;
        if (pp < p1) {
            na[r] = __ldg(seg_lo + pp);
            ne[r] = __ldg(seg_hi + pp);
        }
    }

    // The band of x comes in by bulk asynchronous copies (cp.async.bulk global -> shared, completion counted in
    // bytes on an mbarrier) issued by one thread, so that every thread goes straight on to its first matrix loads
    // and meets the band only when it needs it.  A band that does not start on a 16-byte boundary or has a ragged
    // length (the last one) is loaded by all threads instead.  `ready` is uniform over the block until the wait.
    __shared__ __align__(8) unsigned long long s_bar;
    const unsigned bar = (unsigned)__cvta_generic_to_shared(&s_bar);
    const unsigned band_bytes = (unsigned)n * (unsigned)sizeof(T);
    const bool bulk = (reinterpret_cast<uintptr_t>(xb) & 15) == 0 && (band_bytes & 15u) == 0 && band_bytes > 0;
    bool ready = !bulk;
    if (bulk) {
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(band_bytes) : "memory");
            constexpr unsigned kPiece = 16 * 1024;
            for (unsigned off = 0; off < band_bytes; off += kPiece) {
                const unsigned bytes = band_bytes - off < kPiece ? band_bytes - off : kPiece;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 (unsigned)__cvta_generic_to_shared(band_smem + off)),
                             "l"(reinterpret_cast<const unsigned char *>(xb) + off), "r"(bytes), "r"(bar)
                             : "memory");
            }
        }
    } else {
        for (int i = tid; i < n; i += NT) sx[i] = __ldg(xb + i);
    }
    __syncthreads();  // the barrier is initialised (or the band is in place) for everyone

    // Bounded wait for the band; on a time-out the block records the error word and gives up its segments.
    auto wait_band = [&]() -> bool {
        for (int spin = 0; spin < (1 << 22); spin++) {
            unsigned ok;
            asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                         : "=r"(ok)
                         : "r"(bar), "r"(0u)
                         : "memory");
            if (ok) return true;
        }
        atomicExch(status, 2);
        return false;
    };

    for (int p = s * chunk + g; p < p1; p += NG * R) {
        int a[R], e[R], q[R];
        T acc[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            a[r] = na[r], e[r] = ne[r], acc[r] = T(0);
            q[r] = (a[r] >> 2) + gl;
            const int pn = p + (R + r) * NG;  // the segment this slot takes in the next step
            na[r] = 0, ne[r] = 0;
            if (pn < p1) {
                na[r] = __ldg(seg_lo + pn);
                ne[r] = __ldg(seg_hi + pn);
            }
        }
        bool more = true;
        while (more) {
            int4 cc[R][U];
            BandQuad<T> vv[R][U];
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int qq = q[r] + u * G;
                    if ((qq << 2) < e[r]) {
                        cc[r][u] = __ldcs(reinterpret_cast<const int4 *>(col) + qq);
                        vv[r][u] = band_load_val(val, qq);
                    }
                }
            if (!ready) {  // the first matrix loads are on their way: now the band is needed
                if (!wait_band()) return;
                ready = true;
            }
            more = false;
#pragma unroll
            for (int r = 0; r < R; r++) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int base = (q[r] + u * G) << 2;
                    if (base < e[r]) {
                        if (base + 0 >= a[r]) acc[r] = fma(vv[r][u].v[0], sx[cc[r][u].x - c0], acc[r]);
                        if (base + 1 >= a[r] && base + 1 < e[r]) acc[r] = fma(vv[r][u].v[1], sx[cc[r][u].y - c0], acc[r]);
                        if (base + 2 >= a[r] && base + 2 < e[r]) acc[r] = fma(vv[r][u].v[2], sx[cc[r][u].z - c0], acc[r]);
                        if (base + 3 >= a[r] && base + 3 < e[r]) acc[r] = fma(vv[r][u].v[3], sx[cc[r][u].w - c0], acc[r]);
                    }
                }
                q[r] += G * U;
                more |= (q[r] << 2) < e[r];
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(gmask, acc[r], o, G);
            const int pp = p + r * NG;
            if (gl == 0 && pp < p1) partial[(size_t)pp * bands + b] = acc[r];
        }
    }
    // a thread without segments has not met the band yet: nobody leaves while the copies may still be writing
    // into this block's shared memory
    if (!ready) wait_band();
}

// ---- the same product from the packed copy ------------------------------------------------------------
//
// The long rows are static, so the analysis can lay their elements out the way this kernel walks them: band by band,
// inside a band segment after segment in list order, every segment padded to whole quads.  The block (b, s) then
// streams ONE contiguous piece of memory, neighbouring lane groups read neighbouring addresses, no element has to be
// masked against the row's ends, and the column of an element is its offset inside the band: 16 bits instead of 32
// (10 instead of 12 bytes per fp64 element, 6 instead of 8 per fp32 element).  Padding carries the column 0xffff
// and is skipped, so nothing of x is ever read for it.  The copy costs (sizeof(T) + 2) bytes per long-row element
// of device memory; the caller's CSR arrays stay as they are.
// (Feeding the packed piece through shared memory with a pipeline of bulk copies -- stages of 256 quads on
// mbarriers, one quad per thread, segmented scan over the lanes, run sums combined in warp order -- was built and
// measured too: 1.86 ms per power-law product against 1.24 ms with the lane groups below.  With ~60 elements per
// segment the two block-wide barriers and the ordered combine of every 10 KB stage cost more than the loads they
// take out of the registers.)
template <typename T>
__device__ __forceinline__ BandQuad<T> band_load_packed(const T *__restrict__ val, int q);
template <>
__device__ __forceinline__ BandQuad<float> band_load_packed<float>(const float *__restrict__ val, int q) {
    const float4 t = __ldcs(reinterpret_cast<const float4 *>(val) + q);
    return {{t.x, t.y, t.z, t.w}};
}
template <>
__device__ __forceinline__ BandQuad<double> band_load_packed<double>(const double *__restrict__ val, int q) {
    const double2 a = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q);
    const double2 b = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q + 1);
    return {{a.x, a.y, b.x, b.y}};
}

template <typename T, int G, int U, int R, int NT>
__global__ void __launch_bounds__(NT)
    spmv_band_packed_kernel(int cols, int width, int bands, int nl, int chunk, const int *__restrict__ pk_start,
                            const unsigned short *__restrict__ pk_col, const T *__restrict__ pk_val,
                            const T *__restrict__ x, T *__restrict__ partial, int *__restrict__ status) {
    extern __shared__ __align__(16) unsigned char band_smem[];
    T *sx = reinterpret_cast<T *>(band_smem);
    const int b = blockIdx.x, s = blockIdx.y, tid = threadIdx.x;
    const long long c0l = (long long)b * width;
    const int n = (int)(cols - c0l < width ? cols - c0l : width);
    const T *xb = x + c0l;

    constexpr int NG = NT / G;
    const int g = tid / G, gl = tid % G;
    const unsigned gmask = G == 32 ? 0xffffffffu : (((1u << G) - 1u) << (((tid & 31) / G) * G));
    const int p1 = min(nl, (s + 1) * chunk);
    const int *start = pk_start + (size_t)b * nl;

    int nq[R], ne[R];  // first quad / end quad of the segments of the next step
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int pp = s * chunk + g + r * NG;
        nq[r] = 0, ne[r] = 0;
        if (pp < p1) {
            nq[r] = __ldg(start + pp);
            ne[r] = __ldg(start + pp + 1);
        }
    }

    __shared__ __align__(8) unsigned long long s_bar;
    const unsigned bar = (unsigned)__cvta_generic_to_shared(&s_bar);
    const unsigned band_bytes = (unsigned)n * (unsigned)sizeof(T);
    const bool bulk = (reinterpret_cast<uintptr_t>(xb) & 15) == 0 && (band_bytes & 15u) == 0 && band_bytes > 0;
    bool ready = !bulk;
    if (bulk) {
        if (tid == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(band_bytes) : "memory");
            constexpr unsigned kPiece = 16 * 1024;
            for (unsigned off = 0; off < band_bytes; off += kPiece) {
                const unsigned bytes = band_bytes - off < kPiece ? band_bytes - off : kPiece;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                                 (unsigned)__cvta_generic_to_shared(band_smem + off)),
                             "l"(reinterpret_cast<const unsigned char *>(xb) + off), "r"(bytes), "r"(bar)
                             : "memory");
            }
        }
    } else {
        for (int i = tid; i < n; i += NT) sx[i] = __ldg(xb + i);
    }
    __syncthreads();
    auto wait_band = [&]() -> bool {
        for (int spin = 0; spin < (1 << 22); spin++) {
            unsigned ok;
            asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                         : "=r"(ok)
                         : "r"(bar), "r"(0u)
                         : "memory");
            if (ok) return true;
        }
        atomicExch(status, 2);
        return false;
    };

    for (int p = s * chunk + g; p < p1; p += NG * R) {
        int q[R], e[R];
        T acc[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            q[r] = nq[r] + gl, e[r] = ne[r], acc[r] = T(0);
            const int pn = p + (R + r) * NG;
            nq[r] = 0, ne[r] = 0;
            if (pn < p1) {
                nq[r] = __ldg(start + pn);
                ne[r] = __ldg(start + pn + 1);
            }
        }
        bool more = true;
        while (more) {
            uint2 cc[R][U];
            BandQuad<T> vv[R][U];
#pragma unroll
            for (int r = 0; r < R; r++)
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const int qq = q[r] + u * G;
                    if (qq < e[r]) {
                        cc[r][u] = __ldcs(reinterpret_cast<const uint2 *>(pk_col) + qq);
                        vv[r][u] = band_load_packed<T>(pk_val, qq);
                    }
                }
            if (!ready) {
                if (!wait_band()) return;
                ready = true;
            }
            more = false;
#pragma unroll
            for (int r = 0; r < R; r++) {
#pragma unroll
                for (int u = 0; u < U; u++) {
                    if (q[r] + u * G < e[r]) {
                        const unsigned c0 = cc[r][u].x & 0xffffu, c1 = cc[r][u].x >> 16;
                        const unsigned c2 = cc[r][u].y & 0xffffu, c3 = cc[r][u].y >> 16;
                        if (c0 != 0xffffu) acc[r] = fma(vv[r][u].v[0], sx[c0], acc[r]);
                        if (c1 != 0xffffu) acc[r] = fma(vv[r][u].v[1], sx[c1], acc[r]);
                        if (c2 != 0xffffu) acc[r] = fma(vv[r][u].v[2], sx[c2], acc[r]);
                        if (c3 != 0xffffu) acc[r] = fma(vv[r][u].v[3], sx[c3], acc[r]);
                    }
                }
                q[r] += G * U;
                more |= q[r] < e[r];
            }
        }
#pragma unroll
        for (int r = 0; r < R; r++) {
#pragma unroll
            for (int o = G / 2; o > 0; o >>= 1) acc[r] += __shfl_xor_sync(gmask, acc[r], o, G);
            const int pp = p + r * NG;
            if (gl == 0 && pp < p1) partial[(size_t)pp * bands + b] = acc[r];
        }
    }
    if (!ready) wait_band();
}

// Fills the packed copy: block p copies the elements [a[p], e[p]) of long row p to their places.
template <typename T>
__global__ void band_pack_kernel(int nl, int width, const int *__restrict__ a, const int *__restrict__ e,
                                 const int *__restrict__ seg, const int *__restrict__ pk_start,
                                 const int *__restrict__ col, const T *__restrict__ val,
                                 unsigned short *__restrict__ pk_col, T *__restrict__ pk_val) {
    const int p = blockIdx.x;
    for (long long k = (long long)a[p] + threadIdx.x; k < e[p]; k += blockDim.x) {
        const int c = col[k];
        const int b = c / width;
        const size_t cell = (size_t)b * nl + p;
        const size_t dst = 4 * (size_t)pk_start[cell] + (size_t)(k - seg[cell]);
        pk_col[dst] = (unsigned short)(c - b * width);
        pk_val[dst] = val[k];
    }
}

// One warp per long row: its partial sums in band order (lane j takes bands j, j+32, ..., then a fixed tree over
// the lanes).  ASSIGN: the row belongs to this path alone, y[row] = alpha * total + beta * y[row]; otherwise alpha
// times the total is added to what the merge kernel and its fix-up left in y.
template <typename T, bool ASSIGN>
__global__ void spmv_band_reduce_kernel(int nl, int bands, const int *__restrict__ row,
                                        const T *__restrict__ partial, T *__restrict__ y, T alpha, T beta,
                                        const PeerPush push) {
    const int p = (int)(((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
    const int lane = threadIdx.x & 31;
    if (p >= nl) return;
    const T *src = partial + (size_t)p * bands;
    T acc = T(0);
    for (int b = lane; b < bands; b += 32) acc += src[b];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
        const int r = row[p];
        if (ASSIGN) {
            const T out = (beta == T(0)) ? alpha * acc : fma(beta, y[r], alpha * acc);
            y[r] = out;
            // exchange calls: the finished row also goes to every GPU's next x (push.n == 0 otherwise)
            for (int q = 0; q < push.n; q++) static_cast<T *>(push.dst[q])[push.row_off + r] = out;
        } else {
            y[r] = fma(alpha, acc, y[r]);
        }
    }
}

// flag[p] = 1 when the elements [a[p], e[p]) are not in ascending column order (such a row cannot be cut
// into segments by searching its columns).
__global__ void band_sorted_kernel(const int *__restrict__ a, const int *__restrict__ e, const int *__restrict__ col,
                                   int *__restrict__ flag) {
    const int p = blockIdx.x;
    int bad = 0;
    for (long long k = (long long)a[p] + threadIdx.x; k + 1 < e[p]; k += blockDim.x) bad |= col[k] > col[k + 1];
    if (__syncthreads_or(bad) && threadIdx.x == 0) flag[p] = 1;
}

// seg[b * nl + p] = first element of [a[p], e[p]) whose column is >= b * width (b = 0 .. bands).
__global__ void band_seg_kernel(int nl, int bands, int width, const int *__restrict__ a, const int *__restrict__ e,
                                const int *__restrict__ col, int *__restrict__ seg) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)nl * (bands + 1)) return;
    const int b = (int)(i / nl), p = (int)(i % nl);
    const long long want = (long long)b * width;
    int lo = a[p], hi = e[p];
    if (b == 0) hi = lo;
    else if (b == bands) lo = hi;
    while (lo < hi) {
        const int mid = lo + ((hi - lo) >> 1);
        if ((long long)col[mid] < want) lo = mid + 1;
        else hi = mid;
    }
    seg[i] = lo;
}

void band_destroy(BandTables &b) {
    cudaFree(b.d_row);
    cudaFree(b.d_seg);
    cudaFree(b.d_partial);
    cudaFree(b.d_pk_start);
    cudaFree(b.d_pk_val);
    cudaFree(b.d_pk_col);
    if (b.side) cudaStreamDestroy(b.side);
    if (b.ev_fork) cudaEventDestroy(b.ev_fork);
    if (b.ev_join) cudaEventDestroy(b.ev_join);
    b = BandTables{};
}

struct BandCand {
    int row, a, e;
    int64_t t0, t1;  // merge tiles covered (interior form only)
};

static int64_t band_width_of(const DeviceCtx *ctx) {
    const size_t tsz = ctx->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    int64_t width = option(kOptBandBytes) / (int64_t)tsz & ~31ll;
    if (width < 32) width = 32;
    if (width * (int64_t)tsz > 200 * 1024) width = (200 * 1024 / (int64_t)tsz) & ~31ll;
    return width;
}

int64_t band_long_min(const DeviceCtx *ctx) {
    const int64_t width = band_width_of(ctx);
    const int64_t bands = (ctx->cols + width - 1) / width;
    return std::max<int64_t>(1, option(kOptBandMinSeg) * std::max<int64_t>(bands, 1));
}

// Builds the tables for the candidates (element ranges of rows).  `all_or_nothing`: one candidate out of
// ascending column order drops the whole path (row bins need every long row taken) instead of just that row.
static alphasparse_status_t band_finish(DeviceCtx *ctx, std::vector<BandCand> &cand, int64_t covered, bool all_or_nothing,
                                        cudaStream_t st) {
    const size_t tsz = ctx->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    const int64_t width = band_width_of(ctx);
    const int64_t bands = (ctx->cols + width - 1) / width;
    auto worth = [&] {
        return (int64_t)cand.size() >= std::max<int64_t>(1, option(kOptBandMinRows)) &&
               covered * 100 >= ctx->nnz * option(kOptBandMinSharePct);
    };
    if (bands < 1 || bands > (1 << 20) || cand.empty() || !worth()) return ALPHA_SPARSE_STATUS_SUCCESS;

    // Longest first, dealt round-robin to the `splits` blocks of a band: equal work per block, and the
    // lane groups of a warp meet segments of similar length.
    std::stable_sort(cand.begin(), cand.end(), [](const BandCand &p, const BandCand &q) { return p.e - p.a > q.e - q.a; });
    int nl = (int)cand.size();
    std::vector<int> h_a((size_t)nl), h_e((size_t)nl), h_flag((size_t)nl, 0);
    for (int i = 0; i < nl; i++) h_a[(size_t)i] = cand[(size_t)i].a, h_e[(size_t)i] = cand[(size_t)i].e;

    int *d_a = nullptr, *d_e = nullptr, *d_flag = nullptr;
    BandTables bt;
    auto fail = [&](alphasparse_status_t s) {
        cudaFree(d_a), cudaFree(d_e), cudaFree(d_flag);
        band_destroy(bt);
        return s;
    };
#define TRY(expr, status)                 \
    do {                                  \
        cudaError_t _e = (expr);          \
        if (_e != cudaSuccess) {          \
            record_cuda_error(_e, #expr); \
            return fail(status);          \
        }                                 \
    } while (0)
    TRY(device_alloc(&d_a, sizeof(int) * (size_t)nl), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_e, sizeof(int) * (size_t)nl), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_flag, sizeof(int) * (size_t)nl), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(cudaMemcpyAsync(d_a, h_a.data(), sizeof(int) * (size_t)nl, cudaMemcpyHostToDevice, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(d_e, h_e.data(), sizeof(int) * (size_t)nl, cudaMemcpyHostToDevice, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemsetAsync(d_flag, 0, sizeof(int) * (size_t)nl, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    band_sorted_kernel<<<(unsigned)nl, 256, 0, st>>>(d_a, d_e, ctx->d_col, d_flag);
    count_launch();
    TRY(cudaMemcpyAsync(h_flag.data(), d_flag, sizeof(int) * (size_t)nl, cudaMemcpyDeviceToHost, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    {
        size_t keep = 0;
        for (int i = 0; i < nl; i++) {
            if (h_flag[(size_t)i]) {
                covered -= cand[(size_t)i].e - cand[(size_t)i].a;
                continue;
            }
            cand[keep++] = cand[(size_t)i];
        }
        if (all_or_nothing && keep != cand.size()) keep = 0;
        cand.resize(keep);
        nl = (int)keep;
    }
    if (cand.empty() || !worth()) {
        cand.clear();
        return fail(ALPHA_SPARSE_STATUS_SUCCESS);
    }

    int64_t splits = option(kOptBandSplits);
    if (splits <= 0) {
        splits = (148 * 3 * 8 + bands - 1) / bands;  // about eight waves of blocks ...
        // ... but a block should stream at least four times what it stages (a band of x), or the staging shows: a
        // quarter or an eighth of the power-law matrix (one GPU's share of 4 or 8) ran 2-3 % faster with 2 and 1 blocks
        // per band than with 4
        const int64_t stream = covered * (int64_t)(tsz + 2), staged = 4 * (int64_t)bands * width * (int64_t)tsz;
        splits = std::min<int64_t>(splits, std::max<int64_t>(1, (stream + staged - 1) / staged));
    }
    splits = std::max<int64_t>(1, std::min<int64_t>(splits, std::max(1, nl / (kBandThreads / kBandLanes))));
    splits = std::min<int64_t>(splits, 65535);
    const int chunk = (int)((nl + splits - 1) / splits);
    std::vector<int> h_row((size_t)nl);
    {
        // sorted index i goes to split i % splits; a stable sort by split number makes the positions dense
        std::vector<int> order((size_t)nl);
        std::iota(order.begin(), order.end(), 0);
        std::stable_sort(order.begin(), order.end(), [&](int p, int q) { return p % splits < q % splits; });
        for (int p = 0; p < nl; p++) {
            const BandCand &c = cand[(size_t)order[(size_t)p]];
            h_row[(size_t)p] = c.row, h_a[(size_t)p] = c.a, h_e[(size_t)p] = c.e;
        }
    }

    bt.rows = nl, bt.bands = (int)bands, bt.width = (int)width, bt.splits = (int)splits, bt.chunk = chunk;
    bt.elements = covered;
    TRY(device_alloc(&bt.d_row, sizeof(int) * (size_t)nl), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&bt.d_seg, sizeof(int) * (size_t)nl * (size_t)(bands + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&bt.d_partial, tsz * (size_t)nl * (size_t)bands), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(cudaMemcpyAsync(bt.d_row, h_row.data(), sizeof(int) * (size_t)nl, cudaMemcpyHostToDevice, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(d_a, h_a.data(), sizeof(int) * (size_t)nl, cudaMemcpyHostToDevice, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(d_e, h_e.data(), sizeof(int) * (size_t)nl, cudaMemcpyHostToDevice, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    const long long cells = (long long)nl * (bands + 1);
    band_seg_kernel<<<(unsigned)((cells + 255) / 256), 256, 0, st>>>(nl, (int)bands, (int)width, d_a, d_e, ctx->d_col,
                                                                   bt.d_seg);
    count_launch();
    TRY(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    if (option(kOptBandPacked) && width < 65535) {
        // quads per segment, band-major, from the segment table (a few MB: summed on the host)
        std::vector<int> h_seg((size_t)cells);
        TRY(cudaMemcpyAsync(h_seg.data(), bt.d_seg, sizeof(int) * (size_t)cells, cudaMemcpyDeviceToHost, st),
            ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        const size_t segs = (size_t)nl * (size_t)bands;
        std::vector<int> h_start(segs + 1);
        long long quads = 0;
        for (size_t i = 0; i < segs && quads <= (long long)INT32_MAX / 4; i++) {
            h_start[i] = (int)quads;
            quads += ((long long)h_seg[i + (size_t)nl] - h_seg[i] + 3) >> 2;
        }
        if (quads <= (long long)INT32_MAX / 4) {
            h_start[segs] = (int)quads;
            const size_t slots = 4 * (size_t)quads + 8;  // a little slack behind the last quad
            TRY(device_alloc(&bt.d_pk_start, sizeof(int) * (segs + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
            TRY(device_alloc(&bt.d_pk_val, tsz * slots), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
            TRY(device_alloc(&bt.d_pk_col, sizeof(unsigned short) * slots), ALPHA_SPARSE_STATUS_ALLOC_FAILED);

            TRY(cudaMemcpyAsync(bt.d_pk_start, h_start.data(), sizeof(int) * (segs + 1), cudaMemcpyHostToDevice, st),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            TRY(cudaMemsetAsync(bt.d_pk_val, 0, tsz * slots, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            TRY(cudaMemsetAsync(bt.d_pk_col, 0xff, sizeof(unsigned short) * slots, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            if (tsz == 8)
                band_pack_kernel<double><<<(unsigned)nl, 256, 0, st>>>(nl, (int)width, d_a, d_e, bt.d_seg, bt.d_pk_start,
                                                                      ctx->d_col, static_cast<const double *>(ctx->d_val),
                                                                      bt.d_pk_col, static_cast<double *>(bt.d_pk_val));
            else
                band_pack_kernel<float><<<(unsigned)nl, 256, 0, st>>>(nl, (int)width, d_a, d_e, bt.d_seg, bt.d_pk_start,
                                                                     ctx->d_col, static_cast<const float *>(ctx->d_val),
                                                                     bt.d_pk_col, static_cast<float *>(bt.d_pk_val));
            count_launch();
            TRY(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);  // h_start goes out of scope
            bt.pk_quads = quads;
        }
    }
    if (option(kOptBandOverlap)) {
        TRY(cudaStreamCreateWithFlags(&bt.side, cudaStreamNonBlocking), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(cudaEventCreateWithFlags(&bt.ev_fork, cudaEventDisableTiming), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(cudaEventCreateWithFlags(&bt.ev_join, cudaEventDisableTiming), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    }
    TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
#undef TRY
    cudaFree(d_a), cudaFree(d_e), cudaFree(d_flag);
    ctx->band = bt;
    ctx->device_bytes += (int64_t)(sizeof(int) * (size_t)nl * (size_t)(bands + 2) + tsz * (size_t)nl * (size_t)bands);
    if (bt.pk_quads > 0)
        ctx->device_bytes += (int64_t)((tsz + 2) * 4 * (size_t)bt.pk_quads + sizeof(int) * (size_t)nl * (size_t)bands);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t band_build(DeviceCtx *ctx, const MergeCoord *h_tile, std::vector<char> &skip, cudaStream_t st) {
    if (!option(kOptBandEnable)) return ALPHA_SPARSE_STATUS_SUCCESS;
    const int64_t tiles = ctx->merge_tiles;
    const int64_t min_len = band_long_min(ctx);
    // Candidates: maximal runs of tiles that lie wholly inside one row.
    std::vector<BandCand> cand;
    int64_t covered = 0;
    for (int64_t t = 0; t < tiles;) {
        if (h_tile[t].row != h_tile[t + 1].row || h_tile[t].row >= ctx->rows) {
            t++;
            continue;
        }
        int64_t u = t + 1;
        while (u < tiles && h_tile[u + 1].row == h_tile[t].row) u++;
        const int a = h_tile[t].nz, e = h_tile[u].nz;
        if ((int64_t)e - a >= min_len) {
            cand.push_back({h_tile[t].row, a, e, t, u});
            covered += e - a;
        }
        t = u;
    }
    alphasparse_status_t s = band_finish(ctx, cand, covered, false, st);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS || ctx->band.rows == 0) return s;
    for (const BandCand &c : cand)
        for (int64_t t = c.t0; t < c.t1; t++) skip[(size_t)t] = 1;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t band_build_rows(DeviceCtx *ctx, const int *h_ptr, const std::vector<int> &rows, cudaStream_t st) {
    std::vector<BandCand> cand;
    cand.reserve(rows.size());
    int64_t covered = 0;
    for (int r : rows) {
        cand.push_back({r, h_ptr[r], h_ptr[r + 1], 0, 0});
        covered += (int64_t)h_ptr[r + 1] - h_ptr[r];
    }
    alphasparse_status_t s = band_finish(ctx, cand, covered, true, st);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS && ctx->band.rows > 0) ctx->band.whole_rows = true;
    return s;
}

template <typename K, typename T>
static void launch_band_as(K kernel, int threads, std::atomic<size_t> &granted, DeviceCtx *ctx, const T *x,
                           cudaStream_t st) {
    const BandTables &b = ctx->band;
    const size_t smem = sizeof(T) * (size_t)b.width;
    if (smem > 48 * 1024 && granted.load() < smem) {  // the opt-in limit belongs to the kernel: only ever raise it
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess)
            granted.store(200 * 1024);
    }
    const dim3 grid((unsigned)b.bands, (unsigned)b.splits);
    kernel<<<grid, threads, smem, st>>>((int)ctx->cols, b.width, b.bands, b.rows, b.chunk, b.d_seg, ctx->d_col,
                                        static_cast<const T *>(ctx->d_val), x, static_cast<T *>(b.d_partial),
                                        ctx->d_status);
    count_launch();
}

template <typename K, typename T>
static void launch_band_packed_as(K kernel, std::atomic<size_t> &granted, DeviceCtx *ctx, const T *x, cudaStream_t st) {
    const BandTables &b = ctx->band;
    const size_t smem = sizeof(T) * (size_t)b.width;
    if (smem > 48 * 1024 && granted.load() < smem) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) == cudaSuccess)
            granted.store(200 * 1024);
    }
    const dim3 grid((unsigned)b.bands, (unsigned)b.splits);
    kernel<<<grid, kBandThreads, smem, st>>>((int)ctx->cols, b.width, b.bands, b.rows, b.chunk, b.d_pk_start, b.d_pk_col,
                                             static_cast<const T *>(b.d_pk_val), x, static_cast<T *>(b.d_partial),
                                             ctx->d_status);
    count_launch();
}

template <typename T>
static void launch_band_packed(DeviceCtx *ctx, const T *x, cudaStream_t st) {
    static std::atomic<size_t> granted[2] = {};
    if (option(kOptBandVariant) == 1)
        launch_band_packed_as(spmv_band_packed_kernel<T, 8, 2, 2, kBandThreads>, granted[1], ctx, x, st);
    else
        launch_band_packed_as(spmv_band_packed_kernel<T, 8, 2, 1, kBandThreads>, granted[0], ctx, x, st);
}

template <typename T>
void launch_band(DeviceCtx *ctx, const T *x, cudaStream_t st) {
    if (ctx->band.pk_quads > 0) {
        launch_band_packed<T>(ctx, x, st);
        return;
    }
    static std::atomic<size_t> granted[2] = {};
    if (option(kOptBandVariant) == 1)
        launch_band_as(spmv_band_quad_kernel<T, 4, 2, 1, kBandThreads>, kBandThreads, granted[1], ctx, x, st);
    else
        launch_band_as(spmv_band_quad_kernel<T, 8, 1, 2, kBandThreads>, kBandThreads, granted[0], ctx, x, st);
}

template <typename T>
void launch_band_reduce(DeviceCtx *ctx, T alpha, T beta, T *y, cudaStream_t st, const PeerPush *push) {
    const BandTables &b = ctx->band;
    const unsigned blocks = (unsigned)(((long long)b.rows * 32 + 255) / 256);
    const T *partial = static_cast<const T *>(b.d_partial);
    const PeerPush none{};
    if (b.whole_rows)
        spmv_band_reduce_kernel<T, true><<<blocks, 256, 0, st>>>(b.rows, b.bands, b.d_row, partial, y, alpha, beta,
                                                                 push ? *push : none);
    else
        spmv_band_reduce_kernel<T, false><<<blocks, 256, 0, st>>>(b.rows, b.bands, b.d_row, partial, y, alpha, beta, none);
    count_launch();
}

template void launch_band<float>(DeviceCtx *, const float *, cudaStream_t);
template void launch_band<double>(DeviceCtx *, const double *, cudaStream_t);
template void launch_band_reduce<float>(DeviceCtx *, float, float, float *, cudaStream_t, const PeerPush *);
template void launch_band_reduce<double>(DeviceCtx *, double, double, double *, cudaStream_t, const PeerPush *);

}  // namespace asb
