// Row bins for skewed matrices (sm_100a): one kernel shape per class of row length.
//
// A matrix whose row lengths span five orders of magnitude (half the rows hold one element, a few
// hundred hold 200,000) has no single good kernel shape.  The analysis therefore sorts the rows into
// bins once per handle -- lists of row numbers; the CSR arrays stay as the caller gave them -- and a
// product launches one kernel per non-empty bin on the same stream:
//
//   short   rows of at most 16 elements (option bin_short; empty rows included): one thread per row, straight
//           from the CSR arrays.  Neighbouring threads take neighbouring rows, whose elements are
//           neighbours in memory, so the loads of a warp stay within a few cache lines.
//   mid     three lists (up to 32, up to 256, longer): a group of 4 / 16 / 32 lanes per row, every lane
//           taking whole aligned quads of the row (16-byte loads of col and val) and masking what lies
//           outside it, warp-shuffle reduction.
//   long    rows long enough to average several elements per column band: the column-band kernel
//           (spmv_band.cu), which gathers from a band of x staged in shared memory.
//
// Every row is written by exactly one thread of exactly one kernel, sums are formed in a fixed order:
// results are bit-identical from call to call.  Arithmetic as defined by the reference's gemv kernel,
// src/plain/kernel/level2/mv/gemv/gemv_x_csr_plain.c:4-24.  The reference's device build chooses one
// sub-wavefront width per matrix from nnz / m (src/kernel/dcu/level2/mv/csrmv/dcu_gemv_vector.h:59-182);
// its adaptive variant cuts the rows into blocks of similar work at analysis time
// (src/util_cpp/alphasparse_dcu_x_csrmv_analysis.cpp:58-267).  This is the same idea with other bins.
#include <algorithm>
#include <type_traits>
#include <vector>

#include "internal.h"

namespace asb {

// Delivery of finished rows to the peers; kernels instantiated without PUSH carry no such argument at all.
struct BinNoPush {};
template <bool PUSH>
using BinPushArg = typename std::conditional<PUSH, PeerPush, BinNoPush>::type;
template <typename T>
__device__ __forceinline__ void bin_push_row(const PeerPush &push, long long r, T out) {
#pragma unroll 1
    for (int p = 0; p < push.n; p++) static_cast<T *>(push.dst[p])[push.row_off + r] = out;
}
template <typename T>
__device__ __forceinline__ void bin_push_row(const BinNoPush &, long long, T) {}

// ---- short rows: one thread per row -------------------------------------------------------------
// A thread takes R rows, 256 rows apart (so that every load instruction of a warp covers consecutive rows), and walks
// them together, two elements of each per step.  R = 1 is what is used: see launch_bins.
// PUSH: every finished row also goes into the next-x buffer of every GPU of the row partition (peer-mapped pointers,
// plain stores over NVLink; see PeerPush).  Neighbouring lanes hold neighbouring rows, so these are coalesced.
template <typename T, int R, bool HAS_BETA, bool PUSH>
__global__ void __launch_bounds__(256)
    spmv_short_kernel(int rows, int limit, const int *__restrict__ row_ptr, const int *__restrict__ col,
                      const T *__restrict__ val, const T *__restrict__ x, T *__restrict__ y, T alpha, T beta,
                      const __grid_constant__ BinPushArg<PUSH> push) {
    const long long base = (long long)blockIdx.x * (256 * R) + threadIdx.x;
    int s[R], n[R];
    T acc[R];
    int longest = 0;
#pragma unroll
    for (int u = 0; u < R; u++) {
        const long long r = base + (long long)u * 256;
        s[u] = 0, n[u] = -1, acc[u] = T(0);
        if (r < rows) {
            s[u] = __ldg(row_ptr + r);
            n[u] = __ldg(row_ptr + r + 1) - s[u];
            if (n[u] > limit) n[u] = -1;  // a longer row: some other bin writes it
        }
        longest = max(longest, n[u]);
    }
    for (int j = 0; j < longest; j += 2) {
        int c[R][2];
        T v[R][2];
#pragma unroll
        for (int u = 0; u < R; u++)
#pragma unroll
            for (int w = 0; w < 2; w++)
                if (j + w < n[u]) {
                    c[u][w] = __ldg(col + s[u] + j + w);
                    v[u][w] = __ldg(val + s[u] + j + w);
                }
#pragma unroll
        for (int u = 0; u < R; u++)
#pragma unroll
            for (int w = 0; w < 2; w++)
                if (j + w < n[u]) acc[u] = fma(v[u][w], __ldg(x + c[u][w]), acc[u]);
    }
#pragma unroll
    for (int u = 0; u < R; u++) {
        const long long r = base + (long long)u * 256;
        if (n[u] >= 0) {
            T out = alpha * acc[u];
            if (HAS_BETA) out = fma(beta, y[r], out);
            __stcs(y + r, out);
            bin_push_row<T>(push, r, out);
        }
    }
}

// ---- mid rows: a lane group per listed row ------------------------------------------------------
template <typename T>
struct BinQuad {
    T v[4];
};
__device__ __forceinline__ BinQuad<float> bin_load_val(const float *__restrict__ val, int q) {
    const float4 t = __ldcs(reinterpret_cast<const float4 *>(val) + q);
    return {{t.x, t.y, t.z, t.w}};
}
__device__ __forceinline__ BinQuad<double> bin_load_val(const double *__restrict__ val, int q) {
    const double2 a = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q);
    const double2 b = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q + 1);
    return {{a.x, a.y, b.x, b.y}};
}

template <typename T>
__device__ __forceinline__ T bin_quad_dot(const int4 c, const BinQuad<T> &v, int base, int s, int e,
                                          const T *__restrict__ x) {
    // elements of the quad outside [s, e) belong to a neighbouring row (or to the zero tail of the arrays)
    T acc = T(0);
    if (base + 0 >= s && base + 0 < e) acc = fma(v.v[0], __ldg(x + c.x), acc);
    if (base + 1 >= s && base + 1 < e) acc = fma(v.v[1], __ldg(x + c.y), acc);
    if (base + 2 >= s && base + 2 < e) acc = fma(v.v[2], __ldg(x + c.z), acc);
    if (base + 3 >= s && base + 3 < e) acc = fma(v.v[3], __ldg(x + c.w), acc);
    return acc;
}

// 256 threads = 256 / LANES groups; group g of block b takes list entries b * (GROUPS * R) + g + u * GROUPS,
// u = 0 .. R-1: R rows in flight per group.  U quads per row are requested before any is consumed.
template <typename T, int LANES, int R, int U, bool HAS_BETA, bool PUSH>
__global__ void __launch_bounds__(256)
    spmv_rowlist_kernel(int count, const int *__restrict__ list, const int *__restrict__ row_ptr,
                        const int *__restrict__ row_end, const int *__restrict__ col, const T *__restrict__ val,
                        const T *__restrict__ x, T *__restrict__ y, T alpha, T beta,
                        const __grid_constant__ BinPushArg<PUSH> push) {
    constexpr int GROUPS = 256 / LANES;
    const int lane = threadIdx.x % LANES, grp = threadIdx.x / LANES;
    const long long i0 = (long long)blockIdx.x * (GROUPS * R) + grp;
    int row[R], s[R], e[R], q[R];
    T sum[R];
#pragma unroll
    for (int u = 0; u < R; u++) {
        const long long i = i0 + (long long)u * GROUPS;
        row[u] = -1, s[u] = 0, e[u] = 0, sum[u] = T(0);
        if (i < count) {
            row[u] = __ldg(list + i);
            s[u] = __ldg(row_ptr + row[u]);  // the whole row, or its elements inside one column block (launch_list)
            e[u] = __ldg(row_end + row[u]);
        }
        q[u] = (s[u] >> 2) + lane;
    }
    bool more = true;
    while (more) {
        int4 cc[R][U];
        BinQuad<T> vv[R][U];
#pragma unroll
        for (int u = 0; u < R; u++)
#pragma unroll
            for (int w = 0; w < U; w++) {
                const int qq = q[u] + w * LANES;
                if ((qq << 2) < e[u]) {
                    cc[u][w] = __ldcs(reinterpret_cast<const int4 *>(col) + qq);
                    vv[u][w] = bin_load_val(val, qq);
                }
            }
        more = false;
#pragma unroll
        for (int u = 0; u < R; u++) {
#pragma unroll
            for (int w = 0; w < U; w++) {
                const int qq = q[u] + w * LANES;
                if ((qq << 2) < e[u]) sum[u] += bin_quad_dot(cc[u][w], vv[u][w], qq << 2, s[u], e[u], x);
            }
            q[u] += LANES * U;
            more |= (q[u] << 2) < e[u];
        }
    }
#pragma unroll
    for (int u = 0; u < R; u++) {
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], o);
        if (lane == 0 && row[u] >= 0) {
            T out = alpha * sum[u];
            if (HAS_BETA) out = fma(beta, y[row[u]], out);
            y[row[u]] = out;
            bin_push_row<T>(push, row[u], out);  // the listed rows are few and far apart: single stores
        }
    }
}

// ---- analysis ------------------------------------------------------------------------------------

void bins_destroy(RowBins &b) {
    cudaFree(b.d_list);
    for (int k = 0; k < kMidBins; k++) {
        if (b.side[k]) cudaStreamDestroy(b.side[k]);
        if (b.ev_join[k]) cudaEventDestroy(b.ev_join[k]);
    }
    if (b.ev_fork) cudaEventDestroy(b.ev_fork);
    b = RowBins{};
}

// Sorts the rows into bins.  `h_ptr` is the host copy of the row offsets (rows + 1 entries).  Rows of at least
// `long_min` elements are left to the caller (the column-band tables take them); returns them in `long_rows`.
alphasparse_status_t bins_build(DeviceCtx *ctx, const int *h_ptr, int64_t long_min, std::vector<int> &long_rows,
                                cudaStream_t st) {
    RowBins b;
    b.short_limit = (int)std::max<int64_t>(0, option(kOptBinShort));
    const int bounds[kMidBins] = {(int)option(kOptBinMid0), (int)option(kOptBinMid1), INT32_MAX};
    std::vector<int> lists[kMidBins];
    long_rows.clear();
    for (int64_t r = 0; r < ctx->rows; r++) {
        const int64_t n = (int64_t)h_ptr[r + 1] - h_ptr[r];
        if (n <= b.short_limit) {
            b.short_rows++;
            continue;
        }
        if (n >= long_min) {
            long_rows.push_back((int)r);
            continue;
        }
        for (int k = 0; k < kMidBins; k++)
            if (n <= bounds[k]) {
                lists[k].push_back((int)r);
                break;
            }
    }
    if (option(kOptBinSort)) {
        // A block of the list kernels is busy until its longest row is done: longest rows first, so that the rows
        // of one block are of about one length and the blocks that start last are the short ones.
        // (a counting sort over the lengths, stable in the row number: linear in the list, whatever its size)
        for (int k = 1; k < kMidBins; k++) {
            std::vector<int> &l = lists[k];
            if (l.size() < 2) continue;
            int lo = INT32_MAX, hi = 0;
            for (int r : l) {
                const int n = h_ptr[r + 1] - h_ptr[r];
                lo = std::min(lo, n), hi = std::max(hi, n);
            }
            std::vector<size_t> first((size_t)(hi - lo) + 2, 0);  // first[hi - n + 1]: rows of length n, longest first
            for (int r : l) first[(size_t)(hi - (h_ptr[r + 1] - h_ptr[r])) + 1]++;
            for (size_t i = 1; i < first.size(); i++) first[i] += first[i - 1];
            std::vector<int> sorted(l.size());
            for (int r : l) sorted[first[(size_t)(hi - (h_ptr[r + 1] - h_ptr[r]))]++] = r;
            l.swap(sorted);
        }
    }
    size_t total = 0;
    for (int k = 0; k < kMidBins; k++) {
        b.offset[k] = (int64_t)total;
        b.count[k] = (int64_t)lists[k].size();
        total += lists[k].size();
    }
    if (total > 0) {
        cudaError_t e = device_alloc(&b.d_list, sizeof(int) * total);
        if (e != cudaSuccess) {
            record_cuda_error(e, "device_alloc(&b.d_list, sizeof(int) * total)");
            return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
        }
        for (int k = 0; k < kMidBins && e == cudaSuccess; k++)
            if (!lists[k].empty())
                e = cudaMemcpyAsync(b.d_list + b.offset[k], lists[k].data(), sizeof(int) * lists[k].size(),
                                    cudaMemcpyHostToDevice, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);  // the vectors go out of scope
        if (e != cudaSuccess) {
            cudaFree(b.d_list);
            record_cuda_error(e, "row bins");
            return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
        }
    }
    if (option(kOptBinOverlap)) {
        // Each bin kernel alone leaves the SMs half idle at its tail (a few waves of blocks of uneven length);
        // on streams of their own the next one fills in.  They write disjoint rows of y.
        cudaError_t e = cudaEventCreateWithFlags(&b.ev_fork, cudaEventDisableTiming);
        for (int k = 0; k < kMidBins && e == cudaSuccess; k++) {
            if (b.count[k] == 0) continue;
            e = cudaStreamCreateWithFlags(&b.side[k], cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&b.ev_join[k], cudaEventDisableTiming);
        }
        if (e != cudaSuccess) {
            bins_destroy(b);
            record_cuda_error(e, "row bins");
            return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
        }
    }
    b.active = true;
    ctx->bins = b;
    ctx->device_bytes += (int64_t)(sizeof(int) * total);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- launch --------------------------------------------------------------------------------------

template <typename T, int LANES, int R, int U, bool PUSH>
static void launch_list(DeviceCtx *ctx, int k, T alpha, const T *x, T beta, T *y, cudaStream_t st,
                        const BinPushArg<PUSH> &push) {
    const RowBins &b = ctx->bins;
    if (b.count[k] == 0) return;
    if (b.side[k]) st = b.side[k];
    constexpr int per_block = (256 / LANES) * R;
    const unsigned blocks = (unsigned)((b.count[k] + per_block - 1) / per_block);
    const T *val = static_cast<const T *>(ctx->d_val);
    const int *list = b.d_list + b.offset[k];
    // Column blocks (an x that does not fit L2, see ctx_analyse): one launch per block over the elements of the listed
    // rows that fall into it; the first applies beta, the later ones add to y, the last one delivers (exchange calls).
    const int passes = ctx->mvb.d_split ? ctx->mvb.blocks : 1;
    for (int p = 0; p < passes; p++) {
        const int *lo = passes > 1 ? ctx->mvb.d_split + (size_t)p * ctx->rows : ctx->d_row_ptr;
        const int *hi = passes > 1 ? lo + ctx->rows : lo + 1;
        const T bp = p == 0 ? beta : T(1);
        if (PUSH && p + 1 < passes) {
            if (bp == T(0))
                spmv_rowlist_kernel<T, LANES, R, U, false, false><<<blocks, 256, 0, st>>>((int)b.count[k], list, lo, hi, ctx->d_col,
                                                                                         val, x, y, alpha, bp, BinNoPush{});
            else
                spmv_rowlist_kernel<T, LANES, R, U, true, false><<<blocks, 256, 0, st>>>((int)b.count[k], list, lo, hi, ctx->d_col,
                                                                                        val, x, y, alpha, bp, BinNoPush{});
        } else if (bp == T(0)) {
            spmv_rowlist_kernel<T, LANES, R, U, false, PUSH><<<blocks, 256, 0, st>>>((int)b.count[k], list, lo, hi, ctx->d_col, val,
                                                                                    x, y, alpha, bp, push);
        } else {
            spmv_rowlist_kernel<T, LANES, R, U, true, PUSH><<<blocks, 256, 0, st>>>((int)b.count[k], list, lo, hi, ctx->d_col, val,
                                                                                   x, y, alpha, bp, push);
        }
    }
    count_launch(passes);
}

template <typename T, bool PUSH>
static void launch_short(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y, cudaStream_t st,
                         const BinPushArg<PUSH> &push) {
    const RowBins &b = ctx->bins;
    const T *val = static_cast<const T *>(ctx->d_val);
    const unsigned blocks = (unsigned)((ctx->rows + 255) / 256);
    if (beta == T(0))
        spmv_short_kernel<T, 1, false, PUSH><<<blocks, 256, 0, st>>>((int)ctx->rows, b.short_limit, ctx->d_row_ptr,
                                                                     ctx->d_col, val, x, y, alpha, beta, push);
    else
        spmv_short_kernel<T, 1, true, PUSH><<<blocks, 256, 0, st>>>((int)ctx->rows, b.short_limit, ctx->d_row_ptr,
                                                                    ctx->d_col, val, x, y, alpha, beta, push);
    count_launch();
}

template <typename T, bool PUSH>
static void launch_bins_as(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y, cudaStream_t st,
                           const BinPushArg<PUSH> &push) {
    const RowBins &b = ctx->bins;
    if (b.ev_fork) {
        cudaEventRecord(b.ev_fork, st);
        for (int k = 0; k < kMidBins; k++)
            if (b.side[k]) cudaStreamWaitEvent(b.side[k], b.ev_fork, 0);
    }
    // the longest-running list first, so that the shorter kernels fill in behind it
    launch_list<T, 32, 1, 2, PUSH>(ctx, 2, alpha, x, beta, y, st, push);
    if (b.short_rows > 0) launch_short<T, PUSH>(ctx, alpha, x, beta, y, st, push);
    launch_list<T, 4, 2, 1, PUSH>(ctx, 0, alpha, x, beta, y, st, push);
    launch_list<T, 16, 2, 1, PUSH>(ctx, 1, alpha, x, beta, y, st, push);
    for (int k = 0; k < kMidBins; k++)
        if (b.side[k]) {
            cudaEventRecord(b.ev_join[k], b.side[k]);
            cudaStreamWaitEvent(st, b.ev_join[k], 0);
        }
}

// Short and mid rows of a binned handle (the long rows are the column-band kernel's).  With `push` every kernel
// also stores its rows into the peers' buffers as it finishes them: the exchange overlaps the product.
// Shapes from a sweep on B200 (power-law matrix): one row per thread / two rows per lane group at 32..48 registers
// beat every shape with more rows in flight per thread (4 rows per thread or group: 80..93 registers, 15..25 %
// slower): these kernels live on resident warps, not on loads per thread.
template <typename T>
void launch_bins(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y, cudaStream_t st, const PeerPush *push) {
    if (push) launch_bins_as<T, true>(ctx, alpha, x, beta, y, st, *push);
    else launch_bins_as<T, false>(ctx, alpha, x, beta, y, st, BinNoPush{});
}

template void launch_bins<float>(DeviceCtx *, float, const float *, float, float *, cudaStream_t, const PeerPush *);
template void launch_bins<double>(DeviceCtx *, double, const double *, double, double *, cudaStream_t, const PeerPush *);

}  // namespace asb
