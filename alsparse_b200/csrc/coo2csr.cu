// COO -> CSR on the GPU, for alphasparse_convert_csr on large COO handles.
//
// The reference sorts (row, column, value) records with a serial qsort and then counts rows
// (src/core/format/convert_csr_x_coo.c:14-81); minutes at 2^28 elements.  Here the same output --
// elements ordered by row then column, duplicates kept, in input order among equals (qsort leaves
// that unspecified) -- comes from a stable least-significant-digit radix sort of 64-bit keys
// (row << 32 | column) carrying the element's input position, 4 bits per pass over only the bits the
// matrix dimensions use, followed by one binary search per row for the offsets and one gather of the
// values.  Integer work, HBM-bound: every pass reads and writes 12 bytes per element.
#include <algorithm>

#include "internal.h"

namespace asb {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 8;  // consecutive elements per thread (blocked), so order = thread order
constexpr int kSortTile = kSortThreads * kSortItems;

__global__ void coo_keys_kernel(long long nnz, const int *__restrict__ ri, const int *__restrict__ ci, int rows,
                                int cols, unsigned long long *__restrict__ keys, unsigned *__restrict__ pos,
                                unsigned long long *__restrict__ bad) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    const int r = ri[i], c = ci[i];
    if (r < 0 || r >= rows || c < 0 || c >= cols) atomicAdd(bad, 1ull);
    keys[i] = ((unsigned long long)(unsigned)r << 32) | (unsigned)c;
    pos[i] = (unsigned)i;
}

// Per block: how many of its elements fall into each of the 16 digit values.  hist is digit-major
// (hist[d * blocks + b]) so that one exclusive scan over it yields every block's write offsets.
__global__ void __launch_bounds__(kSortThreads)
    radix_hist_kernel(long long n, const unsigned long long *__restrict__ keys, int shift, unsigned *__restrict__ hist) {
    __shared__ unsigned s_cnt[16];
    if (threadIdx.x < 16) s_cnt[threadIdx.x] = 0;
    __syncthreads();
    const long long base = (long long)blockIdx.x * kSortTile + (long long)threadIdx.x * kSortItems;
    unsigned local[16];
#pragma unroll
    for (int d = 0; d < 16; d++) local[d] = 0;
#pragma unroll
    for (int k = 0; k < kSortItems; k++)
        if (base + k < n) {
            const unsigned d = (unsigned)(keys[base + k] >> shift) & 15u;
#pragma unroll
            for (int q = 0; q < 16; q++) local[q] += (q == d);
        }
#pragma unroll
    for (int d = 0; d < 16; d++)
        if (local[d]) atomicAdd(&s_cnt[d], local[d]);
    __syncthreads();
    if (threadIdx.x < 16) hist[(size_t)threadIdx.x * gridDim.x + blockIdx.x] = s_cnt[threadIdx.x];
}

// Exclusive scan of n unsigned values in three steps (block sums, scan of the sums by one block, add).
constexpr int kScanThreads = 256, kScanItems = 16, kScanTile = kScanThreads * kScanItems;

__device__ __forceinline__ unsigned block_exclusive_scan(unsigned v, unsigned *total) {
    __shared__ unsigned s_warp[kScanThreads / 32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    unsigned inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (lane == 31) s_warp[wid] = inc;
    __syncthreads();
    unsigned before = 0, all = 0;
    for (int w = 0; w < kScanThreads / 32; w++) {
        if (w < wid) before += s_warp[w];
        all += s_warp[w];
    }
    __syncthreads();
    if (total) *total = all;
    return before + inc - v;
}

__global__ void __launch_bounds__(kScanThreads)
    scan_sums_kernel(long long n, const unsigned *__restrict__ in, unsigned *__restrict__ sums) {
    const long long base = (long long)blockIdx.x * kScanTile + (long long)threadIdx.x * kScanItems;
    unsigned s = 0;
    for (int k = 0; k < kScanItems; k++)
        if (base + k < n) s += in[base + k];
    unsigned total;
    block_exclusive_scan(s, &total);
    if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanThreads) scan_top_kernel(int nblocks, unsigned *__restrict__ sums) {
    unsigned carry = 0;  // one block walks the block sums, kScanThreads at a time
    for (int base = 0; base < nblocks; base += kScanThreads) {
        const int i = base + threadIdx.x;
        const unsigned v = i < nblocks ? sums[i] : 0;
        unsigned total;
        const unsigned ex = block_exclusive_scan(v, &total);
        if (i < nblocks) sums[i] = carry + ex;
        carry += total;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kScanThreads)
    scan_apply_kernel(long long n, unsigned *__restrict__ data, const unsigned *__restrict__ sums) {
    const long long base = (long long)blockIdx.x * kScanTile + (long long)threadIdx.x * kScanItems;
    unsigned v[kScanItems], s = 0;
    for (int k = 0; k < kScanItems; k++) {
        v[k] = base + k < n ? data[base + k] : 0;
        s += v[k];
    }
    unsigned run = sums[blockIdx.x] + block_exclusive_scan(s, nullptr);
    for (int k = 0; k < kScanItems; k++)
        if (base + k < n) {
            data[base + k] = run;
            run += v[k];
        }
}

// Stable scatter of one pass: element order inside a block is thread order then item order, so the
// rank of an element among the block's elements with the same digit is (same-digit elements of
// earlier threads) + (same-digit elements earlier in this thread).
__global__ void __launch_bounds__(kSortThreads)
    radix_scatter_kernel(long long n, const unsigned long long *__restrict__ keys_in,
                         const unsigned *__restrict__ pos_in, int shift, const unsigned *__restrict__ offs,
                         unsigned long long *__restrict__ keys_out, unsigned *__restrict__ pos_out) {
    __shared__ unsigned s_cnt[16][kSortThreads + 1];
    const int t = threadIdx.x;
    const long long base = (long long)blockIdx.x * kSortTile + (long long)t * kSortItems;
    unsigned long long key[kSortItems];
    unsigned local[16];
#pragma unroll
    for (int d = 0; d < 16; d++) local[d] = 0;
#pragma unroll
    for (int k = 0; k < kSortItems; k++) {
        key[k] = base + k < n ? keys_in[base + k] : ~0ull;
        if (base + k < n) {
            const unsigned d = (unsigned)(key[k] >> shift) & 15u;
#pragma unroll
            for (int q = 0; q < 16; q++) local[q] += (q == d);
        }
    }
#pragma unroll
    for (int d = 0; d < 16; d++) s_cnt[d][t] = local[d];
    __syncthreads();
    // warp w turns the counts of digits 2w and 2w+1 into exclusive prefixes over the 256 threads
    {
        const int lane = t & 31, w = t >> 5;
        for (int d = 2 * w; d < 2 * w + 2; d++) {
            unsigned carry = 0;
            for (int seg = 0; seg < kSortThreads; seg += 32) {
                const unsigned v = s_cnt[d][seg + lane];
                unsigned inc = v;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const unsigned u = __shfl_up_sync(0xffffffffu, inc, o);
                    if (lane >= o) inc += u;
                }
                s_cnt[d][seg + lane] = carry + inc - v;
                carry += __shfl_sync(0xffffffffu, inc, 31);
            }
        }
    }
    __syncthreads();
    unsigned dst[16];
#pragma unroll
    for (int d = 0; d < 16; d++) dst[d] = offs[(size_t)d * gridDim.x + blockIdx.x] + s_cnt[d][t];
#pragma unroll
    for (int k = 0; k < kSortItems; k++)
        if (base + k < n) {
            const unsigned d = (unsigned)(key[k] >> shift) & 15u;
            unsigned where = 0;
#pragma unroll
            for (int q = 0; q < 16; q++)
                if (q == d) where = dst[q]++;
            keys_out[where] = key[k];
            pos_out[where] = pos_in[base + k];
        }
}

// ptr[r] = first sorted element whose row is >= r (r = 0 .. rows); columns and values in sorted order.
template <typename T>
__global__ void csr_from_sorted_kernel(long long nnz, int rows, const unsigned long long *__restrict__ keys,
                                       const unsigned *__restrict__ pos, const T *__restrict__ vals_in,
                                       int *__restrict__ ptr, int *__restrict__ col, T *__restrict__ val) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= rows) {
        long long lo = 0, hi = nnz;
        while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if ((long long)(keys[mid] >> 32) < i) lo = mid + 1;
            else hi = mid;
        }
        ptr[i] = (int)lo;
    }
    if (i < nnz) {
        col[i] = (int)(unsigned)keys[i];
        val[i] = vals_in[pos[i]];
    }
}

static int bits_for(int64_t n) {
    int b = 1;
    while (b < 31 && (1ll << b) < n) b++;
    return b;
}

static alphasparse_status_t device_exclusive_scan(unsigned *d_data, long long n, unsigned *d_sums, cudaStream_t st) {
    const int nb = (int)((n + kScanTile - 1) / kScanTile);
    scan_sums_kernel<<<nb, kScanThreads, 0, st>>>(n, d_data, d_sums);
    scan_top_kernel<<<1, kScanThreads, 0, st>>>(nb, d_sums);
    scan_apply_kernel<<<nb, kScanThreads, 0, st>>>(n, d_data, d_sums);
    count_launch(3);
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Host COO arrays in, HOST 3-array CSR out (caller-provided buffers of rows+1 / nnz / nnz elements).
// All device memory is temporary.  Returns INVALID_VALUE when an index is out of range.
template <typename T>
alphasparse_status_t coo_to_csr_device(int64_t rows, int64_t cols, int64_t nnz, const int *ri, const int *ci,
                                       const T *v, int *out_ptr, int *out_col, T *out_val) {
    cudaStream_t st = current_stream();
    const long long nblocks = (nnz + kSortTile - 1) / kSortTile;
    const long long hist_n = 16 * nblocks;
    const int scan_blocks = (int)((hist_n + kScanTile - 1) / kScanTile);
    int *d_ri = nullptr, *d_ci = nullptr, *d_ptr = nullptr, *d_col = nullptr;
    T *d_v = nullptr, *d_val = nullptr;
    unsigned long long *d_keys[2] = {nullptr, nullptr}, *d_bad = nullptr;
    unsigned *d_pos[2] = {nullptr, nullptr}, *d_hist = nullptr, *d_sums = nullptr;
    alphasparse_status_t status = ALPHA_SPARSE_STATUS_SUCCESS;
    auto release = [&]() {
        cudaFree(d_ri), cudaFree(d_ci), cudaFree(d_ptr), cudaFree(d_col), cudaFree(d_v), cudaFree(d_val);
        cudaFree(d_keys[0]), cudaFree(d_keys[1]), cudaFree(d_pos[0]), cudaFree(d_pos[1]);
        cudaFree(d_hist), cudaFree(d_sums), cudaFree(d_bad);
    };
#define TRY(expr, code)                       \
    do {                                      \
        cudaError_t _e = (expr);              \
        if (_e != cudaSuccess) {              \
            record_cuda_error(_e, #expr);     \
            release();                        \
            return (code);                    \
        }                                     \
    } while (0)
    const size_t n = (size_t)nnz;
    TRY(device_alloc(&d_ri, sizeof(int) * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_ci, sizeof(int) * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_v, sizeof(T) * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_keys[0], 8 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_keys[1], 8 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_pos[0], 4 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_pos[1], 4 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_hist, sizeof(unsigned) * (size_t)hist_n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_sums, sizeof(unsigned) * (size_t)(scan_blocks + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_bad, 8), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(cudaMemsetAsync(d_bad, 0, 8, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(d_ri, ri, sizeof(int) * n, cudaMemcpyHostToDevice, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(d_ci, ci, sizeof(int) * n, cudaMemcpyHostToDevice, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(d_v, v, sizeof(T) * n, cudaMemcpyHostToDevice, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);

    coo_keys_kernel<<<(unsigned)((nnz + 255) / 256), 256, 0, st>>>(nnz, d_ri, d_ci, (int)rows, (int)cols, d_keys[0],
                                                                  d_pos[0], d_bad);
    count_launch();
    int cur = 0;
    const int col_bits = bits_for(cols), row_bits = bits_for(rows);
    for (int part = 0; part < 2 && status == ALPHA_SPARSE_STATUS_SUCCESS; part++) {
        const int first = part == 0 ? 0 : 32, nbits = part == 0 ? col_bits : row_bits;
        for (int shift = first; shift < first + nbits; shift += 4) {
            radix_hist_kernel<<<(unsigned)nblocks, kSortThreads, 0, st>>>(nnz, d_keys[cur], shift, d_hist);
            count_launch();
            status = device_exclusive_scan(d_hist, hist_n, d_sums, st);
            if (status != ALPHA_SPARSE_STATUS_SUCCESS) break;
            radix_scatter_kernel<<<(unsigned)nblocks, kSortThreads, 0, st>>>(nnz, d_keys[cur], d_pos[cur], shift,
                                                                            d_hist, d_keys[cur ^ 1], d_pos[cur ^ 1]);
            count_launch();
            cur ^= 1;
        }
    }
    if (status != ALPHA_SPARSE_STATUS_SUCCESS) {
        release();
        return status;
    }
    // the input index arrays are no longer needed: reuse them for the result
    d_ptr = nullptr;
    TRY(device_alloc(&d_ptr, sizeof(int) * (size_t)(rows + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_val, sizeof(T) * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    d_col = d_ri;
    d_ri = nullptr;
    const long long work = std::max<long long>(nnz, rows + 1);
    csr_from_sorted_kernel<T><<<(unsigned)((work + 255) / 256), 256, 0, st>>>(nnz, (int)rows, d_keys[cur], d_pos[cur],
                                                                            d_v, d_ptr, d_col, d_val);
    count_launch();
    TRY(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    unsigned long long bad = 0;
    TRY(cudaMemcpyAsync(&bad, d_bad, 8, cudaMemcpyDeviceToHost, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(out_ptr, d_ptr, sizeof(int) * (size_t)(rows + 1), cudaMemcpyDeviceToHost, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(out_col, d_col, sizeof(int) * n, cudaMemcpyDeviceToHost, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemcpyAsync(out_val, d_val, sizeof(T) * n, cudaMemcpyDeviceToHost, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
#undef TRY
    release();
    return bad ? ALPHA_SPARSE_STATUS_INVALID_VALUE : ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- A^T from the device copy of A ------------------------------------------------------------------
//
// The reference materialises the transpose on the host with a counting sort (src/core/format/transpose_x_csr.c:7-62)
// and its transposed gemv adds the elements of a column of A in ascending row order
// (src/plain/kernel/level2/mv/gemv/gemv_x_csr_trans_plain.c:14-25).  Here the same arrays come from the device copy
// without touching the host: the stored elements, taken in storage order (rows ascending), are sorted by column
// with the stable radix sort above (keys = column, over the bits the column count uses; the payload is the
// element's position), so the elements of a column come out by ascending row; the row of each is found again by a
// binary search in the row offsets, the new offsets by a binary search in the sorted columns.
__global__ void transpose_keys_kernel(long long nnz, const int *__restrict__ col, unsigned long long *__restrict__ keys,
                                      unsigned *__restrict__ pos) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    keys[i] = (unsigned)col[i];
    pos[i] = (unsigned)i;
}

template <typename T>
__global__ void transpose_fill_kernel(long long nnz, int rows, int cols, const unsigned long long *__restrict__ keys,
                                      const unsigned *__restrict__ pos, const int *__restrict__ row_ptr,
                                      const T *__restrict__ val, int *__restrict__ tptr, int *__restrict__ tcol,
                                      T *__restrict__ tval) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= cols) {  // first sorted element whose column is >= i
        long long lo = 0, hi = nnz;
        while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if ((long long)(unsigned)keys[mid] < i) lo = mid + 1;
            else hi = mid;
        }
        tptr[i] = (int)lo;
    }
    if (i < nnz) {
        const int k = (int)pos[i];
        int lo = 0, hi = rows;  // last row whose first element is <= k (empty rows share an offset: take the last)
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (row_ptr[mid] <= k) lo = mid;
            else hi = mid;
        }
        tcol[i] = lo;
        tval[i] = val[k];
    }
}

// Device arrays of A^T in the layout ctx_adopt expects (cols + 1 + 4 offsets, nnz + kTailPad columns and values,
// tails zeroed), allocated here and handed to the caller.
template <typename T>
alphasparse_status_t transpose_csr_device(const DeviceCtx *c, int **out_ptr, int **out_col, T **out_val) {
    cudaStream_t st = current_stream();
    const int64_t nnz = c->nnz, rows = c->rows, cols = c->cols;
    const long long nblocks = std::max<long long>(1, (nnz + kSortTile - 1) / kSortTile);
    const long long hist_n = 16 * nblocks;
    const int scan_blocks = (int)((hist_n + kScanTile - 1) / kScanTile);
    unsigned long long *d_keys[2] = {nullptr, nullptr};
    unsigned *d_pos[2] = {nullptr, nullptr}, *d_hist = nullptr, *d_sums = nullptr;
    int *tptr = nullptr, *tcol = nullptr;
    T *tval = nullptr;
    auto release = [&](bool all) {
        cudaFree(d_keys[0]), cudaFree(d_keys[1]), cudaFree(d_pos[0]), cudaFree(d_pos[1]), cudaFree(d_hist), cudaFree(d_sums);
        if (all) cudaFree(tptr), cudaFree(tcol), cudaFree(tval);
    };
#define TRY(expr, code)                   \
    do {                                  \
        cudaError_t _e = (expr);          \
        if (_e != cudaSuccess) {          \
            record_cuda_error(_e, #expr); \
            release(true);                \
            return (code);                \
        }                                 \
    } while (0)
    const size_t n = (size_t)nnz, padded = n + kTailPad;
    TRY(device_alloc(&tptr, sizeof(int) * (size_t)(cols + 1 + 4)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&tcol, sizeof(int) * padded), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&tval, sizeof(T) * padded), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(cudaMemsetAsync(tptr, 0, sizeof(int) * (size_t)(cols + 1 + 4), st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemsetAsync(tcol + n, 0, sizeof(int) * kTailPad, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemsetAsync(tval + n, 0, sizeof(T) * kTailPad, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    if (nnz > 0) {
        TRY(device_alloc(&d_keys[0], 8 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_keys[1], 8 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_pos[0], 4 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_pos[1], 4 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_hist, sizeof(unsigned) * (size_t)hist_n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_sums, sizeof(unsigned) * (size_t)(scan_blocks + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        transpose_keys_kernel<<<(unsigned)((nnz + 255) / 256), 256, 0, st>>>(nnz, c->d_col, d_keys[0], d_pos[0]);
        count_launch();
        int cur = 0;
        const int col_bits = bits_for(cols);
        for (int shift = 0; shift < col_bits; shift += 4) {
            radix_hist_kernel<<<(unsigned)nblocks, kSortThreads, 0, st>>>(nnz, d_keys[cur], shift, d_hist);
            count_launch();
            alphasparse_status_t s = device_exclusive_scan(d_hist, hist_n, d_sums, st);
            if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
                release(true);
                return s;
            }
            radix_scatter_kernel<<<(unsigned)nblocks, kSortThreads, 0, st>>>(nnz, d_keys[cur], d_pos[cur], shift, d_hist,
                                                                            d_keys[cur ^ 1], d_pos[cur ^ 1]);
            count_launch();
            cur ^= 1;
        }
        const long long work = std::max<long long>(nnz, cols + 1);
        transpose_fill_kernel<T><<<(unsigned)((work + 255) / 256), 256, 0, st>>>(
            nnz, (int)rows, (int)cols, d_keys[cur], d_pos[cur], c->d_row_ptr, static_cast<const T *>(c->d_val), tptr, tcol,
            tval);
        count_launch();
        TRY(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }
    TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
#undef TRY
    release(false);
    *out_ptr = tptr, *out_col = tcol, *out_val = tval;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- matrices derived from the device copy of A for structured descriptors -----------------------------
//
// What a SYMMETRIC / TRIANGULAR / DIAGONAL descriptor makes of the stored matrix (the reference's symv / trmv /
// diagmv and symm / trmm / diagmm kernels, src/plain/kernel/level2/mv/{symv,trmv,diagmv},
// src/plain/kernel/level3/mm/{symm,trmm,diagmm}) is an ordinary matrix: the kept triangle, its mirror image for
// SYMMETRIC, its transpose for TRIANGULAR with op = TRANSPOSE, an explicit unit diagonal, or only the diagonal.
// Every stored element emits 0, 1 or 2 (row, column) keys, an exclusive scan places them, the stable radix sort
// orders them by (row, column) -- equal pairs keep storage order -- and the values are gathered at the end.
// Payload of a key: the position of the stored element, or kUnitPayload for an explicit 1 on the diagonal.
constexpr unsigned kUnitPayload = 0xffffffffu;

struct DeriveRule {
    int type;       // ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC / TRIANGULAR / DIAGONAL
    int upper;      // kept triangle
    int unit;       // unit diagonal: stored diagonal entries are ignored
    int flip;       // TRIANGULAR under op = TRANSPOSE: (i, j) becomes (j, i)
    int diag_rule;  // DIAGONAL, rows storing their diagonal more than once: 0 first entry, 1 all, 2 last
};

__device__ __forceinline__ int derive_row_of(const int *__restrict__ row_ptr, int rows, int k) {
    int lo = 0, hi = rows;  // last row whose first element is <= k (empty rows share an offset: take the last)
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (row_ptr[mid] <= k) lo = mid;
        else hi = mid;
    }
    return lo;
}

// DIAGONAL with the first / last rule: the smallest / largest position of a stored diagonal entry per row.
__global__ void derive_diag_pick_kernel(long long nnz, int rows, const int *__restrict__ row_ptr,
                                        const int *__restrict__ col, int last, int *__restrict__ pick) {
    const long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= nnz) return;
    const int i = derive_row_of(row_ptr, rows, (int)k);
    if (col[k] != i) return;
    if (last) atomicMax(pick + i, (int)k);
    else atomicMin(pick + i, (int)k);
}

__device__ __forceinline__ unsigned derive_emits(const DeriveRule &r, int i, int j, int k, const int *__restrict__ pick) {
    if (r.type == ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL) {
        if (r.unit || j != i) return 0;
        return r.diag_rule == 1 || pick[i] == k ? 1u : 0u;
    }
    const bool off = r.upper ? j > i : j < i;
    if (off) return r.type == ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC ? 2u : 1u;
    return j == i && !r.unit ? 1u : 0u;
}

__global__ void derive_count_kernel(long long nnz, int rows, const int *__restrict__ row_ptr, const int *__restrict__ col,
                                    DeriveRule rule, const int *__restrict__ pick, unsigned *__restrict__ count) {
    const long long k = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= nnz) return;
    const int i = derive_row_of(row_ptr, rows, (int)k);
    count[k] = derive_emits(rule, i, col[k], (int)k, pick);
}

// `offset` holds the exclusive scan of the counts; the explicit unit diagonal takes the first `rows` places.
__global__ void derive_emit_kernel(long long nnz, int rows, const int *__restrict__ row_ptr, const int *__restrict__ col,
                                   DeriveRule rule, const int *__restrict__ pick, const unsigned *__restrict__ offset,
                                   unsigned long long *__restrict__ keys, unsigned *__restrict__ pos) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned first = rule.unit ? (unsigned)rows : 0u;
    if (rule.unit && t < rows) {
        keys[t] = ((unsigned long long)(unsigned)t << 32) | (unsigned)t;
        pos[t] = kUnitPayload;
    }
    if (t >= nnz) return;
    const int k = (int)t, i = derive_row_of(row_ptr, rows, k), j = col[k];
    const unsigned n = derive_emits(rule, i, j, k, pick);
    if (n == 0) return;
    const unsigned o = first + offset[k];
    const bool flip = rule.flip && j != i;
    keys[o] = flip ? ((unsigned long long)(unsigned)j << 32) | (unsigned)i : ((unsigned long long)(unsigned)i << 32) | (unsigned)j;
    pos[o] = (unsigned)k;
    if (n == 2) {
        keys[o + 1] = ((unsigned long long)(unsigned)j << 32) | (unsigned)i;
        pos[o + 1] = (unsigned)k;
    }
}

template <typename T>
__global__ void derive_fill_kernel(long long m, int rows, const unsigned long long *__restrict__ keys,
                                   const unsigned *__restrict__ pos, const T *__restrict__ val, int *__restrict__ ptr,
                                   int *__restrict__ col_out, T *__restrict__ val_out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i <= rows) {  // first sorted key whose row is >= i
        long long lo = 0, hi = m;
        while (lo < hi) {
            const long long mid = (lo + hi) >> 1;
            if ((long long)(keys[mid] >> 32) < i) lo = mid + 1;
            else hi = mid;
        }
        ptr[i] = (int)lo;
    }
    if (i < m) {
        col_out[i] = (int)(unsigned)keys[i];
        val_out[i] = pos[i] == kUnitPayload ? T(1) : val[pos[i]];
    }
}

// Device arrays of the derived square matrix in the layout ctx_adopt expects, allocated here and handed to the
// caller with the number of stored elements.
template <typename T>
alphasparse_status_t derive_csr_device(const DeviceCtx *c, int type, int upper, int unit, int flip, int diag_rule,
                                       int **out_ptr, int **out_col, T **out_val, int64_t *out_nnz) {
    cudaStream_t st = current_stream();
    const int64_t nnz = c->nnz, rows = c->rows;
    const DeriveRule rule{type, upper, unit, flip, diag_rule};
    unsigned long long *d_keys[2] = {nullptr, nullptr};
    unsigned *d_pos[2] = {nullptr, nullptr}, *d_hist = nullptr, *d_sums = nullptr, *d_count = nullptr;
    int *d_pick = nullptr, *dptr = nullptr, *dcol = nullptr;
    T *dval = nullptr;
    auto release = [&](bool all) {
        cudaFree(d_keys[0]), cudaFree(d_keys[1]), cudaFree(d_pos[0]), cudaFree(d_pos[1]), cudaFree(d_hist), cudaFree(d_sums);
        cudaFree(d_count), cudaFree(d_pick);
        if (all) cudaFree(dptr), cudaFree(dcol), cudaFree(dval);
    };
#define TRY(expr, code)                   \
    do {                                  \
        cudaError_t _e = (expr);          \
        if (_e != cudaSuccess) {          \
            record_cuda_error(_e, #expr); \
            release(true);                \
            return (code);                \
        }                                 \
    } while (0)
    const unsigned eblocks = (unsigned)((std::max<int64_t>(nnz, 1) + 255) / 256);
    const bool picks = type == ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL && !unit && diag_rule != 1 && nnz > 0;
    if (picks) {
        TRY(device_alloc(&d_pick, sizeof(int) * (size_t)rows), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        // bytes 0x7f.. = a large positive int for the minimum, 0xff.. = -1 for the maximum
        TRY(cudaMemsetAsync(d_pick, diag_rule == 2 ? 0xff : 0x7f, sizeof(int) * (size_t)rows, st),
            ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        derive_diag_pick_kernel<<<eblocks, 256, 0, st>>>(nnz, (int)rows, c->d_row_ptr, c->d_col, diag_rule == 2, d_pick);
        count_launch();
    }
    // how many keys every stored element emits, and where
    unsigned long long emitted = 0;
    if (nnz > 0) {
        const int scan_blocks = (int)((nnz + kScanTile - 1) / kScanTile);
        unsigned last_count = 0, last_offset = 0;
        TRY(device_alloc(&d_count, sizeof(unsigned) * (size_t)nnz), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_sums, sizeof(unsigned) * (size_t)(scan_blocks + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        derive_count_kernel<<<eblocks, 256, 0, st>>>(nnz, (int)rows, c->d_row_ptr, c->d_col, rule, d_pick, d_count);
        count_launch();
        TRY(cudaMemcpyAsync(&last_count, d_count + nnz - 1, 4, cudaMemcpyDeviceToHost, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        alphasparse_status_t s = device_exclusive_scan(d_count, nnz, d_sums, st);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
            release(true);
            return s;
        }
        TRY(cudaMemcpyAsync(&last_offset, d_count + nnz - 1, 4, cudaMemcpyDeviceToHost, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        emitted = (unsigned long long)last_offset + last_count;  // at most 2 * nnz < 2^32: the 32-bit scan is exact
        cudaFree(d_sums), d_sums = nullptr;
    }
    // 32-bit offsets, as for every handle; a symmetric matrix may double its stored elements
    if (emitted + (unit ? (unsigned long long)rows : 0ull) > (unsigned long long)(INT32_MAX - 64)) {
        release(true);
        record_error("the matrix derived for this descriptor would hold more than 2^31 - 65 elements");
        return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    }
    const int64_t m = (int64_t)emitted + (unit ? rows : 0);
    const size_t n = (size_t)m, padded = n + kTailPad;
    TRY(device_alloc(&dptr, sizeof(int) * (size_t)(rows + 1 + 4)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&dcol, sizeof(int) * padded), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&dval, sizeof(T) * padded), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(cudaMemsetAsync(dptr, 0, sizeof(int) * (size_t)(rows + 1 + 4), st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemsetAsync(dcol + n, 0, sizeof(int) * kTailPad, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemsetAsync(dval + n, 0, sizeof(T) * kTailPad, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    if (m > 0) {
        const long long nblocks = (m + kSortTile - 1) / kSortTile;
        const long long hist_n = 16 * nblocks;
        const int scan_blocks = (int)((hist_n + kScanTile - 1) / kScanTile);
        TRY(device_alloc(&d_keys[0], 8 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_keys[1], 8 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_pos[0], 4 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_pos[1], 4 * n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_hist, sizeof(unsigned) * (size_t)hist_n), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        TRY(device_alloc(&d_sums, sizeof(unsigned) * (size_t)(scan_blocks + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        const long long work = std::max<long long>(nnz, unit ? rows : 0);
        derive_emit_kernel<<<(unsigned)((work + 255) / 256), 256, 0, st>>>(nnz, (int)rows, c->d_row_ptr, c->d_col, rule,
                                                                          d_pick, d_count, d_keys[0], d_pos[0]);
        count_launch();
        int cur = 0;
        const int bits = bits_for(rows);  // square: rows == cols
        for (int part = 0; part < 2; part++) {
            const int first = part == 0 ? 0 : 32;
            for (int shift = first; shift < first + bits; shift += 4) {
                radix_hist_kernel<<<(unsigned)nblocks, kSortThreads, 0, st>>>(m, d_keys[cur], shift, d_hist);
                count_launch();
                alphasparse_status_t s = device_exclusive_scan(d_hist, hist_n, d_sums, st);
                if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
                    release(true);
                    return s;
                }
                radix_scatter_kernel<<<(unsigned)nblocks, kSortThreads, 0, st>>>(m, d_keys[cur], d_pos[cur], shift, d_hist,
                                                                                d_keys[cur ^ 1], d_pos[cur ^ 1]);
                count_launch();
                cur ^= 1;
            }
        }
        const long long fill = std::max<long long>(m, rows + 1);
        derive_fill_kernel<T><<<(unsigned)((fill + 255) / 256), 256, 0, st>>>(
            m, (int)rows, d_keys[cur], d_pos[cur], static_cast<const T *>(c->d_val), dptr, dcol, dval);
        count_launch();
        TRY(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }
    TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
#undef TRY
    release(false);
    *out_ptr = dptr, *out_col = dcol, *out_val = dval, *out_nnz = m;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template alphasparse_status_t derive_csr_device<float>(const DeviceCtx *, int, int, int, int, int, int **, int **, float **,
                                                       int64_t *);
template alphasparse_status_t derive_csr_device<double>(const DeviceCtx *, int, int, int, int, int, int **, int **, double **,
                                                        int64_t *);

template alphasparse_status_t transpose_csr_device<float>(const DeviceCtx *, int **, int **, float **);
template alphasparse_status_t transpose_csr_device<double>(const DeviceCtx *, int **, int **, double **);

template alphasparse_status_t coo_to_csr_device<float>(int64_t, int64_t, int64_t, const int *, const int *,
                                                       const float *, int *, int *, float *);
template alphasparse_status_t coo_to_csr_device<double>(int64_t, int64_t, int64_t, const int *, const int *,
                                                        const double *, int *, int *, double *);

}  // namespace asb
