// CSR x dense SpMM kernels for sm_100a, row-major dense operands.
//
// Y[r, :] = beta * Y[r, :] + sum over stored elements (alpha * a) * X[col, :], the operation
// of the reference's gemm_{s,d}_csr_row (arithmetic defined by
// src/plain/kernel/level3/mm/gemm/gemm_x_csr_row_plain.c:4-23: alpha is folded into the
// element before the accumulation).  The reference's own device build has no row-major SpMM
// (src/kernel/dcu/level3/mm/csrmm/dcu_gemm_x_csr_row.cpp:15-36 returns NOT_SUPPORTED).
//
// One warp owns one sparse row; its lanes span the dense columns, VEC consecutive columns
// per lane, so every stored element turns into one fully coalesced read of a row of X
// (64 fp32 columns = 256 bytes = 32 lanes x float2).  The warp fetches 32 (col, alpha*a)
// pairs with one coalesced load each and hands them round with shuffles; the loop over the
// 32 pairs is unrolled so several X rows are in flight per warp.  Bandwidth-bound: the
// traffic is nnz * columns * sizeof(T) of X rows against 2 flops per element, far below what
// would justify staging tiles for tensor cores.
#include <algorithm>

#include "internal.h"

namespace asb {

template <typename T, int VEC>
struct Pack;
template <>
struct Pack<float, 1> { using type = float; };
template <>
struct Pack<float, 2> { using type = float2; };
template <>
struct Pack<float, 4> { using type = float4; };
template <>
struct Pack<double, 1> { using type = double; };
template <>
struct Pack<double, 2> { using type = double2; };

template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T *__restrict__ p, T (&out)[VEC]) {
    using P = typename Pack<T, VEC>::type;
    const P t = __ldg(reinterpret_cast<const P *>(p));
    const T *s = reinterpret_cast<const T *>(&t);
#pragma unroll
    for (int i = 0; i < VEC; i++) out[i] = s[i];
}

// A group of LPR lanes (a power of two up to 32) owns one sparse row; 32/LPR rows share a warp.
// Lane g of the group holds VEC consecutive dense columns starting at ct + g*VEC, so one step of
// the group reads LPR*VEC*sizeof(T) contiguous bytes of an X row (64 fp32 columns: 16 lanes x
// float4 = 256 bytes, two rows per warp instruction).
// VEC > 1 requires: columns % VEC == 0, ldx % VEC == 0, ldy % VEC == 0 and X, Y aligned to
// VEC * sizeof(T); the launcher checks and otherwise uses VEC == 1.
constexpr int kSpmmUnroll = 4;     // X rows in flight per lane group (8 and 16 were slower on B200)
constexpr int kSpmmMinBlocks = 8;  // full occupancy (32 registers) measured fastest
template <typename T, int VEC, int LPR, bool HAS_BETA>
__global__ void __launch_bounds__(256, kSpmmMinBlocks)
    spmm_row_kernel(int rows, const int *__restrict__ row_lo, const int *__restrict__ row_hi,
                    const int *__restrict__ col, const T *__restrict__ val, const T *__restrict__ X, int columns,
                    long long ldx, T *__restrict__ Y, long long ldy, T alpha, T beta) {
    constexpr int UNROLL = kSpmmUnroll;
    constexpr int RPW = 32 / LPR;  // rows per warp
    const int lane = threadIdx.x & 31;
    const int gl = lane % LPR, grp = lane / LPR;
    const unsigned gmask = LPR == 32 ? 0xffffffffu : (((1u << LPR) - 1u) << (grp * LPR));
    const long long row = ((long long)blockIdx.x * 8 + (threadIdx.x >> 5)) * RPW + grp;
    if (row >= rows) return;  // whole groups leave together; shuffles below name only their group
    // [row_lo[row], row_hi[row]) are the stored elements this launch multiplies: the whole row (row_hi = row_lo + 1
    // of the offset array) or the part of it that falls into one column block (see SpmmBlocks)
    const int s = __ldg(row_lo + row), e = __ldg(row_hi + row);

    for (int ct = 0; ct < columns; ct += LPR * VEC) {
        const int c = ct + gl * VEC;
        const bool live = c < columns;
        T acc[VEC];
#pragma unroll
        for (int i = 0; i < VEC; i++) acc[i] = T(0);

        for (int base = s; base < e; base += LPR) {
            const int mine = base + gl;
            int cj = 0;
            T vj = T(0);
            if (mine < e) {
                cj = __ldcs(col + mine);
                vj = alpha * __ldcs(val + mine);
            }
            const int n = min(LPR, e - base);
            int k = 0;
            for (; k + UNROLL <= n; k += UNROLL) {
                T xv[UNROLL][VEC];
                T av[UNROLL];
#pragma unroll
                for (int u = 0; u < UNROLL; u++) {
                    const int cc = __shfl_sync(gmask, cj, k + u, LPR);
                    av[u] = __shfl_sync(gmask, vj, k + u, LPR);
                    if (live) load_vec<T, VEC>(X + (long long)cc * ldx + c, xv[u]);
                }
                if (live) {
#pragma unroll
                    for (int u = 0; u < UNROLL; u++)
#pragma unroll
                        for (int i = 0; i < VEC; i++) acc[i] = fma(av[u], xv[u][i], acc[i]);
                }
            }
            for (; k < n; k++) {
                const int cc = __shfl_sync(gmask, cj, k, LPR);
                const T a = __shfl_sync(gmask, vj, k, LPR);
                if (live) {
                    T xv[VEC];
                    load_vec<T, VEC>(X + (long long)cc * ldx + c, xv);
#pragma unroll
                    for (int i = 0; i < VEC; i++) acc[i] = fma(a, xv[i], acc[i]);
                }
            }
        }

        if (live) {
            T *out = Y + row * ldy + c;
#pragma unroll
            for (int i = 0; i < VEC; i++) {
                T o = acc[i];
                if (HAS_BETA) o = fma(beta, out[i], o);
                acc[i] = o;
            }
            using P = typename Pack<T, VEC>::type;
            P packed;
            T *ps = reinterpret_cast<T *>(&packed);
#pragma unroll
            for (int i = 0; i < VEC; i++) ps[i] = acc[i];
            __stcs(reinterpret_cast<P *>(out), packed);
        }
    }
}

// ---- narrow dense blocks -------------------------------------------------------------------------------
//
// With a handful of dense columns (an X row of at most 32 bytes) the kernel above degenerates: two lanes per row hand
// their elements round two at a time and every round waits for its own X rows (2^21 rows of 32 elements times 1..8
// fp32 columns: 0.68..1.24 ms, where an SpMV of the same matrix takes 0.2 ms).  Here the lanes of a group split the
// ELEMENTS of the row instead, as in the vector SpMV: a lane gathers the whole X row of its element (one or two
// 16-byte loads when the shapes allow, scalars otherwise), carries KC partial sums, two elements in flight, and the
// group reduces them by shuffles.  alpha is folded into the stored value before the sum, as in the kernel above.
template <typename T, int LANES, int KC, bool ALIGNED, bool HAS_BETA>
__global__ void __launch_bounds__(256)
    spmm_row_narrow_kernel(int rows, const int *__restrict__ row_lo, const int *__restrict__ row_hi,
                           const int *__restrict__ col, const T *__restrict__ val, const T *__restrict__ X, int columns,
                           long long ldx, T *__restrict__ Y, long long ldy, T alpha, T beta) {
    constexpr int GROUPS = 256 / LANES;
    constexpr int PER16 = 16 / (int)sizeof(T);  // elements per 16-byte load
    const int lane = threadIdx.x % LANES;
    const long long row = (long long)blockIdx.x * GROUPS + threadIdx.x / LANES;
    int s = 0, e = 0;
    if (row < rows) {
        s = __ldg(row_lo + row);
        e = __ldg(row_hi + row);
    }
    T acc[KC];
#pragma unroll
    for (int k = 0; k < KC; k++) acc[k] = T(0);
    auto take = [&](int j) {
        const int cj = __ldcs(col + j);
        const T vj = alpha * __ldcs(val + j);
        const T *xr = X + (long long)cj * ldx;
        T xv[KC];
        if (ALIGNED) {  // columns == KC, rows of X on 16-byte boundaries
#pragma unroll
            for (int k = 0; k < KC; k += PER16) {
                using P = typename Pack<T, PER16>::type;
                const P t = __ldg(reinterpret_cast<const P *>(xr + k));
                const T *sp = reinterpret_cast<const T *>(&t);
#pragma unroll
                for (int i = 0; i < PER16; i++) xv[k + i] = sp[i];
            }
        } else {
#pragma unroll
            for (int k = 0; k < KC; k++) xv[k] = k < columns ? __ldg(xr + k) : T(0);
        }
#pragma unroll
        for (int k = 0; k < KC; k++) acc[k] = fma(vj, xv[k], acc[k]);
    };
    int j = s + lane;
    for (; j + LANES < e; j += 2 * LANES) {
        take(j);
        take(j + LANES);
    }
    if (j < e) take(j);
#pragma unroll
    for (int k = 0; k < KC; k++) {
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
    }
    if (lane == 0 && row < rows) {
        T *out = Y + row * ldy;
#pragma unroll
        for (int k = 0; k < KC; k++)
            if (k < columns) {
                T o = acc[k];
                if (HAS_BETA) o = fma(beta, out[k], o);
                out[k] = o;
            }
    }
}

// ---- column blocks -----------------------------------------------------------------------------------
//
// Every stored element reads one row of X (columns * sizeof(T) bytes).  With unstructured columns and an X far
// larger than L2 nearly all of these reads come from HBM: 64 fp32 columns on 6.7e7 elements move 17 GB for
// 1.6 GB of operands.  Cutting the columns of A into P blocks and running the product block by block makes the
// rows of X a pass touches a slab of 1/P of X that stays in L2, so X crosses HBM about once; the price is that Y
// is written P times and read P - 1 times.  Rows with ascending columns need no copy of A for this: the part of
// a row inside a block is a contiguous run, described by P + 1 offsets per row.  (An experiment kept as an
// option: see spmm_pick_blocks for what it measured.)
__global__ void rows_ascending_kernel(int rows, const int *__restrict__ row_ptr, const int *__restrict__ col,
                                      unsigned long long *__restrict__ bad) {
    unsigned long long n = 0;
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (long long)gridDim.x * blockDim.x)
        for (int k = row_ptr[r]; k + 1 < row_ptr[r + 1]; k++) n += col[k] > col[k + 1];
    for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
    if ((threadIdx.x & 31) == 0 && n) atomicAdd(bad, n);
}

// split[p * rows + r] = first element of row r whose column is >= p * width (p = 0 .. blocks)
__global__ void spmm_split_kernel(int rows, int blocks, int width, const int *__restrict__ row_ptr,
                                  const int *__restrict__ col, int *__restrict__ split) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)rows * (blocks + 1)) return;
    const int p = (int)(i / rows), r = (int)(i % rows);
    int lo = row_ptr[r], hi = row_ptr[r + 1];
    if (p == 0) hi = lo;
    else if (p == blocks) lo = hi;
    const long long want = (long long)p * width;
    while (lo < hi) {
        const int mid = lo + ((hi - lo) >> 1);
        if ((long long)col[mid] < want) lo = mid + 1;
        else hi = mid;
    }
    split[i] = lo;
}

void spmm_blocks_destroy(SpmmBlocks &b) {
    cudaFree(b.d_split);
    b = SpmmBlocks{};
}

// Column-block table for `blocks` blocks, built on first use and kept until another count is asked for.
// Leaves b.blocks == 1 (no blocking) when the rows are not in ascending column order.
alphasparse_status_t col_blocks_ensure(DeviceCtx *ctx, SpmmBlocks &b, int blocks, cudaStream_t st) {
    if (b.blocks == blocks || (b.unsorted && blocks > 1)) return ALPHA_SPARSE_STATUS_SUCCESS;
    const int64_t old_bytes = b.d_split ? (int64_t)sizeof(int) * ctx->rows * (b.blocks + 1) : 0;
    spmm_blocks_destroy(b);
    ctx->device_bytes -= old_bytes;
    b.blocks = 1;
    if (blocks <= 1) return ALPHA_SPARSE_STATUS_SUCCESS;
    unsigned long long *d_bad = nullptr, h_bad = 0;
    ASB_CUDA_OR(device_alloc(&d_bad, sizeof(h_bad)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    cudaError_t e = cudaMemsetAsync(d_bad, 0, sizeof(h_bad), st);
    if (e == cudaSuccess) {
        rows_ascending_kernel<<<148 * 8, 256, 0, st>>>((int)ctx->rows, ctx->d_row_ptr, ctx->d_col, d_bad);
        count_launch();
        e = cudaMemcpyAsync(&h_bad, d_bad, sizeof(h_bad), cudaMemcpyDeviceToHost, st);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_bad);
    if (e != cudaSuccess) {
        record_cuda_error(e, "column blocks");
        return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    }
    if (h_bad) {
        b.unsorted = true;
        return ALPHA_SPARSE_STATUS_SUCCESS;
    }
    const int width = (int)((ctx->cols + blocks - 1) / blocks);
    const size_t cells = (size_t)ctx->rows * (size_t)(blocks + 1);
    ASB_CUDA_OR(device_alloc(&b.d_split, sizeof(int) * cells), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    spmm_split_kernel<<<(unsigned)((cells + 255) / 256), 256, 0, st>>>((int)ctx->rows, blocks, width, ctx->d_row_ptr,
                                                                     ctx->d_col, b.d_split);
    count_launch();
    e = cudaGetLastError();
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        spmm_blocks_destroy(b);
        b.blocks = 1;
        record_cuda_error(e, "column blocks");
        return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    }
    b.blocks = blocks, b.width = width;
    ctx->device_bytes += (int64_t)(sizeof(int) * cells);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- long rows ------------------------------------------------------------------------------------------

void spmm_split_destroy(SpmmSplit &s) {
    cudaFree(s.d_hi_short), cudaFree(s.d_chunk_lo), cudaFree(s.d_chunk_hi), cudaFree(s.d_long_row), cudaFree(s.d_long_first);
    cudaFree(s.d_part);
    free(s.h_long_row), free(s.h_long_first);
    s = SpmmSplit{};
}

// Y[row, :] += the row's partial sums in chunk order.  One block per long row, threads over the dense columns.
template <typename T>
__global__ void spmm_long_reduce_kernel(const int *__restrict__ long_row, const int *__restrict__ long_first,
                                        const T *__restrict__ part, int columns, T *__restrict__ Y, long long ldy) {
    const int row = long_row[blockIdx.x], k0 = long_first[blockIdx.x], k1 = long_first[blockIdx.x + 1];
    for (int c = threadIdx.x; c < columns; c += blockDim.x) {
        T acc = T(0);
        for (int k = k0; k < k1; k++) acc += part[(size_t)k * columns + c];
        Y[(long long)row * ldy + c] += acc;
    }
}

// Looks at the row lengths once (first row-major product of the handle) and builds the chunk tables when some row
// is longer than spmm_split_min.
static alphasparse_status_t spmm_split_ensure(DeviceCtx *ctx, cudaStream_t st) {
    SpmmSplit &sp = ctx->split;
    if (sp.state != 0) return ALPHA_SPARSE_STATUS_SUCCESS;
    const int64_t min_len = option(kOptSpmmSplitMin), chunk = std::max<int64_t>(64, option(kOptSpmmSplitChunk));
    // (only where the rows are uneven: rows that are all long keep every lane group equally busy as they are)
    if (min_len <= 0 || ctx->max_row_nnz <= min_len || ctx->rows == 0 || (double)ctx->max_row_nnz <= 8.0 * ctx->mean_row_nnz) {
        sp.state = 1;
        return ALPHA_SPARSE_STATUS_SUCCESS;
    }
    std::vector<int> ptr, hi, clo, chi, lrow, lfirst;
    try {
        ptr.resize((size_t)ctx->rows + 1);
    } catch (...) {
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    ASB_CUDA_OR(cudaMemcpyAsync(ptr.data(), ctx->d_row_ptr, sizeof(int) * ptr.size(), cudaMemcpyDeviceToHost, st),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    try {
        hi.resize((size_t)ctx->rows);
        for (int64_t r = 0; r < ctx->rows; r++) {
            const int a = ptr[(size_t)r], e = ptr[(size_t)r + 1];
            hi[(size_t)r] = e;
            if ((int64_t)e - a <= min_len) continue;
            hi[(size_t)r] = a;  // nothing of this row in the row pass
            lrow.push_back((int)r);
            lfirst.push_back((int)clo.size());
            for (int64_t k = a; k < e; k += chunk) {
                clo.push_back((int)k);
                chi.push_back((int)std::min<int64_t>(e, k + chunk));
            }
        }
        lfirst.push_back((int)clo.size());
    } catch (...) {
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    SpmmSplit t;
    t.nlong = (int64_t)lrow.size(), t.nchunks = (int64_t)clo.size();
    t.h_long_row = static_cast<int *>(malloc(sizeof(int) * std::max<size_t>(1, lrow.size())));
    t.h_long_first = static_cast<int *>(malloc(sizeof(int) * lfirst.size()));
    cudaError_t e = (t.h_long_row && t.h_long_first) ? cudaSuccess : cudaErrorMemoryAllocation;
    if (e == cudaSuccess) e = device_alloc(&t.d_hi_short, sizeof(int) * hi.size());
    if (e == cudaSuccess) e = device_alloc(&t.d_chunk_lo, sizeof(int) * clo.size());
    if (e == cudaSuccess) e = device_alloc(&t.d_chunk_hi, sizeof(int) * chi.size());
    if (e == cudaSuccess) e = device_alloc(&t.d_long_row, sizeof(int) * lrow.size());
    if (e == cudaSuccess) e = device_alloc(&t.d_long_first, sizeof(int) * lfirst.size());
    if (e == cudaSuccess) e = cudaMemcpyAsync(t.d_hi_short, hi.data(), sizeof(int) * hi.size(), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t.d_chunk_lo, clo.data(), sizeof(int) * clo.size(), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t.d_chunk_hi, chi.data(), sizeof(int) * chi.size(), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t.d_long_row, lrow.data(), sizeof(int) * lrow.size(), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaMemcpyAsync(t.d_long_first, lfirst.data(), sizeof(int) * lfirst.size(), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);  // the vectors go out of scope
    if (e != cudaSuccess) {
        record_cuda_error(e, "long rows of the dense-block product");
        spmm_split_destroy(t);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    memcpy(t.h_long_row, lrow.data(), sizeof(int) * lrow.size());
    memcpy(t.h_long_first, lfirst.data(), sizeof(int) * lfirst.size());
    t.state = 2;
    sp = t;
    ctx->device_bytes += (int64_t)(sizeof(int) * (hi.size() + clo.size() + chi.size() + lrow.size() + lfirst.size()));
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// The chunk tables (first product of the handle) and room for the partial sums of a product with `columns` columns.
static alphasparse_status_t spmm_split_prepare(DeviceCtx *ctx, size_t tsz, int columns, cudaStream_t st) {
    alphasparse_status_t s = spmm_split_ensure(ctx, st);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS || ctx->split.state != 2) return s;
    SpmmSplit &sp = ctx->split;
    const size_t want = tsz * (size_t)sp.nchunks * (size_t)columns;
    if (sp.part_bytes < want) {
        cudaFree(sp.d_part);
        ctx->device_bytes -= (int64_t)sp.part_bytes;
        sp.d_part = nullptr, sp.part_bytes = 0;
        ASB_CUDA_OR(device_alloc(&sp.d_part, want), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        sp.part_bytes = want;
        ctx->device_bytes += (int64_t)want;
    }
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Column blocks are used only when asked for (option spmm_col_blocks > 1).  Measured on B200 with 64 fp32 columns,
// 2^21 rows of 32 elements and a 537 MB X: 3.51 ms in one pass, 4.08 / 4.60 / 5.16 / 6.37 ms with 4 / 6 / 8 / 12
// blocks.  Blocking does take the reads of X off HBM, but every stored element still pulls a whole row of X from
// L2 into an SM, and that stream (17 GB) already runs at the pace the one-pass kernel reaches from HBM; the
// extra passes over Y and the shorter per-row runs only add to it.
static int spmm_pick_blocks(const DeviceCtx *, size_t) {
    const int64_t blocks = option(kOptSpmmColBlocks);
    return (int)std::max<int64_t>(1, std::min<int64_t>(blocks, 64));
}

template <typename T, int VEC, int LPR>
static void launch_row(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx, T beta, T *Y,
                       int ldy, cudaStream_t st, const RowWindow *w) {
    constexpr int rows_per_block = 8 * (32 / LPR);
    // A window is the same kernel on a slice: offsets are absolute, so shifting the offset arrays and Y
    // by the first row is all it takes.
    const int64_t first = w ? w->begin : 0, rows = w ? w->count : ctx->rows;
    const unsigned blocks = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    const T *val = static_cast<const T *>(ctx->d_val);
    T *const Y0 = Y;
    Y += first * (int64_t)ldy;
    const SpmmSplit &sp = ctx->split;
    const bool split = sp.state == 2;
    const int passes = !split && ctx->spmm.d_split ? ctx->spmm.blocks : 1;
    if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
    for (int p = 0; p < passes; p++) {
        const int *lo = passes > 1 ? ctx->spmm.d_split + (size_t)p * ctx->rows + first : ctx->d_row_ptr + first;
        const int *hi = passes > 1 ? lo + ctx->rows : split ? sp.d_hi_short + first : lo + 1;
        // the first pass applies beta, the later ones add to what is there
        const T b = p == 0 ? beta : T(1);
        if (b == T(0))
            spmm_row_kernel<T, VEC, LPR, false><<<blocks, 256, 0, st>>>(
                (int)rows, lo, hi, ctx->d_col, val, X, columns, ldx, Y, ldy, alpha, b);
        else
            spmm_row_kernel<T, VEC, LPR, true><<<blocks, 256, 0, st>>>(
                (int)rows, lo, hi, ctx->d_col, val, X, columns, ldx, Y, ldy, alpha, b);
    }
    if (split) {
        // the long rows of this window: their chunks through the same kernel into partial sums, then onto Y
        const int *lb = std::lower_bound(sp.h_long_row, sp.h_long_row + sp.nlong, (int)first);
        const int *le = std::lower_bound(sp.h_long_row, sp.h_long_row + sp.nlong, (int)(first + rows));
        const int64_t l0 = lb - sp.h_long_row, l1 = le - sp.h_long_row;
        const int64_t c0 = sp.h_long_first[l0], c1 = sp.h_long_first[l1];
        if (c1 > c0) {
            T *part = static_cast<T *>(sp.d_part) + (size_t)c0 * columns;
            const unsigned cblocks = (unsigned)((c1 - c0 + rows_per_block - 1) / rows_per_block);
            spmm_row_kernel<T, VEC, LPR, false><<<cblocks, 256, 0, st>>>(
                (int)(c1 - c0), sp.d_chunk_lo + c0, sp.d_chunk_hi + c0, ctx->d_col, val, X, columns, ldx, part, columns, alpha,
                T(0));
            const int threads = std::min(256, (columns + 31) / 32 * 32);
            spmm_long_reduce_kernel<T><<<(unsigned)(l1 - l0), threads, 0, st>>>(
                sp.d_long_row + l0, sp.d_long_first + l0, static_cast<const T *>(sp.d_part), columns, Y0, ldy);
            count_launch(2);
        }
    }
    if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
    count_launch(passes);
}

template <typename T, int VEC>
static void launch_row_lanes(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx, T beta, T *Y,
                             int ldy, cudaStream_t st, const RowWindow *w) {
    // smallest group (2 .. 32 lanes) whose lanes cover the dense columns in one pass, if any
    const int need = (columns + VEC - 1) / VEC;
    if (need <= 2) launch_row<T, VEC, 2>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
    else if (need <= 4) launch_row<T, VEC, 4>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
    else if (need <= 8) launch_row<T, VEC, 8>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
    else if (need <= 16) launch_row<T, VEC, 16>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
    else launch_row<T, VEC, 32>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
}

template <typename T, int LANES, int KC, bool ALIGNED>
static void launch_narrow_as(int rows, const int *lo, const int *hi, DeviceCtx *ctx, T alpha, const T *X, int columns,
                             int ldx, T beta, T *Y, long long ldy, cudaStream_t st) {
    const unsigned blocks = (unsigned)(((long long)rows + 256 / LANES - 1) / (256 / LANES));
    const T *val = static_cast<const T *>(ctx->d_val);
    if (beta == T(0))
        spmm_row_narrow_kernel<T, LANES, KC, ALIGNED, false><<<blocks, 256, 0, st>>>(rows, lo, hi, ctx->d_col, val, X, columns,
                                                                                    ldx, Y, ldy, alpha, beta);
    else
        spmm_row_narrow_kernel<T, LANES, KC, ALIGNED, true><<<blocks, 256, 0, st>>>(rows, lo, hi, ctx->d_col, val, X, columns,
                                                                                   ldx, Y, ldy, alpha, beta);
    count_launch();
}

template <typename T, int KC, bool ALIGNED>
static void launch_narrow_lanes(int lanes, int rows, const int *lo, const int *hi, DeviceCtx *ctx, T alpha, const T *X,
                                int columns, int ldx, T beta, T *Y, long long ldy, cudaStream_t st) {
    if (lanes <= 4) launch_narrow_as<T, 4, KC, ALIGNED>(rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else if (lanes <= 8) launch_narrow_as<T, 8, KC, ALIGNED>(rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else if (lanes <= 16) launch_narrow_as<T, 16, KC, ALIGNED>(rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else launch_narrow_as<T, 32, KC, ALIGNED>(rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
}

// One launch of the narrow kernel over `rows` rows (or chunks) in the widest form the shapes allow.
template <typename T>
static void launch_narrow_pick(int lanes, int rows, const int *lo, const int *hi, DeviceCtx *ctx, T alpha, const T *X,
                               int columns, int ldx, T beta, T *Y, long long ldy, cudaStream_t st) {
    constexpr int PER16 = 16 / (int)sizeof(T), WIDE = 2 * PER16;
    const bool aligned = ((uintptr_t)X & 15) == 0 && ldx % PER16 == 0;
    if (aligned && columns == WIDE)
        launch_narrow_lanes<T, WIDE, true>(lanes, rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else if (aligned && columns == PER16)
        launch_narrow_lanes<T, PER16, true>(lanes, rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else if (columns <= PER16)
        launch_narrow_lanes<T, PER16, false>(lanes, rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else
        launch_narrow_lanes<T, WIDE, false>(lanes, rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
}

// The row-major product with an X row of at most 32 bytes: windows and long rows as in launch_row.
template <typename T>
static void launch_narrow(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx, T beta, T *Y, int ldy, cudaStream_t st,
                          const RowWindow *w) {
    const int64_t first = w ? w->begin : 0, rows = w ? w->count : ctx->rows;
    const SpmmSplit &sp = ctx->split;
    const bool split = sp.state == 2;
    const double m = ctx->mean_row_nnz;
    const int lanes = m <= 8 ? 4 : m <= 16 ? 8 : m <= 32 ? 16 : 32;
    if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
    const int *lo = ctx->d_row_ptr + first, *hi = split ? sp.d_hi_short + first : lo + 1;
    launch_narrow_pick<T>(lanes, (int)rows, lo, hi, ctx, alpha, X, columns, ldx, beta, Y + first * (int64_t)ldy, ldy, st);
    if (split) {
        const int *lb = std::lower_bound(sp.h_long_row, sp.h_long_row + sp.nlong, (int)first);
        const int *le = std::lower_bound(sp.h_long_row, sp.h_long_row + sp.nlong, (int)(first + rows));
        const int64_t l0 = lb - sp.h_long_row, l1 = le - sp.h_long_row;
        const int64_t c0 = sp.h_long_first[l0], c1 = sp.h_long_first[l1];
        if (c1 > c0) {
            T *part = static_cast<T *>(sp.d_part) + (size_t)c0 * columns;
            // the partial sums are a dense block of their own: `columns` wide, rows packed
            launch_narrow_pick<T>(32, (int)(c1 - c0), sp.d_chunk_lo + c0, sp.d_chunk_hi + c0, ctx, alpha, X, columns, ldx, T(0),
                                  part, columns, st);
            spmm_long_reduce_kernel<T><<<(unsigned)(l1 - l0), 32, 0, st>>>(sp.d_long_row + l0, sp.d_long_first + l0,
                                                                         static_cast<const T *>(sp.d_part), columns, Y, ldy);
            count_launch();
        }
    }
    if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
}

template <typename T>
alphasparse_status_t launch_spmm_row(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx,
                                     T beta, T *Y, int ldy, cudaStream_t st, const RowWindow *w) {
    if (ctx->rows == 0 || columns <= 0 || (w && w->count <= 0)) return ALPHA_SPARSE_STATUS_SUCCESS;
    alphasparse_status_t bs = spmm_split_prepare(ctx, sizeof(T), columns, st);
    if (bs != ALPHA_SPARSE_STATUS_SUCCESS) return bs;
    bs = col_blocks_ensure(ctx, ctx->spmm, spmm_pick_blocks(ctx, sizeof(T) * (size_t)ctx->cols * (size_t)ldx), st);
    if (bs != ALPHA_SPARSE_STATUS_SUCCESS) return bs;
    if ((size_t)columns * sizeof(T) <= 32 && option(kOptSpmmNarrow)) {
        launch_narrow<T>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
        ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        return ALPHA_SPARSE_STATUS_SUCCESS;
    }
    auto fits = [&](int vec) {
        const uintptr_t mask = (uintptr_t)(vec * sizeof(T) - 1);
        return columns % vec == 0 && ldx % vec == 0 && ldy % vec == 0 &&
               ((uintptr_t)X & mask) == 0 && ((uintptr_t)Y & mask) == 0;
    };
    // Widest 16-byte pack the shapes and alignments allow.
    if constexpr (sizeof(T) == 4) {
        if (fits(4)) launch_row_lanes<T, 4>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
        else if (fits(2)) launch_row_lanes<T, 2>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
        else launch_row_lanes<T, 1>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
    } else {
        if (fits(2)) launch_row_lanes<T, 2>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
        else launch_row_lanes<T, 1>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st, w);
    }
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- column-major dense operands ------------------------------------------------------------------
//
// Y[:, c] = beta * Y[:, c] + alpha * (A * X[:, c]) for every dense column c, element (r, c) of a dense
// operand at [c * ld + r]: the operation of the reference's gemm_{s,d}_csr_col (arithmetic defined by
// src/plain/kernel/level3/mm/gemm/gemm_x_csr_col_plain.c:4-21: a dot product from zero per (row, column),
// then y = y*beta + alpha*dot).  Each dense column is an independent SpMV on the same A, so the kernel
// is the vector SpMV with KC columns carried side by side: a group of LANES lanes owns a sparse row,
// every stored element is loaded once and multiplied into KC accumulators, one gather per column.
// blockIdx.y selects the block of KC columns; A is re-read once per block.
template <typename T, int LANES, int KC, bool HAS_BETA>
__global__ void __launch_bounds__(256)
    spmm_col_kernel(int rows, const int *__restrict__ row_lo, const int *__restrict__ row_hi,
                    const int *__restrict__ col, const T *__restrict__ val, const T *__restrict__ X, int columns,
                    long long ldx, T *__restrict__ Y, long long ldy, T alpha, T beta) {
    constexpr int GROUPS = 256 / LANES;
    const int lane = threadIdx.x % LANES;
    const long long row = (long long)blockIdx.x * GROUPS + threadIdx.x / LANES;
    const int c0 = blockIdx.y * KC;
    int s = 0, e = 0;
    if (row < rows) {  // the whole row, or the chunk of a long row that stands in for a row (see SpmmSplit)
        s = __ldg(row_lo + row);
        e = __ldg(row_hi + row);
    }
    T acc[KC];
#pragma unroll
    for (int k = 0; k < KC; k++) acc[k] = T(0);
    for (int j = s + lane; j < e; j += LANES) {
        const int cj = __ldg(col + j);
        const T vj = __ldg(val + j);
#pragma unroll
        for (int k = 0; k < KC; k++)
            if (c0 + k < columns) acc[k] = fma(vj, __ldg(X + (long long)(c0 + k) * ldx + cj), acc[k]);
    }
#pragma unroll
    for (int k = 0; k < KC; k++) {
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], o);
    }
    if (lane == 0 && row < rows) {
#pragma unroll
        for (int k = 0; k < KC; k++)
            if (c0 + k < columns) {
                T *out = Y + (long long)(c0 + k) * ldy + row;
                T o = alpha * acc[k];
                if (HAS_BETA) o = fma(beta, *out, o);
                *out = o;
            }
    }
}

// Y[c * ldy + row] += the row's partial sums (part[c * nchunks + k]) in chunk order: one thread per (long row, column).
template <typename T>
__global__ void spmm_long_reduce_col_kernel(int nlong, const int *__restrict__ long_row, const int *__restrict__ long_first,
                                            const T *__restrict__ part, long long nchunks, int columns, T *__restrict__ Y,
                                            long long ldy) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)nlong * columns) return;
    const int l = (int)(i % nlong), c = (int)(i / nlong);
    T acc = T(0);
    for (int k = long_first[l]; k < long_first[l + 1]; k++) acc += part[(long long)c * nchunks + k];
    Y[(long long)c * ldy + long_row[l]] += acc;
}

template <typename T, int LANES>
static void launch_col(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx, T beta, T *Y, int ldy,
                       cudaStream_t st) {
    constexpr int KC = 4;
    const dim3 grid((unsigned)((ctx->rows + 256 / LANES - 1) / (256 / LANES)), (unsigned)((columns + KC - 1) / KC));
    const T *val = static_cast<const T *>(ctx->d_val);
    const SpmmSplit &sp = ctx->split;
    const bool split = sp.state == 2;
    const int *hi = split ? sp.d_hi_short : ctx->d_row_ptr + 1;
    if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
    if (beta == T(0))
        spmm_col_kernel<T, LANES, KC, false><<<grid, 256, 0, st>>>((int)ctx->rows, ctx->d_row_ptr, hi, ctx->d_col, val, X,
                                                                  columns, ldx, Y, ldy, alpha, beta);
    else
        spmm_col_kernel<T, LANES, KC, true><<<grid, 256, 0, st>>>((int)ctx->rows, ctx->d_row_ptr, hi, ctx->d_col, val, X,
                                                                 columns, ldx, Y, ldy, alpha, beta);
    count_launch();
    if (split && sp.nchunks > 0) {
        // the chunks of the long rows as rows of their own (a warp each) into partial sums, then onto Y
        T *part = static_cast<T *>(sp.d_part);
        const dim3 cgrid((unsigned)((sp.nchunks + 7) / 8), grid.y);
        spmm_col_kernel<T, 32, KC, false><<<cgrid, 256, 0, st>>>((int)sp.nchunks, sp.d_chunk_lo, sp.d_chunk_hi, ctx->d_col, val,
                                                                X, columns, ldx, part, sp.nchunks, alpha, T(0));
        const long long cells = (long long)sp.nlong * columns;
        spmm_long_reduce_col_kernel<T><<<(unsigned)((cells + 255) / 256), 256, 0, st>>>(
            (int)sp.nlong, sp.d_long_row, sp.d_long_first, part, sp.nchunks, columns, Y, ldy);
        count_launch(2);
    }
    if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
}

// B[f * ld_b + s] = A[s * ld_a + f] for f < n_fast, s < n_slow: a column-major operand (f = row, s = dense column)
// into a row-major one, or back (f = dense column, s = row).  32 x 32 tiles through shared memory; the tiles along the
// longer of the two extents are numbered by blockIdx.x (`slow_on_x`), whose range is the wide one.
template <typename T>
__global__ void __launch_bounds__(256) dense_transpose_kernel(long long n_fast, long long n_slow, const T *__restrict__ A,
                                                              long long ld_a, T *__restrict__ B, long long ld_b,
                                                              int slow_on_x) {
    __shared__ T tile[32][33];
    const long long f0 = (long long)(slow_on_x ? blockIdx.y : blockIdx.x) * 32;
    const long long s0 = (long long)(slow_on_x ? blockIdx.x : blockIdx.y) * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const long long f = f0 + tx, sl = s0 + ty + k;
        if (f < n_fast && sl < n_slow) tile[ty + k][tx] = A[sl * ld_a + f];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const long long f = f0 + ty + k, sl = s0 + tx;
        if (f < n_fast && sl < n_slow) B[f * ld_b + sl] = tile[tx][ty + k];
    }
}

template <typename T>
static void dense_transpose(long long n_fast, long long n_slow, const T *A, long long ld_a, T *B, long long ld_b,
                            cudaStream_t st) {
    const long long tf = (n_fast + 31) / 32, ts = (n_slow + 31) / 32;
    const int slow_on_x = ts > tf;
    const dim3 grid((unsigned)(slow_on_x ? ts : tf), (unsigned)(slow_on_x ? tf : ts));
    dense_transpose_kernel<T><<<grid, 256, 0, st>>>(n_fast, n_slow, A, ld_a, B, ld_b, slow_on_x);
    count_launch();
}

static alphasparse_status_t grow_scratch(DeviceCtx *ctx, void **buf, size_t *have, size_t want) {
    if (*have >= want) return ALPHA_SPARSE_STATUS_SUCCESS;
    cudaFree(*buf);
    ctx->device_bytes -= (int64_t)*have;
    *buf = nullptr, *have = 0;
    ASB_CUDA_OR(device_alloc(buf, want), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    *have = want;
    ctx->device_bytes += (int64_t)want;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template <typename T>
alphasparse_status_t launch_spmm_col(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx, T beta, T *Y,
                                     int ldy, cudaStream_t st) {
    if (ctx->rows == 0 || columns <= 0) return ALPHA_SPARSE_STATUS_SUCCESS;
    // The kernel below gathers one x element per (stored element, dense column): four L2 requests per element and
    // pass of four columns, where the row-major kernels take a whole X row with one or two (2^21 rows of 32 elements
    // times 8 / 64 fp32 columns: 2.0 / 16.2 ms column-major against 0.6 / 3.5 ms row-major).  From spmm_col_via_row
    // columns on the operands are therefore transposed into row-major copies kept with the handle (X, and Y when
    // beta != 0), multiplied there, and Y is transposed back.
    const int64_t via = option(kOptSpmmColViaRow);
    if (via > 0 && columns >= via && columns <= 32 * 65535) {
        const size_t xb = sizeof(T) * (size_t)ctx->cols * (size_t)columns, yb = sizeof(T) * (size_t)ctx->rows * (size_t)columns;
        alphasparse_status_t s = grow_scratch(ctx, &ctx->d_cm_x, &ctx->cm_x_bytes, xb);
        if (s == ALPHA_SPARSE_STATUS_SUCCESS) s = grow_scratch(ctx, &ctx->d_cm_y, &ctx->cm_y_bytes, yb);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        T *xt = static_cast<T *>(ctx->d_cm_x), *yt = static_cast<T *>(ctx->d_cm_y);
        dense_transpose<T>(ctx->cols, columns, X, ldx, xt, columns, st);
        if (beta != T(0)) dense_transpose<T>(ctx->rows, columns, Y, ldy, yt, columns, st);
        s = launch_spmm_row<T>(ctx, alpha, xt, columns, columns, beta, yt, columns, st, nullptr);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        dense_transpose<T>(columns, ctx->rows, yt, columns, Y, ldy, st);
        ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        return ALPHA_SPARSE_STATUS_SUCCESS;
    }
    if ((columns + 3) / 4 > 65535) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    const alphasparse_status_t ps = spmm_split_prepare(ctx, sizeof(T), columns, st);
    if (ps != ALPHA_SPARSE_STATUS_SUCCESS) return ps;
    const double m = ctx->mean_row_nnz;
    if (m <= 8) launch_col<T, 4>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else if (m <= 16) launch_col<T, 8>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else if (m <= 32) launch_col<T, 16>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    else launch_col<T, 32>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template alphasparse_status_t launch_spmm_col<float>(DeviceCtx *, float, const float *, int, int, float, float *,
                                                     int, cudaStream_t);
template alphasparse_status_t launch_spmm_col<double>(DeviceCtx *, double, const double *, int, int, double,
                                                      double *, int, cudaStream_t);

template alphasparse_status_t launch_spmm_row<float>(DeviceCtx *, float, const float *, int, int,
                                                     float, float *, int, cudaStream_t, const RowWindow *);
template alphasparse_status_t launch_spmm_row<double>(DeviceCtx *, double, const double *, int, int,
                                                      double, double *, int, cudaStream_t, const RowWindow *);

}  // namespace asb
