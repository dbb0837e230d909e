/*
 * CPU restatement of the reference's CSR mv / mm path.  TEST INFRASTRUCTURE ONLY: it is the
 * checker the parity tests and the CPU legs of the benchmark compare against, never part of
 * the shipped library, which has no CPU path at all.
 *
 * Every function names the reference source it follows (paths relative to the reference
 * tree).  Arrays are passed flat instead of through the reference's structs so the same
 * functions serve any slice of a matrix.  Built with -ffp-contract=off so that sums are
 * formed exactly as written: left to right, one rounding per multiply and per add.
 *
 * Pinning: tests/test_oracle.py checks these functions against tests/golden/ vectors that
 * were produced by the reference's own sources (oracle/_ref, see oracle/Makefile), and, when
 * oracle/_ref/libalpha_ref.so is present, against that library live on the same inputs.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef int32_t aint;

/* status codes: include/alphasparse/spdef.h:8-19 */
enum { ST_SUCCESS = 0, ST_NOT_INITIALIZED = 1, ST_INVALID_VALUE = 3, ST_NOT_SUPPORTED = 6 };

/* ---------------------------------------------------------------------------------------
 * y = beta*y + alpha*(A x), one row after the other, products added left to right.
 * src/plain/kernel/level2/mv/gemv/gemv_x_csr_plain.c:4-24: y[r] is scaled by beta first,
 * the row's dot product is accumulated from zero, then alpha*dot is added.
 * ------------------------------------------------------------------------------------- */
#define DEF_GEMV(T, sfx)                                                                      \
    void oracle_gemv_csr_##sfx(aint rows, const aint *rs, const aint *re, const aint *col,    \
                               const T *val, T alpha, const T *x, T beta, T *y) {             \
        for (aint r = 0; r < rows; r++) {                                                     \
            T out = y[r] * beta;                                                              \
            T dot = 0;                                                                        \
            for (aint k = rs[r]; k < re[r]; k++) dot += val[k] * x[col[k]];                   \
            y[r] = out + alpha * dot;                                                         \
        }                                                                                     \
    }
DEF_GEMV(float, s)
DEF_GEMV(double, d)

/* ---------------------------------------------------------------------------------------
 * y = beta*y + alpha*(A^T x): y (length cols) scaled first, then every stored element
 * scatters (alpha*a)*x[row] into y[col], rows ascending.
 * src/plain/kernel/level2/mv/gemv/gemv_x_csr_trans_plain.c:4-27.
 * ------------------------------------------------------------------------------------- */
#define DEF_GEMV_T(T, sfx)                                                                    \
    void oracle_gemv_csr_trans_##sfx(aint rows, aint cols, const aint *rs, const aint *re,    \
                                     const aint *col, const T *val, T alpha, const T *x,      \
                                     T beta, T *y) {                                          \
        for (aint c = 0; c < cols; c++) y[c] = y[c] * beta;                                   \
        for (aint r = 0; r < rows; r++)                                                       \
            for (aint k = rs[r]; k < re[r]; k++) {                                            \
                T av = alpha * val[k];                                                        \
                y[col[k]] += av * x[r];                                                       \
            }                                                                                 \
    }
DEF_GEMV_T(float, s)
DEF_GEMV_T(double, d)

/* ---------------------------------------------------------------------------------------
 * Row-major SpMM, Y (rows x columns, leading dimension ldy) = beta*Y + alpha*A*X.
 * src/plain/kernel/level3/mm/gemm/gemm_x_csr_row_plain.c:4-23: the output row is scaled
 * by beta, then each stored element adds (alpha*a) * X[col, :] -- alpha is folded into the
 * element BEFORE the accumulation, unlike the SpMV above.
 * ------------------------------------------------------------------------------------- */
#define DEF_GEMM_ROW(T, sfx)                                                                  \
    void oracle_gemm_csr_row_##sfx(aint rows, const aint *rs, const aint *re,                 \
                                   const aint *col, const T *val, T alpha, const T *X,        \
                                   aint columns, aint ldx, T beta, T *Y, aint ldy) {          \
        for (aint r = 0; r < rows; r++) {                                                     \
            T *out = Y + (size_t)r * ldy;                                                     \
            for (aint c = 0; c < columns; c++) out[c] = out[c] * beta;                        \
            for (aint k = rs[r]; k < re[r]; k++) {                                            \
                T av = alpha * val[k];                                                        \
                const T *in = X + (size_t)col[k] * ldx;                                       \
                for (aint c = 0; c < columns; c++) out[c] += av * in[c];                      \
            }                                                                                 \
        }                                                                                     \
    }
DEF_GEMM_ROW(float, s)
DEF_GEMM_ROW(double, d)

/* ---------------------------------------------------------------------------------------
 * Column-major SpMM: element (r, c) of a dense operand lives at [c*ld + r].
 * src/plain/kernel/level3/mm/gemm/gemm_x_csr_col_plain.c:4-21: for every dense column and
 * every sparse row a dot product from zero, then y = y*beta + alpha*dot.
 * ------------------------------------------------------------------------------------- */
#define DEF_GEMM_COL(T, sfx)                                                                  \
    void oracle_gemm_csr_col_##sfx(aint rows, const aint *rs, const aint *re,                 \
                                   const aint *col, const T *val, T alpha, const T *X,        \
                                   aint columns, aint ldx, T beta, T *Y, aint ldy) {          \
        for (aint c = 0; c < columns; c++)                                                    \
            for (aint r = 0; r < rows; r++) {                                                 \
                T dot = 0;                                                                    \
                for (aint k = rs[r]; k < re[r]; k++)                                          \
                    dot += val[k] * X[(size_t)c * ldx + col[k]];                              \
                T *o = Y + (size_t)c * ldy + r;                                               \
                *o = *o * beta;                                                               \
                *o += alpha * dot;                                                            \
            }                                                                                 \
    }
DEF_GEMM_COL(float, s)
DEF_GEMM_COL(double, d)

/* ---------------------------------------------------------------------------------------
 * The OpenMP kernel of the reference's x86_64 tree (the timed CPU baseline when the
 * reference's own objects are not available): rows are split into one contiguous range
 * per thread by oracle_partition_rows_by_nnz, each row's dot product uses four partial
 * sums over elements k, k+1, k+2, k+3 combined as (t0+t1)+(t2+t3), a scalar tail goes to
 * t0, and then y = y*beta + alpha*dot.
 * src/kernel/x86_64/level2/mv/gemv/gemv_x_csr.c:129-153 (dot), :155-182 (rows), :184-208.
 * ------------------------------------------------------------------------------------- */
void oracle_partition_rows_by_nnz(const aint *acc, aint rows, aint parts, aint *part);

static aint oracle_thread_id(void) {
#ifdef _OPENMP
    return (aint)omp_get_thread_num();
#else
    return 0;
#endif
}

#define DEF_GEMV_OMP(T, sfx)                                                                  \
    void oracle_gemv_csr_omp_##sfx(aint rows, const aint *rs, const aint *re,                 \
                                   const aint *col, const T *val, T alpha, const T *x,        \
                                   T beta, T *y, aint threads) {                              \
        if (threads < 1) threads = 1;                                                         \
        aint *part = (aint *)malloc(sizeof(aint) * ((size_t)threads + 1));                    \
        oracle_partition_rows_by_nnz(re, rows, threads, part);                                \
        _Pragma("omp parallel num_threads(threads)")                                          \
        {                                                                                     \
            const aint t = oracle_thread_id();                                                \
            for (aint r = part[t]; r < part[t + 1]; r++) {                                    \
                const aint b = rs[r], n = re[r] - b, n4 = n & ~3;                             \
                T t0 = 0, t1 = 0, t2 = 0, t3 = 0;                                             \
                aint k = 0;                                                                   \
                for (; k < n4; k += 4) {                                                      \
                    t0 += val[b + k] * x[col[b + k]];                                         \
                    t1 += val[b + k + 1] * x[col[b + k + 1]];                                 \
                    t2 += val[b + k + 2] * x[col[b + k + 2]];                                 \
                    t3 += val[b + k + 3] * x[col[b + k + 3]];                                 \
                }                                                                             \
                for (; k < n; k++) t0 += val[b + k] * x[col[b + k]];                          \
                t0 += t1;                                                                     \
                t2 += t3;                                                                     \
                t0 += t2;                                                                     \
                y[r] = y[r] * beta;                                                           \
                y[r] += alpha * t0;                                                           \
            }                                                                                 \
        }                                                                                     \
        free(part);                                                                           \
    }

DEF_GEMV_OMP(float, s)
DEF_GEMV_OMP(double, d)

/* OpenMP row-major SpMM of the x86_64 tree: a parallel-for over rows around the same
 * arithmetic as the serial kernel.  src/kernel/x86_64/level3/mm/gemm/gemm_x_csr_row.c:4-27 */
#define DEF_GEMM_ROW_OMP(T, sfx)                                                              \
    void oracle_gemm_csr_row_omp_##sfx(aint rows, const aint *rs, const aint *re,             \
                                       const aint *col, const T *val, T alpha, const T *X,    \
                                       aint columns, aint ldx, T beta, T *Y, aint ldy,        \
                                       aint threads) {                                        \
        if (threads < 1) threads = 1;                                                         \
        _Pragma("omp parallel for num_threads(threads)")                                      \
        for (aint r = 0; r < rows; r++) {                                                     \
            T *out = Y + (size_t)r * ldy;                                                     \
            for (aint c = 0; c < columns; c++) out[c] = out[c] * beta;                        \
            for (aint k = rs[r]; k < re[r]; k++) {                                            \
                T av = alpha * val[k];                                                        \
                const T *in = X + (size_t)col[k] * ldx;                                       \
                for (aint c = 0; c < columns; c++) out[c] += av * in[c];                      \
            }                                                                                 \
        }                                                                                     \
    }
DEF_GEMM_ROW_OMP(float, s)
DEF_GEMM_ROW_OMP(double, d)

int oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_num_procs();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------------------------------
 * First index in [lo, hi) whose element is >= value.  src/util/partition.c:46-61.
 * ------------------------------------------------------------------------------------- */
aint oracle_lower_bound(const aint *t, aint lo, aint hi, aint value) {
    while (hi > lo) {
        aint mid = (lo + hi) / 2;
        if (t[mid] < value) lo = mid + 1;
        else hi = mid;
    }
    return lo;
}

/* ---------------------------------------------------------------------------------------
 * nnz-balanced contiguous row split.  src/util/partition.c:79-92.  `acc` is rows_end, the
 * inclusive prefix sums of the row lengths.  Quirks kept on purpose: the average is an
 * integer division; the search range stops at rows-1; a row that crosses a boundary falls
 * into the following part; parts may be empty.
 * ------------------------------------------------------------------------------------- */
void oracle_partition_rows_by_nnz(const aint *acc, aint rows, aint parts, aint *part) {
    const aint total = acc[rows - 1];
    const aint share = total / parts;
    part[0] = 0;
    for (aint p = 1; p < parts; p++) part[p] = oracle_lower_bound(acc, 0, rows - 1, share * p);
    part[parts] = rows;
}

/* ---------------------------------------------------------------------------------------
 * 4-array user CSR -> owned 3-array CSR.  src/core/format/alphasparse_x_create_csr.c:22-55:
 * nnz = rows_end[rows-1] - rows_start[0]; offsets[0] = rows_start[0], offsets[i+1] =
 * rows_end[i]; columns and values are copied from element 0 of the user arrays; with
 * one-based input one is subtracted from every offset and every column.
 * out_ptr has rows+1 entries; out_col / out_val have nnz entries.  Returns nnz.
 * ------------------------------------------------------------------------------------- */
#define DEF_CREATE(T, sfx)                                                                    \
    aint oracle_create_csr_##sfx(aint base, aint rows, const aint *rs, const aint *re,        \
                                 const aint *col, const T *val, aint *out_ptr, aint *out_col, \
                                 T *out_val) {                                                \
        const aint nnz = re[rows - 1] - rs[0];                                                \
        const aint shift = base ? 1 : 0;                                                      \
        if (out_ptr) {                                                                        \
            out_ptr[0] = rs[0] - shift;                                                       \
            for (aint i = 0; i < rows; i++) out_ptr[i + 1] = re[i] - shift;                   \
        }                                                                                     \
        if (out_col)                                                                          \
            for (aint i = 0; i < nnz; i++) {                                                  \
                out_col[i] = col[i] - shift;                                                  \
                out_val[i] = val[i];                                                          \
            }                                                                                 \
        return nnz;                                                                           \
    }
DEF_CREATE(float, s)
DEF_CREATE(double, d)

/* ---------------------------------------------------------------------------------------
 * COO -> CSR.  src/core/format/alphasparse_x_create_coo.c:30-45 (one-based input is
 * rebased) and src/core/format/convert_csr_x_coo.c:14-81: (row, col, value) records are
 * sorted by row then column, offsets come from one sweep over the sorted rows, columns and
 * values are copied in sorted order.  Duplicated (row, col) pairs are all kept.  The
 * reference sorts with qsort, whose order among equal keys is unspecified; this restatement
 * uses a stable merge sort, so it agrees with any outcome of the reference whenever the
 * duplicates carry equal values or there are none.
 * ------------------------------------------------------------------------------------- */
#define DEF_COO2CSR(T, sfx)                                                                   \
    typedef struct { aint r, c; T v; } rec_##sfx;                                             \
    static void msort_##sfx(rec_##sfx *a, rec_##sfx *tmp, size_t n) {                         \
        if (n < 2) return;                                                                    \
        size_t h = n / 2;                                                                     \
        msort_##sfx(a, tmp, h);                                                               \
        msort_##sfx(a + h, tmp, n - h);                                                       \
        size_t i = 0, j = h, o = 0;                                                           \
        while (i < h && j < n) {                                                              \
            int take_right = (a[j].r < a[i].r) || (a[j].r == a[i].r && a[j].c < a[i].c);      \
            tmp[o++] = take_right ? a[j++] : a[i++];                                          \
        }                                                                                     \
        while (i < h) tmp[o++] = a[i++];                                                      \
        while (j < n) tmp[o++] = a[j++];                                                      \
        memcpy(a, tmp, n * sizeof(rec_##sfx));                                                \
    }                                                                                         \
    void oracle_coo_to_csr_##sfx(aint base, aint rows, aint nnz, const aint *ri,              \
                                 const aint *ci, const T *v, aint *out_ptr, aint *out_col,    \
                                 T *out_val) {                                                \
        const aint shift = base ? 1 : 0;                                                      \
        rec_##sfx *a = (rec_##sfx *)malloc(sizeof(rec_##sfx) * (size_t)(nnz > 0 ? nnz : 1));  \
        rec_##sfx *tmp = (rec_##sfx *)malloc(sizeof(rec_##sfx) * (size_t)(nnz > 0 ? nnz : 1));\
        for (aint i = 0; i < nnz; i++) {                                                      \
            a[i].r = ri[i] - shift;                                                           \
            a[i].c = ci[i] - shift;                                                           \
            a[i].v = v[i];                                                                    \
        }                                                                                     \
        msort_##sfx(a, tmp, (size_t)nnz);                                                     \
        for (aint r = 0; r <= rows; r++) out_ptr[r] = 0;                                      \
        for (aint i = 0; i < nnz; i++)                                                        \
            if (a[i].r >= 0 && a[i].r < rows) out_ptr[a[i].r + 1]++;                          \
        for (aint r = 0; r < rows; r++) out_ptr[r + 1] += out_ptr[r];                         \
        for (aint i = 0; i < nnz; i++) {                                                      \
            out_col[i] = a[i].c;                                                              \
            out_val[i] = a[i].v;                                                              \
        }                                                                                     \
        free(a);                                                                              \
        free(tmp);                                                                            \
    }
DEF_COO2CSR(float, s)
DEF_COO2CSR(double, d)

/* ---------------------------------------------------------------------------------------
 * Argument checks of alphasparse_?_mv in the order the reference applies them.
 * src/core/op/level2/alphasparse_x_mv.c:1670-1716 (real precisions):
 *   handle / handle->mat / x / y NULL            -> NOT_INITIALIZED
 *   handle datatype != precision of the call     -> INVALID_VALUE
 *   CONJUGATE_TRANSPOSE on a real type           -> INVALID_VALUE
 *   SYMMETRIC or HERMITIAN on a non-square A     -> INVALID_VALUE
 *   then format CSR + type GENERAL runs gemv; a descriptor type outside 0..4 or an unknown
 *   format -> INVALID_VALUE.
 * Returns ST_SUCCESS when the call reaches the CSR/GENERAL kernel, -1 when it reaches some
 * other kernel of the reference (outside this path), else the error status.
 * ------------------------------------------------------------------------------------- */
int oracle_mv_status(int has_handle, int has_mat, int has_x, int has_y, int handle_datatype,
                     int call_datatype, int operation, int descr_type, int format, aint rows,
                     aint cols) {
    if (!has_handle || !has_mat || !has_x || !has_y) return ST_NOT_INITIALIZED;
    if (handle_datatype != call_datatype) return ST_INVALID_VALUE;
    if (operation == 2) return ST_INVALID_VALUE;
    if ((descr_type == 1 || descr_type == 2) && rows != cols) return ST_INVALID_VALUE;
    if (format == 1 /* CSR */) {
        if (descr_type == 0) return ST_SUCCESS;
        if (descr_type >= 1 && descr_type <= 4) return -1;
        return ST_INVALID_VALUE;
    }
    if (format == 0 || (format >= 2 && format <= 5)) return -1;
    return ST_INVALID_VALUE;
}

/* alphasparse_?_mm applies the same checks in the same order
 * (src/core/op/level3/alphasparse_x_mm.c:2317-2338); the kernel is picked by
 * layout + 2*operation (:47-63). */
int oracle_mm_status(int has_handle, int has_mat, int has_x, int has_y, int handle_datatype,
                     int call_datatype, int operation, int descr_type, int format, aint rows,
                     aint cols) {
    return oracle_mv_status(has_handle, has_mat, has_x, has_y, handle_datatype, call_datatype,
                            operation, descr_type, format, rows, cols);
}

/* ---------------------------------------------------------------------------------------
 * Structured descriptors on a CSR handle (the other branches of alphasparse_?_mv's CSR
 * block, src/core/op/level2/alphasparse_x_mv.c:1693-1716).  A is square; only the stored
 * elements on the requested side of the diagonal take part.
 *
 * TRIANGULAR, src/plain/kernel/level2/mv/trmv/csr/trmv_x_csr_{n,u}_{lo,hi}[_trans]_plain.c:
 *   y = beta*y + alpha*op(T)*x, T = lower (col <= row) or upper (col >= row) part; with a
 *   unit diagonal the stored diagonal is ignored and x[row] is added instead.  Non-transposed:
 *   a dot product per row from zero (from x[row] when unit), scaled by alpha, added to beta*y.
 *   Transposed: y scaled row by row while every kept element scatters (alpha*a)*x[row] into
 *   y[col]; unit adds alpha*x[row] to y[row].
 * SYMMETRIC, .../symv/csr/symv_x_csr_{n,u}_{lo,hi}_plain.c: every kept off-diagonal element a
 *   contributes (alpha*a)*x[row] to y[col] and (alpha*a)*x[col] to y[row]; diagonal elements
 *   once (or alpha*x[row] when unit).  Only operation NON_TRANSPOSE is in the dispatch table
 *   (alphasparse_x_mv.c:89-107); TRANSPOSE returns NOT_SUPPORTED.
 * DIAGONAL, .../diagmv/diagmv_x_csr_{n,u}_plain.c: y = beta*y + alpha*d.*x where d[row] is the
 *   FIRST stored element of the row whose column equals the row (1 when unit, 0 if none).
 * ------------------------------------------------------------------------------------- */
#define DEF_STRUCT(T, sfx)                                                                    \
    void oracle_trmv_csr_##sfx(int upper, int unit, int trans, aint rows, const aint *rs,     \
                               const aint *re, const aint *col, const T *val, T alpha,        \
                               const T *x, T beta, T *y) {                                    \
        if (!trans) {                                                                         \
            for (aint i = 0; i < rows; i++) {                                                 \
                T dot = unit ? x[i] : (T)0;                                                   \
                for (aint k = rs[i]; k < re[i]; k++) {                                        \
                    const aint c = col[k];                                                    \
                    const int keep = upper ? (unit ? c > i : c >= i) : (unit ? c < i : c <= i); \
                    if (keep) dot += val[k] * x[c];                                           \
                }                                                                             \
                dot = dot * alpha;                                                            \
                y[i] = y[i] * beta;                                                           \
                y[i] += dot;                                                                  \
            }                                                                                 \
        } else {                                                                              \
            for (aint i = 0; i < rows; i++) y[i] = y[i] * beta;                               \
            for (aint i = 0; i < rows; i++) {                                                 \
                if (unit) y[i] += alpha * x[i];                                               \
                for (aint k = rs[i]; k < re[i]; k++) {                                        \
                    const aint c = col[k];                                                    \
                    const int keep = upper ? (unit ? c > i : c >= i) : (unit ? c < i : c <= i); \
                    if (keep) {                                                               \
                        T av = alpha * val[k];                                                \
                        y[c] += av * x[i];                                                    \
                    }                                                                         \
                }                                                                             \
            }                                                                                 \
        }                                                                                     \
    }                                                                                         \
    void oracle_symv_csr_##sfx(int upper, int unit, aint rows, const aint *rs, const aint *re, \
                               const aint *col, const T *val, T alpha, const T *x, T beta,    \
                               T *y) {                                                        \
        for (aint i = 0; i < rows; i++) y[i] = y[i] * beta;                                   \
        for (aint i = 0; i < rows; i++) {                                                     \
            if (unit) y[i] += alpha * x[i];                                                   \
            for (aint k = rs[i]; k < re[i]; k++) {                                            \
                const aint c = col[k];                                                        \
                const int off = upper ? c > i : c < i;                                        \
                T av = alpha * val[k];                                                        \
                if (off) {                                                                    \
                    y[c] += av * x[i];                                                        \
                    y[i] += av * x[c];                                                        \
                } else if (c == i && !unit) {                                                 \
                    y[i] += av * x[c];                                                        \
                }                                                                             \
            }                                                                                 \
        }                                                                                     \
    }                                                                                         \
    void oracle_diagmv_csr_##sfx(int unit, aint rows, const aint *rs, const aint *re,         \
                                 const aint *col, const T *val, T alpha, const T *x, T beta,  \
                                 T *y) {                                                      \
        for (aint i = 0; i < rows; i++) {                                                     \
            y[i] = y[i] * beta;                                                               \
            if (unit) {                                                                       \
                y[i] += alpha * x[i];                                                         \
                continue;                                                                     \
            }                                                                                 \
            for (aint k = rs[i]; k < re[i]; k++)                                              \
                if (col[k] == i) {                                                            \
                    T av = alpha * val[k];                                                    \
                    y[i] += av * x[i];                                                        \
                    break;                                                                    \
                }                                                                             \
        }                                                                                     \
    }
DEF_STRUCT(float, s)
DEF_STRUCT(double, d)

/* ---------------------------------------------------------------------------------------
 * The same descriptors in alphasparse_?_mm (src/core/op/level3/alphasparse_x_mm.c:2345-2368;
 * tables :116-151, :303-335, :381-393).  X and Y are dense, `columns` wide; element (r, c) sits at
 * r*ld + c (row-major) or c*ld + r (column-major).
 *
 * SYMMETRIC, src/plain/kernel/level3/mm/symm/csr/symm_x_csr_{n,u}_{lo,hi}_{row,col}_plain.c: Y is
 *   scaled by beta (plus alpha*X when the diagonal is unit), then every kept off-diagonal element a
 *   adds (alpha*a)*X[col,:] to Y[row,:] and (alpha*a)*X[row,:] to Y[col,:]; stored diagonal elements
 *   once.  TRANSPOSE has no table entry (NOT_SUPPORTED).
 * TRIANGULAR, .../trmm/csr/trmm_x_csr_{n,u}_{lo,hi}_{row,col}[_trans]_plain.c: row-major adds
 *   (alpha*a)*X[col,:] per kept element; column-major forms the dot product first and adds
 *   alpha*dot.  The transposed kernels materialise A^T (transpose_csr) and run the kernel of the
 *   opposite triangle on it.
 * DIAGONAL, .../diagmm/diagmm_x_csr_{n,u}_{row,col}_plain.c: the row-major kernel adds EVERY stored
 *   diagonal element of a row, the column-major one keeps the LAST (diagmv keeps the first); the
 *   three agree unless a row stores its diagonal more than once.
 * ------------------------------------------------------------------------------------- */
#define AT(r, c, ld) (col_major ? (size_t)(c) * (size_t)(ld) + (size_t)(r) : (size_t)(r) * (size_t)(ld) + (size_t)(c))
#define DEF_STRUCT_MM(T, sfx)                                                                 \
    void oracle_symm_csr_##sfx(int upper, int unit, int col_major, aint rows, const aint *rs, \
                               const aint *re, const aint *col, const T *val, T alpha,        \
                               const T *x, aint columns, aint ldx, T beta, T *y, aint ldy) {  \
        for (aint r = 0; r < rows; r++)                                                       \
            for (aint c = 0; c < columns; c++) {                                              \
                y[AT(r, c, ldy)] = y[AT(r, c, ldy)] * beta;                                   \
                if (unit) y[AT(r, c, ldy)] += alpha * x[AT(r, c, ldx)];                       \
            }                                                                                 \
        for (aint r = 0; r < rows; r++)                                                       \
            for (aint k = rs[r]; k < re[r]; k++) {                                            \
                const aint j = col[k];                                                        \
                const int off = upper ? j > r : j < r;                                        \
                if (!off && (j != r || unit)) continue;                                       \
                const T av = alpha * val[k];                                                  \
                for (aint c = 0; c < columns; c++) {                                          \
                    y[AT(r, c, ldy)] += av * x[AT(j, c, ldx)];                                \
                    if (off) y[AT(j, c, ldy)] += av * x[AT(r, c, ldx)];                       \
                }                                                                             \
            }                                                                                 \
    }                                                                                         \
    void oracle_trmm_csr_##sfx(int upper, int unit, int trans, int col_major, aint rows,      \
                               const aint *rs, const aint *re, const aint *col, const T *val, \
                               T alpha, const T *x, aint columns, aint ldx, T beta, T *y,     \
                               aint ldy) {                                                    \
        aint *tptr = NULL, *tcol = NULL;                                                      \
        T *tval = NULL;                                                                       \
        if (trans) { /* A^T by a counting sort: rows ascending inside every column */         \
            const aint nnz = rows ? re[rows - 1] - rs[0] : 0;                                 \
            tptr = (aint *)calloc((size_t)rows + 1, sizeof(aint));                            \
            tcol = (aint *)malloc(sizeof(aint) * (size_t)(nnz ? nnz : 1));                    \
            tval = (T *)malloc(sizeof(T) * (size_t)(nnz ? nnz : 1));                          \
            for (aint r = 0; r < rows; r++)                                                   \
                for (aint k = rs[r]; k < re[r]; k++) tptr[col[k] + 1]++;                      \
            for (aint r = 0; r < rows; r++) tptr[r + 1] += tptr[r];                           \
            aint *fill = (aint *)malloc(sizeof(aint) * (size_t)(rows ? rows : 1));            \
            memcpy(fill, tptr, sizeof(aint) * (size_t)rows);                                  \
            for (aint r = 0; r < rows; r++)                                                   \
                for (aint k = rs[r]; k < re[r]; k++) {                                        \
                    const aint p = fill[col[k]]++;                                            \
                    tcol[p] = r, tval[p] = val[k];                                            \
                }                                                                             \
            free(fill);                                                                       \
            rs = tptr, re = tptr + 1, col = tcol, val = tval, upper = !upper;                 \
        }                                                                                     \
        for (aint c = 0; c < columns; c++)                                                    \
            for (aint r = 0; r < rows; r++) {                                                 \
                T *out = &y[AT(r, c, ldy)];                                                   \
                *out = *out * beta;                                                           \
                if (unit) *out += alpha * x[AT(r, c, ldx)];                                   \
                T dot = (T)0;                                                                 \
                for (aint k = rs[r]; k < re[r]; k++) {                                        \
                    const aint j = col[k];                                                    \
                    const int keep = upper ? (unit ? j > r : j >= r) : (unit ? j < r : j <= r); \
                    if (!keep) continue;                                                      \
                    if (col_major) dot += val[k] * x[AT(j, c, ldx)];                          \
                    else { const T av = alpha * val[k]; *out += av * x[AT(j, c, ldx)]; }      \
                }                                                                             \
                if (col_major) *out += dot * alpha;                                           \
            }                                                                                 \
        free(tptr), free(tcol), free(tval);                                                   \
    }                                                                                         \
    void oracle_diagmm_csr_##sfx(int unit, int col_major, aint rows, const aint *rs,          \
                                 const aint *re, const aint *col, const T *val, T alpha,      \
                                 const T *x, aint columns, aint ldx, T beta, T *y, aint ldy) { \
        for (aint r = 0; r < rows; r++)                                                       \
            for (aint c = 0; c < columns; c++) {                                              \
                T *out = &y[AT(r, c, ldy)];                                                   \
                *out = *out * beta;                                                           \
                if (unit) { *out += alpha * x[AT(r, c, ldx)]; continue; }                     \
                if (col_major) {                                                              \
                    T d = (T)0;                                                               \
                    for (aint k = rs[r]; k < re[r]; k++) if (col[k] == r) d = val[k];         \
                    const T av = alpha * d;                                                   \
                    *out += av * x[AT(r, c, ldx)];                                            \
                } else {                                                                      \
                    for (aint k = rs[r]; k < re[r]; k++)                                      \
                        if (col[k] == r) { const T av = alpha * val[k]; *out += av * x[AT(r, c, ldx)]; } \
                }                                                                             \
            }                                                                                 \
    }
DEF_STRUCT_MM(float, s)
DEF_STRUCT_MM(double, d)
#undef AT

/* ---------------------------------------------------------------------------------------
 * A COO handle given straight to mv / mm with a GENERAL descriptor
 * (src/core/op/level2/alphasparse_x_mv.c:1718-1724, src/core/op/level3/alphasparse_x_mm.c:2370-2376).
 *   src/plain/kernel/level2/mv/gemv/gemv_x_coo_plain.c, gemv_x_coo_trans_plain.c: y scaled by beta,
 *   then every entry in stored order adds alpha*(a*x[col]) to y[row] (transposed: alpha*(a*x[row]) to
 *   y[col], y has `cols` entries).
 *   src/plain/kernel/level3/mm/gemm/gemm_x_coo_row_plain.c: every entry adds (alpha*a)*X[col,:] to
 *   Y[row,:]; gemm_x_coo_col_plain.c: alpha*(a*X[col,c]) per dense column c.  The transposed kernels
 *   swap the index arrays (transpose_coo) and run the same loops.
 * ------------------------------------------------------------------------------------- */
#define DEF_COO(T, sfx)                                                                       \
    void oracle_gemv_coo_##sfx(int trans, aint rows, aint cols, aint nnz, const aint *ri,     \
                               const aint *ci, const T *val, T alpha, const T *x, T beta,     \
                               T *y) {                                                        \
        const aint m = trans ? cols : rows;                                                   \
        for (aint i = 0; i < m; i++) y[i] = y[i] * beta;                                      \
        for (aint k = 0; k < nnz; k++) {                                                      \
            const aint r = trans ? ci[k] : ri[k], c = trans ? ri[k] : ci[k];                  \
            const T v = val[k] * x[c];                                                        \
            y[r] += alpha * v;                                                                \
        }                                                                                     \
    }                                                                                         \
    void oracle_gemm_coo_##sfx(int trans, int col_major, aint rows, aint cols, aint nnz,      \
                               const aint *ri, const aint *ci, const T *val, T alpha,         \
                               const T *x, aint columns, aint ldx, T beta, T *y, aint ldy) {  \
        const aint m = trans ? cols : rows;                                                   \
        for (aint r = 0; r < m; r++)                                                          \
            for (aint c = 0; c < columns; c++) {                                              \
                T *out = col_major ? &y[(size_t)c * ldy + r] : &y[(size_t)r * ldy + c];       \
                *out = *out * beta;                                                           \
            }                                                                                 \
        if (col_major) {                                                                      \
            for (aint c = 0; c < columns; c++)                                                \
                for (aint k = 0; k < nnz; k++) {                                              \
                    const aint r = trans ? ci[k] : ri[k], j = trans ? ri[k] : ci[k];          \
                    const T v = val[k] * x[(size_t)c * ldx + j];                              \
                    y[(size_t)c * ldy + r] += alpha * v;                                      \
                }                                                                             \
        } else {                                                                              \
            for (aint k = 0; k < nnz; k++) {                                                  \
                const aint r = trans ? ci[k] : ri[k], j = trans ? ri[k] : ci[k];              \
                const T av = alpha * val[k];                                                  \
                for (aint c = 0; c < columns; c++) y[(size_t)r * ldy + c] += av * x[(size_t)j * ldx + c]; \
            }                                                                                 \
        }                                                                                     \
    }
DEF_COO(float, s)
DEF_COO(double, d)

/* ---------------------------------------------------------------------------------------
 * A CSC handle in mv / mm with a GENERAL descriptor (the CSC blocks of alphasparse_x_mv.c and
 * alphasparse_x_mm.c).  Arrays: cs/ce column offsets, ri row indices.
 *   src/plain/kernel/level2/mv/gemv/gemv_x_csc_plain.c: y scaled by beta, then column by column every
 *   element adds alpha*(a*x[col]) to y[row]; gemv_x_csc_trans_plain.c: per column a dot product with
 *   x[row], times alpha, added to beta*y[col].
 *   src/plain/kernel/level3/mm/gemm/gemm_x_csc_row_plain.c / _col_plain.c: Y scaled by beta, then every
 *   element adds (alpha*a)*X[col,:] to Y[row,:] in column order; the transposed kernels materialise
 *   the CSC of A^T (transpose_csc) and run the same loops on it.
 * ------------------------------------------------------------------------------------- */
#define DEF_CSC(T, sfx)                                                                       \
    void oracle_gemv_csc_##sfx(int trans, aint rows, aint cols, const aint *cs, const aint *ce, \
                               const aint *ri, const T *val, T alpha, const T *x, T beta,     \
                               T *y) {                                                        \
        if (!trans) {                                                                         \
            for (aint j = 0; j < rows; j++) y[j] = y[j] * beta;                               \
            for (aint c = 0; c < cols; c++)                                                   \
                for (aint k = cs[c]; k < ce[c]; k++) {                                        \
                    T t = val[k] * x[c];                                                      \
                    t = alpha * t;                                                            \
                    y[ri[k]] = y[ri[k]] + t;                                                  \
                }                                                                             \
        } else {                                                                              \
            for (aint c = 0; c < cols; c++) {                                                 \
                T t = (T)0;                                                                   \
                y[c] = y[c] * beta;                                                           \
                for (aint k = cs[c]; k < ce[c]; k++) t = t + val[k] * x[ri[k]];               \
                t = alpha * t;                                                                \
                y[c] = y[c] + t;                                                              \
            }                                                                                 \
        }                                                                                     \
    }                                                                                         \
    void oracle_gemm_csc_##sfx(int trans, int col_major, aint rows, aint cols, const aint *cs, \
                               const aint *ce, const aint *ri, const T *val, T alpha,         \
                               const T *x, aint columns, aint ldx, T beta, T *y, aint ldy) {  \
        /* op(A) is m x n; with trans the roles of stored column and row index swap, and the   \
           reference walks A^T's columns (A's rows) in order: same sums, another order */      \
        const aint m = trans ? cols : rows;                                                   \
        for (aint r = 0; r < m; r++)                                                          \
            for (aint c = 0; c < columns; c++) {                                              \
                T *out = col_major ? &y[(size_t)c * ldy + r] : &y[(size_t)r * ldy + c];       \
                *out = *out * beta;                                                           \
            }                                                                                 \
        for (aint c = 0; c < cols; c++)                                                       \
            for (aint k = cs[c]; k < ce[c]; k++) {                                            \
                const aint out_r = trans ? c : ri[k], in_r = trans ? ri[k] : c;               \
                const T av = alpha * val[k];                                                  \
                for (aint d = 0; d < columns; d++) {                                          \
                    if (col_major) y[(size_t)d * ldy + out_r] += av * x[(size_t)d * ldx + in_r]; \
                    else y[(size_t)out_r * ldy + d] += av * x[(size_t)in_r * ldx + d];        \
                }                                                                             \
            }                                                                                 \
    }
DEF_CSC(float, s)
DEF_CSC(double, d)
