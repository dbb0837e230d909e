/*
 * What the reference's dispatch layer does for a CSR matrix under a GENERAL descriptor: it holds a bare
 * spmat_csr_?_t record (made by its own create_csr, host arrays) and calls the kernel symbols of whichever
 * architecture tree was linked -- gemv_d_csr, gemv_s_csr, gemm_d_csr_row, ... (signatures:
 * include/alphasparse/kernel/kernel_csr_{s,d}.h:13-15,65-72 of the reference).  Here the tree is
 * libalphasparse_b200.so.  The prototypes are written out instead of included so that the file compiles
 * against the reference's include/ directory (for spmat.h) as well as against this repository's.
 *
 *   kernel_tree_caller in.bin out.bin
 * in.bin:  int32 rows, cols, nnz, columns; int32 ptr[rows+1]; int32 col[nnz]; double val[nnz];
 *          double x[cols*columns]; double y0[rows*columns]
 * out.bin: double y_mv[rows] (gemv_d_csr, x = first column block entry per row of X);
 *          float  y_mv_s[rows] (gemv_s_csr on the values rounded to float);
 *          double Y[rows*columns] (gemm_d_csr_row); double yt[cols] (gemv_d_csr_trans with x = y0[:rows], beta = 0)
 */
#include <alphasparse/spmat.h>
#include <alphasparse/spdef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

alphasparse_status_t gemv_d_csr(const double alpha, const spmat_csr_d_t *A, const double *x, const double beta, double *y);
alphasparse_status_t gemv_s_csr(const float alpha, const spmat_csr_s_t *A, const float *x, const float beta, float *y);
alphasparse_status_t gemv_d_csr_trans(const double alpha, const spmat_csr_d_t *A, const double *x, const double beta, double *y);
alphasparse_status_t gemm_d_csr_row(const double alpha, const spmat_csr_d_t *mat, const double *x, const ALPHA_INT columns,
                                    const ALPHA_INT ldx, const double beta, double *y, const ALPHA_INT ldy);
alphasparse_status_t alphasparse_cuda_release_csr(const void *record);

static void *take(FILE *fp, size_t bytes) {
    void *p = malloc(bytes ? bytes : 1);
    if (!p || fread(p, 1, bytes, fp) != bytes) exit(4);
    return p;
}

int main(int argc, char **argv) {
    if (argc < 3) return 2;
    FILE *fp = fopen(argv[1], "rb");
    if (!fp) return 2;
    int hdr[4];
    if (fread(hdr, sizeof(int), 4, fp) != 4) return 4;
    const int rows = hdr[0], cols = hdr[1], nnz = hdr[2], columns = hdr[3];
    int *ptr = (int *)take(fp, sizeof(int) * (size_t)(rows + 1));
    int *col = (int *)take(fp, sizeof(int) * (size_t)nnz);
    double *val = (double *)take(fp, sizeof(double) * (size_t)nnz);
    double *X = (double *)take(fp, sizeof(double) * (size_t)cols * columns);
    double *Y0 = (double *)take(fp, sizeof(double) * (size_t)rows * columns);
    fclose(fp);

    spmat_csr_d_t A;
    memset(&A, 0, sizeof(A));
    A.values = val, A.rows_start = ptr, A.rows_end = ptr + 1, A.col_indx = col, A.rows = rows, A.cols = cols;
    float *vals = (float *)malloc(sizeof(float) * (size_t)(nnz ? nnz : 1));
    for (int i = 0; i < nnz; i++) vals[i] = (float)val[i];
    spmat_csr_s_t As;
    memset(&As, 0, sizeof(As));
    As.values = vals, As.rows_start = ptr, As.rows_end = ptr + 1, As.col_indx = col, As.rows = rows, As.cols = cols;

    double *x = (double *)malloc(sizeof(double) * (size_t)cols), *y = (double *)malloc(sizeof(double) * (size_t)rows);
    float *xs = (float *)malloc(sizeof(float) * (size_t)cols), *ys = (float *)malloc(sizeof(float) * (size_t)rows);
    for (int j = 0; j < cols; j++) x[j] = X[(size_t)j * columns], xs[j] = (float)x[j];
    for (int i = 0; i < rows; i++) y[i] = Y0[(size_t)i * columns], ys[i] = (float)y[i];
    double *Y = (double *)malloc(sizeof(double) * (size_t)rows * columns);
    memcpy(Y, Y0, sizeof(double) * (size_t)rows * columns);
    double *yt = (double *)calloc((size_t)cols, sizeof(double));

    int bad = 0;
    bad |= gemv_d_csr(1.5, &A, x, 0.5, y) != ALPHA_SPARSE_STATUS_SUCCESS;
    bad |= gemv_s_csr(1.5f, &As, xs, 0.5f, ys) != ALPHA_SPARSE_STATUS_SUCCESS;
    bad |= gemm_d_csr_row(2.0, &A, X, columns, columns, -1.0, Y, columns) != ALPHA_SPARSE_STATUS_SUCCESS;
    bad |= gemv_d_csr_trans(1.0, &A, Y0, 0.0, yt) != ALPHA_SPARSE_STATUS_SUCCESS; /* first `rows` entries of Y0 as x */
    bad |= gemv_d_csr(1.5, &A, x, 0.5, y) != ALPHA_SPARSE_STATUS_SUCCESS;          /* second call: reuses the device copy */
    bad |= alphasparse_cuda_release_csr(&A) != ALPHA_SPARSE_STATUS_SUCCESS;
    bad |= alphasparse_cuda_release_csr(&As) != ALPHA_SPARSE_STATUS_SUCCESS;
    bad |= alphasparse_cuda_release_csr(&A) != ALPHA_SPARSE_STATUS_SUCCESS;        /* nothing left: still fine */
    if (bad) return 5;

    fp = fopen(argv[2], "wb");
    if (!fp) return 3;
    fwrite(y, sizeof(double), (size_t)rows, fp);
    fwrite(ys, sizeof(float), (size_t)rows, fp);
    fwrite(Y, sizeof(double), (size_t)rows * columns, fp);
    fwrite(yt, sizeof(double), (size_t)cols, fp);
    fclose(fp);
    return 0;
}
