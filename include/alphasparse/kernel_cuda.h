#pragma once
/*
 * Kernel-level entry points of the sm_100a backend: the symbols the reference's dispatch tables call for a
 * CSR matrix under a GENERAL descriptor.  In the reference every architecture tree under src/kernel (plain,
 * arm, hygon, dcu; chosen by src/kernel/Makefile:2-11) defines them; src/core/op/level2/alphasparse_x_mv.c:40-50
 * and src/core/op/level3/alphasparse_x_mm.c:47-63 reach them through gemv_csr / gemm_csr_row / ... macros
 * (include/alphasparse/kernel/def_s.h:118-120,140-143).  Linking this library in place of such a tree gives the
 * reference's own host code (its create_csr, its argument checks, its dispatch) this backend's kernels.
 *
 * Signatures: include/alphasparse/kernel/kernel_csr_s.h:13-15,65-72 and kernel_csr_d.h:13-15,65-72 of the
 * reference.  `A` is the bare host CSR record.  Records of handles created by this library already have a device
 * copy; any other record (zero-based, rows stored back to back) is uploaded and analysed at its first use and
 * stays on the device until alphasparse_cuda_release_csr(record) -- call that from the tree's destroy hook, before
 * the record's arrays are freed or changed.  x / y (X / Y) may be host or device pointers, as in alphasparse_?_mv.
 */
#include "types.h"
#include "spdef.h"
#include "spmat.h"

#ifdef __cplusplus
extern "C" {
#endif

/* y = alpha*A*x + beta*y and y = alpha*A^T*x + beta*y */
alphasparse_status_t gemv_s_csr(const float alpha, const spmat_csr_s_t *A, const float *x, const float beta, float *y);
alphasparse_status_t gemv_d_csr(const double alpha, const spmat_csr_d_t *A, const double *x, const double beta, double *y);
alphasparse_status_t gemv_s_csr_trans(const float alpha, const spmat_csr_s_t *A, const float *x, const float beta, float *y);
alphasparse_status_t gemv_d_csr_trans(const double alpha, const spmat_csr_d_t *A, const double *x, const double beta, double *y);

/* Y = alpha*op(A)*X + beta*Y, dense operands row-major (ld = distance between rows) or column-major */
alphasparse_status_t gemm_s_csr_row(const float alpha, const spmat_csr_s_t *mat, const float *x, const ALPHA_INT columns, const ALPHA_INT ldx, const float beta, float *y, const ALPHA_INT ldy);
alphasparse_status_t gemm_d_csr_row(const double alpha, const spmat_csr_d_t *mat, const double *x, const ALPHA_INT columns, const ALPHA_INT ldx, const double beta, double *y, const ALPHA_INT ldy);
alphasparse_status_t gemm_s_csr_col(const float alpha, const spmat_csr_s_t *mat, const float *x, const ALPHA_INT columns, const ALPHA_INT ldx, const float beta, float *y, const ALPHA_INT ldy);
alphasparse_status_t gemm_d_csr_col(const double alpha, const spmat_csr_d_t *mat, const double *x, const ALPHA_INT columns, const ALPHA_INT ldx, const double beta, double *y, const ALPHA_INT ldy);
alphasparse_status_t gemm_s_csr_row_trans(const float alpha, const spmat_csr_s_t *mat, const float *x, const ALPHA_INT columns, const ALPHA_INT ldx, const float beta, float *y, const ALPHA_INT ldy);
alphasparse_status_t gemm_d_csr_row_trans(const double alpha, const spmat_csr_d_t *mat, const double *x, const ALPHA_INT columns, const ALPHA_INT ldx, const double beta, double *y, const ALPHA_INT ldy);
alphasparse_status_t gemm_s_csr_col_trans(const float alpha, const spmat_csr_s_t *mat, const float *x, const ALPHA_INT columns, const ALPHA_INT ldx, const float beta, float *y, const ALPHA_INT ldy);
alphasparse_status_t gemm_d_csr_col_trans(const double alpha, const spmat_csr_d_t *mat, const double *x, const ALPHA_INT columns, const ALPHA_INT ldx, const double beta, double *y, const ALPHA_INT ldy);

/* Drops the device copy a kernel-level call made for a record this library did not create.  SUCCESS when there
 * is none; INVALID_VALUE for the record of a live handle of this library (alphasparse_destroy releases that). */
alphasparse_status_t alphasparse_cuda_release_csr(const void *record);

#ifdef __cplusplus
}
#endif
