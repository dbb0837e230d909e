#pragma once
/*
 * The alphasparse entry points served by the sm_100a backend.  Each prototype is
 * signature-identical to the one in include/alphasparse/spapi.h of the reference (line
 * ranges given per group) so that a caller relinks without recompiling.
 *
 * Pointer kinds.  The reference takes host pointers.  Here `x` and `y` of mv / mm may be
 * host pointers (copied to the device and back inside the call, which returns when y is
 * complete) or device pointers of the current device (the kernels are enqueued on the
 * library stream and the call returns without waiting, like any CUDA library call).
 * Matrix arrays given to the create calls are host pointers and are deep-copied.
 *
 * Descriptors.  mv and mm serve GENERAL, SYMMETRIC, TRIANGULAR and DIAGONAL on a CSR handle with
 * every fill / diag / operation combination the reference's dispatch tables hold (SYMMETRIC with
 * TRANSPOSE has no entry there and is NOT_SUPPORTED here too).
 *
 * A COO handle may be given to mv / mm directly with a GENERAL descriptor: the product runs on a CSR
 * copy converted on first use and kept with the handle.  CSC handles: see the CSC group below.
 *
 * What is not served.  Complex precisions (and so HERMITIAN), structured descriptors on a COO or CSC
 * handle and formats other than CSR, COO and CSC return ALPHA_SPARSE_STATUS_NOT_SUPPORTED after the argument
 * checks: there is no CPU fallback.
 */
#include "types.h"
#include "spdef.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- handle creation from COO arrays: reference spapi.h:93-127 ------------------------- */
alphasparse_status_t alphasparse_s_create_coo(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              const ALPHA_INT nnz, ALPHA_INT *row_indx,
                                              ALPHA_INT *col_indx, float *values);
alphasparse_status_t alphasparse_d_create_coo(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              const ALPHA_INT nnz, ALPHA_INT *row_indx,
                                              ALPHA_INT *col_indx, double *values);
alphasparse_status_t alphasparse_c_create_coo(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              const ALPHA_INT nnz, ALPHA_INT *row_indx,
                                              ALPHA_INT *col_indx, ALPHA_Complex8 *values);
alphasparse_status_t alphasparse_z_create_coo(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              const ALPHA_INT nnz, ALPHA_INT *row_indx,
                                              ALPHA_INT *col_indx, ALPHA_Complex16 *values);

/* ---- handle creation from 4-array CSR: reference spapi.h:140-174 ------------------------
 * Deep copy into an owned 3-array CSR (base-1 input is rebased to 0), upload to the current
 * device and one-time row-length analysis.  Device memory exhaustion returns ALLOC_FAILED
 * (the reference exits the process on host exhaustion, src/util/malloc.c:25-28). */
alphasparse_status_t alphasparse_s_create_csr(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *rows_start, ALPHA_INT *rows_end,
                                              ALPHA_INT *col_indx, float *values);
alphasparse_status_t alphasparse_d_create_csr(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *rows_start, ALPHA_INT *rows_end,
                                              ALPHA_INT *col_indx, double *values);
alphasparse_status_t alphasparse_c_create_csr(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *rows_start, ALPHA_INT *rows_end,
                                              ALPHA_INT *col_indx, ALPHA_Complex8 *values);
alphasparse_status_t alphasparse_z_create_csr(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *rows_start, ALPHA_INT *rows_end,
                                              ALPHA_INT *col_indx, ALPHA_Complex16 *values);

/* ---- destroy: reference spapi.h:288 (NULL handle is SUCCESS) ---------------------------- */
alphasparse_status_t alphasparse_destroy(alphasparse_matrix_t A);

/* ---- COO -> CSR: reference spapi.h:300-302; only a COO source and NON_TRANSPOSE or
 * TRANSPOSE are accepted, as in src/core/op_/alphasparse_convert_csr.c:100-157 ------------ */
alphasparse_status_t alphasparse_convert_csr(const alphasparse_matrix_t source,
                                             const alphasparse_operation_t operation,
                                             alphasparse_matrix_t *dest);

/* ---- export: reference spapi.h:352-386; returns borrowed pointers to the owned host copy,
 * index base reported as zero --------------------------------------------------------------- */
alphasparse_status_t alphasparse_s_export_csr(const alphasparse_matrix_t source,
                                              alphasparse_index_base_t *indexing,
                                              ALPHA_INT *rows, ALPHA_INT *cols,
                                              ALPHA_INT **rows_start, ALPHA_INT **rows_end,
                                              ALPHA_INT **col_indx, float **values);
alphasparse_status_t alphasparse_d_export_csr(const alphasparse_matrix_t source,
                                              alphasparse_index_base_t *indexing,
                                              ALPHA_INT *rows, ALPHA_INT *cols,
                                              ALPHA_INT **rows_start, ALPHA_INT **rows_end,
                                              ALPHA_INT **col_indx, double **values);

/* ---- CSC handles: reference spapi.h:186-220 (create), :388-422 (export), :17-19 (convert; COO source
 * only, as in src/core/op_/alphasparse_convert_csc.c:101-123).  The arrays of a CSC matrix are the
 * CSR arrays of its transpose: the handle keeps a CSR handle of A^T (host copy, device copy,
 * analysis) in its `inspector` slot, mv / mm run on it with the operation flipped, and export_csc
 * returns that handle's host arrays.  GENERAL descriptor only. ------------------------------------ */
alphasparse_status_t alphasparse_s_create_csc(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *cols_start, ALPHA_INT *cols_end,
                                              ALPHA_INT *row_indx, float *values);
alphasparse_status_t alphasparse_d_create_csc(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *cols_start, ALPHA_INT *cols_end,
                                              ALPHA_INT *row_indx, double *values);
alphasparse_status_t alphasparse_c_create_csc(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *cols_start, ALPHA_INT *cols_end,
                                              ALPHA_INT *row_indx, ALPHA_Complex8 *values);
alphasparse_status_t alphasparse_z_create_csc(alphasparse_matrix_t *A,
                                              const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols,
                                              ALPHA_INT *cols_start, ALPHA_INT *cols_end,
                                              ALPHA_INT *row_indx, ALPHA_Complex16 *values);
alphasparse_status_t alphasparse_s_export_csc(const alphasparse_matrix_t source,
                                              alphasparse_index_base_t *indexing,
                                              ALPHA_INT *rows, ALPHA_INT *cols,
                                              ALPHA_INT **cols_start, ALPHA_INT **cols_end,
                                              ALPHA_INT **row_indx, float **values);
alphasparse_status_t alphasparse_d_export_csc(const alphasparse_matrix_t source,
                                              alphasparse_index_base_t *indexing,
                                              ALPHA_INT *rows, ALPHA_INT *cols,
                                              ALPHA_INT **cols_start, ALPHA_INT **cols_end,
                                              ALPHA_INT **row_indx, double **values);
alphasparse_status_t alphasparse_convert_csc(const alphasparse_matrix_t source,
                                             const alphasparse_operation_t operation,
                                             alphasparse_matrix_t *dest);

/* ---- hints: reference spapi.h:615-671 (declared there, defined nowhere).  Here
 * alphasparse_optimize re-runs the analysis; the hints are accepted and ignored. ----------- */
alphasparse_status_t alphasparse_set_mv_hint(const alphasparse_matrix_t A,
                                             const alphasparse_operation_t operation,
                                             const struct alpha_matrix_descr descr,
                                             const ALPHA_INT expected_calls);
alphasparse_status_t alphasparse_optimize(alphasparse_matrix_t A);

/* ---- y = alpha * op(A) * x + beta * y: reference spapi.h:685-715 ------------------------- */
alphasparse_status_t alphasparse_s_mv(const alphasparse_operation_t operation, const float alpha,
                                      const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr, const float *x,
                                      const float beta, float *y);
alphasparse_status_t alphasparse_d_mv(const alphasparse_operation_t operation, const double alpha,
                                      const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr, const double *x,
                                      const double beta, double *y);
alphasparse_status_t alphasparse_c_mv(const alphasparse_operation_t operation,
                                      const ALPHA_Complex8 alpha, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr,
                                      const ALPHA_Complex8 *x, const ALPHA_Complex8 beta,
                                      ALPHA_Complex8 *y);
alphasparse_status_t alphasparse_z_mv(const alphasparse_operation_t operation,
                                      const ALPHA_Complex16 alpha, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr,
                                      const ALPHA_Complex16 *x, const ALPHA_Complex16 beta,
                                      ALPHA_Complex16 *y);

/* ---- Y = alpha * op(A) * X + beta * Y, X and Y dense: reference spapi.h:899-947 ---------- */
alphasparse_status_t alphasparse_s_mm(const alphasparse_operation_t operation, const float alpha,
                                      const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr,
                                      const alphasparse_layout_t layout, const float *x,
                                      const ALPHA_INT columns, const ALPHA_INT ldx,
                                      const float beta, float *y, const ALPHA_INT ldy);
alphasparse_status_t alphasparse_d_mm(const alphasparse_operation_t operation, const double alpha,
                                      const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr,
                                      const alphasparse_layout_t layout, const double *x,
                                      const ALPHA_INT columns, const ALPHA_INT ldx,
                                      const double beta, double *y, const ALPHA_INT ldy);
alphasparse_status_t alphasparse_c_mm(const alphasparse_operation_t operation,
                                      const ALPHA_Complex8 alpha, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr,
                                      const alphasparse_layout_t layout, const ALPHA_Complex8 *x,
                                      const ALPHA_INT columns, const ALPHA_INT ldx,
                                      const ALPHA_Complex8 beta, ALPHA_Complex8 *y,
                                      const ALPHA_INT ldy);
alphasparse_status_t alphasparse_z_mm(const alphasparse_operation_t operation,
                                      const ALPHA_Complex16 alpha, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr descr,
                                      const alphasparse_layout_t layout, const ALPHA_Complex16 *x,
                                      const ALPHA_INT columns, const ALPHA_INT ldx,
                                      const ALPHA_Complex16 beta, ALPHA_Complex16 *y,
                                      const ALPHA_INT ldy);

#ifdef __cplusplus
}
#endif
