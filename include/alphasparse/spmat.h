#pragma once
/*
 * Host-side matrix records that alphasparse_matrix.mat points at.
 * Field order and types follow include/alphasparse/spmat.h of the reference (COO :64-83,
 * CSR :174-188 single, :203-216 double, CSC :288-297 single, :311-320 double).  The CSR record already carries three device
 * slots in the reference; this backend fills them with the sm_100a device copy.
 */
#include "types.h"

#define ALPHA_DECLARE_SPMAT(T, sfx)                                                         \
    typedef struct {                                                                        \
        T *values;                                                                          \
        ALPHA_INT *rows_start; /* rows+1 offsets; rows_end == rows_start + 1 */             \
        ALPHA_INT *rows_end;                                                                \
        ALPHA_INT *col_indx;                                                                \
        ALPHA_INT rows;                                                                     \
        ALPHA_INT cols;                                                                     \
        bool ordered;                                                                       \
        T *d_values;           /* device copy, 16-byte padded */                            \
        ALPHA_INT *d_row_ptr;  /* device copy of the rows+1 offsets */                      \
        ALPHA_INT *d_col_indx;                                                              \
    } spmat_csr_##sfx##_t;                                                                  \
    typedef struct {                                                                        \
        T *values;                                                                          \
        ALPHA_INT *row_indx;                                                                \
        ALPHA_INT *col_indx;                                                                \
        ALPHA_INT rows;                                                                     \
        ALPHA_INT cols;                                                                     \
        ALPHA_INT nnz;                                                                      \
        bool ordered;                                                                       \
        ALPHA_INT *d_rows_indx; /* unused: COO handles stay on the host */                  \
        ALPHA_INT *d_cols_indx;                                                             \
        T *d_values;                                                                        \
    } spmat_coo_##sfx##_t;                                                                  \
    typedef struct {                                                                        \
        T *values;                                                                          \
        ALPHA_INT *cols_start; /* cols+1 offsets; cols_end == cols_start + 1 */             \
        ALPHA_INT *cols_end;                                                                \
        ALPHA_INT *row_indx;                                                                \
        ALPHA_INT rows;                                                                     \
        ALPHA_INT cols;                                                                     \
        bool ordered;                                                                       \
    } spmat_csc_##sfx##_t;

ALPHA_DECLARE_SPMAT(float, s)
ALPHA_DECLARE_SPMAT(double, d)
