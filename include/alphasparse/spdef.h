#pragma once
/*
 * Enumerations, matrix handle and matrix descriptor of the C ABI.
 * Every constant and field order below matches include/alphasparse/spdef.h of the reference
 * (status :8-19, operation :22-27, matrix type :32-41, index base :46-50, fill :55-59,
 * diag :64-68, layout :73-77, format :120-133, datatype :137-143, handle :162-172,
 * descriptor :178-183), so objects built against either header are interchangeable.
 */

typedef enum {
    ALPHA_SPARSE_STATUS_SUCCESS = 0,
    ALPHA_SPARSE_STATUS_NOT_INITIALIZED = 1,
    ALPHA_SPARSE_STATUS_ALLOC_FAILED = 2,
    ALPHA_SPARSE_STATUS_INVALID_VALUE = 3,
    ALPHA_SPARSE_STATUS_EXECUTION_FAILED = 4,
    ALPHA_SPARSE_STATUS_INTERNAL_ERROR = 5,
    ALPHA_SPARSE_STATUS_NOT_SUPPORTED = 6,
    ALPHA_SPARSE_STATUS_INVALID_POINTER = 7,
    ALPHA_SPARSE_STATUS_INVALID_HANDLE = 8
} alphasparse_status_t;

typedef enum {
    ALPHA_SPARSE_OPERATION_NON_TRANSPOSE = 0,
    ALPHA_SPARSE_OPERATION_TRANSPOSE = 1,
    ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE = 2
} alphasparse_operation_t;

typedef enum {
    ALPHA_SPARSE_MATRIX_TYPE_GENERAL = 0,
    ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC = 1,
    ALPHA_SPARSE_MATRIX_TYPE_HERMITIAN = 2,
    ALPHA_SPARSE_MATRIX_TYPE_TRIANGULAR = 3,
    ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL = 4,
    ALPHA_SPARSE_MATRIX_TYPE_BLOCK_TRIANGULAR = 5,
    ALPHA_SPARSE_MATRIX_TYPE_BLOCK_DIAGONAL = 6
} alphasparse_matrix_type_t;

typedef enum {
    ALPHA_SPARSE_INDEX_BASE_ZERO = 0,
    ALPHA_SPARSE_INDEX_BASE_ONE = 1
} alphasparse_index_base_t;

typedef enum {
    ALPHA_SPARSE_FILL_MODE_LOWER = 0,
    ALPHA_SPARSE_FILL_MODE_UPPER = 1
} alphasparse_fill_mode_t;

typedef enum {
    ALPHA_SPARSE_DIAG_NON_UNIT = 0,
    ALPHA_SPARSE_DIAG_UNIT = 1
} alphasparse_diag_type_t;

typedef enum {
    ALPHA_SPARSE_LAYOUT_ROW_MAJOR = 0,
    ALPHA_SPARSE_LAYOUT_COLUMN_MAJOR = 1
} alphasparse_layout_t;

typedef enum {
    ALPHA_SPARSE_FORMAT_COO = 0,
    ALPHA_SPARSE_FORMAT_CSR = 1,
    ALPHA_SPARSE_FORMAT_CSC = 2,
    ALPHA_SPARSE_FORMAT_BSR = 3,
    ALPHA_SPARSE_FORMAT_SKY = 4,
    ALPHA_SPARSE_FORMAT_DIA = 5,
    ALPHA_SPARSE_FORMAT_ELL = 6,
    ALPHA_SPARSE_FORMAT_GEBSR = 7,
    ALPHA_SPARSE_FORMAT_HYB = 8,
    ALPHA_SPARSE_FORMAT_COO_AOS = 9,
    ALPHA_SPARSE_FORMAT_CSR5 = 10
} alphasparse_format_t;

typedef enum {
    ALPHA_SPARSE_DATATYPE_FLOAT = 0,
    ALPHA_SPARSE_DATATYPE_DOUBLE = 1,
    ALPHA_SPARSE_DATATYPE_FLOAT_COMPLEX = 2,
    ALPHA_SPARSE_DATATYPE_DOUBLE_COMPLEX = 3
} alphasparse_datatype_t;

typedef void *alpha_internal_spmat;

/*
 * The handle.  `mat` points at an spmat_csr_?_t or spmat_coo_?_t (alphasparse/spmat.h).
 * `inspector` of a COO handle holds the CSR copy that mv / mm build on first use (NULL until
 * then); of a CSC handle, the CSR handle of the transposed matrix made at creation; it is always
 * NULL on a CSR handle.  `dcu_info` is the slot the reference reserves for
 * per-matrix device analysis; this backend stores its own device context there (device CSR
 * arrays, row statistics, load-balancing tables, staging buffers).  Both are NULL-initialised
 * by every create call; callers only ever hold the pointer.
 */
typedef struct {
    alpha_internal_spmat mat;
    alphasparse_format_t format;
    alphasparse_datatype_t datatype;
    void *inspector;
    void *dcu_info;
} alphasparse_matrix;

typedef alphasparse_matrix *alphasparse_matrix_t;

/* passed BY VALUE to mv / mm, exactly as in the reference */
struct alpha_matrix_descr {
    alphasparse_matrix_type_t type;
    alphasparse_fill_mode_t mode;
    alphasparse_diag_type_t diag;
};
