#pragma once
/*
 * Host helpers that the reference's umbrella header also declares and that every reference
 * test program calls (include/alphasparse/util/malloc.h:13-23, util/thread.h:10-16,
 * util/partition.h:20-23, util/timing.h:15).  Fresh implementations; two deliberate
 * differences: alpha_memalign returns page-locked memory when a CUDA device is present, so
 * vectors allocated the reference way move over PCIe at full speed, and alpha_free really
 * frees (the reference's only frees NULL, src/util/malloc.c:45-48).
 */
#include "types.h"

#ifdef __cplusplus
extern "C" {
#endif

void *alpha_malloc(size_t bytes);
void *alpha_memalign(size_t bytes, size_t alignment);
void alpha_free(void *point);

int alpha_get_core_num(void);
void alpha_set_thread_num(const int num);
int alpha_get_thread_num(void);

double alpha_timing_wtime(void);

/* Coordinate-text ("%%MatrixMarket ... coordinate"-like) reader: reference include/alphasparse/util/io.h:19-20,
 * src/util/io.c:39-191.  Zero-based output in arrays from alpha_malloc; a "symmetric" first line mirrors
 * off-diagonal entries; a missing value reads as 1.  *nnz_p = -1 on an unreadable or truncated file. */
void alpha_read_coo(const char *file, ALPHA_INT *m_p, ALPHA_INT *n_p, ALPHA_INT *nnz_p, ALPHA_INT **row_index,
                    ALPHA_INT **col_index, float **values);
void alpha_read_coo_d(const char *file, ALPHA_INT *m_p, ALPHA_INT *n_p, ALPHA_INT *nnz_p, ALPHA_INT **row_index,
                      ALPHA_INT **col_index, double **values);

/* first index in [l, r) whose element is >= value: reference src/util/partition.c:46-61 */
int lower_bound_int(const ALPHA_INT *t, ALPHA_INT l, ALPHA_INT r, ALPHA_INT value);

/* nnz-balanced contiguous row split.  acc_sum_arr is rows_end (inclusive prefix sums),
 * partition has num_threads + 1 entries.  Bit-exact with reference
 * src/util/partition.c:79-92, including its quirks (integer average, search range
 * [0, rows-1), the boundary-crossing row goes to the following part, parts may be empty).
 * The multi-GPU row split uses this with num_threads = number of GPUs. */
void balanced_partition_row_by_nnz(const ALPHA_INT *acc_sum_arr, ALPHA_INT rows,
                                   ALPHA_INT num_threads, ALPHA_INT *partition);

#ifdef __cplusplus
}
#endif
