#pragma once
/*
 * Host helpers that the reference's umbrella header also declares and that every reference
 * test program calls (include/alphasparse/util/malloc.h:13-23, util/thread.h:10-16,
 * util/partition.h:20-23, util/timing.h:15).  Fresh implementations; two deliberate
 * differences: alpha_memalign returns page-locked memory when a CUDA device is present, so
 * vectors allocated the reference way move over PCIe at full speed, and alpha_free really
 * frees (the reference's only frees NULL, src/util/malloc.c:45-48).
 */
#include <stdbool.h>
#include <stdio.h>
#include <stdlib.h>

#include "types.h"
#include "spdef.h"

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

/* Wall-clock timer of the reference's test programs: include/alphasparse/util/timing.h:9-23. */
typedef struct {
    double start;
    double end;
} alpha_timer_t;
void alpha_timing_start(alpha_timer_t *timer);
void alpha_timing_end(alpha_timer_t *timer);
double alpha_timing_elapsed_time(const alpha_timer_t *timer);
double alpha_timing_gflops(const alpha_timer_t *timer, int64_t operations);
void alpha_timing_elaped_time_print(const alpha_timer_t *timer, const char *name);
void alpha_timing_gflops_print(const alpha_timer_t *timer, int64_t operations, const char *name);

/* Vector fills: include/alphasparse/util/malloc.h:27-38.  The random ones draw rand() / RAND_MAX after
 * srand(seed); seed 0 seeds from the clock. */
void alpha_fill_s(float *arr, const float num, const size_t size);
void alpha_fill_d(double *arr, const double num, const size_t size);
void alpha_fill_random_s(float *arr, unsigned int seed, const size_t size);
void alpha_fill_random_d(double *arr, unsigned int seed, const size_t size);

/* include/alphasparse/util/malloc.h:23: makes the next call start from cold caches.  Here the cache that
 * holds the operands is the GPU's L2: a 256 MB device buffer (allocated on first use, kept) is overwritten
 * on the current device and the call waits for it; a host buffer is swept as well. */
void alpha_clear_cache(void);

/* Command-line getters of the reference's test programs (include/alphasparse/util/args.h:21-45).  Options
 * are written --name=value (one dash works too; a name may be cut to an unambiguous prefix):
 * --check --thread-num=N --iter=N --columns=N --data-file=F --data-fileA=F --data-fileB=F --layout=R|C
 * --transA=N|T|H --typeA=G|S|H|T|D|BT|BD --fillA=L|U --diagA=N|U (and the B twins).  An unknown value
 * prints a message and exits, as in the reference. */
alphasparse_layout_t alphasparse_layout_parse(const char *arg);
alphasparse_operation_t alphasparse_operation_parse(const char *arg);
alphasparse_matrix_type_t alphasparse_matrix_type_parse(const char *arg);
alphasparse_fill_mode_t alphasparse_fill_mode_parse(const char *arg);
alphasparse_diag_type_t alphasparse_diag_type_parse(const char *arg);
void args_help(const int argc, const char *argv[]);
bool args_get_if_check(const int argc, const char *argv[]);
int args_get_thread_num(const int argc, const char *argv[]);
int args_get_columns(const int argc, const char *argv[], int k);
int args_get_iter(const int argc, const char *argv[]);
const char *args_get_data_file(const int argc, const char *argv[]);
const char *args_get_data_fileA(const int argc, const char *argv[]);
const char *args_get_data_fileB(const int argc, const char *argv[]);
alphasparse_layout_t alpha_args_get_layout_helper(const int argc, const char *argv[], const int layout_opt);
struct alpha_matrix_descr alpha_args_get_matrix_descr_helper(const int argc, const char *argv[], const int type_opt,
                                                              const int fill_opt, const int diag_opt);
alphasparse_operation_t alpha_args_get_trans_helper(const int argc, const char *argv[], const int trans_opt);
alphasparse_layout_t alpha_args_get_layout(const int argc, const char *argv[]);
alphasparse_layout_t alpha_args_get_layoutB(const int argc, const char *argv[]);
alphasparse_layout_t alpha_args_get_layoutC(const int argc, const char *argv[]);
struct alpha_matrix_descr alpha_args_get_matrix_descrA(const int argc, const char *argv[]);
struct alpha_matrix_descr alpha_args_get_matrix_descrB(const int argc, const char *argv[]);
alphasparse_operation_t alpha_args_get_transA(const int argc, const char *argv[]);
alphasparse_operation_t alpha_args_get_transB(const int argc, const char *argv[]);

/* Operation counts the reference's test programs print (include/alphasparse/util/analysis.h:6-8,
 * src/util/analysis.c:8-156): entries below / on / above the diagonal of a coordinate list, and
 * (touched elements * 2 + rows * 3) * columns for real types (9 and 16 for complex). */
void alphasparse_nnz_counter_coo(const ALPHA_INT *row_indx, const ALPHA_INT *col_indx, const ALPHA_INT nnz,
                                 ALPHA_INT *lo_p, ALPHA_INT *diag_p, ALPHA_INT *hi_p);
ALPHA_INT64 alphasparse_operations_mm(const ALPHA_INT rows, const ALPHA_INT cols, const ALPHA_INT lo, const ALPHA_INT diag,
                                      const ALPHA_INT hi, const alphasparse_operation_t operation,
                                      const struct alpha_matrix_descr descr, const ALPHA_INT columns,
                                      const alphasparse_datatype_t datatype);
ALPHA_INT64 alphasparse_operations_mv(const ALPHA_INT rows, const ALPHA_INT cols, const ALPHA_INT lo, const ALPHA_INT diag,
                                      const ALPHA_INT hi, const alphasparse_operation_t operation,
                                      const struct alpha_matrix_descr descr, const alphasparse_datatype_t datatype);

/* The reference's status check for test programs (include/alphasparse/util/error.h:9-48): prints the
 * message and the status name and exits when the call did not succeed. */
#define alpha_call_exit(func, message)                                                          \
    do {                                                                                        \
        alphasparse_status_t alpha_call_status_ = (func);                                       \
        if (alpha_call_status_ != ALPHA_SPARSE_STATUS_SUCCESS) {                                \
            static const char *const alpha_call_names_[] = {                                    \
                "success",        "not initialized", "alloc failed",    "invalid value", "execution failed", \
                "internal error", "not supported",   "invalid pointer", "invalid handle"};      \
            printf("%s\nstatus : %s!!!\n", message,                                             \
                   (unsigned)alpha_call_status_ < 9u ? alpha_call_names_[alpha_call_status_] : "status invalid"); \
            fflush(0);                                                                          \
            exit(-1);                                                                           \
        }                                                                                       \
    } while (0);

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
