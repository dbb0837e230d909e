/*
 * A test program in the style of the reference's own (the flow of test/arm/mv_d_csr_arm_test.c:84-135 of the
 * reference, written fresh): command-line getters -> alpha_read_coo_d -> alphasparse_d_create_coo ->
 * alphasparse_convert_csr -> alpha_fill_random_d -> timed alphasparse_d_mv -> optional dump of y.
 * It includes only <alphasparse.h>, so it compiles against the reference's include/ directory as well as
 * against this repository's, and links against libalphasparse_b200.so in both cases.
 *
 *   mv_d_csr_main --data-file=m.mtx [--iter=3] [--transA=N|T] [--typeA=G ...] [--thread-num=4] [out.bin]
 */
#include <alphasparse.h>
#include <stdio.h>
#include <string.h>

int main(int argc, const char *argv[]) {
    args_help(argc, argv);
    const char *file = args_get_data_file(argc, argv);
    const int threads = args_get_thread_num(argc, argv);
    const int iter = args_get_iter(argc, argv);
    const alphasparse_operation_t transA = alpha_args_get_transA(argc, argv);
    const struct alpha_matrix_descr descr = alpha_args_get_matrix_descrA(argc, argv);
    alpha_set_thread_num(threads);

    ALPHA_INT m, k, nnz, *row_index, *col_index;
    double *values;
    alpha_read_coo_d(file, &m, &k, &nnz, &row_index, &col_index, &values);
    if (nnz < 0) {
        printf("cannot read %s\n", file);
        return 2;
    }
    ALPHA_INT lo, diag, hi;
    alphasparse_nnz_counter_coo(row_index, col_index, nnz, &lo, &diag, &hi);
    const ALPHA_INT64 ops = alphasparse_operations_mv(m, k, lo, diag, hi, transA, descr, ALPHA_SPARSE_DATATYPE_DOUBLE);

    const ALPHA_INT sizex = transA == ALPHA_SPARSE_OPERATION_NON_TRANSPOSE ? k : m;
    const ALPHA_INT sizey = transA == ALPHA_SPARSE_OPERATION_NON_TRANSPOSE ? m : k;
    double *x = (double *)alpha_malloc(sizeof(double) * (size_t)sizex);
    double *y = (double *)alpha_malloc(sizeof(double) * (size_t)sizey);
    alpha_fill_random_d(x, 1, (size_t)sizex);
    alpha_fill_random_d(y, 2, (size_t)sizey);

    alphasparse_matrix_t cooA, csrA;
    alpha_call_exit(alphasparse_d_create_coo(&cooA, ALPHA_SPARSE_INDEX_BASE_ZERO, m, k, nnz, row_index, col_index, values),
                    "alphasparse_d_create_coo");
    alpha_call_exit(alphasparse_convert_csr(cooA, ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, &csrA), "alphasparse_convert_csr");

    const double alpha = 2., beta = 0.5;
    alpha_timer_t timer;
    double total = 0.;
    for (int i = 0; i < iter; i++) {
        alpha_clear_cache();
        alpha_timing_start(&timer);
        alpha_call_exit(alphasparse_d_mv(transA, alpha, csrA, descr, x, beta, y), "alphasparse_d_mv");
        alpha_timing_end(&timer);
        total += alpha_timing_elapsed_time(&timer);
    }
    printf("rows %d cols %d nnz %d lo %d diag %d hi %d ops %lld\n", (int)m, (int)k, (int)nnz, (int)lo, (int)diag, (int)hi,
           (long long)ops);
    printf("alphasparse_d_mv time : %lf[sec]\n", total / iter);
    alpha_timing_gflops_print(&timer, ops, "alphasparse_d_mv");

    const char *out = argc > 1 && argv[argc - 1][0] != '-' ? argv[argc - 1] : NULL;
    if (out) {
        FILE *fp = fopen(out, "wb");
        if (!fp || fwrite(y, sizeof(double), (size_t)sizey, fp) != (size_t)sizey) return 3;
        fclose(fp);
    }
    alphasparse_destroy(cooA);
    alphasparse_destroy(csrA);
    alpha_free(x);
    alpha_free(y);
    alpha_free(row_index);
    alpha_free(col_index);
    alpha_free(values);
    return 0;
}
