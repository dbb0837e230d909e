// The rest of the host utility surface that the reference's test programs call around the
// mv / mm path: command-line getters, timers, vector fills, the cache sweep and the operation
// counts (include/alphasparse/util.h).  Fresh implementations of the behaviour declared in the
// reference's include/alphasparse/util/{args,timing,malloc,analysis}.h; a test program written
// against those headers (for instance the flow of test/arm/mv_d_csr_arm_test.c:84-135) links
// against this library unchanged.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include "alphasparse/util.h"

namespace {

// The option names of the reference's table (src/util/args.c:9-44).  Its getters run
// getopt_long_only over it: one or two leading dashes, the value attached with '=', names may be
// shortened to any prefix that matches exactly one entry.
const char *const kOptionNames[] = {"help",   "check",  "thread-num", "transA",     "transB",     "typeA",
                                    "fillA",  "diagA",  "typeB",      "fillB",      "diagB",      "data-file",
                                    "data-fileA", "data-fileB", "layout", "layoutB", "layoutC",  "columns",
                                    "iter",   "formatA", "formatB",   "data-type"};
constexpr int kOptionCount = (int)(sizeof(kOptionNames) / sizeof(kOptionNames[0]));

// Index + 1 of the option argv[i] names (the reference's option codes are 1-based positions in the
// table), 0 when it names none; *value = text after '=' or null.
int option_code(const char *arg, const char **value) {
    *value = nullptr;
    if (!arg || arg[0] != '-') return 0;
    const char *name = arg + (arg[1] == '-' ? 2 : 1);
    if (!*name) return 0;
    const char *eq = strchr(name, '=');
    const size_t len = eq ? (size_t)(eq - name) : strlen(name);
    if (eq) *value = eq + 1;
    int hit = 0, hits = 0;
    for (int i = 0; i < kOptionCount; i++) {
        if (strlen(kOptionNames[i]) == len && !strncmp(kOptionNames[i], name, len)) return i + 1;  // exact
        if (!strncmp(kOptionNames[i], name, len)) hit = i + 1, hits++;
    }
    return hits == 1 ? hit : 0;
}

// Value of the first occurrence of option `code`, or null.
const char *first_value(int argc, const char *argv[], int code, bool *present = nullptr) {
    if (present) *present = false;
    for (int i = 1; i < argc; i++) {
        const char *v = nullptr;
        if (option_code(argv[i], &v) == code) {
            if (present) *present = true;
            return v;
        }
    }
    return nullptr;
}

const char *data_file_for(int argc, const char *argv[], int own_code) {
    // the matrix-specific name wins wherever it stands; otherwise the last plain --data-file
    const char *plain = nullptr;
    for (int i = 1; i < argc; i++) {
        const char *v = nullptr;
        const int c = option_code(argv[i], &v);
        if (c == own_code && v) return v;
        if (c == 12 && v) plain = v;
    }
    return plain ? plain : "";
}

[[noreturn]] void bad_value(const char *what, const char *arg) {
    printf("invalid %s value!!! %s\n", what, arg ? arg : "(none)");
    exit(-1);
}

bool is_any(const char *arg, const char *a, const char *b, const char *c = nullptr) {
    return arg && (!strcmp(arg, a) || !strcmp(arg, b) || (c && !strcmp(arg, c)));
}

unsigned clock_seed() { return (unsigned)time(nullptr); }

void *g_flush_buf = nullptr;  // device scratch of alpha_clear_cache, kept for the life of the process
constexpr size_t kFlushBytes = (size_t)256 << 20;

}  // namespace

extern "C" {

// ---- command line (reference: include/alphasparse/util/args.h:21-45, src/util/args.c) ---------------

void args_help(const int argc, const char *argv[]) {
    bool present = false;
    first_value(argc, argv, 1, &present);
    if (!present) return;
    printf("--help\n--check\n--thread-num=<int>\n--data-file=<file> --data-fileA=<file> --data-fileB=<file>\n"
           "--columns=<int>\n--iter=<int>\n--layout=<R|C>\n--transA=<N|T|H> --transB=<N|T|H>\n"
           "--typeA=<G|S|H|T|D|BT|BD> --fillA=<L|U> --diagA=<N|U>\n--typeB=... --fillB=... --diagB=...\n");
    exit(-1);
}
bool args_get_if_check(const int argc, const char *argv[]) {
    bool present = false;
    first_value(argc, argv, 2, &present);
    return present;
}
int args_get_thread_num(const int argc, const char *argv[]) {
    const char *v = first_value(argc, argv, 3);
    return v ? atoi(v) : 1;
}
int args_get_columns(const int argc, const char *argv[], int k) {
    const char *v = first_value(argc, argv, 18);
    return v ? atoi(v) : k;
}
int args_get_iter(const int argc, const char *argv[]) {
    const char *v = first_value(argc, argv, 19);
    return v ? atoi(v) : 1;
}
const char *args_get_data_file(const int argc, const char *argv[]) {
    const char *v = first_value(argc, argv, 12);
    return v ? v : "";
}
const char *args_get_data_fileA(const int argc, const char *argv[]) { return data_file_for(argc, argv, 13); }
const char *args_get_data_fileB(const int argc, const char *argv[]) { return data_file_for(argc, argv, 14); }

alphasparse_layout_t alphasparse_layout_parse(const char *arg) {
    if (is_any(arg, "R", "ROW")) return ALPHA_SPARSE_LAYOUT_ROW_MAJOR;
    if (is_any(arg, "C", "COL", "COLUMN")) return ALPHA_SPARSE_LAYOUT_COLUMN_MAJOR;
    bad_value("layout", arg);
}
alphasparse_operation_t alphasparse_operation_parse(const char *arg) {
    if (is_any(arg, "N", "NON_TRANSPOSE")) return ALPHA_SPARSE_OPERATION_NON_TRANSPOSE;
    if (is_any(arg, "T", "TRANSPOSE")) return ALPHA_SPARSE_OPERATION_TRANSPOSE;
    if (is_any(arg, "H", "CONJUGATE_TRANSPOSE")) return ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE;
    bad_value("operation", arg);
}
alphasparse_matrix_type_t alphasparse_matrix_type_parse(const char *arg) {
    if (is_any(arg, "G", "GENERAL")) return ALPHA_SPARSE_MATRIX_TYPE_GENERAL;
    if (is_any(arg, "S", "SYMMETRIC")) return ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC;
    if (is_any(arg, "H", "HERMITIAN")) return ALPHA_SPARSE_MATRIX_TYPE_HERMITIAN;
    if (is_any(arg, "T", "TRIANGULAR")) return ALPHA_SPARSE_MATRIX_TYPE_TRIANGULAR;
    if (is_any(arg, "D", "DIAGONAL")) return ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL;
    if (is_any(arg, "BT", "BLOCK_TRIANGULAR")) return ALPHA_SPARSE_MATRIX_TYPE_BLOCK_TRIANGULAR;
    if (is_any(arg, "BD", "BLOCK_DIAGONAL")) return ALPHA_SPARSE_MATRIX_TYPE_BLOCK_DIAGONAL;
    bad_value("type", arg);
}
alphasparse_fill_mode_t alphasparse_fill_mode_parse(const char *arg) {
    if (is_any(arg, "L", "LOWER")) return ALPHA_SPARSE_FILL_MODE_LOWER;
    if (is_any(arg, "U", "UPPER")) return ALPHA_SPARSE_FILL_MODE_UPPER;
    bad_value("fill", arg);
}
alphasparse_diag_type_t alphasparse_diag_type_parse(const char *arg) {
    if (is_any(arg, "N", "NON_UNIT")) return ALPHA_SPARSE_DIAG_NON_UNIT;
    if (is_any(arg, "U", "UNIT")) return ALPHA_SPARSE_DIAG_UNIT;
    bad_value("diag", arg);
}

alphasparse_layout_t alpha_args_get_layout_helper(const int argc, const char *argv[], const int layout_opt) {
    const char *v = first_value(argc, argv, layout_opt);
    return v ? alphasparse_layout_parse(v) : ALPHA_SPARSE_LAYOUT_ROW_MAJOR;
}
struct alpha_matrix_descr alpha_args_get_matrix_descr_helper(const int argc, const char *argv[], const int type_opt,
                                                              const int fill_opt, const int diag_opt) {
    struct alpha_matrix_descr d;
    d.type = ALPHA_SPARSE_MATRIX_TYPE_GENERAL, d.mode = ALPHA_SPARSE_FILL_MODE_LOWER, d.diag = ALPHA_SPARSE_DIAG_NON_UNIT;
    for (int i = 1; i < argc; i++) {  // every occurrence applies, the last one stands
        const char *v = nullptr;
        const int c = option_code(argv[i], &v);
        if (!v) continue;
        if (c == type_opt) d.type = alphasparse_matrix_type_parse(v);
        else if (c == fill_opt) d.mode = alphasparse_fill_mode_parse(v);
        else if (c == diag_opt) d.diag = alphasparse_diag_type_parse(v);
    }
    return d;
}
alphasparse_operation_t alpha_args_get_trans_helper(const int argc, const char *argv[], const int trans_opt) {
    const char *v = first_value(argc, argv, trans_opt);
    return v ? alphasparse_operation_parse(v) : ALPHA_SPARSE_OPERATION_NON_TRANSPOSE;
}
alphasparse_layout_t alpha_args_get_layout(const int argc, const char *argv[]) { return alpha_args_get_layout_helper(argc, argv, 15); }
alphasparse_layout_t alpha_args_get_layoutB(const int argc, const char *argv[]) { return alpha_args_get_layout_helper(argc, argv, 17); }
alphasparse_layout_t alpha_args_get_layoutC(const int argc, const char *argv[]) { return alpha_args_get_layout_helper(argc, argv, 17); }
struct alpha_matrix_descr alpha_args_get_matrix_descrA(const int argc, const char *argv[]) {
    return alpha_args_get_matrix_descr_helper(argc, argv, 6, 7, 8);
}
struct alpha_matrix_descr alpha_args_get_matrix_descrB(const int argc, const char *argv[]) {
    return alpha_args_get_matrix_descr_helper(argc, argv, 9, 10, 11);
}
alphasparse_operation_t alpha_args_get_transA(const int argc, const char *argv[]) { return alpha_args_get_trans_helper(argc, argv, 4); }
alphasparse_operation_t alpha_args_get_transB(const int argc, const char *argv[]) { return alpha_args_get_trans_helper(argc, argv, 5); }

// ---- timers (reference: include/alphasparse/util/timing.h:17-23, src/util/timer.c) -------------------

void alpha_timing_start(alpha_timer_t *timer) { timer->start = alpha_timing_wtime(); }
void alpha_timing_end(alpha_timer_t *timer) { timer->end = alpha_timing_wtime(); }
double alpha_timing_elapsed_time(const alpha_timer_t *timer) { return timer->end - timer->start; }
double alpha_timing_gflops(const alpha_timer_t *timer, int64_t operations) {
    return (double)operations * 1e-9 / alpha_timing_elapsed_time(timer);
}
void alpha_timing_elaped_time_print(const alpha_timer_t *timer, const char *name) {
    printf("%s elasped time : %lf[sec]\n", name, alpha_timing_elapsed_time(timer));
}
void alpha_timing_gflops_print(const alpha_timer_t *timer, int64_t operations, const char *name) {
    printf("%s gflops : %lf\n", name, alpha_timing_gflops(timer, operations));
}

// ---- fills (reference: include/alphasparse/util/malloc.h:27-38, src/util/malloc.c:62-108) ------------
// The random fills draw rand() / RAND_MAX after srand(seed), seed 0 meaning "seed from the clock":
// a program that fills x with a fixed seed gets the numbers it would get from the reference on the
// same C library.

void alpha_fill_s(float *arr, const float num, const size_t size) {
    for (size_t i = 0; i < size; i++) arr[i] = num;
}
void alpha_fill_d(double *arr, const double num, const size_t size) {
    for (size_t i = 0; i < size; i++) arr[i] = num;
}
void alpha_fill_random_s(float *arr, unsigned int seed, const size_t size) {
    srand(seed ? seed : clock_seed());
    for (size_t i = 0; i < size; i++) arr[i] = (float)rand() / RAND_MAX;
}
void alpha_fill_random_d(double *arr, unsigned int seed, const size_t size) {
    srand(seed ? seed : clock_seed());
    for (size_t i = 0; i < size; i++) arr[i] = (double)rand() / RAND_MAX;
}

// Reference: src/util/malloc.c:50-60 sweeps a buffer larger than the host's last-level cache so that
// the next timed call starts cold.  The operands of this backend live in device memory, so the sweep
// that matters is the GPU's: 256 MB (twice the 126 MB L2 of a B200) are overwritten on the library's
// device; the buffer is allocated on first use and kept.  The host sweep is done as well.
void alpha_clear_cache(void) {
    const size_t host_bytes = (size_t)64 << 20;
    if (unsigned char *h = static_cast<unsigned char *>(malloc(host_bytes))) {
        for (int pass = 0; pass < 2; pass++)
            for (size_t i = 0; i < host_bytes; i += 64) h[i] = (unsigned char)(h[i] + pass + 1);
        free(h);
    }
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        (void)cudaGetLastError();
        return;
    }
    if (!g_flush_buf && cudaMalloc(&g_flush_buf, kFlushBytes) != cudaSuccess) {
        (void)cudaGetLastError();
        g_flush_buf = nullptr;
        return;
    }
    static unsigned char tick = 0;
    cudaMemset(g_flush_buf, ++tick, kFlushBytes);
    cudaDeviceSynchronize();
}

// ---- operation counts (reference: include/alphasparse/util/analysis.h:6-8, src/util/analysis.c) ------

void alphasparse_nnz_counter_coo(const ALPHA_INT *row_indx, const ALPHA_INT *col_indx, const ALPHA_INT nnz,
                                 ALPHA_INT *lo_p, ALPHA_INT *diag_p, ALPHA_INT *hi_p) {
    long long lo = 0, diag = 0, hi = 0;
#pragma omp parallel for reduction(+ : lo, diag, hi) if (nnz > (1 << 16))
    for (ALPHA_INT i = 0; i < nnz; i++) {
        if (row_indx[i] > col_indx[i]) lo++;
        else if (row_indx[i] < col_indx[i]) hi++;
        else diag++;
    }
    *lo_p = (ALPHA_INT)lo, *diag_p = (ALPHA_INT)diag, *hi_p = (ALPHA_INT)hi;
}

// Stored elements a product under `descr` touches (src/util/analysis.c:58-128); -1 for a descriptor
// outside the reference's cases (it asserts there).
static long long touched_elements(long long rows, long long lo, long long diag, long long hi,
                                  alphasparse_operation_t op, struct alpha_matrix_descr d) {
    const long long on_diag = d.diag == ALPHA_SPARSE_DIAG_UNIT ? rows : diag;
    const bool lower = d.mode == ALPHA_SPARSE_FILL_MODE_LOWER;
    switch (d.type) {
        case ALPHA_SPARSE_MATRIX_TYPE_GENERAL: return lo + diag + hi;
        case ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC:
        case ALPHA_SPARSE_MATRIX_TYPE_HERMITIAN: return (lower ? lo : hi) + on_diag;
        case ALPHA_SPARSE_MATRIX_TYPE_TRIANGULAR:
            return ((op == ALPHA_SPARSE_OPERATION_NON_TRANSPOSE) == lower ? lo : hi) + on_diag;
        case ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL: return on_diag;
        default: return -1;
    }
}

ALPHA_INT64 alphasparse_operations_mm(const ALPHA_INT rows, const ALPHA_INT cols, const ALPHA_INT lo, const ALPHA_INT diag,
                                      const ALPHA_INT hi, const alphasparse_operation_t operation,
                                      const struct alpha_matrix_descr descr, const ALPHA_INT columns,
                                      const alphasparse_datatype_t datatype) {
    (void)cols;
    const bool cplx = datatype == ALPHA_SPARSE_DATATYPE_FLOAT_COMPLEX || datatype == ALPHA_SPARSE_DATATYPE_DOUBLE_COMPLEX;
    const long long mul = cplx ? 7 : 1, add = cplx ? 2 : 1, madd = cplx ? 9 : 2;
    const long long nnz = touched_elements(rows, lo, diag, hi, operation, descr);
    if (nnz < 0) return -1;
    return (ALPHA_INT64)((nnz * madd + (long long)rows * (2 * mul + add)) * columns);
}
ALPHA_INT64 alphasparse_operations_mv(const ALPHA_INT rows, const ALPHA_INT cols, const ALPHA_INT lo, const ALPHA_INT diag,
                                      const ALPHA_INT hi, const alphasparse_operation_t operation,
                                      const struct alpha_matrix_descr descr, const alphasparse_datatype_t datatype) {
    return alphasparse_operations_mm(rows, cols, lo, diag, hi, operation, descr, 1, datatype);
}

}  // extern "C"
