// Host helpers exported alongside the sparse entry points (include/alphasparse/util.h).
// Fresh implementations of the small utility surface every reference test program uses.
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#include <atomic>
#include <thread>

#include "alphasparse/util.h"

namespace {
std::atomic<int> g_threads{0};
constexpr size_t kPinThreshold = 1 << 16;  // smaller blocks are not worth a page-locking call
}  // namespace

// Coordinate-text matrix reader with the reference's behaviour (src/util/io.c:39-114 single,
// :116-191 double): comment lines start with '%'; the word "symmetric" on the FIRST line makes every
// off-diagonal entry appear twice, the mirrored copy directly after the original; the first
// non-comment line holds rows, columns and the number of entries; entries are one-based "row col
// [value]", a missing value reads as 1.  Output arrays come from alpha_malloc (release with
// alpha_free) and hold zero-based indices.  Unlike the reference, a file that cannot be opened or
// that ends early yields *nnz_p = -1 and null arrays instead of undefined behaviour.
template <typename T>
static void read_coo(const char *file, ALPHA_INT *m_p, ALPHA_INT *n_p, ALPHA_INT *nnz_p, ALPHA_INT **row_index,
                     ALPHA_INT **col_index, T **values) {
    *nnz_p = -1, *row_index = nullptr, *col_index = nullptr, *values = nullptr;
    FILE *fp = fopen(file, "r");
    if (!fp) return;
    char line[1024];
    bool symmetric = false, first = true, have_sizes = false;
    while (fgets(line, sizeof(line), fp)) {
        if (first && line[0] == '%') {
            for (char *tok = strtok(line, " \n"); tok; tok = strtok(nullptr, " \n"))
                if (!strcmp(tok, "symmetric")) {
                    symmetric = true;
                    break;
                }
            line[0] = '%';
        }
        first = false;
        if (line[0] != '%') {
            have_sizes = true;
            break;
        }
    }
    long long m = 0, n = 0, entries = 0;
    if (!have_sizes || sscanf(line, "%lld %lld %lld", &m, &n, &entries) != 3 || entries < 0) {
        fclose(fp);
        return;
    }
    const size_t cap = (size_t)entries * (symmetric ? 2 : 1);
    ALPHA_INT *ri = static_cast<ALPHA_INT *>(alpha_malloc(sizeof(ALPHA_INT) * (cap ? cap : 1)));
    ALPHA_INT *ci = static_cast<ALPHA_INT *>(alpha_malloc(sizeof(ALPHA_INT) * (cap ? cap : 1)));
    T *v = static_cast<T *>(alpha_malloc(sizeof(T) * (cap ? cap : 1)));
    size_t k = 0;
    bool ok = ri && ci && v;
    for (long long e = 0; ok && e < entries; e++) {
        if (!fgets(line, sizeof(line), fp)) {
            ok = false;
            break;
        }
        char *end = line;
        const long long r = strtoll(end, &end, 10), c = strtoll(end, &end, 10);
        while (*end == ' ' || *end == '\t') end++;
        const T a = (*end && *end != '\n' && *end != '\r') ? (T)strtod(end, nullptr) : T(1);
        ri[k] = (ALPHA_INT)(r - 1), ci[k] = (ALPHA_INT)(c - 1), v[k] = a, k++;
        if (symmetric && r != c) ri[k] = (ALPHA_INT)(c - 1), ci[k] = (ALPHA_INT)(r - 1), v[k] = a, k++;
    }
    fclose(fp);
    if (!ok) {
        alpha_free(ri), alpha_free(ci), alpha_free(v);
        return;
    }
    *m_p = (ALPHA_INT)m, *n_p = (ALPHA_INT)n, *nnz_p = (ALPHA_INT)k;
    *row_index = ri, *col_index = ci, *values = v;
}

extern "C" {

// Reference: src/util/malloc.c:19-48.  Large blocks are page-locked so that vectors a caller
// allocates this way cross PCIe by DMA at full rate; if page-locking is refused (no device,
// limit reached) ordinary aligned memory is returned.
void *alpha_memalign(size_t bytes, size_t alignment) {
    if (bytes >= kPinThreshold && alignment <= 4096) {
        void *p = nullptr;
        if (cudaHostAlloc(&p, bytes, cudaHostAllocPortable) == cudaSuccess) return p;
        (void)cudaGetLastError();
    }
    void *p = nullptr;
    if (alignment < sizeof(void *)) alignment = sizeof(void *);
    if (posix_memalign(&p, alignment, bytes ? bytes : alignment) != 0) return nullptr;
    return p;
}

void *alpha_malloc(size_t bytes) { return alpha_memalign(bytes, 64); }

// Unlike the reference's alpha_free (which only ever frees NULL), this releases the block.
void alpha_free(void *point) {
    if (!point) return;
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, point) == cudaSuccess && at.type == cudaMemoryTypeHost) {
        cudaFreeHost(point);
        return;
    }
    (void)cudaGetLastError();
    free(point);
}

// Reference: src/util/thread.c:13-38.  Only the host-side loops of handle creation use it.
int alpha_get_core_num(void) {
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}
void alpha_set_thread_num(const int num) { g_threads.store(num > 0 ? num : 0); }
int alpha_get_thread_num(void) {
    int t = g_threads.load();
    return t == 0 ? alpha_get_core_num() : t;
}

// Reference: src/util/timer.c:14-24 (wall clock in seconds).
double alpha_timing_wtime(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

void alpha_read_coo(const char *file, ALPHA_INT *m_p, ALPHA_INT *n_p, ALPHA_INT *nnz_p, ALPHA_INT **row_index,
                    ALPHA_INT **col_index, float **values) {
    read_coo<float>(file, m_p, n_p, nnz_p, row_index, col_index, values);
}
void alpha_read_coo_d(const char *file, ALPHA_INT *m_p, ALPHA_INT *n_p, ALPHA_INT *nnz_p, ALPHA_INT **row_index,
                      ALPHA_INT **col_index, double **values) {
    read_coo<double>(file, m_p, n_p, nnz_p, row_index, col_index, values);
}

// Reference: src/util/partition.c:46-61.
int lower_bound_int(const ALPHA_INT *t, ALPHA_INT l, ALPHA_INT r, ALPHA_INT value) {
    while (l < r) {
        const ALPHA_INT m = (l + r) / 2;
        if (t[m] < value) l = m + 1;
        else r = m;
    }
    return l;
}

// Reference: src/util/partition.c:79-92; see include/alphasparse/util.h for the quirks kept.
void balanced_partition_row_by_nnz(const ALPHA_INT *acc_sum_arr, ALPHA_INT rows, ALPHA_INT num_threads,
                                   ALPHA_INT *partition) {
    const ALPHA_INT nnz = acc_sum_arr[rows - 1];
    const ALPHA_INT ave = nnz / num_threads;
    partition[0] = 0;
    for (ALPHA_INT i = 1; i < num_threads; i++)
        partition[i] = lower_bound_int(acc_sum_arr, 0, rows - 1, ave * i);
    partition[num_threads] = rows;
}

}  // extern "C"
