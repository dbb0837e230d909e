// Host helpers exported alongside the sparse entry points (include/alphasparse/util.h).
// Fresh implementations of the small utility surface every reference test program uses.
#include <cuda_runtime.h>
#include <stdlib.h>
#include <time.h>

#include <atomic>
#include <thread>

#include "alphasparse/util.h"

namespace {
std::atomic<int> g_threads{0};
constexpr size_t kPinThreshold = 1 << 16;  // smaller blocks are not worth a page-locking call
}  // namespace

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
