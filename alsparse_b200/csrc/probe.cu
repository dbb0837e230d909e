// A device probe used by the benchmark to put the SpMV numbers in context: the rate at which the
// GPU sustains independent gathers of single elements from random addresses of a table (what a CSR
// matrix with unstructured columns asks of x).  On B200 this rate, not HBM bandwidth, bounds SpMV on
// such matrices: every gather is its own L1->L2 request and the SMs issue one per clock each.
#include "alphasparse/spapi_cuda.h"
#include "internal.h"

namespace asb {

__global__ void probe_fill_kernel(int *idx, size_t n, unsigned long long range) {
    const size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (i >= n) return;
    unsigned long long z = (i + 1) * 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    z ^= z >> 31;
    idx[i] = (int)(z % range);
}

// Shaped like the SpMV inner loop: a 16-byte coalesced load of four indices, four independent gathers.
template <typename T>
__global__ void __launch_bounds__(256) probe_gather_kernel(const int *__restrict__ idx, const T *__restrict__ table,
                                                          T *__restrict__ sink, size_t quads) {
    const size_t q = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if (q >= quads) return;
    const int4 c = __ldcs(reinterpret_cast<const int4 *>(idx) + q);
    const T s = __ldg(table + c.x) + __ldg(table + c.y) + __ldg(table + c.z) + __ldg(table + c.w);
    if (s == T(123456.5)) sink[q] = s;  // never true for a zero table; keeps the loads alive without a store stream
}

template <typename T>
static alphasparse_status_t probe(int64_t table_elems, int64_t gathers, double *per_second) {
    int *idx = nullptr;
    T *table = nullptr, *sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaStream_t st = current_stream();
    const size_t n = (size_t)gathers & ~(size_t)3, quads = n / 4;
    alphasparse_status_t status = ALPHA_SPARSE_STATUS_SUCCESS;
    cudaError_t err = device_alloc(&idx, n * sizeof(int));
    if (err == cudaSuccess) err = device_alloc(&table, (size_t)table_elems * sizeof(T));
    if (err == cudaSuccess) err = device_alloc(&sink, sizeof(T) * 4);
    if (err == cudaSuccess) err = cudaMemsetAsync(table, 0, (size_t)table_elems * sizeof(T), st);
    if (err == cudaSuccess) err = cudaEventCreate(&e0);
    if (err == cudaSuccess) err = cudaEventCreate(&e1);
    if (err == cudaSuccess) {
        probe_fill_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(idx, n, (unsigned long long)table_elems);
        const unsigned blocks = (unsigned)((quads + 255) / 256);
        float best = 1e30f;
        for (int rep = 0; rep < 4 && err == cudaSuccess; rep++) {  // first repetition warms up
            cudaEventRecord(e0, st);
            probe_gather_kernel<T><<<blocks, 256, 0, st>>>(idx, table, sink, quads);
            cudaEventRecord(e1, st);
            err = cudaEventSynchronize(e1);
            float ms = 0.f;
            if (err == cudaSuccess) err = cudaEventElapsedTime(&ms, e0, e1);
            if (rep > 0 && ms < best) best = ms;
        }
        count_launch(5);
        if (err == cudaSuccess) *per_second = (double)n / ((double)best * 1e-3);
    }
    if (err != cudaSuccess) {
        record_cuda_error(err, "gather probe");
        status = ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    }
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(idx), cudaFree(table), cudaFree(sink);
    return status;
}

}  // namespace asb

extern "C" alphasparse_status_t alphasparse_cuda_probe_gather_rate(alphasparse_datatype_t datatype, int64_t table_elems,
                                                                   int64_t gathers, double *per_second) {
    if (!per_second || table_elems <= 0 || table_elems > 0x7fffffff || gathers < 1024)
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (datatype == ALPHA_SPARSE_DATATYPE_FLOAT) return asb::probe<float>(table_elems, gathers, per_second);
    if (datatype == ALPHA_SPARSE_DATATYPE_DOUBLE) return asb::probe<double>(table_elems, gathers, per_second);
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}
