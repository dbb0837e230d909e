// Benchmark-side probe (not part of the library): the rate at which the GPU sustains independent
// gathers of single elements from random addresses of a table, which is what a CSR matrix with
// unstructured columns asks of x.  On B200 this rate, not HBM bandwidth, bounds an SpMV that takes
// every x element from L2: each gather is its own L1 -> L2 request.  bench.py loads the shared
// object built from this file (libbench_gather_probe.so, beside it) and reports the rate next to the
// kernel's time.
//
//   int bench_gather_rate(int elem_bytes, long long table_elems, long long gathers, void *stream,
//                         double *per_second)         returns 0 on success, a cudaError_t otherwise
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

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
int probe(long long table_elems, long long gathers, cudaStream_t st, double *per_second) {
    int *idx = nullptr;
    T *table = nullptr, *sink = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    const size_t n = (size_t)gathers & ~(size_t)3, quads = n / 4;
    cudaError_t err = cudaMalloc(&idx, n * sizeof(int));
    if (err == cudaSuccess) err = cudaMalloc(&table, (size_t)table_elems * sizeof(T));
    if (err == cudaSuccess) err = cudaMalloc(&sink, sizeof(T) * 4);
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
        if (err == cudaSuccess) *per_second = (double)n / ((double)best * 1e-3);
    }
    if (err != cudaSuccess) (void)cudaGetLastError();
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    cudaFree(idx), cudaFree(table), cudaFree(sink);
    return (int)err;
}

}  // namespace

extern "C" int bench_gather_rate(int elem_bytes, long long table_elems, long long gathers, void *stream,
                                 double *per_second) {
    if (!per_second || table_elems <= 0 || table_elems > 0x7fffffff || gathers < 1024) return (int)cudaErrorInvalidValue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (elem_bytes == 4) return probe<float>(table_elems, gathers, st, per_second);
    if (elem_bytes == 8) return probe<double>(table_elems, gathers, st, per_second);
    return (int)cudaErrorInvalidValue;
}
