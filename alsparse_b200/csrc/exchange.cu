// Iterated SpMV across the GPUs of one box: x_{t+1} = alpha * A * x_t (+ beta * y), with A split into
// row blocks (one per GPU, one process per GPU) and x replicated.  The reference has no multi-device
// path; its OpenMP kernel splits rows the same way across threads
// (src/kernel/x86_64/level2/mv/gemv/gemv_x_csr.c:184-208 of the reference) and shares x in host memory.
//
// Here every GPU keeps two full-length x buffers.  The SpMV kernels of alphasparse_?_mv_exchange write
// each finished y row into their own y AND into the *next* x buffer of every GPU, through pointers
// that map the peers' buffers (CUDA IPC; plain stores that travel over NVLink): the allgather is part
// of the product kernel.  A small kernel then tells every peer "my rows of step t are in your buffer"
// (one 64-bit counter per sender, release store at system scope) and waits, with a bounded number of
// polls, until all peers have said the same; after it the buffers swap roles.  No TMA and no multicast
// is involved anywhere; remote memory is only ever written, and read locally afterwards.
#include <string.h>

#include "alphasparse/spapi.h"
#include "internal.h"

namespace asb {

constexpr size_t kIpcBlob = 3 * sizeof(cudaIpcMemHandle_t);  // x buffer 0, x buffer 1, counters

struct Exchange {
    uint64_t magic = 0x4153425845434847ull;
    int device = 0, datatype = 0, rank = 0, world = 1;
    int part[kMaxPeers + 1] = {};
    int64_t total_rows = 0;
    size_t tsz = 4;
    void *xbuf[2] = {nullptr, nullptr};        // local, total_rows elements each
    unsigned long long *counters = nullptr;    // local, one per sender: last step whose rows have arrived
    void *peer_xbuf[2][kMaxPeers] = {};        // peer-mapped (own entries point at the local buffers)
    unsigned long long *peer_counters[kMaxPeers] = {};
    bool opened[kMaxPeers] = {};
    int *d_status = nullptr;                   // 0 fine, 3 = a peer did not arrive within the poll limit
    unsigned long long step = 0;
    int cur = 0;                               // index of the buffer holding the current x
    bool connected = false;
    int mode = 0;                              // alphasparse_cuda_exchange_set_mode
};

// One thread per peer: publish our arrival for `step`, then wait for theirs.
__global__ void exchange_arrive_wait_kernel(unsigned long long step, int rank, int world,
                                            unsigned long long *const *peer_counters,
                                            volatile unsigned long long *my_counters, int *status,
                                            long long max_polls, const int *matrix_status) {
    const int p = threadIdx.x;
    // an error word left by the product's own kernels (a bounded wait that ran out) becomes the exchange's
    if (p == 0 && matrix_status && *matrix_status != 0) atomicCAS(status, 0, *matrix_status);
    if (p >= world) return;
    __threadfence_system();  // everything this GPU wrote before (same stream) is ordered before the flag
    unsigned long long *dst = peer_counters[p] + rank;
    asm volatile("st.release.sys.global.u64 [%0], %1;" :: "l"(dst), "l"(step) : "memory");
    const volatile unsigned long long *src = my_counters + p;
    long long polls = 0;
    for (;;) {
        unsigned long long seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(src) : "memory");
        if (seen >= step) break;
        if (++polls > max_polls) {  // give up: report, leave the context usable
            atomicExch(status, 3);
            break;
        }
        __nanosleep(200);
    }
}

// The waiting half alone, on a counter nobody advances: what a rank sees when a peer never arrives.
__global__ void exchange_wait_only_kernel(volatile unsigned long long *counter, unsigned long long want, int *status,
                                          long long max_polls) {
    long long polls = 0;
    for (;;) {
        unsigned long long seen;
        asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(counter) : "memory");
        if (seen >= want) break;
        if (++polls > max_polls) {
            atomicExch(status, 3);
            break;
        }
        __nanosleep(200);
    }
}

static Exchange *ex_of(alphasparse_cuda_exchange_t h) {
    Exchange *e = reinterpret_cast<Exchange *>(h);
    return (e && e->magic == 0x4153425845434847ull) ? e : nullptr;
}

template <typename T>
static alphasparse_status_t mv_exchange(T alpha, const alphasparse_matrix_t A, struct alpha_matrix_descr descr,
                                        Exchange *e, T beta, T *y) {
    if (!A || !A->mat || !y || !e) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    const alphasparse_datatype_t dt = sizeof(T) == 4 ? ALPHA_SPARSE_DATATYPE_FLOAT : ALPHA_SPARSE_DATATYPE_DOUBLE;
    if (A->datatype != dt || e->datatype != (int)dt) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (A->format != ALPHA_SPARSE_FORMAT_CSR || descr.type != ALPHA_SPARSE_MATRIX_TYPE_GENERAL)
        return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    if (!e->connected) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (c->device != e->device) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    // the block must be this rank's rows of a square matrix
    if (c->rows != e->part[e->rank + 1] - e->part[e->rank] || c->cols != e->total_rows)
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;

    cudaStream_t st = current_stream();
    std::lock_guard<std::mutex> lock(c->mu);
    const int nxt = e->cur ^ 1;
    PeerPush push{};
    push.n = e->world;
    push.row_off = e->part[e->rank];
    push.after = e->mode == 1;
    for (int p = 0; p < e->world; p++) push.dst[p] = e->peer_xbuf[nxt][p];
    alphasparse_status_t s = launch_spmv<T>(c, alpha, static_cast<const T *>(e->xbuf[e->cur]), beta, y, st, &push);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    e->step++;
    // peer_counters table lives in device memory right behind our own counters
    unsigned long long *const *table = reinterpret_cast<unsigned long long *const *>(e->counters + kMaxPeers);
    exchange_arrive_wait_kernel<<<1, 32, 0, st>>>(e->step, e->rank, e->world, table, e->counters, e->d_status,
                                                  4LL << 20, c->d_status);
    count_launch();
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    e->cur = nxt;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// x from host memory, each GPU uploading only its own rows: the block goes over PCIe into this GPU's
// *next* buffer and from there over NVLink into the next buffer of every peer; the same arrive / wait
// and buffer swap as after a product follow, so afterwards every GPU holds all of x in its current
// buffer.  world GPUs move 1/world of x each over their PCIe links instead of all of it each.
template <typename T>
static alphasparse_status_t load_x(Exchange *e, const void *block) {
    const int64_t off = e->part[e->rank], rows = e->part[e->rank + 1] - off;
    if (rows > 0 && !block) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    cudaStream_t st = current_stream();
    const int nxt = e->cur ^ 1;
    T *mine = static_cast<T *>(e->xbuf[nxt]) + off;
    if (rows > 0) {
        ASB_CUDA_OR(cudaMemcpyAsync(mine, block, sizeof(T) * (size_t)rows, cudaMemcpyDefault, st),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        PeerPush push{};
        for (int p = 0; p < e->world; p++)
            if (p != e->rank) push.dst[push.n++] = e->peer_xbuf[nxt][p];
        push.row_off = off;
        launch_push_rows<T>(rows, mine, push, st);
    }
    e->step++;
    unsigned long long *const *table = reinterpret_cast<unsigned long long *const *>(e->counters + kMaxPeers);
    exchange_arrive_wait_kernel<<<1, 32, 0, st>>>(e->step, e->rank, e->world, table, e->counters, e->d_status,
                                                  4LL << 20, nullptr);
    count_launch();
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    e->cur = nxt;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

}  // namespace asb

using namespace asb;

extern "C" {

alphasparse_status_t alphasparse_cuda_exchange_create(alphasparse_cuda_exchange_t *out, alphasparse_datatype_t datatype,
                                                      int rank, int world, const ALPHA_INT *part) {
    if (!out || !part) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    *out = nullptr;
    if (world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (datatype != ALPHA_SPARSE_DATATYPE_FLOAT && datatype != ALPHA_SPARSE_DATATYPE_DOUBLE)
        return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    if (part[0] != 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    for (int p = 0; p < world; p++)
        if (part[p + 1] < part[p]) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    Exchange *e = new (std::nothrow) Exchange();
    if (!e) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    ASB_CUDA_OR(cudaGetDevice(&e->device), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    e->datatype = datatype, e->rank = rank, e->world = world;
    // Measured on B200 (iterated power-law workload): delivering from inside the product kernel wins
    // from 4 GPUs up (0.32 vs 0.41 ms per step at 8); with 2 GPUs a copy kernel afterwards does (0.92 vs 0.98).
    e->mode = world >= 4 ? 0 : 1;
    e->tsz = datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    memcpy(e->part, part, sizeof(int) * (size_t)(world + 1));
    e->total_rows = part[world];
    const size_t xbytes = e->tsz * (size_t)(e->total_rows > 0 ? e->total_rows : 1);
    // counters[kMaxPeers] followed by the table of peer counter addresses [kMaxPeers]
    const size_t cbytes = sizeof(unsigned long long) * kMaxPeers * 2;
    cudaError_t err = device_alloc(&e->xbuf[0], xbytes);
    if (err == cudaSuccess) err = device_alloc(&e->xbuf[1], xbytes);
    if (err == cudaSuccess) err = device_alloc(&e->counters, cbytes);
    if (err == cudaSuccess) err = device_alloc(&e->d_status, sizeof(int));
    if (err == cudaSuccess) err = cudaMemset(e->xbuf[0], 0, xbytes);
    if (err == cudaSuccess) err = cudaMemset(e->xbuf[1], 0, xbytes);
    if (err == cudaSuccess) err = cudaMemset(e->counters, 0, cbytes);
    if (err == cudaSuccess) err = cudaMemset(e->d_status, 0, sizeof(int));
    if (err != cudaSuccess) {
        record_cuda_error(err, "exchange buffers");
        cudaFree(e->xbuf[0]), cudaFree(e->xbuf[1]), cudaFree(e->counters), cudaFree(e->d_status);
        delete e;
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    *out = reinterpret_cast<alphasparse_cuda_exchange_t>(e);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

size_t alphasparse_cuda_exchange_blob_bytes(void) { return kIpcBlob; }

alphasparse_status_t alphasparse_cuda_exchange_export(alphasparse_cuda_exchange_t h, void *blob) {
    Exchange *e = ex_of(h);
    if (!e || !blob) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    cudaIpcMemHandle_t hs[3];
    ASB_CUDA_OR(cudaIpcGetMemHandle(&hs[0], e->xbuf[0]), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaIpcGetMemHandle(&hs[1], e->xbuf[1]), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaIpcGetMemHandle(&hs[2], e->counters), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    memcpy(blob, hs, sizeof(hs));
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t alphasparse_cuda_exchange_connect(alphasparse_cuda_exchange_t h, const void *blobs) {
    Exchange *e = ex_of(h);
    if (!e || !blobs) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    if (e->connected) return ALPHA_SPARSE_STATUS_SUCCESS;
    const char *b = static_cast<const char *>(blobs);
    unsigned long long *table[kMaxPeers] = {};
    for (int p = 0; p < e->world; p++) {
        if (p == e->rank) {
            e->peer_xbuf[0][p] = e->xbuf[0], e->peer_xbuf[1][p] = e->xbuf[1];
            e->peer_counters[p] = e->counters;
        } else {
            cudaIpcMemHandle_t hs[3];
            memcpy(hs, b + (size_t)p * kIpcBlob, sizeof(hs));
            void *ptrs[3] = {nullptr, nullptr, nullptr};
            for (int k = 0; k < 3; k++)
                ASB_CUDA_OR(cudaIpcOpenMemHandle(&ptrs[k], hs[k], cudaIpcMemLazyEnablePeerAccess),
                            ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            e->peer_xbuf[0][p] = ptrs[0], e->peer_xbuf[1][p] = ptrs[1];
            e->peer_counters[p] = static_cast<unsigned long long *>(ptrs[2]);
            e->opened[p] = true;
        }
        table[p] = e->peer_counters[p];
    }
    ASB_CUDA_OR(cudaMemcpy(e->counters + kMaxPeers, table, sizeof(table), cudaMemcpyHostToDevice),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    e->connected = true;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t alphasparse_cuda_exchange_set_mode(alphasparse_cuda_exchange_t h, int mode) {
    Exchange *e = ex_of(h);
    if (!e) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    if (mode != 0 && mode != 1) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    e->mode = mode;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t alphasparse_cuda_exchange_x(alphasparse_cuda_exchange_t h, void **x) {
    Exchange *e = ex_of(h);
    if (!e || !x) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    *x = e->xbuf[e->cur];
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t alphasparse_cuda_exchange_load_x(alphasparse_cuda_exchange_t h, const void *x_block) {
    Exchange *e = ex_of(h);
    if (!e) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    if (!e->connected) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    return e->datatype == ALPHA_SPARSE_DATATYPE_FLOAT ? load_x<float>(e, x_block) : load_x<double>(e, x_block);
}

alphasparse_status_t alphasparse_cuda_exchange_status(alphasparse_cuda_exchange_t h, int *status) {
    Exchange *e = ex_of(h);
    if (!e || !status) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    ASB_CUDA_OR(cudaStreamSynchronize(current_stream()), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaMemcpy(status, e->d_status, sizeof(int), cudaMemcpyDeviceToHost),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return *status == 0 ? ALPHA_SPARSE_STATUS_SUCCESS : ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
}

alphasparse_status_t alphasparse_cuda_exchange_debug_wait(alphasparse_cuda_exchange_t h, int64_t max_polls) {
    Exchange *e = ex_of(h);
    if (!e || max_polls < 1) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    // the last counter slot belongs to a rank that does not exist here unless all eight GPUs take part
    if (e->world >= kMaxPeers) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    exchange_wait_only_kernel<<<1, 1, 0, current_stream()>>>(e->counters + kMaxPeers - 1, ~0ull, e->d_status, max_polls);
    count_launch();
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t alphasparse_cuda_exchange_clear_status(alphasparse_cuda_exchange_t h) {
    Exchange *e = ex_of(h);
    if (!e) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    ASB_CUDA_OR(cudaMemsetAsync(e->d_status, 0, sizeof(int), current_stream()), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t alphasparse_cuda_exchange_destroy(alphasparse_cuda_exchange_t h) {
    Exchange *e = ex_of(h);
    if (!e) return h ? ALPHA_SPARSE_STATUS_INVALID_HANDLE : ALPHA_SPARSE_STATUS_SUCCESS;
    cudaStreamSynchronize(current_stream());
    for (int p = 0; p < e->world; p++)
        if (e->opened[p]) {
            cudaIpcCloseMemHandle(e->peer_xbuf[0][p]);
            cudaIpcCloseMemHandle(e->peer_xbuf[1][p]);
            cudaIpcCloseMemHandle(e->peer_counters[p]);
        }
    cudaFree(e->xbuf[0]), cudaFree(e->xbuf[1]), cudaFree(e->counters), cudaFree(e->d_status);
    e->magic = 0;
    delete e;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t alphasparse_s_mv_exchange(const float alpha, const alphasparse_matrix_t A,
                                               const struct alpha_matrix_descr descr, alphasparse_cuda_exchange_t ex,
                                               const float beta, float *y) {
    return mv_exchange<float>(alpha, A, descr, ex_of(ex), beta, y);
}
alphasparse_status_t alphasparse_d_mv_exchange(const double alpha, const alphasparse_matrix_t A,
                                               const struct alpha_matrix_descr descr, alphasparse_cuda_exchange_t ex,
                                               const double beta, double *y) {
    return mv_exchange<double>(alpha, A, descr, ex_of(ex), beta, y);
}

}  // extern "C"
