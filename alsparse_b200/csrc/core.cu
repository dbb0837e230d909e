// Handle layer and entry points of libalphasparse_b200.so: everything between the C ABI of
// include/alphasparse/spapi.h and the kernels.  Host code only; the kernels live in spmv.cu
// and spmm.cu.  There is no CPU compute path in this library: when no CUDA device can be
// used the create calls fail and mv / mm cannot be reached.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <omp.h>

#include <algorithm>
#include <new>
#include <numeric>
#include <unordered_map>
#include <vector>

#include "alphasparse/kernel_cuda.h"
#include "alphasparse/spapi.h"
#include "alphasparse/util.h"
#include "internal.h"

namespace asb {

// ---- process-wide state ---------------------------------------------------------------------

static std::atomic<cudaStream_t> g_stream{nullptr};
static std::atomic<int> g_alg{-1};
static std::atomic<long long> g_launches{0};
static thread_local char t_error[256] = "";

cudaStream_t current_stream() { return g_stream.load(std::memory_order_relaxed); }

alphasparse_cuda_alg_t forced_algorithm() {
    int a = g_alg.load(std::memory_order_relaxed);
    if (a < 0) {
        a = ALPHA_SPARSE_CUDA_ALG_AUTO;
        if (const char *env = getenv("ALPHASPARSE_CUDA_ALG")) {
            if (!strcmp(env, "vector")) a = ALPHA_SPARSE_CUDA_ALG_VECTOR;
            else if (!strcmp(env, "merge")) a = ALPHA_SPARSE_CUDA_ALG_MERGE;
            else if (!strcmp(env, "rowtile")) a = ALPHA_SPARSE_CUDA_ALG_ROWTILE;
        }
        g_alg.store(a, std::memory_order_relaxed);
    }
    return (alphasparse_cuda_alg_t)a;
}

static std::atomic<long long> g_fail_alloc_in{0};  // > 0: that many allocations from now, the last one fails

cudaError_t device_alloc_bytes(void **p, size_t bytes) {
    long long left = g_fail_alloc_in.load(std::memory_order_relaxed);
    while (left > 0 && !g_fail_alloc_in.compare_exchange_weak(left, left - 1)) {
    }
    if (left == 1) {
        *p = nullptr;
        return cudaErrorMemoryAllocation;
    }
    return cudaMalloc(p, bytes);
}

void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

// ---- tuning options ------------------------------------------------------------------------------
struct OptionDef {
    const char *name;
    int64_t def;
};
static const OptionDef kOptionDefs[kOptCount] = {
    {"band_enable", 1},       {"band_bytes", 64 * 1024}, {"band_min_seg", 12},      {"band_min_rows", 128},
    {"band_min_share_pct", 10}, {"band_splits", 0},      {"band_overlap", 0},      {"band_packed", 1},      {"band_variant", 0},     {"bin_enable", 1},        {"bin_short", 16},         {"bin_mid0", 32},          {"bin_mid1", 256},        {"bin_overlap", 1},      {"bin_mid_max", 16384},   {"bin_push_max_peers", 4}, {"bin_sort", 1}, {"pipe_max_windows", 12}, {"pipe_min_piece_kb", 4096}, {"mv_block_min_kb", 98304}, {"mv_block_kb", 65536}, {"spmm_col_via_row", 2}, {"spmm_narrow", 1}, {"spmm_split_min", 1024}, {"spmm_split_chunk", 512}, {"spmm_col_blocks", 0},
};
static std::atomic<int64_t> g_options[kOptCount];
static std::once_flag g_options_once;

static int option_index(const char *name, size_t len) {
    for (int i = 0; i < kOptCount; i++)
        if (strlen(kOptionDefs[i].name) == len && !strncmp(kOptionDefs[i].name, name, len)) return i;
    return -1;
}

static void options_init() {
    std::call_once(g_options_once, [] {
        for (int i = 0; i < kOptCount; i++) g_options[i].store(kOptionDefs[i].def);
        // ALPHASPARSE_CUDA_OPTIONS="name=value,name=value": initial values
        const char *env = getenv("ALPHASPARSE_CUDA_OPTIONS");
        while (env && *env) {
            while (*env == ' ') env++;  // blanks after a comma
            const char *eq = strchr(env, '='), *end = strchr(env, ',');
            if (!end) end = env + strlen(env);
            if (eq && eq < end) {
                const int i = option_index(env, (size_t)(eq - env));
                if (i >= 0) g_options[i].store(strtoll(eq + 1, nullptr, 10));
            }
            env = *end ? end + 1 : end;
        }
    });
}

int64_t option(Option o) {
    options_init();
    return g_options[o].load(std::memory_order_relaxed);
}

void record_cuda_error(cudaError_t e, const char *what) {
    snprintf(t_error, sizeof(t_error), "%s: %s", what, cudaGetErrorString(e));
    (void)cudaGetLastError();  // clear the sticky-free error so later calls start clean
}

void record_error(const char *what) { snprintf(t_error, sizeof(t_error), "%s", what); }

// ---- device context ----------------------------------------------------------------------------

DeviceCtx *ctx_of(const alphasparse_matrix_t A) {
    if (!A || !A->dcu_info) return nullptr;
    DeviceCtx *c = static_cast<DeviceCtx *>(A->dcu_info);
    return c->magic == kCtxMagic ? c : nullptr;
}

void ctx_destroy(DeviceCtx *c) {
    if (!c) return;
    ctx_destroy(c->transposed);
    c->transposed = nullptr;
    for (DeviceCtx *&d : c->derived) {
        ctx_destroy(d);
        d = nullptr;
    }
    int prev = -1;
    cudaGetDevice(&prev);
    cudaSetDevice(c->device);
    cudaFree(c->d_row_ptr);
    cudaFree(c->d_col);
    cudaFree(c->d_val);
    cudaFree(c->d_tile);
    cudaFree(c->d_carry_row);
    cudaFree(c->d_carry_val);
    cudaFree(c->d_chunk_done);
    cudaFree(c->d_sched);
    band_destroy(c->band);
    bins_destroy(c->bins);
    spmm_blocks_destroy(c->spmm);
    spmm_split_destroy(c->split);
    spmm_blocks_destroy(c->mvb);
    cudaFree(c->d_cm_x);
    cudaFree(c->d_cm_y);
    cudaFree(c->d_x_stage);
    cudaFree(c->d_y_stage);
    cudaFree(c->d_status);
    if (c->copy_in) cudaStreamDestroy(c->copy_in);
    if (c->copy_out) cudaStreamDestroy(c->copy_out);
    for (cudaEvent_t ev : c->ev_pipe)
        if (ev) cudaEventDestroy(ev);
    if (c->ev_start) cudaEventDestroy(c->ev_start);
    if (c->ev_stop) cudaEventDestroy(c->ev_stop);
    if (prev >= 0) cudaSetDevice(prev);
    c->magic = 0;
    delete c;
}

alphasparse_status_t ctx_create(int datatype, int64_t rows, int64_t cols, const int *ptr,
                                const int *col, const void *val, DeviceCtx **out) {
    *out = nullptr;
    int dev = 0;
    ASB_CUDA_OR(cudaGetDevice(&dev), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    DeviceCtx *c = new (std::nothrow) DeviceCtx();
    if (!c) return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    c->device = dev;
    c->datatype = datatype;
    c->rows = rows, c->cols = cols;
    c->nnz = rows > 0 ? (int64_t)ptr[rows] - (int64_t)ptr[0] : 0;
    const size_t tsz = datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    const size_t padded = (size_t)c->nnz + kTailPad;
    cudaStream_t st = current_stream();

    auto fail = [&](alphasparse_status_t s) {
        ctx_destroy(c);
        return s;
    };
#define TRY(expr, status)                        \
    do {                                         \
        cudaError_t _e = (expr);                 \
        if (_e != cudaSuccess) {                 \
            record_cuda_error(_e, #expr);        \
            return fail(status);                 \
        }                                        \
    } while (0)

    // four spare offsets: the row-tile kernel copies offsets in 16-byte units
    TRY(device_alloc(&c->d_row_ptr, sizeof(int) * (size_t)(rows + 1 + 4)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&c->d_status, sizeof(int)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(cudaMemsetAsync(c->d_status, 0, sizeof(int), st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemsetAsync(c->d_row_ptr + rows + 1, 0, sizeof(int) * 4, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(device_alloc(&c->d_col, sizeof(int) * padded), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&c->d_val, tsz * padded), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    c->device_bytes = (int64_t)(sizeof(int) * (size_t)(rows + 1) + (sizeof(int) + tsz) * padded);

    if (rows > 0) {
        TRY(cudaMemcpyAsync(c->d_row_ptr, ptr, sizeof(int) * (size_t)(rows + 1),
                            cudaMemcpyHostToDevice, st),
            ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    } else {
        TRY(cudaMemsetAsync(c->d_row_ptr, 0, sizeof(int), st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }
    if (c->nnz > 0) {
        TRY(cudaMemcpyAsync(c->d_col, col, sizeof(int) * (size_t)c->nnz, cudaMemcpyHostToDevice, st),
            ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        TRY(cudaMemcpyAsync(c->d_val, val, tsz * (size_t)c->nnz, cudaMemcpyHostToDevice, st),
            ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }
    TRY(cudaMemsetAsync(c->d_col + c->nnz, 0, sizeof(int) * kTailPad, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaMemsetAsync(static_cast<char *>(c->d_val) + tsz * (size_t)c->nnz, 0, tsz * kTailPad, st),
        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
#undef TRY

    c->h_row_ptr = rows > 0 ? ptr : nullptr;  // the analysis may bin the rows on the host
    alphasparse_status_t s = ctx_analyse(c);
    c->h_row_ptr = nullptr;
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return fail(s);
    *out = c;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t ctx_adopt(int datatype, int64_t rows, int64_t cols, int64_t nnz, int *d_ptr, int *d_col,
                               void *d_val, DeviceCtx **out) {
    *out = nullptr;
    DeviceCtx *c = new (std::nothrow) DeviceCtx();
    int dev = 0;
    if (!c || cudaGetDevice(&dev) != cudaSuccess) {
        delete c;
        cudaFree(d_ptr), cudaFree(d_col), cudaFree(d_val);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    const size_t tsz = datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    c->device = dev, c->datatype = datatype, c->rows = rows, c->cols = cols, c->nnz = nnz;
    c->d_row_ptr = d_ptr, c->d_col = d_col, c->d_val = d_val;
    c->device_bytes = (int64_t)(sizeof(int) * (size_t)(rows + 1) + (sizeof(int) + tsz) * ((size_t)nnz + kTailPad));
    cudaError_t e = device_alloc(&c->d_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemsetAsync(c->d_status, 0, sizeof(int), current_stream());
    if (e != cudaSuccess) {
        record_cuda_error(e, "ctx_adopt");
        ctx_destroy(c);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    alphasparse_status_t s = ctx_analyse(c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
        ctx_destroy(c);
        return s;
    }
    *out = c;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- host copies ---------------------------------------------------------------------------------

template <typename T>
struct CsrOf;
template <>
struct CsrOf<float> {
    using csr = spmat_csr_s_t;
    using coo = spmat_coo_s_t;
    using csc = spmat_csc_s_t;
    static constexpr alphasparse_datatype_t dt = ALPHA_SPARSE_DATATYPE_FLOAT;
};
template <>
struct CsrOf<double> {
    using csr = spmat_csr_d_t;
    using coo = spmat_coo_d_t;
    using csc = spmat_csc_d_t;
    static constexpr alphasparse_datatype_t dt = ALPHA_SPARSE_DATATYPE_DOUBLE;
};

static void *host_alloc(size_t bytes) {
    void *p = nullptr;
    if (posix_memalign(&p, 64, bytes ? bytes : 64) != 0) return nullptr;
    return p;
}

template <typename T>
static void free_csr_host(typename CsrOf<T>::csr *m) {
    if (!m) return;
    free(m->values);
    free(m->rows_start);
    free(m->col_indx);
    free(m);
}

// Host CSR record -> device context.  The kernel-level entry points (gemv_?_csr, gemm_?_csr_row, ... at the
// end of this file) receive only the record, as the reference's dispatch tables pass it; records of handles
// made by this library are entered at creation and removed by alphasparse_destroy, records the library has
// never seen are uploaded on first use (`adopted`) and stay until alphasparse_cuda_release_csr.
struct RegistryEntry {
    DeviceCtx *ctx;
    bool adopted;
};
static std::mutex g_registry_mu;
static std::unordered_map<const void *, RegistryEntry> &registry() {
    static std::unordered_map<const void *, RegistryEntry> r;
    return r;
}
static void registry_add(const void *record, DeviceCtx *c, bool adopted) {
    std::lock_guard<std::mutex> lock(g_registry_mu);
    registry()[record] = RegistryEntry{c, adopted};
}
static RegistryEntry registry_take(const void *record) {
    std::lock_guard<std::mutex> lock(g_registry_mu);
    auto it = registry().find(record);
    if (it == registry().end()) return RegistryEntry{nullptr, false};
    RegistryEntry e = it->second;
    registry().erase(it);
    return e;
}

// Takes ownership of ptr / col / val (host_alloc'ed, zero-based 3-array CSR) and builds the
// handle around them: host record for export_csr, device copy and analysis for mv / mm.
template <typename T>
static alphasparse_status_t finish_csr_handle(alphasparse_matrix_t *A, int64_t rows, int64_t cols,
                                              int *ptr, int *col, T *val) {
    using M = typename CsrOf<T>::csr;
    alphasparse_matrix *h = static_cast<alphasparse_matrix *>(calloc(1, sizeof(alphasparse_matrix)));
    M *m = static_cast<M *>(calloc(1, sizeof(M)));
    if (!h || !m) {
        free(h), free(m), free(ptr), free(col), free(val);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    m->values = val;
    m->rows_start = ptr;
    m->rows_end = ptr + 1;
    m->col_indx = col;
    m->rows = (ALPHA_INT)rows;
    m->cols = (ALPHA_INT)cols;
    m->ordered = false;
    h->mat = m;
    h->format = ALPHA_SPARSE_FORMAT_CSR;
    h->datatype = CsrOf<T>::dt;

    DeviceCtx *c = nullptr;
    alphasparse_status_t s = ctx_create(CsrOf<T>::dt, rows, cols, ptr, col, val, &c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
        free_csr_host<T>(m);
        free(h);
        return s;
    }
    m->d_values = static_cast<T *>(c->d_val);
    m->d_row_ptr = c->d_row_ptr;
    m->d_col_indx = c->d_col;
    h->dcu_info = c;
    registry_add(m, c, false);
    *A = h;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Reference semantics (src/core/format/alphasparse_x_create_csr.c:22-55): the element count is
// rows_end[rows-1] - rows_start[0]; offsets are rows_start[0] followed by rows_end[*]; columns
// and values are copied from element 0; one-based input loses 1 from every offset and column.
template <typename T>
static alphasparse_status_t create_csr(alphasparse_matrix_t *A, alphasparse_index_base_t indexing,
                                       ALPHA_INT rows, ALPHA_INT cols, const ALPHA_INT *rows_start,
                                       const ALPHA_INT *rows_end, const ALPHA_INT *col_indx,
                                       const T *values) {
    if (!A) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    *A = nullptr;
    if (rows < 0 || cols < 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (rows > 0 && (!rows_start || !rows_end)) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    const int shift = indexing == ALPHA_SPARSE_INDEX_BASE_ONE ? 1 : 0;
    const int64_t nnz = rows > 0 ? (int64_t)rows_end[rows - 1] - (int64_t)rows_start[0] : 0;
    if (nnz < 0 || nnz > (int64_t)INT32_MAX - 2 * kTailPad) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && (!col_indx || !values)) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;

    int *ptr = static_cast<int *>(host_alloc(sizeof(int) * (size_t)(rows + 1)));
    int *col = static_cast<int *>(host_alloc(sizeof(int) * (size_t)nnz));
    T *val = static_cast<T *>(host_alloc(sizeof(T) * (size_t)nnz));
    if (!ptr || !col || !val) {
        free(ptr), free(col), free(val);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    // Offsets are stored relative to the first stored element, which is element 0 of the copied
    // arrays.  (The reference keeps rows_start[0] as is while copying from element 0, which only
    // works when rows_start[0] equals the index base; for that case the two agree bit for bit.)
    const int first = rows > 0 ? rows_start[0] : 0;
    ptr[0] = 0;
#pragma omp parallel for schedule(static) if (rows > (1 << 16))
    for (int64_t i = 0; i < rows; i++) ptr[i + 1] = rows_end[i] - first;
#pragma omp parallel for schedule(static) if (nnz > (1 << 16))
    for (int64_t i = 0; i < nnz; i++) {
        col[i] = col_indx[i] - shift;
        val[i] = values[i];
    }
    return finish_csr_handle<T>(A, rows, cols, ptr, col, val);
}

// A CSC handle around `t`, the CSR handle of the transposed matrix (which it takes over): the CSC
// record borrows t's host arrays -- cols_start / cols_end / row_indx / values of A are
// rows_start / rows_end / col_indx / values of A^T -- and t itself sits in `inspector`.
template <typename T>
static alphasparse_status_t wrap_as_csc(alphasparse_matrix_t t, alphasparse_matrix_t *A) {
    using M = typename CsrOf<T>::csc;
    const typename CsrOf<T>::csr *tm = static_cast<const typename CsrOf<T>::csr *>(t->mat);
    alphasparse_matrix *h = static_cast<alphasparse_matrix *>(calloc(1, sizeof(alphasparse_matrix)));
    M *m = static_cast<M *>(calloc(1, sizeof(M)));
    if (!h || !m) {
        free(h), free(m);
        alphasparse_destroy(t);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    m->values = tm->values;
    m->cols_start = tm->rows_start, m->cols_end = tm->rows_end;
    m->row_indx = tm->col_indx;
    m->rows = tm->cols, m->cols = tm->rows;
    m->ordered = false;
    h->mat = m;
    h->format = ALPHA_SPARSE_FORMAT_CSC;
    h->datatype = CsrOf<T>::dt;
    h->inspector = t;
    *A = h;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Reference semantics: src/core/format/alphasparse_x_create_csc.c:7-57 (deep copy; element count
// cols_end[cols-1]; one-based input rebased).  That file copies cols_end over `rows` entries
// (:35,46), which leaves offsets unset when cols > rows; here all `cols` entries are copied.
template <typename T>
static alphasparse_status_t create_csc(alphasparse_matrix_t *A, alphasparse_index_base_t indexing,
                                       ALPHA_INT rows, ALPHA_INT cols, const ALPHA_INT *cols_start,
                                       const ALPHA_INT *cols_end, const ALPHA_INT *row_indx, const T *values) {
    if (!A) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    *A = nullptr;
    alphasparse_matrix_t t = nullptr;
    alphasparse_status_t s = create_csr<T>(&t, indexing, cols, rows, cols_start, cols_end, row_indx, values);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    return wrap_as_csc<T>(t, A);
}

// Reference semantics: src/core/format/alphasparse_x_create_coo.c:16-45 (deep copy, one-based
// input rebased).  A COO handle never touches the device; it only feeds convert_csr.
template <typename T>
static alphasparse_status_t create_coo(alphasparse_matrix_t *A, alphasparse_index_base_t indexing,
                                       ALPHA_INT rows, ALPHA_INT cols, ALPHA_INT nnz,
                                       const ALPHA_INT *row_indx, const ALPHA_INT *col_indx,
                                       const T *values) {
    using M = typename CsrOf<T>::coo;
    if (!A) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    *A = nullptr;
    if (rows < 0 || cols < 0 || nnz < 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (nnz > 0 && (!row_indx || !col_indx || !values)) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    const int shift = indexing == ALPHA_SPARSE_INDEX_BASE_ONE ? 1 : 0;
    alphasparse_matrix *h = static_cast<alphasparse_matrix *>(calloc(1, sizeof(alphasparse_matrix)));
    M *m = static_cast<M *>(calloc(1, sizeof(M)));
    int *ri = static_cast<int *>(host_alloc(sizeof(int) * (size_t)nnz));
    int *ci = static_cast<int *>(host_alloc(sizeof(int) * (size_t)nnz));
    T *v = static_cast<T *>(host_alloc(sizeof(T) * (size_t)nnz));
    if (!h || !m || !ri || !ci || !v) {
        free(h), free(m), free(ri), free(ci), free(v);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
#pragma omp parallel for schedule(static) if (nnz > (1 << 16))
    for (int64_t i = 0; i < nnz; i++) {
        ri[i] = row_indx[i] - shift;
        ci[i] = col_indx[i] - shift;
        v[i] = values[i];
    }
    m->values = v, m->row_indx = ri, m->col_indx = ci;
    m->rows = rows, m->cols = cols, m->nnz = nnz, m->ordered = false;
    h->mat = m;
    h->format = ALPHA_SPARSE_FORMAT_COO;
    h->datatype = CsrOf<T>::dt;
    *A = h;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// (row, column, value) triples -> 3-array CSR with the elements of a row ordered by column and equal
// (row, column) pairs kept in input order: counting pass by row, then a stable sort of each row, rows
// in parallel.  Output arrays are host_alloc'ed.
template <typename T>
static alphasparse_status_t triples_to_csr(int64_t rows, int64_t nnz, const int *ri, const int *ci, const T *v,
                                           int **out_ptr, int **out_col, T **out_val) {
    int *ptr = static_cast<int *>(host_alloc(sizeof(int) * (size_t)(rows + 1)));
    int *col = static_cast<int *>(host_alloc(sizeof(int) * (size_t)nnz));
    T *val = static_cast<T *>(host_alloc(sizeof(T) * (size_t)nnz));
    std::vector<int> fill, order;
    try {
        fill.assign((size_t)rows + 1, 0);
        order.resize((size_t)nnz);
    } catch (...) {
        free(ptr), free(col), free(val);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    if (!ptr || !col || !val) {
        free(ptr), free(col), free(val);
        return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
    }
    for (int64_t i = 0; i < nnz; i++) fill[(size_t)ri[i] + 1]++;
    ptr[0] = 0;
    for (int64_t r = 0; r < rows; r++) ptr[r + 1] = ptr[r] + fill[(size_t)r + 1];
    for (int64_t r = 0; r < rows; r++) fill[(size_t)r] = ptr[r];
    for (int64_t i = 0; i < nnz; i++) order[(size_t)fill[(size_t)ri[i]]++] = (int)i;
#pragma omp parallel for schedule(dynamic, 1024)
    for (int64_t r = 0; r < rows; r++) {
        int *b = order.data() + ptr[r], *e = order.data() + ptr[r + 1];
        std::stable_sort(b, e, [&](int p, int q) { return ci[p] < ci[q]; });
        for (int *it = b; it != e; ++it) {
            const size_t o = (size_t)(it - order.data());
            col[o] = ci[*it];
            val[o] = v[*it];
        }
    }
    *out_ptr = ptr, *out_col = col, *out_val = val;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// COO -> CSR with the output the reference produces (src/core/format/convert_csr_x_coo.c:14-81):
// elements ordered by (row, column), duplicates all kept, offsets by counting.  The reference
// sorts nnz records with a serial qsort; here a counting pass buckets the elements by row in
// input order and each row is then sorted by column with a stable sort, in parallel over rows.
// Equal (row, column) pairs keep their input order (qsort leaves theirs unspecified).
// With transpose = true rows and columns swap roles (the reference transposes the COO handle
// first, src/core/op_/alphasparse_convert_csr.c:144-151).
template <typename T>
static alphasparse_status_t coo_to_csr(const typename CsrOf<T>::coo *src, bool transpose,
                                       alphasparse_matrix_t *dest) {
    const int64_t rows = transpose ? src->cols : src->rows;
    const int64_t cols = transpose ? src->rows : src->cols;
    const int64_t nnz = src->nnz;
    const int *ri = transpose ? src->col_indx : src->row_indx;
    const int *ci = transpose ? src->row_indx : src->col_indx;
    // Large inputs are sorted on the GPU (radix sort, coo2csr.cu); ALPHASPARSE_CUDA_COO=host|device forces a path.
    static const int forced = [] {
        const char *e = getenv("ALPHASPARSE_CUDA_COO");
        return !e ? 0 : !strcmp(e, "host") ? 1 : !strcmp(e, "device") ? 2 : 0;
    }();
    if (nnz > 0 && forced != 1 && (forced == 2 || nnz >= (1 << 20))) {
        int *ptr = static_cast<int *>(host_alloc(sizeof(int) * (size_t)(rows + 1)));
        int *col = static_cast<int *>(host_alloc(sizeof(int) * (size_t)nnz));
        T *val = static_cast<T *>(host_alloc(sizeof(T) * (size_t)nnz));
        if (!ptr || !col || !val) {
            free(ptr), free(col), free(val);
            return ALPHA_SPARSE_STATUS_ALLOC_FAILED;
        }
        alphasparse_status_t s = coo_to_csr_device<T>(rows, cols, nnz, ri, ci, src->values, ptr, col, val);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
            free(ptr), free(col), free(val);
            return s;
        }
        return finish_csr_handle<T>(dest, rows, cols, ptr, col, val);
    }
    for (int64_t i = 0; i < nnz; i++)
        if (ri[i] < 0 || ri[i] >= rows || ci[i] < 0 || ci[i] >= cols)
            return ALPHA_SPARSE_STATUS_INVALID_VALUE;

    int *ptr = nullptr, *col = nullptr;
    T *val = nullptr;
    alphasparse_status_t s = triples_to_csr<T>(rows, nnz, ri, ci, src->values, &ptr, &col, &val);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    return finish_csr_handle<T>(dest, rows, cols, ptr, col, val);
}

// ---- transpose ---------------------------------------------------------------------------------

// Device CSR of A^T, built once from the handle's DEVICE copy (transpose_csr_device: a stable radix sort by
// column) and kept with the handle.  The reference materialises the transpose on every transposed mm call
// (src/kernel/x86_64/level3/mm/gemm/gemm_x_csr_row_trans.c:5-12 -> src/core/format/transpose_x_csr.c:7-62)
// and scatters with a serial loop in the transposed mv (src/plain/kernel/level2/mv/gemv/gemv_x_csr_trans_plain.c:14-25).
// The elements of a column come out by ascending row -- the order in which the reference's loop adds them.
template <typename T>
static alphasparse_status_t ensure_transposed(DeviceCtx *c, const typename CsrOf<T>::csr *) {
    if (c->transposed) return ALPHA_SPARSE_STATUS_SUCCESS;
    int *tptr = nullptr, *tcol = nullptr;
    T *tval = nullptr;
    alphasparse_status_t s = transpose_csr_device<T>(c, &tptr, &tcol, &tval);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    DeviceCtx *t = nullptr;
    s = ctx_adopt(c->datatype, c->cols, c->rows, c->nnz, tptr, tcol, tval, &t);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    c->transposed = t;
    c->device_bytes += t->device_bytes;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- structured descriptors ---------------------------------------------------------------------

// mv under a SYMMETRIC, TRIANGULAR or DIAGONAL descriptor (the other CSR branches of the reference's
// alphasparse_?_mv, src/core/op/level2/alphasparse_x_mv.c:1693-1716; kernels under
// src/plain/kernel/level2/mv/{symv,trmv,diagmv}) is an ordinary SpMV with a matrix DERIVED from the
// stored one: the kept triangle (plus an explicit unit diagonal), its mirror image for SYMMETRIC, its
// transpose for op = TRANSPOSE, or just the diagonal.  Each variant is built once on the device from the device
// copy of the stored matrix (derive_csr_device), analysed like any matrix and kept with the handle.
//
// The same matrices serve mm (symm / trmm / diagmm, src/core/op/level3/alphasparse_x_mm.c:2345-2368;
// kernels under src/plain/kernel/level3/mm/{symm,trmm,diagmm}).  Only rows that store their diagonal
// more than once tell the reference's three diagonal kernels apart: diagmv stops at the FIRST stored
// diagonal entry (diagmv_x_csr_n_plain.c:12-27), the row-major diagmm adds ALL of them
// (diagmm_x_csr_n_row_plain.c:14-22) and the column-major diagmm keeps the LAST
// (diagmm_x_csr_n_col_plain.c:7-15); `diag_rule` selects which.
enum DiagRule { kDiagFirst = 0, kDiagAll = 1, kDiagLast = 2 };

static int derived_slot(int type, int upper, int unit, int trans, int diag_rule) {
    if (type == ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL) return 16 + diag_rule * 2 + unit;  // 16..21
    const int t = type == ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC ? 0 : 1;
    return t * 8 + upper * 4 + unit * 2 + trans;
}

template <typename T>
static alphasparse_status_t ensure_derived(DeviceCtx *c, const typename CsrOf<T>::csr *m, int type, int upper,
                                           int unit, int trans, int diag_rule, DeviceCtx **out) {
    DeviceCtx *&slot = c->derived[derived_slot(type, upper, unit, trans, diag_rule)];
    if (slot) {
        *out = slot;
        return ALPHA_SPARSE_STATUS_SUCCESS;
    }
    (void)m;
    const int64_t n = c->rows;
    const bool flip = type == ALPHA_SPARSE_MATRIX_TYPE_TRIANGULAR && trans;
    int *dptr = nullptr, *dcol = nullptr;
    T *dval = nullptr;
    int64_t dnnz = 0;
    alphasparse_status_t s = derive_csr_device<T>(c, type, upper, unit, flip, diag_rule, &dptr, &dcol, &dval, &dnnz);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    DeviceCtx *d = nullptr;
    s = ctx_adopt(c->datatype, n, n, dnnz, dptr, dcol, dval, &d);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    c->device_bytes += d->device_bytes;
    slot = d;
    *out = d;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- pointer kinds and staging ------------------------------------------------------------------

// true when `p` can be dereferenced by a kernel running on `device`
static bool is_device_pointer(const void *p, int device) {
    cudaPointerAttributes at;
    cudaError_t e = cudaPointerGetAttributes(&at, p);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (at.type == cudaMemoryTypeDevice) return true;
    if (at.type == cudaMemoryTypeManaged) return true;
    (void)device;
    return false;  // unregistered or page-locked host memory: staged
}

// Device-side address of a page-locked (cudaHostAlloc / cudaHostRegister) host buffer, or null when
// the memory is pageable or not mapped into the device address space.
static void *device_alias_of_pinned(const void *p) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return nullptr;
    }
    return at.type == cudaMemoryTypeHost ? at.devicePointer : nullptr;
}

static alphasparse_status_t grow(void **buf, size_t *have, size_t want, DeviceCtx *c) {
    if (*have >= want) return ALPHA_SPARSE_STATUS_SUCCESS;
    cudaFree(*buf);
    *buf = nullptr;
    c->device_bytes -= (int64_t)*have;
    *have = 0;
    ASB_CUDA_OR(device_alloc(buf, want), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    *have = want;
    c->device_bytes += (int64_t)want;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int want) {
        if (cudaGetDevice(&prev) != cudaSuccess) {
            ok = false;
            return;
        }
        if (prev != want && cudaSetDevice(want) != cudaSuccess) ok = false;
        if (prev == want) prev = -1;
    }
    ~DeviceGuard() {
        if (prev >= 0) cudaSetDevice(prev);
    }
};

// ---- mv / mm -----------------------------------------------------------------------------------------

// Argument checks in the reference's order (src/core/op/level2/alphasparse_x_mv.c:1670-1716,
// src/core/op/level3/alphasparse_x_mm.c:2317-2338).  Returns SUCCESS when the call is one of the
// CSR cases this backend serves (GENERAL, SYMMETRIC, TRIANGULAR, DIAGONAL); every other case the
// reference would run on its CPU kernels is NOT_SUPPORTED here.
static alphasparse_status_t check_call(const alphasparse_matrix_t A, const void *x, const void *y,
                                       alphasparse_datatype_t dt, alphasparse_operation_t op,
                                       struct alpha_matrix_descr descr) {
    if (!A || !A->mat || !x || !y) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (A->datatype != dt) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (op == ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (descr.type == ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC ||
        descr.type == ALPHA_SPARSE_MATRIX_TYPE_HERMITIAN) {
        int64_t r = 0, c = 0;
        if (A->format == ALPHA_SPARSE_FORMAT_CSR) {
            const spmat_csr_s_t *m = static_cast<const spmat_csr_s_t *>(A->mat);  // same prefix for d
            r = m->rows, c = m->cols;
        } else if (A->format == ALPHA_SPARSE_FORMAT_COO) {
            const spmat_coo_s_t *m = static_cast<const spmat_coo_s_t *>(A->mat);
            r = m->rows, c = m->cols;
        } else if (A->format == ALPHA_SPARSE_FORMAT_CSC) {
            const spmat_csc_s_t *m = static_cast<const spmat_csc_s_t *>(A->mat);
            r = m->rows, c = m->cols;
        }
        if (r != c) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    }
    if (A->format == ALPHA_SPARSE_FORMAT_CSR) {
        if (descr.type == ALPHA_SPARSE_MATRIX_TYPE_GENERAL) return ALPHA_SPARSE_STATUS_SUCCESS;
        if (descr.type == ALPHA_SPARSE_MATRIX_TYPE_HERMITIAN) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;  // complex only
        if (descr.type >= ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC &&
            descr.type <= ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL)
            return ALPHA_SPARSE_STATUS_SUCCESS;
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    }
    if (A->format == ALPHA_SPARSE_FORMAT_COO ||   // served for GENERAL through a CSR copy (csr_shadow_of)
        (A->format == ALPHA_SPARSE_FORMAT_CSC && A->inspector)) {  // ... through the CSR handle of A^T
        if (descr.type == ALPHA_SPARSE_MATRIX_TYPE_GENERAL) return ALPHA_SPARSE_STATUS_SUCCESS;
        if (descr.type >= ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC && descr.type <= ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL)
            return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    }
    if (A->format >= ALPHA_SPARSE_FORMAT_CSC && A->format <= ALPHA_SPARSE_FORMAT_DIA)
        return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    return ALPHA_SPARSE_STATUS_INVALID_VALUE;
}

// A COO handle given straight to mv / mm (the COO block of the reference's dispatchers,
// src/core/op/level2/alphasparse_x_mv.c:1718-1741 and src/core/op/level3/alphasparse_x_mm.c:2370-2376; kernels
// src/plain/kernel/level2/mv/gemv/gemv_x_coo[_trans]_plain.c and .../level3/mm/gemm/gemm_x_coo_{row,col}[_trans]_plain.c):
// those kernels add alpha*a*x[col] into y[row] entry by entry, i.e. the general product in another
// summation order.  Here the product runs on a CSR copy of the matrix, converted on first use (the
// device radix sort for large inputs) and kept in the handle's otherwise unused `inspector` slot
// until alphasparse_destroy.
static std::mutex g_shadow_mu;

static alphasparse_status_t csr_shadow_of(const alphasparse_matrix_t A, alphasparse_matrix_t *out) {
    if (A->format == ALPHA_SPARSE_FORMAT_CSC) {  // made at creation; the caller flips the operation
        *out = static_cast<alphasparse_matrix_t>(A->inspector);
        return ALPHA_SPARSE_STATUS_SUCCESS;
    }
    std::lock_guard<std::mutex> lock(g_shadow_mu);
    if (!A->inspector) {
        alphasparse_matrix_t csr = nullptr;
        alphasparse_status_t s = ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
        if (A->datatype == ALPHA_SPARSE_DATATYPE_FLOAT)
            s = coo_to_csr<float>(static_cast<const spmat_coo_s_t *>(A->mat), false, &csr);
        else if (A->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE)
            s = coo_to_csr<double>(static_cast<const spmat_coo_d_t *>(A->mat), false, &csr);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        A->inspector = csr;
    }
    *out = static_cast<alphasparse_matrix_t>(A->inspector);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Host y (and host or device x) on a large matrix: the product runs in row windows so that PCIe and the kernel
// overlap.  Three streams: x and the y0 pieces go in on one, the windows run on the library stream as their inputs
// land, every finished piece of y leaves on the third while the next window is being multiplied (PCIe is full
// duplex).  The call still returns only when all of y is back in host memory.
// The number of windows follows the size of y: pieces of at least pipe_min_piece_kb, at most pipe_max_windows of
// them (on B200 4 / 8 / 12 / 16 windows took a 64 MB y to 3.18 / 2.93 / 2.86 / 2.88 ms end to end; an 8 MB y --
// one GPU's share of the same vector on eight GPUs -- is quicker in two pieces than in eight, where the seventeen
// events and copies of 1 MB cost more than they hide).  The dense-block product keeps kPipelineChunks windows.
constexpr int64_t kPipelineMinRows = 1 << 20;
constexpr int kPipelineChunks = 8;

static int pipeline_windows(size_t y_bytes) {
    const size_t piece = (size_t)std::max<int64_t>(64, option(kOptPipeMinPieceKb)) << 10;
    const size_t most = (size_t)std::max<int64_t>(1, std::min<int64_t>(16, option(kOptPipeMaxWindows)));
    return (int)std::max<size_t>(1, std::min<size_t>(y_bytes / piece, most));
}

// the two copy streams and the events of the host-operand pipelines, created on first use
static alphasparse_status_t ensure_pipe(DeviceCtx *c) {
    if (c->copy_in) return ALPHA_SPARSE_STATUS_SUCCESS;
    ASB_CUDA_OR(cudaStreamCreateWithFlags(&c->copy_in, cudaStreamNonBlocking), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    ASB_CUDA_OR(cudaStreamCreateWithFlags(&c->copy_out, cudaStreamNonBlocking), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    for (cudaEvent_t &ev : c->ev_pipe)
        ASB_CUDA_OR(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template <typename T>
static alphasparse_status_t mv_host_pipelined(DeviceCtx *c, T alpha, const T *x, bool x_dev, T beta, T *y,
                                              cudaStream_t st) {
    alphasparse_status_t s = ALPHA_SPARSE_STATUS_SUCCESS;
    if (!x_dev) s = grow(&c->d_x_stage, &c->x_stage_bytes, sizeof(T) * (size_t)c->cols, c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    s = grow(&c->d_y_stage, &c->y_stage_bytes, sizeof(T) * (size_t)c->rows, c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    s = ensure_pipe(c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    const T *dx = x_dev ? x : static_cast<const T *>(c->d_x_stage);
    T *dy = static_cast<T *>(c->d_y_stage);
    cudaEvent_t ev_x = c->ev_pipe[0];
    // The staging buffers are free: every call that uses them waits for its copies before it returns.  So the
    // inbound copies start at once, beside whatever is still queued on the library stream (for instance the
    // exchange that is bringing a device x together).
    if (!x_dev) {  // a device x is already where the kernels read it (and ordered on the library stream)
        ASB_CUDA_OR(cudaMemcpyAsync(c->d_x_stage, x, sizeof(T) * (size_t)c->cols, cudaMemcpyHostToDevice, c->copy_in),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaEventRecord(ev_x, c->copy_in), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaStreamWaitEvent(st, ev_x, 0), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }

    const int windows = pipeline_windows(sizeof(T) * (size_t)c->rows);
    const int64_t step = ((c->rows + windows - 1) / windows + 1023) & ~1023ll;
    for (int k = 0; k < windows; k++) {
        const int64_t rb = k * step;
        if (rb >= c->rows) break;
        const RowWindow w{rb, std::min<int64_t>(step, c->rows - rb)};
        cudaEvent_t ev_in = c->ev_pipe[1 + 2 * k], ev_done = c->ev_pipe[2 + 2 * k];
        if (beta != T(0)) {
            ASB_CUDA_OR(cudaMemcpyAsync(dy + rb, y + rb, sizeof(T) * (size_t)w.count, cudaMemcpyHostToDevice, c->copy_in),
                        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            ASB_CUDA_OR(cudaEventRecord(ev_in, c->copy_in), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            ASB_CUDA_OR(cudaStreamWaitEvent(st, ev_in, 0), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        }
        s = launch_spmv<T>(c, alpha, dx, beta, dy, st, nullptr, &w);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        ASB_CUDA_OR(cudaEventRecord(ev_done, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaStreamWaitEvent(c->copy_out, ev_done, 0), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaMemcpyAsync(y + rb, dy + rb, sizeof(T) * (size_t)w.count, cudaMemcpyDeviceToHost, c->copy_out),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }
    int kernel_status = 0;
    ASB_CUDA_OR(cudaMemcpyAsync(&kernel_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, c->copy_out),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaStreamSynchronize(c->copy_out), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    if (kernel_status != 0) (void)cudaMemsetAsync(c->d_status, 0, sizeof(int), st);  // reported once
    return kernel_status == 0 ? ALPHA_SPARSE_STATUS_SUCCESS : ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
}

// The matrix a structured (SYMMETRIC / TRIANGULAR / DIAGONAL) mv or mm call multiplies by, in *c.
template <typename T>
static alphasparse_status_t select_structured(DeviceCtx *&c, const alphasparse_matrix_t A, alphasparse_operation_t op,
                                              struct alpha_matrix_descr descr, int diag_rule) {
    // SYMMETRIC has no transposed entry in the reference's tables (NOT_SUPPORTED there too); the
    // diagonal kernels ignore the operation; fill / diag flags outside {0,1} index past its tables
    if (descr.type == ALPHA_SPARSE_MATRIX_TYPE_SYMMETRIC && op != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE)
        return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    if ((unsigned)descr.mode > 1u || (unsigned)descr.diag > 1u) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (c->rows != c->cols) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    const int trans = descr.type == ALPHA_SPARSE_MATRIX_TYPE_TRIANGULAR && op == ALPHA_SPARSE_OPERATION_TRANSPOSE;
    const int upper = descr.type == ALPHA_SPARSE_MATRIX_TYPE_DIAGONAL ? 0 : (int)descr.mode;
    std::lock_guard<std::mutex> build(c->mu);
    DeviceCtx *d = nullptr;
    alphasparse_status_t s = ensure_derived<T>(c, static_cast<const typename CsrOf<T>::csr *>(A->mat), (int)descr.type,
                                               upper, (int)descr.diag, trans, diag_rule, &d);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    c = d;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// y = alpha * (matrix of c) * x + beta * y with x, y in host or device memory: the part of mv that no longer
// looks at the handle.  Host vectors are staged (pipelined in row windows when large) and the call returns when
// y is complete; device vectors are only enqueued.
template <typename T>
static alphasparse_status_t mv_on_ctx(DeviceCtx *c, T alpha, const T *x, T beta, T *y) {
    alphasparse_status_t s = ALPHA_SPARSE_STATUS_SUCCESS;
    if (c->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
    cudaStream_t st = current_stream();
    const bool x_dev = is_device_pointer(x, c->device), y_dev = is_device_pointer(y, c->device);
    std::lock_guard<std::mutex> lock(c->mu);

    if (!y_dev && c->rows >= kPipelineMinRows && spmv_supports_windows(c) && !c->profile)
        return mv_host_pipelined<T>(c, alpha, x, x_dev, beta, y, st);

    const T *dx = x;
    T *dy = y;
    if (!x_dev) {
        const size_t bytes = sizeof(T) * (size_t)c->cols;
        s = grow(&c->d_x_stage, &c->x_stage_bytes, bytes ? bytes : sizeof(T), c);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        if (bytes)
            ASB_CUDA_OR(cudaMemcpyAsync(c->d_x_stage, x, bytes, cudaMemcpyHostToDevice, st),
                        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        dx = static_cast<const T *>(c->d_x_stage);
    }
    if (!y_dev) {
        const size_t bytes = sizeof(T) * (size_t)c->rows;
        s = grow(&c->d_y_stage, &c->y_stage_bytes, bytes, c);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        if (beta != T(0))
            ASB_CUDA_OR(cudaMemcpyAsync(c->d_y_stage, y, bytes, cudaMemcpyHostToDevice, st),
                        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        dy = static_cast<T *>(c->d_y_stage);
    }
    // Merge kernel + page-locked host y on a large matrix: the kernel's chunk delivery (the mechanism
    // that feeds peer GPUs in the multi-GPU exchange) stores finished chunks of y straight into the
    // host buffer over PCIe while later chunks are still being multiplied, instead of a copy afterwards.
    void *y_alias = nullptr;
    if (!y_dev && c->algorithm == ALPHA_SPARSE_CUDA_ALG_MERGE && c->nnz > 0 && c->rows >= kPipelineMinRows)
        y_alias = device_alias_of_pinned(y);
    if (y_alias) {
        PeerPush push{};
        push.n = 1, push.dst[0] = y_alias, push.row_off = 0, push.after = 0, push.runs = 1;
        s = launch_spmv<T>(c, alpha, dx, beta, dy, st, &push);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    } else {
        s = launch_spmv<T>(c, alpha, dx, beta, dy, st);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        if (!y_dev) {
            ASB_CUDA_OR(cudaMemcpyAsync(y, dy, sizeof(T) * (size_t)c->rows, cudaMemcpyDeviceToHost, st),
                        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        }
    }
    if (!y_dev || !x_dev) {
        // a synchronous call can also report a kernel whose bounded wait ran out
        int kernel_status = 0;
        ASB_CUDA_OR(cudaMemcpyAsync(&kernel_status, c->d_status, sizeof(int), cudaMemcpyDeviceToHost, st),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        if (kernel_status != 0) {  // reported once: later calls start clean
            (void)cudaMemsetAsync(c->d_status, 0, sizeof(int), st);
            return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
        }
    }
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template <typename T>
static alphasparse_status_t mv(alphasparse_operation_t op, T alpha, alphasparse_matrix_t A,
                               struct alpha_matrix_descr descr, const T *x, T beta, T *y) {
    alphasparse_status_t s = check_call(A, x, y, CsrOf<T>::dt, op, descr);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    if (A->format != ALPHA_SPARSE_FORMAT_CSR) {
        // A CSC matrix is held as the CSR of its transpose (src/core/op/level2/alphasparse_x_mv.c's CSC block
        // runs gemv_csc / gemv_csc_trans, src/plain/kernel/level2/mv/gemv/gemv_x_csc[_trans]_plain.c: the
        // same products in another summation order)
        if (A->format == ALPHA_SPARSE_FORMAT_CSC)
            op = op == ALPHA_SPARSE_OPERATION_NON_TRANSPOSE ? ALPHA_SPARSE_OPERATION_TRANSPOSE : ALPHA_SPARSE_OPERATION_NON_TRANSPOSE;
        s = csr_shadow_of(A, &A);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    }
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;

    DeviceGuard guard(c->device);
    if (!guard.ok) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    if (descr.type != ALPHA_SPARSE_MATRIX_TYPE_GENERAL) {
        s = select_structured<T>(c, A, op, descr, kDiagFirst);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    } else if (op == ALPHA_SPARSE_OPERATION_TRANSPOSE) {  // y (cols entries) = alpha * A^T * x (rows entries) + beta * y
        {
            std::lock_guard<std::mutex> build(c->mu);
            s = ensure_transposed<T>(c, static_cast<const typename CsrOf<T>::csr *>(A->mat));
            if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        }
        c = c->transposed;
    }
    return mv_on_ctx<T>(c, alpha, x, beta, y);
}

// Row-major mm with host X and host Y on a large dense block: X goes over first (every row of A may
// need any row of X), then the product runs in kPipelineChunks row windows and every finished window
// of Y leaves on its own stream while the next one is multiplied; when Y must come over first
// (beta != 0, or a padded ldy whose gaps belong to the caller) its windows arrive behind X on the
// inbound stream.  Same streams and events as the mv pipeline.
constexpr size_t kMmPipelineMinBytes = (size_t)32 << 20;

template <typename T>
static alphasparse_status_t mm_host_pipelined(DeviceCtx *c, T alpha, const T *x, int columns, int ldx, size_t xbytes,
                                              T beta, T *y, int ldy, size_t y_elems, bool y_in, cudaStream_t st) {
    alphasparse_status_t s = grow(&c->d_x_stage, &c->x_stage_bytes, xbytes, c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    s = grow(&c->d_y_stage, &c->y_stage_bytes, sizeof(T) * y_elems, c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    s = ensure_pipe(c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    const T *dx = static_cast<const T *>(c->d_x_stage);
    T *dy = static_cast<T *>(c->d_y_stage);
    cudaEvent_t ev_x = c->ev_pipe[0];
    ASB_CUDA_OR(cudaEventRecord(ev_x, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaStreamWaitEvent(c->copy_in, ev_x, 0), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaMemcpyAsync(c->d_x_stage, x, xbytes, cudaMemcpyHostToDevice, c->copy_in),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaEventRecord(ev_x, c->copy_in), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaStreamWaitEvent(st, ev_x, 0), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);

    const int64_t step = ((c->rows + kPipelineChunks - 1) / kPipelineChunks + 63) & ~63ll;
    for (int k = 0; k < kPipelineChunks; k++) {
        const int64_t rb = k * step;
        if (rb >= c->rows) break;
        const RowWindow w{rb, std::min<int64_t>(step, c->rows - rb)};
        const size_t e0 = (size_t)rb * (size_t)ldy, e1 = std::min((size_t)(rb + w.count) * (size_t)ldy, y_elems);
        cudaEvent_t ev_in = c->ev_pipe[1 + 2 * k], ev_done = c->ev_pipe[2 + 2 * k];
        if (y_in) {
            ASB_CUDA_OR(cudaMemcpyAsync(dy + e0, y + e0, sizeof(T) * (e1 - e0), cudaMemcpyHostToDevice, c->copy_in),
                        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            ASB_CUDA_OR(cudaEventRecord(ev_in, c->copy_in), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
            ASB_CUDA_OR(cudaStreamWaitEvent(st, ev_in, 0), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        }
        s = launch_spmm_row<T>(c, alpha, dx, columns, ldx, beta, dy, ldy, st, &w);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        ASB_CUDA_OR(cudaEventRecord(ev_done, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaStreamWaitEvent(c->copy_out, ev_done, 0), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaMemcpyAsync(y + e0, dy + e0, sizeof(T) * (e1 - e0), cudaMemcpyDeviceToHost, c->copy_out),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }
    ASB_CUDA_OR(cudaStreamSynchronize(c->copy_out), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Y = alpha * (matrix of c) * X + beta * Y for dense operands in host or device memory: the part of mm that no
// longer looks at the handle.
template <typename T>
static alphasparse_status_t mm_on_ctx(DeviceCtx *c, alphasparse_layout_t layout, T alpha, const T *x, ALPHA_INT columns,
                                      ALPHA_INT ldx, T beta, T *y, ALPHA_INT ldy) {
    alphasparse_status_t s = ALPHA_SPARSE_STATUS_SUCCESS;
    const bool row_major = layout == ALPHA_SPARSE_LAYOUT_ROW_MAJOR;
    // X is (c->cols x columns), Y is (c->rows x columns); ld = distance between rows (row-major) or
    // between columns (column-major)
    if (columns < 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (row_major ? (ldx < columns || ldy < columns) : (ldx < c->cols || ldy < c->rows))
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (c->rows == 0 || columns == 0) return ALPHA_SPARSE_STATUS_SUCCESS;

    cudaStream_t st = current_stream();
    const bool x_dev = is_device_pointer(x, c->device), y_dev = is_device_pointer(y, c->device);
    std::lock_guard<std::mutex> lock(c->mu);

    auto extent = [&](int64_t outer, int64_t inner, int64_t ld) -> size_t {  // elements spanned by a dense operand
        return outer > 0 && inner > 0 ? (size_t)((outer - 1) * ld + inner) : 0;
    };
    const size_t xbytes = sizeof(T) * (row_major ? extent(c->cols, columns, ldx) : extent(columns, c->cols, ldx));
    const size_t ybytes = sizeof(T) * (row_major ? extent(c->rows, columns, ldy) : extent(columns, c->rows, ldy));
    const bool y_tight = row_major ? ldy == columns : ldy == c->rows;
    if (row_major && !x_dev && !y_dev && !c->profile && xbytes > 0 && ybytes >= kMmPipelineMinBytes &&
        c->rows >= 64 * kPipelineChunks)
        return mm_host_pipelined<T>(c, alpha, x, columns, ldx, xbytes, beta, y, ldy, ybytes / sizeof(T),
                                    beta != T(0) || !y_tight, st);
    const T *dx = x;
    T *dy = y;
    if (!x_dev) {
        s = grow(&c->d_x_stage, &c->x_stage_bytes, xbytes ? xbytes : sizeof(T), c);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        if (xbytes)
            ASB_CUDA_OR(cudaMemcpyAsync(c->d_x_stage, x, xbytes, cudaMemcpyHostToDevice, st),
                        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        dx = static_cast<const T *>(c->d_x_stage);
    }
    if (!y_dev) {
        s = grow(&c->d_y_stage, &c->y_stage_bytes, ybytes, c);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        // Gaps left by a padded leading dimension belong to the caller and must survive the round
        // trip, so the whole block is brought over even when beta == 0.
        if (beta != T(0) || !y_tight)
            ASB_CUDA_OR(cudaMemcpyAsync(c->d_y_stage, y, ybytes, cudaMemcpyHostToDevice, st),
                        ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        dy = static_cast<T *>(c->d_y_stage);
    }
    s = row_major ? launch_spmm_row<T>(c, alpha, dx, columns, ldx, beta, dy, ldy, st)
                  : launch_spmm_col<T>(c, alpha, dx, columns, ldx, beta, dy, ldy, st);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    if (!y_dev)
        ASB_CUDA_OR(cudaMemcpyAsync(y, dy, ybytes, cudaMemcpyDeviceToHost, st),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    if (!y_dev || !x_dev)
        ASB_CUDA_OR(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template <typename T>
static alphasparse_status_t mm(alphasparse_operation_t op, T alpha, alphasparse_matrix_t A,
                               struct alpha_matrix_descr descr, alphasparse_layout_t layout,
                               const T *x, ALPHA_INT columns, ALPHA_INT ldx, T beta, T *y,
                               ALPHA_INT ldy) {
    alphasparse_status_t s = check_call(A, x, y, CsrOf<T>::dt, op, descr);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    if (layout != ALPHA_SPARSE_LAYOUT_ROW_MAJOR && layout != ALPHA_SPARSE_LAYOUT_COLUMN_MAJOR)
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (A->format != ALPHA_SPARSE_FORMAT_CSR) {
        if (A->format == ALPHA_SPARSE_FORMAT_CSC)  // held as the CSR of A^T (gemm_x_csc_{row,col}[_trans]_plain.c)
            op = op == ALPHA_SPARSE_OPERATION_NON_TRANSPOSE ? ALPHA_SPARSE_OPERATION_TRANSPOSE : ALPHA_SPARSE_OPERATION_NON_TRANSPOSE;
        s = csr_shadow_of(A, &A);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    }
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    DeviceGuard guard(c->device);
    if (!guard.ok) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    if (descr.type != ALPHA_SPARSE_MATRIX_TYPE_GENERAL) {
        s = select_structured<T>(c, A, op, descr, layout == ALPHA_SPARSE_LAYOUT_ROW_MAJOR ? kDiagAll : kDiagLast);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    } else if (op == ALPHA_SPARSE_OPERATION_TRANSPOSE) {  // the reference also multiplies by a materialised A^T
        {
            std::lock_guard<std::mutex> build(c->mu);
            s = ensure_transposed<T>(c, static_cast<const typename CsrOf<T>::csr *>(A->mat));
            if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        }
        c = c->transposed;
    }
    return mm_on_ctx<T>(c, layout, alpha, x, columns, ldx, beta, y, ldy);
}


// ---- kernel-level entry points ----------------------------------------------------------------------
// The symbols the reference's dispatch tables call for CSR + GENERAL (include/alphasparse/kernel/kernel_csr_s.h:13-17,
// 65-72 and kernel_csr_d.h of the reference; chosen per architecture by src/kernel/Makefile:2-11).  A `cuda` kernel
// tree beside plain / arm / hygon / dcu consists of these: they take the bare CSR record, find (or make) its device
// copy and run the same kernels as alphasparse_?_mv / _mm.

template <typename T>
static alphasparse_status_t ctx_for_record(const typename CsrOf<T>::csr *m, DeviceCtx **out) {
    {
        std::lock_guard<std::mutex> lock(g_registry_mu);
        auto it = registry().find(m);
        if (it != registry().end()) {
            *out = it->second.ctx;
            return ALPHA_SPARSE_STATUS_SUCCESS;
        }
    }
    // A record made elsewhere (the reference's own create_csr, src/core/format/alphasparse_x_create_csr.c:16-55,
    // in a build that links this library as its kernel tree): zero-based host arrays.  Upload and analyse it now.
    const int64_t rows = m->rows;
    if (rows < 0 || m->cols < 0 || (rows > 0 && (!m->rows_start || !m->rows_end))) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    std::vector<int> ptr;
    const int *offsets = m->rows_start;
    if (rows > 0 && m->rows_end != m->rows_start + 1) {  // four-array form: rows must still be contiguous
        ptr.resize((size_t)rows + 1);
        ptr[0] = m->rows_start[0];
        for (int64_t i = 0; i < rows; i++) {
            if (i + 1 < rows && m->rows_end[i] != m->rows_start[i + 1]) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
            ptr[(size_t)i + 1] = m->rows_end[i];
        }
        offsets = ptr.data();
    }
    if (rows > 0 && offsets[0] != 0) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    static const int zero = 0;
    DeviceCtx *c = nullptr;
    alphasparse_status_t s = ctx_create(CsrOf<T>::dt, rows, m->cols, rows > 0 ? offsets : &zero, m->col_indx, m->values, &c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    {
        std::lock_guard<std::mutex> lock(g_registry_mu);
        auto it = registry().find(m);
        if (it != registry().end()) {  // another thread was faster
            ctx_destroy(c);
            c = it->second.ctx;
        } else {
            registry()[m] = RegistryEntry{c, true};
        }
    }
    *out = c;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template <typename T>
static alphasparse_status_t kernel_mv(const typename CsrOf<T>::csr *A, bool trans, T alpha, const T *x, T beta, T *y) {
    if (!A || !x || !y) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    DeviceCtx *c = nullptr;
    alphasparse_status_t s = ctx_for_record<T>(A, &c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    DeviceGuard guard(c->device);
    if (!guard.ok) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    if (trans) {
        std::lock_guard<std::mutex> build(c->mu);
        s = ensure_transposed<T>(c, A);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        c = c->transposed;
    }
    return mv_on_ctx<T>(c, alpha, x, beta, y);
}

template <typename T>
static alphasparse_status_t kernel_mm(const typename CsrOf<T>::csr *A, bool trans, alphasparse_layout_t layout, T alpha,
                                      const T *x, ALPHA_INT columns, ALPHA_INT ldx, T beta, T *y, ALPHA_INT ldy) {
    if (!A || !x || !y) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    DeviceCtx *c = nullptr;
    alphasparse_status_t s = ctx_for_record<T>(A, &c);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    DeviceGuard guard(c->device);
    if (!guard.ok) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    if (trans) {
        std::lock_guard<std::mutex> build(c->mu);
        s = ensure_transposed<T>(c, A);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        c = c->transposed;
    }
    return mm_on_ctx<T>(c, layout, alpha, x, columns, ldx, beta, y, ldy);
}

}  // namespace asb

// =============================================================================================
// C ABI
// =============================================================================================
using namespace asb;

extern "C" {

alphasparse_status_t alphasparse_s_create_csr(alphasparse_matrix_t *A, const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols, ALPHA_INT *rows_start,
                                              ALPHA_INT *rows_end, ALPHA_INT *col_indx, float *values) {
    return create_csr<float>(A, indexing, rows, cols, rows_start, rows_end, col_indx, values);
}
alphasparse_status_t alphasparse_d_create_csr(alphasparse_matrix_t *A, const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols, ALPHA_INT *rows_start,
                                              ALPHA_INT *rows_end, ALPHA_INT *col_indx, double *values) {
    return create_csr<double>(A, indexing, rows, cols, rows_start, rows_end, col_indx, values);
}
alphasparse_status_t alphasparse_c_create_csr(alphasparse_matrix_t *A, const alphasparse_index_base_t,
                                              const ALPHA_INT, const ALPHA_INT, ALPHA_INT *, ALPHA_INT *,
                                              ALPHA_INT *, ALPHA_Complex8 *) {
    if (A) *A = nullptr;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}
alphasparse_status_t alphasparse_z_create_csr(alphasparse_matrix_t *A, const alphasparse_index_base_t,
                                              const ALPHA_INT, const ALPHA_INT, ALPHA_INT *, ALPHA_INT *,
                                              ALPHA_INT *, ALPHA_Complex16 *) {
    if (A) *A = nullptr;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}

alphasparse_status_t alphasparse_s_create_csc(alphasparse_matrix_t *A, const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols, ALPHA_INT *cols_start,
                                              ALPHA_INT *cols_end, ALPHA_INT *row_indx, float *values) {
    return create_csc<float>(A, indexing, rows, cols, cols_start, cols_end, row_indx, values);
}
alphasparse_status_t alphasparse_d_create_csc(alphasparse_matrix_t *A, const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols, ALPHA_INT *cols_start,
                                              ALPHA_INT *cols_end, ALPHA_INT *row_indx, double *values) {
    return create_csc<double>(A, indexing, rows, cols, cols_start, cols_end, row_indx, values);
}
alphasparse_status_t alphasparse_c_create_csc(alphasparse_matrix_t *A, const alphasparse_index_base_t,
                                              const ALPHA_INT, const ALPHA_INT, ALPHA_INT *, ALPHA_INT *,
                                              ALPHA_INT *, ALPHA_Complex8 *) {
    if (A) *A = nullptr;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}
alphasparse_status_t alphasparse_z_create_csc(alphasparse_matrix_t *A, const alphasparse_index_base_t,
                                              const ALPHA_INT, const ALPHA_INT, ALPHA_INT *, ALPHA_INT *,
                                              ALPHA_INT *, ALPHA_Complex16 *) {
    if (A) *A = nullptr;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}

alphasparse_status_t alphasparse_s_create_coo(alphasparse_matrix_t *A, const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols, const ALPHA_INT nnz,
                                              ALPHA_INT *row_indx, ALPHA_INT *col_indx, float *values) {
    return create_coo<float>(A, indexing, rows, cols, nnz, row_indx, col_indx, values);
}
alphasparse_status_t alphasparse_d_create_coo(alphasparse_matrix_t *A, const alphasparse_index_base_t indexing,
                                              const ALPHA_INT rows, const ALPHA_INT cols, const ALPHA_INT nnz,
                                              ALPHA_INT *row_indx, ALPHA_INT *col_indx, double *values) {
    return create_coo<double>(A, indexing, rows, cols, nnz, row_indx, col_indx, values);
}
alphasparse_status_t alphasparse_c_create_coo(alphasparse_matrix_t *A, const alphasparse_index_base_t,
                                              const ALPHA_INT, const ALPHA_INT, const ALPHA_INT, ALPHA_INT *,
                                              ALPHA_INT *, ALPHA_Complex8 *) {
    if (A) *A = nullptr;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}
alphasparse_status_t alphasparse_z_create_coo(alphasparse_matrix_t *A, const alphasparse_index_base_t,
                                              const ALPHA_INT, const ALPHA_INT, const ALPHA_INT, ALPHA_INT *,
                                              ALPHA_INT *, ALPHA_Complex16 *) {
    if (A) *A = nullptr;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}

// Reference: src/core/op_/alphasparse_destroy.c:186-195 (NULL handle is SUCCESS).  Unlike the
// reference, whose alpha_free releases nothing, host and device storage is really returned.
alphasparse_status_t alphasparse_destroy(alphasparse_matrix_t A) {
    if (!A) return ALPHA_SPARSE_STATUS_SUCCESS;
    if (A->mat && A->format == ALPHA_SPARSE_FORMAT_CSR) registry_take(A->mat);
    ctx_destroy(ctx_of(A));
    A->dcu_info = nullptr;
    if (A->mat) {
        if (A->format == ALPHA_SPARSE_FORMAT_CSR) {
            if (A->datatype == ALPHA_SPARSE_DATATYPE_FLOAT) free_csr_host<float>(static_cast<spmat_csr_s_t *>(A->mat));
            else if (A->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE) free_csr_host<double>(static_cast<spmat_csr_d_t *>(A->mat));
        } else if (A->format == ALPHA_SPARSE_FORMAT_CSC) {
            alphasparse_destroy(static_cast<alphasparse_matrix_t>(A->inspector));  // owns the arrays the record borrows
            A->inspector = nullptr;
            free(A->mat);
        } else if (A->format == ALPHA_SPARSE_FORMAT_COO) {
            alphasparse_destroy(static_cast<alphasparse_matrix_t>(A->inspector));  // the CSR copy mv / mm made, if any
            A->inspector = nullptr;
            spmat_coo_s_t *m = static_cast<spmat_coo_s_t *>(A->mat);  // pointer fields first in both precisions
            free(m->values), free(m->row_indx), free(m->col_indx), free(m);
        }
    }
    free(A);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Reference: src/core/op_/alphasparse_convert_csr.c:125-157 (+ :100-123: only a COO source).
alphasparse_status_t alphasparse_convert_csr(const alphasparse_matrix_t source, const alphasparse_operation_t operation,
                                             alphasparse_matrix_t *dest) {
    if (!source || !source->mat) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (!dest) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    *dest = nullptr;
    if (operation == ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    if (operation != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE && operation != ALPHA_SPARSE_OPERATION_TRANSPOSE)
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (source->format != ALPHA_SPARSE_FORMAT_COO) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    const bool tr = operation == ALPHA_SPARSE_OPERATION_TRANSPOSE;
    if (source->datatype == ALPHA_SPARSE_DATATYPE_FLOAT)
        return coo_to_csr<float>(static_cast<const spmat_coo_s_t *>(source->mat), tr, dest);
    if (source->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE)
        return coo_to_csr<double>(static_cast<const spmat_coo_d_t *>(source->mat), tr, dest);
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}

// Reference: src/core/format/alphasparse_x_export_csr.c:5-25.
#define ASB_EXPORT(T, sfx, DT)                                                                              \
    alphasparse_status_t alphasparse_##sfx##_export_csr(                                                    \
        const alphasparse_matrix_t source, alphasparse_index_base_t *indexing, ALPHA_INT *rows,             \
        ALPHA_INT *cols, ALPHA_INT **rows_start, ALPHA_INT **rows_end, ALPHA_INT **col_indx, T **values) {  \
        if (!source) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;                                            \
        if (!source->mat) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;                                         \
        if (source->datatype != DT) return ALPHA_SPARSE_STATUS_INVALID_VALUE;                               \
        if (source->format != ALPHA_SPARSE_FORMAT_CSR) return ALPHA_SPARSE_STATUS_INVALID_VALUE;            \
        spmat_csr_##sfx##_t *m = static_cast<spmat_csr_##sfx##_t *>(source->mat);                           \
        *indexing = ALPHA_SPARSE_INDEX_BASE_ZERO;                                                           \
        *rows = m->rows, *cols = m->cols;                                                                   \
        *rows_start = m->rows_start, *rows_end = m->rows_end;                                               \
        *col_indx = m->col_indx, *values = m->values;                                                       \
        return ALPHA_SPARSE_STATUS_SUCCESS;                                                                 \
    }
ASB_EXPORT(float, s, ALPHA_SPARSE_DATATYPE_FLOAT)
ASB_EXPORT(double, d, ALPHA_SPARSE_DATATYPE_DOUBLE)

// Reference: src/core/format/alphasparse_x_export_csc.c:5-25.
#define ASB_EXPORT_CSC(T, sfx, DT)                                                                          \
    alphasparse_status_t alphasparse_##sfx##_export_csc(                                                    \
        const alphasparse_matrix_t source, alphasparse_index_base_t *indexing, ALPHA_INT *rows,             \
        ALPHA_INT *cols, ALPHA_INT **cols_start, ALPHA_INT **cols_end, ALPHA_INT **row_indx, T **values) {  \
        if (!source) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;                                            \
        if (!source->mat) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;                                         \
        if (source->datatype != DT) return ALPHA_SPARSE_STATUS_INVALID_VALUE;                               \
        if (source->format != ALPHA_SPARSE_FORMAT_CSC) return ALPHA_SPARSE_STATUS_INVALID_VALUE;            \
        spmat_csc_##sfx##_t *m = static_cast<spmat_csc_##sfx##_t *>(source->mat);                           \
        *indexing = ALPHA_SPARSE_INDEX_BASE_ZERO;                                                           \
        *rows = m->rows, *cols = m->cols;                                                                   \
        *cols_start = m->cols_start, *cols_end = m->cols_end;                                               \
        *row_indx = m->row_indx, *values = m->values;                                                       \
        return ALPHA_SPARSE_STATUS_SUCCESS;                                                                 \
    }
ASB_EXPORT_CSC(float, s, ALPHA_SPARSE_DATATYPE_FLOAT)
ASB_EXPORT_CSC(double, d, ALPHA_SPARSE_DATATYPE_DOUBLE)

// Reference: src/core/op_/alphasparse_convert_csc.c:101-150 (only a COO source) ->
// src/core/format/convert_csc_x_coo.c.  CSC of op(A) = CSR arrays of op(A)^T: the COO->CSR conversion
// with the opposite transposition, wrapped.
alphasparse_status_t alphasparse_convert_csc(const alphasparse_matrix_t source, const alphasparse_operation_t operation,
                                             alphasparse_matrix_t *dest) {
    if (!source || !source->mat) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (!dest) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    *dest = nullptr;
    if (operation == ALPHA_SPARSE_OPERATION_CONJUGATE_TRANSPOSE) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    if (operation != ALPHA_SPARSE_OPERATION_NON_TRANSPOSE && operation != ALPHA_SPARSE_OPERATION_TRANSPOSE)
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (source->format != ALPHA_SPARSE_FORMAT_COO) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    const bool tr = operation == ALPHA_SPARSE_OPERATION_TRANSPOSE;
    alphasparse_matrix_t t = nullptr;
    alphasparse_status_t s = ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    if (source->datatype == ALPHA_SPARSE_DATATYPE_FLOAT)
        s = coo_to_csr<float>(static_cast<const spmat_coo_s_t *>(source->mat), !tr, &t);
    else if (source->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE)
        s = coo_to_csr<double>(static_cast<const spmat_coo_d_t *>(source->mat), !tr, &t);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    return source->datatype == ALPHA_SPARSE_DATATYPE_FLOAT ? wrap_as_csc<float>(t, dest) : wrap_as_csc<double>(t, dest);
}

alphasparse_status_t alphasparse_set_mv_hint(const alphasparse_matrix_t A, const alphasparse_operation_t,
                                             const struct alpha_matrix_descr, const ALPHA_INT) {
    return A ? ALPHA_SPARSE_STATUS_SUCCESS : ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
}

alphasparse_status_t alphasparse_optimize(alphasparse_matrix_t A) {
    if (!A || !A->mat) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (A->format == ALPHA_SPARSE_FORMAT_COO || (A->format == ALPHA_SPARSE_FORMAT_CSC && A->inspector)) {
        // builds (or re-analyses) the CSR handle that mv / mm use for this matrix
        alphasparse_status_t s = csr_shadow_of(A, &A);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    }
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
    DeviceGuard guard(c->device);
    if (!guard.ok) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    std::lock_guard<std::mutex> lock(c->mu);
    return ctx_analyse(c);
}

alphasparse_status_t alphasparse_s_mv(const alphasparse_operation_t operation, const float alpha,
                                      const alphasparse_matrix_t A, const struct alpha_matrix_descr descr,
                                      const float *x, const float beta, float *y) {
    return mv<float>(operation, alpha, A, descr, x, beta, y);
}
alphasparse_status_t alphasparse_d_mv(const alphasparse_operation_t operation, const double alpha,
                                      const alphasparse_matrix_t A, const struct alpha_matrix_descr descr,
                                      const double *x, const double beta, double *y) {
    return mv<double>(operation, alpha, A, descr, x, beta, y);
}
alphasparse_status_t alphasparse_c_mv(const alphasparse_operation_t, const ALPHA_Complex8, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr, const ALPHA_Complex8 *x, const ALPHA_Complex8,
                                      ALPHA_Complex8 *y) {
    if (!A || !A->mat || !x || !y) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (A->datatype != ALPHA_SPARSE_DATATYPE_FLOAT_COMPLEX) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}
alphasparse_status_t alphasparse_z_mv(const alphasparse_operation_t, const ALPHA_Complex16, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr, const ALPHA_Complex16 *x, const ALPHA_Complex16,
                                      ALPHA_Complex16 *y) {
    if (!A || !A->mat || !x || !y) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (A->datatype != ALPHA_SPARSE_DATATYPE_DOUBLE_COMPLEX) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}

alphasparse_status_t alphasparse_s_mm(const alphasparse_operation_t operation, const float alpha,
                                      const alphasparse_matrix_t A, const struct alpha_matrix_descr descr,
                                      const alphasparse_layout_t layout, const float *x, const ALPHA_INT columns,
                                      const ALPHA_INT ldx, const float beta, float *y, const ALPHA_INT ldy) {
    return mm<float>(operation, alpha, A, descr, layout, x, columns, ldx, beta, y, ldy);
}
alphasparse_status_t alphasparse_d_mm(const alphasparse_operation_t operation, const double alpha,
                                      const alphasparse_matrix_t A, const struct alpha_matrix_descr descr,
                                      const alphasparse_layout_t layout, const double *x, const ALPHA_INT columns,
                                      const ALPHA_INT ldx, const double beta, double *y, const ALPHA_INT ldy) {
    return mm<double>(operation, alpha, A, descr, layout, x, columns, ldx, beta, y, ldy);
}
alphasparse_status_t alphasparse_c_mm(const alphasparse_operation_t, const ALPHA_Complex8, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr, const alphasparse_layout_t, const ALPHA_Complex8 *x,
                                      const ALPHA_INT, const ALPHA_INT, const ALPHA_Complex8, ALPHA_Complex8 *y,
                                      const ALPHA_INT) {
    if (!A || !A->mat || !x || !y) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (A->datatype != ALPHA_SPARSE_DATATYPE_FLOAT_COMPLEX) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}
alphasparse_status_t alphasparse_z_mm(const alphasparse_operation_t, const ALPHA_Complex16, const alphasparse_matrix_t A,
                                      const struct alpha_matrix_descr, const alphasparse_layout_t, const ALPHA_Complex16 *x,
                                      const ALPHA_INT, const ALPHA_INT, const ALPHA_Complex16, ALPHA_Complex16 *y,
                                      const ALPHA_INT) {
    if (!A || !A->mat || !x || !y) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    if (A->datatype != ALPHA_SPARSE_DATATYPE_DOUBLE_COMPLEX) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    return ALPHA_SPARSE_STATUS_NOT_SUPPORTED;
}


// ---- kernel-level symbols (include/alphasparse/kernel_cuda.h) -------------------------------------------

#define ASB_KERNEL_SYMBOLS(T, sfx)                                                                                  \
    alphasparse_status_t gemv_##sfx##_csr(const T alpha, const spmat_csr_##sfx##_t *A, const T *x, const T beta,   \
                                          T *y) {                                                                   \
        return kernel_mv<T>(A, false, alpha, x, beta, y);                                                           \
    }                                                                                                               \
    alphasparse_status_t gemv_##sfx##_csr_trans(const T alpha, const spmat_csr_##sfx##_t *A, const T *x,           \
                                                const T beta, T *y) {                                               \
        return kernel_mv<T>(A, true, alpha, x, beta, y);                                                            \
    }                                                                                                               \
    alphasparse_status_t gemm_##sfx##_csr_row(const T alpha, const spmat_csr_##sfx##_t *mat, const T *x,           \
                                              const ALPHA_INT columns, const ALPHA_INT ldx, const T beta, T *y,     \
                                              const ALPHA_INT ldy) {                                                \
        return kernel_mm<T>(mat, false, ALPHA_SPARSE_LAYOUT_ROW_MAJOR, alpha, x, columns, ldx, beta, y, ldy);       \
    }                                                                                                               \
    alphasparse_status_t gemm_##sfx##_csr_col(const T alpha, const spmat_csr_##sfx##_t *mat, const T *x,           \
                                              const ALPHA_INT columns, const ALPHA_INT ldx, const T beta, T *y,     \
                                              const ALPHA_INT ldy) {                                                \
        return kernel_mm<T>(mat, false, ALPHA_SPARSE_LAYOUT_COLUMN_MAJOR, alpha, x, columns, ldx, beta, y, ldy);    \
    }                                                                                                               \
    alphasparse_status_t gemm_##sfx##_csr_row_trans(const T alpha, const spmat_csr_##sfx##_t *mat, const T *x,     \
                                                    const ALPHA_INT columns, const ALPHA_INT ldx, const T beta,     \
                                                    T *y, const ALPHA_INT ldy) {                                    \
        return kernel_mm<T>(mat, true, ALPHA_SPARSE_LAYOUT_ROW_MAJOR, alpha, x, columns, ldx, beta, y, ldy);        \
    }                                                                                                               \
    alphasparse_status_t gemm_##sfx##_csr_col_trans(const T alpha, const spmat_csr_##sfx##_t *mat, const T *x,     \
                                                    const ALPHA_INT columns, const ALPHA_INT ldx, const T beta,     \
                                                    T *y, const ALPHA_INT ldy) {                                    \
        return kernel_mm<T>(mat, true, ALPHA_SPARSE_LAYOUT_COLUMN_MAJOR, alpha, x, columns, ldx, beta, y, ldy);     \
    }
ASB_KERNEL_SYMBOLS(float, s)
ASB_KERNEL_SYMBOLS(double, d)

alphasparse_status_t alphasparse_cuda_release_csr(const void *record) {
    if (!record) return ALPHA_SPARSE_STATUS_SUCCESS;
    RegistryEntry e = registry_take(record);
    if (!e.ctx) return ALPHA_SPARSE_STATUS_SUCCESS;
    if (!e.adopted) {  // belongs to a live handle of this library: alphasparse_destroy releases it
        registry_add(record, e.ctx, false);
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    }
    ctx_destroy(e.ctx);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// ---- additions (include/alphasparse/spapi_cuda.h) ---------------------------------------------

alphasparse_status_t alphasparse_cuda_set_stream(void *stream) {
    g_stream.store(static_cast<cudaStream_t>(stream), std::memory_order_relaxed);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_get_stream(void **stream) {
    if (!stream) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    *stream = current_stream();
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_synchronize(void) {
    ASB_CUDA_OR(cudaStreamSynchronize(current_stream()), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_set_algorithm(alphasparse_cuda_alg_t alg) {
    if (alg < ALPHA_SPARSE_CUDA_ALG_AUTO || alg > ALPHA_SPARSE_CUDA_ALG_ROWTILE) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    g_alg.store((int)alg, std::memory_order_relaxed);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_set_option(const char *name, int64_t value) {
    if (!name) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    options_init();
    const int i = option_index(name, strlen(name));
    if (i < 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    g_options[i].store(value < 0 ? kOptionDefs[i].def : value, std::memory_order_relaxed);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_get_option(const char *name, int64_t *value) {
    if (!name || !value) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    options_init();
    const int i = option_index(name, strlen(name));
    if (i < 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    *value = g_options[i].load(std::memory_order_relaxed);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_get_mat_info(const alphasparse_matrix_t A, alphasparse_cuda_mat_info_t *info) {
    if (!info) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    memset(info, 0, sizeof(*info));
    info->rows = c->rows, info->cols = c->cols, info->nnz = c->nnz;
    info->max_row_nnz = c->max_row_nnz, info->empty_rows = c->empty_rows;
    info->mean_row_nnz = c->mean_row_nnz;
    info->algorithm = c->algorithm, info->lanes_per_row = c->lanes;
    info->merge_tiles = c->algorithm == ALPHA_SPARSE_CUDA_ALG_MERGE ? c->merge_tiles : 0;
    info->device_bytes = c->device_bytes, info->device = c->device;
    info->scheduled = c->d_sched != nullptr;
    info->band_rows = c->band.rows, info->band_count = c->band.bands, info->band_width = c->band.width;
    info->band_elements = c->band.elements;
    info->spmm_col_blocks = c->spmm.d_split ? c->spmm.blocks : (c->spmm.blocks ? 1 : 0);
    info->binned = c->bins.active ? 1 : 0;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_get_device_csr(const alphasparse_matrix_t A, ALPHA_INT **d_row_ptr,
                                                     ALPHA_INT **d_col_indx, void **d_values) {
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    if (d_row_ptr) *d_row_ptr = c->d_row_ptr;
    if (d_col_indx) *d_col_indx = c->d_col;
    if (d_values) *d_values = c->d_val;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_kernel_status(const alphasparse_matrix_t A, int *status, int clear) {
    if (!status) return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    DeviceGuard guard(c->device);
    if (!guard.ok) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    std::lock_guard<std::mutex> lock(c->mu);
    cudaStream_t st = current_stream();
    int worst = 0;
    // the handle's own word and those of the matrices derived from it (A^T, structured variants)
    DeviceCtx *all[2 + 24] = {c, c->transposed};
    for (int i = 0; i < 24; i++) all[2 + i] = c->derived[i];
    for (DeviceCtx *d : all) {
        if (!d) continue;
        int code = 0;
        ASB_CUDA_OR(cudaMemcpyAsync(&code, d->d_status, sizeof(int), cudaMemcpyDeviceToHost, st),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        ASB_CUDA_OR(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        if (code != 0 && worst == 0) worst = code;
        if (clear && code != 0)
            ASB_CUDA_OR(cudaMemsetAsync(d->d_status, 0, sizeof(int), st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    }
    *status = worst;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_profile_kernel(const alphasparse_matrix_t A, int enable) {
    DeviceCtx *c = ctx_of(A);
    if (!c) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    DeviceGuard guard(c->device);
    if (!guard.ok) return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    std::lock_guard<std::mutex> lock(c->mu);
    if (enable && !c->ev_start) {
        ASB_CUDA_OR(cudaEventCreate(&c->ev_start), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
        ASB_CUDA_OR(cudaEventCreate(&c->ev_stop), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    }
    c->profile = enable != 0;
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_kernel_ms(const alphasparse_matrix_t A, float *ms) {
    DeviceCtx *c = ctx_of(A);
    if (!c || !ms) return ALPHA_SPARSE_STATUS_INVALID_HANDLE;
    if (!c->ev_start) return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    ASB_CUDA_OR(cudaEventSynchronize(c->ev_stop), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaEventElapsedTime(ms, c->ev_start, c->ev_stop), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
alphasparse_status_t alphasparse_cuda_debug_fail_alloc(int64_t nth) {
    g_fail_alloc_in.store(nth > 0 ? nth : 0, std::memory_order_relaxed);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
int64_t alphasparse_cuda_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char *alphasparse_cuda_last_error(void) { return t_error; }

}  // extern "C"
