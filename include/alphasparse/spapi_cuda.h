#pragma once
/*
 * Additions of the sm_100a backend.  Nothing here is needed for drop-in use of the
 * entry points in spapi.h; a caller that keeps vectors on the device, wants its own
 * stream, or wants to look at what the one-time analysis decided uses these.  They follow
 * the precedent of the reference's device API (include/alphasparse/spapi_dcu.h: device
 * pointers, an explicit stream on the handle, a per-matrix analysis object), not its form.
 */
#include "types.h"
#include "spdef.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Kernels of later mv / mm calls are enqueued on `stream` (a cudaStream_t); NULL restores
 * the default stream.  Process-wide; set it before the calls it should affect. */
alphasparse_status_t alphasparse_cuda_set_stream(void *stream);
alphasparse_status_t alphasparse_cuda_get_stream(void **stream);

/* Blocks until everything enqueued on the library stream has finished. */
alphasparse_status_t alphasparse_cuda_synchronize(void);

typedef enum {
    ALPHA_SPARSE_CUDA_ALG_AUTO = 0,   /* chosen per matrix by the analysis */
    ALPHA_SPARSE_CUDA_ALG_VECTOR = 1, /* a group of 2..32 lanes per row */
    ALPHA_SPARSE_CUDA_ALG_MERGE = 2,  /* merge-path tiles: equal rows+nnz per thread block */
    ALPHA_SPARSE_CUDA_ALG_ROWTILE = 3 /* 128-row tiles staged in shared memory by bulk copies,
                                         one thread per row (falls back when a tile is too large) */
} alphasparse_cuda_alg_t;

/* Forces the SpMV kernel family for handles analysed after the call (A/B measurements);
 * the environment variable ALPHASPARSE_CUDA_ALG=auto|vector|merge|rowtile sets the initial value.
 * ALPHASPARSE_CUDA_NO_SCHEDULE=1 keeps the merge kernel's blocks in natural tile order (see
 * alphasparse_cuda_mat_info_t.scheduled). */
alphasparse_status_t alphasparse_cuda_set_algorithm(alphasparse_cuda_alg_t alg);

/* Tuning values read by the analysis of handles created (or re-analysed by alphasparse_optimize) after the
 * call; a negative value restores the default.  ALPHASPARSE_CUDA_OPTIONS="name=value,..." sets initial values.
 *   band_enable (1)         long rows of a skewed matrix go through the column-band kernel
 *   band_bytes (65536)      bytes of x one column band stages in shared memory
 *   band_min_seg (12)       a row is long when it averages at least this many elements per band
 *   band_min_rows (128)     fewer long rows than this are left to the merge kernel
 *   band_min_share_pct (10) ... and so are long rows holding less than this share of the elements
 *   band_splits (0)         thread blocks per band, 0 = about eight waves of blocks
 *   band_overlap (0)        1: the column-band kernel runs on a second stream beside the other kernels
 *   band_packed (1)         the band kernel streams a packed band-major copy of the long rows (columns relative to
 *                           the band in 16 bits, segments padded to quads): (sizeof(T) + 2) bytes of device
 *                           memory per long-row element; 0 = read the CSR arrays
 *   band_variant (0)        shape of the column-band kernel (lanes x quads in flight x segments per lane group):
 *                           packed copy 0 = 8 x 2 x 1, 1 = 8 x 2 x 2; CSR arrays 0 = 8 x 1 x 2, 1 = 4 x 2 x 1
 *   bin_overlap (1)         the kernels of the mid bins run on streams of their own, side by side
 *   bin_enable (1)          skewed matrices are multiplied bin by bin: thread per row up to bin_short (16)
 *                           elements, a lane group (4 / 16 / 32 lanes for rows up to bin_mid0 (32) / bin_mid1 (256) /
 *                           longer) per row above, the column-band kernel for long rows; merge
 *                           tiles remain for matrices with rows above bin_mid_max (16384; eight times that when the band
 *                           kernel's own threshold lies higher, as it does for wide matrices) that are not long
 *                           enough for the band kernel, with too few long rows, or with unsorted long rows
 *   bin_sort (1)            the two lists of rows above bin_mid0 elements are ordered longest row first, so that the
 *                           rows of one thread block are of about one length; 0 = row order
 *   bin_push_max_peers (4)  exchange calls (alphasparse_?_mv_exchange) over more GPUs than this run over merge tiles,
 *                           whose chunk-wise delivery spreads the NVLink traffic, instead of bins (measured: bins
 *                           0.49 against 0.53 ms per iteration at 4 GPUs, 0.47 against 0.32 ms at 8)
 *   pipe_max_windows (12)   mv with host vectors: the product runs in up to this many row windows (at most 16) that
 *                           overlap the copies of y, each window covering at least pipe_min_piece_kb (4096) KB of y
 *   mv_block_min_kb (98304) vector-kernel SpMV: when x is larger than this many KB (it no longer fits L2) the product runs
 *                           column block by column block, each block covering at most mv_block_kb (65536) KB of
 *                           x, the first launch applying beta and the later ones adding to y; needs rows in
 *                           ascending column order; 0 = never
 *   spmm_col_via_row (2)    column-major dense blocks of at least this many columns are transposed into row-major copies
 *                           kept with the handle (X, and Y when beta != 0), multiplied by the row-major kernels
 *                           and transposed back: device memory for one more X and Y; 0 = never
 *   spmm_narrow (1)         row-major dense blocks whose rows take at most 32 bytes (8 fp32 / 4 fp64 columns) go through
 *                           a kernel whose lanes split the elements of a sparse row instead of the dense columns
 *   spmm_split_min (1024)   row-major dense-block product on a matrix whose longest row exceeds eight times the mean:
 *                           a row above this many elements is multiplied chunk by chunk (spmm_split_chunk (512)
 *                           elements per chunk, partial sums added in chunk order), so that one lane group does
 *                           not walk a hundred thousand elements alone; 0 = never
 *   spmm_col_blocks (0)     row-major dense-block product in this many column blocks (X slab by slab, Y
 *                           accumulated over the passes); 0 or 1 = one pass, which measured faster on B200
 * Unknown names return ALPHA_SPARSE_STATUS_INVALID_VALUE. */
alphasparse_status_t alphasparse_cuda_set_option(const char *name, int64_t value);
alphasparse_status_t alphasparse_cuda_get_option(const char *name, int64_t *value);

/* What the analysis at handle creation found and chose. */
typedef struct {
    int64_t rows, cols, nnz;
    int64_t max_row_nnz;
    int64_t empty_rows;
    double mean_row_nnz;
    int32_t algorithm;     /* alphasparse_cuda_alg_t actually used by mv */
    int32_t lanes_per_row; /* vector kernel: lanes cooperating on one row */
    int64_t merge_tiles;   /* merge kernel: thread blocks per call */
    int64_t device_bytes;  /* device memory held by the handle */
    int32_t device;        /* CUDA device ordinal that owns the device copy */
    int32_t scheduled;     /* merge kernel: 1 when its blocks follow a schedule (column order for large x, and / or
                              without the tiles the column-band kernel covers) */
    int32_t band_rows;     /* long rows handled by the column-band kernel (0: none) */
    int32_t band_count;    /* column bands of band_width columns each */
    int32_t band_width;
    int64_t band_elements; /* stored elements the column-band kernel multiplies */
    int32_t spmm_col_blocks; /* column blocks the last row-major mm call on this handle ran in (0: none yet) */
    int32_t binned;          /* 1: products of this handle run bin by bin (thread per short row, lane group per mid
                                row, column-band kernel for long rows) instead of over merge tiles */
} alphasparse_cuda_mat_info_t;

alphasparse_status_t alphasparse_cuda_get_mat_info(const alphasparse_matrix_t A,
                                                   alphasparse_cuda_mat_info_t *info);

/* Borrowed device pointers of the handle's CSR copy (rows+1 offsets, nnz columns, nnz
 * values of the handle's precision). */
alphasparse_status_t alphasparse_cuda_get_device_csr(const alphasparse_matrix_t A,
                                                     ALPHA_INT **d_row_ptr,
                                                     ALPHA_INT **d_col_indx, void **d_values);

/* y = alpha*A*x + beta*y (double precision, general CSR, non-transposed) on caller-owned
 * DEVICE arrays, with a guarantee: the call never allocates or frees memory, on the device or
 * through any library.  No counterpart in the reference; it exists for callers that cannot
 * allocate at call time -- code running inside a framework whose memory pool already owns the
 * device (a cudaMalloc from a second library fails there even though the pool has room), or a
 * service that cannot tolerate the device-wide synchronisation cudaMalloc / cudaFree carry.
 *
 * d_row_ptr has rows+1 zero-based offsets, d_col_indx / d_values have nnz entries, d_x has cols
 * and d_y rows entries; all five live on the current device (memory of another GPU is refused with
 * ALPHA_SPARSE_STATUS_INVALID_POINTER).  Work is enqueued on the library stream and the call returns
 * without waiting.
 *
 * The matrix is taken as it is: offsets must be non-decreasing and every column index must lie in
 * [0, cols).  Unlike handle creation, which checks both once and refuses a bad matrix, this call does
 * NOT validate them (it would have to read the whole index array on every product): an index outside
 * the range reads outside d_x.  Validate untrusted matrices by creating a handle from them once.
 *
 * Scratch (the merge-path tile table and carries that a handle would own) comes from one fixed
 * 4 MiB array inside the library image, present on every GPU that loads the library until the
 * process exits.  Consequences:
 *   - rows + nnz may not exceed 375,802,112; larger problems return
 *     ALPHA_SPARSE_STATUS_INVALID_VALUE (text via alphasparse_cuda_last_error): create a handle
 *     and use alphasparse_d_mv instead;
 *   - all calls share the array and find the previous call's data in it; each call clears what
 *     it relies on.  Two calls that overlap on the GPU (different streams, different host
 *     threads without ordering) race on it: keep calls on one device in stream order;
 *   - the first call on each device looks up the array's device address (no allocation, but a
 *     runtime query): make that first call before starting any stream capture. */
alphasparse_status_t alphasparse_cuda_d_csrmv_noalloc(ALPHA_INT rows, ALPHA_INT cols, ALPHA_INT nnz,
                                                      double alpha, const ALPHA_INT *d_row_ptr,
                                                      const ALPHA_INT *d_col_indx,
                                                      const double *d_values, const double *d_x,
                                                      double beta, double *d_y);

/* ---- iterated SpMV over the GPUs of one box (one process per GPU) -----------------------------
 * No counterpart in the reference (it has no multi-device path).  A square matrix is split into
 * contiguous row blocks by balanced_partition_row_by_nnz; rank g creates an ordinary handle from its
 * block (local offsets, global columns).  An exchange object holds two full-length x buffers per GPU.
 * alphasparse_?_mv_exchange computes y = alpha*A_block*x + beta*y with x = the current buffer and, in
 * the same kernels, stores every finished y row into the NEXT x buffer of every GPU over NVLink
 * (peer-mapped pointers); it then signals and awaits all peers (bounded wait) and the buffers swap.
 * After the call the current x is the gathered y of all ranks.  Every rank must make the same sequence
 * of calls.  Set-up: create on every rank, export the 192-byte blob, exchange the blobs by any means
 * (e.g. an allgather of bytes), connect with all blobs in rank order. */
typedef struct alphasparse_cuda_exchange *alphasparse_cuda_exchange_t;

alphasparse_status_t alphasparse_cuda_exchange_create(alphasparse_cuda_exchange_t *ex,
                                                      alphasparse_datatype_t datatype, int rank, int world,
                                                      const ALPHA_INT *part /* world + 1 row boundaries */);
size_t alphasparse_cuda_exchange_blob_bytes(void);
alphasparse_status_t alphasparse_cuda_exchange_export(alphasparse_cuda_exchange_t ex, void *blob);
alphasparse_status_t alphasparse_cuda_exchange_connect(alphasparse_cuda_exchange_t ex, const void *blobs);
/* How y reaches the peers: 0 from inside the product kernels, chunk by chunk while later chunks are
 * still being multiplied (default from 4 GPUs up); 1 by one bulk peer-copy kernel after the product
 * (default below 4 GPUs, where there is too little traffic to hide). */
alphasparse_status_t alphasparse_cuda_exchange_set_mode(alphasparse_cuda_exchange_t ex, int mode);
/* Device pointer of the current x (part[world] elements): fill it before the first step, read it after. */
alphasparse_status_t alphasparse_cuda_exchange_x(alphasparse_cuda_exchange_t ex, void **x);
/* Sets x from the ranks' own pieces: every rank passes ITS rows of x (part[rank+1] - part[rank] elements,
 * host or device memory); the piece is copied into this GPU's buffer and stored into every peer's over
 * NVLink, the ranks signal each other as after a product, and the buffers swap: afterwards
 * alphasparse_cuda_exchange_x is the complete vector on every GPU.  With x in host memory each GPU
 * moves 1/world of it over PCIe.  Collective: all ranks call it, in the same order as their products. */
alphasparse_status_t alphasparse_cuda_exchange_load_x(alphasparse_cuda_exchange_t ex, const void *x_block);
/* Waits for the stream and reports whether any bounded wait ran out (status 3) since creation. */
alphasparse_status_t alphasparse_cuda_exchange_status(alphasparse_cuda_exchange_t ex, int *status);
/* Test aids for the bounded wait: enqueue a wait on a counter that no rank ever advances, limited to
 * max_polls polls (it records status 3 and returns, the context stays usable), and reset the status. */
alphasparse_status_t alphasparse_cuda_exchange_debug_wait(alphasparse_cuda_exchange_t ex, int64_t max_polls);
alphasparse_status_t alphasparse_cuda_exchange_clear_status(alphasparse_cuda_exchange_t ex);
alphasparse_status_t alphasparse_cuda_exchange_destroy(alphasparse_cuda_exchange_t ex);
alphasparse_status_t alphasparse_s_mv_exchange(const float alpha, const alphasparse_matrix_t A,
                                               const struct alpha_matrix_descr descr,
                                               alphasparse_cuda_exchange_t ex, const float beta, float *y);
alphasparse_status_t alphasparse_d_mv_exchange(const double alpha, const alphasparse_matrix_t A,
                                               const struct alpha_matrix_descr descr,
                                               alphasparse_cuda_exchange_t ex, const double beta, double *y);

/* Error word of a handle's kernels.  Kernels that wait (the row-tile kernel waits for its bulk copies) give up
 * after a bounded number of polls, leave y untouched for their tile and record a code here: 1 = a tile larger
 * than the kernel was configured for, 2 = a bulk copy did not complete in time.  A call with host vectors
 * reports it as ALPHA_SPARSE_STATUS_EXECUTION_FAILED by itself; a caller that passes device pointers (calls
 * only enqueue) asks here: waits for the library stream, stores the code (0 = fine) and, with clear != 0,
 * resets it so that later calls start clean. */
alphasparse_status_t alphasparse_cuda_kernel_status(const alphasparse_matrix_t A, int *status, int clear);

/* Kernel timing for benchmarks.  With profiling enabled on a handle, every mv / mm call on it
 * brackets its dominant kernel (the SpMV or SpMM kernel itself, not the small fix-up or any
 * copies) with CUDA events on the library stream; alphasparse_cuda_kernel_ms waits for the
 * last such kernel and returns its duration in milliseconds. */
alphasparse_status_t alphasparse_cuda_profile_kernel(const alphasparse_matrix_t A, int enable);
alphasparse_status_t alphasparse_cuda_kernel_ms(const alphasparse_matrix_t A, float *ms);

/* Test aid: makes the nth device allocation the library performs from now on fail as if the device
 * were out of memory (0 cancels).  The failing call returns ALPHA_SPARSE_STATUS_ALLOC_FAILED and
 * releases whatever it had already allocated. */
alphasparse_status_t alphasparse_cuda_debug_fail_alloc(int64_t nth);

/* Number of kernels this library has launched in this process so far. */
int64_t alphasparse_cuda_launch_count(void);

/* Text of the last CUDA error the library met in this thread ("" if none). */
const char *alphasparse_cuda_last_error(void);

#ifdef __cplusplus
}
#endif
