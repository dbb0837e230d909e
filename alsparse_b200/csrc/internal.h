// Internal declarations shared by the translation units of libalphasparse_b200.so.
// Nothing here is part of the C ABI (see include/alphasparse/*.h for that).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "alphasparse/spapi_cuda.h"
#include "alphasparse/spdef.h"
#include "alphasparse/spmat.h"
#include "alphasparse/types.h"

namespace asb {

// ---- process-wide state --------------------------------------------------------------------
cudaStream_t current_stream();
alphasparse_cuda_alg_t forced_algorithm();
void count_launch(int n = 1);
void record_cuda_error(cudaError_t e, const char *what);
void record_error(const char *what);  // text for alphasparse_cuda_last_error without a CUDA error behind it

// Tuning values of the analysis (alphasparse_cuda_set_option / ALPHASPARSE_CUDA_OPTIONS); each has a
// default that measurements on B200 chose, tests shrink them to reach every branch on small matrices.
enum Option {
    kOptBandEnable = 0,   // 1: long rows of a skewed matrix go through the column-band kernel
    kOptBandBytes,        // bytes of x one column band stages in shared memory
    kOptBandMinSeg,       // a row is long when its elements average at least this many per band
    kOptBandMinRows,      // fewer long rows than this: not worth a second kernel
    kOptBandMinSharePct,  // long rows must hold at least this share of the stored elements
    kOptBandSplits,       // thread blocks per band (0: chosen from the band count)
    kOptBandOverlap,      // 1: the band kernel runs on a second stream beside the merge kernel
    kOptBandPacked,       // 1: the band kernel streams a packed, band-major copy of the long rows (16-bit columns)
    kOptBandVariant,      // shape of the band kernel: 0 = 8 lanes x 1 quad x 2 segments, 1 = 4 lanes x 2 quads x 1 segment
    kOptBinEnable,        // 1: skewed matrices are multiplied bin by bin (short / mid / long rows) instead of merge tiles
    kOptBinShort,         // rows of at most this many elements take the thread-per-row kernel
    kOptBinMid0,          // longest row of the first mid list (4 lanes per row)
    kOptBinMid1,          // longest row of the second mid list (16 lanes per row); longer rows: 32 lanes
    kOptBinOverlap,       // 1: the kernels of the bins run on streams of their own, side by side
    kOptBinMidMax,        // longest row the lane-group kernels may be given; longer non-band rows: merge tiles instead
    kOptBinPushMaxPeers,  // exchange calls to more GPUs than this run over merge tiles instead of bins
    kOptBinSort,          // 1: the lists of the two longer mid bins are ordered longest row first
    kOptPipeMaxWindows,   // host-vector mv: most row windows the product is cut into (1..16)
    kOptPipeMinPieceKb,   // ... and the smallest piece of y per window, in KB
    kOptMvBlockMinKb,     // vector-kernel SpMV: an x above this many KB is multiplied column block by column block (0: never)
    kOptMvBlockKb,        // ... each block covering at most this many KB of x
    kOptSpmmColViaRow,    // column-major dense blocks of at least this many columns are transposed and go through the row-major kernels (0: never)
    kOptSpmmNarrow,       // 1: row-major dense blocks with rows of at most 32 bytes go through the narrow kernel
    kOptSpmmSplitMin,     // row-major dense-block product: rows above this many elements are multiplied chunk by chunk (0: never)
    kOptSpmmSplitChunk,   // ... in chunks of this many elements
    kOptSpmmColBlocks,    // column blocks of the row-major dense-block product (0 or 1: one pass)
    kOptCount
};
int64_t option(Option o);

// Every device allocation of the library goes through here: cudaMalloc, except that a test can ask
// for the n-th allocation from now on to fail (alphasparse_cuda_debug_fail_alloc), which is how the
// out-of-memory paths are exercised without exhausting a GPU.
cudaError_t device_alloc_bytes(void **p, size_t bytes);
template <typename P>
inline cudaError_t device_alloc(P **p, size_t bytes) {
    return device_alloc_bytes(reinterpret_cast<void **>(p), bytes);
}

// Maps a failed CUDA call to a status and records its text for alphasparse_cuda_last_error.
#define ASB_CUDA_OR(expr, status)                          \
    do {                                                   \
        cudaError_t _e = (expr);                           \
        if (_e != cudaSuccess) {                           \
            ::asb::record_cuda_error(_e, #expr);           \
            return (status);                               \
        }                                                  \
    } while (0)

// ---- per-handle device context, stored in alphasparse_matrix.dcu_info ---------------------
constexpr uint64_t kCtxMagic = 0x4153423230304358ull;  // guards against foreign pointers

// Elements appended (zero-filled) after the last stored element of the column and value
// arrays so that aligned 16-byte loads that start inside the array never leave it.
constexpr int kTailPad = 16;

// Merge-path tile shape: kMergeThreads threads, each consuming kMergeItems (rows+nnz) items.
constexpr int kMergeThreads = 256;
constexpr int kMergeMinBlocks = 5;  // resident blocks per SM the merge kernel is compiled for (48 registers)
constexpr int kMergeItemsS = 9;  // float
constexpr int kMergeItemsD = 7;  // double

// Row-tile kernel: rows per block (= threads per block) and the most shared memory one block may
// ask for (four blocks per SM must still fit in the 227 KB an SM offers).
constexpr int kRowTile = 128;
constexpr size_t kRowTileMaxSmem = 56 * 1024;

// Where a kernel delivers finished y rows besides its own y: the next-x buffer of every GPU of the
// row partition (peer-mapped device pointers), row r of this block landing at element row_off + r.
constexpr int kMaxPeers = 8;
struct PeerPush {
    void *dst[kMaxPeers];
    int n;
    long long row_off;
    int after;  // 1: deliver with a separate bulk copy after the product instead of from inside it
    int runs;   // 1: the destination wants long contiguous runs (host memory behind PCIe): a binned handle then
                // delivers through its merge tiles, chunk by chunk, not row by row from the bin kernels
    // merge kernel only: progress counters of its chunks of consecutive tiles
    int tiles, chunk_tiles;
    unsigned *chunk_done;  // tiles finished per chunk; reset by the block that completes the chunk
};
constexpr int kPushChunkTiles = 128;  // tiles per delivered chunk (64..512 measured alike on B200)

struct MergeCoord {
    int row;  // rows fully consumed before this point
    int nz;   // stored elements consumed before this point
};

// Long rows of a skewed matrix, handled by the column-band kernel (spmv_band.cu).  Position p of the
// list is row `row[p]`, of which the elements [seg[0*rows+p], seg[bands*rows+p]) -- the part covered by
// merge tiles lying wholly inside the row -- are multiplied band by band; seg[b*rows+p] is the first of
// them whose column is >= b*width.
struct BandTables {
    int rows = 0;       // long rows
    int bands = 0;      // column bands of `width` columns
    int width = 0;
    int splits = 1;     // thread blocks per band; block (b, s) takes positions [s*chunk, (s+1)*chunk)
    int chunk = 0;
    int64_t elements = 0;  // stored elements handled here
    bool whole_rows = false;  // the listed rows are handled from first to last element (row bins) instead of
                              // only where whole merge tiles lie inside them
    int *d_row = nullptr;      // rows
    int *d_seg = nullptr;      // (bands + 1) * rows
    void *d_partial = nullptr; // rows * bands sums, written by every call
    // Packed copy of the long rows' elements, band-major (optional): the segments of band b follow each other in
    // list order, each padded to whole quads; columns are stored relative to the band in 16 bits (0xffff = padding).
    // d_pk_start[b * rows + p] is the first quad of segment (b, p); one more entry closes the last segment.
    int *d_pk_start = nullptr;
    void *d_pk_val = nullptr;
    unsigned short *d_pk_col = nullptr;
    int64_t pk_quads = 0;
    cudaStream_t side = nullptr;  // second stream + fork / join events when the kernels overlap
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
};

// Row bins of a skewed matrix (spmv_bins.cu): rows of at most short_limit elements are found by the thread-per-row
// kernel itself; d_list holds the row numbers of the three mid bins back to back (lengths up to 32, up to 256,
// longer); the long rows are in BandTables.
constexpr int kMidBins = 3;
struct RowBins {
    bool active = false;
    int short_limit = 0;
    int64_t short_rows = 0;
    int64_t offset[kMidBins] = {}, count[kMidBins] = {};
    int *d_list = nullptr;
    // one extra stream per mid list (+ fork / join events) when the bin kernels are to run side by side
    cudaStream_t side[kMidBins] = {};
    cudaEvent_t ev_fork = nullptr, ev_join[kMidBins] = {};
};
void bins_destroy(RowBins &b);

// Column blocks of the row-major dense-block product (spmm.cu): split[p * rows + r] is the first element of
// row r whose column lies in block p or beyond; blocks == 1: the product runs in one pass.
struct SpmmBlocks {
    int blocks = 0;   // 0: nothing decided yet
    int width = 0;    // columns per block
    bool unsorted = false;  // some row is not in ascending column order: no blocking for this matrix
    int *d_split = nullptr;
};
void spmm_blocks_destroy(SpmmBlocks &b);
struct DeviceCtx;
// Builds (or drops, blocks <= 1) the table of `b` for `blocks` column blocks of the matrix in `ctx`; leaves
// b.blocks == 1 when the rows are not in ascending column order.
alphasparse_status_t col_blocks_ensure(DeviceCtx *ctx, SpmmBlocks &b, int blocks, cudaStream_t st);

// Long rows of the row-major dense-block product (spmm.cu).  One lane group per row is fine until a row holds a
// hundred thousand elements and its group is still walking it long after every other row is done: rows above
// `spmm_split_min` elements are left out of the row pass (their end in d_hi_short is their start), cut into chunks of
// `spmm_split_chunk` elements that the same kernel multiplies as if they were rows, into partial sums, and a last
// kernel adds each row's partial sums, in chunk order, onto Y.
struct SpmmSplit {
    int state = 0;  // 0: not looked at yet, 1: no long rows, 2: tables below are in use
    int64_t nlong = 0, nchunks = 0;
    int *d_hi_short = nullptr;                           // rows
    int *d_chunk_lo = nullptr, *d_chunk_hi = nullptr;    // nchunks
    int *d_long_row = nullptr, *d_long_first = nullptr;  // nlong, nlong + 1 (first chunk of each long row)
    int *h_long_row = nullptr, *h_long_first = nullptr;  // host copies: which chunks a row window owns
    void *d_part = nullptr;                              // partial sums, nchunks x columns
    size_t part_bytes = 0;
};
void spmm_split_destroy(SpmmSplit &s);

struct DeviceCtx {
    uint64_t magic = kCtxMagic;
    int device = 0;
    int datatype = 0;  // alphasparse_datatype_t
    int64_t rows = 0, cols = 0, nnz = 0;

    int *d_row_ptr = nullptr;  // rows + 1
    int *d_col = nullptr;      // nnz + kTailPad
    void *d_val = nullptr;     // nnz + kTailPad

    // analysis results
    int64_t max_row_nnz = 0;
    int64_t empty_rows = 0;
    double mean_row_nnz = 0.0;
    double mean_row_quads = 0.0;  // aligned 4-element groups a row touches, on average
    double shifted_rows = 0.0;    // share of sampled elements whose next-row twin sits one column to the right
    int64_t max_tile_span = 0;    // largest quad-aligned element span of kRowTile consecutive rows
    int algorithm = ALPHA_SPARSE_CUDA_ALG_VECTOR;
    int lanes = 4;

    // merge-path tables (only when algorithm == MERGE)
    int merge_items = 0;
    int64_t merge_tiles = 0;
    MergeCoord *d_tile = nullptr;  // merge_tiles + 1
    int *d_carry_row = nullptr;    // merge_tiles
    void *d_carry_val = nullptr;   // merge_tiles
    int *d_sched = nullptr;            // block -> tile order of the merge kernel, or null (tile_key_kernel)
    int64_t sched_tiles = 0;           // tiles the merge kernel runs (= merge_tiles unless long rows are banded)
    RowBins bins;                      // row bins of a skewed matrix; active: products run bin by bin
    const int *h_row_ptr = nullptr;    // host copy of the offsets, valid only while the handle is being created
    SpmmBlocks spmm;                   // column blocks of the row-major dense-block product
    SpmmSplit split;                   // its long rows, cut into chunks
    void *d_cm_x = nullptr, *d_cm_y = nullptr;  // row-major copies of column-major dense operands (spmm.cu), grown on demand
    size_t cm_x_bytes = 0, cm_y_bytes = 0;
    SpmmBlocks mvb;                    // column blocks of the vector-kernel SpMV, for an x that does not fit L2
    bool carry_stale = false;          // a run over ALL tiles wrote carries for tiles the schedule leaves out
    BandTables band;                   // long rows taken out of the merge tiles (spmv_band.cu); rows == 0: none
    unsigned *d_chunk_done = nullptr;  // per chunk of kPushChunkTiles tiles (exchange calls only)

    int *d_status = nullptr;  // error word set by kernels whose bounded waits ran out (0 = fine)

    // staging for calls that pass host vectors (grown on demand, reused)
    void *d_x_stage = nullptr;
    size_t x_stage_bytes = 0;
    void *d_y_stage = nullptr;
    size_t y_stage_bytes = 0;

    // optional timing of the dominant kernel of each mv / mm call (alphasparse_cuda_profile_kernel)
    bool profile = false;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;

    // second and third stream + events of the pipelined host-vector path (created on first use)
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev_pipe[1 + 2 * 16] = {};

    // A^T as a second device CSR, built on the first transposed mv / mm call and kept
    DeviceCtx *transposed = nullptr;
    // matrices derived for SYMMETRIC / TRIANGULAR / DIAGONAL descriptors, built on first use and kept
    DeviceCtx *derived[24] = {};

    int64_t device_bytes = 0;
    std::mutex mu;  // serialises calls that share the carry and staging buffers
};

DeviceCtx *ctx_of(const alphasparse_matrix_t A);

// Upload + analysis.  `ptr` has rows+1 zero-based offsets.  On failure everything allocated
// so far is released and *out stays null.
alphasparse_status_t ctx_create(int datatype, int64_t rows, int64_t cols, const int *ptr,
                                const int *col, const void *val, DeviceCtx **out);
// Wraps device arrays that already have the layout ctx_create produces (rows + 1 + 4 offsets, nnz + kTailPad columns
// and values with zeroed tails) and analyses them.  Takes the arrays over: on failure they are freed.
alphasparse_status_t ctx_adopt(int datatype, int64_t rows, int64_t cols, int64_t nnz, int *d_ptr, int *d_col,
                               void *d_val, DeviceCtx **out);
void ctx_destroy(DeviceCtx *ctx);
alphasparse_status_t ctx_analyse(DeviceCtx *ctx);

// ---- kernel launchers (device pointers, enqueue only) ---------------------------------------
// A contiguous range of rows of the handle: lets a caller run the product in pieces (the
// host-vector path overlaps the pieces with the PCIe copies of y).  begin must be a multiple of
// kRowTile.  Only the vector and row-tile kernels can run on a window.
struct RowWindow {
    int64_t begin, count;
};
bool spmv_supports_windows(const DeviceCtx *ctx);

template <typename T>
alphasparse_status_t launch_spmv(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y,
                                 cudaStream_t stream, const PeerPush *push = nullptr,
                                 const RowWindow *window = nullptr);

// Copies src[0 .. rows) to element push.row_off of every buffer in push.dst (peer-mapped or local).
// Column-band path for long rows (spmv_band.cu).  build: called by the analysis once the merge tiles exist,
// with the tile table copied to the host; marks in `skip` the tiles it takes over.  launch_band: partial sums
// per (long row, band); launch_band_reduce: y[row] += alpha * (sum of the row's partials), after the merge
// kernel and its fix-up have written y.
alphasparse_status_t band_build(DeviceCtx *ctx, const MergeCoord *h_tile, std::vector<char> &skip, cudaStream_t st);
// The same tables for whole rows (row bins): `rows` are the long rows, h_ptr the host copy of the offsets.
// Leaves ctx->band.rows == 0 when one of them is not in ascending column order.
alphasparse_status_t band_build_rows(DeviceCtx *ctx, const int *h_ptr, const std::vector<int> &rows, cudaStream_t st);
int64_t band_long_min(const DeviceCtx *ctx);  // shortest row the column-band kernel takes
alphasparse_status_t bins_build(DeviceCtx *ctx, const int *h_ptr, int64_t long_min, std::vector<int> &long_rows,
                                cudaStream_t st);
template <typename T>
void launch_bins(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y, cudaStream_t st, const PeerPush *push = nullptr);
void band_destroy(BandTables &b);
template <typename T>
void launch_band(DeviceCtx *ctx, const T *x, cudaStream_t st);
// whole_rows tables: y[row] = alpha * sum + beta * y[row]; otherwise y[row] += alpha * sum (beta unused)
template <typename T>
void launch_band_reduce(DeviceCtx *ctx, T alpha, T beta, T *y, cudaStream_t st, const PeerPush *push = nullptr);

template <typename T>
void launch_push_rows(int64_t rows, const T *src, const PeerPush &push, cudaStream_t stream);

template <typename T>
alphasparse_status_t launch_spmm_row(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx,
                                     T beta, T *Y, int ldy, cudaStream_t stream,
                                     const RowWindow *window = nullptr);

template <typename T>
alphasparse_status_t launch_spmm_col(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx,
                                     T beta, T *Y, int ldy, cudaStream_t stream);

// A^T of a handle's device CSR, built on the device (coo2csr.cu); arrays in ctx_adopt's layout.
template <typename T>
alphasparse_status_t transpose_csr_device(const DeviceCtx *c, int **out_ptr, int **out_col, T **out_val);
// Device CSR (ctx_adopt layout) of what a SYMMETRIC / TRIANGULAR / DIAGONAL descriptor makes of the square matrix in `c`.
template <typename T>
alphasparse_status_t derive_csr_device(const DeviceCtx *c, int type, int upper, int unit, int flip, int diag_rule,
                                       int **out_ptr, int **out_col, T **out_val, int64_t *out_nnz);

// COO -> CSR on the device (coo2csr.cu): host arrays in, host 3-array CSR out, same output as the host
// path in core.cu (ordered by row then column, equal pairs in input order).
template <typename T>
alphasparse_status_t coo_to_csr_device(int64_t rows, int64_t cols, int64_t nnz, const int *ri, const int *ci,
                                       const T *v, int *out_ptr, int *out_col, T *out_val);

}  // namespace asb
