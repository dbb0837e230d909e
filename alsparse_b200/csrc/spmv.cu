// CSR SpMV kernels for sm_100a and the one-time analysis that picks between them.
//
// y = alpha * A * x + beta * y for a general CSR matrix, the operation of the reference's
// gemv_{s,d}_csr (arithmetic defined by src/plain/kernel/level2/mv/gemv/gemv_x_csr_plain.c:4-24
// of the reference).  SpMV moves ~12 bytes per flop pair, so the kernels are built around
// HBM traffic, not arithmetic: the value and column streams are read once with 16-byte
// coalesced loads and a streaming cache policy, x is gathered through the read-only path so
// that it stays resident in L2, y is written once.  No tensor cores: there is no reuse to
// feed them.
//
// Two kernel families:
//   vector  a group of LANES (1..32) lanes owns a row; each lane takes whole aligned quads
//           (4 consecutive stored elements) of the row, so every load is a 16-byte load of
//           col and of val regardless of where the row starts.  Used when rows are short and
//           of similar length.
//   merge   every thread block consumes the same number of (row-end + stored-element) items
//           of the merge of the row offsets with the element indices, so a 200000-element
//           row and a run of one-element rows cost the same.  Partial sums that cross a block
//           boundary go through a small carry array and a second kernel adds them, in a fixed
//           order: results do not depend on scheduling and no floating-point atomics are used.
#include <limits.h>
#include <stdio.h>

#include <algorithm>
#include <type_traits>
#include <vector>

#include "internal.h"

namespace asb {

bool spmv_supports_windows(const DeviceCtx *ctx);

// ---- streaming loads / stores ------------------------------------------------------------
// ld.global.cs / st.global.cs: data touched once, first in line for eviction from L1 and L2.

template <typename T>
struct Quad {
    T v[4];
};

__device__ __forceinline__ int4 load_quad_idx(const int *__restrict__ col, int q) {
    return __ldcs(reinterpret_cast<const int4 *>(col) + q);
}
__device__ __forceinline__ Quad<float> load_quad_val(const float *__restrict__ val, int q) {
    float4 t = __ldcs(reinterpret_cast<const float4 *>(val) + q);
    Quad<float> r;
    r.v[0] = t.x, r.v[1] = t.y, r.v[2] = t.z, r.v[3] = t.w;
    return r;
}
__device__ __forceinline__ Quad<double> load_quad_val(const double *__restrict__ val, int q) {
    double2 a = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q);
    double2 b = __ldcs(reinterpret_cast<const double2 *>(val) + 2 * (size_t)q + 1);
    Quad<double> r;
    r.v[0] = a.x, r.v[1] = a.y, r.v[2] = b.x, r.v[3] = b.y;
    return r;
}

// ---- vector kernel -------------------------------------------------------------------------

template <typename T>
__device__ __forceinline__ T quad_dot(const int4 c, const Quad<T> &v, int base, int s, int e,
                                      const T *__restrict__ x) {
    // Elements of the quad outside [s, e) belong to a neighbouring row (or to the zero tail).
    T acc = T(0);
    if (base + 0 >= s && base + 0 < e) acc = fma(v.v[0], __ldg(x + c.x), acc);
    if (base + 1 >= s && base + 1 < e) acc = fma(v.v[1], __ldg(x + c.y), acc);
    if (base + 2 >= s && base + 2 < e) acc = fma(v.v[2], __ldg(x + c.z), acc);
    if (base + 3 >= s && base + 3 < e) acc = fma(v.v[3], __ldg(x + c.w), acc);
    return acc;
}

// 256 threads; 256/LANES row groups; each group handles RPG rows that are 256/LANES apart so
// that every load instruction of a warp covers consecutive rows (consecutive memory).  The
// first quad of all RPG rows is requested before any of them is consumed, which keeps two
// independent chains (offset -> col/val -> x) in flight per thread.
// Measured on B200: with few lanes per row (random gathers, bound by the L2 request rate) two
// rows per group at 6 resident blocks per SM is fastest; with 8 or more lanes per row one row
// per group at full occupancy is.
template <int LANES>
struct VectorShape {
    static constexpr int RPG = LANES <= 4 ? 2 : 1;
    static constexpr int MIN_BLOCKS = LANES <= 4 ? 6 : 8;
};

template <typename T, int LANES, int RPG, bool HAS_BETA>
__global__ void __launch_bounds__(256, VectorShape<LANES>::MIN_BLOCKS)
    spmv_vector_kernel(int rows, const int *__restrict__ row_ptr, const int *__restrict__ row_end,
                       const int *__restrict__ col, const T *__restrict__ val, const T *__restrict__ x,
                       T *__restrict__ y, T alpha, T beta) {
    constexpr int GROUPS = 256 / LANES;
    const int lane = threadIdx.x % LANES;
    const int grp = threadIdx.x / LANES;
    const long long row0 = (long long)blockIdx.x * (GROUPS * RPG) + grp;

    int s[RPG], e[RPG];
#pragma unroll
    for (int u = 0; u < RPG; u++) {
        const long long r = row0 + (long long)u * GROUPS;
        s[u] = 0, e[u] = 0;
        if (r < rows) {
            s[u] = __ldg(row_ptr + r);  // the whole row, or its elements inside one column block (see launch_vector)
            e[u] = __ldg(row_end + r);
        }
    }

    int q[RPG];
    int4 c[RPG];
    Quad<T> v[RPG];
#pragma unroll
    for (int u = 0; u < RPG; u++) {
        q[u] = (s[u] >> 2) + lane;
        if ((q[u] << 2) < e[u]) {
            c[u] = load_quad_idx(col, q[u]);
            v[u] = load_quad_val(val, q[u]);
        }
    }

    T sum[RPG];
#pragma unroll
    for (int u = 0; u < RPG; u++) {
        sum[u] = T(0);
        if ((q[u] << 2) < e[u]) sum[u] = quad_dot(c[u], v[u], q[u] << 2, s[u], e[u], x);
        for (int qq = q[u] + LANES; (qq << 2) < e[u]; qq += LANES) {
            const int4 cc = load_quad_idx(col, qq);
            const Quad<T> vv = load_quad_val(val, qq);
            sum[u] += quad_dot(cc, vv, qq << 2, s[u], e[u], x);
        }
    }

#pragma unroll
    for (int u = 0; u < RPG; u++) {
#pragma unroll
        for (int o = LANES / 2; o > 0; o >>= 1) sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], o);
        const long long r = row0 + (long long)u * GROUPS;
        if (lane == 0 && r < rows) {
            T out = alpha * sum[u];
            if (HAS_BETA) out = fma(beta, y[r], out);
            __stcs(y + r, out);
        }
    }
}

// ---- row-tile kernel ----------------------------------------------------------------------------
//
// One block stages the column indices, values and offsets of kRowTile consecutive rows in
// shared memory with three bulk asynchronous copies (cp.async.bulk global -> shared, completion
// counted in bytes on an mbarrier), then every thread walks ONE row out of shared memory.
// Compared with the vector kernel this turns the x gathers of a banded matrix into coalesced
// accesses (neighbouring lanes = neighbouring rows = neighbouring columns), which is what the
// 27-point stencil needs: there the vector kernel is limited by L1 wavefronts, not by HBM.
// Several blocks are resident per SM, so the copies of one overlap the arithmetic of another.
//
// The element range of a tile is widened to multiples of four elements so that source
// addresses and sizes are multiples of 16 bytes, as the bulk copy requires; the arrays carry a
// zero tail for that.  The wait on the mbarrier is bounded: if it runs out the block records
// an error word and leaves without touching y.

__device__ __forceinline__ unsigned smem_u32(const void *p) {
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void bulk_copy_g2s(unsigned dst, const void *src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

template <typename T, bool HAS_BETA, bool PUSH>
__global__ void __launch_bounds__(kRowTile)
    spmv_rowtile_kernel(int rows, const int *__restrict__ row_ptr, const int *__restrict__ col,
                        const T *__restrict__ val, const T *__restrict__ x, T *__restrict__ y, T alpha,
                        T beta, int cap, int *__restrict__ status, PeerPush push) {
    extern __shared__ __align__(128) unsigned char smem[];
    T *s_val = reinterpret_cast<T *>(smem);
    int *s_col = reinterpret_cast<int *>(smem + (size_t)cap * sizeof(T));
    int *s_ptr = s_col + cap;
    unsigned long long *s_bar = reinterpret_cast<unsigned long long *>(s_ptr + kRowTile + 4);
    __shared__ int s_oversize;

    const int tid = threadIdx.x;
    const int r0 = blockIdx.x * kRowTile;
    const int nr = min(kRowTile, rows - r0);
    const unsigned bar = smem_u32(s_bar);

    if (tid == 0) {
        const int start = __ldg(row_ptr + r0), end = __ldg(row_ptr + r0 + nr);
        const int a0 = start & ~3;
        int n = ((end + 3) & ~3) - a0;
        s_oversize = n > cap;
        if (n > cap) {  // cannot happen for a handle analysed by this library; refuse rather than overrun
            atomicExch(status, 1);
            n = 0;
        }
        const unsigned ptr_bytes = (unsigned)(((nr + 1 + 3) & ~3) * sizeof(int));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        const unsigned bytes = ptr_bytes + (unsigned)n * (unsigned)(sizeof(int) + sizeof(T));
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
        bulk_copy_g2s(smem_u32(s_ptr), row_ptr + r0, ptr_bytes, bar);
        if (n > 0) {
            bulk_copy_g2s(smem_u32(s_col), col + a0, (unsigned)n * sizeof(int), bar);
            bulk_copy_g2s(smem_u32(s_val), val + a0, (unsigned)n * sizeof(T), bar);
        }
    }
    __syncthreads();

    bool arrived = false;
    for (int spin = 0; spin < (1 << 22); spin++) {
        if (mbar_try_wait(bar, 0)) {
            arrived = true;
            break;
        }
    }
    if (!arrived) {
        if (tid == 0) atomicExch(status, 2);
        return;
    }
    if (s_oversize) return;  // nothing was staged: the whole block leaves before it touches the tile or x

    const int a0 = s_ptr[0] & ~3;
    const int b = tid < nr ? s_ptr[tid] - a0 : 0, e = tid < nr ? s_ptr[tid + 1] - a0 : 0;
    const int len = e - b;
    // Neighbouring lanes read rows that start len elements apart: with an even len several lanes hit
    // the same shared-memory bank on every step (16-way for len = 16).  Starting lane t at element
    // t mod len of its row and wrapping round spreads them over the banks; the row is still summed
    // completely, only from a different starting point.  Odd lengths are conflict-free as they are.
    // The choice is made per warp so that no warp runs both loops.
    const bool even = (len & 1) == 0 && len > 0;
    const bool wrap = __any_sync(0xffffffffu, even);
    if (tid < nr) {
        T acc0 = T(0), acc1 = T(0), acc2 = T(0), acc3 = T(0);
        if (!wrap) {
            int k = b;
            for (; k + 4 <= e; k += 4) {
                const int c0 = s_col[k], c1 = s_col[k + 1], c2 = s_col[k + 2], c3 = s_col[k + 3];
                const T x0 = __ldg(x + c0), x1 = __ldg(x + c1), x2 = __ldg(x + c2), x3 = __ldg(x + c3);
                acc0 = fma(s_val[k], x0, acc0);
                acc1 = fma(s_val[k + 1], x1, acc1);
                acc2 = fma(s_val[k + 2], x2, acc2);
                acc3 = fma(s_val[k + 3], x3, acc3);
            }
            for (; k < e; k++) acc0 = fma(s_val[k], __ldg(x + s_col[k]), acc0);
        } else {
            int k = b + (even ? tid % len : 0);
            int left = len;
            for (; left >= 4; left -= 4) {
                const int k0 = k, k1 = (k0 + 1 == e) ? b : k0 + 1, k2 = (k1 + 1 == e) ? b : k1 + 1,
                          k3 = (k2 + 1 == e) ? b : k2 + 1;
                k = (k3 + 1 == e) ? b : k3 + 1;
                const int c0 = s_col[k0], c1 = s_col[k1], c2 = s_col[k2], c3 = s_col[k3];
                const T x0 = __ldg(x + c0), x1 = __ldg(x + c1), x2 = __ldg(x + c2), x3 = __ldg(x + c3);
                acc0 = fma(s_val[k0], x0, acc0);
                acc1 = fma(s_val[k1], x1, acc1);
                acc2 = fma(s_val[k2], x2, acc2);
                acc3 = fma(s_val[k3], x3, acc3);
            }
            for (; left > 0; left--) {
                acc0 = fma(s_val[k], __ldg(x + s_col[k]), acc0);
                k = (k + 1 == e) ? b : k + 1;
            }
        }
        const int r = r0 + tid;
        T out = alpha * ((acc0 + acc1) + (acc2 + acc3));
        if (HAS_BETA) out = fma(beta, y[r], out);
        __stcs(y + r, out);
        if (PUSH) {  // neighbouring lanes hold neighbouring rows: coalesced stores into every peer's next x
#pragma unroll 1
            for (int p = 0; p < push.n; p++) static_cast<T *>(push.dst[p])[push.row_off + r] = out;
        }
    }
}

// ---- merge kernel ----------------------------------------------------------------------------

// One thread block = one tile of NT*IPT merge items.  The tile's start and end coordinates
// (row, element) were computed once at analysis time.
//
// Two paths.  A tile that lies inside a single long row (no row ends in it: about two thirds
// of the tiles of a power-law matrix) is a plain dot product: strided loads, register sums,
// one block reduction, nothing staged.  Any other tile stages its products in shared memory
// in load order and lets every thread walk its IPT consecutive merge items.
//
// With PUSH the same kernel also performs the allgather of y.  Tiles are grouped into chunks of
// `push.chunk_tiles` consecutive tiles; every block counts its tile as done, and the block that
// completes a chunk adds the carries of rows lying wholly inside the chunk and then copies the
// chunk's finished y rows into the next-x buffer of every GPU with wide coalesced stores through
// peer-mapped pointers.  So the transfer of chunk c over NVLink runs while later chunks are still
// being multiplied, the stores are long contiguous runs (pushing each tile's few rows as they
// finish was measured at ~100 GB/s; bulk copies reach several times that), and no block ever waits
// for another.  Rows whose carries cross a chunk boundary are finished, and pushed, by the fix-up
// kernel.
struct NoPush {};  // kernels instantiated without PUSH carry no delivery arguments at all
template <bool PUSH>
using PushArg = typename std::conditional<PUSH, PeerPush, NoPush>::type;


// Copies n elements starting at src (read at L2: other blocks may just have written them) to element
// `at` of every destination buffer.  Each element is read once and stored push.n times; four
// independent loads per thread are in flight, and 16-byte accesses are used when source and
// destinations share their alignment.
template <typename V>
__device__ __forceinline__ void push_units(const V *__restrict__ src, int n, const PeerPush &push, size_t byte_at) {
    const int tid = threadIdx.x, nt = blockDim.x;
    for (int i = tid; i < n; i += 4 * nt) {
        V v[4];
#pragma unroll
        for (int u = 0; u < 4; u++)
            if (i + u * nt < n) v[u] = __ldcg(src + i + u * nt);
        for (int p = 0; p < push.n; p++) {
            V *dst = reinterpret_cast<V *>(static_cast<char *>(push.dst[p]) + byte_at);
#pragma unroll
            for (int u = 0; u < 4; u++)
                if (i + u * nt < n) dst[i + u * nt] = v[u];
        }
    }
}

template <typename T>
__device__ __forceinline__ void push_span(const T *__restrict__ src, int n, const PeerPush &push, long long at) {
    const size_t byte_at = (size_t)at * sizeof(T);
    const uintptr_t sa = (uintptr_t)src, da = (uintptr_t)push.dst[0] + byte_at;
    constexpr int per = 16 / (int)sizeof(T);
    if ((sa & 15) == (da & 15) && n >= 4 * per) {
        int head = (int)(((16 - (sa & 15)) & 15) / sizeof(T));
        const int body = (n - head) / per;
        push_units<T>(src, head, push, byte_at);
        push_units<int4>(reinterpret_cast<const int4 *>(src + head), body, push, byte_at + (size_t)head * sizeof(T));
        const int done = head + body * per;
        push_units<T>(src + done, n - done, push, byte_at + (size_t)done * sizeof(T));
    } else {
        push_units<T>(src, n, push, byte_at);
    }
}

// Called by every thread of a compute block when its tile is finished.  The block that completes a
// chunk of push.chunk_tiles consecutive tiles (whichever arrives last) finishes the chunk: it adds
// the carries of rows that lie wholly inside the chunk and copies the chunk's rows to every GPU.
template <typename T>
__device__ __noinline__ void merge_chunk_deliver(int rows, const int *__restrict__ row_ptr,
                                                 const MergeCoord *__restrict__ tile,
                                                 const T *__restrict__ carry_val, T *__restrict__ y, T alpha,
                                                 const PeerPush &push, int c) {
    const int tid = threadIdx.x, nt = blockDim.x;
    const int t0 = c * push.chunk_tiles, t1 = min(t0 + push.chunk_tiles, push.tiles);
    // Carries of rows that begin and end inside this chunk (tile t stops in row tile[t+1].row).
    const int row_hi = tile[t1].row;  // rows below this one ended in the chunk
    for (int t = t0 + tid; t < t1; t += nt) {
        const int r = tile[t + 1].row;
        if (r >= row_hi || r >= rows) continue;   // ends in a later chunk
        if (t > 0 && tile[t].row == r) continue;  // not the first tile of its run
        T acc = __ldcg(carry_val + t);            // written by other blocks of this grid: read at L2
        for (int u = t + 1; tile[u + 1].row == r; u++) acc += __ldcg(carry_val + u);
        y[r] = fma(alpha, acc, __ldcg(y + r));
    }
    __syncthreads();
    // Finished rows of the chunk: all rows that ended in it, except the first one when it began in
    // an earlier chunk (the fix-up kernel completes and pushes that one).
    int ra = tile[t0].row;
    if (ra < rows && tile[t0].nz > row_ptr[ra]) ra++;
    const int n = row_hi - ra;
    if (n > 0) push_span<T>(y + ra, n, push, push.row_off + ra);
}

template <typename T>
__device__ __forceinline__ void merge_tile_done(int rows, const int *__restrict__ row_ptr,
                                                const MergeCoord *__restrict__ tile,
                                                const T *__restrict__ carry_val, T *__restrict__ y, T alpha,
                                                const PeerPush &push, int tile_id) {
    __shared__ int s_last;
    __syncthreads();  // all of this block's y and carry writes are issued
    const int c = tile_id / push.chunk_tiles;
    if (threadIdx.x == 0) {
        const int in_chunk = min(push.chunk_tiles, push.tiles - c * push.chunk_tiles);
        __threadfence();  // ... and ordered before the count (cumulative over the barrier above)
        const unsigned old = atomicAdd(push.chunk_done + c, 1u);
        s_last = (old + 1u == (unsigned)in_chunk);
        if (s_last) {
            push.chunk_done[c] = 0;  // ready for the next call
            __threadfence();         // the other blocks' writes are visible from here on
        }
    }
    __syncthreads();
    if (s_last) merge_chunk_deliver<T>(rows, row_ptr, tile, carry_val, y, alpha, push, c);
}
template <typename T>
__device__ __forceinline__ void merge_tile_done(int, const int *, const MergeCoord *, const T *, T *, T,
                                                const NoPush &, int) {}

template <typename T, int NT, int IPT, bool HAS_BETA, bool PUSH>
__global__ void __launch_bounds__(NT, kMergeMinBlocks)
    spmv_merge_kernel(int rows, const int *__restrict__ row_ptr, const int *__restrict__ col,
                      const T *__restrict__ val, const T *__restrict__ x, T *__restrict__ y,
                      T alpha, T beta, const MergeCoord *__restrict__ tile, const int *__restrict__ sched,
                      int *__restrict__ carry_row, T *__restrict__ carry_val,
                      const __grid_constant__ PushArg<PUSH> push) {
    constexpr int TILE = NT * IPT;
    constexpr int NW = NT / 32;
    __shared__ T s_prod[TILE];
    __shared__ int s_rend[TILE + 1];
    __shared__ int s_ckey[NT];
    __shared__ T s_cval[NT];
    __shared__ int s_wkey[NW];
    __shared__ T s_wval[NW];

    const int tid = threadIdx.x;
    const int lane = tid & 31, wid = tid >> 5;
    // Block b takes tile sched[b] when a schedule is given (see tile_key_kernel), else tile b.
    const int tile_id = sched ? __ldg(sched + blockIdx.x) : (int)blockIdx.x;
    const MergeCoord c0 = tile[tile_id], c1 = tile[tile_id + 1];
    const int r0 = c0.row, j0 = c0.nz;
    const int tile_rows = c1.row - r0, tile_nnz = c1.nz - j0;

    // All loads of a thread are independent: IPT column/value pairs in flight, then IPT gathers.
    int cc[IPT];
    T vv[IPT];
#pragma unroll
    for (int k = 0; k < IPT; k++) {
        const int i = tid + k * NT;
        cc[k] = 0, vv[k] = T(0);
        if (i < tile_nnz) {
            cc[k] = __ldcs(col + j0 + i);
            vv[k] = __ldcs(val + j0 + i);
        }
    }

    if (tile_rows == 0) {
        // ---- inside one row: block-wide dot product, leftover goes to the carry array --------
        T acc = T(0);
#pragma unroll
        for (int k = 0; k < IPT; k++)
            if (tid + k * NT < tile_nnz) acc = fma(vv[k], __ldg(x + cc[k]), acc);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) s_wval[wid] = acc;
        __syncthreads();
        if (tid == 0) {
            T total = s_wval[0];
#pragma unroll
            for (int w = 1; w < NW; w++) total += s_wval[w];
            carry_row[tile_id] = r0;
            carry_val[tile_id] = total;
        }
        if (PUSH) merge_tile_done<T>(rows, row_ptr, tile, carry_val, y, alpha, push, tile_id);
        return;
    }

    // ---- general tile ---------------------------------------------------------------------------
    const int items = tile_rows + tile_nnz;
    // Row ends relative to the tile's first element; entry tile_rows is the (unfinished) row
    // the tile stops in, or +inf past the last row.
    for (int i = tid; i <= tile_rows; i += NT) {
        const int r = r0 + i;
        s_rend[i] = (r < rows) ? (__ldg(row_ptr + r + 1) - j0) : INT_MAX;
    }
#pragma unroll
    for (int k = 0; k < IPT; k++) {
        const int i = tid + k * NT;
        if (i < tile_nnz) s_prod[i] = vv[k] * __ldg(x + cc[k]);
    }
    __syncthreads();

    // This thread's slice of the merge path: items [d, d + IPT).
    const int d = min(tid * IPT, items);
    int lo = max(0, d - tile_nnz), hi = min(d, tile_rows);
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (s_rend[mid] <= d - mid - 1) lo = mid + 1;
        else hi = mid;
    }
    int i = lo, j = d - lo;
    int cur_end = s_rend[i];  // end of the row being accumulated; re-read only when a row ends

    T run = T(0);
    int first_row = -1;  // first row that ends inside this thread; may have started earlier
    T first_val = T(0);
#pragma unroll
    for (int k = 0; k < IPT; k++) {
        if (d + k < items) {
            if (j < cur_end) {
                run += s_prod[j];
                j++;
            } else {
                if (first_row < 0) {
                    first_row = i;
                    first_val = run;
                } else {
                    const int r = r0 + i;
                    T out = alpha * run;
                    if (HAS_BETA) out = fma(beta, y[r], out);
                    y[r] = out;
                }
                run = T(0);
                i++;
                cur_end = s_rend[i];
            }
        }
    }

    // Segmented inclusive scan of the per-thread leftovers (key = row the thread stopped in).
    // Keys are non-decreasing with the thread index, so equal keys are contiguous.
    int key = i;
    T acc = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int k2 = __shfl_up_sync(0xffffffffu, key, o);
        const T v2 = __shfl_up_sync(0xffffffffu, acc, o);
        if (lane >= o && k2 == key) acc += v2;
    }
    if (lane == 31) {
        s_wkey[wid] = key;
        s_wval[wid] = acc;
    }
    __syncthreads();
    for (int w = wid - 1; w >= 0; w--) {
        if (s_wkey[w] != key) break;
        acc += s_wval[w];
    }
    s_ckey[tid] = key;
    s_cval[tid] = acc;
    __syncthreads();

    if (first_row >= 0) {
        if (tid > 0 && s_ckey[tid - 1] == first_row) first_val += s_cval[tid - 1];
        const int r = r0 + first_row;
        T out = alpha * first_val;
        if (HAS_BETA) out = fma(beta, y[r], out);
        y[r] = out;
    }
    if (tid == NT - 1) {
        carry_row[tile_id] = r0 + key;
        carry_val[tile_id] = acc;
    }
    if (PUSH) merge_tile_done<T>(rows, row_ptr, tile, carry_val, y, alpha, push, tile_id);
}

// Adds the tile leftovers to the rows they belong to.  Consecutive tiles that stopped in the
// same row form a run; the first thread of a run adds the whole run, front to back.
// With PUSH the delivering blocks of the merge kernel have already handled every run that begins
// and ends in one chunk; this kernel takes the runs that cross a chunk boundary and pushes those rows.
template <typename T, bool PUSH>
__global__ void spmv_merge_fixup_kernel(int rows, long long tiles, const int *__restrict__ carry_row,
                                        const T *__restrict__ carry_val, T *__restrict__ y,
                                        T alpha, PeerPush push) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tiles) return;
    const int r = carry_row[t];
    if (r >= rows) return;
    if (t > 0 && carry_row[t - 1] == r) return;
    T acc = carry_val[t];
    long long u = t + 1;
    for (; u < tiles && carry_row[u] == r; u++) acc += carry_val[u];
    // u is now the tile in which row r ends
    if (PUSH && t / push.chunk_tiles == u / push.chunk_tiles && u < tiles) return;
    const T out = fma(alpha, acc, y[r]);
    y[r] = out;
    if (PUSH) {
        for (int p = 0; p < push.n; p++) static_cast<T *>(push.dst[p])[push.row_off + r] = out;
    }
}

// Copies this GPU's finished y block into the next-x buffer of every peer: the exchange step for
// the kernels that do not push from their own epilogue.
template <typename T>
__global__ void push_rows_kernel(long long rows, const T *__restrict__ y, const __grid_constant__ PeerPush push) {
    // each block takes a contiguous slice, so that its stores to a peer are long runs
    const long long per_block = ((rows + gridDim.x - 1) / gridDim.x + 63) & ~63ll;
    const long long lo = (long long)blockIdx.x * per_block;
    const long long n = lo < rows ? (rows - lo < per_block ? rows - lo : per_block) : 0;
    if (n > 0) push_span<T>(y + lo, (int)n, push, push.row_off + lo);
}

template <typename T>
void launch_push_rows(int64_t rows, const T *src, const PeerPush &push, cudaStream_t st) {
    if (rows <= 0 || push.n <= 0) return;
    push_rows_kernel<T><<<148 * 4, 256, 0, st>>>(rows, src, push);
    count_launch();
}
template void launch_push_rows<float>(int64_t, const float *, const PeerPush &, cudaStream_t);
template void launch_push_rows<double>(int64_t, const double *, const PeerPush &, cudaStream_t);

// y = beta * y for a matrix without stored elements (the reference still scales y).
template <typename T>
__global__ void scale_kernel(long long n, T *__restrict__ y, T beta) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) y[i] = (beta == T(0)) ? T(0) : y[i] * beta;
}

// ---- analysis kernels --------------------------------------------------------------------------

// out[0] = max row length, out[1] = empty rows, out[2] = aligned quads touched (summed over
// rows), out[3] = rows whose end offset is below their start offset (malformed input),
// out[5] = largest quad-aligned element span of a tile of kRowTile consecutive rows.
__global__ void row_stats_kernel(int rows, const int *__restrict__ row_ptr,
                                 unsigned long long *__restrict__ out) {
    unsigned long long mx = 0, empty = 0, quads = 0, bad = 0, span = 0;
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r < rows;
         r += (long long)gridDim.x * blockDim.x) {
        const int s = row_ptr[r], e = row_ptr[r + 1];
        if (e < s) {
            bad++;
            continue;
        }
        const unsigned long long len = (unsigned long long)(e - s);
        mx = len > mx ? len : mx;
        if (len == 0) empty++;
        else quads += (unsigned long long)(((e + 3) >> 2) - (s >> 2));
        if (r % kRowTile == 0) {
            const long long last = r + kRowTile < rows ? r + kRowTile : rows;
            const int te = row_ptr[last];
            if (te >= s) {
                const unsigned long long sp = (unsigned long long)(((te + 3) & ~3) - (s & ~3));
                span = sp > span ? sp : span;
            }
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long m2 = __shfl_xor_sync(0xffffffffu, mx, o);
        mx = m2 > mx ? m2 : mx;
        const unsigned long long s2 = __shfl_xor_sync(0xffffffffu, span, o);
        span = s2 > span ? s2 : span;
        empty += __shfl_xor_sync(0xffffffffu, empty, o);
        quads += __shfl_xor_sync(0xffffffffu, quads, o);
        bad += __shfl_xor_sync(0xffffffffu, bad, o);
    }
    if ((threadIdx.x & 31) == 0) {
        atomicMax(out + 0, mx);
        atomicMax(out + 5, span);
        if (empty) atomicAdd(out + 1, empty);
        if (quads) atomicAdd(out + 2, quads);
        if (bad) atomicAdd(out + 3, bad);
    }
}

// out[0] = stored column indices outside [0, cols).  A kernel given such an index would read
// outside x, so handle creation refuses the matrix instead.
__global__ void col_range_kernel(long long nnz, int cols, const int *__restrict__ col,
                                 unsigned long long *__restrict__ out) {
    unsigned long long bad = 0;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nnz;
         i += (long long)gridDim.x * blockDim.x) {
        const int c = col[i];
        if (c < 0 || c >= cols) bad++;
    }
    for (int o = 16; o > 0; o >>= 1) bad += __shfl_xor_sync(0xffffffffu, bad, o);
    if ((threadIdx.x & 31) == 0 && bad) atomicAdd(out, bad);
}

// Shifted-row structure: out[0] counts sampled positions k (first, middle, last element) of rows r
// for which row r+1 holds column col(r, k) + 1 at the same position, out[1] the positions sampled.
// Close to 1 for stencils and other banded matrices in natural ordering (neighbouring rows gather
// neighbouring x elements), close to 0 for unstructured columns.
__global__ void row_shift_kernel(int rows, const int *__restrict__ row_ptr, const int *__restrict__ col,
                                 unsigned long long *__restrict__ out) {
    unsigned long long hit = 0, seen = 0;
    for (long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x; r + 1 < rows;
         r += (long long)gridDim.x * blockDim.x) {
        const int s0 = row_ptr[r], s1 = row_ptr[r + 1], e1 = row_ptr[r + 2];
        const int len0 = s1 - s0, len1 = e1 - s1;
        if (len0 <= 0 || len1 <= 0) continue;
        const int ks[3] = {0, len0 / 2, len0 - 1};
        for (int i = 0; i < 3; i++) {
            if (i > 0 && ks[i] == ks[i - 1]) continue;
            seen++;
            if (ks[i] < len1 && col[s1 + ks[i]] == col[s0 + ks[i]] + 1) hit++;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        hit += __shfl_xor_sync(0xffffffffu, hit, o);
        seen += __shfl_xor_sync(0xffffffffu, seen, o);
    }
    if ((threadIdx.x & 31) == 0 && seen) {
        atomicAdd(out + 0, hit);
        atomicAdd(out + 1, seen);
    }
}

// Start coordinate of every merge tile: the point on diagonal t*items of the merge of the row
// end offsets (row_ptr[1..rows]) with the element indices 0..nnz-1.
__global__ void merge_tiles_kernel(int rows, int nnz, const int *__restrict__ row_ptr, int items,
                                   long long tiles, MergeCoord *__restrict__ out) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t > tiles) return;
    long long diag = t * items;
    const long long total = (long long)rows + nnz;
    if (diag > total) diag = total;
    long long lo = diag > nnz ? diag - nnz : 0, hi = diag < rows ? diag : rows;
    while (lo < hi) {
        const long long mid = (lo + hi) >> 1;
        if ((long long)row_ptr[mid + 1] <= diag - mid - 1) lo = mid + 1;
        else hi = mid;
    }
    out[t].row = (int)lo;
    out[t].nz = (int)(diag - lo);
}

// Sort key of every merge tile for the block schedule.  A tile that lies inside ONE row of a matrix
// with ascending columns gathers from a narrow band of x that starts at its first column; when the
// blocks that run at the same time take such tiles in the order of that column -- across all long
// rows -- the part of x in use at any moment is a small window that stays in L2, whatever the size
// of x.  (Measured on B200 with 1550 rows of 200,000 elements in fp64: 347 / 287 / 229 / 105 G
// elements/s when x is 16 / 33 / 67 / 134 MB, i.e. the gathers are fast only while x is L2-resident.)
// Tiles that span several rows touch all of x anyway: key -1, they run first in their own order.
// (A separate kernel for the single-row tiles -- 16-byte loads, no shared memory, 5 to 8 blocks per SM --
// ran no faster than the branch of the merge kernel: the gathers, not the loads of A, set the pace.)
__global__ void tile_key_kernel(long long tiles, const MergeCoord *__restrict__ tile, const int *__restrict__ col,
                                int *__restrict__ key) {
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tiles) return;
    const MergeCoord a = tile[t], b = tile[t + 1];
    key[t] = (a.row == b.row && b.nz > a.nz) ? col[a.nz] : -1;
}

// ---- analysis (host) ------------------------------------------------------------------------------

// Dynamic shared memory of one row-tile block: values | columns | offsets (+4 pad) | mbarrier.
static size_t rowtile_smem_bytes(const DeviceCtx *ctx) {
    const size_t cap = (size_t)((ctx->max_tile_span + 3) & ~3ll);
    const size_t tsz = ctx->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    return cap * (tsz + sizeof(int)) + (kRowTile + 4) * sizeof(int) + 16;
}

static int pick_lanes(double mean_quads) {
    // Lanes per row = aligned quads an average row touches, rounded to a power of two.
    int lanes = 1;
    while (lanes < 32 && (double)lanes < mean_quads * 0.75) lanes <<= 1;
    return lanes;
}

// Block schedule of the merge kernel (tile_key_kernel): single-row tiles by first column, behind the
// others.  Built when x is too large to stay in L2 next to the matrix stream and enough of the tiles
// are single-row ones for the order to matter; the sort runs on the host (one key per tile).
constexpr size_t kScheduleMinXBytes = (size_t)24 << 20;

static bool schedule_disabled() {
    static const bool off = [] {
        const char *v = getenv("ALPHASPARSE_CUDA_NO_SCHEDULE");
        return v && *v && *v != '0';
    }();
    return off;
}

// Decides which tiles the merge kernel runs and in which order.  Tiles covered by the column-band path
// (band_build) drop out; the remaining single-row tiles are taken in the order of their first column when
// x is large (tile_key_kernel).  Leaves d_sched null when the natural order over all tiles is what is wanted.
static alphasparse_status_t build_tile_schedule(DeviceCtx *ctx, cudaStream_t st) {
    const size_t tsz = ctx->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    const long long tiles = ctx->merge_tiles;
    ctx->sched_tiles = tiles;
    if (tiles < 2) return ALPHA_SPARSE_STATUS_SUCCESS;
    std::vector<MergeCoord> h_tile((size_t)tiles + 1);
    cudaError_t e = cudaMemcpyAsync(h_tile.data(), ctx->d_tile, sizeof(MergeCoord) * ((size_t)tiles + 1),
                                    cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        record_cuda_error(e, "tile schedule");
        return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    }
    std::vector<char> skip((size_t)tiles, 0);
    if (!ctx->bins.active) {  // a binned handle runs its merge tiles only in the delivering form: all of them
        alphasparse_status_t s = band_build(ctx, h_tile.data(), skip, st);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    }
    const bool banded = ctx->band.rows > 0 && !ctx->band.whole_rows;
    const bool by_column = !schedule_disabled() && (size_t)ctx->cols * tsz >= kScheduleMinXBytes;
    if (!banded && !by_column) return ALPHA_SPARSE_STATUS_SUCCESS;

    std::vector<int> order;
    order.reserve((size_t)tiles);
    long long single = 0;
    for (long long t = 0; t < tiles; t++) {
        if (skip[(size_t)t]) continue;
        order.push_back((int)t);
        single += h_tile[(size_t)t].row == h_tile[(size_t)t + 1].row;
    }
    const bool sort_it = by_column && single * 8 >= (long long)order.size();  // fewer than one tile in eight: leave it
    if (!banded && !sort_it) return ALPHA_SPARSE_STATUS_SUCCESS;
    int *d_key = nullptr;
    ASB_CUDA_OR(device_alloc(&d_key, sizeof(int) * (size_t)tiles), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    if (sort_it) {
        tile_key_kernel<<<(unsigned)((tiles + 255) / 256), 256, 0, st>>>(tiles, ctx->d_tile, ctx->d_col, d_key);
        count_launch();
        std::vector<int> key((size_t)tiles);
        e = cudaMemcpyAsync(key.data(), d_key, sizeof(int) * (size_t)tiles, cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) {
            cudaFree(d_key);
            record_cuda_error(e, "tile schedule");
            return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
        }
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return key[(size_t)a] < key[(size_t)b]; });
    }
    e = cudaMemcpyAsync(d_key, order.data(), sizeof(int) * order.size(), cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) {
        cudaFree(d_key);
        record_cuda_error(e, "tile schedule");
        return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    }
    ctx->d_sched = d_key;
    ctx->sched_tiles = (long long)order.size();
    ctx->device_bytes += (int64_t)(sizeof(int) * (size_t)tiles);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Row bins (spmv_bins.cu) for a matrix the analysis found skewed.  Declined -- the handle then multiplies over merge
// tiles -- when some row is too long for a lane group yet not long enough for the column-band kernel, when there
// are long rows but too few (or holding too little) to be worth that kernel, or when a long row is not in ascending
// column order.
static alphasparse_status_t try_row_bins(DeviceCtx *ctx, cudaStream_t st) {
    if (!option(kOptBinEnable)) return ALPHA_SPARSE_STATUS_SUCCESS;
    std::vector<int> fetched;
    const int *h_ptr = ctx->h_row_ptr;
    if (!h_ptr) {  // re-analysis of a live handle: the offsets come back from the device
        fetched.resize((size_t)ctx->rows + 1);
        cudaError_t e = cudaMemcpyAsync(fetched.data(), ctx->d_row_ptr, sizeof(int) * ((size_t)ctx->rows + 1),
                                        cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) {
            record_cuda_error(e, "row bins");
            return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
        }
        h_ptr = fetched.data();
    }
    const int64_t long_min = option(kOptBandEnable) ? band_long_min(ctx) : INT64_MAX;
    // With many column bands (a wide matrix) the rows that are long enough for the band kernel start far above
    // bin_mid_max; the 32-lane list then takes the rows in between as well, up to eight times the limit (its rows are
    // ordered longest first), rather than the whole matrix falling back to merge tiles for them (power-law, 2^24 rows:
    // long rows start at 24,576 elements).
    int64_t mid_max = option(kOptBinMidMax);
    if (long_min != INT64_MAX) mid_max = std::max(mid_max, std::min(long_min - 1, 8 * mid_max));
    for (int64_t r = 0; r < ctx->rows; r++) {
        const int64_t n = (int64_t)h_ptr[r + 1] - h_ptr[r];
        if (n > mid_max && n < long_min) return ALPHA_SPARSE_STATUS_SUCCESS;
    }
    std::vector<int> long_rows;
    alphasparse_status_t s = bins_build(ctx, h_ptr, long_min, long_rows, st);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    if (!long_rows.empty()) {
        s = band_build_rows(ctx, h_ptr, long_rows, st);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS || ctx->band.rows == 0) {
            const int64_t freed = (int64_t)sizeof(int) * (ctx->bins.count[0] + ctx->bins.count[1] + ctx->bins.count[2]);
            bins_destroy(ctx->bins);
            ctx->device_bytes -= freed;
            return s;
        }
    }
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// Merge-path tables of a handle: tile coordinates, carry arrays, chunk counters, block schedule and the
// column-band tables.  Everything is built into `tmp` and handed to the handle only when all of it exists,
// so a failure half-way (alphasparse_optimize on a live handle) leaves the handle as it was.
static alphasparse_status_t build_merge_tables(DeviceCtx *ctx, cudaStream_t st) {
    const int ipt = (ctx->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE) ? kMergeItemsD : kMergeItemsS;
    const size_t tsz = (ctx->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE) ? 8 : 4;
    const int items = kMergeThreads * ipt;
    const int64_t total = ctx->rows + ctx->nnz;
    const int64_t tiles = (total + items - 1) / items;
    const size_t nchunks = (size_t)(tiles + kPushChunkTiles - 1) / kPushChunkTiles;
    MergeCoord *d_tile = nullptr;
    int *d_carry_row = nullptr;
    void *d_carry_val = nullptr;
    unsigned *d_chunk_done = nullptr;
    auto undo = [&] {
        cudaFree(d_tile), cudaFree(d_carry_row), cudaFree(d_carry_val), cudaFree(d_chunk_done);
        cudaFree(ctx->d_sched);
        ctx->d_sched = nullptr;
        band_destroy(ctx->band);
        bins_destroy(ctx->bins);
        ctx->d_tile = nullptr, ctx->d_carry_row = nullptr, ctx->d_carry_val = nullptr, ctx->d_chunk_done = nullptr;
        ctx->merge_tiles = 0, ctx->sched_tiles = 0;
    };
#define TRY(expr, status)                 \
    do {                                  \
        cudaError_t _e = (expr);          \
        if (_e != cudaSuccess) {          \
            record_cuda_error(_e, #expr); \
            undo();                       \
            return (status);              \
        }                                 \
    } while (0)
    TRY(device_alloc(&d_tile, sizeof(MergeCoord) * (size_t)(tiles + 1)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_carry_row, sizeof(int) * (size_t)tiles), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_carry_val, tsz * (size_t)tiles), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(device_alloc(&d_chunk_done, sizeof(unsigned) * nchunks), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    TRY(cudaMemsetAsync(d_chunk_done, 0, sizeof(unsigned) * nchunks, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    // 0x7f7f7f7f lies beyond any row: the fix-up kernel ignores tiles that never ran
    TRY(cudaMemsetAsync(d_carry_row, 0x7f, sizeof(int) * (size_t)tiles, st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    const int threads = 256;
    const int blocks = (int)((tiles + 1 + threads - 1) / threads);
    merge_tiles_kernel<<<blocks, threads, 0, st>>>((int)ctx->rows, (int)ctx->nnz, ctx->d_row_ptr, items, tiles, d_tile);
    count_launch();
    TRY(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    TRY(cudaStreamSynchronize(st), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
#undef TRY
    // the schedule and the band tables read these through the handle
    ctx->merge_items = items, ctx->merge_tiles = tiles;
    ctx->d_tile = d_tile, ctx->d_carry_row = d_carry_row, ctx->d_carry_val = d_carry_val, ctx->d_chunk_done = d_chunk_done;
    ctx->carry_stale = false;
    alphasparse_status_t s = try_row_bins(ctx, st);
    if (s == ALPHA_SPARSE_STATUS_SUCCESS) s = build_tile_schedule(ctx, st);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) {
        undo();
        return s;
    }
    ctx->device_bytes += (int64_t)(sizeof(MergeCoord) * (size_t)(tiles + 1) + (sizeof(int) + tsz) * (size_t)tiles);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

alphasparse_status_t ctx_analyse(DeviceCtx *ctx) {
    cudaStream_t st = current_stream();
    ctx->algorithm = ALPHA_SPARSE_CUDA_ALG_VECTOR;
    ctx->lanes = 4;
    ctx->max_row_nnz = 0, ctx->empty_rows = ctx->rows, ctx->mean_row_nnz = 0.0;
    if (ctx->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;

    unsigned long long *d_out = nullptr, h_out[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    ASB_CUDA_OR(device_alloc(&d_out, sizeof(h_out)), ALPHA_SPARSE_STATUS_ALLOC_FAILED);
    cudaError_t e = cudaMemsetAsync(d_out, 0, sizeof(h_out), st);
    if (e == cudaSuccess) {
        const int threads = 256;
        long long want = (ctx->rows + threads - 1) / threads;
        int blocks = (int)(want < 148 * 16 ? want : 148 * 16);
        row_stats_kernel<<<blocks, threads, 0, st>>>((int)ctx->rows, ctx->d_row_ptr, d_out);
        count_launch();
        if (ctx->nnz > 0) {
            want = (ctx->nnz + threads - 1) / threads;
            blocks = (int)(want < 148 * 16 ? want : 148 * 16);
            col_range_kernel<<<blocks, threads, 0, st>>>(ctx->nnz, (int)ctx->cols, ctx->d_col,
                                                         d_out + 4);
            want = (ctx->rows + threads - 1) / threads;
            blocks = (int)(want < 148 * 16 ? want : 148 * 16);
            row_shift_kernel<<<blocks, threads, 0, st>>>((int)ctx->rows, ctx->d_row_ptr, ctx->d_col,
                                                         d_out + 6);
            count_launch(2);
        }
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_out, d_out, sizeof(h_out), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    cudaFree(d_out);
    if (e != cudaSuccess) {
        record_cuda_error(e, "row analysis");
        return ALPHA_SPARSE_STATUS_EXECUTION_FAILED;
    }
    if (h_out[3] != 0 || h_out[4] != 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;

    ctx->max_row_nnz = (int64_t)h_out[0];
    ctx->empty_rows = (int64_t)h_out[1];
    ctx->mean_row_nnz = (double)ctx->nnz / (double)ctx->rows;
    ctx->mean_row_quads = (double)h_out[2] / (double)ctx->rows;
    ctx->max_tile_span = (int64_t)h_out[5];
    ctx->shifted_rows = h_out[7] ? (double)h_out[6] / (double)h_out[7] : 0.0;
    ctx->lanes = pick_lanes(ctx->mean_row_quads);

    // A row longer than eight passes of its lane group would leave that group running long
    // after the rest of the grid has drained: switch to equal-work tiles.
    int alg = forced_algorithm();
    const bool rowtile_fits = rowtile_smem_bytes(ctx) <= kRowTileMaxSmem;
    if (alg == ALPHA_SPARSE_CUDA_ALG_ROWTILE && !rowtile_fits) alg = ALPHA_SPARSE_CUDA_ALG_AUTO;
    if (alg == ALPHA_SPARSE_CUDA_ALG_AUTO) {
        const int64_t comfortable = (int64_t)ctx->lanes * 4 * 8;
        if (ctx->max_row_nnz > comfortable) alg = ALPHA_SPARSE_CUDA_ALG_MERGE;
        else if (rowtile_fits && (ctx->shifted_rows >= 0.5 || ctx->mean_row_nnz <= 4.0))
            alg = ALPHA_SPARSE_CUDA_ALG_ROWTILE;  // banded: thread-per-row makes the x gathers coalesce;
                                                  // very short rows: a whole lane group per row is wasteful
        else alg = ALPHA_SPARSE_CUDA_ALG_VECTOR;
    }
    if (alg == ALPHA_SPARSE_CUDA_ALG_MERGE && ctx->d_tile == nullptr) {
        // on failure the handle keeps the algorithm it had (or the vector kernel, which needs no tables)
        alphasparse_status_t s = build_merge_tables(ctx, st);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    }
    ctx->algorithm = alg;
    // An x that L2 cannot hold turns most gathers into 32-byte sector reads from HBM (2^24 x 16 in fp64, x = 134 MB:
    // 3.3 ms against 1.07 ms for the fp32 matrix).  The vector kernel then runs once per column block of at most
    // mv_block_kb of x; rows in ascending column order need only an offset per row and block for that.
    int blocks = 1;
    const int64_t tsz = ctx->datatype == ALPHA_SPARSE_DATATYPE_DOUBLE ? 8 : 4;
    const int64_t x_kb = ctx->cols * tsz >> 10, min_kb = option(kOptMvBlockMinKb), block_kb = std::max<int64_t>(1, option(kOptMvBlockKb));
    if ((alg == ALPHA_SPARSE_CUDA_ALG_VECTOR || (alg == ALPHA_SPARSE_CUDA_ALG_MERGE && ctx->bins.active)) && min_kb > 0 &&
        x_kb > min_kb && ctx->nnz > 0)  // (of a binned handle the lists of mid rows run block by block)
        blocks = (int)std::min<int64_t>(64, (x_kb + block_kb - 1) / block_kb);
    return col_blocks_ensure(ctx, ctx->mvb, blocks, st);
}

// ---- launchers -----------------------------------------------------------------------------------

template <typename T, int LANES>
static void launch_vector(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y, cudaStream_t st,
                          const RowWindow &w) {
    constexpr int RPG = VectorShape<LANES>::RPG;
    constexpr int rows_per_block = (256 / LANES) * RPG;
    const unsigned blocks = (unsigned)((w.count + rows_per_block - 1) / rows_per_block);
    const T *val = static_cast<const T *>(ctx->d_val);
    if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
    // A window is just an offset view: offsets stay absolute, so col / val need no shift.
    // Column blocks (an x that does not fit L2, see ctx_analyse): one launch per block over the elements of every row
    // that fall into it, so that the gathers of a launch stay inside a slice of x that L2 holds; the first launch
    // applies beta, the later ones add to y.
    const int passes = ctx->mvb.d_split ? ctx->mvb.blocks : 1;
    for (int p = 0; p < passes; p++) {
        const int *lo = passes > 1 ? ctx->mvb.d_split + (size_t)p * ctx->rows + w.begin : ctx->d_row_ptr + w.begin;
        const int *hi = passes > 1 ? lo + ctx->rows : lo + 1;
        const T b = p == 0 ? beta : T(1);
        if (b == T(0))
            spmv_vector_kernel<T, LANES, RPG, false><<<blocks, 256, 0, st>>>((int)w.count, lo, hi, ctx->d_col, val, x,
                                                                            y + w.begin, alpha, b);
        else
            spmv_vector_kernel<T, LANES, RPG, true><<<blocks, 256, 0, st>>>((int)w.count, lo, hi, ctx->d_col, val, x,
                                                                           y + w.begin, alpha, b);
    }
    if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
    count_launch(passes);
}

template <typename T, int IPT, bool HAS_BETA, bool PUSH>
static void launch_merge_as(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y, cudaStream_t st,
                            const PeerPush &push) {
    const T *val = static_cast<const T *>(ctx->d_val);
    T *carry = static_cast<T *>(ctx->d_carry_val);
    // In-kernel delivery wants chunks of neighbouring tiles to finish together: every tile, natural order,
    // and therefore no column-band path either.
    // Exchange calls over many GPUs stay on the merge tiles: their chunk-by-chunk delivery spreads the NVLink traffic
    // over the whole product, while the bins would send 88 % of the rows in one burst from the short-row kernel
    // (iterated power-law step on 8 GPUs: 0.32 ms with tiles, 0.47 ms with bins; on 2 GPUs 0.99 against 0.78 ms).
    // So do deliveries into page-locked host memory: single 8-byte stores over PCIe made the end-to-end power-law
    // product 5.4 ms, the tiles' 16-byte runs 3.1 ms.
    bool binned = ctx->bins.active;
    if constexpr (PUSH) binned = binned && !push.runs && push.n <= (int)option(kOptBinPushMaxPeers);
    if (binned) {
        // bin by bin: the column-band kernel (long rows) first, on its own stream when there is one, then
        // the short and mid rows; its partial sums are folded into y last.  In an exchange call (PUSH) every
        // kernel that finishes rows stores them into the peers' buffers itself.
        const PeerPush *deliver = PUSH ? &push : nullptr;
        BandTables &bt = ctx->band;
        if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
        if (bt.rows > 0) {
            cudaStream_t band_st = st;
            if (bt.side) {
                cudaEventRecord(bt.ev_fork, st);
                cudaStreamWaitEvent(bt.side, bt.ev_fork, 0);
                band_st = bt.side;
            }
            launch_band<T>(ctx, x, band_st);
        }
        launch_bins<T>(ctx, alpha, x, beta, y, st, deliver);
        if (bt.rows > 0) {
            if (bt.side) {
                cudaEventRecord(bt.ev_join, bt.side);
                cudaStreamWaitEvent(st, bt.ev_join, 0);
            }
            launch_band_reduce<T>(ctx, alpha, beta, y, st, deliver);
        }
        if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
        return;
    }
    const bool banded = !PUSH && ctx->band.rows > 0 && !ctx->band.whole_rows;
    const int *sched = PUSH ? nullptr : ctx->d_sched;
    const unsigned blocks = (unsigned)(PUSH ? ctx->merge_tiles : ctx->sched_tiles);
    if (PUSH && ctx->band.rows > 0 && !ctx->band.whole_rows) ctx->carry_stale = true;  // tiles the schedule leaves out write carries now
    if (banded && ctx->carry_stale) {
        cudaMemsetAsync(ctx->d_carry_row, 0x7f, sizeof(int) * (size_t)ctx->merge_tiles, st);
        ctx->carry_stale = false;
    }
    if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
    BandTables &bt = ctx->band;
    cudaStream_t band_st = st;
    if (banded) {
        // The band kernel only reads the matrix and x and writes its own partial sums: with a second stream
        // it runs beside the merge kernel (one is bound by HBM, the other by L2 requests).
        if (bt.side) {
            cudaEventRecord(bt.ev_fork, st);
            cudaStreamWaitEvent(bt.side, bt.ev_fork, 0);
            band_st = bt.side;
        }
        launch_band<T>(ctx, x, band_st);
    }
    PushArg<PUSH> arg{};
    if constexpr (PUSH) arg = push;
    if (blocks > 0)
        spmv_merge_kernel<T, kMergeThreads, IPT, HAS_BETA, PUSH><<<blocks, kMergeThreads, 0, st>>>(
            (int)ctx->rows, ctx->d_row_ptr, ctx->d_col, val, x, y, alpha, beta, ctx->d_tile, sched,
            ctx->d_carry_row, carry, arg);
    if (ctx->profile && !banded) cudaEventRecord(ctx->ev_stop, st);
    const unsigned fblocks = (unsigned)((ctx->merge_tiles + 255) / 256);
    spmv_merge_fixup_kernel<T, PUSH><<<fblocks, 256, 0, st>>>((int)ctx->rows, ctx->merge_tiles,
                                                             ctx->d_carry_row, carry, y, alpha, push);
    count_launch(2);
    if (banded) {
        if (bt.side) {
            cudaEventRecord(bt.ev_join, bt.side);
            cudaStreamWaitEvent(st, bt.ev_join, 0);
        }
        launch_band_reduce<T>(ctx, alpha, beta, y, st);
        // with two large kernels the timed span is the whole product
        if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
    }
}

template <typename T, int IPT>
static void launch_merge(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y, cudaStream_t st,
                         const PeerPush *push) {
    const PeerPush none{};
    if (push && push->after) {  // deliver with one bulk copy kernel once the product is complete
        if (beta == T(0)) launch_merge_as<T, IPT, false, false>(ctx, alpha, x, beta, y, st, none);
        else launch_merge_as<T, IPT, true, false>(ctx, alpha, x, beta, y, st, none);
        push_rows_kernel<T><<<148 * 4, 256, 0, st>>>(ctx->rows, y, *push);
        count_launch();
        return;
    }
    if (push) {
        PeerPush p = *push;
        p.tiles = (int)ctx->merge_tiles;
        p.chunk_tiles = kPushChunkTiles;
        p.chunk_done = ctx->d_chunk_done;
        if (beta == T(0)) launch_merge_as<T, IPT, false, true>(ctx, alpha, x, beta, y, st, p);
        else launch_merge_as<T, IPT, true, true>(ctx, alpha, x, beta, y, st, p);
    } else {
        if (beta == T(0)) launch_merge_as<T, IPT, false, false>(ctx, alpha, x, beta, y, st, none);
        else launch_merge_as<T, IPT, true, false>(ctx, alpha, x, beta, y, st, none);
    }
}

template <typename T>
static alphasparse_status_t launch_rowtile(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y,
                                           cudaStream_t st, const PeerPush *pushp, const RowWindow &w) {
    const int cap = (int)((ctx->max_tile_span + 3) & ~3ll);
    const size_t smem = rowtile_smem_bytes(ctx);
    const T *val = static_cast<const T *>(ctx->d_val);
    const unsigned blocks = (unsigned)((w.count + kRowTile - 1) / kRowTile);
    const bool in_kernel = pushp && !pushp->after;
    const PeerPush push = in_kernel ? *pushp : PeerPush{};
    const int which = (beta == T(0) ? 0 : 1) + (in_kernel ? 2 : 0);
    decltype(&spmv_rowtile_kernel<T, false, false>) variants[4] = {
        spmv_rowtile_kernel<T, false, false>, spmv_rowtile_kernel<T, true, false>,
        spmv_rowtile_kernel<T, false, true>, spmv_rowtile_kernel<T, true, true>};
    auto kernel = variants[which];
    // The opt-in limit is a property of the kernel, shared by all handles: only ever raise it.
    static std::atomic<size_t> granted[4] = {{0}, {0}, {0}, {0}};
    if (smem > 48 * 1024 && granted[which].load() < smem) {
        ASB_CUDA_OR(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kRowTileMaxSmem),
                    ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        granted[which].store(kRowTileMaxSmem);
    }
    if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
    // w.begin is a multiple of kRowTile (the caller's duty): tiles, and the 16-byte alignment of the
    // offset copies, are the same as in a full launch
    kernel<<<blocks, kRowTile, smem, st>>>((int)w.count, ctx->d_row_ptr + w.begin, ctx->d_col, val, x,
                                           y + w.begin, alpha, beta, cap, ctx->d_status, push);
    if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
    count_launch();
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template <typename T>
alphasparse_status_t launch_spmv(DeviceCtx *ctx, T alpha, const T *x, T beta, T *y,
                                 cudaStream_t st, const PeerPush *push, const RowWindow *window) {
    if (ctx->rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
    const RowWindow w = window ? *window : RowWindow{0, ctx->rows};
    if (window && (push || !spmv_supports_windows(ctx))) return ALPHA_SPARSE_STATUS_INTERNAL_ERROR;
    bool pushed = false;  // whether the kernel's own epilogue delivered y to the peers
    if (ctx->nnz == 0) {
        const unsigned blocks = (unsigned)((ctx->rows + 255) / 256);
        scale_kernel<T><<<blocks, 256, 0, st>>>(ctx->rows, y, beta);
        count_launch();
    } else if (ctx->algorithm == ALPHA_SPARSE_CUDA_ALG_MERGE) {
        constexpr int IPT = sizeof(T) == 8 ? kMergeItemsD : kMergeItemsS;
        launch_merge<T, IPT>(ctx, alpha, x, beta, y, st, push);
        pushed = true;
    } else if (ctx->algorithm == ALPHA_SPARSE_CUDA_ALG_ROWTILE) {
        alphasparse_status_t s = launch_rowtile<T>(ctx, alpha, x, beta, y, st, push, w);
        if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
        pushed = push && !push->after;
    } else {
        int lanes = ctx->lanes;  // a pass over one of P column blocks sees 1/P of every row
        for (int p = ctx->mvb.d_split ? ctx->mvb.blocks : 1; p > 1 && lanes > 1; p >>= 1) lanes >>= 1;
        switch (lanes) {
            case 1: launch_vector<T, 1>(ctx, alpha, x, beta, y, st, w); break;
            case 2: launch_vector<T, 2>(ctx, alpha, x, beta, y, st, w); break;
            case 4: launch_vector<T, 4>(ctx, alpha, x, beta, y, st, w); break;
            case 8: launch_vector<T, 8>(ctx, alpha, x, beta, y, st, w); break;
            case 16: launch_vector<T, 16>(ctx, alpha, x, beta, y, st, w); break;
            default: launch_vector<T, 32>(ctx, alpha, x, beta, y, st, w); break;
        }
    }
    if (push && !pushed) {
        push_rows_kernel<T><<<148 * 4, 256, 0, st>>>(ctx->rows, y, *push);
        count_launch();
    }
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template alphasparse_status_t launch_spmv<float>(DeviceCtx *, float, const float *, float, float *,
                                                 cudaStream_t, const PeerPush *, const RowWindow *);
template alphasparse_status_t launch_spmv<double>(DeviceCtx *, double, const double *, double,
                                                  double *, cudaStream_t, const PeerPush *, const RowWindow *);

bool spmv_supports_windows(const DeviceCtx *ctx) {
    return ctx->nnz > 0 && (ctx->algorithm == ALPHA_SPARSE_CUDA_ALG_VECTOR ||
                            ctx->algorithm == ALPHA_SPARSE_CUDA_ALG_ROWTILE);
}

}  // namespace asb

// =============================================================================================
// alphasparse_cuda_d_csrmv_noalloc: the merge-path SpMV without any allocation
// =============================================================================================
//
// Everything above keeps its load-balancing tables and carry buffers in memory obtained with
// cudaMalloc when a handle is created.  Some callers cannot afford that: a solver running
// inside a framework whose caching pool has already claimed the whole device (a cudaMalloc
// from a second library then fails although plenty of memory is "free" in the pool), or a
// service that must never hit the device-wide synchronisation cudaMalloc and cudaFree imply.
// For them this entry point works on caller-owned device CSR arrays and takes its scratch
// from one fixed array that is part of the library image.  The array costs kScratchBytes on
// every GPU that loads the library, for the lifetime of the process.

namespace {

constexpr size_t kScratchBytes = 4u << 20;  // 4 MiB per device
constexpr int kNoAllocItems = asb::kMergeThreads * asb::kMergeItemsD;
// per tile: start coordinate (8 bytes) + carry row (4) + carry value (8); one extra coordinate
constexpr long long kNoAllocMaxTiles = (long long)((kScratchBytes - 64) / 20) - 1;

// In host code this name is only a handle for cudaGetSymbolAddress, never a usable address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char *g_noalloc_ptr[kMaxDevices] = {};

// Device address of the scratch array on the CURRENT device, resolved on first use per device.
alphasparse_status_t noalloc_scratch(unsigned char **out) {
    int dev = -1;
    ASB_CUDA_OR(cudaGetDevice(&dev), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    if (dev < 0 || dev >= kMaxDevices) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[dev]) {
        void *p = nullptr;
        ASB_CUDA_OR(cudaGetSymbolAddress(&p, g_noalloc_scratch), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        g_noalloc_ptr[dev] = static_cast<unsigned char *>(p);
    }
    *out = g_noalloc_ptr[dev];
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

// true when `p` is memory the kernels of device `dev` can use: allocated on that device, or managed
bool on_device(const void *p, int dev) {
    cudaPointerAttributes at;
    if (cudaPointerGetAttributes(&at, p) != cudaSuccess) {
        (void)cudaGetLastError();
        return false;
    }
    if (at.type == cudaMemoryTypeManaged) return true;
    return at.type == cudaMemoryTypeDevice && at.device == dev;
}

}  // namespace

extern "C" alphasparse_status_t alphasparse_cuda_d_csrmv_noalloc(
    ALPHA_INT rows, ALPHA_INT cols, ALPHA_INT nnz, double alpha, const ALPHA_INT *d_row_ptr,
    const ALPHA_INT *d_col_indx, const double *d_values, const double *d_x, double beta, double *d_y) {
    using namespace asb;
    // cols only documents the length of d_x: the stored column indices are NOT checked against it here (a handle
    // checks them once, at creation; this call would have to read the whole index array on every product)
    if (rows < 0 || cols < 0 || nnz < 0) return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    if (rows == 0) return ALPHA_SPARSE_STATUS_SUCCESS;
    if (!d_row_ptr || !d_y || (nnz > 0 && (!d_col_indx || !d_values || !d_x)))
        return ALPHA_SPARSE_STATUS_NOT_INITIALIZED;
    int dev = -1;
    ASB_CUDA_OR(cudaGetDevice(&dev), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    if (!on_device(d_row_ptr, dev) || !on_device(d_y, dev) ||
        (nnz > 0 && (!on_device(d_col_indx, dev) || !on_device(d_values, dev) || !on_device(d_x, dev)))) {
        record_cuda_error(cudaErrorInvalidValue,
                          "alphasparse_cuda_d_csrmv_noalloc takes pointers to memory of the current device only");
        return ALPHA_SPARSE_STATUS_INVALID_POINTER;
    }
    const long long total = (long long)rows + nnz;
    const long long tiles = (total + kNoAllocItems - 1) / kNoAllocItems;
    if (tiles > kNoAllocMaxTiles) {
        char msg[200];
        snprintf(msg, sizeof(msg),
                 "alphasparse_cuda_d_csrmv_noalloc: rows + nnz = %lld exceeds the fixed scratch (limit %lld); "
                 "create a handle and use alphasparse_d_mv",
                 total, kNoAllocMaxTiles * kNoAllocItems);
        record_cuda_error(cudaErrorInvalidValue, msg);
        return ALPHA_SPARSE_STATUS_INVALID_VALUE;
    }
    cudaStream_t st = current_stream();
    if (nnz == 0) {
        scale_kernel<double><<<(unsigned)((rows + 255) / 256), 256, 0, st>>>(rows, d_y, beta);
        count_launch();
        ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
        return ALPHA_SPARSE_STATUS_SUCCESS;
    }

    unsigned char *scratch = nullptr;
    alphasparse_status_t s = noalloc_scratch(&scratch);
    if (s != ALPHA_SPARSE_STATUS_SUCCESS) return s;
    // Layout inside the scratch array: carry values | tile coordinates | carry rows.
    double *carry_val = reinterpret_cast<double *>(scratch);
    MergeCoord *tile = reinterpret_cast<MergeCoord *>(scratch + 8 * (size_t)kNoAllocMaxTiles);
    int *carry_row = reinterpret_cast<int *>(scratch + 16 * (size_t)(kNoAllocMaxTiles + 1));

    // The array still holds whatever the previous call left.  The tile table is rewritten in
    // full below; the carries are cleared so that a tile that writes none contributes zero.
    ASB_CUDA_OR(cudaMemsetAsync(carry_val, 0, sizeof(double) * (size_t)tiles, st),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    ASB_CUDA_OR(cudaMemsetAsync(carry_row, 0x7f, sizeof(int) * (size_t)tiles, st),
                ALPHA_SPARSE_STATUS_EXECUTION_FAILED);  // 0x7f7f7f7f: beyond any row, ignored by the fix-up
    merge_tiles_kernel<<<(unsigned)((tiles + 1 + 255) / 256), 256, 0, st>>>(rows, nnz, d_row_ptr, kNoAllocItems,
                                                                          tiles, tile);
    const PeerPush none{};
    const NoPush nopush{};
    if (beta == 0.0)
        spmv_merge_kernel<double, kMergeThreads, kMergeItemsD, false, false>
            <<<(unsigned)tiles, kMergeThreads, 0, st>>>(rows, d_row_ptr, d_col_indx, d_values, d_x, d_y, alpha,
                                                        beta, tile, nullptr, carry_row, carry_val, nopush);
    else
        spmv_merge_kernel<double, kMergeThreads, kMergeItemsD, true, false>
            <<<(unsigned)tiles, kMergeThreads, 0, st>>>(rows, d_row_ptr, d_col_indx, d_values, d_x, d_y, alpha,
                                                        beta, tile, nullptr, carry_row, carry_val, nopush);
    spmv_merge_fixup_kernel<double, false><<<(unsigned)((tiles + 255) / 256), 256, 0, st>>>(
        rows, tiles, carry_row, carry_val, d_y, alpha, none);
    count_launch(4);
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}
