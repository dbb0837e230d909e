/*
 * Seeded synthetic sparse matrices and vectors for the parity tests and the benchmark.
 *
 * The reference's tests read user-supplied Matrix-Market-like files or the output of its
 * time-seeded generator (tools/sparse_gen.c:35-102: uniform random points, sorted, duplicates
 * dropped); neither is reproducible.  These generators produce the same kinds of matrices
 * deterministically: every random draw is a pure function of (seed, stream, row, draw index),
 * so any row range can be generated on its own (one GPU's share of a row-partitioned matrix)
 * and the result does not depend on the thread count.
 *
 * All matrices come out as 3-array CSR pieces: row lengths first (so the caller can build
 * offsets and split rows), then columns (ascending, distinct within a row) and values.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef uint64_t u64;
typedef int64_t i64;
typedef int32_t i32;

static inline u64 mix64(u64 z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
/* draw number k of row `row` in stream `stream` */
static inline u64 draw(u64 seed, u64 stream, u64 row, u64 k) {
    return mix64(mix64(mix64(seed ^ (stream << 56)) + row) + k);
}
static inline double unit(u64 r) { return (double)(r >> 11) * (1.0 / 9007199254740992.0); }
static inline u64 below(u64 r, u64 n) { return (u64)(((unsigned __int128)r * n) >> 64); }

enum { STREAM_LEN = 1, STREAM_COL = 2, STREAM_VAL = 3 };

/* ---- row lengths --------------------------------------------------------------------- */

/* Poisson(lambda) by inversion of the cumulative distribution with one uniform per row. */
void synth_rowlen_poisson(u64 seed, i64 row0, i64 nrows, double lambda, i32 cap, i32 *len) {
    const double p0 = exp(-lambda);
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < nrows; i++) {
        double u = unit(draw(seed, STREAM_LEN, (u64)(row0 + i), 0));
        double p = p0, c = p0;
        i32 k = 0;
        while (u > c && k < cap) {
            k++;
            p *= lambda / k;
            c += p;
            if (p < 1e-300) break;
        }
        len[i] = k;
    }
}

/* Zipf (zeta) distribution with exponent s > 1 by the rejection method of Devroye
 * (Non-Uniform Random Variate Generation, 1986, ch. X.6), then clipped to [lo, hi]. */
void synth_rowlen_zipf(u64 seed, i64 row0, i64 nrows, double s, i32 lo, i32 hi, i32 *len) {
    const double am1 = s - 1.0, b = pow(2.0, am1);
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < nrows; i++) {
        u64 k = 0;
        double X;
        for (;;) {
            double U = 1.0 - unit(draw(seed, STREAM_LEN, (u64)(row0 + i), k++)); /* (0,1] */
            double V = unit(draw(seed, STREAM_LEN, (u64)(row0 + i), k++));
            X = floor(pow(U, -1.0 / am1));
            if (!(X >= 1.0) || X > 1e18) continue;
            double T = pow(1.0 + 1.0 / X, am1);
            if (V * X * (T - 1.0) / (b - 1.0) <= T / b) break;
        }
        double c = X < (double)lo ? (double)lo : (X > (double)hi ? (double)hi : X);
        len[i] = (i32)c;
    }
}

/* exclusive prefix sum of lengths into nrows+1 offsets; returns the total (may exceed 2^31,
 * in which case the offsets are unusable and the caller must shrink the matrix) */
i64 synth_offsets(i64 nrows, const i32 *len, i32 *ptr) {
    i64 acc = 0;
    for (i64 i = 0; i < nrows; i++) {
        ptr[i] = (i32)acc;
        acc += len[i];
    }
    ptr[nrows] = (i32)acc;
    return acc;
}

/* ---- distinct ascending uniform columns + values ---------------------------------------- */

static int cmp_i32(const void *a, const void *b) {
    i32 x = *(const i32 *)a, y = *(const i32 *)b;
    return (x > y) - (x < y);
}

/* L distinct values in [0, cols), ascending, for one row.  Short rows: rejection against the
 * values already held.  Long rows: draw, sort, drop duplicates, top up with further draws
 * until L distinct values are held.  Dense rows (L > cols/2): choose the complement. */
static void row_columns(u64 seed, u64 row, i32 L, i32 cols, i32 *out, i32 *scratch) {
    u64 k = 0;
    if (L <= 0) return;
    if (L > cols) L = cols;
    if ((i64)L * 2 > (i64)cols) {
        /* partial Fisher-Yates over the identity, then sort the chosen prefix */
        for (i32 i = 0; i < cols; i++) scratch[i] = i;
        for (i32 i = 0; i < L; i++) {
            i32 j = i + (i32)below(draw(seed, STREAM_COL, row, k++), (u64)(cols - i));
            i32 t = scratch[i];
            scratch[i] = scratch[j];
            scratch[j] = t;
        }
        memcpy(out, scratch, sizeof(i32) * (size_t)L);
        qsort(out, (size_t)L, sizeof(i32), cmp_i32);
        return;
    }
    if (L <= 48) {
        i32 n = 0;
        while (n < L) {
            i32 c = (i32)below(draw(seed, STREAM_COL, row, k++), (u64)cols);
            i32 p = n;
            int dup = 0;
            for (i32 q = 0; q < n; q++)
                if (out[q] == c) { dup = 1; break; }
            if (dup) continue;
            while (p > 0 && out[p - 1] > c) { out[p] = out[p - 1]; p--; }
            out[p] = c;
            n++;
        }
        return;
    }
    i32 n = 0;
    while (n < L) {
        for (i32 q = n; q < L; q++) out[q] = (i32)below(draw(seed, STREAM_COL, row, k++), (u64)cols);
        qsort(out, (size_t)L, sizeof(i32), cmp_i32);
        i32 w = 0;
        for (i32 q = 0; q < L; q++)
            if (w == 0 || out[q] != out[w - 1]) out[w++] = out[q];
        n = w;
    }
}

#define DEF_FILL(T, sfx)                                                                      \
    void synth_fill_uniform_##sfx(u64 seed, i64 row0, i64 nrows, i32 cols, const i32 *ptr,    \
                                  i32 *col, T *val) {                                         \
        _Pragma("omp parallel")                                                               \
        {                                                                                     \
            i32 *scratch = NULL;                                                              \
            _Pragma("omp for schedule(dynamic, 256)")                                         \
            for (i64 i = 0; i < nrows; i++) {                                                 \
                const i32 b = ptr[i], L = ptr[i + 1] - ptr[i];                                \
                const u64 row = (u64)(row0 + i);                                              \
                if ((i64)L * 2 > (i64)cols && !scratch)                                       \
                    scratch = (i32 *)malloc(sizeof(i32) * (size_t)cols);                      \
                row_columns(seed, row, L, cols, col + b, scratch);                            \
                for (i32 q = 0; q < L; q++)                                                   \
                    val[b + q] = (T)(2.0 * unit(draw(seed, STREAM_VAL, row, (u64)q)) - 1.0);  \
            }                                                                                 \
            free(scratch);                                                                    \
        }                                                                                     \
    }
DEF_FILL(float, s)
DEF_FILL(double, d)

/* ---- 27-point stencil on an n x n x n grid, x fastest, neighbours clipped at the faces ---- */

void synth_stencil27_rowlen(i32 n, i64 row0, i64 nrows, i32 *len) {
#pragma omp parallel for schedule(static)
    for (i64 i = 0; i < nrows; i++) {
        i64 r = row0 + i;
        i32 x = (i32)(r % n), y = (i32)((r / n) % n), z = (i32)(r / ((i64)n * n));
        i32 cx = 1 + (x > 0) + (x < n - 1), cy = 1 + (y > 0) + (y < n - 1),
            cz = 1 + (z > 0) + (z < n - 1);
        len[i] = cx * cy * cz;
    }
}

#define DEF_STENCIL(T, sfx)                                                                   \
    void synth_stencil27_fill_##sfx(i32 n, i64 row0, i64 nrows, const i32 *ptr, i32 *col,     \
                                    T *val, double diag, double off) {                        \
        _Pragma("omp parallel for schedule(static)")                                          \
        for (i64 i = 0; i < nrows; i++) {                                                     \
            i64 r = row0 + i;                                                                 \
            i32 x = (i32)(r % n), y = (i32)((r / n) % n), z = (i32)(r / ((i64)n * n));        \
            i32 w = ptr[i];                                                                   \
            for (i32 dz = -1; dz <= 1; dz++) {                                                \
                if (z + dz < 0 || z + dz >= n) continue;                                      \
                for (i32 dy = -1; dy <= 1; dy++) {                                            \
                    if (y + dy < 0 || y + dy >= n) continue;                                  \
                    for (i32 dx = -1; dx <= 1; dx++) {                                        \
                        if (x + dx < 0 || x + dx >= n) continue;                              \
                        i64 c = ((i64)(z + dz) * n + (y + dy)) * n + (x + dx);                \
                        col[w] = (i32)c;                                                      \
                        val[w] = (T)((dx == 0 && dy == 0 && dz == 0) ? diag : off);           \
                        w++;                                                                  \
                    }                                                                         \
                }                                                                             \
            }                                                                                 \
        }                                                                                     \
    }
DEF_STENCIL(float, s)
DEF_STENCIL(double, d)

/* ---- dense vectors / blocks: element i of stream `stream` uniform in [lo, hi) ----------- */

#define DEF_VEC(T, sfx)                                                                       \
    void synth_vector_##sfx(u64 seed, u64 stream, i64 first, i64 n, double lo, double hi,     \
                            T *out) {                                                         \
        _Pragma("omp parallel for schedule(static)")                                          \
        for (i64 i = 0; i < n; i++)                                                           \
            out[i] = (T)(lo + (hi - lo) * unit(draw(seed, 16 + stream, (u64)(first + i), 0)));\
    }
DEF_VEC(float, s)
DEF_VEC(double, d)
