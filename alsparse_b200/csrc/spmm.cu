// CSR x dense SpMM kernels for sm_100a, row-major dense operands.
//
// Y[r, :] = beta * Y[r, :] + sum over stored elements (alpha * a) * X[col, :], the operation
// of the reference's gemm_{s,d}_csr_row (arithmetic defined by
// src/plain/kernel/level3/mm/gemm/gemm_x_csr_row_plain.c:4-23: alpha is folded into the
// element before the accumulation).  The reference's own device build has no row-major SpMM
// (src/kernel/dcu/level3/mm/csrmm/dcu_gemm_x_csr_row.cpp:15-36 returns NOT_SUPPORTED).
//
// One warp owns one sparse row; its lanes span the dense columns, VEC consecutive columns
// per lane, so every stored element turns into one fully coalesced read of a row of X
// (64 fp32 columns = 256 bytes = 32 lanes x float2).  The warp fetches 32 (col, alpha*a)
// pairs with one coalesced load each and hands them round with shuffles; the loop over the
// 32 pairs is unrolled so several X rows are in flight per warp.  Bandwidth-bound: the
// traffic is nnz * columns * sizeof(T) of X rows against 2 flops per element, far below what
// would justify staging tiles for tensor cores.
#include "internal.h"

namespace asb {

template <typename T, int VEC>
struct Pack;
template <>
struct Pack<float, 1> { using type = float; };
template <>
struct Pack<float, 2> { using type = float2; };
template <>
struct Pack<float, 4> { using type = float4; };
template <>
struct Pack<double, 1> { using type = double; };
template <>
struct Pack<double, 2> { using type = double2; };

template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T *__restrict__ p, T (&out)[VEC]) {
    using P = typename Pack<T, VEC>::type;
    const P t = __ldg(reinterpret_cast<const P *>(p));
    const T *s = reinterpret_cast<const T *>(&t);
#pragma unroll
    for (int i = 0; i < VEC; i++) out[i] = s[i];
}

// VEC > 1 requires: columns % VEC == 0, ldx % VEC == 0, ldy % VEC == 0 and X, Y aligned to
// VEC * sizeof(T); the launcher checks and otherwise uses VEC == 1.
template <typename T, int VEC, bool HAS_BETA>
__global__ void __launch_bounds__(256)
    spmm_row_kernel(int rows, const int *__restrict__ row_ptr, const int *__restrict__ col,
                    const T *__restrict__ val, const T *__restrict__ X, int columns,
                    long long ldx, T *__restrict__ Y, long long ldy, T alpha, T beta) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (row >= rows) return;  // whole warp leaves together
    const int s = __ldg(row_ptr + row), e = __ldg(row_ptr + row + 1);

    for (int ct = 0; ct < columns; ct += 32 * VEC) {
        const int c = ct + lane * VEC;
        const bool live = c < columns;
        T acc[VEC];
#pragma unroll
        for (int i = 0; i < VEC; i++) acc[i] = T(0);

        for (int base = s; base < e; base += 32) {
            const int mine = base + lane;
            int cj = 0;
            T vj = T(0);
            if (mine < e) {
                cj = __ldcs(col + mine);
                vj = alpha * __ldcs(val + mine);
            }
            const int n = min(32, e - base);
            int k = 0;
            for (; k + 4 <= n; k += 4) {
                T xv[4][VEC];
                T av[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int cc = __shfl_sync(0xffffffffu, cj, k + u);
                    av[u] = __shfl_sync(0xffffffffu, vj, k + u);
                    if (live) load_vec<T, VEC>(X + (long long)cc * ldx + c, xv[u]);
                }
                if (live) {
#pragma unroll
                    for (int u = 0; u < 4; u++)
#pragma unroll
                        for (int i = 0; i < VEC; i++) acc[i] = fma(av[u], xv[u][i], acc[i]);
                }
            }
            for (; k < n; k++) {
                const int cc = __shfl_sync(0xffffffffu, cj, k);
                const T a = __shfl_sync(0xffffffffu, vj, k);
                if (live) {
                    T xv[VEC];
                    load_vec<T, VEC>(X + (long long)cc * ldx + c, xv);
#pragma unroll
                    for (int i = 0; i < VEC; i++) acc[i] = fma(a, xv[i], acc[i]);
                }
            }
        }

        if (live) {
            T *out = Y + row * ldy + c;
#pragma unroll
            for (int i = 0; i < VEC; i++) {
                T o = acc[i];
                if (HAS_BETA) o = fma(beta, out[i], o);
                acc[i] = o;
            }
            using P = typename Pack<T, VEC>::type;
            P packed;
            T *ps = reinterpret_cast<T *>(&packed);
#pragma unroll
            for (int i = 0; i < VEC; i++) ps[i] = acc[i];
            __stcs(reinterpret_cast<P *>(out), packed);
        }
    }
}

template <typename T, int VEC>
static void launch_row(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx, T beta, T *Y,
                       int ldy, cudaStream_t st) {
    const unsigned blocks = (unsigned)((ctx->rows + 7) / 8);
    const T *val = static_cast<const T *>(ctx->d_val);
    if (ctx->profile) cudaEventRecord(ctx->ev_start, st);
    if (beta == T(0))
        spmm_row_kernel<T, VEC, false><<<blocks, 256, 0, st>>>(
            (int)ctx->rows, ctx->d_row_ptr, ctx->d_col, val, X, columns, ldx, Y, ldy, alpha, beta);
    else
        spmm_row_kernel<T, VEC, true><<<blocks, 256, 0, st>>>(
            (int)ctx->rows, ctx->d_row_ptr, ctx->d_col, val, X, columns, ldx, Y, ldy, alpha, beta);
    if (ctx->profile) cudaEventRecord(ctx->ev_stop, st);
    count_launch();
}

template <typename T>
alphasparse_status_t launch_spmm_row(DeviceCtx *ctx, T alpha, const T *X, int columns, int ldx,
                                     T beta, T *Y, int ldy, cudaStream_t st) {
    if (ctx->rows == 0 || columns <= 0) return ALPHA_SPARSE_STATUS_SUCCESS;
    constexpr int MAXVEC = sizeof(T) == 4 ? 4 : 2;
    auto fits = [&](int vec) {
        const uintptr_t mask = (uintptr_t)(vec * sizeof(T) - 1);
        return columns % vec == 0 && ldx % vec == 0 && ldy % vec == 0 &&
               ((uintptr_t)X & mask) == 0 && ((uintptr_t)Y & mask) == 0;
    };
    // Widest pack that still gives every lane of the warp a column to work on.
    int vec = 1;
    if (MAXVEC >= 4 && columns >= 128 && fits(4)) vec = 4;
    else if (columns >= 64 && fits(2)) vec = 2;
    if constexpr (sizeof(T) == 4) {
        if (vec == 4) launch_row<T, 4>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
        else if (vec == 2) launch_row<T, 2>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
        else launch_row<T, 1>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    } else {
        if (vec == 2) launch_row<T, 2>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
        else launch_row<T, 1>(ctx, alpha, X, columns, ldx, beta, Y, ldy, st);
    }
    ASB_CUDA_OR(cudaGetLastError(), ALPHA_SPARSE_STATUS_EXECUTION_FAILED);
    return ALPHA_SPARSE_STATUS_SUCCESS;
}

template alphasparse_status_t launch_spmm_row<float>(DeviceCtx *, float, const float *, int, int,
                                                     float, float *, int, cudaStream_t);
template alphasparse_status_t launch_spmm_row<double>(DeviceCtx *, double, const double *, int, int,
                                                      double, double *, int, cudaStream_t);

}  // namespace asb
