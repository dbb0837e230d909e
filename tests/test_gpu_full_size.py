"""Parity at the full sizes of the benchmark configurations, through checks that need no full-size CPU run:

* a few thousand sampled rows (the first, the last, the longest and random ones) against the oracle's plain kernel,
  fed with those rows cut out of the same matrix and the full-length x;
* identical bits from one call to the next;
* linearity, A(2 x1 - 3 x2) = 2 A x1 - 3 A x2, within the parity tolerance on every row;
* a checksum, sum(A x) = (column sums of A) . x, within the tolerance on the whole sum;
* the reference's own pass criterion (the residual of its check_{s,d}_l2 / _l3, at most 50), computed on the whole
  result against the oracle's OpenMP kernel on the whole matrix, and printed beside the per-row gate.

The per-row scale |A||x| that the tolerances multiply is computed with torch on the GPU from the same arrays.
"""
import numpy as np
import pytest
import torch

import bench
import oracle
from alsparse_b200 import capi, spblas, synth
from gpu_util import TORCH, make_handle
from helpers import TOL, assert_rows_close, mm_scale, row_scale

pytestmark = pytest.mark.gpu


def build(name):
    cfg = bench.WORKLOADS[name]
    lens = bench.global_row_lengths(name, cfg)
    return cfg, bench.local_block(name, cfg, lens, 0, len(lens))


def cut_rows(m, rng, n_random):
    """Sorted distinct row numbers and those rows as a small CSR (local offsets, global columns)."""
    lens = np.diff(m.ptr)
    longest = np.argpartition(lens, -8)[-8:]
    pick = np.unique(np.concatenate([rng.integers(0, m.nrows, n_random), [0, m.nrows - 1], longest]))
    sub_lens = lens[pick]
    ptr = np.concatenate([[0], np.cumsum(sub_lens)]).astype(np.int32)
    idx = np.concatenate([np.arange(m.ptr[r], m.ptr[r + 1], dtype=np.int64) for r in pick])
    return pick, ptr, m.col[idx], m.val[idx]


def abs_row_sums(m, absx):
    """|A| |x| per row in double precision, on the GPU."""
    col = torch.from_numpy(m.col).cuda()
    prod = torch.from_numpy(m.val).cuda().abs().double() * absx.double().index_select(0, col)
    del col
    lens = torch.from_numpy(np.diff(m.ptr).astype(np.int64)).cuda()
    return torch.segment_reduce(prod, "sum", lengths=lens)


@pytest.mark.parametrize("name", ["uniform16", "stencil27", "powerlaw"])
def test_full_size_mv(name):
    cfg, m = build(name)
    kind, alpha, beta = cfg["kind"], cfg["alpha"], cfg["beta"]
    A = make_handle(kind, m)
    x1, x2, y0 = synth.vector(kind, 1, 1, m.cols), synth.vector(kind, 1, 2, m.cols), synth.vector(kind, 1, 3, m.nrows)
    dx1, dx2 = torch.from_numpy(x1).cuda(), torch.from_numpy(x2).cuda()
    descr = spblas.descr()

    def product(dx, a, b):
        dy = torch.from_numpy(y0).cuda()
        assert spblas.mv(kind, 0, a, A, descr, dx, b, dy) == capi.SUCCESS, spblas.last_error()
        return dy

    # sampled rows against the oracle, with the configuration's own scalars
    y = product(dx1, alpha, beta)
    pick, sptr, scol, sval = cut_rows(m, np.random.default_rng(1), 4000)
    y_ref = oracle.gemv(kind, sptr[:-1], sptr[1:], scol, sval, alpha, x1, beta, y0[pick].copy())
    y_host = y.cpu().numpy()
    assert_rows_close(kind, y_host[pick], y_ref, row_scale(sptr, scol, sval, x1, alpha, beta, y0[pick]), f"{name} sampled rows")
    assert np.isfinite(y_host).all()
    # the reference's own criterion on the whole vector (its tests compare two implementations this way)
    y_all = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, alpha, x1, beta, y0.copy(), threads=oracle.max_threads())
    resid = oracle.check_l2_residual(kind, y_all, y_host, x1, alpha, beta, m.nrows, m.cols, m.col, m.val)
    print(f"{name}: reference check_{kind}_l2 residual {resid:.3g} (passes at <= {oracle.CHECK_THRESHOLD:g})")
    assert resid <= oracle.CHECK_THRESHOLD
    # identical bits on a second call
    assert torch.equal(y, product(dx1, alpha, beta))

    # linearity and the checksum, beta = 0
    ya, yb, yc = product(dx1, 1.0, 0.0), product(dx2, 1.0, 0.0), product(2.0 * dx1 - 3.0 * dx2, 1.0, 0.0)
    scale = abs_row_sums(m, 2.0 * dx1.abs() + 3.0 * dx2.abs())
    err = (yc.double() - (2.0 * ya.double() - 3.0 * yb.double())).abs()
    # three products and the combination each round once: four times the single-product tolerance
    worst = (err - 4.0 * TOL[kind] * scale).max().item()
    assert worst <= 0.0, f"{name}: linearity off by {worst:g} beyond the tolerance"
    colsum = torch.zeros(m.cols, dtype=torch.float64, device="cuda")
    colsum.index_add_(0, torch.from_numpy(m.col).cuda(), torch.from_numpy(m.val).cuda().double())
    want = torch.dot(colsum, dx1.double()).item()
    got = ya.double().sum().item()
    total_scale = abs_row_sums(m, dx1.abs()).sum().item()
    assert abs(got - want) <= TOL[kind] * total_scale, (name, got, want, total_scale)
    spblas.destroy(A)


def test_full_size_mm():
    cfg, m = build("spmm64")
    kind, columns = cfg["kind"], cfg["columns"]
    A = make_handle(kind, m)
    X = synth.vector(kind, 2, 1, m.cols * columns)
    Y0 = synth.vector(kind, 2, 2, m.nrows * columns)
    dX = torch.from_numpy(X).cuda()

    def product(a, b):
        dY = torch.from_numpy(Y0).cuda()
        assert spblas.mm(kind, 0, a, A, spblas.descr(), capi.ROW_MAJOR, dX, columns, columns, b, dY, columns) == capi.SUCCESS
        return dY

    Y = product(1.5, 0.5)
    pick, sptr, scol, sval = cut_rows(m, np.random.default_rng(2), 3000)
    Y0s = np.ascontiguousarray(Y0.reshape(m.nrows, columns)[pick]).reshape(-1)
    Y_ref = oracle.gemm(kind, "row", sptr[:-1], sptr[1:], scol, sval, 1.5, X, columns, columns, 0.5, Y0s.copy(), columns)
    got = Y.cpu().numpy().reshape(m.nrows, columns)[pick].reshape(-1)
    scale = mm_scale(sptr, scol, sval, X, columns, columns, 1.5, 0.5, Y0s, columns)
    assert_rows_close(kind, got, Y_ref, scale.reshape(-1), "spmm64 sampled rows")
    Y_all = oracle.gemm(kind, "row", m.rows_start, m.rows_end, m.col, m.val, 1.5, X, columns, columns, 0.5, Y0.copy(), columns,
                        threads=oracle.max_threads())
    resid = oracle.check_l3_residual(kind, Y_all, Y.cpu().numpy(), X, m.nrows, m.cols, columns, columns, columns, columns,
                                     m.col, m.val)
    print(f"spmm64: reference check_{kind}_l3 residual {resid:.3g} (passes at <= {oracle.CHECK_THRESHOLD:g})")
    assert resid <= oracle.CHECK_THRESHOLD
    assert torch.equal(Y, product(1.5, 0.5))
    assert TORCH[kind] == Y.dtype
    spblas.destroy(A)
