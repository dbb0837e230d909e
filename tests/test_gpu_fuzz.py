"""Seeded random shapes, row-length distributions and analysis options through mv and both mm layouts against the
oracle's plain kernels (fp64 comparand, so that single-precision rows of thousands of elements can be judged)."""
import numpy as np
import pytest
import torch

import oracle
from alsparse_b200 import capi, spblas, synth
from helpers import TOL

pytestmark = pytest.mark.gpu


def _lengths(rng, rows, cols):
    shape = int(rng.integers(4))
    seed = int(rng.integers(1 << 30))
    if shape == 0:      # power law
        lens = synth.rowlen_zipf(seed, rows, 1.5 + rng.random(), 1, min(cols, int(rng.integers(1, 60000))))
    elif shape == 1:    # even
        lens = synth.rowlen_poisson(seed, rows, rng.random() * 40, cols)
    elif shape == 2:    # short rows and a few very long ones
        lens = synth.rowlen_poisson(seed, rows, 3.0, cols).copy()
        for _ in range(int(rng.integers(1, 8))):
            lens[rng.integers(rows)] = min(cols, int(rng.integers(100, 70000)))
    else:               # mostly empty
        lens = np.zeros(rows, np.int32)
        lens[rng.integers(rows, size=max(1, rows // 50))] = min(cols, int(rng.integers(1, 3000)))
    lens = np.minimum(lens, cols).astype(np.int32)
    if lens.sum() > 3_000_000:
        lens = (lens * (3_000_000 / lens.sum())).astype(np.int32)
    return lens


def _options(rng):
    if rng.random() < 0.3:
        return {}
    pick = lambda *v: int(rng.choice(v))
    return dict(band_bytes=pick(1024, 4096, 16384, 65536), band_min_seg=pick(1, 2, 6, 12), band_min_rows=pick(1, 4, 128),
                band_min_share_pct=pick(0, 10), bin_short=pick(0, 2, 16), bin_mid0=pick(8, 32), bin_mid1=pick(64, 256),
                bin_mid_max=pick(512, 16384), band_packed=pick(0, 1), bin_sort=pick(0, 1), spmm_split_min=pick(0, 64, 1024),
                spmm_split_chunk=pick(64, 512), mv_block_min_kb=pick(0, 1, 98304), mv_block_kb=pick(16, 256))


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_and_options(seed):
    rng = np.random.default_rng(seed)
    seen = set()
    for it in range(10):
        kind = "sd"[int(rng.integers(2))]
        rows, cols = int(rng.integers(1, 60000)), int(rng.integers(1, 90000))
        m = synth.from_lengths(kind, int(rng.integers(1 << 30)), _lengths(rng, rows, cols), cols)
        opts = _options(rng)
        try:
            for k, v in opts.items():
                assert spblas.set_option(k, v) == capi.SUCCESS, k
            st, A = spblas.create_csr(kind, capi.BASE_ZERO, rows, cols, m.rows_start, m.rows_end, m.col, m.val)
            assert st == capi.SUCCESS, spblas.last_error()
            info = spblas.mat_info(A)[1]
            seen.add((int(info.algorithm), int(info.binned), info.band_rows > 0))
            what = f"seed {seed} case {it} {kind} {rows}x{cols} nnz {m.nnz} options {opts}"
            alpha, beta = float(rng.choice([1.0, 1.5, -0.5])), float(rng.choice([0.0, 0.5, 1.0]))
            v64 = m.val.astype(np.float64)
            rid = np.repeat(np.arange(rows), np.diff(m.ptr))
            slack = 4 if kind == "s" else 1     # the comparand is fp64: room for the rounding of the fp32 result itself

            x, y0 = synth.vector(kind, it, 1, cols), synth.vector(kind, it, 2, rows)
            x64 = x.astype(np.float64)
            ref = oracle.gemv("d", m.rows_start, m.rows_end, m.col, v64, alpha, x64, beta, y0.astype(np.float64))
            scale = np.abs(beta * y0) + abs(alpha) * np.bincount(rid, weights=np.abs(v64 * x64[m.col]), minlength=rows)
            dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
            assert spblas.mv(kind, 0, alpha, A, spblas.descr(), dx, beta, dy) == capi.SUCCESS, what
            err = np.abs(dy.cpu().numpy().astype(np.float64) - ref)
            assert (err <= slack * TOL[kind] * scale + 1e-300).all(), "mv " + what

            columns = int(rng.choice([1, 3, 8, 64]))
            X, Y0 = synth.vector(kind, it, 3, cols * columns), synth.vector(kind, it, 4, rows * columns)
            X64 = X.astype(np.float64)
            for lay, layout in (("row", capi.ROW_MAJOR), ("col", capi.COLUMN_MAJOR)):
                ldx, ldy = (columns, columns) if lay == "row" else (cols, rows)
                ref = oracle.gemm("d", lay, m.rows_start, m.rows_end, m.col, v64, alpha, X64, columns, ldx, beta,
                                  Y0.astype(np.float64), ldy)
                dX, dY = torch.from_numpy(X).cuda(), torch.from_numpy(Y0).cuda()
                assert spblas.mm(kind, 0, alpha, A, spblas.descr(), layout, dX, columns, ldx, beta, dY, ldy) == capi.SUCCESS, what
                if lay == "row":
                    sc = np.abs(beta * Y0.reshape(rows, columns)).astype(np.float64)
                    np.add.at(sc, rid, abs(alpha) * np.abs(v64[:, None] * X64.reshape(cols, columns)[m.col]))
                    sc = sc.reshape(-1)
                else:
                    sc = np.abs(beta * Y0).astype(np.float64)
                    for c in range(columns):
                        sc[c * rows:(c + 1) * rows] += abs(alpha) * np.bincount(
                            rid, weights=np.abs(v64 * X64[c * cols:(c + 1) * cols][m.col]), minlength=rows)
                err = np.abs(dY.cpu().numpy().astype(np.float64) - ref)
                assert (err <= slack * TOL[kind] * sc + 1e-300).all(), f"mm {lay} x{columns} " + what
            assert spblas.kernel_status(A) == (capi.SUCCESS, 0), what
            spblas.destroy(A)
        finally:
            for k in opts:
                spblas.set_option(k, -1)
    assert len(seen) >= 2, seen   # the draws reached more than one kernel family


@pytest.mark.parametrize("seed", [21, 22])
def test_random_transposed_and_structured_products(seed):
    """The matrices derived on the device (A^T, kept triangle, mirror image, unit diagonal, diagonal only) from random
    square matrices, half of them with rows in shuffled column order and diagonals stored twice."""
    rng = np.random.default_rng(seed)
    for it in range(8):
        n = int(rng.integers(1, 40000))
        shape, s = int(rng.integers(3)), int(rng.integers(1 << 30))
        if shape == 0:
            lens = synth.rowlen_zipf(s, n, 1.6 + rng.random(), 1, min(n, int(rng.integers(1, 30000))))
        elif shape == 1:
            lens = synth.rowlen_poisson(s, n, rng.random() * 30, n)
        else:
            lens = synth.rowlen_poisson(s, n, 2.0, n).copy()
            for _ in range(3):
                lens[rng.integers(n)] = min(n, int(rng.integers(50, 30000)))
        lens = np.minimum(lens, n).astype(np.int32)
        if lens.sum() > 2_000_000:
            lens = (lens * (2_000_000 / lens.sum())).astype(np.int32)
        m = synth.from_lengths("d", s, lens, n)
        col, val = m.col.copy(), m.val.copy()
        if rng.random() < 0.5:
            for r in rng.integers(0, n, 200):
                a, b = m.ptr[r], m.ptr[r + 1]
                p = rng.permutation(b - a)
                col[a:b], val[a:b] = col[a:b][p], val[a:b][p]
                if b - a >= 2 and rng.random() < 0.5:
                    col[a] = col[b - 1] = r
        st, A = spblas.create_csr("d", capi.BASE_ZERO, n, n, m.rows_start, m.rows_end, col, val)
        assert st == capi.SUCCESS, spblas.last_error()
        x, y0 = synth.vector("d", it, 1, n), synth.vector("d", it, 2, n)
        rid = np.repeat(np.arange(n), np.diff(m.ptr))
        scale = np.abs(0.5 * y0) + 1.25 * (np.bincount(rid, weights=np.abs(val * x[col]), minlength=n) +
                                           np.bincount(col, weights=np.abs(val * x[rid]), minlength=n) + np.abs(x))
        cases = [(capi.GENERAL, 0, 0, 1)]
        for t in (capi.SYMMETRIC, capi.TRIANGULAR, capi.DIAGONAL):
            cases.append((t, int(rng.integers(2)), int(rng.integers(2)), int(rng.integers(2)) if t == capi.TRIANGULAR else 0))
        for t, upper, unit, trans in cases:
            if t == capi.GENERAL:
                ref = oracle.gemv_trans("d", n, m.rows_start, m.rows_end, col, val, 1.25, x, 0.5, y0.copy())
                descr = spblas.descr()
            else:
                ref = oracle.structured_mv("d", t, upper, unit, trans, m.rows_start, m.rows_end, col, val, 1.25, x, 0.5, y0.copy())
                descr = spblas.descr(t, upper, unit)
            dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
            assert spblas.mv("d", trans, 1.25, A, descr, dx, 0.5, dy) == capi.SUCCESS, spblas.last_error()
            err = np.abs(dy.cpu().numpy() - ref)
            assert (err <= TOL["d"] * scale + 1e-300).all(), f"seed {seed} case {it} n {n} type {t} {upper}{unit}{trans}"
        spblas.destroy(A)
