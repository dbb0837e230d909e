"""Parity of alphasparse_{s,d}_mm (row-major) on the GPU with the reference's plain kernel."""
import numpy as np
import pytest
import torch

import oracle
from alsparse_b200 import capi, spblas, synth
from gpu_util import make_handle
from helpers import assert_rows_close, golden, mm_scale, structured_scale

pytestmark = pytest.mark.gpu


def run_mm(kind, A, m, X, columns, ldx, alpha, beta, Y0, ldy, device):
    if device:
        dX, dY = torch.from_numpy(X).cuda(), torch.from_numpy(Y0).cuda()
        st = spblas.mm(kind, 0, alpha, A, spblas.descr(), capi.ROW_MAJOR, dX, columns, ldx, beta, dY, ldy)
        torch.cuda.synchronize()
        Y = dY.cpu().numpy()
    else:
        Y = Y0.copy()
        st = spblas.mm(kind, 0, alpha, A, spblas.descr(), capi.ROW_MAJOR, X, columns, ldx, beta, Y, ldy)
    assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
    return Y


def compare(kind, m, Y, Yref, X, columns, ldx, alpha, beta, Y0, ldy, what):
    rows = m.nrows
    scale = mm_scale(m.ptr, m.col, m.val, X, columns, ldx, alpha, beta, Y0, ldy)
    assert_rows_close(kind, Y.reshape(rows, ldy)[:, :columns].reshape(-1),
                      Yref.reshape(rows, ldy)[:, :columns].reshape(-1), scale.reshape(-1), what)
    assert np.array_equal(Y.reshape(rows, ldy)[:, columns:], Y0.reshape(rows, ldy)[:, columns:]), "padding written"


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("case", ["w64", "w5"])
@pytest.mark.parametrize("device", [False, True])
def test_golden_vectors(kind, case, device):
    g = golden(f"mm_{kind}.npz")
    m = synth.Csr(int(g["rows"]), int(g["cols"]), 0, g["ptr"], g["col"], g["val"])
    columns, ldx, ldy = (int(v) for v in g[f"{case}_par"][:3])
    alpha, beta = float(g[f"{case}_par"][5]), float(g[f"{case}_par"][6])
    A = make_handle(kind, m)
    Y = run_mm(kind, A, m, g[f"{case}_X"], columns, ldx, alpha, beta, g[f"{case}_Y0"], ldy, device)
    compare(kind, m, Y, g[f"{case}_row"], g[f"{case}_X"], columns, ldx, alpha, beta, g[f"{case}_Y0"], ldy, case)
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("columns,ldx,ldy", [(64, 64, 64), (64, 80, 72), (1, 1, 1), (3, 3, 5), (32, 32, 32),
                                             (100, 100, 100), (128, 128, 128), (130, 131, 133), (256, 256, 256)])
def test_widths_and_leading_dimensions(kind, columns, ldx, ldy):
    m = synth.poisson(kind, 12, 3000, 2500, 32.0)
    lens = np.diff(m.ptr).copy()
    lens[::50] = 0
    lens[7] = 700
    m = synth.from_lengths(kind, 12, lens, 2500)
    X, Y0 = synth.vector(kind, 12, 3, m.cols * ldx), synth.vector(kind, 12, 4, m.nrows * ldy)
    A = make_handle(kind, m)
    for alpha, beta in ((1.0, 0.0), (1.5, 0.5)):
        Yref = oracle.gemm(kind, "row", m.rows_start, m.rows_end, m.col, m.val, alpha, X, columns, ldx, beta,
                           Y0.copy(), ldy)
        for device in (False, True):
            Y = run_mm(kind, A, m, X, columns, ldx, alpha, beta, Y0, ldy, device)
            compare(kind, m, Y, Yref, X, columns, ldx, alpha, beta, Y0, ldy, f"{columns}/{ldx}/{ldy} dev={device}")
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
def test_column_blocks_give_the_same_product(kind):
    """Row-major mm in column blocks (X slab by slab, Y accumulated over the passes): forced block counts on a
    small matrix against the oracle, with beta != 0 (applied by the first pass only), padded leading dimensions,
    empty rows, more blocks than some rows have elements, host operands; a matrix whose rows are not in ascending
    column order must fall back to one pass."""
    lens = synth.rowlen_poisson(13, 4000, 12.0, 3000).copy()
    lens[::40] = 0
    lens[11] = 900
    m = synth.from_lengths(kind, 13, lens, 3000)
    columns, ldx, ldy = 24, 28, 26
    X, Y0 = synth.vector(kind, 13, 3, m.cols * ldx), synth.vector(kind, 13, 4, m.nrows * ldy)
    A = make_handle(kind, m)
    try:
        for blocks in (1, 2, 5, 16):
            assert spblas.set_option("spmm_col_blocks", blocks) == capi.SUCCESS
            for alpha, beta in ((1.0, 0.0), (1.5, 0.5)):
                Yref = oracle.gemm(kind, "row", m.rows_start, m.rows_end, m.col, m.val, alpha, X, columns, ldx, beta,
                                   Y0.copy(), ldy)
                for device in (False, True):
                    Y = run_mm(kind, A, m, X, columns, ldx, alpha, beta, Y0, ldy, device)
                    compare(kind, m, Y, Yref, X, columns, ldx, alpha, beta, Y0, ldy, f"{blocks} column blocks dev={device}")
            assert spblas.mat_info(A)[1].spmm_col_blocks == blocks
        spblas.destroy(A)
        A = None
        # descending columns inside the rows: the blocks cannot be cut by searching, one pass it is
        ptr = m.ptr
        col, val = m.col.copy(), m.val.copy()
        for r in range(m.nrows):
            col[ptr[r]:ptr[r + 1]] = col[ptr[r]:ptr[r + 1]][::-1]
            val[ptr[r]:ptr[r + 1]] = val[ptr[r]:ptr[r + 1]][::-1]
        mr = synth.Csr(m.nrows, m.cols, 0, ptr, col, val)
        A = make_handle(kind, mr)
        assert spblas.set_option("spmm_col_blocks", 4) == capi.SUCCESS
        Yref = oracle.gemm(kind, "row", mr.rows_start, mr.rows_end, mr.col, mr.val, 2.0, X, columns, ldx, -1.0, Y0.copy(), ldy)
        Y = run_mm(kind, A, mr, X, columns, ldx, 2.0, -1.0, Y0, ldy, True)
        compare(kind, mr, Y, Yref, X, columns, ldx, 2.0, -1.0, Y0, ldy, "unsorted rows")
        assert spblas.mat_info(A)[1].spmm_col_blocks == 1
    finally:
        spblas.set_option("spmm_col_blocks", -1)
        if A is not None:
            spblas.destroy(A)


def test_status_codes():
    m = synth.poisson("s", 8, 30, 40, 4.0)
    A = make_handle("s", m)
    X, Y = np.zeros(40 * 4, np.float32), np.zeros(30 * 4, np.float32)
    g = spblas.descr()
    assert spblas.mm("s", 0, 1.0, A, g, 0, None, 4, 4, 0.0, Y, 4) == capi.NOT_INITIALIZED
    assert spblas.mm("d", 0, 1.0, A, g, 0, X, 4, 4, 0.0, Y, 4) == capi.INVALID_VALUE
    assert spblas.mm("s", capi.CONJUGATE_TRANSPOSE, 1.0, A, g, 0, X, 4, 4, 0.0, Y, 4) == capi.INVALID_VALUE
    assert spblas.mm("s", 0, 1.0, A, spblas.descr(capi.SYMMETRIC), 0, X, 4, 4, 0.0, Y, 4) == capi.INVALID_VALUE
    assert spblas.mm("s", 0, 1.0, A, spblas.descr(capi.TRIANGULAR), 0, X, 4, 4, 0.0, Y, 4) == capi.NOT_SUPPORTED  # not square
    assert spblas.mm("s", 0, 1.0, A, g, 0, X, 4, 3, 0.0, Y, 4) == capi.INVALID_VALUE           # ldx < columns
    assert spblas.mm("s", 0, 1.0, A, g, capi.COLUMN_MAJOR, X, 4, 39, 0.0, Y, 30) == capi.INVALID_VALUE  # ldx < cols
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("case", ["w64", "w5"])
def test_column_major_golden(kind, case):
    """Column-major operands against the reference's plain gemm_csr_col (golden vectors)."""
    g = golden(f"mm_{kind}.npz")
    m = synth.Csr(int(g["rows"]), int(g["cols"]), 0, g["ptr"], g["col"], g["val"])
    columns, _, _, ldxc, ldyc = (int(v) for v in g[f"{case}_par"][:5])
    alpha, beta = float(g[f"{case}_par"][5]), float(g[f"{case}_par"][6])
    A = make_handle(kind, m)
    Xc, Yc0, Yref = g[f"{case}_Xc"], g[f"{case}_Yc0"], g[f"{case}_col"]
    for dev in (False, True):
        if dev:
            dX, dY = torch.from_numpy(Xc).cuda(), torch.from_numpy(Yc0).cuda()
            st = spblas.mm(kind, 0, alpha, A, spblas.descr(), capi.COLUMN_MAJOR, dX, columns, ldxc, beta, dY, ldyc)
            Y = dY.cpu().numpy()
        else:
            Y = Yc0.copy()
            st = spblas.mm(kind, 0, alpha, A, spblas.descr(), capi.COLUMN_MAJOR, Xc, columns, ldxc, beta, Y, ldyc)
        assert st == capi.SUCCESS, capi.STATUS_NAMES[st]
        # compare through the row-major view of the same numbers
        rows, cols = m.nrows, m.cols
        Xr = Xc.reshape(columns, ldxc)[:, :cols].T.copy()
        Y0r = Yc0.reshape(columns, ldyc)[:, :rows].T.copy()
        scale = mm_scale(m.ptr, m.col, m.val, Xr.reshape(-1), columns, columns, alpha, beta, Y0r.reshape(-1), columns)
        assert_rows_close(kind, Y.reshape(columns, ldyc)[:, :rows].T.reshape(-1),
                          Yref.reshape(columns, ldyc)[:, :rows].T.reshape(-1), scale.reshape(-1), f"col {case} dev={dev}")
        assert np.array_equal(Y.reshape(columns, ldyc)[:, rows:], Yc0.reshape(columns, ldyc)[:, rows:]), "padding written"
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
def test_transposed_mm_both_layouts(kind):
    """op = TRANSPOSE: Y (cols x columns) = alpha * A^T * X (rows x columns) + beta * Y, checked against the
    oracle applied to the explicitly transposed matrix (what the reference's trans kernels do)."""
    m = synth.poisson(kind, 51, 900, 1300, 12.0)
    order = np.lexsort((np.repeat(np.arange(m.nrows), np.diff(m.ptr)), m.col))     # by column, then row
    trow = m.col[order]
    tptr = np.concatenate([[0], np.cumsum(np.bincount(trow, minlength=m.cols))]).astype(np.int32)
    tcol = np.repeat(np.arange(m.nrows), np.diff(m.ptr))[order].astype(np.int32)
    tval = m.val[order]
    A = make_handle(kind, m)
    columns, alpha, beta = 24, 0.75, -0.5
    # row-major
    X, Y0 = synth.vector(kind, 51, 3, m.nrows * columns), synth.vector(kind, 51, 4, m.cols * columns)
    Yref = oracle.gemm(kind, "row", tptr[:-1], tptr[1:], tcol, tval, alpha, X, columns, columns, beta, Y0.copy(), columns)
    Y = Y0.copy()
    assert spblas.mm(kind, capi.TRANSPOSE, alpha, A, spblas.descr(), capi.ROW_MAJOR, X, columns, columns, beta, Y,
                     columns) == capi.SUCCESS
    scale = mm_scale(tptr, tcol, tval, X, columns, columns, alpha, beta, Y0, columns)
    assert_rows_close(kind, Y, Yref, scale.reshape(-1), "transposed row-major")
    # column-major
    Xc, Yc0 = synth.vector(kind, 51, 5, m.nrows * columns), synth.vector(kind, 51, 6, m.cols * columns)
    Ycref = oracle.gemm(kind, "col", tptr[:-1], tptr[1:], tcol, tval, alpha, Xc, columns, m.nrows, beta, Yc0.copy(),
                        m.cols)
    dX, dY = torch.from_numpy(Xc).cuda(), torch.from_numpy(Yc0).cuda()
    assert spblas.mm(kind, capi.TRANSPOSE, alpha, A, spblas.descr(), capi.COLUMN_MAJOR, dX, columns, m.nrows, beta, dY,
                     m.cols) == capi.SUCCESS
    Xr = Xc.reshape(columns, m.nrows).T.copy()
    Y0r = Yc0.reshape(columns, m.cols).T.copy()
    sc = mm_scale(tptr, tcol, tval, Xr.reshape(-1), columns, columns, alpha, beta, Y0r.reshape(-1), columns)
    assert_rows_close(kind, dY.cpu().numpy().reshape(columns, m.cols).T.reshape(-1),
                      Ycref.reshape(columns, m.cols).T.reshape(-1), sc.reshape(-1), "transposed column-major")
    spblas.destroy(A)


def test_structured_descriptors_mm():
    """SYMMETRIC / TRIANGULAR / DIAGONAL descriptors in mm: every fill / diag / operation variant of the reference's
    symm / trmm / diagmm tables in both layouts against its plain kernels (golden vectors; the matrix stores some
    diagonals twice and some not at all), host and device operands; then a larger matrix against the oracle."""
    g = golden("struct_mm_d.npz")
    ptr, a, b = g["ptr"], float(g["alpha"]), float(g["beta"])
    columns, ldx, ldy, ldxc, ldyc = (int(v) for v in g["par"])
    n = 160
    m = synth.Csr(n, n, 0, ptr, g["col"], g["val"])
    A = make_handle("d", m)
    cases = 0
    for key in (k[4:] for k in g.files if k.startswith("row_")):
        t, upper, unit, tr = (int(f[1:]) for f in key.split("_"))
        for lay, layout, X, Y0, lx, ly in (("row", capi.ROW_MAJOR, g["Xr"], g["Yr"], ldx, ldy),
                                           ("col", capi.COLUMN_MAJOR, g["Xc"], g["Yc"], ldxc, ldyc)):
            view = (lambda v: v.reshape(n, ly)[:, :columns]) if lay == "row" else (lambda v: v.reshape(columns, ly)[:, :n].T)
            pad = (lambda v: v.reshape(n, ly)[:, columns:]) if lay == "row" else (lambda v: v.reshape(columns, ly)[:, n:])
            xv = X.reshape(n, lx)[:, :columns] if lay == "row" else X.reshape(columns, lx)[:, :n].T
            sc = structured_scale(n, ptr, g["col"], g["val"], xv, view(Y0), a, b)
            for dev in (False, True):
                if dev:
                    dX, dY = torch.from_numpy(X).cuda(), torch.from_numpy(Y0).cuda()
                    st = spblas.mm("d", tr, a, A, spblas.descr(t, upper, unit), layout, dX, columns, lx, b, dY, ly)
                    Y = dY.cpu().numpy()
                else:
                    Y = Y0.copy()
                    st = spblas.mm("d", tr, a, A, spblas.descr(t, upper, unit), layout, X, columns, lx, b, Y, ly)
                assert st == capi.SUCCESS, (key, lay, capi.STATUS_NAMES[st], spblas.last_error())
                assert_rows_close("d", view(Y).reshape(-1), view(g[f"{lay}_{key}"]).reshape(-1), sc.reshape(-1),
                                  f"{lay} {key} dev={dev}")
                assert np.array_equal(pad(Y), pad(Y0)), "padding written"
                cases += 1
    assert cases == 4 * (4 + 8 + 2)
    # no transposed symmetric kernel for real types in the reference's table; flags outside {0, 1} index past it
    X, Y = g["Xr"], g["Yr"].copy()
    assert spblas.mm("d", capi.TRANSPOSE, a, A, spblas.descr(capi.SYMMETRIC), 0, X, columns, ldx, b, Y, ldy) == capi.NOT_SUPPORTED
    assert spblas.mm("d", 0, a, A, spblas.descr(capi.TRIANGULAR, 2, 0), 0, X, columns, ldx, b, Y, ldy) == capi.INVALID_VALUE
    assert np.array_equal(Y, g["Yr"])
    spblas.destroy(A)

    for kind in ("s", "d"):
        n, columns = 3000, 16
        m = synth.poisson(kind, 73, n, n, 9.0)
        X, Y0 = synth.vector(kind, 73, 1, n * columns), synth.vector(kind, 73, 2, n * columns)
        A = make_handle(kind, m)
        sc = structured_scale(n, m.ptr, m.col, m.val, X.reshape(n, columns), Y0.reshape(n, columns), 1.25, 0.5)
        for t, upper, unit, tr in ((capi.SYMMETRIC, 0, 1, 0), (capi.TRIANGULAR, 1, 0, 1), (capi.TRIANGULAR, 0, 0, 0),
                                   (capi.DIAGONAL, 0, 0, 0)):
            Yref = oracle.structured_mm(kind, t, upper, unit, tr, "row", m.rows_start, m.rows_end, m.col, m.val, 1.25, X,
                                        columns, columns, 0.5, Y0.copy(), columns)
            dX, dY = torch.from_numpy(X).cuda(), torch.from_numpy(Y0).cuda()
            assert spblas.mm(kind, tr, 1.25, A, spblas.descr(t, upper, unit), capi.ROW_MAJOR, dX, columns, columns, 0.5, dY,
                             columns) == capi.SUCCESS
            assert_rows_close(kind, dY.cpu().numpy(), Yref, sc.reshape(-1), f"{kind} mm type {t}")
        spblas.destroy(A)


@pytest.mark.parametrize("ldy,beta", [(64, 0.0), (72, 0.5)])
def test_large_host_operands_take_the_windowed_path(ldy, beta):
    """Host X and Y above 32 MB: the product runs in row windows that overlap the copies of Y; results and the
    caller's padding must be what the single-launch path gives."""
    rows, cols, columns, ldx = 140001, 50000, 64, 64
    m = synth.poisson("s", 77, rows, cols, 6.0)
    X, Y0 = synth.vector("s", 77, 1, cols * ldx), synth.vector("s", 77, 2, rows * ldy)
    A = make_handle("s", m)
    Yref = oracle.gemm("s", "row", m.rows_start, m.rows_end, m.col, m.val, 1.25, X, columns, ldx, beta, Y0.copy(), ldy)
    Y = run_mm("s", A, m, X, columns, ldx, 1.25, beta, Y0, ldy, device=False)
    compare("s", m, Y, Yref, X, columns, ldx, 1.25, beta, Y0, ldy, f"windowed ldy={ldy}")
    Yd = run_mm("s", A, m, X, columns, ldx, 1.25, beta, Y0, ldy, device=True)
    assert np.array_equal(Y.reshape(rows, ldy)[:, :columns], Yd.reshape(rows, ldy)[:, :columns])  # same kernel, same sums
    spblas.destroy(A)


def _with_long_rows(kind, seed, rows, cols, mean, long_rows):
    """A Poisson(mean) matrix in which the rows named in `long_rows` (row -> length) are replaced by long ones."""
    base = synth.poisson(kind, seed, rows, cols, mean)
    rng = np.random.default_rng(seed)
    lens = np.diff(base.ptr).astype(np.int64)
    pieces_c, pieces_v = [], []
    for r in range(rows):
        if r in long_rows:
            c = np.sort(rng.choice(cols, long_rows[r], replace=False)).astype(np.int32)
            pieces_c.append(c)
            pieces_v.append(rng.uniform(-1, 1, len(c)).astype(base.val.dtype))
            lens[r] = len(c)
        else:
            pieces_c.append(base.col[base.ptr[r]:base.ptr[r + 1]])
            pieces_v.append(base.val[base.ptr[r]:base.ptr[r + 1]])
    ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    return synth.Csr(rows, cols, 0, ptr, np.concatenate(pieces_c), np.concatenate(pieces_v))


@pytest.mark.parametrize("kind", ["s", "d"])
def test_long_rows_are_multiplied_in_chunks(kind):
    """Rows above spmm_split_min elements leave the row pass and are multiplied chunk by chunk into partial sums that
    a last kernel adds onto Y: same product (fp32 rows stay short enough for the serial fp32 oracle), padding of Y
    untouched, beta applied once, first / last / neighbouring rows long, every pack width, transposed handle too."""
    rows, cols = 3000, 4000
    long_rows = {0: 1400, 1: 700, 1500: 1100, 2999: 900}
    m = _with_long_rows(kind, 95, rows, cols, 6.0, long_rows)
    try:
        assert spblas.set_option("spmm_split_min", 512) == capi.SUCCESS
        assert spblas.set_option("spmm_split_chunk", 128) == capi.SUCCESS
        A = make_handle(kind, m)
        for columns, ldx, ldy, beta in ((64, 64, 64, 0.0), (64, 72, 80, 0.5), (7, 7, 9, 0.5), (1, 1, 1, 0.0), (16, 16, 16, 1.0)):
            X, Y0 = synth.vector(kind, 95, 1, cols * ldx), synth.vector(kind, 95, 2, rows * ldy)
            Yref = oracle.gemm(kind, "row", m.rows_start, m.rows_end, m.col, m.val, 1.25, X, columns, ldx, beta, Y0.copy(), ldy)
            for device in (True, False):
                Y = run_mm(kind, A, m, X, columns, ldx, 1.25, beta, Y0, ldy, device)
                compare(kind, m, Y, Yref, X, columns, ldx, 1.25, beta, Y0, ldy, f"long rows {columns}/{ldx}/{ldy} dev={device}")
        # column-major operands: the same chunk tables, partial sums laid out column by column
        for columns, beta in ((6, 0.5), (1, 0.0)):
            ldx, ldy = cols + 3, rows + 5
            X, Y0 = synth.vector(kind, 99, 1, ldx * columns), synth.vector(kind, 99, 2, ldy * columns)
            Yref = oracle.gemm(kind, "col", m.rows_start, m.rows_end, m.col, m.val, 1.25, X, columns, ldx, beta, Y0.copy(), ldy)
            dX, dY = torch.from_numpy(X).cuda(), torch.from_numpy(Y0).cuda()
            assert spblas.mm(kind, 0, 1.25, A, spblas.descr(), capi.COLUMN_MAJOR, dX, columns, ldx, beta, dY, ldy) == capi.SUCCESS
            Y = dY.cpu().numpy()
            rid = np.repeat(np.arange(rows), np.diff(m.ptr))
            sc = np.zeros((columns, ldy))
            for c in range(columns):
                xs = X[c * ldx:c * ldx + cols].astype(np.float64)
                sc[c, :rows] = np.abs(beta * Y0[c * ldy:c * ldy + rows]) + 1.25 * np.bincount(
                    rid, weights=np.abs(m.val.astype(np.float64) * xs[m.col]), minlength=rows)
            assert_rows_close(kind, Y, Yref, sc.reshape(-1), f"column-major long rows, {columns} columns")
            pad = np.ones(ldy * columns, bool).reshape(columns, ldy)
            pad[:, :rows] = False
            assert np.array_equal(Y[pad.reshape(-1)], Y0[pad.reshape(-1)]), "padding written"
        # the same handle transposed: A^T has its own long rows (none here, its columns are short) and its own tables
        X, Y0 = synth.vector(kind, 96, 1, rows * 8), synth.vector(kind, 96, 2, cols * 8)
        st = spblas.mm(kind, capi.TRANSPOSE, 1.0, A, spblas.descr(), capi.ROW_MAJOR, torch.from_numpy(X).cuda(), 8, 8, 0.0,
                       torch.from_numpy(Y0).cuda(), 8)
        assert st == capi.SUCCESS
        spblas.destroy(A)
        # a matrix whose longest row stays under the limit builds no tables and runs the one pass
        small = synth.poisson(kind, 97, 2000, 2000, 5.0)
        A = make_handle(kind, small)
        X, Y0 = synth.vector(kind, 97, 1, 2000 * 8), synth.vector(kind, 97, 2, 2000 * 8)
        Yref = oracle.gemm(kind, "row", small.rows_start, small.rows_end, small.col, small.val, 1.0, X, 8, 8, 0.0, Y0.copy(), 8)
        before = spblas.launch_count()
        Y = run_mm(kind, A, small, X, 8, 8, 1.0, 0.0, Y0, 8, True)
        assert spblas.launch_count() - before == 1
        compare(kind, small, Y, Yref, X, 8, 8, 1.0, 0.0, Y0, 8, "no long rows")
        spblas.destroy(A)
    finally:
        spblas.set_option("spmm_split_min", -1)
        spblas.set_option("spmm_split_chunk", -1)


def test_long_rows_in_row_windows():
    """Host operands above 32 MB run in row windows; each window multiplies the chunks of its own long rows."""
    rows, cols, columns, ld = 140001, 50000, 64, 64
    long_rows = {0: 30000, 17500: 20000, 17501: 9000, 70000: 45000, 140000: 12000}
    m = _with_long_rows("s", 98, rows, cols, 6.0, long_rows)
    A = make_handle("s", m)          # default limits: rows above 1024 elements, chunks of 512
    X, Y0 = synth.vector("s", 98, 1, cols * ld), synth.vector("s", 98, 2, rows * ld)
    # fp32 rows of tens of thousands of elements: compare against the product accumulated in fp64
    Yref = oracle.gemm("d", "row", m.rows_start, m.rows_end, m.col, m.val.astype(np.float64), 1.25, X.astype(np.float64),
                       columns, ld, 0.5, Y0.astype(np.float64), ld).astype(np.float32)
    Y = run_mm("s", A, m, X, columns, ld, 1.25, 0.5, Y0, ld, device=False)
    compare("s", m, Y, Yref, X, columns, ld, 1.25, 0.5, Y0, ld, "windows")
    Yd = run_mm("s", A, m, X, columns, ld, 1.25, 0.5, Y0, ld, device=True)
    assert np.array_equal(Y, Yd)  # same kernels, same chunks, same sums
    spblas.destroy(A)
