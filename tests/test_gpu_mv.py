"""Parity of alphasparse_{s,d}_mv on the GPU with the reference's plain kernel (through the oracle),
against the committed golden vectors and on fresh seeded inputs, including the edge cases."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle
from alsparse_b200 import capi, spblas, synth
from gpu_util import TORCH, check_mv, download, make_handle
from helpers import NP, assert_rows_close, golden, row_scale

pytestmark = pytest.mark.gpu
ALGS = [capi.ALG_VECTOR, capi.ALG_MERGE, capi.ALG_ROWTILE]


def _csr(g):
    return synth.Csr(int(g["rows"]), int(g["cols"]), 0, g["ptr"], g["col"], g["val"])


def test_kat_3x3_and_index_base():
    g = golden("kat3x3.npz")
    for base in (0, 1):
        st, A = spblas.create_csr("s", base, 3, 3, g["rs"] + base, g["re"] + base, g["col"] + base, g["val"])
        assert st == capi.SUCCESS
        y = np.ones(3, np.float32)
        assert spblas.mv("s", 0, 2.0, A, spblas.descr(), g["x"], 3.0, y) == capi.SUCCESS
        assert y.tolist() == [405.0, 63.0, 11.0]
        st, b, rows, cols, rs, re_, col, val = spblas.export_csr("s", A)
        assert (st, b, rows, cols) == (0, 0, 3, 3)
        assert rs.tolist() == [0, 2, 3] and re_.tolist() == [2, 3, 4] and col.tolist() == [0, 2, 1, 0]
        Y = np.zeros(6, np.float32)
        assert spblas.mm("s", 0, 1.0, A, spblas.descr(), capi.ROW_MAJOR, g["B"], 2, 2, 0.0, Y, 2) == capi.SUCCESS
        assert Y.tolist() == g["mm_row"].tolist()
        spblas.destroy(A)


@pytest.mark.parametrize("alg", [None] + ALGS)
@pytest.mark.parametrize("name,kind", [("cfg1_s.npz", "s"), ("zipf_d.npz", "d"), ("stencil8_d.npz", "d")])
def test_golden_vectors(name, kind, alg):
    """Known answers produced by the reference's own objects."""
    g = golden(name)
    m = _csr(g)
    if alg is not None:
        spblas.set_algorithm(alg)
    A = make_handle(kind, m)
    spblas.set_algorithm(capi.ALG_AUTO)
    cases = [(float(g["alpha"]), float(g["beta"]), g["y"])]
    if name == "cfg1_s.npz":
        cases.append((1.5, 0.5, g["y_ab"]))
    for alpha, beta, y_ref in cases:
        for dev in (False, True):
            if dev:
                dx, dy = torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g["y0"]).cuda()
                assert spblas.mv(kind, 0, alpha, A, spblas.descr(), dx, beta, dy) == capi.SUCCESS
                y = dy.cpu().numpy()
            else:
                y = g["y0"].copy()
                assert spblas.mv(kind, 0, alpha, A, spblas.descr(), g["x"], beta, y) == capi.SUCCESS
            assert_rows_close(kind, y, y_ref, row_scale(m.ptr, m.col, m.val, g["x"], alpha, beta, g["y0"]), name)
    spblas.destroy(A)


def test_device_copy_and_coo_conversion_are_bit_exact():
    """Index handling: device CSR == oracle create_csr; COO->CSR == the reference's conversion."""
    g = golden("cfg1_s.npz")
    st, coo = spblas.create_coo("s", capi.BASE_ONE, 1000, 1000, len(g["coo_ri"]), g["coo_ri"] + 1, g["coo_ci"] + 1,
                                g["coo_v"])
    assert st == capi.SUCCESS
    st, A = spblas.convert_csr(coo, capi.NON_TRANSPOSE)
    assert st == capi.SUCCESS, spblas.last_error()
    st, base, rows, cols, rs, re_, col, val = spblas.export_csr("s", A)
    assert (st, base, rows, cols) == (0, 0, 1000, 1000)
    ptr = np.concatenate([rs[:1], re_])
    assert np.array_equal(ptr, g["csr_ptr"]) and np.array_equal(col, g["csr_col"])
    assert np.array_equal(val.view(np.uint32), g["csr_val"].view(np.uint32))
    st, d_ptr, d_col, d_val = spblas.device_csr(A)
    assert st == capi.SUCCESS
    assert np.array_equal(download(d_ptr, 1001, torch.int32), g["csr_ptr"])
    assert np.array_equal(download(d_col, 5000, torch.int32), g["csr_col"])
    assert np.array_equal(download(d_val, 5000, torch.float32).view(np.uint32), g["csr_val"].view(np.uint32))
    y = np.zeros(1000, np.float32)
    assert spblas.mv("s", 0, 1.0, A, spblas.descr(), g["x"], 0.0, y) == capi.SUCCESS
    assert_rows_close("s", y, g["y"], row_scale(g["ptr"], g["col"], g["val"], g["x"], 1.0, 0.0, g["y0"]), "coo path")
    # transposed conversion: A^T built from the COO, checked against the oracle on swapped indices
    st, At = spblas.convert_csr(coo, capi.TRANSPOSE)
    assert st == capi.SUCCESS
    _, _, _, _, trs, tre, tcol, tval = spblas.export_csr("s", At)
    op, oc, ov = oracle.coo_to_csr("s", 0, 1000, g["coo_ci"], g["coo_ri"], g["coo_v"])
    assert np.array_equal(np.concatenate([trs[:1], tre]), op) and np.array_equal(tcol, oc) and np.array_equal(tval, ov)
    for h in (coo, A, At):
        spblas.destroy(h)
    # one-based create_csr against the oracle's create_csr
    m = synth.poisson("d", 2, 700, 900, 7.0)
    op, oc, ov = oracle.create_csr("d", 1, m.rows_start + 1, m.rows_end + 1, m.col + 1, m.val)
    A = make_handle("d", m, base=1)
    _, d_ptr, d_col, d_val = spblas.device_csr(A)
    assert np.array_equal(download(d_ptr, 701, torch.int32), op)
    assert np.array_equal(download(d_col, m.nnz, torch.int32), oc)
    assert np.array_equal(download(d_val, m.nnz, torch.float64), ov)
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("alg", ALGS)
@pytest.mark.parametrize("pointers", ["host", "device"])
def test_shapes_and_scalars(kind, alg, pointers):
    """Row-length regimes of the benchmark configurations at sizes the oracle finishes instantly."""
    mats = [synth.uniform_fixed(kind, 1, 20000, 20000, 16), synth.poisson(kind, 2, 9000, 7000, 32.0),
            synth.stencil27(kind, 14), synth.uniform_fixed(kind, 3, 5000, 300, 1),
            synth.uniform_fixed(kind, 4, 777, 50, 3)]
    # rows of up to 200,000 elements in both precisions (single precision is compared with a double-precision sum)
    mats.append(synth.zipf(kind, 5, 30000, 250000, 1.8, 1, 200000))
    for m in mats:
        for alpha, beta in ((1.0, 0.0), (1.5, 0.5), (-2.0, 1.0), (0.0, 3.0)):
            check_mv(kind, m, alpha, beta, pointers=pointers, alg=alg)


@pytest.mark.parametrize("alg", ALGS)
def test_edge_cases(alg):
    kind = "d"
    # empty rows at the front, in runs, at the back; a single row; a single element
    lens = np.zeros(3000, np.int32)
    lens[100:200] = 5
    lens[1500] = 2500
    lens[2000:2500:3] = 1
    check_mv(kind, synth.from_lengths(kind, 1, lens, 4000), 2.0, 0.5, alg=alg)
    check_mv(kind, synth.from_lengths(kind, 2, np.array([7]), 9), 1.0, 0.0, alg=alg)
    check_mv(kind, synth.from_lengths(kind, 3, np.array([1]), 1), 3.0, 2.0, alg=alg)
    check_mv(kind, synth.from_lengths(kind, 4, np.array([0, 0, 1, 0]), 5), 3.0, 2.0, alg=alg)
    # one row of 200000 elements (the clip of the power-law configuration) between short rows
    lens = np.ones(2001, np.int32)
    lens[1000] = 200000
    check_mv(kind, synth.from_lengths(kind, 5, lens, 300000), 1.0, 0.0, alg=alg)
    # a dense row (every column) and more rows than columns
    lens = np.full(64, 64, np.int32)
    check_mv(kind, synth.from_lengths(kind, 6, lens, 64), -1.0, 1.0, alg=alg)
    # beta == 0 must not read y: NaNs in y0 do not propagate (the oracle computes y*0 = NaN, so compare to a clean run)
    m = synth.poisson(kind, 7, 500, 500, 6.0)
    x = synth.vector(kind, 7, 1, 500)
    spblas.set_algorithm(alg)
    A = make_handle(kind, m)
    spblas.set_algorithm(capi.ALG_AUTO)
    y = np.full(500, np.nan)
    assert spblas.mv(kind, 0, 1.0, A, spblas.descr(), x, 0.0, y) == capi.SUCCESS
    y_ref = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, 1.0, x, 0.0, np.zeros(500))
    assert_rows_close(kind, y, y_ref, row_scale(m.ptr, m.col, m.val, x, 1.0, 0.0, np.zeros(500)), "beta=0")
    spblas.destroy(A)


def test_no_stored_elements_and_no_rows():
    # nnz == 0: the CPU kernels still scale y by beta
    ptr = np.zeros(6, np.int32)
    st, A = spblas.create_csr("s", 0, 5, 4, ptr[:-1], ptr[1:], np.zeros(0, np.int32), np.zeros(0, np.float32))
    assert st == capi.SUCCESS
    y = np.arange(5, dtype=np.float32)
    assert spblas.mv("s", 0, 1.0, A, spblas.descr(), np.ones(4, np.float32), 2.0, y) == capi.SUCCESS
    assert y.tolist() == [0, 2, 4, 6, 8]
    spblas.destroy(A)
    # rows == 0: success, nothing touched (the reference would read rows_end[-1])
    st, A = spblas.create_csr("d", 0, 0, 4, None, None, None, None)
    assert st == capi.SUCCESS
    y = np.ones(1)
    assert spblas.mv("d", 0, 1.0, A, spblas.descr(), np.ones(4), 2.0, y) == capi.SUCCESS and y[0] == 1.0
    spblas.destroy(A)


def test_unsorted_columns_and_duplicates():
    """create_csr does not sort or merge: duplicates are summed by the product, as on the CPU."""
    rng = np.random.default_rng(3)
    rows, cols = 400, 60
    lens = rng.integers(0, 40, rows).astype(np.int32)
    ptr = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    col = rng.integers(0, cols, ptr[-1]).astype(np.int32)  # unsorted, with repeats
    val = rng.uniform(-1, 1, ptr[-1])
    m = synth.Csr(rows, cols, 0, ptr, col, val)
    for alg in ALGS:
        check_mv("d", m, 1.25, -0.5, alg=alg)


def test_status_codes_on_live_handles():
    m = synth.poisson("s", 8, 30, 40, 4.0)
    A = make_handle("s", m)
    x, y = np.zeros(40, np.float32), np.zeros(30, np.float32)
    g = spblas.descr()
    assert spblas.mv("s", 0, 1.0, A, g, None, 0.0, y) == capi.NOT_INITIALIZED
    assert spblas.mv("s", 0, 1.0, A, g, x, 0.0, None) == capi.NOT_INITIALIZED
    assert spblas.mv("d", 0, 1.0, A, g, x, 0.0, y) == capi.INVALID_VALUE
    assert spblas.mv("s", capi.CONJUGATE_TRANSPOSE, 1.0, A, g, x, 0.0, y) == capi.INVALID_VALUE
    assert spblas.mv("s", 0, 1.0, A, spblas.descr(capi.SYMMETRIC), x, 0.0, y) == capi.INVALID_VALUE  # 30 x 40
    assert spblas.mv("s", 0, 1.0, A, spblas.descr(7), x, 0.0, y) == capi.INVALID_VALUE
    assert spblas.mv("s", 0, 1.0, A, spblas.descr(capi.DIAGONAL), x, 0.0, y) == capi.NOT_SUPPORTED
    # the same precedence the oracle's restatement of the reference's checks gives
    assert oracle.mv_status(has_x=0) == capi.NOT_INITIALIZED
    assert oracle.mv_status(handle_datatype=0, call_datatype=1) == capi.INVALID_VALUE
    assert oracle.mv_status(descr_type=1, rows=30, cols=40) == capi.INVALID_VALUE
    st, info = spblas.mat_info(A)
    assert st == capi.SUCCESS and (info.rows, info.cols, info.nnz) == (30, 40, m.nnz)
    assert info.max_row_nnz == int(np.diff(m.ptr).max()) and info.empty_rows == int((np.diff(m.ptr) == 0).sum())
    spblas.destroy(A)
    # out-of-range column index: refused at creation instead of faulting later
    bad = m.col.copy()
    bad[3] = 40
    st, B = spblas.create_csr("s", 0, 30, 40, m.rows_start, m.rows_end, bad, m.val)
    assert st == capi.INVALID_VALUE and not B.value


def test_analysis_picks_by_row_shape():
    A = make_handle("s", synth.uniform_fixed("s", 1, 4096, 4096, 16))
    _, info = spblas.mat_info(A)
    assert info.algorithm == capi.ALG_VECTOR and info.lanes_per_row == 4   # random columns: no row tiles
    spblas.destroy(A)
    A = make_handle("d", synth.stencil27("d", 24))
    _, info = spblas.mat_info(A)
    assert info.algorithm == capi.ALG_ROWTILE                               # neighbouring rows, neighbouring columns
    spblas.destroy(A)
    A = make_handle("d", synth.zipf("d", 1, 20000, 300000, 1.8, 1, 200000))
    _, info = spblas.mat_info(A)
    assert info.algorithm == capi.ALG_MERGE and info.merge_tiles > 0
    spblas.destroy(A)


def test_linearity_and_repeatability():
    """Size-independent properties: A(ax1 + bx2) = aAx1 + bAx2 within tolerance; identical bits run to run."""
    kind = "d"
    m = synth.zipf(kind, 9, 100000, 100000, 1.8, 1, 50000)
    A = make_handle(kind, m)
    x1, x2 = (torch.from_numpy(synth.vector(kind, 9, s, m.cols)).cuda() for s in (1, 2))
    ys = []
    for x in (x1, x2, 2.0 * x1 - 3.0 * x2, x1):
        y = torch.zeros(m.nrows, dtype=torch.float64, device="cuda")
        assert spblas.mv(kind, 0, 1.0, A, spblas.descr(), x, 0.0, y) == capi.SUCCESS
        ys.append(y)
    torch.cuda.synchronize()
    assert torch.equal(ys[0], ys[3])
    xs = np.abs(synth.vector(kind, 9, 1, m.cols)) * 2 + np.abs(synth.vector(kind, 9, 2, m.cols)) * 3
    scale = np.bincount(np.repeat(np.arange(m.nrows), np.diff(m.ptr)), weights=np.abs(m.val) * xs[m.col],
                        minlength=m.nrows)
    err = (ys[2] - (2.0 * ys[0] - 3.0 * ys[1])).abs().cpu().numpy()
    assert (err <= 4e-12 * scale + 1e-300).all()
    spblas.destroy(A)


@pytest.mark.parametrize("kind,make", [("s", lambda: synth.uniform_fixed("s", 31, (1 << 20) + 12345, 1 << 20, 8)),
                                       ("d", lambda: synth.stencil27("d", 104))])
def test_large_host_vectors_take_the_pipelined_path(kind, make):
    """Host x and y on more than 2^20 rows: the product runs in row windows overlapped with the PCIe
    copies; the result must not depend on that."""
    m = make()
    assert m.nrows >= 1 << 20
    for alpha, beta in ((1.5, 0.5), (1.0, 0.0)):
        y_host = check_mv(kind, m, alpha, beta, seed=31, pointers="host")
        y_dev = check_mv(kind, m, alpha, beta, seed=31, pointers="device")
        assert np.array_equal(y_host, y_dev)  # same kernels on the same rows: identical bits
        y_mixed = check_mv(kind, m, alpha, beta, seed=31, pointers="device_x_host_y")   # windows, x already on the GPU
        assert np.array_equal(y_mixed, y_dev)


def test_transposed_mv():
    """y = alpha * A^T * x + beta * y against the reference's plain transposed kernel (golden vector
    from its own objects, and the oracle on fresh rectangular inputs)."""
    g = golden("trans_d.npz")
    m = _csr(g)
    A = make_handle("d", m)
    y = g["y0"].copy()
    assert spblas.mv("d", capi.TRANSPOSE, float(g["alpha"]), A, spblas.descr(), g["x"], float(g["beta"]), y) == capi.SUCCESS
    prod = np.abs(g["val"] * np.repeat(g["x"], np.diff(g["ptr"])))
    scale = np.abs(g["beta"] * g["y0"]) + abs(g["alpha"]) * np.bincount(g["col"], weights=prod, minlength=len(y))
    assert_rows_close("d", y, g["y"], scale, "transposed mv (golden)")
    spblas.destroy(A)
    for kind in ("s", "d"):
        lens = synth.rowlen_zipf(41, 5000, 1.8, 1, 900 if kind == "s" else 4000)
        lens[::9] = 0
        m = synth.from_lengths(kind, 41, lens, 7000)      # 5000 x 7000: x has 5000 entries, y 7000
        x, y0 = synth.vector(kind, 41, 1, m.nrows), synth.vector(kind, 41, 2, m.cols)
        A = make_handle(kind, m)
        for alpha, beta in ((1.0, 0.0), (-0.5, 2.0)):
            y_ref = oracle.gemv_trans(kind, m.cols, m.rows_start, m.rows_end, m.col, m.val, alpha, x, beta, y0.copy())
            prod = np.abs(m.val.astype(np.float64) * np.repeat(x.astype(np.float64), np.diff(m.ptr)))
            scale = np.abs(beta * y0.astype(np.float64)) + abs(alpha) * np.bincount(m.col, weights=prod, minlength=m.cols)
            for dev in (False, True):
                if dev:
                    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
                    assert spblas.mv(kind, capi.TRANSPOSE, alpha, A, spblas.descr(), dx, beta, dy) == capi.SUCCESS
                    y = dy.cpu().numpy()
                else:
                    y = y0.copy()
                    assert spblas.mv(kind, capi.TRANSPOSE, alpha, A, spblas.descr(), x, beta, y) == capi.SUCCESS
                assert_rows_close(kind, y, y_ref, scale, f"transposed mv {kind} dev={dev}")
        # the non-transposed product of the same handle is unaffected
        check_mv(kind, m, 1.5, 0.5, A=A)
        spblas.destroy(A)


def test_structured_descriptors():
    """SYMMETRIC / TRIANGULAR / DIAGONAL descriptors on a CSR handle: every fill / diag / operation variant the
    reference's dispatch table holds, against its plain symv / trmv / diagmv kernels (golden vectors), then on a
    larger random matrix against the oracle."""
    g = golden("struct_d.npz")
    ptr, a, b = g["ptr"], float(g["alpha"]), float(g["beta"])
    m = synth.Csr(160, 160, 0, ptr, g["col"], g["val"])
    A = make_handle("d", m)

    def scale_of(mm_, x, y0, alpha, beta):
        rid = np.repeat(np.arange(mm_.nrows), np.diff(mm_.ptr))
        return np.abs(beta * y0) + abs(alpha) * (np.bincount(rid, weights=np.abs(mm_.val * x[mm_.col]), minlength=mm_.nrows) +
                                                 np.bincount(mm_.col, weights=np.abs(mm_.val * x[rid]), minlength=mm_.nrows) +
                                                 np.abs(x))
    sc = scale_of(m, g["x"], g["y0"], a, b)
    for t, transes in ((capi.SYMMETRIC, (0,)), (capi.TRIANGULAR, (0, 1)), (capi.DIAGONAL, (0,))):
        for upper in (0, 1):
            for unit in (0, 1):
                for tr in transes:
                    y = g["y0"].copy()
                    st = spblas.mv("d", tr, a, A, spblas.descr(t, upper, unit), g["x"], b, y)
                    assert st == capi.SUCCESS, (t, upper, unit, tr, capi.STATUS_NAMES[st])
                    assert_rows_close("d", y, g[f"y_t{t}_u{upper}_d{unit}_o{tr}"], sc, f"type {t} {upper}{unit}{tr}")
    # the reference has no transposed symmetric kernel for real types: NULL table entry
    assert spblas.mv("d", capi.TRANSPOSE, a, A, spblas.descr(capi.SYMMETRIC), g["x"], b, g["y0"].copy()) == capi.NOT_SUPPORTED
    # the general product of the same handle still sees the whole matrix
    check_mv("d", m, 1.0, 0.0, A=A)
    spblas.destroy(A)

    for kind in ("s", "d"):
        m = synth.poisson(kind, 71, 4000, 4000, 10.0)
        x, y0 = synth.vector(kind, 71, 1, 4000), synth.vector(kind, 71, 2, 4000)
        A = make_handle(kind, m)
        sc = scale_of(m, x.astype(np.float64), y0.astype(np.float64), 1.25, 0.5)
        for t, upper, unit, tr in ((capi.SYMMETRIC, 1, 0, 0), (capi.TRIANGULAR, 0, 1, 1), (capi.TRIANGULAR, 1, 0, 0),
                                   (capi.DIAGONAL, 0, 0, 0)):
            y_ref = oracle.structured_mv(kind, t, upper, unit, tr, m.rows_start, m.rows_end, m.col, m.val, 1.25, x, 0.5,
                                         y0.copy())
            dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
            assert spblas.mv(kind, tr, 1.25, A, spblas.descr(t, upper, unit), dx, 0.5, dy) == capi.SUCCESS
            assert_rows_close(kind, dy.cpu().numpy(), y_ref, sc, f"{kind} type {t}")
        spblas.destroy(A)


def test_structured_descriptors_on_unsorted_rows_with_repeated_diagonals():
    """The derived matrices are built on the device from the device copy (key emission, scan, radix sort over more
    than one block of keys).  Rows in shuffled column order, diagonals stored up to three times (diagmv takes the
    FIRST stored one, the row-major diagmm ALL, the column-major diagmm the LAST), pairs stored twice, empty rows."""
    n = 60000
    base = synth.poisson("d", 91, n, n, 20.0)
    assert base.nnz > 1 << 20
    rng = np.random.default_rng(91)
    rows_of = np.repeat(np.arange(n, dtype=np.int64), np.diff(base.ptr))
    extra_diag = np.concatenate([rng.integers(0, n, 9000), rng.integers(0, n, 4000)])  # some rows get 2 or 3
    dup = rng.integers(0, base.nnz, 3000)
    ri = np.concatenate([rows_of, extra_diag, rows_of[dup]])
    ci = np.concatenate([base.col.astype(np.int64), extra_diag, base.col[dup].astype(np.int64)])
    v = np.concatenate([base.val, rng.uniform(-1, 1, len(extra_diag)), rng.uniform(-1, 1, len(dup))])
    keep = ri % 97 != 5  # empty rows
    ri, ci, v = ri[keep], ci[keep], v[keep]
    order = np.lexsort((rng.random(len(ri)), ri))  # rows ascending, random order inside a row
    ri, ci, v = ri[order], ci[order].astype(np.int32), v[order]
    ptr = np.concatenate([[0], np.cumsum(np.bincount(ri, minlength=n))]).astype(np.int32)
    m = synth.Csr(n, n, 0, ptr, ci, v)
    A = make_handle("d", m)
    x, y0 = synth.vector("d", 91, 1, n), synth.vector("d", 91, 2, n)
    rid = np.repeat(np.arange(n), np.diff(ptr))
    sc = np.abs(0.5 * y0) + 1.25 * (np.bincount(rid, weights=np.abs(v * x[ci]), minlength=n) +
                                    np.bincount(ci, weights=np.abs(v * x[rid]), minlength=n) + np.abs(x))
    for t, transes in ((capi.SYMMETRIC, (0,)), (capi.TRIANGULAR, (0, 1)), (capi.DIAGONAL, (0,))):
        for upper in (0, 1):
            for unit in (0, 1):
                for tr in transes:
                    y_ref = oracle.structured_mv("d", t, upper, unit, tr, m.rows_start, m.rows_end, m.col, m.val, 1.25, x,
                                                 0.5, y0.copy())
                    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
                    assert spblas.mv("d", tr, 1.25, A, spblas.descr(t, upper, unit), dx, 0.5, dy) == capi.SUCCESS, spblas.last_error()
                    assert_rows_close("d", dy.cpu().numpy(), y_ref, sc, f"type {t} {upper}{unit}{tr}")
    # the two diagmm rules for repeated diagonals
    columns = 4
    X, Y0 = synth.vector("d", 92, 1, n * columns), synth.vector("d", 92, 2, n * columns)
    for lay, layout in (("row", capi.ROW_MAJOR), ("col", capi.COLUMN_MAJOR)):
        ld = columns if lay == "row" else n
        Yref = oracle.structured_mm("d", capi.DIAGONAL, 0, 0, 0, lay, m.rows_start, m.rows_end, m.col, m.val, 1.25, X, columns,
                                    ld, 0.5, Y0.copy(), ld)
        dX, dY = torch.from_numpy(X).cuda(), torch.from_numpy(Y0).cuda()
        assert spblas.mm("d", 0, 1.25, A, spblas.descr(capi.DIAGONAL, 0, 0), layout, dX, columns, ld, 0.5, dY, ld) == capi.SUCCESS
        d_abs = np.bincount(rid[ci == rid], weights=np.abs(v[ci == rid]), minlength=n)
        scm = np.abs(0.5 * Y0) + 1.25 * np.abs(X) * (np.repeat(d_abs, columns) if lay == "row" else np.tile(d_abs, columns))
        assert_rows_close("d", dY.cpu().numpy(), Yref, scm, f"diagmm {lay}")
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
def test_vector_kernel_in_column_blocks(kind):
    """An x that does not fit L2 makes the vector kernel run once per column block (limits shrunk here so that a small
    matrix is cut into 2 .. 64 blocks): every scalar combination, host and device vectors, empty rows, rows with fewer
    elements than blocks; rows in descending column order must fall back to one launch."""
    rows, cols = 30011, 40009
    lens = synth.rowlen_poisson(31, rows, 14.0, cols).copy()
    lens[::97] = 0
    m = synth.from_lengths(kind, 31, lens, cols)
    x, y0 = synth.vector(kind, 31, 1, cols), synth.vector(kind, 31, 2, rows)
    tsz = 4 if kind == "s" else 8
    for block_kb in (cols * tsz // 2048 + 1, 16, 1):
        with _Options(mv_block_min_kb=1, mv_block_kb=block_kb):
            A = make_handle(kind, m)
        assert spblas.mat_info(A)[1].algorithm == capi.ALG_VECTOR
        for alpha, beta in ((1.0, 0.0), (1.5, 0.5), (-0.5, 1.0)):
            check_mv(kind, m, alpha, beta, A=A)
            check_mv(kind, m, alpha, beta, A=A, pointers="device")
        before = spblas.launch_count()
        dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
        assert spblas.mv(kind, 0, 1.0, A, spblas.descr(), dx, 0.0, dy) == capi.SUCCESS
        want = min(64, -(-(cols * tsz // 1024) // block_kb))
        assert spblas.launch_count() - before == want, (block_kb, want)
        spblas.destroy(A)
    col, val = m.col.copy(), m.val.copy()
    for r in range(rows):
        col[m.ptr[r]:m.ptr[r + 1]] = col[m.ptr[r]:m.ptr[r + 1]][::-1]
        val[m.ptr[r]:m.ptr[r + 1]] = val[m.ptr[r]:m.ptr[r + 1]][::-1]
    mr = synth.Csr(rows, cols, 0, m.ptr, col, val)
    with _Options(mv_block_min_kb=1, mv_block_kb=16):
        A = make_handle(kind, mr)
    before = spblas.launch_count()
    check_mv(kind, mr, 1.5, 0.5, A=A, pointers="device")
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
def test_large_coo_is_sorted_on_the_device(kind):
    """More than 2^20 COO entries take the GPU radix-sort path of alphasparse_convert_csr; the CSR must be
    the one the reference's conversion produces (bit-exact, duplicates kept in input order)."""
    m = synth.poisson(kind, 81, 90000, 70000, 14.0)
    assert m.nnz > 1 << 20
    rng = np.random.default_rng(81)
    ri = np.repeat(np.arange(m.nrows, dtype=np.int32), np.diff(m.ptr))
    # shuffle, then append repeated (row, col) pairs with different values: stable order keeps them as given
    dup = rng.integers(0, m.nnz, 5000)
    ri2 = np.concatenate([ri, ri[dup]])
    ci2 = np.concatenate([m.col, m.col[dup]])
    v2 = np.concatenate([m.val, rng.uniform(-1, 1, 5000).astype(m.val.dtype)])
    perm = rng.permutation(len(ri2))
    ri2, ci2, v2 = ri2[perm], ci2[perm], v2[perm]
    for op, rows, cols, a, b in ((capi.NON_TRANSPOSE, m.nrows, m.cols, ri2, ci2), (capi.TRANSPOSE, m.cols, m.nrows, ci2, ri2)):
        st, coo = spblas.create_coo(kind, capi.BASE_ONE, m.nrows, m.cols, len(ri2), ri2 + 1, ci2 + 1, v2)
        assert st == capi.SUCCESS
        st, A = spblas.convert_csr(coo, op)
        assert st == capi.SUCCESS, spblas.last_error()
        _, _, r, c, rs, re_, col, val = spblas.export_csr(kind, A)
        optr, ocol, oval = oracle.coo_to_csr(kind, 0, rows, a, b, v2)
        assert (r, c) == (rows, cols)
        assert np.array_equal(np.concatenate([rs[:1], re_]), optr) and np.array_equal(col, ocol)
        assert np.array_equal(val.view(np.uint8), oval.view(np.uint8))
        spblas.destroy(A)
        spblas.destroy(coo)
    # an index outside the matrix is refused
    bad = ri2.copy()
    bad[7] = m.nrows
    st, coo = spblas.create_coo(kind, capi.BASE_ZERO, m.nrows, m.cols, len(bad), bad, ci2, v2)
    st, A = spblas.convert_csr(coo, capi.NON_TRANSPOSE)
    assert st == capi.INVALID_VALUE and not A.value
    spblas.destroy(coo)


def test_merge_kernel_delivers_into_page_locked_host_y():
    """Large skewed matrix + page-locked host y: finished chunks of y are stored into the host buffer from
    inside the merge kernel, which then runs over all tiles (the delivering form has no column-band path, so
    long rows are summed in another order than in the device-pointer call: equal within the tolerance, and
    bit-identical from one such call to the next).  Pageable host memory takes the device-pointer kernels."""
    kind = "d"
    m = synth.zipf(kind, 91, (1 << 20) + 777, 1 << 20, 1.8, 1, 100000)
    A = make_handle(kind, m)
    _, info = spblas.mat_info(A)
    assert info.algorithm == capi.ALG_MERGE
    x = synth.vector(kind, 91, 1, m.cols)
    y0 = synth.vector(kind, 91, 2, m.nrows)
    for alpha, beta in ((1.0, 0.0), (0.5, -1.5)):
        dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
        assert spblas.mv(kind, 0, alpha, A, spblas.descr(), dx, beta, dy) == capi.SUCCESS
        want = dy.cpu().numpy()
        scale = row_scale(m.ptr, m.col, m.val, x, alpha, beta, y0)
        exact = oracle.gemv_exact(m.rows_start, m.rows_end, m.col, m.val, alpha, x, beta, y0)
        pinned = torch.from_numpy(y0.copy()).pin_memory()
        assert spblas.mv(kind, 0, alpha, A, spblas.descr(), x, beta, pinned.numpy()) == capi.SUCCESS
        assert_rows_close(kind, pinned.numpy(), exact, scale, "delivered into page-locked y")
        again = torch.from_numpy(y0.copy()).pin_memory()
        assert spblas.mv(kind, 0, alpha, A, spblas.descr(), x, beta, again.numpy()) == capi.SUCCESS
        assert np.array_equal(pinned.numpy(), again.numpy())
        pageable = y0.copy()
        assert spblas.mv(kind, 0, alpha, A, spblas.descr(), x, beta, pageable) == capi.SUCCESS
        assert np.array_equal(pageable, want)
    y_ref = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, 0.5, x, -1.5, y0.copy())
    assert_rows_close(kind, want, y_ref, row_scale(m.ptr, m.col, m.val, x, 0.5, -1.5, y0), "merge e2e")
    spblas.destroy(A)


def test_coo_handle_goes_straight_to_mv_and_mm():
    """A COO handle with a GENERAL descriptor is served by mv / mm directly (a CSR copy is made on first use):
    both operations and both dense layouts against the reference's plain COO kernels (golden vectors, unsorted
    one-based entries with repeated pairs), host and device operands."""
    g = golden("coo_d.npz")
    ri, ci, val, a, b = g["ri"], g["ci"], g["val"], float(g["alpha"]), float(g["beta"])
    rows, cols = int(g["rows"]), int(g["cols"])
    columns, ldx, ldy = (int(v) for v in g["par"])
    st, A = spblas.create_coo("d", capi.BASE_ONE, rows, cols, len(ri), ri + 1, ci + 1, val)
    assert st == capi.SUCCESS

    def scale(m_out, r, c, X, Y0):
        out = np.zeros((m_out, X.shape[1]))
        np.add.at(out, r, np.abs(val)[:, None] * np.abs(X)[c])
        return (np.abs(b * Y0) + abs(a) * out).reshape(-1)

    for tr in (0, 1):
        m_out, m_in = (cols, rows) if tr else (rows, cols)
        r, c = (ci, ri) if tr else (ri, ci)
        x, y0 = g[f"x_o{tr}"], g[f"y0_o{tr}"]
        for dev in (False, True):
            if dev:
                dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
                assert spblas.mv("d", tr, a, A, spblas.descr(), dx, b, dy) == capi.SUCCESS
                y = dy.cpu().numpy()
            else:
                y = y0.copy()
                assert spblas.mv("d", tr, a, A, spblas.descr(), x, b, y) == capi.SUCCESS, spblas.last_error()
            assert_rows_close("d", y, g[f"y_o{tr}"], scale(m_out, r, c, x[:, None], y0[:, None]), f"coo mv op {tr}")
        Xr, Yr0 = g[f"Xr_o{tr}"], g[f"Yr0_o{tr}"]
        Y = Yr0.copy()
        assert spblas.mm("d", tr, a, A, spblas.descr(), capi.ROW_MAJOR, Xr, columns, ldx, b, Y, ldy) == capi.SUCCESS
        view = lambda v: v.reshape(m_out, ldy)[:, :columns]  # noqa: E731
        assert_rows_close("d", view(Y).reshape(-1), view(g[f"Yr_o{tr}"]).reshape(-1),
                          scale(m_out, r, c, Xr.reshape(m_in, ldx)[:, :columns], view(Yr0)), f"coo mm row op {tr}")
        assert np.array_equal(Y.reshape(m_out, ldy)[:, columns:], Yr0.reshape(m_out, ldy)[:, columns:])
        lx, ly = m_in + 2, m_out + 1
        Xc, Yc0 = g[f"Xc_o{tr}"], g[f"Yc0_o{tr}"]
        dX, dY = torch.from_numpy(Xc).cuda(), torch.from_numpy(Yc0).cuda()
        assert spblas.mm("d", tr, a, A, spblas.descr(), capi.COLUMN_MAJOR, dX, columns, lx, b, dY, ly) == capi.SUCCESS
        viewc = lambda v: v.reshape(columns, ly)[:, :m_out].T  # noqa: E731
        assert_rows_close("d", viewc(dY.cpu().numpy()).reshape(-1), viewc(g[f"Yc_o{tr}"]).reshape(-1),
                          scale(m_out, r, c, Xc.reshape(columns, lx)[:, :m_in].T, viewc(Yc0)), f"coo mm col op {tr}")
    # checks keep the reference's order; structured descriptors on a COO handle are not served
    x, y = g["x_o0"], g["y0_o0"].copy()
    assert spblas.mv("s", 0, 1.0, A, spblas.descr(), x, 0.0, y) == capi.INVALID_VALUE
    assert spblas.mv("d", 0, a, A, spblas.descr(capi.SYMMETRIC), x, b, y) == capi.INVALID_VALUE      # 150 x 210
    assert spblas.mv("d", 0, a, A, spblas.descr(capi.TRIANGULAR), x, b, y) == capi.NOT_SUPPORTED
    assert spblas.mv("d", 0, a, A, spblas.descr(9), x, b, y) == capi.INVALID_VALUE
    assert np.array_equal(y, g["y0_o0"])
    # the conversion entry point still works on the same handle, and destroy releases the copy made by mv
    st, B = spblas.convert_csr(A, capi.NON_TRANSPOSE)
    assert st == capi.SUCCESS
    assert spblas.destroy(B) == capi.SUCCESS and spblas.destroy(A) == capi.SUCCESS

    # a larger single-precision matrix against the oracle, entries in random order
    m = synth.poisson("s", 91, 30000, 20000, 9.0)
    rng = np.random.default_rng(91)
    perm = rng.permutation(m.nnz)
    ri = np.repeat(np.arange(m.nrows, dtype=np.int32), np.diff(m.ptr))[perm]
    ci, v = m.col[perm], m.val[perm]
    st, A = spblas.create_coo("s", capi.BASE_ZERO, m.nrows, m.cols, m.nnz, ri, ci, v)
    assert capi.load().alphasparse_optimize(A) == capi.SUCCESS      # converts ahead of the first product
    assert C.cast(A, C.POINTER(capi.Matrix)).contents.inspector is not None
    x, y0 = synth.vector("s", 91, 1, m.cols), synth.vector("s", 91, 2, m.nrows)
    y_ref = oracle.gemv_coo("s", 0, m.nrows, m.cols, ri, ci, v, 1.5, x, 0.5, y0.copy())
    y = y0.copy()
    assert spblas.mv("s", 0, 1.5, A, spblas.descr(), x, 0.5, y) == capi.SUCCESS
    assert_rows_close("s", y, y_ref, row_scale(m.ptr, m.col, m.val, x, 1.5, 0.5, y0), "coo mv s")
    spblas.destroy(A)


def test_merge_blocks_follow_the_column_schedule_when_x_is_large():
    """With an x too large to sit in L2 beside the matrix stream the merge kernel's blocks take the single-row
    tiles in the order of their first column; the product must be what the natural order gives (the order only
    changes which block computes which tile), and small matrices keep the natural order."""
    cols = 1 << 22                                             # 32 MB of fp64 x
    lens = np.concatenate([np.full(30, 70000), synth.rowlen_zipf(5, 20000, 1.8, 1, 3000), np.full(10, 120001)])
    m = synth.from_lengths("d", 5, lens, cols)
    A = make_handle("d", m)
    st, info = spblas.mat_info(A)
    assert st == capi.SUCCESS and info.algorithm == capi.ALG_MERGE and info.scheduled == 1
    x, y0 = synth.vector("d", 5, 1, cols), synth.vector("d", 5, 2, m.nrows)
    y_ref = oracle.gemv("d", m.rows_start, m.rows_end, m.col, m.val, 1.5, x, -0.25, y0.copy())
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
    assert spblas.mv("d", 0, 1.5, A, spblas.descr(), dx, -0.25, dy) == capi.SUCCESS
    first = dy.cpu().numpy()
    assert_rows_close("d", first, y_ref, row_scale(m.ptr, m.col, m.val, x, 1.5, -0.25, y0), "scheduled merge")
    dy = torch.from_numpy(y0).cuda()
    assert spblas.mv("d", 0, 1.5, A, spblas.descr(), dx, -0.25, dy) == capi.SUCCESS
    assert np.array_equal(first, dy.cpu().numpy())             # same schedule, same sums: bit-identical repeats
    spblas.destroy(A)
    small = synth.from_lengths("d", 6, np.concatenate([np.full(4, 30000), np.full(500, 3)]), 1 << 16)
    B = make_handle("d", small)
    st, info = spblas.mat_info(B)
    assert info.algorithm == capi.ALG_MERGE and info.scheduled == 0
    spblas.destroy(B)


class _Options:
    """Sets analysis options for the handles created inside the block and restores the defaults after it."""

    def __init__(self, **kw):
        self.kw = kw

    def __enter__(self):
        for k, v in self.kw.items():
            assert spblas.set_option(k, v) == capi.SUCCESS
        return self

    def __exit__(self, *exc):
        for k in self.kw:
            spblas.set_option(k, -1)


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("overlap", [0, 1])
@pytest.mark.parametrize("mode", ["binned", "binned_unpacked", "binned_unsorted", "tiles", "tiles_unsorted"])
def test_row_bins_and_the_column_band_path(kind, overlap, mode):
    """Row binning of the analysis on a skewed matrix, with limits small enough for a small matrix to fill every bin.

    binned: thread per row up to 2 elements, lane groups for the three mid lists, and the five long rows (long = at
    least 30 elements per column band on average) whole in the column-band kernel (bands of x staged in shared
    memory; several splits per band, a ragged last band, long rows first / last / adjacent).
    binned_unsorted: one long row has two columns swapped; it cannot be cut into bands, so the handle must fall back
    to merge tiles, where the other four long rows still give their inner tiles to the band kernel.
    binned_unpacked: the band kernel reads the long rows from the CSR arrays instead of from its packed band-major
    copy (16-bit columns relative to the band, segments padded to quads).
    tiles / tiles_unsorted: the same with binning switched off.
    All scalar combinations, host and device vectors, bit-identical repeats, and a run of the delivering merge kernel
    (every tile) in between."""
    cols = 70001
    body = np.concatenate([[40000], synth.rowlen_zipf(9, 6000, 1.8, 1, 900), [9000, 25000, 3],
                           synth.rowlen_zipf(10, 3000, 1.8, 1, 50), [12000, 1, 1]])
    # square (the exchange below wants that): empty rows fill up, the last row is long
    lens = np.concatenate([body, np.zeros(cols - len(body) - 1), [30000]]).astype(np.int32)
    m = synth.from_lengths(kind, 9, lens, cols)
    ptr = m.ptr
    unsorted = mode.endswith("unsorted")
    if unsorted:
        row = 6002                                               # the 25000-element row: swap two of its columns
        assert ptr[row + 1] - ptr[row] == 25000
        a = int(ptr[row]) + 7000
        m.col[a], m.col[a + 1] = m.col[a + 1], m.col[a]
        m.val[a], m.val[a + 1] = m.val[a + 1], m.val[a]
    binned = mode.startswith("binned")
    with _Options(band_bytes=4096, band_min_seg=30, band_min_rows=1, band_min_share_pct=0, band_splits=3,
                  band_overlap=overlap, bin_enable=int(binned), bin_short=2, band_packed=int(mode != "binned_unpacked")):
        spblas.set_algorithm(capi.ALG_MERGE)
        try:
            A = make_handle(kind, m)
        finally:
            spblas.set_algorithm(capi.ALG_AUTO)
    st, info = spblas.mat_info(A)
    assert st == capi.SUCCESS and info.algorithm == capi.ALG_MERGE
    assert info.band_width == 4096 // m.val.itemsize and info.band_count == -(-cols // info.band_width)
    long_total = 40000 + 9000 + 12000 + 30000 + (0 if unsorted else 25000)
    assert info.band_rows == (4 if unsorted else 5), info.band_rows
    if binned and not unsorted:
        assert info.binned == 1 and info.band_elements == long_total
    else:
        tile = 256 * (7 if kind == "d" else 9)
        assert info.binned == 0 and info.scheduled == 1
        assert long_total - 2 * info.band_rows * tile <= info.band_elements <= long_total
    x, y0 = synth.vector(kind, 9, 1, cols), synth.vector(kind, 9, 2, m.nrows)
    dx = torch.from_numpy(x).cuda()
    results = {}
    for alpha, beta in ((1.0, 0.0), (1.5, 0.5), (-2.0, 1.0), (0.0, 3.0)):
        y_ref = oracle.gemv_exact(m.rows_start, m.rows_end, m.col, m.val, alpha, x, beta, y0)
        dy = torch.from_numpy(y0).cuda()
        assert spblas.mv(kind, 0, alpha, A, spblas.descr(), dx, beta, dy) == capi.SUCCESS
        y = dy.cpu().numpy()
        assert_rows_close(kind, y, y_ref, row_scale(m.ptr, m.col, m.val, x, alpha, beta, y0), f"{mode} {kind} {alpha} {beta}")
        results[(alpha, beta)] = y
        yh = y0.copy()                                           # host vectors through the same handle
        assert spblas.mv(kind, 0, alpha, A, spblas.descr(), x, beta, yh) == capi.SUCCESS
        assert np.array_equal(yh, y)
    # the delivering merge kernel runs every tile (and leaves carries behind for the tiles a schedule skips)
    from alsparse_b200 import multi
    ex = multi.FusedExchange(kind, np.array([0, m.nrows], np.int32), 0, 1, deliver_after=False)
    ex.x_tensor().copy_(dx)
    dy = torch.from_numpy(y0).cuda()
    assert ex.step(1.5, A, 0.5, dy) == capi.SUCCESS
    y_ref = oracle.gemv_exact(m.rows_start, m.rows_end, m.col, m.val, 1.5, x, 0.5, y0)
    assert_rows_close(kind, dy.cpu().numpy(), y_ref, row_scale(m.ptr, m.col, m.val, x, 1.5, 0.5, y0), "all tiles")
    assert np.array_equal(ex.x_tensor().cpu().numpy(), dy.cpu().numpy())
    ex.destroy()
    dy = torch.from_numpy(y0).cuda()
    assert spblas.mv(kind, 0, 1.5, A, spblas.descr(), dx, 0.5, dy) == capi.SUCCESS
    assert np.array_equal(dy.cpu().numpy(), results[(1.5, 0.5)])
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
def test_row_bins_without_long_rows_and_declined_bins(kind):
    """A skewed matrix whose longest rows stay below the column-band kernel's threshold is binned without that kernel;
    a row longer than the lane-group kernels may take (eight times bin_mid_max when the band kernel's threshold lies
    above that) but too short for the band kernel keeps the handle on merge tiles."""
    lens = np.concatenate([synth.rowlen_zipf(3, 20000, 1.8, 1, 2500), np.zeros(50), [2999, 1]]).astype(np.int32)
    m = synth.from_lengths(kind, 3, lens, 1 << 23)              # 512 / 1024 bands: a row is long from 4096 / 8192 elements
    for mid_max, expect in ((16384, 1), (2000, 1), (300, 0)):
        with _Options(bin_mid_max=mid_max):
            spblas.set_algorithm(capi.ALG_MERGE)
            try:
                A = make_handle(kind, m)
            finally:
                spblas.set_algorithm(capi.ALG_AUTO)
        _, info = spblas.mat_info(A)
        assert info.binned == expect and info.band_rows == 0, (info.binned, info.band_rows)
        check_mv(kind, m, 1.5, 0.5, pointers="device", A=A)
        check_mv(kind, m, 1.0, 0.0, pointers="host", A=A)
        assert spblas.optimize(A) == capi.SUCCESS                # re-analysis of a live handle keeps it usable
        check_mv(kind, m, -1.0, 2.0, pointers="device", A=A)
        spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
def test_large_transpose_keeps_the_reference_order(kind):
    """A^T of a matrix with more than a million stored elements, some pairs stored twice: the transposed product
    must agree with the oracle's transposed kernel, and bit for bit with the plain product of a handle created
    from the explicitly transposed arrays (a column's elements by ascending row, repeated pairs in stored order)."""
    m = synth.poisson(kind, 83, 90000, 70000, 14.0)
    assert m.nnz > 1 << 20
    # repeat some stored pairs with other values, in place: create_csr keeps them as they come
    rid = np.repeat(np.arange(m.nrows), np.diff(m.ptr))
    rng = np.random.default_rng(83)
    dup = np.sort(rng.choice(m.nnz, 3000, replace=False))       # each copy lands right after its original
    col = np.insert(m.col, dup + 1, m.col[dup])
    val = np.insert(m.val, dup + 1, rng.uniform(-1, 1, len(dup)).astype(m.val.dtype))
    rid2 = np.insert(rid, dup + 1, rid[dup])
    ptr = np.concatenate([[0], np.cumsum(np.bincount(rid2, minlength=m.nrows))]).astype(np.int32)
    st, A = spblas.create_csr(kind, 0, m.nrows, m.cols, ptr[:-1], ptr[1:], col, val)
    assert st == capi.SUCCESS
    x, y0 = synth.vector(kind, 83, 1, m.nrows), synth.vector(kind, 83, 2, m.cols)
    y_ref = oracle.gemv_trans(kind, m.cols, ptr[:-1], ptr[1:], col, val, 1.5, x, 0.5, y0.copy())
    dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
    assert spblas.mv(kind, capi.TRANSPOSE, 1.5, A, spblas.descr(), dx, 0.5, dy) == capi.SUCCESS, spblas.last_error()
    order = np.lexsort((np.arange(len(col)), rid2, col))       # by column, then row, then stored position
    tptr = np.concatenate([[0], np.cumsum(np.bincount(col, minlength=m.cols))]).astype(np.int32)
    tcol, tval = rid2[order].astype(np.int32), val[order]
    scale = row_scale(tptr, tcol, tval, x, 1.5, 0.5, y0)
    assert_rows_close(kind, dy.cpu().numpy(), y_ref, scale, "transposed, large")
    st, B = spblas.create_csr(kind, 0, m.cols, m.nrows, tptr[:-1], tptr[1:], tcol, tval)
    assert st == capi.SUCCESS
    dy2 = torch.from_numpy(y0).cuda()
    assert spblas.mv(kind, 0, 1.5, B, spblas.descr(), dx, 0.5, dy2) == capi.SUCCESS
    assert torch.equal(dy, dy2)
    spblas.destroy(A)
    spblas.destroy(B)


def test_csc_handle_in_mv_and_mm():
    """A CSC handle (created from one-based arrays, more columns than rows) in mv / mm: both operations and both
    dense layouts against the reference's plain CSC kernels (golden vectors); export_csc; convert_csc from COO."""
    g = golden("csc_d.npz")
    ptr, ri, val, a, b = g["ptr"], g["ri"], g["val"], float(g["alpha"]), float(g["beta"])
    rows, cols = int(g["rows"]), int(g["cols"])
    columns, ldx, ldy = (int(v) for v in g["par"])
    st, A = spblas.create_csc("d", capi.BASE_ONE, rows, cols, ptr[:-1] + 1, ptr[1:] + 1, ri + 1, val)
    assert st == capi.SUCCESS, spblas.last_error()
    st, base, er, ec, cs, ce, eri, ev = spblas.export_csc("d", A)
    assert (st, base, er, ec) == (capi.SUCCESS, 0, rows, cols)
    assert np.array_equal(cs, ptr[:-1]) and np.array_equal(ce, ptr[1:]) and np.array_equal(eri, ri) and np.array_equal(ev, val)
    cid = np.repeat(np.arange(cols), np.diff(ptr))

    def scale(m_out, r, c, X, Y0):
        out = np.zeros((m_out, X.shape[1]))
        np.add.at(out, r, np.abs(val)[:, None] * np.abs(X)[c])
        return (np.abs(b * Y0) + abs(a) * out).reshape(-1)

    for tr in (0, 1):
        m_out, m_in = (cols, rows) if tr else (rows, cols)
        r, c = (cid, ri) if tr else (ri, cid)
        x, y0 = g[f"x_o{tr}"], g[f"y0_o{tr}"]
        for dev in (False, True):
            if dev:
                dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
                assert spblas.mv("d", tr, a, A, spblas.descr(), dx, b, dy) == capi.SUCCESS
                y = dy.cpu().numpy()
            else:
                y = y0.copy()
                assert spblas.mv("d", tr, a, A, spblas.descr(), x, b, y) == capi.SUCCESS, spblas.last_error()
            assert_rows_close("d", y, g[f"y_o{tr}"], scale(m_out, r, c, x[:, None], y0[:, None]), f"csc mv op {tr}")
        Xr, Yr0 = g[f"Xr_o{tr}"], g[f"Yr0_o{tr}"]
        Y = Yr0.copy()
        assert spblas.mm("d", tr, a, A, spblas.descr(), capi.ROW_MAJOR, Xr, columns, ldx, b, Y, ldy) == capi.SUCCESS
        view = lambda v: v.reshape(m_out, ldy)[:, :columns]  # noqa: E731
        assert_rows_close("d", view(Y).reshape(-1), view(g[f"Yr_o{tr}"]).reshape(-1),
                          scale(m_out, r, c, Xr.reshape(m_in, ldx)[:, :columns], view(Yr0)), f"csc mm row op {tr}")
        assert np.array_equal(Y.reshape(m_out, ldy)[:, columns:], Yr0.reshape(m_out, ldy)[:, columns:])
        lx, ly = m_in + 2, m_out + 1
        Xc, Yc0 = g[f"Xc_o{tr}"], g[f"Yc0_o{tr}"]
        dX, dY = torch.from_numpy(Xc).cuda(), torch.from_numpy(Yc0).cuda()
        assert spblas.mm("d", tr, a, A, spblas.descr(), capi.COLUMN_MAJOR, dX, columns, lx, b, dY, ly) == capi.SUCCESS
        viewc = lambda v: v.reshape(columns, ly)[:, :m_out].T  # noqa: E731
        assert_rows_close("d", viewc(dY.cpu().numpy()).reshape(-1), viewc(g[f"Yc_o{tr}"]).reshape(-1),
                          scale(m_out, r, c, Xc.reshape(columns, lx)[:, :m_in].T, viewc(Yc0)), f"csc mm col op {tr}")
    x, y = g["x_o0"], g["y0_o0"].copy()
    assert spblas.mv("s", 0, 1.0, A, spblas.descr(), x, 0.0, y) == capi.INVALID_VALUE
    assert spblas.mv("d", 0, a, A, spblas.descr(capi.SYMMETRIC), x, b, y) == capi.INVALID_VALUE      # 130 x 170
    assert spblas.mv("d", 0, a, A, spblas.descr(capi.DIAGONAL), x, b, y) == capi.NOT_SUPPORTED
    assert np.array_equal(y, g["y0_o0"])
    assert spblas.destroy(A) == capi.SUCCESS

    # COO -> CSC, as is and transposed: column-major sorted arrays of op(A), and products that agree with the COO handle's
    m = synth.poisson("s", 93, 700, 900, 7.0)
    rng = np.random.default_rng(93)
    perm = rng.permutation(m.nnz)
    cri = np.repeat(np.arange(m.nrows, dtype=np.int32), np.diff(m.ptr))[perm]
    cci, cv = m.col[perm], m.val[perm]
    st, coo = spblas.create_coo("s", capi.BASE_ZERO, m.nrows, m.cols, m.nnz, cri, cci, cv)
    for op, orows, ocols, oi, oj in ((capi.NON_TRANSPOSE, m.nrows, m.cols, cri, cci), (capi.TRANSPOSE, m.cols, m.nrows, cci, cri)):
        st, B = spblas.convert_csc(coo, op)
        assert st == capi.SUCCESS, spblas.last_error()
        st, base, er, ec, cs, ce, eri, ev = spblas.export_csc("s", B)
        assert (st, er, ec) == (capi.SUCCESS, orows, ocols)
        order = np.lexsort((np.arange(m.nnz), oi, oj))           # by column, then row, then stored position
        assert np.array_equal(eri, oi[order]) and np.array_equal(ev, cv[order])
        assert np.array_equal(np.concatenate([cs[:1], ce]), np.concatenate([[0], np.cumsum(np.bincount(oj, minlength=ocols))]))
        x, y0 = synth.vector("s", 93, 1, ocols), synth.vector("s", 93, 2, orows)
        y_ref = oracle.gemv_coo("s", 0, orows, ocols, oi, oj, cv, 1.5, x, 0.5, y0.copy())
        y = y0.copy()
        assert spblas.mv("s", 0, 1.5, B, spblas.descr(), x, 0.5, y) == capi.SUCCESS
        sc = np.abs(0.5 * y0.astype(np.float64)) + 1.5 * np.bincount(oi, weights=np.abs(cv.astype(np.float64) * x[oj]), minlength=orows)
        assert_rows_close("s", y, y_ref, sc, f"converted csc op {op}")
        spblas.destroy(B)
    spblas.destroy(coo)
