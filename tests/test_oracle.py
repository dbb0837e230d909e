"""Pins the C restatement (oracle/oracle.c) to the reference: against the golden vectors the
reference's own objects produced, and live against those objects where they are present."""
import numpy as np
import pytest

import oracle
from alsparse_b200 import synth
from helpers import NP, assert_rows_close, golden, mm_scale, row_scale, structured_scale

# The reference is built with -Ofast (reassociation, FMA contraction); the restatement sums strictly
# left to right.  Both are one summation order of the same products, so they agree to a few
# roundings of the row scale -- far inside the parity tolerance, which is what is asserted.


def test_kat_3x3():
    g = golden("kat3x3.npz")
    y = oracle.gemv("s", g["rs"], g["re"], g["col"], g["val"], 2.0, g["x"], 3.0, np.ones(3, np.float32))
    assert y.tolist() == [405.0, 63.0, 11.0] == g["y_a2_b3"].tolist() == g["y_base1"].tolist()
    ptr, col, val = oracle.create_csr("s", 1, g["rs"] + 1, g["re"] + 1, g["col"] + 1, g["val"])
    assert ptr.tolist() == g["base1_ptr"].tolist() and col.tolist() == g["base1_col"].tolist()
    Y = oracle.gemm("s", "row", g["rs"], g["re"], g["col"], g["val"], 1.0, g["B"], 2, 2, 0.0, np.zeros(6, np.float32), 2)
    assert Y.tolist() == g["mm_row"].tolist() == [11, 14, 9, 12, 4, 8]
    Y = oracle.gemm("s", "col", g["rs"], g["re"], g["col"], g["val"], 1.0, g["B"], 2, 3, 0.0, np.zeros(6, np.float32), 3)
    assert Y.tolist() == g["mm_col"].tolist()


@pytest.mark.parametrize("name,kind", [("cfg1_s.npz", "s"), ("zipf_d.npz", "d"), ("stencil8_d.npz", "d")])
def test_gemv_golden(name, kind):
    g = golden(name)
    ptr, alpha, beta = g["ptr"], float(g["alpha"]), float(g["beta"])
    scale = row_scale(ptr, g["col"], g["val"], g["x"], alpha, beta, g["y0"])
    y = oracle.gemv(kind, ptr[:-1], ptr[1:], g["col"], g["val"], alpha, g["x"], beta, g["y0"].copy())
    assert_rows_close(kind, y, g["y"], scale, name)
    yo = oracle.gemv(kind, ptr[:-1], ptr[1:], g["col"], g["val"], alpha, g["x"], beta, g["y0"].copy(), threads=3)
    assert_rows_close(kind, yo, g["y"], scale, name + " (OpenMP form)")
    if name == "cfg1_s.npz":
        y = oracle.gemv(kind, ptr[:-1], ptr[1:], g["col"], g["val"], 1.5, g["x"], 0.5, g["y0"].copy())
        assert_rows_close(kind, y, g["y_ab"], row_scale(ptr, g["col"], g["val"], g["x"], 1.5, 0.5, g["y0"]), "a,b")


def test_gemv_trans_golden():
    g = golden("trans_d.npz")
    ptr = g["ptr"]
    y = oracle.gemv_trans("d", int(g["cols"]), ptr[:-1], ptr[1:], g["col"], g["val"], float(g["alpha"]), g["x"],
                          float(g["beta"]), g["y0"].copy())
    prod = np.abs(g["val"] * np.repeat(g["x"], np.diff(ptr)))
    scale = np.abs(g["beta"] * g["y0"]) + abs(g["alpha"]) * np.bincount(g["col"], weights=prod, minlength=len(y))
    assert_rows_close("d", y, g["y"], scale, "transpose")


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("case", ["w64", "w5"])
def test_gemm_golden(kind, case):
    g = golden(f"mm_{kind}.npz")
    ptr = g["ptr"]
    columns, ldx, ldy, ldxc, ldyc = (int(v) for v in g[f"{case}_par"][:5])
    alpha, beta = float(g[f"{case}_par"][5]), float(g[f"{case}_par"][6])
    Y = oracle.gemm(kind, "row", ptr[:-1], ptr[1:], g["col"], g["val"], alpha, g[f"{case}_X"], columns, ldx, beta,
                    g[f"{case}_Y0"].copy(), ldy)
    rows = len(ptr) - 1
    scale = mm_scale(ptr, g["col"], g["val"], g[f"{case}_X"], columns, ldx, alpha, beta, g[f"{case}_Y0"], ldy)
    got = Y.reshape(rows, ldy)[:, :columns].reshape(-1)
    ref = g[f"{case}_row"].reshape(rows, ldy)[:, :columns].reshape(-1)
    assert_rows_close(kind, got, ref, scale.reshape(-1), f"mm row {case}")
    # padding between rows is never written
    assert np.array_equal(Y.reshape(rows, ldy)[:, columns:], g[f"{case}_Y0"].reshape(rows, ldy)[:, columns:])
    Yc = oracle.gemm(kind, "col", ptr[:-1], ptr[1:], g["col"], g["val"], alpha, g[f"{case}_Xc"], columns, ldxc, beta,
                     g[f"{case}_Yc0"].copy(), ldyc)
    # same operation in the other layout: compare with the tolerance of the transposed scale
    Xc = g[f"{case}_Xc"].reshape(columns, ldxc)[:, : int(g["cols"])].T.copy()
    Yc0 = g[f"{case}_Yc0"].reshape(columns, ldyc)[:, :rows].T.copy()
    sc = mm_scale(ptr, g["col"], g["val"], Xc.reshape(-1), columns, columns, alpha, beta, Yc0.reshape(-1), columns)
    assert_rows_close(kind, Yc.reshape(columns, ldyc)[:, :rows].T.reshape(-1),
                      g[f"{case}_col"].reshape(columns, ldyc)[:, :rows].T.reshape(-1), sc.reshape(-1), f"mm col {case}")


def test_structured_descriptors_golden():
    """symv / trmv / diagmv restatements against the reference's plain kernels (all fill / diag / op variants)."""
    g = golden("struct_d.npz")
    ptr, a, b = g["ptr"], float(g["alpha"]), float(g["beta"])
    full = np.abs(b * g["y0"]) + abs(a) * (np.bincount(np.repeat(np.arange(160), np.diff(ptr)),
                                                       weights=np.abs(g["val"] * g["x"][g["col"]]), minlength=160) +
                                           np.bincount(g["col"], weights=np.abs(g["val"] * np.repeat(g["x"], np.diff(ptr))),
                                                       minlength=160) + np.abs(g["x"]))
    n = 0
    for t, transes in ((1, (0,)), (3, (0, 1)), (4, (0,))):
        for upper in (0, 1):
            for unit in (0, 1):
                for tr in transes:
                    y = oracle.structured_mv("d", t, upper, unit, tr, ptr[:-1], ptr[1:], g["col"], g["val"], a, g["x"],
                                             b, g["y0"].copy())
                    assert_rows_close("d", y, g[f"y_t{t}_u{upper}_d{unit}_o{tr}"], full, f"type {t} {upper}{unit}{tr}")
                    n += 1
    assert n == 16


def test_structured_mm_golden():
    """symm / trmm / diagmm restatements against the reference's plain kernels: every fill / diag / operation
    variant in both layouts with padded leading dimensions."""
    g = golden("struct_mm_d.npz")
    ptr, a, b = g["ptr"], float(g["alpha"]), float(g["beta"])
    columns, ldx, ldy, ldxc, ldyc = (int(v) for v in g["par"])
    n, n_cases = 160, 0
    for key in (k[4:] for k in g.files if k.startswith("row_")):
        t, upper, unit, tr = (int(f[1:]) for f in key.split("_"))
        for lay, X, Y0, lx, ly in (("row", g["Xr"], g["Yr"], ldx, ldy), ("col", g["Xc"], g["Yc"], ldxc, ldyc)):
            Y = oracle.structured_mm("d", t, upper, unit, tr, lay, ptr[:-1], ptr[1:], g["col"], g["val"], a, X, columns,
                                     lx, b, Y0.copy(), ly)
            ref = g[f"{lay}_{key}"]
            view = (lambda v: v.reshape(n, ly)[:, :columns]) if lay == "row" else (lambda v: v.reshape(columns, ly)[:, :n].T)
            xv = X.reshape(n, lx)[:, :columns] if lay == "row" else X.reshape(columns, lx)[:, :n].T
            sc = structured_scale(n, ptr, g["col"], g["val"], xv, view(Y0), a, b)
            assert_rows_close("d", view(Y).reshape(-1), view(ref).reshape(-1), sc.reshape(-1), f"{lay} {key}")
            pad = (lambda v: v.reshape(n, ly)[:, columns:]) if lay == "row" else (lambda v: v.reshape(columns, ly)[:, n:])
            assert np.array_equal(pad(Y), pad(Y0)) and np.array_equal(pad(ref), pad(Y0))
            n_cases += 1
    assert n_cases == 2 * (4 + 8 + 2)


def coo_scale(rows_out, r, c, val, X, Y0, alpha, beta):
    """|beta*Y0| + |alpha| * sum |a * X[c, :]| scattered to row r; X, Y0 two-dimensional (rows, dense columns)."""
    out = np.zeros((rows_out, X.shape[1]))
    np.add.at(out, r, np.abs(val.astype(np.float64))[:, None] * np.abs(X.astype(np.float64))[c])
    return np.abs(beta * Y0.astype(np.float64)) + abs(alpha) * out


def test_coo_products_golden():
    """gemv_coo / gemm_coo restatements (both operations and layouts) against the reference's plain kernels on
    unsorted entries with repeated pairs."""
    g = golden("coo_d.npz")
    ri, ci, val, a, b = g["ri"], g["ci"], g["val"], float(g["alpha"]), float(g["beta"])
    rows, cols = int(g["rows"]), int(g["cols"])
    columns, ldx, ldy = (int(v) for v in g["par"])
    for tr in (0, 1):
        m_out, m_in = (cols, rows) if tr else (rows, cols)
        r, c = (ci, ri) if tr else (ri, ci)
        y = oracle.gemv_coo("d", tr, rows, cols, ri, ci, val, a, g[f"x_o{tr}"], b, g[f"y0_o{tr}"].copy())
        sc = coo_scale(m_out, r, c, val, g[f"x_o{tr}"][:, None], g[f"y0_o{tr}"][:, None], a, b)
        assert_rows_close("d", y, g[f"y_o{tr}"], sc.reshape(-1), f"coo mv op {tr}")
        Y = oracle.gemm_coo("d", tr, "row", rows, cols, ri, ci, val, a, g[f"Xr_o{tr}"], columns, ldx, b,
                            g[f"Yr0_o{tr}"].copy(), ldy)
        sc = coo_scale(m_out, r, c, val, g[f"Xr_o{tr}"].reshape(m_in, ldx)[:, :columns],
                       g[f"Yr0_o{tr}"].reshape(m_out, ldy)[:, :columns], a, b)
        assert_rows_close("d", Y.reshape(m_out, ldy)[:, :columns].reshape(-1),
                          g[f"Yr_o{tr}"].reshape(m_out, ldy)[:, :columns].reshape(-1), sc.reshape(-1), f"coo mm row op {tr}")
        assert np.array_equal(Y.reshape(m_out, ldy)[:, columns:], g[f"Yr0_o{tr}"].reshape(m_out, ldy)[:, columns:])
        lx, ly = m_in + 2, m_out + 1
        Y = oracle.gemm_coo("d", tr, "col", rows, cols, ri, ci, val, a, g[f"Xc_o{tr}"], columns, lx, b,
                            g[f"Yc0_o{tr}"].copy(), ly)
        sc = coo_scale(m_out, r, c, val, g[f"Xc_o{tr}"].reshape(columns, lx)[:, :m_in].T,
                       g[f"Yc0_o{tr}"].reshape(columns, ly)[:, :m_out].T, a, b)
        assert_rows_close("d", Y.reshape(columns, ly)[:, :m_out].T.reshape(-1),
                          g[f"Yc_o{tr}"].reshape(columns, ly)[:, :m_out].T.reshape(-1), sc.reshape(-1), f"coo mm col op {tr}")


def test_csc_products_golden():
    """gemv_csc / gemm_csc restatements (both operations and layouts) against the reference's plain kernels on a
    matrix with more columns than rows."""
    g = golden("csc_d.npz")
    ptr, ri, val, a, b = g["ptr"], g["ri"], g["val"], float(g["alpha"]), float(g["beta"])
    rows, cols = int(g["rows"]), int(g["cols"])
    columns, ldx, ldy = (int(v) for v in g["par"])
    cid = np.repeat(np.arange(cols), np.diff(ptr))
    for tr in (0, 1):
        m_out, m_in = (cols, rows) if tr else (rows, cols)
        r, c = (cid, ri) if tr else (ri, cid)
        y = oracle.gemv_csc("d", tr, rows, cols, ptr[:-1], ptr[1:], ri, val, a, g[f"x_o{tr}"], b, g[f"y0_o{tr}"].copy())
        sc = coo_scale(m_out, r, c, val, g[f"x_o{tr}"][:, None], g[f"y0_o{tr}"][:, None], a, b)
        assert_rows_close("d", y, g[f"y_o{tr}"], sc.reshape(-1), f"csc mv op {tr}")
        Y = oracle.gemm_csc("d", tr, "row", rows, cols, ptr[:-1], ptr[1:], ri, val, a, g[f"Xr_o{tr}"], columns, ldx, b,
                            g[f"Yr0_o{tr}"].copy(), ldy)
        sc = coo_scale(m_out, r, c, val, g[f"Xr_o{tr}"].reshape(m_in, ldx)[:, :columns],
                       g[f"Yr0_o{tr}"].reshape(m_out, ldy)[:, :columns], a, b)
        assert_rows_close("d", Y.reshape(m_out, ldy)[:, :columns].reshape(-1),
                          g[f"Yr_o{tr}"].reshape(m_out, ldy)[:, :columns].reshape(-1), sc.reshape(-1), f"csc mm row op {tr}")
        assert np.array_equal(Y.reshape(m_out, ldy)[:, columns:], g[f"Yr0_o{tr}"].reshape(m_out, ldy)[:, columns:])
        lx, ly = m_in + 2, m_out + 1
        Y = oracle.gemm_csc("d", tr, "col", rows, cols, ptr[:-1], ptr[1:], ri, val, a, g[f"Xc_o{tr}"], columns, lx, b,
                            g[f"Yc0_o{tr}"].copy(), ly)
        sc = coo_scale(m_out, r, c, val, g[f"Xc_o{tr}"].reshape(columns, lx)[:, :m_in].T,
                       g[f"Yc0_o{tr}"].reshape(columns, ly)[:, :m_out].T, a, b)
        assert_rows_close("d", Y.reshape(columns, ly)[:, :m_out].T.reshape(-1),
                          g[f"Yc_o{tr}"].reshape(columns, ly)[:, :m_out].T.reshape(-1), sc.reshape(-1), f"csc mm col op {tr}")


def test_coo_to_csr_golden():
    g = golden("cfg1_s.npz")
    ptr, col, val = oracle.coo_to_csr("s", 1, 1000, g["coo_ri"] + 1, g["coo_ci"] + 1, g["coo_v"])
    assert np.array_equal(ptr, g["csr_ptr"]) and np.array_equal(col, g["csr_col"])
    assert np.array_equal(val.view(np.uint32), g["csr_val"].view(np.uint32))
    # and it is the matrix the COO was cut from
    assert np.array_equal(ptr, g["ptr"]) and np.array_equal(col, g["col"]) and np.array_equal(val, g["val"])


def test_partition_golden():
    g = golden("partition.npz")
    for name in ("tiny", "cfg1", "zipf", "one_row", "flat"):
        for p in (1, 2, 3, 4, 8):
            assert np.array_equal(oracle.partition_rows_by_nnz(g[f"{name}_acc"], p), g[f"{name}_p{p}"]), (name, p)
    assert g["tiny_p2"].tolist() == [0, 0, 3]  # the crossing row goes to the next part; parts may be empty


def test_mv_status_order():
    S = oracle.mv_status
    assert S(has_handle=0) == 1 and S(has_mat=0) == 1 and S(has_x=0) == 1 and S(has_y=0) == 1
    assert S(has_x=0, handle_datatype=1) == 1          # NULL checks come before the datatype check
    assert S(handle_datatype=1, call_datatype=0) == 3
    assert S(operation=2) == 3
    assert S(descr_type=1, rows=3, cols=4) == 3 and S(descr_type=1, rows=3, cols=3) == -1
    assert S(descr_type=0) == 0 and S(descr_type=6) == 3 and S(fmt=9) == 3 and S(fmt=0) == -1


@pytest.mark.skipif(not oracle.ref_available(), reason="reference objects not built on this machine")
@pytest.mark.parametrize("kind", ["s", "d"])
def test_live_against_reference_objects(kind):
    """Fresh seeded inputs through both the restatement and the reference's compiled sources."""
    lens = synth.rowlen_zipf(11, 4000, 1.8, 1, 900)
    lens[5::11] = 0
    m = synth.from_lengths(kind, 11, lens, 3000)
    x, y0 = synth.vector(kind, 11, 1, 3000), synth.vector(kind, 11, 2, 4000)
    A = oracle.RefCsr.from_csr(kind, 0, 4000, 3000, m.rows_start, m.rows_end, m.col, m.val)
    p, c, v = A.export()
    op, oc, ov = oracle.create_csr(kind, 0, m.rows_start, m.rows_end, m.col, m.val)
    assert np.array_equal(p, op) and np.array_equal(c, oc) and np.array_equal(v, ov)
    scale = row_scale(m.ptr, m.col, m.val, x, 0.7, -1.3, y0)
    y_ref = A.gemv(0.7, x, -1.3, y0.copy())
    assert_rows_close(kind, oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, 0.7, x, -1.3, y0.copy()), y_ref,
                      scale, "plain")
    assert_rows_close(kind, A.gemv(0.7, x, -1.3, y0.copy(), omp_threads=4), y_ref, scale, "reference OpenMP kernel")
    for parts in (2, 4, 8):
        assert np.array_equal(oracle.partition_rows_by_nnz(m.rows_end, parts),
                              oracle.ref_partition_rows_by_nnz(m.rows_end, parts))
    X, Y0 = synth.vector(kind, 11, 3, 3000 * 8), synth.vector(kind, 11, 4, 4000 * 8)
    Yr = A.gemm("row", 1.25, X, 8, 8, 0.5, Y0.copy(), 8)
    Yo = oracle.gemm(kind, "row", m.rows_start, m.rows_end, m.col, m.val, 1.25, X, 8, 8, 0.5, Y0.copy(), 8)
    assert_rows_close(kind, Yo, Yr, mm_scale(m.ptr, m.col, m.val, X, 8, 8, 1.25, 0.5, Y0, 8).reshape(-1), "mm")


@pytest.mark.skipif(not oracle.ref_available(), reason="reference objects not built on this machine")
@pytest.mark.parametrize("kind", ["s", "d"])
def test_live_structured_and_coo_against_reference_objects(kind):
    """Fresh seeded square matrix through the restatements of symm / trmm / diagmm and of the COO kernels and
    through the reference's compiled sources: every variant, both precisions."""
    n, columns = 300, 4
    m = synth.poisson(kind, 17, n, n, 6.0)
    A = oracle.RefCsr.from_csr(kind, 0, n, n, m.rows_start, m.rows_end, m.col, m.val)
    X, Y0 = synth.vector(kind, 17, 1, n * columns), synth.vector(kind, 17, 2, n * columns)
    checked = 0
    for t, transes in ((1, (0,)), (3, (0, 1)), (4, (0,))):
        for upper in ((0,) if t == 4 else (0, 1)):
            for unit in (0, 1):
                for tr in transes:
                    for lay in ("row", "col"):
                        ld = columns if lay == "row" else n
                        want = A.structured_mm(t, upper, unit, tr, lay, 1.5, X, columns, ld, -0.5, Y0.copy(), ld)
                        got = oracle.structured_mm(kind, t, upper, unit, tr, lay, m.rows_start, m.rows_end, m.col, m.val,
                                                   1.5, X, columns, ld, -0.5, Y0.copy(), ld)
                        as2d = (lambda v: v.reshape(n, columns)) if lay == "row" else (lambda v: v.reshape(columns, n).T)
                        sc = structured_scale(n, m.ptr, m.col, m.val, as2d(X), as2d(Y0), 1.5, -0.5)
                        assert_rows_close(kind, as2d(got).reshape(-1), as2d(want).reshape(-1), sc.reshape(-1),
                                          f"type {t} {upper}{unit}{tr} {lay}")
                        checked += 1
    assert checked == 28
    rng = np.random.default_rng(17)
    perm = rng.permutation(m.nnz)
    ri = np.repeat(np.arange(n, dtype=np.int32), np.diff(m.ptr))[perm]
    ci, v = m.col[perm], m.val[perm]
    K = oracle.RefCoo(kind, 0, n, n, ri, ci, v)
    x, y0 = synth.vector(kind, 17, 3, n), synth.vector(kind, 17, 4, n)
    for tr in (0, 1):
        r, c = (ci, ri) if tr else (ri, ci)
        sc = coo_scale(n, r, c, v, x[:, None], y0[:, None], 0.75, 1.25).reshape(-1)
        assert_rows_close(kind, oracle.gemv_coo(kind, tr, n, n, ri, ci, v, 0.75, x, 1.25, y0.copy()),
                          K.gemv(tr, 0.75, x, 1.25, y0.copy()), sc, f"coo mv {tr}")
        for lay in ("row", "col"):
            ld = columns if lay == "row" else n
            as2d = (lambda w: w.reshape(n, columns)) if lay == "row" else (lambda w: w.reshape(columns, n).T)
            sc = coo_scale(n, r, c, v, as2d(X), as2d(Y0), 0.75, 1.25)
            got = oracle.gemm_coo(kind, tr, lay, n, n, ri, ci, v, 0.75, X, columns, ld, 1.25, Y0.copy(), ld)
            want = K.gemm(tr, lay, 0.75, X, columns, ld, 1.25, Y0.copy(), ld)
            assert_rows_close(kind, as2d(got).reshape(-1), as2d(want).reshape(-1), sc.reshape(-1), f"coo mm {tr} {lay}")
