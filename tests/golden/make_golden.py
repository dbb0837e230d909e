"""Regenerates the golden vectors in this directory from the REFERENCE'S OWN code.

    python tests/golden/make_golden.py        (needs oracle/_ref/libalpha_ref.so, i.e. the
                                               reference tree mounted and `make -C oracle ref`)

Inputs come from the seeded generators in alsparse_b200.synth; every expected output is
produced by the reference's objects (its plain serial kernels, create_csr, create_coo +
COO->CSR conversion, balanced_partition_row_by_nnz), compiled with the reference's -Ofast.
The files pin the C restatement in oracle/oracle.c (tests/test_oracle.py) and serve as known
answers for the CUDA library on machines where the reference tree is absent.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402
from alsparse_b200 import synth  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
NP = {"s": np.float32, "d": np.float64}


def mv_case(kind, m, alpha, beta, seed, base=0):
    """Reference plain-kernel result for matrix m (synth.Csr) with seeded x, y0."""
    x = synth.vector(kind, seed, 1, m.cols)
    y0 = synth.vector(kind, seed, 2, m.nrows)
    A = oracle.RefCsr.from_csr(kind, base, m.nrows, m.cols, m.rows_start + base, m.rows_end + base, m.col + base,
                               m.val)
    y = A.gemv(alpha, x, beta, y0.copy())
    return dict(ptr=m.ptr, col=m.col, val=m.val, x=x, y0=y0, y=y, alpha=alpha, beta=beta, rows=m.nrows, cols=m.cols)


def main():
    if not oracle.ref_available():
        sys.exit("oracle/_ref/libalpha_ref.so not built: the reference tree is needed")

    # -- the 3x3 hand case: zero- and one-based create_csr, mv and row-major mm -----------------
    rs, re_ = np.array([0, 2, 3], np.int32), np.array([2, 3, 4], np.int32)
    col, val = np.array([0, 2, 1, 0], np.int32), np.array([1, 2, 3, 4], np.float32)
    x = np.array([1, 10, 100], np.float32)
    A0 = oracle.RefCsr.from_csr("s", 0, 3, 3, rs, re_, col, val)
    A1 = oracle.RefCsr.from_csr("s", 1, 3, 3, rs + 1, re_ + 1, col + 1, val)
    B = np.arange(1, 7, dtype=np.float32)
    np.savez(os.path.join(OUT, "kat3x3.npz"), rs=rs, re=re_, col=col, val=val, x=x,
             y_a2_b3=A0.gemv(2.0, x, 3.0, np.ones(3, np.float32)),
             y_base1=A1.gemv(2.0, x, 3.0, np.ones(3, np.float32)),
             base1_ptr=A1.export()[0], base1_col=A1.export()[1],
             B=B, mm_row=A0.gemm("row", 1.0, B, 2, 2, 0.0, np.zeros(6, np.float32), 2),
             mm_col=A0.gemm("col", 1.0, B, 2, 3, 0.0, np.zeros(6, np.float32), 3))

    # -- configuration 1: 1000 x 1000, 5000 stored elements, fp32 --------------------------------
    m = synth.poisson("s", 0, 1000, 1000, 5.0, total=5000)
    c = mv_case("s", m, 1.0, 0.0, 0)
    c2 = mv_case("s", m, 1.5, 0.5, 0)
    # the same matrix as shuffled COO through the reference's create_coo + COO->CSR, one-based
    perm = np.random.default_rng(0).permutation(m.nnz)
    ri = np.repeat(np.arange(1000, dtype=np.int32), np.diff(m.ptr))[perm]
    ci, cv = m.col[perm], m.val[perm]
    R = oracle.RefCsr.from_coo("s", 1, 1000, 1000, ri + 1, ci + 1, cv)
    cp, cc, cvv = R.export()
    np.savez_compressed(os.path.join(OUT, "cfg1_s.npz"), y_ab=c2["y"], coo_ri=ri, coo_ci=ci, coo_v=cv, csr_ptr=cp,
                        csr_col=cc, csr_val=cvv, **c)

    # -- fp64: a small power-law matrix (long and empty rows) and a small 27-point stencil -------
    lens = synth.rowlen_zipf(3, 1500, 1.8, 1, 700)
    lens[::7] = 0  # empty rows
    z = synth.from_lengths("d", 3, lens, 1200)
    np.savez_compressed(os.path.join(OUT, "zipf_d.npz"), **mv_case("d", z, -0.75, 1.25, 3))
    s = synth.stencil27("d", 8)
    np.savez_compressed(os.path.join(OUT, "stencil8_d.npz"), **mv_case("d", s, 1.0, 0.0, 4))

    # -- transpose mv (plain kernel), rectangular ---------------------------------------------------
    t = synth.poisson("d", 5, 300, 450, 6.0)
    xt, y0t = synth.vector("d", 5, 1, 300), synth.vector("d", 5, 2, 450)
    T = oracle.RefCsr.from_csr("d", 0, 300, 450, t.rows_start, t.rows_end, t.col, t.val)
    np.savez_compressed(os.path.join(OUT, "trans_d.npz"), ptr=t.ptr, col=t.col, val=t.val, x=xt, y0=y0t,
                        y=T.gemv(0.5, xt, -2.0, y0t.copy(), trans=True), alpha=0.5, beta=-2.0, rows=300, cols=450)

    # -- SpMM: 64 columns tight, and 5 columns with padded leading dimensions, both layouts -----------
    for kind in "sd":
        a = synth.poisson(kind, 6, 96, 120, 8.0)
        A = oracle.RefCsr.from_csr(kind, 0, 96, 120, a.rows_start, a.rows_end, a.col, a.val)
        out = dict(ptr=a.ptr, col=a.col, val=a.val, rows=96, cols=120)
        for name, columns, ldx, ldy, alpha, beta in (("w64", 64, 64, 64, 1.0, 0.0), ("w5", 5, 7, 9, 1.5, 0.5)):
            X = synth.vector(kind, 6, 3, 120 * ldx)
            Y0 = synth.vector(kind, 6, 4, 96 * ldy)
            out[f"{name}_X"], out[f"{name}_Y0"] = X, Y0
            out[f"{name}_row"] = A.gemm("row", alpha, X, columns, ldx, beta, Y0.copy(), ldy)
            # column-major: X is (ldx_c x columns) with ldx_c >= cols; reuse the streams with new shapes
            ldxc, ldyc = 120 + (ldx - columns), 96 + (ldy - columns)
            Xc = synth.vector(kind, 6, 5, ldxc * columns)
            Yc0 = synth.vector(kind, 6, 6, ldyc * columns)
            out[f"{name}_Xc"], out[f"{name}_Yc0"] = Xc, Yc0
            out[f"{name}_col"] = A.gemm("col", alpha, Xc, columns, ldxc, beta, Yc0.copy(), ldyc)
            out[f"{name}_par"] = np.array([columns, ldx, ldy, ldxc, ldyc, alpha, beta])
        np.savez_compressed(os.path.join(OUT, f"mm_{kind}.npz"), **out)

    # -- structured descriptors (symmetric / triangular / diagonal) on a square matrix with missing and
    #    repeated diagonal entries: the reference's plain symv / trmv / diagmv kernels ---------------------
    q = synth.poisson("d", 9, 160, 160, 7.0)
    rid = np.repeat(np.arange(160), np.diff(q.ptr))
    keep = ~((q.col == rid) & (rid % 3 == 0))                     # every third row loses its diagonal
    qcol, qval, qlens = q.col[keep], q.val[keep], np.bincount(rid[keep], minlength=160)
    extra_r = np.arange(1, 160, 5)                                # some rows get a second diagonal entry at the end
    order = np.argsort(np.concatenate([rid[keep], extra_r]), kind="stable")
    qcol = np.concatenate([qcol, extra_r])[order].astype(np.int32)
    qval = np.concatenate([qval, np.full(len(extra_r), 0.25)])[order]
    qlens[extra_r] += 1
    qptr = np.concatenate([[0], np.cumsum(qlens)]).astype(np.int32)
    xs, ys = synth.vector("d", 9, 1, 160), synth.vector("d", 9, 2, 160)
    Q = oracle.RefCsr.from_csr("d", 0, 160, 160, qptr[:-1], qptr[1:], qcol, qval)
    out = dict(ptr=qptr, col=qcol, val=qval, x=xs, y0=ys, alpha=0.75, beta=-0.5)
    for t, transes in ((1, (0,)), (3, (0, 1)), (4, (0,))):
        for upper in (0, 1):
            for unit in (0, 1):
                for tr in transes:
                    out[f"y_t{t}_u{upper}_d{unit}_o{tr}"] = Q.structured_mv(t, upper, unit, tr, 0.75, xs, -0.5, ys.copy())
    np.savez_compressed(os.path.join(OUT, "struct_d.npz"), **out)

    # -- the same descriptors in mm: the reference's plain symm / trmm / diagmm kernels, both layouts, padded
    #    leading dimensions (the repeated diagonal entries separate "all" / "last" / "first") --------------
    columns, ldx, ldy, ldxc, ldyc = 5, 7, 6, 163, 161
    Xr, Yr = synth.vector("d", 9, 3, 160 * ldx), synth.vector("d", 9, 4, 160 * ldy)
    Xc, Yc = synth.vector("d", 9, 5, ldxc * columns), synth.vector("d", 9, 6, ldyc * columns)
    out = dict(ptr=qptr, col=qcol, val=qval, Xr=Xr, Yr=Yr, Xc=Xc, Yc=Yc, alpha=0.75, beta=-0.5,
               par=np.array([columns, ldx, ldy, ldxc, ldyc]))
    for t, transes in ((1, (0,)), (3, (0, 1)), (4, (0,))):
        for upper in ((0,) if t == 4 else (0, 1)):
            for unit in (0, 1):
                for tr in transes:
                    key = f"t{t}_u{upper}_d{unit}_o{tr}"
                    out[f"row_{key}"] = Q.structured_mm(t, upper, unit, tr, "row", 0.75, Xr, columns, ldx, -0.5, Yr.copy(), ldy)
                    out[f"col_{key}"] = Q.structured_mm(t, upper, unit, tr, "col", 0.75, Xc, columns, ldxc, -0.5, Yc.copy(), ldyc)
    np.savez_compressed(os.path.join(OUT, "struct_mm_d.npz"), **out)

    # -- a COO handle given straight to mv / mm: the reference's plain gemv_coo / gemm_coo kernels on unsorted
    #    one-based entries with a few repeated (row, col) pairs ---------------------------------------------
    cm = synth.poisson("d", 13, 150, 210, 5.0)
    rng = np.random.default_rng(13)
    cri = np.repeat(np.arange(150, dtype=np.int32), np.diff(cm.ptr))
    dup = rng.integers(0, cm.nnz, 40)
    cri, cci = np.concatenate([cri, cri[dup]]), np.concatenate([cm.col, cm.col[dup]])
    cv = np.concatenate([cm.val, rng.uniform(-1, 1, 40)])
    perm = rng.permutation(len(cri))
    cri, cci, cv = cri[perm].astype(np.int32), cci[perm].astype(np.int32), cv[perm]
    K = oracle.RefCoo("d", 1, 150, 210, cri + 1, cci + 1, cv)
    columns, ldx, ldy = 6, 8, 7
    out = dict(ri=cri, ci=cci, val=cv, rows=150, cols=210, alpha=1.25, beta=-0.75, par=np.array([columns, ldx, ldy]))
    for tr, m_out, m_in in ((0, 150, 210), (1, 210, 150)):
        xk, yk = synth.vector("d", 13, 1 + tr, m_in), synth.vector("d", 13, 3 + tr, m_out)
        out[f"x_o{tr}"], out[f"y0_o{tr}"] = xk, yk
        out[f"y_o{tr}"] = K.gemv(tr, 1.25, xk, -0.75, yk.copy())
        Xr, Yr = synth.vector("d", 13, 5 + tr, m_in * ldx), synth.vector("d", 13, 7 + tr, m_out * ldy)
        Xc, Yc = synth.vector("d", 13, 9 + tr, (m_in + 2) * columns), synth.vector("d", 13, 11 + tr, (m_out + 1) * columns)
        out[f"Xr_o{tr}"], out[f"Yr0_o{tr}"], out[f"Xc_o{tr}"], out[f"Yc0_o{tr}"] = Xr, Yr, Xc, Yc
        out[f"Yr_o{tr}"] = K.gemm(tr, "row", 1.25, Xr, columns, ldx, -0.75, Yr.copy(), ldy)
        out[f"Yc_o{tr}"] = K.gemm(tr, "col", 1.25, Xc, columns, m_in + 2, -0.75, Yc.copy(), m_out + 1)
    np.savez_compressed(os.path.join(OUT, "coo_d.npz"), **out)

    # -- a CSC handle in mv / mm: the reference's plain gemv_csc / gemm_csc kernels on a matrix with more columns
    #    than rows (one-based input to the product library) ------------------------------------------------
    rows_c, cols_c = 130, 170
    t = synth.poisson("d", 19, cols_c, rows_c, 5.0)            # the CSR of A^T holds the CSC arrays of A
    Kc = oracle.RefCsc("d", rows_c, cols_c, t.ptr[:-1], t.ptr[1:], t.col, t.val)
    columns, ldx, ldy = 6, 8, 7
    out = dict(ptr=t.ptr, ri=t.col, val=t.val, rows=rows_c, cols=cols_c, alpha=1.25, beta=-0.75,
               par=np.array([columns, ldx, ldy]))
    for tr, m_out, m_in in ((0, rows_c, cols_c), (1, cols_c, rows_c)):
        xk, yk = synth.vector("d", 19, 1 + tr, m_in), synth.vector("d", 19, 3 + tr, m_out)
        out[f"x_o{tr}"], out[f"y0_o{tr}"] = xk, yk
        out[f"y_o{tr}"] = Kc.gemv(tr, 1.25, xk, -0.75, yk.copy())
        Xr, Yr = synth.vector("d", 19, 5 + tr, m_in * ldx), synth.vector("d", 19, 7 + tr, m_out * ldy)
        Xc, Yc = synth.vector("d", 19, 9 + tr, (m_in + 2) * columns), synth.vector("d", 19, 11 + tr, (m_out + 1) * columns)
        out[f"Xr_o{tr}"], out[f"Yr0_o{tr}"], out[f"Xc_o{tr}"], out[f"Yc0_o{tr}"] = Xr, Yr, Xc, Yc
        out[f"Yr_o{tr}"] = Kc.gemm(tr, "row", 1.25, Xr, columns, ldx, -0.75, Yr.copy(), ldy)
        out[f"Yc_o{tr}"] = Kc.gemm(tr, "col", 1.25, Xc, columns, m_in + 2, -0.75, Yc.copy(), m_out + 1)
    np.savez_compressed(os.path.join(OUT, "csc_d.npz"), **out)

    # -- nnz-balanced row partition: known answers incl. the quirks ---------------------------------
    cases = {}
    accs = {"tiny": np.array([2, 3, 4], np.int32), "cfg1": m.ptr[1:], "zipf": z.ptr[1:],
            "one_row": np.array([9], np.int32), "flat": np.arange(1, 65, dtype=np.int32) * 16}
    for name, acc in accs.items():
        cases[f"{name}_acc"] = acc
        for p in (1, 2, 3, 4, 8):
            cases[f"{name}_p{p}"] = oracle.ref_partition_rows_by_nnz(acc, p)
    np.savez_compressed(os.path.join(OUT, "partition.npz"), **cases)
    print("golden vectors written to", OUT)


if __name__ == "__main__":
    main()
