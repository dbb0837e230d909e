"""The two places where the reference's own code meets this library, exercised with real C callers.

* A test program in the reference's style (tests/ref_style/mv_d_csr_main.c: getters, matrix file reader, COO ->
  CSR, random fill, timed alphasparse_d_mv) compiled against the REFERENCE's include/ directory when it is on
  this machine (ALPHASPARSE_REFERENCE_DIR or a `reference` checkout beside the repository), else against this repository's, and linked to the library.
* A caller of the kernel-level symbols (tests/ref_style/kernel_tree_caller.c: gemv_{s,d}_csr, gemv_d_csr_trans,
  gemm_d_csr_row on a bare CSR record), which is what the reference's dispatch tables do with the tree they link.

Compiling and linking need no GPU; the runs are marked gpu and checked against the oracle."""
import os
import subprocess

import numpy as np
import pytest

import oracle
from alsparse_b200 import capi, synth
from helpers import TOL, assert_rows_close, mm_scale, reference_dir, row_scale

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "ref_style")
REF_INC = os.path.join(reference_dir() or "", "include")
INCLUDES = [os.path.join(ROOT, "include")] + ([REF_INC] if os.path.isfile(os.path.join(REF_INC, "alphasparse.h")) else [])


def _compile(name, inc, out_dir):
    exe = os.path.join(out_dir, name + ("_ref" if inc == REF_INC else ""))
    capi.load()  # builds nothing, but fails loudly when the library is missing
    subprocess.check_call(["/usr/bin/gcc", "-std=gnu11", "-O1", "-w", "-I", inc, os.path.join(SRC, name + ".c"), "-o", exe,
                           capi.LIB_PATH, "-Wl,-rpath," + os.path.dirname(capi.LIB_PATH), "-lm"])
    return exe


@pytest.mark.parametrize("inc", INCLUDES)
def test_reference_style_programs_compile_and_link(inc, tmp_path):
    for name in ("mv_d_csr_main", "kernel_tree_caller"):
        exe = _compile(name, inc, str(tmp_path))
        undefined = subprocess.run(["ldd", "-r", exe], capture_output=True, text=True).stdout
        assert "undefined symbol" not in undefined, undefined


def test_command_line_getters_follow_the_reference():
    """args_* / alpha_args_*: --name=value with one or two dashes, unambiguous prefixes, defaults, first
    occurrence wins (last for the descriptor fields), --data-fileA overrides --data-file wherever it stands."""
    import ctypes as C
    lib = capi.load()

    def argv(*a):
        arr = (C.c_char_p * (len(a) + 1))(b"prog", *[s.encode() for s in a])
        return len(a) + 1, arr

    n, v = argv("--data-file=a.mtx", "-iter=7", "--thread-num=3", "--check", "--transA=T", "--typeA=S", "--fillA=U",
                "--diagA=U", "--columns=5", "--layout=C", "--data-fileB=b.mtx", "--iter=9")
    assert lib.args_get_data_file(n, v) == b"a.mtx" and lib.args_get_iter(n, v) == 7
    assert lib.args_get_thread_num(n, v) == 3 and lib.args_get_if_check(n, v) is True
    assert lib.alpha_args_get_transA(n, v) == capi.TRANSPOSE and lib.alpha_args_get_transB(n, v) == capi.NON_TRANSPOSE
    d = lib.alpha_args_get_matrix_descrA(n, v)
    assert (d.type, d.mode, d.diag) == (capi.SYMMETRIC, 1, 1)
    d = lib.alpha_args_get_matrix_descrB(n, v)
    assert (d.type, d.mode, d.diag) == (capi.GENERAL, 0, 0)
    assert lib.args_get_columns(n, v, 11) == 5 and lib.alpha_args_get_layout(n, v) == capi.COLUMN_MAJOR
    assert lib.args_get_data_fileA(n, v) == b"a.mtx" and lib.args_get_data_fileB(n, v) == b"b.mtx"
    n, v = argv("--thread=2", "positional")                       # a prefix that names one option only
    assert lib.args_get_thread_num(n, v) == 2 and lib.args_get_iter(n, v) == 1 and lib.args_get_if_check(n, v) is False
    assert lib.args_get_data_file(n, v) == b"" and lib.args_get_columns(n, v, 11) == 11
    n, v = argv("--data-file=x", "--data-file=y")                  # ambiguous prefixes name nothing: --data is skipped
    assert lib.args_get_data_fileA(n, v) == b"y" and lib.args_get_data_file(n, v) == b"x"
    assert lib.alphasparse_matrix_type_parse(b"BT") == 5 and lib.alphasparse_layout_parse(b"ROW") == capi.ROW_MAJOR


def test_timers_fills_and_operation_counts():
    import ctypes as C
    lib = capi.load()
    t = capi.AlphaTimer()
    lib.alpha_timing_start(C.byref(t))
    lib.alpha_timing_end(C.byref(t))
    assert 0.0 <= lib.alpha_timing_elapsed_time(C.byref(t)) < 1.0
    t.start, t.end = 1.0, 3.0
    assert lib.alpha_timing_gflops(C.byref(t), 4 * 10 ** 9) == 2.0
    a, b = np.empty(1000), np.empty(1000)
    lib.alpha_fill_random_d(a.ctypes.data, 7, 1000)
    lib.alpha_fill_random_d(b.ctypes.data, 7, 1000)
    assert np.array_equal(a, b) and a.min() >= 0.0 and a.max() <= 1.0 and len(np.unique(a)) > 900
    f = np.empty(10, np.float32)
    lib.alpha_fill_s(f.ctypes.data, 2.5, 10)
    assert (f == 2.5).all()
    ri, ci = np.array([0, 1, 2, 2, 0], np.int32), np.array([0, 0, 2, 1, 2], np.int32)
    lo, di, hi = C.c_int32(), C.c_int32(), C.c_int32()
    lib.alphasparse_nnz_counter_coo(ri.ctypes.data, ci.ctypes.data, 5, C.byref(lo), C.byref(di), C.byref(hi))
    assert (lo.value, di.value, hi.value) == (2, 2, 1)
    # the reference's count (src/util/analysis.c:130-156): (touched * 2 + rows * 3) * columns for real types
    G = capi.MatrixDescr(capi.GENERAL, 0, 0)
    assert lib.alphasparse_operations_mv(3, 3, 2, 2, 1, capi.NON_TRANSPOSE, G, capi.DOUBLE) == 5 * 2 + 3 * 3
    assert lib.alphasparse_operations_mm(3, 3, 2, 2, 1, capi.NON_TRANSPOSE, G, 4, capi.FLOAT) == (5 * 2 + 9) * 4
    T = capi.MatrixDescr(capi.TRIANGULAR, 1, 1)                   # upper, unit diagonal, transposed: lo + rows
    assert lib.alphasparse_operations_mv(3, 3, 2, 2, 1, capi.TRANSPOSE, T, capi.DOUBLE) == (2 + 3) * 2 + 9
    assert lib.alphasparse_operations_mv(3, 3, 2, 2, 1, capi.NON_TRANSPOSE, G, capi.DOUBLE_COMPLEX) == 5 * 9 + 3 * 16


def _write_mtx(path, m):
    with open(path, "w") as fp:
        fp.write("%%MatrixMarket matrix coordinate real general\n")
        fp.write(f"{m.nrows} {m.cols} {m.nnz}\n")
        rows = np.repeat(np.arange(m.nrows), np.diff(m.ptr))
        order = np.random.default_rng(3).permutation(m.nnz)          # the file is in no particular order
        for k in order:
            fp.write(f"{rows[k] + 1} {m.col[k] + 1} {float(m.val[k])!r}\n")


@pytest.mark.gpu
@pytest.mark.parametrize("inc", INCLUDES)
@pytest.mark.parametrize("trans", ["N", "T"])
def test_reference_style_main_runs(inc, trans, tmp_path):
    import ctypes as C
    exe = _compile("mv_d_csr_main", inc, str(tmp_path))
    m = synth.poisson("d", 21, 3000, 2500, 9.0)
    mtx, out = str(tmp_path / "m.mtx"), str(tmp_path / "y.bin")
    _write_mtx(mtx, m)
    res = subprocess.run([exe, f"--data-file={mtx}", "--iter=1", f"--transA={trans}", "--thread-num=2", out],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert f"rows 3000 cols 2500 nnz {m.nnz}" in res.stdout and "alphasparse_d_mv time" in res.stdout
    lib = capi.load()
    nx, ny = (2500, 3000) if trans == "N" else (3000, 2500)
    x, y0 = np.empty(nx), np.empty(ny)
    lib.alpha_fill_random_d(x.ctypes.data, 1, nx)
    lib.alpha_fill_random_d(y0.ctypes.data, 2, ny)
    y = np.fromfile(out, dtype=np.float64)
    if trans == "N":
        ref = oracle.gemv("d", m.rows_start, m.rows_end, m.col, m.val, 2.0, x, 0.5, y0.copy())
        scale = row_scale(m.ptr, m.col, m.val, x, 2.0, 0.5, y0)
    else:
        ref = oracle.gemv_trans("d", m.cols, m.rows_start, m.rows_end, m.col, m.val, 2.0, x, 0.5, y0.copy())
        prod = np.abs(m.val * x[np.repeat(np.arange(m.nrows), np.diff(m.ptr))])
        scale = np.abs(0.5 * y0) + 2.0 * np.bincount(m.col, weights=prod, minlength=m.cols)
    assert_rows_close("d", y, ref, scale, f"reference-style main, op {trans}")


@pytest.mark.gpu
@pytest.mark.parametrize("inc", INCLUDES)
def test_kernel_level_symbols_serve_a_bare_record(inc, tmp_path):
    exe = _compile("kernel_tree_caller", inc, str(tmp_path))
    columns = 6
    m = synth.zipf("d", 22, 4000, 3500, 1.8, 1, 3000)
    X = synth.vector("d", 22, 1, m.cols * columns)
    Y0 = synth.vector("d", 22, 2, m.nrows * columns)
    inp, out = str(tmp_path / "in.bin"), str(tmp_path / "out.bin")
    with open(inp, "wb") as fp:
        np.array([m.nrows, m.cols, m.nnz, columns], np.int32).tofile(fp)
        m.ptr.astype(np.int32).tofile(fp), m.col.astype(np.int32).tofile(fp), m.val.tofile(fp), X.tofile(fp), Y0.tofile(fp)
    res = subprocess.run([exe, inp, out], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, (res.returncode, res.stdout + res.stderr)
    raw = open(out, "rb").read()
    off = 0

    def take(n, dt):
        nonlocal off
        a = np.frombuffer(raw, dtype=dt, count=n, offset=off)
        off += a.nbytes
        return a
    y, ys, Y, yt = take(m.nrows, np.float64), take(m.nrows, np.float32), take(m.nrows * columns, np.float64), take(m.cols, np.float64)
    x, y0 = X[::columns].copy(), Y0[::columns].copy()
    y1 = oracle.gemv("d", m.rows_start, m.rows_end, m.col, m.val, 1.5, x, 0.5, y0.copy())
    y2 = oracle.gemv("d", m.rows_start, m.rows_end, m.col, m.val, 1.5, x, 0.5, y1.copy())
    s1 = row_scale(m.ptr, m.col, m.val, x, 1.5, 0.5, y0)
    assert_rows_close("d", y, y2, row_scale(m.ptr, m.col, m.val, x, 1.5, 0.5, y1) + 0.5 * s1, "gemv_d_csr twice")
    vs, xs, y0s = m.val.astype(np.float32), x.astype(np.float32), y0.astype(np.float32)
    ref_s = oracle.gemv_exact(m.rows_start, m.rows_end, m.col, vs, 1.5, xs, 0.5, y0s)
    assert_rows_close("s", ys, ref_s, row_scale(m.ptr, m.col, vs, xs, 1.5, 0.5, y0s), "gemv_s_csr")
    Yr = oracle.gemm("d", "row", m.rows_start, m.rows_end, m.col, m.val, 2.0, X, columns, columns, -1.0, Y0.copy(), columns)
    sc = mm_scale(m.ptr, m.col, m.val, X, columns, columns, 2.0, -1.0, Y0, columns)
    assert (np.abs(Y - Yr).reshape(m.nrows, columns) <= TOL["d"] * sc + 1e-300).all(), "gemm_d_csr_row"
    xt = Y0[: m.nrows].copy()
    ref_t = oracle.gemv_trans("d", m.cols, m.rows_start, m.rows_end, m.col, m.val, 1.0, xt, 0.0, np.zeros(m.cols))
    prod = np.abs(m.val * xt[np.repeat(np.arange(m.nrows), np.diff(m.ptr))])
    assert_rows_close("d", yt, ref_t, np.bincount(m.col, weights=prod, minlength=m.cols), "gemv_d_csr_trans")
