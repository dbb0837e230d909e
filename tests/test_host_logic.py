"""Host-side pieces of the library that need no GPU: the row partition, COO handles, generators."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import oracle
from alsparse_b200 import capi, spblas, synth
from helpers import golden


def test_partition_matches_reference_rule():
    g = golden("partition.npz")
    for name in ("tiny", "cfg1", "zipf", "one_row", "flat"):
        for p in (1, 2, 3, 4, 8):
            assert np.array_equal(spblas.partition_rows_by_nnz(g[f"{name}_acc"], p), g[f"{name}_p{p}"]), (name, p)
    rng = np.random.default_rng(1)
    for _ in range(50):
        rows = int(rng.integers(1, 400))
        acc = np.cumsum(rng.integers(0, 40, rows)).astype(np.int32)
        for p in (2, 4, 8, 16):
            assert np.array_equal(spblas.partition_rows_by_nnz(acc, p), oracle.partition_rows_by_nnz(acc, p))


def test_lower_bound():
    lib = capi.load()
    t = np.array([1, 3, 3, 7, 9], np.int32)
    for v in range(0, 11):
        assert lib.lower_bound_int(t.ctypes.data, 0, 5, v) == int(np.searchsorted(t, v, "left"))


def test_coo_handle_lives_on_the_host():
    ri, ci = np.array([1, 3, 2], np.int32), np.array([2, 1, 3], np.int32)
    v = np.array([1.5, 2.5, 3.5])
    st, A = spblas.create_coo("d", capi.BASE_ONE, 3, 3, 3, ri, ci, v)
    assert st == capi.SUCCESS and A.value
    h = C.cast(A, C.POINTER(capi.Matrix)).contents
    assert h.format == capi.FORMAT_COO and h.datatype == capi.DOUBLE and h.dcu_info is None
    # structured descriptors on a COO handle are refused without touching a device; the general product needs
    # one (it runs on a device CSR copy) and fails loudly, y untouched, where there is none
    y = v.copy()
    assert spblas.mv("d", 0, 1.0, A, spblas.descr(capi.TRIANGULAR), v, 0.0, y) == capi.NOT_SUPPORTED
    if not torch.cuda.is_available():
        assert spblas.mv("d", 0, 1.0, A, spblas.descr(), v, 0.0, y) not in (capi.SUCCESS, capi.NOT_SUPPORTED)
        assert spblas.last_error() != "" and h.inspector is None
    assert np.array_equal(y, v)
    st, _ = spblas.convert_csr(A, capi.CONJUGATE_TRANSPOSE)
    assert st == capi.NOT_SUPPORTED
    assert spblas.destroy(A) == capi.SUCCESS


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-device behaviour")
def test_no_device_means_failure_not_fallback():
    m = synth.uniform_fixed("s", 0, 64, 64, 4)
    st, A = spblas.create_csr("s", 0, 64, 64, m.rows_start, m.rows_end, m.col, m.val)
    assert st != capi.SUCCESS and not A.value
    assert spblas.last_error() != ""


def test_generators_are_deterministic_and_sliceable():
    for make in (lambda **k: synth.uniform_fixed("s", 7, 5000, 4000, 16, **k),
                 lambda **k: synth.poisson("d", 7, 5000, 4000, 9.0, **k),
                 lambda **k: synth.zipf("d", 7, 5000, 4000, 1.8, 1, 3000, **k),
                 lambda **k: synth.stencil27("d", 12, **k)):
        whole, again = make(), make()
        assert np.array_equal(whole.ptr, again.ptr) and np.array_equal(whole.col, again.col)
        assert np.array_equal(whole.val, again.val)
        rows = whole.nrows
        a, b = rows // 3, rows - rows // 3
        part = make(row0=a, nrows=b - a)
        lo, hi = whole.ptr[a], whole.ptr[b]
        assert np.array_equal(part.ptr, whole.ptr[a:b + 1] - lo)
        assert np.array_equal(part.col, whole.col[lo:hi]) and np.array_equal(part.val, whole.val[lo:hi])
        # columns ascending and distinct within every row, inside the matrix
        d = np.diff(whole.col)
        starts = whole.ptr[1:-1]
        inner = np.ones(len(d), bool)
        inner[starts[(starts > 0) & (starts < whole.nnz)] - 1] = False
        assert (d[inner] > 0).all() and whole.col.min() >= 0 and whole.col.max() < whole.cols


def test_generator_shapes():
    m = synth.poisson("s", 0, 1000, 1000, 5.0, total=5000)
    assert m.nnz == 5000 and m.nrows == 1000
    s = synth.stencil27("d", 10)
    assert s.nnz == (3 * 10 - 2) ** 3 and np.diff(s.ptr).max() == 27
    assert set(np.unique(s.val)) == {-1.0, 26.0}
    lens = synth.rowlen_zipf(0, 200000, 1.8, 1, 200000)
    assert 0.50 < (lens == 1).mean() < 0.56 and lens.max() > 10000
    lens = synth.rowlen_poisson(0, 200000, 32.0, 1 << 20)
    assert abs(lens.mean() - 32.0) < 0.1 and abs(lens.var() - 32.0) < 0.5
    x = synth.vector("d", 0, 1, 100000, 0.0, 1.0)
    assert 0.0 <= x.min() and x.max() < 1.0 and abs(x.mean() - 0.5) < 0.01
    assert np.array_equal(synth.vector("d", 0, 1, 100, 0.0, 1.0, first=50), x[50:150])


def test_matrix_file_reader(tmp_path):
    """alpha_read_coo / alpha_read_coo_d against the reference's reader on the same files."""
    files = {
        "general.mtx": "%%MatrixMarket matrix coordinate real general\n% a comment\n3 5 4\n1 1 2.5\n3 5 -1e-3\n2 4 7\n1 2 0.5\n",
        "symmetric.mtx": "%%MatrixMarket matrix coordinate real symmetric\n4 4 5\n1 1 2.5\n3 1 -1\n4 2 0.125\n2 2\n4 4 7e-1\n",
        "pattern.mtx": "% no banner at all\n%\n2 2 3\n1 2\n2 1\n2 2\n",
    }
    expect = {"general.mtx": (3, 5, [0, 2, 1, 0], [0, 4, 3, 1], [2.5, -1e-3, 7, 0.5]),
              "symmetric.mtx": (4, 4, [0, 2, 0, 3, 1, 1, 3], [0, 0, 2, 1, 3, 1, 3], [2.5, -1, -1, 0.125, 0.125, 1, 0.7]),
              "pattern.mtx": (2, 2, [0, 1, 1], [1, 0, 1], [1, 1, 1])}
    for name, text in files.items():
        path = str(tmp_path / name)
        open(path, "w").write(text)
        for kind in "sd":
            m, n, ri, ci, v = spblas.read_coo(kind, path)
            em, en, eri, eci, ev = expect[name]
            assert (m, n) == (em, en) and ri.tolist() == eri and ci.tolist() == eci
            assert np.array_equal(v, np.array(ev, dtype=v.dtype))
            if oracle.ref_available():
                rm, rn, rri, rci, rv = oracle.ref_read_coo(kind, path)
                assert (m, n) == (rm, rn) and np.array_equal(ri, rri) and np.array_equal(ci, rci)
                assert np.array_equal(v.view(np.uint8), rv.view(np.uint8))
    with pytest.raises(OSError):
        spblas.read_coo("s", str(tmp_path / "missing.mtx"))


def test_tuning_options_table_matches_the_header():
    """Every option the public header documents as `name (default)` exists with that default, set / restore work
    without a GPU, unknown names are refused, and ALPHASPARSE_CUDA_OPTIONS seeds the values of a fresh process."""
    import re
    import subprocess
    import sys
    from helpers import ROOT
    text = open(os.path.join(ROOT, "include", "alphasparse", "spapi_cuda.h")).read()
    block = text[text.index("ALPHASPARSE_CUDA_OPTIONS="):text.index("alphasparse_cuda_set_option(const char")]
    documented = {n: int(d) for n, d in re.findall(r"\*\s+([a-z][a-z0-9_]+) \((\d+)\)", block)}
    documented.update({n: int(d) for n, d in re.findall(r"\b(bin_[a-z0-9_]+) \((\d+)\)", block)})  # named inside a sentence
    assert len(documented) >= 15, documented
    for name, default in documented.items():
        assert spblas.get_option(name) == default, name
        assert spblas.set_option(name, default + 3) == capi.SUCCESS
        assert spblas.get_option(name) == default + 3
        assert spblas.set_option(name, -1) == capi.SUCCESS
        assert spblas.get_option(name) == default, name
    assert spblas.set_option("no_such_option", 1) == capi.INVALID_VALUE
    code = ("from alsparse_b200 import spblas; "
            "print(spblas.get_option('band_min_seg'), spblas.get_option('bin_short'), spblas.get_option('band_bytes'))")
    env = dict(os.environ, ALPHASPARSE_CUDA_OPTIONS="band_min_seg=7, bin_short=9,bogus=1")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd=ROOT, timeout=120)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == ["7", "9", str(documented["band_bytes"])]
