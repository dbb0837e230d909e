"""Seeded synthetic CSR matrices and vectors (ctypes wrapper of synth.c).

Every generator can produce any row range ``[row0, row0 + nrows)`` of its matrix on its own,
with offsets local to the range and column indices global: that is the share of one GPU of a
row-partitioned matrix.  The shapes follow the benchmark configurations:

* ``uniform_fixed``  -- exactly k distinct uniform columns per row, values U[-1, 1)
* ``poisson``        -- Poisson(lam) row lengths, distinct uniform columns
* ``zipf``           -- Zipf(s) row lengths clipped to [lo, hi], distinct uniform columns
* ``stencil27``      -- 27-point stencil on an n^3 grid, diagonal 26, off-diagonals -1
"""
import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsynth.so")
_lib = None
_NP = {"s": np.float32, "d": np.float64}


def _load():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            from .. import build
            build.build_synth()
        lib = C.CDLL(_LIB_PATH)
        u64, i64, i32, dbl, p = C.c_uint64, C.c_int64, C.c_int32, C.c_double, C.c_void_p
        lib.synth_rowlen_poisson.argtypes = [u64, i64, i64, dbl, i32, p]
        lib.synth_rowlen_zipf.argtypes = [u64, i64, i64, dbl, i32, i32, p]
        lib.synth_offsets.argtypes = [i64, p, p]
        lib.synth_offsets.restype = i64
        lib.synth_stencil27_rowlen.argtypes = [i32, i64, i64, p]
        for k in "sd":
            getattr(lib, f"synth_fill_uniform_{k}").argtypes = [u64, i64, i64, i32, p, p, p]
            getattr(lib, f"synth_stencil27_fill_{k}").argtypes = [i32, i64, i64, p, p, p, dbl, dbl]
            getattr(lib, f"synth_vector_{k}").argtypes = [u64, u64, i64, i64, dbl, dbl, p]
        _lib = lib
    return _lib


class Csr:
    """3-array CSR piece: rows [row0, row0+nrows) of a (rows x cols) matrix."""

    def __init__(self, rows, cols, row0, ptr, col, val):
        self.rows, self.cols, self.row0 = rows, cols, row0
        self.ptr, self.col, self.val = ptr, col, val

    @property
    def nrows(self):
        return len(self.ptr) - 1

    @property
    def nnz(self):
        return int(self.ptr[-1])

    @property
    def rows_start(self):
        return self.ptr[:-1]

    @property
    def rows_end(self):
        return self.ptr[1:]


def _offsets(lens):
    lib = _load()
    ptr = np.empty(len(lens) + 1, dtype=np.int32)
    total = lib.synth_offsets(len(lens), lens.ctypes.data, ptr.ctypes.data)
    if total >= 2**31 - 64:
        raise ValueError(f"{total} stored elements do not fit 32-bit offsets")
    return ptr


def _fill_uniform(kind, seed, row0, lens, rows, cols):
    lib = _load()
    ptr = _offsets(lens)
    col = np.empty(int(ptr[-1]), dtype=np.int32)
    val = np.empty(int(ptr[-1]), dtype=_NP[kind])
    getattr(lib, f"synth_fill_uniform_{kind}")(seed, row0, len(lens), cols, ptr.ctypes.data, col.ctypes.data,
                                                val.ctypes.data)
    return Csr(rows, cols, row0, ptr, col, val)


def _range(rows, row0, nrows):
    return (0, rows) if row0 is None else (row0, nrows)


def rowlen_fixed(rows, k, row0=None, nrows=None):
    row0, nrows = _range(rows, row0, nrows)
    return np.full(nrows, k, dtype=np.int32)


def rowlen_poisson(seed, rows, lam, cap, row0=None, nrows=None):
    row0, nrows = _range(rows, row0, nrows)
    lens = np.empty(nrows, dtype=np.int32)
    _load().synth_rowlen_poisson(seed, row0, nrows, lam, cap, lens.ctypes.data)
    return lens


def rowlen_zipf(seed, rows, s, lo, hi, row0=None, nrows=None):
    row0, nrows = _range(rows, row0, nrows)
    lens = np.empty(nrows, dtype=np.int32)
    _load().synth_rowlen_zipf(seed, row0, nrows, s, lo, hi, lens.ctypes.data)
    return lens


def uniform_fixed(kind, seed, rows, cols, k, row0=None, nrows=None):
    row0, nrows = _range(rows, row0, nrows)
    return _fill_uniform(kind, seed, row0, rowlen_fixed(rows, k, row0, nrows), rows, cols)


def poisson(kind, seed, rows, cols, lam, row0=None, nrows=None, total=None):
    """Poisson(lam) row lengths.  ``total`` (whole-matrix generation only) trims or tops up the
    lengths round-robin so that exactly that many elements are stored."""
    row0, nrows = _range(rows, row0, nrows)
    lens = rowlen_poisson(seed, rows, lam, cols, row0, nrows)
    if total is not None:
        assert row0 == 0 and nrows == rows
        lens = lens.astype(np.int64)
        diff, r = int(lens.sum()) - total, 0
        while diff != 0:
            if diff > 0 and lens[r] > 0:
                lens[r] -= 1
                diff -= 1
            elif diff < 0 and lens[r] < cols:
                lens[r] += 1
                diff += 1
            r = (r + 1) % rows
        lens = lens.astype(np.int32)
    return _fill_uniform(kind, seed, row0, lens, rows, cols)


def zipf(kind, seed, rows, cols, s=1.8, lo=1, hi=200000, row0=None, nrows=None):
    row0, nrows = _range(rows, row0, nrows)
    return _fill_uniform(kind, seed, row0, rowlen_zipf(seed, rows, s, lo, min(hi, cols), row0, nrows), rows, cols)


def from_lengths(kind, seed, lens, cols, row0=0, rows=None):
    """Distinct uniform columns / U[-1,1) values for caller-chosen row lengths."""
    lens = np.ascontiguousarray(lens, dtype=np.int32)
    return _fill_uniform(kind, seed, row0, lens, len(lens) if rows is None else rows, cols)


def stencil27(kind, n, row0=None, nrows=None, diag=26.0, off=-1.0):
    rows = n ** 3
    row0, nrows = _range(rows, row0, nrows)
    lib = _load()
    lens = np.empty(nrows, dtype=np.int32)
    lib.synth_stencil27_rowlen(n, row0, nrows, lens.ctypes.data)
    ptr = _offsets(lens)
    col = np.empty(int(ptr[-1]), dtype=np.int32)
    val = np.empty(int(ptr[-1]), dtype=_NP[kind])
    getattr(lib, f"synth_stencil27_fill_{kind}")(n, row0, nrows, ptr.ctypes.data, col.ctypes.data, val.ctypes.data,
                                                  diag, off)
    return Csr(rows, rows, row0, ptr, col, val)


def vector(kind, seed, stream, n, lo=-1.0, hi=1.0, first=0, out=None):
    """n elements of dense stream ``stream`` starting at element ``first``, uniform in [lo, hi)."""
    if out is None:
        out = np.empty(n, dtype=_NP[kind])
    getattr(_load(), f"synth_vector_{kind}")(seed, stream, first, n, lo, hi, out.ctypes.data)
    return out
