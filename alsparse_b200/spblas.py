"""Host-side mirror of the reference's operator interface for the CSR mv / mm path.

Same names, argument order and status codes as the C API (include/alphasparse/spapi.h); the
functions take numpy arrays (host pointers) or torch CUDA tensors (device pointers) where the
C API takes pointers and return the ``alphasparse_status_t`` as an int, so a test written
against the reference's C entry points reads the same here:

    st, A = create_coo('s', BASE_ZERO, rows, cols, nnz, ri, ci, v)
    st, B = convert_csr(A, NON_TRANSPOSE)
    st = mv('s', NON_TRANSPOSE, 2.0, B, descr(GENERAL), x, 2.0, y)      # y updated in place
"""
import ctypes as C

import numpy as np

from . import capi
from .capi import (BASE_ONE, BASE_ZERO, COLUMN_MAJOR, GENERAL, NON_TRANSPOSE, ROW_MAJOR, SUCCESS,  # noqa: F401
                   TRANSPOSE, MatInfo, MatrixDescr)

_NP = {"s": np.float32, "d": np.float64}


def descr(type_=capi.GENERAL, mode=0, diag=0):
    return MatrixDescr(type_, mode, diag)


def _ptr(a):
    """Raw address of a numpy array, a torch tensor, an int address or None."""
    if a is None:
        return None
    if isinstance(a, int):
        return a
    if isinstance(a, np.ndarray):
        return a.ctypes.data
    if hasattr(a, "data_ptr"):
        return a.data_ptr()
    raise TypeError(f"cannot take the address of {type(a)!r}")


def _i32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.int32)


def create_csr(kind, indexing, rows, cols, rows_start, rows_end, col_indx, values):
    """alphasparse_{s,d}_create_csr.  Returns (status, handle)."""
    lib = capi.load()
    rs, re_, ci = _i32(rows_start), _i32(rows_end), _i32(col_indx)
    v = None if values is None else np.ascontiguousarray(values, dtype=_NP.get(kind, np.float32))
    h = C.c_void_p()
    st = getattr(lib, f"alphasparse_{kind}_create_csr")(C.byref(h), indexing, rows, cols, _ptr(rs), _ptr(re_),
                                                         _ptr(ci), _ptr(v))
    return st, h


def create_coo(kind, indexing, rows, cols, nnz, row_indx, col_indx, values):
    """alphasparse_{s,d}_create_coo.  Returns (status, handle)."""
    lib = capi.load()
    ri, ci = _i32(row_indx), _i32(col_indx)
    v = None if values is None else np.ascontiguousarray(values, dtype=_NP.get(kind, np.float32))
    h = C.c_void_p()
    st = getattr(lib, f"alphasparse_{kind}_create_coo")(C.byref(h), indexing, rows, cols, nnz, _ptr(ri), _ptr(ci),
                                                         _ptr(v))
    return st, h


def convert_csr(source, operation=capi.NON_TRANSPOSE):
    """alphasparse_convert_csr.  Returns (status, handle)."""
    h = C.c_void_p()
    st = capi.load().alphasparse_convert_csr(source, operation, C.byref(h))
    return st, h


def export_csr(kind, source):
    """alphasparse_{s,d}_export_csr.  Returns (status, base, rows, cols, rows_start, rows_end, col_indx,
    values); the arrays are numpy views of the handle's own storage (borrowed, like the C pointers)."""
    lib = capi.load()
    base, rows, cols = C.c_int(), C.c_int32(), C.c_int32()
    rs, re_, ci, v = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    st = getattr(lib, f"alphasparse_{kind}_export_csr")(source, C.byref(base), C.byref(rows), C.byref(cols),
                                                         C.byref(rs), C.byref(re_), C.byref(ci), C.byref(v))
    if st != SUCCESS:
        return (st,) + (None,) * 7
    m = rows.value

    def view(p, n, ct):
        if n == 0 or not p.value:
            return np.zeros(0, dtype=np.dtype(ct))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=(n,))

    ptr = view(rs, m + 1, C.c_int32)
    nnz = int(ptr[m] - ptr[0]) if m > 0 else 0
    ct = C.c_float if kind == "s" else C.c_double
    return (st, base.value, m, cols.value, ptr[:m], ptr[1:m + 1] if m > 0 else ptr[:0], view(ci, nnz, C.c_int32),
            view(v, nnz, ct))


def create_csc(kind, indexing, rows, cols, cols_start, cols_end, row_indx, values):
    """alphasparse_{s,d}_create_csc.  Returns (status, handle)."""
    lib = capi.load()
    cs, ce, ri = _i32(cols_start), _i32(cols_end), _i32(row_indx)
    v = None if values is None else np.ascontiguousarray(values, dtype=_NP.get(kind, np.float32))
    h = C.c_void_p()
    st = getattr(lib, f"alphasparse_{kind}_create_csc")(C.byref(h), indexing, rows, cols, _ptr(cs), _ptr(ce),
                                                         _ptr(ri), _ptr(v))
    return st, h


def convert_csc(source, operation=capi.NON_TRANSPOSE):
    """alphasparse_convert_csc (COO source).  Returns (status, handle)."""
    h = C.c_void_p()
    st = capi.load().alphasparse_convert_csc(source, operation, C.byref(h))
    return st, h


def export_csc(kind, source):
    """alphasparse_{s,d}_export_csc.  Returns (status, base, rows, cols, cols_start, cols_end, row_indx, values)
    as borrowed numpy views, like export_csr."""
    lib = capi.load()
    base, rows, cols = C.c_int(), C.c_int32(), C.c_int32()
    cs, ce, ri, v = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
    st = getattr(lib, f"alphasparse_{kind}_export_csc")(source, C.byref(base), C.byref(rows), C.byref(cols),
                                                         C.byref(cs), C.byref(ce), C.byref(ri), C.byref(v))
    if st != SUCCESS:
        return (st,) + (None,) * 7
    n = cols.value

    def view(p, k, ct):
        if k == 0 or not p.value:
            return np.zeros(0, dtype=np.dtype(ct))
        return np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=(k,))

    ptr = view(cs, n + 1, C.c_int32)
    nnz = int(ptr[n] - ptr[0]) if n > 0 else 0
    ct = C.c_float if kind == "s" else C.c_double
    return (st, base.value, rows.value, n, ptr[:n], ptr[1:n + 1] if n > 0 else ptr[:0], view(ri, nnz, C.c_int32),
            view(v, nnz, ct))


def destroy(handle):
    return capi.load().alphasparse_destroy(handle)


def mv(kind, operation, alpha, A, descr_, x, beta, y):
    """alphasparse_{s,d}_mv: y = alpha*op(A)*x + beta*y, y updated in place.  Returns the status."""
    return getattr(capi.load(), f"alphasparse_{kind}_mv")(operation, alpha, A, descr_, _ptr(x), beta, _ptr(y))


def mm(kind, operation, alpha, A, descr_, layout, x, columns, ldx, beta, y, ldy):
    """alphasparse_{s,d}_mm: Y = alpha*op(A)*X + beta*Y, Y updated in place.  Returns the status."""
    return getattr(capi.load(), f"alphasparse_{kind}_mm")(operation, alpha, A, descr_, layout, _ptr(x), columns, ldx,
                                                           beta, _ptr(y), ldy)


def optimize(A):
    """alphasparse_optimize: re-runs the analysis of the handle."""
    return capi.load().alphasparse_optimize(A)


def mat_info(A):
    info = MatInfo()
    st = capi.load().alphasparse_cuda_get_mat_info(A, C.byref(info))
    return st, info


def device_csr(A):
    """(status, d_row_ptr, d_col_indx, d_values) as integer device addresses."""
    a, b, c = C.c_void_p(), C.c_void_p(), C.c_void_p()
    st = capi.load().alphasparse_cuda_get_device_csr(A, C.byref(a), C.byref(b), C.byref(c))
    return st, a.value, b.value, c.value


def set_stream(stream_ptr):
    return capi.load().alphasparse_cuda_set_stream(stream_ptr)


def set_algorithm(alg):
    return capi.load().alphasparse_cuda_set_algorithm(alg)


def set_option(name, value):
    """alphasparse_cuda_set_option: a tuning value of the analysis (negative restores the default)."""
    return capi.load().alphasparse_cuda_set_option(name.encode(), int(value))


def get_option(name):
    v = C.c_int64()
    st = capi.load().alphasparse_cuda_get_option(name.encode(), C.byref(v))
    assert st == SUCCESS, capi.STATUS_NAMES[st]
    return v.value


def launch_count():
    return capi.load().alphasparse_cuda_launch_count()


def last_error():
    return capi.load().alphasparse_cuda_last_error().decode()


def partition_rows_by_nnz(rows_end, parts):
    """balanced_partition_row_by_nnz: nnz-balanced contiguous row split, parts+1 boundaries."""
    acc = _i32(rows_end)
    out = np.zeros(parts + 1, dtype=np.int32)
    capi.load().balanced_partition_row_by_nnz(_ptr(acc), len(acc), parts, _ptr(out))
    return out


def kernel_status(A, clear=False):
    """alphasparse_cuda_kernel_status: (status, code) -- the error word of the handle's kernels (0 = fine)."""
    code = C.c_int()
    st = capi.load().alphasparse_cuda_kernel_status(A, C.byref(code), 1 if clear else 0)
    return st, code.value


def profile_kernel(A, enable=True):
    return capi.load().alphasparse_cuda_profile_kernel(A, 1 if enable else 0)


def kernel_ms(A):
    """Duration in ms of the dominant kernel of the last mv / mm call on A (profiling enabled)."""
    ms = C.c_float()
    st = capi.load().alphasparse_cuda_kernel_ms(A, C.byref(ms))
    assert st == SUCCESS, capi.STATUS_NAMES[st]
    return ms.value


def csrmv_noalloc(rows, cols, nnz, alpha, d_row_ptr, d_col_indx, d_values, d_x, beta, d_y):
    """alphasparse_cuda_d_csrmv_noalloc: double-precision SpMV on device arrays that never allocates
    (scratch lives in a fixed 4 MiB array inside the library; rows + nnz <= 375,802,112)."""
    return capi.load().alphasparse_cuda_d_csrmv_noalloc(rows, cols, nnz, alpha, _ptr(d_row_ptr), _ptr(d_col_indx),
                                                         _ptr(d_values), _ptr(d_x), beta, _ptr(d_y))


def read_coo(kind, path):
    """alpha_read_coo / alpha_read_coo_d: (rows, cols, row_indx, col_indx, values) as numpy copies (zero-based)."""
    lib = capi.load()
    m, n, nnz = C.c_int32(), C.c_int32(), C.c_int32()
    ri, ci, v = C.c_void_p(), C.c_void_p(), C.c_void_p()
    getattr(lib, "alpha_read_coo" if kind == "s" else "alpha_read_coo_d")(path.encode(), C.byref(m), C.byref(n),
                                                                          C.byref(nnz), C.byref(ri), C.byref(ci),
                                                                          C.byref(v))
    if nnz.value < 0:
        raise OSError(f"cannot read {path}")
    k = nnz.value

    def take(p, ct):
        a = np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=(max(k, 1),))[:k].copy()
        lib.alpha_free(p)
        return a
    return m.value, n.value, take(ri, C.c_int32), take(ci, C.c_int32), take(v, C.c_float if kind == "s" else C.c_double)
