"""CPU checkers for the CSR mv / mm path -- TEST INFRASTRUCTURE ONLY.

Two libraries, both built by ``make -C oracle``:

* ``liboracle.so``  -- the C restatement in ``oracle.c`` (always available);
* ``_ref/libalpha_ref.so`` -- the reference's own source files for this path compiled in place
  (plain serial kernels, x86_64 OpenMP kernels, create / convert / partition).  It is built
  where the reference tree is mounted and travels as a prebuilt file elsewhere.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU legs of ``bench.py`` may import this
module; the product library never does.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_LIB = os.path.join(HERE, "liboracle.so")
REF_LIB = os.path.join(HERE, "_ref", "libalpha_ref.so")
_NP = {"s": np.float32, "d": np.float64}
_CT = {"s": C.c_float, "d": C.c_double}
_i32, _p = C.c_int32, C.c_void_p


def _a(x):
    return x.ctypes.data


def _i(x):
    return np.ascontiguousarray(x, dtype=np.int32)


# ---------------------------------------------------------------------------------------------
# the C restatement
# ---------------------------------------------------------------------------------------------
_oracle = None


def lib():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_LIB):
            raise ImportError(f"{ORACLE_LIB} missing: run `make -C oracle`")
        L = C.CDLL(ORACLE_LIB)
        for k, T in _CT.items():
            getattr(L, f"oracle_gemv_csr_{k}").argtypes = [_i32, _p, _p, _p, _p, T, _p, T, _p]
            getattr(L, f"oracle_gemv_csr_trans_{k}").argtypes = [_i32, _i32, _p, _p, _p, _p, T, _p, T, _p]
            getattr(L, f"oracle_gemv_csr_omp_{k}").argtypes = [_i32, _p, _p, _p, _p, T, _p, T, _p, _i32]
            for lay in ("row", "col"):
                getattr(L, f"oracle_gemm_csr_{lay}_{k}").argtypes = [_i32, _p, _p, _p, _p, T, _p, _i32, _i32, T, _p,
                                                                      _i32]
            getattr(L, f"oracle_gemm_csr_row_omp_{k}").argtypes = [_i32, _p, _p, _p, _p, T, _p, _i32, _i32, T, _p,
                                                                    _i32, _i32]
            getattr(L, f"oracle_trmv_csr_{k}").argtypes = [C.c_int, C.c_int, C.c_int, _i32, _p, _p, _p, _p, T, _p, T, _p]
            getattr(L, f"oracle_symv_csr_{k}").argtypes = [C.c_int, C.c_int, _i32, _p, _p, _p, _p, T, _p, T, _p]
            getattr(L, f"oracle_diagmv_csr_{k}").argtypes = [C.c_int, _i32, _p, _p, _p, _p, T, _p, T, _p]
            mm_tail = [_i32, _p, _p, _p, _p, T, _p, _i32, _i32, T, _p, _i32]
            getattr(L, f"oracle_symm_csr_{k}").argtypes = [C.c_int] * 3 + mm_tail
            getattr(L, f"oracle_trmm_csr_{k}").argtypes = [C.c_int] * 4 + mm_tail
            getattr(L, f"oracle_diagmm_csr_{k}").argtypes = [C.c_int] * 2 + mm_tail
            getattr(L, f"oracle_gemv_coo_{k}").argtypes = [C.c_int, _i32, _i32, _i32, _p, _p, _p, T, _p, T, _p]
            getattr(L, f"oracle_gemm_coo_{k}").argtypes = [C.c_int, C.c_int, _i32, _i32, _i32, _p, _p, _p, T, _p, _i32,
                                                            _i32, T, _p, _i32]
            getattr(L, f"oracle_gemv_csc_{k}").argtypes = [C.c_int, _i32, _i32, _p, _p, _p, _p, T, _p, T, _p]
            getattr(L, f"oracle_gemm_csc_{k}").argtypes = [C.c_int, C.c_int, _i32, _i32, _p, _p, _p, _p, T, _p, _i32,
                                                            _i32, T, _p, _i32]
            getattr(L, f"oracle_create_csr_{k}").argtypes = [_i32, _i32, _p, _p, _p, _p, _p, _p, _p]
            getattr(L, f"oracle_create_csr_{k}").restype = _i32
            getattr(L, f"oracle_coo_to_csr_{k}").argtypes = [_i32, _i32, _i32, _p, _p, _p, _p, _p, _p]
        L.oracle_partition_rows_by_nnz.argtypes = [_p, _i32, _i32, _p]
        L.oracle_lower_bound.argtypes = [_p, _i32, _i32, _i32]
        L.oracle_lower_bound.restype = _i32
        L.oracle_mv_status.argtypes = [C.c_int] * 9 + [_i32, _i32]
        L.oracle_mm_status.argtypes = [C.c_int] * 9 + [_i32, _i32]
        L.oracle_max_threads.restype = C.c_int
        _oracle = L
    return _oracle


def gemv(kind, rows_start, rows_end, col, val, alpha, x, beta, y, threads=0):
    """y (modified in place and returned) = beta*y + alpha*A*x; threads>0 uses the OpenMP form."""
    rs, re_, ci = _i(rows_start), _i(rows_end), _i(col)
    args = [len(rs), _a(rs), _a(re_), _a(ci), _a(val), alpha, _a(x), beta, _a(y)]
    if threads:
        getattr(lib(), f"oracle_gemv_csr_omp_{kind}")(*args, threads)
    else:
        getattr(lib(), f"oracle_gemv_csr_{kind}")(*args)
    return y


def gemv_exact(rows_start, rows_end, col, val, alpha, x, beta, y0):
    """The product of the reference's gemv kernel (src/plain/kernel/level2/mv/gemv/gemv_x_csr_plain.c:4-24:
    y[r] = beta*y[r] + alpha * sum a_rj * x[col_rj]) with every product and sum carried in double precision,
    returned as float64.  The comparand for single-precision rows so long that the reference's own serial
    float sum leaves the parity tolerance (1e-5 of the row's sum of |a*x|): against this one the tolerance
    is spent on the tested kernel alone.  Requires rows_end[r] == rows_start[r+1] (3-array CSR)."""
    rs, re_ = np.asarray(rows_start, dtype=np.int64), np.asarray(rows_end, dtype=np.int64)
    prod = np.asarray(val, dtype=np.float64) * np.asarray(x, dtype=np.float64)[np.asarray(col)]
    # each row summed on its own (differences of one running sum would cancel badly on large matrices)
    out = np.add.reduceat(np.concatenate([prod, [0.0]]), np.minimum(rs - rs[0], len(prod))) if len(rs) else prod[:0]
    out = np.where(re_ > rs, out, 0.0)
    return beta * np.asarray(y0, dtype=np.float64) + alpha * out


CHECK_THRESHOLD = 50.0   # THRESH of the reference's checks (include/alphasparse/util/check.h:39)


def _check_eps(kind):
    # CalEpisilon_{s,d} (src/util/norm.c:6-32): ten times the machine epsilon of the type
    return 10.0 * float(np.finfo(np.float32 if kind == "s" else np.float64).eps)


def _norm1_of_columns(cols, col, val):
    # GeNorm1_{s,d} (src/util/norm.c:207-222): the largest column sum of |a|
    return float(np.bincount(np.asarray(col), weights=np.abs(np.asarray(val, dtype=np.float64)), minlength=cols).max()) \
        if len(col) else 0.0


def check_l2_residual(kind, answer, result, x, alpha, beta, rows, cols, col, val):
    """The figure the reference's own mv tests judge a result by (check_{s,d}_l2, src/util/check.c:7-57 and its
    double twin): max|answer - result| over (max(|A|_1, 1) * max(|x|_inf, 1) * max(|result|_inf, 1) * eps * max(rows,
    cols)), with |x|_inf multiplied by alpha and |result|_inf by beta when their magnitude exceeds one (by the signed
    scalar, as the reference does) and eps ten machine epsilons.  A result passes when the residual is <= 50."""
    a, r = np.asarray(answer, dtype=np.float64), np.asarray(result, dtype=np.float64)
    norm_d = float(np.abs(a - r).max()) if len(a) else 0.0
    norm_x = float(np.abs(np.asarray(x, dtype=np.float64)).max()) if len(x) else 0.0
    if abs(alpha) > 1.0:
        norm_x *= alpha
    norm_y = float(np.abs(r).max()) if len(r) else 0.0
    if abs(beta) > 1.0:
        norm_y *= beta
    norm_a = _norm1_of_columns(cols, col, val)
    return norm_d / (max(norm_a, 1.0) * max(norm_x, 1.0) * max(norm_y, 1.0) * _check_eps(kind) * max(rows, cols))


def check_l3_residual(kind, answer, result, X, rows, cols, columns, ld_answer, ld_result, ldx, col, val):
    """check_{s,d}_l3 for row-major mm (src/util/check.c:217-334, the branch with one matrix file): the largest column
    sum of |answer - result| over (max(|A|_1, 1) * max(|X|_1, 1) * max(|result|_1, 1) * eps * max(rows, cols, columns)),
    |.|_1 the largest column sum of magnitudes (DesNorm1, DesDiffNorm1 of src/util/norm.c:303-354)."""
    def dense(v, n, ld):
        return np.asarray(v, dtype=np.float64).reshape(-1)[: n * ld].reshape(n, ld)[:, :columns]
    A_, R_, X_ = dense(answer, rows, ld_answer), dense(result, rows, ld_result), dense(X, cols, ldx)
    norm_d = float(np.abs(A_ - R_).sum(axis=0).max())
    norm_x = float(np.abs(X_).sum(axis=0).max())
    norm_y = float(np.abs(R_).sum(axis=0).max())
    norm_a = _norm1_of_columns(cols, col, val)
    return norm_d / (max(norm_a, 1.0) * max(norm_x, 1.0) * max(norm_y, 1.0) * _check_eps(kind) * max(rows, cols, columns))


def gemv_trans(kind, cols, rows_start, rows_end, col, val, alpha, x, beta, y):
    rs, re_, ci = _i(rows_start), _i(rows_end), _i(col)
    getattr(lib(), f"oracle_gemv_csr_trans_{kind}")(len(rs), cols, _a(rs), _a(re_), _a(ci), _a(val), alpha, _a(x),
                                                     beta, _a(y))
    return y


def gemm(kind, layout, rows_start, rows_end, col, val, alpha, X, columns, ldx, beta, Y, ldy, threads=0):
    rs, re_, ci = _i(rows_start), _i(rows_end), _i(col)
    args = [len(rs), _a(rs), _a(re_), _a(ci), _a(val), alpha, _a(X), columns, ldx, beta, _a(Y), ldy]
    if threads:
        assert layout == "row"
        getattr(lib(), f"oracle_gemm_csr_row_omp_{kind}")(*args, threads)
    else:
        getattr(lib(), f"oracle_gemm_csr_{layout}_{kind}")(*args)
    return Y


def structured_mv(kind, descr_type, upper, unit, trans, rows_start, rows_end, col, val, alpha, x, beta, y):
    """mv under a TRIANGULAR (3), SYMMETRIC (1) or DIAGONAL (4) descriptor; y modified in place."""
    rs, re_, ci = _i(rows_start), _i(rows_end), _i(col)
    tail = [len(rs), _a(rs), _a(re_), _a(ci), _a(val), alpha, _a(x), beta, _a(y)]
    if descr_type == 3:
        getattr(lib(), f"oracle_trmv_csr_{kind}")(int(upper), int(unit), int(trans), *tail)
    elif descr_type == 1:
        getattr(lib(), f"oracle_symv_csr_{kind}")(int(upper), int(unit), *tail)
    elif descr_type == 4:
        getattr(lib(), f"oracle_diagmv_csr_{kind}")(int(unit), *tail)
    else:
        raise ValueError(descr_type)
    return y


def structured_mm(kind, descr_type, upper, unit, trans, layout, rows_start, rows_end, col, val, alpha, X, columns,
                  ldx, beta, Y, ldy):
    """mm under a TRIANGULAR (3), SYMMETRIC (1) or DIAGONAL (4) descriptor; Y modified in place."""
    rs, re_, ci = _i(rows_start), _i(rows_end), _i(col)
    cm = int(layout == "col")
    tail = [len(rs), _a(rs), _a(re_), _a(ci), _a(val), alpha, _a(X), columns, ldx, beta, _a(Y), ldy]
    if descr_type == 3:
        getattr(lib(), f"oracle_trmm_csr_{kind}")(int(upper), int(unit), int(trans), cm, *tail)
    elif descr_type == 1:
        getattr(lib(), f"oracle_symm_csr_{kind}")(int(upper), int(unit), cm, *tail)
    elif descr_type == 4:
        getattr(lib(), f"oracle_diagmm_csr_{kind}")(int(unit), cm, *tail)
    else:
        raise ValueError(descr_type)
    return Y


def gemv_coo(kind, trans, rows, cols, row_indx, col_indx, val, alpha, x, beta, y):
    """mv on a COO matrix (zero-based entries in stored order); y modified in place."""
    ri, ci = _i(row_indx), _i(col_indx)
    getattr(lib(), f"oracle_gemv_coo_{kind}")(int(trans), rows, cols, len(ri), _a(ri), _a(ci), _a(val), alpha, _a(x),
                                               beta, _a(y))
    return y


def gemm_coo(kind, trans, layout, rows, cols, row_indx, col_indx, val, alpha, X, columns, ldx, beta, Y, ldy):
    ri, ci = _i(row_indx), _i(col_indx)
    getattr(lib(), f"oracle_gemm_coo_{kind}")(int(trans), int(layout == "col"), rows, cols, len(ri), _a(ri), _a(ci),
                                               _a(val), alpha, _a(X), columns, ldx, beta, _a(Y), ldy)
    return Y


def gemv_csc(kind, trans, rows, cols, cols_start, cols_end, row_indx, val, alpha, x, beta, y):
    """mv on a CSC matrix (zero-based); y modified in place."""
    cs, ce, ri = _i(cols_start), _i(cols_end), _i(row_indx)
    getattr(lib(), f"oracle_gemv_csc_{kind}")(int(trans), rows, cols, _a(cs), _a(ce), _a(ri), _a(val), alpha, _a(x),
                                               beta, _a(y))
    return y


def gemm_csc(kind, trans, layout, rows, cols, cols_start, cols_end, row_indx, val, alpha, X, columns, ldx, beta, Y, ldy):
    cs, ce, ri = _i(cols_start), _i(cols_end), _i(row_indx)
    getattr(lib(), f"oracle_gemm_csc_{kind}")(int(trans), int(layout == "col"), rows, cols, _a(cs), _a(ce), _a(ri),
                                               _a(val), alpha, _a(X), columns, ldx, beta, _a(Y), ldy)
    return Y


def create_csr(kind, base, rows_start, rows_end, col, val):
    """(offsets[rows+1], col[nnz], val[nnz]) as the reference's create_csr would store them."""
    rs, re_, ci = _i(rows_start), _i(rows_end), _i(col)
    v = np.ascontiguousarray(val, dtype=_NP[kind])
    f = getattr(lib(), f"oracle_create_csr_{kind}")
    nnz = f(base, len(rs), _a(rs), _a(re_), _a(ci), _a(v), None, None, None)
    ptr, oc, ov = np.empty(len(rs) + 1, np.int32), np.empty(nnz, np.int32), np.empty(nnz, _NP[kind])
    f(base, len(rs), _a(rs), _a(re_), _a(ci), _a(v), _a(ptr), _a(oc), _a(ov))
    return ptr, oc, ov


def coo_to_csr(kind, base, rows, row_indx, col_indx, val):
    ri, ci = _i(row_indx), _i(col_indx)
    v = np.ascontiguousarray(val, dtype=_NP[kind])
    ptr, oc, ov = np.empty(rows + 1, np.int32), np.empty(len(ri), np.int32), np.empty(len(ri), _NP[kind])
    getattr(lib(), f"oracle_coo_to_csr_{kind}")(base, rows, len(ri), _a(ri), _a(ci), _a(v), _a(ptr), _a(oc), _a(ov))
    return ptr, oc, ov


def partition_rows_by_nnz(rows_end, parts):
    acc = _i(rows_end)
    out = np.zeros(parts + 1, np.int32)
    lib().oracle_partition_rows_by_nnz(_a(acc), len(acc), parts, _a(out))
    return out


def mv_status(has_handle=1, has_mat=1, has_x=1, has_y=1, handle_datatype=0, call_datatype=0, operation=0,
              descr_type=0, fmt=1, rows=1, cols=1):
    return lib().oracle_mv_status(has_handle, has_mat, has_x, has_y, handle_datatype, call_datatype, operation,
                                  descr_type, fmt, rows, cols)


def max_threads():
    return lib().oracle_max_threads()


# ---------------------------------------------------------------------------------------------
# the reference's own objects
# ---------------------------------------------------------------------------------------------
class _RefHandle(C.Structure):
    _fields_ = [("mat", C.c_void_p), ("format", C.c_int), ("datatype", C.c_int), ("inspector", C.c_void_p),
                ("dcu_info", C.c_void_p)]


_ref = None


def ref_available():
    return os.path.exists(REF_LIB)


def ref():
    """The reference's objects, loaded RTLD_LOCAL (it exports the same names as the product)."""
    global _ref
    if _ref is None:
        if not ref_available():
            raise ImportError(f"{REF_LIB} missing (built only where the reference tree is mounted)")
        L = C.CDLL(REF_LIB, mode=C.RTLD_LOCAL)
        for k, T in _CT.items():
            getattr(L, f"alphasparse_{k}_create_csr").argtypes = [_p, C.c_int, _i32, _i32, _p, _p, _p, _p]
            getattr(L, f"alphasparse_{k}_create_coo").argtypes = [_p, C.c_int, _i32, _i32, _i32, _p, _p, _p]
            getattr(L, f"convert_csr_{k}_coo").argtypes = [_p, _p]
            for name in (f"gemv_{k}_csr_plain", f"gemv_{k}_csr", f"gemv_{k}_csr_trans_plain"):
                getattr(L, name).argtypes = [T, _p, _p, T, _p]
            for name in (f"gemm_{k}_csr_row_plain", f"gemm_{k}_csr_col_plain", f"gemm_{k}_csr_row",
                         f"gemm_{k}_csr_col", f"gemm_{k}_csr_row_trans_plain", f"gemm_{k}_csr_col_trans_plain"):
                getattr(L, name).argtypes = [T, _p, _p, _i32, _i32, T, _p, _i32]
            for name in [f"symv_{k}_csr_{d}_{m}_plain" for d in "nu" for m in ("lo", "hi")] + \
                        [f"trmv_{k}_csr_{d}_{m}{t}_plain" for d in "nu" for m in ("lo", "hi") for t in ("", "_trans")] + \
                        [f"diagmv_{k}_csr_{d}_plain" for d in "nu"]:
                getattr(L, name).argtypes = [T, _p, _p, T, _p]
            for name in [f"symm_{k}_csr_{d}_{m}_{lay}_plain" for d in "nu" for m in ("lo", "hi") for lay in ("row", "col")] + \
                        [f"trmm_{k}_csr_{d}_{m}_{lay}{t}_plain" for d in "nu" for m in ("lo", "hi")
                         for lay in ("row", "col") for t in ("", "_trans")] + \
                        [f"diagmm_{k}_csr_{d}_{lay}_plain" for d in "nu" for lay in ("row", "col")]:
                getattr(L, name).argtypes = [T, _p, _p, _i32, _i32, T, _p, _i32]
            for name in (f"gemv_{k}_coo_plain", f"gemv_{k}_coo_trans_plain"):
                getattr(L, name).argtypes = [T, _p, _p, T, _p]
            for name in [f"gemm_{k}_coo_{lay}{t}_plain" for lay in ("row", "col") for t in ("", "_trans")]:
                getattr(L, name).argtypes = [T, _p, _p, _i32, _i32, T, _p, _i32]
            for name in (f"gemv_{k}_csc_plain", f"gemv_{k}_csc_trans_plain"):
                getattr(L, name).argtypes = [T, _p, _p, T, _p]
            for name in [f"gemm_{k}_csc_{lay}{t}_plain" for lay in ("row", "col") for t in ("", "_trans")]:
                getattr(L, name).argtypes = [T, _p, _p, _i32, _i32, T, _p, _i32]
            getattr(L, f"alphasparse_{k}_export_csr").argtypes = [_p] * 8
        L.balanced_partition_row_by_nnz.argtypes = [_p, _i32, _i32, _p]
        for name in ("alpha_read_coo", "alpha_read_coo_d"):
            getattr(L, name).argtypes = [C.c_char_p] + [_p] * 6
        L.alpha_set_thread_num.argtypes = [C.c_int]
        L.alpha_get_core_num.restype = C.c_int
        _ref = L
    return _ref


class RefCsr:
    """A CSR handle owned by the reference library.  The reference never frees (its alpha_free is
    a no-op for non-NULL pointers), so create few of these."""

    def __init__(self, kind, handle):
        self.kind, self.handle = kind, handle
        self.mat = C.cast(handle, C.POINTER(_RefHandle)).contents.mat

    @classmethod
    def from_csr(cls, kind, base, rows, cols, rows_start, rows_end, col, val):
        rs, re_, ci = _i(rows_start), _i(rows_end), _i(col)
        v = np.ascontiguousarray(val, dtype=_NP[kind])
        h = C.c_void_p()
        st = getattr(ref(), f"alphasparse_{kind}_create_csr")(C.byref(h), base, rows, cols, _a(rs), _a(re_), _a(ci),
                                                               _a(v))
        assert st == 0
        return cls(kind, h)

    @classmethod
    def from_coo(cls, kind, base, rows, cols, row_indx, col_indx, val):
        """create_coo then the COO->CSR conversion, as every reference test builds its matrix."""
        ri, ci = _i(row_indx), _i(col_indx)
        v = np.ascontiguousarray(val, dtype=_NP[kind])
        h = C.c_void_p()
        st = getattr(ref(), f"alphasparse_{kind}_create_coo")(C.byref(h), base, rows, cols, len(ri), _a(ri), _a(ci),
                                                               _a(v))
        assert st == 0
        coo = C.cast(h, C.POINTER(_RefHandle)).contents.mat
        out = C.c_void_p()
        st = getattr(ref(), f"convert_csr_{kind}_coo")(coo, C.byref(out))
        assert st == 0
        fake = _RefHandle(out.value, 1, 0 if kind == "s" else 1, None, None)
        obj = cls.__new__(cls)
        obj.kind, obj._keep, obj.mat = kind, fake, out.value
        obj.handle = C.cast(C.pointer(fake), C.c_void_p)
        return obj

    def export(self):
        base, rows, cols = C.c_int(), C.c_int32(), C.c_int32()
        rs, re_, ci, v = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        st = getattr(ref(), f"alphasparse_{self.kind}_export_csr")(self.handle, C.byref(base), C.byref(rows),
                                                                   C.byref(cols), C.byref(rs), C.byref(re_),
                                                                   C.byref(ci), C.byref(v))
        assert st == 0
        m = rows.value
        ptr = np.ctypeslib.as_array(C.cast(rs, C.POINTER(C.c_int32)), shape=(m + 1,)).copy()
        nnz = int(ptr[m] - ptr[0])
        col = np.ctypeslib.as_array(C.cast(ci, C.POINTER(C.c_int32)), shape=(max(nnz, 1),))[:nnz].copy()
        val = np.ctypeslib.as_array(C.cast(v, C.POINTER(_CT[self.kind])), shape=(max(nnz, 1),))[:nnz].copy()
        return ptr, col, val

    def gemv(self, alpha, x, beta, y, omp_threads=0, trans=False):
        """The reference's plain serial kernel (omp_threads == 0) or its x86_64 OpenMP kernel."""
        L = ref()
        if trans:
            fn = getattr(L, f"gemv_{self.kind}_csr_trans_plain")
        elif omp_threads:
            L.alpha_set_thread_num(omp_threads)
            fn = getattr(L, f"gemv_{self.kind}_csr")
        else:
            fn = getattr(L, f"gemv_{self.kind}_csr_plain")
        st = fn(alpha, self.mat, _a(x), beta, _a(y))
        assert st == 0
        return y

    def structured_mv(self, descr_type, upper, unit, trans, alpha, x, beta, y):
        """The reference's plain symv / trmv / diagmv kernel for the given descriptor."""
        d, m = "u" if unit else "n", "hi" if upper else "lo"
        name = {1: f"symv_{self.kind}_csr_{d}_{m}_plain", 3: f"trmv_{self.kind}_csr_{d}_{m}{'_trans' if trans else ''}_plain",
                4: f"diagmv_{self.kind}_csr_{d}_plain"}[descr_type]
        st = getattr(ref(), name)(alpha, self.mat, _a(x), beta, _a(y))
        assert st == 0
        return y

    def structured_mm(self, descr_type, upper, unit, trans, layout, alpha, X, columns, ldx, beta, Y, ldy):
        """The reference's plain symm / trmm / diagmm kernel for the given descriptor and layout."""
        d, m = "u" if unit else "n", "hi" if upper else "lo"
        name = {1: f"symm_{self.kind}_csr_{d}_{m}_{layout}_plain",
                3: f"trmm_{self.kind}_csr_{d}_{m}_{layout}{'_trans' if trans else ''}_plain",
                4: f"diagmm_{self.kind}_csr_{d}_{layout}_plain"}[descr_type]
        st = getattr(ref(), name)(alpha, self.mat, _a(X), columns, ldx, beta, _a(Y), ldy)
        assert st == 0
        return Y

    def gemm(self, layout, alpha, X, columns, ldx, beta, Y, ldy, omp_threads=0, trans=False):
        L = ref()
        if trans:
            fn = getattr(L, f"gemm_{self.kind}_csr_{layout}_trans_plain")
        elif omp_threads:
            L.alpha_set_thread_num(omp_threads)
            fn = getattr(L, f"gemm_{self.kind}_csr_{layout}")
        else:
            fn = getattr(L, f"gemm_{self.kind}_csr_{layout}_plain")
        st = fn(alpha, self.mat, _a(X), columns, ldx, beta, _a(Y), ldy)
        assert st == 0
        return Y


class RefCoo:
    """A COO handle owned by the reference library (never freed, like RefCsr)."""

    def __init__(self, kind, base, rows, cols, row_indx, col_indx, val):
        ri, ci = _i(row_indx), _i(col_indx)
        v = np.ascontiguousarray(val, dtype=_NP[kind])
        h = C.c_void_p()
        st = getattr(ref(), f"alphasparse_{kind}_create_coo")(C.byref(h), base, rows, cols, len(ri), _a(ri), _a(ci), _a(v))
        assert st == 0
        self.kind, self.mat = kind, C.cast(h, C.POINTER(_RefHandle)).contents.mat

    def gemv(self, trans, alpha, x, beta, y):
        st = getattr(ref(), f"gemv_{self.kind}_coo{'_trans' if trans else ''}_plain")(alpha, self.mat, _a(x), beta, _a(y))
        assert st == 0
        return y

    def gemm(self, trans, layout, alpha, X, columns, ldx, beta, Y, ldy):
        st = getattr(ref(), f"gemm_{self.kind}_coo_{layout}{'_trans' if trans else ''}_plain")(
            alpha, self.mat, _a(X), columns, ldx, beta, _a(Y), ldy)
        assert st == 0
        return Y


class _CscRecord(C.Structure):
    """spmat_csc_?_t of the reference (include/alphasparse/spmat.h:288-297, :311-320)."""
    _fields_ = [("values", C.c_void_p), ("cols_start", C.c_void_p), ("cols_end", C.c_void_p), ("row_indx", C.c_void_p),
                ("rows", C.c_int32), ("cols", C.c_int32), ("ordered", C.c_bool)]


class RefCsc:
    """A CSC record laid out for the reference's kernels.  Built here rather than by the reference's create_csc,
    which copies only `rows` of the `cols` column offsets (src/core/format/alphasparse_x_create_csc.c:35)."""

    def __init__(self, kind, rows, cols, cols_start, cols_end, row_indx, val):
        self.kind = kind
        self._keep = (_i(cols_start), _i(cols_end), _i(row_indx), np.ascontiguousarray(val, dtype=_NP[kind]))
        cs, ce, ri, v = self._keep
        self.rec = _CscRecord(_a(v), _a(cs), _a(ce), _a(ri), rows, cols, False)

    def gemv(self, trans, alpha, x, beta, y):
        st = getattr(ref(), f"gemv_{self.kind}_csc{'_trans' if trans else ''}_plain")(alpha, C.addressof(self.rec), _a(x),
                                                                                    beta, _a(y))
        assert st == 0
        return y

    def gemm(self, trans, layout, alpha, X, columns, ldx, beta, Y, ldy):
        st = getattr(ref(), f"gemm_{self.kind}_csc_{layout}{'_trans' if trans else ''}_plain")(
            alpha, C.addressof(self.rec), _a(X), columns, ldx, beta, _a(Y), ldy)
        assert st == 0
        return Y


def ref_partition_rows_by_nnz(rows_end, parts):
    acc = _i(rows_end)
    out = np.zeros(parts + 1, np.int32)
    ref().balanced_partition_row_by_nnz(_a(acc), len(acc), parts, _a(out))
    return out


def ref_cores():
    return ref().alpha_get_core_num()


def ref_read_coo(kind, path):
    """The reference's own reader (src/util/io.c): (rows, cols, row_indx, col_indx, values)."""
    m, n, nnz = C.c_int32(), C.c_int32(), C.c_int32()
    ri, ci, v = C.c_void_p(), C.c_void_p(), C.c_void_p()
    getattr(ref(), "alpha_read_coo" if kind == "s" else "alpha_read_coo_d")(path.encode(), C.byref(m), C.byref(n),
                                                                            C.byref(nnz), C.byref(ri), C.byref(ci),
                                                                            C.byref(v))
    k = nnz.value
    get = lambda p, ct: np.ctypeslib.as_array(C.cast(p, C.POINTER(ct)), shape=(max(k, 1),))[:k].copy()  # noqa: E731
    return m.value, n.value, get(ri, C.c_int32), get(ci, C.c_int32), get(v, _CT[kind])
