"""ctypes binding of libalphasparse_b200.so: one prototype per declaration in include/alphasparse/*.h.

This is the whole Python <-> C boundary: plain pointers, 32-bit indices, enums as C ints and the
matrix descriptor passed by value, exactly as a C caller of the reference's <alphasparse.h> sees
them.  No torch types cross it; a torch tensor is passed as ``tensor.data_ptr()``.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libalphasparse_b200.so")

# alphasparse_status_t (include/alphasparse/spdef.h)
SUCCESS, NOT_INITIALIZED, ALLOC_FAILED, INVALID_VALUE, EXECUTION_FAILED = 0, 1, 2, 3, 4
INTERNAL_ERROR, NOT_SUPPORTED, INVALID_POINTER, INVALID_HANDLE = 5, 6, 7, 8
STATUS_NAMES = ["SUCCESS", "NOT_INITIALIZED", "ALLOC_FAILED", "INVALID_VALUE", "EXECUTION_FAILED",
                "INTERNAL_ERROR", "NOT_SUPPORTED", "INVALID_POINTER", "INVALID_HANDLE"]
# alphasparse_operation_t
NON_TRANSPOSE, TRANSPOSE, CONJUGATE_TRANSPOSE = 0, 1, 2
# alphasparse_matrix_type_t
GENERAL, SYMMETRIC, HERMITIAN, TRIANGULAR, DIAGONAL = 0, 1, 2, 3, 4
# alphasparse_index_base_t
BASE_ZERO, BASE_ONE = 0, 1
# alphasparse_layout_t
ROW_MAJOR, COLUMN_MAJOR = 0, 1
# alphasparse_format_t / alphasparse_datatype_t
FORMAT_COO, FORMAT_CSR, FORMAT_CSC = 0, 1, 2
FLOAT, DOUBLE, FLOAT_COMPLEX, DOUBLE_COMPLEX = 0, 1, 2, 3
# alphasparse_cuda_alg_t
ALG_AUTO, ALG_VECTOR, ALG_MERGE, ALG_ROWTILE = 0, 1, 2, 3


class MatrixDescr(C.Structure):
    """struct alpha_matrix_descr, passed by value."""
    _fields_ = [("type", C.c_int), ("mode", C.c_int), ("diag", C.c_int)]


class Matrix(C.Structure):
    """alphasparse_matrix: what an alphasparse_matrix_t points at."""
    _fields_ = [("mat", C.c_void_p), ("format", C.c_int), ("datatype", C.c_int),
                ("inspector", C.c_void_p), ("dcu_info", C.c_void_p)]


class MatInfo(C.Structure):
    """alphasparse_cuda_mat_info_t"""
    _fields_ = [("rows", C.c_int64), ("cols", C.c_int64), ("nnz", C.c_int64),
                ("max_row_nnz", C.c_int64), ("empty_rows", C.c_int64), ("mean_row_nnz", C.c_double),
                ("algorithm", C.c_int32), ("lanes_per_row", C.c_int32), ("merge_tiles", C.c_int64),
                ("device_bytes", C.c_int64), ("device", C.c_int32), ("scheduled", C.c_int32),
                ("band_rows", C.c_int32), ("band_count", C.c_int32), ("band_width", C.c_int32),
                ("band_elements", C.c_int64), ("spmm_col_blocks", C.c_int32), ("binned", C.c_int32)]


class AlphaTimer(C.Structure):
    """alpha_timer_t"""
    _fields_ = [("start", C.c_double), ("end", C.c_double)]


class Complex8(C.Structure):
    _fields_ = [("real", C.c_float), ("imag", C.c_float)]


class Complex16(C.Structure):
    _fields_ = [("real", C.c_double), ("imag", C.c_double)]


_H = C.c_void_p           # alphasparse_matrix_t
_HP = C.POINTER(C.c_void_p)
_I = C.c_int32
_P = C.c_void_p

_REAL = {"s": C.c_float, "d": C.c_double}
_CPLX = {"c": Complex8, "z": Complex16}


def prototypes():
    """name -> (restype, argtypes) for every exported function the headers declare."""
    p = {}
    for k, T in list(_REAL.items()) + list(_CPLX.items()):
        p[f"alphasparse_{k}_create_coo"] = (C.c_int, [_HP, C.c_int, _I, _I, _I, _P, _P, _P])
        p[f"alphasparse_{k}_create_csr"] = (C.c_int, [_HP, C.c_int, _I, _I, _P, _P, _P, _P])
        p[f"alphasparse_{k}_create_csc"] = (C.c_int, [_HP, C.c_int, _I, _I, _P, _P, _P, _P])
        p[f"alphasparse_{k}_mv"] = (C.c_int, [C.c_int, T, _H, MatrixDescr, _P, T, _P])
        p[f"alphasparse_{k}_mm"] = (C.c_int, [C.c_int, T, _H, MatrixDescr, C.c_int, _P, _I, _I, T, _P, _I])
    for k in _REAL:
        p[f"alphasparse_{k}_export_csr"] = (C.c_int, [_H, C.POINTER(C.c_int), C.POINTER(_I), C.POINTER(_I),
                                                       _HP, _HP, _HP, _HP])
        p[f"alphasparse_{k}_export_csc"] = (C.c_int, [_H, C.POINTER(C.c_int), C.POINTER(_I), C.POINTER(_I),
                                                       _HP, _HP, _HP, _HP])
    p["alphasparse_destroy"] = (C.c_int, [_H])
    p["alphasparse_convert_csr"] = (C.c_int, [_H, C.c_int, _HP])
    p["alphasparse_convert_csc"] = (C.c_int, [_H, C.c_int, _HP])
    p["alphasparse_set_mv_hint"] = (C.c_int, [_H, C.c_int, MatrixDescr, _I])
    p["alphasparse_optimize"] = (C.c_int, [_H])
    # include/alphasparse/spapi_cuda.h
    p["alphasparse_cuda_set_stream"] = (C.c_int, [_P])
    p["alphasparse_cuda_get_stream"] = (C.c_int, [_HP])
    p["alphasparse_cuda_synchronize"] = (C.c_int, [])
    p["alphasparse_cuda_set_algorithm"] = (C.c_int, [C.c_int])
    p["alphasparse_cuda_set_option"] = (C.c_int, [C.c_char_p, C.c_int64])
    p["alphasparse_cuda_get_option"] = (C.c_int, [C.c_char_p, C.POINTER(C.c_int64)])
    p["alphasparse_cuda_get_mat_info"] = (C.c_int, [_H, C.POINTER(MatInfo)])
    p["alphasparse_cuda_get_device_csr"] = (C.c_int, [_H, _HP, _HP, _HP])
    p["alphasparse_cuda_d_csrmv_noalloc"] = (C.c_int, [_I, _I, _I, C.c_double, _P, _P, _P, _P, C.c_double, _P])
    p["alphasparse_cuda_exchange_create"] = (C.c_int, [_HP, C.c_int, C.c_int, C.c_int, _P])
    p["alphasparse_cuda_exchange_blob_bytes"] = (C.c_size_t, [])
    p["alphasparse_cuda_exchange_export"] = (C.c_int, [_H, _P])
    p["alphasparse_cuda_exchange_connect"] = (C.c_int, [_H, _P])
    p["alphasparse_cuda_exchange_set_mode"] = (C.c_int, [_H, C.c_int])
    p["alphasparse_cuda_exchange_x"] = (C.c_int, [_H, _HP])
    p["alphasparse_cuda_exchange_load_x"] = (C.c_int, [_H, _P])
    p["alphasparse_cuda_exchange_status"] = (C.c_int, [_H, C.POINTER(C.c_int)])
    p["alphasparse_cuda_exchange_debug_wait"] = (C.c_int, [_H, C.c_int64])
    p["alphasparse_cuda_exchange_clear_status"] = (C.c_int, [_H])
    p["alphasparse_cuda_exchange_destroy"] = (C.c_int, [_H])
    p["alphasparse_s_mv_exchange"] = (C.c_int, [C.c_float, _H, MatrixDescr, _H, C.c_float, _P])
    p["alphasparse_d_mv_exchange"] = (C.c_int, [C.c_double, _H, MatrixDescr, _H, C.c_double, _P])
    p["alphasparse_cuda_kernel_status"] = (C.c_int, [_H, C.POINTER(C.c_int), C.c_int])
    p["alphasparse_cuda_profile_kernel"] = (C.c_int, [_H, C.c_int])
    p["alphasparse_cuda_kernel_ms"] = (C.c_int, [_H, C.POINTER(C.c_float)])
    p["alphasparse_cuda_debug_fail_alloc"] = (C.c_int, [C.c_int64])
    p["alphasparse_cuda_launch_count"] = (C.c_int64, [])
    p["alphasparse_cuda_last_error"] = (C.c_char_p, [])
    # include/alphasparse/kernel_cuda.h
    for k, T in _REAL.items():
        for name in (f"gemv_{k}_csr", f"gemv_{k}_csr_trans"):
            p[name] = (C.c_int, [T, _P, _P, T, _P])
        for name in (f"gemm_{k}_csr_row", f"gemm_{k}_csr_col", f"gemm_{k}_csr_row_trans", f"gemm_{k}_csr_col_trans"):
            p[name] = (C.c_int, [T, _P, _P, _I, _I, T, _P, _I])
    p["alphasparse_cuda_release_csr"] = (C.c_int, [_P])
    # include/alphasparse/util.h
    p["alpha_malloc"] = (C.c_void_p, [C.c_size_t])
    p["alpha_memalign"] = (C.c_void_p, [C.c_size_t, C.c_size_t])
    p["alpha_free"] = (None, [C.c_void_p])
    p["alpha_get_core_num"] = (C.c_int, [])
    p["alpha_set_thread_num"] = (None, [C.c_int])
    p["alpha_get_thread_num"] = (C.c_int, [])
    p["alpha_timing_wtime"] = (C.c_double, [])
    _T = C.POINTER(AlphaTimer)
    p["alpha_timing_start"] = (None, [_T])
    p["alpha_timing_end"] = (None, [_T])
    p["alpha_timing_elapsed_time"] = (C.c_double, [_T])
    p["alpha_timing_gflops"] = (C.c_double, [_T, C.c_int64])
    p["alpha_timing_elaped_time_print"] = (None, [_T, C.c_char_p])
    p["alpha_timing_gflops_print"] = (None, [_T, C.c_int64, C.c_char_p])
    p["alpha_fill_s"] = (None, [_P, C.c_float, C.c_size_t])
    p["alpha_fill_d"] = (None, [_P, C.c_double, C.c_size_t])
    p["alpha_fill_random_s"] = (None, [_P, C.c_uint, C.c_size_t])
    p["alpha_fill_random_d"] = (None, [_P, C.c_uint, C.c_size_t])
    p["alpha_clear_cache"] = (None, [])
    _ARGV = [C.c_int, C.POINTER(C.c_char_p)]
    for name, res in (("alphasparse_layout_parse", C.c_int), ("alphasparse_operation_parse", C.c_int),
                      ("alphasparse_matrix_type_parse", C.c_int), ("alphasparse_fill_mode_parse", C.c_int),
                      ("alphasparse_diag_type_parse", C.c_int)):
        p[name] = (res, [C.c_char_p])
    p["args_help"] = (None, _ARGV)
    p["args_get_if_check"] = (C.c_bool, _ARGV)
    p["args_get_thread_num"] = (C.c_int, _ARGV)
    p["args_get_columns"] = (C.c_int, _ARGV + [C.c_int])
    p["args_get_iter"] = (C.c_int, _ARGV)
    for name in ("args_get_data_file", "args_get_data_fileA", "args_get_data_fileB"):
        p[name] = (C.c_char_p, _ARGV)
    p["alpha_args_get_layout_helper"] = (C.c_int, _ARGV + [C.c_int])
    p["alpha_args_get_matrix_descr_helper"] = (MatrixDescr, _ARGV + [C.c_int, C.c_int, C.c_int])
    p["alpha_args_get_trans_helper"] = (C.c_int, _ARGV + [C.c_int])
    for name in ("alpha_args_get_layout", "alpha_args_get_layoutB", "alpha_args_get_layoutC", "alpha_args_get_transA",
                 "alpha_args_get_transB"):
        p[name] = (C.c_int, _ARGV)
    p["alpha_args_get_matrix_descrA"] = (MatrixDescr, _ARGV)
    p["alpha_args_get_matrix_descrB"] = (MatrixDescr, _ARGV)
    p["alphasparse_nnz_counter_coo"] = (None, [_P, _P, _I, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I)])
    p["alphasparse_operations_mm"] = (C.c_int64, [_I, _I, _I, _I, _I, C.c_int, MatrixDescr, _I, C.c_int])
    p["alphasparse_operations_mv"] = (C.c_int64, [_I, _I, _I, _I, _I, C.c_int, MatrixDescr, C.c_int])
    p["alpha_read_coo"] = (None, [C.c_char_p, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), _HP, _HP, _HP])
    p["alpha_read_coo_d"] = (None, [C.c_char_p, C.POINTER(_I), C.POINTER(_I), C.POINTER(_I), _HP, _HP, _HP])
    p["lower_bound_int"] = (C.c_int, [_P, _I, _I, _I])
    p["balanced_partition_row_by_nnz"] = (None, [_P, _I, _I, _P])
    return p


_lib = None


def load():
    """Loads the library (once).  Fails loudly when it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python -m alsparse_b200.build` "
                              "(the CUDA library is the only compute path)")
        lib = C.CDLL(LIB_PATH, mode=C.RTLD_LOCAL)
        for name, (res, args) in prototypes().items():
            fn = getattr(lib, name)  # AttributeError if a declared symbol is not exported
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
