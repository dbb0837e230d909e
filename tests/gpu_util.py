"""Helpers for the GPU parity tests: every call goes through the C ABI (alsparse_b200.spblas)."""
import ctypes as C

import numpy as np
import torch

import oracle
from alsparse_b200 import capi, spblas
from helpers import NP, assert_rows_close, mm_scale, row_scale

TORCH = {"s": torch.float32, "d": torch.float64}


def make_handle(kind, m, base=0):
    st, A = spblas.create_csr(kind, base, m.nrows, m.cols, m.rows_start + base, m.rows_end + base, m.col + base, m.val)
    assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
    return A


class _DeviceArray:
    """Wraps a raw device address so torch can view it (CUDA array interface, version 2)."""

    def __init__(self, addr, n, typestr):
        self.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (addr, False), "version": 2}


def download(addr, n, dtype):
    """n elements of `dtype` read back from device address `addr`."""
    if n == 0:
        return torch.empty(0, dtype=dtype).numpy()
    typestr = {torch.int32: "<i4", torch.float32: "<f4", torch.float64: "<f8"}[dtype]
    return torch.as_tensor(_DeviceArray(addr, n, typestr), device="cuda").cpu().numpy()


def check_mv(kind, m, alpha, beta, seed=1, pointers="host", alg=None, A=None):
    """One mv through the C ABI against the oracle's plain kernel on the same inputs."""
    from alsparse_b200 import synth
    x = synth.vector(kind, seed, 1, m.cols)
    y0 = synth.vector(kind, seed, 2, m.nrows)
    own = A is None
    if alg is not None:
        spblas.set_algorithm(alg)
    try:
        if own:
            A = make_handle(kind, m)
    finally:
        if alg is not None:
            spblas.set_algorithm(capi.ALG_AUTO)
    if kind == "s" and m.nnz and int(np.diff(m.ptr).max()) > 1000:
        # the reference's serial float sum over thousands of elements leaves the tolerance by itself: compare with
        # the same products summed in double precision instead
        y_ref = oracle.gemv_exact(m.rows_start, m.rows_end, m.col, m.val, alpha, x, beta, y0)
    else:
        y_ref = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, alpha, x, beta, y0.copy())
    if pointers == "host":
        y = y0.copy()
        st = spblas.mv(kind, capi.NON_TRANSPOSE, alpha, A, spblas.descr(), x, beta, y)
    elif pointers == "device_x_host_y":
        dx, y = torch.from_numpy(x).cuda(), y0.copy()
        st = spblas.mv(kind, capi.NON_TRANSPOSE, alpha, A, spblas.descr(), dx, beta, y)
    else:
        dx, dy = torch.from_numpy(x).cuda(), torch.from_numpy(y0).cuda()
        st = spblas.mv(kind, capi.NON_TRANSPOSE, alpha, A, spblas.descr(), dx, beta, dy)
        torch.cuda.synchronize()
        y = dy.cpu().numpy()
    assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
    assert_rows_close(kind, y, y_ref, row_scale(m.ptr, m.col, m.val, x, alpha, beta, y0),
                      f"mv {kind} rows={m.nrows} nnz={m.nnz} alg={alg} ptr={pointers}")
    if own:
        spblas.destroy(A)
    return y
