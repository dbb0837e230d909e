"""alphasparse_cuda_d_csrmv_noalloc against the oracle's plain kernel and against alphasparse_d_mv.

The no-allocation entry point exists for callers that cannot call cudaMalloc when they need a
product (a memory pool already owns the device, or the device-wide synchronisation of an
allocation is not acceptable).  It must give what the reference's kernel gives (the oracle, within
the parity tolerance) and what the handle-based call gives.  This file sorts
last on purpose: a run that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest
import torch

import oracle
from alsparse_b200 import capi, spblas, synth
from helpers import TOL, assert_rows_close, row_scale

pytestmark = pytest.mark.gpu


def _both(m, alpha, beta, seed, check_free_memory=False):
    """(y from the handle-based mv, y from the no-allocation call, y from the oracle, per-row tolerance scale)."""
    x = synth.vector("d", seed, 1, m.cols)
    y0 = synth.vector("d", seed, 2, m.nrows)
    st, A = spblas.create_csr("d", 0, m.nrows, m.cols, m.rows_start, m.rows_end, m.col, m.val)
    assert st == capi.SUCCESS, spblas.last_error()
    dx = torch.from_numpy(x).cuda()
    y_handle = torch.from_numpy(y0).cuda()
    assert spblas.mv("d", 0, alpha, A, spblas.descr(), dx, beta, y_handle) == capi.SUCCESS
    # the caller owns every array the new entry point touches
    d_ptr, d_col, d_val = (torch.from_numpy(a).cuda() for a in (m.ptr, m.col, m.val))
    y_noalloc = torch.from_numpy(y0).cuda()
    torch.cuda.synchronize()
    before, free_before = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    st = spblas.csrmv_noalloc(m.nrows, m.cols, m.nnz, alpha, d_ptr, d_col, d_val, dx, beta, y_noalloc)
    assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    if check_free_memory:  # once every kernel involved has been loaded, device free memory does not move
        assert torch.cuda.mem_get_info()[0] == free_before
    spblas.destroy(A)
    y_oracle = oracle.gemv("d", m.rows_start, m.rows_end, m.col, m.val, alpha, x, beta, y0.copy())
    return y_handle.cpu().numpy(), y_noalloc.cpu().numpy(), y_oracle, row_scale(m.ptr, m.col, m.val, x, alpha, beta, y0)


def test_two_calls_in_a_row_match_the_handle_based_mv():
    # Different shapes back to back: the second call finds the first call's tables and carries in
    # the shared scratch array and must not be affected by them.
    first = synth.zipf("d", 21, 60000, 80000, 1.8, 1, 50000)          # long rows: carries across tiles
    lens = np.full(40000, 3, np.int32)
    lens[::5] = 0
    second = synth.from_lengths("d", 22, lens, 1000)                   # short and empty rows, fewer tiles
    for m, alpha, beta, seed, settled in ((first, 1.5, 0.5, 21, False), (second, -2.0, 0.0, 22, False),
                                          (first, 1.0, 0.0, 23, True)):
        y_handle, y_noalloc, y_oracle, scale = _both(m, alpha, beta, seed, settled)
        assert_rows_close("d", y_noalloc, y_oracle, scale, "no-allocation call against the oracle")
        err = np.abs(y_noalloc - y_handle)
        assert (err <= 2 * TOL["d"] * scale).all(), f"max ratio {np.max(err / np.maximum(scale, 1e-300)):.3g}"


def test_limits_and_pointer_checks():
    x = torch.zeros(8, dtype=torch.float64, device="cuda")
    ip = torch.zeros(9, dtype=torch.int32, device="cuda")
    # beyond the fixed scratch: refused with a message, nothing launched
    st = spblas.csrmv_noalloc(2_000_000_000, 8, 0x7fffffff, 1.0, ip, ip, x, x, 0.0, x)
    assert st == capi.INVALID_VALUE and "exceeds the fixed scratch" in spblas.last_error()
    if torch.cuda.device_count() > 1:  # memory of another GPU is refused, not dereferenced
        other = torch.zeros(8, dtype=torch.float64, device="cuda:1")
        assert spblas.csrmv_noalloc(8, 8, 8, 1.0, ip, ip, x, other, 0.0, x) == capi.INVALID_POINTER
    # host memory is not accepted
    hx = np.zeros(8)
    assert spblas.csrmv_noalloc(8, 8, 8, 1.0, ip, ip, x, hx, 0.0, x) == capi.INVALID_POINTER
    assert spblas.csrmv_noalloc(8, 8, 8, 1.0, ip, ip, x, x, 0.0, None) == capi.NOT_INITIALIZED
    assert spblas.csrmv_noalloc(0, 8, 0, 1.0, None, None, None, None, 0.0, None) == capi.SUCCESS
    # no stored elements: y is scaled by beta, as alphasparse_d_mv does
    y = torch.arange(8, dtype=torch.float64, device="cuda")
    assert spblas.csrmv_noalloc(8, 8, 0, 1.0, ip, None, None, None, 2.0, y) == capi.SUCCESS
    assert y.cpu().tolist() == [0.0, 2.0, 4.0, 6.0, 8.0, 10.0, 12.0, 14.0]
