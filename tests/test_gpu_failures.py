"""Failure paths, produced on the host or by a bounded wait that is allowed to run out -- never by a GPU fault:
device allocation failures at every allocation of handle creation, a peer that never arrives, and concurrent
callers on one handle."""
import ctypes as C
import threading

import numpy as np
import pytest
import torch

import oracle
from alsparse_b200 import capi, multi, spblas, synth
from gpu_util import make_handle
from helpers import assert_rows_close, row_scale

pytestmark = pytest.mark.gpu


def test_allocation_failures_leave_nothing_behind():
    lib = capi.load()
    m = synth.zipf("d", 3, 20000, 20000, 1.8, 1, 5000)      # merge path: the creation allocates its tables too
    free0 = torch.cuda.mem_get_info()[0]
    failures = 0
    for nth in range(1, 40):
        lib.alphasparse_cuda_debug_fail_alloc(nth)
        st, A = spblas.create_csr("d", 0, m.nrows, m.cols, m.rows_start, m.rows_end, m.col, m.val)
        lib.alphasparse_cuda_debug_fail_alloc(0)
        if st == capi.SUCCESS:          # fewer than nth allocations were needed: every earlier one has been covered
            spblas.destroy(A)
            break
        assert st == capi.ALLOC_FAILED and not A.value and "device_alloc" in spblas.last_error()
        failures += 1
    # row_ptr, status, col, val, analysis scratch, tile table, carries, chunk counters, row lists, band tables
    assert 8 <= failures < 39
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] >= free0 - (4 << 20)   # nothing leaked (allow allocator granularity)
    # a staging-buffer failure inside mv is reported and the handle keeps working
    A = make_handle("d", m)
    x, y = synth.vector("d", 3, 1, m.cols), np.zeros(m.nrows)
    lib.alphasparse_cuda_debug_fail_alloc(1)
    assert spblas.mv("d", 0, 1.0, A, spblas.descr(), x, 0.0, y) == capi.ALLOC_FAILED
    lib.alphasparse_cuda_debug_fail_alloc(0)
    assert spblas.mv("d", 0, 1.0, A, spblas.descr(), x, 0.0, y) == capi.SUCCESS
    y_ref = oracle.gemv("d", m.rows_start, m.rows_end, m.col, m.val, 1.0, x, 0.0, np.zeros(m.nrows))
    assert_rows_close("d", y, y_ref, row_scale(m.ptr, m.col, m.val, x, 1.0, 0.0, y * 0), "after failed call")
    spblas.destroy(A)


def test_a_peer_that_never_arrives_is_reported_not_waited_for():
    lib = capi.load()
    m = synth.uniform_fixed("d", 4, 4096, 4096, 8)
    A = make_handle("d", m)
    ex = multi.FusedExchange("d", np.array([0, m.nrows], np.int32), 0, 1)
    ex.x_tensor().copy_(torch.from_numpy(synth.vector("d", 4, 1, m.cols)))
    y = torch.zeros(m.nrows, dtype=torch.float64, device="cuda")
    assert ex.step(1.0, A, 0.0, y) == capi.SUCCESS and ex.status() == (capi.SUCCESS, 0)
    assert lib.alphasparse_cuda_exchange_debug_wait(ex.handle, 2000) == capi.SUCCESS   # ~ a millisecond of polling
    st, code = ex.status()
    assert st == capi.EXECUTION_FAILED and code == 3
    # the context is intact: clear the status and carry on
    assert lib.alphasparse_cuda_exchange_clear_status(ex.handle) == capi.SUCCESS
    assert ex.step(1.0, A, 0.0, y) == capi.SUCCESS and ex.status() == (capi.SUCCESS, 0)
    assert torch.isfinite(y).all()
    ex.destroy()
    spblas.destroy(A)


def test_concurrent_callers_on_one_handle():
    m = synth.poisson("s", 6, 50000, 50000, 12.0)
    A = make_handle("s", m)
    xs = [synth.vector("s", 6, 10 + i, m.cols) for i in range(4)]
    ys = [np.zeros(m.nrows, np.float32) for _ in range(4)]
    errs = []

    def work(i):
        for _ in range(5):
            st = spblas.mv("s", 0, 1.0, A, spblas.descr(), xs[i], 0.0, ys[i])   # host pointers share the staging buffers
            if st != capi.SUCCESS:
                errs.append(st)
    threads = [threading.Thread(target=work, args=(i,)) for i in range(4)]
    [t.start() for t in threads]
    [t.join() for t in threads]
    assert not errs
    for i in range(4):
        y_ref = oracle.gemv("s", m.rows_start, m.rows_end, m.col, m.val, 1.0, xs[i], 0.0, np.zeros(m.nrows, np.float32))
        assert_rows_close("s", ys[i], y_ref, row_scale(m.ptr, m.col, m.val, xs[i], 1.0, 0.0, y_ref * 0), f"thread {i}")
    spblas.destroy(A)
