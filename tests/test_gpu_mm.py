"""Parity of alphasparse_{s,d}_mm (row-major) on the GPU with the reference's plain kernel."""
import numpy as np
import pytest
import torch

import oracle
from alsparse_b200 import capi, spblas, synth
from gpu_util import make_handle
from helpers import assert_rows_close, golden, mm_scale

pytestmark = pytest.mark.gpu


def run_mm(kind, A, m, X, columns, ldx, alpha, beta, Y0, ldy, device):
    if device:
        dX, dY = torch.from_numpy(X).cuda(), torch.from_numpy(Y0).cuda()
        st = spblas.mm(kind, 0, alpha, A, spblas.descr(), capi.ROW_MAJOR, dX, columns, ldx, beta, dY, ldy)
        torch.cuda.synchronize()
        Y = dY.cpu().numpy()
    else:
        Y = Y0.copy()
        st = spblas.mm(kind, 0, alpha, A, spblas.descr(), capi.ROW_MAJOR, X, columns, ldx, beta, Y, ldy)
    assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
    return Y


def compare(kind, m, Y, Yref, X, columns, ldx, alpha, beta, Y0, ldy, what):
    rows = m.nrows
    scale = mm_scale(m.ptr, m.col, m.val, X, columns, ldx, alpha, beta, Y0, ldy)
    assert_rows_close(kind, Y.reshape(rows, ldy)[:, :columns].reshape(-1),
                      Yref.reshape(rows, ldy)[:, :columns].reshape(-1), scale.reshape(-1), what)
    assert np.array_equal(Y.reshape(rows, ldy)[:, columns:], Y0.reshape(rows, ldy)[:, columns:]), "padding written"


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("case", ["w64", "w5"])
@pytest.mark.parametrize("device", [False, True])
def test_golden_vectors(kind, case, device):
    g = golden(f"mm_{kind}.npz")
    m = synth.Csr(int(g["rows"]), int(g["cols"]), 0, g["ptr"], g["col"], g["val"])
    columns, ldx, ldy = (int(v) for v in g[f"{case}_par"][:3])
    alpha, beta = float(g[f"{case}_par"][5]), float(g[f"{case}_par"][6])
    A = make_handle(kind, m)
    Y = run_mm(kind, A, m, g[f"{case}_X"], columns, ldx, alpha, beta, g[f"{case}_Y0"], ldy, device)
    compare(kind, m, Y, g[f"{case}_row"], g[f"{case}_X"], columns, ldx, alpha, beta, g[f"{case}_Y0"], ldy, case)
    spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("columns,ldx,ldy", [(64, 64, 64), (64, 80, 72), (1, 1, 1), (3, 3, 5), (32, 32, 32),
                                             (100, 100, 100), (128, 128, 128), (130, 131, 133), (256, 256, 256)])
def test_widths_and_leading_dimensions(kind, columns, ldx, ldy):
    m = synth.poisson(kind, 12, 3000, 2500, 32.0)
    lens = np.diff(m.ptr).copy()
    lens[::50] = 0
    lens[7] = 700
    m = synth.from_lengths(kind, 12, lens, 2500)
    X, Y0 = synth.vector(kind, 12, 3, m.cols * ldx), synth.vector(kind, 12, 4, m.nrows * ldy)
    A = make_handle(kind, m)
    for alpha, beta in ((1.0, 0.0), (1.5, 0.5)):
        Yref = oracle.gemm(kind, "row", m.rows_start, m.rows_end, m.col, m.val, alpha, X, columns, ldx, beta,
                           Y0.copy(), ldy)
        for device in (False, True):
            Y = run_mm(kind, A, m, X, columns, ldx, alpha, beta, Y0, ldy, device)
            compare(kind, m, Y, Yref, X, columns, ldx, alpha, beta, Y0, ldy, f"{columns}/{ldx}/{ldy} dev={device}")
    spblas.destroy(A)


def test_status_codes():
    m = synth.poisson("s", 8, 30, 40, 4.0)
    A = make_handle("s", m)
    X, Y = np.zeros(40 * 4, np.float32), np.zeros(30 * 4, np.float32)
    g = spblas.descr()
    assert spblas.mm("s", 0, 1.0, A, g, 0, None, 4, 4, 0.0, Y, 4) == capi.NOT_INITIALIZED
    assert spblas.mm("d", 0, 1.0, A, g, 0, X, 4, 4, 0.0, Y, 4) == capi.INVALID_VALUE
    assert spblas.mm("s", capi.CONJUGATE_TRANSPOSE, 1.0, A, g, 0, X, 4, 4, 0.0, Y, 4) == capi.INVALID_VALUE
    assert spblas.mm("s", 0, 1.0, A, spblas.descr(capi.SYMMETRIC), 0, X, 4, 4, 0.0, Y, 4) == capi.INVALID_VALUE
    assert spblas.mm("s", 0, 1.0, A, spblas.descr(capi.TRIANGULAR), 0, X, 4, 4, 0.0, Y, 4) == capi.NOT_SUPPORTED
    spblas.destroy(A)
