"""Shared pieces of the parity tests."""
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NP = {"s": np.float32, "d": np.float64}
# Tolerance of the parity gate: |y - y_ref| <= TOL * (|beta*y0| + |alpha| * sum_j |a_ij * x_j|) per row
# (1e-5 in single, 1e-12 in double precision).
TOL = {"s": 1e-5, "d": 1e-12}


def reference_dir():
    """The reference's source tree, when this machine has it: ALPHASPARSE_REFERENCE_DIR, else a checkout
    named ``reference`` next to this repository.  None when neither exists."""
    for cand in (os.environ.get("ALPHASPARSE_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.isfile(os.path.join(cand, "include", "alphasparse.h")):
            return cand
    return None


def golden(name):
    return np.load(os.path.join(GOLDEN, name))


def row_ids(ptr):
    return np.repeat(np.arange(len(ptr) - 1), np.diff(ptr))


def row_scale(ptr, col, val, x, alpha, beta, y0):
    """S_r = |beta*y0[r]| + |alpha| * sum_j |a_rj * x_j| in double precision."""
    prod = np.abs(val.astype(np.float64) * x.astype(np.float64)[col])
    s = np.bincount(row_ids(ptr), weights=prod, minlength=len(ptr) - 1)
    return np.abs(beta * y0.astype(np.float64)) + abs(alpha) * s


def assert_rows_close(kind, y, y_ref, scale, what=""):
    err = np.abs(y.astype(np.float64) - y_ref.astype(np.float64))
    bound = TOL[kind] * scale
    bad = err > bound
    # rows whose scale is exactly zero must match exactly
    assert not bad.any(), (f"{what}: {int(bad.sum())} of {len(y)} rows outside tolerance; worst ratio "
                           f"{np.max(err[bad] / np.maximum(bound[bad], 1e-300)):.3g} at row {int(np.argmax(bad))}")


def mm_scale(ptr, col, val, X, columns, ldx, alpha, beta, Y0, ldy):
    """Per (row, column) scale for row-major SpMM, shape (rows, columns)."""
    rows = len(ptr) - 1
    Xv = np.abs(X.astype(np.float64).reshape(-1)[: (X.size // ldx) * ldx].reshape(-1, ldx)[:, :columns])
    out = np.zeros((rows, columns))
    np.add.at(out, row_ids(ptr), np.abs(val.astype(np.float64))[:, None] * Xv[col])
    Y0v = np.abs(Y0.astype(np.float64).reshape(-1)[: rows * ldy].reshape(rows, ldy)[:, :columns])
    return abs(beta) * Y0v + abs(alpha) * out


def structured_scale(n, ptr, col, val, X, Y0, alpha, beta):
    """Per (row, column) scale for a product under a SYMMETRIC / TRIANGULAR / DIAGONAL descriptor: the bound
    of the widest variant, (|A| + |A|^T + I) |X|, on an n x n matrix small enough to hold densely."""
    dense = np.zeros((n, n))
    np.add.at(dense, (row_ids(ptr), col), np.abs(val.astype(np.float64)))
    return np.abs(beta * Y0.astype(np.float64)) + abs(alpha) * ((dense + dense.T + np.eye(n)) @ np.abs(X.astype(np.float64)))
