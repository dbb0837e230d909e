"""The C-ABI library loads, exports every symbol its headers declare, and its headers are valid C
with the layouts the reference's callers were compiled against.  No compute calls: runs without a GPU."""
import ctypes as C
import os
import re
import subprocess
import tempfile

import numpy as np
import pytest

from alsparse_b200 import capi, spblas
from helpers import reference_dir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INC = os.path.join(ROOT, "include")
REF_INC = os.path.join(reference_dir() or "", "include")


def declared_functions():
    names = set()
    for h in ("spapi.h", "spapi_cuda.h", "util.h", "kernel_cuda.h"):
        text = open(os.path.join(INC, "alphasparse", h)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"#define(?:.*\\\n)*.*\n", "", text)   # macros (with their continuation lines) are not exports
        names |= set(re.findall(r"\b(alpha\w+|args_\w+|gem[vm]_\w+|lower_bound_int|balanced_partition_row_by_nnz)\s*\(", text))
    return {n for n in names if not n.startswith(("alphasparse_status_t", "alphasparse_cuda_alg_t"))}


def test_every_declared_symbol_is_exported_and_bound():
    lib = capi.load()
    declared = declared_functions()
    assert len(declared) >= 35
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert declared == set(capi.prototypes()), declared ^ set(capi.prototypes())


def test_headers_compile_as_c_and_layouts_match():
    src = r"""
    #include <alphasparse.h>
    #include <stdio.h>
    #include <stddef.h>
    int main(void) {
        printf("%zu %zu %zu %zu %zu %zu %zu %d %d %d %d\n", sizeof(alphasparse_matrix),
               offsetof(alphasparse_matrix, format), offsetof(alphasparse_matrix, datatype),
               offsetof(alphasparse_matrix, inspector), offsetof(alphasparse_matrix, dcu_info),
               sizeof(struct alpha_matrix_descr), sizeof(ALPHA_INT), (int)ALPHA_SPARSE_STATUS_INVALID_HANDLE,
               (int)ALPHA_SPARSE_FORMAT_CSR, (int)ALPHA_SPARSE_DATATYPE_DOUBLE, (int)ALPHA_SPARSE_LAYOUT_COLUMN_MAJOR);
        return 0;
    }"""
    outs = []
    for inc in [INC] + ([REF_INC] if os.path.isdir(REF_INC) else []):
        with tempfile.TemporaryDirectory() as d:
            open(os.path.join(d, "t.c"), "w").write(src)
            subprocess.check_call(["/usr/bin/gcc", "-std=gnu11", "-I", inc, os.path.join(d, "t.c"), "-o",
                                   os.path.join(d, "t")])
            outs.append(subprocess.check_output([os.path.join(d, "t")]).decode().split())
    assert outs[0] == ["32", "8", "12", "16", "24", "12", "4", "8", "1", "1", "1"]
    assert all(o == outs[0] for o in outs)  # identical when built against the reference's own header
    assert C.sizeof(capi.Matrix) == 32 and C.sizeof(capi.MatrixDescr) == 12


@pytest.mark.skipif(not os.path.isdir(REF_INC), reason="reference headers not on this machine")
def test_reference_style_caller_links_against_the_library():
    """A caller compiled against the REFERENCE'S header links to this library without changes."""
    src = r"""
    #include <alphasparse.h>
    int main(void) {
        alphasparse_matrix_t A = 0;
        struct alpha_matrix_descr d = {ALPHA_SPARSE_MATRIX_TYPE_GENERAL, 0, 0};
        float x[1] = {0}, y[1] = {0};
        /* NULL handle: rejected before any device work */
        int a = alphasparse_s_mv(ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, 1.f, A, d, x, 0.f, y);
        int b = alphasparse_d_mm(ALPHA_SPARSE_OPERATION_NON_TRANSPOSE, 1., A, d, ALPHA_SPARSE_LAYOUT_ROW_MAJOR,
                                 (double *)x, 1, 1, 0., (double *)y, 1);
        int c = alphasparse_destroy(A);
        return (a == ALPHA_SPARSE_STATUS_NOT_INITIALIZED && b == ALPHA_SPARSE_STATUS_NOT_INITIALIZED &&
                c == ALPHA_SPARSE_STATUS_SUCCESS) ? 0 : 1;
    }"""
    with tempfile.TemporaryDirectory() as d:
        open(os.path.join(d, "t.c"), "w").write(src)
        subprocess.check_call(["/usr/bin/gcc", "-std=gnu11", "-w", "-I", REF_INC, os.path.join(d, "t.c"), "-o",
                               os.path.join(d, "t"), capi.LIB_PATH, "-Wl,-rpath," + os.path.dirname(capi.LIB_PATH)])
        assert subprocess.call([os.path.join(d, "t")]) == 0


def test_argument_checks_need_no_device():
    x = np.zeros(4, np.float32)
    g = spblas.descr()
    assert spblas.mv("s", 0, 1.0, None, g, x, 0.0, x) == capi.NOT_INITIALIZED
    h = capi.Matrix(None, capi.FORMAT_CSR, capi.FLOAT, None, None)
    assert spblas.mv("s", 0, 1.0, C.byref(h), g, x, 0.0, x) == capi.NOT_INITIALIZED      # mat == NULL
    h.mat = x.ctypes.data  # any non-NULL pointer: the checks below never dereference it
    assert spblas.mv("s", 0, 1.0, C.byref(h), g, None, 0.0, x) == capi.NOT_INITIALIZED
    assert spblas.mv("d", 0, 1.0, C.byref(h), g, x, 0.0, x) == capi.INVALID_VALUE        # datatype mismatch
    assert spblas.mv("s", capi.CONJUGATE_TRANSPOSE, 1.0, C.byref(h), g, x, 0.0, x) == capi.INVALID_VALUE
    assert spblas.mv("s", 0, 1.0, C.byref(h), spblas.descr(6), x, 0.0, x) == capi.INVALID_VALUE
    assert spblas.mv("s", 0, 1.0, C.byref(h), spblas.descr(capi.TRIANGULAR), x, 0.0, x) == capi.INVALID_HANDLE  # no device context behind it
    h.format = 9
    assert spblas.mv("s", 0, 1.0, C.byref(h), g, x, 0.0, x) == capi.INVALID_VALUE
    h.format = capi.FORMAT_CSR
    assert spblas.mm("s", 0, 1.0, C.byref(h), g, 0, x, 1, 1, 0.0, None, 1) == capi.NOT_INITIALIZED
    assert spblas.mm("d", 0, 1.0, C.byref(h), g, 0, x, 1, 1, 0.0, x, 1) == capi.INVALID_VALUE
    assert spblas.destroy(None) == capi.SUCCESS
    lib = capi.load()
    for k in "cz":  # complex entry points exist and refuse
        assert getattr(lib, f"alphasparse_{k}_create_csr")(C.byref(C.c_void_p()), 0, 1, 1, None, None, None,
                                                            None) == capi.NOT_SUPPORTED


def test_product_does_not_touch_the_oracle():
    """The shipped code (package sources, headers) never refers to the CPU checkers."""
    bad = []
    pkg = os.path.join(ROOT, "alsparse_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".h", ".c", ".cpp")) and f != "build.py":
                text = open(os.path.join(base, f), errors="ignore").read()
                if re.search(r"\boracle\b|liboracle|libalpha_ref", text):
                    bad.append(os.path.join(base, f))
    assert not bad, bad
