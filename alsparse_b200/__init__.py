"""B200 (sm_100a) backend for the CSR SpMV / SpMM path of the AlphaSparse C API.

The product is ``libalphasparse_b200.so`` (C ABI declared in ``include/alphasparse/*.h``);
this package holds its sources (``csrc/``), the build step (``build.py``), the ctypes binding
(``capi``), a host-side mirror of the reference's operator interface (``spblas``), seeded input
generators (``synth``) and the one-process-per-GPU row-partitioned driver (``multi``).
"""
__all__ = ["capi", "spblas", "synth", "build"]
