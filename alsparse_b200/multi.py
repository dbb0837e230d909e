"""Row-partitioned SpMV across the GPUs of one box: one process per GPU (torch.distributed).

The reference splits rows across OpenMP threads with ``balanced_partition_row_by_nnz``
(src/util/partition.c:79-92 of the reference, used at src/kernel/x86_64/level2/mv/gemv/gemv_x_csr.c:193-206);
here the same rule, bit for bit, splits them across GPUs: rank g owns the contiguous rows
``[part[g], part[g+1])`` with offsets rebased to its block and GLOBAL column indices, x is replicated
on every GPU, y stays partitioned.  There is no exchange on the data path unless y must become the
next x (iterated SpMV): then every rank's y block is gathered into every rank's next-x buffer.

Only host-side logic lives here; it runs unchanged over the ``gloo`` backend on CPU tensors, which
is how it is tested without GPUs.
"""
import ctypes as C

import numpy as np
import torch
import torch.distributed as dist

from . import capi, spblas


def row_partition(rows_end, world):
    """``world + 1`` row boundaries from the inclusive prefix sums of the row lengths (rows_end)."""
    return spblas.partition_rows_by_nnz(np.ascontiguousarray(rows_end, dtype=np.int32), world)


def local_rows(part, rank):
    return int(part[rank]), int(part[rank + 1])


def slice_csr(ptr, col, val, r0, r1):
    """Rows [r0, r1) of a 3-array CSR as (local offsets, columns, values): offsets rebased to zero,
    column indices untouched."""
    lo, hi = int(ptr[r0]), int(ptr[r1])
    return (ptr[r0:r1 + 1] - ptr[r0]).astype(np.int32), col[lo:hi], val[lo:hi]


def gather_sizes(part):
    return [int(part[i + 1] - part[i]) for i in range(len(part) - 1)]


def allgather_rows(y_local, out_full, part, group=None):
    """Gathers every rank's y block into ``out_full`` (length = total rows) on every rank.

    Blocks have unequal sizes (the nnz-balanced rule) and may be empty, so this is an
    allgather-v: ``out_full`` is split at the partition boundaries and each piece is filled from
    its owner.  Works on CUDA tensors over NCCL and on CPU tensors over gloo.
    """
    sizes = gather_sizes(part)
    pieces = list(torch.split(out_full, sizes))
    if dist.get_backend(group) == "gloo":
        # gloo's all_gather wants equal shapes: pad to the largest block, then trim
        width = max(max(sizes), 1)
        padded = torch.zeros(width, dtype=y_local.dtype)
        padded[: y_local.numel()] = y_local
        bufs = [torch.empty(width, dtype=y_local.dtype) for _ in sizes]
        dist.all_gather(bufs, padded, group=group)
        for piece, buf, n in zip(pieces, bufs, sizes):
            piece.copy_(buf[:n])
    else:
        dist.all_gather(pieces, y_local, group=group)
    return out_full


class IteratedSpmv:
    """x_{t+1} = alpha * A * x_t (+ beta * y_t) with A row-partitioned and y all-gathered into the
    next x after every product.  ``local_mv(x_full, y_local)`` performs this rank's product; it is
    a parameter so that the exchange logic can be exercised on CPU with a stand-in product."""

    def __init__(self, part, rank, x0, y_local, local_mv, group=None):
        self.part, self.rank, self.group = part, rank, group
        self.x, self.x_next = x0, torch.empty_like(x0)
        self.y_local, self.local_mv = y_local, local_mv

    def step(self):
        self.local_mv(self.x, self.y_local)
        allgather_rows(self.y_local, self.x_next, self.part, self.group)
        self.x, self.x_next = self.x_next, self.x
        return self.x


class FusedExchange:
    """The product-plus-allgather in one kernel (``alphasparse_?_mv_exchange``): every rank's SpMV
    stores its finished y rows straight into the next-x buffer of every GPU over NVLink, then the
    ranks signal each other and the buffers swap.  CUDA only; set-up exchanges 192-byte IPC blobs
    through ``torch.distributed`` (any backend)."""

    def __init__(self, kind, part, rank, world, group=None, deliver_after=None):
        lib = capi.load()
        self.kind, self.part, self.rank, self.world = kind, np.ascontiguousarray(part, dtype=np.int32), rank, world
        self.handle = C.c_void_p()
        dt = capi.FLOAT if kind == "s" else capi.DOUBLE
        st = lib.alphasparse_cuda_exchange_create(C.byref(self.handle), dt, rank, world, self.part.ctypes.data)
        assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
        nbytes = lib.alphasparse_cuda_exchange_blob_bytes()
        blob = (C.c_ubyte * nbytes)()
        st = lib.alphasparse_cuda_exchange_export(self.handle, blob)
        assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
        if world > 1:
            blobs = [None] * world
            dist.all_gather_object(blobs, bytes(blob), group=group)
        else:
            blobs = [bytes(blob)]
        joined = b"".join(blobs)
        st = lib.alphasparse_cuda_exchange_connect(self.handle, joined)
        assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
        if deliver_after is not None:  # None keeps the library's choice for this number of GPUs
            lib.alphasparse_cuda_exchange_set_mode(self.handle, 1 if deliver_after else 0)
        if world > 1:
            dist.barrier(group=group)  # nobody starts pushing before every rank has mapped every buffer

    def x_ptr(self):
        p = C.c_void_p()
        st = capi.load().alphasparse_cuda_exchange_x(self.handle, C.byref(p))
        assert st == capi.SUCCESS
        return p.value

    def x_tensor(self):
        """The current x as a torch view of the library's buffer (valid until the next step)."""
        n = int(self.part[-1])
        typestr = "<f4" if self.kind == "s" else "<f8"

        class _Raw:
            __cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (self.x_ptr(), False), "version": 2}
        return torch.as_tensor(_Raw(), device="cuda")

    def load_x(self, x_block):
        """Sets x on every GPU from the ranks' own rows of it (numpy / pinned host tensor or CUDA tensor of
        part[rank+1] - part[rank] elements): each GPU uploads 1/world of x and the pieces cross NVLink."""
        return capi.load().alphasparse_cuda_exchange_load_x(self.handle, spblas._ptr(x_block))

    def step(self, alpha, A, beta, y_local):
        fn = getattr(capi.load(), f"alphasparse_{self.kind}_mv_exchange")
        return fn(alpha, A, spblas.descr(), self.handle, beta, spblas._ptr(y_local))

    def status(self):
        code = C.c_int()
        st = capi.load().alphasparse_cuda_exchange_status(self.handle, C.byref(code))
        return st, code.value

    def destroy(self):
        if self.handle:
            capi.load().alphasparse_cuda_exchange_destroy(self.handle)
            self.handle = C.c_void_p()
