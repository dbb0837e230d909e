"""alphasparse_?_mv_exchange: the SpMV kernels that also deliver y into every GPU's next x.

With one rank the exchange degenerates to "y is also written into my own next-x buffer", which
exercises the pushing epilogues of all kernel families on a single GPU.  The two-rank test needs
two GPUs and runs one process per GPU (kernels of different ranks wait on each other, so they must
never share a GPU)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import oracle
from alsparse_b200 import capi, multi, spblas, synth
from gpu_util import make_handle
from helpers import TOL, row_scale

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _matrices(kind):
    hi = 20000 if kind == "d" else 1500
    return [("merge", capi.ALG_MERGE, synth.zipf(kind, 3, 30000, 30000, 1.8, 1, hi)),
            ("rowtile", capi.ALG_ROWTILE, synth.stencil27(kind, 20)),
            ("vector", capi.ALG_VECTOR, synth.uniform_fixed(kind, 4, 20000, 20000, 16))]


@pytest.mark.parametrize("kind", ["s", "d"])
@pytest.mark.parametrize("after", [False, True])
def test_single_rank_push_matches_oracle(kind, after):
    for name, alg, m in _matrices(kind):
        spblas.set_algorithm(alg)
        A = make_handle(kind, m)
        spblas.set_algorithm(capi.ALG_AUTO)
        part = np.array([0, m.nrows], np.int32)
        ex = multi.FusedExchange(kind, part, 0, 1, deliver_after=after)
        x0 = synth.vector(kind, 3, 1, m.cols)
        ex.x_tensor().copy_(torch.from_numpy(x0))
        y0 = synth.vector(kind, 3, 2, m.nrows)
        y = torch.from_numpy(y0).cuda()
        x_ref, y_ref = x0.copy(), y0.copy()
        for it in range(3):
            alpha, beta = (0.125, 0.5) if it % 2 else (0.25, 0.0)
            assert ex.step(alpha, A, beta, y) == capi.SUCCESS
            scale = row_scale(m.ptr, m.col, m.val, x_ref, alpha, beta, y_ref)
            y_ref = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, alpha, x_ref, beta, y_ref)
            got_y, got_x = y.cpu().numpy(), ex.x_tensor().cpu().numpy()
            assert np.array_equal(got_y, got_x), f"{name}: pushed x differs from y"
            err = np.abs(got_y.astype(np.float64) - y_ref)
            assert (err <= (it + 1) * TOL[kind] * scale + 1e-300).all(), (name, it, float(np.max(err / np.maximum(scale, 1e-300))))
            x_ref = got_y.copy()   # follow the GPU's own iterate (teacher forcing), as y feeds back as x
            y_ref = got_y.copy()
        assert ex.status() == (capi.SUCCESS, 0)
        ex.destroy()
        spblas.destroy(A)


@pytest.mark.parametrize("kind", ["s", "d"])
def test_single_rank_push_with_column_blocks(kind):
    """Handles whose x counts as too large for L2 (limit shrunk): the vector kernel and the lists of a binned handle run
    column block by column block, and only the last launch of a list delivers to the peers."""
    opts = dict(mv_block_min_kb=1, mv_block_kb=32, band_bytes=4096, band_min_seg=2, band_min_rows=1, band_min_share_pct=0,
                bin_short=2, bin_mid0=8, bin_mid1=64)
    hi = 20000 if kind == "d" else 1500
    cases = [("binned", synth.zipf(kind, 5, 30000, 30000, 1.8, 1, hi)), ("vector", synth.uniform_fixed(kind, 6, 20000, 20000, 16))]
    for name, m in cases:
        try:
            for k, v in opts.items():
                assert spblas.set_option(k, v) == capi.SUCCESS
            A = make_handle(kind, m)
        finally:
            for k in opts:
                spblas.set_option(k, -1)
        info = spblas.mat_info(A)[1]
        assert (info.binned == 1) == (name == "binned"), (name, info.binned, info.algorithm)
        ex = multi.FusedExchange(kind, np.array([0, m.nrows], np.int32), 0, 1, deliver_after=False)
        x_ref = synth.vector(kind, 5, 1, m.cols)
        ex.x_tensor().copy_(torch.from_numpy(x_ref))
        y_ref = synth.vector(kind, 5, 2, m.nrows)
        y = torch.from_numpy(y_ref).cuda()
        for it in range(3):
            alpha, beta = (0.125, 0.5) if it % 2 else (0.25, 0.0)
            assert ex.step(alpha, A, beta, y) == capi.SUCCESS
            scale = row_scale(m.ptr, m.col, m.val, x_ref, alpha, beta, y_ref)
            want = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, alpha, x_ref, beta, y_ref)
            got_y, got_x = y.cpu().numpy(), ex.x_tensor().cpu().numpy()
            assert np.array_equal(got_y, got_x), f"{name}: pushed x differs from y"
            err = np.abs(got_y.astype(np.float64) - want)
            assert (err <= (it + 1) * TOL[kind] * scale + 1e-300).all(), (name, it, float(np.max(err / np.maximum(scale, 1e-300))))
            x_ref, y_ref = got_y.copy(), got_y.copy()
        assert ex.status() == (capi.SUCCESS, 0)
        ex.destroy()
        spblas.destroy(A)


def test_single_rank_load_x():
    """alphasparse_cuda_exchange_load_x with one rank: the piece is the whole vector; buffers swap as after a product."""
    m = synth.uniform_fixed("s", 4, 5000, 5000, 8)
    A = make_handle("s", m)
    ex = multi.FusedExchange("s", np.array([0, m.nrows], np.int32), 0, 1)
    xa, xb = synth.vector("s", 5, 1, m.cols), synth.vector("s", 5, 2, m.cols)
    before = ex.x_ptr()
    assert ex.load_x(xa) == capi.SUCCESS
    assert ex.x_ptr() != before and np.array_equal(ex.x_tensor().cpu().numpy(), xa)
    y = torch.zeros(m.nrows, device="cuda")
    assert ex.step(1.0, A, 0.0, y) == capi.SUCCESS
    ref = oracle.gemv("s", m.rows_start, m.rows_end, m.col, m.val, 1.0, xa, 0.0, np.zeros(m.nrows, np.float32))
    assert (np.abs(y.cpu().numpy() - ref) <= TOL["s"] * row_scale(m.ptr, m.col, m.val, xa, 1.0, 0.0, ref * 0) + 1e-30).all()
    assert ex.load_x(torch.from_numpy(xb).cuda()) == capi.SUCCESS
    assert np.array_equal(ex.x_tensor().cpu().numpy(), xb)
    assert ex.load_x(None) == capi.INVALID_POINTER
    assert ex.status() == (capi.SUCCESS, 0)
    ex.destroy()
    spblas.destroy(A)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        kind = "d"
        m = synth.zipf(kind, 8, 60000, 60000, 1.8, 1, 30000)
        part = multi.row_partition(m.rows_end, world)
        r0, r1 = multi.local_rows(part, rank)
        ptr, col, val = multi.slice_csr(m.ptr, m.col, m.val, r0, r1)
        st, A = spblas.create_csr(kind, 0, r1 - r0, m.cols, ptr[:-1], ptr[1:], col, val)
        assert st == capi.SUCCESS, spblas.last_error()
        ex = multi.FusedExchange(kind, part, rank, world)
        x0 = synth.vector(kind, 8, 1, m.cols)
        ex.x_tensor().copy_(torch.from_numpy(x0))
        torch.cuda.synchronize()
        dist.barrier()
        y = torch.zeros(r1 - r0, dtype=torch.float64, device="cuda")
        x_ref = x0.copy()
        for it in range(4):
            assert ex.step(0.2, A, 0.0, y) == capi.SUCCESS
            x_new = ex.x_tensor().cpu().numpy()            # gathered y of ALL ranks
            scale = row_scale(m.ptr, m.col, m.val, x_ref, 0.2, 0.0, np.zeros(m.nrows))
            ref = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, 0.2, x_ref, 0.0, np.zeros(m.nrows))
            err = np.abs(x_new - ref)
            assert (err <= TOL[kind] * scale + 1e-300).all(), (rank, it, float(np.max(err / np.maximum(scale, 1e-300))))
            assert np.array_equal(x_new[r0:r1], y.cpu().numpy())
            x_ref = x_new
        # x set from the ranks' own rows of a host vector: every GPU ends up with all of it, and the
        # products carry on from there
        x1 = synth.vector(kind, 8, 5, m.cols)
        assert ex.load_x(x1[r0:r1].copy()) == capi.SUCCESS
        assert np.array_equal(ex.x_tensor().cpu().numpy(), x1)
        assert ex.step(0.2, A, 0.0, y) == capi.SUCCESS
        ref = oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, 0.2, x1, 0.0, np.zeros(m.nrows))
        scale = row_scale(m.ptr, m.col, m.val, x1, 0.2, 0.0, np.zeros(m.nrows))
        assert (np.abs(ex.x_tensor().cpu().numpy() - ref) <= TOL[kind] * scale + 1e-300).all()
        assert ex.load_x(torch.from_numpy(x0[r0:r1].copy()).cuda()) == capi.SUCCESS      # a device piece works too
        assert np.array_equal(ex.x_tensor().cpu().numpy(), x0)
        assert ex.status() == (capi.SUCCESS, 0)
        dist.barrier()
        ex.destroy()
        spblas.destroy(A)
        open(os.path.join(out_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs (one process per GPU)")
def test_two_ranks_gather_through_the_kernel(tmp_path):
    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
