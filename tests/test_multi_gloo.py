"""The N > 1 path on CPU: two `gloo` ranks run the row partition, the block slicing and the
allgather of y into the next x, with the oracle standing in for the GPU product of each rank."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from alsparse_b200 import multi, synth

        # a skewed square matrix: the nnz-balanced blocks have very different row counts
        lens = synth.rowlen_zipf(5, 3000, 1.8, 1, 1500)
        lens[:40] = 0
        m = synth.from_lengths("d", 5, lens, 3000)
        part = multi.row_partition(m.rows_end, world)
        assert part[0] == 0 and part[-1] == m.nrows and np.all(np.diff(part) >= 0)
        assert np.array_equal(part, oracle.partition_rows_by_nnz(m.rows_end, world))
        r0, r1 = multi.local_rows(part, rank)
        ptr, col, val = multi.slice_csr(m.ptr, m.col, m.val, r0, r1)
        assert ptr[0] == 0 and ptr[-1] == len(col) == len(val) and col.max(initial=0) < m.cols

        # every rank must hold the same partition
        mine = torch.from_numpy(part.astype(np.int64))
        seen = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(seen, mine)
        assert all(torch.equal(s, mine) for s in seen)

        def local_mv(x_full, y_local):  # the oracle stands in for alphasparse_d_mv on this rank's block
            oracle.gemv("d", ptr[:-1], ptr[1:], col, val, 0.5, x_full.numpy(), 0.0, y_local.numpy())

        x0 = torch.from_numpy(synth.vector("d", 5, 1, m.cols))
        it = multi.IteratedSpmv(part, rank, x0.clone(), torch.zeros(r1 - r0, dtype=torch.float64), local_mv)
        x_ref = x0.numpy().copy()
        for _ in range(3):
            x = it.step()
            x_ref = oracle.gemv("d", m.rows_start, m.rows_end, m.col, m.val, 0.5, x_ref, 0.0, np.zeros(m.nrows))
            assert np.array_equal(x.numpy(), x_ref)  # same kernel, same order per row: bit-identical

        # a partition with an empty block (the reference's rule allows it)
        acc = np.array([2, 3, 4], np.int32)
        p2 = multi.row_partition(acc, world)
        assert p2.tolist() == ([0, 0, 3] if world == 2 else [0, 0, 0, 1, 3])
        a, b = multi.local_rows(p2, rank)
        out = multi.allgather_rows(torch.arange(a, b, dtype=torch.float64), torch.empty(3, dtype=torch.float64), p2)
        assert out.tolist() == [0.0, 1.0, 2.0]
        open(os.path.join(result_dir, f"ok{rank}"), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_partitioned_iteration_over_gloo(tmp_path, world):
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))
