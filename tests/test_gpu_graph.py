"""Device-pointer calls only enqueue kernels on the library stream, so a caller can record them in a CUDA
graph and replay the graph: the way to run a launch-bound inner loop (many small products) without
per-call host cost."""
import numpy as np
import pytest
import torch

from alsparse_b200 import capi, spblas, synth
from gpu_util import make_handle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("kind,make", [("d", lambda: synth.stencil27("d", 16)),
                                       ("s", lambda: synth.uniform_fixed("s", 5, 6000, 6000, 16)),
                                       ("d", lambda: synth.zipf("d", 5, 6000, 6000, 1.8, 1, 3000))])
def test_products_replay_from_a_cuda_graph(kind, make):
    m = make()
    A = make_handle(kind, m)
    dt = torch.float32 if kind == "s" else torch.float64
    x = torch.from_numpy(synth.vector(kind, 5, 1, m.cols)).cuda()
    y = torch.zeros(m.nrows, dtype=dt, device="cuda")
    z = torch.zeros(m.nrows, dtype=dt, device="cuda")

    def chain():  # y = 0.1 A x ; z = 0.1 A y + 0.5 z   (square matrices)
        assert spblas.mv(kind, 0, 0.1, A, spblas.descr(), x, 0.0, y) == capi.SUCCESS
        assert spblas.mv(kind, 0, 0.1, A, spblas.descr(), y, 0.5, z) == capi.SUCCESS

    side = torch.cuda.Stream()
    spblas.set_stream(side.cuda_stream)
    try:
        with torch.cuda.stream(side):
            chain()                      # warm-up outside capture (first launches load the kernels)
            side.synchronize()
            z.zero_()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                chain()
            z.zero_()
            for _ in range(3):
                graph.replay()
            side.synchronize()
            z_graph = z.clone()
            z.zero_()
            for _ in range(3):
                chain()
            side.synchronize()
        assert torch.equal(z_graph, z)   # same kernels, same order: identical bits
        assert float(z.abs().sum()) > 0
    finally:
        spblas.set_stream(None)
        spblas.destroy(A)
