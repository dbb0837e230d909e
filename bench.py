"""Benchmark of the CSR SpMV / SpMM path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One "step" is one pass of the hot path over the whole matrix: one alphasparse_?_mv (or _mm) call
per GPU on its row block.  The metric is effective GB/s = algorithmic bytes / step time, where
algorithmic bytes = values + col_idx + row_ptr + x + y, each array counted once for the whole
matrix (also reported: GFLOP/s = 2*nnz[*columns] / step time).

Workloads (seeded synthetic stand-ins for the user-supplied matrix files the reference's tests read):
  uniform16   fp32, 2^24 x 2^24, exactly 16 distinct uniform columns per row, alpha=1.5, beta=0.5
              (default: the configuration that is row-partitioned over 1/2/4/8 GPUs)
  stencil27   fp64, 27-point stencil on a 160^3 grid, alpha=1, beta=0
  powerlaw    fp64, 2^23 rows, Zipf(1.8) row lengths clipped to [1, 200000], alpha=1, beta=0;
              with more than one GPU every step ends with the allgather of y into the next x
  spmm64      fp32, 2^21 rows Poisson(32), times a 2^21 x 64 row-major dense block, alpha=1, beta=0

With N > 1 (launched by torch.distributed.run, one process per GPU) the rows are split by the
reference's nnz-balanced rule, x is replicated, y stays partitioned: total work is fixed, so the
scaling is "strong".  `--impl reference` times the reference's own OpenMP CPU kernel instead.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only without MEASURED_PEAKS.json

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu
# captures summarised under profiles/ (bytes; None where no capture exists yet).
NCU_TRAFFIC = {"uniform16": 3937436144, "stencil27": 1393600664, "powerlaw": None, "spmm64": 17518304000}

WORKLOADS = {
    "uniform16": dict(kind="s", rows_log2=24, alpha=1.5, beta=0.5, op="mv"),
    "stencil27": dict(kind="d", grid=160, alpha=1.0, beta=0.0, op="mv"),
    "powerlaw": dict(kind="d", rows_log2=23, alpha=1.0, beta=0.0, op="mv"),
    "spmm64": dict(kind="s", rows_log2=21, alpha=1.0, beta=0.0, op="mm", columns=64),
}
TSIZE = {"s": 4, "d": 8}


# ------------------------------------------------------------------------------------------------
# workload construction
# ------------------------------------------------------------------------------------------------
def global_row_lengths(name, cfg, seed=0):
    """Row lengths of the whole matrix (cheap; needed for the nnz-balanced split)."""
    from alsparse_b200 import synth
    if name == "stencil27":
        import ctypes  # noqa: F401
        n = cfg["grid"]
        lens = np.empty(n ** 3, dtype=np.int32)
        synth._load().synth_stencil27_rowlen(n, 0, n ** 3, lens.ctypes.data)
        return lens
    rows = 1 << cfg["rows_log2"]
    if name == "uniform16":
        return synth.rowlen_fixed(rows, 16)
    if name == "powerlaw":
        return synth.rowlen_zipf(seed, rows, 1.8, 1, min(200000, rows))
    if name == "spmm64":
        return synth.rowlen_poisson(seed, rows, 32.0, rows)
    raise ValueError(name)


def local_block(name, cfg, lens, r0, r1, seed=0):
    """Rows [r0, r1) as a CSR piece with local offsets and global columns."""
    from alsparse_b200 import synth
    kind = cfg["kind"]
    if name == "stencil27":
        return synth.stencil27(kind, cfg["grid"], row0=r0, nrows=r1 - r0)
    rows = len(lens)
    return synth._fill_uniform(kind, seed, r0, np.ascontiguousarray(lens[r0:r1]), rows, rows)


def algorithmic_bytes(cfg, rows, cols, nnz):
    t = TSIZE[cfg["kind"]]
    k = cfg.get("columns", 1)
    return nnz * t + nnz * 4 + (rows + 1) * 4 + cols * k * t + rows * k * t


def flops(cfg, nnz):
    return 2 * nnz * cfg.get("columns", 1)


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples the SM clock and the throttle reasons of one GPU in a background thread: through NVML every
    2 ms when the bindings are present, else through `nvidia-smi -lms 50`.  Read-only."""
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index, uuid=None):
        self.samples, self.proc, self.stop_flag, self.max_mhz = [], None, False, None
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            h = None
            if uuid:
                for cand in (f"GPU-{uuid}", str(uuid)):
                    try:
                        h = pynvml.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                        break
                    except Exception:
                        h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
            reasons_fn = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                pynvml.nvmlDeviceGetCurrentClocksThrottleReasons

            def pump():
                while not self.stop_flag:
                    try:
                        mhz = float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                        mask = int(reasons_fn(h))
                        self.samples.append((time.time(), mhz, [n for b, n in self.REASONS.items() if mask & b]))
                    except Exception:
                        pass
                    time.sleep(0.002)
            self.thread = threading.Thread(target=pump, daemon=True)
            self.thread.start()
            self.source = "nvml"
            return
        except Exception:
            pass
        self.source = "nvidia-smi"
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50", "-i",
                 str(gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump_smi, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump_smi(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            p = [x.strip() for x in line.split(",")]
            try:
                self.max_mhz = float(p[1])
                self.samples.append((time.time(), float(p[0]),
                                     [names[i] for i, f in enumerate(p[3:7]) if f.lower().startswith("active")]))
            except (ValueError, IndexError):
                pass

    def stop(self):
        self.stop_flag = True
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, t0, t1):
        window = [x for x in self.samples if t0 <= x[0] <= t1]
        scope = "timed region"
        if len(window) < 3:
            window, scope = list(self.samples), "warm-up + timed region + kernel-timing pass (timed region too short to sample)"
        if not window:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "scope": "no sampler available"}
        return {"sm_mhz": statistics.median(w[1] for w in window), "sm_max_mhz": self.max_mhz,
                "reasons": sorted({r for w in window for r in w[2]}), "samples": len(window), "scope": scope,
                "source": self.source}


# ------------------------------------------------------------------------------------------------
# the reference arm / CPU baseline
# ------------------------------------------------------------------------------------------------
def cpu_reference_run(name, cfg, steps, warmup, sample_rows_log2=22):
    """The reference's own OpenMP kernel (oracle/_ref) -- or the oracle port of it when those objects
    are absent -- on a bounded sample: the first 2^sample_rows_log2 rows of the workload's matrix with
    x at full length, all host threads.  Returns (GB/s, GFLOP/s, ms per step, descriptor dict)."""
    import oracle
    from alsparse_b200 import synth
    kind = cfg["kind"]
    lens = global_row_lengths(name, cfg)
    rows, cols = len(lens), len(lens)
    n = min(rows, 1 << sample_rows_log2)
    if cfg["op"] == "mm":
        n = min(n, 1 << 19)
    m = local_block(name, cfg, lens, 0, n)
    columns = cfg.get("columns", 1)
    x = synth.vector(kind, 0, 1, cols * columns, 0.0 if name == "stencil27" else -1.0, 1.0)
    y = synth.vector(kind, 0, 2, n * columns)
    use_ref = oracle.ref_available()
    threads = oracle.ref_cores() if use_ref else oracle.max_threads()
    A = oracle.RefCsr.from_csr(kind, 0, n, cols, m.rows_start, m.rows_end, m.col, m.val) if use_ref else None

    def step():
        if cfg["op"] == "mv":
            if use_ref:
                A.gemv(cfg["alpha"], x, cfg["beta"], y, omp_threads=threads)
            else:
                oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, cfg["alpha"], x, cfg["beta"], y,
                            threads=threads)
        else:
            if use_ref:
                A.gemm("row", cfg["alpha"], x, columns, columns, cfg["beta"], y, columns, omp_threads=threads)
            else:
                oracle.gemm(kind, "row", m.rows_start, m.rows_end, m.col, m.val, cfg["alpha"], x, columns, columns,
                            cfg["beta"], y, columns, threads=threads)

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = (time.perf_counter() - t0) / max(steps, 1)
    nbytes = algorithmic_bytes(cfg, n, cols, m.nnz)
    desc = {"kind": "reference" if use_ref else "port", "cores": threads,
            "sample": f"rows [0, {n}) of {rows} ({m.nnz} stored elements), x at full length {cols}"
                      f"{' x ' + str(columns) if columns > 1 else ''}; {steps} timed calls after {warmup} warm-up"}
    return nbytes / dt / 1e9, flops(cfg, m.nnz) / dt / 1e9, dt * 1e3, desc


def run_reference_arm(args, name, cfg, rank):
    if rank != 0:
        return
    gbs, gfl, ms, desc = cpu_reference_run(name, cfg, args.steps, max(args.warmup, 1))
    line = {"impl": "reference", "metric": "csr_spmv_effective_gbs" if cfg["op"] == "mv" else "csr_spmm_effective_gbs",
            "value": gbs, "unit": "GB/s", "gflops": gfl, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": max(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32" if cfg["kind"] == "s" else "f64", "data": "synthetic",
            "config": {"workload": name}, "cpu_baseline": dict(value=gbs, unit="GB/s", **desc),
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# the GPU arm
# ------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default="uniform16", choices=sorted(WORKLOADS))
    ap.add_argument("--rows-log2", type=int, default=None, help="shrink the matrix (development only)")
    ap.add_argument("--grid", type=int, default=None, help="shrink the stencil grid (development only)")
    ap.add_argument("--alg", default="auto", choices=["auto", "vector", "merge", "rowtile"])
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "push", "nccl"],
                    help="iterated workload with several GPUs: y reaches the next x from inside the SpMV kernels "
                         "over peer memory (fused), by one peer-copy kernel after them (push), "
                         "whichever of the two the library prefers for this many GPUs (auto) or by a NCCL allgather (nccl)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-others", action="store_true",
                    help="do not append the short device-resident runs of the other three workloads (N=1 only)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    name = args.workload
    cfg = dict(WORKLOADS[name])
    reduced = False
    if args.rows_log2 is not None and "rows_log2" in cfg:
        reduced, cfg["rows_log2"] = cfg["rows_log2"] != args.rows_log2, args.rows_log2
    if args.grid is not None and "grid" in cfg:
        reduced, cfg["grid"] = cfg["grid"] != args.grid, args.grid

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, name, cfg, rank)
        return

    import torch
    import torch.distributed as dist

    from alsparse_b200 import capi, multi, spblas, synth

    assert torch.cuda.is_available(), "bench.py needs a CUDA device: there is no CPU path"
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    kind, alpha, beta, op = cfg["kind"], cfg["alpha"], cfg["beta"], cfg["op"]
    tdt = torch.float32 if kind == "s" else torch.float64
    columns = cfg.get("columns", 1)
    # y becomes the next x through an allgather; on one GPU only when the in-library exchange is asked for
    # by name (its kernels then deliver into this GPU's own next-x buffer: the form an ncu capture can take)
    iterate = name == "powerlaw" and (world > 1 or args.exchange in ("fused", "push"))

    # ---- build this rank's row block ---------------------------------------------------------------
    lens = global_row_lengths(name, cfg)
    rows = cols = len(lens)
    rows_end = np.cumsum(lens, dtype=np.int64)
    nnz_total = int(rows_end[-1])
    assert nnz_total < 2 ** 31
    part = multi.row_partition(rows_end, world)
    r0, r1 = multi.local_rows(part, rank)
    m = local_block(name, cfg, lens, r0, r1)
    spblas.set_algorithm({"auto": capi.ALG_AUTO, "vector": capi.ALG_VECTOR, "merge": capi.ALG_MERGE,
                          "rowtile": capi.ALG_ROWTILE}[args.alg])
    stream = torch.cuda.Stream()
    spblas.set_stream(stream.cuda_stream)
    st, A = spblas.create_csr(kind, capi.BASE_ZERO, m.nrows, cols, m.rows_start, m.rows_end, m.col, m.val)
    assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
    _, info = spblas.mat_info(A)

    x_lo = 0.0 if name == "stencil27" else -1.0
    x_h = torch.from_numpy(synth.vector(kind, 0, 1, cols * columns, x_lo, 1.0)).pin_memory()
    y0_h = torch.from_numpy(synth.vector(kind, 0, 2, rows * columns)[r0 * columns:r1 * columns].copy()).pin_memory()
    y_h = torch.empty_like(y0_h).pin_memory()
    x_d = x_h.cuda()
    y_d = y0_h.cuda()
    xn_d = torch.empty_like(x_d) if iterate else None
    descr = spblas.descr()
    fused = None
    if iterate and args.exchange != "nccl":
        if args.exchange == "auto":
            args.exchange = "fused" if world >= 4 else "push"   # the library's own default
        fused = multi.FusedExchange(kind, part, rank, world, deliver_after=args.exchange == "push")
        fused.x_tensor().copy_(x_d)
        torch.cuda.synchronize()

    def step_device(xd, yd):
        if op == "mv":
            s = spblas.mv(kind, 0, alpha, A, descr, xd, beta, yd)
        else:
            s = spblas.mm(kind, 0, alpha, A, descr, capi.ROW_MAJOR, xd, columns, columns, beta, yd, columns)
        assert s == capi.SUCCESS, capi.STATUS_NAMES[s]

    def step():
        nonlocal x_d, xn_d
        if fused is not None:
            s = fused.step(alpha, A, beta, y_d)
            assert s == capi.SUCCESS, capi.STATUS_NAMES[s]
            return
        step_device(x_d, y_d)
        if iterate:
            multi.allgather_rows(y_d, xn_d, part)
            x_d, xn_d = xn_d, x_d

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def sum_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([float(v)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = None
    if rank == 0:
        try:
            uuid = torch.cuda.get_device_properties(local_rank).uuid
        except Exception:
            uuid = None
        sampler = ClockSampler(local_rank, uuid)
    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step()
        barrier()
        launches0 = spblas.launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall0 = time.time()
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        e1.synchronize()
        t_wall1 = time.time()
        barrier()
        launches = spblas.launch_count() - launches0
        ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)

        # ---- duration of the dominant kernel, launch by launch, same stream -----------------------
        # The library brackets the kernel with one pair of events per handle; reading them waits for the
        # stream.  Launches are queued back to back, as in the timed region, and the events of the last one
        # of each batch are read, so that no sample comes from a kernel started on an idle GPU.
        spblas.profile_kernel(A, True)
        kms = []
        batches = min(args.steps, 5)
        for b in range(batches):
            for _ in range(max(1, args.steps // batches)):
                step()
            kms.append(spblas.kernel_ms(A))
        spblas.profile_kernel(A, False)
        barrier()
        kernel_ms = max_over_ranks(sum(kms) / len(kms))

        # ---- end to end: host vectors through the same entry point ----------------------------------
        e2e = None
        if not args.no_e2e and not iterate:
            xh, y0h, yh = x_h.numpy(), y0_h.numpy(), y_h.numpy()

            yh[:] = y0h

            # Several GPUs, square matrix: every rank uploads only its own rows of x and the pieces are exchanged
            # over NVLink (alphasparse_cuda_exchange_load_x) instead of every rank pulling all of x over PCIe.
            loader, x_upload = None, "every rank uploads all of x"
            if world > 1 and op == "mv" and rows == cols:
                try:
                    loader = multi.FusedExchange(kind, part, rank, world)
                    x_block_h = x_h[r0:r1].clone().pin_memory()
                    x_upload = "each rank uploads its own rows of x; the pieces cross NVLink to every GPU"
                except Exception as exc:  # e.g. no peer access between these GPUs: keep the plain path
                    print(f"[bench] sharded upload of x unavailable: {exc}", file=sys.stderr)
                    loader = None

            def step_host():  # y is updated in place; with beta = 0.5 it converges, no reset needed
                if loader is not None:
                    s = loader.load_x(x_block_h)
                    assert s == capi.SUCCESS, capi.STATUS_NAMES[s]
                    s = spblas.mv(kind, 0, alpha, A, descr, loader.x_ptr(), beta, yh)
                elif op == "mv":
                    s = spblas.mv(kind, 0, alpha, A, descr, xh, beta, yh)
                else:
                    s = spblas.mm(kind, 0, alpha, A, descr, capi.ROW_MAJOR, xh, columns, columns, beta, yh, columns)
                assert s == capi.SUCCESS
            for _ in range(2):
                step_host()
            barrier()
            n_e2e = max(3, min(args.steps, 10))
            t0 = time.perf_counter()
            e0.record(stream)
            for _ in range(n_e2e):
                step_host()
            e1.record(stream)
            e1.synchronize()
            wall = (time.perf_counter() - t0) / n_e2e * 1e3
            barrier()
            ms_e2e = max_over_ranks(max(e0.elapsed_time(e1) / n_e2e, wall))
            x_bytes = (x_block_h if loader is not None else x_h)
            h2d = x_bytes.numel() * x_bytes.element_size() + (y0_h.numel() * y0_h.element_size() if beta != 0.0 else 0)
            d2h = y_h.numel() * y_h.element_size()
            if loader is not None:
                st_code, code = loader.status()
                assert st_code == capi.SUCCESS and code == 0, f"a bounded wait of the exchange ran out (status {code})"
                loader.destroy()
            # bytes of the whole job: every rank's copies added up
            e2e = (ms_e2e, sum_over_ranks(h2d), sum_over_ranks(d2h), x_upload)
    if sampler:
        sampler.stop()

    nbytes = algorithmic_bytes(cfg, rows, cols, nnz_total)
    fl = flops(cfg, nnz_total)
    # per-launch algorithmic bytes of THIS rank's kernel: its rows' share of A, row_ptr, y plus all of x
    t = TSIZE[kind]
    launch_bytes = m.nnz * (t + 4) + (m.nrows + 1) * 4 + cols * columns * t + m.nrows * columns * t
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    achieved = launch_bytes / (kernel_ms * 1e-3) / 1e9
    # Matrices with unstructured columns: one gather of x per stored element.  The measured gather rate
    # of this GPU gives a floor for the kernel that no SpMV can beat, whatever its HBM traffic.
    gather = None
    if op == "mv" and name != "stencil27":
        rate = spblas.probe_gather_rate(kind, cols)
        floor_ms = m.nnz / rate * 1e3
        gather = {"gathers_per_s": rate, "table_elems": cols, "kernel_floor_ms": floor_ms,
                  "kernel_vs_floor": floor_ms / kernel_ms}

    if rank == 0:
        line = {
            "metric": "csr_spmv_effective_gbs" if op == "mv" else "csr_spmm_effective_gbs",
            "value": nbytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s", "gflops": fl / (ms_step * 1e-3) / 1e9,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32" if kind == "s" else "f64", "data": "synthetic",
            "config": {"workload": name + (" (REDUCED SIZE: development run)" if reduced else ""), "rows": rows,
                       "cols": cols, "nnz": nnz_total, "alpha": alpha, "beta": beta, "columns": columns,
                       "partition": f"nnz-balanced contiguous row blocks over {world} GPU(s), x replicated",
                       "collective": ("none" if not iterate else
                                      "allgather of y into the next x each step: " +
                                      ({"fused": "peer stores from inside the SpMV kernel + flag exchange",
                                        "push": "peer-copy kernel after the SpMV + flag exchange"}[args.exchange]
                                       if fused is not None
                                       else "NCCL all_gather after the SpMV")),
                       "algorithm": ["auto", "vector", "merge", "rowtile"][info.algorithm], "lanes_per_row": info.lanes_per_row,
                       "l2": f"inputs ({nbytes / 1e6:.0f} MB per step) exceed the 126 MB L2; no flush between steps",
                       "algorithmic_bytes_per_step": nbytes},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": NCU_TRAFFIC.get(name) if not reduced and world == 1 else None,
                         "peak_source": peak_src, "kernel_ms": kernel_ms, "bytes_per_launch": launch_bytes,
                         "gather_bound": gather},
            "clocks": sampler.summary(t_wall0, t_wall1) if sampler else None,
        }
        if e2e:
            line["e2e"] = {"value": nbytes / (e2e[0] * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e[0],
                           "h2d_bytes_per_step": int(e2e[1]), "d2h_bytes_per_step": int(e2e[2]), "x_upload": e2e[3]}
        else:
            line["e2e"] = None
        if world == 1 and not args.no_cpu_baseline:
            gbs, gfl, ms, desc = cpu_reference_run(name, cfg, 3, 1)
            line["cpu_baseline"] = dict(value=gbs, unit="GB/s", gflops=gfl, ms_per_step=ms, **desc)
        if world == 1 and not args.no_others and not reduced:
            # The other single-GPU configurations, each in a fresh process, device-resident numbers only:
            # context for the headline above (they are parity-test cases, not separate bench lines).
            others = {}
            for w in sorted(WORKLOADS):
                if w == name:
                    continue
                try:
                    out = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", w, "--steps", "10",
                                          "--warmup", "3", "--no-e2e", "--no-cpu-baseline", "--no-others"],
                                         capture_output=True, text=True, timeout=600)
                    d = json.loads(out.stdout.strip().splitlines()[-1])
                    others[w] = {"value": d["value"], "unit": d["unit"], "ms_per_step": d["ms_per_step"],
                                 "gflops": d["gflops"], "roofline_frac": d["roofline"]["frac"],
                                 "algorithm": d["config"]["algorithm"], "nnz": d["config"]["nnz"]}
                except Exception as exc:  # the headline must not depend on these
                    others[w] = {"error": repr(exc)[:200]}
            line["other_workloads"] = others
        print(json.dumps(line), flush=True)

    if fused is not None:
        st_, code = fused.status()
        assert code == 0, f"a bounded wait of the exchange ran out (status {code})"
        fused.destroy()
    spblas.destroy(A)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
