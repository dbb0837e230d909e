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
scaling is "strong"; the default run then also measures, in the same process group, the iterated
power-law SpMV whose y becomes the next x on every GPU (other_workloads.powerlaw_iterated: the
allgather done inside the SpMV kernels, by a peer-copy kernel, and by NCCL; checked against the
oracle).  `--impl reference` times the reference's own OpenMP CPU kernel on the same workload.
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

FALLBACK_HBM_GBS = 6650.0  # B200 copy bandwidth used only when MEASURED_PEAKS.json is absent

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


def gather_rate(elem_bytes, table_elems, stream_ptr, gathers=1 << 27):
    """Random single-element gathers per second this GPU sustains from a table of that many elements: the probe
    built from bench_gather_probe.cu beside this file (python -m alsparse_b200.build)."""
    import ctypes as C
    path = os.path.join(ROOT, "libbench_gather_probe.so")
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: run `python -m alsparse_b200.build`")
    lib = C.CDLL(path, mode=C.RTLD_LOCAL)
    lib.bench_gather_rate.restype = C.c_int
    lib.bench_gather_rate.argtypes = [C.c_int, C.c_longlong, C.c_longlong, C.c_void_p, C.POINTER(C.c_double)]
    rate = C.c_double()
    err = lib.bench_gather_rate(elem_bytes, table_elems, gathers, stream_ptr, C.byref(rate))
    assert err == 0, f"gather probe failed (cudaError {err})"
    return rate.value


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
# what both arms say about the workload (identical dictionaries: the two lines describe the same job)
# ------------------------------------------------------------------------------------------------
def workload_config(name, cfg, rows, cols, nnz, reduced):
    nbytes = algorithmic_bytes(cfg, rows, cols, nnz)
    return {"workload": name + (" (REDUCED SIZE: development run)" if reduced else ""), "rows": rows, "cols": cols,
            "nnz": nnz, "alpha": cfg["alpha"], "beta": cfg["beta"], "columns": cfg.get("columns", 1),
            "l2": f"inputs ({nbytes / 1e6:.0f} MB per step) exceed the 126 MB L2; no flush between steps",
            "algorithmic_bytes_per_step": nbytes}


def metric_name(cfg):
    return "csr_spmv_effective_gbs" if cfg["op"] == "mv" else "csr_spmm_effective_gbs"


# ------------------------------------------------------------------------------------------------
# the reference arm / CPU baseline
# ------------------------------------------------------------------------------------------------
def cpu_reference_time(cfg, m, cols, x, y, steps, warmup):
    """Times the reference's own OpenMP kernel (oracle/_ref) -- or the oracle port of it when those objects are
    absent -- on the WHOLE matrix `m` with all host threads.  y is updated in place, as a caller's would be.
    Returns (ms per call, descriptor dict)."""
    import oracle
    kind, columns = cfg["kind"], cfg.get("columns", 1)
    use_ref = oracle.ref_available()
    threads = oracle.ref_cores() if use_ref else oracle.max_threads()
    A = oracle.RefCsr.from_csr(kind, 0, m.nrows, cols, m.rows_start, m.rows_end, m.col, m.val) if use_ref else None

    def step():
        if cfg["op"] == "mv":
            if use_ref:
                A.gemv(cfg["alpha"], x, cfg["beta"], y, omp_threads=threads)
            else:
                oracle.gemv(kind, m.rows_start, m.rows_end, m.col, m.val, cfg["alpha"], x, cfg["beta"], y, threads=threads)
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
    desc = {"kind": "reference" if use_ref else "port", "cores": threads,
            "sample": f"the whole matrix ({m.nrows} rows, {m.nnz} stored elements); {steps} timed calls after {warmup} warm-up"}
    return dt * 1e3, desc


def run_reference_arm(args, name, cfg, reduced, rank):
    """The reference's CPU implementation of the path on this box's host cores, same workload as the GPU arm.
    Under torchrun rank 0 alone works."""
    if rank != 0:
        return
    from alsparse_b200 import synth
    kind, columns = cfg["kind"], cfg.get("columns", 1)
    lens = global_row_lengths(name, cfg)
    rows = cols = len(lens)
    m = local_block(name, cfg, lens, 0, rows)
    x = synth.vector(kind, 0, 1, cols * columns, 0.0 if name == "stencil27" else -1.0, 1.0)
    y = synth.vector(kind, 0, 2, rows * columns)
    warmup = max(args.warmup, 1)
    ms, desc = cpu_reference_time(cfg, m, cols, x, y, args.steps, warmup)
    nbytes = algorithmic_bytes(cfg, rows, cols, m.nnz)
    gbs = nbytes / (ms * 1e-3) / 1e9
    line = {"impl": "reference", "metric": metric_name(cfg), "value": gbs, "unit": "GB/s",
            "gflops": flops(cfg, m.nnz) / (ms * 1e-3) / 1e9, "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32" if kind == "s" else "f64", "data": "synthetic",
            "config": workload_config(name, cfg, rows, cols, m.nnz, reduced),
            "cpu_baseline": dict(value=gbs, unit="GB/s", **desc),
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# ncu traffic figures (profiles/ncu_traffic.json): reported only for the kernel they were captured on
# ------------------------------------------------------------------------------------------------
def ncu_traffic(name, kernel, reduced, world):
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    if reduced or world != 1 or not os.path.exists(path):
        return None, None
    rec = json.load(open(path)).get(name)
    if not isinstance(rec, dict) or rec.get("kernel") != kernel:
        return None, (f"no capture of {kernel} (profiles/ncu_traffic.json has {rec.get('kernel')})"
                      if isinstance(rec, dict) else None)
    how = "scaled from a capture at reduced size, see the summary" if rec.get("scaled") else "full-size capture"
    return rec["dram_bytes_per_launch"], f"ncu: {rec['summary']} ({rec['kernel']}, at commit {rec['commit']}; {how})"


def sampled_rows(m, rng, n_random):
    """Sorted distinct local row numbers (first, last, the eight longest, random ones) and those rows as a small
    CSR with local offsets and the matrix's own columns."""
    lens = np.diff(m.ptr)
    longest = np.argpartition(lens, -min(8, len(lens)))[-8:]
    pick = np.unique(np.concatenate([rng.integers(0, m.nrows, n_random), [0, m.nrows - 1], longest]))
    ptr = np.concatenate([[0], np.cumsum(lens[pick])]).astype(np.int32)
    idx = np.concatenate([np.arange(m.ptr[r], m.ptr[r + 1], dtype=np.int64) for r in pick])
    return pick, ptr, m.col[idx], m.val[idx]


# ------------------------------------------------------------------------------------------------
# iterated power-law SpMV over several GPUs: y of every step becomes the next x on all GPUs
# ------------------------------------------------------------------------------------------------
def measure_iterated(args, rank, world, stream, iterations=50):
    """x_{t+1} = A x_t on the power-law matrix, rows split over the GPUs, the allgather of y done three ways:
    inside the SpMV kernels (peer stores), by one peer-copy kernel after them, and by a NCCL all_gather.
    Every way is checked on its first step against the oracle (sampled rows of this rank, x0 known) and timed
    over `iterations` steps; the time of a step is the maximum over ranks."""
    import torch
    import torch.distributed as dist

    import oracle
    from alsparse_b200 import capi, multi, spblas, synth

    name = "powerlaw"
    cfg = dict(WORKLOADS[name])
    if args.iter_rows_log2:
        cfg["rows_log2"] = args.iter_rows_log2
    kind, tol = cfg["kind"], 1e-12
    lens = global_row_lengths(name, cfg)
    rows = cols = len(lens)
    rows_end = np.cumsum(lens, dtype=np.int64)
    nnz_total = int(rows_end[-1])
    part = multi.row_partition(rows_end, world)
    r0, r1 = multi.local_rows(part, rank)
    m = local_block(name, cfg, lens, r0, r1)
    st, A = spblas.create_csr(kind, capi.BASE_ZERO, m.nrows, cols, m.rows_start, m.rows_end, m.col, m.val)
    assert st == capi.SUCCESS, (capi.STATUS_NAMES[st], spblas.last_error())
    x0 = synth.vector(kind, 0, 1, cols)
    x0_d = torch.from_numpy(x0).cuda()
    y_d = torch.zeros(m.nrows, dtype=torch.float64, device="cuda")
    xa, xb = torch.empty_like(x0_d), torch.empty_like(x0_d)
    descr = spblas.descr()

    # the comparand of step 1: this rank's sampled rows through the oracle's plain kernel
    pick, sptr, scol, sval = sampled_rows(m, np.random.default_rng(100 + rank), max(64, 4000 // world)) if m.nrows else \
        (np.zeros(0, np.int64), np.zeros(1, np.int32), m.col[:0], m.val[:0])
    y_ref = oracle.gemv(kind, sptr[:-1], sptr[1:], scol, sval, 1.0, x0, 0.0, np.zeros(len(pick)))
    prod = np.abs(sval * x0[scol])
    scale = np.add.reduceat(np.concatenate([prod, [0.0]]), np.minimum(sptr[:-1], len(prod))) * (np.diff(sptr) > 0)

    def all_max(v):
        t = torch.tensor([float(v)], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    out = {"iterations": iterations, "rows": rows, "nnz": nnz_total, "dtype": "f64", "alpha": 1.0, "beta": 0.0,
           "rows_of_rank0": int(part[1] - part[0]),
           "nvlink_bytes_per_gpu_per_iteration": {"sent": int(m.nrows) * 8 * (world - 1), "received": int(rows - m.nrows) * 8},
           "parity": {"against": "oracle plain kernel, sampled rows of every rank, step 1 (x0 known)", "tolerance": tol,
                      "rows_checked_on_rank0": int(len(pick))}, "modes": {}}
    nbytes = algorithmic_bytes(cfg, rows, cols, nnz_total)
    collectives = {"fused": "peer stores from inside the SpMV kernels + flag exchange",
                   "push": "one peer-copy kernel after the SpMV + flag exchange",
                   "nccl": "torch.distributed all_gather (NCCL) after the SpMV"}
    with torch.cuda.stream(stream):
        for mode in ("fused", "push", "nccl"):
            ex = None
            cur, nxt = xa, xb
            if mode != "nccl":
                ex = multi.FusedExchange(kind, part, rank, world, deliver_after=(mode == "push"))
                ex.x_tensor().copy_(x0_d)
            else:
                cur.copy_(x0_d)
            barrier()

            def step():
                nonlocal cur, nxt
                if ex is not None:
                    s = ex.step(1.0, A, 0.0, y_d)
                else:
                    s = spblas.mv(kind, 0, 1.0, A, descr, cur, 0.0, y_d)
                    multi.allgather_rows(y_d, nxt, part)
                    cur, nxt = nxt, cur
                assert s == capi.SUCCESS, capi.STATUS_NAMES[s]

            step()
            barrier()
            y1 = y_d.cpu().numpy()
            x1 = (ex.x_tensor() if ex is not None else cur)
            err = np.abs(y1[pick] - y_ref)
            rows_ok = bool((err <= tol * scale + 1e-300).all()) if len(pick) else True
            worst = float(np.max(err / np.maximum(tol * scale, 1e-300))) if len(pick) else 0.0
            own_ok = bool(torch.equal(x1[r0:r1], y_d))                   # my rows arrived in my own next x
            # every rank must hold the same gathered vector: compare a checksum of it across ranks
            chk = float(x1.double().abs().sum().item())
            same = all_max(chk) == -all_max(-chk)
            ok = all_max(0.0 if (rows_ok and own_ok and same) else 1.0) == 0.0
            for _ in range(max(args.warmup, 3)):
                step()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(iterations):
                step()
            e1.record(stream)
            e1.synchronize()
            barrier()
            ms = all_max(e0.elapsed_time(e1) / iterations)
            status = 0
            if ex is not None:
                st_, status = ex.status()
                ex.destroy()
            status = int(all_max(status))
            finite = all_max(0.0 if bool(torch.isfinite(y_d).all()) else 1.0) == 0.0
            out["modes"][mode] = {"ms_per_iteration": ms, "value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
                                  "collective": collectives[mode], "parity_ok": ok,
                                  "worst_row_error_over_tolerance": all_max(worst), "exchange_status": status,
                                  "finite_after_all_iterations": finite}
        # the product alone on the same handle (x fixed, nothing exchanged): what the three modes add to it
        xa.copy_(x0_d)
        for _ in range(max(args.warmup, 3)):
            assert spblas.mv(kind, 0, 1.0, A, descr, xa, 0.0, y_d) == capi.SUCCESS
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iterations):
            spblas.mv(kind, 0, 1.0, A, descr, xa, 0.0, y_d)
        e1.record(stream)
        e1.synchronize()
        barrier()
        out["product_without_exchange_ms"] = all_max(e0.elapsed_time(e1) / iterations)
    out["parity"]["ok"] = all(v["parity_ok"] and v["exchange_status"] == 0 for v in out["modes"].values())
    out["fused_vs_nccl"] = out["modes"]["nccl"]["ms_per_iteration"] / out["modes"]["fused"]["ms_per_iteration"]
    spblas.destroy(A)
    return out


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
    ap.add_argument("--iter-rows-log2", type=int, default=None,
                    help="shrink the iterated power-law matrix of multi-GPU runs (development only)")
    ap.add_argument("--alg", default="auto", choices=["auto", "vector", "merge", "rowtile"])
    ap.add_argument("--exchange", default="auto", choices=["auto", "fused", "push", "nccl"],
                    help="iterated workload with several GPUs: y reaches the next x from inside the SpMV kernels "
                         "over peer memory (fused), by one peer-copy kernel after them (push), "
                         "whichever of the two the library prefers for this many GPUs (auto) or by a NCCL allgather (nccl)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cold", action="store_true", help="skip the cold-L2 variant")
    ap.add_argument("--no-others", action="store_true",
                    help="do not append the other workloads (N=1: the three other configurations, each in a fresh "
                         "process; N>1: the iterated power-law SpMV with its allgather, in this process group)")
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
        run_reference_arm(args, name, cfg, reduced, rank)
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
    x_np = synth.vector(kind, 0, 1, cols * columns, x_lo, 1.0)
    y0_np = synth.vector(kind, 0, 2, rows * columns)[r0 * columns:r1 * columns].copy()
    x_h = torch.from_numpy(x_np).pin_memory()
    y0_h = torch.from_numpy(y0_np).pin_memory()
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

        # ---- duration of the product's kernels, launch by launch, same stream -----------------------
        # The library brackets the kernels of the product with one pair of events per handle (one kernel for
        # the vector and row-tile families; for a skewed matrix the span from the first to the last kernel of
        # the product, since two large kernels share the work); reading them waits for the stream.  Launches
        # are queued back to back, as in the timed region, and the events of the last one of each batch are
        # read, so that no sample comes from a kernel started on an idle GPU.
        spblas.profile_kernel(A, True)
        kms = []
        batches = min(args.steps, 5)
        for b in range(batches):
            for _ in range(max(1, args.steps // batches)):
                step()
            kms.append(spblas.kernel_ms(A))
        spblas.profile_kernel(A, False)
        barrier()
        kernel_ms = max_over_ranks(float(np.median(kms)))  # median: one sample taken beside a clock sample or a host hiccup must not move it

        # ---- cold L2: 256 MB are overwritten on the device before every timed step ---------------------
        cold = None
        if not args.no_cold and not iterate:
            flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
            n_cold = max(3, min(args.steps, 10))
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_cold)]
            for a, b in pairs:
                flush.fill_(1)
                a.record(stream)
                step()
                b.record(stream)
            torch.cuda.synchronize()
            cold_ms = max_over_ranks(statistics.median(a.elapsed_time(b) for a, b in pairs))
            del flush
            barrier()
            cold = cold_ms

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

            phase = {"load_x_ms": 0.0, "product_ms": 0.0}

            def step_host(timed=False):  # y is updated in place; with beta = 0.5 it converges, no reset needed
                t0 = time.perf_counter()
                if loader is not None:
                    s = loader.load_x(x_block_h)
                    assert s == capi.SUCCESS, capi.STATUS_NAMES[s]
                    if timed:
                        torch.cuda.synchronize()
                        phase["load_x_ms"] += (time.perf_counter() - t0) * 1e3
                        t0 = time.perf_counter()
                    s = spblas.mv(kind, 0, alpha, A, descr, loader.x_ptr(), beta, yh)
                elif op == "mv":
                    s = spblas.mv(kind, 0, alpha, A, descr, xh, beta, yh)
                else:
                    s = spblas.mm(kind, 0, alpha, A, descr, capi.ROW_MAJOR, xh, columns, columns, beta, yh, columns)
                assert s == capi.SUCCESS
                if timed:
                    phase["product_ms"] += (time.perf_counter() - t0) * 1e3
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
            # the same steps once more with a host-side wait between their two halves: where the time goes
            # (outside the timed region; the extra wait makes these steps slower than the timed ones)
            breakdown = None
            if loader is not None:
                for _ in range(3):
                    step_host(timed=True)
                barrier()
                breakdown = {"x_piece_upload_and_nvlink_exchange_ms": max_over_ranks(phase["load_x_ms"] / 3),
                             "product_with_y_copies_ms": max_over_ranks(phase["product_ms"] / 3),
                             "note": "measured in separate steps with a wait between the two halves (max over ranks)"}
            x_bytes = (x_block_h if loader is not None else x_h)
            h2d = x_bytes.numel() * x_bytes.element_size() + (y0_h.numel() * y0_h.element_size() if beta != 0.0 else 0)
            d2h = y_h.numel() * y_h.element_size()
            # What the host side of the box allows for these copies alone: every rank moves the bytes of one step
            # (same pinned buffers, inbound and outbound on two streams at once, no kernel), all ranks at the same
            # time.  With several GPUs the ranks share the host's memory and PCIe root, so this floor does not
            # shrink like the per-GPU byte count does.
            up, down = torch.cuda.Stream(), torch.cuda.Stream()
            dev_in = [torch.empty_like(x_bytes, device="cuda"), torch.empty_like(y0_h, device="cuda")]
            dev_out = torch.empty_like(y_h, device="cuda")

            def copies():
                with torch.cuda.stream(up):
                    dev_in[0].copy_(x_bytes, non_blocking=True)
                    if beta != 0.0:
                        dev_in[1].copy_(y0_h, non_blocking=True)
                with torch.cuda.stream(down):
                    y_h.copy_(dev_out, non_blocking=True)
                up.synchronize()
                down.synchronize()
            for _ in range(2):
                copies()
            barrier()
            t0 = time.perf_counter()
            for _ in range(5):
                copies()
            copy_floor = max_over_ranks((time.perf_counter() - t0) / 5 * 1e3)
            del dev_in, dev_out
            barrier()
            if loader is not None:
                st_code, code = loader.status()
                assert st_code == capi.SUCCESS and code == 0, f"a bounded wait of the exchange ran out (status {code})"
                loader.destroy()
            # bytes of the whole job: every rank's copies added up
            e2e = (ms_e2e, sum_over_ranks(h2d), sum_over_ranks(d2h), x_upload, breakdown, copy_floor)
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
    # of this GPU gives a floor for a kernel that gathers every element of x from L2, whatever its HBM traffic.
    gather = None
    if op == "mv" and name != "stencil27":
        rate = gather_rate(TSIZE[kind], cols, stream.cuda_stream)
        through_l2 = m.nnz - int(info.band_elements)
        floor_ms = through_l2 / rate * 1e3
        gather = {"gathers_per_s": rate, "table_elems": cols, "elements_gathered_from_l2": through_l2,
                  "elements_gathered_from_shared_memory": int(info.band_elements),
                  "kernel_floor_ms": floor_ms, "kernel_vs_floor": floor_ms / kernel_ms}

    algorithm = ["auto", "vector", "merge", "rowtile"][info.algorithm]
    kernel = {"vector": f"spmv_vector_kernel lanes={info.lanes_per_row}", "rowtile": "spmv_rowtile_kernel",
              "merge": ("row bins: spmv_short_kernel + spmv_rowlist_kernel x3" if info.binned else "spmv_merge_kernel") +
                       (" + spmv_band_packed_kernel + spmv_band_reduce_kernel" if info.band_rows else "")}[algorithm] \
        if op == "mv" else "spmm_row_kernel"
    if rank == 0:
        traffic, traffic_src = ncu_traffic(name, kernel, reduced, world)
        line = {
            "metric": metric_name(cfg),
            "value": nbytes / (ms_step * 1e-3) / 1e9, "unit": "GB/s", "gflops": fl / (ms_step * 1e-3) / 1e9,
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32" if kind == "s" else "f64", "data": "synthetic",
            "config": workload_config(name, cfg, rows, cols, nnz_total, reduced),
            "execution": {"partition": f"nnz-balanced contiguous row blocks over {world} GPU(s), x replicated",
                          "collective": ("none" if not iterate else
                                         "allgather of y into the next x each step: " +
                                         ({"fused": "peer stores from inside the SpMV kernel + flag exchange",
                                           "push": "peer-copy kernel after the SpMV + flag exchange"}[args.exchange]
                                          if fused is not None
                                          else "NCCL all_gather after the SpMV")),
                          "algorithm": algorithm, "lanes_per_row": info.lanes_per_row, "kernel": kernel,
                          "rows_in_column_band_kernel": info.band_rows, "elements_in_column_band_kernel": int(info.band_elements)},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_source": traffic_src,
                         "peak_source": peak_src, "kernel_ms": kernel_ms, "bytes_per_launch": launch_bytes,
                         "gather_bound": gather},
            "clocks": sampler.summary(t_wall0, t_wall1) if sampler else None,
        }
        if cold is not None:
            line["cold_l2"] = {"ms_per_step": cold, "value": nbytes / (cold * 1e-3) / 1e9, "unit": "GB/s",
                               "how": "256 MB overwritten on the device before every timed step; median of the steps"}
        if e2e:
            line["e2e"] = {"value": nbytes / (e2e[0] * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e[0],
                           "h2d_bytes_per_step": int(e2e[1]), "d2h_bytes_per_step": int(e2e[2]), "x_upload": e2e[3]}
            if e2e[4]:
                line["e2e"]["phases"] = e2e[4]
            line["e2e"]["copies_alone_ms"] = e2e[5]
            line["e2e"]["copies_alone_note"] = ("the same host<->device bytes moved by plain copies on two streams, all "
                                                "ranks at once, no kernel: the share of the step that belongs to the "
                                                "host's memory and PCIe links")
        else:
            line["e2e"] = None
        if world == 1 and not args.no_cpu_baseline:
            # the reference's OpenMP kernel on this box's host cores, the whole matrix, the same vectors
            ms_cpu, desc = cpu_reference_time(cfg, m, cols, x_np, y0_np.copy(), 3, 1)
            line["cpu_baseline"] = dict(value=nbytes / (ms_cpu * 1e-3) / 1e9, unit="GB/s",
                                        gflops=fl / (ms_cpu * 1e-3) / 1e9, ms_per_step=ms_cpu, **desc)

    if fused is not None:
        st_, code = fused.status()
        assert code == 0, f"a bounded wait of the exchange ran out (status {code})"
        fused.destroy()
    spblas.destroy(A)
    del x_d, y_d, xn_d
    torch.cuda.empty_cache()

    others = None
    if world > 1 and not args.no_others and not reduced and name == "uniform16":
        # the iterated configuration, in the same process group: SpMV fused with its allgather against NCCL
        try:
            others = {"powerlaw_iterated": measure_iterated(args, rank, world, stream)}
        except Exception as exc:  # the headline must not depend on it; all ranks fail or pass together
            others = {"powerlaw_iterated": {"error": repr(exc)[:300]}}
    if rank == 0:
        if world == 1 and not args.no_others and not reduced:
            # The other single-GPU configurations, each in a fresh process with its own end-to-end, CPU-baseline
            # and roofline figures: context for the headline above (parity-test cases, not separate bench lines).
            others = {}
            for w in sorted(WORKLOADS):
                if w == name:
                    continue
                try:
                    out = subprocess.run([sys.executable, os.path.abspath(__file__), "--workload", w, "--steps", "10",
                                          "--warmup", "3", "--no-others"], capture_output=True, text=True, timeout=900)
                    d = json.loads(out.stdout.strip().splitlines()[-1])
                    others[w] = {k: d.get(k) for k in ("value", "unit", "ms_per_step", "gflops", "dtype", "config",
                                                        "execution", "roofline", "e2e", "cpu_baseline", "cold_l2",
                                                        "gpu_launches")}
                except Exception as exc:  # the headline must not depend on these
                    others[w] = {"error": repr(exc)[:200]}
        if others is not None:
            line["other_workloads"] = others
        print(json.dumps(line), flush=True)

    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
