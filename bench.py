"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c1..c5]

Default workload (c2): CSR SpMV fp32 on a 1,048,576 x 1,048,576 matrix with power-law row lengths
(Zipf s = 1.8, mean about 30, cap 16384, about 30 M non-zeros), y = 1.5 A x + 0.5 y.  All inputs
are seeded synthetic data (no matrix collection is read).  One "step" is one such product.

Our arm prints one JSON line with
  value          GFLOP/s (2 * nnz * N per step) with every input resident in HBM, CUDA-event timed
  e2e            the same metric through the aclsparse C API with x and y in pinned HOST memory:
                 x and y are copied to the device, aclsparseSpMV runs, y is copied back, every step
                 (A stays resident and analysed once, as the API's Preprocess contract intends)
  roofline       algorithmic bytes per launch / measured launch time, against the measured HBM peak
  cpu_baseline   the reference's own CPU golden timed on this host's cores
`--impl reference` times that CPU golden alone (all host threads) and prints the same line shape.

With --gpus N > 1 (launched by torchrun, one rank per GPU) the matrix is cut into N row blocks of
equal non-zero count (strong scaling: the total work is fixed), x is broadcast from rank 0 over
NCCL inside every timed step, y stays sharded; time is the maximum over ranks.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
NOMINAL_HBM_GBS = 8000.0


def measured_peaks() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.dev = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.dev, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.nv = None

    def sample(self):
        if not self.ok:
            return
        nv = self.nv
        try:
            self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.dev, nv.NVML_CLOCK_SM)))
            bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.dev))
            names = {
                "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
                "hw_power_brake": getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80),
            }
            for name, bit in names.items():
                if bits & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def run(self):
        while not self._stop_evt.is_set():
            self.sample()
            time.sleep(0.002)

    def stop(self) -> dict:
        self.sample()
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": int(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def physical_gpu_index(local_index: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_index])
        except Exception:
            return local_index
    return local_index


# ------------------------------------------------------------------------------- workloads

def build_config(name: str, synth):
    return {"c1": synth.config1, "c2": synth.config2, "c3": synth.config3, "c4": synth.config4,
            "c5": synth.config5}[name]()


def describe(name: str, cfg) -> dict:
    A = cfg["A"]
    d = {"workload": cfg["name"], "rows": A.rows, "cols": A.cols, "nnz": A.nnz, "alpha": cfg["alpha"],
         "beta": cfg["beta"], "values": cfg["val"], "output": cfg["out"], "index": "int32",
         "max_row_nnz": int(A.lengths().max())}
    if "B" in cfg:
        d["n"] = int(cfg["B"].shape[1])
    return d


def bytes_and_flops(cfg, synth, rows=None, nnz=None):
    A = cfg["A"]
    rows = A.rows if rows is None else rows
    nnz = A.nnz if nnz is None else nnz
    vb = {"f32": 4, "f16": 2, "bf16": 2}[cfg["val"]]
    ob = {"f32": 4, "f16": 2, "bf16": 2}[cfg["out"]]
    if "B" in cfg:
        n = cfg["B"].shape[1]
        return synth.algorithmic_bytes_spmm(rows, A.cols, nnz, n, vb, ob, cfg["beta"]), 2.0 * nnz * n
    return synth.algorithmic_bytes_spmv(rows, A.cols, nnz, vb, ob, cfg["beta"]), 2.0 * nnz


# ------------------------------------------------------------------------------- CPU arm

class CpuGolden:
    """The reference's CPU golden on a bounded sample of the workload: its leading rows."""

    def __init__(self, cfg, oracle, threads: int):
        self.cfg, self.oracle, self.threads = cfg, oracle, threads
        self.A = cfg["A"]
        self.is_spmm = "B" in cfg
        self.n = cfg["B"].shape[1] if self.is_spmm else 1
        to32 = lambda a: np.ascontiguousarray(a, dtype=np.float32)
        self.dense = to32(cfg["B"] if self.is_spmm else cfg["x"])
        self.out = to32(cfg["C"] if self.is_spmm else cfg["y"])
        self.kind = "port"

    def passes(self, rows: int, reps: int) -> tuple[np.ndarray, int]:
        """(seconds of each of `reps` passes, nnz of the sample); only the golden loop is clocked."""
        S = self.A.row_slice(0, rows)
        c = self.cfg
        fn = self.oracle.time_spmm_f32 if self.is_spmm else self.oracle.time_spmv_f32
        per, self.kind = fn(S.row_ptr, S.col_ind, S.values, self.dense, self.out[:rows], c["alpha"], c["beta"],
                            self.threads, reps)
        return per, S.nnz

    def run(self, rows: int, reps: int) -> tuple[float, int]:
        per, nnz = self.passes(rows, reps)
        return float(per.mean()), nnz

    def rows_for(self, seconds_per_pass: float) -> int:
        """Leading rows whose golden pass takes about `seconds_per_pass` (whole matrix if it fits)."""
        probe = min(self.A.rows, 2048 if self.is_spmm else 65536)
        sec, nnz = self.run(probe, 1)
        per_nnz = max(sec, 1e-7) / max(nnz, 1)
        if per_nnz * self.A.nnz <= seconds_per_pass:
            return self.A.rows
        rows = int(np.searchsorted(self.A.row_ptr, seconds_per_pass / per_nnz))
        return max(min(rows, self.A.rows), 1)

    def report(self, rows: int, reps: int) -> dict:
        sec, nnz = self.run(rows, reps)
        return {"value": 2.0 * nnz * self.n / sec / 1e9, "unit": "GFLOP/s", "cores": self.threads, "kind": self.kind,
                "sample": f"rows [0, {rows}) of {self.A.rows} ({nnz} of {self.A.nnz} nnz), {reps} passes, "
                          f"{sec * 1e3:.2f} ms per pass; 16-bit configurations are timed on fp32-widened values",
                "ms_per_pass": sec * 1e3}


def cpu_baseline(cfg, oracle, threads: int, budget_s: float = 12.0) -> dict:
    """At most about `budget_s` seconds of wall time on all host threads: the whole matrix when a pass is
    short (repeated until about a second has been spent), else its leading rows, 3 passes.  The same loop
    on one thread (the golden as the reference's harness runs it) is timed beside it on a sample a
    tenth as long."""
    g = CpuGolden(cfg, oracle, threads)
    rows = g.rows_for(budget_s / 3)
    sec, _ = g.run(rows, 1)  # also the warm-up pass
    reps = int(min(200, max(3, round(1.0 / max(sec, 1e-4)))))
    rep = g.report(rows, reps)
    one = CpuGolden(cfg, oracle, 1)
    rows1 = one.rows_for(budget_s / 30)
    one.run(rows1, 1)
    r1 = one.report(rows1, 3)
    rep["single_core"] = {"value": r1["value"], "unit": r1["unit"], "sample": r1["sample"]}
    return rep


def reference_arm(args, synth, oracle):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU golden runs once per job: the other ranks have nothing to do
    cfg = build_config(args.config, synth)
    g = CpuGolden(cfg, oracle, oracle.hardware_threads())
    # one step = one golden pass over a bounded sample; K + W steps must end within a few minutes
    per_step = max(0.002, min(4.0, 150.0 / max(args.steps + args.warmup, 1)))
    rows = g.rows_for(per_step)
    t0 = time.perf_counter()
    per, nnz = g.passes(rows, args.warmup + args.steps)  # W untimed passes, then exactly K timed ones
    wall = time.perf_counter() - t0
    sec = float(per[args.warmup:].mean())
    v = 2.0 * nnz * g.n / sec / 1e9
    line = {
        "impl": "reference", "metric": metric_name(cfg), "value": v, "unit": "GFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": dtype_name(cfg), "data": "synthetic (seeded)",
        "config": describe(args.config, cfg),
        "cpu_baseline": {"value": v, "unit": "GFLOP/s", "cores": g.threads, "kind": g.kind,
                         "sample": f"rows [0, {rows}) of {g.A.rows} ({nnz} of {g.A.nnz} nnz) per step; the clock "
                                   f"covers the golden loop only (whole run {wall:.1f} s with argument set-up)"},
        "e2e": {"value": v, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def metric_name(cfg) -> str:
    return "csr_spmm_gflops" if "B" in cfg else "csr_spmv_gflops"


def dtype_name(cfg) -> str:
    return {"f32": "f32", "f16": "f16 values, f32 accumulate", "bf16": "bf16 values, f32 accumulate"}[cfg["val"]]


# ------------------------------------------------------------------------------- GPU arm

# DRAM bytes per launch of the dominant kernel from ncu captures (dram__bytes_read.sum +
# dram__bytes_write.sum); filled from the summaries committed under profiles/.  None = not captured.
NCU_TRAFFIC_BYTES = {
    "c2": 284_459_008,  # both kernels of one product: 147.7 MB (long rows) + 136.8 MB (medium + short rows)
    "c3": 353_516_032,
    "c4": 641_619_968,
}
# What the counters show to be the busy resource where it is not DRAM.
BOUND_NOTES = {
    "c2": "x gathers from uniformly random columns cost one 32-byte L2 sector request each and an SM issues one "
          "request per clock: the medium + short kernel keeps that port 74 % busy (DRAM 25 %); the long rows "
          "(56 % of the non-zeros) gather from x blocks staged in shared memory and run beside it",
    "c4": "B (67 MB) is gathered from L2: 4.48 GB through L2->L1 per product, L2 slices 71 % and L1 78 % busy",
    "c5": "B (1.07 GB) exceeds L2: the row gather is DRAM traffic, about 18.8 GB per product (5.5 x the algorithmic "
          "bytes, which count B once); against that traffic the product runs at about 6.4 TB/s",
}


def dominant_kernels(is_spmm: bool, launches_per_step: float, b_row_bytes: int) -> str:
    """The kernels one step launches, as the library's routing rules give them."""
    if is_spmm:
        if b_row_bytes in (512, 1024):
            return ("SpmmRowStreamKernel (rows <= 1024 nnz)" +
                    (" + SpmmFastKernel (segment CTAs of longer rows)" if launches_per_step > 1 else ""))
        return "SpmmFastKernel"
    if launches_per_step > 1:
        return "SpmvLongBlockKernel | SpmvLongListKernel (side stream) + SpmvMediumShortKernel"
    return "SpmvShortRowsKernel | SpmvMediumShortKernel"


class SpMVOpStep:
    """The same product through the SpMVOp plan API (compensated row sums), Z aliasing Y; `step` like the
    sharded operators so that the timing loops do not care."""

    def __init__(self, d_rp, d_ci, d_v, cols, x, y, alg):
        from ops_sparse_b200 import api
        self.h = api.Handle()
        self.A = api.CsrMatrix(d_rp, d_ci, d_v, d_rp.numel() - 1, cols)
        self.x, self.y = api.DnVec(x), api.DnVec(y)
        self.plan = api.SpMVOpPlan(self.h, self.A, self.x, self.y, self.y, alg=alg)

    def step(self, alpha, beta, broadcast=False):
        self.plan.run(self.x, self.y, self.y, alpha, beta)

    def close(self):
        self.plan.close()
        self.h.close()


def torch_dtype(kind: str):
    import torch
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[kind]


def gpu_arm(args, synth, oracle):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU implementation")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    from ops_sparse_b200 import mg
    pkg = entry.load_package()

    cfg = build_config(args.config, synth)  # every rank draws the same matrix from the same seed
    A = cfg["A"]
    is_spmm = "B" in cfg
    alpha, beta = cfg["alpha"], cfg["beta"]
    vt, ot = torch_dtype(cfg["val"]), torch_dtype(cfg["out"])
    cuts = mg.partition_rows(A.row_ptr, world)
    r0, r1 = mg.local_rows(cuts, rank)
    rp, ci, v = mg.slice_csr(A.row_ptr, A.col_ind, A.values, r0, r1)
    d_rp, d_ci = torch.from_numpy(rp).to(dev), torch.from_numpy(np.ascontiguousarray(ci)).to(dev)
    d_v = torch.from_numpy(np.ascontiguousarray(v)).to(dev).to(vt)
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    if is_spmm:
        n = cfg["B"].shape[1]
        dense_h = pin(cfg["B"]).to(vt) if False else torch.from_numpy(cfg["B"]).to(vt).pin_memory()
        out_h = torch.from_numpy(cfg["C"][r0:r1]).to(ot).pin_memory()
        dense = dense_h.to(dev) if rank == 0 else torch.zeros_like(dense_h, device=dev)
        out = out_h.to(dev)
        op = mg.ShardedSpmm(d_rp, d_ci, d_v, A.cols, dense, out)
    else:
        n = 1
        dense_h = torch.from_numpy(cfg["x"]).to(vt).pin_memory()
        out_h = torch.from_numpy(cfg["y"][r0:r1]).to(ot).pin_memory()
        dense = dense_h.to(dev) if rank == 0 else torch.zeros_like(dense_h, device=dev)
        out = out_h.to(dev)
        op = mg.ShardedSpmv(d_rp, d_ci, d_v, A.cols, dense, out)
        if args.api != "spmv":
            if cfg["val"] != "f32" or world > 1:
                raise SystemExit("--api spmvop-alg1 / spmvop-alg2: fp32 SpMV configurations (c1, c2), one GPU")
            op.close()
            op = SpMVOpStep(d_rp, d_ci, d_v, A.cols, dense, out, 2 if args.api == "spmvop-alg2" else 1)
    result_h = torch.empty_like(out_h).pin_memory()
    bcast = world > 1

    def step():
        op.step(alpha, beta, broadcast=bcast)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    K, W = args.steps, args.warmup
    for _ in range(W):
        step()
    barrier()

    # ---- timed region: exactly K steps, inputs resident, CUDA events on the launching stream
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    count = pkg.lib().b200sp_kernel_launches
    count.restype = ctypes.c_ulonglong
    launches_before = count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    launches = int(count() - launches_before)  # this rank's kernels inside the timed region
    sampler.sample()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    barrier()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = total_ms / K

    # ---- compute-only steps (no broadcast): launch duration for the roofline.  A step is one
    # launch of the dominant kernel (plus, for the binned SpMV, the long-row kernel running beside
    # it on a side stream), so the duration is the event-bracketed region divided by the steps.
    KL = min(K, 200)
    barrier()
    e0.record()
    for _ in range(KL):
        op.step(alpha, beta, broadcast=False)
    e1.record()
    torch.cuda.synchronize()
    launch_ms_mean = max_over_ranks(e0.elapsed_time(e1) / KL)

    # ---- end to end: host buffers in, host result out, every step.  The package's host-operand API cuts the
    # rows into panels so that the copies of one panel overlap the product of another.
    from ops_sparse_b200 import hostio
    KE = min(K, 200)
    pipe = hostio.HostOperandProduct(rp, d_ci, d_v, A.cols, dense, out, panels=args.e2e_panels)
    graph = pipe.capture(dense_h, out_h, result_h, alpha, beta) if (world == 1 and not args.no_graph) else None

    def e2e_step():
        if graph is not None:
            graph.replay()  # the recorded step: x / B up, per panel y / C up -> product -> result down
        else:
            pipe.step(dense_h, out_h, result_h, alpha, beta, upload_dense=(rank == 0))

    for _ in range(3):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(KE):
        e2e_step()
        torch.cuda.synchronize()  # the caller needs the result before the next step
    e1.record()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1)) / KE
    pipe.close()
    # bytes this rank moves per step (rank 0 also uploads x / B; y / C goes up only when beta != 0 reads it)
    out_bytes = (r1 - r0) * n * out_h.element_size()
    h2d = (dense_h.numel() * dense_h.element_size() if rank == 0 else 0) + (out_bytes if beta != 0 else 0)
    d2h = out_bytes

    # ---- spot check of the last end-to-end result against the CPU oracle (first local rows)
    check_rows = min(r1 - r0, 20000 if not is_spmm else 512)
    S = A.row_slice(r0, r0 + check_rows)
    got = result_h[:check_rows].to(torch.float32).numpy().astype(np.float64)
    if is_spmm:
        Bw = dense_h.to(torch.float32).numpy()
        C0 = out_h[:check_rows].to(torch.float32).numpy()
        vw = torch.from_numpy(S.values).to(vt).to(torch.float32).numpy()
        gold = oracle.spmm_f32(S.row_ptr, S.col_ind, vw, Bw, C0, alpha, beta)
        scale = abs(alpha) * oracle.spmm_abs_sum(S.row_ptr, S.col_ind, vw, Bw) + np.abs(beta * C0)
    else:
        xw = dense_h.to(torch.float32).numpy()
        y0 = out_h[:check_rows].to(torch.float32).numpy()
        vw = torch.from_numpy(S.values).to(vt).to(torch.float32).numpy()
        gold = oracle.spmv(S.row_ptr, S.col_ind, vw, xw, y0, alpha, beta)
        scale = abs(alpha) * oracle.spmv_abs_rowsum(S.row_ptr, S.col_ind, vw, xw) + np.abs(beta * y0)
    tol = 1e-5 if cfg["val"] == "f32" else 2e-3
    parity_ok = bool(np.all(np.abs(got - gold) <= tol * scale + 1e-30))

    alg_bytes, flops = bytes_and_flops(cfg, synth)
    my_bytes, _ = bytes_and_flops(cfg, synth, rows=r1 - r0, nnz=int(ci.size))
    peak, peak_src = measured_peaks()
    achieved = my_bytes / (launch_ms_mean * 1e-3) / 1e9
    value = flops / (ms_per_step * 1e-3) / 1e9

    base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(cfg, oracle, oracle.hardware_threads())

    if rank == 0:
        line = {
            "metric": metric_name(cfg), "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": dtype_name(cfg), "data": "synthetic (seeded)",
            "config": describe(args.config, cfg) | {
                "parallelism": f"rows split by nnz over {world} GPU(s); x/B broadcast from rank 0 inside every step"
                if world > 1 else "single GPU",
                "l2_policy": "no flush between steps: A (col_ind + values) alone is larger than L2 "
                             f"({(4 + d_v.element_size()) * A.nnz / 1e6:.0f} MB vs 126 MB); x / B may stay cached"
                if (4 + d_v.element_size()) * A.nnz > L2_BYTES else
                "inputs fit in L2: this configuration is launch-latency bound, bandwidth fractions are not meaningful",
                "analysis": "aclsparse*Preprocess once, outside the timed region",
                "api": args.api,
            },
            "effective_gbs": alg_bytes / (ms_per_step * 1e-3) / 1e9,
            "algorithmic_bytes_per_step": alg_bytes,
            "roofline": {
                "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS, "peak_source": peak_src,
                "kernel": ("SpmvOpLongRowsKernel + SpmvOpRowsKernel per length class" if args.api == "spmvop-alg2"
                           else "SpmvOpRowsKernel" if args.api == "spmvop-alg1"
                           else dominant_kernels(is_spmm, launches / K, n * dense.element_size() if is_spmm else 0)),
                "launch_ms_mean": launch_ms_mean,
                "algorithmic_bytes_per_launch": my_bytes, "traffic": NCU_TRAFFIC_BYTES.get(args.config) if (world == 1 and args.api == "spmv") else None,
                "note": BOUND_NOTES.get(args.config) if args.api == "spmv" else None,
            },
            "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": KE,
                    "row_panels": args.e2e_panels, "cuda_graph": graph is not None},
            "compute_only": {"value": flops / (launch_ms_mean * 1e-3) / 1e9, "unit": "GFLOP/s",
                             "ms_per_step": launch_ms_mean,
                             "broadcast_ms_per_step": max(ms_per_step - launch_ms_mean, 0.0) if world > 1 else 0.0,
                             "note": "max-over-ranks mean product time without the broadcast (an event after "
                                     "every single step would add its own 15-30 us to a 95 us step, so no "
                                     "per-step spread is reported)"},
            "gpu_launches": launches * world, "kernels_per_step": launches / K, "clocks": clocks, "parity_spot_check": parity_ok,
        }
        if base is not None:
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "single_core")
                                    if k in base}
        print(json.dumps(line))
    op.close()
    if world > 1:
        dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit("parity spot check against the CPU oracle failed")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=["c1", "c2", "c3", "c4", "c5"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU golden timing leg")
    ap.add_argument("--api", default="spmv", choices=["spmv", "spmvop-alg1", "spmvop-alg2"],
                    help="resident-operand legs through aclsparseSpMV (default) or the SpMVOp plan API")
    ap.add_argument("--no-graph", action="store_true", help="end-to-end leg: issue every step's operations one by one")
    ap.add_argument("--e2e-panels", type=int, default=4,
                    help="row panels the end-to-end leg pipelines its host copies over (1 = copy, compute, copy)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    entry.load_package()
    from ops_sparse_b200 import synth
    entry._load("b200sp_build_oracle", ROOT / "oracle" / "build_oracle.py").build_oracle()
    oracle = entry.load_oracle()
    if args.impl == "reference":
        reference_arm(args, synth, oracle)
    else:
        gpu_arm(args, synth, oracle)


if __name__ == "__main__":
    main()
