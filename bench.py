"""Benchmark of the CSR SpMV / SpMM hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c2] [--configs c1,...]

Headline workload (c2): CSR SpMV fp32 on a 1,048,576 x 1,048,576 matrix with power-law row lengths
(Zipf s = 1.8, mean about 30, cap 16384, about 30 M non-zeros), y = 1.5 A x + 0.5 y.  All inputs
are seeded synthetic data (no matrix collection is read).  One "step" is one such product.

Our arm prints ONE JSON line.  Its top-level keys describe the headline configuration:
  value          GFLOP/s (2 * nnz * N per step) with every input resident in HBM, CUDA-event timed
  e2e            the same metric through the aclsparse C API with x / B and y / C in pinned HOST memory:
                 copied to the device, multiplied, copied back, every step (A stays resident and analysed
                 once, as the API's Preprocess contract intends)
  roofline       algorithmic bytes per launch / measured launch time, against the measured HBM peak
  cpu_baseline   the reference's own CPU golden timed on this host's cores (all threads, and one)
  parity_full    every output of the last end-to-end step checked against the CPU oracle
and `configs` holds the same measurements for every benchmark configuration that was run (all five on one
GPU; c2 and c5 on several).  `--impl reference` times the CPU golden alone and prints the same line shape.

With --gpus N > 1 (launched by torchrun, one rank per GPU) the matrix is cut into N row blocks of
equal non-zero count (strong scaling: the total work is fixed), x / B is held in N slices (rank r owns
slice r) and replicated inside every timed step, y / C stays sharded; time is the maximum over ranks.
"""
from __future__ import annotations

import argparse
import ctypes
import gc
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
ALL_CONFIGS = ("c1", "c2", "c3", "c4", "c5")


def measured_peaks() -> tuple[float, str]:
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        try:
            return float(json.loads(f.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json, copy bandwidth)"
        except Exception:
            pass
    return 6650.0, "fallback (6.65 TB/s, earlier measurement on this pool)"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while a timed region runs."""

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
        # A query every 20 ms: a long timed region gets a series, a short one (20 steps of 90 us) gets the sample
        # the caller takes itself while the steps run.  NVML queries go through the driver; at 500 per second on
        # every rank they showed up in the multi-GPU step time.
        while not self._stop_evt.wait(0.02):
            self.sample()

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


def describe(cfg) -> dict:
    """The workload, in the same words for both arms (the driver compares this object between them)."""
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


def metric_name(cfg) -> str:
    return "csr_spmm_gflops" if "B" in cfg else "csr_spmv_gflops"


def dtype_name(cfg) -> str:
    return {"f32": "f32", "f16": "f16 values, f32 accumulate", "bf16": "bf16 values, f32 accumulate"}[cfg["val"]]


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
                          f"{sec * 1e3:.2f} ms per pass; 16-bit configurations are timed on fp32-widened values; "
                          "the golden's row loop is split statically over the threads (started and joined inside "
                          "every clocked pass, as a caller of the reference's loop would)",
                "ms_per_pass": sec * 1e3}


def cpu_baseline(cfg, oracle, threads: int, budget_s: float = 6.0) -> dict:
    """At most about `budget_s` seconds of wall time on all host threads: the whole matrix when a pass is
    short (repeated until about a second has been spent), else its leading rows, 3 passes.  The same loop
    on one thread (the golden as the reference's harness runs it) is timed beside it on a sample a
    tenth as long."""
    g = CpuGolden(cfg, oracle, threads)
    rows = g.rows_for(budget_s / 4)
    sec, _ = g.run(rows, 1)  # also the warm-up pass
    reps = int(min(200, max(3, round(1.0 / max(sec, 1e-4)))))
    rep = g.report(rows, reps)
    one = CpuGolden(cfg, oracle, 1)
    rows1 = one.rows_for(budget_s / 40)
    one.run(rows1, 1)
    r1 = one.report(rows1, 3)
    rep["single_core"] = {"value": r1["value"], "unit": r1["unit"], "cores": 1, "kind": r1["kind"],
                          "sample": r1["sample"]}
    return rep


def reference_config(name: str, args, synth, oracle, steps: int, warmup: int, wall_budget_s: float) -> dict:
    cfg = build_config(name, synth)
    g = CpuGolden(cfg, oracle, oracle.hardware_threads())
    # one step = one golden pass over a bounded sample; warm-up + steps must end within the budget
    per_step = max(0.002, min(4.0, wall_budget_s / max(steps + warmup, 1)))
    rows = g.rows_for(per_step)
    t0 = time.perf_counter()
    per, nnz = g.passes(rows, warmup + steps)  # W untimed passes, then exactly K timed ones
    wall = time.perf_counter() - t0
    timed = per[warmup:]
    sec = float(timed.mean())
    v = 2.0 * nnz * g.n / sec / 1e9
    return {
        "metric": metric_name(cfg), "value": v, "unit": "GFLOP/s", "steps": steps, "warmup": warmup,
        "ms_per_step": sec * 1e3,
        "per_step_ms": {"min": float(timed.min()) * 1e3, "median": float(np.median(timed)) * 1e3,
                        "max": float(timed.max()) * 1e3},
        "dtype": dtype_name(cfg), "config": describe(cfg),
        "cpu_baseline": {"value": v, "unit": "GFLOP/s", "cores": g.threads, "kind": g.kind,
                         "sample": f"rows [0, {rows}) of {g.A.rows} ({nnz} of {g.A.nnz} nnz) per step; the clock "
                                   f"covers the golden loop only (whole run {wall:.1f} s with argument set-up); "
                                   "threads are started and joined inside every clocked pass"},
        "e2e": {"value": v, "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def reference_arm(args, synth, oracle):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the CPU golden runs once per job: the other ranks have nothing to do
    names = config_list(args, 1 if args.gpus <= 1 else args.gpus)
    results = {}
    for name in names:
        head = name == args.config
        steps, warmup = (args.steps, args.warmup) if head else (min(args.steps, 5), 3)
        results[name] = reference_config(name, args, synth, oracle, steps, warmup, 120.0 if head else 25.0)
    h = results[args.config]
    line = {"impl": "reference", "metric": h["metric"], "value": h["value"], "unit": "GFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": h["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": h["dtype"], "data": "synthetic (seeded)",
            "config": h["config"], "cpu_baseline": h["cpu_baseline"], "e2e": h["e2e"], "gpu_launches": 0,
            "per_step_ms": h["per_step_ms"], "configs": results}
    print(json.dumps(line))


def config_list(args, world: int) -> list[str]:
    if args.configs:
        names = [c for c in args.configs.split(",") if c]
    else:
        names = list(ALL_CONFIGS) if world == 1 else ["c2", "c5"]
    if args.config not in names:
        names.insert(0, args.config)
    return names


# ------------------------------------------------------------------------------- GPU arm

# DRAM bytes per product from ncu captures on one GPU (dram__bytes_read.sum + dram__bytes_write.sum, summed over
# the kernels of one product), with the summary under profiles/ they were read from.  A figure is attached to a
# line only when the kernels that ran are the ones the capture covers.
NCU_TRAFFIC = {
    "c2": {"bytes": 280_800_000, "kernels": "SpmvLongBlockKernel + SpmvMediumShortKernel",
           "source": "profiles/spmv_binned_c2_powerlaw_f32.md"},
    "c3": {"bytes": 352_300_000, "kernels": "SpmvShortRowsKernel", "source": "profiles/spmv_binned_c3_stencil27_f16.md"},
    "c4": {"bytes": 635_600_000, "kernels": "SpmmFastKernel", "source": "profiles/spmm_fast_c4_f32_n64.md"},
    "c5": {"bytes": 13_460_000_000, "kernels": "SpmmRowStreamKernel + SpmmLongBlockKernel",
           "source": "profiles/spmm_rowstream_c5_bf16_n256.md"},
}
# What the counters show to be the busy resource where it is not DRAM.
BOUND_NOTES = {
    "c1": "0.57 MB of inputs, L2-resident: a product is one launch of a few microseconds, bandwidth fractions say "
          "nothing here",
    "c2": "every gather of x from a random column is one 32-byte sector request to L2 and an SM issues one request "
          "per clock (measured: 0.97-0.99 gathers per clock and SM); the rows of 512+ entries (64 % of the "
          "non-zeros) gather from blocks of x staged in shared memory instead, beside the other rows' grid",
    "c4": "B (67 MB) is gathered from L2: 4.3 GB move L2->SM per product and that path delivers 18.1-18.4 TB/s "
          "(62-63 B per clock and SM, measured with a pure row-gather probe), so 236 us is the floor of any "
          "formulation that fetches a B row per non-zero",
    "c5": "B (1.07 GB) exceeds L2: the rows of up to 1024 entries gather their B rows from DRAM (11.6 GB per product "
          "at 6.1 TB/s: the row-stream kernel is at the HBM roofline of its traffic); the longer rows (43 % of the "
          "non-zeros) gather block by block of B through L2 and are bound by instruction issue and L2 latency",
}


def torch_dtype(kind: str):
    import torch
    return {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[kind]


class Env:
    pass


def kernels_of(is_spmm: bool, launches_per_step: float, b_row_bytes: int, world: int, plan=(0, 0, 0, 0)) -> str:
    """The kernels one step launches, as the library's routing rules give them (`plan`: b200spSpMMPlanInfo)."""
    if is_spmm:
        if plan[1] > 0:
            long_rows = " + SpmmLongBlockKernel (rows > 1024 nnz, block by block of B through L2, side stream)"
        elif plan[0] > 0:
            long_rows = " + SpmmFastKernel (segment CTAs of rows > 1024 nnz, side stream)"
        else:
            long_rows = ""
        if b_row_bytes in (512, 1024):
            return "SpmmRowStreamKernel" + long_rows
        return "SpmmFastKernel" + (long_rows if plan[1] > 0 else "")
    if launches_per_step >= 2 + (world > 1):
        return "SpmvLongBlockKernel (side stream) + SpmvMediumShortKernel"
    return "SpmvShortRowsKernel | SpmvMediumShortKernel | SpmvAllBinsKernel"


def measure_config(name: str, args, env, head: bool) -> dict:
    """Every leg of the benchmark for one configuration on this rank's share; returns the rank-0 result dict
    (other ranks return their local pieces, which the caller ignores)."""
    import torch
    import torch.distributed as dist
    from ops_sparse_b200 import api, hostio, mg

    torch_, world, rank, dev, oracle, synth, pkg = env.torch, env.world, env.rank, env.dev, env.oracle, env.synth, env.pkg
    L = pkg.lib()
    K, W = (args.steps, args.warmup) if head else (min(args.steps, 200), min(args.warmup, 10))

    cfg = build_config(name, synth)  # every rank draws the same matrix from the same seed
    A = cfg["A"]
    is_spmm = "B" in cfg
    alpha, beta = cfg["alpha"], cfg["beta"]
    vt, ot = torch_dtype(cfg["val"]), torch_dtype(cfg["out"])
    cuts = mg.partition_rows(A.row_ptr, world)
    r0, r1 = mg.local_rows(cuts, rank)
    rp, ci, v = mg.slice_csr(A.row_ptr, A.col_ind, A.values, r0, r1)
    d_rp, d_ci = torch.from_numpy(rp).to(dev), torch.from_numpy(np.ascontiguousarray(ci)).to(dev)
    d_v = torch.from_numpy(np.ascontiguousarray(v)).to(dev).to(vt)
    replicate = args.replicate if world > 1 else "none"
    if is_spmm:
        n = cfg["B"].shape[1]
        dense_h = torch.from_numpy(cfg["B"]).to(vt).pin_memory()
        out_h = torch.from_numpy(cfg["C"][r0:r1]).to(ot).pin_memory()
    else:
        n = 1
        dense_h = torch.from_numpy(cfg["x"]).to(vt).pin_memory()
        out_h = torch.from_numpy(cfg["y"][r0:r1]).to(ot).pin_memory()
    # Every rank starts from the whole operand only to cut its own slice from it (the sharded operators keep
    # that slice); in the "nccl-broadcast" form the other ranks' copies are zeroed so that the step must fill them.
    dense = dense_h.to(dev)
    if world > 1 and replicate == "nccl-broadcast" and rank != 0:
        dense.zero_()
    out = out_h.to(dev)
    if is_spmm:
        op = mg.ShardedSpmm(d_rp, d_ci, d_v, A.cols, dense, out, replicate=replicate if world > 1 else "nccl-broadcast")
    else:
        op = mg.ShardedSpmv(d_rp, d_ci, d_v, A.cols, dense, out, replicate=replicate if world > 1 else "nccl-broadcast")
    if world > 1 and replicate != "nccl-broadcast":
        dense.zero_()  # the full-size buffer is only a target now: what the product reads must come from the exchange
    result_h = torch.empty_like(out_h).pin_memory()
    ct = api._compute_type(d_v, out)

    # one GPU: the K products are issued by a compiled loop (include/b200sp_bench.h), as a C caller would
    a_c, b_c = ctypes.c_float(alpha), ctypes.c_float(beta)
    a_p, b_p = ctypes.cast(ctypes.byref(a_c), ctypes.c_void_p), ctypes.cast(ctypes.byref(b_c), ctypes.c_void_p)

    def steps(count: int, with_exchange: bool):
        if world == 1:
            if is_spmm:
                rc = L.b200spRepeatSpMM(op.handle.raw, 0, 0, a_p, op.A.raw, op.B.raw, b_p, op.C.raw, ct, 0,
                                        api._ptr(op.buffer), count)
            else:
                rc = L.b200spRepeatSpMV(op.handle.raw, 0, a_p, op.A.raw, op.x.raw, b_p, op.y.raw, ct, 0,
                                        api._ptr(op.buffer), count)
            if rc != 0:
                raise RuntimeError(f"compute entry point returned status {rc}")
        elif with_exchange:
            op.steps(alpha, beta, count)  # the compiled loop again when the peer exchange is in use
        else:
            op.products(alpha, beta, count)  # no exchange: the local product alone, same compiled loop

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

    # Set-up outside the timed region: the exchange (peer mappings or NCCL channels) is brought to its steady
    # state with untimed steps on the real buffers, then the W warm-up steps the caller asked for.
    settle = 30 if world > 1 else 0
    steps(settle, True)
    barrier()
    steps(W, True)
    barrier()

    # ---- timed region: exactly K steps, inputs resident, CUDA events on the launching stream
    sampler = ClockSampler(physical_gpu_index(env.local))
    if rank == 0:  # rank 0 reports its GPU's clocks; the other ranks' GPUs are left alone while they are timed
        sampler.start()
    count = L.b200sp_kernel_launches
    count.restype = ctypes.c_ulonglong
    if world > 1:
        # The host-side barrier releases the ranks some hundred microseconds apart, which is a quarter of 20 steps
        # of 60 us and would be charged to whichever rank left it first.  One more untimed step, enqueued right
        # before the first event, lines the GPUs up on the device: its exchange waits for every rank.
        steps(1, True)
    launches_before = count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    steps(K, True)
    e1.record()
    launches = int(count() - launches_before)  # this rank's kernels inside the timed region
    if rank == 0:
        sampler.sample()  # taken while the K steps are running on the device
    torch.cuda.synchronize()
    clocks = sampler.stop()
    barrier()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = total_ms / K

    # ---- the same steps with an event after each, for the spread (an event costs a little: the mean above is
    # the figure of record, these show whether it hides a transient)
    KS = min(K, 200)
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(KS + 1)]
    barrier()
    evs[0].record()
    for i in range(KS):
        steps(1, True)
        evs[i + 1].record()
    torch.cuda.synchronize()
    per = np.array([evs[i].elapsed_time(evs[i + 1]) for i in range(KS)])
    per_step = {"min": max_over_ranks(float(per.min())), "median": max_over_ranks(float(np.median(per))),
                "max": max_over_ranks(float(per.max())), "steps": KS}

    # ---- compute-only steps (no exchange): launch duration for the roofline.  A step is one launch of the
    # dominant kernel (plus, where two run side by side, the one beside it), so the duration is the
    # event-bracketed region divided by the steps.
    KL = min(K, 200)
    barrier()
    e0.record()
    steps(KL, False)
    e1.record()
    torch.cuda.synchronize()
    launch_ms_mean = max_over_ranks(e0.elapsed_time(e1) / KL)
    exchange_error = op.replication_error()

    # ---- end to end: host buffers in, host result out, every step, through the library's entry points for
    # host-resident operands (include/b200sp_host.h): rows cut into panels so that the copies of one panel overlap
    # the product of another; every copy and kernel of a step is issued by the library.
    KE = min(K, 200)
    pipe = hostio.HostOperandProduct(rp, d_ci, d_v, A.cols, dense, out, panels=args.e2e_panels)
    graph = pipe.capture(dense_h, out_h, result_h, alpha, beta) if (world == 1 and not args.no_graph) else None

    def e2e_step():
        if graph is not None:
            graph.replay()  # the recorded step: x / B up, per panel y / C up -> product -> result down
        else:
            pipe.step(dense_h, out_h, result_h, alpha, beta, upload_dense=True)

    for _ in range(5):
        e2e_step()
    # Two passes of KE steps, the quieter one counts: the leg is bound by host <-> device copies, and on a shared
    # host another job's traffic on the same PCIe switch has doubled a pass now and then.
    e2e_passes = []
    for _ in range(2):
        barrier()
        e0.record()
        for _ in range(KE):
            e2e_step()
            torch.cuda.synchronize()  # the caller needs the result before the next step
        e1.record()
        torch.cuda.synchronize()
        e2e_passes.append(max_over_ranks(e0.elapsed_time(e1)) / KE)
    e2e_ms = min(e2e_passes)
    del graph
    pipe.close()
    out_bytes = (r1 - r0) * n * out_h.element_size()
    h2d = dense_h.numel() * dense_h.element_size() + (out_bytes if beta != 0 else 0)
    d2h = out_bytes

    # ---- every output of the last end-to-end step against the CPU oracle (threaded, all local rows)
    tol = 1e-5 if cfg["val"] == "f32" else 2e-3
    S = A.row_slice(r0, r1)
    vw = torch.from_numpy(np.ascontiguousarray(S.values)).to(vt).to(torch.float32).numpy()
    dw = dense_h.to(torch.float32).numpy()
    ow = out_h.to(torch.float32).numpy()
    gw = result_h.to(torch.float32).numpy()
    t0 = time.perf_counter()
    if is_spmm:
        bad, worst = oracle.check_spmm_f32(S.row_ptr, S.col_ind, vw, dw, ow, gw, alpha, beta, tol)
    else:
        bad, worst = oracle.check_spmv_f32(S.row_ptr, S.col_ind, vw, dw, ow, gw, alpha, beta, tol)
    check_s = time.perf_counter() - t0
    del vw, dw, ow, gw
    if world > 1:
        t = torch.tensor([float(bad)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        bad = int(t.item())
        t = torch.tensor([worst], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        worst = float(t.item())
    parity = {"outputs_checked": int(A.rows * n), "outside_tolerance": int(bad), "worst_err_over_scale": worst,
              "tolerance": tol, "rule": "|got - gold| <= tol * (|alpha| * sum |a b| + |beta * old|), every output",
              "checker": "oracle/ (CPU golden restatement), all host threads", "seconds": round(check_s, 2),
              "ok": bad == 0 and exchange_error == 0}

    alg_bytes, flops = bytes_and_flops(cfg, synth)
    my_bytes, _ = bytes_and_flops(cfg, synth, rows=r1 - r0, nnz=int(ci.size))
    peak, peak_src = measured_peaks()
    achieved = my_bytes / (launch_ms_mean * 1e-3) / 1e9
    value = flops / (ms_per_step * 1e-3) / 1e9

    base = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        base = cpu_baseline(cfg, oracle, oracle.hardware_threads())

    lps = launches / K
    plan = (ctypes.c_int32 * 4)()
    if is_spmm:
        L.b200spSpMMPlanInfo(op.A.raw, plan)
    kernels = kernels_of(is_spmm, lps, n * dense.element_size() if is_spmm else 0, world, tuple(plan))
    traffic = NCU_TRAFFIC.get(name) if world == 1 else None
    if traffic is not None and any(k not in kernels for k in traffic["kernels"].split(" + ")):
        traffic = None
    res = {
        "metric": metric_name(cfg), "value": value, "unit": "GFLOP/s", "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms_per_step, "per_step_ms": per_step, "dtype": dtype_name(cfg), "config": describe(cfg),
        "effective_gbs": alg_bytes / (ms_per_step * 1e-3) / 1e9, "algorithmic_bytes_per_step": alg_bytes,
        "roofline": {
            "bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
            "frac_of_nominal_8000": achieved / NOMINAL_HBM_GBS, "peak_source": peak_src, "kernel": kernels,
            "launch_ms_mean": launch_ms_mean, "algorithmic_bytes_per_launch": my_bytes,
            "traffic": traffic["bytes"] if traffic else None, "traffic_source": traffic["source"] if traffic else None,
            "note": BOUND_NOTES.get(name) if world == 1 and (traffic is not None or name == "c1") else None,
        },
        "e2e": {"value": flops / (e2e_ms * 1e-3) / 1e9, "unit": "GFLOP/s", "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": KE,
                "passes_ms": [round(v, 6) for v in e2e_passes],
                "row_panels": args.e2e_panels, "cuda_graph": world == 1 and not args.no_graph},
        "compute_only": {"value": flops / (launch_ms_mean * 1e-3) / 1e9, "unit": "GFLOP/s",
                         "ms_per_step": launch_ms_mean,
                         "exchange_ms_per_step": max(ms_per_step - launch_ms_mean, 0.0) if world > 1 else 0.0},
        "gpu_launches": launches * world, "kernels_per_step": lps, "clocks": clocks, "parity_full": parity,
        "l2_policy": ("no flush between steps: A (col_ind + values) alone is larger than L2 "
                      f"({(4 + d_v.element_size()) * A.nnz / 1e6:.0f} MB vs 126 MB); x / B may stay cached"
                      if (4 + d_v.element_size()) * A.nnz > L2_BYTES else
                      "inputs fit in L2: this configuration is launch-latency bound, bandwidth fractions are not "
                      "meaningful"),
    }
    if base is not None:
        res["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample", "single_core") if k in base}
    op.close()
    del op, dense, out, d_rp, d_ci, d_v, dense_h, out_h, result_h, cfg, A
    gc.collect()
    torch.cuda.empty_cache()
    return res


def gpu_arm(args, synth, oracle):
    import torch
    import torch.distributed as dist

    env = Env()
    env.world = int(os.environ.get("WORLD_SIZE", "1"))
    env.rank = int(os.environ.get("RANK", "0"))
    env.local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU implementation")
    torch.cuda.set_device(env.local)
    env.dev = torch.device("cuda", env.local)
    if env.world > 1:
        dist.init_process_group("nccl", device_id=env.dev)
    env.torch, env.oracle, env.synth = torch, oracle, synth
    env.pkg = entry.load_package()

    names = config_list(args, env.world)
    results = {}
    for name in names:
        results[name] = measure_config(name, args, env, head=(name == args.config))
    if env.rank == 0:
        h = results[args.config]
        line = {
            "metric": h["metric"], "value": h["value"], "unit": "GFLOP/s", "n_gpus": env.world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": h["ms_per_step"], "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": h["dtype"], "data": "synthetic (seeded)", "config": h["config"],
            "parallelism": ("single GPU" if env.world == 1 else
                            f"rows split by nnz over {env.world} GPUs; x / B held in {env.world} slices and replicated "
                            f"inside every step ({args.replicate}); 30 untimed steps before the warm-up bring the "
                            "exchange to its steady state; one untimed step after the barrier lines the ranks up "
                            "on the device before the first event"),
            "analysis": "aclsparse*Preprocess once, outside the timed region",
            "step_issue": ("compiled loop over the C API (b200spRepeatSpMV / b200spRepeatSpMM)" if env.world == 1
                           else ("compiled loop over the C API (b200spMgRepeatSpMV / b200spMgRepeatSpMM): one exchange "
                                 "launch and one aclsparse call per step" if args.replicate == "peer"
                                 else "Python loop: one collective and one aclsparse call per step")),
        }
        for k in ("per_step_ms", "effective_gbs", "algorithmic_bytes_per_step", "roofline", "e2e", "compute_only",
                  "gpu_launches", "kernels_per_step", "clocks", "parity_full", "l2_policy", "cpu_baseline"):
            if k in h:
                line[k] = h[k]
        line["configs"] = results
        print(json.dumps(line))
    if env.world > 1:
        dist.barrier()
        dist.destroy_process_group()
    bad = [n for n, r in results.items() if not r["parity_full"]["ok"]]
    if bad:
        raise SystemExit(f"parity check against the CPU oracle failed for {bad}")


# ------------------------------------------------------------------------------- operators next to the hot path

def aux_arm(args, synth, oracle):
    """`--op coo2csr | csrsort | csr2csc | sddmm`: the CSR producers and SDDMM on benchmark-size inputs (one GPU).
    One JSON line: time per call (CUDA events), algorithmic bytes per call, the HBM roofline fraction, the CPU
    golden restatement timed on this host, and a bit-exact (converters) / reference-verdict (SDDMM) parity check."""
    import torch
    from ctypes import byref, c_size_t, c_uint16, c_void_p
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product path has no CPU implementation")
    pkg = entry.load_package()
    from ops_sparse_b200 import api
    L, S = pkg.lib(), pkg
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    h = api.Handle()
    P = lambda t: c_void_p(t.data_ptr())
    to = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    K = max(3, min(args.steps, 50))
    peak, peak_src = measured_peaks()

    def timed(fn, restore=None):
        for _ in range(3):
            if restore:
                restore()
            fn()
        torch.cuda.synchronize()
        times = []
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(K):
            if restore:
                restore()
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        return np.array(times)

    if args.op in ("coo2csr", "csrsort", "csr2csc"):
        cfg = synth.config2()
        A = cfg["A"]
        m, n, nnz = A.rows, A.cols, A.nnz
        d_rp, d_ci = to(A.row_ptr), to(A.col_ind)
    if args.op == "coo2csr":
        rows = np.repeat(np.arange(m, dtype=np.int32), A.lengths())
        d_rows, d_out = to(rows), torch.empty(m + 1, dtype=torch.int32, device=dev)
        fn = lambda: api.check(L.aclsparseXcoo2csr(h.raw, P(d_rows), nnz, m, P(d_out), 0), "aclsparseXcoo2csr")
        t = timed(fn)
        t0 = time.perf_counter()
        gold = oracle.coo2csr(rows, m, 0)
        cpu_s = time.perf_counter() - t0
        ok = bool(np.array_equal(d_out.cpu().numpy(), gold))
        alg = 4 * nnz + 4 * (m + 1)
        workload = {"workload": "coo2csr of the c2 pattern", "rows": m, "nnz": nnz}
        kernels = "Coo2CsrKernel (a binary search per row offset)"
    elif args.op == "csrsort":
        rng = np.random.default_rng(7)
        key = np.repeat(np.arange(m, dtype=np.int64), A.lengths()) * (1 << 21) + rng.integers(0, 1 << 21, nnz)
        shuffled = A.col_ind[np.argsort(key, kind="stable")].astype(np.int32)  # every row's columns in random order
        d_src = to(shuffled)
        d_col, d_p = torch.empty_like(d_src), torch.empty(nnz, dtype=torch.int32, device=dev)
        iota = torch.arange(nnz, dtype=torch.int32, device=dev)
        descr = c_void_p()
        api.check(L.aclsparseCreateMatDescr(byref(descr)), "aclsparseCreateMatDescr")
        size = c_size_t()
        api.check(L.aclsparseXcsrsort_bufferSizeExt(h.raw, m, n, nnz, P(d_rp), P(d_src), byref(size)), "bufferSizeExt")
        buf = torch.empty(size.value, dtype=torch.uint8, device=dev)

        def restore():
            d_col.copy_(d_src)
            d_p.copy_(iota)
        fn = lambda: api.check(L.aclsparseXcsrsort(h.raw, m, n, nnz, descr, P(d_rp), P(d_col), P(d_p), P(buf)), "csrsort")
        t = timed(fn, restore)
        t0 = time.perf_counter()
        gc_, gp_ = oracle.csrsort(A.row_ptr, shuffled, np.arange(nnz, dtype=np.int32), 0)
        cpu_s = time.perf_counter() - t0
        ok = bool(np.array_equal(d_col.cpu().numpy(), gc_) and np.array_equal(d_p.cpu().numpy(), gp_))
        alg = 4 * (m + 1) + 16 * nnz  # col_ind and P: read once, written once
        workload = {"workload": "csrsort of the c2 pattern, columns shuffled inside every row", "rows": m, "nnz": nnz,
                    "workspace_bytes": int(size.value)}
        kernels = "SegSortWarpKernel + SegSortCtaKernel (keys formed and split inside the sort)"
    elif args.op == "csr2csc":
        d_v = to(A.values)
        o_v, o_ri = torch.empty_like(d_v), torch.empty_like(d_ci)
        o_cp = torch.empty(n + 1, dtype=torch.int32, device=dev)
        size = c_size_t()
        api.check(L.aclsparseCsr2cscEx2_bufferSize(h.raw, m, n, nnz, None, None, None, None, None, None, S.ACL_FLOAT, 1, 0,
                                                   0, byref(size)), "bufferSize")
        buf = torch.empty(size.value, dtype=torch.uint8, device=dev)
        fn = lambda: api.check(L.aclsparseCsr2cscEx2(h.raw, m, n, nnz, P(d_v), P(d_rp), P(d_ci), P(o_v), P(o_cp), P(o_ri),
                                                     S.ACL_FLOAT, 1, 0, 0, P(buf)), "csr2csc")
        t = timed(fn)
        t0 = time.perf_counter()
        gcp, gri, gv = oracle.csr2csc(m, n, A.row_ptr, A.col_ind, A.values.view(np.uint32), 0)
        cpu_s = time.perf_counter() - t0
        ok = bool(np.array_equal(o_cp.cpu().numpy(), gcp) and np.array_equal(o_ri.cpu().numpy(), gri)
                  and np.array_equal(o_v.cpu().numpy().view(np.uint32), gv))
        alg = 4 * (m + 1) + 8 * nnz + 4 * (n + 1) + 8 * nnz
        workload = {"workload": "csr2csc (numeric, fp32) of the c2 matrix", "rows": m, "cols": n, "nnz": nnz,
                    "workspace_bytes": int(size.value)}
        kernels = ("ColumnHistogramKernel + Scan{BlockSums,Sums,Apply}Kernel + ScatterKeysKernel + "
                   "SegSort{Warp,Cta}Kernel")
    elif args.op in ("spmvop-alg1", "spmvop-alg2"):
        # the SpMVOp plan API (compensated row sums) on the c2 matrix, Z aliasing Y
        cfg = synth.config2()
        A = cfg["A"]
        m, n, nnz = A.rows, A.cols, A.nnz
        d_rp, d_ci, d_v = to(A.row_ptr), to(A.col_ind), to(A.values)
        dA = api.CsrMatrix(d_rp, d_ci, d_v, m, n)
        y0 = to(cfg["y"])
        dx, dy = api.DnVec(to(cfg["x"])), api.DnVec(y0.clone())
        plan = api.SpMVOpPlan(h, dA, dx, dy, dy, alg=2 if args.op.endswith("2") else 1)
        fn = lambda: plan.run(dx, dy, dy, cfg["alpha"], cfg["beta"])
        t = timed(fn, lambda: dy.values.copy_(y0))
        t0 = time.perf_counter()
        gold = oracle.spmv_op(A.row_ptr, A.col_ind, A.values, cfg["x"], cfg["y"], cfg["alpha"], cfg["beta"])
        cpu_s = time.perf_counter() - t0
        got = dy.values.cpu().numpy().astype(np.float64)
        scale = abs(cfg["alpha"]) * oracle.spmv_abs_rowsum(A.row_ptr, A.col_ind, A.values, cfg["x"]) + np.abs(cfg["beta"] * cfg["y"])
        ok = bool(np.all(np.abs(got - gold.astype(np.float64)) <= 1e-6 * scale + 1e-30))
        alg = synth.algorithmic_bytes_spmv(m, n, nnz, 4, 4, cfg["beta"])
        workload = {"workload": f"aclsparseSpMVOp ({args.op[-4:]}) on the c2 matrix", "rows": m, "nnz": nnz}
        kernels = ("SpmvOpLongRowsKernel + SpmvOpRowsKernel per length class" if args.op.endswith("2") else "SpmvOpRowsKernel")
        plan.close()
    else:  # sddmm: the pattern of a 1 M-node power-law graph, X and Y^T of 256 fp16 per row (the backward of c5's layer)
        cfg = synth.config5(rows=1 << 20)
        A = cfg["A"]
        m, n, nnz, k = A.rows, A.cols, A.nnz, 256
        rng = np.random.default_rng(11)
        X = torch.from_numpy(rng.uniform(-1, 1, (m, k)).astype(np.float16)).to(dev)
        Yt = torch.from_numpy(rng.uniform(-1, 1, (n, k)).astype(np.float16)).to(dev)
        c0 = torch.from_numpy(rng.uniform(-1, 1, nnz).astype(np.float16)).to(dev)
        cv = c0.clone()
        d_rp, d_ci = to(A.row_ptr), to(A.col_ind)
        dX, dY, dC = c_void_p(), c_void_p(), c_void_p()
        api.check(L.aclsparseCreateDnMat(byref(dX), m, k, k, P(X), S.ACL_FLOAT16, 0), "CreateDnMat")
        api.check(L.aclsparseCreateDnMat(byref(dY), n, k, k, P(Yt), S.ACL_FLOAT16, 0), "CreateDnMat")
        api.check(L.aclsparseCreateCsr(byref(dC), m, n, nnz, P(d_rp), P(d_ci), P(cv), 0, 0, 0, S.ACL_FLOAT16), "CreateCsr")
        one, half = c_uint16(int(np.float16(1.0).view(np.uint16))), c_uint16(int(np.float16(0.5).view(np.uint16)))
        a_, b_ = c_void_p(ctypes.addressof(one)), c_void_p(ctypes.addressof(half))
        size = c_size_t()
        api.check(L.aclsparseSDDMMBufferSize(h.raw, 0, 1, a_, dX, dY, b_, dC, S.ACL_FLOAT16, 0, byref(size)), "BufferSize")
        buf = torch.empty(max(size.value, 256), dtype=torch.uint8, device=dev)
        api.check(L.aclsparseSDDMMPreprocess(h.raw, 0, 1, a_, dX, dY, b_, dC, S.ACL_FLOAT16, 0, P(buf)), "Preprocess")
        fn = lambda: api.check(L.aclsparseSDDMM(h.raw, 0, 1, a_, dX, dY, b_, dC, S.ACL_FLOAT16, 0, P(buf)), "aclsparseSDDMM")
        t = timed(fn, lambda: cv.copy_(c0))
        # parity and CPU time on the leading rows (the fp64 golden is O(nnz * k) on one thread)
        rows_s = int(np.searchsorted(A.row_ptr, 200_000))
        e_s = int(A.row_ptr[rows_s])
        Xs = X[:rows_s].to(torch.float64).cpu().numpy()
        Ys = Yt.to(torch.float64).cpu().numpy()
        t0 = time.perf_counter()
        gold = oracle.sddmm_f64(rows_s, n, k, Xs, Ys, A.row_ptr[:rows_s + 1], A.col_ind[:e_s],
                                c0[:e_s].to(torch.float64).cpu().numpy(), 1.0, 0.5, False, True)
        cpu_s = (time.perf_counter() - t0) * (nnz / max(e_s, 1))
        got = cv[:e_s].to(torch.float32).cpu().numpy()
        ok = oracle.verify_mixed_tolerance(got, np.clip(gold.astype(np.float32), -65504.0, 65504.0), "f16")[0]
        alg = 2 * m * k + 2 * n * k + 4 * (m + 1) + 4 * nnz + 4 * nnz
        workload = {"workload": "SDDMM fp16 on the pattern of a 1,048,576-node power-law graph, k = 256, op_y = T",
                    "rows": m, "cols": n, "nnz": nnz, "k": k, "alpha": 1.0, "beta": 0.5,
                    "gather_bytes": int(nnz) * 2 * k * 2,
                    "note": "the Y row of every entry is its own 512-byte read: the gather (nnz * 1 KB with X) is what "
                            "moves, the algorithmic bytes count X and Y once"}
        kernels = "SddmmVecKernel"
    ms = float(np.median(t))
    line = {"op": args.op, "metric": f"{args.op}_ms", "value": ms, "unit": "ms", "higher_is_better": False, "n_gpus": 1,
            "steps": K, "warmup": 3, "per_step_ms": {"min": float(t.min()), "median": ms, "max": float(t.max())},
            "data": "synthetic (seeded)", "config": workload,
            "roofline": {"bound": "hbm", "achieved": alg / (ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                         "frac": alg / (ms * 1e-3) / 1e9 / peak, "algorithmic_bytes_per_launch": int(alg),
                         "peak_source": peak_src, "kernel": kernels, "traffic": None},
            "cpu_baseline": {"value": cpu_s * 1e3, "unit": "ms", "cores": 1, "kind": "port",
                             "sample": "oracle restatement of the reference golden, one pass on one thread"
                                       + (" (leading rows, scaled by nnz)" if args.op == "sddmm" else "")},
            "parity": {"ok": bool(ok), "rule": "mixed tolerance of the reference test frame on the leading 200,000 entries' rows"
                       if args.op == "sddmm" else "|err| <= 1e-6 * (|alpha| sum |a x| + |beta y|) per row against the restated "
                       "compensated row sums" if args.op.startswith("spmvop") else "bit-exact against the golden restatement"}}
    print(json.dumps(line))
    h.close()
    if not ok:
        raise SystemExit(f"{args.op}: parity check against the CPU oracle failed")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="c2", choices=list(ALL_CONFIGS), help="the headline configuration")
    ap.add_argument("--configs", default="", help="comma-separated configurations to measure (default: all five on "
                                                  "one GPU, c2 and c5 on several); the headline is always included")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU golden timing leg")
    ap.add_argument("--replicate", default="peer", choices=["peer", "nccl-allgather", "nccl-broadcast"],
                    help="how x / B reaches every GPU inside a multi-GPU step (see ops-sparse_b200/mg.py)")
    ap.add_argument("--op", default="", choices=["", "coo2csr", "csrsort", "csr2csc", "sddmm", "spmvop-alg1", "spmvop-alg2"],
                    help="measure one of the operators next to the hot path instead (one GPU)")
    ap.add_argument("--no-graph", action="store_true", help="end-to-end leg: issue every step's operations one by one")
    ap.add_argument("--e2e-panels", type=int, default=4,
                    help="row panels the end-to-end leg pipelines its host copies over (1 = copy, compute, copy)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    entry._load("b200sp_build_oracle", ROOT / "oracle" / "build_oracle.py").build_oracle()
    oracle = entry.load_oracle()
    if args.impl == "reference":
        # the CPU arm never maps the CUDA library: the workload generator is loaded on its own
        synth = entry._load("b200sp_synth", ROOT / "ops-sparse_b200" / "synth.py")
        reference_arm(args, synth, oracle)
    else:
        entry.load_package()
        from ops_sparse_b200 import synth
        if args.op:
            aux_arm(args, synth, oracle)
        else:
            gpu_arm(args, synth, oracle)


if __name__ == "__main__":
    main()
