"""Benchmark of the hc tiled-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one pass of the hot path (one GEMM) over one batch of seeded synthetic input.

  N = 1   workload "gemm_8192": M=N=K=8192, float16, fp32 accumulate/output (the configuration
          the metric is quoted on). `--workload skinny|ragged|sim_64|sharded` time the others.
  N > 1   workload "sharded": M=16384, N=32768, K=16384 with B and C split by columns over the
          ranks and A replicated; no data-path collective (strong scaling: the total work is
          fixed). The optional NCCL all-gather of the C slabs is timed separately.

The JSON line printed by rank 0 carries: `value` (aggregate TFLOP/s, inputs resident in HBM,
CUDA-event time, max over ranks), `e2e` (the same metric through the public
`hc.compile(..., target="nvidia-sm100a")` handle on pinned NumPy buffers, host<->device copies
inside the timed region), `roofline` for the dominant kernel, `cpu_baseline` (the CPU oracle
timed on this box's host cores on a bounded sample) and the SM clocks sampled while timing.

`--impl reference` times the reference's own CPU implementation of the path instead. The
reference is Python and cannot run here without its un-vendored dependencies, so this arm
runs the bit-exact C restatement of its arithmetic (oracle/) on all host threads, on a
bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

REPO = Path(__file__).resolve().parent
for _entry in (str(REPO), str(REPO / "5_b200")):
    if _entry not in sys.path:
        sys.path.insert(0, _entry)

import workloads  # noqa: E402

METRIC = "gemm_tflops"
UNIT = "TFLOP/s"
NOMINAL_PEAK_TFLOPS = 2250.0  # dense fp16/bf16, for context
NOMINAL_HBM_GBS = 8000.0
NOMINAL_SM_MHZ = 1965  # clocks.max.sm of the B200s of this pool
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}

# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum) as
# (bytes, where the figure comes from): ncu captures summarised under profiles/, NOT measured by
# the run that prints them. Workloads without a capture carry no figure.
NCU_DRAM_TRAFFIC = {
    "gemm_8192": (1.105e9, "ncu capture, profiles/gemm_dense_wide_kernel__gemm_8192.md"),
    "gemm_8192:float8_e4m3fn": (0.618e9, "ncu capture, profiles/gemm_dense_wide_kernel__gemm_8192_float8.md (B stored [N, K])"),
    "skinny": (272.4e6, "ncu capture, profiles/gemm_skinny_kernel__skinny_8x16384x8192.md"),
    "ragged": (21.1e6, "ncu capture, profiles/ragged_4095x3073x1031__launches.md (GEMM kernel only)"),
    "long_k": (33.6e6, "ncu capture, profiles/gemm_dense_cluster_kernel__512x512x16384.md"),
}


def measured_peaks() -> tuple[dict, str]:
    path = REPO / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except (OSError, ValueError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# ---------------------------------------------------------------- clocks ----------------


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU in a background thread (read-only)."""

    REASONS = {
        0x0000000000000001: "gpu_idle",
        0x0000000000000002: "applications_clocks_setting",
        0x0000000000000010: "sync_boost",
        0x0000000000000100: "display_clock_setting",
        0x0000000000000004: "sw_power_cap",
        0x0000000000000008: "hw_slowdown",
        0x0000000000000020: "sw_thermal_slowdown",
        0x0000000000000040: "hw_thermal_slowdown",
        0x0000000000000080: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int, period_s: float = 0.002) -> None:
        self.device_index = device_index
        self.period_s = period_s
        self.samples: list[tuple[float, int, int]] = []  # (time, sm_mhz, reasons bitmask)
        self.sm_max_mhz: int | None = None
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._nvml = None
        self._handle = None
        self.error: str | None = None

    def start(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.sm_max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # NVML missing: report, do not fail the benchmark
            self.error = f"{type(exc).__name__}: {exc}"
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self) -> None:
        nv = self._nvml
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                try:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                except Exception:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception as exc:
                self.error = f"{type(exc).__name__}: {exc}"
                return
            self._stop.wait(self.period_s)

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)

    def summary(self, begin: float, end: float) -> dict:
        inside = [(mhz, reasons) for t, mhz, reasons in self.samples if begin <= t <= end]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max_mhz, "reasons": [], "samples": 0,
                    "note": self.error or "no sample fell inside the timed region"}
        clocks = sorted(mhz for mhz, _ in inside)
        mask = 0
        for _, reasons in inside:
            mask |= reasons
        names = sorted(name for bit, name in self.REASONS.items() if mask & bit)
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": self.sm_max_mhz, "reasons": names,
                "samples": len(inside), "sm_mhz_min": clocks[0], "sm_mhz_highest": clocks[-1]}


# ---------------------------------------------------------------- distributed plumbing ---


class Ranks:
    """torch.distributed used for rendezvous only: barrier, max-reduce of a float, broadcast."""

    def __init__(self, connect: bool = True) -> None:
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.dist = None
        self.torch = None
        if self.world > 1 and connect:
            import torch
            import torch.distributed as dist

            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            torch.cuda.set_device(self.local_rank)
            dist.init_process_group("cpu:gloo,cuda:nccl", rank=self.rank, world_size=self.world)
            self.dist, self.torch = dist, torch

    def barrier(self) -> None:
        if self.dist is not None:
            self.dist.all_reduce(self.torch.zeros(1))  # CPU tensor: goes over gloo

    def device_sync(self) -> None:
        if self.torch is not None:
            self.torch.cuda.synchronize()

    def max(self, value: float) -> float:
        if self.dist is None:
            return value
        box = self.torch.tensor([value], dtype=self.torch.float64)
        self.dist.all_reduce(box, op=self.dist.ReduceOp.MAX)
        return float(box[0])

    def gather_objects(self, obj):
        if self.dist is None:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj)
        return out

    def broadcast_bytes(self, payload):
        if self.dist is None:
            return payload
        box = [payload]
        self.dist.broadcast_object_list(box, src=0)
        return box[0]

    def close(self) -> None:
        if self.dist is not None:
            self.dist.destroy_process_group()


# ---------------------------------------------------------------- CPU legs ---------------


def time_cpu_oracle(a: np.ndarray, b: np.ndarray, target_seconds: float = 12.0) -> dict:
    """Times the CPU oracle (C restatement of the reference's arithmetic, all host threads) on
    a bounded sample: the first R rows of C, R chosen so the run takes about `target_seconds`."""
    from oracle import cpu_ref

    m, k = a.shape
    n = b.shape[1]
    threads = cpu_ref.max_threads()
    probe_rows = min(m, max(threads, 8))
    start = time.perf_counter()
    cpu_ref.matmul_k_ascending(a, b, rows=(0, probe_rows))
    probe = time.perf_counter() - start
    # The probe includes widening B once; assume the same fixed cost in the real sample.
    rows = int(min(m, max(probe_rows, probe_rows * target_seconds / max(probe, 1e-3))))
    rows = max(threads, rows - rows % threads) if rows >= threads else rows
    rows = min(rows, m)
    start = time.perf_counter()
    cpu_ref.matmul_k_ascending(a, b, rows=(0, rows))
    seconds = time.perf_counter() - start
    return {
        "value": workloads.flops(rows, n, k) / seconds / 1e12,
        "unit": UNIT,
        "cores": threads,
        "kind": "port",
        "seconds": seconds,
        "sample": f"rows [0,{rows}) of C: {rows}x{n}x{k} multiply-accumulates of the {m}x{n}x{k} workload",
    }


_SIMULATOR_SCRIPT = r"""
import importlib, json, os, sys, time
import numpy as np
sys.path.insert(0, sys.argv[2]); sys.path.insert(0, sys.argv[1])
ex = importlib.import_module("examples.amdgpu_gfx11_wmma_matmul")
rng = np.random.default_rng(0)
a = rng.standard_normal((64, 64)).astype(np.float16)
b = rng.standard_normal((64, 64)).astype(np.float16)
start = time.perf_counter()
c = ex.simulate_gfx11_wmma_matmul(a, b)
print(json.dumps({"seconds": time.perf_counter() - start, "checksum": float(np.abs(c).sum())}))
"""


def time_reference_simulator() -> dict:
    """The reference's own executor, `hc.simulator`, on benchmark configuration 1 (64^3, float16,
    seed 0): the unmodified Python package from the checkout that $HC_REFERENCE_DIR names, with
    oracle/standins/ in place of its two absent third-party dependencies (neither carries
    arithmetic). One core: the simulator is a Python interpreter loop. Without a checkout the
    record says so; the C restatement above is then the only CPU figure."""
    reference = os.environ.get("HC_REFERENCE_DIR", "")
    if not reference or not (Path(reference) / "hc" / "simulator.py").exists():
        return {"unavailable": "unavailable on this box: no reference checkout ($HC_REFERENCE_DIR is not set "
                               "or has no hc/simulator.py)"}
    env = dict(os.environ)
    env["HC_IXSIMPL_VENDOR_DIR"] = str(REPO / "oracle" / "standins" / "ixsimpl_vendor")
    try:
        result = subprocess.run([sys.executable, "-c", _SIMULATOR_SCRIPT, reference, str(REPO / "oracle" / "standins")],
                                capture_output=True, text=True, timeout=300, env=env)
        if result.returncode != 0:
            return {"unavailable": f"the reference simulator did not run: {result.stderr.strip()[-200:]}"}
        out = json.loads(result.stdout.strip().splitlines()[-1])
    except Exception as exc:
        return {"unavailable": f"the reference simulator did not run: {type(exc).__name__}: {exc}"}
    flops = workloads.flops(64, 64, 64)
    return {"seconds": out["seconds"], "value": flops / out["seconds"] / 1e12, "unit": UNIT, "cores": 1,
            "kind": "reference", "sample": "hc.simulator on the whole of configuration 1 (64x64x64, float16, seed 0)"}


def time_numpy_matmul(a: np.ndarray, b: np.ndarray, budget_rows: int = 8192) -> dict:
    """NumPy/BLAS float32 matmul of the same shape (inputs widened first), for context."""
    rows = min(a.shape[0], budget_rows)
    a32 = a[:rows].astype(np.float32)
    b32 = b.astype(np.float32)
    start = time.perf_counter()
    _ = a32 @ b32
    seconds = time.perf_counter() - start
    threads = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_info

        pools = [p.get("num_threads") for p in threadpool_info() if p.get("user_api") == "blas"]
        if pools:
            threads = int(pools[0])
    except Exception:
        pass
    return {"value": workloads.flops(rows, b.shape[1], a.shape[1]) / seconds / 1e12, "unit": UNIT,
            "threads": threads, "seconds": seconds, "sample": f"{rows}x{b.shape[1]}x{a.shape[1]} float32 matmul"}


def time_cublas(a: np.ndarray, b: np.ndarray, steps: int) -> dict:
    """Library yardstick, same protocol as the timed region: cuBLAS through torch.mm on the same
    inputs, once with fp32 output (the same problem as the hc kernel) and once with 16-bit output
    (what the pod's measured tensor peak was taken with). Context only; never on the hot path."""
    try:
        import torch
    except Exception as exc:  # pragma: no cover
        return {"error": f"{type(exc).__name__}: {exc}"}
    if a.dtype.name == "bfloat16":
        ta = torch.from_numpy(a.view(np.uint16).copy()).view(torch.bfloat16).cuda()
        tb = torch.from_numpy(b.view(np.uint16).copy()).view(torch.bfloat16).cuda()
    else:
        ta, tb = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    flops = workloads.flops(a.shape[0], b.shape[1], a.shape[1])
    out = {}
    variants = {"out_16bit": lambda: torch.mm(ta, tb)}
    try:
        torch.mm(ta, tb, out_dtype=torch.float32)
        variants["out_fp32"] = lambda: torch.mm(ta, tb, out_dtype=torch.float32)
    except Exception as exc:
        out["out_fp32"] = {"error": f"{type(exc).__name__}: {exc}"}
    for name, fn in variants.items():
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        out[name] = {"ms_per_step": ms, "tflops": flops / (ms * 1e-3) / 1e12}
    return out


# ---------------------------------------------------------------- arms -------------------


def choose_workload(args, world: int) -> str:
    if args.workload:
        return args.workload
    return "gemm_8192" if world == 1 else "sharded"


def run_reference_arm(args, ranks: Ranks) -> None:
    if ranks.rank != 0:
        return
    name = choose_workload(args, ranks.world)
    w = workloads.CONFIGS[name]
    if name == "sharded":
        # One 2048-column block of B is a faithful sample of the sharded product.
        a, b = workloads.make_sharded_inputs(0, workloads.SHARDED_BLOCK_COLUMNS)
    else:
        a, b = workloads.make_inputs(name)
    per_step = max(2.0, min(20.0, 120.0 / max(1, args.steps + args.warmup)))
    results = [time_cpu_oracle(a, b, target_seconds=per_step) for _ in range(args.warmup + args.steps)]
    timed = results[args.warmup:]
    seconds = sum(r["seconds"] for r in timed)
    value = sum(float(r["value"]) * r["seconds"] for r in timed) / seconds
    baseline = dict(timed[-1])
    baseline["value"] = value
    baseline["simulator"] = time_reference_simulator()
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": ranks.world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / len(timed) * 1e3,
        "higher_is_better": True, "scaling": "strong" if ranks.world > 1 else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": name, "m": w.m, "n": w.n, "k": w.k, "input_dtype": w.dtype},
        "detail": {"note": "CPU restatement of the reference simulator's arithmetic on host cores; "
                           "each step is the bounded sample named in cpu_baseline.sample"},
        "cpu_baseline": baseline,
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


L2_BYTES = 126e6


def timed_region(ctx, ranks: Ranks, sampler: ClockSampler, launch, steps: int) -> tuple[float, dict]:
    """`steps` launches between two CUDA events on the context's stream, bracketed by a barrier and
    a device synchronise on both sides. Returns (device milliseconds, max over ranks; clocks sampled
    between the two host time stamps)."""
    start_ev, stop_ev = ctx.event(), ctx.event()
    ranks.barrier()
    ctx.synchronize()
    ranks.device_sync()
    t_begin = time.perf_counter()
    start_ev.record()
    for i in range(steps):
        launch(i)
    stop_ev.record()
    elapsed_ms = stop_ev.elapsed_ms_since(start_ev)
    ctx.synchronize()
    ranks.device_sync()
    t_end = time.perf_counter()
    ranks.barrier()
    return ranks.max(elapsed_ms), sampler.summary(t_begin, t_end)


class DeviceRun:
    """One workload resident in HBM on this rank: buffers, the compiled handle's plan, the timed
    launches, parity of what was timed, and the roofline of its dominant kernel."""

    def __init__(self, ctx, ranks: Ranks, name: str, *, b_transposed: bool = False, member: str = "plain",
                 rotate: bool = False) -> None:
        from examples.b200_wmma_matmul import compiled_for
        from hc.distributed import column_slab

        self.ctx, self.ranks, self.name = ctx, ranks, name
        w = self.w = workloads.CONFIGS[name]
        if name == "sharded":
            slab = column_slab(w.n, ranks.world, ranks.rank, align=workloads.SHARDED_BLOCK_COLUMNS)
            self.a, self.b = workloads.make_sharded_inputs(slab.begin, slab.end)
            self.local_n = slab.width
        else:
            self.a, self.b = workloads.make_inputs(name)
            self.local_n = w.n
        self.m, self.k = w.m, w.k
        self.b_transposed = b_transposed
        self.host_b = np.ascontiguousarray(self.b.T) if b_transposed else self.b
        self.handle = compiled_for(w.dtype, ranks.local_rank, b_transposed, member)
        if self.handle.plan is None:
            raise SystemExit(f"kernel not recognised: {self.handle.pipeline_diagnostics}")
        contract = self.contract = self.handle.plan
        self.bias = self.dbias = None
        if contract.bias_param is not None:
            self.bias = np.random.default_rng(99).standard_normal(self.local_n).astype(np.float32)
            self.dbias = ctx.to_device(self.bias)
        self.gemm_kwargs = {"b_transposed": b_transposed, "accumulate": contract.accumulate,
                            "epilogue": contract.epilogue, "bias": self.dbias}
        self.c_type = self.a.dtype if contract.output_dtype != "float32" else np.dtype(np.float32)
        # A working set smaller than L2 would be served from L2 on every launch after the first:
        # such a workload is run on several copies of its buffers in turn, enough of them that a
        # copy has left L2 by the time it is used again.
        c_bytes = self.m * self.local_n * self.c_type.itemsize
        self.working_set = self.a.nbytes + self.host_b.nbytes + c_bytes
        copies = 1
        if rotate and self.working_set < 1.5 * L2_BYTES and self.working_set >= 4e6:
            copies = min(8, int(np.ceil(1.5 * L2_BYTES / self.working_set)))
        self.sets = []
        for _ in range(copies):
            dc = ctx.empty((self.m, self.local_n), self.c_type)
            dc.fill_bytes(0)
            self.sets.append((ctx.to_device(self.a), ctx.to_device(self.host_b), dc))
        self.da, self.db, self.dc = self.sets[0]
        self.bound = [ctx.bind_gemm(da, db, dc, **self.gemm_kwargs) for da, db, dc in self.sets]
        self.plan = ctx.plan(self.m, self.local_n, self.k, w.dtype, b_transposed=b_transposed,
                             accumulate=contract.accumulate, epilogue=contract.epilogue,
                             c_dtype=contract.output_dtype)
        self.local_flops = workloads.flops(self.m, self.local_n, self.k)
        self.total_flops = workloads.flops(w.m, w.n, w.k)
        if self.working_set > L2_BYTES:
            self.l2 = "inputs larger than L2 (A+B+C per GPU exceed 126 MB)"
        elif copies > 1:
            self.l2 = (f"{copies} copies of A, B, C used in turn ({copies * self.working_set / 1e6:.0f} MB in all, "
                       f"larger than L2)")
        else:
            self.l2 = "working set fits L2: a launch-latency figure, not a bandwidth or tensor one"

    def launch(self, i: int) -> None:
        self.bound[i % len(self.bound)].launch()

    def time(self, sampler: ClockSampler, steps: int, warmup: int, sustained_seconds: float = 0.0) -> None:
        for i in range(max(warmup, 3) * len(self.bound)):
            self.launch(i)
        self.ctx.synchronize()
        self.steps = steps
        elapsed_ms, self.clocks = timed_region(self.ctx, self.ranks, sampler, self.launch, steps)
        self.region_ms = elapsed_ms
        self.ms_per_step = elapsed_ms / steps
        self.sustained = None
        if sustained_seconds > 0:
            # The same launches for at least `sustained_seconds` of device time, so that every N and
            # every workload is also seen in the power state a long job runs in.
            count = int(max(steps, np.ceil(sustained_seconds * 1e3 / self.ms_per_step)))
            long_ms, long_clocks = timed_region(self.ctx, self.ranks, sampler, self.launch, count)
            self.sustained = {"launches": count, "seconds": long_ms / 1e3, "ms_per_step": long_ms / count,
                              "clocks": long_clocks}

    def check(self) -> dict:
        """Parity of what was timed: sampled rows of C against the float64 rule."""
        contract, ctx = self.contract, self.ctx
        if contract.accumulate:
            # The timed launches kept adding to C; check one launch on top of zeros.
            self.dc.fill_bytes(0)
            ctx.gemm(self.da, self.db, self.dc, **self.gemm_kwargs)
            ctx.synchronize()
        c = self.c = self.dc.to_numpy()
        a, b = self.a, self.b
        rows = self.rows = np.unique(np.linspace(0, self.m - 1, 16).astype(np.int64))
        parity = workloads.check_against_float64(c, a, b, rows=rows, epilogue=contract.epilogue, bias=self.bias)
        if contract.output_dtype != "float32":
            # A 16-bit C carries half a unit in its last place on top of the float32 bound.
            ulp = 2.0 ** -11 if contract.output_dtype == "float16" else 2.0 ** -8
            exact = a[rows].astype(np.float64) @ b.astype(np.float64)
            bound = np.abs(a[rows].astype(np.float64)) @ np.abs(b.astype(np.float64))
            diff = np.abs(c[rows].astype(np.float64) - exact)
            parity["ok"] = bool(parity["finite"] and (diff <= 1e-2 * bound + ulp * np.abs(exact)).all())
            parity["output_rounding"] = (f"{contract.output_dtype}: half a unit in the last place added to the "
                                         f"element bound")
        self.parity_all = self.ranks.gather_objects(parity)
        return self.parity_summary()

    def parity_summary(self) -> dict:
        return {"rule": "vs float64 product: rel Frobenius <= 1e-3, |err| <= 1e-2*(|A||B|)",
                "rows_checked_per_rank": int(len(self.rows)), "ok": all(p["ok"] for p in self.parity_all),
                "rel_frobenius": max(p["rel_frobenius"] for p in self.parity_all),
                "max_element_ratio": max(p["max_element_ratio"] for p in self.parity_all)}

    def kernel_name(self) -> str:
        if self.plan.variant == "skinny":
            return "gemm_skinny_kernel"
        if self.m >= 1024 and self.plan.tiles_m == -(-self.m // 512):
            return "gemm_dense_wide_kernel"
        pairs = self.m > 128 and self.plan.tiles_m == -(-self.m // 256)
        return "gemm_dense_pair_kernel" if pairs else "gemm_dense_kernel"

    def roofline(self, peaks: dict, peaks_source: str) -> dict:
        """Achieved rate of the dominant kernel over the timed region against the measured peak that
        bounds it. `traffic` is only ever a figure from a committed ncu capture of the same kernel
        and workload, named in `traffic_source`; nothing measured in this run stands behind it."""
        traffic, source = NCU_DRAM_TRAFFIC.get(self.name, (None, None)) if self.ranks.world == 1 else (None, None)
        seconds = self.ms_per_step * 1e-3
        out: dict = {}
        if self.plan.variant == "skinny":
            algo = workloads.algorithmic_bytes(self.m, self.local_n, self.k) \
                - (4 - self.c_type.itemsize) * self.m * self.local_n \
                - (2 - self.a.dtype.itemsize) * (self.m * self.k + self.k * self.local_n)
            algo += (4 * self.m * self.local_n if self.contract.accumulate else 0) \
                + (0 if self.bias is None else self.bias.nbytes)
            achieved, peak = algo / seconds / 1e9, float(peaks["hbm_gbs"])
            out = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                   "algorithmic_bytes_per_launch": algo, "peak_source": f"{peaks_source} HBM copy bandwidth",
                   "frac_of_nominal": achieved / NOMINAL_HBM_GBS}
            if self.sustained:
                rate = algo / (self.sustained["ms_per_step"] * 1e-3) / 1e9
                out["sustained"] = {**self.sustained, "achieved": rate, "frac": rate / peak}
        else:
            achieved = self.local_flops / seconds / 1e12
            burst, long_run = float(peaks["bf16_tflops"]), float(peaks["bf16_tflops_sustained"])
            # A timed region shorter than a second is a burst (the clocks sampled inside it say so
            # too); a longer one is compared with the figure cuBLAS sustains under the power cap.
            is_burst = self.region_ms < 1000.0
            peak = burst if is_burst else long_run
            eight_bit = self.w.dtype.startswith("float8")
            out = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                   "frac": achieved / peak, "flops_per_launch": self.local_flops,
                   "peak_source": f"{peaks_source} cuBLAS bf16 8192^3 (16-bit output), "
                                  + ("burst: the timed region lasted under a second" if is_burst
                                     else "sustained: the timed region lasted over a second"),
                   "timed_region_ms": self.region_ms,
                   "frac_of_burst_peak": achieved / burst, "frac_of_sustained_peak": achieved / long_run,
                   "frac_of_nominal": achieved / (NOMINAL_PEAK_TFLOPS * (2 if eight_bit else 1))}
            if eight_bit:
                out["note"] = ("8-bit operands: no peak was measured for them on this pool, so `peak` is still the "
                               "16-bit cuBLAS figure (a fraction above 1 is expected); frac_of_nominal is against "
                               "the nominal dense fp8 rate, 4500 TFLOP/s")
            if self.sustained:
                rate = self.local_flops / (self.sustained["ms_per_step"] * 1e-3) / 1e12
                out["sustained"] = {**self.sustained, "achieved": rate, "peak": long_run, "frac": rate / long_run,
                                    "peak_source": f"{peaks_source} cuBLAS bf16, back to back for seconds"}
        out["kernel"] = self.kernel_name()
        out["traffic"] = traffic
        out["traffic_source"] = source if traffic is not None else "not captured for this workload"
        return out

    def free(self) -> None:
        for bufs in self.sets:
            for buf in bufs:
                buf.free()
        if self.dbias is not None:
            self.dbias.free()
        self.sets, self.bound = [], []


def side_record(ctx, ranks: Ranks, sampler: ClockSampler, name: str, steps: int, peaks: dict, peaks_source: str,
                sustained_seconds: float = 0.0) -> dict:
    """One of the other benchmark configurations on this GPU: ms, achieved rate, roofline, parity,
    clocks -- the same protocol as the headline workload, without the end-to-end and CPU legs."""
    try:
        run = DeviceRun(ctx, ranks, name, rotate=True)
        run.time(sampler, steps, 5, sustained_seconds)
        parity = run.check()
        record = {
            "m": run.m, "n": run.local_n, "k": run.k, "input_dtype": run.w.dtype, "steps": steps,
            "ms_per_step": run.ms_per_step, "tflops": run.local_flops / (run.ms_per_step * 1e-3) / 1e12,
            "gbs": workloads.algorithmic_bytes(run.m, run.local_n, run.k) / (run.ms_per_step * 1e-3) / 1e9,
            "variant": run.plan.variant, "grid": run.plan.grid, "splits": run.plan.splits,
            "launches_per_step": run.plan.kernel_launches, "l2": run.l2,
            "roofline": run.roofline(peaks, peaks_source), "parity": parity, "clocks": run.clocks,
        }
        run.free()
        return record
    except Exception as exc:  # a side record must not take the headline number down with it
        return {"error": f"{type(exc).__name__}: {exc}"}


def map_record(ctx, ranks: Ranks, sampler: ClockSampler, steps: int, peaks: dict, peaks_source: str) -> dict:
    """The masked element-wise kernel class (examples/b200_elementwise.py: scaled_clamp, seven float32
    operations with a second input) on 2^27 elements per buffer: HBM-bound, 12 bytes per element
    (two inputs read, one output written), checked bit for bit against the NumPy oracle."""
    try:
        from examples.b200_elementwise import compiled as compiled_map
        from oracle import cpu_ref

        n = 1 << 27
        plan = compiled_map("scaled_clamp", ranks.local_rank).plan
        rng = np.random.default_rng(16)
        x = rng.standard_normal(n, dtype=np.float32)
        y = rng.standard_normal(n, dtype=np.float32)
        dx, dy, dout = ctx.to_device(x), ctx.to_device(y), ctx.empty((n,), np.float32)
        launch = lambda i: ctx.map(dx, dout, plan.ops, other=dy)  # noqa: E731
        for i in range(5):
            launch(i)
        ctx.synchronize()
        elapsed_ms, clocks = timed_region(ctx, ranks, sampler, launch, steps)
        ms = elapsed_ms / steps
        sample = slice(0, 1 << 20)
        got = dout.to_numpy()
        want = cpu_ref.map_elementwise(x[sample], plan.ops, other=y[sample])
        tail = cpu_ref.map_elementwise(x[-4099:], plan.ops, other=y[-4099:])
        ok = bool(np.array_equal(got[sample].view(np.uint32), want.view(np.uint32))
                  and np.array_equal(got[-4099:].view(np.uint32), tail.view(np.uint32)))
        algo = 12.0 * n
        achieved, peak = algo / (ms * 1e-3) / 1e9, float(peaks["hbm_gbs"])
        for buf in (dx, dy, dout):
            buf.free()
        return {"kernel_class": "masked element-wise map (scaled_clamp: 7 float32 operations, 2 inputs)",
                "n": n, "steps": steps, "ms_per_step": ms, "gbs": achieved,
                "l2": "inputs larger than L2 (1.5 GiB per launch)",
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "algorithmic_bytes_per_launch": algo,
                             "peak_source": f"{peaks_source} HBM copy bandwidth", "kernel": "map_f32_kernel",
                             "frac_of_nominal": achieved / NOMINAL_HBM_GBS, "traffic": None,
                             "traffic_source": "not captured for this workload"},
                "parity": {"rule": "bit-identical to the NumPy oracle (first 2^20 and last 4099 elements)", "ok": ok},
                "clocks": clocks}
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"}


def pairwise_record(ctx, ranks: Ranks, sampler: ClockSampler, steps: int) -> dict:
    """The pairwise-distance kernel class (examples/b200_pairwise.py: the reference simulator's own
    two-dimensional test kernel) on 8192 x 8192 outputs over 128 values: three float32 instructions per
    (i, j, h), none of them fusable, so the bound is the float32 issue rate; checked bit for bit against
    the NumPy oracle on sampled rows."""
    try:
        from oracle import cpu_ref

        w1 = w2 = 8192
        h = 128
        rng = np.random.default_rng(18)
        x1 = rng.standard_normal((w1, h), dtype=np.float32)
        x2 = rng.standard_normal((w2, h), dtype=np.float32)
        d1, d2, dout = ctx.to_device(x1), ctx.to_device(x2), ctx.empty((w1, w2), np.float32)
        launch = lambda i: ctx.pairwise(d1, d2, dout)  # noqa: E731
        for i in range(3):
            launch(i)
        ctx.synchronize()
        elapsed_ms, clocks = timed_region(ctx, ranks, sampler, launch, steps)
        ms = elapsed_ms / steps
        rows = np.r_[0:24, w1 - 24 : w1]
        got = dout.to_numpy()[rows]
        want = cpu_ref.pairwise_distance(x1[rows], x2)
        ok = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
        flops = 3.0 * w1 * w2 * h
        achieved = flops / (ms * 1e-3) / 1e12
        sm_count = ctx.sm_count
        peak = sm_count * 128 * NOMINAL_SM_MHZ * 1e6 / 1e12  # one float32 instruction per lane and clock
        for buf in (d1, d2, dout):
            buf.free()
        return {"kernel_class": "pairwise distances (pairwise: sqrt of the sum of squared differences)",
                "w1": w1, "w2": w2, "h": h, "steps": steps, "ms_per_step": ms, "tflops": achieved,
                "l2": "output larger than L2 (256 MiB per launch); inputs (8 MiB) stay resident, as in the kernel's use",
                "roofline": {"bound": "fp32", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                             "algorithmic_flops_per_launch": flops,
                             "peak_source": f"nominal: {sm_count} SMs x 128 float32 lanes x {NOMINAL_SM_MHZ} MHz, one "
                                            "instruction per lane and clock (no fused multiply-add: every operation "
                                            "of the kernel rounds)",
                             "kernel": "pairwise_f32_kernel", "traffic": None,
                             "traffic_source": "not captured for this workload"},
                "parity": {"rule": "bit-identical to the NumPy oracle (first and last 24 rows)", "ok": ok},
                "clocks": clocks}
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"}


def row_sum_record(ctx, ranks: Ranks, sampler: ClockSampler, steps: int, peaks: dict, peaks_source: str) -> dict:
    """The row-sum kernel class (examples/b200_rowsum.py: row_norms, the square root of the sum of the
    squared values of each row) on 2^19 rows of 512 values: HBM-bound, 4 bytes read per value and 4
    written per row, checked bit for bit against the NumPy oracle (the additions follow the order of
    NumPy's sum)."""
    try:
        from oracle import cpu_ref

        w, h = 1 << 19, 512
        rng = np.random.default_rng(19)
        x = rng.standard_normal((w, h), dtype=np.float32)
        dx, dout = ctx.to_device(x), ctx.empty((w,), np.float32)
        launch = lambda i: ctx.row_sum(dx, dout, square=True, take_sqrt=True)  # noqa: E731
        for i in range(5):
            launch(i)
        ctx.synchronize()
        elapsed_ms, clocks = timed_region(ctx, ranks, sampler, launch, steps)
        ms = elapsed_ms / steps
        rows = np.r_[0:8192, w - 8192 : w]
        got = dout.to_numpy()[rows]
        want = cpu_ref.row_sums(x[rows], square=True, take_sqrt=True)
        ok = bool(np.array_equal(got.view(np.uint32), want.view(np.uint32)))
        algo = 4.0 * w * h + 4.0 * w
        achieved, peak = algo / (ms * 1e-3) / 1e9, float(peaks["hbm_gbs"])
        for buf in (dx, dout):
            buf.free()
        return {"kernel_class": "row sums (row_norms: sqrt of the sum of the squared values of a row)",
                "w": w, "h": h, "steps": steps, "ms_per_step": ms, "gbs": achieved,
                "l2": "input larger than L2 (1 GiB per launch)",
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "algorithmic_bytes_per_launch": algo,
                             "peak_source": f"{peaks_source} HBM copy bandwidth", "kernel": "row_sum_f32_kernel",
                             "frac_of_nominal": achieved / NOMINAL_HBM_GBS, "traffic": None,
                             "traffic_source": "not captured for this workload"},
                "parity": {"rule": "bit-identical to the NumPy oracle (first and last 8192 rows)", "ok": ok},
                "clocks": clocks}
    except Exception as exc:
        return {"error": f"{type(exc).__name__}: {exc}"}


def run_gpu_arm(args, ranks: Ranks) -> None:
    from hc import cuda
    from hc.distributed import column_slab, init_communicator

    name = choose_workload(args, ranks.world)
    w = workloads.CONFIGS[name]
    if name != "sharded" and ranks.world > 1:
        raise SystemExit(f"workload {name} does not shard; run it with --gpus 1")
    ctx = cuda.Context(ranks.local_rank)
    peaks, peaks_source = measured_peaks()
    run = DeviceRun(ctx, ranks, name, b_transposed=args.b_transposed, member=args.member)
    a, b, m, k, local_n = run.a, run.b, run.m, run.k, run.local_n
    da, db, dc = run.da, run.db, run.dc
    contract, plan, handle, bias = run.contract, run.plan, run.handle, run.bias
    c_type, total_flops = run.c_type, run.total_flops

    # ---- warm-up, then the timed region (device time, max over ranks), then >= 2 s of the same ----
    sampler = ClockSampler(ranks.local_rank)
    sampler.start()
    run.time(sampler, args.steps, args.warmup, 0.0 if args.quick else args.sustained_seconds)
    ms_per_step, clocks = run.ms_per_step, run.clocks
    value = total_flops / (ms_per_step * 1e-3) / 1e12

    # ---- correctness of what was timed (sampled rows, float64 rule) ------------------------
    parity = run.check()
    c, rows = run.c, run.rows

    if args.quick:
        sampler.stop()
        if ranks.rank == 0:
            print(json.dumps({"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": ranks.world,
                              "steps": args.steps, "ms_per_step": ms_per_step, "quick": True,
                              "config": {"workload": name, "variant": plan.variant, "splits": plan.splits,
                                         "grid": plan.grid, "launches_per_step": plan.kernel_launches},
                              "parity_ok": parity["ok"], "clocks": clocks}), flush=True)
        return

    # ---- end to end through the public handle on pinned host buffers ---------------------
    e2e_steps = max(1, min(args.steps, args.e2e_steps))
    pa = cuda.pinned_empty(a.shape, a.dtype)
    host_b = run.host_b
    pb = cuda.pinned_empty(host_b.shape, host_b.dtype)
    pc = cuda.pinned_empty((m, local_n), c_type)
    pa[...] = a
    pb[...] = host_b
    pc[...] = 0
    call_args = (pa, pb, pc) if bias is None else (pa, pb, pc, bias)
    e2e_api = "hc.compile(kernel, target='nvidia-sm100a')(a, b, c) on pinned NumPy arrays"
    e2e_h2d_a = a.nbytes
    comm_ready = False
    if ranks.world > 1:
        # The sharded product from host arrays: every rank holds A in host memory but uploads only
        # its share of the rows; the shares are exchanged over NVLink instead of crossing PCIe once
        # per rank. Needs the NCCL communicator the gather leg uses as well.
        try:
            from hc.distributed import ShardedMatmul

            init_communicator(ctx, ranks.world, ranks.rank, ranks.broadcast_bytes)
            comm_ready = True
            sharded_host = ShardedMatmul(handle, ctx, w.n, ranks.world, ranks.rank,
                                         align=workloads.SHARDED_BLOCK_COLUMNS)
            e2e_call = lambda: sharded_host.host_product(pa, pb, pc)  # noqa: E731
            e2e_ctx = ctx
            e2e_api = ("hc.distributed.ShardedMatmul.host_product(a, b_slab, c_slab) on pinned NumPy arrays: each "
                       "rank uploads 1/N of A's rows, the shares are exchanged over NVLink (NCCL all-gather), the "
                       "B slab travels in column panels while earlier panels are multiplied and sent back")
            e2e_h2d_a = a.nbytes // ranks.world if m % ranks.world == 0 else a.nbytes
        except Exception as exc:
            e2e_api += f" (sharded host path unavailable: {type(exc).__name__}: {exc})"
            e2e_call = lambda: handle(*call_args)  # noqa: E731
            e2e_ctx = cuda.default_context(ranks.local_rank)
    else:
        e2e_call = lambda: handle(*call_args)  # noqa: E731
        e2e_ctx = cuda.default_context(ranks.local_rank)
    e2e_call()  # warm-up: allocates the context's staging buffers
    e0, e1 = e2e_ctx.event(), e2e_ctx.event()
    ranks.barrier()
    e2e_ctx.synchronize()
    e0.record()
    for _ in range(e2e_steps):
        e2e_call()
    e1.record()
    e2e_ms = ranks.max(e1.elapsed_ms_since(e0)) / e2e_steps
    if contract.accumulate:  # the host C has taken the product 1 + e2e_steps times
        e2e_ok = bool(np.allclose(pc[rows], (1 + e2e_steps) * c[rows], rtol=1e-4, atol=1e-5))
    else:
        e2e_ok = bool(np.array_equal(pc[rows], c[rows]))
        if not e2e_ok and plan.splits > 1:
            # The device launch split some tiles over k; the host call's panels never do, so the two
            # differ by fp32 reassociation in those tiles.
            scale = float(np.abs(c[rows].astype(np.float64)).max())
            e2e_ok = bool(np.allclose(pc[rows].astype(np.float64), c[rows].astype(np.float64), rtol=1e-4,
                                      atol=1e-5 * max(scale, 1.0)))
    h2d_bytes = e2e_h2d_a + b.nbytes + (pc.nbytes if contract.accumulate else 0) + (0 if bias is None else bias.nbytes)
    e2e = {"value": total_flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
           "steps": e2e_steps, "h2d_bytes_per_step": int(h2d_bytes),
           "d2h_bytes_per_step": int(pc.nbytes), "matches_device_path": e2e_ok,
           "api": e2e_api}

    # ---- optional all-gather of the C slabs (N > 1), reported separately ---------------------
    gather = None
    if ranks.world > 1 and not args.no_gather:
        try:
            if not comm_ready:
                init_communicator(ctx, ranks.world, ranks.rank, ranks.broadcast_bytes)
            gathered = ctx.empty((ranks.world, m, local_n), np.float32)
            g0, g1 = ctx.event(), ctx.event()
            ctx.all_gather(dc, gathered)
            ctx.synchronize()
            ranks.barrier()
            g0.record()
            for _ in range(3):
                ctx.all_gather(dc, gathered)
            g1.record()
            gather_ms = ranks.max(g1.elapsed_ms_since(g0)) / 3
            received = (ranks.world - 1) * dc.nbytes
            gather = {"ms": gather_ms, "bytes_received_per_gpu": int(received),
                      "gbs_per_gpu": received / (gather_ms * 1e-3) / 1e9, "layout": "slab-major [rank][M][N/ranks]",
                      "library": "NCCL over NVLink"}
            ctx.comm_destroy()
        except Exception as exc:
            gather = {"error": f"{type(exc).__name__}: {exc}"}

    if comm_ready and (args.no_gather or (gather is not None and "error" in gather)):
        try:
            ctx.comm_destroy()
        except Exception:
            pass

    # ---- the same product with the gather fused into the epilogue (N > 1) ------------------
    fused = None
    if ranks.world > 1 and not args.no_gather:
        try:
            import hashlib

            from hc.distributed import PushedMatmul

            pushed = PushedMatmul(ctx, m, w.n, ranks.world, ranks.rank, align=workloads.SHARDED_BLOCK_COLUMNS)
            full_c = pushed.setup(ranks.gather_objects)
            pushed.run(da, db)
            ctx.synchronize()
            ranks.barrier()
            fused_steps = max(1, min(args.steps, 10))
            f0, f1 = ctx.event(), ctx.event()
            f0.record()
            for _ in range(fused_steps):
                pushed.run(da, db)
            f1.record()
            fused_ms = ranks.max(f1.elapsed_ms_since(f0)) / fused_steps
            ctx.synchronize()
            ranks.barrier()
            # Every rank must now hold every slab exactly as its owner computed it.
            digests = []
            for r in range(ranks.world):
                lo, hi = column_slab(w.n, ranks.world, r, align=workloads.SHARDED_BLOCK_COLUMNS).begin, \
                    column_slab(w.n, ranks.world, r, align=workloads.SHARDED_BLOCK_COLUMNS).end
                sample = np.concatenate([full_c.window(int(row), int(row) + 1, lo, hi).to_numpy() for row in rows[:8]])
                digests.append(hashlib.sha256(sample.tobytes()).hexdigest())
            everyone = ranks.gather_objects(digests)
            consistent = all(view == everyone[0] for view in everyone)
            own = np.concatenate([c[int(row):int(row) + 1] for row in rows[:8]])
            matches_plain = hashlib.sha256(own.tobytes()).hexdigest() == digests[ranks.rank]
            fused = {"ms": fused_ms, "aggregate_tflops": total_flops / (fused_ms * 1e-3) / 1e12,
                     "steps": fused_steps, "bytes_pushed_per_gpu": int((ranks.world - 1) * dc.nbytes),
                     "layout": "row-major C[M,N] on every rank", "all_ranks_identical": bool(consistent),
                     "matches_unfused_slab": bool(matches_plain),
                     "mechanism": "GEMM epilogue stores each tile to all peers through CUDA IPC pointers (NVLink)"}
            pushed.close()
            ranks.barrier()
            full_c.free()
        except Exception as exc:
            fused = {"error": f"{type(exc).__name__}: {exc}"}

    # ---- the other benchmark configurations on this GPU (single-GPU line only) --------------
    side = {}
    if ranks.world == 1 and name == "gemm_8192" and args.member == "plain" and not args.b_transposed \
            and not args.no_side_workloads:
        run.free()  # config 5 on one GPU needs 3.5 GiB of its own
        side["skinny"] = side_record(ctx, ranks, sampler, "skinny", 400, peaks, peaks_source)
        side["ragged"] = side_record(ctx, ranks, sampler, "ragged", 400, peaks, peaks_source)
        side["sim_64"] = side_record(ctx, ranks, sampler, "sim_64", 1000, peaks, peaks_source)
        side["long_k"] = side_record(ctx, ranks, sampler, "long_k", 1000, peaks, peaks_source)
        side["elementwise_map"] = map_record(ctx, ranks, sampler, 50, peaks, peaks_source)
        side["pairwise"] = pairwise_record(ctx, ranks, sampler, 20)
        side["row_sum"] = row_sum_record(ctx, ranks, sampler, 50, peaks, peaks_source)
        side["sharded_1gpu"] = side_record(ctx, ranks, sampler, "sharded", 10, peaks, peaks_source,
                                           sustained_seconds=args.sustained_seconds)
    sampler.stop()

    if ranks.rank != 0:
        return

    roofline = run.roofline(peaks, peaks_source)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": ranks.world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if ranks.world > 1 else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": {"workload": name, "m": w.m, "n": w.n, "k": w.k, "input_dtype": w.dtype},
        "detail": {"accumulate": "fp32", "variant": plan.variant, "per_gpu_n": local_n,
                   "b_layout": "[N, K] (transposed)" if args.b_transposed else "[K, N]",
                   "member": args.member,
                   "parallelism": f"n-sharded x{ranks.world}" if ranks.world > 1 else "single GPU",
                   "l2": run.l2, "device": ctx.name, "sm_count": ctx.sm_count},
        "roofline": roofline,
        "e2e": e2e,
        "gpu_launches": args.steps * plan.kernel_launches,
        "clocks": clocks,
        "parity": parity,
    }
    if run.sustained is not None:
        per_step = run.sustained["ms_per_step"]
        line["sustained"] = {"value": total_flops / (per_step * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": per_step,
                             "launches": run.sustained["launches"], "seconds": run.sustained["seconds"],
                             "clocks": run.sustained["clocks"],
                             "note": "the timed launches repeated for at least this long, CUDA-event time, max "
                                     "over ranks: the rate in the power state of a long job"}
    if side:
        line["workloads"] = side
    if gather is not None:
        line["all_gather"] = gather
    if fused is not None:
        if gather is not None and "ms" in gather and "ms" in fused:
            fused["product_then_nccl_all_gather_ms"] = ms_per_step + gather["ms"]
        line["fused_gather"] = fused
    if args.cublas and ranks.world == 1:
        line["cublas"] = time_cublas(a, b, args.steps)
    if ranks.world == 1 and not args.no_cpu_baseline:
        baseline = time_cpu_oracle(a, b)
        baseline["numpy_f32_matmul"] = time_numpy_matmul(a, b)
        baseline["simulator"] = time_reference_simulator()
        line["cpu_baseline"] = baseline
    print(json.dumps(line), flush=True)


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--impl", choices=("b200", "reference"), default="b200")
    parser.add_argument("--workload", choices=sorted(workloads.CONFIGS), default=None)  # (aliases are added below)
    parser.add_argument("--shape", default=None, metavar="MxNxK",
                        help="an arbitrary float16 shape instead of a named workload (single GPU), e.g. 8192x8192x512")
    parser.add_argument("--input-dtype", default=None, choices=("float16", "bfloat16", "float8_e4m3fn", "float8_e5m2"),
                        help="single GPU: run the workload with A and B of this element type (same shape, seed and "
                             "distribution, values rounded to it) instead of the type the configuration names")
    parser.add_argument("--e2e-steps", type=int, default=5)
    parser.add_argument("--sustained-seconds", type=float, default=2.0,
                        help="after the timed steps, repeat the same launches for at least this long and report "
                             "that rate too (0 = skip)")
    parser.add_argument("--no-side-workloads", action="store_true",
                        help="single GPU: leave out the records of the other benchmark configurations")
    parser.add_argument("--no-gather", action="store_true")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--b-transposed", action="store_true",
                        help="hand B over stored [N, K] and use the Buffer[N, K] member of the kernel family")
    parser.add_argument("--member", choices=("plain", "accumulate", "fused", "narrow"), default="plain",
                        help="kernel family member: C = A.B (the reference example, default), C += A.B, "
                             "C = maximum(0.125 * A.B + bias, 0) folded into the store, or C in the input type")
    parser.add_argument("--cublas", action="store_true",
                        help="also time cuBLAS (torch.mm) on the same inputs with the same loop, for context")
    parser.add_argument("--quick", action="store_true",
                        help="timed region and parity only (for profiler captures): no e2e, CPU or gather legs")
    args = parser.parse_args()
    if args.steps < 1:
        parser.error("--steps must be at least 1")
    if args.shape is not None:
        try:
            dims = [int(x) for x in args.shape.lower().split("x")]
            assert len(dims) == 3 and min(dims) >= 1
        except (ValueError, AssertionError):
            parser.error("--shape takes MxNxK, e.g. 8192x8192x512")
        if args.gpus > 1 or args.workload is not None:
            parser.error("--shape is a single-GPU measurement and excludes --workload")
        args.workload = workloads.register_custom(*dims)
    if args.input_dtype is not None:
        if args.gpus > 1:
            parser.error("--input-dtype is a single-GPU measurement")
        args.workload = workloads.with_input_dtype(args.workload or "gemm_8192", args.input_dtype)
    if (args.b_transposed or args.member != "plain") and args.gpus > 1:
        parser.error("--b-transposed and --member are single-GPU measurements")
    if args.b_transposed and args.member != "plain":
        parser.error("the transposed-B example is built as the plain member only")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1 and args.impl != "reference":
        # Launched without torchrun: start one rank per GPU ourselves.
        cmd = [sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
               "--nnodes=1", f"--nproc-per-node={args.gpus}", str(Path(__file__).resolve()), *sys.argv[1:]]
        return subprocess.call(cmd)

    ranks = Ranks(connect=args.impl != "reference")  # the CPU arm runs on rank 0 alone
    try:
        if args.impl == "reference":
            run_reference_arm(args, ranks)
        else:
            run_gpu_arm(args, ranks)
    finally:
        ranks.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
