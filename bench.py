#!/usr/bin/env python
"""Benchmark of the cuda backend's hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl cuda|reference]
                    [--skip-extras | --only-configs | --only-mlp]

Headline workload (`config.workload` = "softmax_lse_argmax_f32_8192x4096"): one jit program
computing softmax, log-sum-exp and argmax over the last axis of f32 X[8192, 4096] ~ N(0, 1):
ten Kernels (row max x3, exp, row sum, scale, a copy of the row max, fused exp-sum, max+log,
int32 arg-index max).  A step is one replay of that step list as a user of `jit` gets it: captured
once through the C ABI, then one CUDA graph launch per call, inside which the backend runs the
ten Kernels as one row-resident kernel.  The metric is the bytes the program must move (X in,
softmax / lse / argmax out: 268.5 MB per step) per second, summed over all GPUs; the same list
dispatched kernel by kernel is reported beside it under "unfused" with per-Kernel bytes.

With N > 1 every rank runs the same program on its own rows (independent units, no
data-path collective: "weak" scaling); the data-parallel MLP step that does exchange
gradients is reported beside it under "mlp_train".

The line also carries: `roofline` for the dominant kernel (timed with CUDA events inside the
timed region, against MEASURED_PEAKS.json), `e2e` (same program with the host->device copy
of X from pinned memory and the device->host read of all results inside every step; the reads
are the Promise form of Backend.read, so a step's read-back overlaps the next step's upload),
`cpu_baseline` (the CPU oracle, a restatement of the reference's Wasm backend, on a bounded
sample of rows), `configs` (the other benchmark configurations, one figure each) and `clocks`.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS = 8192, 4096
WORKLOAD = f"softmax_lse_argmax_f32_{ROWS}x{COLS}"
METRIC = "fused-kernel algorithmic HBM throughput (softmax + logsumexp + argmax program: bytes the program must move per second)"
UNIT = "GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the row-fused kernel, from the committed
# ncu capture named in NCU_TRAFFIC_SOURCE (not a property of this run)
NCU_TRAFFIC_ROWFUSE_BYTES = 218.5e6
NCU_TRAFFIC_SOURCE = "ncu capture of jx_rowfuse at this workload, profiles/softmax_lse_argmax_f32_8192x4096.md (a constant of that capture, not measured in this run)"


def config_dict():
    """The workload, identically in both arms."""
    return {"workload": WORKLOAD, "rows_per_gpu": ROWS, "cols": COLS, "sharding": "rows, no collective",
            "program": "jit computing softmax, logsumexp and argmax over the last axis; ten Kernels",
            "program_bytes_per_step": program_bytes(ROWS)}


def program_bytes(rows):
    """Distinct bytes the program must move: X and the index constant in, softmax, lse and argmax out."""
    return 2 * rows * COLS * 4 + 2 * rows * 4 + COLS * 4


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons while the timed region runs: NVML read calls from a
    thread every 5 ms (the region lasts tens of milliseconds, less than one period of nvidia-smi's
    loop mode); nvidia-smi in loop mode where NVML cannot be loaded.  Nothing is set, only read."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    REASON_BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        self.samples = []          # (time, sm_mhz, sm_max_mhz, [reasons])
        self.proc = None
        self.stop_flag = False
        self.source = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            try:       # the CUDA device's own UUID: NVML may number the GPUs of the machine differently
                import torch
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{torch.cuda.get_device_properties(index).uuid}")
            except Exception:
                visible = [v for v in os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",") if v.strip().isdigit()]
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(int(visible[index]) if index < len(visible) else index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self._read_nvml()
            self.source = "nvml, every 5 ms"
            self.thread = threading.Thread(target=self._poll_nvml, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.samples.clear()
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(index)], stdout=subprocess.PIPE, text=True)
            self.source = "nvidia-smi -lms 100"
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read_nvml(self):
        n = self.nvml
        mhz = int(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
        mask = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
        self.samples.append((time.time(), mhz, self.sm_max, [name for name, bit in self.REASON_BITS if mask & bit]))

    def _poll_nvml(self):
        while not self.stop_flag:
            try:
                self._read_nvml()
            except Exception:
                return
            time.sleep(0.005)

    def _pump(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7 and parts[0].isdigit():
                names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
                self.samples.append((time.time(), int(parts[0]), int(parts[1]),
                                     [n for n, v in zip(names, parts[3:7]) if v.lower().startswith("active")]))

    def inside(self, t0: float, t1: float) -> int:
        return sum(1 for s in self.samples if t0 <= s[0] <= t1)

    def stop(self, t0: float, t1: float, note: str = "") -> dict:
        """Summary of the samples taken between t0 and t1 (host clock)."""
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
        self.stop_flag = True
        rows = [s for s in self.samples if t0 <= s[0] <= t1]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "source": self.source}
        out = {"sm_mhz": statistics.median(s[1] for s in rows), "sm_max_mhz": rows[0][2],
               "reasons": sorted({r for s in rows for r in s[3]}), "samples": len(rows), "source": self.source}
        if note:
            out["note"] = note
        return out


def time_kernel(be, kernel, arrays, iters=20, warmup=3, copies=1):
    """Mean device time (ms) of one Kernel with resident inputs; returns (ms, exe).  With copies > 1
    the launches rotate over that many copies of the inputs, so that a working set smaller than the
    126 MB L2 is still streamed from HBM."""
    sets = [[be.put(a) for a in arrays] for _ in range(copies)]
    out = be.malloc(kernel.bytes)
    exe = be.prepare_kernel(kernel)
    for i in range(warmup):
        be.dispatch(exe, sets[i % copies], [out])
    be.event_record(0)
    for i in range(iters):
        be.dispatch(exe, sets[i % copies], [out])
    be.event_record(1)
    ms = be.event_elapsed_ms(0, 1) / iters
    for s in [x for st in sets for x in st] + [out]:
        be.dec_ref(s)
    return ms, exe


def other_configs(be, peaks, iters=None, warmup=None):
    """One figure for each remaining benchmark configuration (resident inputs, CUDA events).  `warmup`
    overrides every config's own warm-up count (the profiler run wants few launches)."""
    from jax_js_b200 import DType
    from jax_js_b200 import programs as P
    rng = np.random.default_rng(0)
    out = {}
    n = 1024
    a, b = rng.uniform(-1, 1, (n, n)).astype(np.float32), rng.uniform(-1, 1, (n, n)).astype(np.float32)
    ms, exe = time_kernel(be, P.dot_kernel(n, n, n), [a, b], iters=iters or 50, warmup=warmup or 3)
    out["matmul_f32_1024"] = {"tflops": 2 * n**3 / ms / 1e9, "ms": ms, "kernel": exe.describe}
    w = (rng.standard_normal((4096, 11008)) * 0.02).astype(np.float16)
    x = (rng.standard_normal(4096) * 0.02).astype(np.float16)
    for name, k, args in (("matvec_f16_xW_4096x11008", P.matvec_kernel(4096, 11008, DType.Float16, orientation="xW"), [x, w]),
                          ("matvec_f16_Wx_11008x4096", P.matvec_kernel(11008, 4096, DType.Float16, orientation="Wx"),
                           [w.reshape(11008, 4096), x])):
        ms, exe = time_kernel(be, k, args, iters=iters or 60, warmup=warmup or 3, copies=3)
        nbytes = exe.cost()[0]
        out[name] = {"gbs": nbytes / ms / 1e6, "frac_hbm": nbytes / ms / 1e6 / peaks["hbm_gbs"], "ms": ms,
                     "kernel": exe.describe, "l2": "launches rotate over 3 copies of W (270 MB), larger than L2"}
    n = 4096
    a = (rng.standard_normal((n, n)) * 0.02).astype(np.float16)
    b = (rng.standard_normal((n, n)) * 0.02).astype(np.float16)
    ms, exe = time_kernel(be, P.dot_kernel(n, n, n, DType.Float16), [a, b], iters=iters or 10, warmup=warmup or 2)
    tf = 2 * n**3 / ms / 1e9
    out["matmul_f16_4096"] = {"tflops": tf, "frac_tensor_burst": tf / peaks["bf16_tflops"], "ms": ms, "kernel": exe.describe}
    # a convolution as `jitRules[Conv]` emits it: NCHW 32 x 64 x 56 x 56, 128 filters of 3 x 3, padding 1.
    # No TF32 peak is measured: the stand-in ceiling for 3xTF32 is the measured bf16 burst / 2 / 3.
    N, Ci, H, Co = 32, 64, 56, 128
    x = rng.standard_normal((N, Ci, H, H)).astype(np.float32)
    w = (rng.standard_normal((Co, Ci, 3, 3)) * 0.05).astype(np.float32)
    flops = 2.0 * N * Co * H * H * Ci * 9
    ms, exe = time_kernel(be, P.conv2d_kernel(N, Ci, H, H, Co, 3, 3, 1, 1), [x, w], iters=iters or 10, warmup=warmup or 2)
    out["conv2d_f32_32x64x56x56_k3"] = {"tflops": flops / ms / 1e9, "frac_3xtf32_ceiling": flops / ms / 1e9 / (peaks["bf16_tflops"] / 6),
                                        "ms": ms, "kernel": exe.describe,
                                        "stages": "implicit GEMM: warp groups of the tcgen05 kernel evaluate the patch operand (and its 3xTF32 remainder) into the shared-memory stages; TMA loads the weights"}
    x16, w16 = x.astype(np.float16), w.astype(np.float16)
    ms, exe = time_kernel(be, P.conv2d_kernel(N, Ci, H, H, Co, 3, 3, 1, 1, DType.Float16), [x16, w16], iters=iters or 10, warmup=warmup or 2)
    out["conv2d_f16_32x64x56x56_k3"] = {"tflops": flops / ms / 1e9, "frac_tensor_burst": flops / ms / 1e9 / peaks["bf16_tflops"],
                                        "ms": ms, "kernel": exe.describe}
    return out


def mlp_train(be, rank, world, dist, steps=8, warmup=2):
    """Config 5: data-parallel Adam step of the 784-2048-2048-10 MLP, global batch 65536 split over
    the ranks, gradients summed with NCCL on the backend's stream.  Returns steps/s (strong scaling)."""
    import torch
    from jax_js_b200 import mlp
    from jax_js_b200.backend import CudaBackend
    dims, GB = [784, 2048, 2048, 10], 65536
    local = GB // world
    if world > 1:
        uid = [CudaBackend.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(uid, src=0)
        be.comm_init(rank, world, uid[0])
    # the same global batch at every N: 8 seeded chunks of 8192 examples, of which a rank takes its share
    chunk = GB // 8
    xs, ys = [], []
    for c in range(rank * local // chunk, ((rank + 1) * local + chunk - 1) // chunk):
        rng = np.random.default_rng(100 + c)
        xs.append(rng.uniform(0, 1, (chunk, dims[0])).astype(np.float32))
        ys.append(rng.integers(0, 10, chunk).astype(np.int32))
    off = rank * local - (rank * local // chunk) * chunk
    sx = be.put(np.concatenate(xs)[off:off + local])
    sy = be.put(np.concatenate(ys)[off:off + local])
    hoist = os.environ.get("BENCH_MLP_HOIST", "0") == "1"   # the hoisted order measured slower on eight GPUs; off
    tr = mlp.MlpTrainer(be, dims, local, GB, overlap=os.environ.get("BENCH_MLP_OVERLAP", "1") != "0", hoist=hoist)
    losses = []
    for _ in range(warmup):
        be.dec_ref(tr.step(sx, sy, world))
    be.sync()
    if dist:
        dist.barrier()
    be.event_record(2)
    for _ in range(3):                                  # the same step dispatched kernel by kernel
        be.dec_ref(tr.step(sx, sy, world))
    be.event_record(3)
    be.sync()
    eager_ms = be.event_elapsed_ms(2, 3) / 3
    tr.capture(sx, sy, world)                           # from here on a step is one graph launch
    be.dec_ref(tr.step(sx, sy, world))
    be.sync()
    if dist:
        dist.barrier()
    l0 = be.launch_count()
    be.event_record(0)
    for _ in range(steps):
        s = tr.step(sx, sy, world)
        losses.append(s)
    be.event_record(1)
    be.sync()
    ms = be.event_elapsed_ms(0, 1)
    launches = be.launch_count() - l0
    vals = [float(be.get(losses[-1], "float32")[0])] * 2   # a captured step rewrites one loss slot in place
    for s in losses:
        be.dec_ref(s)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    flops = 2.0 * GB * (784 * 2048 + 2048 * 2048 + 2048 * 10) * 3 - 2.0 * GB * 784 * 2048
    tr.close()
    phases = None
    if world > 1:
        # the same shard without the sums (a trainer of its own, world 1 on the local batch): what the
        # step costs in kernels alone; the rest of the step is sums that nothing hides and waiting
        # for the slowest rank
        solo = mlp.MlpTrainer(be, dims, local, GB, hoist=hoist)
        for _ in range(2):
            be.dec_ref(solo.step(sx, sy, 1))
        solo.capture(sx, sy, 1)
        be.dec_ref(solo.step(sx, sy, 1))
        be.sync()
        be.event_record(4)
        for _ in range(steps):
            be.dec_ref(solo.step(sx, sy, 1))
        be.event_record(5)
        be.sync()
        ts = torch.tensor([be.event_elapsed_ms(4, 5) / steps], dtype=torch.float64, device="cuda")
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        solo.close()
        phases = {"shard_kernels_ms": float(ts.item()), "sums_and_waiting_ms": ms / steps - float(ts.item()),
                  "note": "shard_kernels_ms: the same local batch replayed without the gradient sums (max over ranks)"}
    be.dec_ref(sx)
    be.dec_ref(sy)
    return {"steps_per_s": steps / ms * 1e3, "ms_per_step": ms / steps, "global_batch": GB, "local_batch": local,
            "tflops_algorithmic": flops * steps / ms / 1e9, "scaling": "strong", "launches_per_step": launches / steps,
            "allreduce_bytes": 4 * sum(mlp.leaf_sizes(dims)), "loss_last": vals[-1],
            "replay": "one CUDA graph launch per step (gradient program + NCCL sum + Adam program; two graphs alternate between two state buffers)",
            "gradient_sum": "per layer on a second stream, under back-propagation" if tr.overlap and world > 1 else "after the gradient program",
            "kernel_order": "the reference's list with the weight-gradient Kernels of layers 2.. moved to where their inputs exist (same Kernels, same bits)"
                            if tr.hoist else "the reference's list",
            "eager_ms_per_step": eager_ms, "phases": phases,
            "gemm": "3xTF32 on tcgen05 (f32 accuracy), f32 accumulate"}


def vmap_grad(be, rank, world, dist, steps=30, warmup=3):
    """Config 4: per-example value-and-gradient of the 784-1024-10 MLP under vmap, batch 64 split in
    contiguous chunks over the ranks (independent units, no collective).  Returns steps/s."""
    import torch
    from jax_js_b200 import mlp
    dims, GB = [784, 1024, 10], 64
    local = GB // world
    rng = np.random.default_rng(7)
    x = rng.uniform(0, 1, (GB, dims[0])).astype(np.float32)[rank * local:(rank + 1) * local]
    y = rng.integers(0, 10, GB).astype(np.int32)[rank * local:(rank + 1) * local]
    prog = mlp.mlp_grad_program(local, dims, per_example=True)
    prog.prepare(be)
    slots = [be.put(x), be.put(y), be.put(np.eye(10, dtype=np.float32))] + [be.put(p) for p in mlp.init_params(dims)]
    nbytes = prog.cost(be)[0]

    for _ in range(warmup):
        for s in prog.execute(be, slots):
            be.dec_ref(s)
    graph, outs = prog.capture(be, slots)
    launches, graph_bytes, fused = be.graph_cost(graph)
    be.graph_launch(graph)
    be.sync()
    if dist:
        dist.barrier()
    be.event_record(0)
    for _ in range(steps):
        be.graph_launch(graph)
    be.event_record(1)
    be.sync()
    for s in outs:
        be.dec_ref(s)
    be.graph_destroy(graph)
    t = torch.tensor([be.event_elapsed_ms(0, 1)], dtype=torch.float64, device="cuda")
    if dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    for s in slots:
        be.dec_ref(s)
    return {"steps_per_s": steps / ms * 1e3, "ms_per_step": ms / steps, "batch": GB, "local_batch": local,
            "algorithmic_gbs": graph_bytes * world * steps / ms / 1e6, "scaling": "strong",
            "bytes_per_step": graph_bytes, "bytes_per_step_kernel_by_kernel": nbytes,
            "kernels_per_step": launches, "fused_runs": fused,
            "memory": "L2-resident: this rank's arrays fit the 126 MB L2, so the figure is not HBM throughput"
                      if graph_bytes < 126e6 else "streams from HBM",
            "note": "per-example dW1 is f32[batch,784,1024]; the reference's list writes it batch-last and moves the batch axis "
                    "first in a second Kernel, the captured replay substitutes the product into that Kernel and writes it once; "
                    "bytes are what the launched kernels address (inputs + outputs), summed"}


def oracle_program_runner(rows, threads):
    """Builds the program and its inputs once; returns a function that replays the Kernel list on the
    CPU oracle and gives the seconds it took."""
    import oracle
    from jax_js_b200 import np_dtype
    from jax_js_b200 import programs as P
    oracle.build()
    prog = P.softmax_lse_argmax_program(rows, COLS)
    x = np.random.default_rng(1).standard_normal((rows, COLS)).astype(np.float32)
    iota = P.argmax_iota(COLS)
    bufs = {s.name: np.empty(s.kernel.size, np_dtype(s.kernel.dtype)) for s in prog.steps if s.kind == "execute"}

    def run():
        env = {"x": x, "iota": iota}
        t0 = time.perf_counter()
        for s in prog.steps:
            if s.kind == "execute":
                env[s.name] = oracle.run_kernel(s.kernel, [env[n] for n in s.inputs], out=bufs[s.name], threads=threads,
                                                mode=oracle.MODE_WASM)
        return time.perf_counter() - t0
    return run


def cpu_baseline(budget_s=10.0, threads=1):
    """The oracle (port of the reference's Wasm backend arithmetic) on a bounded sample of rows."""
    probe_rows = 64
    t = oracle_program_runner(probe_rows, threads)()
    rows = int(min(ROWS, max(probe_rows, probe_rows * budget_s / max(t, 1e-6))))
    rows = max(64, rows // 64 * 64)
    t = oracle_program_runner(rows, threads)()
    return {"value": program_bytes(rows) / t / 1e9, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"{rows} of {ROWS} rows of the same program (ten Kernels, unfused), {t:.2f} s, oracle in Wasm-semantics mode",
            "host_cores": os.cpu_count()}


def run_reference(args):
    """The reference arm: the CPU restatement of the reference's Wasm arithmetic on all host threads.
    A step is one replay of the program on a bounded sample of rows; only the replays are timed."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    threads = len(os.sched_getaffinity(0))
    warmup = args.warmup if args.warmup is not None else 1
    steps = args.steps if args.steps is not None else 3
    probe = oracle_program_runner(64, threads)
    probe()
    t = probe()
    # rows per step so that warm-up plus timed steps take about 40 s at most
    rows = int(min(ROWS, max(64, 64 * 40.0 / max(t, 1e-6) / max(1, steps + warmup))))
    rows = max(64, rows // 64 * 64)
    run = oracle_program_runner(rows, threads)
    for _ in range(max(1, warmup)):
        run()
    dt = sum(run() for _ in range(steps))
    v = program_bytes(rows) * steps / dt / 1e9
    base = {"value": v, "unit": UNIT, "cores": threads, "kind": "port", "host_cores": os.cpu_count(),
            "sample": f"{rows} of {ROWS} rows per step, {steps} steps, {dt:.2f} s; reference Wasm-under-Node unavailable on this box "
                      "(no JS runtime): C++ restatement of its arithmetic, OpenMP over the output range as the browser worker pool splits it"}
    return {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
            "warmup": warmup, "ms_per_step": dt / steps * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config_dict(), "cpu_baseline": base,
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}


def main():
    # stdout carries exactly one JSON line: libraries that print there (NCCL's version banner) are
    # sent to stderr for the duration of the run
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        line = _run()
    finally:
        sys.stdout.flush()
        os.dup2(real_stdout, 1)
    if line:
        print(json.dumps(line), flush=True)


def _run():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--skip-extras", action="store_true", help="only the headline program (used under ncu)")
    ap.add_argument("--only-configs", action="store_true",
                    help="run each remaining config kernel a few times and print their figures (used under ncu)")
    ap.add_argument("--only-mlp", action="store_true", help="only the data-parallel MLP training step")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.only_configs:
        from jax_js_b200.backend import CudaBackend
        be = CudaBackend(int(os.environ.get("LOCAL_RANK", "0")))
        out = {"configs": other_configs(be, measured_peaks(), iters=args.steps or 2, warmup=args.warmup)}
        be.close()
        return out
    steps = args.steps if args.steps is not None else 1000
    warmup = max(3, args.warmup if args.warmup is not None else 10)

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    import torch
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    from jax_js_b200 import DType
    from jax_js_b200 import programs as P
    from jax_js_b200.backend import CudaBackend
    be = CudaBackend(local)           # raises when the library or the GPU is missing: no fallback
    peaks = measured_peaks()
    if args.only_mlp:
        train = mlp_train(be, rank, world, dist, steps=args.steps or 50)
        be.close()
        if dist:
            dist.barrier()
            dist.destroy_process_group()
        return {"n_gpus": world, "mlp_train": train} if rank == 0 else None

    rng = np.random.default_rng(rank)
    x_host = be.host_alloc(ROWS * COLS * 4)
    x_host.view(np.float32)[:] = rng.standard_normal(ROWS * COLS, dtype=np.float32)
    iota = P.argmax_iota(COLS)
    prog = P.softmax_lse_argmax_program(ROWS, COLS)
    prog.prepare(be)
    A, R4 = ROWS * COLS * 4, ROWS * 4
    # two copies of X and two captured replays that alternate: between two reads of the same copy the
    # GPU moves four times the 126 MB L2
    sxs, si = [be.malloc(A), be.malloc(A)], be.put(iota)
    for s_ in sxs:
        be.write(s_, x_host)
    exec_steps = [s for s in prog.steps if s.kind == "execute"]
    nk = len(exec_steps)
    unfused_bytes = prog.cost(be)[0]

    def barrier():
        be.sync()
        if dist:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        if dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def run_step(ev_base=None, x_slot=None):
        """Replays the jit step list kernel by kernel; with ev_base, brackets every dispatch with events."""
        env, j = {"x": sxs[0] if x_slot is None else x_slot, "iota": si}, 0
        for s in prog.steps:
            if s.kind == "malloc":
                env[s.name] = be.malloc(s.nbytes)
            elif s.kind == "execute":
                if ev_base is not None:
                    be.event_record(ev_base + 2 * j)
                be.dispatch(prog._exes[id(s)], [env[n] for n in s.inputs], [env[s.name]])
                if ev_base is not None:
                    be.event_record(ev_base + 2 * j + 1)
                j += 1
            elif s.kind == "free":
                be.dec_ref(env.pop(s.name))
        return [env[n] for n in prog.outputs]

    def drop(outs):
        for s in outs:
            be.dec_ref(s)

    # the call a user makes: the jit program captured once, then one graph launch per step
    graphs, gouts = [], []
    for s_ in sxs:
        g, o = prog.capture(be, [s_, si])
        graphs.append(g)
        gouts.append(o)
    launches_per_step, step_bytes, fused_groups = be.graph_cost(graphs[0])
    for i in range(warmup):
        be.graph_launch(graphs[i % 2])
    sampler = ClockSampler(local) if rank == 0 else None
    barrier()
    launches0 = be.launch_count()
    t0 = time.time()
    be.event_record(0)
    for i in range(steps):
        be.graph_launch(graphs[i % 2])
    be.event_record(1)
    barrier()
    t1 = time.time()
    ms_max = max_over_ranks(be.event_elapsed_ms(0, 1))
    launches = be.launch_count() - launches0
    clocks = None
    if sampler:
        note = ""
        if sampler.inside(t0, t1) < 3:
            # the sampler was slower than the region: keep the GPU on the same step (untimed) until it has seen it
            t_ext = time.time()
            while time.time() - t_ext < 0.6 and sampler.inside(t0, time.time()) < 5:
                for i in range(100):
                    be.graph_launch(graphs[i % 2])
                be.sync()
            t1 = time.time()
            note = "the timed region was shorter than the sampling period: samples include the same step replayed right after it"
        clocks = sampler.stop(t0, t1, note)
    value = step_bytes * steps * world / ms_max / 1e6

    # beside it: the same step list dispatched kernel by kernel (what the backend does outside a
    # capture), first untimed per kernel, then a separate pass with an event pair around every dispatch
    un_steps = max(3, min(steps, 200))
    for _ in range(3):
        drop(run_step())
    barrier()
    be.event_record(0)
    for i in range(un_steps):
        drop(run_step(x_slot=sxs[i % 2]))
    be.event_record(1)
    barrier()
    unfused_ms = max_over_ranks(be.event_elapsed_ms(0, 1)) / un_steps
    traced = min(un_steps, 50)
    for i in range(traced):
        drop(run_step(2 + i * 2 * nk, x_slot=sxs[i % 2]))
    barrier()
    per_kernel = []
    for j, s in enumerate(exec_steps):
        ms = statistics.mean(be.event_elapsed_ms(2 + i * 2 * nk + 2 * j, 2 + i * 2 * nk + 2 * j + 1) for i in range(traced))
        b, _, _ = prog._exes[id(s)].cost()
        per_kernel.append({"out": s.name, "kernel": prog._exes[id(s)].describe, "ms": ms, "bytes": b, "gbs": b / ms / 1e6})

    # end to end: pinned host X in, all three results out, every step, through the same public calls.
    # The reads are the Promise form of Backend.read (read_async / read_wait): step i's results come
    # back while step i+1 uploads and computes, as a JS caller awaiting the previous step would see it;
    # every step's upload and read-back completes inside the timed region.
    e2e_steps = max(3, min(steps, 20))
    h2d, d2h = A, A + 2 * R4
    out_hosts = [be.host_alloc(A + 2 * R4) for _ in range(2)]

    def e2e_issue(i):
        k, oh = i % 2, out_hosts[i % 2]
        be.write_async(sxs[k], x_host)
        be.graph_launch(graphs[k])
        o = gouts[k]
        return [be.read_async(o[0], oh[:A]), be.read_async(o[1], oh[A: A + R4]), be.read_async(o[2], oh[A + R4:])]

    def e2e_finish(tickets):
        for t in tickets:
            be.read_wait(t)

    e2e_finish(e2e_issue(0))
    barrier()
    te = time.perf_counter()
    pending = None
    for i in range(e2e_steps):
        cur = e2e_issue(i)
        if pending:
            e2e_finish(pending)
        pending = cur
    e2e_finish(pending)
    barrier()
    e2e_s = max_over_ranks(time.perf_counter() - te)
    e2e_value = step_bytes * e2e_steps * world / e2e_s / 1e9
    # the same with blocking calls (write, launch, read, one after the other), for comparison
    tb = time.perf_counter()
    for _ in range(3):
        be.write(sxs[0], x_host)
        be.graph_launch(graphs[0])
        be.read_into(gouts[0][0], out_hosts[0][:A])
        be.read_into(gouts[0][1], out_hosts[0][A: A + R4])
        be.read_into(gouts[0][2], out_hosts[0][A + R4:])
    e2e_blocking_ms = (time.perf_counter() - tb) / 3 * 1e3

    line = None
    if rank == 0:
        kernel_ms = ms_max / steps / max(1, launches_per_step)
        fused_desc = "row-fused kernel" if fused_groups else "unfused"
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_max / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": config_dict(),
            # placed early so that a reader of the line's head sees them
            "configs_head": None,
            "step": {"replay": "captured step list, one CUDA graph launch per step; two graphs alternate between two copies of X",
                     "kernels_per_step": int(launches_per_step), "fused_runs": int(fused_groups),
                     "algorithmic_bytes_per_step": step_bytes, "timed_region_ms": ms_max,
                     "l2": "each step streams 268 MB (X in, softmax out) through the 126 MB L2; a copy of X is read again only after 537 MB of other traffic"},
            "unfused": {"value": unfused_bytes * world / unfused_ms / 1e6, "unit": UNIT, "ms_per_step": unfused_ms,
                        "kernels_per_step": nk, "algorithmic_bytes_per_step": unfused_bytes,
                        "program_bytes_gbs": step_bytes * world / unfused_ms / 1e6,
                        "note": "the same step list dispatched kernel by kernel (outside a capture); bytes are per Kernel: distinct input bytes + output bytes"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_s / e2e_steps * 1e3,
                    "calls": "write_async + graph_launch + read_async per step, read_wait one step later",
                    "blocking_calls_ms_per_step": e2e_blocking_ms},
            "gpu_launches": int(launches),
            "roofline": {"bound": "hbm", "achieved": step_bytes / kernel_ms / 1e6 if launches_per_step == 1 else None,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": step_bytes / kernel_ms / 1e6 / peaks["hbm_gbs"] if launches_per_step == 1 else None,
                         "traffic": NCU_TRAFFIC_ROWFUSE_BYTES, "traffic_source": NCU_TRAFFIC_SOURCE,
                         "kernel": fused_desc, "ms": kernel_ms, "algorithmic_bytes": step_bytes,
                         "timing": "CUDA events around the timed steps on the backend's stream; each step is this one kernel",
                         "peak_source": peaks["source"]},
            "kernels": [{k: (round(v, 5) if isinstance(v, float) else v) for k, v in pk.items()} for pk in per_kernel],
            "clocks": clocks,
        }
        if launches_per_step != 1:      # fusion off (JAXCUDA_FUSE=0): the dominant kernel of the unfused list
            top = max(per_kernel, key=lambda k: k["ms"])
            line["roofline"].update({"achieved": top["gbs"], "frac": top["gbs"] / peaks["hbm_gbs"], "kernel": top["kernel"],
                                     "ms": top["ms"], "algorithmic_bytes": top["bytes"], "traffic": None})
        if world == 1 and not args.skip_extras:
            cfgs = other_configs(be, peaks)
            line["configs_head"] = {k: {kk: vv for kk, vv in v.items() if kk in ("tflops", "gbs", "ms", "frac_hbm", "frac_tensor_burst", "frac_3xtf32_ceiling")}
                                    for k, v in cfgs.items()}
            line["configs"] = cfgs
            line["cpu_baseline"] = cpu_baseline(budget_s=10.0, threads=1)
    if not args.skip_extras:
        train = mlp_train(be, rank, world, dist)
        vg = vmap_grad(be, rank, world, dist)
        if line:
            line["mlp_train"] = train
            line["vmap_grad"] = vg
    for g, o in zip(graphs, gouts):
        drop(o)
        be.graph_destroy(g)
    for s in sxs + [si]:
        be.dec_ref(s)
    be.host_free(x_host)
    for oh in out_hosts:
        be.host_free(oh)
    be.close()
    if dist:
        dist.barrier()
        dist.destroy_process_group()
    return line


if __name__ == "__main__":
    main()
