#!/usr/bin/env python
"""Benchmark of the B200 execution backend on its five configured workloads.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Headline (one JSON line on stdout): fused row softmax, fp32 65,536 x 4,096 per
GPU, launched through the Triton driver plugin.  A "step" is one launch of the
kernel over one batch of rows.  `value` is timed with inputs resident in HBM;
`e2e` repeats the measurement through the same public call with pinned HOST
buffers, the host->device and device->host copies inside the timed region.
The other workloads (masked vector add 2^30, LayerNorm 4096x8192 fp16, strided
masked reduction 8192x12288, bf16 matmul 8192^3) are timed the same way after
the headline region and reported under "workloads".

Multi-GPU (torchrun, one rank per GPU): every rank owns a contiguous range of
the global grid's programs (N x the single-GPU rows) and its shard of the data;
there is no data-path collective (only the strided-reduction workload combines
one scalar with an NCCL all-reduce).  Timing: CUDA events per rank, max over ranks.

`--impl reference` times the CPU restatement of the reference backend (oracle/)
on the host cores for the same workload on a bounded sample; the reference's own
CPU backend needs MLIR/LLVM tools that this environment does not have.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

SOFTMAX_ROWS, SOFTMAX_COLS = 65_536, 4_096
ADD_N = 1 << 30
LN_M, LN_N = 4_096, 8_192
RED_M, RED_N, RED_NV = 8_192, 12_288, 12_000
MM = 8_192

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per launch from the ncu
# captures summarised under profiles/; None until a capture exists for the kernel.
# Captures on reduced cases are scaled to the full-size launch by rows / elements (traffic is
# proportional for these kernels); the summaries give the raw figures and the commands.
NCU_TRAFFIC_BYTES = {
    "softmax": 1.94216e9,         # 65,536 x 4,096: 4 x (268.46 MB read + 217.08 MB written) at 16,384 rows
    "vec_add": 12.5733e9,         # n = 2^30: 8 x (1.0738 GB + 497.8 MB) at n = 2^27
    "layernorm": 121.3e6,         # 4,096 x 8,192 fp16: 485.2 MB / 4 at 16,384 rows
    "strided_reduce": 396.7e6,    # full size, the cluster row kernel
    "matmul": 1.57206e9,          # 8192^3 bf16, two-CTA kernel: 1.4427 GB read + 129.3 MB written
    "block_copy": 1.86488e9,      # 16,000 x 16,000 fp32: 4 x (256.04 MB + 210.18 MB) at 8,000 x 8,000
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            j = json.load(f)
        return {"hbm": float(j["hbm_gbs"]), "tensor": float(j["bf16_tflops"]),
                "tensor_sustained": float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), "src": "measured"}
    return {"hbm": 6650.0, "tensor": 1590.0, "tensor_sustained": 1400.0, "src": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in self.lines:
            f = [x.strip() for x in l.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(names, f[5:9]):
                if v.lower() == "active":
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def bind_to_gpu_numa_node(gpu_index: int):
    """Restrict this process to the CPUs of the NUMA node the GPU hangs off, so that pinned host
    buffers allocated afterwards are local to it.  Best effort: returns what was done."""
    try:
        import torch
        bus = torch.cuda.get_device_properties(gpu_index).pci_bus_id
        dom = getattr(torch.cuda.get_device_properties(gpu_index), "pci_domain_id", 0)
        dev = torch.cuda.get_device_properties(gpu_index).pci_device_id
        path = f"/sys/bus/pci/devices/{dom:04x}:{bus:02x}:{dev:02x}.0/numa_node"
        with open(path) as f:
            node = int(f.read().strip())
        if node < 0:
            return {"node": None, "note": "the platform reports no NUMA node for the GPU"}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"node": node, "note": "none of the node's CPUs is available to this process"}
        os.sched_setaffinity(0, allowed)
        return {"node": node, "cpus": len(allowed)}
    except Exception as e:  # noqa: BLE001 - placement is an optimisation, never a failure
        return {"node": None, "note": f"{type(e).__name__}: {e}"[:120]}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all",
                    help="which secondary workloads to time after the softmax headline: all, none, or a "
                         "comma-separated subset of vec_add,layernorm,strided_reduce,matmul")
    ap.add_argument("--small", action="store_true",
                    help="reduced sizes (still larger than L2) and 3 timed steps, for profiler captures")
    ap.add_argument("--rows", type=int, default=SOFTMAX_ROWS, help="softmax rows per GPU (smaller for profiling captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="time eager plugin launches instead of a replayed CUDA graph")
    return ap.parse_args()


# ----------------------------------------------------------------------------------------
# CPU legs (oracle): the one place besides tests where oracle/ is executed

def cpu_softmax_rate(seconds_target=10.0, threads=None):
    """GB/s of the oracle's softmax on a bounded sample of the 4,096-column workload: passes over
    (at most) the full 65,536-row batch are repeated until about `seconds_target` of CPU work."""
    import numpy as np
    import oracle
    oracle.build()
    threads = threads or oracle.max_threads()
    rng = np.random.default_rng(1)
    rows = min(SOFTMAX_ROWS, 1024 * threads)
    rows -= rows % threads
    x = rng.standard_normal((rows, SOFTMAX_COLS), dtype=np.float32)
    out = np.empty_like(x)
    oracle.softmax(x, 4096, threads=threads, out=out)  # warm-up (page faults, thread start)
    passes, t0 = 0, time.perf_counter()
    while True:
        oracle.softmax(x, 4096, threads=threads, out=out)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= seconds_target or passes >= 200:
            break
    gbs = rows * SOFTMAX_COLS * 8 * passes / dt / 1e9
    return gbs, threads, (rows, passes), dt


def cpu_baselines(seconds_each=1.5):
    """The oracle (CPU restatement of the reference's lowered loops) on bounded samples of the other
    workloads, at one thread (the reference launcher runs the grid serially on one thread,
    backend/driver.py:116-133) and at all host threads.  Rates are in the workload's own unit."""
    import numpy as np
    import oracle
    oracle.build()
    nthr = oracle.max_threads()
    rng = np.random.default_rng(7)
    out = {}

    def rate(fn, work, unit):
        res = {}
        for label, t in (("one_thread", 1), ("all_threads", nthr)):
            fn(t)  # warm-up
            n, t0 = 0, time.perf_counter()
            while True:
                fn(t)
                n += 1
                dt = time.perf_counter() - t0
                if dt >= seconds_each or n >= 50:
                    break
            res[label] = {"value": work * n / dt / unit[1], "cores": t, "passes": n, "seconds": round(dt, 2)}
        res["unit"], res["kind"] = unit[0], "port"
        return res

    n = 1 << 22
    x, y = rng.random(n, dtype=np.float32), rng.random(n, dtype=np.float32)
    o = np.empty(n, dtype=np.float32)
    out["vec_add"] = rate(lambda t: oracle.vec_add(x, y, n, 1024, threads=t, out=o), 12 * n, ("GB/s", 1e9))
    out["vec_add"]["sample"] = f"{n} of {ADD_N} elements per pass"
    rows = 64
    xh = rng.standard_normal((rows, LN_N), dtype=np.float32).astype(np.float16)
    w = (rng.random(LN_N, dtype=np.float32) + 0.5).astype(np.float16)
    b = (0.1 * rng.standard_normal(LN_N, dtype=np.float32)).astype(np.float16)
    out["layernorm"] = rate(lambda t: oracle.layernorm_fwd(xh, w, b, 1e-5, 1024, threads=t), 4 * rows * LN_N, ("GB/s", 1e9))
    out["layernorm"]["sample"] = f"{rows} of {LN_M} rows x {LN_N} columns per pass"
    M, NT, NV = 1024, 1536, 1500
    flat = rng.standard_normal(M * NT, dtype=np.float32)
    out["strided_reduce"] = rate(lambda t: oracle.reduce_rows(flat, M, NV, 1, M, 64, 64, threads=t), 4 * M * NV, ("GB/s", 1e9))
    out["strided_reduce"]["sample"] = f"{M} x {NV} of {RED_M} x {RED_NV} (strides [1, {M}]) per pass"
    mm, mk = 1024, 128
    bits = lambda a: (a.view(np.uint32) >> 16).astype(np.uint16)  # bf16 by truncation: timing only
    A = bits(rng.random((mm, mk), dtype=np.float32) * 2 - 1)
    B = bits(rng.random((mk, mm), dtype=np.float32) * 2 - 1)
    out["matmul"] = rate(lambda t: oracle.matmul(A, B, oracle.BF16, 128, 256, 64, 8, threads=t), 2.0 * mm * mm * mk, ("TFLOP/s", 1e12))
    out["matmul"]["sample"] = f"{mm} x {mm} x {mk} of {MM}^3 per pass ({(mm // 128) * (mm // 256)} programs)"
    return out


def run_reference(args):
    """Reference arm: the CPU restatement of the reference backend on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import oracle
    oracle.build()
    threads = oracle.max_threads()
    rows = 256 * threads  # bounded sample of the 65,536-row batch per step
    rng = np.random.default_rng(1)
    x = rng.standard_normal((rows, SOFTMAX_COLS), dtype=np.float32)
    out = np.empty_like(x)
    for _ in range(args.warmup):
        oracle.softmax(x, 4096, threads=threads, out=out)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.softmax(x, 4096, threads=threads, out=out)
    dt = time.perf_counter() - t0
    gbs = rows * SOFTMAX_COLS * 8 * args.steps / dt / 1e9
    sample = f"{rows} of {SOFTMAX_ROWS} rows x {SOFTMAX_COLS} cols per step, {threads} host threads"
    line = {
        "impl": "reference", "metric": "row softmax throughput (algorithmic bytes: 1 read + 1 write per element)",
        "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"fused row softmax fp32 {SOFTMAX_ROWS}x{SOFTMAX_COLS}, BLOCK 4096", "sample": sample},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "reference CPU backend needs triton-shared-opt/mlir-opt/llc (absent here); this times its C++ restatement",
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------

def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist
    import triton_shared_b200
    import kernels as K

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    # libraries (NCCL's version banner, for one) write to file descriptor 1: send that to stderr
    # until the result line is printed
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this backend has no CPU execution path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        # keep stdout to the one JSON line: NCCL prints its version banner there at VERSION level
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    drv = triton_shared_b200.activate()
    peaks = measured_peaks()
    stream = torch.cuda.current_stream()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, steps, warmup, launches_per_call=1, graph=True):
        """Time `steps` calls of fn on the current stream with CUDA events.

        graph=True: one call of fn is captured into a CUDA graph after warm-up and the graph is
        replayed `steps` times, so the device never waits for the Python host between launches
        (the kernels here run for tens of microseconds; an eager loop would time the host).
        Returns (total ms, max over ranks; mean ms per kernel launch on this rank)."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize()
        run = fn
        if graph:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                fn()
            run = g.replay
            run()
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(torch.cuda.current_stream())
        for _ in range(steps):
            run()
        e1.record(torch.cuda.current_stream())
        torch.cuda.synchronize()
        total = e0.elapsed_time(e1)
        barrier()
        return max_over_ranks(total), total / (steps * launches_per_call)

    # ------------------------------------------------------------------ headline: softmax
    rows, cols = args.rows, SOFTMAX_COLS
    g_rows = rows * world  # global grid; this rank owns programs [rank*rows, (rank+1)*rows)
    torch.manual_seed(1 + rank)
    x = torch.randn(rows, cols, device="cuda")
    y = torch.empty_like(x)
    lo = rank * rows
    # kernels index rows by the global program id: pass pointers to virtual row 0
    DP = triton_shared_b200.DevicePtr
    x_virt = DP(x.data_ptr() - lo * cols * 4, torch.float32)
    y_virt = DP(y.data_ptr() - lo * cols * 4, torch.float32)

    def softmax_step():
        with drv.partition(rank, world):
            K.softmax_kernel[(g_rows,)](y_virt, x_virt, cols, cols, cols, BLOCK_SIZE=4096)

    sampler = ClockSampler(local_rank)
    sampler.start()
    time.sleep(0.3)  # let the sampler deliver its first lines before the timed region
    total_ms, per_launch_ms = timed(softmax_step, args.steps, max(args.warmup, 3), graph=not args.eager)
    eager_ms, _ = timed(softmax_step, args.steps, 3, graph=False)
    alg_bytes = rows * cols * 8  # per rank per launch
    value = alg_bytes * world * args.steps / (total_ms * 1e-3) / 1e9
    achieved = alg_bytes / (per_launch_ms * 1e-3) / 1e9
    ok = torch.allclose(y.sum(dim=1), torch.ones(rows, device="cuda"), rtol=1e-4)

    # end to end: pinned host buffers, H2D + launch + D2H inside the timed region.  The rank's host
    # threads (and so the pages it pins) are first bound to the CPUs of the GPU's own NUMA node.
    numa = bind_to_gpu_numa_node(local_rank)
    hx = torch.randn(rows, cols).pin_memory()
    hy = torch.empty(rows, cols).pin_memory()

    # One step = the whole batch from host memory to host memory.  The batch is cut into
    # chunks of rows; chunk c is launched as the program range of its rows as soon as its
    # host->device copy has landed, and is copied back while later chunks are still in flight,
    # so the two copy directions and the kernel overlap (three streams, events between them).
    n_chunks = 32 if rows % 32 == 0 and rows >= 1024 else (8 if rows % 8 == 0 and rows >= 64 else 1)
    crow = rows // n_chunks
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(n_chunks)]
    ev_k = [torch.cuda.Event() for _ in range(n_chunks)]

    def e2e_step():
        main = torch.cuda.current_stream()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for c in range(n_chunks):
            r0, r1 = c * crow, (c + 1) * crow
            with torch.cuda.stream(s_in):
                x[r0:r1].copy_(hx[r0:r1], non_blocking=True)
                ev_in[c].record(s_in)
            main.wait_event(ev_in[c])
            with drv.program_range(lo + r0, lo + r1):
                K.softmax_kernel[(g_rows,)](y_virt, x_virt, cols, cols, cols, BLOCK_SIZE=4096)
            ev_k[c].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_k[c])
                hy[r0:r1].copy_(y[r0:r1], non_blocking=True)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    e2e_steps = max(3, min(args.steps, 10))
    e2e_ms, _ = timed(e2e_step, e2e_steps, 3, graph=False)
    e2e_value = alg_bytes * world * e2e_steps / (e2e_ms * 1e-3) / 1e9
    e2e_ok = bool(torch.allclose(hy.sum(dim=1), torch.ones(rows), rtol=1e-4))

    # the host-side ceiling of that pipeline: the same chunked H2D and D2H copies with no kernel
    # between them, all ranks at once (what the host's memory system and PCIe give N GPUs together)
    def copy_only_step():
        main = torch.cuda.current_stream()
        s_in.wait_stream(main)
        s_out.wait_stream(main)
        for c in range(n_chunks):
            r0, r1 = c * crow, (c + 1) * crow
            with torch.cuda.stream(s_in):
                x[r0:r1].copy_(hx[r0:r1], non_blocking=True)
                ev_in[c].record(s_in)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_in[c])
                hy[r0:r1].copy_(y[r0:r1], non_blocking=True)
        main.wait_stream(s_out)
        main.wait_stream(s_in)
    copy_ms, _ = timed(copy_only_step, e2e_steps, 2, graph=False)
    copy_value = alg_bytes * world * e2e_steps / (copy_ms * 1e-3) / 1e9
    clocks = sampler.stop()  # sampled across the headline and end-to-end timed regions
    del hx, hy

    line = {
        "metric": "row softmax throughput (algorithmic bytes: 1 read + 1 write per element)",
        "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"fused row softmax fp32 {rows}x{cols} per GPU, BLOCK 4096, one program per row",
                   "l2": "inputs (1 GiB read + 1 GiB written per launch) exceed the 126 MB L2",
                   "partition": f"contiguous program ranges, {rows} rows per GPU, no collective",
                   "timing": ("one launch captured in a CUDA graph, replayed K times" if not args.eager else "eager launches"),
                   "eager_ms_per_step": eager_ms / args.steps,
                   "result_check": "row sums == 1" if ok else "FAILED row-sum check"},
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm"],
                     "traffic": NCU_TRAFFIC_BYTES["softmax"] * rows / SOFTMAX_ROWS,
                     "peak_source": f"of {peaks['src']}", "frac_of_nominal_8TBs": achieved / 8000.0},
        "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": rows * cols * 4 * world,
                "d2h_bytes_per_step": rows * cols * 4 * world, "steps": e2e_steps,
                "pipeline": f"{n_chunks} row chunks per step: H2D, kernel and D2H on three streams",
                "host_numa": numa,
                "copy_only": {"value": copy_value, "unit": "GB/s",
                              "note": "same pinned H2D + D2H chunks with no kernel, all ranks at once: the host-side ceiling"},
                "result_check": e2e_ok},
        "gpu_launches": args.steps,
        "clocks": clocks,
    }
    del x, y
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ secondary workloads
    # the five configured workloads, the block copy, and three kernels that run on the general engines
    # (elementwise VM, block programs, device-side loops) rather than on dedicated kernels
    names = {"vec_add", "layernorm", "strided_reduce", "matmul", "block_copy", "gelu_bias", "bias_chain", "rmsnorm", "row_stats", "wrap_rows",
             "gather_rows"}
    chosen = names if args.workload == "all" else {w for w in args.workload.split(",") if w in names}
    if chosen:
        wl = {}
        steps2, warm2 = (3, 3) if args.small else (10, 3)

        def record(name, fn, alg, unit_scale, bound, unit, nbuf=1, launches=1, graph=True):
            """fn runs the workload once per rotating buffer set (nbuf passes of `alg` work)."""
            smp = ClockSampler(local_rank)
            smp.start()
            time.sleep(0.25)
            try:
                tot, per = timed(fn, steps2, warm2, launches_per_call=nbuf, graph=graph and not args.eager)
            except Exception as e:  # an unsupported family is reported, never hidden
                smp.stop()
                wl[name] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
                return
            clk = smp.stop()
            rate = alg / (per * 1e-3) / unit_scale
            peak = peaks["hbm"] if bound == "hbm" else peaks["tensor"]
            wl[name] = {"value": alg * world * steps2 * nbuf / (tot * 1e-3) / unit_scale, "unit": unit,
                        "ms_per_pass": per, "roofline": {"bound": bound, "achieved": rate, "peak": peak,
                                                         "frac": rate / peak, "unit": unit,
                                                         "traffic": NCU_TRAFFIC_BYTES.get(name),
                                                         "peak_source": f"of {peaks['src']}"},
                        "gpu_launches": steps2 * launches * nbuf, "rotating_buffers": nbuf, "clocks": clk}

        def host_us_per_launch(fn, n=200):
            """Host time to enqueue one launch through the plugin (plan evaluation, ctypes call, kernel
            launch): wall time of a burst of eager launches that is not synchronised until its end."""
            fn()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            dt = time.perf_counter() - t0
            torch.cuda.synchronize()
            return dt / n * 1e6

        def wl_vec_add():
            # masked vector add, 2^30 fp32 per GPU
            n = ADD_N >> 3 if args.small else ADD_N
            a = torch.rand(n, device="cuda")
            b = torch.rand(n, device="cuda")
            c = torch.empty(n, device="cuda")
            off = rank * n * 4
            grid = ((n * world + 1023) // 1024,)

            def add_step():
                with drv.partition(rank, world):
                    K.add_kernel[grid](DP(a.data_ptr() - off, torch.float32), DP(b.data_ptr() - off, torch.float32),
                                       DP(c.data_ptr() - off, torch.float32), n * world, BLOCK_SIZE=1024)
            record("vec_add", add_step, n * 12, 1e9, "hbm", "GB/s")
            if "value" in wl["vec_add"]:
                wl["vec_add"]["n"] = n
                wl["vec_add"]["result_check"] = bool(torch.equal(c[:1 << 20], a[:1 << 20] + b[:1 << 20]))
                wl["vec_add"]["host_us_per_launch"] = host_us_per_launch(add_step, 20)

        def wl_layernorm():
            # LayerNorm forward 4096 x 8192 fp16 per GPU; rotating buffer sets (134 MB each is about the L2 size)
            nb = 2 if args.small else 8
            m = LN_M * 4 if args.small else LN_M  # one 537 MB pass exceeds L2 by itself in a capture
            xs = [torch.randn(m, LN_N, device="cuda").half() for _ in range(nb)]
            ys = [torch.empty_like(xs[0]) for _ in range(nb)]
            w = (torch.rand(LN_N, device="cuda") + 0.5).half()
            bb = (0.1 * torch.randn(LN_N, device="cuda")).half()
            mean = torch.empty(m * world, device="cuda")
            rstd = torch.empty(m * world, device="cuda")
            lo_ln = rank * m

            def ln_step():
                for i in range(nb):
                    with drv.partition(rank, world):
                        K.layernorm_fwd_kernel[(m * world,)](DP(xs[i].data_ptr() - lo_ln * LN_N * 2, torch.float16),
                                                            DP(ys[i].data_ptr() - lo_ln * LN_N * 2, torch.float16),
                                                            w, bb, mean, rstd, LN_N, LN_N, 1e-5, BLOCK_SIZE=1024)
            record("layernorm", ln_step, 4 * m * LN_N + 4 * LN_N + 8 * m, 1e9, "hbm", "GB/s", nbuf=nb)
            if "value" in wl["layernorm"]:
                wl["layernorm"]["rows"] = m
                ref = torch.nn.functional.layer_norm(xs[0][:256].float(), (LN_N,), w.float(), bb.float(), 1e-5)
                err = (ys[0][:256].float() - ref).abs().max().item()
                mu = xs[nb - 1].float().mean(dim=1)  # mean / rstd hold the last buffer set's rows
                merr = (mean[lo_ln:lo_ln + m] - mu).abs().max().item()
                wl["layernorm"]["result_check"] = {"max_abs_err_y": err, "max_abs_err_mean": merr,
                                                   "ok": bool(err <= 2e-2 and merr <= 1e-5)}

                def one_launch():
                    with drv.partition(rank, world):
                        K.layernorm_fwd_kernel[(m * world,)](DP(xs[0].data_ptr() - lo_ln * LN_N * 2, torch.float16),
                                                            DP(ys[0].data_ptr() - lo_ln * LN_N * 2, torch.float16),
                                                            w, bb, mean, rstd, LN_N, LN_N, 1e-5, BLOCK_SIZE=1024)
                wl["layernorm"]["host_us_per_launch"] = host_us_per_launch(one_launch)

        def wl_strided_reduce():
            # strided masked reduction 8192 x 12288 (strides [1, 8192]) masked to 12000 columns + scalar total
            nb = 2 if args.small else 4
            fl = [torch.randn(RED_M * RED_N, device="cuda") for _ in range(nb)]
            rs = [torch.empty(RED_M, device="cuda") for _ in range(nb)]
            tots = torch.zeros(nb, device="cuda")  # one scalar total per pass

            def red_step():
                # every GPU reduces its own 8192-row matrix (weak scaling); the per-pass scalars are combined
                # across GPUs with ONE all-reduce per step, after the last pass, so no pass waits on NCCL
                for i in range(nb):
                    K.row_sum_kernel[(RED_M // 64,)](fl[i], rs[i], RED_M, RED_NV, 1, RED_M, BLOCK_M=64, BLOCK_N=64)
                    K.total_kernel[(1,)](rs[i], tots[i:i + 1], RED_M, BLOCK=1024)
                if world > 1:
                    dist.all_reduce(tots)
            record("strided_reduce", red_step, 4 * RED_M * RED_NV + 4 * RED_M + 4, 1e9, "hbm", "GB/s", nbuf=nb,
                   launches=2)
            if "unavailable" in wl["strided_reduce"] and world > 1:
                # the all-reduce could not be captured into a graph here: time eager launches instead
                record("strided_reduce", red_step, 4 * RED_M * RED_NV + 4 * RED_M + 4, 1e9, "hbm", "GB/s", nbuf=nb,
                       launches=2, graph=False)
            if "value" in wl["strided_reduce"]:
                # row sums against an fp64 sum, to 1e-5 of sum|x| (sums of N(0,1) data cancel); the scalar total
                # against the same sums combined over all GPUs
                v = fl[0].view(RED_N, RED_M)[:RED_NV]
                exact, scale = v.double().sum(dim=0), v.abs().double().sum(dim=0)
                rows_ok = bool(torch.all((rs[0].double() - exact).abs() <= 1e-5 * scale))
                red_step()
                torch.cuda.synchronize()
                want = torch.stack([fl[i].view(RED_N, RED_M)[:RED_NV].double().sum() for i in range(nb)])
                mag = torch.stack([fl[i].view(RED_N, RED_M)[:RED_NV].abs().double().sum() for i in range(nb)])
                if world > 1:
                    dist.all_reduce(want)
                    dist.all_reduce(mag)
                tot_ok = bool(torch.all((tots.double() - want).abs() <= 1e-5 * mag))
                wl["strided_reduce"]["result_check"] = {"row_sums": rows_ok, "scalar_total_all_gpus": tot_ok,
                                                        "ok": rows_ok and tot_ok}
                wl["strided_reduce"]["launches_per_pass"] = "2: the row-sum kernel and the single-program total kernel " \
                                                            "(two Triton kernels; the reference has no atomics)"

        def wl_matmul():
            # bf16 matmul 8192^3, blocks 128/256/64, fp32 accumulation
            A = (2 * torch.rand(MM, MM, device="cuda") - 1).bfloat16()
            B = (2 * torch.rand(MM, MM, device="cuda") - 1).bfloat16()
            C = torch.empty(MM, MM, device="cuda", dtype=torch.bfloat16)
            mm_grid = ((MM // 128) * (MM // 256),)

            def mm_step():
                K.matmul_kernel[mm_grid](A, B, C, MM, MM, MM, A.stride(0), A.stride(1), B.stride(0), B.stride(1),
                                         C.stride(0), C.stride(1), BLOCK_M=128, BLOCK_N=256, BLOCK_K=64, GROUP_M=8)
            record("matmul", mm_step, 2.0 * MM * MM * MM, 1e12, "tensor", "TFLOP/s")
            if "value" in wl.get("matmul", {}):
                # single launches with idle gaps between them: the burst figure (the measured peak is
                # quoted the same two ways: best single cuBLAS call, and seconds of back-to-back calls)
                best = float("inf")
                for _ in range(10):
                    torch.cuda.synchronize()
                    time.sleep(0.05)
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    mm_step()
                    e1.record()
                    torch.cuda.synchronize()
                    best = min(best, e0.elapsed_time(e1))
                burst = 2.0 * MM * MM * MM / (best * 1e-3) / 1e12
                wl["matmul"]["burst"] = {"best_ms": best, "value": burst, "unit": "TFLOP/s",
                                         "frac_of_burst_peak": burst / peaks["tensor"]}
                # seconds of back-to-back launches, the way the sustained peak itself was measured
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    for _ in range(20):
                        mm_step()
                g.replay()
                torch.cuda.synchronize()
                smp = ClockSampler(local_rank)
                smp.start()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps, t0 = 0, time.perf_counter()
                e0.record()
                while time.perf_counter() - t0 < 2.5:
                    for _ in range(8):
                        g.replay()
                    reps += 8
                    torch.cuda.synchronize()
                e1.record()
                torch.cuda.synchronize()
                sus = 2.0 * MM * MM * MM * 20 * reps / (e0.elapsed_time(e1) * 1e-3) / 1e12
                wl["matmul"]["sustained"] = {"seconds": e0.elapsed_time(e1) * 1e-3, "launches": 20 * reps, "value": sus,
                                             "unit": "TFLOP/s", "frac_of_sustained_peak": sus / peaks["tensor_sustained"],
                                             "clocks": smp.stop()}
                ref = (A[:256].float() @ B.float())
                err = (C[:256].float() - ref).abs().max().item() / ref.abs().max().item()
                wl["matmul"]["result_check_rel_err"] = err

        def wl_gelu_bias():
            # register-VM elementwise body (25 ops, fp16 I/O, broadcast bias), 16,384 x 8,192
            R, C = (4096, 8192) if args.small else (16384, 8192)
            x = torch.randn(R, C, device="cuda").half()
            b = torch.randn(C, device="cuda").half()
            o = torch.empty_like(x)

            def step():
                K.gelu_bias_kernel[(R, C // 1024)](x, b, o, C, BLOCK=1024)
            record("gelu_bias", step, 4 * R * C + 2 * C, 1e9, "hbm", "GB/s")

        def wl_bias_chain():
            # 5-op fp32 body with a row-broadcast operand on a 2-D grid (elementwise VM, lean accessors), 8,192 x 8,192
            R, C = (4096, 8192) if args.small else (8192, 8192)
            x = torch.randn(R, C, device="cuda")
            b = torch.randn(C, device="cuda")
            o = torch.empty_like(x)

            def step():
                K.bias_chain_kernel[(R, C // 1024)](x, b, o, C, NIT=2, BLOCK=1024)
            record("bias_chain", step, 8 * R * C + 4 * C, 1e9, "hbm", "GB/s")
            if "value" in wl["bias_chain"]:
                v = x[:64] + b
                for _ in range(2):
                    v = v * 1.0001 + b
                wl["bias_chain"]["result_check"] = bool(torch.equal(o[:64], v))

        def wl_rmsnorm():
            # a full fold inside the body (elementwise VM with a per-program fold), fp16 16,384 x 4,096
            R, C = (4096, 4096) if args.small else (16384, 4096)
            x = torch.randn(R, C, device="cuda").half()
            w = (torch.rand(C, device="cuda") + 0.5).half()
            y = torch.empty_like(x)

            def step():
                K.rmsnorm_kernel[(R,)](x, w, y, C, C, 1e-6, BLOCK=4096)
            record("rmsnorm", step, 4 * R * C + 2 * C, 1e9, "hbm", "GB/s")

        def wl_row_stats():
            # block-program kernel (loop-carried block accumulators, folds to scalars), fp32 16,384 x 4,096
            R, C = (4096, 4096) if args.small else (16384, 4096)
            x = torch.randn(R, C, device="cuda")
            sums = torch.empty(R, device="cuda")
            maxs = torch.empty(R, device="cuda")

            def step():
                K.row_stats_kernel[(R,)](x, sums, maxs, C, C, BLOCK=1024)
            record("row_stats", step, 4 * R * C + 8 * R, 1e9, "hbm", "GB/s")
            if "value" in wl["row_stats"]:
                wl["row_stats"]["result_check"] = bool(torch.equal(maxs, x.max(dim=1).values) and
                                                       torch.allclose(sums.double(), x.double().sum(dim=1), rtol=1e-5, atol=1e-3))

        def wl_wrap_rows():
            # wrap-around row gather copy: 64 programs' worth in one program is tiny, so use many column steps
            M, N = 4096, 16384
            A = torch.randn(M, N, device="cuda")
            Cc = torch.empty(64, N, device="cuda")

            def step():
                K.wrap_rows_kernel[(1,)](A, Cc, M, N, 1, N, 1, START=4090, BM=64, BN=64, STEPS=N // 64)
            record("wrap_rows", step, 8 * 64 * N, 1e9, "hbm", "GB/s")  # one launch: the column loop runs on the device
            if "value" in wl["wrap_rows"]:
                wl["wrap_rows"]["result_check"] = bool(torch.equal(Cc, torch.cat([A[4090:], A[:58]])))
                wl["wrap_rows"]["note"] = "a single program (one CTA) walks 256 column steps: bound by one SM, not by HBM"

        def wl_gather_rows():
            # row gather through a loaded int64 index (one unstructured dim, contiguous rows), fp32 65,536 x 1,024
            R, C = (16384, 1024) if args.small else (65536, 1024)
            x = torch.randn(R, C, device="cuda")
            idx = torch.randperm(R, device="cuda")
            o = torch.empty_like(x)

            def step():
                K.gather_rows_kernel[(R // 16, C // 128)](x, idx, o, R, C, C, C, BLOCK_M=16, BLOCK_N=128)
            record("gather_rows", step, 8 * R * C + 8 * R, 1e9, "hbm", "GB/s")
            if "value" in wl["gather_rows"]:
                wl["gather_rows"]["result_check"] = bool(torch.equal(o, x[idx]))

        def wl_block_copy():
            # masked strided 2-D block copy, fp32 16,000 x 16,000 (ragged against 64 x 128 tiles), row-major to row-major
            M = N = 8000 if args.small else 16000
            src = torch.randn(M, N, device="cuda")
            dst = torch.empty(M, N, device="cuda")
            grid2 = ((M + 63) // 64, (N + 127) // 128)

            def step():
                K.copy_2d_kernel[grid2](src, dst, M, N, N, 1, N, 1, BM=64, BN=128)
            record("block_copy", step, 8 * M * N, 1e9, "hbm", "GB/s")
            if "value" in wl["block_copy"]:
                wl["block_copy"]["result_check"] = bool(torch.equal(src, dst))

        for name, fn in (("vec_add", wl_vec_add), ("layernorm", wl_layernorm),
                         ("strided_reduce", wl_strided_reduce), ("matmul", wl_matmul),
                         ("gelu_bias", wl_gelu_bias), ("bias_chain", wl_bias_chain), ("rmsnorm", wl_rmsnorm), ("row_stats", wl_row_stats), ("wrap_rows", wl_wrap_rows), ("gather_rows", wl_gather_rows),
                         ("block_copy", wl_block_copy)):
            if name in chosen:
                fn()
                torch.cuda.empty_cache()
        line["workloads"] = wl

    # ------------------------------------------------------------------ strong scaling: shards of ONE grid
    if world > 1 and chosen:
        from triton_shared_b200 import partition_range
        strong = {}
        steps3, warm3 = 10, 3

        def nbuf_for(shard_bytes):
            # enough rotating buffer sets that consecutive passes cannot be served from the 126 MB L2
            return int(max(2, min(32, -(-400_000_000 // max(shard_bytes, 1)))))

        def srecord(name, fn, alg_total, unit_scale, bound, unit, nbuf, check=None):
            try:
                tot, per = timed(fn, steps3, warm3, launches_per_call=nbuf)
            except Exception as e:
                strong[name] = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
                return
            peak = peaks["hbm"] if bound == "hbm" else peaks["tensor"]
            per_gpu = alg_total / world / (per * 1e-3) / unit_scale
            strong[name] = {"value": alg_total * steps3 * nbuf / (tot * 1e-3) / unit_scale, "unit": unit,
                            "ms_per_pass": per, "per_gpu_frac_of_peak": per_gpu / peak, "rotating_buffers": nbuf,
                            "problem": "fixed total size, contiguous program ranges per GPU, num_programs = full grid"}
            if check is not None:
                strong[name]["result_check"] = check()

        def s_vec_add():
            n = ADD_N
            progs = n // 1024
            lo_p, hi_p = partition_range(progs, rank, world)
            ne = (hi_p - lo_p) * 1024
            nb = nbuf_for(ne * 12)
            bufs = [(torch.rand(ne, device="cuda"), torch.rand(ne, device="cuda"), torch.empty(ne, device="cuda")) for _ in range(nb)]
            off = lo_p * 1024 * 4

            def step():
                for a, b, c in bufs:
                    with drv.partition(rank, world):
                        K.add_kernel[(progs,)](DP(a.data_ptr() - off, torch.float32), DP(b.data_ptr() - off, torch.float32),
                                               DP(c.data_ptr() - off, torch.float32), n, BLOCK_SIZE=1024)
            srecord("vec_add", step, n * 12, 1e9, "hbm", "GB/s", nb,
                    lambda: bool(torch.equal(bufs[0][2], bufs[0][0] + bufs[0][1])))

        def s_softmax():
            R, C = SOFTMAX_ROWS, SOFTMAX_COLS
            lo_r, hi_r = partition_range(R, rank, world)
            nr = hi_r - lo_r
            nb = nbuf_for(nr * C * 8)
            bufs = [(torch.randn(nr, C, device="cuda"), torch.empty(nr, C, device="cuda")) for _ in range(nb)]
            off = lo_r * C * 4

            def step():
                for xi, yi in bufs:
                    with drv.partition(rank, world):
                        K.softmax_kernel[(R,)](DP(yi.data_ptr() - off, torch.float32), DP(xi.data_ptr() - off, torch.float32),
                                               C, C, C, BLOCK_SIZE=4096)
            srecord("softmax", step, R * C * 8, 1e9, "hbm", "GB/s", nb,
                    lambda: bool(torch.allclose(bufs[0][1].sum(dim=1), torch.ones(nr, device="cuda"), rtol=1e-4)))

        def s_layernorm():
            lo_r, hi_r = partition_range(LN_M, rank, world)
            nr = hi_r - lo_r
            nb = nbuf_for(nr * LN_N * 4)
            bufs = [(torch.randn(nr, LN_N, device="cuda").half(), torch.empty(nr, LN_N, device="cuda", dtype=torch.float16))
                    for _ in range(nb)]
            w = (torch.rand(LN_N, device="cuda") + 0.5).half()
            bb = (0.1 * torch.randn(LN_N, device="cuda")).half()
            mean, rstd = torch.empty(LN_M, device="cuda"), torch.empty(LN_M, device="cuda")
            off = lo_r * LN_N * 2

            def step():
                for xi, yi in bufs:
                    with drv.partition(rank, world):
                        K.layernorm_fwd_kernel[(LN_M,)](DP(xi.data_ptr() - off, torch.float16), DP(yi.data_ptr() - off, torch.float16),
                                                        w, bb, mean, rstd, LN_N, LN_N, 1e-5, BLOCK_SIZE=1024)

            def check():
                ref = torch.nn.functional.layer_norm(bufs[0][0].float(), (LN_N,), w.float(), bb.float(), 1e-5)
                return bool((bufs[0][1].float() - ref).abs().max().item() <= 2e-2)
            srecord("layernorm", step, 4 * LN_M * LN_N + 4 * LN_N + 8 * LN_M, 1e9, "hbm", "GB/s", nb, check)

        def s_reduce():
            progs = RED_M // 64
            lo_p, hi_p = partition_range(progs, rank, world)
            lo_r, nr = lo_p * 64, (hi_p - lo_p) * 64
            nb = nbuf_for(nr * RED_N * 4)
            # this rank's rows of the [1, M]-strided matrix, stored compactly: element (i, j) at (i - lo_r) + j * nr
            fl = [torch.randn(RED_N * nr, device="cuda") for _ in range(nb)]
            rs = torch.empty(nr, device="cuda")
            tots = torch.zeros(nb, device="cuda")

            def step():
                for i in range(nb):
                    with drv.partition(rank, world):
                        K.row_sum_kernel[(progs,)](DP(fl[i].data_ptr() - lo_r * 4, torch.float32), DP(rs.data_ptr() - lo_r * 4, torch.float32),
                                                   RED_M, RED_NV, 1, nr, BLOCK_M=64, BLOCK_N=64)
                    K.total_kernel[(1,)](rs, tots[i:i + 1], nr, BLOCK=1024)
                dist.all_reduce(tots)  # the global scalar of every pass, one NCCL all-reduce per step

            def check():
                step()
                torch.cuda.synchronize()
                want = torch.stack([f.view(RED_N, nr)[:RED_NV].double().sum() for f in fl])
                mag = torch.stack([f.view(RED_N, nr)[:RED_NV].abs().double().sum() for f in fl])
                dist.all_reduce(want)
                dist.all_reduce(mag)
                return bool(torch.all((tots.double() - want).abs() <= 1e-5 * mag))
            srecord("strided_reduce", step, 4 * RED_M * RED_NV + 4 * RED_M + 4, 1e9, "hbm", "GB/s", nb, check)

        def s_matmul():
            progs = (MM // 128) * (MM // 256)
            lo_p, hi_p = partition_range(progs, rank, world)
            per_group = 8 * (MM // 256)  # programs of one group of GROUP_M = 8 tile rows
            if lo_p % per_group or hi_p % per_group:
                strong["matmul"] = {"unavailable": "program ranges do not fall on tile-row groups at this GPU count"}
                return
            r0, r1 = lo_p // per_group * 8 * 128, hi_p // per_group * 8 * 128  # this rank's band of A / C rows
            A = (2 * torch.rand(r1 - r0, MM, device="cuda") - 1).bfloat16()
            B = (2 * torch.rand(MM, MM, device="cuda") - 1).bfloat16()  # replicated
            C = torch.empty(r1 - r0, MM, device="cuda", dtype=torch.bfloat16)

            def step():
                with drv.partition(rank, world):
                    K.matmul_kernel[(progs,)](DP(A.data_ptr() - r0 * MM * 2, torch.bfloat16), B, DP(C.data_ptr() - r0 * MM * 2, torch.bfloat16),
                                              MM, MM, MM, MM, 1, MM, 1, MM, 1, BLOCK_M=128, BLOCK_N=256, BLOCK_K=64, GROUP_M=8)

            def check():
                ref = A[:256].float() @ B.float()
                return bool(((C[:256].float() - ref).abs().max() / ref.abs().max()).item() <= 1e-2)
            srecord("matmul", step, 2.0 * MM ** 3, 1e12, "tensor", "TFLOP/s", 1, check)

        for nm, fn in (("vec_add", s_vec_add), ("softmax", s_softmax), ("layernorm", s_layernorm),
                       ("strided_reduce", s_reduce), ("matmul", s_matmul)):
            if nm == "softmax" or nm in chosen:
                fn()
                torch.cuda.empty_cache()
        line["strong_scaling"] = strong

    # ------------------------------------------------------------------ CPU baseline (rank 0, N = 1)
    if world == 1 and rank == 0 and not args.no_cpu_baseline:
        gbs, threads, (srows, passes), dt = cpu_softmax_rate()
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                                "sample": f"{srows} of {SOFTMAX_ROWS} rows x {SOFTMAX_COLS} cols, {passes} passes, {dt:.1f} s"}
        g1, _, (r1_, p1_), d1_ = cpu_softmax_rate(seconds_target=3.0, threads=1)
        line["cpu_baseline"]["one_thread"] = {"value": g1, "cores": 1, "sample": f"{r1_} rows, {p1_} passes, {d1_:.1f} s",
                                              "note": "the reference launcher runs the grid serially on one thread"}
        for name, cb in cpu_baselines().items():
            if name in line.get("workloads", {}):
                line["workloads"][name]["cpu_baseline"] = cb
    if world > 1:
        dist.destroy_process_group()
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)  # stdout carries exactly one line
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
