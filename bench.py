"""Benchmark of the INT4 fused SwiGLU MLP path (BASELINE config 1: Llama-3.2-1B shape,
hidden 2048 / intermediate 8192, group 64, rows M in {1,2,4,8,16,32,128}).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one sweep: the fused MLP (gate|up SwiGLU -> down + residual) once for every M of
the sweep, each call on the next of a rotating set of weight copies larger than L2.  `value` is
the weight bytes streamed per second over the whole step with all inputs resident in HBM (the
sweep replayed as a CUDA graph); `e2e` is the same metric through the public executor with HOST
activations (pinned), host->device and device->host copies inside the timed region.  The JSON
line also carries per-M times, the roofline of the dominant kernel, and a CPU baseline.

With --gpus N > 1 (launched by torch.distributed.run, one rank per GPU) the workload is the
tensor-parallel MLP of BASELINE config 4 (hidden 5120 / intermediate 27648): gate|up
column-sharded, down row-sharded, one NCCL all-reduce per MLP; scaling is "strong".

--impl reference times the reference semantics on the host cores (the C + OpenMP port under
oracle/, because MLX itself cannot be installed here) on the same workload and prints the same
line shape with "impl": "reference".
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

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

SWEEP = (1, 2, 4, 8, 16, 32, 128)
HIDDEN, INTERMEDIATE = 2048, 8192
TP_HIDDEN, TP_INTERMEDIATE = 5120, 27648
TP_SWEEP = (1, 16, 128)
NOMINAL_HBM_GBS = 8000.0


def weight_bytes(hidden, intermediate):
    """Packed nibbles + bf16 scale and bias per group of 64, three projections."""
    per_weight = 0.5 + 2 * 2 / 64
    return int(3 * hidden * intermediate * per_weight)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as handle:
            data = json.load(handle)
        return float(data["hbm_gbs"]), float(data.get("bf16_tflops_sustained", 1420.5)), "measured"
    return 6650.0, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self):
        try:
            self._run_nvml()
        except Exception:
            self._run_smi()

    def _run_nvml(self):
        """In-process NVML queries (read-only): no fork while CUDA / NCCL threads are running."""
        import pynvml

        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
        self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(handle, pynvml.NVML_CLOCK_SM))
        bits = {
            "hw_slowdown": pynvml.nvmlClocksThrottleReasonHwSlowdown,
            "hw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonHwThermalSlowdown,
            "sw_thermal_slowdown": pynvml.nvmlClocksThrottleReasonSwThermalSlowdown,
            "sw_power_cap": pynvml.nvmlClocksThrottleReasonSwPowerCap,
        }
        while not self._stop.is_set():
            self.samples.append(float(pynvml.nvmlDeviceGetClockInfo(handle, pynvml.NVML_CLOCK_SM)))
            reasons = pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
            for name, bit in bits.items():
                if reasons & bit:
                    self.reasons.add(name)
            self._stop.wait(0.05)

    def _run_smi(self):
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        while not self._stop.is_set():
            try:
                out = subprocess.run(
                    ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                     "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                fields = [f.strip() for f in out.strip().splitlines()[0].split(",")]
                self.samples.append(float(fields[0]))
                self.max_mhz = float(fields[1])
                for name, value in zip(names, fields[2:6]):
                    if value.lower().startswith("active"):
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.2)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


def bits_triple(triple):
    from metile_b200 import synth

    return triple[0].cpu().numpy(), synth.to_numpy_bits(triple[1]), synth.to_numpy_bits(triple[2])


def cpu_sweep_seconds(hidden, intermediate, sweep, repeats):
    """Time the C + OpenMP port of the reference semantics on the host cores."""
    from metile_b200 import synth
    from oracle import cport

    gate, up, down = synth.mlp_weights(100, hidden, intermediate)
    triples = [bits_triple(t) for t in (gate, up, down)]
    inputs = [(synth.to_numpy_bits(synth.activations(5, m, hidden)),
               synth.to_numpy_bits(synth.activations(6, m, hidden))) for m in sweep]
    cport.mlp(inputs[0][0], *triples, inputs[0][1])  # warm-up (thread pool, page faults)
    times = []
    for _ in range(repeats):
        start = time.perf_counter()
        for x, r in inputs:
            cport.mlp(x, *triples, r)
        times.append(time.perf_counter() - start)
    return times, cport.num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tp = args.gpus > 1
    hidden, inter, sweep = (TP_HIDDEN, TP_INTERMEDIATE, TP_SWEEP) if tp else (HIDDEN, INTERMEDIATE, SWEEP)
    total_bytes = weight_bytes(hidden, inter) * len(sweep)
    times, cores = cpu_sweep_seconds(hidden, inter, sweep, args.warmup + args.steps)
    timed = times[args.warmup:]
    seconds = sum(timed) / len(timed)
    value = total_bytes / seconds / 1e9
    line = {
        "impl": "reference",
        "metric": "int4_fused_mlp_weight_GBps",
        "value": value,
        "unit": "GB/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": seconds * 1e3,
        "higher_is_better": True,
        "scaling": "strong" if tp else "weak",
        "vs_baseline": None,
        "dtype": "bf16 activations, u4 weights, fp32 accumulate",
        "data": "synthetic",
        "config": workload_config(hidden, inter, sweep, args.gpus, "host memory (CPU run)"),
        "tokens_per_s": sum(sweep) / seconds,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{len(timed)} full sweeps M={list(sweep)} of the same MLP"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "MLX-CPU (the reference's own CPU path) is unavailable on this box; this is the C + OpenMP "
                "port of its semantics under oracle/",
    }
    print(json.dumps(line))


def workload_config(hidden, inter, sweep, gpus, l2_note):
    return {
        "workload": ("int4_swiglu_mlp_llama3.2-1b" if hidden == HIDDEN else "int4_swiglu_mlp_qwen2.5-32b_tp"),
        "hidden": hidden,
        "intermediate": inter,
        "group_size": 64,
        "bits": 4,
        "rows_sweep": list(sweep),
        "weight_bytes_per_mlp": weight_bytes(hidden, inter),
        "parallelism": "single GPU" if gpus == 1 else f"tp{gpus} (gate|up column-sharded, down row-sharded, 1 all-reduce)",
        "l2": l2_note,
    }


def log(message):
    """Progress on stderr (the JSON line alone goes to stdout)."""
    if os.environ.get("RANK", "0") == "0":
        print(f"[bench {time.strftime('%H:%M:%S')}] {message}", file=sys.stderr, flush=True)


def run_ours(args):
    import torch

    from metile_b200 import _lib
    from metile_b200 import backends as B
    from metile_b200 import synth
    from metile_b200 import tp as tensor_parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} does not match WORLD_SIZE {world}")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
    tp = distributed
    hidden, inter, sweep = (TP_HIDDEN, TP_INTERMEDIATE, TP_SWEEP) if tp else (HIDDEN, INTERMEDIATE, SWEEP)
    per_mlp_bytes = weight_bytes(hidden, inter)
    local_bytes = per_mlp_bytes // world
    l2_bytes = torch.cuda.get_device_properties(device).L2_cache_size
    copies = max(2, -(-2 * l2_bytes // local_bytes) + 1)
    copies = min(copies, 24)

    log(f"world {world}, workload hidden {hidden} / intermediate {inter}, {copies} weight sets")
    # ---- build the rotating weight sets and executors -------------------------------------------
    executors = []
    for c in range(copies):
        if tp:
            executors.append(tensor_parallel.TensorParallelMLP.from_seed(100, hidden, inter, device, rank, world))
        else:
            gate, up, down = synth.mlp_weights(100, hidden, inter, device)
            sample = synth.activations(5, 1, hidden, device)
            executors.append(B.mlx_affine_mlp_executor(sample, *gate, *up, *down, sample))
    inputs = {m: (synth.activations(5, m, hidden, device), synth.activations(6, m, hidden, device)) for m in sweep}
    # Activations and residual of one call share a page-locked buffer, residual right after the
    # activations, so that the host entry point can move both with one copy.
    host_inputs = {}
    for m in sweep:
        both = torch.empty((2, m, hidden), dtype=torch.bfloat16).pin_memory()
        both[0].copy_(inputs[m][0])
        both[1].copy_(inputs[m][1])
        host_inputs[m] = (both[0], both[1])
    host_outputs = {m: torch.empty((m, hidden), dtype=torch.bfloat16).pin_memory() for m in sweep}
    cursor = [0]

    def next_executor():
        cursor[0] = (cursor[0] + 1) % copies
        return executors[cursor[0]]

    def sweep_once():
        for m in sweep:
            x, r = inputs[m]
            next_executor()(x, r)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.Stream()

    def capture(fn, repeats):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(stream):
            fn()
            stream.synchronize()
            with torch.cuda.graph(graph, stream=stream):
                for _ in range(repeats):
                    fn()
        torch.cuda.synchronize()
        return graph

    def time_graph(graph, replays):
        with torch.cuda.stream(stream):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            for _ in range(replays):
                graph.replay()
            stop.record(stream)
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e-3

    log("weights resident; warm-up")
    def time_eager(fn, repeats):
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(repeats):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e-3

    # ---- headline: K steps, each one sweep, replayed as a CUDA graph ------------------------------
    # (single GPU).  The tensor-parallel run times eager launches instead: replaying graphs that
    # contain NCCL collectives did not make progress on this pool, eager collectives do.
    for _ in range(3):
        sweep_once()
    torch.cuda.synchronize()
    log("eager warm-up done; capturing the sweep")
    if tp:
        run_steps = lambda n: time_eager(sweep_once, n)  # noqa: E731
    else:
        step_graph = capture(sweep_once, 1)
        log("graph captured")
        run_steps = lambda n: time_graph(step_graph, n)  # noqa: E731
    run_steps(max(args.warmup, 3))
    barrier()
    with ClockSampler(local_rank) as clocks:
        seconds = run_steps(args.steps)
        barrier()
        # Keep the sampler alive long enough for a few samples when the steps are very short.
        if seconds < 0.5 and not tp:
            filler = run_steps(max(1, int(0.5 / max(seconds / args.steps, 1e-6))))
            del filler
    if distributed:
        t = torch.tensor([seconds], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())
    step_seconds = seconds / args.steps
    total_bytes = per_mlp_bytes * len(sweep)
    value = total_bytes / step_seconds / 1e9

    log(f"headline: {step_seconds * 1e3:.3f} ms per step")
    # ---- per-M detail (graph of 8 MLP calls per M) ------------------------------------------------
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    detail = []
    for m in sweep:
        log(f"detail M={m}")
        x, r = inputs[m]

        def one(x=x, r=r):
            next_executor()(x, r)

        if tp:
            time_eager(one, 8)
            barrier()
            per_call = time_eager(one, 80) / 80
        else:
            graph = capture(one, 8)
            graph.replay()
            barrier()
            per_call = time_graph(graph, 10) / 80
        if distributed:
            t = torch.tensor([per_call], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            per_call = float(t.item())
        flops = 2.0 * 3 * hidden * inter * m
        hbm_seconds = (local_bytes) / (hbm_peak * 1e9)
        tensor_seconds = flops / world / (tensor_peak * 1e12)
        detail.append({
            "rows": m,
            "us": per_call * 1e6,
            "weight_GBps": per_mlp_bytes / per_call / 1e9,
            "tokens_per_s": m / per_call,
            "frac_of_hbm": (local_bytes / per_call / 1e9) / hbm_peak,
            "frac_of_nominal_8TBps": (local_bytes / per_call / 1e9) / NOMINAL_HBM_GBS,
            "bound": "hbm" if hbm_seconds >= tensor_seconds else "tensor",
            "frac_of_roofline": max(hbm_seconds, tensor_seconds) / per_call,
        })

    # ---- roofline per kernel family, each timed alone; the headline one is the family with the largest
    # share of the step (launches in a sweep x its duration) ------------------------------------------
    roofline = None
    roofline_kernels = []
    if not tp:
        library = _lib.load()
        weight_sets = [synth.mlp_weights(100, hidden, inter, device) for _ in range(copies)]
        cursor = [0]

        def per_launch_seconds(fn, launches_per_call):
            graph = capture(fn, 16)
            graph.replay()
            torch.cuda.synchronize()
            return time_graph(graph, 10) / (160 * launches_per_call)

        def entry(kernel, rows_served, seconds, algorithmic, traffic, profile):
            achieved = algorithmic / seconds / 1e9
            return {
                "kernel": kernel,
                "bound": "hbm",
                "achieved": achieved,
                "peak": hbm_peak,
                "unit": "GB/s",
                "frac": achieved / hbm_peak,
                "peak_kind": f"of {peak_kind}",
                # dram__bytes_read.sum + dram__bytes_write.sum of one launch, from the ncu capture
                # summarised in the named file under profiles/.
                "traffic": traffic,
                "traffic_source": profile,
                "algorithmic_bytes_per_launch": int(algorithmic),
                "us_per_launch": seconds * 1e6,
                "launches_per_sweep": sum(1 for m in sweep if m in rows_served),
            }

        packed = hidden * inter * (0.5 + 4 / 64)  # one projection: nibbles + bf16 scales and biases
        single_rows = [m for m in sweep if library.mt_affine_mlp_launches(m, hidden, inter, 0) == 1]
        # One launch per MLP: the CUDA-core kernel for one row, the warp-MMA kernel from two to eight.
        for rows_served, label, traffic, profile in (
                ([m for m in single_rows if m <= 1], "single-launch MLP on CUDA cores (affine_mlp_fused_kernel)", 28381952,
                 "profiles/affine_mlp_fused_m1_llama1b.md"),
                ([m for m in single_rows if m > 1], "single-launch MLP on mma.sync (affine_mlp_fused_mma_kernel)", 28458496,
                 "profiles/affine_mlp_fused_mma_m8_llama1b.md")):
            if not rows_served:
                continue
            m = rows_served[0] if rows_served[0] <= 1 else rows_served[-1]
            xm, rm = inputs[m]
            executors_m = [B.mlx_affine_mlp_executor(xm, *w[0], *w[1], *w[2], rm) for w in weight_sets]

            def whole_mlp(executors_m=executors_m, xm=xm, rm=rm):
                cursor[0] = (cursor[0] + 1) % copies
                executors_m[cursor[0]](xm, rm)

            seconds = per_launch_seconds(whole_mlp, 1)
            roofline_kernels.append(entry(
                f"{label}, M={m}", rows_served, seconds,
                3 * packed + 2 * m * hidden * 2 + 2 * m * inter * 2 + m * hidden * 2, traffic, profile))
        two_kernel_rows = [m for m in sweep if m not in single_rows]
        small = [m for m in two_kernel_rows if m <= 16]
        if small:
            m = small[-1]
            xs = inputs[m][0]
            hs = synth.activations(11, m, inter, device, std=0.3)
            rs = inputs[m][1]

            def gate_up():
                cursor[0] = (cursor[0] + 1) % copies
                gate, up, _ = weight_sets[cursor[0]]
                B.mlx_affine_swiglu(xs, *gate, *up)

            def down_projection():
                cursor[0] = (cursor[0] + 1) % copies
                B.mlx_affine_residual_qmv(hs, *weight_sets[cursor[0]][2], rs)

            roofline_kernels.append(entry(
                f"gate|up SwiGLU on tcgen05, 16-row instance at M={m} (affine_umma_kernel<2,16>)", small,
                per_launch_seconds(gate_up, 1), 2 * packed + m * hidden * 2 + m * inter * 2, 19020544,
                "profiles/affine_umma_swiglu_m1_llama1b.md"))
            roofline_kernels.append(entry(
                f"down projection on tcgen05, 16-row instance at M={m} (affine_umma_kernel<1,16>)", small,
                per_launch_seconds(down_projection, 1), packed + m * inter * 2 + 2 * m * hidden * 2, None, None))
        if roofline_kernels:
            roofline = max(roofline_kernels, key=lambda e: e["launches_per_sweep"] * e["us_per_launch"])
        del weight_sets

    # ---- tensor-parallel run: the SAME workload unsharded on one GPU (this rank's own), so that the
    # strong-scaling ratio can be read from one line; eager launches and CUDA events like the headline.
    one_gpu = None
    if tp:
        full_sets = [synth.mlp_weights(100, hidden, inter, device) for _ in range(2)]
        sample = synth.activations(5, 1, hidden, device)
        full_executors = [B.mlx_affine_mlp_executor(sample, *w[0], *w[1], *w[2], sample) for w in full_sets]
        flip = [0]

        def unsharded_sweep():
            for m in sweep:
                flip[0] ^= 1
                full_executors[flip[0]](*inputs[m])

        time_eager(unsharded_sweep, 3)
        barrier()
        one_seconds = time_eager(unsharded_sweep, args.steps) / args.steps
        t = torch.tensor([one_seconds], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        one_seconds = float(t.item())
        one_gpu = {"value": per_mlp_bytes * len(sweep) / one_seconds / 1e9, "unit": "GB/s",
                   "ms_per_step": one_seconds * 1e3,
                   "note": "same sweep, unsharded, one GPU (every rank runs it at once; slowest rank), "
                           f"two weight sets of {per_mlp_bytes / 1e6:.0f} MB alternating"}
        del full_executors, full_sets

    log("per-M detail done")
    # ---- end to end with host buffers ---------------------------------------------------------------
    # Single GPU: the C-ABI host entry point (mt_affine_mlp_host through mlx_affine_mlp_host_executor):
    # one call queues the two host->device copies, the MLP and the device->host copy.  Tensor-parallel:
    # the sharded executor on device tensors with the copies issued around it.
    if tp:
        def e2e_step():
            for m in sweep:
                hx, hr = host_inputs[m]
                x = hx.to(device, non_blocking=True)
                r = hr.to(device, non_blocking=True)
                y = next_executor()(x, r)
                host_outputs[m].copy_(y, non_blocking=True)
            torch.cuda.synchronize()
    else:
        host_executors = [B.mlx_affine_mlp_host_executor(max(sweep), hidden, *e.weights) for e in executors]

        def e2e_step():
            for m in sweep:
                hx, hr = host_inputs[m]
                cursor[0] = (cursor[0] + 1) % copies
                host_executors[cursor[0]](hx, hr, host_outputs[m])
            torch.cuda.synchronize()

    log("e2e warm-up")
    for _ in range(3):
        e2e_step()
    barrier()
    log("e2e timed")
    start = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_seconds = (time.perf_counter() - start) / args.steps
    if distributed:
        t = torch.tensor([e2e_seconds], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_seconds = float(t.item())
    h2d = sum(2 * m * hidden * 2 for m in sweep)
    d2h = sum(m * hidden * 2 for m in sweep)

    # ---- CPU baseline (rank 0, single-GPU run only) -----------------------------------------------
    cpu_baseline = None
    if rank == 0 and not tp:
        times, cores = cpu_sweep_seconds(hidden, inter, sweep, 3)
        cpu_seconds = min(times)
        cpu_baseline = {"value": total_bytes / cpu_seconds / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                        "sample": f"3 full sweeps M={list(sweep)} of the same MLP (best), C + OpenMP port of the "
                                  "reference semantics; MLX-CPU is unavailable on this box"}

    if rank == 0:
        launches_per_sweep = sum(_lib.load().mt_affine_mlp_launches(m, hidden, inter, 0) for m in sweep)
        line = {
            "metric": "int4_fused_mlp_weight_GBps",
            "value": value,
            "unit": "GB/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": step_seconds * 1e3,
            "higher_is_better": True,
            "scaling": "strong" if tp else "weak",
            "vs_baseline": None,
            "dtype": "bf16 activations, u4 weights, fp32 accumulate",
            "data": "synthetic",
            "config": workload_config(hidden, inter, sweep, world,
                                      f"rotating {copies} weight sets ({copies * local_bytes / 1e6:.0f} MB per GPU) "
                                      f"> 2x L2 ({l2_bytes / 1e6:.0f} MB)"),
            "tokens_per_s": sum(sweep) / step_seconds,
            "frac_of_hbm_peak": (local_bytes * len(sweep) / step_seconds / 1e9) / hbm_peak,
            "sweep": detail,
            "roofline": roofline,
            "roofline_kernels": roofline_kernels,
            "one_gpu_same_workload": one_gpu,
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": total_bytes / e2e_seconds / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_seconds * 1e3},
            "gpu_launches": launches_per_sweep * args.steps,
            "timing": "eager launches, CUDA events" if tp else "CUDA-graph replay, CUDA events",
            "clocks": clocks.summary(),
        }
        print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


def run_capture(spec):
    """Six launches of one operator at the Llama-3.2-1B shape over six weight sets (170 MB, larger than
    L2), nothing timed and nothing printed but a status line: the process profilers attach to."""
    import torch

    from metile_b200 import _lib
    from metile_b200 import backends as B
    from metile_b200 import synth

    op, family, rows = spec.split(":")
    rows = int(rows)
    family = None if family == "default" else family
    hidden, inter = 2048, 8192
    device = torch.device("cuda:0")
    sets = [synth.mlp_weights(200 + i, hidden, inter, device) for i in range(6)]
    x = synth.activations(5, rows, hidden, device)
    h = synth.activations(6, rows, inter, device, std=0.3)
    r = synth.activations(7, rows, hidden, device)
    executors = [B.mlx_affine_mlp_executor(x, *w[0], *w[1], *w[2], r) for w in sets]
    with B.force_kernel(family):
        for i, (gate, up, down) in enumerate(sets):
            if op == "mlp":
                executors[i](x, r)
            elif op == "swiglu":
                B.mlx_affine_swiglu(x, *gate, *up)
            elif op == "down":
                B.mlx_affine_residual_qmv(h, *down, r)
            else:
                raise SystemExit(f"unknown operator {op!r}")
    torch.cuda.synchronize()
    ok, words = _lib.device_status()
    print(json.dumps({"capture": spec, "device_status_ok": bool(ok)}))
    return 0 if ok else 1


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=10)
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--capture", default=None, metavar="OP:FAMILY:ROWS",
                        help="run a few launches of one operator and exit (a small target for ncu): OP is mlp, "
                             "swiglu or down; FAMILY is default, mlp_fused, mlp_fused_mma, gemv or umma")
    args = parser.parse_args()
    if args.capture:
        return run_capture(args.capture)
    if args.impl == "reference":
        if args.steps > 20:
            args.steps = 20  # each CPU step is a full sweep (~1 s); keep the run within minutes
        if args.warmup > 3:
            args.warmup = 3
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
