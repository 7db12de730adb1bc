"""Benchmark of the INT4 fused SwiGLU MLP path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads
  llama1b   (default at N = 1)  Llama-3.2-1B MLP, hidden 2048 / intermediate 8192, group 64, swept over
            M in {1,2,4,8,16,32,128} activation rows.
  qwen32b   (default at N > 1)  Qwen2.5-32B MLP, hidden 5120 / intermediate 27648, M in {1,16,128}; with
            N > 1 ranks (torch.distributed.run, one rank per GPU) it is tensor-parallel: gate|up
            column-sharded, down row-sharded, one all-reduce per MLP; scaling is "strong".

One "step" is one sweep: the fused MLP (gate|up SwiGLU -> down + residual) once for every M of the
sweep, each call on the next of a rotating set of weight copies larger than L2.  `value` is the weight
bytes streamed per second over the whole step with all inputs resident in HBM; `e2e` is the same metric
through the public executor with HOST activations (pinned), host->device and device->host copies inside
the timed region.  The JSON line also carries per-M times (median and minimum over interleaved rounds),
the roofline of every kernel family, the other named workloads (single projection, dense rows, decoder
block, add+RMSNorm, decode attention) and a CPU baseline.

--impl reference times the reference semantics on the host cores (the C + OpenMP port under oracle/,
because MLX itself cannot be installed here) on the same workload, with every core the process may use,
and prints the same line shape with "impl": "reference".
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

WORKLOADS = {
    "llama1b": {"name": "int4_swiglu_mlp_llama3.2-1b", "hidden": 2048, "intermediate": 8192,
                "sweep": (1, 2, 4, 8, 16, 32, 128)},
    "qwen32b": {"name": "int4_swiglu_mlp_qwen2.5-32b_tp", "hidden": 5120, "intermediate": 27648,
                "sweep": (1, 16, 128)},
}
NOMINAL_HBM_GBS = 8000.0
ROUNDS = 25

# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the kernel families, from the
# ncu captures summarised in the named files under profiles/; None where no capture exists.
PROFILE_K2 = "profiles/affine_umma_llama1b.md"
TRAFFIC = {"swiglu_16": 19019264, "down_16": 9845248, "swiglu_128": 19482880, "down_128": 12145408}


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
    """Samples SM clocks and throttle reasons (read-only queries) while a timed region runs."""

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
        """In-process NVML queries: no fork while CUDA / NCCL threads are running."""
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


def host_cores():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_sweep_seconds(hidden, intermediate, sweep, repeats):
    """Time the C + OpenMP port of the reference semantics on every host core the process may use
    (launchers such as torchrun export OMP_NUM_THREADS=1, so the count is set explicitly)."""
    from metile_b200 import synth
    from oracle import cport

    cores = cport.set_threads(host_cores())
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
    return times, cores


def workload_config(workload, gpus):
    return {
        "workload": workload["name"],
        "hidden": workload["hidden"],
        "intermediate": workload["intermediate"],
        "group_size": 64,
        "bits": 4,
        "rows_sweep": list(workload["sweep"]),
        "weight_bytes_per_mlp": weight_bytes(workload["hidden"], workload["intermediate"]),
        "parallelism": "single GPU" if gpus == 1 else f"tp{gpus} (gate|up column-sharded, down row-sharded, 1 all-reduce)",
    }


def pick_workload(args):
    if args.workload:
        return WORKLOADS[args.workload]
    return WORKLOADS["qwen32b" if args.gpus > 1 else "llama1b"]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    workload = pick_workload(args)
    hidden, inter, sweep = workload["hidden"], workload["intermediate"], workload["sweep"]
    sample_sweep = sweep
    if workload is WORKLOADS["qwen32b"]:
        sample_sweep = (1, 16)  # a bounded sample: the 128-row MLP alone takes the host tens of seconds
    total_bytes = weight_bytes(hidden, inter) * len(sample_sweep)
    times, cores = cpu_sweep_seconds(hidden, inter, sample_sweep, args.warmup + args.steps)
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
        "scaling": "strong" if args.gpus > 1 else "weak",
        "vs_baseline": None,
        "dtype": "bf16 activations, u4 weights, fp32 accumulate",
        "data": "synthetic",
        "config": workload_config(workload, args.gpus),
        "tokens_per_s": sum(sample_sweep) / seconds,
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": f"{len(timed)} sweeps M={list(sample_sweep)} of the same MLP"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "timing_notes": "host memory (CPU run)",
        "note": "MLX-CPU (the reference's own CPU path) is unavailable on this box; this is the C + OpenMP "
                "port of its semantics under oracle/",
    }
    print(json.dumps(line))


def log(message):
    """Progress on stderr (the JSON line alone goes to stdout)."""
    if os.environ.get("RANK", "0") == "0":
        print(f"[bench {time.strftime('%H:%M:%S')}] {message}", file=sys.stderr, flush=True)


class Timer:
    """CUDA-graph capture / replay and CUDA-event timing on one side stream."""

    def __init__(self, torch):
        self.torch = torch
        self.stream = torch.cuda.Stream()

    def capture(self, fn, repeats):
        torch = self.torch
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(self.stream):
            fn()
            self.stream.synchronize()
            with torch.cuda.graph(graph, stream=self.stream):
                for _ in range(repeats):
                    fn()
        torch.cuda.synchronize()
        return graph

    def warm(self, graph):
        """One untimed replay on the timer's stream, finished before anything else is queued."""
        self.replay_seconds(graph, 1)

    def replay_seconds(self, graph, replays):
        torch = self.torch
        with torch.cuda.stream(self.stream):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(self.stream)
            for _ in range(replays):
                graph.replay()
            stop.record(self.stream)
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e-3

    def eager_seconds(self, fn, repeats):
        torch = self.torch
        torch.cuda.synchronize()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(repeats):
            fn()
        stop.record()
        torch.cuda.synchronize()
        return start.elapsed_time(stop) * 1e-3

    def interleaved_rounds(self, graphs, calls_per_replay, rounds=ROUNDS):
        """{key: [seconds per call, one entry per round]}: every round replays every graph once, in an
        order that alternates from round to round, so that slow drifts hit all of them alike."""
        samples = {key: [] for key in graphs}
        keys = list(graphs)
        for r in range(rounds):
            for key in (keys if r % 2 == 0 else keys[::-1]):
                samples[key].append(self.replay_seconds(graphs[key], 1) / calls_per_replay)
        return samples


def summarise(seconds_list):
    return {"median_us": statistics.median(seconds_list) * 1e6, "min_us": min(seconds_list) * 1e6,
            "rounds": len(seconds_list)}


def other_workloads(torch, device, timer, hbm_peak):
    """The other named workloads on one GPU: single INT4 projection, dense bf16 rows, the
    Qwen2.5-1.5B-shaped decoder block (prefill and decode), add+RMSNorm and decode attention."""
    from metile_b200 import backends as B
    from metile_b200 import synth
    from metile_b200.integrations import blocks, torch_lm

    out = {}

    def per_call(fn, calls_in_fn):
        graph = timer.capture(fn, 4)
        timer.warm(graph)
        return summarise([timer.replay_seconds(graph, 1) / (4 * calls_in_fn) for _ in range(ROUNDS)])

    def with_rates(stats, bytes_per_call):
        gbps = bytes_per_call / (stats["median_us"] * 1e-6) / 1e9
        return {**stats, "algorithmic_bytes": int(bytes_per_call), "GBps": gbps, "frac_of_hbm": gbps / hbm_peak}

    # ---- single projection: M = 1, K = 1536, N = 8960 ------------------------------------------------
    k, n = 1536, 8960
    copies = 40  # 40 x 7.7 MB = 310 MB > 2 x L2
    weights = [synth.affine_weight(900 + i, n, k, device) for i in range(copies)]
    x = synth.activations(1, 1, k, device)

    def gemv():
        for w in weights:
            B.mlx_affine_qmv(x, *w)

    out["int4_projection_m1_k1536_n8960"] = with_rates(per_call(gemv, copies),
                                                       n * k * (0.5 + 4 / 64) + x.numel() * 2 + n * 2)
    del weights

    # ---- dense bf16 rows: K = 1536, N = 8960, M swept; rows bit-identical to running alone ------------
    copies = 12  # 12 x 27.5 MB = 330 MB
    dense = [synth.dense_weight(950 + i, n, k, device) for i in range(copies)]
    rows_full = synth.activations(2, 128, k, device)
    dense_detail = []
    alone = torch.cat([B.mlx_dense_residual_qmv(rows_full[i:i + 1], dense[0]) for i in range(8)])
    for m in (1, 2, 4, 8, 16, 32, 128):
        xm = rows_full[:m]

        def dense_rows(xm=xm):
            for w in dense:
                B.mlx_dense_residual_qmv(xm, w)

        batch = B.mlx_dense_residual_qmv(xm, dense[0])
        identical = bool((batch[:min(m, 8)].view(torch.uint16) == alone[:min(m, 8)].view(torch.uint16)).all())
        dense_detail.append({"rows": m, **with_rates(per_call(dense_rows, copies), n * k * 2 + m * k * 2 + m * n * 2),
                             "rows_bit_identical_to_running_alone": identical})
    out["dense_bf16_rows_k1536_n8960"] = dense_detail
    del dense

    # ---- add + RMSNorm ---------------------------------------------------------------------------------
    norm_w = synth.norm_weight(3, 1536, device)
    for rows in (16, 512):
        a = synth.activations(4, rows, 1536, device)
        r = synth.activations(5, rows, 1536, device)

        def add_norm(a=a, r=r):
            B.mlx_add_rms_norm(a, r, norm_w, 1e-6)

        entry = with_rates(per_call(add_norm, 1), rows * 1536 * 2 * 4 + 1536 * 2)
        entry["note"] = "inputs and outputs fit L2: bound by launch latency at this size, not by HBM"
        out[f"add_rmsnorm_{rows}x1536"] = entry

    # ---- decode attention: 16 sequences, 12 query / 2 KV heads of 128, KV length 2048 -------------------
    batch, q_heads, kv_heads, tokens, dim = 16, 12, 2, 2048, 128
    caches = 12  # 12 x 33.5 MB = 400 MB of keys and values
    q = synth.activations(6, batch * q_heads, dim, device).reshape(batch, q_heads, 1, dim)
    kvs = []
    for _ in range(caches):
        keys = torch.empty((batch, kv_heads, tokens, dim), dtype=torch.bfloat16, device=device).normal_(0, 0.5)
        kvs.append((keys, torch.empty_like(keys).normal_(0, 0.5)))

    def attention():
        for keys, values in kvs:
            B.mlx_attention_decode(q, keys, values, scale=dim ** -0.5)

    entry = with_rates(per_call(attention, caches), 2 * batch * kv_heads * tokens * dim * 2)
    entry["kernels_per_call"] = 2
    out["decode_attention_16x12q2kv_d128_kv2048"] = entry
    del kvs

    # ---- the Qwen2.5-1.5B-shaped decoder block: prefill of 512 tokens, 16-row decode at KV 2048 ---------
    hidden, inter = 1536, 8960

    def linear(seed, fan_in, fan_out):
        return blocks.QuantizedLinear.from_seed(seed, fan_in, fan_out, device)

    block_copies = 8  # 8 x 26.3 MB of INT4 weights + 8 x 33.5 MB of cache
    block_list = []
    for c in range(block_copies):
        base = 100 * c
        attn = blocks.Attention(linear(base + 1, hidden, 1536), linear(base + 2, hidden, 256), linear(base + 3, hidden, 256),
                                linear(base + 4, 1536, hidden), 12, 2, 128, 1e6)
        mlp = blocks.GatedMLP(linear(base + 5, hidden, inter), linear(base + 6, hidden, inter), linear(base + 7, inter, hidden))
        block_list.append(blocks.DecoderBlock(blocks.RMSNorm(synth.norm_weight(base + 8, hidden, device), 1e-6), attn,
                                              blocks.RMSNorm(synth.norm_weight(base + 9, hidden, device), 1e-6), mlp))
    model = torch.nn.Module()
    model.layers = torch.nn.ModuleList(block_list)
    decode_x = synth.activations(7, 16, hidden, device, std=0.5).reshape(16, 1, hidden)
    prefill_x = synth.activations(8, 512, hidden, device, std=0.5).reshape(1, 512, hidden)
    decode_caches = []
    for c in range(block_copies):
        cache = blocks.KVCache(16, 2, 2048, 128, device)
        cache.keys.normal_(0, 0.5)
        cache.values.normal_(0, 0.5)
        decode_caches.append(cache)

    def rewind(cache):
        cache.length = 2047
        cache.positions.fill_(2047)

    def count_kernels(fn):
        """Kernels launched by one call of `fn` (torch profiler, CUDA activity; nothing here is timed)."""
        try:
            from torch.profiler import ProfilerActivity, profile

            with profile(activities=[ProfilerActivity.CUDA]) as prof:
                fn()
                torch.cuda.synchronize()
            return sum(1 for event in prof.events() if "kernel" in str(event.device_type).lower()
                       or event.device_type.name == "CUDA")
        except Exception:
            return None

    results = {}
    launches = {}
    with torch.no_grad():
        for patched in (False, True):
            key = "patched" if patched else "unpatched"
            handle = torch_lm.apply_metile_to_torch_lm(model, attention=True) if patched else None
            try:
                def decode_step():
                    for block, cache in zip(block_list, decode_caches):
                        rewind(cache)
                        block(decode_x, cache)

                def prefill_step():
                    for block in block_list:
                        block(prefill_x, blocks.KVCache(1, 2, 512, 128, device))

                for fn, label in ((decode_step, "decode_16_rows_kv2048"), (prefill_step, "prefill_512")):
                    fn()
                    torch.cuda.synchronize()
                    times = [timer.eager_seconds(fn, 1) / block_copies for _ in range(ROUNDS)]
                    results.setdefault(label, {})[key] = summarise(times)

                def one_decode():
                    rewind(decode_caches[0])
                    block_list[0](decode_x, decode_caches[0])

                launches[key] = count_kernels(one_decode)
                if patched:
                    results["refusals"] = dict(handle.refusals)
                    # The same patched step replayed as a CUDA graph: what the kernels take without the
                    # interpreter between them (the eager numbers above are bound by Python dispatch).
                    try:
                        graph = timer.capture(decode_step, 1)
                        timer.warm(graph)
                        replays = [timer.replay_seconds(graph, 1) / block_copies for _ in range(ROUNDS)]
                        results["decode_16_rows_kv2048"]["patched_graph_replay"] = summarise(replays)
                    except Exception as error:  # capture is a convenience of the harness, not of the library
                        results["decode_16_rows_kv2048"]["patched_graph_replay"] = {"unavailable": str(error)[:200]}
            finally:
                if handle is not None:
                    handle.restore()
    block_bytes = 26320896
    kv_bytes = 2 * 16 * 2 * 2048 * 128 * 2
    for label in ("decode_16_rows_kv2048", "prefill_512"):
        entry = results[label]
        entry["speedup_patched_over_unpatched"] = entry["unpatched"]["median_us"] / entry["patched"]["median_us"]
    decode = results["decode_16_rows_kv2048"]
    decode["algorithmic_bytes"] = block_bytes + kv_bytes
    decode["patched_GBps"] = (block_bytes + kv_bytes) / (decode["patched"]["median_us"] * 1e-6) / 1e9
    decode["patched_frac_of_hbm"] = decode["patched_GBps"] / hbm_peak
    decode["gpu_kernels_per_decode_step"] = launches
    replay = decode.get("patched_graph_replay", {})
    if "median_us" in replay:
        decode["patched_graph_GBps"] = (block_bytes + kv_bytes) / (replay["median_us"] * 1e-6) / 1e9
        decode["patched_graph_frac_of_hbm"] = decode["patched_graph_GBps"] / hbm_peak
    results["timing"] = "eager launches, CUDA events (the unpatched block runs torch operators)"
    out["qwen2.5-1.5b_decoder_block"] = results
    del block_list, decode_caches, model
    torch.cuda.empty_cache()

    # ---- output projection at vocabulary size: N = 128256, K = 2048 (Llama-3.2-1B lm_head) -------------
    vocabulary, width = 128256, 2048
    heads_w = [synth.affine_weight(980 + i, vocabulary, width, device) for i in range(2)]  # 2 x 148 MB
    lm_head = []
    for m in (1, 16):
        xm = synth.activations(9, m, width, device, std=0.5)

        def project(xm=xm):
            for w in heads_w:
                B.mlx_affine_qmv(xm, *w)

        lm_head.append({"rows": m, **with_rates(per_call(project, 2),
                                                vocabulary * width * (0.5 + 4 / 64) + m * width * 2 + m * vocabulary * 2)})
    out["int4_lm_head_k2048_n128256"] = lm_head
    del heads_w

    # ---- the 32B-shaped MLP (hidden 5120 / intermediate 27648) unsharded: the one-GPU point of the
    # tensor-parallel series that `--gpus N` runs ---------------------------------------------------------
    big_h, big_i = 5120, 27648
    big_sets = [synth.mlp_weights(100, big_h, big_i, device) for _ in range(2)]  # 2 x 239 MB
    sample = synth.activations(5, 1, big_h, device)
    big_execs = [B.mlx_affine_mlp_executor(sample, *w[0], *w[1], *w[2], sample) for w in big_sets]
    big_bytes = 3 * big_h * big_i * (0.5 + 4 / 64)
    big_rows = []
    for m in (1, 16, 128):
        xm = synth.activations(6, m, big_h, device)
        rm = synth.activations(7, m, big_h, device)

        def big_mlp(xm=xm, rm=rm):
            for execute in big_execs:
                execute(xm, rm)

        big_rows.append({"rows": m, **with_rates(per_call(big_mlp, 2), big_bytes + 3 * m * big_h * 2)})
    sweep_us = sum(r["median_us"] for r in big_rows)
    out["qwen2.5-32b_mlp_5120_27648_one_gpu"] = {
        "per_rows": big_rows, "sweep_ms": sweep_us * 1e-3,
        "value_GBps": 3 * big_bytes / (sweep_us * 1e-6) / 1e9,
        "note": "same sweep M = 1, 16, 128 and the same value definition as the tensor-parallel runs (--gpus N)"}
    del big_sets, big_execs
    torch.cuda.empty_cache()

    # ---- feature plan of a four-layer model at the block's shape, chosen by timing its decode loop -------
    from metile_b200.integrations import autotune

    lm = blocks.random_model(seed=21, hidden=1536, intermediate=8960, heads=12, kv_heads=2, head_dim=128, layers=4,
                             vocab=32768, device=device, tie_word_embeddings=True)
    prompt = torch.randint(1, 32768, (1, 32), generator=torch.Generator().manual_seed(3)).to(device)
    plan = autotune.autotune_metile_for_torch_lm(lm, prompt, decode_steps=8, trials=5)
    chosen = next((m for m in plan.report.measurements if m.plan == plan), None)
    # The selected plan with its decode step captured as a CUDA graph (device-side argmax feeds the next
    # step): what the kernels take per token without the interpreter between them.
    graphed_us = None
    try:
        from metile_b200.integrations.graphed import GraphedDecoder

        with plan.apply(lm):
            decoder = GraphedDecoder(lm, batch=1, capacity=256)
            first = decoder.prefill(prompt).argmax(dim=-1)
            decoder.generate(first, 4)
            torch.cuda.synchronize()
            samples = []
            for _ in range(5):
                first = decoder.prefill(prompt).argmax(dim=-1)
                torch.cuda.synchronize()
                begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                begin.record()
                decoder.generate(first, 32)
                end.record()
                torch.cuda.synchronize()
                samples.append(begin.elapsed_time(end) * 1e3 / 32)
            graphed_us = statistics.median(samples)
    except Exception as error:  # the harness is a convenience; the plan numbers above stand without it
        graphed_us = f"unavailable: {str(error)[:160]}"
    out["feature_plan_4_layers_1536_8960"] = {
        "selected": [name for name, on in plan.flags.items() if on],
        "unpatched_us_per_token": plan.report.baseline_seconds_per_token * 1e6,
        "selected_us_per_token": None if chosen is None else chosen.seconds_per_token * 1e6,
        "selected_us_per_token_cuda_graph": graphed_us,
        "subsets_measured": len(plan.report.measurements),
        "subsets_rejected": [m.reason for m in plan.report.measurements if not m.valid],
        "timing": "eager decode loop, batch 1, 8 steps, median of 5 interleaved rounds",
    }
    return out


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
    workload = pick_workload(args)
    hidden, inter, sweep = workload["hidden"], workload["intermediate"], workload["sweep"]
    per_mlp_bytes = weight_bytes(hidden, inter)
    local_bytes = per_mlp_bytes // world
    l2_bytes = torch.cuda.get_device_properties(device).L2_cache_size
    copies = max(2, -(-2 * l2_bytes // local_bytes) + 1)
    copies = min(copies, 24)
    hbm_peak, tensor_peak, peak_kind = measured_peaks()
    timer = Timer(torch)
    library = _lib.load()

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

    def max_over_ranks(value):
        if not distributed:
            return value
        t = torch.tensor([value], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- headline: K steps, each one sweep ------------------------------------------------------------
    # The sweep is replayed as a CUDA graph, on one GPU and tensor-parallel alike: the sum over the ranks
    # is the library's own kernel (its call counter lives on the device), so every rank replays the same
    # graph and no NCCL call sits inside it.
    log("weights resident; warm-up")
    for _ in range(3):
        sweep_once()
    torch.cuda.synchronize()
    barrier()
    step_graph = timer.capture(sweep_once, 1)
    run_steps = lambda n: timer.replay_seconds(step_graph, n)  # noqa: E731
    run_steps(max(args.warmup, 3))
    barrier()
    with ClockSampler(local_rank) as clocks:
        seconds = run_steps(args.steps)
        barrier()
        seconds = max_over_ranks(seconds)
        # Keep the sampler alive long enough for a few samples when the steps are very short.  The number
        # of extra replays comes from the rank-agreed time: every rank must launch the same number of
        # exchange kernels.
        if seconds < 0.5:
            run_steps(max(1, int(0.5 / max(seconds / args.steps, 1e-6))))
    step_seconds = seconds / args.steps
    total_bytes = per_mlp_bytes * len(sweep)
    value = total_bytes / step_seconds / 1e9
    log(f"headline: {step_seconds * 1e3:.3f} ms per step")

    def check_device(where):
        """Stop at once if a bounded device-side wait gave up (ranks out of step would otherwise spend
        the wait limit on every later exchange)."""
        ok, words = _lib.device_status()
        if not ok:
            raise SystemExit(f"a device-side wait gave up {where}: status words {[hex(w) for w in words]}")

    check_device("during the headline steps")

    # ---- per-M detail: interleaved rounds, median and minimum -------------------------------------------
    def detail_for(flags=0):
        graphs = {}
        for m in sweep:
            x, r = inputs[m]

            def one(x=x, r=r):
                next_executor()(x, r)

            graphs[m] = timer.capture(one, 8)
            timer.warm(graphs[m])
        barrier()
        samples = timer.interleaved_rounds(graphs, 8)
        if tp:  # the slowest rank of every round
            samples = {m: [max_over_ranks(v) for v in values] for m, values in samples.items()}
        rows = []
        for m in sweep:
            stats = summarise(samples[m])
            per_call = stats["median_us"] * 1e-6
            flops = 2.0 * 3 * hidden * inter * m
            hbm_seconds = local_bytes / (hbm_peak * 1e9)
            tensor_seconds = flops / world / (tensor_peak * 1e12)
            rows.append({
                "rows": m,
                "us": stats["median_us"],
                "min_us": stats["min_us"],
                "rounds": stats["rounds"],
                "weight_GBps": per_mlp_bytes / per_call / 1e9,
                "tokens_per_s": m / per_call,
                "frac_of_hbm": (local_bytes / per_call / 1e9) / hbm_peak,
                "frac_of_nominal_8TBps": (local_bytes / per_call / 1e9) / NOMINAL_HBM_GBS,
                "bound": "hbm" if hbm_seconds >= tensor_seconds else "tensor",
                "frac_of_roofline": max(hbm_seconds, tensor_seconds) / per_call,
                "kernels_per_mlp": library.mt_affine_mlp_launches(m, hidden, inter // world, flags),
            })
        return rows

    log("per-M detail")
    detail = detail_for()
    check_device("during the per-M rounds")
    sweep_invariant = None
    if not tp:
        log("per-M detail, batch-invariant mode (one kernel family for every batch size)")
        with B.batch_invariant():
            sweep_invariant = detail_for(_lib.FLAG_FORCE_UMMA)

    # ---- roofline per kernel family, each timed alone; the headline one is the family with the largest
    # share of the step (launches in a sweep x its duration) ------------------------------------------
    roofline = None
    roofline_kernels = []
    tp_extra = {}
    if not tp:
        weight_sets = [synth.mlp_weights(100, hidden, inter, device) for _ in range(copies)]
        cursor = [0]

        def per_launch_seconds(fn, launches_per_call):
            graph = timer.capture(fn, 16)
            timer.warm(graph)
            return statistics.median([timer.replay_seconds(graph, 1) / (16 * launches_per_call) for _ in range(ROUNDS)])

        def entry(kernel, rows_served, seconds, algorithmic, traffic, profile, bound="hbm", flops=0.0):
            achieved = algorithmic / seconds / 1e9
            item = {
                "kernel": kernel,
                "bound": bound,
                "achieved": achieved,
                "peak": hbm_peak,
                "unit": "GB/s",
                "frac": achieved / hbm_peak,
                "peak_kind": f"of {peak_kind}",
                "traffic": traffic,
                "traffic_source": profile,
                "algorithmic_bytes_per_launch": int(algorithmic),
                "us_per_launch": seconds * 1e6,
                "launches_per_sweep": sum(1 for m in sweep if m in rows_served),
            }
            if bound == "tensor":
                item.update({"achieved": flops / seconds / 1e12, "peak": tensor_peak, "unit": "TFLOP/s",
                             "frac": flops / seconds / 1e12 / tensor_peak, "hbm_frac": achieved / hbm_peak})
            return item

        packed = hidden * inter * (0.5 + 4 / 64)  # one projection: nibbles + bf16 scales and biases
        single_rows = [m for m in sweep if library.mt_affine_mlp_launches(m, hidden, inter, 0) == 1]
        for rows_served, label, traffic, profile in (
                ([m for m in single_rows if m <= 1], "single-launch MLP on CUDA cores (affine_mlp_fused_kernel)", 28378368,
                 "profiles/affine_mlp_fused_m1_llama1b.md"),
                ([m for m in single_rows if m > 1], "single-launch MLP on mma.sync (affine_mlp_fused_mma_kernel)", 28456192,
                 "profiles/affine_mlp_fused_mma_m8_llama1b.md")):
            if not rows_served:
                continue
            m = rows_served[0] if rows_served[0] <= 1 else rows_served[-1]
            xm, rm = inputs[m]
            executors_m = [B.mlx_affine_mlp_executor(xm, *w[0], *w[1], *w[2], rm) for w in weight_sets]

            def whole_mlp(executors_m=executors_m, xm=xm, rm=rm):
                cursor[0] = (cursor[0] + 1) % copies
                executors_m[cursor[0]](xm, rm)

            roofline_kernels.append(entry(
                f"{label}, M={m}", rows_served, per_launch_seconds(whole_mlp, 1),
                3 * packed + 2 * m * hidden * 2 + 2 * m * inter * 2 + m * hidden * 2, traffic, profile))
        two_kernel_rows = [m for m in sweep if m not in single_rows]
        for m, rows_served in ((16, [r for r in two_kernel_rows if r <= 32]), (128, [r for r in two_kernel_rows if r > 32])):
            if not rows_served or m not in inputs:
                continue
            xs, rs = inputs[m]
            hs = synth.activations(11, m, inter, device, std=0.3)

            def gate_up(xs=xs):
                cursor[0] = (cursor[0] + 1) % copies
                gate, up, _ = weight_sets[cursor[0]]
                B.mlx_affine_swiglu(xs, *gate, *up)

            def down_projection(hs=hs, rs=rs):
                cursor[0] = (cursor[0] + 1) % copies
                B.mlx_affine_residual_qmv(hs, *weight_sets[cursor[0]][2], rs)

            bound = "tensor" if m >= 128 else "hbm"
            roofline_kernels.append(entry(
                f"gate|up SwiGLU on tcgen05, {m}-row instance (affine_umma_kernel<2,{m}>)", rows_served,
                per_launch_seconds(gate_up, 1), 2 * packed + m * hidden * 2 + m * inter * 2, TRAFFIC[f"swiglu_{m}"],
                PROFILE_K2, bound, 2.0 * 2 * hidden * inter * m))
            roofline_kernels.append(entry(
                f"down projection on tcgen05, {m}-row instance (affine_umma_kernel<1,{m}>)", rows_served,
                per_launch_seconds(down_projection, 1), packed + m * inter * 2 + 2 * m * hidden * 2,
                TRAFFIC[f"down_{m}"], PROFILE_K2, bound, 2.0 * hidden * inter * m))
        if roofline_kernels:
            roofline = max(roofline_kernels, key=lambda e: e["launches_per_sweep"] * e["us_per_launch"])
        del weight_sets
    else:
        # ---- tensor-parallel extras -------------------------------------------------------------------
        # (1) this rank's shard MLP alone (no collective), replayed as a graph: the roofline of its kernels;
        # (2) the all-reduce alone; (3) the SAME workload unsharded on one GPU; (4) parity of the sharded
        # result against the unsharded executor on the same inputs (every rank's GPU holds both).
        shard_detail = []
        for m in sweep:
            x, r = inputs[m]

            def shard_only(x=x, r=r):
                next_executor().partial(x, r)

            graph = timer.capture(shard_only, 8)
            timer.warm(graph)
            shard_seconds = statistics.median([timer.replay_seconds(graph, 1) / 8 for _ in range(ROUNDS)])
            buffer = torch.empty((m, hidden), dtype=torch.bfloat16, device=device)

            peer_sum = tensor_parallel.shared_peer_all_reduce(device, rank, world, 128 * hidden)

            def reduce_only(buffer=buffer):
                peer_sum(buffer)

            def nccl_only(buffer=buffer):
                dist.all_reduce(buffer)

            buffer.zero_()
            reduce_only()
            torch.cuda.synchronize()
            barrier()
            reduce_graph = timer.capture(reduce_only, 8)
            timer.warm(reduce_graph)
            barrier()
            reduce_times = [max_over_ranks(statistics.median(
                [timer.replay_seconds(reduce_graph, 1) / 8 for _ in range(ROUNDS)]))]
            buffer.zero_()
            timer.eager_seconds(nccl_only, 8)
            barrier()
            reduce_times.append(max_over_ranks(
                statistics.median([timer.eager_seconds(nccl_only, 16) / 16 for _ in range(ROUNDS)])))
            reduce_seconds, nccl_seconds = reduce_times
            shard_seconds = max_over_ranks(shard_seconds)
            shard_detail.append({"rows": m, "shard_mlp_us": shard_seconds * 1e6, "all_reduce_us": reduce_seconds * 1e6,
                                 "nccl_all_reduce_us": nccl_seconds * 1e6,
                                 "shard_GBps": local_bytes / shard_seconds / 1e9,
                                 "shard_frac_of_hbm": local_bytes / shard_seconds / 1e9 / hbm_peak})
        worst = max(shard_detail, key=lambda e: e["shard_mlp_us"])
        tp_extra["decomposition"] = shard_detail
        roofline = {
            "kernel": f"this rank's shard MLP (gate|up + down kernels, no collective), M={worst['rows']}",
            "bound": "hbm", "achieved": worst["shard_GBps"], "peak": hbm_peak, "unit": "GB/s",
            "frac": worst["shard_frac_of_hbm"], "peak_kind": f"of {peak_kind}", "traffic": None,
            "algorithmic_bytes_per_launch": int(local_bytes), "us_per_launch": worst["shard_mlp_us"],
        }

        full_sets = [synth.mlp_weights(100, hidden, inter, device) for _ in range(2)]
        sample = synth.activations(5, 1, hidden, device)
        full_executors = [B.mlx_affine_mlp_executor(sample, *w[0], *w[1], *w[2], sample) for w in full_sets]
        flip = [0]

        def unsharded_sweep():
            for m in sweep:
                flip[0] ^= 1
                full_executors[flip[0]](*inputs[m])

        timer.eager_seconds(unsharded_sweep, 3)
        barrier()
        one_seconds = max_over_ranks(timer.eager_seconds(unsharded_sweep, args.steps) / args.steps)
        tp_extra["one_gpu_same_workload"] = {
            "value": per_mlp_bytes * len(sweep) / one_seconds / 1e9, "unit": "GB/s", "ms_per_step": one_seconds * 1e3,
            "note": "same sweep, unsharded, one GPU (every rank runs it at once; slowest rank), "
                    f"two weight sets of {per_mlp_bytes / 1e6:.0f} MB alternating"}
        tp_extra["tp_speedup"] = one_seconds / step_seconds
        parity = []
        for m in sweep:
            x, r = inputs[m]
            sharded = executors[0](x, r).float()
            unsharded = full_executors[0](x, r).float()
            peak = float(unsharded.abs().max().item())
            error = float((sharded - unsharded).abs().max().item())
            # Every rank must hold the same bits: the exchange adds the partials in rank order everywhere.
            digest = sharded.double().sum().reshape(1)
            lowest, highest = digest.clone(), digest.clone()
            dist.all_reduce(lowest, op=dist.ReduceOp.MIN)
            dist.all_reduce(highest, op=dist.ReduceOp.MAX)
            parity.append({"rows": m, "max_err_over_peak": error / peak, "ok": bool(error <= 6e-3 * peak),
                           "same_on_every_rank": bool((lowest == highest).item())})
        ok_everywhere = max_over_ranks(0.0 if all(p["ok"] and p["same_on_every_rank"] for p in parity) else 1.0) == 0.0
        tp_extra["tp_parity"] = {"per_rows": parity, "ok": ok_everywhere,
                                 "bound": "6e-3 of the unsharded result's peak: each of the two results is within 3e-3 "
                                          "of the exact-arithmetic MLP (the bound of the parity tests against the "
                                          "oracle, sharded shapes included), so they are within 6e-3 of each other",
                                 "reference": "the unsharded executor on each rank's own GPU, same inputs; ok on every rank"}
        del full_executors, full_sets

    log("roofline / tensor-parallel extras done")
    # ---- end to end with host buffers ---------------------------------------------------------------
    # Single GPU: the C-ABI host entry point (mt_affine_mlp_host through mlx_affine_mlp_host_executor):
    # one call queues the two host->device copies, the MLP and the device->host copy.  Tensor-parallel:
    # the sharded executor on device tensors with the copies issued around it.
    host_executors = None
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

    log("e2e")
    for _ in range(3):
        e2e_step()
    barrier()
    start = time.perf_counter()
    for _ in range(args.steps):
        e2e_step()
    barrier()
    e2e_seconds = max_over_ranks((time.perf_counter() - start) / args.steps)
    h2d = sum(2 * m * hidden * 2 for m in sweep)
    d2h = sum(m * hidden * 2 for m in sweep)

    # ---- the other named workloads (single GPU) -------------------------------------------------------
    others = None
    if not tp and not args.skip_other:
        log("other workloads")
        host_executors = None
        executors.clear()
        torch.cuda.empty_cache()
        others = other_workloads(torch, device, timer, hbm_peak)

    # ---- CPU baseline (rank 0): a bounded sample of the same workload on the host cores ----------------
    cpu_baseline = None
    if rank == 0:
        log("cpu baseline")
        cpu_sweep = sweep if workload is WORKLOADS["llama1b"] else (1, 16)
        times, cores = cpu_sweep_seconds(hidden, inter, cpu_sweep, 3 if workload is WORKLOADS["llama1b"] else 2)
        cpu_seconds = min(times)
        cpu_baseline = {"value": per_mlp_bytes * len(cpu_sweep) / cpu_seconds / 1e9, "unit": "GB/s", "cores": cores,
                        "kind": "port",
                        "sample": f"{len(times)} sweeps M={list(cpu_sweep)} of the same MLP (best), C + OpenMP port of "
                                  "the reference semantics; MLX-CPU is unavailable on this box"}

    if rank == 0:
        launches_per_sweep = sum(library.mt_affine_mlp_launches(m, hidden, inter // world, 0) for m in sweep)
        if tp:
            launches_per_sweep += len(sweep)  # the exchange kernel after every shard MLP
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
            "config": workload_config(workload, world),
            "timing_notes": f"rotating {copies} weight sets ({copies * local_bytes / 1e6:.0f} MB per GPU) > 2x L2 "
                            f"({l2_bytes / 1e6:.0f} MB); per-M numbers are medians of {ROUNDS} interleaved rounds",
            "tokens_per_s": sum(sweep) / step_seconds,
            "frac_of_hbm_peak": (local_bytes * len(sweep) / step_seconds / 1e9) / hbm_peak,
            "sweep": detail,
            "sweep_invariant": sweep_invariant,
            "roofline": roofline,
            "roofline_kernels": roofline_kernels,
            **tp_extra,
            "other_workloads": others,
            "cpu_baseline": cpu_baseline,
            "e2e": {"value": total_bytes / e2e_seconds / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": e2e_seconds * 1e3},
            "gpu_launches": launches_per_sweep * args.steps,
            "timing": "CUDA-graph replay, CUDA events",
            "clocks": clocks.summary(),
        }
        print(json.dumps(line))
    failed = bool(tp_extra) and not tp_extra["tp_parity"]["ok"]
    if distributed:
        if tp:
            tensor_parallel.close_peer_groups()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("tensor-parallel result differs from the unsharded result beyond the bound")


def run_capture(spec):
    """Six launches of one operator over rotating weight sets larger than L2 (the Llama-3.2-1B MLP and
    its projections, decode attention, dense bf16 rows, the LM head), nothing timed and nothing printed
    but a status line: the process profilers attach to."""
    import torch

    from metile_b200 import _lib
    from metile_b200 import backends as B
    from metile_b200 import synth

    op, family, rows = spec.split(":")
    rows = int(rows)
    family = None if family == "default" else family
    hidden, inter = 2048, 8192
    device = torch.device("cuda:0")
    if op == "attention":
        # `rows` sequences x 2 KV heads x 2048 tokens x 128: six caches of 4 MB per sequence rotate.
        heads, kv_heads, tokens, dim = 12, 2, 2048, 128
        query = synth.activations(1, rows * heads, dim, device).reshape(rows, heads, 1, dim)
        caches = [(synth.activations(10 + i, rows * kv_heads * tokens, dim, device, std=0.5).reshape(rows, kv_heads, tokens, dim),
                   synth.activations(20 + i, rows * kv_heads * tokens, dim, device, std=0.5).reshape(rows, kv_heads, tokens, dim))
                  for i in range(6)]
        for keys, values in caches:
            B.mlx_attention_decode(query, keys, values, scale=dim ** -0.5)
        torch.cuda.synchronize()
        ok, words = _lib.device_status()
        print(json.dumps({"capture": spec, "device_status_ok": bool(ok)}))
        return 0 if ok else 1
    if op in ("dense", "lm_head"):
        # dense: bf16 rows against six 1536 x 8960 matrices (165 MB); lm_head: the INT4 projection onto a
        # 128256-token vocabulary, two weight sets (148 MB each).
        if op == "dense":
            k, n = 1536, 8960
            weights = [synth.dense_weight(950 + i, n, k, device) for i in range(6)]
        else:
            k, n = 2048, 128256
            weights = [synth.affine_weight(700 + i, n, k, device) for i in range(2)] * 3
        values = synth.activations(5, rows, k, device)
        with B.force_kernel(family):
            for weight in weights:
                if op == "dense":
                    B.mlx_dense_residual_qmv(values, weight)
                else:
                    B.mlx_affine_qmv(values, *weight)
        torch.cuda.synchronize()
        ok, words = _lib.device_status()
        print(json.dumps({"capture": spec, "device_status_ok": bool(ok)}))
        return 0 if ok else 1
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
    parser.add_argument("--workload", choices=tuple(WORKLOADS), default=None,
                        help="llama1b (default on one GPU) or qwen32b (default with --gpus > 1; on one GPU it "
                             "runs unsharded: the N = 1 point of the tensor-parallel series)")
    parser.add_argument("--skip-other", action="store_true", help="leave out the other named workloads")
    parser.add_argument("--capture", default=None, metavar="OP:FAMILY:ROWS",
                        help="run a few launches of one operator and exit (a small target for ncu): OP is mlp, "
                             "swiglu, down, attention (ROWS = sequences), dense or lm_head; FAMILY is default, mlp_fused, "
                             "mlp_fused_mma, gemv or umma")
    args = parser.parse_args()
    if args.capture:
        return run_capture(args.capture)
    if args.impl == "reference":
        # Each CPU step is a full sweep (about a second): the same warm-up as the other arm up to ten
        # steps, and as many timed steps as keep the run within minutes.
        args.warmup = min(max(args.warmup, 3), 10)
        args.steps = min(args.steps, 20)
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
