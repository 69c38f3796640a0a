#!/usr/bin/env python
"""Benchmark of the SPN joint log-likelihood hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--config 2]

One "step" = one pass of the engine over one resident batch of synthetic samples.  The default
workload is BASELINE.json's second configuration (the one the metric is quoted on): a seeded random
SPN over 26 Gaussian features (~2,000 nodes, depth 8), 10 M float32 samples per GPU, f32 log-space.
With N > 1 (launched under torchrun, one rank per GPU) every rank evaluates its own 10 M-sample shard
of the batch with the replicated model: weak scaling, no collective on the data path.

Rank 0 prints ONE JSON line.  `value` is samples/s with inputs resident in HBM (CUDA-event timed on
the launching stream, max over ranks); `e2e` is the same metric through the host-pointer C-ABI call
(pinned host buffers, H2D and D2H inside the timed region); `roofline` relates the kernel's
algorithmic bytes to the measured HBM peak and `roofline_compute` its algorithmic FP32 / SFU
operations to issue rates measured on the same device; `cpu_baseline` times the CPU restatement of
the reference's vectorised path on the host cores for a bounded sample.

`--impl reference` times that CPU restatement alone (the reference itself cannot be built here).
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "spn-compiler_b200", "python"))

CONFIGS = {
    1: dict(name="cfg1: 16 categorical features, ~400 nodes, int32 in, f64 linear", n=1_000_000, log_space=False,
            marginal=False),
    2: dict(name="cfg2: 26 Gaussian features, ~2000 nodes, depth 8, f32 log-space", n=10_000_000, log_space=True,
            marginal=True),
    3: dict(name="cfg3: 100 histogram features, ~8000 nodes, depth 10, 10% NaN, f32 log-space", n=4_000_000,
            log_space=True, marginal=True),
    4: dict(name="cfg4: 256 mixed features, ~50000-node DAG, f32 log-space", n=4_000_000,
            log_space=True, marginal=True),
    5: dict(name="cfg5: RAT-SPN-style layered SPN, 784 Gaussian features, 16 repetitions, 32x1024 dense sums, f32 log-space",
            n=2_000_000, log_space=True, marginal=True,
            layered=dict(num_features=784, depth=4, repetitions=16, width=32)),   # synth.config5's defaults
}


MEASURED_DRAM_BYTES_PER_SAMPLE = {2: 108.398}


def build_workload(cfg_id, workdir):
    """-> (xspn query path, function n -> inputs)"""
    from spnb import synth
    spn = getattr(synth, "config%d" % cfg_id)()
    path = os.path.join(workdir, "bench_cfg%d.bin" % cfg_id)
    with open(path, "wb") as f:
        f.write(spn.to_xspn_bytes(support_marginal=CONFIGS[cfg_id]["marginal"]))
    gen = {1: lambda n, seed: synth.config1_inputs(spn, n, seed), 2: synth.config2_inputs, 3: synth.config3_inputs,
           4: synth.config4_inputs, 5: synth.config5_inputs}[cfg_id]
    return path, gen


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz, mx, reasons = [], None, set()
        for ln in self.lines:
            p = [q.strip() for q in ln.split(",")]
            if len(p) < 6:
                continue
            try:
                mhz.append(float(p[0]))
                mx = float(p[1])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(mhz)) if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(mhz)}


def host_threads():
    """Hardware threads this process may run on.  Asked from the scheduler and handed to the oracle
    explicitly: under torchrun OMP_NUM_THREADS is 1, which would make the OpenMP default one thread."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


def cpu_baseline(query_path, gen, cfg, seconds=12.0):
    """Times the CPU restatement of the reference's batch-vectorised path (oracle, libmvec build) on all
    host threads for a bounded sample of the workload."""
    from oracle import oracle
    model = oracle.load_model(query_path)
    mode = "log_f32_cpu" if cfg["log_space"] else "linear_f64"
    threads = host_threads()
    n = 65536
    x = gen(n, 2999)
    oracle.evaluate(model, x[:4096], mode, vectorized=True, threads=threads)
    t0 = time.perf_counter()
    oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
    dt = time.perf_counter() - t0
    n2 = int(min(max(n * seconds / max(dt, 1e-6), n), 4_000_000))
    if n2 > n:
        x = gen(n2, 2999)
        t0 = time.perf_counter()
        oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
        dt = time.perf_counter() - t0
        n = n2
    return {"value": n / dt, "unit": "samples/s", "cores": threads, "kind": "port",
            "sample": "%d samples of the same workload, all %d host threads, AVX-512 libmvec, chunks of 4096" % (n, threads)}


def run_reference(args, rank):
    """--impl reference: the reference's CPU path (restated; the original needs LLVM 13/MLIR and cannot be
    built here) on the host cores.  Rank 0 alone does the work."""
    if rank != 0:
        return
    import tempfile
    from oracle import oracle
    cfg = CONFIGS[args.config]
    with tempfile.TemporaryDirectory() as wd:
        query, gen = build_workload(args.config, wd)
        model = oracle.load_model(query)
    mode = "log_f32_cpu" if cfg["log_space"] else "linear_f64"
    threads = host_threads()
    n = args.ref_samples
    x = gen(n, 2000 + args.config)
    for _ in range(args.warmup):
        oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
    dt = time.perf_counter() - t0
    val = n * args.steps / dt
    sample = "%d samples per step of the same workload, all %d host threads" % (n, threads)
    print(json.dumps({
        "impl": "reference", "metric": "SPN log-likelihood samples/sec", "value": val, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32" if cfg["log_space"] else "f64",
        "data": "synthetic", "config": {"workload": cfg["name"], "samples_per_step": n},
        "cpu_baseline": {"value": val, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS))
    ap.add_argument("--samples", type=int, default=0, help="samples per GPU per step (default: the config's batch)")
    ap.add_argument("--ref-samples", type=int, default=400_000)
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--opt", action="append", default=[], help="extra compile option key=value")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import tempfile
    import torch
    import torch.distributed as dist
    from spnb import capi  # fails loudly if libspnb.so is missing
    from spnb.shard import dataset_mean, max_over_ranks

    if capi.device_count() == 0:
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = CONFIGS[args.config]
    n = args.samples or cfg["n"]
    workdir = tempfile.mkdtemp(prefix="spnb_bench_")
    query, gen = build_workload(args.config, workdir)
    opts = {"target": "CUDA", "use-log-space": "true" if cfg["log_space"] else "false"}
    for kv in args.opt:
        k, v = kv.split("=", 1)
        opts[k] = v
    t0 = time.perf_counter()
    plan_path, info = capi.compile_query(query, opts, os.path.join(workdir, "bench_rank%d.plan" % rank))
    compile_s = time.perf_counter() - t0
    plan = capi.Plan(plan_path)
    plan.set_device(local_rank)
    stats = plan.stats

    # inputs: each rank owns a different shard of the synthetic batch, generated on the host and copied once
    host_x = gen(n, 2000 + args.config + 17 * rank)
    in_dtype = host_x.dtype
    dx = torch.from_numpy(host_x).cuda()
    out_dtype = torch.float32 if cfg["log_space"] else torch.float64
    dout = torch.empty(n, dtype=out_dtype, device="cuda")
    stream = torch.cuda.current_stream()

    def step():
        plan.execute_device(local_rank, n, dx.data_ptr(), dout.data_ptr(), stream.cuda_stream)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    torch.cuda.synchronize()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    ms_total = e0.elapsed_time(e1)
    # A short timed region ends before nvidia-smi (started with it, one line per 100 ms, 8 GPUs queried at
    # once under torchrun) has printed a line.  The same steps then keep running, untimed, until a few samples
    # of the clocks under this load exist; the JSON says which window the samples cover.
    window = "timed region"
    t_wait = time.perf_counter()
    while len(sampler.lines) < 3 and sampler.proc is not None and time.perf_counter() - t_wait < 3.0:
        step()
        torch.cuda.synchronize()
        window = "timed region and an untimed continuation of the same steps"
    clocks = sampler.stop()
    clocks["window"] = window
    if world > 1:
        dist.barrier()
        ms_total = max_over_ranks(ms_total)
    ms_step = ms_total / args.steps
    value = n * world / (ms_step * 1e-3)

    # optional dataset-mean log-likelihood: the only place a collective is used
    mean_ll = float(dout.double().sum().item())
    mean_ll = dataset_mean(mean_ll, n) if world > 1 else mean_ll / n

    # end to end through the host-pointer entry point, pinned host buffers, copies inside the timed region
    pin_x = torch.from_numpy(host_x).pin_memory()
    pin_out = torch.empty(n, dtype=out_dtype).pin_memory()
    plan.execute_host_ptr(n, pin_x.data_ptr(), pin_out.data_ptr())
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        plan.execute_host_ptr(n, pin_x.data_ptr(), pin_out.data_ptr())
    e2e_s = (time.perf_counter() - t0) / args.e2e_steps
    e2e_kernel_ms = plan.last_kernel_ms
    if world > 1:
        e2e_s = max_over_ranks(e2e_s)
    same = bool(torch.equal(pin_out.cuda(), dout))

    if rank == 0:
        peaks = {}
        pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
        hbm_peak, peak_src = 6650.0, "fallback"
        if os.path.exists(pk):
            peaks = json.load(open(pk))
            hbm_peak, peak_src = float(peaks.get("hbm_gbs", hbm_peak)), "measured"
        alg_bytes = stats["bytes_per_sample"] * n
        achieved = alg_bytes / (ms_step * 1e-3) / 1e9
        # dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture, per sample (traffic grows in
        # proportion to the samples of a launch): profiles/spnb_kernel_cfg2_gaussian26.md
        per_sample = MEASURED_DRAM_BYTES_PER_SAMPLE.get(args.config)
        traffic = per_sample * n if per_sample else None
        fp32 = capi.measure_peak("fp32")
        ex2 = capi.measure_peak("ex2")
        lg2 = capi.measure_peak("lg2")
        fp64 = capi.measure_peak("fp64")
        fp32x2 = capi.measure_peak("fp32x2")
        if cfg["log_space"]:
            sfu_rate = min(ex2, lg2)
            t_fp32 = stats["ops_fp32"] * n / fp32
            t_sfu = stats["ops_sfu"] * n / sfu_rate
            t_comp, bound = (t_fp32, "fp32") if t_fp32 >= t_sfu else (t_sfu, "sfu")
            ops, peak_ops = (stats["ops_fp32"], fp32) if bound == "fp32" else (stats["ops_sfu"], sfu_rate)
        else:
            t_comp, bound, ops, peak_ops = stats["ops_fp64"] * n / fp64, "fp64", stats["ops_fp64"], fp64
        launches = args.steps
        if stats["strategy"] == "layered":
            # Layered models are counted in their factorised formulation: per inner region (two operands of
            # `width` values, `width` sums) width*2 exponentials + width logarithms and one
            # [1 x width^2] x [width^2 x width] contraction (2 * width^3 flops); the leaf layer as a product of
            # [x^2, x] (2 F entries) with a 2 F x width parameter matrix per repetition.  The contraction and
            # the leaf layer run on the tensor cores, so the tensor term joins the maximum; its peak is the
            # measured dense 16-bit GEMM rate (sustained).
            m = cfg["layered"]
            inner = m["repetitions"] * (2 ** m["depth"] - 1)
            w = m["width"]
            flops_tc = inner * 2 * w ** 3 + m["repetitions"] * 2 * w * w + 2 * (2 * m["num_features"]) * w * m["repetitions"]
            sfu_ops = inner * 3 * w + m["repetitions"] * (2 * w + 1)
            tc_peak = float(peaks.get("bf16_tflops_sustained", 1400.0)) * 1e12
            t_tc = flops_tc * n / tc_peak
            t_sfu = sfu_ops * n / min(ex2, lg2)
            if t_tc >= t_sfu:
                t_comp, bound, ops, peak_ops = t_tc, "tensor", flops_tc, tc_peak
            else:
                t_comp, bound, ops, peak_ops = t_sfu, "sfu", sfu_ops, min(ex2, lg2)
            # per launch of the entry point: one transposition and one evaluation kernel per 512 Ki samples
            launches = args.steps * 2 * ((n + 524287) // 524288)
        t_hbm = alg_bytes / (hbm_peak * 1e9)
        t_roof = max(t_comp, t_hbm)
        line = {
            "metric": "SPN log-likelihood samples/sec", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32" if cfg["log_space"] else "f64", "data": "synthetic",
            "config": {"workload": cfg["name"], "samples_per_gpu": n, "input_dtype": str(in_dtype),
                       "nodes": stats["nodes"], "strategy": stats["strategy"], "l2": "inputs larger than L2 (%.0f MB per step)" % (host_x.nbytes / 1e6),
                       "parallelism": "batch sharded over %d GPU(s), model replicated, no data-path collective" % world,
                       "compile_s": round(compile_s, 2), "launch": list(plan.launch_config(local_rank)),
                       "registers": stats["registers"], "options": opts},
            "clocks": clocks,
            "e2e": {"value": n * world / e2e_s, "unit": "samples/s", "h2d_bytes_per_step": int(host_x.nbytes),
                    "d2h_bytes_per_step": int(n * (4 if cfg["log_space"] else 8)), "ms_per_step": e2e_s * 1e3,
                    "kernel_ms_inside": e2e_kernel_ms, "host_buffers": "pinned", "matches_device_path": same},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": traffic, "peak_source": peak_src,
                         "note": "algorithmic bytes = %d B/sample x %d samples per launch; this workload is compute-bound, see roofline_compute" % (stats["bytes_per_sample"], n)},
            "roofline_compute": {"bound": bound, "ops_per_sample": ops, "achieved": ops * n / (ms_step * 1e-3),
                                 "peak": peak_ops, "unit": "flop/s" if bound == "tensor" else "op/s", "frac": (ops * n / peak_ops) / (ms_step * 1e-3),
                                 "measured_rates": {"fp32_fma": fp32, "fp32_fma_packed_pairs": fp32x2, "ex2": ex2, "lg2": lg2, "fp64_fma": fp64},
                                 "per_config_roofline_frac": t_roof / (ms_step * 1e-3), "t_roof_ms": t_roof * 1e3},
            "mean_ll": mean_ll,
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(query, gen, cfg)
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
