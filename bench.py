#!/usr/bin/env python
"""Benchmark of the SPN joint log-likelihood hot path.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--config 2]

One "step" = one pass of the engine over one batch of synthetic samples resident in HBM.  The headline
workload is BASELINE.json's second configuration: a seeded random SPN over 26 Gaussian features (~2,000
nodes, depth 8), ONE batch of 10 M float32 samples, f32 log-space.  With N > 1 (launched under torchrun, one
rank per GPU) that one batch is cut into N contiguous shards, one per rank, the model replicated: strong
scaling, no collective on the data path.  The batch is made of eight seeded blocks, so it is the same batch
for every N.

Rank 0 prints ONE JSON line.  `value` is samples/s with inputs resident in HBM (CUDA-event timed on the
launching stream, max over ranks); `e2e` is the same metric through the host-pointer C-ABI call (host
buffers, H2D and D2H inside the timed region; pinned buffers for the headline figure, a pageable numpy
array -- what the Python entry point hands over -- beside it); `roofline` relates the kernel's algorithmic
bytes to the measured HBM peak and `roofline_compute` its algorithmic FP32 / SFU / tensor operations to rates
measured on the same device; `cpu_baseline` times the CPU restatement of the reference's vectorised path
on the host cores for a bounded sample.  At N = 1 the line also carries `per_config`: the other four
BASELINE configurations at their full batch sizes (fewer steps), each with its time, throughput, compute
roofline fraction, the error of a subset against the oracle and the clocks seen.  At N > 1 it carries
`strong_cfg5` (the 2 M-sample layered batch cut the same way) and `weak` (every rank on a full 10 M batch).

`--impl reference` times the CPU restatement alone on the same batch (the reference itself cannot be built
here).  `--config K` makes configuration K the headline and skips the `per_config` block.
"""
import argparse
import hashlib
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
PLAN_CACHE = os.path.join(ROOT, "spn-compiler_b200", "plan_cache")
BLOCKS = 8   # the global batch of a configuration is made of this many seeded blocks

CONFIGS = {
    1: dict(name="cfg1: 16 categorical features, ~400 nodes, int32 in, f64 linear", n=1_000_000, log_space=False,
            marginal=False, steps=20),
    2: dict(name="cfg2: 26 Gaussian features, ~2000 nodes, depth 8, f32 log-space", n=10_000_000, log_space=True,
            marginal=True, steps=20),
    3: dict(name="cfg3: 100 histogram features, ~8000 nodes, depth 10, 10% NaN, f32 log-space", n=4_000_000,
            log_space=True, marginal=True, steps=10),
    4: dict(name="cfg4: 256 mixed features, ~50000-node DAG, f32 log-space", n=4_000_000,
            log_space=True, marginal=True, steps=3),
    5: dict(name="cfg5: RAT-SPN-style layered SPN, 784 Gaussian features, 16 repetitions, 32x1024 dense sums, f32 log-space",
            n=2_000_000, log_space=True, marginal=True, steps=3,
            layered=dict(num_features=784, depth=4, repetitions=16, width=32)),   # synth.config5's defaults
}

# dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture, per sample (traffic grows in proportion to
# the samples of a launch)
L2_FLUSH_BYTES = 256 * 2**20   # twice the 126 MB L2

MEASURED_DRAM_BYTES_PER_SAMPLE = {1: 64.6, 2: 108.158, 3: 1234.5, 4: 24721.0, 5: 35818.0}


def make_model(cfg_id):
    from spnb import synth
    return getattr(synth, "config%d" % cfg_id)()


def input_block(cfg_id, spn, rows, block):
    """Rows of block `block` (0..BLOCKS-1) of the configuration's global batch."""
    from spnb import synth
    seed = 2000 + cfg_id + 100 * block
    if cfg_id == 1:
        return synth.config1_inputs(spn, rows, seed)
    return getattr(synth, "config%d_inputs" % cfg_id)(rows, seed)


def shard_inputs(cfg_id, spn, n_total, world, rank):
    """This rank's contiguous shard of the global batch of n_total samples: blocks [rank*B/world, (rank+1)*B/world)."""
    per = n_total // BLOCKS
    lo, hi = rank * BLOCKS // world, (rank + 1) * BLOCKS // world
    parts = [input_block(cfg_id, spn, per if b < BLOCKS - 1 else n_total - per * (BLOCKS - 1), b) for b in range(lo, hi)]
    return np.ascontiguousarray(np.concatenate(parts)) if len(parts) > 1 else parts[0]


def compile_opts(cfg_id, extra=()):
    opts = {"target": "CUDA", "use-log-space": "true" if CONFIGS[cfg_id]["log_space"] else "false"}
    for kv in extra:
        k, v = kv.split("=", 1)
        opts[k] = v
    return opts


def cached_plan(cfg_id, spn, opts, workdir, rank=0):
    """-> (query path, plan path, seconds spent compiling; 0 on a cache hit).  Plans are keyed by the query
    bytes, the options and the engine library, and kept beside the package (built artefacts, not sources):
    __graft_entry__.build() fills the cache, so that a 50 k-node model's JIT is not paid inside a bench run."""
    from spnb import capi
    data = spn.to_xspn_bytes(support_marginal=CONFIGS[cfg_id]["marginal"])
    query = os.path.join(workdir, "bench_cfg%d.bin" % cfg_id)
    with open(query, "wb") as f:
        f.write(data)
    h = hashlib.sha256()
    h.update(data)
    h.update(json.dumps(opts, sort_keys=True).encode())
    with open(capi.LIB_PATH, "rb") as f:     # a plan holds code generated by this very library
        h.update(hashlib.sha256(f.read()).digest())
    cached = os.path.join(PLAN_CACHE, "cfg%d_%s.plan" % (cfg_id, h.hexdigest()[:20]))
    if os.path.exists(cached):
        return query, cached, 0.0
    t0 = time.perf_counter()
    target = os.path.join(workdir, "bench_cfg%d_rank%d.plan" % (cfg_id, rank))
    plan_path, _ = capi.compile_query(query, opts, target)
    dt = time.perf_counter() - t0
    try:
        os.makedirs(PLAN_CACHE, exist_ok=True)
        tmp = cached + ".tmp%d" % os.getpid()
        with open(plan_path, "rb") as src, open(tmp, "wb") as dst:
            dst.write(src.read())
        os.replace(tmp, cached)
    except OSError:
        pass
    return query, plan_path, dt


def warm_plan_cache(configs=(1, 2, 3, 4, 5), prune=True):
    """Compile the bench plans into the cache (needs no GPU) and drop plans made by an earlier build of the
    library.  Called by __graft_entry__.build()."""
    import tempfile
    keep = set()
    with tempfile.TemporaryDirectory() as wd:
        for c in configs:
            _, path, dt = cached_plan(c, make_model(c), compile_opts(c), wd)
            if os.path.dirname(path) != PLAN_CACHE:      # compiled just now: the cache holds a copy
                path = [os.path.join(PLAN_CACHE, f) for f in os.listdir(PLAN_CACHE) if f.startswith("cfg%d_" % c)]
                path = max(path, key=os.path.getmtime)
            keep.add(os.path.basename(path))
            print("plan cache: cfg%d %s (%.1f s)" % (c, os.path.basename(path), dt), flush=True)
    if prune and os.path.isdir(PLAN_CACHE):
        for f in os.listdir(PLAN_CACHE):
            if f not in keep:
                os.remove(os.path.join(PLAN_CACHE, f))


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


CPU_PORT_NOTE = ("CPU restatement of the reference's batch-vectorised path: a block interpreter over chunks of 4096 "
                 "samples (not model-specialised compiled code), AVX-512 libmvec, discrete leaves gathered from "
                 "pre-computed log tables")


def cpu_baseline(query_path, cfg_id, spn, seconds=12.0):
    """Times the CPU restatement of the reference's batch-vectorised path (oracle, libmvec build) on all
    host threads for a bounded sample of the workload."""
    from oracle import oracle
    cfg = CONFIGS[cfg_id]
    model = oracle.load_model(query_path)
    mode = "log_f32_cpu" if cfg["log_space"] else "linear_f64"
    threads = host_threads()
    n = 65536
    x = input_block(cfg_id, spn, n, 0)
    oracle.evaluate(model, x[:4096], mode, vectorized=True, threads=threads)
    t0 = time.perf_counter()
    oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
    dt = time.perf_counter() - t0
    n2 = int(min(max(n * seconds / max(dt, 1e-6), n), 4_000_000))
    if n2 > n:
        x = input_block(cfg_id, spn, n2, 0)
        t0 = time.perf_counter()
        oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
        dt = time.perf_counter() - t0
        n = n2
    return {"value": n / dt, "unit": "samples/s", "cores": threads, "kind": "port",
            "sample": "%d samples of the same workload, all %d host threads; %s" % (n, threads, CPU_PORT_NOTE)}


def run_reference(args, rank):
    """--impl reference: the reference's CPU path (restated; the original needs LLVM 13/MLIR and cannot be
    built here) on the host cores, on the same batch as the engine's arm.  Rank 0 alone does the work."""
    if rank != 0:
        return
    import tempfile
    from oracle import oracle
    cfg = CONFIGS[args.config]
    spn = make_model(args.config)
    with tempfile.TemporaryDirectory() as wd:
        query = os.path.join(wd, "ref.bin")
        with open(query, "wb") as f:
            f.write(spn.to_xspn_bytes(support_marginal=cfg["marginal"]))
        model = oracle.load_model(query)
    mode = "log_f32_cpu" if cfg["log_space"] else "linear_f64"
    threads = host_threads()
    n_total = args.samples or cfg["n"]
    # one step = the same batch as the engine's step when the CPU gets through it in about a second; otherwise a
    # bounded leading part of that batch, sized from a probe, so that the whole run ends within minutes
    probe = shard_inputs(args.config, spn, n_total, BLOCKS, 0)[:65536]
    oracle.evaluate(model, probe[:4096], mode, vectorized=True, threads=threads)
    t0 = time.perf_counter()
    oracle.evaluate(model, probe, mode, vectorized=True, threads=threads)
    rate = len(probe) / max(time.perf_counter() - t0, 1e-6)
    budget_s = 150.0 / max(args.steps + args.warmup, 1)
    n = n_total if args.ref_samples == 0 else min(args.ref_samples, n_total)
    if args.ref_samples == 0 and n_total / rate > budget_s:
        n = max(65536, int(rate * budget_s) // 4096 * 4096)
    x = shard_inputs(args.config, spn, n_total, 1, 0)[:n] if n > len(probe) else probe[:n]
    for _ in range(args.warmup):
        oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.evaluate(model, x, mode, vectorized=True, threads=threads)
    dt = time.perf_counter() - t0
    val = n * args.steps / dt
    whole = n == n_total
    sample = ("%s of the engine's batch (%d of %d samples) per step, all %d host threads; %s"
              % ("all" if whole else "a leading part", n, n_total, threads, CPU_PORT_NOTE))
    emit_result(({
        "impl": "reference", "metric": "SPN log-likelihood samples/sec", "value": val, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32" if cfg["log_space"] else "f64",
        "data": "synthetic", "config": {"workload": cfg["name"], "samples_total": n_total, "samples_per_step": n,
                                        "same_batch_as_engine_arm": whole},
        "cpu_baseline": {"value": val, "unit": "samples/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def compute_roofline(cfg, stats, n, ms_step, rates, peaks):
    """Algorithmic operations of one launch against the issue / tensor rates measured on this device."""
    fp32, ex2, lg2, fp64 = rates["fp32_fma"], rates["ex2"], rates["lg2"], rates["fp64_fma"]
    if stats["strategy"] == "layered" and "layered" in cfg:
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
        t_tc, t_sfu = flops_tc * n / tc_peak, sfu_ops * n / min(ex2, lg2)
        if t_tc >= t_sfu:
            t_comp, bound, ops, peak_ops = t_tc, "tensor", flops_tc, tc_peak
        else:
            t_comp, bound, ops, peak_ops = t_sfu, "sfu", sfu_ops, min(ex2, lg2)
    elif cfg["log_space"]:
        sfu_rate = min(ex2, lg2)
        t_fp32 = stats["ops_fp32"] * n / fp32
        t_sfu = stats["ops_sfu"] * n / sfu_rate
        t_comp, bound = (t_fp32, "fp32") if t_fp32 >= t_sfu else (t_sfu, "sfu")
        ops, peak_ops = (stats["ops_fp32"], fp32) if bound == "fp32" else (stats["ops_sfu"], sfu_rate)
    else:
        t_comp, bound, ops, peak_ops = stats["ops_fp64"] * n / fp64, "fp64", stats["ops_fp64"], fp64
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    t_hbm = stats["bytes_per_sample"] * n / (hbm_peak * 1e9)
    t_roof = max(t_comp, t_hbm)
    return {"bound": bound, "ops_per_sample": ops, "achieved": ops * n / (ms_step * 1e-3), "peak": peak_ops,
            "unit": "flop/s" if bound == "tensor" else "op/s", "frac": (ops * n / peak_ops) / (ms_step * 1e-3),
            "per_config_roofline_frac": t_roof / (ms_step * 1e-3), "t_roof_ms": t_roof * 1e3}


class Workload:
    """One configuration set up on this rank's GPU: model, plan, resident shard."""

    def __init__(self, cfg_id, n_total, world, rank, local_rank, workdir, extra_opts=(), whole_batch=False):
        import torch
        from spnb import capi
        self.cfg_id, self.cfg = cfg_id, CONFIGS[cfg_id]
        self.local_rank = local_rank
        self.spn = make_model(cfg_id)
        self.opts = compile_opts(cfg_id, extra_opts)
        self.query, plan_path, self.compile_s = cached_plan(cfg_id, self.spn, self.opts, workdir, rank)
        self.plan = capi.Plan(plan_path)
        self.plan.set_device(local_rank)
        self.stats = self.plan.stats
        self.host_x = shard_inputs(cfg_id, self.spn, n_total, 1, 0) if whole_batch else \
            shard_inputs(cfg_id, self.spn, n_total, world, rank)
        self.n = self.host_x.shape[0]
        self.dx = torch.from_numpy(self.host_x).cuda()
        self.out_dtype = torch.float32 if self.cfg["log_space"] else torch.float64
        self.dout = torch.empty(self.n, dtype=self.out_dtype, device="cuda")
        self.stream = torch.cuda.current_stream()
        moved = self.host_x.nbytes + self.dout.numel() * self.dout.element_size()
        self.flush = torch.zeros(L2_FLUSH_BYTES // 4, dtype=torch.int32, device="cuda") if moved < L2_FLUSH_BYTES else None

    def l2_note(self):
        mb = self.host_x.nbytes / 1e6
        if self.flush is None:
            return "inputs larger than L2 (%.0f MB per GPU per step)" % mb
        return "%.0f MB of inputs per GPU per step: a %d MB buffer is rewritten before every timed step (L2 flush), steps timed one by one" % (mb, L2_FLUSH_BYTES // 2**20)

    def step(self):
        self.plan.execute_device(self.local_rank, self.n, self.dx.data_ptr(), self.dout.data_ptr(), self.stream.cuda_stream)

    def timed(self, steps, warmup, world, sample_clocks=True):
        """-> (ms per step: CUDA events on the launching stream, max over ranks; clocks record)"""
        import torch
        import torch.distributed as dist
        from spnb.shard import max_over_ranks
        for _ in range(warmup):
            self.step()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        sampler = ClockSampler(self.local_rank)
        if sample_clocks:
            sampler.start()
        torch.cuda.synchronize()
        if self.flush is None:
            e0 = torch.cuda.Event(enable_timing=True)
            e1 = torch.cuda.Event(enable_timing=True)
            e0.record(self.stream)
            for _ in range(steps):
                self.step()
            e1.record(self.stream)
            torch.cuda.synchronize()
            ms_total = e0.elapsed_time(e1)
        else:
            # shard smaller than twice the L2: a buffer larger than L2 is rewritten before every timed step,
            # each step has its own pair of events and the flushes stay outside the sum
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            for a, b in pairs:
                self.flush.add_(1)
                a.record(self.stream)
                self.step()
                b.record(self.stream)
            torch.cuda.synchronize()
            ms_total = sum(a.elapsed_time(b) for a, b in pairs)
        # a bounded wait that gave up would end the kernels early and publish a fast number: ask the engine
        self.plan.device_status(self.local_rank)
        clocks = None
        if sample_clocks:
            # A short timed region ends before nvidia-smi (one line per 100 ms) has printed a line.  The same
            # steps then keep running, untimed, until a few samples of the clocks under this load exist; the
            # record says which window the samples cover.
            window = "timed region"
            t_wait = time.perf_counter()
            while len(sampler.lines) < 3 and sampler.proc is not None and time.perf_counter() - t_wait < 3.0:
                self.step()
                torch.cuda.synchronize()
                window = "timed region and an untimed continuation of the same steps"
            clocks = sampler.stop()
            clocks["window"] = window
        if world > 1:
            dist.barrier()
            ms_total = max_over_ranks(ms_total)
        return ms_total / steps, clocks

    def subset_error(self, count, chunk=256):
        """Largest relative error (in log space, |ll| floored at 1) of `count` evenly spaced samples of the
        resident result against the f64 oracle."""
        from oracle import oracle
        idx = np.linspace(0, self.n - 1, num=min(count, self.n)).astype(np.int64)
        got = self.dout[idx.tolist()].double().cpu().numpy()
        want = oracle.evaluate(oracle.load_model(self.query), np.ascontiguousarray(self.host_x[idx]),
                               "log_f64" if self.cfg["log_space"] else "linear_f64", threads=host_threads(), chunk=chunk)
        fin = np.isfinite(want)
        if not np.array_equal(np.isfinite(got), fin):
            return float("inf")
        return float(np.max(np.abs(got[fin] - want[fin]) / np.maximum(np.abs(want[fin]), 1.0))) if fin.any() else 0.0

    def launches_per_step(self):
        if self.stats["strategy"] == "layered" or self.stats.get("scoped_staging"):
            # per call of the entry point: one transposition and one evaluation kernel per 512 Ki samples
            return 2 * ((self.n + 524287) // 524288)
        return 1

    def close(self):
        self.plan.close()
        self.dx = self.dout = self.flush = None


def e2e_host(w, steps, world, pinned):
    """Same metric through the host-pointer entry point: inputs in host memory, copies inside the timed region."""
    import torch
    import torch.distributed as dist
    from spnb.shard import max_over_ranks
    if pinned:
        hx = torch.from_numpy(w.host_x).pin_memory()
        hout = torch.empty(w.n, dtype=w.out_dtype).pin_memory()
        call = lambda: w.plan.execute_host_ptr(w.n, hx.data_ptr(), hout.data_ptr())
        result = lambda: hout
    else:
        box = {}
        def call():
            box["out"] = w.plan.execute_host(w.host_x)   # pageable numpy in, fresh numpy out: what CUDACompiler.execute does
        result = lambda: torch.from_numpy(box["out"])
    call()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        call()
    dt = (time.perf_counter() - t0) / steps
    # sum of the per-chunk event intervals of the last call: chunks on rotating streams queue behind one another
    # for the SMs, so the sum can exceed the step's wall time
    kernel_ms = w.plan.last_kernel_ms
    if world > 1:
        dt = max_over_ranks(dt)
    same = bool(torch.equal(result().cuda(), w.dout))
    return dt, kernel_ms, same


_RESULT_OUT = None


def claim_stdout():
    """The process's stdout carries the one JSON line and nothing else: whatever libraries print on file
    descriptor 1 (NCCL's version banner, for one) is sent to stderr, the line goes out through a copy of the
    original descriptor."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit_result(line):
    claim_stdout()
    _RESULT_OUT.write(json.dumps(line) + "\n")
    _RESULT_OUT.flush()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=0, choices=[0] + sorted(CONFIGS),
                    help="headline configuration (default 2, with the other four in per_config)")
    ap.add_argument("--samples", type=int, default=0, help="samples of the whole batch per step (default: the config's batch)")
    ap.add_argument("--ref-samples", type=int, default=0,
                    help="--impl reference: samples per step (default: the engine's batch, bounded by a time budget)")
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-per-config", action="store_true")
    ap.add_argument("--warm-plan-cache", action="store_true", help="compile the bench plans into the cache and exit")
    ap.add_argument("--opt", action="append", default=[], help="extra compile option key=value")
    args = ap.parse_args()
    if args.warm_plan_cache:
        warm_plan_cache()
        return
    claim_stdout()
    per_config_wanted = args.config == 0 and not args.no_per_config and not args.samples and not args.opt
    args.config = args.config or 2
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
    from spnb.shard import dataset_mean

    if capi.device_count() == 0:
        raise SystemExit("bench.py needs a CUDA device: the engine has no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    cfg = CONFIGS[args.config]
    n_total = args.samples or cfg["n"]
    workdir = tempfile.mkdtemp(prefix="spnb_bench_")

    # ---- headline: one batch of n_total samples cut into `world` shards --------------------------------------
    w = Workload(args.config, n_total, world, rank, local_rank, workdir, args.opt)
    ms_step, clocks = w.timed(args.steps, args.warmup, world)
    value = n_total / (ms_step * 1e-3)
    local_sum = float(w.dout.double().sum().item())
    mean_ll = dataset_mean(local_sum, w.n) if world > 1 else local_sum / w.n   # the only collective: optional mean
    e2e_s, e2e_kernel_ms, same = e2e_host(w, args.e2e_steps, world, pinned=True)
    e2e_pg_s, _, same_pg = e2e_host(w, max(1, min(args.e2e_steps, 2)), world, pinned=False)

    peaks = {}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    hbm_peak, peak_src = 6650.0, "fallback"
    if os.path.exists(pk):
        peaks = json.load(open(pk))
        hbm_peak, peak_src = float(peaks.get("hbm_gbs", hbm_peak)), "measured"
    rates = None
    if rank == 0:
        rates = {"fp32_fma": capi.measure_peak("fp32"), "fp32_fma_packed_pairs": capi.measure_peak("fp32x2"),
                 "ex2": capi.measure_peak("ex2"), "lg2": capi.measure_peak("lg2"), "fp64_fma": capi.measure_peak("fp64")}

    line = None
    if rank == 0:
        stats = w.stats
        alg_bytes = stats["bytes_per_sample"] * w.n          # of this rank's launch
        achieved = alg_bytes / (ms_step * 1e-3) / 1e9
        per_sample = MEASURED_DRAM_BYTES_PER_SAMPLE.get(args.config)
        rc = compute_roofline(cfg, stats, w.n, ms_step, rates, peaks)
        rc["measured_rates"] = rates
        out_bytes = 4 if cfg["log_space"] else 8
        line = {
            "metric": "SPN log-likelihood samples/sec", "value": value, "unit": "samples/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32" if cfg["log_space"] else "f64", "data": "synthetic",
            "config": {"workload": cfg["name"], "samples_total": n_total, "samples_per_gpu": w.n,
                       "input_dtype": str(w.host_x.dtype), "nodes": stats["nodes"], "strategy": stats["strategy"],
                       "l2": w.l2_note(),
                       "parallelism": "one batch cut into %d contiguous shard(s), one per GPU, model replicated, no data-path collective" % world,
                       "compile_s": round(w.compile_s, 2), "launch": list(w.plan.launch_config(local_rank)),
                       "registers": stats["registers"], "options": w.opts},
            "clocks": clocks,
            "e2e": {"value": n_total / e2e_s, "unit": "samples/s", "h2d_bytes_per_step": int(w.host_x.nbytes) * world,
                    "d2h_bytes_per_step": int(n_total * out_bytes), "ms_per_step": e2e_s * 1e3,
                    "chunk_kernel_intervals_ms": e2e_kernel_ms, "host_buffers": "pinned", "matches_device_path": same,
                    "pageable": {"value": n_total / e2e_pg_s, "ms_per_step": e2e_pg_s * 1e3,
                                 "host_buffers": "pageable numpy array in, new numpy array out (what CUDACompiler.execute passes)",
                                 "matches_device_path": same_pg}},
            "gpu_launches": args.steps * w.launches_per_step(),
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": per_sample * w.n if per_sample else None, "peak_source": peak_src,
                         "note": "algorithmic bytes = %d B/sample x %d samples per launch; this workload is compute-bound, see roofline_compute" % (stats["bytes_per_sample"], w.n)},
            "roofline_compute": rc,
            "mean_ll": mean_ll,
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(w.query, args.config, w.spn)
    w.close()
    torch.cuda.empty_cache()

    # ---- N = 1: the other configurations at their full batch ---------------------------------------------
    if world == 1 and per_config_wanted:
        per = {}
        for c in (1, 3, 4, 5):
            t0 = time.perf_counter()
            try:
                wc = Workload(c, CONFIGS[c]["n"], 1, 0, local_rank, workdir)
                steps = CONFIGS[c]["steps"]
                ms_c, clk = wc.timed(steps, 3, 1)
                rc = compute_roofline(CONFIGS[c], wc.stats, wc.n, ms_c, rates, peaks)
                per["cfg%d" % c] = {
                    "workload": CONFIGS[c]["name"], "samples": wc.n, "steps": steps, "warmup": 3, "ms_per_step": ms_c,
                    "value": wc.n / (ms_c * 1e-3), "unit": "samples/s", "strategy": wc.stats["strategy"],
                    "launch": list(wc.plan.launch_config(local_rank)), "l2": wc.l2_note(),
                    "gpu_launches": steps * wc.launches_per_step(),
                    "roofline_compute": {k: rc[k] for k in ("bound", "frac", "ops_per_sample", "per_config_roofline_frac", "t_roof_ms")},
                    "max_rel_err_vs_oracle": wc.subset_error(128 if c == 5 else 2000, chunk=16 if c == 5 else 256),
                    "tolerance": 1e-5 if CONFIGS[c]["log_space"] else 1e-12,
                    "clocks": clk, "compile_s": round(wc.compile_s, 2), "wall_s": None}
                wc.close()
            except Exception as e:   # one configuration failing must not cost the headline line
                per["cfg%d" % c] = {"error": "%s: %s" % (type(e).__name__, e)}
            per["cfg%d" % c]["wall_s"] = round(time.perf_counter() - t0, 1)
            torch.cuda.empty_cache()
        line["per_config"] = per

    # ---- N > 1: the layered batch cut the same way, and the weak figure ------------------------------------
    if world > 1 and per_config_wanted:
        w5 = Workload(5, CONFIGS[5]["n"], world, rank, local_rank, workdir)
        ms5, clk5 = w5.timed(CONFIGS[5]["steps"], 3, world)
        if rank == 0:
            line["strong_cfg5"] = {"workload": CONFIGS[5]["name"], "samples_total": CONFIGS[5]["n"], "samples_per_gpu": w5.n,
                                   "steps": CONFIGS[5]["steps"], "ms_per_step": ms5, "value": CONFIGS[5]["n"] / (ms5 * 1e-3),
                                   "unit": "samples/s", "scaling": "strong", "clocks": clk5}
        w5.close()
        torch.cuda.empty_cache()
        ww = Workload(args.config, n_total, world, rank, local_rank, workdir, args.opt, whole_batch=True)
        msw, _ = ww.timed(args.steps, 3, world, sample_clocks=False)
        if rank == 0:
            line["weak"] = {"samples_per_gpu": ww.n, "ms_per_step": msw, "value": ww.n * world / (msw * 1e-3),
                            "unit": "samples/s", "scaling": "weak"}
        ww.close()

    if rank == 0:
        emit_result(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
