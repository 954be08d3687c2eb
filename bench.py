"""Benchmark of the QR hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A step is LAUNCHES_PER_STEP passes of the hot path over one batch: reduced QR of
BATCH float32 32 x 32 N(0,1) matrices per GPU (the shape the headline metric is
quoted on, at a batch that saturates the GPU and is larger than L2: 1 GiB in, 2 GiB
out per GPU), launched back to back so that the timed region lasts over a second
and the clock samples fall inside it. The batch axis is sharded over the GPUs with
no collective; per-GPU work is fixed as N grows (weak scaling). Rank 0 prints one
JSON line.

  value      matrices/s with the inputs resident in HBM: K launches of the C-ABI
             call on device pointers, timed with CUDA events, max over ranks
  e2e        the same through the C-ABI call on HOST (pinned) buffers: the
             host-to-device copy of the inputs and the device-to-host copy of Q
             and R are inside the timed region
  roofline   the small-matrix kernel against the measured HBM copy bandwidth
  cpu_baseline  the reference's own CPU path (src/qr_cpu.mm compiled into
             oracle/_ref; all host cores) on a bounded sample of the same workload
  peaks      (1 GPU only) the FP32 FMA pipe and the dense TF32 tensor pipe measured by microbenchmarks
             (metal-linalg_b200/bench/peaks.cu) in this run, with the SM clock sampled beside them
  roofline_4096  (1 GPU only) the metric's second half: one 4096 x 4096 QR against those measured peaks
  mode_r     (1 GPU only) R alone against reduced, per kernel family
  others     (1 GPU only) the remaining benchmark configurations, each timed the same way
  weak_scaled  (several GPUs) configurations 2, 3, 4 and 5b, one shard per GPU, timed as the headline is
  svd        (1 GPU only) the SVD that calls the QR, on tall and small batches

--impl reference times the reference's CPU path alone, on the host cores.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path[:0] = [os.path.join(ROOT, "metal-linalg_b200")]

METRIC = "fp32 QR matrices/s (32x32 batch)"
UNIT = "matrices/s"
ROWS = COLS = 32
BATCH = 262144                       # per GPU
LAUNCHES_PER_STEP = 50               # passes over the batch in one step
BYTES_PER_MATRIX = 3 * ROWS * COLS * 4   # A read, Q and R written
# DRAM bytes per matrix of the small kernel, from one ncu capture of one launch on 65 536 matrices:
# (dram__bytes_read.sum + dram__bytes_write.sum) / 65 536. Traffic grows in proportion to the batch.
MEASURED_TRAFFIC_PER_MATRIX = 11785
TRAFFIC_SOURCE = "ncu, one launch on 65 536 matrices, scaled by the batch"
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except OSError:
        return {"hbm_gbs": FALLBACK_HBM_GBS}, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.lines, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
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
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


_cpu_inputs = {}


def cpu_reference(sample_batch, reps):
    """The reference's CPU QR on `sample_batch` 32 x 32 matrices: (matrices/s, cores, kind, best seconds)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import numpy as np

    import harness
    if sample_batch not in _cpu_inputs:       # drawn once per size: the draw takes longer than the factorisation
        _cpu_inputs.clear()
        out = np.empty((sample_batch, ROWS, COLS), np.float32)
        parts = max(1, min(os.cpu_count() or 1, sample_batch // 1024))      # seeded per part, drawn on all cores
        seeds = np.random.SeedSequence(0).spawn(parts)
        edges = [sample_batch * i // parts for i in range(parts + 1)]

        def draw(i):
            np.random.default_rng(seeds[i]).standard_normal(out=out[edges[i]:edges[i + 1]], dtype=np.float32)
        workers = [threading.Thread(target=draw, args=(i,)) for i in range(parts)]
        for w in workers:
            w.start()
        for w in workers:
            w.join()
        _cpu_inputs[sample_batch] = out
    a = _cpu_inputs[sample_batch]
    if harness.load_ref() is not None:
        run, kind, cores = (lambda: harness.ref_qr(a)), "reference", int(harness.load_ref().ref_cpu_threads())
    else:
        run, kind, cores = (lambda: harness.oracle_qr(a)), "port", os.cpu_count() or 1
    best = float("inf")
    for _ in range(reps):
        t0 = time.perf_counter()
        run()
        best = min(best, time.perf_counter() - t0)
    return sample_batch / best, cores, kind, best


def run_reference(args, rank):
    if rank != 0:
        return
    t_all = time.perf_counter()
    # one step = the whole batch of the GPU arm's workload, once (under a second on 16 cores)
    _, cores, kind, _ = cpu_reference(4096, 1)
    sample = BATCH
    for _ in range(args.warmup):
        cpu_reference(sample, 1)
    times = []
    for _ in range(args.steps):
        _, _, _, t = cpu_reference(sample, 1)
        times.append(t)
    value = sample * len(times) / sum(times)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"reduced QR of {BATCH} float32 {ROWS}x{COLS} N(0,1) matrices per GPU (the first "
                               f"benchmark configuration's shape at a batch that saturates the GPU)",
                   "batch_per_gpu": BATCH, "rows": ROWS, "cols": COLS, "mode": "reduced", "passes_per_step": 1,
                   "cpu_arm": f"the reference's CPU path on all {cores} host cores, the whole batch of "
                              f"{sample} matrices once per step"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": f"the whole batch, {sample} matrices, once per step, {args.steps} steps"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "wall_s": time.perf_counter() - t_all,
    }
    print(json.dumps(line), flush=True)


def time_config(torch, mlt, _lib, a, mode, steps, warmup, flush):
    """Seconds per launch of the C-ABI call on device tensor `a`, CUDA events on the launching stream."""
    b, m, n = a.shape
    k = min(m, n)
    qc = {"reduced": k, "complete": m, "r": 0}[mode]
    rr = m if mode == "complete" else k
    q = torch.empty(b, m, qc, device=a.device) if qc else None
    r = torch.empty(b, rr, n, device=a.device)
    stream = torch.cuda.current_stream().cuda_stream

    def call():
        _lib.qr(a.data_ptr(), b, m, n, q.data_ptr() if qc else None, r.data_ptr(), mode, stream)

    for _ in range(warmup):
        call()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(steps):
        if flush is not None:
            flush.add_(1.0)            # rewrites a buffer larger than L2 between iterations
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        call()
        e1.record()
        e1.synchronize()
        total += e0.elapsed_time(e1) * 1e-3
    return total / steps, (q, r)


def load_peaks_library():
    import ctypes
    path = os.path.join(ROOT, "metal-linalg_b200", "lib", "libmlb_peaks.so")
    lib = ctypes.CDLL(path)
    d, i = ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_int)
    lib.mlb_peak_ffma.restype = ctypes.c_int
    lib.mlb_peak_ffma.argtypes = [ctypes.c_double, ctypes.c_int, d, d, i]
    lib.mlb_peak_tf32.restype = ctypes.c_int
    lib.mlb_peak_tf32.argtypes = [ctypes.c_double, d, d, i]
    return lib


def measure_compute_peaks(local_rank, seconds=2.0):
    """The FP32 FMA pipe and the dense TF32 tensor pipe of this GPU, each a loop of `seconds` with the SM
    clock sampled meanwhile: TFLOP/s sustained over the loop and of the best launch."""
    import ctypes
    out = {"how": "metal-linalg_b200/bench/peaks.cu: register-resident FMA chains (2 x 1024 threads a multiprocessor); "
                  "tcgen05.mma kind::tf32 128x256x8 from shared memory, one block a multiprocessor",
           "seconds_each": seconds}
    try:
        lib = load_peaks_library()
    except OSError as e:
        out["error"] = f"libmlb_peaks.so: {e}"
        return out
    for name, call in (("ffma", lambda *r: lib.mlb_peak_ffma(seconds, 0, *r)),
                       ("ffma_packed", lambda *r: lib.mlb_peak_ffma(seconds, 1, *r)),
                       ("tf32_dense", lambda *r: lib.mlb_peak_tf32(seconds, *r))):
        sustained, burst, launches = ctypes.c_double(0), ctypes.c_double(0), ctypes.c_int(0)
        sampler = ClockSampler(local_rank)
        sampler.start()
        rc = call(ctypes.byref(sustained), ctypes.byref(burst), ctypes.byref(launches))
        clocks = sampler.stop()
        out[name] = {"tflops_sustained": sustained.value, "tflops_burst": burst.value, "launches": launches.value,
                     "status": rc, "sm_mhz": clocks.get("sm_mhz"), "reasons": clocks.get("reasons")}
    return out


def copy_bound(torch, ha, hq, hr, a, q, r, reps):
    """Seconds per step of nothing but the step's copies: the pinned input to the device on one stream while Q
    and R go back to pinned memory on another (what a perfectly overlapped staging pipeline is left with)."""
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps + 1):
        t0 = time.perf_counter()
        with torch.cuda.stream(s_in):
            a.copy_(ha, non_blocking=True)
        with torch.cuda.stream(s_out):
            hq.copy_(q, non_blocking=True)
            hr.copy_(r, non_blocking=True)
        s_in.synchronize()
        s_out.synchronize()
        best = min(best, time.perf_counter() - t0)
    return best


def run_ours(args, rank, world, local_rank):
    import torch

    import metal_linalg_torch as mlt
    from metal_linalg_torch import _lib, workloads

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a GPU: this library has no CPU path")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"      # keeps NCCL's version banner off stdout: rank 0 prints one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    t_all = time.perf_counter()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(seconds):
        t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.item()

    g = torch.Generator(device="cuda").manual_seed(1000 + rank)
    a = torch.randn(BATCH, ROWS, COLS, generator=g, device="cuda", dtype=torch.float32)
    q = torch.empty(BATCH, ROWS, COLS, device="cuda")
    r = torch.empty(BATCH, ROWS, COLS, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream

    def step():
        for _ in range(LAUNCHES_PER_STEP):
            _lib.qr(a.data_ptr(), BATCH, ROWS, COLS, q.data_ptr(), r.data_ptr(), "reduced", stream)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.12)       # the first sample is taken before the region starts
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    seconds = e0.elapsed_time(e1) * 1e-3
    clocks = sampler.stop() if rank == 0 else None
    seconds = max_over_ranks(seconds)
    _lib.synchronize()         # and no kernel gave up on a wait

    # correctness of what was timed: a sample against float64 products on the GPU
    sl = slice(0, 4096)
    a64, q64, r64 = a[sl].double(), q[sl].double(), r[sl].double()
    recon = (torch.linalg.matrix_norm(a64 - q64 @ r64) / torch.linalg.matrix_norm(a64)).max().item()
    orth = torch.linalg.matrix_norm(q64.mT @ q64 - torch.eye(COLS, device="cuda", dtype=torch.float64)).max().item()
    del a64, q64, r64

    # end to end: host (pinned) buffers through the C-ABI call, copies inside the timed region
    e2e_steps = max(1, min(args.steps, 3))
    ha = torch.empty(BATCH, ROWS, COLS, dtype=torch.float32).pin_memory()
    ha.copy_(a)
    hq = torch.empty(BATCH, ROWS, COLS, dtype=torch.float32).pin_memory()
    hr = torch.empty(BATCH, ROWS, COLS, dtype=torch.float32).pin_memory()
    _lib.lib.metal_linalg_set_device(local_rank)

    def host_step():
        _lib.qr(ha.data_ptr(), BATCH, ROWS, COLS, hq.data_ptr(), hr.data_ptr(), "reduced")

    host_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        host_step()
    e2e_seconds = max_over_ranks(time.perf_counter() - t0)
    e2e_ok = bool(torch.equal(hq[:64], q[:64].cpu()) and torch.equal(hr[:64], r[:64].cpu()))
    # the same bytes with no kernel in between, every rank at once: what the machine's copy engines and host memory allow
    barrier()
    copy_seconds = max_over_ranks(copy_bound(torch, ha, hq, hr, a, q, r, e2e_steps))
    del ha, hq, hr

    scaled = weak_scaled_configs(torch, mlt, _lib, args, rank, world, barrier, max_over_ranks) if world > 1 else None

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    launches = args.steps * LAUNCHES_PER_STEP
    per_launch = seconds / launches
    achieved = BATCH * BYTES_PER_MATRIX / per_launch / 1e9
    line = {
        "metric": METRIC, "value": world * BATCH * launches / seconds, "unit": UNIT, "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * seconds / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"reduced QR of {BATCH} float32 {ROWS}x{COLS} N(0,1) matrices per GPU (the first "
                               f"benchmark configuration's shape at a batch that saturates the GPU)",
                   "batch_per_gpu": BATCH, "rows": ROWS, "cols": COLS, "mode": "reduced",
                   "passes_per_step": LAUNCHES_PER_STEP,
                   "sharding": f"batch axis over {world} GPU(s), no collective",
                   "l2": "inputs and outputs (3 GiB per GPU) are larger than L2; no flush needed",
                   "kernel": mlt.qr_kernel(ROWS, COLS, BATCH)},
        "ms_per_launch": 1e3 * per_launch,
        "e2e": {"value": world * BATCH * e2e_steps / e2e_seconds, "unit": UNIT,
                "h2d_bytes_per_step": BATCH * ROWS * COLS * 4, "d2h_bytes_per_step": 2 * BATCH * ROWS * COLS * 4,
                "steps": e2e_steps, "ms_per_step": 1e3 * e2e_seconds / e2e_steps,
                "copy_bound_ms": 1e3 * copy_seconds,
                "copy_bound": "the step's pinned H2D and D2H copies alone, on two streams at once, every rank at the "
                              "same time, best of the repetitions, max over ranks",
                "frac_of_copy_bound": copy_seconds / (e2e_seconds / e2e_steps),
                "path": "metal_linalg_qr_with_mode on pinned host pointers (staged in chunks); one pass per step",
                "matches_device_path": e2e_ok},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peaks["hbm_gbs"], "of": peak_kind,
                     "traffic": (MEASURED_TRAFFIC_PER_MATRIX * BATCH if MEASURED_TRAFFIC_PER_MATRIX else None),
                     "traffic_source": TRAFFIC_SOURCE,
                     "kernel": "qr_small_kernel<32,16,2,true>", "algorithmic_bytes_per_launch": BATCH * BYTES_PER_MATRIX},
        "clocks": clocks,
        "check": {"recon_max": recon, "orth_max": orth, "tolerance": workloads.tolerance(COLS)},
    }
    if scaled is not None:
        line["weak_scaled"] = scaled

    if world == 1 and not args.headline_only:
        del a, q, r
        torch.cuda.empty_cache()
        line["peaks"] = measure_compute_peaks(local_rank)
        line["others"] = other_configs(torch, mlt, _lib, workloads, args)
        line["roofline_4096"] = roofline_4096(line["others"], line["peaks"])
        line["mode_r"] = mode_r_configs(torch, mlt, _lib, workloads, args)
        line["svd"] = svd_configs(torch, mlt, _lib, args)
        rate, cores, kind, best = cpu_reference(4096, 2)
        sample = int(min(BATCH, max(4096, rate * 3.0)))
        rate, cores, kind, best = cpu_reference(sample, 3)
        line["cpu_baseline"] = {"value": rate, "unit": UNIT, "cores": cores, "kind": kind,
                                "sample": f"{sample} of the {BATCH} matrices, best of 3 ({best:.2f} s each)"}
    line["wall_s"] = time.perf_counter() - t_all
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def roofline_4096(others, peaks):
    """The metric's second half: one 4096 x 4096 QR as algorithmic TFLOP/s against the FP32-equivalent roofline,
    max(FP32 FMA peak, dense TF32 peak / 3), both measured in this run (sustained figures: the call is a chain
    of hundreds of kernels, not a burst)."""
    entry = next((o for o in others if o.get("config", "").startswith("c5a_4096x4096") and o.get("batch") == 1
                  and "gflops" in o), None)
    if entry is None:
        return {"error": "the 4096 x 4096 configuration did not run"}
    tflops = entry["gflops"] / 1e3
    ffma = (peaks.get("ffma") or {}).get("tflops_sustained") or 0.0
    tf32 = (peaks.get("tf32_dense") or {}).get("tflops_sustained") or 0.0
    out = {"bound": "tensor", "achieved": tflops, "unit": "TFLOP/s", "ms": entry["ms"],
           "algorithmic_gflop": entry["gflops"] * entry["ms"] / 1e3,
           "ffma_peak": ffma, "tf32_dense_peak": tf32, "tf32_over_3": tf32 / 3.0,
           "peak": max(ffma, tf32 / 3.0), "of": "measured in this run (peaks)"}
    if ffma:
        out["frac_of_ffma"] = tflops / ffma
    if tf32:
        out["frac_of_tf32_over_3"] = tflops / (tf32 / 3.0)
    if out["peak"]:
        out["frac"] = tflops / out["peak"]
    return out


def mode_r_configs(torch, mlt, _lib, workloads, args):
    """R alone against the reduced QR of the same input, a shape per kernel family (the reference quotes
    1.14-1.77x for R alone on its GPU backends, docs/qr.md:305-317)."""
    out = []
    flush = torch.zeros(64 << 20, device="cuda")
    for name, a, need_flush, steps in (
            ("c1_32x32 (batch 1024)", workloads.generate("c1_32x32").cuda(), True, args.steps),
            ("32x32 (batch 262144)", torch.randn(BATCH, 32, 32, device="cuda"), False, args.steps),
            ("c3_256x256_rank224 (batch 512)", workloads.generate("c3_256x256_rank224", batch=512, device="cuda").cuda(), False, 5),
            ("c4_65536x64_tall (batch 16)", workloads.generate("c4_65536x64_tall", batch=16).cuda(), False, 5),
            ("c5a_4096x4096", workloads.generate("c5a_4096x4096").cuda(), False, 3)):
        try:
            b, m, n = a.shape
            t_full, _ = time_config(torch, mlt, _lib, a, "reduced", steps, 3, flush if need_flush else None)
            t_r, _ = time_config(torch, mlt, _lib, a, "r", steps, 3, flush if need_flush else None)
            out.append({"config": name, "kernel": mlt.qr_kernel(m, n, b, "r"), "batch": b, "rows": m, "cols": n,
                        "ms_reduced": t_full * 1e3, "ms_r": t_r * 1e3, "speedup_r": t_full / t_r,
                        "gflops_r": b * workloads.qr_flops(m, n, "r") / t_r / 1e9})
        except Exception as e:
            out.append({"config": name, "error": f"{type(e).__name__}: {e}"})
        del a
        torch.cuda.synchronize()
    return out


def weak_scaled_configs(torch, mlt, _lib, args, rank, world, barrier, max_over_ranks):
    """Configurations 2, 3, 4 and 5b with one shard per GPU (5b: one 8192 x 8192 matrix per GPU, as the
    configuration is defined), each timed as the headline is: barrier, CUDA events, max over ranks. Inputs are
    drawn on each GPU with the configurations' shapes and distributions (the seeded CPU generators, which the
    parity tests use, would have every rank draw gigabytes on the one host at once)."""
    from metal_linalg_torch import workloads
    out = []
    g = torch.Generator(device="cuda").manual_seed(2000 + rank)

    def leg(name, make, mode, launches):
        try:
            a = make()
            b, m, n = a.shape
            k = min(m, n)
            q = torch.empty(b, m, k, device="cuda")
            r = torch.empty(b, k, n, device="cuda")
            stream = torch.cuda.current_stream().cuda_stream

            def call():
                _lib.qr(a.data_ptr(), b, m, n, q.data_ptr(), r.data_ptr(), mode, stream)
            for _ in range(3):
                call()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(launches):
                call()
            e1.record()
            barrier()
            sec = max_over_ranks(e0.elapsed_time(e1) * 1e-3) / launches
            out.append({"config": name, "mode": mode, "kernel": mlt.qr_kernel(m, n, b, mode), "batch_per_gpu": b,
                        "rows": m, "cols": n, "n_gpus": world, "ms": sec * 1e3, "matrices_per_s": world * b / sec,
                        "gflops": world * b * workloads.qr_flops(m, n, mode) / sec / 1e9,
                        "gbs": world * b * workloads.qr_bytes(m, n, mode) / sec / 1e9, "data": "drawn on each GPU"})
            del a, q, r
        except Exception as e:
            out.append({"config": name, "error": f"{type(e).__name__}: {e}"})
        torch.cuda.synchronize()
        torch.cuda.empty_cache()

    def c2():
        x = torch.randn(262144, 16, 16, generator=g, device="cuda")
        u = torch.rand(262144, generator=g, device="cuda", dtype=torch.float64) * 67.0 - 30.0
        return (x.double() * torch.pow(torch.tensor(10.0, device="cuda", dtype=torch.float64), u)[:, None, None]).float()

    def c3():
        uu = torch.linalg.qr(torch.randn(4096, 256, 256, generator=g, device="cuda", dtype=torch.float64))[0]
        vv = torch.linalg.qr(torch.randn(4096, 256, 256, generator=g, device="cuda", dtype=torch.float64))[0]
        s = torch.logspace(0.0, -7.0, 256, device="cuda", dtype=torch.float64)
        s[224:] = 0.0
        return ((uu * s) @ vv.mT).float()

    leg("c2_16x16_magnitudes", c2, "reduced", 20)
    leg("c3_256x256_rank224", c3, "reduced", 5)
    leg("c4_65536x64_tall", lambda: torch.randn(64, 65536, 64, generator=g, device="cuda"), "reduced", 5)
    leg("c5b_8192x8192 (one matrix per GPU)", lambda: torch.rand(1, 8192, 8192, generator=g, device="cuda") * 2 - 1,
        "reduced", 3)
    return out


def other_configs(torch, mlt, _lib, workloads, args):
    """The remaining benchmark configurations on one GPU: seconds per launch, matrices/s, GFLOP/s and
    GB/s from the algorithmic counts. Inputs come from the configurations' seeded CPU generators
    (metal_linalg_torch.workloads, as in the parity tests; the third configuration's float64 orthogonal
    factors are formed on the GPU from the seeded draws)."""
    out = []
    flush = torch.zeros(64 << 20, device="cuda")      # 256 MiB, larger than L2

    def add(name, a, mode, need_flush, steps=None):
        b, m, n = a.shape
        try:
            kernel = mlt.qr_kernel(m, n, b, mode)
            sec, (q, r) = time_config(torch, mlt, _lib, a, mode, steps or args.steps, max(3, min(args.warmup, 3)),
                                      flush if need_flush else None)
            s = slice(0, min(b, 2))
            a64, q64, r64 = a[s].double(), q[s].double(), r[s].double()
            recon = (torch.linalg.matrix_norm(a64 - q64 @ r64) / torch.linalg.matrix_norm(a64)).max().item()
            out.append({"config": name, "mode": mode, "kernel": kernel, "batch": b, "rows": m, "cols": n,
                        "ms": sec * 1e3, "matrices_per_s": b / sec,
                        "gflops": b * workloads.qr_flops(m, n, mode) / sec / 1e9,
                        "gbs": b * workloads.qr_bytes(m, n, mode) / sec / 1e9,
                        "l2_flush": bool(need_flush), "recon_max": recon})
        except Exception as e:   # a configuration whose kernel is not built yet is reported, not hidden
            out.append({"config": name, "mode": mode, "error": f"{type(e).__name__}: {e}"})
        torch.cuda.synchronize()

    add("c1_32x32 (batch 1024)", workloads.generate("c1_32x32").cuda(), "reduced", True)
    add("c2_16x16_magnitudes", workloads.generate("c2_16x16_magnitudes").cuda(), "reduced", False)
    try:
        a = workloads.generate("c3_256x256_rank224", device="cuda").cuda()
        add("c3_256x256_rank224", a, "reduced", False)
        add("c3_256x256_rank224", a, "complete", False)
        del a
    except Exception as e:
        out.append({"config": "c3_256x256_rank224", "error": f"{type(e).__name__}: {e}"})
    add("c4_65536x64_tall", workloads.generate("c4_65536x64_tall").cuda(), "reduced", False)
    add("c5a_4096x4096", workloads.generate("c5a_4096x4096").cuda(), "reduced", False, steps=min(args.steps, 5))
    a8 = workloads.generate("c5b_8192x8192").cuda()
    add("c5b_8192x8192 (one of the eight matrices: one per GPU)", a8[:1], "reduced", False, steps=2)
    add("c5b_8192x8192 x 8 (the whole configuration on one GPU)", a8, "reduced", False, steps=1)
    del a8
    g = torch.Generator(device="cuda").manual_seed(7)
    add("c5a_4096x4096 x 8 (a batch, drawn on the GPU: several matrices at a time)",
        torch.rand(8, 4096, 4096, generator=g, device="cuda") * 2 - 1, "reduced", False, steps=2)
    return out


def svd_configs(torch, mlt, _lib, args):
    """The SVD that calls the QR (min(M, N) <= 128), on one GPU: seconds per call by CUDA events through
    the C ABI on device pointers, matrices/s, and GB/s from the algorithmic bytes (A read once; s, and with
    vectors U and Vt, written once). Beside each, LAPACK's sgesdd (the routine the reference's CPU SVD calls)
    on one host core over a bounded sample."""
    import numpy as np
    import scipy.linalg
    out = []
    g = torch.Generator(device="cuda").manual_seed(11)

    def add(name, b, m, n, vectors):
        try:
            a = torch.randn(b, m, n, generator=g, device="cuda")
            k = min(m, n)
            s = torch.empty(b, k, device="cuda")
            u = torch.empty(b, m, k, device="cuda") if vectors else None
            vt = torch.empty(b, k, n, device="cuda") if vectors else None
            info = torch.zeros(b, dtype=torch.int32, device="cuda")
            stream = torch.cuda.current_stream().cuda_stream

            def call():
                _lib.svd(a.data_ptr(), b, m, n, u.data_ptr() if vectors else None, s.data_ptr(),
                         vt.data_ptr() if vectors else None, info.data_ptr(), stream)
            for _ in range(3):
                call()
            torch.cuda.synchronize()
            steps = max(2, min(args.steps, 5))
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                call()
            e1.record()
            e1.synchronize()
            sec = e0.elapsed_time(e1) / 1e3 / steps
            ref = torch.linalg.svdvals(a[:64].double())
            err = ((s[:64].double() - ref).abs().amax(-1) / torch.linalg.matrix_norm(a[:64].double())).max().item()
            converged = bool(((info >> 16) & 1).all().item())
            bytes_ = 4 * b * (m * n + k + ((m * k + k * n) if vectors else 0))
            host = a[:max(1, min(b, 200000 // (m * n) + 1))].cpu().numpy()
            t0 = time.perf_counter()
            for x in host:
                scipy.linalg.svd(x, compute_uv=vectors, full_matrices=False, lapack_driver="gesdd")
            cpu = len(host) / (time.perf_counter() - t0)
            out.append({"config": name, "vectors": vectors, "backend": mlt.svd_backend(m, n, b),
                        "qr_kernel": mlt.qr_kernel(max(m, n), k, b, "reduced" if vectors else "r"),
                        "batch": b, "rows": m, "cols": n, "ms": sec * 1e3, "matrices_per_s": b / sec,
                        "gbs": bytes_ / sec / 1e9, "sval_err_max": err, "converged": converged,
                        "cpu_sgesdd_matrices_per_s": cpu, "cpu_cores": 1, "cpu_sample": len(host)})
            del a, s, u, vt
        except Exception as e:
            out.append({"config": name, "error": f"{type(e).__name__}: {e}"})
        torch.cuda.synchronize()

    add("svdvals 4096 x 2048x32 (tall: R alone, then Jacobi)", 4096, 2048, 32, False)
    add("svd 4096 x 2048x32", 4096, 2048, 32, True)
    add("svd 262144 x 32x32", 262144, 32, 32, True)
    add("svdvals 262144 x 32x32", 262144, 32, 32, False)
    add("svd 262144 x 16x16", 262144, 16, 16, True)
    add("svdvals 64 x 65536x32", 64, 65536, 32, False)
    add("svdvals 64 x 65536x64 (the fourth configuration's shape)", 64, 65536, 64, False)
    add("svd 64 x 65536x64 (the fourth configuration's shape)", 64, 65536, 64, True)
    add("svd 1024 x 512x128", 1024, 512, 128, True)
    return out


PROFILE_CASES = {
    # name: (batch, rows, cols, mode): small enough for an ncu capture to end by itself, larger than L2
    "small32": (65536, 32, 32, "reduced"),
    "small16": (262144, 16, 16, "reduced"),
    "mid256": (592, 256, 256, "reduced"),
    "tsqr": (8, 65536, 64, "reduced"),
    "blocked4096": (1, 4096, 4096, "reduced"),
    "blocked8192": (1, 8192, 8192, "reduced"),
    # the SVD that calls the QR (mode "svd": U, S and Vt)
    "svd32": (65536, 32, 32, "svd"),
    "svd128": (592, 512, 128, "svd"),
}


def run_profile_case(name, launches):
    """A few launches of one configuration and nothing else: the target of the ncu captures."""
    import torch

    import metal_linalg_torch as mlt
    from metal_linalg_torch import _lib
    b, m, n, mode = PROFILE_CASES[name]
    g = torch.Generator(device="cuda").manual_seed(5)
    a = torch.randn(b, m, n, generator=g, device="cuda")
    if mode == "svd":
        mlt.svd(a)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(launches):
            mlt.svd(a)
        e1.record()
        e1.synchronize()
        print(json.dumps({"profile_case": name, "backend": mlt.svd_backend(m, n, b), "batch": b, "rows": m, "cols": n,
                          "ms_per_launch": e0.elapsed_time(e1) / launches}), flush=True)
        return
    sec, _ = time_config(torch, mlt, _lib, a, mode, launches, 1, None)
    print(json.dumps({"profile_case": name, "kernel": mlt.qr_kernel(m, n, b, mode), "batch": b, "rows": m, "cols": n,
                      "ms_per_launch": sec * 1e3}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--headline-only", action="store_true", help="skip the other configurations and the CPU baseline")
    ap.add_argument("--profile-case", choices=sorted(PROFILE_CASES), help="run a few launches of one small case and exit")
    ap.add_argument("--launches", type=int, default=3)
    args = ap.parse_args()
    if args.profile_case:
        return run_profile_case(args.profile_case, args.launches)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
