"""Benchmark of the BCPNN hidden-layer train step (forward + softmax + trace/weight/
bias/mask update) on synthetic STL-10-shaped data.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
                    [--workload stl10_f32|mnist_f32|mnist_f64|wide_f32|stl10_dp_f32]

One "step" is one pass of the layer over one batch: ``compute_activation`` then
``train_step`` with a mask update (every step: the worst case of the reference's
schedule).  Default workload: 55296 -> 30x100 units, float32, batch 256 per GPU
(``stl10_f32``); with N > 1 every rank takes its own 256 samples of a 256*N global
batch and one sum-allreduce of the batch deltas precedes the trace update (weak
scaling).  ``stl10_dp_f32`` is the fixed global batch 8192 split over the ranks.

Prints ONE JSON line (rank 0).  ``value`` is samples/s with the batches resident in
HBM, ``e2e`` the same metric through the host-buffer C-ABI call (pinned host input
copied in, activations copied out, every step).  ``--impl reference`` times the
reference's own CPU implementation (compiled OpenMP module under oracle/_ref, else
the C restatement) on the host cores for the same workload.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import statistics
import sys
import time


def host_cores() -> int:
    """Host cores this process may run on."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


if "reference" in sys.argv[1:]:
    # The CPU arm uses every host core whatever the launcher exported (torch.distributed.run sets
    # OMP_NUM_THREADS=1 for its workers): the OpenMP and OpenBLAS runtimes read these when they load,
    # which is after this line.
    os.environ["OMP_NUM_THREADS"] = os.environ["OPENBLAS_NUM_THREADS"] = str(host_cores())

import numpy as np

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

from streambrain_b200 import synthetic  # noqa: E402

POOL = 8  # distinct resident batches cycled through (8 x 56.6 MB of inputs > 126 MB of L2)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-mask", action="store_true", help="skip the per-step mask update")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg")
    ap.add_argument("--dp-path", action="store_true",
                    help="at N = 1, run the data-parallel step (row-block products, reduction, row-block "
                         "apply) with nothing to reduce: the kernels every rank runs at N > 1")
    ap.add_argument("--no-dp-large", action="store_true",
                    help="skip the extra leg on the large-batch data-parallel workload (stl10_dp_f32)")
    ap.add_argument("--dp-mode", default="sharded", choices=["sharded", "allreduce"],
                    help="data-parallel step at N > 1: the layer's input rows sharded over the ranks (inputs exchanged "
                         "by columns over peer-mapped memory, supports summed, every row updated once by its "
                         "owner) or all-reduce of the batch sums and replicated update")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="skip the short legs on the other configurations (mnist_f32, mnist_f64, wide_f32)")
    ap.add_argument("--contraction", default="tensor", choices=["tensor", "general"],
                    help="tcgen05 tensor-core kernels (default) or the general-shape FFMA kernels")
    return ap.parse_args()


def measured_peaks():
    try:
        with open(os.path.join(REPO, "MEASURED_PEAKS.json")) as f:
            return json.load(f), "measured"
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


def algorithmic_work(N, M, H, B, s):
    """Bytes and flops one step must move / do, per phase: the forward product reads W, x and the
    bias and writes y; the trace update reads Cij and writes Cij and W (3 N M), reads x, y and the mask."""
    fwd_bytes = (N * M + B * N + B * M + M) * s
    upd_bytes = (3 * N * M + B * N + B * M) * s + N * H
    flops = 2.0 * B * N * M
    return fwd_bytes, upd_bytes, flops


def workload_config(wl, p, batch, world, mask, dp_path=False):
    """The ``config`` object of the JSON line: the workload, identical for the GPU arm and the CPU arm."""
    hp = p["hidden"]
    N, H, Mc = hp["in_features"], hp["hypercolumns"], hp["minicolumns"]
    s = np.dtype(p["dtype"]).itemsize
    return {"workload": wl, "layer": "%d->%dx%d" % (N, H, Mc), "batch_per_gpu": batch,
            "global_batch": batch * world, "mask_update": "every step" if mask else "none",
            "start_state": "traces at the independent steady state (mask scores finite, as from epoch 2 on)",
            "l2": "inputs larger than L2: %d resident batches cycled, %.0f MB of state streamed per step" % (
                POOL, 2 * N * H * Mc * s / 1e6),
            "parallelism": "dp%d" % world + (" (data-parallel step on one rank, nothing to exchange)"
                                             if dp_path and world == 1 else "")}


def host_description():
    """CPU model, OpenMP threads in force and the BLAS behind the reference module."""
    model = "unknown"
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    model = line.split(":", 1)[1].strip()
                    break
    except OSError:
        pass
    threads = None
    try:
        threads = int(ctypes.CDLL("libgomp.so.1").omp_get_max_threads())
    except OSError:
        pass
    blas = None
    try:
        sys.path.insert(0, os.path.join(REPO, "oracle"))
        import build as oracle_build
        info = os.path.join(os.path.dirname(oracle_build.ref_module_path()), "BUILD_INFO.txt")
        with open(info) as f:
            for line in f:
                if line.startswith("blas:"):
                    blas = line.split(":", 1)[1].strip()
    except Exception:
        pass
    return {"cpu_model": model, "host_cores": host_cores(), "omp_max_threads": threads,
            "OMP_NUM_THREADS": os.environ.get("OMP_NUM_THREADS"),
            "OPENBLAS_NUM_THREADS": os.environ.get("OPENBLAS_NUM_THREADS"), "blas": blas}


def use_all_host_cores():
    """Make the OpenMP runtime already loaded in this process (if any) use every host core."""
    n = host_cores()
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(n)
    except OSError:
        pass
    return n


class ClockSampler:
    """SM clock and throttle-reason samples during the timed region, read through NVML every few
    milliseconds on a thread of this process (read only; nothing is set)."""

    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"), (0x20, "sw_thermal_slowdown"),
               (0x4, "sw_power_cap"))

    def __init__(self, gpu_index, period_s=0.001):
        import threading
        self.sm, self.reasons, self.max_mhz = [], set(), None
        self.stop_flag = threading.Event()
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            try:   # the CUDA ordinal may be remapped by CUDA_VISIBLE_DEVICES: find the board by UUID
                import torch
                h = pynvml.nvmlDeviceGetHandleByUUID("GPU-" + str(torch.cuda.get_device_properties(gpu_index).uuid))
            except Exception:
                h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            return

        def poll():
            while not self.stop_flag.is_set():
                try:
                    self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    bits = int(pynvml.nvmlDeviceGetCurrentClocksThrottleReasons(h))
                    for bit, name in self.REASONS:
                        if bits & bit:
                            self.reasons.add(name)
                except Exception:
                    pass
                self.stop_flag.wait(period_s)
        self.thread = threading.Thread(target=poll, daemon=True)
        self.thread.start()

    def stop(self):
        self.stop_flag.set()
        if self.thread is not None:
            self.thread.join(timeout=2)
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(sm)}


def make_batches(p, batch, count, seed):
    xs = []
    for k in range(count):
        x, _ = synthetic.make_inputs(batch, p["n_pixels"], p["sparsity"], p["dtype"], seed=seed + k)
        xs.append(x)
    return xs


# --------------------------------------------------------------------------- CPU
def cpu_layer(p, kernels, seed=0):
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import oracle
    hp = p["hidden"]
    np.random.seed(seed)
    return oracle.OracleLayer(kernels, "plastic", hp["in_features"], hp["hypercolumns"], hp["minicolumns"],
                              hp["taupdt"], hp["initial_counters"], p["dtype"], khalf=hp["khalf"], pmin=hp["pmin"],
                              taubdt=hp["taubdt"], density=hp["density"])


def global_batches(p, batch, world, count):
    """The global batches of the GPU arm: rank r's batch k is drawn from seed DATA_SEED + 1000 r + k."""
    out = []
    for k in range(count):
        parts = [make_batches(p, batch, 1, synthetic.DATA_SEED + 1000 * r + k)[0] for r in range(world)]
        out.append(parts[0] if world == 1 else np.ascontiguousarray(np.concatenate(parts, axis=0)))
    return out


def cpu_time_steps(p, batch, world, steps, warmup, budget_s, mask=True, pool=2):
    """Time the reference CPU implementation of the same step on the global batch (batch * world
    samples: the reference's data-parallel backend equals its cpu backend on the concatenated batch,
    BCPNN/backend/_kernels/test_mpi.py:48-59).  Returns (samples_per_s, mean_s, steps_timed, kind, cores)."""
    sys.path.insert(0, os.path.join(REPO, "oracle"))
    import oracle
    cores = use_all_host_cores()
    kernels = oracle.best_kernels()
    layer = cpu_layer(p, kernels)
    xs = global_batches(p, batch, world, pool)
    layer.Ci, layer.Cj, layer.Cij = synthetic.steady_state_traces(p, xs[0][:batch])
    H = p["hidden"]["hypercolumns"]
    times = []
    t_start = time.perf_counter()
    warmed = 0
    s = 0
    while len(times) < steps:
        x = xs[s % len(xs)]
        t0 = time.perf_counter()
        act = layer.compute_activation(x)
        layer.train_step(x, act, (s % H) if mask else None)
        dt = time.perf_counter() - t0
        s += 1
        elapsed = time.perf_counter() - t_start
        # on a slow host the warm-up may not eat the budget: it ends after `warmup` steps or a quarter of it
        if warmed < warmup and not times and (warmed == 0 or elapsed < 0.25 * budget_s):
            warmed += 1
            continue
        times.append(dt)
        if len(times) >= 2 and elapsed + dt > budget_s:
            break
    mean = sum(times) / len(times)
    cpu_time_steps.warmup_done = warmed
    return batch * world / mean, mean, len(times), kernels.kind, cores


def run_reference(args, wl, p, batch):
    """The reference arm: the same workload (the global batch the GPU arm processes at this N), same
    steps and warm-up, on the host cores.  Under a multi-rank launcher rank 0 alone works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    mask = not args.no_mask
    sps, mean, done, kind, cores = cpu_time_steps(p, batch, world, args.steps, args.warmup, budget_s=240.0,
                                                  mask=mask, pool=min(POOL, 4))
    sample = "%d of %d full steps (forward + train_step%s) of %s at the global batch %d, %d warm-up" % (
        done, args.steps, " + mask update" if mask else "", wl, batch * world,
        getattr(cpu_time_steps, "warmup_done", args.warmup))
    line = {
        "impl": "reference", "metric": "training samples/sec per layer", "value": sps, "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": mean * 1e3,
        "higher_is_better": True, "scaling": "strong" if wl == "stl10_dp_f32" else "weak", "vs_baseline": None,
        "dtype": "f32" if p["dtype"] == np.float32 else "f64", "data": "synthetic",
        "config": workload_config(wl, p, batch, world, mask),
        "cpu_baseline": {"value": sps, "unit": "samples/s", "cores": cores, "kind": kind, "sample": sample,
                         "steps_timed": done, "host": host_description()},
        "e2e": {"value": sps, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU
FP64_PEAK_TFLOPS = 37.2   # 148 SMs x 64 FP64 lanes x 2 flops x 1.965 GHz (nominal; this pool measures no FP64 peak)
FFMA_PEAK_TFLOPS = 74.4   # 148 SMs x 128 FP32 lanes x 2 flops x 1.965 GHz (nominal)


_FP64_RATES = {}


def fp64_rates(lib):
    """Measured DFMA and float64 tensor-core (mma.sync m8n8k4) rates of the device, TFLOP/s (measured once)."""
    if not _FP64_RATES:
        a, b = ctypes.c_double(0), ctypes.c_double(0)
        if lib.sbb_measure_fp64_rates(ctypes.byref(a), ctypes.byref(b)) == 0 and a.value > 0:
            _FP64_RATES.update(dfma=a.value, dmma=b.value)
        else:
            _FP64_RATES.update(dfma=None, dmma=None)
    return _FP64_RATES


def step_roofline_of(p, batch, ms_per_step, peaks, tensor_path, fp64=None):
    """Whole-step roofline: each of the two phases (forward, trace update) bounded by the larger of its
    memory time and its compute time at the peak of the datapath that ran it.  float32 on the tensor
    path costs three TF32 products per product, i.e. a sixth of the measured bf16 rate; both the burst
    and the sustained measurement of that rate are given, ``frac`` uses the burst (stricter) one."""
    hp = p["hidden"]
    N, H, Mc = hp["in_features"], hp["hypercolumns"], hp["minicolumns"]
    s = np.dtype(p["dtype"]).itemsize
    fwd_b, upd_b, flops = algorithmic_work(N, H * Mc, H, batch, s)
    hbm = float(peaks["hbm_gbs"]) * 1e9
    if s == 8 and fp64 and fp64.get("dfma"):
        burst = sustained = max(fp64["dfma"], fp64.get("dmma") or 0.0)
        note = ("peak = float64 rate measured on this device: DFMA loop %.1f TFLOP/s, mma.sync m8n8k4 loop %.1f "
                "TFLOP/s (tcgen05 has no float64 kind)" % (fp64["dfma"], fp64.get("dmma") or 0.0))
    elif s == 8:
        burst = sustained = FP64_PEAK_TFLOPS
        note = "peak = nominal FP64 rate (DFMA), no tensor-core path exists for float64"
    elif tensor_path:
        burst = float(peaks["bf16_tflops"]) / 6.0
        sustained = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])) / 6.0
        note = "peak = measured bf16 rate / 6 (float32 by three TF32 products): burst, and sustained under the power cap"
    else:
        burst = sustained = FFMA_PEAK_TFLOPS
        note = "peak = nominal FP32 FFMA rate (general-shape kernels)"

    def t_roof(peak_tf):
        c = flops / (peak_tf * 1e12)
        return (max(fwd_b / hbm, c) + max(upd_b / hbm, c)) * 1e3
    return {"t_roof_ms": t_roof(burst), "frac": t_roof(burst) / ms_per_step, "compute_peak_tflops": burst,
            "t_roof_ms_sustained_peak": t_roof(sustained), "frac_sustained_peak": t_roof(sustained) / ms_per_step,
            "compute_peak_tflops_sustained": sustained, "note": note}


def short_leg(B200, lib, check, torch, wl, peaks, steps=20, warmup=3, profile_phases=False):
    """One of the other configurations, timed the same way as the headline (resident batches, mask update
    every step, CUDA events) over a short region."""
    p = synthetic.layer_params(wl)
    hp = p["hidden"]
    N, H, Mc, batch = hp["in_features"], hp["hypercolumns"], hp["minicolumns"], p["batch"]
    M = H * Mc
    np.random.seed(0)
    layer = B200.StructuralPlasticityLayer(N, H, Mc, hp["taupdt"], hp["khalf"], hp["pmin"], hp["taubdt"],
                                           hp["density"], 16, hp["initial_counters"], dtype=p["dtype"])
    state_mb = 2 * N * M * np.dtype(p["dtype"]).itemsize / 1e6
    pool = 4 if state_mb > 126 else 16   # small layers are L2-resident by nature; their inputs still cycle
    xs_host = make_batches(p, batch, pool, synthetic.DATA_SEED)
    layer.Ci, layer.Cj, layer.Cij = synthetic.steady_state_traces(p, xs_host[0])
    xs = [torch.from_numpy(x).cuda() for x in xs_host]
    y = torch.empty((batch, M), dtype=xs[0].dtype, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def step(k):
        x = xs[k % pool]
        check(lib.sbb_layer_forward(layer._handle, x.data_ptr(), batch, y.data_ptr(), stream))
        check(lib.sbb_layer_train_step(layer._handle, x.data_ptr(), y.data_ptr(), batch, k % H, stream))
    for k in range(warmup):
        step(k)
    torch.cuda.synchronize()
    if profile_phases:
        check(lib.sbb_layer_profile(layer._handle, 1))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for k in range(steps):
        step(warmup + k)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    tensor_path = bool(lib.sbb_tensor_path_available()) and bool(lib.sbb_get_contraction_path()) and \
        p["dtype"] == np.float32
    phases = None
    if profile_phases:   # the two contractions alone, against the float64 rate of the device
        def mean_ms(phase):
            n = ctypes.c_long(0)
            check(lib.sbb_layer_phase_calls(layer._handle, phase, ctypes.byref(n)))
            out = []
            for i in range(max(0, n.value - 64), n.value):
                t = ctypes.c_float(0)
                check(lib.sbb_layer_phase_ms(layer._handle, phase, i, ctypes.byref(t)))
                out.append(t.value)
            return sum(out) / len(out) if out else None
        fwd, upd = mean_ms(0), mean_ms(1)
        check(lib.sbb_layer_profile(layer._handle, 0))
        flops = 2.0 * batch * N * M
        rates = fp64_rates(lib) if p["dtype"] == np.float64 else {}
        peak = max(rates.get("dfma") or 0.0, rates.get("dmma") or 0.0) or None
        phases = {"forward_ms": fwd, "trace_update_ms": upd,
                  "forward_tflops": flops / (fwd * 1e-3) / 1e12 if fwd else None,
                  "trace_update_tflops": flops / (upd * 1e-3) / 1e12 if upd else None,
                  "fp64_rates_tflops": rates or None,
                  "forward_frac_of_fp64_rate": flops / (fwd * 1e-3) / 1e12 / peak if fwd and peak else None,
                  "trace_update_frac_of_fp64_rate": flops / (upd * 1e-3) / 1e12 / peak if upd and peak else None}
    fp64 = fp64_rates(lib) if p["dtype"] == np.float64 else None
    return {"workload": wl, "layer": "%d->%dx%d" % (N, H, Mc), "batch": batch,
            "dtype": "f32" if p["dtype"] == np.float32 else "f64", "value": batch / (ms * 1e-3), "unit": "samples/s",
            "ms_per_step": ms, "steps": steps, "warmup": warmup,
            "l2": "state %.0f MB %s" % (state_mb, "> L2, streamed every step" if state_mb > 126 else
                                         "(fits the 126 MB L2: this configuration is L2-resident by nature)"),
            "contractions": phases,
            "step_roofline": step_roofline_of(p, batch, ms, peaks, tensor_path, fp64)}


def data_parallel_checks(B200, lib, check, torch, dist, layer, world, rank, all_reduce, sharded):
    """Outside the timed region, at N > 1: (1) the replicas of the timed layer are bit-identical
    (checksums of Cij, weights and mask agree over ranks); (2) on a reduced shape one data-parallel
    step over the ranks equals the fused single-GPU step at the same global batch."""
    if sharded:   # a rank holds current weights and traces only for the rows it owns until they are shared
        layer.share_rows(all_reduce)
    sums = []
    for name in ("Cij", "weights", "wmask"):
        t = layer.state_tensor(name)
        bits = t.view(torch.int32) if t.dtype != torch.uint8 else t
        sums.append(bits.to(torch.int64).sum())
    lo = torch.stack(sums)
    hi = lo.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    identical = bool(torch.equal(lo, hi))

    N, H, Mc, b_local, h = 4096, 30, 100, 128, 3
    M = H * Mc
    hp = synthetic.layer_params("stl10_f32", batch=b_local * world)["hidden"]
    rs = np.random.RandomState(4321)
    pix = rs.rand(b_local * world, N // 2).astype(np.float32)
    xg = synthetic.complementary_code(pix)
    small_p = {"hidden": dict(hp, in_features=N), "dtype": np.dtype(np.float32)}
    traces = synthetic.steady_state_traces(small_p, xg)

    def make():
        np.random.seed(0)
        l = B200.StructuralPlasticityLayer(N, H, Mc, hp["taupdt"], hp["khalf"], hp["pmin"], hp["taubdt"],
                                           hp["density"], 16, hp["initial_counters"], dtype=np.float32)
        l.Ci, l.Cj, l.Cij = traces
        return l
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    dp = make()
    if sharded:
        from streambrain_b200 import parallel
        dp.shard_rows(rank, world, parallel.all_gather_bytes_over(dist), b_local)
    xl = torch.from_numpy(np.ascontiguousarray(xg[rank * b_local:(rank + 1) * b_local])).cuda()
    yl = torch.empty((b_local, M), dtype=torch.float32, device="cuda")
    if sharded:
        dp.sharded_step(xl, h, all_reduce, out=yl)
        dp.share_rows(all_reduce)
    else:
        check(lib.sbb_layer_forward(dp._handle, xl.data_ptr(), b_local, yl.data_ptr(), stream))
        dp.dp_train_step(xl, yl, h, world, all_reduce)
    torch.cuda.synchronize()
    err, masks_equal = None, None
    if rank == 0:
        one = make()
        xa = torch.from_numpy(xg).cuda()
        ya = torch.empty((b_local * world, M), dtype=torch.float32, device="cuda")
        check(lib.sbb_layer_forward(one._handle, xa.data_ptr(), b_local * world, ya.data_ptr(), stream))
        check(lib.sbb_layer_train_step(one._handle, xa.data_ptr(), ya.data_ptr(), b_local * world, h, stream))
        torch.cuda.synchronize()
        err = 0.0
        for name in ("Ci", "Cj", "Cij"):
            a, b = getattr(dp, name).astype(np.float64), getattr(one, name).astype(np.float64)
            err = max(err, float(np.abs(a - b).max() / np.abs(b).max()))
        masks_equal = bool(np.array_equal(dp.wmask, one.wmask))
        if masks_equal:
            a, b = dp.weights.astype(np.float64), one.weights.astype(np.float64)
            err = max(err, float(np.abs(a - b).max() / max(1.0, np.abs(b).max())) / 10)
    return {"mode": "row-sharded layer over peer-mapped memory" if sharded else "all-reduce, replicated update",
            "replicas_identical": identical, "dp_vs_single_rel_err": err, "dp_vs_single_masks_equal": masks_equal,
            "dp_vs_single_shape": "%d->%dx%d, global batch %d, one step with a mask update; traces relative "
                                  "to their maximum, weights / 10 (their tolerance is 10x the traces')" % (
                                      N, H, Mc, b_local * world)}


def run_b200(args, wl, p, batch):
    import torch
    import torch.distributed as dist
    import streambrain_b200 as B200
    from streambrain_b200._lib import check, lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl b200 needs a CUDA device (there is no CPU fallback)")
    torch.cuda.set_device(local_rank)
    check(lib.sbb_set_contraction_path(1 if args.contraction == "tensor" else 0))
    tensor_path = args.contraction == "tensor" and bool(lib.sbb_tensor_path_available()) and p["dtype"] == np.float32
    if world > 1:
        # NCCL's kernels on a high-priority stream: their few CTAs are scheduled ahead of the pending
        # CTAs of the step's own kernels, so the reduction of a row block runs beside the next block
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), pg_options=opts)
    hp = p["hidden"]
    N, H, Mc = hp["in_features"], hp["hypercolumns"], hp["minicolumns"]
    M = H * Mc
    np_dtype = p["dtype"]
    s = np.dtype(np_dtype).itemsize
    np.random.seed(0)  # identical replicas on every rank
    layer = B200.StructuralPlasticityLayer(N, H, Mc, hp["taupdt"], hp["khalf"], hp["pmin"], hp["taubdt"],
                                           hp["density"], 16, hp["initial_counters"], dtype=np_dtype)
    xs_host = make_batches(p, batch, POOL, synthetic.DATA_SEED + 1000 * rank)
    ref_batch = xs_host[0] if rank == 0 else make_batches(p, batch, 1, synthetic.DATA_SEED)[0]
    layer.Ci, layer.Cj, layer.Cij = synthetic.steady_state_traces(p, ref_batch)   # identical on every rank
    sharded = world > 1 and args.dp_mode == "sharded"
    if sharded:
        from streambrain_b200 import parallel
        layer.shard_rows(rank, world, parallel.all_gather_bytes_over(dist), batch)
    elif world == 1 and args.dp_path and args.dp_mode == "sharded":
        layer.shard_rows(0, 1, lambda blob: [blob], batch)   # the sharded step's kernels on one rank (nothing crosses NVLink)
    shard_step = getattr(layer, "_shard", None) is not None
    xs = [torch.from_numpy(x).cuda() for x in xs_host]
    ys = [torch.empty((batch, M), dtype=xs[0].dtype, device="cuda") for _ in range(2)]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    class _Reduced:   # a finished reduction, for --dp-path at N = 1
        def wait(self):
            pass
    dp_path = world > 1 or args.dp_path
    all_reduce = (lambda t: dist.all_reduce(t, async_op=True)) if world > 1 else (lambda t: _Reduced())
    mask = not args.no_mask

    def step(k):
        x, y = xs[k % POOL], ys[k % 2]
        h = (k % H) if mask else None
        if shard_step:   # forward + train in one: the layer's rows are spread over the ranks; the next batch's
            # exchange is staged beside this step
            layer.sharded_step(x, h, all_reduce, out=y, next_inputs=xs[(k + 1) % POOL])
            return
        check(lib.sbb_layer_forward(layer._handle, x.data_ptr(), batch, y.data_ptr(), stream))
        if dp_path:
            layer.dp_train_step(x, y, h, world, all_reduce)
        else:
            check(lib.sbb_layer_train_step(layer._handle, x.data_ptr(), y.data_ptr(), batch, -1 if h is None else h,
                                           stream))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for k in range(args.warmup):
        step(k)
    barrier()
    check(lib.sbb_layer_profile(layer._handle, 1))
    sampler = ClockSampler(local_rank) if rank == 0 else None
    launches0 = int(lib.sbb_kernel_launches())
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for k in range(args.steps):
        step(args.warmup + k)
    ev1.record()
    barrier()
    elapsed_ms = ev0.elapsed_time(ev1)
    launches = int(lib.sbb_kernel_launches()) - launches0
    if shard_step:
        layer.drop_staged()   # the batch staged by the last timed step is not consumed
    clocks = sampler.stop() if sampler else None
    if world > 1:
        t = torch.tensor([elapsed_ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())

    # per-kernel durations recorded inside the timed region
    def phase_ms(phase):
        n = ctypes.c_long(0)
        check(lib.sbb_layer_phase_calls(layer._handle, phase, ctypes.byref(n)))
        out = []
        for i in range(max(0, n.value - 64), n.value):
            ms = ctypes.c_float(0)
            check(lib.sbb_layer_phase_ms(layer._handle, phase, i, ctypes.byref(ms)))
            out.append(ms.value)
        return out, n.value
    fwd_ms, _ = phase_ms(0)
    trace_ms, trace_calls = phase_ms(1)
    check(lib.sbb_layer_profile(layer._handle, 0))
    wait_status = ctypes.c_int(0)
    check(lib.sbb_device_wait_status(ctypes.byref(wait_status)))

    # The data-parallel workload of the same layer (global batch 8192 cut evenly over the ranks, strong
    # scaling), timed the same way and reported beside the headline under "dp_large_batch".
    dp_large = None
    if wl == "stl10_f32" and not args.no_dp_large:
        del xs, ys
        pl = synthetic.layer_params("stl10_dp_f32")
        gb = pl["batch"]
        bl = gb // world
        hl = pl["hidden"]
        np.random.seed(0)
        big = B200.StructuralPlasticityLayer(N, H, Mc, hl["taupdt"], hl["khalf"], hl["pmin"], hl["taubdt"],
                                             hl["density"], 16, hl["initial_counters"], dtype=np_dtype)
        big.Ci, big.Cj, big.Cij = synthetic.steady_state_traces(pl, ref_batch)
        if sharded:
            big.shard_rows(rank, world, parallel.all_gather_bytes_over(dist), bl)
        elif shard_step:
            big.shard_rows(0, 1, lambda blob: [blob], bl)
        gen = torch.Generator(device="cuda")
        gen.manual_seed(synthetic.DATA_SEED + 17 * rank)
        xl = []
        for _ in range(2):   # uniform pixels, complementary-coded (p, 1 - p), made on the device: 1.8 GB per batch at N = 1
            pix = torch.rand((bl, N // 2), device="cuda", generator=gen, dtype=torch.float32)
            xl.append(torch.stack((pix, 1.0 - pix), dim=2).reshape(bl, N).contiguous())
            del pix
        yl = torch.empty((bl, M), dtype=torch.float32, device="cuda")

        def big_step(k):
            x = xl[k % 2]
            h = (k % H) if mask else None
            if shard_step:
                big.sharded_step(x, h, all_reduce, out=yl, next_inputs=xl[(k + 1) % 2])
                return
            check(lib.sbb_layer_forward(big._handle, x.data_ptr(), bl, yl.data_ptr(), stream))
            if dp_path:
                big.dp_train_step(x, yl, h, world, all_reduce)
            else:
                check(lib.sbb_layer_train_step(big._handle, x.data_ptr(), yl.data_ptr(), bl, -1 if h is None else h,
                                               stream))
        n_big = max(3, min(args.steps, 8))
        for k in range(3):
            big_step(k)
        barrier()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for k in range(n_big):
            big_step(3 + k)
        b1.record()
        barrier()
        big_ms = b0.elapsed_time(b1)
        if world > 1:
            t = torch.tensor([big_ms], dtype=torch.float64, device="cuda")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            big_ms = float(t.item())
        dp_large = {"workload": "stl10_dp_f32", "global_batch": gb, "batch_per_gpu": bl, "scaling": "strong",
                    "value": gb * n_big / (big_ms * 1e-3), "unit": "samples/s", "ms_per_step": big_ms / n_big,
                    "steps": n_big, "warmup": 3, "data": "synthetic, made on the device"}
        del xl, yl, big
        xs = [torch.from_numpy(x).cuda() for x in xs_host[:4]]

    # end to end: at N = 1 through the host-buffer C-ABI call; under data parallelism (further down)
    # through the device-tensor calls with every rank's copies on a copy stream.
    e2e = None
    if world == 1 and not args.no_e2e:
        # Every step uploads its own batch from page-locked host memory and reads its activation back;
        # sbb_layer_step_host_async double-buffers the two copies against the previous / next step.
        pinned = [torch.from_numpy(x).pin_memory() for x in xs_host[:4]]
        y_host = [torch.empty((batch, M), dtype=xs[0].dtype).pin_memory() for _ in range(2)]

        def host_step(k):
            check(lib.sbb_layer_step_host_async(layer._handle, ctypes.c_void_p(pinned[k % 4].data_ptr()), None, batch,
                                                (k % H) if mask else -1, ctypes.c_void_p(y_host[k % 2].data_ptr())))
        for k in range(3):
            host_step(k)
        check(lib.sbb_layer_wait(layer._handle))
        e_steps = max(args.steps, 60)   # wall-clock timed: long enough for the host's scheduling noise to average out
        t0 = time.perf_counter()
        for k in range(e_steps):
            host_step(3 + k)
        check(lib.sbb_layer_wait(layer._handle))
        dt = time.perf_counter() - t0
        # the same loop with the blocking call (copy, step, copy back, one after the other)
        yp = ctypes.c_void_p(y_host[0].data_ptr())
        b_steps = max(3, min(args.steps, 10))
        check(lib.sbb_layer_step_host(layer._handle, ctypes.c_void_p(pinned[0].data_ptr()), None, batch, -1, yp))  # warm-up: its staging buffers
        t0 = time.perf_counter()
        for k in range(b_steps):
            check(lib.sbb_layer_step_host(layer._handle, ctypes.c_void_p(pinned[k % 4].data_ptr()), None, batch,
                                          (k % H) if mask else -1, yp))
        dt_block = time.perf_counter() - t0
        e2e = {"value": batch * e_steps / dt, "unit": "samples/s", "h2d_bytes_per_step": batch * N * s,
               "d2h_bytes_per_step": batch * M * s, "ms_per_step": dt / e_steps * 1e3,
               "call": "sbb_layer_step_host_async (pinned host buffers, copies double-buffered)",
               "blocking_call_value": batch * b_steps / dt_block}

    if world > 1 and not args.no_e2e:
        # Data parallel: every rank uploads its slice of the batch from page-locked host memory on a copy
        # stream (two device slots), runs forward + the data-parallel train step on device tensors (the
        # reduction needs them on the device), and reads its activation back; timed with the wall clock
        # between barriers, maximum over ranks.
        pinned = [torch.from_numpy(x).pin_memory() for x in xs_host[:4]]
        y_host = [torch.empty((batch, M), dtype=xs[0].dtype).pin_memory() for _ in range(2)]
        x_dev = [torch.empty((batch, N), dtype=xs[0].dtype, device="cuda") for _ in range(3 if shard_step else 2)]
        y_dev = [torch.empty((batch, M), dtype=xs[0].dtype, device="cuda") for _ in range(2)]
        copy_stream = torch.cuda.Stream()
        compute = torch.cuda.current_stream()
        landed = [torch.cuda.Event() for _ in range(3)]
        used = [torch.cuda.Event() for _ in range(3)]

        def upload(k):
            slot = k % 3
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(used[slot])          # the exchange that last read this slot has run
                x_dev[slot].copy_(pinned[k % 4], non_blocking=True)
                landed[slot].record(copy_stream)

        def sharded_host_step(k):
            # batch k + 1 is uploaded and exchanged while step k computes; batch k was staged by step k - 1
            upload(k + 1)
            layer.sharded_step(x_dev[k % 3], (k % H) if mask else None, all_reduce, out=y_dev[k % 2],
                               next_inputs=x_dev[(k + 1) % 3], next_ready=landed[(k + 1) % 3])
            used[(k + 1) % 3] = layer.staged_event
            if k == 0:   # the first batch was exchanged on the compute stream by this very call
                used[0] = torch.cuda.Event()
                used[0].record(compute)
            y_host[k % 2].copy_(y_dev[k % 2], non_blocking=True)

        def host_step(k):
            if shard_step:
                return sharded_host_step(k)
            slot = k % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(used[slot])          # the step that last read this slot has finished
                x_dev[slot].copy_(pinned[k % 4], non_blocking=True)
                landed[slot].record(copy_stream)
            compute.wait_event(landed[slot])
            check(lib.sbb_layer_forward(layer._handle, x_dev[slot].data_ptr(), batch, y_dev[slot].data_ptr(), stream))
            layer.dp_train_step(x_dev[slot], y_dev[slot], (k % H) if mask else None, world, all_reduce)
            y_host[slot].copy_(y_dev[slot], non_blocking=True)
            used[slot].record(compute)
        if shard_step:   # the first step's batch is not staged by a step before it
            upload(0)
            compute.wait_event(landed[0])
        for k in range(3):
            host_step(k)
        barrier()
        e_steps = max(args.steps, 60)   # wall-clock timed: long enough for the host's scheduling noise to average out
        t0 = time.perf_counter()
        for k in range(e_steps):
            host_step(3 + k)
        torch.cuda.synchronize()
        dt = torch.tensor([time.perf_counter() - t0], dtype=torch.float64, device="cuda")
        dist.all_reduce(dt, op=dist.ReduceOp.MAX)
        dt = float(dt.item())
        e2e = {"value": world * batch * e_steps / dt, "unit": "samples/s", "h2d_bytes_per_step": world * batch * N * s,
               "d2h_bytes_per_step": world * batch * M * s, "ms_per_step": dt / e_steps * 1e3,
               "call": ("sharded_step" if shard_step else "compute_activation + dp_train_step") +
                       " on device tensors, per-rank batch slice uploaded from pinned host memory on a copy stream"}

    if shard_step:
        layer.drop_staged()
    dp_checks = None
    if world > 1:
        dp_checks = data_parallel_checks(B200, lib, check, torch, dist, layer, world, rank, all_reduce, sharded)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    fwd_b, upd_b, flops = algorithmic_work(N, M, H, batch, s)
    if shard_step and world > 1:   # a rank's launch updates its own rows from the global batch
        _, upd_b, flops = algorithmic_work(layer.owned_rows()[1] - layer.owned_rows()[0], M, H, batch * world, s)
    ms_per_step = elapsed_ms / args.steps
    value = world * batch * args.steps / (elapsed_ms * 1e-3)
    # one launch per step on one GPU; under data parallelism the product is cut into row blocks,
    # so the per-step time is the sum over its launches
    per_step_trace = (sum(trace_ms) / len(trace_ms)) * (trace_calls / args.steps) if trace_ms else None
    hbm = float(peaks["hbm_gbs"])
    roofline = None
    if per_step_trace:
        achieved = upd_b / (per_step_trace * 1e-3) / 1e9
        tf32_sustained = float(peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])) / 2.0   # dense TF32 = half of bf16
        tf32_burst = float(peaks["bf16_tflops"]) / 2.0
        tf = 3 * flops / (per_step_trace * 1e-3) / 1e12
        roofline = {"bound": "hbm", "kernel": "trace update (x^T y + EMA + log-ratio weights + mask)",
                    "achieved": achieved, "peak": hbm, "unit": "GB/s", "frac": achieved / hbm,
                    # DRAM bytes are not measured by this program: the ncu capture of this kernel is summarised
                    # in the named profile
                    "traffic": None,
                    "traffic_source": "profiles/tc_contraction_kernels_stl10_f32.txt (dram__bytes_read.sum + "
                                      "dram__bytes_write.sum of one launch under ncu)" if tensor_path else
                                      "profiles/trace_update_simt_stl10_f32.txt",
                    "peak_source": peak_kind, "algorithmic_bytes": upd_b,
                    "ms_per_launch": per_step_trace,
                    "forward_ms": (sum(fwd_ms) / len(fwd_ms)) if fwd_ms else None,
                    # the same launch against the tensor pipe: three TF32 products per float32 product
                    "tensor": {"achieved": tf, "unit": "TFLOP/s (TF32)", "peak": tf32_burst, "frac": tf / tf32_burst,
                               "peak_sustained": tf32_sustained, "frac_sustained_peak": tf / tf32_sustained}
                    if tensor_path else None}
    step_roofline = step_roofline_of(p, batch, ms_per_step, peaks, tensor_path)

    other = None
    if world == 1 and wl == "stl10_f32" and not args.no_other_configs:
        del xs
        torch.cuda.empty_cache()
        other = []
        # the three other reference configurations, and the float64 kernels at the large shape (not a reference
        # configuration: it shows their rate where launch and pipeline-fill overheads do not dominate)
        for name, kw in (("mnist_f32", {}), ("mnist_f64", {"profile_phases": True}), ("wide_f32", {}),
                         ("stl10_f64", {"steps": 5, "warmup": 2, "profile_phases": True})):
            try:
                other.append(short_leg(B200, lib, check, torch, name, peaks, **kw))
            except Exception as e:
                other.append({"workload": name, "error": str(e)[:200]})

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        try:
            sps, mean, done, kind, cores = cpu_time_steps(p, batch, 1, 12, 1, budget_s=30.0, mask=mask)
            cpu = {"value": sps, "unit": "samples/s", "cores": cores, "kind": kind, "ms_per_step": mean * 1e3,
                   "sample": "%d full steps of the same workload (batch %d) after 1 warm-up" % (done, batch),
                   "host": host_description()}
        except Exception as e:  # the CPU leg must never take the GPU line down
            cpu = {"value": None, "unit": "samples/s", "cores": 0, "kind": "unavailable", "sample": str(e)[:200]}

    line = {
        "metric": "training samples/sec per layer", "value": value, "unit": "samples/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong" if wl == "stl10_dp_f32" else "weak", "vs_baseline": None,
        "dtype": "f32" if np_dtype == np.float32 else "f64", "data": "synthetic",
        "config": workload_config(wl, p, batch, world, mask, args.dp_path),
        "contraction": "tcgen05 3xTF32" if tensor_path else ("FFMA" if np_dtype == np.float32 else "DFMA"),
        "dp_step": ("row-sharded layer over peer-mapped memory (inputs exchanged by columns, supports summed)"
                    if shard_step else "all-reduce, replicated update") if dp_path else None,
        "roofline": roofline, "step_roofline": step_roofline, "dp_large_batch": dp_large,
        "dp_checks": dp_checks, "other_configs": other, "cpu_baseline": cpu, "e2e": e2e,
        "gpu_launches": launches, "clocks": clocks,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse_args()
    wl = args.workload or "stl10_f32"
    p = synthetic.layer_params(wl)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    batch = p["batch"] // world if wl == "stl10_dp_f32" else p["batch"]
    if args.impl == "reference":
        run_reference(args, wl, p, batch)
    else:
        run_b200(args, wl, p, batch)


if __name__ == "__main__":
    main()
