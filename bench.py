"""Benchmark of the fused batch-norm + activation path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload (one "step"): training-mode batch norm fused with PReLU then ELU, forward and backward, on
x[256, 256, 28, 28] fp32 PER GPU (weak scaling: the global batch is 256*N entries, sharded on the
batch axis; training batch norm all-reduces 2*C floats forward and 2*C floats backward over NCCL).
Inputs are seeded synthetic tensors (x ~ N(0.5, 2), dy ~ N(0, 1), gamma ~ U(0.5, 1.5),
beta ~ N(0, 0.1), slope ~ U(0, 0.3)); each tensor is 205 MB, larger than the 126 MB L2, so timed
iterations stream from HBM without an explicit flush.

Metric: achieved HBM GB/s over all GPUs, counting ALGORITHMIC bytes only: forward 8 B/element (read
x, write y) + backward 12 B/element (read x, dy, write dx) = 20 B/element/step.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_PER_GPU, C, H, W = 256, 256, 28, 28
EPS = 1e-5
BYTES_PER_ELEM_FWD = 8
BYTES_PER_ELEM_BWD = 12
METRIC = "fused BN+activation fwd/bwd achieved HBM GB/s"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/ (same shape:
# bn_train_chain_kernel_x256x256x28x28.md, bn_bwd_apply_kernel_cfg2_..., bn_bwd_stats_kernel_cfg2_..., bn_stats_..., bn_apply_channel_...)
NCU_TRAFFIC_BYTES = {"forward": 364772352, "backward": 625849344, "bwd_apply": 580634624, "bwd_stats": 417700000, "stats": 210000000,
                     "apply": 363633664}
WORKLOAD = "bn_train+prelu+elu fwd+bwd, x[256,256,28,28] fp32 per GPU"
KINK = 1e-5   # |bn output| below which an element is at PReLU's kink for the parity checks of dx


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
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
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        for line in self.lines:
            f = [t.strip() for t in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                smax = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        # under load = the upper half of the samples (idle samples before/after the region read low or max)
        med = sm[len(sm) // 2] if sm else None
        return {"sm_mhz": med, "sm_max_mhz": smax, "reasons": sorted(reasons), "samples": len(sm)}


def elements_per_gpu():
    return N_PER_GPU * C * H * W


def cpu_step_seconds(n_sample, threads_hint=None, reps=2):
    """One unfused, layer-by-layer training step of the same chain on the host cores, the way the
    reference schedules its plain backend: BN(batch stats) -> PReLU -> ELU, then ELU', PReLU' (data and
    weights), BN'. PReLU and ELU run nnForge's own plain sources when the reference-backed library was
    built; training batch norm has no CPU implementation in the reference, so that layer always runs
    our C restatement. Returns (seconds per step, threads, description)."""
    import numpy as np
    from oracle import Oracle, Reference
    orc = Oracle(parallel=True)
    ref = Reference(parallel=True)
    g = np.random.Generator(np.random.PCG64(1002))
    shape = (n_sample, C, H, W)
    x = (g.standard_normal(shape, dtype=np.float32) * 2 + np.float32(0.5)).astype(np.float32)
    dy = g.standard_normal(shape, dtype=np.float32)
    gamma = (g.random(C, dtype=np.float32) + np.float32(0.5)).astype(np.float32)
    beta = (g.standard_normal(C, dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    slope = (g.random(C, dtype=np.float32) * np.float32(0.3)).astype(np.float32)
    m = n_sample * H * W
    best = None
    for _ in range(reps):
        t = 0.0
        t0 = time.perf_counter()
        s, q = orc.bn_train_sums(x, f32=True)
        saved = orc.bn_train_finalize(s, q, m, EPS)
        u = orc.bn_train_apply(x, gamma, beta, saved)
        t += time.perf_counter() - t0
        if ref.available:
            v, dt1 = ref.prelu_fwd(u, slope)
            y, dt2 = ref.elu_fwd(v)
            dv, dt3 = ref.elu_bwd(dy, y)
            du, dt4 = ref.prelu_bwd_data(dv, u, slope)
            _, dt5 = ref.prelu_bwd_weights(dv, u)
            t += dt1 + dt2 + dt3 + dt4 + dt5
        else:
            t0 = time.perf_counter()
            v = orc.prelu_fwd(u, slope)
            y = orc.elu_fwd(v)
            dv = orc.elu_bwd(dy, y)
            du = orc.prelu_bwd_data(dv, u, slope)
            orc.prelu_bwd_weights(dv, u)
            t += time.perf_counter() - t0
        t0 = time.perf_counter()
        db, dg = orc.bn_train_bwd_sums(du, x, saved)
        orc.bn_train_bwd_apply(du, x, gamma, saved, db, dg, m)
        t += time.perf_counter() - t0
        best = t if best is None else min(best, t)
    kind = "port"  # the dominant layer (training batch norm) has no reference CPU code; see the description
    desc = ("%d of %d entries of the workload, unfused layer by layer (BN-train fwd/bwd: C restatement, no reference CPU code exists; "
            "PReLU/ELU fwd/bwd: %s), OpenMP on all host threads, best of %d"
            % (n_sample, N_PER_GPU, "nnForge plain sources" if ref.available else "C restatement", reps))
    return best, orc.threads, kind, desc


def make_config(world):
    """The `config` object of the JSON line: the same for the GPU arm and the reference arm at a given N."""
    return {"workload": WORKLOAD, "global_batch": N_PER_GPU * world, "parallelism": "dp%d" % world,
            "collective": "2 x sum of 2*C floats per step" if world > 1 else "none",
            "l2": "inputs larger than L2 (205 MB per tensor vs 126 MB), no flush needed",
            "bytes_per_element": {"forward": BYTES_PER_ELEM_FWD, "backward": BYTES_PER_ELEM_BWD}}


def use_all_host_threads():
    """torch.distributed.run exports OMP_NUM_THREADS=1 to its workers; the CPU arm is meant to use every core."""
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    os.environ["OMP_NUM_THREADS"] = str(cores)
    return cores


def run_reference(args):
    """The reference arm: the reference's CPU path for the same workload, timed on the host cores (rank 0 only; the
    other ranks leave at once). One step = the whole per-GPU batch of 256 entries, unfused, layer by layer."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    use_all_host_threads()
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    n_sample = N_PER_GPU
    warmup = max(args.warmup, 1)
    for _ in range(min(warmup, 3)):
        cpu_step_seconds(n_sample, reps=1)
    times = []
    budget_end = time.time() + 150.0          # the arm ends within a few minutes whatever the host
    for _ in range(max(1, args.steps)):
        sec, threads, kind, desc = cpu_step_seconds(n_sample, reps=1)
        times.append(sec)
        if time.time() > budget_end:
            break
    sec = sum(times) / len(times)
    elems = n_sample * C * H * W
    gbs = elems * (BYTES_PER_ELEM_FWD + BYTES_PER_ELEM_BWD) / sec / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": len(times), "warmup": warmup,
        "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": make_config(world),
        "note": "CPU path on rank 0's host cores; one step = one GPU's batch of %d entries (the CPU arm does not grow with N)" % n_sample,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": kind, "sample": desc},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_sweep(args):
    """Prints the per-configuration kernel table on stderr and one JSON line on stdout."""
    import torch
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    peak, peak_kind = measured_peaks()
    rows = collect_sweep(args, quick=False)
    print(json.dumps({"sweep": rows, "peak_GBps": peak, "peak_source": peak_kind}))


def collect_sweep(args, quick):
    """Per-configuration kernel table (all five benchmark configurations, single GPU): device time per
    launch by CUDA events, algorithmic GB/s and fraction of the measured copy bandwidth. Tensors smaller
    than L2 are rotated through enough buffers to exceed it and replayed from a CUDA graph, so that the
    figure is neither an L2 number nor a Python launch-overhead number. quick: only the rows of the five
    configurations themselves (what the benchmark line carries under "configs"), a few seconds in all."""
    import torch
    import nnforge_b200.capi as capi
    peak, peak_kind = measured_peaks()
    rows = []

    def bnp(c):
        return [torch.rand(c, device="cuda") + 0.5, torch.randn(c, device="cuda") * 0.1, torch.randn(c, device="cuda") * 0.1,
                1 / torch.sqrt(torch.rand(c, device="cuda") * 1.5 + 0.5)]

    def timeit(fn, nbuf, reps=20):
        for i in range(max(3, nbuf)):
            fn(i % nbuf)
        torch.cuda.synchronize()
        graph = None
        if nbuf > 1:  # small tensors: replay `reps` launches from a graph, rotating buffers
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(reps):
                        fn(i % nbuf)
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        if graph is not None:
            graph.replay()
        else:
            for i in range(reps):
                fn(i % nbuf)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    def nbufs(bytes_per_set):
        return max(1, min(24, int(2 * 126e6 / bytes_per_set) + 1)) if bytes_per_set < 200e6 else 1

    def report(config, name, ms, alg_bytes, note=""):
        gbs = alg_bytes / (ms * 1e-3) / 1e9
        rows.append({"config": config, "kernel": name, "us": ms * 1e3, "GBps": gbs, "frac_of_peak": gbs / peak, "algorithmic_bytes": alg_bytes, "note": note})
        print("cfg%-2s %-58s %9.1f us %8.1f GB/s %6.1f%% of %s peak %s" % (config, name, ms * 1e3, gbs, 100 * gbs / peak, peak_kind, note), file=sys.stderr, flush=True)

    # config 0: inference BN + ReLU
    shape = (64, 64, 32, 32)
    e = 64 * 64 * 32 * 32
    nb = nbufs(8 * e)
    xs = [torch.randn(shape, device="cuda") for _ in range(nb)]
    ys = [torch.empty(shape, device="cuda") for _ in range(nb)]
    bn = bnp(64)
    relu = [capi.relu(0.0)]
    report(0, "bn_infer+relu x[64,64,32,32]", timeit(lambda i: capi.bn_infer_act(ys[i], xs[i], bn=bn, acts=relu), nb), 8 * e, "%d rotating buffers, graph replay" % nb)
    if not quick:
        # what a plain copy of a tensor this small reaches under the same procedure: the launch's ramp-up and tail are a fixed
        # few microseconds, so 16.8 MB in and out cannot reach the figure of a 200 MB copy
        report(0, "reference point: torch copy_ of x[64,64,32,32]", timeit(lambda i: ys[i].copy_(xs[i]), nb), 8 * e, "%d rotating buffers, graph replay" % nb)
    del xs, ys
    # config 1: channel softmax
    for shape in [(256, 1000, 1, 1), (32, 21, 128, 128)]:
        e = shape[0] * shape[1] * shape[2] * shape[3]
        nb = nbufs(8 * e)
        xs = [torch.randn(shape, device="cuda") * 3 for _ in range(nb)]
        ys = [torch.empty(shape, device="cuda") for _ in range(nb)]
        dx = torch.empty(shape, device="cuda")
        report(1, "softmax fwd %s" % (list(shape),), timeit(lambda i: capi.softmax_fwd(ys[i], xs[i]), nb), 8 * e, "%d rotating buffers, graph replay" % nb)
        report(1, "softmax bwd %s" % (list(shape),), timeit(lambda i: capi.softmax_bwd(dx, xs[i], ys[i]), nb), 12 * e, "%d rotating buffers, graph replay" % nb)
        if not quick:
            report(1, "reference point: torch copy_ of %s" % (list(shape),), timeit(lambda i: ys[i].copy_(xs[i]), nb), 8 * e, "%d rotating buffers, graph replay" % nb)
        del xs, ys, dx
    # beyond the five configurations: softmax fused with the loss behind it, at sizes above L2
    for shape in ([] if quick else [(65536, 1000, 1, 1), (512, 21, 128, 128)]):
        e = shape[0] * shape[1] * shape[2] * shape[3]
        logits = torch.randn(shape, device="cuda") * 3
        labels = torch.randint(0, shape[1], (shape[0],) + shape[2:], device="cuda")
        targets = torch.zeros(shape, device="cuda").scatter_(1, labels.unsqueeze(1), 1.0)
        probs, dl = torch.empty_like(logits), torch.empty_like(logits)
        err = torch.empty((shape[0], 1) + shape[2:], device="cuda")
        report(1, "softmax+nll fwd fused %s" % (list(shape),), timeit(lambda i: capi.softmax_nll_fwd(probs, err, logits, targets), 1), 12 * e)
        report(1, "softmax+nll bwd fused %s" % (list(shape),), timeit(lambda i: capi.softmax_nll_bwd(dl, probs, targets), 1), 12 * e)
        del logits, labels, targets, probs, dl, err
    # config 2: training BN + PReLU + ELU (the default benchmark's kernels, timed one by one)
    shape = (N_PER_GPU, C, H, W)
    e = elements_per_gpu()
    x = torch.randn(shape, device="cuda") * 2 + 0.5
    dy = torch.randn(shape, device="cuda")
    y, dx = torch.empty_like(x), torch.empty_like(x)
    g, b, sl = torch.rand(C, device="cuda") + 0.5, torch.randn(C, device="cuda") * 0.1, torch.rand(C, device="cuda") * 0.3
    ws = torch.empty(capi.bn_train_workspace_bytes(N_PER_GPU, C, H * W), dtype=torch.uint8, device="cuda")
    sums, saved, bs = torch.empty(2 * C, device="cuda"), torch.empty(2 * C, device="cuda"), torch.empty(3 * C, device="cuda")
    acts = [capi.prelu(sl), capi.elu()]
    m = N_PER_GPU * H * W
    report(2, "bn_train fwd, one launch (statistics + apply items)", timeit(lambda i: capi.bn_train_fwd(y, saved, sums, x, g, b, EPS, acts, workspace=ws), 1), 8 * e)
    report(2, "bn_train bwd, one launch (statistics + apply items)", timeit(lambda i: capi.bn_train_bwd(dx, bs, dy, x, g, b, saved, acts, workspace=ws), 1), 12 * e)
    if not quick:
        report(2, "bn_train stats", timeit(lambda i: capi.bn_train_stats(sums, x, ws), 1), 4 * e)
        report(2, "bn_train apply+prelu+elu", timeit(lambda i: capi.bn_train_apply_act(y, saved, x, g, b, sums, m, EPS, acts), 1), 8 * e)
        report(2, "bn_train bwd stats", timeit(lambda i: capi.bn_train_bwd_stats(bs, dy, x, g, b, saved, acts, ws), 1), 8 * e)
        report(2, "bn_train bwd apply", timeit(lambda i: capi.bn_train_bwd_apply(dx, dy, x, g, b, saved, bs, bs, m, acts), 1), 12 * e)
        report(2, "reference point: torch copy_ of one tensor", timeit(lambda i: y.copy_(x), 1), 8 * e)
    del x, dy, y, dx
    # config 3: BN -> add -> ReLU -> max-pool 3x3/2, forward and backward, four stages
    for c, hw in [(64, 56), (128, 28), (256, 14), (512, 7)]:
        shape = (256, c, hw, hw)
        e = 256 * c * hw * hw
        p = capi.pool((3, 3), (2, 2))
        oh, ow = capi.pool_out_shape(hw, hw, p)
        rho = oh * ow / float(hw * hw)
        x, r, z = [torch.randn(shape, device="cuda") for _ in range(3)]
        pooled = torch.empty((256, c, oh, ow), device="cuda")
        idx = torch.empty((256, c, oh, ow), device="cuda", dtype=torch.int32)
        bn = bnp(c)
        dpo, dx, dr = torch.randn_like(pooled), torch.empty_like(x), torch.empty_like(x)
        nb = 1
        report(3, "bn+add+relu+maxpool fwd C=%d %dx%d" % (c, hw, hw), timeit(lambda i: capi.bn_add_relu_maxpool_fwd(z, pooled, idx, x, r, bn, 0.0, p), nb), (12 + 8 * rho) * e)
        report(3, "bn+add+relu+maxpool bwd C=%d %dx%d" % (c, hw, hw), timeit(lambda i: capi.bn_add_relu_maxpool_bwd(dx, dr, dpo, idx, z, bn[0], bn[3], 0.0, p), nb), (12 + 8 * rho) * e)
        if not quick and hw <= 14:
            # the ceiling for launches this short: two plain copies back to back move the same 16 bytes per element
            def two_copies(i):
                dx.copy_(x)
                dr.copy_(r)
            report(3, "reference point: two torch copy_ back to back C=%d %dx%d" % (c, hw, hw), timeit(two_copies, nb) , 16 * e, "two launches")
        del x, r, z, pooled, idx, dpo, dx, dr
    # beyond the five configurations: the tail of a residual network - BN -> add -> ReLU -> global average pooling
    for c, hw in ([] if quick else [(512, 7), (256, 14)]):
        shape = (1024, c, hw, hw)
        e = shape[0] * c * hw * hw
        x, r, z = [torch.randn(shape, device="cuda") for _ in range(3)]
        pooled = torch.empty((shape[0], c, 1, 1), device="cuda")
        bn = bnp(c)
        mult = 1.0 / (hw * hw)
        report(3, "bn+add+relu+global avgpool fwd N=1024 C=%d %dx%d" % (c, hw, hw),
               timeit(lambda i: capi.bn_add_relu_avgpool_fwd(z, pooled, x, r, bn, 0.0, (hw, hw), mult), 1), 12 * e)
        dpo = torch.randn_like(pooled)
        dx, dr = torch.empty_like(x), torch.empty_like(x)
        report(3, "bn+add+relu+global avgpool bwd N=1024 C=%d %dx%d" % (c, hw, hw),
               timeit(lambda i: capi.bn_add_relu_avgpool_bwd(dx, dr, dpo, z, bn[0], bn[3], 0.0, (hw, hw), mult), 1), 12 * e)
        del x, r, z, pooled, dpo, dx, dr
    # the stand-alone subsampling layers (no batch norm in front): max 3x3/2 and 2x2/2, average 2x2
    for c, hw, win in ([] if quick else [(64, 56, 3), (128, 28, 3), (128, 28, 2), (256, 14, 2)]):
        n = 1024
        shape = (n, c, hw, hw)
        e = n * c * hw * hw
        p = capi.pool((win, win), (2, 2))
        oh, ow = capi.pool_out_shape(hw, hw, p)
        rho = oh * ow / float(hw * hw)
        x = torch.randn(shape, device="cuda")
        pooled = torch.empty((n, c, oh, ow), device="cuda")
        idx = torch.empty((n, c, oh, ow), device="cuda", dtype=torch.int32)
        dpo, dx = torch.randn_like(pooled), torch.empty_like(x)
        report(3, "maxpool %dx%d/2 fwd N=%d C=%d %dx%d" % (win, win, n, c, hw, hw), timeit(lambda i: capi.maxpool_fwd(pooled, idx, x, p), 1), (4 + 8 * rho) * e)
        report(3, "maxpool %dx%d/2 bwd N=%d C=%d %dx%d" % (win, win, n, c, hw, hw), timeit(lambda i: capi.maxpool_bwd(dx, dpo, idx, p), 1), (4 + 8 * rho) * e)
        if win == 2:
            report(3, "avgpool 2x2 fwd N=%d C=%d %dx%d" % (n, c, hw, hw), timeit(lambda i: capi.avgpool_fwd(pooled, x, (2, 2), 0.25), 1), 5 * e)
            report(3, "avgpool 2x2 bwd N=%d C=%d %dx%d" % (n, c, hw, hw), timeit(lambda i: capi.avgpool_bwd(dx, dpo, (2, 2), 0.25), 1), 5 * e)
        del x, pooled, idx, dpo, dx
    # training batch norm + ReLU on the last stage's 7x7 planes (not whole float4s: the channel-group kernels)
    for n, c, hw in ([] if quick else [(1024, 512, 7), (256, 2048, 7)]):
        shape = (n, c, hw, hw)
        e = n * c * hw * hw
        x, dy = torch.randn(shape, device="cuda"), torch.randn(shape, device="cuda")
        y, dx = torch.empty_like(x), torch.empty_like(x)
        gamma, beta = torch.rand(c, device="cuda") + 0.5, torch.randn(c, device="cuda") * 0.1
        saved, sums, bsums = torch.empty(2 * c, device="cuda"), torch.empty(2 * c, device="cuda"), torch.empty(3 * c, device="cuda")
        ws = torch.empty(capi.bn_train_workspace_bytes(n, c, hw * hw), dtype=torch.uint8, device="cuda")
        acts = [capi.relu(0.0)]
        report(3, "bn_train+relu fwd N=%d C=%d %dx%d, one launch (channel-group items)" % (n, c, hw, hw),
               timeit(lambda i: capi.bn_train_fwd(y, saved, sums, x, gamma, beta, 1e-5, acts, workspace=ws), 1), 8 * e)
        report(3, "bn_train+relu bwd N=%d C=%d %dx%d, one launch (channel-group items)" % (n, c, hw, hw),
               timeit(lambda i: capi.bn_train_bwd(dx, bsums, dy, x, gamma, beta, saved, acts, workspace=ws), 1), 12 * e)
        del x, dy, y, dx
    # beyond the five configurations: inference BN + ReLU on planes that are not whole float4s (the channel-group kernel)
    for n, c, hw in ([] if quick else [(1024, 512, 7), (1024, 2048, 7)]):
        e = n * c * hw * hw
        x = torch.randn((n, c, hw, hw), device="cuda")
        y = torch.empty_like(x)
        bn = bnp(c)
        report(3, "bn_infer+relu N=%d C=%d %dx%d (channel groups)" % (n, c, hw, hw), timeit(lambda i: capi.bn_infer_act(y, x, bn=bn, acts=[capi.relu(0.0)]), 1), 8 * e)
        del x, y
    if not quick:
        # the layers either side of the path, each at a size well above L2 (rows "n": neighbours, not one of the five configurations)
        shape = (256, 256, 28, 28)
        e = 256 * 256 * 28 * 28
        x, dy = torch.randn(shape, device="cuda"), torch.randn(shape, device="cuda")
        y, dx = torch.empty_like(x), torch.empty_like(x)
        slope = torch.rand(256, device="cuda") * 0.3
        capi.act_fwd(y, x, capi.elu())
        report("n", "ELU backward (dy, y -> dx) x[256,256,28,28]", timeit(lambda i: capi.act_bwd(dx, dy, y, capi.elu()), 1), 12 * e)
        report("n", "PReLU backward, data (dy, x -> dx) x[256,256,28,28]", timeit(lambda i: capi.act_bwd(dx, dy, x, capi.prelu(slope)), 1), 12 * e)
        dslope = torch.empty(256, device="cuda")
        wsp = torch.empty(capi.lib.nnf_prelu_bwd_weights_workspace_bytes(256, 256, 784), dtype=torch.uint8, device="cuda")
        report("n", "PReLU backward, slopes (dy, x -> dslope) x[256,256,28,28]", timeit(lambda i: capi.prelu_bwd_weights(dslope, dy, x, workspace=wsp), 1), 8 * e)
        report("n", "add forward, two inputs x[256,256,28,28]", timeit(lambda i: capi.add_fwd(y, [x, dy]), 1), 12 * e)
        report("n", "add backward (dy * alpha -> dx) x[256,256,28,28]", timeit(lambda i: capi.add_bwd(dx, dy, alpha=0.5), 1), 8 * e)
        del x, dy, y, dx
        # channel softmax outside the shapes of configuration 1: many channels per pixel (tile kernel), rows that are not whole
        # float4s (scalar warp kernel), rows longer than a warp holds (CTA per row)
        for shape in [(16, 150, 128, 128), (65536, 1001, 1, 1), (8192, 32000, 1, 1)]:
            e = shape[0] * shape[1] * shape[2] * shape[3]
            x = torch.randn(shape, device="cuda")
            y, dy, dx = torch.empty_like(x), torch.randn(shape, device="cuda"), torch.empty_like(x)
            report("n", "softmax fwd %s" % (list(shape),), timeit(lambda i: capi.softmax_fwd(y, x), 1), 8 * e)
            report("n", "softmax bwd %s" % (list(shape),), timeit(lambda i: capi.softmax_bwd(dx, dy, y), 1), 12 * e)
            del x, y, dy, dx
        # top-n accuracy beside the loss (predictions and targets in, top_n + 1 values per row or pixel out)
        for shape in [(65536, 1000, 1, 1), (512, 21, 128, 128)]:
            e = shape[0] * shape[1] * shape[2] * shape[3]
            pr = torch.softmax(torch.randn(shape, device="cuda"), dim=1)
            tg = torch.zeros(shape, device="cuda")
            tg.scatter_(1, torch.randint(0, shape[1], (shape[0], 1) + shape[2:], device="cuda"), 1.0)
            out = torch.empty((shape[0], 2) + shape[2:], device="cuda")
            report("n", "top-1 accuracy %s" % (list(shape),), timeit(lambda i: capi.accuracy_fwd(out, pr, tg, None, 1), 1), 8 * e + 8 * (e // shape[1]))
            del pr, tg, out
        # training statistics and apply through the separate channel-group kernels (what the single launch replaces at 7x7)
        n, c, hw = 1024, 512, 7
        shape = (n, c, hw, hw)
        e = n * c * hw * hw
        x, dy = torch.randn(shape, device="cuda"), torch.randn(shape, device="cuda")
        y, dx = torch.empty_like(x), torch.empty_like(x)
        gamma, beta = torch.rand(c, device="cuda") + 0.5, torch.randn(c, device="cuda") * 0.1
        saved, sums, bsums = torch.empty(2 * c, device="cuda"), torch.empty(2 * c, device="cuda"), torch.empty(3 * c, device="cuda")
        ws = torch.empty(capi.bn_train_workspace_bytes(n, c, hw * hw), dtype=torch.uint8, device="cuda")
        acts = [capi.relu(0.0)]
        report("n", "bn_train stats, channel groups N=1024 C=512 7x7", timeit(lambda i: capi.bn_train_stats(sums, x, ws), 1), 4 * e)
        report("n", "bn_train apply+relu, channel groups N=1024 C=512 7x7", timeit(lambda i: capi.bn_train_apply_act(y, saved, x, gamma, beta, sums, n * hw * hw, 1e-5, acts), 1), 8 * e)
        report("n", "bn_train bwd stats, channel groups N=1024 C=512 7x7", timeit(lambda i: capi.bn_train_bwd_stats(bsums, dy, x, gamma, beta, saved, acts, ws), 1), 8 * e)
        report("n", "bn_train bwd apply, channel groups N=1024 C=512 7x7", timeit(lambda i: capi.bn_train_bwd_apply(dx, dy, x, gamma, beta, saved, bsums, bsums, n * hw * hw, acts), 1), 12 * e)
        # running-statistics calibration pass over the same tensor (one read)
        acc = capi.bn_calibrate_accumulator(c)
        mean, invsigma = torch.randn(c, device="cuda") * 0.1, torch.rand(c, device="cuda") + 0.5
        cws = torch.empty(capi.lib.nnf_bn_calibrate_workspace_bytes(c), dtype=torch.uint8, device="cuda")
        report("n", "bn calibration statistics N=1024 C=512 7x7", timeit(lambda i: capi.bn_calibrate_accumulate(acc, x, mean, invsigma, workspace=cws), 1), 4 * e)
        del x, dy, y, dx
        # optimiser step: one launch over a table of weight chunks (vanilla momentum: data, gradient, previous update in; data, previous
        # update and the cleared gradient out)
        parts = []
        for k in range(16):
            m = 4 * 1024 * 1024
            parts.append({"data": torch.randn(m, device="cuda"), "gradient": torch.randn(m, device="cuda"), "prev_upd": torch.zeros(m, device="cuda"),
                          "update_accum": torch.zeros(1, dtype=torch.float64, device="cuda"), "learning_rate": 0.01, "weight_decay": 1e-4})
        w = 16 * 4 * 1024 * 1024
        report("n", "optimiser step, vanilla momentum, 16 chunks of 4 M weights", timeit(lambda i: capi.apply_gradient(parts, momentum_type=capi.MOMENTUM_VANILLA, normalizer=256.0), 1), 24 * w)
        del parts
    # config 4: inference BN + TanH / Sigmoid bandwidth sweep
    sizes = [128, 1024] if quick else [128, 1024, 4096] + ([8192] if args.sweep_full else [])
    for n in sizes:
        shape = (n, 128, 64, 64)
        e = n * 128 * 64 * 64
        x = torch.randn(shape, device="cuda") * 1.5
        y = torch.empty_like(x)
        bn = bnp(128)
        for name, act in (("tanh", capi.tanh()), ("sigmoid", capi.sigmoid())):
            report(4, "bn_infer+%s N=%d (%.2f GiB in)" % (name, n, e * 4 / 2.0 ** 30), timeit(lambda i: capi.bn_infer_act(y, x, bn=bn, acts=[act]), 1, reps=10), 8 * e)
        del x, y
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=8)
    ap.add_argument("--no-configs", action="store_true", help="leave out the table of the other four configurations")
    ap.add_argument("--tune", action="append", default=[], metavar="KNOB=VALUE", help="a knob of the launch plans (nnf_set_tuning), for experiments")
    ap.add_argument("--sweep", action="store_true", help="time every kernel family at all five configurations (single GPU) instead of the benchmark step")
    ap.add_argument("--sweep-full", action="store_true", help="with --sweep: include the 16 GiB case of configuration 4")
    ap.add_argument("--ceilings", action="store_true", help="run the stand-alone memory-ceiling program (copy, read-only, L2 re-reads, the two-read launch "
                    "without arithmetic) and print its table")
    args = ap.parse_args()
    if args.ceilings:
        import subprocess
        exe = os.path.join(os.path.dirname(os.path.abspath(__file__)), "nnforge_b200", "nnf_ceilings")
        if not os.path.exists(exe):
            sys.exit("nnforge_b200/nnf_ceilings is missing: build it with `python -m nnforge_b200.build`")
        peak, kind = measured_peaks()
        print("rates against the %s copy bandwidth, %.1f GB/s" % (kind, peak), flush=True)
        sys.exit(subprocess.call([exe, "%.1f" % peak]))
    if args.sweep:
        run_sweep(args)
        return
    if args.impl == "reference":
        run_reference(args)
        return

    # Libraries (NCCL prints its version banner) write to file descriptor 1; keep the real stdout for the one
    # JSON line and send everything else to stderr.
    sys.stdout.flush()
    result_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    import torch
    import nnforge_b200.capi as capi  # raises if the CUDA library is missing: there is no fallback

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    warmup = max(args.warmup, 3)
    for item in args.tune:
        knob, value = item.split("=")
        capi.set_tuning(knob, int(value))

    gen = torch.Generator(device="cuda")
    gen.manual_seed(1002 + rank)
    shape = (N_PER_GPU, C, H, W)
    x = torch.randn(shape, device="cuda", generator=gen) * 2 + 0.5
    dy = torch.randn(shape, device="cuda", generator=gen)
    pgen = torch.Generator(device="cuda")
    pgen.manual_seed(1002)
    gamma = torch.rand(C, device="cuda", generator=pgen) + 0.5
    beta = torch.randn(C, device="cuda", generator=pgen) * 0.1
    slope = torch.rand(C, device="cuda", generator=pgen) * 0.3
    y, dx = torch.empty_like(x), torch.empty_like(x)
    hw = H * W
    m_total = float(N_PER_GPU * world * hw)
    ws = torch.empty(capi.bn_train_workspace_bytes(N_PER_GPU, C, hw), dtype=torch.uint8, device="cuda")
    sums, saved = torch.empty(2 * C, device="cuda"), torch.empty(2 * C, device="cuda")
    bsums, gsums = torch.empty(3 * C, device="cuda"), torch.empty(2 * C, device="cuda")
    grads = [torch.zeros(C, device="cuda") for _ in range(3)]
    acts = [capi.prelu(slope), capi.elu()]
    single = dist is None
    # kernels of ours per step: single GPU = 1 forward + 1 backward launch (each holds the statistics and the
    # apply work items); sharded = 2 + 1 + 2 + 1 with the exchange after each statistics step
    launches_per_step = 2 if single else 6  # + 2 x 2 small exchange kernels when the peer-memory exchange is used
    in_launch = (not single) and os.environ.get("NNF_EXCHANGE", "launch") == "launch"
    if in_launch:
        launches_per_step = 2
    phases = ("forward", "backward") if (single or in_launch) else ("stats", "apply", "bwd_stats", "bwd_apply")

    from nnforge_b200.sharded import ShardedBatchNormAct
    current = {"ev": None}
    order = {"start": 0, "stats": 1, "allreduce_fwd": 2, "apply": 3, "bwd_stats": 4, "allreduce_bwd": 5, "bwd_apply": 6}

    # One launch per direction: an event record between two launches costs about 2.5 us of device time (the step ran 229 us
    # with no marks inside it, 239 us with four, 249 us with seven), so only every fourth step of the timed region is marked,
    # at the start of its forward launch, between its two launches and at its end; the launches' durations are averages over
    # the marked steps. The forms with several kernels per direction mark every phase of every step.
    lean = single   # set again below, once it is known which exchange runs

    def on_phase(name):
        if current["ev"] is not None and (not lean or name in ("start", "bwd_stats", "bwd_apply")):
            current["ev"][order[name]].record()

    exchange, exchange_name = None, "none"
    if not single:
        from nnforge_b200.sharded import NcclExchange, PeerExchange
        exchange, exchange_name = NcclExchange(), "NCCL all-reduce"
        mode = os.environ.get("NNF_EXCHANGE", "launch")
        if mode in ("peer", "fused", "launch"):
            try:
                if mode == "launch":
                    from nnforge_b200.sharded import InLaunchExchange
                    exchange = InLaunchExchange(capi, C, torch.device("cuda", local))
                    exchange_name = "per-channel peer-memory stores and waits inside the one launch per direction (no NCCL call)"
                elif mode == "fused":
                    from nnforge_b200.sharded import FusedPeerExchange
                    exchange = FusedPeerExchange(capi, 2 * C, torch.device("cuda", local))
                    exchange_name = "peer-memory stores from the reducing kernel, summed in the consuming kernel's prologue (no NCCL call)"
                else:
                    exchange = PeerExchange(capi, 2 * C, torch.device("cuda", local))
                    exchange_name = "peer-memory stores + local sum (nnf_peer_exchange_sum)"
            except Exception as e:  # no symmetric memory on this machine: NCCL does the same sum
                print("peer exchange unavailable (%s); using NCCL" % (e,), file=sys.stderr)
    lean = single or getattr(exchange, "in_launch", False)
    layer = ShardedBatchNormAct(capi, C, EPS, acts, "cuda", on_phase=on_phase, exchange=exchange)
    grad_map = {"gamma": grads[0], "beta": grads[1], "slope": grads[2]}

    def step(ev=None):
        current["ev"] = ev
        if single:
            # one GPU: the single-GPU entry points (one launch per direction)
            on_phase("start")
            capi.bn_train_fwd(y, saved, sums, x, gamma, beta, EPS, acts, workspace=ws)
            on_phase("stats")
            on_phase("bwd_stats")
            capi.bn_train_bwd(dx, bsums, dy, x, gamma, beta, saved, acts, grad_gamma=grads[0], grad_beta=grads[1], grad_slope=grads[2], workspace=ws)
            on_phase("bwd_apply")
        else:
            layer.forward(y, x, gamma, beta)
            layer.backward(dx, dy, x, gamma, beta, grads=grad_map)
        current["ev"] = None

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(args.steps)]
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    host_t0 = time.perf_counter()
    # (not the first steps after the pause in front of the timed region: the clocks are still coming up)
    marked = [k for k in range(args.steps) if not lean or args.steps <= 4 or k % 4 == 2]
    for k in range(args.steps):
        step(evs[k] if k in marked else None)
    host_enqueue_us = (time.perf_counter() - host_t0) * 1e6 / args.steps   # how long the host took to enqueue a step
    t_end.record()
    barrier()
    ms_total = t_start.elapsed_time(t_end)
    if rank == 0:
        time.sleep(0.2)
        clocks = sampler.stop()
    if dist is not None:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    elems = elements_per_gpu()
    bytes_step_all = elems * (BYTES_PER_ELEM_FWD + BYTES_PER_ELEM_BWD) * world
    value = bytes_step_all / (ms_step * 1e-3) / 1e9

    # per-kernel durations from the events recorded inside the timed region (this rank)
    if in_launch and not getattr(exchange, "in_launch", False):
        in_launch = False  # symmetric memory was not available: the NCCL sequence ran
        launches_per_step = 6
        phases = ("stats", "apply", "bwd_stats", "bwd_apply")
    if lean:
        idx = None
        alg_bytes = {"forward": 8 * elems, "backward": 12 * elems}
        names = {"forward": "bn_train_chain_kernel<forward> (x in, y out; statistics and apply items in one launch)",
                 "backward": "bn_train_chain_kernel<backward> (x, dy in, dx out; statistics and apply items in one launch)"}
    else:
        idx = {"stats": (0, 1), "apply": (2, 3), "bwd_stats": (3, 4), "bwd_apply": (5, 6)}
        alg_bytes = {"stats": 4 * elems, "apply": 8 * elems, "bwd_stats": 8 * elems, "bwd_apply": 12 * elems}
        names = {"stats": "bn_stats_kernel (x in)", "apply": "bn_act_kernel (x in, y out)", "bwd_stats": "bn_bwd_stats_kernel (x, dy in)",
                 "bwd_apply": "bn_bwd_apply_kernel (x, dy in, dx out)"}
    evs = [evs[k] for k in marked]
    if idx is None:
        # marks: [0] before the forward launch, [4] before the backward launch, [6] behind it
        kernel_ms = {"forward": sum(e[0].elapsed_time(e[4]) for e in evs) / len(evs),
                     "backward": sum(e[4].elapsed_time(e[6]) for e in evs) / len(evs)}
    else:
        kernel_ms = {name: sum(e[a].elapsed_time(e[b]) for e in evs) / len(evs) for name, (a, b) in idx.items()}
    peak, peak_kind = measured_peaks()
    dominant = max(kernel_ms, key=kernel_ms.get)
    achieved = alg_bytes[dominant] / (kernel_ms[dominant] * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": names[dominant], "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": peak_kind + " copy bandwidth (MEASURED_PEAKS.json hbm_gbs)", "traffic": NCU_TRAFFIC_BYTES.get(dominant),
                "algorithmic_bytes_per_launch": alg_bytes[dominant],
                "kernels": {k: {"ms": kernel_ms[k], "algorithmic_GBps": alg_bytes[k] / (kernel_ms[k] * 1e-3) / 1e9,
                                "frac_of_peak": alg_bytes[k] / (kernel_ms[k] * 1e-3) / 1e9 / peak} for k in phases},
                "step_frac_of_peak": (value / world) / peak}

    # ---- checks, outside the timed region: nothing above is a number unless these hold ------------------------
    checks = []

    def note(name, ok, **detail):
        checks.append(dict({"check": name, "ok": bool(ok)}, **detail))

    def worst(got, want, rtol=1e-5, atol=1e-6, skip=None):
        """max over elements of |got - want| / (atol + rtol |want|): <= 1 is inside the tolerance"""
        ratio = (got - want).abs() / (atol + rtol * want.abs())
        if skip is not None:
            ratio = ratio.masked_fill(skip, 0.0)
        return float(ratio.max().item())

    def exact_step():
        """The step in float64 (torch on the GPU; per-channel sums all-reduced in float64 over the ranks)."""
        m = float(N_PER_GPU * world * hw)
        xd = x.double()
        s1, s2 = xd.sum(dim=(0, 2, 3)), (xd * xd).sum(dim=(0, 2, 3))
        if dist is not None:
            dist.all_reduce(s1)
            dist.all_reduce(s2)
        mean = s1 / m
        inv = 1.0 / torch.sqrt(s2 / m - mean * mean + EPS)
        xh = (xd - mean[None, :, None, None]) * inv[None, :, None, None]
        del xd
        u = xh * gamma.double()[None, :, None, None] + beta.double()[None, :, None, None]
        a = slope.double()[None, :, None, None]
        t1 = torch.where(u >= 0, u, u * a)
        yw = torch.where(t1 >= 0, t1, torch.expm1(t1))
        du = dy.double() * torch.where(t1 >= 0, torch.ones_like(t1), yw + 1.0) * torch.where(u >= 0, torch.ones_like(u), a.expand_as(u))
        del u, t1
        sb, sg = du.sum(dim=(0, 2, 3)), (du * xh).sum(dim=(0, 2, 3))
        if dist is not None:
            dist.all_reduce(sb)
            dist.all_reduce(sg)
        dxw = (gamma.double() * inv)[None, :, None, None] * ((du - sb[None, :, None, None] / m) - xh * sg[None, :, None, None] / m)
        # PReLU's derivative jumps at u = 0 (from the slope to 1): an element whose u is within rounding of 0 may fall on either
        # side in fp32, and two correct implementations then differ there by |dy| * (1 - slope) * gamma * invstd. Such elements
        # (a few hundred of 51 million) are left out of the comparisons of dx, and counted.
        kink = (xh * gamma.double()[None, :, None, None] + beta.double()[None, :, None, None]).abs() < KINK
        return yw, dxw, kink

    err_word = capi.fused_error_check()
    timed_out = None
    if not single:
        from nnforge_b200.sharded import ExchangeTimeout
        try:
            layer.check(block=True)
        except ExchangeTimeout as e:
            timed_out = str(e)
    note("no bounded wait ran out in the warm-up and timed steps", err_word == 0 and timed_out is None, error_word=err_word, report=timed_out)
    waits = None
    if not single and getattr(exchange, "in_launch", False):
        # how long the items of one step's two launches waited (for this GPU's statistics and for the other ranks'), per rank
        step()
        torch.cuda.synchronize()
        total_ns, longest_ns = layer.last_wait_ns()
        layer.check(block=True)
        t = torch.tensor([float(total_ns), float(longest_ns)], device="cuda")
        gathered = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(gathered, t)
        waits = {"per_rank_item_wait_us_summed": [round(float(g[0]) / 1e3, 1) for g in gathered],
                 "per_rank_longest_wait_us": [round(float(g[1]) / 1e3, 1) for g in gathered]}
    step()
    torch.cuda.synchronize()
    y_run, dx_run, saved_run = y.clone(), dx.clone(), (saved if single else layer.saved).clone()
    yw, dxw, kink = exact_step()
    kinks = int(kink.sum().item())
    wy, wdx = worst(y_run, yw, atol=2e-6), worst(dx_run, dxw, atol=5e-6, skip=kink)
    if dist is not None:
        t = torch.tensor([wy, wdx], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        wy, wdx = float(t[0].item()), float(t[1].item())
    note("the timed path against a float64 evaluation of the step with all-reduced sums (1e-5 relative + 2e-6 / 5e-6 absolute: the fp32 "
         "chain itself is that far from it where du and dx cancel), worst rank", wy <= 1.0 and wdx <= 1.0 and kinks <= 2e-5 * elements_per_gpu(), y=wy, dx=wdx,
         elements_left_out_at_the_prelu_kink=kinks, kink_halfwidth=KINK)
    del yw
    y2, dx2 = torch.empty_like(x), torch.empty_like(x)
    if single:
        # (a) another path of this library: statistics kernel, apply kernel, backward statistics kernel, backward apply kernel
        saved2, sums2, bsums2 = torch.empty(2 * C, device="cuda"), torch.empty(2 * C, device="cuda"), torch.empty(3 * C, device="cuda")
        capi.bn_train_stats(sums2, x, ws)
        capi.bn_train_apply_act(y2, saved2, x, gamma, beta, sums2, float(N_PER_GPU * hw), EPS, acts)
        capi.bn_train_bwd_stats(bsums2, dy, x, gamma, beta, saved2, acts, ws)
        capi.bn_train_bwd_apply(dx2, dy, x, gamma, beta, saved2, bsums2, bsums2, float(N_PER_GPU * hw), acts)
        torch.cuda.synchronize()
        note("single launch against the two-kernel form of this library (1e-5 relative + 1e-6 absolute)",
             max(worst(saved_run, saved2), worst(y_run, y2), worst(dx_run, dx2, skip=kink)) <= 1.0,
             saved=worst(saved_run, saved2), y=worst(y_run, y2), dx=worst(dx_run, dx2, skip=kink))
        # (b) the reference's own arithmetic for this layer: cuDNN's spatial batch norm (the two calls of
        # nnforge/cuda/batch_norm_layer_updater_cuda.cu:89,145), followed by torch's PReLU and ELU, forward and autograd backward
        if torch.backends.cudnn.is_available():
            xr = x.detach().clone().requires_grad_(True)
            u = torch.nn.functional.batch_norm(xr, None, None, gamma, beta, training=True, momentum=0.1, eps=EPS)
            yr = torch.nn.functional.elu(torch.nn.functional.prelu(u, slope))
            yr.backward(dy)
            torch.cuda.synchronize()
            wy = worst(y_run, yr.detach(), atol=2e-6)
            wdx = worst(dx_run, xr.grad, atol=5e-6, skip=kink)
            note("single launch against cuDNN batch norm + torch PReLU, ELU (1e-5 relative + 2e-6 / 5e-6 absolute: du and dx cancel)",
                 wy <= 1.0 and wdx <= 1.0, y=wy, dx=wdx)
            del xr, u, yr
    else:
        from nnforge_b200.sharded import NcclExchange
        other = ShardedBatchNormAct(capi, C, EPS, acts, "cuda", exchange=NcclExchange())
        other.forward(y2, x, gamma, beta)
        other.backward(dx2, dy, x, gamma, beta)
        torch.cuda.synchronize()
        w = (worst(saved_run, other.saved), worst(y_run, y2), worst(dx_run, dx2, atol=5e-6, skip=kink), worst(dx2, dxw, atol=5e-6, skip=kink))
        t = torch.tensor([max(w[:3])], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        note("%s against statistics kernel + NCCL all-reduce + apply kernel on the same shards (1e-5 relative + 1e-6 absolute; dx 5e-6), worst rank" % exchange_name,
             float(t.item()) <= 1.0, worst=float(t.item()), this_rank={"saved": w[0], "y": w[1], "dx": w[2], "dx of the NCCL form against float64": w[3]})
        gathered = [torch.empty_like(saved_run) for _ in range(world)]
        dist.all_gather(gathered, saved_run)
        same = all(bool((g.view(torch.int32) == gathered[0].view(torch.int32)).all().item()) for g in gathered)
        note("saved {mean, invstd} bit-identical on all ranks", same)
        err_word = capi.fused_error_check()
        note("no bounded wait ran out in the checked steps", err_word == 0, error_word=err_word)
    del y2, dx2, dxw, kink
    parity = {"ok": all(c["ok"] for c in checks), "checks": checks}
    if dist is not None:
        ok = torch.tensor([1 if parity["ok"] else 0], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        parity["ok"] = bool(ok.item())       # every rank's checks
        parity["ranks"] = world

    # End to end through the C ABI with HOST buffers: every step copies its x and dy from pinned host memory and
    # its y and dx back, all inside the timed region. The copies of one step overlap the kernels and the opposite
    # copies of its neighbours (three streams, two sets of device buffers): host->device of x, forward, device->host
    # of y while dy comes in, backward, device->host of dx while the next step's x comes in.
    # The calls of this leg are those of an nnForge scheduler: the schema of the benchmarked chain is planned, the C++ factory
    # makes the fused head (and the two no-op follower objects), and every step enqueues the head's forward and
    # backward_data_and_weights actions with the buffers its size queries asked for. With several GPUs each rank's head owns
    # a mailbox in symmetric memory of its own (published with the peers' mapped addresses before the objects are created).
    from nnforge_b200 import host as nnf_host
    objects = None
    peers = None
    if not single and in_launch and getattr(exchange, "in_launch", False):
        from nnforge_b200.sharded import InLaunchExchange
        object_mailboxes = InLaunchExchange(capi, C, torch.device("cuda", local))
        peers = nnf_host.PeerDirectory()
        for r, address in enumerate(object_mailboxes.ptrs):
            peers.publish("bn", r, address)
    if single or peers is not None:
        net = nnf_host.Net("bn BatchNorm x eps=%r\nprelu PReLU bn\nelu ELU prelu\n" % EPS, {"x": (C, W, H)}, training=True,
                           device_pos=rank, device_count=world, peers=peers)
        head = net.objects[0]
        assert (head.role, head.kind, head.data, head.outputs) == ("head", "bn_train_act", ["bn", "prelu"], ["elu"])
        objects = {
            "net": net, "head": head, "followers": net.objects[1:],
            "data": [gamma, beta, torch.zeros(C, device="cuda"), torch.ones(C, device="cuda"), slope],
            "gradient": [torch.zeros(C, device="cuda") for _ in range(5)],
            "saved": torch.empty(head.get_temporary_fixed_buffer_size() // 4, device="cuda"),
            "ws_fwd": torch.empty(head.get_temporary_working_fixed_buffer_size(nnf_host.FORWARD), dtype=torch.uint8, device="cuda"),
            "ws_bwd": torch.empty(head.get_temporary_working_fixed_buffer_size(nnf_host.BACKWARD_DATA_AND_WEIGHTS), dtype=torch.uint8, device="cuda"),
        }

    def objects_forward(st):
        o = objects
        o["head"].enqueue_forward_propagation([st["y"]], o["data"], [st["x"]], N_PER_GPU, temporary_working_fixed_buffer=o["ws_fwd"], temporary_fixed_buffer=o["saved"])
        for f in o["followers"]:   # a per-layer scheduler enqueues them too; they launch nothing
            f.enqueue_forward_propagation([st["y"]], [], [st["y"]], N_PER_GPU)

    def objects_backward(st):
        o = objects
        for f in reversed(o["followers"]):
            f.enqueue_backward_data_propagation(0, st["dy"], st["dy"], [], [None], None, N_PER_GPU)
        o["head"].enqueue_backward_data_and_weights_propagation([st["dx"]], st["dy"], o["gradient"], o["data"], [st["x"]], None, N_PER_GPU,
                                                                temporary_working_fixed_buffer=o["ws_bwd"], temporary_fixed_buffer=o["saved"])

    if objects is not None:
        # the objects' step gives what the entry points gave (checked once, outside any timed region)
        y_obj, dx_obj = torch.empty_like(x), torch.empty_like(x)
        st0 = {"x": x, "dy": dy, "y": y_obj, "dx": dx_obj}
        objects_forward(st0)
        objects_backward(st0)
        report_words = torch.zeros(capi.REPORT_WORDS, dtype=torch.int64).pin_memory()
        capi.read_report(report_words, objects["ws_bwd"])
        step()
        torch.cuda.synchronize()
        report = capi.parse_report(report_words)
        # the same kernels on the same inputs: the same bits (several GPUs: unless a timed-out exchange made the host layer fall back)
        differing = int((y_obj != y).sum().item()) + int((dx_obj != dx).sum().item())
        note_ok = differing == 0 and report["status"] == 0
        parity["checks"].append({"check": "layer objects (planned schema -> fused head) reproduce the entry points' y and dx bit for bit", "ok": note_ok,
                                 "differing_elements": differing, "launch_status": report["status"]})
        if dist is not None:
            flag = torch.tensor([1 if note_ok else 0], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            note_ok = bool(flag.item())
        parity["ok"] = parity["ok"] and note_ok
        del y_obj, dx_obj

    xh, dyh = x.cpu().pin_memory(), dy.cpu().pin_memory()
    yh, dxh = torch.empty_like(xh).pin_memory(), torch.empty_like(xh).pin_memory()
    s_in, s_comp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    sets = [{"x": x, "dy": dy, "y": y, "dx": dx}, {"x": torch.empty_like(x), "dy": torch.empty_like(x), "y": torch.empty_like(x), "dx": torch.empty_like(x)}]
    for st in sets:
        for name in ("ev_x", "ev_dy", "ev_y", "ev_dx", "ev_out"):
            st[name] = torch.cuda.Event()
            st[name].record()

    def e2e_step(k):
        st = sets[k & 1]
        with torch.cuda.stream(s_in):
            s_in.wait_event(st["ev_dx"])          # the step two back has finished reading this set's x and dy
            st["x"].copy_(xh, non_blocking=True)
            st["ev_x"].record(s_in)
            st["dy"].copy_(dyh, non_blocking=True)
            st["ev_dy"].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(st["ev_x"])
            s_comp.wait_event(st["ev_out"])       # ... and its y and dx have been copied out
            if objects is not None:
                objects_forward(st)
            else:
                layer.forward(st["y"], st["x"], gamma, beta)
            st["ev_y"].record(s_comp)
            s_comp.wait_event(st["ev_dy"])
            if objects is not None:
                objects_backward(st)
            else:
                layer.backward(st["dx"], st["dy"], st["x"], gamma, beta, grads=grad_map)
            st["ev_dx"].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(st["ev_y"])
            yh.copy_(st["y"], non_blocking=True)
            s_out.wait_event(st["ev_dx"])
            dxh.copy_(st["dx"], non_blocking=True)
            st["ev_out"].record(s_out)

    current["ev"] = None
    e2e_step(0)
    e2e_step(1)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for stream in (s_in, s_comp, s_out):
        stream.wait_stream(torch.cuda.current_stream())
    e0.record()
    for stream in (s_in, s_comp, s_out):
        stream.wait_event(e0)
    for k in range(args.e2e_steps):
        e2e_step(k)
    for stream in (s_in, s_comp, s_out):
        torch.cuda.current_stream().wait_stream(stream)
    e1.record()
    barrier()
    e2e_ms = e0.elapsed_time(e1) / args.e2e_steps
    if dist is not None:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    tensor_bytes = elems * 4
    e2e = {"value": bytes_step_all / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": e2e_ms,
           "h2d_bytes_per_step": 2 * tensor_bytes, "d2h_bytes_per_step": 2 * tensor_bytes, "steps": args.e2e_steps,
           "overlap": "copies of neighbouring steps overlap the kernels (3 streams, 2 buffer sets)",
           "api": "layer_updater objects made by the C++ factory from the planned schema (fused head + no-op followers)" if objects is not None
                  else "ShardedBatchNormAct over the C ABI"}

    # the other configurations of the benchmark (one GPU each), outside the headline's timed region
    configs = None
    if world == 1 and not args.no_configs:
        del sets, xh, dyh, yh, dxh
        torch.cuda.empty_cache()
        configs = [{"config": r["config"], "kernel": r["kernel"], "us": r["us"], "GBps": r["GBps"], "frac": r["frac_of_peak"], "note": r["note"]}
                   for r in collect_sweep(args, quick=True)]

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sec, threads, kind, desc = cpu_step_seconds(32, reps=2)
        cpu = {"value": 32 * C * H * W * (BYTES_PER_ELEM_FWD + BYTES_PER_ELEM_BWD) / sec / 1e9, "unit": "GB/s", "cores": threads, "kind": kind, "sample": desc}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": make_config(world), "exchange": exchange_name,
            "gelem_per_s": elems * world / (ms_step * 1e-3) / 1e9,
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
            "host_enqueue_us_per_step": host_enqueue_us,
            "parity_check": parity, "configs": configs, "waits": waits, "tuning": args.tune,
        }
        result_out.write(json.dumps(line) + "\n")
        result_out.flush()
    if dist is not None:
        dist.destroy_process_group()
    if not parity["ok"]:
        print("parity check failed: %s" % json.dumps(parity), file=sys.stderr)
        sys.exit(3)


if __name__ == "__main__":
    main()
