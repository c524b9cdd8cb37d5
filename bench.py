#!/usr/bin/env python3
"""Benchmark of the Lyapunov-fractal hot path on B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode exact|fast64|fast32] [--impl reference] [--config 3|4]

One "step" renders one frame end to end on the device: lambda kernel -> min/max -> normalise -> colour.
Workload at N = 1: the 4096x4096 "AABAB" frame, 200 warm-up + 2000 accumulated steps per pixel, exact fp64.
At N > 1 (one process per GPU, launched by torch.distributed.run) the frame grows to 4096 x (4096*N) and
each rank renders one 4096-row band (weak scaling); the only exchange is the all-reduce of the frame's
min/max (two doubles) before the colour stage, and each rank recomputes its two halo rows.

--config 3 (16384^2, "BBBBBBAAAAAA", 500 + 4000) and --config 4 (65536^2, "AB", 100 + 1000) render that one frame
split into N row bands instead (strong scaling; device-resident only, no end-to-end leg at those sizes).

Metric: logistic-map steps per second (executed steps of all ranks / max-over-ranks device time).
PyTorch appears here only as plumbing: CUDA events on the launching stream, pinned host buffers,
torch.distributed for the barrier and the two-double all-reduce.  The engine is liblyap_b200.so.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG2 = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=4096, height=4096, sequence="AABAB",
            iterations=2000, warmup=200)
CFG3 = dict(min_x=3.4, max_x=4.0, min_y=2.5, max_y=3.4, width=16384, height=16384, sequence="BBBBBBAAAAAA",
            iterations=4000, warmup=500)
CFG4 = dict(min_x=2.0, max_x=4.0, min_y=2.0, max_y=4.0, width=65536, height=65536, sequence="AB",
            iterations=1000, warmup=100)
# fp64 instructions per logistic step in the exact kernel's main path, counted from its source:
#   warm-up step      3  (r*x, 1-x, product)
#   accumulated step 13  (fma(-2,x,1), r*|.|, 7 for the log incl. its last addition, sum +=, r*x, 1-x, product)
# The log's other two products, e*ln2hi and (e-1023)*ln2lo, come from a 4096-entry shared-memory table.
OPS_WARM, OPS_ACC = 3, 13
FAST_OPS = 4   # fast modes: 4 fused instructions per step on the fp64 / fp32 pipe


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        rows = [l.split(", ") for t, l in self.lines if t0 <= t <= t1 + 0.2] or [l.split(", ") for _t, l in self.lines]
        sm, reasons, smax, power = [], set(), None, []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[0]))
                smax = float(r[1])
                power.append(float(r[2]))
                for n, v in zip(names, r[3:7]):
                    if v.strip() == "Active":
                        reasons.add(n)
            except (ValueError, IndexError):
                pass
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


def reference_arm(args, rank, world):
    """The reference's own CPU implementation (unmodified header, host libm, OpenMP over rows) on a bounded
    sample of the same workload: a window of the 4096-wide frame a few rows tall, same steps per pixel."""
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O   # the one place outside tests/ that runs the CPU checker: it is what is being timed
    ref, kind = O.ref("stock"), "reference"
    port = O.port()
    if ref is None:
        kind = "port"
    cores = os.cpu_count()
    w, per_px = CFG2["width"], CFG2["warmup"] + CFG2["iterations"]

    def run(rows):
        dy = (CFG2["max_y"] - CFG2["min_y"]) / (CFG2["height"] - 1.0)
        y0 = 1500
        a = (CFG2["min_x"], CFG2["max_x"], CFG2["min_y"] + dy * y0, CFG2["min_y"] + dy * (y0 + rows - 1), w, rows,
             CFG2["sequence"], CFG2["iterations"], CFG2["warmup"])
        t = time.perf_counter()
        if ref is not None:
            lam = ref.compute_fractal(*a)
            ref.normalize(lam)
        else:
            lam, _ = port.lambda_rows(*a)
            port.normalize(lam)
        return time.perf_counter() - t

    t8 = run(8)
    rows = max(8, min(4096, int(8 * 4.0 / max(t8, 1e-3))))     # about 4 s per step
    for _ in range(args.warmup if args.warmup < 2 else 1):
        run(rows)
    times = [run(rows) for _ in range(args.steps)]
    total = sum(times)
    value = rows * w * per_px * args.steps / total
    sample = "%d of 4096 rows of the 4096-wide frame per step (%.2e nominal steps), lambda + normalizeData" % (
        rows, rows * w * per_px)
    line = {"impl": "reference", "metric": "logistic-map steps/s", "value": value, "unit": "steps/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "cfg2: 4096x4096 'AABAB' 200+2000 exact fp64 (bounded row sample)"},
            "cpu_baseline": {"value": value, "unit": "steps/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def cpu_baseline_leg():
    """~10 s of the reference's CPU path on this box's cores, reported beside the GPU number."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    ref, kind = O.ref("stock"), "reference"
    port = O.port()
    w, per_px = CFG2["width"], CFG2["warmup"] + CFG2["iterations"]
    dy = (CFG2["max_y"] - CFG2["min_y"]) / (CFG2["height"] - 1.0)

    def run(rows):
        a = (CFG2["min_x"], CFG2["max_x"], CFG2["min_y"] + dy * 1500, CFG2["min_y"] + dy * (1500 + rows - 1), w, rows,
             CFG2["sequence"], CFG2["iterations"], CFG2["warmup"])
        t = time.perf_counter()
        if ref is not None:
            ref.compute_fractal(*a)
        else:
            port.lambda_rows(*a)
        return time.perf_counter() - t

    if ref is None:
        kind = "port"
    t8 = run(8)
    rows = max(8, min(4096, int(8 * 5.0 / max(t8, 1e-3))))
    best = min(run(rows) for _ in range(2))
    return {"value": rows * w * per_px / best, "unit": "steps/s", "cores": os.cpu_count(), "kind": kind,
            "sample": "%d rows of the 4096-wide cfg2 frame (%.2e nominal steps), computeFractal, best of 2, OpenMP on all cores"
                      % (rows, rows * w * per_px)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--mode", default="exact", choices=["exact", "fast64", "fast32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4],
                    help="2 (default): the 4096-wide frame, one 4096-row band per GPU; 3, 4: that frame split over the GPUs")
    ap.add_argument("--no-gather", action="store_true", help="skip the optional NCCL gather of the RGBA bands to rank 0 (N > 1)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank, world)
        return

    # stdout carries exactly one JSON line: anything a library prints there (NCCL's version banner, ...) goes to stderr
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import numpy as np
    import torch
    import lyapunovfractalwasm_b200 as L
    from lyapunovfractalwasm_b200 import bands

    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    eng = L.Engine(local_rank)
    stream = torch.cuda.Stream()          # a real stream handle: the engine, the events and NCCL's waits all use it
    torch.cuda.set_stream(stream)
    eng.set_stream(ctypes.c_void_p(stream.cuda_stream))
    mode = {"exact": L.MODE_EXACT, "fast64": L.MODE_FAST_FP64, "fast32": L.MODE_FAST_FP32}[args.mode]

    # the frame: cfg2 at N = 1; N bands of 4096 rows at N > 1
    strong = args.config != 2
    kw = dict({3: CFG3, 4: CFG4}[args.config], mode=mode) if strong else dict(CFG2, height=CFG2["height"] * world, mode=mode)
    width, height = kw["width"], kw["height"]
    b0, b1 = bands.band_rows(height, world, rank)
    above, below = bands.halo_rows(height, b0, b1)
    rows_all, rows_own = (b1 - b0) + above + below, b1 - b0
    p_band = L.make_params(**kw, row_begin=b0 - above, row_end=b1 + below)

    dev = torch.device("cuda", local_rank)
    d_lambda = torch.empty(rows_all * width, dtype=torch.float64, device=dev)
    d_norm = torch.empty(rows_all * width, dtype=torch.float64, device=dev)
    d_rgba = torch.empty(rows_own * width * 4, dtype=torch.uint8, device=dev)
    d_minmax = torch.empty(2, dtype=torch.float64, device=dev)
    d_steps = torch.zeros(1, dtype=torch.int64, device=dev)
    own_off = above * width * 8

    lam_events = []

    def step(record=False, norm=None, rgba=None):
        norm = d_norm if norm is None else norm
        rgba = d_rgba if rgba is None else rgba
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
        eng.lambda_device(p_band, d_lambda.data_ptr(), None, d_steps.data_ptr())
        if record:
            e1.record(stream)
            lam_events.append((e0, e1))
        eng.minmax_device(d_lambda.data_ptr() + own_off, rows_own * width, d_minmax.data_ptr())
        if dist is not None:
            dist.all_reduce(d_minmax[0:1], op=dist.ReduceOp.MIN)
            dist.all_reduce(d_minmax[1:2], op=dist.ReduceOp.MAX)
        eng.normalize_device(d_lambda.data_ptr(), rows_all * width, d_minmax.data_ptr(), norm.data_ptr())
        eng.colorize_device(norm.data_ptr() + own_off, width, rows_own, above, below, 0, rgba.data_ptr())

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    fp64_peak = eng.fp64_peak()
    fp32_peak = eng.fp32_peak()
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    d_steps.zero_()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    barrier()
    t0 = time.time()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        step(record=True)
    ev1.record(stream)
    torch.cuda.synchronize()
    t1 = time.time()
    barrier()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ms = ev0.elapsed_time(ev1)
    ms_lambda = sum(a.elapsed_time(b) for a, b in lam_events) / len(lam_events)
    executed = int(d_steps.item()) * rows_own // rows_all     # halo rows excluded pro rata
    t = torch.tensor([ms, ms_lambda], dtype=torch.float64, device=dev)
    s = torch.tensor([executed], dtype=torch.int64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(s, op=dist.ReduceOp.SUM)
    ms, ms_lambda = float(t[0]), float(t[1])
    executed_all = int(s[0])
    value = executed_all / (ms * 1e-3)

    # ---- end to end: same frame through the host-buffer path, copies inside the timed region ----
    def end_to_end():
        p_full = L.make_params(**kw)
        stats = L.RenderStats()
        # two sets of pinned host buffers and (N > 1) of device outputs: step k's copies run on their own stream
        # while step k + 1 computes into the other set
        h_norm = [torch.empty(rows_own * width, dtype=torch.float64).pin_memory() for _ in range(2)]
        h_rgba = [torch.empty(rows_own * width * 4, dtype=torch.uint8).pin_memory() for _ in range(2)]
        counter = [0]
        if world > 1:
            copy_stream = torch.cuda.Stream()
            dn = [d_norm, torch.empty_like(d_norm)]
            dr = [d_rgba, torch.empty_like(d_rgba)]
            computed = [torch.cuda.Event(), torch.cuda.Event()]
            copied = [torch.cuda.Event(), torch.cuda.Event()]
            own0 = above * width

        def e2e_step():
            b = counter[0] & 1
            counter[0] += 1
            if world == 1:
                # the call a user makes: lyap_render with host pointers (parameters in, normalised + RGBA out)
                L._check(eng.lib.lyap_render(eng.ctx, ctypes.byref(p_full), None, None, h_norm[b].data_ptr(),
                                             h_rgba[b].data_ptr(), None, ctypes.byref(stats)))
                return stats.executed_steps
            if counter[0] > 2:
                stream.wait_event(copied[b])          # this set's previous copies have left the device buffers
            step(norm=dn[b], rgba=dr[b])
            computed[b].record(stream)
            copy_stream.wait_event(computed[b])
            with torch.cuda.stream(copy_stream):
                h_norm[b].copy_(dn[b][own0:own0 + rows_own * width], non_blocking=True)
                h_rgba[b].copy_(dr[b], non_blocking=True)
                copied[b].record(copy_stream)
            return None

        e2e_step()
        barrier()
        d_steps.zero_()
        ev0.record(stream)
        te = time.perf_counter()
        e2e_executed = 0
        for _ in range(args.steps):
            r = e2e_step()
            e2e_executed += r if r is not None else 0
        ev1.record(stream)
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - te) * 1e3
        if world > 1:
            e2e_executed = int(d_steps.item()) * rows_own // rows_all
        t = torch.tensor([wall_ms], dtype=torch.float64, device=dev)
        s = torch.tensor([e2e_executed], dtype=torch.int64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(s, op=dist.ReduceOp.SUM)
        return int(s[0]) / (float(t[0]) * 1e-3)

    e2e_value = None if strong else end_to_end()

    # ---- the same K frames as one batch call: copies of frame k overlap the kernels of frame k + 1 ----
    def end_to_end_batch():
        n = args.steps
        frames = (L.LyapParams * n)()
        p_full = L.make_params(**kw)
        for i in range(n):
            ctypes.memmove(ctypes.byref(frames[i]), ctypes.byref(p_full), ctypes.sizeof(L.LyapParams))
        h_norms = [torch.empty(rows_own * width, dtype=torch.float64).pin_memory() for _ in range(n)]
        h_rgbas = [torch.empty(rows_own * width * 4, dtype=torch.uint8).pin_memory() for _ in range(n)]
        norm_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in h_norms])
        rgba_ptrs = (ctypes.c_void_p * n)(*[t.data_ptr() for t in h_rgbas])
        devs = (ctypes.c_int32 * 1)(local_rank)
        stats = (L.RenderStats * n)()
        best = None
        for _ in range(2):      # the first call also pays for the worker's context and buffers being set up cold
            te = time.perf_counter()
            L._check(eng.lib.lyap_render_frames(frames, n, 1, devs, norm_ptrs, rgba_ptrs, stats))
            wall = time.perf_counter() - te
            rate = sum(st.executed_steps for st in stats) / wall
            best = rate if best is None else max(best, rate)
        return {"value": best, "unit": "steps/s", "frames_per_call": n,
                "what": "lyap_render_frames(host pointers): one call for all K frames, two buffer sets per device, "
                        "device-to-host copies on their own stream; wall clock of the whole call, worker and buffer set-up included"}

    e2e_batch = end_to_end_batch() if (world == 1 and not strong) else None

    # ---- optional: gather the finished RGBA bands to rank 0 over NCCL (outside the timed regions above) ----
    gather = None
    if dist is not None and not args.no_gather:
        parts = [torch.empty_like(d_rgba) for _ in range(world)] if rank == 0 else None
        dist.gather(d_rgba, parts, dst=0)          # warm-up (connection set-up)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        dist.gather(d_rgba, parts, dst=0)
        g1.record(stream)
        torch.cuda.synchronize()
        tg = torch.tensor([g0.elapsed_time(g1)], dtype=torch.float64, device=dev)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        nbytes = d_rgba.numel() * (world - 1)
        gather = {"ms": float(tg[0]), "bytes_into_rank0": nbytes, "gbs": nbytes / (float(tg[0]) * 1e-3) / 1e9,
                  "what": "torch.distributed.gather (NCCL) of each rank's RGBA8 band into rank 0's memory, timed apart from the steps"}

    if rank == 0:
        hbm_peak = None
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                hbm_peak = json.load(f).get("hbm_gbs")
        except OSError:
            pass
        per_px_ops = (OPS_WARM * kw["warmup"] + OPS_ACC * kw["iterations"]) if mode == L.MODE_EXACT else \
            FAST_OPS * (kw["warmup"] + kw["iterations"])
        steps_per_launch = executed_all / args.steps / world * rows_all / rows_own   # one rank's launch, halo included
        instr_per_launch = steps_per_launch * per_px_ops / (kw["warmup"] + kw["iterations"])
        achieved = instr_per_launch / (ms_lambda * 1e-3)
        peak = fp32_peak if mode == L.MODE_FAST_FP32 else fp64_peak
        out_bytes = rows_all * width * 8
        roofline = {
            "kernel": {L.MODE_EXACT: "k_lambda_exact_spec (k_lambda_exact compiled at run time for this sequence; LYAP_JIT=0: precompiled)"
                       if os.environ.get("LYAP_JIT", "1") != "0" else "k_lambda_exact", L.MODE_FAST_FP64: "k_lambda_fast<double>",
                       L.MODE_FAST_FP32: "k_lambda_fast<float>"}[mode],
            "bound": "fp32_pipe" if mode == L.MODE_FAST_FP32 else "fp64_pipe",
            "achieved": achieved / 1e12, "peak": peak / 1e12, "unit": "T thread-instr/s", "frac": achieved / peak,
            "peak_source": "measured in this run: independent FMA chains on all SMs (lyap_fp64_peak / lyap_fp32_peak); "
                           "MEASURED_PEAKS.json has no fp64/fp32 vector entry",
            "instr_per_step": {"warmup": OPS_WARM, "accumulated": OPS_ACC} if mode == L.MODE_EXACT else FAST_OPS,
            "ms_per_launch": ms_lambda,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch on the 4096x4096 frame (ncu, profiles/):
            # 1.9 MB read + 76.1 MB written; less than the 134 MB of stores because the tail is still in L2 at kernel end
            "traffic": 78.0e6 * rows_all / 4096 if mode == L.MODE_EXACT and not strong else None,
            "hbm": {"algorithmic_bytes_per_launch": out_bytes, "store_gbs": out_bytes / (ms_lambda * 1e-3) / 1e9,
                    "peak_gbs": hbm_peak, "peak_source": "MEASURED_PEAKS.json (measured)" if hbm_peak else "absent"},
        }
        what = "%s mode; step = lambda + min/max + normalise + RGBA8 on the device" % args.mode
        if strong:
            workload = ("cfg%d: %dx%d '%s', %d warm-up + %d accumulated steps, %s; the one frame as %d row band(s) of %d rows"
                        % (args.config, width, height, kw["sequence"], kw["warmup"], kw["iterations"], what, world, rows_own))
        else:
            workload = ("cfg2: 4096x4096 'AABAB', a,b in [2.5,4], 200 warm-up + 2000 accumulated steps, " + what
                        + ("" if world == 1 else "; frame 4096x%d as %d row bands of 4096 rows, halo rows "
                           "recomputed and excluded from the step count pro rata" % (height, world)))
        line = {
            "metric": "logistic-map steps/s", "value": value, "unit": "steps/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong" if strong else "weak",
            "vs_baseline": None, "dtype": "f32" if mode == L.MODE_FAST_FP32 else "f64", "data": "synthetic",
            "config": {"workload": workload,
                       "l2": "each step rewrites %.0f MiB of outputs per GPU (> 126 MB L2); the path has no input arrays"
                             % ((rows_all * width * 16 + rows_own * width * 4) / 2 ** 20),
                       "executed_over_nominal": executed_all / (args.steps * width * height * (kw["warmup"] + kw["iterations"]))},
            ("ms_per_frame" if strong else "ms_per_frame_4096"): ms / args.steps,
            "roofline": roofline,
            "e2e": None if e2e_value is None else {"value": e2e_value, "unit": "steps/s", "h2d_bytes_per_step": ctypes.sizeof(L.LyapParams) + len(kw["sequence"]),
                    "d2h_bytes_per_step": rows_own * width * 12 + ctypes.sizeof(L.RenderStats),
                    "what": "lyap_render(host pointers): parameters in, normalised fp64 + RGBA8 frame out to pinned host memory"
                            if world == 1 else "band path (device entry points + the min/max all-reduce), then the band's normalised fp64 "
                            "+ RGBA8 copied to pinned host memory on a second stream from one of two buffer sets, so the copies "
                            "of step k overlap the kernels of step k + 1; all copies are inside the timed region"},
            "gpu_launches": 4 * args.steps,
            "clocks": clocks,
        }
        if gather is not None:
            line["gather"] = gather
        if e2e_batch is not None:
            line["e2e_batch"] = e2e_batch
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg()
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    eng.close()


if __name__ == "__main__":
    main()
