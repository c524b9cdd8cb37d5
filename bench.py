#!/usr/bin/env python3
"""Benchmark of the Lyapunov-fractal hot path on B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode exact|fast64|fast32] [--impl reference] [--config 3|4]
                    [--no-extras] [--no-cpu-baseline] [--no-gather]

One "step" renders one frame end to end on the device: lambda kernel -> min/max -> normalise -> colour.
Workload at N = 1: the 4096x4096 "AABAB" frame, 200 warm-up + 2000 accumulated steps per pixel, exact fp64.
At N > 1 (one process per GPU, launched by torch.distributed.run) the frame grows to 4096 x (4096*N) and
each rank renders one 4096-row band (weak scaling); the only exchange is one all-reduce(MIN) of the pair
(min, -max) of the frame's lambda values before the colour stage, and each rank recomputes its two halo rows.

Beside that headline the JSON line carries (unless --no-extras):
  strong_cfg4   the one 65536x65536 "AB" frame split into N row bands (strong scaling; N = 1 holds 80 GiB)
  modes         (N = 1) the fast kernels (fused fp64, fused fp32, fp64 on the exact orbit) on the 4096x4096 frame: ms per
                frame, pipe fraction, per-pixel deviation from the exact frame
  c_abi_multi   rank 0 alone drives all N devices from one process through the C ABI's lyap_multi object:
                the 16384x16384 frame as N bands with the NCCL gather of the RGBA bands into device 0, and a
                batch of zoom frames dealt round-robin (the other ranks wait on the host meanwhile)
--config 3 / --config 4 make that frame the headline workload instead (strong scaling).

Metric: logistic-map steps per second (executed steps of all ranks / max-over-ranks device time).
`e2e` is the same metric through host buffers with every frame's outputs copied to pinned host memory inside the timed
region, the copies of frame k overlapping the kernels of frame k + 1 (N = 1: one lyap_multi_render_frames call for the K
frames; N > 1: the band path with two buffer sets); `e2e_blocking` (N = 1) is one blocking lyap_render call per frame.
PyTorch appears here only as plumbing: CUDA events on the launching stream, pinned host buffers,
torch.distributed for the barrier and the all-reduce.  The engine is liblyap_b200.so.

--impl reference times the reference's own CPU code (its header built natively, host libm, OpenMP over rows) on a
bounded row sample of the same frame, on this box's host cores.
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
# the same steps in flops (a fused multiply-add counts 2): warm-up 3 (none fused); accumulated 19 = 13 instructions,
# 6 of them fused (fma(-2,x,1), r = fma(d,inv,-1), three for the cubic, s = fma(r,w,klo))
FLOPS_WARM, FLOPS_ACC = 3, 19
FAST_OPS = 4   # fast modes: 4 instructions per step on the fp64 / fp32 pipe, 2 of them fused (6 flops)
FAST_FLOPS = 6


def config5_frame(k):
    h = 0.5 * 0.97 ** k
    return dict(min_x=3.82 - h, max_x=3.82 + h, min_y=3.45 - h, max_y=3.45 + h, width=1920, height=1080,
                sequence="ABC", iterations=3000, warmup=300, c=3.7)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 100 ms while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
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


# ---------------------------------------------------------------------------------------------------------------
# The reference's CPU path, timed on this box's host cores.
# ---------------------------------------------------------------------------------------------------------------

def cpu_model():
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("model name"):
                    return line.split(":", 1)[1].strip()
    except OSError:
        pass
    return "unknown"


class CpuReference:
    """A row window of the 4096-wide frame through the reference's computeFractal / normalizeData
    (oracle/_ref/libref_stock.so: the unmodified header, host libm; this project's restatement when that build is
    absent).  The header turns its OpenMP loop on only for frames TALLER THAN 100 ROWS
    (src/lyapunov_fractal.hpp:40), so every threaded sample here is at least 128 rows and a multiple of the
    thread count."""

    def __init__(self):
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as O   # bench.py's CPU legs are the one place outside tests/ that runs the CPU checker
        self.ref = O.ref("stock")
        self.port = O.port()
        self.kind = "reference" if self.ref is not None else "port"
        # all the host CPUs this process may run on, whatever OMP_NUM_THREADS says (torch.distributed.run sets it to 1 for
        # every worker it starts); what the header's loop will really use is read back from the OpenMP runtime
        cpus = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
        if self.ref is not None:
            self.ref.set_threads(cpus)
            self.threads = self.ref.max_threads()
        else:
            os.environ["OMP_NUM_THREADS"] = str(cpus)
            self.threads = cpus
        self.w = CFG2["width"]
        self.per_px = CFG2["warmup"] + CFG2["iterations"]

    def window(self, rows):
        dy = (CFG2["max_y"] - CFG2["min_y"]) / (CFG2["height"] - 1.0)
        y0 = 1500
        return (CFG2["min_x"], CFG2["max_x"], CFG2["min_y"] + dy * y0, CFG2["min_y"] + dy * (y0 + rows - 1), self.w, rows,
                CFG2["sequence"], CFG2["iterations"], CFG2["warmup"])

    def run(self, rows):
        """(seconds in computeFractal, seconds in normalizeData)."""
        a = self.window(rows)
        t0 = time.perf_counter()
        lam = self.ref.compute_fractal(*a) if self.ref is not None else self.port.lambda_rows(*a)[0]
        t1 = time.perf_counter()
        if self.ref is not None:
            self.ref.normalize(lam)
        else:
            self.port.normalize(lam)
        t2 = time.perf_counter()
        return t1 - t0, t2 - t1

    def round_rows(self, rows):
        t = max(1, self.threads)
        rows = max(128, min(4096, int(rows)))
        return max(128, (rows + t - 1) // t * t)

    def rows_for(self, seconds):
        """Rows whose threaded run takes about `seconds`, from a threaded probe of >= 128 rows."""
        probe = self.round_rows(128)
        tc, tn = self.run(probe)
        return self.round_rows(probe * seconds / max(tc + tn, 1e-3))

    def one_thread_rate(self, seconds=2.0):
        """steps/s of computeFractal on one thread (a short sample: the loop is serial below 101 rows anyway)."""
        if self.ref is None:
            return None
        self.ref.set_threads(1)
        try:
            rows = 8
            tc, _ = self.run(rows)
            rows = max(8, min(100, int(rows * seconds / max(tc, 1e-3))))
            tc, _ = self.run(rows)
        finally:
            self.ref.set_threads(self.threads)
        return rows * self.w * self.per_px / tc

    def describe(self, rows, tc, tn, what):
        steps = rows * self.w * self.per_px
        return {"value": steps / tc, "unit": "steps/s", "cores": self.threads, "kind": self.kind,
                "threads_used": self.threads, "host_logical_cpus": os.cpu_count(), "cpu_model": cpu_model(),
                "sample": "%d of 4096 rows of the 4096-wide cfg2 frame (%.2e nominal steps); %s; the sample is taller than 100 "
                          "rows, so the header's OpenMP row loop is on (schedule(dynamic), %d threads)" % (rows, steps, what, self.threads),
                "compute_fractal_ms": 1e3 * tc,
                "normalize_data": {"ms": 1e3 * tn, "mpixels_per_s": rows * self.w / tn / 1e6}}


def reference_arm(args, rank):
    """--impl reference: K steps, each one threaded row sample of the frame through computeFractal + normalizeData."""
    if rank != 0:
        return
    cpu = CpuReference()
    rows = cpu.rows_for(4.0)                       # about 4 s per step
    for _ in range(min(args.warmup, 1)):
        cpu.run(rows)
    runs = [cpu.run(rows) for _ in range(args.steps)]
    tc, tn = sum(r[0] for r in runs), sum(r[1] for r in runs)
    steps = rows * cpu.w * cpu.per_px * args.steps
    value = steps / (tc + tn)
    base = cpu.describe(rows, tc / args.steps, tn / args.steps, "computeFractal then normalizeData per step")
    base["value"] = value
    base["one_thread_steps_per_s"] = cpu.one_thread_rate()
    line = {"impl": "reference", "metric": "logistic-map steps/s", "value": value, "unit": "steps/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * (tc + tn) / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64", "data": "synthetic",
            "config": {"workload": "cfg2: 4096x4096 'AABAB' 200+2000 exact fp64 (bounded row sample, %d rows per step)" % rows},
            "cpu_baseline": base,
            "e2e": {"value": value, "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def cpu_baseline_leg():
    """About 10 s of the reference's CPU path on this box's cores, reported beside the GPU number."""
    cpu = CpuReference()
    rows = cpu.rows_for(4.0)
    tc, tn = min((cpu.run(rows) for _ in range(2)), key=lambda r: r[0])
    out = cpu.describe(rows, tc, tn, "computeFractal, best of 2")
    out["one_thread_steps_per_s"] = cpu.one_thread_rate()
    return out


# ---------------------------------------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--mode", default="exact", choices=["exact", "fast64", "fast32", "orbit64"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4],
                    help="2 (default): the 4096-wide frame, one 4096-row band per GPU; 3, 4: that frame split over the GPUs")
    ap.add_argument("--no-gather", action="store_true", help="skip the optional NCCL gather of the RGBA bands to rank 0 (N > 1)")
    ap.add_argument("--no-extras", action="store_true", help="headline workload only (no strong_cfg4 / modes / c_abi_multi)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, rank)
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
    dist = host_pg = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        host_pg = dist.new_group(backend="gloo")     # host-side waits: no kernel of a waiting rank sits on its GPU

    eng = L.Engine(local_rank)
    stream = torch.cuda.Stream()          # a real stream handle: the engine, the events and NCCL's waits all use it
    torch.cuda.set_stream(stream)
    eng.set_stream(ctypes.c_void_p(stream.cuda_stream))
    modes = {"exact": L.MODE_EXACT, "fast64": L.MODE_FAST_FP64, "fast32": L.MODE_FAST_FP32, "orbit64": L.MODE_FAST_FP64_ORBIT}
    mode = modes[args.mode]
    dev = torch.device("cuda", local_rank)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    class BandRunner:
        """This rank's band of one frame: buffers on the device and the per-step launches."""

        def __init__(self, kw):
            self.kw = kw
            self.width, self.height = kw["width"], kw["height"]
            b0, b1 = bands.band_rows(self.height, world, rank)
            self.above, self.below = bands.halo_rows(self.height, b0, b1)
            self.rows_own, self.rows_all = b1 - b0, (b1 - b0) + self.above + self.below
            self.p_band = L.make_params(**kw, row_begin=b0 - self.above, row_end=b1 + self.below)
            n_all = self.rows_all * self.width
            self.d_lambda = torch.empty(n_all, dtype=torch.float64, device=dev)
            self.d_norm = torch.empty(n_all, dtype=torch.float64, device=dev)
            self.d_rgba = torch.empty(self.rows_own * self.width * 4, dtype=torch.uint8, device=dev)
            self.d_minmax = torch.empty(2, dtype=torch.float64, device=dev)
            self.d_pair = torch.empty(2, dtype=torch.float64, device=dev)
            self.sign = torch.tensor([1.0, -1.0], dtype=torch.float64, device=dev)
            self.d_steps = torch.zeros(1, dtype=torch.int64, device=dev)
            self.own_off = self.above * self.width * 8
            self.lam_events = []
            self.launches = 0
            self.kernel_name = ""

        def step(self, record=False, norm=None, rgba=None):
            norm = self.d_norm if norm is None else norm
            rgba = self.d_rgba if rgba is None else rgba
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
            eng.lambda_device(self.p_band, self.d_lambda.data_ptr(), None, self.d_steps.data_ptr())
            if record:
                e1.record(stream)
                self.lam_events.append((e0, e1))
            eng.minmax_device(self.d_lambda.data_ptr() + self.own_off, self.rows_own * self.width, self.d_minmax.data_ptr())
            if dist is not None:
                # one all-reduce serves both ends: min over (min, -max)
                torch.mul(self.d_minmax, self.sign, out=self.d_pair)     # exact: times 1, times -1
                dist.all_reduce(self.d_pair, op=dist.ReduceOp.MIN)
                torch.mul(self.d_pair, self.sign, out=self.d_minmax)
            eng.normalize_device(self.d_lambda.data_ptr(), self.rows_all * self.width, self.d_minmax.data_ptr(), norm.data_ptr())
            eng.colorize_device(norm.data_ptr() + self.own_off, self.width, self.rows_own, self.above, self.below, 0, rgba.data_ptr())
            self.launches += 4

        def measure(self, steps, warmup, sample_clocks=False):
            """W untimed steps, then K timed ones between barriers; max over ranks; executed steps of all ranks."""
            for _ in range(warmup):
                self.step()
            self.kernel_name = eng.lib.lyap_last_kernel().decode()
            barrier()
            self.d_steps.zero_()
            self.lam_events, self.launches = [], 0
            sampler = ClockSampler(local_rank) if (sample_clocks and rank == 0) else None
            if sampler:
                sampler.start()
                time.sleep(0.3)
            barrier()
            t0 = time.time()
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record(stream)
            for _ in range(steps):
                self.step(record=True)
            ev1.record(stream)
            torch.cuda.synchronize()
            t1 = time.time()
            barrier()
            clocks = sampler.stop(t0, t1) if sampler else None
            ms = ev0.elapsed_time(ev1)
            ms_lambda = sum(a.elapsed_time(b) for a, b in self.lam_events) / len(self.lam_events)
            executed = int(self.d_steps.item()) * self.rows_own // self.rows_all     # halo rows excluded pro rata
            t = torch.tensor([ms, ms_lambda], dtype=torch.float64, device=dev)
            s = torch.tensor([executed], dtype=torch.int64, device=dev)
            if dist is not None:
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dist.all_reduce(s, op=dist.ReduceOp.SUM)
            return {"ms": float(t[0]), "ms_lambda": float(t[1]), "executed": int(s[0]), "clocks": clocks,
                    "launches": self.launches, "steps": steps}

        def pipe_numbers(self, m, peak64, peak32):
            """Fractions of the pipe's issue rate and of its flop rate for the lambda kernel of measurement m."""
            kw, md = self.kw, self.kw.get("mode", L.MODE_EXACT)
            per_px_steps = kw["warmup"] + kw["iterations"]
            if md == L.MODE_EXACT:
                ops = OPS_WARM * kw["warmup"] + OPS_ACC * kw["iterations"]
                flops = FLOPS_WARM * kw["warmup"] + FLOPS_ACC * kw["iterations"]
            elif md == L.MODE_FAST_FP64_ORBIT:      # the reference's 3 orbit operations; fma(-2,x,1) and the product when accumulating
                ops = 3 * kw["warmup"] + 5 * kw["iterations"]
                flops = 3 * kw["warmup"] + 6 * kw["iterations"]
            else:
                ops, flops = FAST_OPS * per_px_steps, FAST_FLOPS * per_px_steps
            steps_per_launch = m["executed"] / m["steps"] / world * self.rows_all / self.rows_own   # one rank's launch, halo included
            sec = m["ms_lambda"] * 1e-3
            peak = peak32 if md == L.MODE_FAST_FP32 else peak64
            instr = steps_per_launch * ops / per_px_steps / sec
            fl = steps_per_launch * flops / per_px_steps / sec
            return {"achieved": instr / 1e12, "peak": peak / 1e12, "frac": instr / peak,
                    "achieved_tflops": fl / 1e12, "peak_tflops": 2 * peak / 1e12, "frac_flops": fl / (2 * peak)}

        def free(self):
            for n in ("d_lambda", "d_norm", "d_rgba"):
                setattr(self, n, None)
            torch.cuda.empty_cache()

    # the frame: cfg2 at N = 1; N bands of 4096 rows at N > 1; or one of the two large frames split over the ranks
    strong = args.config != 2
    kw = dict({3: CFG3, 4: CFG4}[args.config], mode=mode) if strong else dict(CFG2, height=CFG2["height"] * world, mode=mode)
    width, height = kw["width"], kw["height"]
    run = BandRunner(kw)
    rows_own, rows_all, above = run.rows_own, run.rows_all, run.above

    fp64_peak = eng.fp64_peak()
    fp32_peak = eng.fp32_peak()
    m = run.measure(args.steps, max(args.warmup, 3), sample_clocks=True)
    ms, ms_lambda, executed_all, clocks = m["ms"], m["ms_lambda"], m["executed"], m["clocks"]
    value = executed_all / (ms * 1e-3)
    main_launches = m["launches"]
    main_kernel = run.kernel_name
    pipe = run.pipe_numbers(m, fp64_peak, fp32_peak)

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
            dn = [run.d_norm, torch.empty_like(run.d_norm)]
            dr = [run.d_rgba, torch.empty_like(run.d_rgba)]
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
            run.step(norm=dn[b], rgba=dr[b])
            computed[b].record(stream)
            copy_stream.wait_event(computed[b])
            with torch.cuda.stream(copy_stream):
                h_norm[b].copy_(dn[b][own0:own0 + rows_own * width], non_blocking=True)
                h_rgba[b].copy_(dr[b], non_blocking=True)
                copied[b].record(copy_stream)
            return None

        e2e_step()
        barrier()
        run.d_steps.zero_()
        te = time.perf_counter()
        e2e_executed = 0
        for _ in range(args.steps):
            r = e2e_step()
            e2e_executed += r if r is not None else 0
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - te) * 1e3
        if world > 1:
            e2e_executed = int(run.d_steps.item()) * rows_own // rows_all
        t = torch.tensor([wall_ms], dtype=torch.float64, device=dev)
        s = torch.tensor([e2e_executed], dtype=torch.int64, device=dev)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.all_reduce(s, op=dist.ReduceOp.SUM)
        return int(s[0]) / (float(t[0]) * 1e-3)

    e2e_value = None if strong else end_to_end()

    # ---- the same K frames as one batch call on a kept lyap_multi object: copies of frame k overlap the kernels of frame k + 1 ----
    def end_to_end_batch():
        n = args.steps
        p_full = L.make_params(**kw)
        frames = [p_full] * n
        h_norms = [torch.empty(rows_own * width, dtype=torch.float64).pin_memory() for _ in range(n)]
        h_rgbas = [torch.empty(rows_own * width * 4, dtype=torch.uint8).pin_memory() for _ in range(n)]
        with L.Multi([local_rank]) as mo:
            mo.render_frames(frames, [t.data_ptr() for t in h_norms], [t.data_ptr() for t in h_rgbas])   # warm-up: grows the object's buffers
            te = time.perf_counter()
            stats = mo.render_frames(frames, [t.data_ptr() for t in h_norms], [t.data_ptr() for t in h_rgbas])
            wall = time.perf_counter() - te
            rate = sum(st.executed_steps for st in stats) / wall
        return {"value": rate, "unit": "steps/s", "frames_per_call": n,
                "h2d_bytes_per_step": ctypes.sizeof(L.LyapParams) + len(kw["sequence"]),
                "d2h_bytes_per_step": rows_own * width * 12 + 48,
                "what": "lyap_multi_render_frames(host pointers) on a lyap_multi object kept between calls: ONE call renders the K "
                        "frames; every frame's normalised fp64 + RGBA8 (192 MiB) is copied to pinned host memory inside the timed "
                        "region, on a second stream from one of two buffer sets, so the copies of frame k overlap the kernels of "
                        "frame k + 1 (the same policy as the N > 1 legs); wall clock of the whole call"}

    e2e_batch = end_to_end_batch() if (world == 1 and not strong) else None

    # ---- optional: gather the finished RGBA bands to rank 0 over NCCL (outside the timed regions above) ----
    gather = None
    if dist is not None and not args.no_gather:
        parts = [torch.empty_like(run.d_rgba) for _ in range(world)] if rank == 0 else None
        dist.gather(run.d_rgba, parts, dst=0)          # warm-up (connection set-up)
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record(stream)
        dist.gather(run.d_rgba, parts, dst=0)
        g1.record(stream)
        torch.cuda.synchronize()
        tg = torch.tensor([g0.elapsed_time(g1)], dtype=torch.float64, device=dev)
        dist.all_reduce(tg, op=dist.ReduceOp.MAX)
        nbytes = run.d_rgba.numel() * (world - 1)
        gather = {"ms": float(tg[0]), "bytes_into_rank0": nbytes, "gbs": nbytes / (float(tg[0]) * 1e-3) / 1e9,
                  "what": "torch.distributed.gather (NCCL) of each rank's RGBA8 band into rank 0's memory, timed apart from the steps"}
        parts = None

    extras = {}
    if not args.no_extras and mode == L.MODE_EXACT:
        # ---- (N = 1) the fast modes on the same frame: time, pipe fraction, deviation from the exact frame ----
        if world == 1 and not strong:
            exact = run.d_lambda.clone()
            stable = (exact < 0) & (exact > -4)
            chaotic = exact >= 0
            out = {}
            for name, md in (("fast64", L.MODE_FAST_FP64), ("fast32", L.MODE_FAST_FP32), ("orbit64", L.MODE_FAST_FP64_ORBIT)):
                fr = BandRunner(dict(kw, mode=md))
                fm = fr.measure(5, 3)
                fp = fr.pipe_numbers(fm, fp64_peak, fp32_peak)
                lam = fr.d_lambda
                rel = (lam[stable] - exact[stable]).abs() / exact[stable].abs()
                clear = exact[stable].abs() > 1e-3          # away from lambda = 0, where a relative bound means little
                absd = (lam[chaotic] - exact[chaotic]).abs()
                out[name] = {
                    "ms_per_frame_4096": fm["ms"] / fm["steps"], "ms_lambda_kernel": fm["ms_lambda"],
                    "steps_per_s": fm["executed"] / (fm["ms"] * 1e-3), "kernel": fr.kernel_name,
                    "pipe": "fp32" if md == L.MODE_FAST_FP32 else "fp64", "frac": fp["frac"], "frac_flops": fp["frac_flops"],
                    "deviation_from_exact": {
                        "stable_pixels": int(stable.sum()), "stable_share_beyond_1e-6_relative": float((rel > 1e-6).float().mean()),
                        "stable_share_beyond_1e-6_relative_where_abs_lambda_above_1e-3": float((rel[clear] > 1e-6).float().mean()),
                        "stable_median_relative": float(rel.median()),
                        "chaotic_pixels": int(chaotic.sum()), "chaotic_share_beyond_1e-3_absolute": float((absd > 1e-3).float().mean()),
                        "chaotic_mean_lambda_difference": float((lam[chaotic].mean() - exact[chaotic].mean()).abs()),
                        "sentinel_mismatches": int(((lam == -5.0) != (exact == -5.0)).sum())}}
                fr.free()
                del fr, lam, rel, absd, clear
            extras["modes"] = out
            del exact, stable, chaotic
        # ---- the 65536^2 frame as N row bands (strong scaling) ----
        if not strong:
            run.free()
            torch.cuda.empty_cache()
            try:
                sr = BandRunner(dict(CFG4, mode=L.MODE_EXACT))
                sm = sr.measure(2, 1)
                sp = sr.pipe_numbers(sm, fp64_peak, fp32_peak)
                extras["strong_cfg4"] = {
                    "workload": "65536x65536 'AB' 100+1000 exact fp64, the one frame as %d row band(s) of %d rows; lambda + min/max + "
                                "normalise + RGBA8 on the device; 1 warm-up frame, 2 timed" % (world, sr.rows_own),
                    "n_gpus": world, "ms_per_frame": sm["ms"] / sm["steps"], "ms_lambda_kernel": sm["ms_lambda"],
                    "steps_per_s": sm["executed"] / (sm["ms"] * 1e-3), "frac": sp["frac"], "frac_flops": sp["frac_flops"],
                    "kernel": sr.kernel_name, "device_bytes_per_gpu": sr.rows_all * sr.width * 16 + sr.rows_own * sr.width * 4}
                sr.free()
                del sr
            except torch.OutOfMemoryError as e:       # a smaller part: say so instead of failing the headline
                extras["strong_cfg4"] = {"unavailable": "device allocation failed: %s" % str(e).split("\n")[0]}
            torch.cuda.empty_cache()
        # ---- the C ABI's one-process multi-device object, driven by rank 0 over all N devices ----
        if not strong:
            torch.cuda.synchronize()
            if host_pg is not None:
                dist.barrier(group=host_pg)           # every rank is idle on its GPU from here (host-side wait below)
            if rank == 0:
                extras["c_abi_multi"] = c_abi_multi(L, world, np)
            if host_pg is not None:
                dist.barrier(group=host_pg)

    if rank == 0:
        hbm_peak = None
        try:
            with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
                hbm_peak = json.load(f).get("hbm_gbs")
        except OSError:
            pass
        out_bytes = rows_all * width * 8
        roofline = {
            "kernel": main_kernel,
            "kernel_source": "lyap_last_kernel(): what the library launched for the lambda stage; lyap_jit_note() = %r"
                             % eng.lib.lyap_jit_note().decode(),
            "bound": "fp32_pipe" if mode == L.MODE_FAST_FP32 else "fp64_pipe",
            "achieved": pipe["achieved"], "peak": pipe["peak"], "unit": "T thread-instr/s", "frac": pipe["frac"],
            "frac_flops": pipe["frac_flops"], "achieved_tflops": pipe["achieved_tflops"], "peak_tflops": pipe["peak_tflops"],
            "flops_note": "a fused multiply-add counts 2 flops, so the flop peak is 2 x the issue-rate peak; the exact mode may fuse "
                          "only where the reference's rounding allows (6 of its 13 instructions per accumulated step), which "
                          "caps frac_flops at 19/26 of frac",
            "peak_source": "measured in this run: independent FMA chains on all SMs (lyap_fp64_peak / lyap_fp32_peak); "
                           "MEASURED_PEAKS.json has no fp64/fp32 vector entry",
            "instr_per_step": {"warmup": OPS_WARM, "accumulated": OPS_ACC} if mode == L.MODE_EXACT else FAST_OPS,
            "flops_per_step": {"warmup": FLOPS_WARM, "accumulated": FLOPS_ACC} if mode == L.MODE_EXACT else FAST_FLOPS,
            "ms_per_launch": ms_lambda,
            # dram__bytes_read.sum + dram__bytes_write.sum of one launch on the 4096x4096 frame, from the ncu capture summarised
            # under profiles/ (not re-measured by this run): 2.7 MB read + 77.1 MB written; less than the 134 MB of stores
            # because the tail is still in L2 at kernel end
            "traffic": 79.7e6 * rows_all / 4096 if mode == L.MODE_EXACT and not strong else None,
            "traffic_source": "constant from the committed ncu capture of this kernel on this frame, scaled by rows; not measured live",
            "co_bound": {"pipe": "shared-memory data pipe (the logarithm's two 16-byte table look-ups)", "busy": 0.795,
                         "source": "l1tex__data_pipe_lsu_wavefronts_mem_shared, % of peak, from the committed ncu capture of this "
                                   "kernel on the 4096x4096 frame (not measured live); the fp64 stream without the look-ups "
                                   "runs at 0.96 of the issue rate"} if mode == L.MODE_EXACT else None,
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
            "e2e": None if e2e_value is None else e2e_batch if (world == 1 and e2e_batch is not None) else
                   {"value": e2e_value, "unit": "steps/s", "h2d_bytes_per_step": ctypes.sizeof(L.LyapParams) + len(kw["sequence"]),
                    "d2h_bytes_per_step": rows_own * width * 12 + ctypes.sizeof(L.RenderStats),
                    "what": "band path (device entry points + the min/max all-reduce), then the band's normalised fp64 "
                            "+ RGBA8 copied to pinned host memory on a second stream from one of two buffer sets, so the copies "
                            "of step k overlap the kernels of step k + 1; all copies are inside the timed region"},
            "gpu_launches": main_launches,
            "gpu_launches_note": "this library's kernels enqueued by this rank inside the timed region, counted call by call "
                                 "(lambda, min/max, normalise, colour per step)",
            "clocks": clocks,
        }
        if gather is not None:
            line["gather"] = gather
        if world == 1 and e2e_value is not None:
            line["e2e_blocking"] = {
                "value": e2e_value, "unit": "steps/s",
                "what": "lyap_render(host pointers), one BLOCKING call per frame (the reference's call shape: one computeLyapunovFractal "
                        "per view): parameters in, normalised fp64 + RGBA8 frame out to pinned host memory.  The 192 MiB cannot leave "
                        "before the frame's min/max is known, i.e. after the last lambda pixel, so a single blocking frame costs "
                        "kernel time + copy time; `e2e` overlaps them across frames"}
        line.update(extras)
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline_leg()
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    eng.close()


def c_abi_multi(L, world, np):
    """Rank 0 alone, one process over all N devices through lyap_multi: a banded frame with the gather into device 0,
    and a batch of zoom frames dealt round-robin."""
    out = {"n_devices": world}
    devices = list(range(world))
    try:
        with L.Multi(devices, use_nccl=True) as mo:
            out["nccl_note"] = mo.note()
            p = L.make_params(**CFG3)
            flags = L.MULTI_GATHER_RGBA
            mo.render(p, want=(), flags=flags)                      # grows the buffers, sets the NCCL connections up
            best = None
            for _ in range(2):
                st = mo.render(p, want=(), flags=flags)["stats"]
                if best is None or st.ms_wall < best.ms_wall:
                    best = st
            st = best
            out["bands_cfg3"] = {
                "workload": "16384x16384 'BBBBBBAAAAAA' 500+4000 exact fp64 as %d row band(s), one host thread per device; min/max by "
                            "one all-reduce(MIN) of (min, -max); RGBA8 bands gathered into device 0's frame buffer" % world,
                "ms_wall": st.ms_wall, "ms_lambda_slowest_band": st.ms_lambda_max, "ms_device_slowest_band": st.ms_device_max,
                "steps_per_s_wall": st.executed_steps / (st.ms_wall * 1e-3), "used_nccl": int(st.used_nccl),
                "kernel_launches": int(st.kernel_launches),
                "gather": {"ms": st.ms_gather, "bytes_into_device0": int(st.gather_bytes),
                           "gbs": (st.gather_bytes / (st.ms_gather * 1e-3) / 1e9) if st.ms_gather > 0 else None,
                           "how": "ncclSend on each other device, one group of ncclRecv on device 0" if st.used_nccl else
                                  ("nothing to move on one device" if world == 1 else "cudaMemcpyPeerAsync (NCCL not in use)")}}
            # a zoom batch: 4 frames per device, RGBA8 to pinned host memory
            nf = 4 * world
            frames = [L.make_params(**config5_frame(k)) for k in range(nf)]
            nbytes = 1920 * 1080 * 4
            ptrs = []
            for _ in range(nf):
                q = ctypes.c_void_p()
                L._check(mo.lib.lyap_host_alloc(ctypes.byref(q), nbytes))
                ptrs.append(q.value)
            try:
                mo.render_frames(frames, None, ptrs)
                t0 = time.perf_counter()
                stats = mo.render_frames(frames, None, ptrs)
                wall = time.perf_counter() - t0
            finally:
                for q in ptrs:
                    mo.lib.lyap_host_free(q)
            out["frames_cfg5"] = {
                "workload": "zoom frames 0..%d (1920x1080 'ABC' c=3.7 300+3000), frame k on device k mod %d, RGBA8 out to pinned host memory"
                            % (nf - 1, world),
                "frames": nf, "ms_wall": 1e3 * wall, "frames_per_s": nf / wall,
                "steps_per_s_wall": sum(s.executed_steps for s in stats) / wall}
    except L.LyapError as e:
        out["error"] = str(e)
    return out


if __name__ == "__main__":
    main()
