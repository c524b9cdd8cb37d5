"""GPU tests of the C ABI's behaviour around the kernels: host entry points, device entry points per
band, error statuses, the progress callback, fast modes within their stated tolerance."""
import ctypes

import numpy as np
import pytest

import lyapunovfractalwasm_b200 as L
from lyapunovfractalwasm_b200 import bands
from conftest import CONFIGS

pytestmark = pytest.mark.gpu


def test_normalize_data_entry_point(engine, port):
    rng = np.random.default_rng(3)
    v = rng.uniform(-6, 1.5, size=100003)
    v[::97] = -5.0
    v[5] = np.nan
    v[6] = np.inf
    v[7] = -np.inf
    got = engine.normalize_data(v)
    assert np.array_equal(got.view(np.uint64), port.normalize(v).view(np.uint64))
    assert np.all(engine.normalize_data(np.full(1000, 0.3)) == 0.0)       # min >= max (:122)
    assert np.all(engine.normalize_data(np.full(7, -5.0)) == 0.0)         # nothing passes the filter
    assert engine.normalize_data(np.empty(0)).size == 0                   # empty in, empty out (:106)
    one = engine.normalize_data(np.array([0.5]))
    assert one[0] == 0.0


def test_colorize_entry_point_all_palettes(engine, port):
    rng = np.random.default_rng(4)
    norm = rng.uniform(0, 1, size=(37, 53))
    norm[0, 0] = 0.0
    norm[1, 1] = 1.0
    norm[2, 2] = 0.5
    for pal in range(7):
        assert np.array_equal(engine.colorize(norm, pal), port.colorize(norm, pal)), pal
    assert np.array_equal(engine.colorize(norm, 42), port.colorize(norm, 0))


def test_device_entry_points_band_by_band(engine, port):
    """Three bands with recomputed halo rows and an exchanged min/max give the single-frame bytes."""
    kw = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=300, height=101, sequence="AABAB", iterations=150,
              warmup=30)
    whole = engine.render(L.make_params(**kw), want=("lambda", "norm", "rgba"))
    backend = bands.GpuBackend(engine, L.make_params)
    world = 3
    local = []
    for rank in range(world):
        b, e = bands.band_rows(kw["height"], world, rank)
        h = backend.lambda_rows(kw, b, e)
        local.append(backend.minmax(h))
    glo, ghi = min(m[0] for m in local), max(m[1] for m in local)
    parts = [bands.render_band(backend, kw, rank, world, lambda lo, hi: (glo, ghi)) for rank in range(world)]
    lam = np.vstack([backend.to_host(p["lambda"]) for p in parts])
    norm = np.vstack([backend.to_host(p["norm"]) for p in parts])
    rgba = np.vstack([backend.to_host(p["rgba"]) for p in parts])
    assert np.array_equal(lam.view(np.uint64), whole["lambda"].view(np.uint64))
    assert np.array_equal(norm.view(np.uint64), whole["norm"].view(np.uint64))
    assert np.array_equal(rgba, whole["rgba"])


def test_error_statuses(engine):
    lib = engine.lib
    out = np.empty(64)

    def status(**kw):
        p = L.make_params(**dict(dict(width=8, height=8, sequence="AB", iterations=10, warmup=2), **kw))
        return lib.lyap_compute_fractal(engine.ctx, ctypes.byref(p), out.ctypes.data, None)

    assert status() == 0
    assert status(sequence="") == 2 and b"empty" in lib.lyap_last_error()
    assert status(width=0) == 1 and status(height=-3) == 1
    assert status(iterations=-1) == 1 and status(warmup=-1) == 1
    assert status(mode=7) == 1 and status(mode=3) == 0
    assert status(mode=1, iterations=2 ** 24) == 3          # the fast modes' 32-bit exponent sums: at most 2^24 steps
    assert status(row_begin=5, row_end=3) == 1 and status(row_begin=0, row_end=9) == 1
    assert status(iterations=20000) == 0                 # a long run of a short sequence wraps round its period
    assert status(iterations=20000, warmup=20000, sequence="".join("AB"[(i * i) % 3 == 0] for i in range(449))) == 3
    p = L.make_params(width=8, height=8, sequence="AB", iterations=10, warmup=2)
    assert lib.lyap_compute_fractal(engine.ctx, ctypes.byref(p), None, None) == 1
    assert lib.lyap_compute_fractal(None, ctypes.byref(p), out.ctypes.data, None) == 1
    # a band cannot be normalised by the host entry point (needs the frame's min/max)
    pb = L.make_params(width=8, height=8, sequence="AB", iterations=10, warmup=2, row_begin=2, row_end=4)
    assert lib.lyap_render(engine.ctx, ctypes.byref(pb), None, None, out.ctypes.data, None, None, None) == 1
    bad = ctypes.c_void_p()
    assert lib.lyap_create(ctypes.byref(bad), 9999) == 1


def test_progress_callback_is_ordered_and_ends_with_one(engine, port):
    kw = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=2048, height=2048, sequence="AB", iterations=60,
              warmup=10)
    seen = []
    lam = engine.compute_fractal(L.make_params(**kw), progress=seen.append)
    assert len(seen) >= 2 and seen[-1] == 1.0
    assert all(0.0 < a < b <= 1.0 for a, b in zip(seen, seen[1:]))
    # chunked launches do not change the result
    again = engine.compute_fractal(L.make_params(**kw))
    assert np.array_equal(lam.view(np.uint64), again.view(np.uint64))


def test_fast_modes_within_stated_tolerance(engine):
    """Fast modes against exact on the config-1 frame.  Stated bounds: fp64 fast mode keeps 99% of the
    stable pixels (lambda < 0, > -4) within 1e-6 relative; fp32 fast mode keeps their median within 1e-5
    relative.  Chaotic pixels (lambda >= 0) agree only statistically: mean lambda over them within 2e-3 (fp64) and
    1e-2 (fp32, whose 24-bit orbits fall into short cycles sooner)."""
    kw = CONFIGS[1]
    exact = engine.render(L.make_params(**kw), want=("lambda",))["lambda"]
    stable = (exact < 0) & (exact > -4)
    chaotic = exact >= 0
    for mode, frac_bound, median_bound, mean_bound in ((L.MODE_FAST_FP64, 0.01, 1e-12, 2e-3),
                                                        (L.MODE_FAST_FP32, 1.0, 1e-5, 1e-2)):
        fast = engine.render(L.make_params(**kw, mode=mode), want=("lambda", "rgba"))
        lam = fast["lambda"]
        # same sentinel pixels, except on the last row / column where a parameter is exactly 4: there
        # the full-range map can land on x == 1.0 at a different step in rearranged arithmetic
        differs = (lam == -5.0) != (exact == -5.0)
        assert not differs[:-1, :-1].any()
        rel = np.abs(lam[stable] - exact[stable]) / np.abs(exact[stable])
        assert np.mean(rel > 1e-6) <= frac_bound, (mode, np.mean(rel > 1e-6))
        assert np.median(rel) < median_bound, (mode, np.median(rel))
        bias = abs(np.mean(lam[chaotic]) - np.mean(exact[chaotic]))
        assert bias < mean_bound, (mode, bias)
        assert fast["rgba"].shape == (512, 512, 4) and np.all(fast["rgba"][..., 3] == 255)


def test_orbit_mode_differs_from_exact_only_by_the_accumulation(engine):
    """LYAP_MODE_FAST_FP64_ORBIT runs the reference's own operations for the orbit and each derivative and only
    accumulates differently (a running product, one log per pixel).  Stated bounds against the exact frame, on config 1
    and on the page call (mid-run exits): the same sentinel pixels everywhere, the same executed steps, |d lambda| below
    1e-12, every stable pixel within 1e-6 relative, and at most one RGBA byte in ten thousand off by one level."""
    page = dict(min_x=0.0, max_x=4.0, min_y=0.0, max_y=4.0, width=800, height=800, sequence="AB", iterations=1000, warmup=100)
    for kw in (CONFIGS[1], page):
        exact = engine.render(L.make_params(**kw), want=("lambda", "rgba"))
        orbit = engine.render(L.make_params(**kw, mode=L.MODE_FAST_FP64_ORBIT), want=("lambda", "rgba"))
        le, lo = exact["lambda"], orbit["lambda"]
        assert np.array_equal(le == -5.0, lo == -5.0)
        assert orbit["stats"].executed_steps == exact["stats"].executed_steps
        assert np.max(np.abs(le - lo)) < 1e-12
        stable = (le < 0) & (le > -4)
        rel = np.abs(lo[stable] - le[stable]) / np.abs(le[stable])
        assert np.mean(rel > 1e-6) == 0.0, np.mean(rel > 1e-6)
        diff = exact["rgba"].astype(int) - orbit["rgba"].astype(int)
        assert np.max(np.abs(diff)) <= 1 and np.mean(diff != 0) < 1e-4, (np.max(np.abs(diff)), np.mean(diff != 0))


def test_peak_microbenchmarks_report_plausible_rates(engine):
    f64, f32 = engine.fp64_peak(), engine.fp32_peak()
    assert 5e12 < f64 < 3e13 and 1e13 < f32 < 6e13


def test_render_multi_bands_equal_single_device(engine):
    """lyap_render_multi with three bands (all on device 0 here) gives the single-device bytes."""
    kw = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=257, height=100, sequence="AABAB", iterations=120,
              warmup=25, palette="aurora")
    one = engine.render(L.make_params(**kw), want=("lambda", "norm", "rgba"))
    multi = L.render_multi(L.make_params(**kw), [0, 0, 0])
    assert np.array_equal(multi["lambda"].view(np.uint64), one["lambda"].view(np.uint64))
    assert np.array_equal(multi["norm"].view(np.uint64), one["norm"].view(np.uint64))
    assert np.array_equal(multi["rgba"], one["rgba"])
    assert multi["stats"].executed_steps == one["stats"].executed_steps
    assert (multi["stats"].lambda_min, multi["stats"].lambda_max) == (one["stats"].lambda_min, one["stats"].lambda_max)


def test_render_multi_deadline_when_a_band_never_arrives(engine):
    """A band whose worker never reaches the min/max exchange (ordinal -1 stands for it) ends the call with
    LYAP_ERR_TIMEOUT after the host-side deadline; no GPU is made to hang for this."""
    import time
    p = L.make_params(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=64, height=32, sequence="AB", iterations=50,
                      warmup=5)
    t0 = time.time()
    with pytest.raises(L.LyapError) as ei:
        L.render_multi(p, [0, -1], timeout_seconds=0.5)
    assert ei.value.status == 6 and "deadline" in str(ei.value)
    assert 0.4 < time.time() - t0 < 10
    # the library is still usable afterwards
    ok = L.render_multi(p, [0, 0], want=("rgba",))
    assert ok["rgba"].shape == (32, 64, 4)
    with pytest.raises(L.LyapError):
        L.render_multi(L.make_params(width=8, height=2, sequence="AB", iterations=5, warmup=1), [0, 0, 0])


def test_cli_reproduces_the_page_call(engine, port, tmp_path):
    """lyap_cli with no arguments is the page's call (800x800, [0,4]^2, 'AB', 1000 iterations, warm-up 100, cosmic)."""
    import json
    import os
    import subprocess
    from lyapunovfractalwasm_b200 import build
    out = tmp_path / "frame.rgba"
    r = subprocess.run([build.CLI, "--out", str(out)], check=True, capture_output=True, text=True)
    info = json.loads(r.stdout.strip().splitlines()[-1])
    assert (info["width"], info["height"], info["sequence"]) == (800, 800, "AB")
    rgba = np.fromfile(out, dtype=np.uint8).reshape(800, 800, 4)
    lam, steps = port.lambda_rows(0.0, 4.0, 0.0, 4.0, 800, 800, "AB", 1000, 100)
    assert info["executed_steps"] == steps
    assert np.array_equal(rgba, port.colorize(port.normalize(lam), 0))
    ppm = tmp_path / "two.ppm"
    subprocess.run([build.CLI, "--config", "1", "--gpus", "2", "--palette", "rainbow", "--out", str(ppm)], check=False)
    if os.path.exists(ppm):   # needs two devices; on a one-GPU box the CLI reports the error instead
        assert ppm.stat().st_size == 512 * 512 * 3 + len(b"P6\n512 512\n255\n")


def test_glow_matches_the_cpu_restatement(engine, port):
    """applyGlow as the engine defines it (the browser defines it in the reference: parity unpinned there)."""
    kw = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=301, height=123, sequence="AB", iterations=150, warmup=30)
    rgba = engine.render(L.make_params(**kw), want=("rgba",))["rgba"]
    got = engine.glow(rgba)
    want = port.glow(rgba)
    assert np.array_equal(got, want)
    assert np.all(got[..., 3] == 255) and np.all(got[..., :3].astype(int) >= rgba[..., :3].astype(int))   # 'screen' only brightens
    tiny = np.zeros((3, 5, 4), dtype=np.uint8)
    tiny[..., 3] = 255
    tiny[1, 2, :3] = 200
    assert np.array_equal(engine.glow(tiny), port.glow(tiny))


def test_render_frames_batch_equals_frame_by_frame(engine, port):
    """lyap_render_frames (two buffer sets, copies on their own stream) against lyap_render frame by frame and the
    oracle: frames of different sizes and sequences, more frames than buffer sets, the same device listed twice."""
    from conftest import config5_frame
    frames_kw = [dict(config5_frame(k), width=320, height=180, iterations=300, warmup=30) for k in (0, 20, 40, 60, 80)]
    frames_kw.insert(2, dict(min_x=2.0, max_x=4.0, min_y=2.0, max_y=4.0, width=257, height=131, sequence="AB",
                             iterations=200, warmup=20))
    frames_kw.append(dict(min_x=0.0, max_x=4.0, min_y=0.0, max_y=4.0, width=64, height=48, sequence="BBA",
                          iterations=100, warmup=10, palette=3))
    frames = [L.make_params(**kw) for kw in frames_kw]
    for devices, pinned in (([0], False), ([0, 0], True)):
        out, stats = L.render_frames(frames, devices, pinned=pinned)
        for i, kw in enumerate(frames_kw):
            one = engine.render(frames[i], want=("norm", "rgba"))
            assert np.array_equal(out["norm"][i].view(np.uint64), one["norm"].view(np.uint64)), i
            assert np.array_equal(out["rgba"][i], one["rgba"]), i
            st = stats[i]
            assert st.executed_steps == one["stats"].executed_steps and st.nominal_steps == one["stats"].nominal_steps
            assert (st.lambda_min, st.lambda_max) == (one["stats"].lambda_min, one["stats"].lambda_max)
            assert st.ms_lambda > 0 and st.ms_total_device >= st.ms_lambda and st.ms_copies > 0
        lam, _ = port.lambda_rows(*[frames_kw[2][k] for k in ("min_x", "max_x", "min_y", "max_y", "width", "height",
                                                               "sequence", "iterations", "warmup")])
        assert np.array_equal(out["norm"][2].view(np.uint64), port.normalize(lam).view(np.uint64))
    # only RGBA wanted; no frames at all
    out, stats = L.render_frames(frames[:3], [0], want=("rgba",))
    assert "norm" not in out and np.array_equal(out["rgba"][1], engine.render(frames[1], want=("rgba",))["rgba"])
    out, stats = L.render_frames([], [0])
    assert out == {"norm": [], "rgba": []} and stats == []


def test_multi_object_gather_and_reuse(engine):
    """lyap_multi on this device listed three times (NCCL cannot have one GPU twice, so the object takes its host
    exchange and peer-copy gather; the NCCL legs run where there are distinct devices): the gathered RGBA8 / fp32
    lambda frames in the first device's memory and every host output equal the one-device render; the object is reused
    for another frame size and for a frame batch without being rebuilt."""
    kw = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=301, height=100, sequence="AABAB", iterations=120,
              warmup=25, palette="nebula")
    one = engine.render(L.make_params(**kw), want=("lambda", "lambda32", "norm", "rgba"))
    with L.Multi([0, 0, 0], use_nccl=True) as m:
        assert "more than once" in m.note()
        r = m.render(L.make_params(**kw), want=("lambda", "lambda32", "norm", "rgba"),
                     flags=L.MULTI_GATHER_RGBA | L.MULTI_GATHER_LAMBDA32)
        st = r["stats"]
        assert st.used_nccl == 0 and st.gather_bytes == 2 * (100 - 34) * 301 * 4 and st.ms_gather > 0
        assert np.array_equal(r["lambda"].view(np.uint64), one["lambda"].view(np.uint64))
        assert np.array_equal(r["lambda32"], one["lambda32"])
        assert np.array_equal(r["norm"].view(np.uint64), one["norm"].view(np.uint64))
        assert np.array_equal(r["rgba"], one["rgba"])
        assert st.executed_steps == one["stats"].executed_steps
        assert (st.lambda_min, st.lambda_max) == (one["stats"].lambda_min, one["stats"].lambda_max)
        # the gathered frames themselves, read back from the first device
        d_rgba, d_l32 = m.gathered()
        got = np.empty((100, 301, 4), dtype=np.uint8)
        L._check(engine.lib.lyap_copy_to_host(engine.ctx, got.ctypes.data, d_rgba, got.nbytes))
        assert np.array_equal(got, one["rgba"])
        got32 = np.empty((100, 301), dtype=np.float32)
        L._check(engine.lib.lyap_copy_to_host(engine.ctx, got32.ctypes.data, d_l32, got32.nbytes))
        assert np.array_equal(got32, one["lambda32"])
        # gather only (no host buffers), a larger frame, then without gather
        kw2 = dict(kw, width=640, height=333, sequence="AB", palette="cosmic")
        one2 = engine.render(L.make_params(**kw2), want=("rgba",))
        r2 = m.render(L.make_params(**kw2), want=(), flags=L.MULTI_GATHER_RGBA)
        d_rgba, _ = m.gathered()
        got = np.empty((333, 640, 4), dtype=np.uint8)
        L._check(engine.lib.lyap_copy_to_host(engine.ctx, got.ctypes.data, d_rgba, got.nbytes))
        assert np.array_equal(got, one2["rgba"]) and r2["stats"].gather_bytes == (333 - 111) * 640 * 4
        r3 = m.render(L.make_params(**kw2), want=("rgba",))
        assert np.array_equal(r3["rgba"], one2["rgba"]) and r3["stats"].gather_bytes == 0
        # lambda only: no colour stage, no exchange needed
        r4 = m.render(L.make_params(**kw), want=("lambda",))
        assert np.array_equal(r4["lambda"].view(np.uint64), one["lambda"].view(np.uint64))
        # a batch of frames on the same object
        frames = [L.make_params(**dict(kw, width=64 + 16 * i, height=40 + i)) for i in range(5)]
        norms = [np.empty((f.height, f.width)) for f in frames]
        rgbas = [np.empty((f.height, f.width, 4), dtype=np.uint8) for f in frames]
        stats = m.render_frames(frames, [a.ctypes.data for a in norms], [a.ctypes.data for a in rgbas])
        for f, nrm, img, fs in zip(frames, norms, rgbas, stats):
            ref = engine.render(f, want=("norm", "rgba"))
            assert np.array_equal(nrm.view(np.uint64), ref["norm"].view(np.uint64)) and np.array_equal(img, ref["rgba"])
            assert fs.executed_steps == ref["stats"].executed_steps


def test_multi_object_single_device_with_nccl(engine):
    """One device, NCCL asked for: a one-rank communicator; the min/max all-reduce goes through it."""
    kw = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=200, height=64, sequence="AB", iterations=100, warmup=10)
    one = engine.render(L.make_params(**kw), want=("norm", "rgba"))
    with L.Multi([0], use_nccl=True) as m:
        r = m.render(L.make_params(**kw), want=("norm", "rgba"), flags=L.MULTI_GATHER_RGBA)
        assert m.note() == "" and r["stats"].used_nccl == 1
        assert np.array_equal(r["norm"].view(np.uint64), one["norm"].view(np.uint64))
        assert np.array_equal(r["rgba"], one["rgba"])
        r = m.render(L.make_params(**kw), want=("rgba",), flags=L.MULTI_HOST_EXCHANGE)
        assert r["stats"].used_nccl == 0 and np.array_equal(r["rgba"], one["rgba"])


def test_multi_object_deadline_and_errors(engine):
    import time
    p = L.make_params(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=64, height=32, sequence="AB", iterations=50, warmup=5)
    with L.Multi([0, -1], use_nccl=True) as m:      # a band that never arrives: no NCCL, the deadline fires on the host
        assert "no device" in m.note()
        t0 = time.time()
        with pytest.raises(L.LyapError) as ei:
            m.render(p, want=("rgba",), flags=L.MULTI_GATHER_RGBA, timeout_seconds=0.4)
        assert ei.value.status == 6 and 0.3 < time.time() - t0 < 10
    with L.Multi([0, 0]) as m:
        with pytest.raises(L.LyapError) as ei:
            m.render(L.make_params(width=8, height=8, sequence="", iterations=5, warmup=1))
        assert ei.value.status == 2
        with pytest.raises(L.LyapError) as ei:
            m.render(L.make_params(width=8, height=1, sequence="AB", iterations=5, warmup=1))
        assert ei.value.status == 1                   # more bands than rows
        ok = m.render(p, want=("rgba",))               # still usable
        assert ok["rgba"].shape == (32, 64, 4)
    with pytest.raises(L.LyapError):
        L.Multi([9999])


def test_drop_in_header_program_runs_and_matches_the_oracle(port, engine, tmp_path):
    """A program written against the reference's header API (struct, computeFractal with a callback, normalizeData:
    the calls of src/wasm_bindings.cpp:112-119) compiled against include/lyapunov_fractal.hpp and RUN: its lambda and
    normalised arrays equal the oracle's."""
    import os
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = tmp_path / "user.cpp"
    src.write_text(
        '#include "lyapunov_fractal.hpp"\n'
        "#include <cstdio>\n"
        "static int calls = 0; static double last = 0;\n"
        "static void cb(double f) { ++calls; last = f; }\n"
        "int main(int, char** argv) {\n"
        "  lyapunov::FractalComputer::ComputationParams params;\n"
        "  params.min_x = 2.4; params.max_x = 4.0; params.min_y = 2.5; params.max_y = 3.9;\n"
        '  params.width = 200; params.height = 90; params.sequence = "ABBAB"; params.iterations = 150; params.warmup = 30;\n'
        "  lyapunov::FractalComputer computer;\n"
        "  std::vector<double> fractal_data = computer.computeFractal(params, cb);\n"
        "  std::vector<double> normalized_data = lyapunov::normalizeData(fractal_data);\n"
        '  FILE* f = std::fopen(argv[1], "wb");\n'
        "  std::fwrite(fractal_data.data(), 8, fractal_data.size(), f);\n"
        "  std::fwrite(normalized_data.data(), 8, normalized_data.size(), f);\n"
        "  std::fclose(f);\n"
        "  return (calls >= 1 && last == 1.0 && normalized_data.size() == 18000) ? 0 : 1;\n"
        "}\n")
    exe, out = tmp_path / "user", tmp_path / "out.bin"
    libdir = os.path.join(root, "lyapunovfractalwasm_b200")
    subprocess.run(["g++", "-std=c++23", "-Wall", "-Werror", "-I", os.path.join(root, "include"), str(src),
                    "-L", libdir, "-llyap_b200", "-Wl,-rpath," + libdir, "-o", str(exe)], check=True)
    subprocess.run([str(exe), str(out)], check=True)
    data = np.fromfile(out, dtype=np.float64)
    lam, _ = port.lambda_rows(2.4, 4.0, 2.5, 3.9, 200, 90, "ABBAB", 150, 30)
    assert np.array_equal(data[:18000].view(np.uint64), lam.ravel().view(np.uint64))
    assert np.array_equal(data[18000:].view(np.uint64), port.normalize(lam).ravel().view(np.uint64))


def device_count(lib):
    n = ctypes.c_int(0)
    lib.lyap_device_count(ctypes.byref(n))
    return n.value


def test_multi_object_on_distinct_devices_with_nccl(engine):
    """Needs two or more GPUs (skipped on a one-GPU box): every device its own band, the frame's min/max by one NCCL
    all-reduce, the RGBA8 and fp32 lambda bands gathered into device 0 by ncclSend / grouped ncclRecv.  The bytes equal
    the one-device render, the host-assembled frame (no gather, host exchange) and the peer-copy gather."""
    n = device_count(engine.lib)
    if n < 2:
        pytest.skip("one GPU here")
    n = min(n, 8)
    kw = dict(min_x=2.5, max_x=4.0, min_y=2.5, max_y=4.0, width=1500, height=1003, sequence="AABAB", iterations=300,
              warmup=40, palette="aurora")
    one = engine.render(L.make_params(**kw), want=("lambda", "lambda32", "norm", "rgba"))
    with L.Multi(list(range(n)), use_nccl=True) as m:
        assert m.note() == ""
        for _ in range(2):     # second pass: warm connections, reused buffers
            r = m.render(L.make_params(**kw), want=("lambda", "lambda32", "norm", "rgba"),
                         flags=L.MULTI_GATHER_RGBA | L.MULTI_GATHER_LAMBDA32)
            st = r["stats"]
            assert st.used_nccl == 1 and st.ms_gather > 0
            own0 = 1003 // n + (1 if 1003 % n else 0)
            assert st.gather_bytes == 2 * (1003 - own0) * 1500 * 4
            assert np.array_equal(r["lambda"].view(np.uint64), one["lambda"].view(np.uint64))
            assert np.array_equal(r["lambda32"], one["lambda32"])
            assert np.array_equal(r["norm"].view(np.uint64), one["norm"].view(np.uint64))
            assert np.array_equal(r["rgba"], one["rgba"])
            assert st.executed_steps == one["stats"].executed_steps
            assert (st.lambda_min, st.lambda_max) == (one["stats"].lambda_min, one["stats"].lambda_max)
        host = m.render(L.make_params(**kw), want=("norm", "rgba"), flags=L.MULTI_HOST_EXCHANGE)
        assert host["stats"].used_nccl == 0 and host["stats"].gather_bytes == 0
        assert np.array_equal(host["rgba"], one["rgba"]) and np.array_equal(host["norm"].view(np.uint64), one["norm"].view(np.uint64))
        peer = m.render(L.make_params(**kw), want=("rgba",), flags=L.MULTI_HOST_EXCHANGE | L.MULTI_GATHER_RGBA)
        assert peer["stats"].used_nccl == 0 and peer["stats"].gather_bytes == (1003 - own0) * 1500 * 4
        assert np.array_equal(peer["rgba"], one["rgba"])
        # frames of a batch dealt to distinct devices
        frames = [L.make_params(**dict(kw, width=200 + 8 * i, height=120 + i, iterations=100)) for i in range(2 * n + 1)]
        rgbas = [np.empty((f.height, f.width, 4), dtype=np.uint8) for f in frames]
        m.render_frames(frames, None, [a.ctypes.data for a in rgbas])
        for f, img in zip(frames, rgbas):
            assert np.array_equal(img, engine.render(f, want=("rgba",))["rgba"])
    # the one-call form over distinct devices
    multi = L.render_multi(L.make_params(**kw), list(range(n)))
    assert np.array_equal(multi["rgba"], one["rgba"]) and np.array_equal(multi["lambda"].view(np.uint64), one["lambda"].view(np.uint64))
