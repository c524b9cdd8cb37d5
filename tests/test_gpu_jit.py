"""The instances of the lambda kernels made for one sequence -- compiled with the library (csrc/lyap_prebuilt.cu) or at
run time (csrc/lyap_jit.cu) -- against the CPU oracle and against the generic kernel: same bits, same executed-step
counts.  The kernel_path fixture picks which of the three a launch takes."""
import os

import numpy as np
import pytest

import lyapunovfractalwasm_b200 as L
from conftest import CONFIGS, config5_frame

pytestmark = pytest.mark.gpu


def oracle(port, kw):
    return port.lambda_rows(kw["min_x"], kw["max_x"], kw["min_y"], kw["max_y"], kw["width"], kw["height"],
                            kw["sequence"], kw["iterations"], kw["warmup"], c=kw.get("c"))


CASES = [
    dict(sequence="AB", iterations=1000, warmup=100),                  # period 2: one group pattern
    dict(sequence="AABAB", iterations=333, warmup=37),                 # period 5 -> 5 group patterns, odd warm-up phase
    dict(sequence="BBBBBBAAAAAA", iterations=500, warmup=500),         # period 12, accumulation starts at phase 8
    dict(sequence="ABC", iterations=301, warmup=29, c=3.7),            # three parameters
    dict(sequence="ABC", iterations=301, warmup=29),                   # 'C' is B without the extension
    dict(sequence="A", iterations=77, warmup=5),                       # period 1
    dict(sequence="ABBABAABBBABAABABBBAABAB" * 3 + "A", iterations=200, warmup=20),   # no short period: precompiled kernel
    dict(sequence="AB", iterations=7, warmup=3),                       # shorter than one chunk
    dict(sequence="AAB", iterations=18, warmup=18),                    # exactly one chunk of three periods
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: "%s_%d_%d" % (c["sequence"][:12], c["iterations"], c["warmup"]))
def test_specialised_kernel_is_bit_exact(engine, port, kernel_path, case):
    kw = dict(min_x=2.3, max_x=4.1, min_y=2.2, max_y=4.05, width=333, height=67, **case)
    want, steps = oracle(port, kw)
    got = {}
    names = {}
    for mode in ("jit", "prebuilt", "generic"):
        kernel_path(mode)
        r = engine.render(L.make_params(**kw), want=("lambda",))
        assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64)), mode
        assert r["stats"].executed_steps == steps, mode
        got[mode] = r["lambda"]
        names[mode] = engine.lib.lyap_last_kernel().decode()
    assert np.array_equal(got["generic"].view(np.uint64), got["jit"].view(np.uint64))
    assert engine.lib.lyap_jit_note() == b""      # nothing fell back
    assert "generic" in names["generic"]
    periodic = len(case["sequence"]) <= 12
    assert ("compiled at run time" in names["jit"]) == periodic, names
    if case == CASES[0]:
        assert "built for the patterns" in names["prebuilt"], names


def test_specialised_kernel_on_the_page_call_with_mid_run_exits(engine, port, kernel_path):
    kw = dict(min_x=0.0, max_x=4.0, min_y=0.0, max_y=4.0, width=800, height=800, sequence="AB", iterations=1000, warmup=100)
    want, steps = oracle(port, kw)
    for mode in ("jit", "prebuilt"):
        kernel_path(mode)
        r = engine.render(L.make_params(**kw), want=("lambda",))
        assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64)) and r["stats"].executed_steps == steps, mode
        assert "generic" not in engine.lib.lyap_last_kernel().decode()


def test_every_benchmark_sequence_has_a_prebuilt_instance(engine, port, kernel_path):
    """Bands of the five benchmark frames (and "ABC" without the third parameter): the library's own instance for the
    sequence is what launches -- no run-time compiler involved -- and it gives the oracle's bits; so does NVRTC's."""
    shapes = [(CONFIGS[1], 100, 140), (CONFIGS[2], 1000, 1016), (CONFIGS[3], 9000, 9004), (CONFIGS[4], 40000, 40001),
              (config5_frame(3), 100, 108), (dict(config5_frame(3), c=None), 100, 108)]
    for kw, y0, y1 in shapes:
        kw = dict(kw)
        c = kw.pop("c", None)
        want, _ = port.lambda_rows(kw["min_x"], kw["max_x"], kw["min_y"], kw["max_y"], kw["width"], kw["height"],
                                   kw["sequence"], kw["iterations"], kw["warmup"], c=c, y0=y0, y1=y1)
        for mode in ("prebuilt", "jit"):
            kernel_path(mode)
            lam = engine.compute_fractal(L.make_params(**kw, c=c, row_begin=y0, row_end=y1))
            assert np.array_equal(lam.view(np.uint64), want.view(np.uint64)), (kw["sequence"], mode)
            name = engine.lib.lyap_last_kernel().decode()
            assert ("built for the patterns" in name) == (mode == "prebuilt"), (kw["sequence"], mode, name)
        for fast in (L.MODE_FAST_FP64, L.MODE_FAST_FP32, L.MODE_FAST_FP64_ORBIT):
            kernel_path("prebuilt")
            engine.render(L.make_params(**kw, c=c, row_begin=y0, row_end=y1, mode=fast), want=("lambda",))
            assert "built for the patterns" in engine.lib.lyap_last_kernel().decode(), (kw["sequence"], fast)


def test_no_warmup_many_small_launches(engine, port, kernel_path):
    """warmup = 0: the first logarithm comes right after the kernel has filled its shared-memory tables, so a missing
    barrier between the fill and the first look-up would show here.  Many small launches, every kernel path."""
    rng = np.random.default_rng(5)
    shapes = [(int(rng.integers(1, 2000)), int(rng.integers(1, 5))) for _ in range(40)] + [(1536, 148), (4096, 37)]
    for seq in ("AB", "AABAB"):
        for mode in ("generic", "prebuilt", "jit"):
            kernel_path(mode)
            for w, h in shapes:
                kw = dict(min_x=2.5, max_x=3.99, min_y=2.6, max_y=3.97, width=w, height=h, sequence=seq, iterations=24, warmup=0)
                r = engine.render(L.make_params(**kw), want=("lambda",))
                want, steps = oracle(port, kw)
                assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64)), (seq, mode, w, h)
                assert r["stats"].executed_steps == steps


@pytest.mark.parametrize("mode", [L.MODE_FAST_FP64, L.MODE_FAST_FP32, L.MODE_FAST_FP64_ORBIT])
def test_specialised_fast_kernels_agree_with_the_precompiled_ones(engine, kernel_path, mode):
    """Fast modes: moving the exponent out of the running product is exact, so where the products are stripped does
    not change their value: pixels whose run was regular get the precompiled kernel's bits.  Pixels that had a chunk
    redone step by step (an exit, a zero derivative) may differ in the last digits, because the two kernels cut the
    run into chunks at different steps and a redone chunk adds logs one by one instead of multiplying."""
    tol = 2e-4 if mode == L.MODE_FAST_FP32 else 1e-10
    for case in CASES[:6]:
        kw = dict(min_x=2.3, max_x=4.1, min_y=2.2, max_y=4.05, width=257, height=45, mode=mode, **case)
        got = {}
        for m in ("jit", "prebuilt", "generic"):
            kernel_path(m)
            r = engine.render(L.make_params(**kw), want=("lambda",))
            got[m] = (r["lambda"], r["stats"].executed_steps)
        for m in ("jit", "prebuilt"):
            same = got["generic"][0].view(np.uint64) == got[m][0].view(np.uint64)
            assert same.mean() > 0.9, (case, m, same.mean())
            assert np.array_equal(got["generic"][0] == -5.0, got[m][0] == -5.0)
            assert np.max(np.abs(got["generic"][0] - got[m][0])) < tol, (case, m)
            assert got["generic"][1] == got[m][1], (case, m)
    assert engine.lib.lyap_jit_note() == b""


LONG_RUNS = [
    dict(sequence="AB", iterations=20011, warmup=3001),                # beyond the 14336 steps the selector table holds:
    dict(sequence="AABAB", iterations=30005, warmup=17),               # the regions are walked by the sequence's period
    dict(sequence="BBBBBBAAAAAA", iterations=9000, warmup=9000),
    dict(sequence="ABCAC", iterations=15000, warmup=2000, c=3.3),
    dict(sequence="ABBABAABBBABAABABBBAABABAABBBABBAAABABBBABAABBABAAABBBABABBAABBAB", iterations=16000, warmup=1000),
    dict(sequence="ABBABAABBBABAABABBBAABABAABBBABBAAABABBBABAABBABAAABBBABABBAABBABA", iterations=16001, warmup=999),
]


@pytest.mark.parametrize("case", LONG_RUNS, ids=lambda c: "%d_%d_%d" % (len(c["sequence"]), c["iterations"], c["warmup"]))
def test_runs_longer_than_the_selector_table(engine, port, kernel_path, case):
    """Specialised and precompiled kernels, exact mode, bit for bit; the fast modes on the same frame to their tolerance."""
    kw = dict(min_x=2.4, max_x=4.0, min_y=2.4, max_y=4.0, width=50, height=21, **case)
    want, steps = oracle(port, kw)
    for mode in ("jit", "generic"):
        kernel_path(mode)
        r = engine.render(L.make_params(**kw), want=("lambda",))
        assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64)), mode
        assert r["stats"].executed_steps == steps, mode
        for fast, tol in ((L.MODE_FAST_FP64, 1e-9), (L.MODE_FAST_FP32, 5e-2)):
            f = engine.render(L.make_params(**kw, mode=fast), want=("lambda",))["lambda"][:-1, :-1]
            w = want[:-1, :-1]
            assert np.array_equal(f == -5.0, w == -5.0)
            assert np.median(np.abs(f - w)) < tol, (mode, fast)


def test_default_mode_compiles_in_the_background(engine, port):
    """The default (LYAP_JIT=1): once about 2e10 steps of work with a sequence have been asked for, an instance is
    compiled on a background thread; launches meanwhile use the generic kernel (no stall), later ones the new instance,
    and the bits are the same before and after."""
    import os
    import time
    old = {k: os.environ.get(k) for k in ("LYAP_JIT", "LYAP_PREBUILT")}
    os.environ["LYAP_JIT"], os.environ["LYAP_PREBUILT"] = "1", "0"
    try:
        kw = dict(min_x=2.6, max_x=3.95, min_y=2.7, max_y=3.9, width=1024, height=1024, sequence="ABAAB", iterations=9000,
                  warmup=1000)                                          # 1.05e10 steps a frame
        small = dict(kw, width=96, height=8)
        want, _ = oracle(port, small)
        first = engine.render(L.make_params(**kw), want=("lambda",))["lambda"]
        assert "generic" in engine.lib.lyap_last_kernel().decode()       # below the threshold
        t0 = time.time()
        second = engine.render(L.make_params(**kw), want=("lambda",))["lambda"]     # crosses it: compilation starts, no wait
        assert time.time() - t0 < 0.5 and "generic" in engine.lib.lyap_last_kernel().decode()
        name = ""
        while time.time() - t0 < 60 and "compiled at run time" not in name:
            time.sleep(0.2)
            r = engine.render(L.make_params(**small), want=("lambda",))
            assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64))
            # the small frame takes another shape (2 pixels per thread): keep asking with the large one's shape too
            third = engine.render(L.make_params(**kw), want=("lambda",))["lambda"]
            name = engine.lib.lyap_last_kernel().decode()
        assert "compiled at run time" in name, (name, engine.lib.lyap_jit_note())
        assert np.array_equal(first.view(np.uint64), second.view(np.uint64))
        assert np.array_equal(first.view(np.uint64), third.view(np.uint64))
    finally:
        for k, v in old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v
