"""The run-time specialised instance of the exact kernel (csrc/lyap_jit.cu) against the CPU oracle and against the
precompiled kernel: same bits, same executed-step counts.  LYAP_JIT=2 compiles on first use, 0 turns it off."""
import os

import numpy as np
import pytest

import lyapunovfractalwasm_b200 as L
from conftest import CONFIGS, config5_frame

pytestmark = pytest.mark.gpu


@pytest.fixture()
def jit_mode():
    old = os.environ.get("LYAP_JIT")

    def set_mode(m):
        os.environ["LYAP_JIT"] = str(m)
    yield set_mode
    if old is None:
        os.environ.pop("LYAP_JIT", None)
    else:
        os.environ["LYAP_JIT"] = old


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
def test_specialised_kernel_is_bit_exact(engine, port, jit_mode, case):
    kw = dict(min_x=2.3, max_x=4.1, min_y=2.2, max_y=4.05, width=333, height=67, **case)
    want, steps = oracle(port, kw)
    got = {}
    for mode in (2, 0):
        jit_mode(mode)
        r = engine.render(L.make_params(**kw), want=("lambda",))
        assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64)), mode
        assert r["stats"].executed_steps == steps, mode
        got[mode] = r["lambda"]
    assert np.array_equal(got[0].view(np.uint64), got[2].view(np.uint64))
    assert engine.lib.lyap_jit_note() == b""      # nothing fell back


def test_specialised_kernel_on_the_page_call_with_mid_run_exits(engine, port, jit_mode):
    jit_mode(2)
    kw = dict(min_x=0.0, max_x=4.0, min_y=0.0, max_y=4.0, width=800, height=800, sequence="AB", iterations=1000, warmup=100)
    r = engine.render(L.make_params(**kw), want=("lambda",))
    want, steps = oracle(port, kw)
    assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64)) and r["stats"].executed_steps == steps


def test_specialised_kernel_on_benchmark_shapes(engine, port, jit_mode):
    jit_mode(2)
    kw = CONFIGS[2]
    lam = engine.compute_fractal(L.make_params(**kw, row_begin=1000, row_end=1016))
    want, _ = port.lambda_rows(kw["min_x"], kw["max_x"], kw["min_y"], kw["max_y"], kw["width"], kw["height"],
                               kw["sequence"], kw["iterations"], kw["warmup"], y0=1000, y1=1016)
    assert np.array_equal(lam.view(np.uint64), want.view(np.uint64))
    kw = config5_frame(3)
    lam = engine.compute_fractal(L.make_params(**kw, row_begin=100, row_end=108))
    want, _ = port.lambda_rows(kw["min_x"], kw["max_x"], kw["min_y"], kw["max_y"], kw["width"], kw["height"],
                               kw["sequence"], kw["iterations"], kw["warmup"], c=kw["c"], y0=100, y1=108)
    assert np.array_equal(lam.view(np.uint64), want.view(np.uint64))


@pytest.mark.parametrize("mode", [L.MODE_FAST_FP64, L.MODE_FAST_FP32])
def test_specialised_fast_kernels_agree_with_the_precompiled_ones(engine, jit_mode, mode):
    """Fast modes: moving the exponent out of the running product is exact, so where the products are stripped does
    not change their value: pixels whose run was regular get the precompiled kernel's bits.  Pixels that had a chunk
    redone step by step (an exit, a zero derivative) may differ in the last digits, because the two kernels cut the
    run into chunks at different steps and a redone chunk adds logs one by one instead of multiplying."""
    tol = 1e-10 if mode == L.MODE_FAST_FP64 else 2e-4
    for case in CASES[:6]:
        kw = dict(min_x=2.3, max_x=4.1, min_y=2.2, max_y=4.05, width=257, height=45, mode=mode, **case)
        got = {}
        for m in (2, 0):
            jit_mode(m)
            r = engine.render(L.make_params(**kw), want=("lambda",))
            got[m] = (r["lambda"], r["stats"].executed_steps)
        same = got[0][0].view(np.uint64) == got[2][0].view(np.uint64)
        assert same.mean() > 0.9, (case, same.mean())
        assert np.array_equal(got[0][0] == -5.0, got[2][0] == -5.0)
        assert np.max(np.abs(got[0][0] - got[2][0])) < tol, case
        assert got[0][1] == got[2][1], case
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
def test_runs_longer_than_the_selector_table(engine, port, jit_mode, case):
    """Specialised and precompiled kernels, exact mode, bit for bit; the fast modes on the same frame to their tolerance."""
    kw = dict(min_x=2.4, max_x=4.0, min_y=2.4, max_y=4.0, width=50, height=21, **case)
    want, steps = oracle(port, kw)
    for mode in (2, 0):
        jit_mode(mode)
        r = engine.render(L.make_params(**kw), want=("lambda",))
        assert np.array_equal(r["lambda"].view(np.uint64), want.view(np.uint64)), mode
        assert r["stats"].executed_steps == steps, mode
        for fast, tol in ((L.MODE_FAST_FP64, 1e-9), (L.MODE_FAST_FP32, 5e-2)):
            f = engine.render(L.make_params(**kw, mode=fast), want=("lambda",))["lambda"][:-1, :-1]
            w = want[:-1, :-1]
            assert np.array_equal(f == -5.0, w == -5.0)
            assert np.median(np.abs(f - w)) < tol, (mode, fast)
