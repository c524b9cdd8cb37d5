"""Accuracy of the engine's own elementary functions (csrc/lyap_math.h) against mpmath.

These functions define "bit-exact" for the engine (CPU oracle and CUDA kernels share them), so the
test is about their quality, i.e. how far the engine can be from a libm-linked reference."""
import math
import random

import mpmath as mp
import pytest

mp.mp.prec = 200


def ulps(got, exact):
    e = float(exact)
    u = math.ulp(e) if e != 0 else 5e-324
    return float(abs(mp.mpf(got) - exact) / mp.mpf(u))


def test_log_accuracy(port):
    L = port.lib
    rng = random.Random(7)
    worst, worst_abs_near1 = 0.0, 0.0
    for t in range(40000):
        mode = t % 4
        d = (rng.uniform(0, 4), 2.0 ** rng.uniform(-60, 2), rng.uniform(0.9, 1.1), 2.0 ** rng.uniform(-1070, 1023))[mode]
        if d == 0.0:
            continue
        got, ex = L.oracle_log(d), mp.log(mp.mpf(d))
        if abs(float(ex)) >= 2.0 ** -4:
            worst = max(worst, ulps(got, ex))
        else:
            worst_abs_near1 = max(worst_abs_near1, float(abs(mp.mpf(got) - ex)))
    assert worst <= 0.55, worst
    assert worst_abs_near1 < 2.0 ** -57, worst_abs_near1


def test_log_special_values(port):
    L = port.lib
    assert L.oracle_log(2.0) == math.log(2.0) == float.fromhex("0x1.62e42fefa39efp-1")
    assert L.oracle_log(0.0) == -math.inf and L.oracle_log(-0.0) == -math.inf
    assert L.oracle_log(math.inf) == math.inf
    assert math.isnan(L.oracle_log(-1.0)) and math.isnan(L.oracle_log(math.nan))
    assert abs(L.oracle_log(1.0)) < 2.0 ** -58
    d = 5e-324
    assert ulps(L.oracle_log(d), mp.log(mp.mpf(d))) < 0.55
    d = 2.2250738585072014e-308
    assert ulps(L.oracle_log(d), mp.log(mp.mpf(d))) < 0.55


def test_exp_pow_accuracy(port):
    L = port.lib
    rng = random.Random(11)
    worst = 0.0
    for t in range(20000):
        x = rng.uniform(-20, 20) if t % 2 else rng.uniform(-700, 700)
        worst = max(worst, ulps(L.oracle_exp(x), mp.exp(mp.mpf(x))))
    assert worst < 1.0, worst
    assert L.oracle_exp(0.0) == 1.0 and L.oracle_exp(-1000.0) == 0.0 and L.oracle_exp(1000.0) == math.inf
    worst = 0.0
    for y in (1.2, 1.5):
        for t in range(20000):
            x = rng.uniform(0, 1) if t % 2 else 2.0 ** rng.uniform(-300, 1)
            worst = max(worst, ulps(L.oracle_pow(x, y), mp.power(mp.mpf(x), mp.mpf(y))))
    assert worst < 1.5, worst
    assert L.oracle_pow(0.0, 1.2) == 0.0 and L.oracle_pow(1.0, 1.2) == 1.0
    assert math.isnan(L.oracle_pow(-0.5, 1.2))


def test_sin_cos_accuracy(port):
    L = port.lib
    rng = random.Random(13)
    ws = wc = 0.0
    for t in range(40000):
        x = rng.uniform(0, math.pi) if t % 2 else rng.uniform(-30, 30)
        if abs(math.sin(x)) > 1e-3:
            ws = max(ws, ulps(L.oracle_sin(x), mp.sin(mp.mpf(x))))
        if abs(math.cos(x)) > 1e-3:
            wc = max(wc, ulps(L.oracle_cos(x), mp.cos(mp.mpf(x))))
    assert ws < 2.0 and wc < 2.0, (ws, wc)
    assert L.oracle_sin(0.0) == 0.0 and L.oracle_cos(0.0) == 1.0
