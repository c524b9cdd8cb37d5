#!/usr/bin/env python3
"""Generate lyap_tables.h: every constant used by lyap_math.h.

The engine's exact mode must give the same bits on the CPU (oracle) and on the
GPU, so its transcendental functions are this project's own: a table-driven
natural logarithm (1024 bins, cubic correction) plus polynomial exp / sin / cos.
This script derives all tables and coefficients from first principles with
mpmath (arbitrary precision) and writes them as hexadecimal floating literals.

log(d), d = 2^(ke-1023) * m, m in [1,2), bin i = top 10 mantissa bits:
    r   = m*invc[i] - 1                     |r| <= ~2^-11
    log = (ke-1023)*ln2 + L[i] + log1p(r),  L[i] = -log(invc[i])
invc[i] is chosen (a search over nearby grid points) such that L[i] lies on the
2^-42 grid up to a residual < 2^-61; ln2hi is ln2 truncated to that grid.  Then
(ke-1023)*ln2hi + L[i] is exact in one fma and the only significant rounding is
the last addition.

Run:  python gen_tables.py > lyap_tables.h
"""
import sys
from fractions import Fraction
import mpmath as mp

mp.mp.prec = 260
NB = 1024          # bins
GRID = 42          # L and ln2hi are multiples of 2^-GRID
SEARCH = 8192      # candidates per bin, each side
STRIDE = 997       # grid-point stride between candidates (window +-2^-19 relative)


def to_double(x):
    """Round an mpf to the nearest double, returned as Python float."""
    return float(mp.mpf(x))


def hexf(x):
    return float(x).hex()


def frac_of_float(x):
    return Fraction(float(x))


def is_exact_double(fr):
    return Fraction(float(fr)) == fr


def gen_log():
    g = mp.mpf(2) ** -GRID
    ln2 = mp.log(2)
    ln2hi_fr = Fraction(int(mp.floor(ln2 * 2 ** GRID)), 2 ** GRID)
    assert is_exact_double(ln2hi_fr)
    ln2hi = float(ln2hi_fr)
    ln2lo = to_double(ln2 - mp.mpf(ln2hi_fr.numerator) / ln2hi_fr.denominator)
    klo_bias = to_double(-1023 * mp.mpf(ln2lo))
    rows = []
    worst_resid = 0
    rmax = 0
    for i in range(NB):
        c = mp.mpf(1) + (mp.mpf(i) + mp.mpf(1) / 2) / NB
        j0 = int(mp.nint(mp.log(c) / g))
        # candidates j = j0 + t*STRIDE, |t| <= SEARCH, walked in 240-bit fixed point
        FP = 240
        jlo = j0 - SEARCH * STRIDE
        e_fx = int(mp.floor(mp.exp(-mp.mpf(jlo) * g) * 2 ** FP))
        q_fx = int(mp.floor(mp.exp(-mp.mpf(STRIDE) * g) * 2 ** FP))
        best = None
        sh = FP - 53                      # e in [0.5,1): ulp = 2^-53
        half = 1 << (sh - 1)
        mask = (1 << sh) - 1
        for t in range(2 * SEARCH + 1):
            fracpart = e_fx & mask
            dist = fracpart if fracpart < half else (1 << sh) - fracpart
            if best is None or dist < best[0]:
                best = (dist, jlo + t * STRIDE)
            e_fx = (e_fx * q_fx) >> FP
        j = best[1]
        e = mp.exp(-mp.mpf(j) * g)
        ed = to_double(e)
        best = (abs((e - mp.mpf(ed)) / e), j, ed)
        delta, j, invc = best
        L_fr = Fraction(j, 2 ** GRID)
        Lp_fr = L_fr - 1023 * ln2hi_fr
        assert is_exact_double(L_fr) and is_exact_double(Lp_fr), i
        # true residual
        resid = abs(-mp.log(mp.mpf(invc)) - mp.mpf(j) * g)
        worst_resid = max(worst_resid, resid)
        lo_m = mp.mpf(1) + mp.mpf(i) / NB
        hi_m = mp.mpf(1) + mp.mpf(i + 1) / NB
        rmax = max(rmax, abs(lo_m * invc - 1), abs(hi_m * invc - 1))
        rows.append((float(Lp_fr), invc, float(L_fr)))
    return ln2hi, ln2lo, klo_bias, rows, worst_resid, rmax


def fit_even_or_general(func, a, b, deg):
    """Near-minimax polynomial (Chebyshev fit) of func on [a,b]; coefficients low->high."""
    coeffs = mp.chebyfit(func, [a, b], deg + 1)
    return [to_double(cf) for cf in reversed(coeffs)]


def main():
    out = []
    w = out.append
    ln2hi, ln2lo, klo_bias, rows, worst_resid, rmax = gen_log()
    R = rmax * mp.mpf("1.0005")

    def f(r):
        if r == 0:
            return mp.mpf(-1) / 2
        return (mp.log1p(r) - r) / (r * r)

    c = fit_even_or_general(f, -R, R, 2)   # q(r) = c2 + c3 r + c4 r^2

    # exp: Taylor coefficients 1/k!, k = 2..14 (|r| <= ln2/2)
    exp_c = [to_double(mp.mpf(1) / mp.factorial(k)) for k in range(2, 15)]
    invln2 = to_double(1 / mp.log(2))

    # sin / cos kernels on |x| <= pi/4 (slightly widened), in u = x^2
    U = (mp.pi / 4 * mp.mpf("1.01")) ** 2

    def fs(u):  # (sin(x)/x - 1)/u
        if u == 0:
            return mp.mpf(-1) / 6
        x = mp.sqrt(u)
        return (mp.sin(x) / x - 1) / u

    def fc(u):  # (cos(x) - 1 + u/2)/u^2
        if u == 0:
            return mp.mpf(1) / 24
        x = mp.sqrt(u)
        return (mp.cos(x) - 1 + u / 2) / (u * u)

    sin_c = fit_even_or_general(fs, 0, U, 6)
    cos_c = fit_even_or_general(fc, 0, U, 6)

    # pi/2 in three pieces (33 + 33 bits + rest) for Cody-Waite reduction
    pio2 = mp.pi / 2
    p1 = mp.floor(pio2 * 2 ** 32) / 2 ** 32           # 33 significant bits
    p2 = mp.floor((pio2 - p1) * 2 ** 65) / 2 ** 65
    p3 = to_double(pio2 - p1 - p2)
    two_over_pi = to_double(2 / mp.pi)

    w("// GENERATED by gen_tables.py -- do not edit; regenerate instead.")
    w("// Constants of the engine's own fp64 math (log/exp/sin/cos); see lyap_math.h.")
    w("#pragma once")
    w("")
    w("#define LYAP_LOG_BINS %d" % NB)
    w("#define LYAP_LN2HI   %s  /* ln2 truncated to a multiple of 2^-%d */" % (hexf(ln2hi), GRID))
    w("#define LYAP_LN2LO   %s  /* ln2 - LN2HI */" % hexf(ln2lo))
    w("#define LYAP_KLO_BIAS %s /* -1023 * LN2LO */" % hexf(klo_bias))
    w("#define LYAP_LN2     %s  /* ln2 correctly rounded */" % hexf(to_double(mp.log(2))))
    w("#define LYAP_LOG_C2  %s" % hexf(c[0]))
    w("#define LYAP_LOG_C3  %s" % hexf(c[1]))
    w("#define LYAP_LOG_C4  %s" % hexf(c[2]))
    w("// table residual max |-log(invc)-L| = %s ; max |r| = %s" %
      (mp.nstr(worst_resid, 5), mp.nstr(rmax, 8)))
    w("#define LYAP_INVLN2  %s" % hexf(invln2))
    for k, v in enumerate(exp_c):
        w("#define LYAP_EXP_C%d %s  /* 1/%d! */" % (k + 2, hexf(v), k + 2))
    for k, v in enumerate(sin_c):
        w("#define LYAP_SIN_C%d %s" % (k, hexf(v)))
    for k, v in enumerate(cos_c):
        w("#define LYAP_COS_C%d %s" % (k, hexf(v)))
    w("#define LYAP_PIO2_1  %s" % hexf(to_double(p1)))
    w("#define LYAP_PIO2_2  %s" % hexf(to_double(p2)))
    w("#define LYAP_PIO2_3  %s" % hexf(p3))
    w("#define LYAP_2OVERPI %s" % hexf(two_over_pi))
    w("#define LYAP_PI      %s" % hexf(to_double(mp.pi)))
    w("")
    w("// entry i: { L[i] - 1023*LN2HI (exact), invc[i] }")
    w("#define LYAP_LOG_TABLE_INIT \\")
    for i, (lp, invc, _l) in enumerate(rows):
        sep = ", \\" if i + 1 < NB else ""
        w("  {%s, %s}%s" % (hexf(lp), hexf(invc), sep))
    w("")
    sys.stdout.write("\n".join(out))
    sys.stdout.write("\n")


if __name__ == "__main__":
    main()
