// lyap_math.h -- the engine's own fp64 elementary functions, identical bits on
// host (g++) and device (nvcc).
//
// The reference (src/lyapunov_fractal.hpp:72,132,133) calls libm's log, pow and
// exp; the browser side (web/fractal_renderer.js:214-216,223,262-264) calls
// Math.sin/cos/pow.  libm's results differ between libm builds in the last bit,
// so "bit-exact" needs one fixed definition.  These functions are that
// definition: IEEE add/mul/fma/div only, every fma explicit, no contraction
// allowed anywhere else (build host code with -ffp-contract=off -mfma and
// device code with -fmad=false).  The CPU oracle links the unmodified reference
// header against these same functions.
//
// Accuracy (measured against mpmath, see tests/test_math.py):
//   lyap_log : <= 0.54 ulp for |log d| >= 2^-4, absolute error < 2^-57 nearer 1 (log(1) = 1.3e-18)
//   lyap_exp : < 1 ulp;  lyap_pow(t, 1.2 | 1.5) : < 1.5 ulp;  lyap_sin, lyap_cos : < 2 ulp for |x| <= 30
#pragma once

#if defined(__CUDACC_RTC__)
// run-time compilation has no host headers: the few fixed-width names used below
typedef unsigned int uint32_t;
typedef unsigned long long uint64_t;
typedef long long int64_t;
typedef unsigned long long uintptr_t;
#else
#include <stdint.h>
#include <string.h>
#endif
#include "lyap_tables.h"

#if defined(__CUDACC__)
#define LYAP_HD __host__ __device__ __forceinline__
#else
#define LYAP_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define LYAP_FMA(a, b, c) __fma_rn((a), (b), (c))
#else
#define LYAP_FMA(a, b, c) __builtin_fma((a), (b), (c))
#endif

struct __attribute__((aligned(16))) lyap_logtab_entry {
    double lp;    // L[i] - 1023*LN2HI, exact
    double invc;  // ~ 1/centre of bin i
};

#if defined(__CUDA_ARCH__)
// device copy lives in lyap_kernels.cu (g_lyap_logtab); kernels stage it in shared memory
#else
static const lyap_logtab_entry lyap_logtab_host[LYAP_LOG_BINS] = {LYAP_LOG_TABLE_INIT};
#endif

LYAP_HD uint64_t lyap_bits(double x) {
#if defined(__CUDA_ARCH__)
    return (uint64_t)__double_as_longlong(x);
#else
    uint64_t u;
    memcpy(&u, &x, 8);
    return u;
#endif
}

LYAP_HD double lyap_from_bits(uint64_t u) {
#if defined(__CUDA_ARCH__)
    return __longlong_as_double((long long)u);
#else
    double x;
    memcpy(&x, &u, 8);
    return x;
#endif
}

// Core of the logarithm for a positive normal double given as (hi word, lo word).
// ke_adj is added to the biased exponent (used for pre-scaled subnormals).
// Returns the exact high part in *hi_out and the small part in *s_out; the
// logarithm is hi + s (one rounding).  8 fp64 instructions with the addition.
// tab[i * stride] is entry i (stride > 1: interleaved copies, see the lambda kernel).
LYAP_HD void lyap_log_core(uint32_t hw, uint32_t lw, int ke_adj, const lyap_logtab_entry* tab, int stride,
                           double* hi_out, double* s_out) {
    const int ke = (int)(hw >> 20) + ke_adj;
    const uint32_t i = (hw >> 10) & (LYAP_LOG_BINS - 1);
    const uint32_t mh = (hw & 0x000FFFFFu) | 0x3FF00000u;
    const double m = lyap_from_bits(((uint64_t)mh << 32) | lw);
    const lyap_logtab_entry ent = tab[i * stride];
    const double lp = ent.lp;
    const double invc = ent.invc;
    const double kd = (double)ke;
    const double r = LYAP_FMA(m, invc, -1.0);
    double q = LYAP_FMA(r, LYAP_LOG_C4, LYAP_LOG_C3);
    q = LYAP_FMA(r, q, LYAP_LOG_C2);
    const double w = LYAP_FMA(r, q, 1.0);
    const double klo = LYAP_FMA(kd, LYAP_LN2LO, LYAP_KLO_BIAS);
    *s_out = LYAP_FMA(r, w, klo);
    *hi_out = LYAP_FMA(kd, LYAP_LN2HI, lp);
}

// True when the fast core applies directly: d positive, normal, finite.
LYAP_HD bool lyap_log_fast_domain(uint32_t hw) { return (hw - 0x00100000u) < 0x7FE00000u; }

// Natural logarithm, all inputs.  tab = 1024-entry table (host or shared copy).
LYAP_HD double lyap_log_tab(double d, const lyap_logtab_entry* tab, int stride) {
    uint64_t b = lyap_bits(d);
    uint32_t hw = (uint32_t)(b >> 32), lw = (uint32_t)b;
    int adj = 0;
    if (!lyap_log_fast_domain(hw)) {
        if ((b << 1) == 0) return lyap_from_bits(0xFFF0000000000000ull);        // log(+-0) = -inf
        if (b == 0x7FF0000000000000ull) return d;                               // log(+inf) = +inf
        if ((b >> 63) || (hw & 0x7FF00000u) == 0x7FF00000u)                     // negative or NaN
            return lyap_from_bits(0x7FF8000000000000ull);
        d = d * 0x1p52;  // subnormal: exact scaling
        b = lyap_bits(d);
        hw = (uint32_t)(b >> 32);
        lw = (uint32_t)b;
        adj = -52;
    }
    double hi, s;
    lyap_log_core(hw, lw, adj, tab, stride, &hi, &s);
    return hi + s;
}

#if !defined(__CUDA_ARCH__)
static inline double lyap_log(double d) { return lyap_log_tab(d, lyap_logtab_host, 1); }
#endif

// 2^n * p for p in [0.5, 4), any n: two-step scaling keeps subnormal results single-rounded enough
// for our use (results below 2^-1022 are rounded twice; never reached by the colour path).
LYAP_HD double lyap_scalbn_small(double p, int n) {
    if (n > 1000) {
        p = p * 0x1p1000;
        n -= 1000;
        if (n > 1000) n = 1000;
    } else if (n < -1000) {
        p = p * 0x1p-1000;
        n += 1000;
        if (n < -1000) n = -1000;
    }
    return p * lyap_from_bits((uint64_t)(uint32_t)(1023 + n) << 52);
}

// e^x
LYAP_HD double lyap_exp(double x) {
    if (x != x) return x;
    if (x > 709.782712893384) return lyap_from_bits(0x7FF0000000000000ull);
    if (x < -745.2) return 0.0;
    const double magic = 0x1.8p52;
    const double nf = LYAP_FMA(x, LYAP_INVLN2, magic) - magic;  // nearest integer to x/ln2
    const int n = (int)nf;
    double r = LYAP_FMA(-nf, LYAP_LN2HI, x);  // exact: LN2HI has 42 significant bits
    r = LYAP_FMA(-nf, LYAP_LN2LO, r);
    double p = LYAP_EXP_C14;
    p = LYAP_FMA(p, r, LYAP_EXP_C13);
    p = LYAP_FMA(p, r, LYAP_EXP_C12);
    p = LYAP_FMA(p, r, LYAP_EXP_C11);
    p = LYAP_FMA(p, r, LYAP_EXP_C10);
    p = LYAP_FMA(p, r, LYAP_EXP_C9);
    p = LYAP_FMA(p, r, LYAP_EXP_C8);
    p = LYAP_FMA(p, r, LYAP_EXP_C7);
    p = LYAP_FMA(p, r, LYAP_EXP_C6);
    p = LYAP_FMA(p, r, LYAP_EXP_C5);
    p = LYAP_FMA(p, r, LYAP_EXP_C4);
    p = LYAP_FMA(p, r, LYAP_EXP_C3);
    p = LYAP_FMA(p, r, LYAP_EXP_C2);
    const double r2 = r * r;
    const double t = LYAP_FMA(p, r2, r);  // e^r - 1
    return lyap_scalbn_small(1.0 + t, n);
}

// t^y for t >= 0 and finite y > 0 (the colour path uses y = 1.2 and y = 1.5).
LYAP_HD double lyap_pow_tab(double t, double y, const lyap_logtab_entry* tab, int stride) {
    if (t != t || t < 0.0) return lyap_from_bits(0x7FF8000000000000ull);
    if (t == 0.0) return 0.0;
    if (t == 1.0) return 1.0;
    uint64_t b = lyap_bits(t);
    if (b == 0x7FF0000000000000ull) return t;
    uint32_t hw = (uint32_t)(b >> 32), lw = (uint32_t)b;
    int adj = 0;
    if (hw < 0x00100000u) {
        t = t * 0x1p52;
        b = lyap_bits(t);
        hw = (uint32_t)(b >> 32);
        lw = (uint32_t)b;
        adj = -52;
    }
    double hi, s;
    lyap_log_core(hw, lw, adj, tab, stride, &hi, &s);
    // log t = zh + zl (TwoSum)
    const double zh = hi + s;
    const double bb = zh - hi;
    const double zl = (hi - (zh - bb)) + (s - bb);
    const double ph = y * zh;
    const double pl = LYAP_FMA(y, zh, -ph) + y * zl;
    const double e = lyap_exp(ph);
    return LYAP_FMA(e, pl, e);
}

#if !defined(__CUDA_ARCH__)
static inline double lyap_pow(double t, double y) { return lyap_pow_tab(t, y, lyap_logtab_host, 1); }
#endif

// sin/cos kernels on |r| <= pi/4
LYAP_HD double lyap_sin_kernel(double r) {
    const double u = r * r;
    double p = LYAP_SIN_C6;
    p = LYAP_FMA(p, u, LYAP_SIN_C5);
    p = LYAP_FMA(p, u, LYAP_SIN_C4);
    p = LYAP_FMA(p, u, LYAP_SIN_C3);
    p = LYAP_FMA(p, u, LYAP_SIN_C2);
    p = LYAP_FMA(p, u, LYAP_SIN_C1);
    p = LYAP_FMA(p, u, LYAP_SIN_C0);
    return LYAP_FMA(r * u, p, r);
}

LYAP_HD double lyap_cos_kernel(double r) {
    const double u = r * r;
    double p = LYAP_COS_C6;
    p = LYAP_FMA(p, u, LYAP_COS_C5);
    p = LYAP_FMA(p, u, LYAP_COS_C4);
    p = LYAP_FMA(p, u, LYAP_COS_C3);
    p = LYAP_FMA(p, u, LYAP_COS_C2);
    p = LYAP_FMA(p, u, LYAP_COS_C1);
    p = LYAP_FMA(p, u, LYAP_COS_C0);
    const double h = LYAP_FMA(u, -0.5, 1.0);
    return LYAP_FMA(u * u, p, h);
}

// Argument reduction to r in [-pi/4, pi/4], quadrant in *q.  Meant for |x| < 2^20.
LYAP_HD double lyap_trig_reduce(double x, int* q) {
    const double magic = 0x1.8p52;
    const double nf = LYAP_FMA(x, LYAP_2OVERPI, magic) - magic;
    double r = LYAP_FMA(-nf, LYAP_PIO2_1, x);
    r = LYAP_FMA(-nf, LYAP_PIO2_2, r);
    r = LYAP_FMA(-nf, LYAP_PIO2_3, r);
    *q = (int)nf & 3;
    return r;
}

LYAP_HD double lyap_sin(double x) {
    int q;
    const double r = lyap_trig_reduce(x, &q);
    const double v = (q & 1) ? lyap_cos_kernel(r) : lyap_sin_kernel(r);
    return (q & 2) ? -v : v;
}

LYAP_HD double lyap_cos(double x) {
    int q;
    const double r = lyap_trig_reduce(x, &q);
    const double v = (q & 1) ? lyap_sin_kernel(r) : lyap_cos_kernel(r);
    return ((q + 1) & 2) ? -v : v;
}
