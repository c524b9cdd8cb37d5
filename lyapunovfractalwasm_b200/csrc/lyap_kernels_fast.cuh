// lyap_kernels_fast.cuh -- fast-mode lambda kernels (included by lyap_kernels.cu after lyap_exact_kernel.cuh, and, as
// text, by the run-time specialiser).
//
// Same pixel mapping, sequence handling, sentinel and early-exit rules as the exact kernel, but the
// arithmetic is rearranged for speed and is NOT bit-compatible with the reference:
//   t = r*x;  deriv = fma(-2,t,r) = r(1-2x);  x' = fma(-t,x,t) = r x (1-x)         (4 fused ops/step)
// and instead of one log per step the |deriv| are multiplied together; the product's exponent is
// moved into an integer at least every 32 (fp64) or 20 (fp32) steps, and one log of the remaining mantissa is
// taken per pixel at the end:  sum log|deriv| = E*ln2 + log(mantissa product).
// A chunk in which the orbit left (0,1) or a derivative was exactly zero is rolled back and redone
// step by step with the reference's rules (skip zero terms, stop at the exit, keep the partial sum).
#pragma once

namespace lyap {

template <typename T>
struct FastTraits;

template <>
struct FastTraits<double> {
    static constexpr int kRenorm = 32;
    static __device__ __forceinline__ double fma_(double a, double b, double c) { return __fma_rn(a, b, c); }
    static __device__ __forceinline__ double mul(double a, double b) { return __dmul_rn(a, b); }
    static __device__ __forceinline__ double sub(double a, double b) { return __dsub_rn(a, b); }
    static __device__ __forceinline__ double abs_(double a) { return fabs(a); }
    // returns biased exponent; rewrites v's exponent to 0 (mantissa in [1,2)); sign assumed +
    static __device__ __forceinline__ int strip(double& v) {
        const unsigned hw = (unsigned)__double2hiint(v);
        v = __hiloint2double((int)((hw & 0x000FFFFFu) | 0x3FF00000u), __double2loint(v));
        return (int)(hw >> 20);
    }
    static constexpr int kBias = 1023;
    static constexpr int kExpMax = 2047;
};

template <>
struct FastTraits<float> {
    // A product that is subnormal or zero when it is stripped sends the chunk to the step-by-step path.  Falling below
    // 2^-126 from [1,2) within 20 steps takes derivatives that average below 2^-6 (x within a percent of 0.5 step after
    // step); only a product that did so and was multiplied back above 2^-126 before the strip would lose low bits
    // unnoticed.  Where the strips fall does not change a regular pixel's bits (moving the exponent out is exact).
    static constexpr int kRenorm = 20;
    static __device__ __forceinline__ float fma_(float a, float b, float c) { return __fmaf_rn(a, b, c); }
    static __device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
    static __device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
    static __device__ __forceinline__ float abs_(float a) { return fabsf(a); }
    static __device__ __forceinline__ int strip(float& v) {
        const unsigned u = __float_as_uint(v);
        v = __uint_as_float((u & 0x007FFFFFu) | 0x3F800000u);
        return (int)(u >> 23);
    }
    static constexpr int kBias = 127;
    static constexpr int kExpMax = 255;
};

// The three fast kernels: which type the orbit and the product run in, and whether the orbit and the derivative use the
// reference's own operations (then x and every derivative have the exact kernel's bits and only the accumulation --
// a running product instead of a sum of logarithms -- differs) or the fused ones.
struct FusedF64 { using real = double; static constexpr bool same_orbit = false; };
struct FusedF32 { using real = float; static constexpr bool same_orbit = false; };
struct OrbitF64 { using real = double; static constexpr bool same_orbit = true; };

// One step of one pixel: the derivative at x (times into prod when ACC), then the update.
//   fused:      t = r*x;  deriv = fma(-2,t,r) = r(1-2x);  x' = fma(-t,x,t) = r x (1-x)            4 instructions
//   same orbit: |fma(-2,x,1)| into the product (deriv = r*|1-2x|, :69; the r's are added as n*log r at the end);
//               x' = (r*x)*(1-x) (:76)                                                             5 instructions
template <typename FL, bool ACC>
__device__ __forceinline__ void fast_step_one(typename FL::real& x, typename FL::real& prod, typename FL::real r) {
    using T = typename FL::real;
    using F = FastTraits<T>;
    if (FL::same_orbit) {
        // |r*(1-2x)| = r*|1-2x| for r > 0: only |1-2x| (exact: 2x and 1-2x round nowhere near 0.5) goes into the product;
        // the factors r are accounted for per pixel at the end, from how many steps used which parameter
        if (ACC) prod = F::mul(prod, F::abs_(F::fma_((T)-2, x, (T)1)));
        x = F::mul(F::mul(r, x), F::sub((T)1, x));
    } else {
        const T t = F::mul(r, x);
        if (ACC) prod = F::mul(prod, F::abs_(F::fma_((T)-2, t, r)));
        x = F::fma_(-t, x, t);
    }
}

template <typename T>
struct FastPixel {
    T x;
    double extra;   // log terms added one by one by the careful path
    int valid;
};

template <typename FL, bool ACC>
__device__ __noinline__ bool fast_careful_chunk(FastPixel<typename FL::real>* ps, typename FL::real rA, typename FL::real rB,
                                                typename FL::real rC, unsigned word, int n, unsigned long long* steps) {
    using T = typename FL::real;
    using F = FastTraits<T>;
    T x = ps->x;
    double extra = ps->extra;
    int valid = ps->valid;
    bool dead = false;
    int j = 0;
    for (; j < n; ++j) {
        const unsigned sel = (word >> (2 * j)) & 3u;
        const T r = sel == 0 ? rA : (sel == 1 ? rB : rC);
        const T t = F::mul(r, x);
        if (ACC) {
            const T d = FL::same_orbit ? F::mul(r, F::abs_(F::fma_((T)-2, x, (T)1))) : F::abs_(F::fma_((T)-2, t, r));
            if (d > (T)0) {
                extra = __dadd_rn(extra, lyap_log_tab((double)d, g_lyap_logtab, 1));
                ++valid;
            }
        }
        x = FL::same_orbit ? F::mul(t, F::sub((T)1, x)) : F::fma_(-t, x, t);
        if (!(x > (T)0 && x < (T)1)) {
            dead = true;
            ++j;
            break;
        }
    }
    *steps += (unsigned long long)j;
    ps->x = x;
    ps->extra = extra;
    ps->valid = valid;
    return dead;
}

template <typename FL, int P, bool ACC>
__device__ __forceinline__ void fast_mode_steps(typename FL::real (&x)[P], typename FL::real (&prod)[P],
                                                const typename FL::real (&r)[P]) {
#pragma unroll
    for (int p = 0; p < P; ++p) fast_step_one<FL, ACC>(x[p], prod[p], r[p]);
}

// fast_careful_chunk for steps [first, first + n) of a region whose selector words start at `sel`.
template <typename FL, bool ACC>
__device__ __noinline__ bool fast_careful_steps(FastPixel<typename FL::real>* ps, typename FL::real rA, typename FL::real rB,
                                                typename FL::real rC, const unsigned* sel, int wrap, int first, int n,
                                                unsigned long long* steps) {
    bool dead = false;
    int j = first;
    const int end = first + n;
    while (j < end && !dead) {
        const int in_word = j & (kStepsPerWord - 1);
        const int m = min(kStepsPerWord - in_word, end - j);
        dead = fast_careful_chunk<FL, ACC>(ps, rA, rB, rC, sel[(j / kStepsPerWord) % wrap] >> (2 * in_word), m, steps);
        j += m;
    }
    return dead;
}

// Moves the exponent of every pixel's running product into its integer sum and notes the smallest exponent field seen.
// The sum takes the BIASED field; the caller subtracts the bias once per strip when it accepts the chunk.  Only the
// low end needs watching: while x stays inside (0,1) every derivative is below r in magnitude, so a product of at most
// kRenorm of them cannot overflow, and an x that left (0,1) is found by the test on x itself.
template <typename T, int P>
__device__ __forceinline__ void strip_products(T (&prod)[P], int (&esum)[P], int (&emin)[P]) {
    using F = FastTraits<T>;
#pragma unroll
    for (int p = 0; p < P; ++p) {
        const int e = F::strip(prod[p]);
        emin[p] = min(emin[p], e);
        esum[p] += e;
    }
}

// strips fast_fixed_groups makes in NG groups
template <typename T>
__host__ __device__ constexpr int strips_in_groups(int ng) {
    int n = 0;
    for (int gi = 0; gi < ng; ++gi)
        if ((2 * (gi + 1)) % FastTraits<T>::kRenorm == 0 || gi == ng - 1) ++n;
    return n;
}

// Run-time specialisation (see lyap_jit.cu): NG two-step groups whose patterns are compile-time constants
// (PATS: 4 bits per group, repeating every KG groups), as one straight-line block; the products are stripped
// every kRenorm steps and after the last group.
template <typename FL, int P, bool ACC, int KG, unsigned long long PATS, int NG, int GI = 0>
__device__ __forceinline__ void fast_fixed_groups(typename FL::real (&x)[P], typename FL::real (&prod)[P], int (&esum)[P],
                                                  int (&emin)[P], const typename FL::real (&rA)[P],
                                                  const typename FL::real (&rB)[P], const typename FL::real (&rC)[P]) {
    using T = typename FL::real;
    using F = FastTraits<T>;
    if constexpr (GI < NG) {
        constexpr unsigned pat = (unsigned)((PATS >> (4 * (GI % KG))) & 15ull);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            constexpr unsigned code0 = pat & 3u, code1 = (pat >> 2) & 3u;
            const unsigned code = j == 0 ? code0 : code1;
#pragma unroll
            for (int p = 0; p < P; ++p) {
                const T r = code == 0 ? rA[p] : (code == 1 ? rB[p] : rC[p]);
                fast_step_one<FL, ACC>(x[p], prod[p], r);
            }
        }
        if (ACC && ((2 * (GI + 1)) % F::kRenorm == 0 || GI == NG - 1)) strip_products<T, P>(prod, esum, emin);
        fast_fixed_groups<FL, P, ACC, KG, PATS, NG, GI + 1>(x, prod, esum, emin, rA, rB, rC);
    }
}

template <typename T>
__device__ __forceinline__ bool ordinary_param_t(T r);
template <>
__device__ __forceinline__ bool ordinary_param_t<double>(double r) { return r > 0x1p-40 && r < 0x1p40; }
template <>
__device__ __forceinline__ bool ordinary_param_t<float>(float r) { return r > 0x1p-20f && r < 0x1p5f; }

// how many of the `steps` 2-bit codes in `pats` (step j at bits 2j, 2j+1) equal `code`
__host__ __device__ constexpr int count_code(unsigned long long pats, int steps, unsigned code) {
    int n = 0;
    for (int j = 0; j < steps; ++j) n += ((pats >> (2 * j)) & 3ull) == code ? 1 : 0;
    return n;
}

// the same for the first n (<= 16) steps of a selector word, at run time
__device__ __forceinline__ void count_word_codes(unsigned word, int n, int& c0, int& c1, int& c2) {
    const unsigned live = n >= 16 ? 0x55555555u : ((1u << (2 * n)) - 1u) & 0x55555555u;
    const unsigned lo = word & 0x55555555u, hi = (word >> 1) & 0x55555555u;
    c0 = __popc(~lo & ~hi & live);
    c1 = __popc(lo & ~hi & live);
    c2 = __popc(hi & ~lo & live);
}

// Body shared by the precompiled kernel (KG == 0) and a run-time specialised instance (KG > 0).
template <typename FL, int P, int THREADS, int KG, unsigned long long WU_PATS, unsigned long long ACC_PATS>
__device__ __forceinline__ void lambda_fast_body(const LambdaArgs& a, double* __restrict__ out64, float* __restrict__ out32,
                                                 unsigned long long* __restrict__ steps_out) {
    using T = typename FL::real;
    using F = FastTraits<T>;
    unsigned long long my_steps = 0;
    const long long tile_px = (long long)THREADS * P;

    for (long long tile = blockIdx.x; tile * tile_px < a.n_pixels; tile += gridDim.x) {
        const long long idx0 = tile * tile_px + (long long)threadIdx.x * P;
        T x[P], prod[P], rA[P], rB[P], rC[P];
        double extra[P], lam[P];
        int valid[P], esum[P];   // 32 bits are enough: the host admits at most 2^24 steps per pixel in the fast modes
        int nuse[P][3];          // same-orbit flavour: accumulated steps of accepted chunks by the parameter they used (A, B, C)
        bool done[P], careful_only[P];
        {
            long long row = idx0 / a.width;
            int col = (int)(idx0 - row * a.width);
            row += a.row_begin;
#pragma unroll
            for (int p = 0; p < P; ++p) {
                const bool inside = idx0 + p < a.n_pixels;
                const double rb = __dadd_rn(a.min_y, __dmul_rn(a.dy, (double)(int)row));
                const double ra = __dadd_rn(a.min_x, __dmul_rn(a.dx, (double)col));
                rA[p] = (T)ra;
                rB[p] = (T)rb;
                rC[p] = (T)a.c_value;
                x[p] = (T)0.5;
                prod[p] = (T)1;
                extra[p] = 0.0;
                valid[p] = 0;
                esum[p] = 0;
                if constexpr (FL::same_orbit) nuse[p][0] = nuse[p][1] = nuse[p][2] = 0;
                lam[p] = -5.0;
                done[p] = !inside || ra <= 0.0 || rb <= 0.0;
                careful_only[p] = !(ordinary_param_t<T>(rA[p]) && ordinary_param_t<T>(rB[p]) && a.fast_ok_c);
                if (++col == a.width) {
                    col = 0;
                    ++row;
                }
            }
        }

        // lambda from the partial sums: esum*ln2 + log(mantissa product) + terms logged one by one
        // (+ n_A log r_A + n_B log r_B + n_C log r_C where the product left the parameters out)
        auto finish = [&](int p) -> double {
            double lsum = __dadd_rn(__fma_rn((double)esum[p], LYAP_LN2, lyap_log_tab((double)prod[p], g_lyap_logtab, 1)), extra[p]);
            if constexpr (FL::same_orbit) {
                double rsum = 0.0;
                if (nuse[p][0] > 0) rsum = __fma_rn((double)nuse[p][0], lyap_log_tab((double)rA[p], g_lyap_logtab, 1), rsum);
                if (nuse[p][1] > 0) rsum = __fma_rn((double)nuse[p][1], lyap_log_tab((double)rB[p], g_lyap_logtab, 1), rsum);
                if (nuse[p][2] > 0) rsum = __fma_rn((double)nuse[p][2], lyap_log_tab((double)rC[p], g_lyap_logtab, 1), rsum);
                lsum = __dadd_rn(lsum, rsum);
            }
            return valid[p] > 0 ? __ddiv_rn(lsum, __dmul_rn((double)valid[p], LYAP_LN2)) : -5.0;
        };

        for (int region = 0; region < 2; ++region) {
            const bool acc = region == 1;
            const int nsteps = acc ? a.iterations : a.warmup;
            const int word0 = acc ? a.acc_word0 : 0;
            const int wrap = acc ? a.acc_wrap : a.wu_wrap;
            if constexpr (KG > 0) {
                // exit tests after REP straight-line blocks of CB whole periods (measured: 1 -> 4 blocks saves 12 % (fp64) and
                // 16 % (fp32) of a large frame's time, 8 another 2 %; a pixel that leaves (0,1) replays at most one such chunk)
                constexpr int BS = 2 * KG, CB = (kStepsPerWord + BS - 1) / BS, REP = 8, CS = CB * BS * REP;
                const unsigned* sel = a.sel + word0;
                int s = 0;
                while (s < nsteps) {
                    bool all_done = true;
#pragma unroll
                    for (int p = 0; p < P; ++p) all_done = all_done && done[p];
                    if (__all_sync(0xFFFFFFFFu, all_done)) break;
                    const int left = nsteps - s;
                    const int n = left >= CS ? CS : (left >= CB * BS ? CB * BS : (left >= BS ? left / BS * BS : left));
                    T sx[P], sp[P];
                    int se[P], emin[P];
                    int nstrip = 0;   // strips made in this chunk (the same for every pixel): their bias leaves the sums below
                    int cuse[3] = {0, 0, 0};   // accumulated steps of this chunk by parameter (same for every pixel)
                    constexpr int kPer0 = count_code(ACC_PATS, BS, 0), kPer1 = count_code(ACC_PATS, BS, 1), kPer2 = count_code(ACC_PATS, BS, 2);
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        sx[p] = x[p];
                        sp[p] = prod[p];
                        se[p] = esum[p];
                        emin[p] = F::kExpMax;
                    }
                    if (left >= CS) {
#pragma unroll 1
                        for (int rep = 0; rep < REP; ++rep) {
                            if (acc) fast_fixed_groups<FL, P, true, KG, ACC_PATS, CB * KG>(x, prod, esum, emin, rA, rB, rC);
                            else fast_fixed_groups<FL, P, false, KG, WU_PATS, CB * KG>(x, prod, esum, emin, rA, rB, rC);
                        }
                        nstrip = REP * strips_in_groups<T>(CB * KG);
                        if constexpr (FL::same_orbit) cuse[0] = REP * CB * kPer0, cuse[1] = REP * CB * kPer1, cuse[2] = REP * CB * kPer2;
                    } else if (left >= CB * BS) {
                        if (acc) fast_fixed_groups<FL, P, true, KG, ACC_PATS, CB * KG>(x, prod, esum, emin, rA, rB, rC);
                        else fast_fixed_groups<FL, P, false, KG, WU_PATS, CB * KG>(x, prod, esum, emin, rA, rB, rC);
                        nstrip = strips_in_groups<T>(CB * KG);
                        if constexpr (FL::same_orbit) cuse[0] = CB * kPer0, cuse[1] = CB * kPer1, cuse[2] = CB * kPer2;
                    } else if (left >= BS) {
#pragma unroll 1
                        for (int b = 0; b < n / BS; ++b) {
                            if (acc) fast_fixed_groups<FL, P, true, KG, ACC_PATS, KG>(x, prod, esum, emin, rA, rB, rC);
                            else fast_fixed_groups<FL, P, false, KG, WU_PATS, KG>(x, prod, esum, emin, rA, rB, rC);
                        }
                        nstrip = (n / BS) * strips_in_groups<T>(KG);
                        if constexpr (FL::same_orbit) cuse[0] = (n / BS) * kPer0, cuse[1] = (n / BS) * kPer1, cuse[2] = (n / BS) * kPer2;
                    } else {
#pragma unroll 1
                        for (int j = s; j < nsteps; ++j) {
                            const unsigned code = (sel[(j / kStepsPerWord) % wrap] >> (2 * (j & (kStepsPerWord - 1)))) & 3u;
                            if (acc) {
                                if constexpr (FL::same_orbit) {
                                    if (code == 0) ++cuse[0];
                                    else if (code == 1) ++cuse[1];
                                    else ++cuse[2];
                                }
                                if (code == 0) fast_mode_steps<FL, P, true>(x, prod, rA);
                                else if (code == 1) fast_mode_steps<FL, P, true>(x, prod, rB);
                                else fast_mode_steps<FL, P, true>(x, prod, rC);
                                if ((j - s + 1) % F::kRenorm == 0 || j == nsteps - 1) {
                                    strip_products<T, P>(prod, esum, emin);
                                    ++nstrip;
                                }
                            } else {
                                if (code == 0) fast_mode_steps<FL, P, false>(x, prod, rA);
                                else if (code == 1) fast_mode_steps<FL, P, false>(x, prod, rB);
                                else fast_mode_steps<FL, P, false>(x, prod, rC);
                            }
                        }
                    }
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        if (done[p]) continue;
                        const bool regular = !careful_only[p] && (x[p] > (T)0 && x[p] < (T)1) && (!acc || emin[p] != 0);
                        if (regular) {
                            if (acc) {
                                valid[p] += n;
                                esum[p] -= F::kBias * nstrip;
                                if constexpr (FL::same_orbit) {
                                    nuse[p][0] += cuse[0];
                                    nuse[p][1] += cuse[1];
                                    nuse[p][2] += cuse[2];
                                }
                            }
                            my_steps += (unsigned long long)n;
                        } else {
                            esum[p] = se[p];
                            prod[p] = sp[p];
                            FastPixel<T> ps{sx[p], extra[p], valid[p]};
                            const bool dead =
                                acc ? fast_careful_steps<FL, true>(&ps, rA[p], rB[p], rC[p], sel, wrap, s, n, &my_steps)
                                    : fast_careful_steps<FL, false>(&ps, rA[p], rB[p], rC[p], sel, wrap, s, n, &my_steps);
                            x[p] = ps.x;
                            extra[p] = ps.extra;
                            valid[p] = ps.valid;
                            if (dead) {
                                done[p] = true;
                                lam[p] = finish(p);
                                x[p] = (T)0.25;
                            }
                        }
                    }
                    s += n;
                }
                continue;
            }
            const int nchunks = nsteps / kStepsPerWord + (nsteps % kStepsPerWord != 0);
            for (int c = 0, wi = 0; c < nchunks; ++c) {
                bool all_done = true;
#pragma unroll
                for (int p = 0; p < P; ++p) all_done = all_done && done[p];
                if (__all_sync(0xFFFFFFFFu, all_done)) break;

                const unsigned word = a.sel[word0 + wi];
                if (++wi == wrap) wi = 0;
                const int n = min(kStepsPerWord, nsteps - c * kStepsPerWord);
                T sx[P], sp[P];
                int se[P], emin[P];
                int nstrip = 0;
                int cuse[3] = {0, 0, 0};
                if constexpr (FL::same_orbit) {
                    if (acc) count_word_codes(word, n, cuse[0], cuse[1], cuse[2]);
                }
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    sx[p] = x[p];
                    sp[p] = prod[p];
                    se[p] = esum[p];
                    emin[p] = F::kExpMax;
                }
                unsigned w = word;
                if (acc) {
                    for (int j0 = 0; j0 < n; j0 += F::kRenorm, ++nstrip) {
                        const int jn = min(F::kRenorm, n - j0);
                        for (int j = 0; j < jn; ++j, w >>= 2) {
                            const unsigned sel = w & 3u;
                            if (sel == 0) fast_mode_steps<FL, P, true>(x, prod, rA);
                            else if (sel == 1) fast_mode_steps<FL, P, true>(x, prod, rB);
                            else fast_mode_steps<FL, P, true>(x, prod, rC);
                        }
                        strip_products<T, P>(prod, esum, emin);
                    }
                } else {
                    for (int j = 0; j < n; ++j, w >>= 2) {
                        const unsigned sel = w & 3u;
                        if (sel == 0) fast_mode_steps<FL, P, false>(x, prod, rA);
                        else if (sel == 1) fast_mode_steps<FL, P, false>(x, prod, rB);
                        else fast_mode_steps<FL, P, false>(x, prod, rC);
                    }
                }
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    if (done[p]) continue;
                    // a zero derivative (or a product that underflowed) shows as exponent field 0
                    const bool regular = !careful_only[p] && (x[p] > (T)0 && x[p] < (T)1) && (!acc || emin[p] != 0);
                    if (regular) {
                        if (acc) {
                            valid[p] += n;
                            esum[p] -= F::kBias * nstrip;
                            if constexpr (FL::same_orbit) {
                                nuse[p][0] += cuse[0];
                                nuse[p][1] += cuse[1];
                                nuse[p][2] += cuse[2];
                            }
                        }
                        my_steps += (unsigned long long)n;
                    } else {
                        esum[p] = se[p];
                        prod[p] = sp[p];
                        FastPixel<T> ps{sx[p], extra[p], valid[p]};
                        const bool dead =
                            acc ? fast_careful_chunk<FL, true>(&ps, rA[p], rB[p], rC[p], word, n, &my_steps)
                                : fast_careful_chunk<FL, false>(&ps, rA[p], rB[p], rC[p], word, n, &my_steps);
                        x[p] = ps.x;
                        extra[p] = ps.extra;
                        valid[p] = ps.valid;
                        if (dead) {
                            // freeze the result now: the abandoned lane keeps running on garbage
                            done[p] = true;
                            lam[p] = finish(p);
                            x[p] = (T)0.25;
                        }
                    }
                }
            }
        }

#pragma unroll
        for (int p = 0; p < P; ++p)
            if (!done[p]) lam[p] = finish(p);
        // stores through the warp's own staging row in shared memory: 16 bytes per lane, consecutive 512-byte runs per
        // instruction, no block-wide barrier (plain stores for a ragged last tile or a misaligned output pointer)
        const long long tile0 = tile * tile_px;
        const bool full_tile = tile0 + tile_px <= a.n_pixels;
        __shared__ __align__(16) double stage_all[THREADS * P];
        const int lane = threadIdx.x & 31, warp_px0 = (threadIdx.x & ~31) * P;
        double* stage = stage_all + warp_px0;
        if (out64) {
            if (full_tile && ((reinterpret_cast<uintptr_t>(out64 + tile0) & 15) == 0)) {
                __syncwarp();
#pragma unroll
                for (int p = 0; p < P; ++p) stage[lane * P + p] = lam[p];
                __syncwarp();
                double2* dst = reinterpret_cast<double2*>(out64 + tile0 + warp_px0);
                const double2* src = reinterpret_cast<const double2*>(stage);
#pragma unroll
                for (int i = lane; i < 16 * P; i += 32) dst[i] = src[i];
            } else {
#pragma unroll
                for (int p = 0; p < P; ++p)
                    if (idx0 + p < a.n_pixels) out64[idx0 + p] = lam[p];
            }
        }
        if (out32) {
            if (full_tile && ((reinterpret_cast<uintptr_t>(out32 + tile0) & 15) == 0)) {
                float* stage32 = reinterpret_cast<float*>(stage);
                __syncwarp();
#pragma unroll
                for (int p = 0; p < P; ++p) stage32[lane * P + p] = (float)lam[p];
                __syncwarp();
                float4* dst = reinterpret_cast<float4*>(out32 + tile0 + warp_px0);
                const float4* src = reinterpret_cast<const float4*>(stage32);
#pragma unroll
                for (int i = lane; i < 8 * P; i += 32) dst[i] = src[i];
            } else {
#pragma unroll
                for (int p = 0; p < P; ++p)
                    if (idx0 + p < a.n_pixels) out32[idx0 + p] = (float)lam[p];
            }
        }
    }

    if (steps_out) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) my_steps += __shfl_down_sync(0xFFFFFFFFu, my_steps, o);
        if ((threadIdx.x & 31) == 0 && my_steps) atomicAdd(steps_out, my_steps);
    }
}

constexpr int kFastThreads = 256;

template <typename FL, int P, int THREADS>
__global__ void __launch_bounds__(THREADS)
k_lambda_fast(const __grid_constant__ LambdaArgs a, double* __restrict__ out64, float* __restrict__ out32,
              unsigned long long* __restrict__ steps_out) {
    lambda_fast_body<FL, P, THREADS, 0, 0ull, 0ull>(a, out64, out32, steps_out);
}

#if defined(LYAP_SPEC_FAST)
// The specialised instance; LYAP_SPEC_* are given on the run-time compiler's command line.
extern "C" __global__ void __launch_bounds__(LYAP_SPEC_THREADS)
k_lambda_fast_spec(const __grid_constant__ LambdaArgs a, double* __restrict__ out64, float* __restrict__ out32,
                   unsigned long long* __restrict__ steps_out) {
    lambda_fast_body<LYAP_SPEC_FAST, LYAP_SPEC_P, LYAP_SPEC_THREADS, LYAP_SPEC_KG, LYAP_SPEC_WU_PATS, LYAP_SPEC_ACC_PATS>(
        a, out64, out32, steps_out);
}
#endif


}  // namespace lyap
