// lyap_exact_kernel.cuh -- the exact lambda kernel (FractalComputer::computeFractal, reference
// src/lyapunov_fractal.hpp:41-86).  Included by lyap_kernels.cu (compiled by nvcc into the library) and, as text,
// by the run-time specialiser (lyap_jit.cu), which compiles one more instance of the same code with the sequence's
// group patterns as compile-time constants.  Keep it free of host-only headers.
#pragma once

#include "lyap_args.h"
#include "lyap_math.h"

namespace lyap {

static __device__ const lyap_logtab_entry g_lyap_logtab[LYAP_LOG_BINS] = {LYAP_LOG_TABLE_INIT};

// ---------------------------------------------------------------------------------------------
// Exact lambda kernel.
//
// One thread owns P horizontally adjacent pixels for their whole orbit: x, the running log sum and
// the two parameter values stay in registers.  The per-step A/B(/C) choice is the same for every
// pixel, so steps are taken in groups of U whose pattern (e.g. "AB", "BA") picks, by one warp-uniform
// multiway branch, a straight-line body compiled for exactly that pattern: no per-step select or branch.
// Inside a body the orbit runs ahead and the U*P logarithms that hang off it are independent chains.
//
// The log table (1024 entries x 16 B) sits in shared memory in 8 interleaved copies: entry i of
// copy c is at slot i*8+c and a lane uses copy (lane & 7).  A 16-byte load per lane is served per
// quarter warp, whose 8 lanes then hit 8 different 16-byte bank groups whatever their indices are,
// so the lookups never conflict.
//
// Steps run in chunks of 16 to about 40 without per-step exit tests.  That is sound because leaving (0,1)
// is permanent for x <- r x (1-x) with r > 0 (x >= 1 gives x <= 0 next, x <= 0 stays <= 0, NaN stays
// NaN), so testing x after the chunk finds every exit, and the only other irregular event, a zero
// derivative (x == 0.5 exactly, skipped and not counted by the reference, :71-74), has exponent field 0,
// for which the exponent table holds -inf: the running sum turns non-finite.  A chunk in which anything irregular
// happened is rolled back and redone by `careful_chunk` / `careful_steps`, which follow the reference step by step.
// ---------------------------------------------------------------------------------------------

constexpr int kTabCopies = 8;
constexpr size_t kTabSmemBytes = (size_t)LYAP_LOG_BINS * kTabCopies * sizeof(lyap_logtab_entry);  // 128 KB
// Second shared table, indexed by the top 12 bits of the derivative (sign + exponent field e): {e*LN2HI (exact),
// (e-1023)*LN2LO}.  It replaces an integer->double conversion and one fma per logarithm, and it carries the
// irregular cases: entry 0 (zero or subnormal derivative) is -inf and entries >= 2047 (inf, NaN, sign bit) are NaN,
// so such a step poisons the running sum and the chunk is redone step by step.
constexpr int kExpEntries = 4096;
constexpr size_t kExpSmemBytes = (size_t)kExpEntries * sizeof(double2);                              // 64 KB
constexpr size_t kExactSmemBytes = kTabSmemBytes + kExpSmemBytes;
// after the tables: one staging row per warp (32 * P doubles each) for 16-byte-per-lane stores of the results
__host__ __device__ constexpr size_t exact_smem_bytes(int threads, int pixels_per_thread) {
    return kExactSmemBytes + (size_t)threads * pixels_per_thread * sizeof(double);
}

__device__ __forceinline__ bool in_unit_interval(double x) { return x > 0.0 && x < 1.0; }

// parameter values the chunked fast path may be used with: positive, finite, 2^-500 < r < 2^500
__device__ __forceinline__ bool ordinary_param(double r) {
    const unsigned hw = (unsigned)__double2hiint(r);
    return (hw - 0x20B00000u) < (0x5F300000u - 0x20B00000u);
}

struct PixelState {
    double x, lyap;
    int valid;
};

// Reference semantics, one step at a time, for `n` steps of selector word `word`.
// Returns true when the orbit left (0,1) (the reference's break).  *steps counts executed updates.
template <bool ACC>
__device__ __noinline__ bool careful_chunk(PixelState* ps, double rA, double rB, double rC, unsigned word, int n,
                                           unsigned long long* steps) {
    double x = ps->x, lyap = ps->lyap;
    int valid = ps->valid;
    bool dead = false;
    int j = 0;
    for (; j < n; ++j) {
        const unsigned sel = (word >> (2 * j)) & 3u;
        const double r = sel == 0 ? rA : (sel == 1 ? rB : rC);
        if (ACC) {
            const double deriv = fabs(__dmul_rn(r, __dsub_rn(1.0, __dmul_rn(2.0, x))));   // :69
            if (deriv > 0.0) {                                                              // :71
                lyap = __dadd_rn(lyap, lyap_log_tab(deriv, g_lyap_logtab, 1));              // :72
                ++valid;
            }
        }
        x = __dmul_rn(__dmul_rn(r, x), __dsub_rn(1.0, x));                                  // :58,76
        if (!in_unit_interval(x)) {                                                         // :60,78
            dead = true;
            ++j;
            break;
        }
    }
    *steps += (unsigned long long)j;
    ps->x = x;
    ps->lyap = lyap;
    ps->valid = valid;
    return dead;
}

// Constants of the log core in constant memory: fp64 instructions take them as constant-bank
// operands, which costs no instruction (64-bit immediates would each need two moves).
struct LogConsts {
    double c2, c3, c4, ln2hi, ln2lo, klo_bias;
};
static __constant__ LogConsts c_logk = {LYAP_LOG_C2, LYAP_LOG_C3, LYAP_LOG_C4, LYAP_LN2HI, LYAP_LN2LO, LYAP_KLO_BIAS};
static __constant__ int c_minus_2p20 = -(1 << 20);   // read as a constant-bank operand so the product below stays one multiply-add

// lyap_log_core (lyap_math.h) for a positive normal d, written against the two shared-memory tables, which start
// at the beginning of the dynamic shared memory: `lane_off` is the byte offset of this lane's copy inside a
// mantissa-table entry group ((lane & 7) * 16; groups are kTabCopies*16 bytes apart), or'ed into the bin offset so
// that the address is one logic operation plus a constant.  Same values in the same order as
// lyap_log_core (e*LN2HI + lp and (e-1023)*LN2LO are tabulated instead of computed), so same bits.
__device__ __forceinline__ double log_fast(double d, unsigned lane_off) {
    const unsigned hw = (unsigned)__double2hiint(d);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // bin index * 128 bytes, or'ed with this lane's copy offset (lane_off = (lane & 7) * 16)
    const unsigned off = ((hw >> 3) & (unsigned)((LYAP_LOG_BINS - 1) * kTabCopies * 16)) | lane_off;
    const double2 me = *reinterpret_cast<const double2*>(smem_raw + off);
    const double lp = me.x, invcb = me.y;
    const unsigned ke = hw >> 20;
    const double2 ee = reinterpret_cast<const double2*>(smem_raw + kTabSmemBytes)[ke];
    const double khi = ee.x, klo = ee.y;
    // The mantissa table holds invc with 0x3FF00000 added to its high word, so subtracting d's exponent field
    // gives invc * 2^-(exponent of d): d * that == mantissa(d) * invc exactly (a power-of-two rescaling),
    // without assembling the mantissa as a separate double.
    int invs_hi;
    asm("mad.lo.s32 %0, %1, %2, %3;" : "=r"(invs_hi) : "r"((int)ke), "r"(c_minus_2p20), "r"(__double2hiint(invcb)));
    const double invs = __hiloint2double(invs_hi, __double2loint(invcb));
    const double r = __fma_rn(d, invs, -1.0);
    double q = __fma_rn(r, c_logk.c4, c_logk.c3);
    q = __fma_rn(r, q, c_logk.c2);
    const double w = __fma_rn(r, q, 1.0);
    const double s = __fma_rn(r, w, klo);
    const double hi = __dadd_rn(khi, lp);      // exact: both on the 2^-42 grid
    return __dadd_rn(hi, s);
}

// careful_chunk for steps [first, first + n) of a region whose selector words start at `sel`.
template <bool ACC>
__device__ __noinline__ bool careful_steps(PixelState* ps, double rA, double rB, double rC, const unsigned* sel, int wrap, int first,
                                           int n, unsigned long long* steps) {
    bool dead = false;
    int j = first;
    const int end = first + n;
    while (j < end && !dead) {
        const int in_word = j & (kStepsPerWord - 1);
        const int m = min(kStepsPerWord - in_word, end - j);
        dead = careful_chunk<ACC>(ps, rA, rB, rC, sel[(j / kStepsPerWord) % wrap] >> (2 * in_word), m, steps);
        j += m;
    }
    return dead;
}

// U consecutive logistic steps of all P pixels, selector bits in `word` (step j at bits 2j, 2j+1).
// Written as one straight-line block: the orbit x (3 dependent fp64 operations per step) runs ahead
// and leaves the U derivatives behind, whose logarithms are independent of each other and of the orbit,
// so the scheduler has U*P log chains to interleave.  The sum is still accumulated in step order.
// The warp-uniform parameter choice is a select (no branch, so the block stays one scheduling region).
template <int P, bool ACC, bool HAS_C, int U>
__device__ __forceinline__ void fast_group(double (&x)[P], double (&lyap)[P], const double (&rA)[P],
                                           const double (&rB)[P], double rC, unsigned word, unsigned lane_off) {
    double d[U][P];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const bool not_a = (word >> (2 * j)) & 1u;
        const bool is_c = (word >> (2 * j + 1)) & 1u;
#pragma unroll
        for (int p = 0; p < P; ++p) {
            double r = not_a ? rB[p] : rA[p];
            if (HAS_C) r = is_c ? rC : r;
            if (ACC) {
                const double t = __fma_rn(-2.0, x[p], 1.0);      // == fl(1 - fl(2x)): 2x is exact
                d[j][p] = __dmul_rn(r, fabs(t));                 // == |r*(1-2x)| for r > 0
            }
            x[p] = __dmul_rn(__dmul_rn(r, x[p]), __dsub_rn(1.0, x[p]));
        }
    }
    if (ACC) {
        double z[U][P];
#pragma unroll
        for (int j = 0; j < U; ++j)
#pragma unroll
            for (int p = 0; p < P; ++p) z[j][p] = log_fast(d[j][p], lane_off);
#pragma unroll
        for (int p = 0; p < P; ++p) {
#pragma unroll
            for (int j = 0; j < U; ++j) lyap[p] = __dadd_rn(lyap[p], z[j][p]);
        }
    }
}

// U steps whose parameter choices are known at compile time (PAT: 2 bits per step, 0 = A, 1 = B, 2 = C):
// no selects, no per-step branches; every operand is fixed.
template <int P, bool ACC, int U, unsigned PAT>
__device__ __forceinline__ void fixed_group(double (&x)[P], double (&lyap)[P], const double (&rA)[P],
                                            const double (&rB)[P], double rC, unsigned lane_off) {
    double d[U][P];
#pragma unroll
    for (int j = 0; j < U; ++j) {
        const unsigned code = (PAT >> (2 * j)) & 3u;
#pragma unroll
        for (int p = 0; p < P; ++p) {
            const double r = code == 0 ? rA[p] : (code == 1 ? rB[p] : rC);
            if (ACC) {
                const double t = __fma_rn(-2.0, x[p], 1.0);      // == fl(1 - fl(2x)): 2x is exact
                d[j][p] = __dmul_rn(r, fabs(t));                 // == |r*(1-2x)| for r > 0
            }
            x[p] = __dmul_rn(__dmul_rn(r, x[p]), __dsub_rn(1.0, x[p]));
        }
    }
    if (ACC) {
        double z[U][P];
#pragma unroll
        for (int j = 0; j < U; ++j)
#pragma unroll
            for (int p = 0; p < P; ++p) z[j][p] = log_fast(d[j][p], lane_off);
#pragma unroll
        for (int p = 0; p < P; ++p) {
#pragma unroll
            for (int j = 0; j < U; ++j) lyap[p] = __dadd_rn(lyap[p], z[j][p]);
        }
    }
}

// 1 bit per step -> 2 bits per step (A/B patterns)
__host__ __device__ constexpr unsigned spread_bits(unsigned m) {
    return (m & 1u) | ((m & 2u) << 1) | ((m & 4u) << 2) | ((m & 8u) << 3);
}

// One group of U steps, dispatched on its pattern index to the matching straight-line body: one
// warp-uniform multiway branch per U steps instead of a choice per step.
//   !HAS_C: idx has one bit per step (0 = A, 1 = B), U is 2 or 4.   HAS_C: idx is the raw 2-bit codes, U is 2.
template <int P, bool ACC, bool HAS_C, int U>
__device__ __forceinline__ void dispatch_group(double (&x)[P], double (&lyap)[P],
                                               const double (&rA)[P], const double (&rB)[P], double rC, unsigned idx,
                                               unsigned lane_off) {
#define LYAP_CASE_AB(N) \
    case N: fixed_group<P, ACC, U, spread_bits(N)>(x, lyap, rA, rB, rC, lane_off); break;
#define LYAP_CASE_RAW(N) \
    case N: fixed_group<P, ACC, U, N>(x, lyap, rA, rB, rC, lane_off); break;
    if (HAS_C) {
        static_assert(!HAS_C || U == 2, "three-parameter groups are two steps long");
        switch (idx) {
            LYAP_CASE_RAW(0x0) LYAP_CASE_RAW(0x1) LYAP_CASE_RAW(0x2) LYAP_CASE_RAW(0x4) LYAP_CASE_RAW(0x5)
            LYAP_CASE_RAW(0x6) LYAP_CASE_RAW(0x8) LYAP_CASE_RAW(0x9) LYAP_CASE_RAW(0xA)
            default: break;   // code 3 is never produced by the host packing
        }
    } else if (U == 2) {
        if (idx & 1u) {
            if (idx & 2u) fixed_group<P, ACC, U, spread_bits(3)>(x, lyap, rA, rB, rC, lane_off);
            else fixed_group<P, ACC, U, spread_bits(1)>(x, lyap, rA, rB, rC, lane_off);
        } else {
            if (idx & 2u) fixed_group<P, ACC, U, spread_bits(2)>(x, lyap, rA, rB, rC, lane_off);
            else fixed_group<P, ACC, U, spread_bits(0)>(x, lyap, rA, rB, rC, lane_off);
        }
    } else {
        switch (idx) {
            LYAP_CASE_AB(0) LYAP_CASE_AB(1) LYAP_CASE_AB(2) LYAP_CASE_AB(3) LYAP_CASE_AB(4) LYAP_CASE_AB(5)
            LYAP_CASE_AB(6) LYAP_CASE_AB(7) LYAP_CASE_AB(8) LYAP_CASE_AB(9) LYAP_CASE_AB(10) LYAP_CASE_AB(11)
            LYAP_CASE_AB(12) LYAP_CASE_AB(13) LYAP_CASE_AB(14) LYAP_CASE_AB(15)
            default: break;
        }
    }
#undef LYAP_CASE_AB
#undef LYAP_CASE_RAW
}

// even bits of w packed into the low 16 bits
__device__ __forceinline__ unsigned compress_even_bits(unsigned w) {
    w &= 0x55555555u;
    w = (w | (w >> 1)) & 0x33333333u;
    w = (w | (w >> 2)) & 0x0F0F0F0Fu;
    w = (w | (w >> 4)) & 0x00FF00FFu;
    w = (w | (w >> 8)) & 0x0000FFFFu;
    return w;
}

// n steps of selector word `word` (2 bits per step: 0 = A, 1 = B, 2 = C).
template <int P, bool ACC, bool HAS_C, int UNROLL>
__device__ __forceinline__ void fast_chunk(double (&x)[P], double (&lyap)[P], const double (&rA)[P],
                                           const double (&rB)[P], double rC, unsigned word, int n, unsigned lane_off) {
    if (n == kStepsPerWord) {
        constexpr int U = HAS_C ? 2 : UNROLL;
        unsigned pat = HAS_C ? word : compress_even_bits(word);
        constexpr int kBits = HAS_C ? 2 * U : U;
#pragma unroll 1
        for (int h = 0; h < kStepsPerWord / U; ++h) {
            dispatch_group<P, ACC, HAS_C, U>(x, lyap, rA, rB, rC, pat & ((1u << kBits) - 1u), lane_off);
            pat >>= kBits;
        }
    } else {
#pragma unroll 1
        for (int j = 0; j < n; ++j, word >>= 2) fast_group<P, ACC, HAS_C, 1>(x, lyap, rA, rB, rC, word, lane_off);
    }
}

// ---- run-time specialisation -------------------------------------------------------------------
// For a periodic sequence the pattern of every 2-step group repeats every KG groups (KG = lcm(period, 2) / 2).
// With the KG patterns known at compile time (PATS: 4 bits per group = two 2-bit codes) a whole period is one
// straight-line block: no dispatch at all.
template <int P, bool ACC, int KG, unsigned long long PATS, int G = 0>
__device__ __forceinline__ void period_block(double (&x)[P], double (&lyap)[P], const double (&rA)[P], const double (&rB)[P],
                                             double rC, unsigned lane_off) {
    if constexpr (G < KG) {
        fixed_group<P, ACC, 2, (unsigned)((PATS >> (4 * G)) & 15ull)>(x, lyap, rA, rB, rC, lane_off);
        period_block<P, ACC, KG, PATS, G + 1>(x, lyap, rA, rB, rC, lane_off);
    }
}

__host__ __device__ constexpr bool pats_use_c(unsigned long long pats) {
    return (pats & 0xAAAAAAAAAAAAAAAAull) != 0;
}

// Body shared by the library's generic kernel (KG == 0: patterns dispatched at run time) and by a specialised
// instance (KG > 0: WU_PATS / ACC_PATS are the group patterns of the warm-up and accumulation regions).
template <int P, int THREADS, bool HAS_C, int UNROLL, int KG, unsigned long long WU_PATS, unsigned long long ACC_PATS>
__device__ __forceinline__ void lambda_exact_body(const LambdaArgs& a, double* __restrict__ out64, float* __restrict__ out32,
                  unsigned long long* __restrict__ steps_out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    lyap_logtab_entry* tab_all = reinterpret_cast<lyap_logtab_entry*>(smem_raw);
    for (int e = threadIdx.x; e < LYAP_LOG_BINS * kTabCopies; e += THREADS) {
        lyap_logtab_entry t = g_lyap_logtab[e / kTabCopies];
        t.invc = __hiloint2double(__double2hiint(t.invc) + 0x3FF00000, __double2loint(t.invc));   // see log_fast
        tab_all[e] = t;
    }
    const unsigned lane_off = (threadIdx.x & (kTabCopies - 1)) * 16u;
    double2* exp_tab = reinterpret_cast<double2*>(smem_raw + kTabSmemBytes);
    for (int e = threadIdx.x; e < kExpEntries; e += THREADS) {
        double2 v;
        if (e == 0) v = make_double2(__longlong_as_double(0xFFF0000000000000LL), 0.0);                       // zero / subnormal derivative
        else if (e >= 2047) v = make_double2(__longlong_as_double(0x7FF8000000000000LL), 0.0);                // inf, NaN, or a set sign bit
        else v = make_double2(__dmul_rn((double)e, LYAP_LN2HI), __fma_rn((double)e, LYAP_LN2LO, LYAP_KLO_BIAS));
        exp_tab[e] = v;
    }
    __syncthreads();   // both tables are read across warps from the first logarithm on (at once when warmup == 0)

    unsigned long long my_steps = 0;
    // Work is dealt out per WARP: warp-tile t is the 32*P consecutive pixels from t*32*P, and the warps of the grid take
    // them round-robin, warp index first (tile t goes to warp t / gridDim of block t % gridDim), so that when the tiles
    // do not fill a whole number of rounds every SM gets the same mix of busier and idler warps.  (Dealt out per block,
    // a frame of 9.1 rounds costs 10; this way it costs about 9.1.)
    const long long tile_px = 32LL * P;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long warps_in_grid = (long long)gridDim.x * (THREADS / 32);
    const int n_regions = 2;

    for (long long tile = (long long)warp * gridDim.x + blockIdx.x; tile * tile_px < a.n_pixels; tile += warps_in_grid) {
        const long long idx0 = tile * tile_px + (long long)lane * P;
        double x[P], lyap[P], rA[P], rB[P], lam[P];
        const double rC = a.c_value;
        int valid[P];
        bool done[P], careful_only[P];

        {
            long long row = idx0 / a.width;
            int col = (int)(idx0 - row * a.width);
            row += a.row_begin;
#pragma unroll
            for (int p = 0; p < P; ++p) {
                const bool inside = idx0 + p < a.n_pixels;
                rB[p] = __dadd_rn(a.min_y, __dmul_rn(a.dy, (double)(int)row));   // :42
                rA[p] = __dadd_rn(a.min_x, __dmul_rn(a.dx, (double)col));        // :45
                x[p] = 0.5;                                                       // :31,52
                lyap[p] = 0.0;
                valid[p] = 0;
                lam[p] = -5.0;
                done[p] = !inside || rA[p] <= 0.0 || rB[p] <= 0.0;                // :47-50
                careful_only[p] = !(ordinary_param(rA[p]) && ordinary_param(rB[p]) && a.fast_ok_c);
                if (++col == a.width) {
                    col = 0;
                    ++row;
                }
            }
        }

        for (int region = 0; region < n_regions; ++region) {
            const bool acc = region == 1;
            const int nsteps = acc ? a.iterations : a.warmup;
            const int word0 = acc ? a.acc_word0 : 0;
            const int wrap = acc ? a.acc_wrap : a.wu_wrap;
            if constexpr (KG > 0) {
                // specialised walk: chunks of REP blocks of CB whole periods (>= 16 steps each), then one block, whole periods, single steps
                // REP = 2 blocks between exit tests measured best (1: more tests and state copies; 3 and more: slower code)
                constexpr int BS = 2 * KG, CB = (kStepsPerWord + BS - 1) / BS, REP = 2, CS = CB * BS * REP;
                const unsigned* sel = a.sel + word0;
                int s = 0;
                while (s < nsteps) {
                    bool all_done = true;
#pragma unroll
                    for (int p = 0; p < P; ++p) all_done = all_done && done[p];
                    if (__all_sync(0xFFFFFFFFu, all_done)) break;
                    const int left = nsteps - s;
                    const int n = left >= CS ? CS : (left >= CB * BS ? CB * BS : (left >= BS ? left / BS * BS : left));
                    double sx[P], sl[P];
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        sx[p] = x[p];
                        sl[p] = lyap[p];
                    }
                    if (left >= CS) {             // CB whole periods, straight-line, REP times
#pragma unroll 1
                        for (int rep = 0; rep < REP; ++rep) {
#pragma unroll
                            for (int b = 0; b < CB; ++b) {
                                if (acc) period_block<P, true, KG, ACC_PATS>(x, lyap, rA, rB, rC, lane_off);
                                else period_block<P, false, KG, WU_PATS>(x, lyap, rA, rB, rC, lane_off);
                            }
                        }
                    } else if (left >= CB * BS) { // one straight-line block
#pragma unroll
                        for (int b = 0; b < CB; ++b) {
                            if (acc) period_block<P, true, KG, ACC_PATS>(x, lyap, rA, rB, rC, lane_off);
                            else period_block<P, false, KG, WU_PATS>(x, lyap, rA, rB, rC, lane_off);
                        }
                    } else if (left >= BS) {      // the last few whole periods
#pragma unroll 1
                        for (int b = 0; b < n / BS; ++b) {
                            if (acc) period_block<P, true, KG, ACC_PATS>(x, lyap, rA, rB, rC, lane_off);
                            else period_block<P, false, KG, WU_PATS>(x, lyap, rA, rB, rC, lane_off);
                        }
                    } else {                      // less than one period: one step at a time
#pragma unroll 1
                        for (int j = s; j < nsteps; ++j) {
                            const unsigned code = (sel[(j / kStepsPerWord) % wrap] >> (2 * (j & (kStepsPerWord - 1)))) & 3u;
                            if (acc) fast_group<P, true, HAS_C, 1>(x, lyap, rA, rB, rC, code, lane_off);
                            else fast_group<P, false, HAS_C, 1>(x, lyap, rA, rB, rC, code, lane_off);
                        }
                    }
#pragma unroll
                    for (int p = 0; p < P; ++p) {
                        if (done[p]) continue;
                        const bool regular = !careful_only[p] && in_unit_interval(x[p]) && isfinite(lyap[p]);
                        if (regular) {
                            if (acc) valid[p] += n;
                            my_steps += (unsigned long long)n;
                        } else {
                            PixelState ps{sx[p], sl[p], valid[p]};
                            const bool dead = acc ? careful_steps<true>(&ps, rA[p], rB[p], rC, sel, wrap, s, n, &my_steps)
                                                  : careful_steps<false>(&ps, rA[p], rB[p], rC, sel, wrap, s, n, &my_steps);
                            x[p] = ps.x;
                            lyap[p] = ps.lyap;
                            valid[p] = ps.valid;
                            if (dead) {
                                done[p] = true;
                                lam[p] = ps.valid > 0 ? __ddiv_rn(ps.lyap, __dmul_rn((double)ps.valid, LYAP_LN2)) : -5.0;   // :84-85
                                x[p] = 0.25;
                            }
                        }
                    }
                    s += n;
                }
                continue;
            }
            // generic walk: the selector words one after the other, exit tests after every second full word
            const unsigned* sel = a.sel + word0;
            int s = 0, wi = 0;
            while (s < nsteps) {
                bool all_done = true;
#pragma unroll
                for (int p = 0; p < P; ++p) all_done = all_done && done[p];
                if (__all_sync(0xFFFFFFFFu, all_done)) break;

                const int left = nsteps - s;
                const int n = left >= 2 * kStepsPerWord ? 2 * kStepsPerWord : (left >= kStepsPerWord ? kStepsPerWord : left);
                double sx[P], sl[P];
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    sx[p] = x[p];
                    sl[p] = lyap[p];
                }
#pragma unroll 1
                for (int k = 0; k < n; k += kStepsPerWord) {
                    const unsigned word = sel[wi];
                    if (++wi == wrap) wi = 0;
                    const int m = min(kStepsPerWord, n - k);
                    if (acc) fast_chunk<P, true, HAS_C, UNROLL>(x, lyap, rA, rB, rC, word, m, lane_off);
                    else fast_chunk<P, false, HAS_C, UNROLL>(x, lyap, rA, rB, rC, word, m, lane_off);
                }
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    if (done[p]) continue;
                    // an irregular derivative (zero, subnormal, non-finite) has made the sum non-finite through the exponent table
                    const bool regular = !careful_only[p] && in_unit_interval(x[p]) && isfinite(lyap[p]);
                    if (regular) {
                        if (acc) valid[p] += n;
                        my_steps += (unsigned long long)n;
                    } else {
                        PixelState ps{sx[p], sl[p], valid[p]};
                        const bool dead = acc ? careful_steps<true>(&ps, rA[p], rB[p], rC, sel, wrap, s, n, &my_steps)
                                              : careful_steps<false>(&ps, rA[p], rB[p], rC, sel, wrap, s, n, &my_steps);
                        x[p] = ps.x;
                        lyap[p] = ps.lyap;
                        valid[p] = ps.valid;
                        if (dead) {
                            done[p] = true;
                            lam[p] = ps.valid > 0 ? __ddiv_rn(ps.lyap, __dmul_rn((double)ps.valid, LYAP_LN2)) : -5.0;   // :84-85
                            x[p] = 0.25;   // keep the abandoned lane's arithmetic tame
                        }
                    }
                }
                s += n;
            }
        }

#pragma unroll
        for (int p = 0; p < P; ++p) {
            if (!done[p]) lam[p] = valid[p] > 0 ? __ddiv_rn(lyap[p], __dmul_rn((double)valid[p], LYAP_LN2)) : -5.0;
        }

        // stores: each warp's 32*P consecutive values go through the warp's own staging row in shared memory, so that every
        // lane writes 16 bytes and a store instruction covers consecutive 512-byte runs whatever P is (no block-wide barrier:
        // warps stay out of step with each other); a ragged last tile or a misaligned output pointer takes plain stores
        const long long tile0 = tile * tile_px;
        const bool full_tile = tile0 + tile_px <= a.n_pixels;
        double* stage = reinterpret_cast<double*>(smem_raw + kExactSmemBytes) + warp * (32 * P);
        if (out64) {
            if (full_tile && ((reinterpret_cast<uintptr_t>(out64 + tile0) & 15) == 0)) {
                __syncwarp();   // the row is free (this warp's reads of the previous tile are done)
#pragma unroll
                for (int p = 0; p < P; ++p) stage[lane * P + p] = lam[p];
                __syncwarp();
                double2* dst = reinterpret_cast<double2*>(out64 + tile0);
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
                float4* dst = reinterpret_cast<float4*>(out32 + tile0);
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


template <int P, int THREADS, bool HAS_C, int UNROLL>
__global__ void __launch_bounds__(THREADS, 1)
k_lambda_exact(const __grid_constant__ LambdaArgs a, double* __restrict__ out64, float* __restrict__ out32,
               unsigned long long* __restrict__ steps_out) {
    lambda_exact_body<P, THREADS, HAS_C, UNROLL, 0, 0ull, 0ull>(a, out64, out32, steps_out);
}

#if defined(LYAP_SPEC_EXACT)
// The specialised instance; LYAP_SPEC_* are given on the run-time compiler's command line.
extern "C" __global__ void __launch_bounds__(LYAP_SPEC_THREADS, 1)
k_lambda_exact_spec(const __grid_constant__ LambdaArgs a, double* __restrict__ out64, float* __restrict__ out32,
                    unsigned long long* __restrict__ steps_out) {
    lambda_exact_body<LYAP_SPEC_P, LYAP_SPEC_THREADS, pats_use_c(LYAP_SPEC_WU_PATS | LYAP_SPEC_ACC_PATS), 2, LYAP_SPEC_KG,
                      LYAP_SPEC_WU_PATS, LYAP_SPEC_ACC_PATS>(a, out64, out32, steps_out);
}
#endif

}  // namespace lyap
