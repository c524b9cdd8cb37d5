// lyap_kernels.cu -- sm_100a kernels of the Lyapunov-fractal engine.
//
//   k_lambda_exact   FractalComputer::computeFractal  (reference src/lyapunov_fractal.hpp:41-86)
//   k_minmax         normalizeData pass 1             (src/lyapunov_fractal.hpp:110-120)
//   k_normalize      normalizeData pass 2             (src/lyapunov_fractal.hpp:122-137)
//   k_colorize       box mean + palette + RGBA store  (web/fractal_renderer.js:283-311,207-281,191-198)
//
// Build with -fmad=false: the exact kernels may only fuse where an fma is written out.
#include <cfloat>
#include <math_constants.h>
#include <cstdint>
#include <cstdlib>

#include "lyap_engine.h"
#include "lyap_math.h"

namespace lyap {

__device__ const lyap_logtab_entry g_lyap_logtab[LYAP_LOG_BINS] = {LYAP_LOG_TABLE_INIT};

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
// Steps run in chunks of up to 16 without per-step exit tests.  That is sound because leaving (0,1)
// is permanent for x <- r x (1-x) with r > 0 (x >= 1 gives x <= 0 next, x <= 0 stays <= 0, NaN stays
// NaN), so testing x after the chunk finds every exit, and the only other irregular event, a zero
// derivative (x == 0.5 exactly, skipped and not counted by the reference, :71-74), has exponent field 0,
// for which the exponent table holds -inf: the running sum turns non-finite.  A chunk in which anything irregular
// happened is rolled back and redone by `careful_chunk`, which follows the reference step by step.
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
__constant__ LogConsts c_logk = {LYAP_LOG_C2, LYAP_LOG_C3, LYAP_LOG_C4, LYAP_LN2HI, LYAP_LN2LO, LYAP_KLO_BIAS};
__constant__ int c_minus_2p20 = -(1 << 20);   // read as a constant-bank operand so the product below stays one multiply-add

// lyap_log_core (lyap_math.h) for a positive normal d, written against the two shared-memory tables:
// `tab_addr` is the shared-window byte address of this lane's copy of entry 0 of the mantissa table (entries are
// kTabCopies*16 bytes apart), `exp_addr` that of the exponent table.  Same values in the same order as
// lyap_log_core (e*LN2HI + lp and (e-1023)*LN2LO are tabulated instead of computed), so same bits.
__device__ __forceinline__ double log_fast(double d, unsigned tab_addr, unsigned exp_addr) {
    const unsigned hw = (unsigned)__double2hiint(d);
    const unsigned off = (hw >> 3) & (unsigned)((LYAP_LOG_BINS - 1) * kTabCopies * 16);   // bin index * 128 bytes
    double lp, invcb;
    asm("ld.shared.v2.f64 {%0, %1}, [%2];" : "=d"(lp), "=d"(invcb) : "r"(tab_addr + off));
    const unsigned ke = hw >> 20;
    double khi, klo;
    asm("ld.shared.v2.f64 {%0, %1}, [%2];" : "=d"(khi), "=d"(klo) : "r"(exp_addr + ke * 16u));
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

// U consecutive logistic steps of all P pixels, selector bits in `word` (step j at bits 2j, 2j+1).
// Written as one straight-line block: the orbit x (3 dependent fp64 operations per step) runs ahead
// and leaves the U derivatives behind, whose logarithms are independent of each other and of the orbit,
// so the scheduler has U*P log chains to interleave.  The sum is still accumulated in step order.
// The warp-uniform parameter choice is a select (no branch, so the block stays one scheduling region).
template <int P, bool ACC, bool HAS_C, int U>
__device__ __forceinline__ void fast_group(double (&x)[P], double (&lyap)[P], const double (&rA)[P],
                                           const double (&rB)[P], double rC, unsigned word, unsigned tab_addr, unsigned exp_addr) {
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
            for (int p = 0; p < P; ++p) z[j][p] = log_fast(d[j][p], tab_addr, exp_addr);
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
                                            const double (&rB)[P], double rC, unsigned tab_addr, unsigned exp_addr) {
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
            for (int p = 0; p < P; ++p) z[j][p] = log_fast(d[j][p], tab_addr, exp_addr);
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
                                               unsigned tab_addr, unsigned exp_addr) {
#define LYAP_CASE_AB(N) \
    case N: fixed_group<P, ACC, U, spread_bits(N)>(x, lyap, rA, rB, rC, tab_addr, exp_addr); break;
#define LYAP_CASE_RAW(N) \
    case N: fixed_group<P, ACC, U, N>(x, lyap, rA, rB, rC, tab_addr, exp_addr); break;
    if (HAS_C) {
        static_assert(!HAS_C || U == 2, "three-parameter groups are two steps long");
        switch (idx) {
            LYAP_CASE_RAW(0x0) LYAP_CASE_RAW(0x1) LYAP_CASE_RAW(0x2) LYAP_CASE_RAW(0x4) LYAP_CASE_RAW(0x5)
            LYAP_CASE_RAW(0x6) LYAP_CASE_RAW(0x8) LYAP_CASE_RAW(0x9) LYAP_CASE_RAW(0xA)
            default: break;   // code 3 is never produced by the host packing
        }
    } else if (U == 2) {
        if (idx & 1u) {
            if (idx & 2u) fixed_group<P, ACC, U, spread_bits(3)>(x, lyap, rA, rB, rC, tab_addr, exp_addr);
            else fixed_group<P, ACC, U, spread_bits(1)>(x, lyap, rA, rB, rC, tab_addr, exp_addr);
        } else {
            if (idx & 2u) fixed_group<P, ACC, U, spread_bits(2)>(x, lyap, rA, rB, rC, tab_addr, exp_addr);
            else fixed_group<P, ACC, U, spread_bits(0)>(x, lyap, rA, rB, rC, tab_addr, exp_addr);
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
                                           const double (&rB)[P], double rC, unsigned word, int n, unsigned tab_addr, unsigned exp_addr) {
    if (n == kStepsPerWord) {
        constexpr int U = HAS_C ? 2 : UNROLL;
        unsigned pat = HAS_C ? word : compress_even_bits(word);
        constexpr int kBits = HAS_C ? 2 * U : U;
#pragma unroll 1
        for (int h = 0; h < kStepsPerWord / U; ++h) {
            dispatch_group<P, ACC, HAS_C, U>(x, lyap, rA, rB, rC, pat & ((1u << kBits) - 1u), tab_addr, exp_addr);
            pat >>= kBits;
        }
    } else {
#pragma unroll 1
        for (int j = 0; j < n; ++j, word >>= 2) fast_group<P, ACC, HAS_C, 1>(x, lyap, rA, rB, rC, word, tab_addr, exp_addr);
    }
}

template <int P, int THREADS, bool HAS_C, int UNROLL>
__global__ void __launch_bounds__(THREADS, 1)
k_lambda_exact(const __grid_constant__ LambdaArgs a, double* __restrict__ out64, float* __restrict__ out32,
               unsigned long long* __restrict__ steps_out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    lyap_logtab_entry* tab_all = reinterpret_cast<lyap_logtab_entry*>(smem_raw);
    for (int e = threadIdx.x; e < LYAP_LOG_BINS * kTabCopies; e += THREADS) {
        lyap_logtab_entry t = g_lyap_logtab[e / kTabCopies];
        t.invc = __hiloint2double(__double2hiint(t.invc) + 0x3FF00000, __double2loint(t.invc));   // see log_fast
        tab_all[e] = t;
    }
    __syncthreads();
    const lyap_logtab_entry* tab = tab_all + (threadIdx.x & (kTabCopies - 1));
    const unsigned tab_addr = (unsigned)__cvta_generic_to_shared(tab);
    double2* exp_tab = reinterpret_cast<double2*>(smem_raw + kTabSmemBytes);
    for (int e = threadIdx.x; e < kExpEntries; e += THREADS) {
        double2 v;
        if (e == 0) v = make_double2(-CUDART_INF, 0.0);                       // zero / subnormal derivative
        else if (e >= 2047) v = make_double2(CUDART_NAN, 0.0);                // inf, NaN, or a set sign bit
        else v = make_double2(__dmul_rn((double)e, LYAP_LN2HI), __fma_rn((double)e, LYAP_LN2LO, LYAP_KLO_BIAS));
        exp_tab[e] = v;
    }
    const unsigned exp_addr = (unsigned)__cvta_generic_to_shared(exp_tab);

    unsigned long long my_steps = 0;
    const long long tile_px = (long long)THREADS * P;
    const int n_regions = 2;

    for (long long tile = blockIdx.x; tile * tile_px < a.n_pixels; tile += gridDim.x) {
        const long long idx0 = tile * tile_px + (long long)threadIdx.x * P;
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
            const int nchunks = (nsteps + kStepsPerWord - 1) / kStepsPerWord;
            for (int c = 0; c < nchunks; ++c) {
                bool all_done = true;
#pragma unroll
                for (int p = 0; p < P; ++p) all_done = all_done && done[p];
                if (__all_sync(0xFFFFFFFFu, all_done)) break;

                const unsigned word = a.sel[word0 + c];
                const int n = min(kStepsPerWord, nsteps - c * kStepsPerWord);
                double sx[P], sl[P];
#pragma unroll
                for (int p = 0; p < P; ++p) {
                    sx[p] = x[p];
                    sl[p] = lyap[p];
                }
                if (acc) fast_chunk<P, true, HAS_C, UNROLL>(x, lyap, rA, rB, rC, word, n, tab_addr, exp_addr);
                else fast_chunk<P, false, HAS_C, UNROLL>(x, lyap, rA, rB, rC, word, n, tab_addr, exp_addr);
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
                        const bool dead = acc ? careful_chunk<true>(&ps, rA[p], rB[p], rC, word, n, &my_steps)
                                              : careful_chunk<false>(&ps, rA[p], rB[p], rC, word, n, &my_steps);
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
            }
        }

#pragma unroll
        for (int p = 0; p < P; ++p) {
            if (!done[p]) lam[p] = valid[p] > 0 ? __ddiv_rn(lyap[p], __dmul_rn((double)valid[p], LYAP_LN2)) : -5.0;
        }

        // stores: one 16-byte (fp64) / 8-byte (fp32) store per pixel pair when aligned
        if (out64) {
            if (P % 2 == 0 && idx0 + P <= a.n_pixels && ((reinterpret_cast<uintptr_t>(out64 + idx0) & 15) == 0)) {
#pragma unroll
                for (int p = 0; p < P; p += 2)
                    *reinterpret_cast<double2*>(out64 + idx0 + p) = make_double2(lam[p], lam[p + 1 < P ? p + 1 : p]);
            } else {
#pragma unroll
                for (int p = 0; p < P; ++p)
                    if (idx0 + p < a.n_pixels) out64[idx0 + p] = lam[p];
            }
        }
        if (out32) {
            if (P % 2 == 0 && idx0 + P <= a.n_pixels && ((reinterpret_cast<uintptr_t>(out32 + idx0) & 7) == 0)) {
#pragma unroll
                for (int p = 0; p < P; p += 2)
                    *reinterpret_cast<float2*>(out32 + idx0 + p) =
                        make_float2((float)lam[p], (float)lam[p + 1 < P ? p + 1 : p]);
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
static cudaError_t launch_exact_variant(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                        int sm_count, cudaStream_t st) {
    auto kern = k_lambda_exact<P, THREADS, HAS_C, UNROLL>;
    // the attribute is per device and cheap to set; doing it on every launch keeps this thread- and device-safe
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kExactSmemBytes);
    if (e != cudaSuccess) return e;
    const long long tile_px = (long long)THREADS * P;
    const long long tiles = (a.n_pixels + tile_px - 1) / tile_px;
    if (tiles <= 0) return cudaSuccess;
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    kern<<<grid, THREADS, kExactSmemBytes, st>>>(a, out64, out32, steps);
    return cudaGetLastError();
}

// Pixels per thread for a launch of n pixels.  Large frames: 3 (measured best on B200).  Small frames are
// dominated by how many rounds of tiles the busiest SM runs, so the count that minimises rounds * pixels-per-thread
// (weighted by each shape's measured per-pixel cost) is taken.  LYAP_EXACT_VARIANT=0..4 overrides (tuning knob).
static int exact_pixels_per_thread(long long n_pixels, int sm_count, int* threads) {
    static const int env = [] {
        const char* e = getenv("LYAP_EXACT_VARIANT");
        return e ? atoi(e) : -1;
    }();
    *threads = 512;
    switch (env) {
        case 0: return 3;
        case 1: return 2;
        case 3: return 4;
        case 4: *threads = 1024; return 2;
        default: break;
    }
    const int cand[3] = {3, 2, 4};
    const double cost[3] = {1.0, 1.035, 1.015};
    int best = 3;
    double best_t = 1e300;
    for (int i = 0; i < 3; ++i) {
        const long long tiles = (n_pixels + 512LL * cand[i] - 1) / (512LL * cand[i]);
        const long long rounds = (tiles + sm_count - 1) / sm_count;
        const double t = (double)rounds * cand[i] * cost[i];
        if (t < best_t * 0.999) {
            best_t = t;
            best = cand[i];
        }
    }
    return best;
}

cudaError_t launch_lambda_exact(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                int sm_count, cudaStream_t st) {
    bool has_c = false;
    const int words = a.acc_word0 + (a.iterations + kStepsPerWord - 1) / kStepsPerWord;
    for (int i = 0; i < words; ++i) has_c = has_c || (a.sel[i] & 0xAAAAAAAAu);
#define LYAP_VARIANT(P, T, U)                                                                    \
    (has_c ? launch_exact_variant<P, T, true, U>(a, out64, out32, steps, sm_count, st)            \
           : launch_exact_variant<P, T, false, U>(a, out64, out32, steps, sm_count, st))
    int threads = 512;
    const int ppt = exact_pixels_per_thread(a.n_pixels, sm_count, &threads);
    if (threads == 1024) return LYAP_VARIANT(2, 1024, 2);
    if (ppt == 2) return LYAP_VARIANT(2, 512, 2);
    if (ppt == 4) return LYAP_VARIANT(4, 512, 2);
    return LYAP_VARIANT(3, 512, 2);
#undef LYAP_VARIANT
}

// ---------------------------------------------------------------------------------------------
// normalizeData pass 1: min / max over finite values > -4.
// Results are selections, so any reduction order gives the reference's bits.
// ---------------------------------------------------------------------------------------------
constexpr int kMinmaxThreads = 256;

__device__ __forceinline__ void minmax_take(double v, double& lo, double& hi) {
    if (isfinite(v) && v > -4.0) {     // :116
        lo = fmin(lo, v);
        hi = fmax(hi, v);
    }
}

__global__ void __launch_bounds__(kMinmaxThreads)
k_minmax(const double* __restrict__ v, unsigned long long n, double* __restrict__ minmax, double* partial,
         unsigned int* ticket) {
    double lo = DBL_MAX, hi = -DBL_MAX;   // :110-111
    const unsigned long long tid = (unsigned long long)blockIdx.x * kMinmaxThreads + threadIdx.x;
    const unsigned long long nthreads = (unsigned long long)gridDim.x * kMinmaxThreads;
    const bool aligned = (reinterpret_cast<uintptr_t>(v) & 15) == 0;
    if (aligned) {
        const unsigned long long n2 = n / 2;
        const double2* v2 = reinterpret_cast<const double2*>(v);
        for (unsigned long long i = tid; i < n2; i += nthreads) {
            const double2 q = v2[i];
            minmax_take(q.x, lo, hi);
            minmax_take(q.y, lo, hi);
        }
        if (tid == 0 && (n & 1)) minmax_take(v[n - 1], lo, hi);
    } else {
        for (unsigned long long i = tid; i < n; i += nthreads) minmax_take(v[i], lo, hi);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        lo = fmin(lo, __shfl_down_sync(0xFFFFFFFFu, lo, o));
        hi = fmax(hi, __shfl_down_sync(0xFFFFFFFFu, hi, o));
    }
    __shared__ double s_lo[kMinmaxThreads / 32], s_hi[kMinmaxThreads / 32];
    __shared__ bool s_last;
    if ((threadIdx.x & 31) == 0) {
        s_lo[threadIdx.x >> 5] = lo;
        s_hi[threadIdx.x >> 5] = hi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kMinmaxThreads / 32; ++w) {
            lo = fmin(lo, s_lo[w]);
            hi = fmax(hi, s_hi[w]);
        }
        partial[2 * blockIdx.x] = lo;
        partial[2 * blockIdx.x + 1] = hi;
        __threadfence();
        const unsigned t = atomicAdd(ticket, 1u);
        s_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (s_last) {
        __threadfence();
        lo = DBL_MAX;
        hi = -DBL_MAX;
        for (unsigned b = threadIdx.x; b < gridDim.x; b += kMinmaxThreads) {
            lo = fmin(lo, __ldcg(&partial[2 * b]));
            hi = fmax(hi, __ldcg(&partial[2 * b + 1]));
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            lo = fmin(lo, __shfl_down_sync(0xFFFFFFFFu, lo, o));
            hi = fmax(hi, __shfl_down_sync(0xFFFFFFFFu, hi, o));
        }
        __syncthreads();
        if ((threadIdx.x & 31) == 0) {
            s_lo[threadIdx.x >> 5] = lo;
            s_hi[threadIdx.x >> 5] = hi;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w = 1; w < kMinmaxThreads / 32; ++w) {
                lo = fmin(lo, s_lo[w]);
                hi = fmax(hi, s_hi[w]);
            }
            minmax[0] = lo;
            minmax[1] = hi;
            *ticket = 0;   // ready for the next launch
        }
    }
}

cudaError_t launch_minmax(const double* v, unsigned long long n, double* minmax, void* scratch, cudaStream_t st) {
    double* partial = static_cast<double*>(scratch);
    unsigned int* ticket = reinterpret_cast<unsigned int*>(partial + 2 * kMinmaxBlocks);
    unsigned long long want = (n / 2 + kMinmaxThreads - 1) / kMinmaxThreads;
    if (want < 1) want = 1;
    const int grid = (int)(want < (unsigned long long)kMinmaxBlocks ? want : kMinmaxBlocks);
    k_minmax<<<grid, kMinmaxThreads, 0, st>>>(v, n, minmax, partial, ticket);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Min/max without any allocation (lyap_minmax_device_noalloc in the public header).
//
// Same kernel as above; its scratch (per-block partial results and the arrival ticket) is this fixed
// array in the library image instead of memory owned by a context.  In host code the array's name is
// only a handle: the address a kernel can use is obtained once per device with cudaGetSymbolAddress,
// with that device current, and cached.
// ---------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_minmax_fixed_scratch[(kMinmaxScratchBytes + 255) / 256 * 256];

}  // namespace lyap

#include <mutex>

#include "../../include/lyap_b200.h"

extern "C" int lyap_minmax_device_noalloc(const double* d_values, uint64_t n, double* d_minmax, void* cuda_stream) {
    using namespace lyap;
    if (!d_minmax || (!d_values && n)) return set_error(LYAP_ERR_INVALID, "lyap_minmax_device_noalloc: null pointer");
    if (n > LYAP_NOALLOC_MAX_VALUES)
        return set_error(LYAP_ERR_TOO_LARGE, "lyap_minmax_device_noalloc: n exceeds LYAP_NOALLOC_MAX_VALUES (2^32 values)");
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void* scratch_of_device[kMaxDevices] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return set_error(LYAP_ERR_INVALID, "lyap_minmax_device_noalloc: device ordinal out of range");
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!scratch_of_device[dev]) {   // one-time set-up for this device (it is the current one)
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_minmax_fixed_scratch);
            if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
            scratch_of_device[dev] = p;
        }
        scratch = scratch_of_device[dev];
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    // the arrival ticket must start at zero; the array keeps whatever the last call (or an aborted one) left
    unsigned int* ticket = reinterpret_cast<unsigned int*>(static_cast<double*>(scratch) + 2 * kMinmaxBlocks);
    e = cudaMemsetAsync(ticket, 0, 16, st);
    if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
    e = launch_minmax(d_values, n, d_minmax, scratch, st);
    if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
    return LYAP_OK;
}

namespace lyap {

// ---------------------------------------------------------------------------------------------
// normalizeData pass 2.
// ---------------------------------------------------------------------------------------------
constexpr int kNormThreads = 256;

__device__ __forceinline__ double normalize_one(double val, double mn, double range_inv, const lyap_logtab_entry* tab) {
    if (isfinite(val) && val > -4.0) {                                                   // :130
        const double t = __dmul_rn(__dsub_rn(val, mn), range_inv);                       // :131
        const double s = lyap_pow_tab(t, 1.2, tab, 1);                                   // :132
        return __ddiv_rn(1.0, __dadd_rn(1.0, lyap_exp(__dmul_rn(-7.0, __dsub_rn(s, 0.5)))));   // :133
    }
    return 0.0;                                                                          // :135
}

__global__ void __launch_bounds__(kNormThreads)
k_normalize(const double* __restrict__ v, unsigned long long n, const double* __restrict__ minmax,
            double* __restrict__ out) {
    __shared__ lyap_logtab_entry tab[LYAP_LOG_BINS];
    for (int e = threadIdx.x; e < LYAP_LOG_BINS; e += kNormThreads) tab[e] = g_lyap_logtab[e];
    __syncthreads();
    const double mn = minmax[0], mx = minmax[1];
    const bool degenerate = mn >= mx;                                                    // :122
    const double range_inv = __ddiv_rn(1.0, __dsub_rn(mx, mn));                          // :124-125
    const unsigned long long tid = (unsigned long long)blockIdx.x * kNormThreads + threadIdx.x;
    const unsigned long long nthreads = (unsigned long long)gridDim.x * kNormThreads;
    const bool aligned = ((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15) == 0;
    if (aligned) {
        const unsigned long long n2 = n / 2;
        const double2* v2 = reinterpret_cast<const double2*>(v);
        double2* o2 = reinterpret_cast<double2*>(out);
        for (unsigned long long i = tid; i < n2; i += nthreads) {
            const double2 q = v2[i];
            double2 r;
            r.x = degenerate ? 0.0 : normalize_one(q.x, mn, range_inv, tab);
            r.y = degenerate ? 0.0 : normalize_one(q.y, mn, range_inv, tab);
            o2[i] = r;
        }
        if (tid == 0 && (n & 1)) out[n - 1] = degenerate ? 0.0 : normalize_one(v[n - 1], mn, range_inv, tab);
    } else {
        for (unsigned long long i = tid; i < n; i += nthreads)
            out[i] = degenerate ? 0.0 : normalize_one(v[i], mn, range_inv, tab);
    }
}

cudaError_t launch_normalize(const double* v, unsigned long long n, const double* minmax, double* out,
                             int sm_count, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    unsigned long long want = (n / 2 + kNormThreads - 1) / kNormThreads;
    if (want < 1) want = 1;
    const unsigned long long cap = (unsigned long long)sm_count * 8;
    const int grid = (int)(want < cap ? want : cap);
    k_normalize<<<grid, kNormThreads, 0, st>>>(v, n, minmax, out);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Colour stage: 3x3 mean (edge-aware, fixed summation order) -> palette -> clamped bytes, alpha 255.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned clamp_u8(double v) {   // Uint8ClampedArray store of an integer-valued double
    if (!(v > 0.0)) return 0u;                              // negatives and NaN -> 0
    if (v >= 255.0) return 255u;
    return (unsigned)(int)v;
}

__device__ __forceinline__ double hue2rgb(double p, double q, double t) {   // web/fractal_renderer.js:32-39
    if (t < 0) t = __dadd_rn(t, 1.0);
    if (t > 1) t = __dsub_rn(t, 1.0);
    if (t < 1.0 / 6) return __dadd_rn(p, __dmul_rn(__dmul_rn(__dsub_rn(q, p), 6.0), t));
    if (t < 1.0 / 2) return q;
    if (t < 2.0 / 3) return __dadd_rn(p, __dmul_rn(__dmul_rn(__dsub_rn(q, p), __dsub_rn(2.0 / 3, t)), 6.0));
    return p;
}

__device__ __forceinline__ double scale255(double v) { return floor(__dmul_rn(255.0, v)); }

__device__ unsigned palette_rgba(double t, int palette, const lyap_logtab_entry* tab) {
    const double PI = LYAP_PI;
    const double mid = __dmul_rn(fabs(__dsub_rn(t, 0.5)), 2.0);
    const double I = __dsub_rn(1.0, mid);
    double r, g, b;
    switch (palette) {
        default:
        case 0: {   // cosmic :209-218
            const double ph = __dmul_rn(mid, PI);
            r = scale255(__dadd_rn(__dmul_rn(I, 0.8), __dmul_rn(0.2, lyap_sin(ph))));
            g = scale255(__dmul_rn(I, 0.3));
            b = scale255(__dadd_rn(__dmul_rn(I, 0.9), __dmul_rn(0.1, lyap_cos(ph))));
        } break;
        case 1:     // nebula :219-227
            r = scale255(__dadd_rn(__dmul_rn(I, 0.9), __dmul_rn(0.1, lyap_pow_tab(t, 1.5, tab, 1))));
            g = scale255(__dmul_rn(I, 0.5));
            b = scale255(__dmul_rn(I, 0.8));
            break;
        case 2: {   // aurora :228-237
            const double ph = __dmul_rn(mid, PI);
            r = scale255(__dmul_rn(I, 0.6));
            g = scale255(__dadd_rn(__dmul_rn(I, 0.9), __dmul_rn(0.1, lyap_sin(ph))));
            b = scale255(__dmul_rn(I, 0.7));
        } break;
        case 3:     // solarflare :238-246
            r = scale255(__dmul_rn(I, 0.95));
            g = scale255(__dmul_rn(I, 0.6));
            b = scale255(__dmul_rn(I, 0.2));
            break;
        case 4: {   // blackhole :247-256
            const double ph = __dmul_rn(mid, PI);
            r = scale255(__dmul_rn(I, 0.5));
            g = scale255(__dmul_rn(I, 0.7));
            b = scale255(__dadd_rn(__dmul_rn(I, 0.9), __dmul_rn(0.1, lyap_sin(ph))));
        } break;
        case 5: {   // psychedelic :257-266
            const double ph = __dmul_rn(__dmul_rn(t, PI), 6.0);
            const double o1 = __ddiv_rn(__dmul_rn(2.0, PI), 3.0), o2 = __ddiv_rn(__dmul_rn(4.0, PI), 3.0);
            r = scale255(__dmul_rn(I, __dadd_rn(0.5, __dmul_rn(0.5, lyap_sin(ph)))));
            g = scale255(__dmul_rn(I, __dadd_rn(0.5, __dmul_rn(0.5, lyap_sin(__dadd_rn(ph, o1))))));
            b = scale255(__dmul_rn(I, __dadd_rn(0.5, __dmul_rn(0.5, lyap_sin(__dadd_rn(ph, o2))))));
        } break;
        case 6: {   // rainbow :267-278 with hslToRgb(hue, 1, 0.5) :26-47
            const double h = __ddiv_rn(__dmul_rn(t, 360.0), 360.0);
            const double q = 1.0, p = 0.0;
            const double cr = hue2rgb(p, q, __dadd_rn(h, 1.0 / 3));
            const double cg = hue2rgb(p, q, h);
            const double cb = hue2rgb(p, q, __dsub_rn(h, 1.0 / 3));
            r = scale255(__dmul_rn(I, cr));
            g = scale255(__dmul_rn(I, cg));
            b = scale255(__dmul_rn(I, cb));
        } break;
    }
    return clamp_u8(r) | (clamp_u8(g) << 8) | (clamp_u8(b) << 16) | 0xFF000000u;
}

constexpr int kColorThreads = 256;

__global__ void __launch_bounds__(kColorThreads)
k_colorize(const double* __restrict__ norm, int width, long long rows, int rows_above, int rows_below, int palette,
           unsigned int* __restrict__ rgba) {
    __shared__ lyap_logtab_entry tab[LYAP_LOG_BINS];
    if (palette == 1) {
        for (int e = threadIdx.x; e < LYAP_LOG_BINS; e += kColorThreads) tab[e] = g_lyap_logtab[e];
        __syncthreads();
    }
    const long long n = rows * (long long)width;
    const long long nthreads = (long long)gridDim.x * kColorThreads;
    for (long long idx = (long long)blockIdx.x * kColorThreads + threadIdx.x; idx < n; idx += nthreads) {
        const long long y = idx / width;
        const int x = (int)(idx - y * width);
        double sum = norm[idx];                       // :292
        int count = 1;
#pragma unroll
        for (int dy = -1; dy <= 1; ++dy) {
            const long long ny = y + dy;
            const bool row_ok = (ny >= 0 || rows_above) && (ny < rows || rows_below);
#pragma unroll
            for (int dx = -1; dx <= 1; ++dx) {
                if (dx == 0 && dy == 0) continue;
                const int nx = x + dx;
                if (row_ok && nx >= 0 && nx < width) {       // :301
                    sum = __dadd_rn(sum, norm[ny * width + nx]);
                    ++count;
                }
            }
        }
        const double t = __ddiv_rn(sum, (double)count);      // :307
        rgba[idx] = palette_rgba(t, palette, tab);
    }
}

cudaError_t launch_colorize(const double* norm, int width, long long rows, int rows_above, int rows_below,
                            int palette, unsigned char* rgba, cudaStream_t st) {
    const long long n = rows * (long long)width;
    if (n <= 0) return cudaSuccess;
    long long want = (n + kColorThreads - 1) / kColorThreads;
    const long long cap = 148LL * 64;
    const int grid = (int)(want < cap ? want : cap);
    k_colorize<<<grid, kColorThreads, 0, st>>>(norm, width, rows, rows_above, rows_below, palette,
                                                reinterpret_cast<unsigned int*>(rgba));
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Pipe issue-rate micro-benchmarks: 8 independent FMA chains per thread, nothing else in the loop.
// ---------------------------------------------------------------------------------------------
constexpr int kPeakThreads = 512;
constexpr int kPeakChains = 8;
constexpr int kPeakInner = 64;

__global__ void __launch_bounds__(kPeakThreads) k_fp64_peak(double* sink, int iters) {
    double acc[kPeakChains];
#pragma unroll
    for (int c = 0; c < kPeakChains; ++c) acc[c] = 1.0 + 1e-9 * (threadIdx.x + c);
    const double m = 0.999999, k = 1e-7;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int u = 0; u < kPeakInner; ++u) {
#pragma unroll
            for (int c = 0; c < kPeakChains; ++c) acc[c] = __fma_rn(acc[c], m, k);
        }
    }
    double s = 0;
#pragma unroll
    for (int c = 0; c < kPeakChains; ++c) s += acc[c];
    if (s == 12345.678) sink[0] = s;
}

__global__ void __launch_bounds__(kPeakThreads) k_fp32_peak(float* sink, int iters) {
    float acc[kPeakChains];
#pragma unroll
    for (int c = 0; c < kPeakChains; ++c) acc[c] = 1.0f + 1e-6f * (threadIdx.x + c);
    const float m = 0.9999f, k = 1e-5f;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int u = 0; u < kPeakInner; ++u) {
#pragma unroll
            for (int c = 0; c < kPeakChains; ++c) acc[c] = __fmaf_rn(acc[c], m, k);
        }
    }
    float s = 0;
#pragma unroll
    for (int c = 0; c < kPeakChains; ++c) s += acc[c];
    if (s == 12345.678f) sink[0] = s;
}

cudaError_t launch_fp64_peak(double* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st) {
    const int grid = sm_count * 2;
    k_fp64_peak<<<grid, kPeakThreads, 0, st>>>(sink, iters);
    *instr = (unsigned long long)grid * kPeakThreads * kPeakChains * kPeakInner * (unsigned long long)iters;
    return cudaGetLastError();
}

cudaError_t launch_fp32_peak(float* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st) {
    const int grid = sm_count * 4;
    k_fp32_peak<<<grid, kPeakThreads, 0, st>>>(sink, iters);
    *instr = (unsigned long long)grid * kPeakThreads * kPeakChains * kPeakInner * (unsigned long long)iters;
    return cudaGetLastError();
}

}  // namespace lyap

#include "lyap_kernels_fast.cuh"
