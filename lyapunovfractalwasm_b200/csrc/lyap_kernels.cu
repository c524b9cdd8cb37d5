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

#include "lyap_exact_kernel.cuh"
#include "lyap_kernels_fast.cuh"

namespace lyap {

template <int P, int THREADS, bool HAS_C, int UNROLL>
static cudaError_t launch_exact_variant(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                        int sm_count, cudaStream_t st) {
    auto kern = k_lambda_exact<P, THREADS, HAS_C, UNROLL>;
    constexpr size_t smem = exact_smem_bytes(THREADS, P);
    // the attribute is per device and cheap to set; doing it on every launch keeps this thread- and device-safe
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const long long tile_px = (long long)THREADS * P;     // one round of a block's warps (work is dealt out per warp)
    const long long tiles = (a.n_pixels + tile_px - 1) / tile_px;
    if (tiles <= 0) return cudaSuccess;
    const int grid = (int)(tiles < sm_count ? tiles : sm_count);
    kern<<<grid, THREADS, smem, st>>>(a, out64, out32, steps);
    static const char* const names[2] = {"k_lambda_exact<2,512> (generic: patterns dispatched every 2 steps)",
                                         "k_lambda_exact<3,512> (generic: patterns dispatched every 2 steps)"};
    note_lambda_kernel(names[P - 2]);
    return cudaGetLastError();
}

// Pixels per thread for a launch of n pixels.  Large frames: 3 (measured best on B200).  A frame of only a few rounds of
// warp-tiles is dominated by its last, partly filled round, in which the few warps still working run faster than in a
// full round but not in proportion (one warp alone reaches under half of its scheduler's fp64 rate); the shape with the
// smaller estimate of (full rounds + last round) x per-pixel cost is taken.  `spec`: the shapes run as instances made for
// the sequence, which are faster.
static int exact_pixels_per_thread(long long n_pixels, int sm_count, bool spec) {
    const int cand[2] = {3, 2};
    const double cost[2] = {spec ? 0.92 : 1.0, spec ? 0.95 : 1.035};
    const double warps = (double)sm_count * 16.0;
    int best = 3;
    double best_t = 1e300;
    for (int i = 0; i < 2; ++i) {
        const double tiles = (double)((n_pixels + 32LL * cand[i] - 1) / (32LL * cand[i]));
        const double rounds = tiles / warps;
        const double full = (double)(long long)rounds, frac = rounds - full;
        const double last = frac <= 0.0 ? 0.0 : (frac < 0.45 ? 0.45 : frac);
        const double t = (full + last) * cand[i] * cost[i];
        if (t < best_t * 0.999) {
            best_t = t;
            best = cand[i];
        }
    }
    return best;
}

// LYAP_JIT: 0 never compile at run time, 1 (default) once enough work with a sequence has been seen, 2 at once.
// LYAP_PREBUILT=0: ignore the instances compiled at build time (with LYAP_JIT=0 that forces the generic kernels).
static int spec_mode() {
    const char* je = getenv("LYAP_JIT");
    const char* pe = getenv("LYAP_PREBUILT");
    const int jit = je ? atoi(je) : 1;
    const int pre = pe ? atoi(pe) : 1;
    return (jit < 0 ? 0 : (jit > 2 ? 2 : jit)) | (pre ? kSpecUsePrebuilt : 0);
}

cudaError_t launch_lambda_exact(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                int sm_count, cudaStream_t st) {
    bool has_c = false;
    const int words = a.acc_word0 + (a.iterations > 0 ? min(a.acc_wrap, (a.iterations - 1) / kStepsPerWord + 1) : 0);
    for (int i = 0; i < words; ++i) has_c = has_c || (a.sel[i] & 0xAAAAAAAAu);
#define LYAP_VARIANT(P, T, U)                                                                    \
    (has_c ? launch_exact_variant<P, T, true, U>(a, out64, out32, steps, sm_count, st)            \
           : launch_exact_variant<P, T, false, U>(a, out64, out32, steps, sm_count, st))
    // a periodic sequence can run an instance of this kernel made for its patterns
    const int mode = spec_mode();
    unsigned long long wu_pats = 0, acc_pats = 0;
    const bool spec = mode != 0 && sequence_group_period(a, &wu_pats, &acc_pats) > 0;
    const int ppt = exact_pixels_per_thread(a.n_pixels, sm_count, spec);
    {
        bool launched = false;
        const cudaError_t e = launch_lambda_spec(a, out64, out32, steps, sm_count, st, 0, ppt, 512, exact_smem_bytes(512, ppt),
                                                 mode, &launched);
        if (e != cudaSuccess) return e;
        if (launched) return cudaSuccess;
    }
    if (ppt == 2) return LYAP_VARIANT(2, 512, 2);
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

cudaError_t launch_minmax(const double* v, unsigned long long n, double* minmax, void* scratch, int sm_count, cudaStream_t st) {
    double* partial = static_cast<double*>(scratch);
    unsigned int* ticket = reinterpret_cast<unsigned int*>(partial + 2 * kMinmaxBlocks);
    unsigned long long want = (n / 2 + kMinmaxThreads - 1) / kMinmaxThreads;
    if (want < 1) want = 1;
    // 8 blocks per SM of this device, never more than the scratch has room for
    const unsigned long long cap = (unsigned long long)(8 * sm_count < kMinmaxBlocks && sm_count > 0 ? 8 * sm_count : kMinmaxBlocks);
    const int grid = (int)(want < cap ? want : cap);
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
    constexpr int kMaxDevices = LYAP_NOALLOC_MAX_DEVICES;
    static std::mutex mu;
    static void* scratch_of_device[kMaxDevices] = {};
    static int sm_count_of_device[kMaxDevices] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices)
        return set_error(LYAP_ERR_INVALID, "lyap_minmax_device_noalloc: device ordinal beyond LYAP_NOALLOC_MAX_DEVICES");
    void* scratch = nullptr;
    int sm_count = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!scratch_of_device[dev]) {   // one-time set-up for this device (it is the current one)
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_minmax_fixed_scratch);
            if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
            sm_count_of_device[dev] = sms;
            scratch_of_device[dev] = p;
        }
        scratch = scratch_of_device[dev];
        sm_count = sm_count_of_device[dev];
    }
    cudaStream_t st = static_cast<cudaStream_t>(cuda_stream);
    // the arrival ticket must start at zero; the array keeps whatever the last call (or an aborted one) left
    unsigned int* ticket = reinterpret_cast<unsigned int*>(static_cast<double*>(scratch) + 2 * kMinmaxBlocks);
    e = cudaMemsetAsync(ticket, 0, 16, st);
    if (e != cudaSuccess) return set_error(LYAP_ERR_CUDA, cudaGetErrorString(e));
    e = launch_minmax(d_values, n, d_minmax, scratch, sm_count, st);
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

// one pixel: 3x3 mean in the page's summation order, then the palette
__device__ __forceinline__ unsigned int colorize_one(const double* __restrict__ norm, long long idx, int width, long long rows,
                                                     int rows_above, int rows_below, int palette, const lyap_logtab_entry* tab) {
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
    return palette_rgba(t, palette, tab);
}

// Four consecutive pixels per thread, written as one 16-byte store (a warp writes 512 consecutive bytes); the last few
// pixels of a frame whose size is not a multiple of four, and a misaligned output, take 4-byte stores.
__global__ void __launch_bounds__(kColorThreads)
k_colorize(const double* __restrict__ norm, int width, long long rows, int rows_above, int rows_below, int palette,
           unsigned int* __restrict__ rgba) {
    __shared__ lyap_logtab_entry tab[LYAP_LOG_BINS];
    if (palette == 1) {
        for (int e = threadIdx.x; e < LYAP_LOG_BINS; e += kColorThreads) tab[e] = g_lyap_logtab[e];
        __syncthreads();
    }
    const long long n = rows * (long long)width;
    const long long nquads = (n + 3) / 4;
    const long long nthreads = (long long)gridDim.x * kColorThreads;
    const bool aligned = (reinterpret_cast<uintptr_t>(rgba) & 15) == 0;
    for (long long q = (long long)blockIdx.x * kColorThreads + threadIdx.x; q < nquads; q += nthreads) {
        const long long idx0 = 4 * q;
        if (aligned && idx0 + 4 <= n) {
            uint4 px;
            px.x = colorize_one(norm, idx0, width, rows, rows_above, rows_below, palette, tab);
            px.y = colorize_one(norm, idx0 + 1, width, rows, rows_above, rows_below, palette, tab);
            px.z = colorize_one(norm, idx0 + 2, width, rows, rows_above, rows_below, palette, tab);
            px.w = colorize_one(norm, idx0 + 3, width, rows, rows_above, rows_below, palette, tab);
            *reinterpret_cast<uint4*>(rgba + idx0) = px;
        } else {
            for (long long idx = idx0; idx < n && idx < idx0 + 4; ++idx)
                rgba[idx] = colorize_one(norm, idx, width, rows, rows_above, rows_below, palette, tab);
        }
    }
}

cudaError_t launch_colorize(const double* norm, int width, long long rows, int rows_above, int rows_below,
                            int palette, unsigned char* rgba, int sm_count, cudaStream_t st) {
    const long long n = rows * (long long)width;
    if (n <= 0) return cudaSuccess;
    long long want = ((n + 3) / 4 + kColorThreads - 1) / kColorThreads;
    const long long cap = (long long)sm_count * 64;
    const int grid = (int)(want < cap ? want : cap);
    k_colorize<<<grid, kColorThreads, 0, st>>>(norm, width, rows, rows_above, rows_below, palette,
                                                reinterpret_cast<unsigned int*>(rgba));
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------------
// Glow (web/fractal_renderer.js:313-334): the canvas drawn onto itself three times with 'screen' compositing,
// blur(6px) at alpha 0.3, blur(2px) at alpha 0.4, unfiltered at alpha 0.1.  The browser's compositor defines
// the exact arithmetic in the reference; these kernels implement this project's reading of the Canvas / CSS
// rules (stated in full beside oracle_glow in the CPU checker): Gaussian truncated at ceil(3 sigma),
// transparent black outside, opaque backdrop, out = Cb + alpha * Sp * (1 - Cb), 8-bit rounding per draw.
// ---------------------------------------------------------------------------------------------
constexpr int kGlowMaxRadius = 18;
struct GlowArgs {
    double w[2 * kGlowMaxRadius + 1];
    double alpha;
    int radius;   // 0: no filter
};
constexpr int kGlowThreads = 256;

__global__ void __launch_bounds__(kGlowThreads)
k_glow_blur_rows(const __grid_constant__ GlowArgs g, const unsigned char* __restrict__ canvas, int width, long long n,
                 double* __restrict__ tmp) {
    __shared__ double unit[256];
    unit[threadIdx.x] = __ddiv_rn((double)threadIdx.x, 255.0);
    __syncthreads();
    const long long nthreads = (long long)gridDim.x * kGlowThreads;
    for (long long i = (long long)blockIdx.x * kGlowThreads + threadIdx.x; i < n; i += nthreads) {
        const int x = (int)(i % width);
        double s0 = 0.0, s1 = 0.0, s2 = 0.0;
        for (int k = -g.radius; k <= g.radius; ++k) {
            const int xx = x + k;
            if (xx >= 0 && xx < width) {
                const uchar4 c = *reinterpret_cast<const uchar4*>(canvas + (i + k) * 4);
                const double wk = g.w[k + g.radius];
                s0 = __dadd_rn(s0, __dmul_rn(wk, unit[c.x]));
                s1 = __dadd_rn(s1, __dmul_rn(wk, unit[c.y]));
                s2 = __dadd_rn(s2, __dmul_rn(wk, unit[c.z]));
            }
        }
        tmp[i * 3] = s0;
        tmp[i * 3 + 1] = s1;
        tmp[i * 3 + 2] = s2;
    }
}

__device__ __forceinline__ unsigned char glow_mix(double cb, double sp, double alpha) {
    const double out = __dadd_rn(cb, __dmul_rn(__dmul_rn(alpha, sp), __dsub_rn(1.0, cb)));
    const double q = floor(__dadd_rn(__dmul_rn(out, 255.0), 0.5));
    return (unsigned char)(q < 0.0 ? 0.0 : (q > 255.0 ? 255.0 : q));
}

__global__ void __launch_bounds__(kGlowThreads)
k_glow_blur_cols_mix(const __grid_constant__ GlowArgs g, unsigned char* __restrict__ canvas, int width, int height,
                     long long n, const double* __restrict__ tmp) {
    __shared__ double unit[256];
    unit[threadIdx.x] = __ddiv_rn((double)threadIdx.x, 255.0);
    __syncthreads();
    const long long nthreads = (long long)gridDim.x * kGlowThreads;
    for (long long i = (long long)blockIdx.x * kGlowThreads + threadIdx.x; i < n; i += nthreads) {
        const uchar4 cb = *reinterpret_cast<const uchar4*>(canvas + i * 4);
        double s0, s1, s2;
        if (g.radius > 0) {
            const int y = (int)(i / width);
            s0 = s1 = s2 = 0.0;
            for (int k = -g.radius; k <= g.radius; ++k) {
                const int yy = y + k;
                if (yy >= 0 && yy < height) {
                    const double* t = tmp + (i + (long long)k * width) * 3;
                    const double wk = g.w[k + g.radius];
                    s0 = __dadd_rn(s0, __dmul_rn(wk, t[0]));
                    s1 = __dadd_rn(s1, __dmul_rn(wk, t[1]));
                    s2 = __dadd_rn(s2, __dmul_rn(wk, t[2]));
                }
            }
        } else {
            s0 = unit[cb.x];
            s1 = unit[cb.y];
            s2 = unit[cb.z];
        }
        uchar4 o;
        o.x = glow_mix(unit[cb.x], s0, g.alpha);
        o.y = glow_mix(unit[cb.y], s1, g.alpha);
        o.z = glow_mix(unit[cb.z], s2, g.alpha);
        o.w = cb.w;
        *reinterpret_cast<uchar4*>(canvas + i * 4) = o;
    }
}

cudaError_t launch_glow(unsigned char* canvas, int width, int height, double* scratch, int sm_count, cudaStream_t st) {
    const long long n = (long long)width * height;
    if (n <= 0) return cudaSuccess;
    const long long want = (n + kGlowThreads - 1) / kGlowThreads;
    const long long cap = (long long)sm_count * 32;
    const int grid = (int)(want < cap ? want : cap);
    const double sigmas[3] = {6.0, 2.0, 0.0}, alphas[3] = {0.3, 0.4, 0.1};
    for (int pass = 0; pass < 3; ++pass) {
        GlowArgs g{};
        g.alpha = alphas[pass];
        g.radius = (int)ceil(3.0 * sigmas[pass]);
        if (g.radius > 0) {
            double sum = 0.0;
            for (int k = -g.radius; k <= g.radius; ++k) {
                g.w[k + g.radius] = lyap_exp(-(double)(k * k) / (2.0 * sigmas[pass] * sigmas[pass]));
                sum += g.w[k + g.radius];
            }
            for (int k = 0; k <= 2 * g.radius; ++k) g.w[k] /= sum;
            k_glow_blur_rows<<<grid, kGlowThreads, 0, st>>>(g, canvas, width, n, scratch);
            if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
        }
        k_glow_blur_cols_mix<<<grid, kGlowThreads, 0, st>>>(g, canvas, width, height, n, scratch);
        if (cudaError_t e = cudaGetLastError(); e != cudaSuccess) return e;
    }
    return cudaSuccess;
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

namespace lyap {

template <typename FL, int P>
static cudaError_t launch_lambda_fast_t(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                        int sm_count, cudaStream_t st, int kind, int spec_ppt, const char* generic_name) {
    {   // a periodic sequence can run an instance made for its patterns (same switches as the exact kernel)
        bool launched = false;
        const cudaError_t e = launch_lambda_spec(a, out64, out32, steps, sm_count, st, kind, spec_ppt, 512, 0, spec_mode(), &launched);
        if (e != cudaSuccess) return e;
        if (launched) return cudaSuccess;
    }
    const long long tile_px = (long long)kFastThreads * P;
    const long long tiles = (a.n_pixels + tile_px - 1) / tile_px;
    if (tiles <= 0) return cudaSuccess;
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_lambda_fast<FL, P, kFastThreads>,
                                                                  kFastThreads, 0);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) per_sm = 1;
    const long long cap = (long long)sm_count * per_sm;
    const int grid = (int)(tiles < cap ? tiles : cap);
    k_lambda_fast<FL, P, kFastThreads><<<grid, kFastThreads, 0, st>>>(a, out64, out32, steps);
    note_lambda_kernel(generic_name);
    return cudaGetLastError();
}

// measured best shapes for the instances made for a sequence: fused fp64 4 pixels/thread, fp32 2, same-orbit fp64 3; 512 threads
cudaError_t launch_lambda_fast64(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st) {
    return launch_lambda_fast_t<FusedF64, 4>(a, out64, out32, steps, sm_count, st, 1, 4, "k_lambda_fast<FusedF64,4,256> (generic)");
}

cudaError_t launch_lambda_fast32(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st) {
    return launch_lambda_fast_t<FusedF32, 4>(a, out64, out32, steps, sm_count, st, 2, 2, "k_lambda_fast<FusedF32,4,256> (generic)");
}

cudaError_t launch_lambda_orbit64(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                  int sm_count, cudaStream_t st) {
    return launch_lambda_fast_t<OrbitF64, 4>(a, out64, out32, steps, sm_count, st, 3, 3, "k_lambda_fast<OrbitF64,4,256> (generic)");
}

}  // namespace lyap
