/* lyap_b200.h -- C ABI of the B200 (sm_100a) Lyapunov-fractal engine.
 *
 * One shared library, liblyap_b200.so, plain C types only.  It replaces the compute path of the
 * reference project (emeraldant/LyapunovFractalWASM); every entry point names the reference
 * interface it stands in for (paths relative to the reference project).  There is no CPU
 * fallback: without a CUDA device every compute entry point returns LYAP_ERR_CUDA.
 *
 * Conventions
 *   - every function returns an int status (LYAP_OK == 0); no exception crosses this boundary;
 *     lyap_last_error() gives the message of the calling thread's last failure.
 *   - "_device" entry points take DEVICE pointers and only enqueue work on the context's stream;
 *     the others take HOST pointers, copy, and return when the result is in the host buffer.
 *   - frames are row-major, row 0 = min_y, column 0 = min_x, like the reference
 *     (src/lyapunov_fractal.hpp:42,45,84).  Pixel counts are 64-bit here.
 */
#ifndef LYAP_B200_H
#define LYAP_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LYAP_ABI_VERSION 2

enum lyap_status {
    LYAP_OK = 0,
    LYAP_ERR_INVALID = 1,      /* bad dimension, null pointer, bad row range, unknown mode/palette */
    LYAP_ERR_SEQUENCE = 2,     /* empty sequence (the reference divides by zero there, :34,37) */
    LYAP_ERR_TOO_LARGE = 3,    /* step count or size beyond what an entry point supports */
    LYAP_ERR_CUDA = 4,         /* CUDA runtime failure, or no device */
    LYAP_ERR_NOMEM = 5,
    LYAP_ERR_TIMEOUT = 6,      /* a host-side deadline expired (multi-device orchestration) */
    LYAP_ERR_COMM = 7          /* gather / peer-copy failure */
};

enum lyap_mode {
    LYAP_MODE_EXACT = 0,       /* fp64, reference operation order, one log per step: bit-exact */
    LYAP_MODE_FAST_FP64 = 1,   /* fp64 FMA orbit, running product of derivatives, one log per pixel */
    LYAP_MODE_FAST_FP32 = 2,   /* fp32 orbit and products, integer exponent sum, one log per pixel */
    LYAP_MODE_FAST_FP64_ORBIT = 3  /* the reference's own operations for the orbit and for 1 - 2x (so x, the exits and
                                      the sentinels are the exact mode's), but the factors |1 - 2x| multiplied into a
                                      running product with one log per pixel, and the factors r added as n_A log r_A +
                                      n_B log r_B (+ n_C log c): lambda differs from the exact mode's only by the
                                      rounding of that accumulation (below 1e-12) */
};
/* The fast modes accept at most 2^24 steps per pixel (warmup + iterations): LYAP_ERR_TOO_LARGE beyond. */

enum lyap_palette {            /* web/fractal_renderer.js:207-281; unknown names mean cosmic (:280) */
    LYAP_PALETTE_COSMIC = 0,
    LYAP_PALETTE_NEBULA = 1,
    LYAP_PALETTE_AURORA = 2,
    LYAP_PALETTE_SOLARFLARE = 3,
    LYAP_PALETTE_BLACKHOLE = 4,
    LYAP_PALETTE_PSYCHEDELIC = 5,
    LYAP_PALETTE_RAINBOW = 6
};

/* Mirrors lyapunov::FractalComputer::ComputationParams field for field
 * (src/lyapunov_fractal.hpp:15-25), then an extension block.  lyap_params_default() fills the
 * reference's defaults (0..4 x 0..4, 800x600, "ABABABAB", 10000 iterations, 100 warm-up). */
typedef struct lyap_params {
    double min_x, max_x, min_y, max_y;  /* parameter window: columns -> A, rows -> B */
    int32_t width, height;
    const char* sequence;               /* any byte other than 'A' selects B (:37) ... */
    int32_t sequence_len;
    int32_t iterations, warmup;
    /* ---- extension block (all zero = reference behaviour) ---- */
    int32_t mode;                       /* enum lyap_mode */
    int32_t palette;                    /* enum lyap_palette */
    int32_t c_enabled;                  /* ... unless c_enabled: then 'C' selects c_value */
    int32_t reserved0;
    double c_value;
    int64_t row_begin, row_end;         /* rows [row_begin,row_end) of the frame; both 0 = all rows.
                                           r_y always uses the global row index and global dy, so a
                                           band has the bits the whole frame would have. */
} lyap_params;

typedef struct lyap_ctx lyap_ctx;      /* one device, one stream, scratch buffers */

/* Progress callback, same shape as the reference's void(*)(double) (src/lyapunov_fractal.hpp:27).
 * Called on the calling host thread, in increasing order, after each finished row chunk with
 * rows_done/height, and once with 1.0 at the end (reference: every 10th row from worker threads
 * in any order, then 1.0; :88-90,97-99). */
typedef void (*lyap_progress_fn)(double fraction);

typedef struct lyap_render_stats {
    uint64_t executed_steps;           /* logistic updates actually performed (early exits excluded) */
    uint64_t nominal_steps;            /* pixels * (warmup + iterations) */
    double lambda_min, lambda_max;     /* over finite values > -4 (normalizeData's filter) */
    float ms_lambda, ms_minmax, ms_normalize, ms_colorize, ms_total_device, ms_copies;
    int32_t kernel_launches;
    int32_t reserved;
} lyap_render_stats;

/* ---- library ---- */
int lyap_abi_version(void);
/* Stand-in for testFunction() (src/wasm_bindings.cpp:19-22): returns 42. */
int lyap_self_test(void);
const char* lyap_last_error(void);
const char* lyap_status_string(int status);
void lyap_params_default(lyap_params* p);
/* palette id for a name as used by the page's <select> (web/index.html:115-123); unknown -> cosmic */
int lyap_palette_from_name(const char* name);
int lyap_device_count(int* count);

/* ---- context ---- */
int lyap_create(lyap_ctx** ctx, int device);
int lyap_destroy(lyap_ctx* ctx);
/* Use a caller-owned cudaStream_t (passed as void*) for all work of this context; NULL = own stream. */
int lyap_set_stream(lyap_ctx* ctx, void* cuda_stream);
int lyap_sync(lyap_ctx* ctx);
int lyap_device_alloc(lyap_ctx* ctx, void** dptr, size_t bytes);
int lyap_device_free(lyap_ctx* ctx, void* dptr);
int lyap_host_alloc(void** hptr, size_t bytes);     /* pinned */
int lyap_host_free(void* hptr);
int lyap_copy_to_host(lyap_ctx* ctx, void* host, const void* dev, size_t bytes);   /* waits */
int lyap_copy_to_device(lyap_ctx* ctx, void* dev, const void* host, size_t bytes); /* waits */

/* ---- device-pointer entry points (enqueue only) ---- */

/* FractalComputer::computeFractal (src/lyapunov_fractal.hpp:27-102) for rows [row_begin,row_end).
 * d_lambda: rows*width doubles, or NULL; d_lambda32: same count of floats ((float)lambda), or NULL.
 * d_steps: one uint64 the kernel ADDS executed steps to, or NULL. */
int lyap_lambda_device(lyap_ctx* ctx, const lyap_params* p, double* d_lambda, float* d_lambda32,
                       uint64_t* d_steps);

/* normalizeData pass 1 (src/lyapunov_fractal.hpp:110-120): d_minmax[0]=min, [1]=max over finite
 * values > -4; starts from +DBL_MAX / -DBL_MAX like the reference. */
int lyap_minmax_device(lyap_ctx* ctx, const double* d_values, uint64_t n, double* d_minmax);

/* normalizeData pass 2 (src/lyapunov_fractal.hpp:122-137) with min/max read from device memory
 * (for a band: the whole frame's min/max).  min >= max gives all zeros (:122). */
int lyap_normalize_device(lyap_ctx* ctx, const double* d_values, uint64_t n, const double* d_minmax,
                          double* d_out);

/* applyPostProcessing + palette + ImageData store (web/fractal_renderer.js:283-311,207-281,191-198).
 * d_norm points at the first of `rows` rows of `width` normalised values; rows_above / rows_below
 * (0 or 1) say whether the row before / after that block exists in memory (a band's neighbour rows);
 * where they do not, the image edge rule applies.  d_rgba: rows*width*4 bytes, R,G,B,255. */
int lyap_colorize_device(lyap_ctx* ctx, const double* d_norm, int32_t width, int64_t rows,
                         int32_t rows_above, int32_t rows_below, int32_t palette, uint8_t* d_rgba);

/* applyGlow (web/fractal_renderer.js:313-334) on an RGBA8 frame in place: three self-draws with 'screen' compositing
 * (blur 6 px at alpha 0.3, blur 2 px at 0.4, unfiltered at 0.1).  The reference leaves the arithmetic to the
 * browser's compositor; this is the engine's own reading of the Canvas / CSS filter rules (Gaussian of the given
 * standard deviation truncated at 3 sigma, transparent outside the canvas, 8-bit rounding after each draw).
 * d_scratch: width*height*24 bytes of device memory. */
int lyap_glow_device(lyap_ctx* ctx, uint8_t* d_rgba, int32_t width, int32_t height, void* d_scratch);

/* ---- host-pointer entry points (blocking) ---- */

/* computeFractal (src/lyapunov_fractal.hpp:27): out_lambda holds rows*width doubles. */
int lyap_compute_fractal(lyap_ctx* ctx, const lyap_params* p, double* out_lambda, lyap_progress_fn progress);

/* normalizeData (src/lyapunov_fractal.hpp:105): n == 0 is allowed and does nothing (:106). */
int lyap_normalize_data(lyap_ctx* ctx, const double* values, uint64_t n, double* out);

/* renderFractal up to putImageData (web/fractal_renderer.js:177-200) for a whole frame. */
int lyap_colorize(lyap_ctx* ctx, const double* norm, int32_t width, int32_t height, int32_t palette,
                  uint8_t* out_rgba);

/* applyGlow for a frame in host memory (see lyap_glow_device); rgba_in and rgba_out may be the same buffer. */
int lyap_glow(lyap_ctx* ctx, const uint8_t* rgba_in, int32_t width, int32_t height, uint8_t* rgba_out);

/* The binding's whole call order (src/wasm_bindings.cpp:109-125: parse, computeFractal,
 * normalizeData) followed by the page's colour stage, on the whole frame.  Any output may be NULL.
 * out_norm is what the WASM export returns. */
int lyap_render(lyap_ctx* ctx, const lyap_params* p, double* out_lambda, float* out_lambda32, double* out_norm,
                uint8_t* out_rgba, lyap_progress_fn progress, lyap_render_stats* stats);

/* ---- several devices of this machine, from one process ---- */

/* A set of devices kept ready for frames split into row bands and for batches of whole frames: per device one
 * engine context, two streams, its buffers (grown on demand, kept between calls) and a pinned read-back record;
 * with use_nccl != 0 also one NCCL communicator per device (ncclCommInitAll; the NCCL library is looked up with
 * dlopen("libnccl.so.2"), path override: environment LYAP_NCCL_PATH).  The same ordinal may be listed more than
 * once and a negative ordinal stands for a band whose worker never arrives (the tests use it to exercise the
 * deadline without disturbing a GPU); in both cases, and when the library is missing or its set-up fails, the object
 * works without NCCL (min/max through the host, gather by peer copies) and lyap_multi_note() says why.
 * One call at a time per object. */
typedef struct lyap_multi lyap_multi;
int lyap_multi_create(lyap_multi** m, int32_t n_devices, const int32_t* devices, int32_t use_nccl);
int lyap_multi_destroy(lyap_multi* m);
/* "" while NCCL is in use (or was not asked for), otherwise the reason it is not. */
const char* lyap_multi_note(lyap_multi* m);

enum lyap_multi_flags {
    LYAP_MULTI_GATHER_RGBA = 1,      /* collect every band's RGBA8 in the first device's own frame buffer */
    LYAP_MULTI_GATHER_LAMBDA32 = 2,  /* likewise the (float)lambda bands */
    LYAP_MULTI_HOST_EXCHANGE = 4     /* this call without NCCL even where it is available: frame min/max through the
                                        host, a gather by peer copies (cudaMemcpyPeerAsync) */
};

typedef struct lyap_multi_stats {
    uint64_t executed_steps, nominal_steps;
    double lambda_min, lambda_max;
    float ms_wall;                 /* the whole call, host clock */
    float ms_lambda_max;           /* slowest band: its lambda kernels (CUDA events on its stream) */
    float ms_device_max;           /* slowest band: lambda ... RGBA */
    float ms_gather;               /* first device: gather posted ... last byte in its frame buffer (CUDA events) */
    uint64_t gather_bytes;         /* bytes that came from the other devices */
    int32_t kernel_launches;       /* this library's kernels, all devices */
    int32_t used_nccl;             /* 1: all-reduce / send / recv went through NCCL; 0: host exchange, peer copies */
} lyap_multi_stats;

/* One frame as contiguous row bands, one per listed device (the reference's rows loop, src/lyapunov_fractal.hpp:41,
 * and its result vector, :28,84,101).  Each band recomputes one halo row per inner side for the page's 3x3 mean; the
 * one exchange is the frame's min/max (normalizeData, :110-125): a single all-reduce(MIN) of (min, -max).
 * Host outputs (any may be NULL) receive every band in its place, so the bytes equal lyap_render's on one device.
 * With a GATHER flag the bands are first sent to the first listed device -- ncclSend on each other device, the
 * matching ncclRecvs posted as one group on the first; peer copies without NCCL -- into ONE contiguous frame in that
 * device's memory (lyap_multi_gathered), and out_rgba / out_lambda32, if given, are copied from there.  The gather is
 * posted only after every band has finished, and is timed on its own (stats->ms_gather).
 * Failure handling: every step that needs all bands is preceded by a host-side rendezvous with the deadline
 * (timeout_seconds; it covers the kernels too; <= 0: 60 s plus the frame's steps / (1e11 per device)), so a band that
 * fails or never arrives gives its error / LYAP_ERR_TIMEOUT before
 * any collective is enqueued; afterwards completion is polled (stream state, ncclCommGetAsyncError) against the same
 * deadline, and on expiry or an NCCL error the communicators are aborted: LYAP_ERR_TIMEOUT / LYAP_ERR_COMM. */
int lyap_multi_render(lyap_multi* m, const lyap_params* p, int32_t flags, double* out_lambda, float* out_lambda32,
                      double* out_norm, uint8_t* out_rgba, double timeout_seconds, lyap_multi_stats* stats);

/* Device pointers (first listed device) of the frames the last GATHER render filled; valid until the next render that
 * needs a larger one, or lyap_multi_destroy.  NULL for a kind never gathered. */
int lyap_multi_gathered(lyap_multi* m, uint8_t** d_rgba, float** d_lambda32);

/* A batch of independent whole frames -- a zoom sequence: each frame its own window, hence its own min/max
 * (the page calls computeLyapunovFractal once per view, web/fractal_renderer.js:132-154) -- dealt round-robin to
 * the object's devices: frame k goes to device k % n.  On each device the kernels of successive frames run back to
 * back on one stream while the previous frame's outputs are copied to the host on a second stream from a second set
 * of buffers, so copies cost no device time as long as they are shorter than a frame.  out_norm / out_rgba are arrays
 * of n_frames host pointers (either array, or single entries, may be NULL; pinned memory from lyap_host_alloc copies
 * fastest); stats, if given, is an array of n_frames records (ms_copies = time from the frame's last kernel to its
 * last byte on the host).  Every frame's bytes equal those of lyap_render on that frame. */
int lyap_multi_render_frames(lyap_multi* m, const lyap_params* frames, int32_t n_frames, double* const* out_norm,
                             uint8_t* const* out_rgba, lyap_render_stats* stats);

/* One-call forms: a temporary lyap_multi (without NCCL) around one lyap_multi_render (host min/max exchange, no
 * gather) / lyap_multi_render_frames.  They pay for contexts and buffers on every call; keep a lyap_multi for
 * repeated use.  stats->ms_total_device of lyap_render_multi is the wall-clock time of the render inside. */
int lyap_render_multi(const lyap_params* p, int32_t n_devices, const int32_t* devices, double* out_lambda,
                      double* out_norm, uint8_t* out_rgba, double timeout_seconds, lyap_render_stats* stats);
int lyap_render_frames(const lyap_params* frames, int32_t n_frames, int32_t n_devices, const int32_t* devices,
                       double* const* out_norm, uint8_t* const* out_rgba, lyap_render_stats* stats);

/* ---- for callers that must not allocate ---- */

/* No counterpart in the reference.  Same result as lyap_minmax_device, for hosts that are not allowed to
 * allocate device memory at the time of the call: a renderer that fixed its memory budget at start-up, code
 * running between frames of a real-time loop where an allocation may stall the whole device, or a plug-in whose
 * host forbids driver allocations after initialisation.  It needs no lyap_ctx (creating one allocates): it runs on
 * the CURRENT device, on the given cudaStream_t (NULL = default stream), and its reduction scratch is a fixed
 * array inside the library image (about 19 KB, resident on every GPU that loads the library until exit).
 * It calls no cudaMalloc / cudaFree and no allocating routine.
 *   - n may be at most LYAP_NOALLOC_MAX_VALUES; larger sizes return LYAP_ERR_TOO_LARGE.
 *   - The first call on each device looks up the array's device address (one-time set-up); make that first call
 *     outside any stream capture.
 *   - All calls on a device share the one array: calls that may overlap on the GPU (different streams,
 *     different threads) race and give wrong results; order them on one stream or with events.
 *   - d_values / d_minmax are device pointers supplied by the caller; only enqueues work.
 *   - The looked-up addresses are kept in a fixed table of LYAP_NOALLOC_MAX_DEVICES entries (no host allocation
 *     either): on a device whose ordinal is that or larger the call returns LYAP_ERR_INVALID. */
#define LYAP_NOALLOC_MAX_VALUES (1ull << 32)
#define LYAP_NOALLOC_MAX_DEVICES 64
int lyap_minmax_device_noalloc(const double* d_values, uint64_t n, double* d_minmax, void* cuda_stream);

/* No counterpart in the reference.  For a periodic sequence the lambda kernels run as an instance made for that
 * sequence's A/B(/C) patterns (same source, same bits, no per-step choice left): one compiled with the library for
 * the patterns of "AB", "AABAB", "BBBBBBAAAAAA" (500 warm-up steps), "ABC" with a third parameter and "ABB", else one
 * compiled at run time (NVRTC) once about 2e10 steps of work with the sequence have been asked for.  Environment:
 * LYAP_JIT=0 never compiles at run time, 2 compiles on first use; LYAP_PREBUILT=0 ignores the library's own instances
 * (both 0: the generic kernels, which choose the pattern every two steps).
 * lyap_jit_note: why the last attempt to build or use a run-time instance fell back ("" if none did).
 * lyap_last_kernel: which lambda kernel the calling thread's last launch used, and how it was made. */
const char* lyap_jit_note(void);
const char* lyap_last_kernel(void);

/* No counterpart in the reference (host only, needs no GPU).  Writes to *code which parameter step `step` of the
 * warm-up (region 0) or of the accumulation (region 1) uses under `params` -- 0 = column parameter ('A'),
 * 1 = row parameter, 2 = c_value -- read back from the packed selector table the kernels are given, i.e. what
 * sequence[(region ? warmup + step : step) % len] selects (src/lyapunov_fractal.hpp:37).  A region too long to store
 * whole is stored as one period of the sequence in whole 16-step words and walked cyclically, so any warmup and
 * iterations are accepted while 2 * len / gcd(len, 16) <= 896; longer sequences are limited to 14336 steps. */
int lyap_selector_code(const lyap_params* params, int region, int64_t step, int* code);

/* No counterpart in the reference (host only, needs no GPU).  The key under which a launch with `params` looks for a
 * lambda-kernel instance made for its sequence: *groups = number of two-step groups after which the parameter choices
 * of both regions repeat (0: none up to 16, the generic kernel runs), and the 2-bit codes of one such period of the
 * warm-up and of the accumulation region (4 bits per group).  The build recipe computes the same key for the instances it
 * embeds; the CPU tests compare the two. */
int lyap_group_patterns(const lyap_params* params, int* groups, uint64_t* warmup_patterns, uint64_t* accumulation_patterns);

/* ---- measurement ---- */

/* Issue-rate micro-benchmark of the fp64 pipe on the context's device: independent DFMA chains,
 * all SMs.  Writes thread-level fp64 instructions per second. */
int lyap_fp64_peak(lyap_ctx* ctx, double* instr_per_second);
/* Same for the fp32 FMA pipe. */
int lyap_fp32_peak(lyap_ctx* ctx, double* instr_per_second);

#ifdef __cplusplus
}
#endif
#endif /* LYAP_B200_H */
