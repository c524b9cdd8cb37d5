// lyap_abi.cu -- implementation of the C ABI declared in include/lyap_b200.h.
//
// Host-side orchestration only: parameter checks, the sequence-to-selector packing
// (reference src/lyapunov_fractal.hpp:34-38), buffer management, launches, copies, timing.
// There is deliberately no CPU implementation behind these entry points.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <numeric>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>   // header-only: ranges cost nothing unless a profiler attaches

#include "../../include/lyap_b200.h"
#include "lyap_engine.h"

namespace {

thread_local std::string g_last_error;

int fail(int status, const std::string& msg) {
    g_last_error = msg;
    return status;
}

int fail_cuda(cudaError_t e, const char* what) {
    g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
    return LYAP_ERR_CUDA;
}

#define CU(call)                                              \
    do {                                                      \
        cudaError_t e_ = (call);                              \
        if (e_ != cudaSuccess) return fail_cuda(e_, #call);   \
    } while (0)

struct Buffer {
    void* p = nullptr;
    size_t cap = 0;
};

// NVTX range around the enqueueing of one stage (shows as a named span in a profiler's timeline)
struct Range {
    explicit Range(const char* name) { nvtxRangePushA(name); }
    ~Range() { nvtxRangePop(); }
};

}  // namespace

struct lyap_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t own_stream = nullptr;
    Buffer lambda, lambda32, norm, rgba;   // frame-sized work buffers of the host-pointer entry points
    void* small = nullptr;                 // [0,16) min/max, [16,24) step counter, then min/max scratch
    cudaEvent_t ev[8] = {};
    std::vector<cudaEvent_t> chunk_events;
};

namespace {

double* ctx_minmax(lyap_ctx* c) { return static_cast<double*>(c->small); }
unsigned long long* ctx_steps(lyap_ctx* c) {
    return reinterpret_cast<unsigned long long*>(static_cast<char*>(c->small) + 16);
}
void* ctx_scratch(lyap_ctx* c) { return static_cast<char*>(c->small) + 32; }

int ensure(lyap_ctx* c, Buffer& b, size_t bytes) {
    if (b.cap >= bytes) return LYAP_OK;
    if (b.p) {
        CU(cudaStreamSynchronize(c->stream));
        CU(cudaFree(b.p));
        b.p = nullptr;
        b.cap = 0;
    }
    cudaError_t e = cudaMalloc(&b.p, bytes);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return fail(LYAP_ERR_NOMEM, "device allocation of " + std::to_string(bytes) + " bytes failed");
    }
    if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc");
    b.cap = bytes;
    return LYAP_OK;
}

struct Geometry {
    long long row_begin, rows;
    long long n_pixels;
};

// Validates p and packs everything the lambda kernels need.
int build_args(const lyap_params* p, lyap::LambdaArgs* a, Geometry* g) {
    if (!p) return fail(LYAP_ERR_INVALID, "params is null");
    if (p->width < 1 || p->height < 1) return fail(LYAP_ERR_INVALID, "width and height must be >= 1");
    if (p->iterations < 0 || p->warmup < 0) return fail(LYAP_ERR_INVALID, "iterations and warmup must be >= 0");
    if (p->mode < LYAP_MODE_EXACT || p->mode > LYAP_MODE_FAST_FP64_ORBIT) return fail(LYAP_ERR_INVALID, "unknown mode");
    // the fast kernels keep each pixel's exponent sum in 32 bits: a derivative's exponent is at most 2 and, short of an
    // exact zero (handled apart), no less than about -60, so 2^24 steps stay far inside the range
    if (p->mode != LYAP_MODE_EXACT && (long long)p->iterations + p->warmup > (1LL << 24))
        return fail(LYAP_ERR_TOO_LARGE, "the fast modes take at most 2^24 steps per pixel (warmup + iterations)");
    if (!p->sequence) return fail(LYAP_ERR_SEQUENCE, "sequence is null");
    const long long seq_len = p->sequence_len < 0 ? (long long)std::strlen(p->sequence) : p->sequence_len;
    if (seq_len < 1) return fail(LYAP_ERR_SEQUENCE, "sequence is empty");
    long long rb = p->row_begin, re = p->row_end;
    if (rb == 0 && re == 0) re = p->height;
    if (rb < 0 || re > p->height || rb >= re) return fail(LYAP_ERR_INVALID, "row range must satisfy 0 <= begin < end <= height");

    // A region is stored whole when it fits; otherwise as one period of the sequence in whole words
    // (lcm(len, 16) steps = len / gcd(len, 16) words), which the kernels walk round and round.
    const long long period_words = seq_len / std::gcd(seq_len, (long long)lyap::kStepsPerWord);
    const long long wu_need = ((long long)p->warmup + lyap::kStepsPerWord - 1) / lyap::kStepsPerWord;
    const long long acc_need = ((long long)p->iterations + lyap::kStepsPerWord - 1) / lyap::kStepsPerWord;
    const long long wu_words = std::min(wu_need, period_words), acc_words = std::min(acc_need, period_words);
    if (wu_words + acc_words > lyap::kMaxSelWords)
        return fail(LYAP_ERR_TOO_LARGE, "warmup + iterations beyond " +
                                            std::to_string(lyap::kMaxSelWords * lyap::kStepsPerWord) +
                                            " steps with a sequence too long to store by its period");

    std::memset(a, 0, sizeof(*a));
    a->min_x = p->min_x;
    a->min_y = p->min_y;
    a->dx = (p->max_x - p->min_x) / (p->width - 1.0);    // src/lyapunov_fractal.hpp:29
    a->dy = (p->max_y - p->min_y) / (p->height - 1.0);   // :30
    a->c_value = p->c_value;
    a->row_begin = rb;
    a->n_pixels = (re - rb) * (long long)p->width;
    a->width = p->width;
    a->warmup = p->warmup;
    a->iterations = p->iterations;
    a->acc_word0 = (int)wu_words;
    a->wu_wrap = (int)std::max(1LL, wu_words);
    a->acc_wrap = (int)std::max(1LL, acc_words);
    const bool use_c = p->c_enabled != 0;
    bool seq_has_c = false;
    // step i uses sequence[i % len]; 'A' -> column parameter, anything else -> row parameter (:37),
    // except 'C' -> c_value when the extension is on
    auto code = [&](long long i) -> unsigned {
        const char ch = p->sequence[i % seq_len];
        if (ch == 'A') return 0u;
        if (use_c && ch == 'C') {
            seq_has_c = true;
            return 2u;
        }
        return 1u;
    };
    const long long wu_stored = std::min<long long>(p->warmup, wu_words * lyap::kStepsPerWord);
    const long long acc_stored = std::min<long long>(p->iterations, acc_words * lyap::kStepsPerWord);
    for (long long i = 0; i < wu_stored; ++i) a->sel[i / 16] |= code(i) << (2 * (i % 16));
    for (long long i = 0; i < acc_stored; ++i)
        a->sel[wu_words + i / 16] |= code((long long)p->warmup + i) << (2 * (i % 16));
    const double c = p->c_value;
    a->fast_ok_c = (!seq_has_c || (c > 0x1p-20 && c < 0x1p20)) ? 1 : 0;
    g->row_begin = rb;
    g->rows = re - rb;
    g->n_pixels = a->n_pixels;
    return LYAP_OK;
}

int launch_lambda(lyap_ctx* c, int mode, const lyap::LambdaArgs& a, double* d64, float* d32, unsigned long long* steps) {
    Range range("lyap: lambda");
    cudaError_t e;
    if (mode == LYAP_MODE_EXACT) e = lyap::launch_lambda_exact(a, d64, d32, steps, c->sm_count, c->stream);
    else if (mode == LYAP_MODE_FAST_FP64) e = lyap::launch_lambda_fast64(a, d64, d32, steps, c->sm_count, c->stream);
    else if (mode == LYAP_MODE_FAST_FP64_ORBIT) e = lyap::launch_lambda_orbit64(a, d64, d32, steps, c->sm_count, c->stream);
    else e = lyap::launch_lambda_fast32(a, d64, d32, steps, c->sm_count, c->stream);
    if (e != cudaSuccess) return fail_cuda(e, "lambda kernel launch");
    return LYAP_OK;
}

int check_ctx(lyap_ctx* c) {
    if (!c) return fail(LYAP_ERR_INVALID, "context is null");
    CU(cudaSetDevice(c->device));
    return LYAP_OK;
}

}  // namespace

namespace lyap {
int set_error(int status, const char* message) { return fail(status, message); }

int validate_whole_frame(const lyap_params* p) {
    LambdaArgs a;
    Geometry g;
    if (int r = build_args(p, &a, &g)) return r;
    if (g.rows != p->height) return fail(LYAP_ERR_INVALID, "whole frames only here (row_begin = row_end = 0)");
    return LYAP_OK;
}
}  // namespace lyap

extern "C" {

int lyap_abi_version(void) { return LYAP_ABI_VERSION; }

int lyap_self_test(void) { return 42; }

const char* lyap_jit_note(void) { return lyap::jit_last_note(); }

const char* lyap_last_kernel(void) { return lyap::last_lambda_kernel(); }

int lyap_selector_code(const lyap_params* p, int region, int64_t step, int* code) {
    if (!code || region < 0 || region > 1) return fail(LYAP_ERR_INVALID, "lyap_selector_code: bad region or null output");
    lyap::LambdaArgs a;
    Geometry g;
    if (int rc = build_args(p, &a, &g)) return rc;
    const long long n = region ? a.iterations : a.warmup;
    if (step < 0 || step >= n) return fail(LYAP_ERR_INVALID, "lyap_selector_code: step outside the region");
    const int word0 = region ? a.acc_word0 : 0, wrap = region ? a.acc_wrap : a.wu_wrap;
    *code = (int)((a.sel[word0 + (step / lyap::kStepsPerWord) % wrap] >> (2 * (step % lyap::kStepsPerWord))) & 3u);
    return LYAP_OK;
}

int lyap_group_patterns(const lyap_params* p, int* groups, uint64_t* warmup_patterns, uint64_t* accumulation_patterns) {
    if (!groups || !warmup_patterns || !accumulation_patterns) return fail(LYAP_ERR_INVALID, "lyap_group_patterns: null output");
    lyap::LambdaArgs a;
    Geometry g;
    if (int rc = build_args(p, &a, &g)) return rc;
    unsigned long long wu = 0, acc = 0;
    *groups = lyap::sequence_group_period(a, &wu, &acc);
    *warmup_patterns = wu;
    *accumulation_patterns = acc;
    return LYAP_OK;
}

const char* lyap_last_error(void) { return g_last_error.c_str(); }

const char* lyap_status_string(int s) {
    switch (s) {
        case LYAP_OK: return "ok";
        case LYAP_ERR_INVALID: return "invalid argument";
        case LYAP_ERR_SEQUENCE: return "empty or missing sequence";
        case LYAP_ERR_TOO_LARGE: return "too large";
        case LYAP_ERR_CUDA: return "CUDA error";
        case LYAP_ERR_NOMEM: return "out of device memory";
        case LYAP_ERR_TIMEOUT: return "timeout";
        case LYAP_ERR_COMM: return "communication error";
        default: return "unknown status";
    }
}

void lyap_params_default(lyap_params* p) {
    if (!p) return;
    std::memset(p, 0, sizeof(*p));
    p->min_x = 0.0;   // src/lyapunov_fractal.hpp:16-24
    p->max_x = 4.0;
    p->min_y = 0.0;
    p->max_y = 4.0;
    p->width = 800;
    p->height = 600;
    p->sequence = "ABABABAB";
    p->sequence_len = 8;
    p->iterations = 10000;
    p->warmup = 100;
}

int lyap_palette_from_name(const char* name) {
    static const char* names[] = {"cosmic", "nebula", "aurora", "solarflare", "blackhole", "psychedelic", "rainbow"};
    if (name)
        for (int i = 0; i < 7; ++i)
            if (std::strcmp(name, names[i]) == 0) return i;
    return LYAP_PALETTE_COSMIC;   // web/fractal_renderer.js:280
}

int lyap_device_count(int* count) {
    if (!count) return fail(LYAP_ERR_INVALID, "count is null");
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) {
        *count = 0;
        return fail_cuda(e, "cudaGetDeviceCount");
    }
    *count = n;
    return LYAP_OK;
}

int lyap_create(lyap_ctx** out, int device) {
    if (!out) return fail(LYAP_ERR_INVALID, "ctx pointer is null");
    *out = nullptr;
    int n = 0;
    CU(cudaGetDeviceCount(&n));
    if (device < 0 || device >= n) return fail(LYAP_ERR_INVALID, "no such device");
    CU(cudaSetDevice(device));
    cudaDeviceProp prop;
    CU(cudaGetDeviceProperties(&prop, device));
    if (prop.major < 10) return fail(LYAP_ERR_CUDA, "this library holds sm_100a code only; device is sm_" +
                                                        std::to_string(prop.major) + std::to_string(prop.minor));
    lyap_ctx* c = new (std::nothrow) lyap_ctx;
    if (!c) return fail(LYAP_ERR_NOMEM, "host allocation failed");
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    cudaError_t e = cudaStreamCreateWithFlags(&c->own_stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&c->small, 32 + lyap::kMinmaxScratchBytes);
    if (e == cudaSuccess) e = cudaMemset(c->small, 0, 32 + lyap::kMinmaxScratchBytes);
    for (int i = 0; i < 8 && e == cudaSuccess; ++i) e = cudaEventCreate(&c->ev[i]);
    if (e != cudaSuccess) {
        lyap_destroy(c);
        return fail_cuda(e, "context setup");
    }
    c->stream = c->own_stream;
    *out = c;
    return LYAP_OK;
}

int lyap_destroy(lyap_ctx* c) {
    if (!c) return LYAP_OK;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (Buffer* b : {&c->lambda, &c->lambda32, &c->norm, &c->rgba})
        if (b->p) cudaFree(b->p);
    if (c->small) cudaFree(c->small);
    for (auto& ev : c->ev)
        if (ev) cudaEventDestroy(ev);
    for (auto& ev : c->chunk_events) cudaEventDestroy(ev);
    if (c->own_stream) cudaStreamDestroy(c->own_stream);
    delete c;
    return LYAP_OK;
}

int lyap_set_stream(lyap_ctx* c, void* s) {
    if (int r = check_ctx(c)) return r;
    CU(cudaStreamSynchronize(c->stream));
    c->stream = s ? static_cast<cudaStream_t>(s) : c->own_stream;
    return LYAP_OK;
}

int lyap_sync(lyap_ctx* c) {
    if (int r = check_ctx(c)) return r;
    CU(cudaStreamSynchronize(c->stream));
    return LYAP_OK;
}

int lyap_device_alloc(lyap_ctx* c, void** dptr, size_t bytes) {
    if (int r = check_ctx(c)) return r;
    if (!dptr) return fail(LYAP_ERR_INVALID, "dptr is null");
    *dptr = nullptr;
    cudaError_t e = cudaMalloc(dptr, bytes ? bytes : 1);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return fail(LYAP_ERR_NOMEM, "device allocation of " + std::to_string(bytes) + " bytes failed");
    }
    if (e != cudaSuccess) return fail_cuda(e, "cudaMalloc");
    return LYAP_OK;
}

int lyap_device_free(lyap_ctx* c, void* dptr) {
    if (int r = check_ctx(c)) return r;
    CU(cudaFree(dptr));
    return LYAP_OK;
}

int lyap_host_alloc(void** hptr, size_t bytes) {
    if (!hptr) return fail(LYAP_ERR_INVALID, "hptr is null");
    *hptr = nullptr;
    cudaError_t e = cudaMallocHost(hptr, bytes ? bytes : 1);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return e == cudaErrorMemoryAllocation ? fail(LYAP_ERR_NOMEM, "pinned allocation failed") : fail_cuda(e, "cudaMallocHost");
    }
    return LYAP_OK;
}

int lyap_host_free(void* hptr) {
    if (!hptr) return LYAP_OK;
    CU(cudaFreeHost(hptr));
    return LYAP_OK;
}

int lyap_copy_to_host(lyap_ctx* c, void* host, const void* dev, size_t bytes) {
    if (int r = check_ctx(c)) return r;
    if (bytes == 0) return LYAP_OK;
    if (!host || !dev) return fail(LYAP_ERR_INVALID, "null pointer");
    CU(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    return LYAP_OK;
}

int lyap_copy_to_device(lyap_ctx* c, void* dev, const void* host, size_t bytes) {
    if (int r = check_ctx(c)) return r;
    if (bytes == 0) return LYAP_OK;
    if (!host || !dev) return fail(LYAP_ERR_INVALID, "null pointer");
    CU(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, c->stream));
    CU(cudaStreamSynchronize(c->stream));
    return LYAP_OK;
}

// ---- device-pointer entry points ----

int lyap_lambda_device(lyap_ctx* c, const lyap_params* p, double* d_lambda, float* d_lambda32, uint64_t* d_steps) {
    if (int r = check_ctx(c)) return r;
    lyap::LambdaArgs a;
    Geometry g;
    if (int r = build_args(p, &a, &g)) return r;
    if (!d_lambda && !d_lambda32) return fail(LYAP_ERR_INVALID, "both outputs are null");
    return launch_lambda(c, p->mode, a, d_lambda, d_lambda32, reinterpret_cast<unsigned long long*>(d_steps));
}

int lyap_minmax_device(lyap_ctx* c, const double* d_values, uint64_t n, double* d_minmax) {
    if (int r = check_ctx(c)) return r;
    if (!d_minmax || (!d_values && n)) return fail(LYAP_ERR_INVALID, "null pointer");
    Range range("lyap: min/max");
    cudaError_t e = lyap::launch_minmax(d_values, n, d_minmax, ctx_scratch(c), c->sm_count, c->stream);
    if (e != cudaSuccess) return fail_cuda(e, "minmax launch");
    return LYAP_OK;
}

int lyap_normalize_device(lyap_ctx* c, const double* d_values, uint64_t n, const double* d_minmax, double* d_out) {
    if (int r = check_ctx(c)) return r;
    if (n == 0) return LYAP_OK;
    if (!d_values || !d_minmax || !d_out) return fail(LYAP_ERR_INVALID, "null pointer");
    Range range("lyap: normalise");
    cudaError_t e = lyap::launch_normalize(d_values, n, d_minmax, d_out, c->sm_count, c->stream);
    if (e != cudaSuccess) return fail_cuda(e, "normalize launch");
    return LYAP_OK;
}

int lyap_colorize_device(lyap_ctx* c, const double* d_norm, int32_t width, int64_t rows, int32_t rows_above,
                         int32_t rows_below, int32_t palette, uint8_t* d_rgba) {
    if (int r = check_ctx(c)) return r;
    if (width < 1 || rows < 0) return fail(LYAP_ERR_INVALID, "bad dimensions");
    if (rows == 0) return LYAP_OK;
    if (!d_norm || !d_rgba) return fail(LYAP_ERR_INVALID, "null pointer");
    if (palette < 0 || palette > LYAP_PALETTE_RAINBOW) palette = LYAP_PALETTE_COSMIC;
    Range range("lyap: colour");
    cudaError_t e = lyap::launch_colorize(d_norm, width, rows, rows_above ? 1 : 0, rows_below ? 1 : 0, palette, d_rgba,
                                          c->sm_count, c->stream);
    if (e != cudaSuccess) return fail_cuda(e, "colorize launch");
    return LYAP_OK;
}

int lyap_glow_device(lyap_ctx* c, uint8_t* d_rgba, int32_t width, int32_t height, void* d_scratch) {
    if (int r = check_ctx(c)) return r;
    if (width < 1 || height < 1) return fail(LYAP_ERR_INVALID, "bad dimensions");
    if (!d_rgba || !d_scratch) return fail(LYAP_ERR_INVALID, "null pointer");
    cudaError_t e = lyap::launch_glow(d_rgba, width, height, static_cast<double*>(d_scratch), c->sm_count, c->stream);
    if (e != cudaSuccess) return fail_cuda(e, "glow launch");
    return LYAP_OK;
}

// ---- host-pointer entry points ----

int lyap_render(lyap_ctx* c, const lyap_params* p, double* out_lambda, float* out_lambda32, double* out_norm,
                uint8_t* out_rgba, lyap_progress_fn progress, lyap_render_stats* stats) {
    if (int r = check_ctx(c)) return r;
    lyap::LambdaArgs a;
    Geometry g;
    if (int r = build_args(p, &a, &g)) return r;
    const size_t n = (size_t)g.n_pixels;
    const bool want_colour = out_norm || out_rgba;
    if (want_colour && g.rows != p->height)
        return fail(LYAP_ERR_INVALID, "normalised / RGBA output needs the whole frame's min and max: "
                                      "render all rows, or use the device entry points per band");
    if (int r = ensure(c, c->lambda, n * sizeof(double))) return r;
    if (out_lambda32)
        if (int r = ensure(c, c->lambda32, n * sizeof(float))) return r;
    if (want_colour)
        if (int r = ensure(c, c->norm, n * sizeof(double))) return r;
    if (out_rgba)
        if (int r = ensure(c, c->rgba, n * 4)) return r;

    double* d_lambda = static_cast<double*>(c->lambda.p);
    float* d_l32 = out_lambda32 ? static_cast<float*>(c->lambda32.p) : nullptr;
    double* d_norm = static_cast<double*>(c->norm.p);
    uint8_t* d_rgba = static_cast<uint8_t*>(c->rgba.p);
    cudaStream_t st = c->stream;
    int launches = 0;

    CU(cudaMemsetAsync(ctx_steps(c), 0, 8, st));
    CU(cudaEventRecord(c->ev[0], st));
    if (!progress) {
        if (int r = launch_lambda(c, p->mode, a, d_lambda, d_l32, ctx_steps(c))) return r;
        ++launches;
    } else {
        // row chunks so the callback can follow completed rows; each chunk keeps every SM busy for
        // several tiles, and there are at most ~64 chunks
        const long long min_rows = (8LL * c->sm_count * 1024 + p->width - 1) / p->width;
        long long chunk_rows = (g.rows + 63) / 64;
        if (chunk_rows < min_rows) chunk_rows = min_rows;
        const long long nchunks = (g.rows + chunk_rows - 1) / chunk_rows;
        while ((long long)c->chunk_events.size() < nchunks) {
            cudaEvent_t ev;
            CU(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
            c->chunk_events.push_back(ev);
        }
        for (long long k = 0; k < nchunks; ++k) {
            lyap::LambdaArgs ak = a;
            const long long r0 = k * chunk_rows;
            const long long r1 = r0 + chunk_rows < g.rows ? r0 + chunk_rows : g.rows;
            ak.row_begin = g.row_begin + r0;
            ak.n_pixels = (r1 - r0) * (long long)p->width;
            const size_t off = (size_t)r0 * p->width;
            if (int r = launch_lambda(c, p->mode, ak, d_lambda + off, d_l32 ? d_l32 + off : nullptr, ctx_steps(c)))
                return r;
            ++launches;
            CU(cudaEventRecord(c->chunk_events[k], st));
        }
        for (long long k = 0; k < nchunks; ++k) {
            CU(cudaEventSynchronize(c->chunk_events[k]));
            const long long done_rows = (k + 1) * chunk_rows < g.rows ? (k + 1) * chunk_rows : g.rows;
            if (done_rows < g.rows) progress((double)(g.row_begin + done_rows) / p->height);
        }
    }
    CU(cudaEventRecord(c->ev[1], st));
    if (want_colour) {
        nvtxRangePushA("lyap: min/max");
        cudaError_t e = lyap::launch_minmax(d_lambda, n, ctx_minmax(c), ctx_scratch(c), c->sm_count, st);
        nvtxRangePop();
        if (e != cudaSuccess) return fail_cuda(e, "minmax launch");
        CU(cudaEventRecord(c->ev[2], st));
        Range range("lyap: normalise");
        e = lyap::launch_normalize(d_lambda, n, ctx_minmax(c), d_norm, c->sm_count, st);
        if (e != cudaSuccess) return fail_cuda(e, "normalize launch");
        launches += 2;
    } else {
        CU(cudaEventRecord(c->ev[2], st));
    }
    CU(cudaEventRecord(c->ev[3], st));
    if (out_rgba) {
        int pal = p->palette;
        if (pal < 0 || pal > LYAP_PALETTE_RAINBOW) pal = LYAP_PALETTE_COSMIC;
        Range range("lyap: colour");
        cudaError_t e = lyap::launch_colorize(d_norm, p->width, p->height, 0, 0, pal, d_rgba, c->sm_count, st);
        if (e != cudaSuccess) return fail_cuda(e, "colorize launch");
        ++launches;
    }
    CU(cudaEventRecord(c->ev[4], st));
    Range copies("lyap: copies to host");
    if (out_lambda) CU(cudaMemcpyAsync(out_lambda, d_lambda, n * sizeof(double), cudaMemcpyDeviceToHost, st));
    if (out_lambda32) CU(cudaMemcpyAsync(out_lambda32, d_l32, n * sizeof(float), cudaMemcpyDeviceToHost, st));
    if (out_norm) CU(cudaMemcpyAsync(out_norm, d_norm, n * sizeof(double), cudaMemcpyDeviceToHost, st));
    if (out_rgba) CU(cudaMemcpyAsync(out_rgba, d_rgba, n * 4, cudaMemcpyDeviceToHost, st));
    struct {
        double mm[2];
        unsigned long long steps;
    } small;
    CU(cudaMemcpyAsync(&small, c->small, sizeof(small), cudaMemcpyDeviceToHost, st));
    CU(cudaEventRecord(c->ev[5], st));
    CU(cudaStreamSynchronize(st));
    if (progress) progress(1.0);   // src/lyapunov_fractal.hpp:97-99
    if (stats) {
        std::memset(stats, 0, sizeof(*stats));
        stats->executed_steps = small.steps;
        stats->nominal_steps = (uint64_t)n * (uint64_t)((long long)p->warmup + p->iterations);
        stats->lambda_min = want_colour ? small.mm[0] : NAN;
        stats->lambda_max = want_colour ? small.mm[1] : NAN;
        cudaEventElapsedTime(&stats->ms_lambda, c->ev[0], c->ev[1]);
        cudaEventElapsedTime(&stats->ms_minmax, c->ev[1], c->ev[2]);
        cudaEventElapsedTime(&stats->ms_normalize, c->ev[2], c->ev[3]);
        cudaEventElapsedTime(&stats->ms_colorize, c->ev[3], c->ev[4]);
        cudaEventElapsedTime(&stats->ms_total_device, c->ev[0], c->ev[4]);
        cudaEventElapsedTime(&stats->ms_copies, c->ev[4], c->ev[5]);
        stats->kernel_launches = launches;
    }
    return LYAP_OK;
}

int lyap_compute_fractal(lyap_ctx* c, const lyap_params* p, double* out_lambda, lyap_progress_fn progress) {
    if (!out_lambda) return fail(LYAP_ERR_INVALID, "out_lambda is null");
    return lyap_render(c, p, out_lambda, nullptr, nullptr, nullptr, progress, nullptr);
}

int lyap_normalize_data(lyap_ctx* c, const double* values, uint64_t n, double* out) {
    if (int r = check_ctx(c)) return r;
    if (n == 0) return LYAP_OK;   // src/lyapunov_fractal.hpp:106
    if (!values || !out) return fail(LYAP_ERR_INVALID, "null pointer");
    if (int r = ensure(c, c->lambda, n * sizeof(double))) return r;
    if (int r = ensure(c, c->norm, n * sizeof(double))) return r;
    cudaStream_t st = c->stream;
    CU(cudaMemcpyAsync(c->lambda.p, values, n * sizeof(double), cudaMemcpyHostToDevice, st));
    cudaError_t e = lyap::launch_minmax(static_cast<double*>(c->lambda.p), n, ctx_minmax(c), ctx_scratch(c), c->sm_count, st);
    if (e != cudaSuccess) return fail_cuda(e, "minmax launch");
    e = lyap::launch_normalize(static_cast<double*>(c->lambda.p), n, ctx_minmax(c), static_cast<double*>(c->norm.p),
                               c->sm_count, st);
    if (e != cudaSuccess) return fail_cuda(e, "normalize launch");
    CU(cudaMemcpyAsync(out, c->norm.p, n * sizeof(double), cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    return LYAP_OK;
}

int lyap_colorize(lyap_ctx* c, const double* norm, int32_t width, int32_t height, int32_t palette, uint8_t* out_rgba) {
    if (int r = check_ctx(c)) return r;
    if (width < 1 || height < 1) return fail(LYAP_ERR_INVALID, "bad dimensions");
    if (!norm || !out_rgba) return fail(LYAP_ERR_INVALID, "null pointer");
    const size_t n = (size_t)width * height;
    if (int r = ensure(c, c->norm, n * sizeof(double))) return r;
    if (int r = ensure(c, c->rgba, n * 4)) return r;
    if (palette < 0 || palette > LYAP_PALETTE_RAINBOW) palette = LYAP_PALETTE_COSMIC;
    cudaStream_t st = c->stream;
    CU(cudaMemcpyAsync(c->norm.p, norm, n * sizeof(double), cudaMemcpyHostToDevice, st));
    cudaError_t e = lyap::launch_colorize(static_cast<double*>(c->norm.p), width, height, 0, 0, palette,
                                          static_cast<uint8_t*>(c->rgba.p), c->sm_count, st);
    if (e != cudaSuccess) return fail_cuda(e, "colorize launch");
    CU(cudaMemcpyAsync(out_rgba, c->rgba.p, n * 4, cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    return LYAP_OK;
}

}  // extern "C"

extern "C" {

int lyap_glow(lyap_ctx* c, const uint8_t* rgba_in, int32_t width, int32_t height, uint8_t* rgba_out) {
    if (int r = check_ctx(c)) return r;
    if (width < 1 || height < 1) return fail(LYAP_ERR_INVALID, "bad dimensions");
    if (!rgba_in || !rgba_out) return fail(LYAP_ERR_INVALID, "null pointer");
    const size_t n = (size_t)width * height;
    if (int r = ensure(c, c->rgba, n * 4)) return r;
    if (int r = ensure(c, c->norm, n * 24)) return r;   // the blur's scratch shares the normalised-frame buffer
    cudaStream_t st = c->stream;
    CU(cudaMemcpyAsync(c->rgba.p, rgba_in, n * 4, cudaMemcpyHostToDevice, st));
    cudaError_t e = lyap::launch_glow(static_cast<uint8_t*>(c->rgba.p), width, height, static_cast<double*>(c->norm.p), c->sm_count, st);
    if (e != cudaSuccess) return fail_cuda(e, "glow launch");
    CU(cudaMemcpyAsync(rgba_out, c->rgba.p, n * 4, cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    return LYAP_OK;
}

// ---- measurement ----

static int peak_common(lyap_ctx* c, bool fp64, double* out) {
    if (int r = check_ctx(c)) return r;
    if (!out) return fail(LYAP_ERR_INVALID, "null pointer");
    cudaStream_t st = c->stream;
    void* sink = ctx_minmax(c);   // never written (the kernel's store condition is never true)
    unsigned long long instr = 0;
    double best = 0;
    for (int rep = 0; rep < 4; ++rep) {
        CU(cudaEventRecord(c->ev[6], st));
        cudaError_t e = fp64 ? lyap::launch_fp64_peak(static_cast<double*>(sink), c->sm_count, 400, &instr, st)
                             : lyap::launch_fp32_peak(static_cast<float*>(sink), c->sm_count, 800, &instr, st);
        if (e != cudaSuccess) return fail_cuda(e, "peak kernel launch");
        CU(cudaEventRecord(c->ev[7], st));
        CU(cudaEventSynchronize(c->ev[7]));
        float ms = 0;
        CU(cudaEventElapsedTime(&ms, c->ev[6], c->ev[7]));
        const double rate = (double)instr / (ms * 1e-3);
        if (rep > 0 && rate > best) best = rate;
    }
    *out = best;
    return LYAP_OK;
}

int lyap_fp64_peak(lyap_ctx* c, double* instr_per_second) { return peak_common(c, true, instr_per_second); }
int lyap_fp32_peak(lyap_ctx* c, double* instr_per_second) { return peak_common(c, false, instr_per_second); }

}  // extern "C"
