// lyap_abi.cu -- implementation of the C ABI declared in include/lyap_b200.h.
//
// Host-side orchestration only: parameter checks, the sequence-to-selector packing
// (reference src/lyapunov_fractal.hpp:34-38), buffer management, launches, copies, timing.
// There is deliberately no CPU implementation behind these entry points.
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <chrono>
#include <condition_variable>
#include <mutex>
#include <new>
#include <numeric>
#include <thread>
#include <string>
#include <vector>

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
    if (p->mode < LYAP_MODE_EXACT || p->mode > LYAP_MODE_FAST_FP32) return fail(LYAP_ERR_INVALID, "unknown mode");
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
    cudaError_t e;
    if (mode == LYAP_MODE_EXACT) e = lyap::launch_lambda_exact(a, d64, d32, steps, c->sm_count, c->stream);
    else if (mode == LYAP_MODE_FAST_FP64) e = lyap::launch_lambda_fast64(a, d64, d32, steps, c->sm_count, c->stream);
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
}  // namespace lyap

extern "C" {

int lyap_abi_version(void) { return LYAP_ABI_VERSION; }

int lyap_self_test(void) { return 42; }

const char* lyap_jit_note(void) { return lyap::jit_last_note(); }

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
    cudaError_t e = lyap::launch_minmax(d_values, n, d_minmax, ctx_scratch(c), c->stream);
    if (e != cudaSuccess) return fail_cuda(e, "minmax launch");
    return LYAP_OK;
}

int lyap_normalize_device(lyap_ctx* c, const double* d_values, uint64_t n, const double* d_minmax, double* d_out) {
    if (int r = check_ctx(c)) return r;
    if (n == 0) return LYAP_OK;
    if (!d_values || !d_minmax || !d_out) return fail(LYAP_ERR_INVALID, "null pointer");
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
    cudaError_t e = lyap::launch_colorize(d_norm, width, rows, rows_above ? 1 : 0, rows_below ? 1 : 0, palette, d_rgba,
                                          c->stream);
    if (e != cudaSuccess) return fail_cuda(e, "colorize launch");
    return LYAP_OK;
}

int lyap_glow_device(lyap_ctx* c, uint8_t* d_rgba, int32_t width, int32_t height, void* d_scratch) {
    if (int r = check_ctx(c)) return r;
    if (width < 1 || height < 1) return fail(LYAP_ERR_INVALID, "bad dimensions");
    if (!d_rgba || !d_scratch) return fail(LYAP_ERR_INVALID, "null pointer");
    cudaError_t e = lyap::launch_glow(d_rgba, width, height, static_cast<double*>(d_scratch), c->stream);
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
        cudaError_t e = lyap::launch_minmax(d_lambda, n, ctx_minmax(c), ctx_scratch(c), st);
        if (e != cudaSuccess) return fail_cuda(e, "minmax launch");
        CU(cudaEventRecord(c->ev[2], st));
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
        cudaError_t e = lyap::launch_colorize(d_norm, p->width, p->height, 0, 0, pal, d_rgba, st);
        if (e != cudaSuccess) return fail_cuda(e, "colorize launch");
        ++launches;
    }
    CU(cudaEventRecord(c->ev[4], st));
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
    cudaError_t e = lyap::launch_minmax(static_cast<double*>(c->lambda.p), n, ctx_minmax(c), ctx_scratch(c), st);
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
                                          static_cast<uint8_t*>(c->rgba.p), st);
    if (e != cudaSuccess) return fail_cuda(e, "colorize launch");
    CU(cudaMemcpyAsync(out_rgba, c->rgba.p, n * 4, cudaMemcpyDeviceToHost, st));
    CU(cudaStreamSynchronize(st));
    return LYAP_OK;
}

}  // extern "C"

// ---- one frame over several devices ----

namespace {

struct MultiShared {
    std::mutex mu;
    std::condition_variable cv;
    int arrived = 0, expected = 0;
    bool failed = false;
    double lo = 0, hi = 0;
    bool have = false;
    unsigned long long steps = 0;
    int status = LYAP_OK;
    std::string error;
};

void multi_fail(MultiShared& sh, int status, const char* msg) {
    std::lock_guard<std::mutex> lk(sh.mu);
    if (sh.status == LYAP_OK) {
        sh.status = status;
        sh.error = msg;
    }
    sh.failed = true;
    sh.cv.notify_all();
}

// One band on one device.  Returns after its part of the host buffers is written, or after a failure anywhere.
void multi_worker(MultiShared& sh, const lyap_params& base, int device, long long b0, long long b1, double* out_lambda,
                  double* out_norm, uint8_t* out_rgba, double timeout_s) {
    lyap_ctx* c = nullptr;
    if (lyap_create(&c, device) != LYAP_OK) return multi_fail(sh, LYAP_ERR_CUDA, lyap_last_error());
    const long long H = base.height, W = base.width;
    const int above = b0 > 0 ? 1 : 0, below = b1 < H ? 1 : 0;
    const long long rows_all = (b1 - b0) + above + below, rows_own = b1 - b0;
    // one device allocation for the band: lambda | normalised | RGBA | min/max + step counter (allocations are
    // serialised across the workers of a process, so they are kept few)
    void *block = nullptr, *d_lam = nullptr, *d_norm = nullptr, *d_rgba = nullptr, *d_small = nullptr;
    auto cleanup = [&]() {
        if (block) lyap_device_free(c, block);
        lyap_destroy(c);
    };
    auto bail = [&](int st) {
        multi_fail(sh, st, lyap_last_error());
        cleanup();
    };
    const bool colour = out_norm || out_rgba;
    const size_t lam_bytes = ((size_t)rows_all * W * 8 + 255) / 256 * 256;
    const size_t norm_bytes = colour ? lam_bytes : 0;
    const size_t rgba_bytes = out_rgba ? ((size_t)rows_own * W * 4 + 255) / 256 * 256 : 0;
    int st = lyap_device_alloc(c, &block, lam_bytes + norm_bytes + rgba_bytes + 256);
    if (st != LYAP_OK) return bail(st);
    d_lam = block;
    d_norm = colour ? static_cast<char*>(block) + lam_bytes : nullptr;
    d_rgba = out_rgba ? static_cast<char*>(block) + lam_bytes + norm_bytes : nullptr;
    d_small = static_cast<char*>(block) + lam_bytes + norm_bytes + rgba_bytes;
    double* d_mm = static_cast<double*>(d_small);
    uint64_t* d_steps = reinterpret_cast<uint64_t*>(d_mm + 2);
    uint64_t zero = 0;
    double* own = static_cast<double*>(d_lam) + (size_t)above * W;
    st = lyap_copy_to_device(c, d_steps, &zero, 8);
    {   // the band's own rows (counted), then the halo rows (same kernel, not counted)
        lyap_params p = base;
        p.row_begin = b0;
        p.row_end = b1;
        if (st == LYAP_OK) st = lyap_lambda_device(c, &p, own, nullptr, d_steps);
        if (st == LYAP_OK && above) {
            p.row_begin = b0 - 1;
            p.row_end = b0;
            st = lyap_lambda_device(c, &p, static_cast<double*>(d_lam), nullptr, nullptr);
        }
        if (st == LYAP_OK && below) {
            p.row_begin = b1;
            p.row_end = b1 + 1;
            st = lyap_lambda_device(c, &p, own + (size_t)rows_own * W, nullptr, nullptr);
        }
    }
    if (st == LYAP_OK) st = lyap_minmax_device(c, own, (uint64_t)rows_own * W, d_mm);
    double mm[2];
    uint64_t steps = 0;
    if (st == LYAP_OK) st = lyap_copy_to_host(c, mm, d_mm, 16);
    if (st == LYAP_OK) st = lyap_copy_to_host(c, &steps, d_steps, 8);
    if (st != LYAP_OK) return bail(st);
    {   // the one exchange: min of mins, max of maxes, with a deadline
        std::unique_lock<std::mutex> lk(sh.mu);
        sh.lo = sh.have ? std::fmin(sh.lo, mm[0]) : mm[0];
        sh.hi = sh.have ? std::fmax(sh.hi, mm[1]) : mm[1];
        sh.have = true;
        sh.steps += steps;
        ++sh.arrived;
        sh.cv.notify_all();
        const bool ok = sh.cv.wait_for(lk, std::chrono::duration<double>(timeout_s),
                                       [&] { return sh.arrived == sh.expected || sh.failed; });
        if (!ok && sh.status == LYAP_OK) {
            sh.status = LYAP_ERR_TIMEOUT;
            sh.error = "lyap_render_multi: a band did not reach the min/max exchange before the deadline";
            sh.failed = true;
            sh.cv.notify_all();
        }
        if (sh.failed) {
            lk.unlock();
            cleanup();
            return;
        }
        mm[0] = sh.lo;
        mm[1] = sh.hi;
    }
    if (out_lambda) st = lyap_copy_to_host(c, out_lambda + (size_t)b0 * W, own, (size_t)rows_own * W * 8);
    if (st == LYAP_OK && colour) {
        st = lyap_copy_to_device(c, d_mm, mm, 16);
        if (st == LYAP_OK) st = lyap_normalize_device(c, static_cast<double*>(d_lam), (uint64_t)rows_all * W, d_mm, static_cast<double*>(d_norm));
        double* norm_own = static_cast<double*>(d_norm) + (size_t)above * W;
        if (st == LYAP_OK && out_rgba)
            st = lyap_colorize_device(c, norm_own, base.width, rows_own, above, below, base.palette, static_cast<uint8_t*>(d_rgba));
        if (st == LYAP_OK && out_norm) st = lyap_copy_to_host(c, out_norm + (size_t)b0 * W, norm_own, (size_t)rows_own * W * 8);
        if (st == LYAP_OK && out_rgba) st = lyap_copy_to_host(c, out_rgba + (size_t)b0 * W * 4, d_rgba, (size_t)rows_own * W * 4);
    }
    if (st != LYAP_OK) return bail(st);
    cleanup();
}

}  // namespace

extern "C" int lyap_render_multi(const lyap_params* p, int32_t n_devices, const int32_t* devices, double* out_lambda,
                                 double* out_norm, uint8_t* out_rgba, double timeout_seconds, lyap_render_stats* stats) {
    lyap::LambdaArgs args;
    Geometry g;
    if (int r = build_args(p, &args, &g)) return r;
    if (g.rows != p->height) return fail(LYAP_ERR_INVALID, "lyap_render_multi renders whole frames (row_begin = row_end = 0)");
    if (n_devices < 1 || !devices) return fail(LYAP_ERR_INVALID, "need at least one device");
    if (n_devices > p->height) return fail(LYAP_ERR_INVALID, "more bands than rows");
    if (timeout_seconds <= 0) timeout_seconds = 60.0;
    const auto t0 = std::chrono::steady_clock::now();
    MultiShared sh;
    sh.expected = n_devices;
    std::vector<std::thread> workers;
    const long long H = p->height, base = H / n_devices, extra = H % n_devices;
    for (int r = 0; r < n_devices; ++r) {
        const long long b0 = r * base + (r < extra ? r : extra);
        const long long b1 = b0 + base + (r < extra ? 1 : 0);
        if (devices[r] < 0) continue;   // a band whose worker never arrives
        workers.emplace_back(multi_worker, std::ref(sh), std::cref(*p), (int)devices[r], b0, b1, out_lambda, out_norm,
                             out_rgba, timeout_seconds);
    }
    for (auto& w : workers) w.join();
    if (workers.empty()) return fail(LYAP_ERR_TIMEOUT, "lyap_render_multi: no band arrived");
    if (sh.status != LYAP_OK) return fail(sh.status, sh.error);
    if (stats) {
        std::memset(stats, 0, sizeof(*stats));
        stats->executed_steps = sh.steps;
        stats->nominal_steps = (uint64_t)g.n_pixels * (uint64_t)((long long)p->warmup + p->iterations);
        stats->lambda_min = sh.lo;
        stats->lambda_max = sh.hi;
        stats->ms_total_device = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
        stats->kernel_launches = 6 * n_devices - 2;   // per band: lambda for own rows + up to two halo rows, min/max, normalise, colour
    }
    return LYAP_OK;
}

// ---- a batch of independent frames (a zoom sequence) over several devices ----

namespace {

struct FramesShared {
    std::mutex mu;
    bool failed = false;
    int status = LYAP_OK;
    std::string error;
};

void frames_fail(FramesShared& sh, int status, const char* msg) {
    std::lock_guard<std::mutex> lk(sh.mu);
    if (sh.status == LYAP_OK) {
        sh.status = status;
        sh.error = msg;
    }
    sh.failed = true;
}

struct FrameSmall {
    double mm[2];
    unsigned long long steps;
};

// One set of device buffers; a worker alternates between two, so that one frame's copies to the host run
// while the next frame is computed.
struct FrameSlot {
    void* block = nullptr;           // one device allocation: lambda | normalised | RGBA | min/max + step counter
    void *lam = nullptr, *norm = nullptr, *rgba = nullptr, *small = nullptr;
    FrameSmall* h_small = nullptr;   // pinned, owned by the caller of the workers
    cudaEvent_t begun = nullptr, lambda_done = nullptr, computed = nullptr, copied = nullptr;
    int frame = -1;
};

// Frames first, first + stride, ... on one device: kernels in order on the context's stream, copies on a second
// stream behind an event, two buffer sets.
void frames_worker(FramesShared& sh, int device, int first, int stride, const lyap_params* frames, int n_frames,
                   double* const* out_norm, uint8_t* const* out_rgba, lyap_render_stats* stats, FrameSmall* pinned) {
    lyap_ctx* c = nullptr;
    if (lyap_create(&c, device) != LYAP_OK) return frames_fail(sh, LYAP_ERR_CUDA, lyap_last_error());
    cudaStream_t copy = nullptr;
    FrameSlot slots[2];
    size_t max_px = 0;
    bool any_rgba = false;
    for (int k = first; k < n_frames; k += stride) {
        max_px = std::max(max_px, (size_t)frames[k].width * (size_t)frames[k].height);
        any_rgba = any_rgba || (out_rgba && out_rgba[k]);
    }
    auto cleanup = [&]() {
        cudaStreamSynchronize(c->stream);
        if (copy) cudaStreamSynchronize(copy);
        for (FrameSlot& s : slots) {
            if (s.block) cudaFree(s.block);
            for (cudaEvent_t e : {s.begun, s.lambda_done, s.computed, s.copied})
                if (e) cudaEventDestroy(e);
        }
        if (copy) cudaStreamDestroy(copy);
        lyap_destroy(c);
    };
    auto bail_cuda = [&](cudaError_t e, const char* what) {
        fail_cuda(e, what);
        frames_fail(sh, LYAP_ERR_CUDA, lyap_last_error());
        cleanup();
    };
#define FR(call)                                                   \
    do {                                                           \
        cudaError_t fr_e = (call);                                 \
        if (fr_e != cudaSuccess) return bail_cuda(fr_e, #call);    \
    } while (0)
    FR(cudaStreamCreateWithFlags(&copy, cudaStreamNonBlocking));
    // allocations are few on purpose: with several devices in one process every cudaMalloc / cudaFree and, far more,
    // every pinned allocation is serialised across the workers
    const size_t px8 = (max_px * 8 + 255) / 256 * 256, px4 = any_rgba ? (max_px * 4 + 255) / 256 * 256 : 0;
    for (int i = 0; i < 2; ++i) {
        FrameSlot& s = slots[i];
        FR(cudaMalloc(&s.block, 2 * px8 + px4 + 256));
        char* base = static_cast<char*>(s.block);
        s.lam = base;
        s.norm = base + px8;
        s.rgba = any_rgba ? base + 2 * px8 : nullptr;
        s.small = base + 2 * px8 + px4;
        s.h_small = pinned + i;
        for (cudaEvent_t* e : {&s.begun, &s.lambda_done, &s.computed, &s.copied}) FR(cudaEventCreate(e));
    }
    // the slot's frame has reached the host: fill in its statistics
    auto finish = [&](FrameSlot& s) -> cudaError_t {
        if (s.frame < 0) return cudaSuccess;
        cudaError_t e = cudaEventSynchronize(s.copied);
        if (e != cudaSuccess) return e;
        if (stats) {
            const lyap_params& p = frames[s.frame];
            lyap_render_stats& r = stats[s.frame];
            std::memset(&r, 0, sizeof(r));
            r.executed_steps = s.h_small->steps;
            r.nominal_steps = (uint64_t)p.width * (uint64_t)p.height * (uint64_t)((long long)p.warmup + p.iterations);
            r.lambda_min = s.h_small->mm[0];
            r.lambda_max = s.h_small->mm[1];
            cudaEventElapsedTime(&r.ms_lambda, s.begun, s.lambda_done);
            cudaEventElapsedTime(&r.ms_total_device, s.begun, s.computed);
            cudaEventElapsedTime(&r.ms_copies, s.computed, s.copied);
            r.kernel_launches = (out_rgba && out_rgba[s.frame]) ? 4 : 3;
        }
        s.frame = -1;
        return cudaSuccess;
    };
    int local = 0;
    for (int k = first; k < n_frames; k += stride, ++local) {
        {
            std::lock_guard<std::mutex> lk(sh.mu);
            if (sh.failed) break;
        }
        FrameSlot& s = slots[local & 1];
        FR(finish(s));   // its buffers are free again
        const lyap_params& p = frames[k];
        const size_t n = (size_t)p.width * (size_t)p.height;
        double* d_mm = static_cast<double*>(s.small);
        uint64_t* d_steps = reinterpret_cast<uint64_t*>(d_mm + 2);
        cudaStream_t st = c->stream;
        FR(cudaMemsetAsync(d_steps, 0, 8, st));
        FR(cudaEventRecord(s.begun, st));
        int rc = lyap_lambda_device(c, &p, static_cast<double*>(s.lam), nullptr, d_steps);
        if (rc == LYAP_OK) {
            FR(cudaEventRecord(s.lambda_done, st));
            rc = lyap_minmax_device(c, static_cast<double*>(s.lam), n, d_mm);
        }
        if (rc == LYAP_OK) rc = lyap_normalize_device(c, static_cast<double*>(s.lam), n, d_mm, static_cast<double*>(s.norm));
        uint8_t* h_rgba = out_rgba ? out_rgba[k] : nullptr;
        double* h_norm = out_norm ? out_norm[k] : nullptr;
        if (rc == LYAP_OK && h_rgba)
            rc = lyap_colorize_device(c, static_cast<double*>(s.norm), p.width, p.height, 0, 0, p.palette, static_cast<uint8_t*>(s.rgba));
        if (rc != LYAP_OK) {
            frames_fail(sh, rc, lyap_last_error());
            cleanup();
            return;
        }
        FR(cudaEventRecord(s.computed, st));
        FR(cudaStreamWaitEvent(copy, s.computed, 0));
        if (h_norm) FR(cudaMemcpyAsync(h_norm, s.norm, n * 8, cudaMemcpyDeviceToHost, copy));
        if (h_rgba) FR(cudaMemcpyAsync(h_rgba, s.rgba, n * 4, cudaMemcpyDeviceToHost, copy));
        FR(cudaMemcpyAsync(s.h_small, s.small, sizeof(FrameSmall), cudaMemcpyDeviceToHost, copy));
        FR(cudaEventRecord(s.copied, copy));
        s.frame = k;
    }
    for (FrameSlot& s : slots) FR(finish(s));
#undef FR
    cleanup();
}

}  // namespace

extern "C" int lyap_render_frames(const lyap_params* frames, int32_t n_frames, int32_t n_devices, const int32_t* devices,
                                  double* const* out_norm, uint8_t* const* out_rgba, lyap_render_stats* stats) {
    if (n_frames < 0 || (n_frames > 0 && !frames)) return fail(LYAP_ERR_INVALID, "lyap_render_frames: bad frame list");
    if (n_devices < 1 || !devices) return fail(LYAP_ERR_INVALID, "need at least one device");
    for (int k = 0; k < n_frames; ++k) {
        lyap::LambdaArgs a;
        Geometry g;
        if (int r = build_args(&frames[k], &a, &g)) return r;
        if (g.rows != frames[k].height)
            return fail(LYAP_ERR_INVALID, "lyap_render_frames renders whole frames (row_begin = row_end = 0)");
    }
    if (n_frames == 0) return LYAP_OK;
    // one pinned block for every worker's two small read-back records
    int n_dev_present = 0;
    CU(cudaGetDeviceCount(&n_dev_present));
    if (devices[0] < 0 || devices[0] >= n_dev_present) return fail(LYAP_ERR_INVALID, "no such device");
    CU(cudaSetDevice(devices[0]));
    FrameSmall* pinned = nullptr;
    CU(cudaMallocHost(reinterpret_cast<void**>(&pinned), (size_t)n_devices * 2 * sizeof(FrameSmall)));
    FramesShared sh;
    std::vector<std::thread> workers;
    for (int r = 0; r < n_devices && r < n_frames; ++r)
        workers.emplace_back(frames_worker, std::ref(sh), (int)devices[r], r, (int)n_devices, frames, (int)n_frames, out_norm,
                             out_rgba, stats, pinned + 2 * r);
    for (auto& w : workers) w.join();
    cudaFreeHost(pinned);
    if (sh.status != LYAP_OK) return fail(sh.status, sh.error);
    return LYAP_OK;
}

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
    cudaError_t e = lyap::launch_glow(static_cast<uint8_t*>(c->rgba.p), width, height, static_cast<double*>(c->norm.p), st);
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
