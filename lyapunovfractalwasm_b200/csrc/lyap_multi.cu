// lyap_multi.cu -- one frame, or a batch of frames, over several GPUs of one machine from ONE process.
//
// A lyap_multi object keeps, per listed device, an engine context, two streams, its device buffers and a pinned
// read-back record, and (optionally) one NCCL communicator per device (ncclCommInitAll).  Work is driven by one host
// thread per device for the length of a call.
//
// One frame (lyap_multi_render): the rows loop of the reference (src/lyapunov_fractal.hpp:41) is cut into contiguous
// bands; a band recomputes one halo row per inner side for the page's 3x3 mean (web/fractal_renderer.js:283-311).
// The only exchange the algorithm needs is normalizeData's whole-frame min/max (src/lyapunov_fractal.hpp:110-125):
// one all-reduce(MIN) over the pair (min, -max), on the device through NCCL, or through the host.  Optionally the
// finished RGBA8 bands (and the fp32 lambda bands) are gathered into the first device's own contiguous frame buffer:
// NCCL has no gather, so the other devices ncclSend their band and the first device posts the matching ncclRecvs as
// one group; the data crosses NVLink / NVSwitch once and lands in local memory.  No kernel of this library reads
// another GPU's memory.
//
// Nothing here can leave a GPU waiting on a peer that will not come: every collective is posted only after ALL
// workers have met at a host-side rendezvous with a deadline, so a missing or failed worker turns into
// LYAP_ERR_TIMEOUT / its own error before any NCCL kernel is enqueued.  After posting, completion is polled from the
// host (cudaStreamQuery + ncclCommGetAsyncError) against the same deadline; on expiry or an asynchronous NCCL error
// the communicators are aborted (ncclCommAbort), the object stops using NCCL and the call returns
// LYAP_ERR_TIMEOUT / LYAP_ERR_COMM.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>   // declarations only: the library itself is looked up at run time
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <condition_variable>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include "../../include/lyap_b200.h"
#include "lyap_engine.h"

namespace {

using Clock = std::chrono::steady_clock;

// ---- NCCL, found with dlopen so that the engine library loads (and single-device use works) without it ----
struct Nccl {
    void* lib = nullptr;
    decltype(&ncclCommInitAll) comm_init_all = nullptr;
    decltype(&ncclCommDestroy) comm_destroy = nullptr;
    decltype(&ncclCommAbort) comm_abort = nullptr;
    decltype(&ncclCommGetAsyncError) comm_async_error = nullptr;
    decltype(&ncclGroupStart) group_start = nullptr;
    decltype(&ncclGroupEnd) group_end = nullptr;
    decltype(&ncclAllReduce) all_reduce = nullptr;
    decltype(&ncclSend) send = nullptr;
    decltype(&ncclRecv) recv = nullptr;
    decltype(&ncclGetErrorString) error_string = nullptr;
    decltype(&ncclGetVersion) get_version = nullptr;
    bool ok = false;
};

Nccl& nccl() {
    static Nccl n = [] {
        Nccl r;
        const char* env = getenv("LYAP_NCCL_PATH");
        // a process that already holds an NCCL with this soname (for instance one that came with a framework) gets that one
        const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char* nm : names) {
            if (!nm || !*nm) continue;
            r.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
            if (r.lib) break;
        }
        if (!r.lib) return r;
#define LYAP_SYM(field, name) r.field = reinterpret_cast<decltype(r.field)>(dlsym(r.lib, name))
        LYAP_SYM(comm_init_all, "ncclCommInitAll");
        LYAP_SYM(comm_destroy, "ncclCommDestroy");
        LYAP_SYM(comm_abort, "ncclCommAbort");
        LYAP_SYM(comm_async_error, "ncclCommGetAsyncError");
        LYAP_SYM(group_start, "ncclGroupStart");
        LYAP_SYM(group_end, "ncclGroupEnd");
        LYAP_SYM(all_reduce, "ncclAllReduce");
        LYAP_SYM(send, "ncclSend");
        LYAP_SYM(recv, "ncclRecv");
        LYAP_SYM(error_string, "ncclGetErrorString");
        LYAP_SYM(get_version, "ncclGetVersion");
#undef LYAP_SYM
        r.ok = r.comm_init_all && r.comm_destroy && r.comm_abort && r.comm_async_error && r.group_start && r.group_end &&
               r.all_reduce && r.send && r.recv && r.error_string && r.get_version;
        return r;
    }();
    return n;
}

// (min, max) <-> (min, -max): one all-reduce with MIN then serves both
__global__ void k_pack_minmax(const double* __restrict__ mm, double* __restrict__ pair) {
    pair[0] = mm[0];
    pair[1] = -mm[1];
}
__global__ void k_unpack_minmax(const double* __restrict__ pair, double* __restrict__ mm) {
    mm[0] = pair[0];
    mm[1] = -pair[1];
}

struct Small {            // device record and its pinned mirror
    double mm[2];
    unsigned long long steps;
    unsigned long long pad;
    double pair[2];
};

struct Block {
    void* p = nullptr;
    size_t cap = 0;
};

struct FrameBuffers {    // one of a device's two buffer sets for frame batches
    Block block;
    Small* d_small = nullptr;
    cudaEvent_t begun = nullptr, lambda_done = nullptr, computed = nullptr, copied = nullptr;
    int frame = -1;
};

struct Slot {
    int device = -1;      // < 0: stands for a band whose worker never arrives (exercises the deadline on the host only)
    lyap_ctx* ctx = nullptr;
    cudaStream_t stream = nullptr, copy = nullptr;
    Block band;           // lambda (+ halo rows) | normalised | RGBA band | fp32 lambda band
    Small* d_small = nullptr;
    Small* h_small = nullptr;       // pinned: [0] band render, [1], [2] the two frame-buffer sets
    cudaEvent_t ev[6] = {};
    ncclComm_t comm = nullptr;
    FrameBuffers fb[2];
};

struct Rendezvous {
    std::mutex mu;
    std::condition_variable cv;
    int arrived[3] = {0, 0, 0};
    int expected = 0;
    bool failed = false;
    int status = LYAP_OK;
    std::string error;
    double lo = 0, hi = 0;
    bool have = false;
    unsigned long long steps = 0;
    float ms_lambda_max = 0, ms_device_max = 0;
};

void fail_all(Rendezvous& rv, int status, const std::string& msg) {
    std::lock_guard<std::mutex> lk(rv.mu);
    if (rv.status == LYAP_OK) {
        rv.status = status;
        rv.error = msg;
    }
    rv.failed = true;
    rv.cv.notify_all();
}

// All workers meet here before anything that needs every one of them.  False: someone failed or did not come in time.
bool meet(Rendezvous& rv, int which, Clock::time_point deadline, const char* what) {
    std::unique_lock<std::mutex> lk(rv.mu);
    ++rv.arrived[which];
    rv.cv.notify_all();
    const bool ok = rv.cv.wait_until(lk, deadline, [&] { return rv.arrived[which] == rv.expected || rv.failed; });
    if (!ok && rv.status == LYAP_OK) {
        rv.status = LYAP_ERR_TIMEOUT;
        rv.error = std::string("lyap_multi: ") + what + ": a band did not arrive before the deadline";
        rv.failed = true;
        rv.cv.notify_all();
    }
    return !rv.failed;
}

int grow(Block& b, size_t bytes) {
    if (b.cap >= bytes) return LYAP_OK;
    if (b.p) cudaFree(b.p);
    b.p = nullptr;
    b.cap = 0;
    const cudaError_t e = cudaMalloc(&b.p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return lyap::set_error(e == cudaErrorMemoryAllocation ? LYAP_ERR_NOMEM : LYAP_ERR_CUDA,
                               (std::string("device allocation of ") + std::to_string(bytes) + " bytes: " + cudaGetErrorString(e)).c_str());
    }
    b.cap = bytes;
    return LYAP_OK;
}

size_t round256(size_t v) { return (v + 255) / 256 * 256; }

}  // namespace

struct lyap_multi {
    std::vector<Slot> slots;
    bool want_nccl = false, nccl_ready = false, nccl_broken = false;
    std::string nccl_note;            // why NCCL is not in use ("" when it is)
    Block gathered_rgba, gathered_l32;   // on slots[0].device
    std::mutex call_mu;               // one call at a time per object
};

namespace {

#define MCU(call)                                                                                       \
    do {                                                                                                \
        cudaError_t e_ = (call);                                                                        \
        if (e_ != cudaSuccess)                                                                          \
            return lyap::set_error(LYAP_ERR_CUDA, (std::string(#call) + ": " + cudaGetErrorString(e_)).c_str()); \
    } while (0)

int slot_setup(Slot& s) {
    if (s.device < 0) return LYAP_OK;
    if (int rc = lyap_create(&s.ctx, s.device)) return rc;
    MCU(cudaSetDevice(s.device));
    MCU(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
    MCU(cudaStreamCreateWithFlags(&s.copy, cudaStreamNonBlocking));
    if (int rc = lyap_set_stream(s.ctx, s.stream)) return rc;
    MCU(cudaMalloc(reinterpret_cast<void**>(&s.d_small), 3 * sizeof(Small)));
    MCU(cudaMemset(s.d_small, 0, 3 * sizeof(Small)));
    MCU(cudaMallocHost(reinterpret_cast<void**>(&s.h_small), 3 * sizeof(Small)));
    for (auto& e : s.ev) MCU(cudaEventCreate(&e));
    for (int i = 0; i < 2; ++i) {
        s.fb[i].d_small = s.d_small + 1 + i;
        for (cudaEvent_t* e : {&s.fb[i].begun, &s.fb[i].lambda_done, &s.fb[i].computed, &s.fb[i].copied}) MCU(cudaEventCreate(e));
    }
    return LYAP_OK;
}

void slot_teardown(Slot& s) {
    if (s.device < 0) return;
    cudaSetDevice(s.device);
    if (s.stream) cudaStreamSynchronize(s.stream);
    if (s.copy) cudaStreamSynchronize(s.copy);
    if (s.band.p) cudaFree(s.band.p);
    for (auto& f : s.fb) {
        if (f.block.p) cudaFree(f.block.p);
        for (cudaEvent_t e : {f.begun, f.lambda_done, f.computed, f.copied})
            if (e) cudaEventDestroy(e);
    }
    if (s.d_small) cudaFree(s.d_small);
    if (s.h_small) cudaFreeHost(s.h_small);
    for (auto& e : s.ev)
        if (e) cudaEventDestroy(e);
    if (s.ctx) lyap_destroy(s.ctx);   // synchronises the stream it was given, so the streams go after it
    if (s.copy) cudaStreamDestroy(s.copy);
    if (s.stream) cudaStreamDestroy(s.stream);
    s = Slot{};
}

// Communicators for the listed devices (one process, one per device).  Not possible when a device is listed twice or
// a band is absent; then, and when the library is missing, the object works through the host and with plain copies.
void nccl_setup(lyap_multi* m) {
    if (m->nccl_ready || m->nccl_broken || !m->want_nccl) return;
    const int n = (int)m->slots.size();
    std::vector<int> devs(n);
    for (int i = 0; i < n; ++i) {
        devs[i] = m->slots[i].device;
        if (devs[i] < 0) { m->nccl_note = "a listed band has no device"; m->nccl_broken = true; return; }
        for (int j = 0; j < i; ++j)
            if (devs[j] == devs[i]) { m->nccl_note = "a device is listed more than once"; m->nccl_broken = true; return; }
    }
    Nccl& nc = nccl();
    if (!nc.ok) { m->nccl_note = "NCCL library (libnccl.so.2) not found"; m->nccl_broken = true; return; }
    std::vector<ncclComm_t> comms(n, nullptr);
    const ncclResult_t r = nc.comm_init_all(comms.data(), n, devs.data());
    if (r != ncclSuccess) {
        m->nccl_note = std::string("ncclCommInitAll: ") + nc.error_string(r);
        m->nccl_broken = true;
        return;
    }
    for (int i = 0; i < n; ++i) m->slots[i].comm = comms[i];
    m->nccl_ready = true;
}

void nccl_abort(lyap_multi* m, const char* why) {
    if (!m->nccl_ready) return;
    Nccl& nc = nccl();
    for (Slot& s : m->slots)
        if (s.comm) {
            nc.comm_abort(s.comm);
            s.comm = nullptr;
        }
    m->nccl_ready = false;
    m->nccl_broken = true;
    m->nccl_note = why;
}

// Waits on the host until everything enqueued on the slot's streams is done, polling so that a deadline and an
// asynchronous NCCL error can end the wait.  Never blocks inside the driver on work that may depend on a peer.
int wait_streams(lyap_multi* m, Slot& s, Clock::time_point deadline, bool watch_nccl, Rendezvous* rv = nullptr) {
    for (;;) {
        if (rv) {   // another band has failed: what this one waits for may depend on it, so stop waiting now
            std::lock_guard<std::mutex> lk(rv->mu);
            if (rv->failed) return lyap::set_error(rv->status, rv->error.c_str());
        }
        const cudaError_t a = cudaStreamQuery(s.stream), b = cudaStreamQuery(s.copy);
        if (a != cudaSuccess && a != cudaErrorNotReady)
            return lyap::set_error(LYAP_ERR_CUDA, (std::string("stream: ") + cudaGetErrorString(a)).c_str());
        if (b != cudaSuccess && b != cudaErrorNotReady)
            return lyap::set_error(LYAP_ERR_CUDA, (std::string("copy stream: ") + cudaGetErrorString(b)).c_str());
        if (a == cudaSuccess && b == cudaSuccess) return LYAP_OK;
        if (watch_nccl && s.comm) {
            ncclResult_t async = ncclSuccess;
            if (nccl().comm_async_error(s.comm, &async) == ncclSuccess && async != ncclSuccess && async != ncclInProgress)
                return lyap::set_error(LYAP_ERR_COMM, (std::string("NCCL reported: ") + nccl().error_string(async)).c_str());
        }
        if (Clock::now() > deadline)
            return lyap::set_error(LYAP_ERR_TIMEOUT, "lyap_multi: the device did not finish before the deadline");
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
}

struct BandCall {
    lyap_multi* m;
    const lyap_params* p;
    int flags;
    double* out_lambda;
    double* out_norm;
    uint8_t* out_rgba;
    float* out_l32;
    Clock::time_point deadline;
    Rendezvous rv;
    bool use_nccl = false;
    float ms_gather = 0;
    uint64_t gather_bytes = 0;
    int launches = 0;
    std::mutex stat_mu;
};

void band_rows(long long H, int n, int r, long long* b0, long long* b1) {
    const long long base = H / n, extra = H % n;
    *b0 = r * base + (r < extra ? r : extra);
    *b1 = *b0 + base + (r < extra ? 1 : 0);
}

void band_worker(BandCall& c, int r) {
    lyap_multi* m = c.m;
    Slot& s = m->slots[r];
    Rendezvous& rv = c.rv;
    auto bail = [&](int st) { fail_all(rv, st, lyap_last_error()); };
    auto bail_cuda = [&](cudaError_t e, const char* what) { fail_all(rv, LYAP_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e)); };
#define WCU(call)                                                \
    do {                                                         \
        cudaError_t e_ = (call);                                 \
        if (e_ != cudaSuccess) return bail_cuda(e_, #call);      \
    } while (0)
    const lyap_params& base = *c.p;
    const int n = (int)m->slots.size();
    const long long H = base.height, W = base.width;
    long long b0, b1;
    band_rows(H, n, r, &b0, &b1);
    const int above = b0 > 0 ? 1 : 0, below = b1 < H ? 1 : 0;
    const long long rows_own = b1 - b0, rows_all = rows_own + above + below;
    const bool gather_rgba = (c.flags & LYAP_MULTI_GATHER_RGBA) != 0, gather_l32 = (c.flags & LYAP_MULTI_GATHER_LAMBDA32) != 0;
    const bool want_rgba = c.out_rgba || gather_rgba, want_l32 = c.out_l32 || gather_l32;
    const bool colour = c.out_norm || want_rgba;
    WCU(cudaSetDevice(s.device));
    Slot& s0 = m->slots[0];

    // the band's buffers: lambda (with halo rows) | normalised | RGBA band | fp32 lambda band; the first device writes its
    // RGBA / fp32 bands straight into the gathered frame when there is one
    const size_t lam_bytes = round256((size_t)rows_all * W * 8), norm_bytes = colour ? lam_bytes : 0;
    const bool rgba_in_frame = gather_rgba && r == 0, l32_in_frame = gather_l32 && r == 0;
    const size_t rgba_bytes = (want_rgba && !rgba_in_frame) ? round256((size_t)rows_own * W * 4) : 0;
    const size_t l32_bytes = (want_l32 && !l32_in_frame) ? round256((size_t)rows_own * W * 4) : 0;
    if (int st = grow(s.band, lam_bytes + norm_bytes + rgba_bytes + l32_bytes)) return bail(st);
    if (r == 0 && gather_rgba)
        if (int st = grow(m->gathered_rgba, (size_t)H * W * 4)) return bail(st);
    if (r == 0 && gather_l32)
        if (int st = grow(m->gathered_l32, (size_t)H * W * 4)) return bail(st);
    char* blk = static_cast<char*>(s.band.p);
    double* d_lam = reinterpret_cast<double*>(blk);
    double* d_norm = colour ? reinterpret_cast<double*>(blk + lam_bytes) : nullptr;
    uint8_t* d_rgba = !want_rgba ? nullptr
                      : rgba_in_frame ? static_cast<uint8_t*>(m->gathered_rgba.p) + (size_t)b0 * W * 4
                                      : reinterpret_cast<uint8_t*>(blk + lam_bytes + norm_bytes);
    float* d_l32 = !want_l32 ? nullptr
                   : l32_in_frame ? static_cast<float*>(m->gathered_l32.p) + (size_t)b0 * W
                                  : reinterpret_cast<float*>(blk + lam_bytes + norm_bytes + rgba_bytes);
    double* own = d_lam + (size_t)above * W;
    double* d_mm = s.d_small->mm;
    uint64_t* d_steps = reinterpret_cast<uint64_t*>(&s.d_small->steps);
    cudaStream_t st = s.stream;
    int launches = 0;

    WCU(cudaMemsetAsync(d_steps, 0, 8, st));
    WCU(cudaEventRecord(s.ev[0], st));
    {   // the band's own rows (counted), then the halo rows (same kernel, not counted)
        lyap_params p = base;
        p.row_begin = b0;
        p.row_end = b1;
        int rc = lyap_lambda_device(s.ctx, &p, own, d_l32, d_steps);
        ++launches;
        if (rc == LYAP_OK && colour && above) {
            p.row_begin = b0 - 1;
            p.row_end = b0;
            rc = lyap_lambda_device(s.ctx, &p, d_lam, nullptr, nullptr);
            ++launches;
        }
        if (rc == LYAP_OK && colour && below) {
            p.row_begin = b1;
            p.row_end = b1 + 1;
            rc = lyap_lambda_device(s.ctx, &p, own + (size_t)rows_own * W, nullptr, nullptr);
            ++launches;
        }
        if (rc != LYAP_OK) return bail(rc);
    }
    WCU(cudaEventRecord(s.ev[1], st));
    if (colour) {
        if (int rc = lyap_minmax_device(s.ctx, own, (uint64_t)rows_own * W, d_mm)) return bail(rc);
        ++launches;
        if (c.use_nccl) {
            k_pack_minmax<<<1, 1, 0, st>>>(d_mm, s.d_small->pair);
            WCU(cudaGetLastError());
            ++launches;
        } else {
            WCU(cudaMemcpyAsync(s.h_small, s.d_small, sizeof(Small), cudaMemcpyDeviceToHost, st));
            WCU(cudaStreamSynchronize(st));   // own kernels only: nothing on this stream depends on a peer yet
            std::lock_guard<std::mutex> lk(rv.mu);
            rv.lo = rv.have ? std::fmin(rv.lo, s.h_small->mm[0]) : s.h_small->mm[0];
            rv.hi = rv.have ? std::fmax(rv.hi, s.h_small->mm[1]) : s.h_small->mm[1];
            rv.have = true;
        }
    }
    // ---- every band is enqueued (or its min/max is in): from here on steps may need all of them ----
    if (!meet(rv, 0, c.deadline, "min/max exchange")) return;
    if (colour) {
        if (c.use_nccl) {
            const ncclResult_t nr = nccl().all_reduce(s.d_small->pair, s.d_small->pair, 2, ncclFloat64, ncclMin, s.comm, st);
            if (nr != ncclSuccess) return fail_all(rv, LYAP_ERR_COMM, std::string("ncclAllReduce: ") + nccl().error_string(nr));
            k_unpack_minmax<<<1, 1, 0, st>>>(s.d_small->pair, d_mm);
            WCU(cudaGetLastError());
            launches += 2;
        } else {
            double mm[2];
            {
                std::lock_guard<std::mutex> lk(rv.mu);
                mm[0] = rv.lo;
                mm[1] = rv.hi;
            }
            s.h_small->pair[0] = mm[0];
            s.h_small->pair[1] = mm[1];
            WCU(cudaMemcpyAsync(d_mm, s.h_small->pair, 16, cudaMemcpyHostToDevice, st));
        }
        if (int rc = lyap_normalize_device(s.ctx, d_lam, (uint64_t)rows_all * W, d_mm, d_norm)) return bail(rc);
        ++launches;
        if (want_rgba) {
            if (int rc = lyap_colorize_device(s.ctx, d_norm + (size_t)above * W, base.width, rows_own, above, below, base.palette, d_rgba))
                return bail(rc);
            ++launches;
        }
    }
    WCU(cudaEventRecord(s.ev[2], st));
    // the band's outputs to the host, behind the kernels, on the copy stream
    WCU(cudaStreamWaitEvent(s.copy, s.ev[2], 0));
    if (c.out_lambda) WCU(cudaMemcpyAsync(c.out_lambda + (size_t)b0 * W, own, (size_t)rows_own * W * 8, cudaMemcpyDeviceToHost, s.copy));
    if (c.out_norm) WCU(cudaMemcpyAsync(c.out_norm + (size_t)b0 * W, d_norm + (size_t)above * W, (size_t)rows_own * W * 8, cudaMemcpyDeviceToHost, s.copy));
    if (c.out_rgba && !gather_rgba) WCU(cudaMemcpyAsync(c.out_rgba + (size_t)b0 * W * 4, d_rgba, (size_t)rows_own * W * 4, cudaMemcpyDeviceToHost, s.copy));
    if (c.out_l32 && !gather_l32) WCU(cudaMemcpyAsync(c.out_l32 + (size_t)b0 * W, d_l32, (size_t)rows_own * W * 4, cudaMemcpyDeviceToHost, s.copy));
    WCU(cudaMemcpyAsync(s.h_small, s.d_small, sizeof(Small), cudaMemcpyDeviceToHost, s.copy));

    // ---- optional gather of the finished bands into the first device's frame ----
    if ((gather_rgba || gather_l32) && n > 1) {
        // The gather is posted only once every band is known to be finished and healthy: a send never waits on a device
        // that is still computing (so the gather's time is its own) and never on one that failed.
        if (int rc = wait_streams(m, s, c.deadline, c.use_nccl, &rv)) return bail(rc);
        if (!meet(rv, 1, c.deadline, "gather")) return;
        const size_t band_px = (size_t)rows_own * W;
        nvtxRangePushA("lyap: gather to the first device");
        struct Pop { ~Pop() { nvtxRangePop(); } } pop_range;
        if (c.use_nccl) {
            Nccl& nc = nccl();
            ncclResult_t nr = ncclSuccess;
            if (r == 0) {
                WCU(cudaEventRecord(s.ev[3], st));
                nr = nc.group_start();
                for (int q = 1; q < n && nr == ncclSuccess; ++q) {
                    long long q0, q1;
                    band_rows(H, n, q, &q0, &q1);
                    const size_t qpx = (size_t)(q1 - q0) * W;
                    if (gather_rgba) nr = nc.recv(static_cast<uint8_t*>(m->gathered_rgba.p) + (size_t)q0 * W * 4, qpx * 4, ncclUint8, q, s.comm, st);
                    if (gather_l32 && nr == ncclSuccess) nr = nc.recv(static_cast<float*>(m->gathered_l32.p) + (size_t)q0 * W, qpx, ncclFloat32, q, s.comm, st);
                }
                const ncclResult_t ge = nc.group_end();
                if (nr == ncclSuccess) nr = ge;
                WCU(cudaEventRecord(s.ev[4], st));
            } else {
                nr = nc.group_start();
                if (gather_rgba && nr == ncclSuccess) nr = nc.send(d_rgba, band_px * 4, ncclUint8, 0, s.comm, st);
                if (gather_l32 && nr == ncclSuccess) nr = nc.send(d_l32, band_px, ncclFloat32, 0, s.comm, st);
                const ncclResult_t ge = nc.group_end();
                if (nr == ncclSuccess) nr = ge;
            }
            if (nr != ncclSuccess) return fail_all(rv, LYAP_ERR_COMM, std::string("NCCL send/recv: ") + nc.error_string(nr));
        } else {
            // plain peer copies into the first device's frame, each on the sending device's stream; the first device's
            // stream then waits for all of them
            if (r == 0) WCU(cudaEventRecord(s.ev[3], st));
            if (r > 0) {
                if (gather_rgba)
                    WCU(cudaMemcpyPeerAsync(static_cast<uint8_t*>(m->gathered_rgba.p) + (size_t)b0 * W * 4, s0.device, d_rgba, s.device, band_px * 4, st));
                if (gather_l32)
                    WCU(cudaMemcpyPeerAsync(static_cast<float*>(m->gathered_l32.p) + (size_t)b0 * W, s0.device, d_l32, s.device, band_px * 4, st));
                WCU(cudaEventRecord(s.ev[5], st));
            }
            if (!meet(rv, 2, c.deadline, "gather copies")) return;   // the senders' events are recorded
            if (r == 0) {
                for (int q = 1; q < n; ++q) WCU(cudaStreamWaitEvent(st, m->slots[q].ev[5], 0));
                WCU(cudaEventRecord(s.ev[4], st));
            }
        }
        if (r == 0) {
            std::lock_guard<std::mutex> lk(c.stat_mu);
            c.gather_bytes = (gather_rgba ? (size_t)(H - rows_own) * W * 4 : 0) + (gather_l32 ? (size_t)(H - rows_own) * W * 4 : 0);
        }
    }
    if (r == 0) {   // the gathered frame to the host, when the caller gave host buffers for it
        if (gather_rgba && c.out_rgba) WCU(cudaMemcpyAsync(c.out_rgba, m->gathered_rgba.p, (size_t)H * W * 4, cudaMemcpyDeviceToHost, st));
        if (gather_l32 && c.out_l32) WCU(cudaMemcpyAsync(c.out_l32, m->gathered_l32.p, (size_t)H * W * 4, cudaMemcpyDeviceToHost, st));
    }
    if (int rc = wait_streams(m, s, c.deadline, c.use_nccl, &rv)) return bail(rc);
    {
        float ms_l = 0, ms_d = 0, ms_g = 0;
        cudaEventElapsedTime(&ms_l, s.ev[0], s.ev[1]);
        cudaEventElapsedTime(&ms_d, s.ev[0], s.ev[2]);
        if (r == 0 && (gather_rgba || gather_l32) && n > 1) cudaEventElapsedTime(&ms_g, s.ev[3], s.ev[4]);
        std::lock_guard<std::mutex> lk(rv.mu);
        rv.steps += s.h_small->steps;
        rv.ms_lambda_max = std::max(rv.ms_lambda_max, ms_l);
        rv.ms_device_max = std::max(rv.ms_device_max, ms_d);
        if (colour && r == 0) {   // after the exchange every device holds the frame's min/max
            rv.lo = s.h_small->mm[0];
            rv.hi = s.h_small->mm[1];
        }
        std::lock_guard<std::mutex> lk2(c.stat_mu);
        if (r == 0) c.ms_gather = ms_g;
        c.launches += launches;
    }
#undef WCU
}

}  // namespace

extern "C" {

int lyap_multi_create(lyap_multi** out, int32_t n_devices, const int32_t* devices, int32_t use_nccl) {
    if (!out) return lyap::set_error(LYAP_ERR_INVALID, "lyap_multi_create: null output");
    *out = nullptr;
    if (n_devices < 1 || !devices) return lyap::set_error(LYAP_ERR_INVALID, "need at least one device");
    int present = 0;
    MCU(cudaGetDeviceCount(&present));
    for (int i = 0; i < n_devices; ++i)
        if (devices[i] >= present) return lyap::set_error(LYAP_ERR_INVALID, "no such device");
    lyap_multi* m = new (std::nothrow) lyap_multi;
    if (!m) return lyap::set_error(LYAP_ERR_NOMEM, "host allocation failed");
    m->slots.resize(n_devices);
    m->want_nccl = use_nccl != 0;
    {   // contexts, streams, pinned records: one thread per device (done one after the other this takes ~10 ms per device)
        std::vector<int> rc(n_devices, LYAP_OK);
        std::vector<std::string> msg(n_devices);
        std::vector<std::thread> setup;
        for (int i = 0; i < n_devices; ++i) {
            m->slots[i].device = devices[i];
            setup.emplace_back([m, i, &rc, &msg] {
                rc[i] = slot_setup(m->slots[i]);
                if (rc[i] != LYAP_OK) msg[i] = lyap_last_error();   // the message is per thread: carry it over
            });
        }
        for (auto& t : setup) t.join();
        for (int i = 0; i < n_devices; ++i)
            if (rc[i] != LYAP_OK) {
                lyap_multi_destroy(m);
                return lyap::set_error(rc[i], msg[i].c_str());
            }
    }
    nccl_setup(m);   // a failure here is not fatal: the object then works through the host (see lyap_multi_note)
    if (m->slots[0].device >= 0) {
        // a gather without NCCL uses peer copies into the first device: let them go over NVLink instead of through the host
        for (int i = 1; i < n_devices; ++i) {
            const int d = m->slots[i].device;
            int can = 0;
            if (d < 0 || d == m->slots[0].device) continue;
            if (cudaDeviceCanAccessPeer(&can, d, m->slots[0].device) == cudaSuccess && can && cudaSetDevice(d) == cudaSuccess) {
                const cudaError_t pe = cudaDeviceEnablePeerAccess(m->slots[0].device, 0);
                if (pe != cudaSuccess) cudaGetLastError();   // already enabled, or not possible: the copy still works
            }
        }
    }
    *out = m;
    return LYAP_OK;
}

int lyap_multi_destroy(lyap_multi* m) {
    if (!m) return LYAP_OK;
    for (Slot& s : m->slots) {   // let every stream drain before a communicator goes away
        if (s.device < 0) continue;
        cudaSetDevice(s.device);
        if (s.stream) cudaStreamSynchronize(s.stream);
        if (s.copy) cudaStreamSynchronize(s.copy);
    }
    if (m->nccl_ready)
        for (Slot& s : m->slots)
            if (s.comm) {
                nccl().comm_destroy(s.comm);
                s.comm = nullptr;
            }
    if (!m->slots.empty() && m->slots[0].device >= 0) {
        cudaSetDevice(m->slots[0].device);
        if (m->gathered_rgba.p) cudaFree(m->gathered_rgba.p);
        if (m->gathered_l32.p) cudaFree(m->gathered_l32.p);
    }
    for (Slot& s : m->slots) slot_teardown(s);
    delete m;
    return LYAP_OK;
}

const char* lyap_multi_note(lyap_multi* m) {
    thread_local std::string copy;
    copy = m ? m->nccl_note : std::string("null object");
    return copy.c_str();
}

int lyap_multi_render(lyap_multi* m, const lyap_params* p, int32_t flags, double* out_lambda, float* out_lambda32,
                      double* out_norm, uint8_t* out_rgba, double timeout_seconds, lyap_multi_stats* stats) {
    if (!m) return lyap::set_error(LYAP_ERR_INVALID, "lyap_multi_render: null object");
    if (int rc = lyap::validate_whole_frame(p)) return rc;
    const int n = (int)m->slots.size();
    if (n > p->height) return lyap::set_error(LYAP_ERR_INVALID, "more bands than rows");
    if (timeout_seconds <= 0) {
        // default: a minute, plus the frame's work at a tenth of one device's real rate spread over the devices (the
        // deadline covers the kernels too, so it has to grow with the frame)
        const double steps = (double)p->width * (double)p->height * ((double)p->warmup + (double)p->iterations);
        timeout_seconds = 60.0 + steps / (1e11 * n);
    }
    std::lock_guard<std::mutex> call_lock(m->call_mu);
    const auto t0 = Clock::now();
    BandCall c;
    c.m = m;
    c.p = p;
    c.flags = flags;
    c.out_lambda = out_lambda;
    c.out_l32 = out_lambda32;
    c.out_norm = out_norm;
    c.out_rgba = out_rgba;
    c.deadline = t0 + std::chrono::duration_cast<Clock::duration>(std::chrono::duration<double>(timeout_seconds));
    c.rv.expected = n;
    c.use_nccl = m->nccl_ready && !(flags & LYAP_MULTI_HOST_EXCHANGE);
    std::vector<std::thread> workers;
    for (int r = 0; r < n; ++r) {
        if (m->slots[r].device < 0) continue;   // a band whose worker never arrives
        workers.emplace_back(band_worker, std::ref(c), r);
    }
    for (auto& w : workers) w.join();
    if (workers.empty()) return lyap::set_error(LYAP_ERR_TIMEOUT, "lyap_multi_render: no band arrived");
    if (c.rv.status != LYAP_OK) {
        // once every band had passed the first rendezvous, collectives may have been posted that a failed band will never
        // join: abort them before waiting for the streams below
        if (c.use_nccl && c.rv.arrived[0] == n) nccl_abort(m, "aborted after a failed or overdue call");
        for (Slot& s : m->slots) {   // whatever was enqueued must be off the buffers before the next call
            if (s.device < 0) continue;
            cudaSetDevice(s.device);
            cudaStreamSynchronize(s.stream);
            cudaStreamSynchronize(s.copy);
        }
        return lyap::set_error(c.rv.status, c.rv.error.c_str());
    }
    if (stats) {
        std::memset(stats, 0, sizeof(*stats));
        stats->executed_steps = c.rv.steps;
        stats->nominal_steps = (uint64_t)p->width * (uint64_t)p->height * (uint64_t)((long long)p->warmup + p->iterations);
        const bool colour = out_norm || out_rgba || (flags & LYAP_MULTI_GATHER_RGBA);
        stats->lambda_min = colour ? c.rv.lo : NAN;
        stats->lambda_max = colour ? c.rv.hi : NAN;
        stats->ms_wall = std::chrono::duration<float, std::milli>(Clock::now() - t0).count();
        stats->ms_lambda_max = c.rv.ms_lambda_max;
        stats->ms_device_max = c.rv.ms_device_max;
        stats->ms_gather = c.ms_gather;
        stats->gather_bytes = c.gather_bytes;
        stats->kernel_launches = c.launches;
        stats->used_nccl = c.use_nccl ? 1 : 0;
    }
    return LYAP_OK;
}

int lyap_multi_gathered(lyap_multi* m, uint8_t** d_rgba, float** d_lambda32) {
    if (!m) return lyap::set_error(LYAP_ERR_INVALID, "null object");
    if (d_rgba) *d_rgba = static_cast<uint8_t*>(m->gathered_rgba.p);
    if (d_lambda32) *d_lambda32 = static_cast<float*>(m->gathered_l32.p);
    return LYAP_OK;
}

}  // extern "C"

// ---- a batch of independent frames (a zoom sequence) ----

namespace {

struct FramesCall {
    lyap_multi* m;
    const lyap_params* frames;
    int n_frames;
    double* const* out_norm;
    uint8_t* const* out_rgba;
    lyap_render_stats* stats;
    std::mutex mu;
    bool failed = false;
    int status = LYAP_OK;
    std::string error;
};

void frames_fail(FramesCall& c, int status, const std::string& msg) {
    std::lock_guard<std::mutex> lk(c.mu);
    if (c.status == LYAP_OK) {
        c.status = status;
        c.error = msg;
    }
    c.failed = true;
}

// Frames r, r + stride, ... on one device: kernels in order on the slot's stream, copies on its copy stream behind an
// event, two buffer sets, so one frame's copies run while the next frame is computed.
void frames_worker(FramesCall& c, int r) {
    lyap_multi* m = c.m;
    Slot& s = m->slots[r];
    const int stride = (int)m->slots.size();
    auto bail_cuda = [&](cudaError_t e, const char* what) { frames_fail(c, LYAP_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e)); };
#define FR(call)                                                  \
    do {                                                          \
        cudaError_t fr_e = (call);                                \
        if (fr_e != cudaSuccess) return bail_cuda(fr_e, #call);   \
    } while (0)
    FR(cudaSetDevice(s.device));
    size_t max_px = 0;
    bool any_rgba = false;
    for (int k = r; k < c.n_frames; k += stride) {
        max_px = std::max(max_px, (size_t)c.frames[k].width * (size_t)c.frames[k].height);
        any_rgba = any_rgba || (c.out_rgba && c.out_rgba[k]);
    }
    const size_t px8 = round256(max_px * 8), px4 = any_rgba ? round256(max_px * 4) : 0;
    for (FrameBuffers& f : s.fb) {
        if (grow(f.block, 2 * px8 + px4) != LYAP_OK) return frames_fail(c, LYAP_ERR_NOMEM, lyap_last_error());
        f.frame = -1;
    }
    auto finish = [&](FrameBuffers& f, int which) -> cudaError_t {   // the set's frame has reached the host: its statistics
        if (f.frame < 0) return cudaSuccess;
        const cudaError_t e = cudaEventSynchronize(f.copied);
        if (e != cudaSuccess) return e;
        if (c.stats) {
            const lyap_params& p = c.frames[f.frame];
            lyap_render_stats& o = c.stats[f.frame];
            const Small& h = s.h_small[1 + which];
            std::memset(&o, 0, sizeof(o));
            o.executed_steps = h.steps;
            o.nominal_steps = (uint64_t)p.width * (uint64_t)p.height * (uint64_t)((long long)p.warmup + p.iterations);
            o.lambda_min = h.mm[0];
            o.lambda_max = h.mm[1];
            cudaEventElapsedTime(&o.ms_lambda, f.begun, f.lambda_done);
            cudaEventElapsedTime(&o.ms_total_device, f.begun, f.computed);
            cudaEventElapsedTime(&o.ms_copies, f.computed, f.copied);
            o.kernel_launches = (c.out_rgba && c.out_rgba[f.frame]) ? 4 : 3;
        }
        f.frame = -1;
        return cudaSuccess;
    };
    int local = 0;
    for (int k = r; k < c.n_frames; k += stride, ++local) {
        {
            std::lock_guard<std::mutex> lk(c.mu);
            if (c.failed) break;
        }
        const int which = local & 1;
        FrameBuffers& f = s.fb[which];
        FR(finish(f, which));   // its buffers are free again
        const lyap_params& p = c.frames[k];
        const size_t n = (size_t)p.width * (size_t)p.height;
        char* base = static_cast<char*>(f.block.p);
        double* d_lam = reinterpret_cast<double*>(base);
        double* d_norm = reinterpret_cast<double*>(base + px8);
        uint8_t* d_rgba = any_rgba ? reinterpret_cast<uint8_t*>(base + 2 * px8) : nullptr;
        double* d_mm = f.d_small->mm;
        uint64_t* d_steps = reinterpret_cast<uint64_t*>(&f.d_small->steps);
        cudaStream_t st = s.stream;
        FR(cudaMemsetAsync(d_steps, 0, 8, st));
        FR(cudaEventRecord(f.begun, st));
        int rc = lyap_lambda_device(s.ctx, &p, d_lam, nullptr, d_steps);
        if (rc == LYAP_OK) {
            FR(cudaEventRecord(f.lambda_done, st));
            rc = lyap_minmax_device(s.ctx, d_lam, n, d_mm);
        }
        if (rc == LYAP_OK) rc = lyap_normalize_device(s.ctx, d_lam, n, d_mm, d_norm);
        uint8_t* h_rgba = c.out_rgba ? c.out_rgba[k] : nullptr;
        double* h_norm = c.out_norm ? c.out_norm[k] : nullptr;
        if (rc == LYAP_OK && h_rgba) rc = lyap_colorize_device(s.ctx, d_norm, p.width, p.height, 0, 0, p.palette, d_rgba);
        if (rc != LYAP_OK) return frames_fail(c, rc, lyap_last_error());
        FR(cudaEventRecord(f.computed, st));
        FR(cudaStreamWaitEvent(s.copy, f.computed, 0));
        if (h_norm) FR(cudaMemcpyAsync(h_norm, d_norm, n * 8, cudaMemcpyDeviceToHost, s.copy));
        if (h_rgba) FR(cudaMemcpyAsync(h_rgba, d_rgba, n * 4, cudaMemcpyDeviceToHost, s.copy));
        FR(cudaMemcpyAsync(&s.h_small[1 + which], f.d_small, sizeof(Small), cudaMemcpyDeviceToHost, s.copy));
        FR(cudaEventRecord(f.copied, s.copy));
        f.frame = k;
    }
    for (int i = 0; i < 2; ++i) FR(finish(s.fb[i], i));
#undef FR
}

}  // namespace

extern "C" {

int lyap_multi_render_frames(lyap_multi* m, const lyap_params* frames, int32_t n_frames, double* const* out_norm,
                             uint8_t* const* out_rgba, lyap_render_stats* stats) {
    if (!m) return lyap::set_error(LYAP_ERR_INVALID, "lyap_multi_render_frames: null object");
    if (n_frames < 0 || (n_frames > 0 && !frames)) return lyap::set_error(LYAP_ERR_INVALID, "lyap_multi_render_frames: bad frame list");
    for (int k = 0; k < n_frames; ++k)
        if (int rc = lyap::validate_whole_frame(&frames[k])) return rc;
    if (n_frames == 0) return LYAP_OK;
    for (const Slot& s : m->slots)
        if (s.device < 0) return lyap::set_error(LYAP_ERR_INVALID, "a listed device is absent");
    std::lock_guard<std::mutex> call_lock(m->call_mu);
    FramesCall c;
    c.m = m;
    c.frames = frames;
    c.n_frames = n_frames;
    c.out_norm = out_norm;
    c.out_rgba = out_rgba;
    c.stats = stats;
    std::vector<std::thread> workers;
    for (int r = 0; r < (int)m->slots.size() && r < n_frames; ++r) workers.emplace_back(frames_worker, std::ref(c), r);
    for (auto& w : workers) w.join();
    if (c.status != LYAP_OK) {
        for (Slot& s : m->slots) {
            cudaSetDevice(s.device);
            cudaStreamSynchronize(s.stream);
            cudaStreamSynchronize(s.copy);
        }
        return lyap::set_error(c.status, c.error.c_str());
    }
    return LYAP_OK;
}

// ---- the one-call forms: a temporary object around a single call ----

int lyap_render_multi(const lyap_params* p, int32_t n_devices, const int32_t* devices, double* out_lambda,
                      double* out_norm, uint8_t* out_rgba, double timeout_seconds, lyap_render_stats* stats) {
    if (int rc = lyap::validate_whole_frame(p)) return rc;
    if (n_devices < 1 || !devices) return lyap::set_error(LYAP_ERR_INVALID, "need at least one device");
    if (n_devices > p->height) return lyap::set_error(LYAP_ERR_INVALID, "more bands than rows");
    lyap_multi* m = nullptr;
    if (int rc = lyap_multi_create(&m, n_devices, devices, 0)) return rc;
    lyap_multi_stats ms;
    const int rc = lyap_multi_render(m, p, LYAP_MULTI_HOST_EXCHANGE, out_lambda, nullptr, out_norm, out_rgba, timeout_seconds, &ms);
    const std::string msg = rc != LYAP_OK ? lyap_last_error() : "";
    lyap_multi_destroy(m);
    if (rc != LYAP_OK) return lyap::set_error(rc, msg.c_str());
    if (stats) {
        std::memset(stats, 0, sizeof(*stats));
        stats->executed_steps = ms.executed_steps;
        stats->nominal_steps = ms.nominal_steps;
        stats->lambda_min = ms.lambda_min;
        stats->lambda_max = ms.lambda_max;
        stats->ms_lambda = ms.ms_lambda_max;
        stats->ms_total_device = ms.ms_wall;   // wall clock of the render itself (set-up of the temporary object excluded)
        stats->kernel_launches = ms.kernel_launches;
    }
    return LYAP_OK;
}

int lyap_render_frames(const lyap_params* frames, int32_t n_frames, int32_t n_devices, const int32_t* devices,
                       double* const* out_norm, uint8_t* const* out_rgba, lyap_render_stats* stats) {
    if (n_frames < 0 || (n_frames > 0 && !frames)) return lyap::set_error(LYAP_ERR_INVALID, "lyap_render_frames: bad frame list");
    if (n_devices < 1 || !devices) return lyap::set_error(LYAP_ERR_INVALID, "need at least one device");
    for (int k = 0; k < n_frames; ++k)
        if (int rc = lyap::validate_whole_frame(&frames[k])) return rc;
    if (n_frames == 0) return LYAP_OK;
    lyap_multi* m = nullptr;
    if (int rc = lyap_multi_create(&m, n_devices, devices, 0)) return rc;
    const int rc = lyap_multi_render_frames(m, frames, n_frames, out_norm, out_rgba, stats);
    const std::string msg = rc != LYAP_OK ? lyap_last_error() : "";
    lyap_multi_destroy(m);
    if (rc != LYAP_OK) return lyap::set_error(rc, msg.c_str());
    return LYAP_OK;
}

}  // extern "C"
