// lyap_jit.cu -- run-time specialisation of the exact lambda kernel for one sequence.
//
// The library's precompiled kernel picks, every two steps, the straight-line body that matches the next A/B(/C)
// pattern (one warp-uniform multiway branch).  For a periodic sequence that choice is known in advance, so this
// file compiles, once per (device, sequence patterns), an instance of the SAME kernel source
// (lyap_exact_kernel.cuh, embedded as text at build time) in which a whole period is one straight-line block.
// NVRTC does the compilation (found with dlopen: no link-time dependency); the driver entry points for loading and
// launching come from cudaGetDriverEntryPoint.  Everything here is optional: if any step fails, the caller falls
// back to the precompiled kernel, which computes the same bits.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nvrtc.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <thread>
#include <tuple>
#include <vector>

#include "lyap_engine.h"
#include "lyap_jit_source.inc"   // generated: kSrc_lyap_exact_kernel_cuh, kSrc_lyap_kernels_fast_cuh, kSrc_lyap_args_h, ...

namespace lyap {

namespace {

struct Nvrtc {
    void* lib = nullptr;
    decltype(&nvrtcCreateProgram) create = nullptr;
    decltype(&nvrtcCompileProgram) compile = nullptr;
    decltype(&nvrtcGetCUBINSize) cubin_size = nullptr;
    decltype(&nvrtcGetCUBIN) cubin = nullptr;
    decltype(&nvrtcGetProgramLogSize) log_size = nullptr;
    decltype(&nvrtcGetProgramLog) log = nullptr;
    decltype(&nvrtcDestroyProgram) destroy = nullptr;
    bool ok = false;
};

struct Driver {
    CUresult (*module_load_data)(CUmodule*, const void*) = nullptr;
    CUresult (*module_unload)(CUmodule) = nullptr;
    CUresult (*module_get_function)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*func_set_attribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*launch_kernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                              void**, void**) = nullptr;
    bool ok = false;
};

// Process-wide state lives in objects that are never destroyed: a background compilation may still be running when the
// process leaves main, and must not find them gone.
std::mutex& g_mu = *new std::mutex;
std::string& g_note = *new std::string;   // last reason a specialised kernel could not be used

Nvrtc& nvrtc() {
    static Nvrtc n = [] {
        Nvrtc r;
        const char* env = getenv("LYAP_NVRTC_PATH");
        const char* names[] = {env, "libnvrtc.so.12", "/usr/local/cuda/lib64/libnvrtc.so.12", "libnvrtc.so"};
        for (const char* nm : names) {
            if (!nm || !*nm) continue;
            r.lib = dlopen(nm, RTLD_NOW | RTLD_LOCAL);
            if (r.lib) break;
        }
        if (!r.lib) return r;
#define LYAP_SYM(field, name) r.field = reinterpret_cast<decltype(r.field)>(dlsym(r.lib, name))
        LYAP_SYM(create, "nvrtcCreateProgram");
        LYAP_SYM(compile, "nvrtcCompileProgram");
        LYAP_SYM(cubin_size, "nvrtcGetCUBINSize");
        LYAP_SYM(cubin, "nvrtcGetCUBIN");
        LYAP_SYM(log_size, "nvrtcGetProgramLogSize");
        LYAP_SYM(log, "nvrtcGetProgramLog");
        LYAP_SYM(destroy, "nvrtcDestroyProgram");
#undef LYAP_SYM
        r.ok = r.create && r.compile && r.cubin_size && r.cubin && r.log_size && r.log && r.destroy;
        return r;
    }();
    return n;
}

Driver& driver() {
    static Driver d = [] {
        Driver r;
        auto get = [](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult st;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &st) == cudaSuccess &&
                   st == cudaDriverEntryPointSuccess && *fn;
        };
        r.ok = get("cuModuleLoadData", reinterpret_cast<void**>(&r.module_load_data)) &&
               get("cuModuleUnload", reinterpret_cast<void**>(&r.module_unload)) &&
               get("cuModuleGetFunction", reinterpret_cast<void**>(&r.module_get_function)) &&
               get("cuFuncSetAttribute", reinterpret_cast<void**>(&r.func_set_attribute)) &&
               get("cuLaunchKernel", reinterpret_cast<void**>(&r.launch_kernel));
        return r;
    }();
    return d;
}

// device, P, KG, warm-up pats, acc pats, kind, threads, origin (0: compiled at run time, 1: embedded at build time)
using Key = std::tuple<int, int, int, unsigned long long, unsigned long long, int, int, int>;

struct Entry {
    CUfunction fn = nullptr;
    bool failed = false;
    double work_seen = 0;   // nominal steps asked for so far with this key (decides when compiling pays off)
};

std::map<Key, Entry>& g_cache = *new std::map<Key, Entry>;
// compiled code does not depend on the device ordinal: one compilation serves every GPU of the process
using CodeKey = std::tuple<int, int, unsigned long long, unsigned long long, int, int, int>;   // Key without the device
std::map<CodeKey, std::vector<char>>& g_cubins = *new std::map<CodeKey, std::vector<char>>;
// run-time compilations handed to a background thread: 1 = running, 2 = failed (a finished one is in g_cubins)
std::map<CodeKey, int>& g_background = *new std::map<CodeKey, int>;

// NVRTC: source text + pattern macros -> cubin for sm_100a.
bool compile_cubin(const Key& key, std::vector<char>* out, std::string* note) {
    Nvrtc& n = nvrtc();
    const int kind = std::get<5>(key);
    std::vector<char>& cubin = *out;
    if (!n.ok) { *note = "NVRTC library not found"; return false; }
    char o_p[64], o_kg[64], o_wu[96], o_acc[96], o_thr[64];
    snprintf(o_thr, sizeof o_thr, "-DLYAP_SPEC_THREADS=%d", std::get<6>(key));
    // the exact instance is compiled when LYAP_SPEC_EXACT is defined; a fast one when LYAP_SPEC_FAST names its flavour
    static const char* const kind_opts[4] = {"-DLYAP_SPEC_EXACT=1", "-DLYAP_SPEC_FAST=FusedF64", "-DLYAP_SPEC_FAST=FusedF32",
                                             "-DLYAP_SPEC_FAST=OrbitF64"};
    const char* o_kind = kind_opts[kind];
    snprintf(o_p, sizeof o_p, "-DLYAP_SPEC_P=%d", std::get<1>(key));
    snprintf(o_kg, sizeof o_kg, "-DLYAP_SPEC_KG=%d", std::get<2>(key));
    snprintf(o_wu, sizeof o_wu, "-DLYAP_SPEC_WU_PATS=0x%llxull", std::get<3>(key));
    snprintf(o_acc, sizeof o_acc, "-DLYAP_SPEC_ACC_PATS=0x%llxull", std::get<4>(key));
    // build.py compiles the embedded instances with exactly these options (keep the two lists the same)
    const char* opts[] = {"--gpu-architecture=sm_100a", "--fmad=false", "--std=c++17", "-lineinfo", o_thr, o_kind,
                          o_p, o_kg, o_wu, o_acc};
    const char* header_src[] = {kSrc_lyap_exact_kernel_cuh, kSrc_lyap_kernels_fast_cuh, kSrc_lyap_args_h, kSrc_lyap_math_h,
                                kSrc_lyap_tables_h};
    const char* header_names[] = {"lyap_exact_kernel.cuh", "lyap_kernels_fast.cuh", "lyap_args.h", "lyap_math.h", "lyap_tables.h"};
    static const char kMain[] = "#include \"lyap_exact_kernel.cuh\"\n#include \"lyap_kernels_fast.cuh\"\n";
    nvrtcProgram prog = nullptr;
    if (n.create(&prog, kMain, "lyap_spec.cu", 5, header_src, header_names) != NVRTC_SUCCESS) {
        *note = "nvrtcCreateProgram failed";
        return false;
    }
    const nvrtcResult rc = n.compile(prog, (int)(sizeof(opts) / sizeof(opts[0])), opts);
    if (rc != NVRTC_SUCCESS) {
        size_t ls = 0;
        n.log_size(prog, &ls);
        std::string log(ls, '\0');
        if (ls) n.log(prog, log.data());
        *note = "run-time compilation failed: " + log.substr(0, 600);
        n.destroy(&prog);
        return false;
    }
    size_t cs = 0;
    if (n.cubin_size(prog, &cs) != NVRTC_SUCCESS || cs == 0) {
        *note = "no cubin produced";
        n.destroy(&prog);
        return false;
    }
    cubin.resize(cs);
    n.cubin(prog, cubin.data());
    n.destroy(&prog);
    return true;
}

// Loads the (cached) cubin into the current device's context and looks the kernel up.
bool compile_entry(const Key& key, Entry* e, size_t smem_bytes, const PrebuiltKernel* embedded = nullptr) {
    Driver& d = driver();
    if (!d.ok) { g_note = "driver entry points not available"; return false; }
    const int kind = std::get<5>(key);
    const CodeKey ck{std::get<1>(key), std::get<2>(key), std::get<3>(key), std::get<4>(key), kind, std::get<6>(key), std::get<7>(key)};
    std::vector<char>& cubin = g_cubins[ck];
    if (cubin.empty() && embedded) cubin.assign(reinterpret_cast<const char*>(embedded->cubin),
                                                reinterpret_cast<const char*>(embedded->cubin) + embedded->cubin_bytes);
    if (cubin.empty() && !compile_cubin(key, &cubin, &g_note)) {
        cubin.clear();
        return false;
    }
    cudaFree(nullptr);   // make sure the primary context of the current device exists and is current
    CUmodule mod = nullptr;
    if (d.module_load_data(&mod, cubin.data()) != CUDA_SUCCESS) { g_note = "cuModuleLoadData failed"; return false; }
    CUfunction fn = nullptr;
    if (d.module_get_function(&fn, mod, kind == 0 ? "k_lambda_exact_spec" : "k_lambda_fast_spec") != CUDA_SUCCESS) {
        g_note = "kernel symbol not found";
        d.module_unload(mod);
        return false;
    }
    if (smem_bytes && d.func_set_attribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, (int)smem_bytes) != CUDA_SUCCESS) {
        g_note = "cuFuncSetAttribute failed";
        d.module_unload(mod);
        return false;
    }
    e->fn = fn;
    return true;
}

}  // namespace

// The note is written by whichever thread compiled or launched last; a reader gets its own copy.
const char* jit_last_note() {
    thread_local std::string copy;
    std::lock_guard<std::mutex> lk(g_mu);
    copy = g_note;
    return copy.c_str();
}

namespace {
thread_local std::string t_last_kernel;
std::vector<PrebuiltKernel>& prebuilt_list() {
    static std::vector<PrebuiltKernel> v;
    return v;
}
}  // namespace

const char* last_lambda_kernel() { return t_last_kernel.c_str(); }
void note_lambda_kernel(const char* text) { t_last_kernel = text; }

void register_prebuilt(const PrebuiltKernel& k) { prebuilt_list().push_back(k); }   // static initialisers only

// Finds the group-pattern period of both regions of `a`.  Returns KG (1..16) and the two pattern words, or 0.
int sequence_group_period(const LambdaArgs& a, unsigned long long* wu_pats, unsigned long long* acc_pats) {
    auto code = [&](bool acc_region, long long i) {
        const int word0 = acc_region ? a.acc_word0 : 0, wrap = acc_region ? a.acc_wrap : a.wu_wrap;
        return (a.sel[word0 + (i / kStepsPerWord) % wrap] >> (2 * (i % kStepsPerWord))) & 3u;
    };
    for (int kg = 1; kg <= 16; ++kg) {
        const int bs = 2 * kg;
        bool ok = true;
        // a wrapped region repeats after wrap words: one stored period plus bs steps covers every residue
        const long long wu_n = std::min<long long>(a.warmup, (long long)a.wu_wrap * kStepsPerWord + bs);
        const long long acc_n = std::min<long long>(a.iterations, (long long)a.acc_wrap * kStepsPerWord + bs);
        for (long long i = bs; i < wu_n && ok; ++i) ok = code(false, i) == code(false, i - bs);
        for (long long i = bs; i < acc_n && ok; ++i) ok = code(true, i) == code(true, i - bs);
        if (!ok) continue;
        unsigned long long wu = 0, acc = 0;
        for (int i = 0; i < bs; ++i) {
            if (i < a.warmup) wu |= (unsigned long long)code(false, i) << (2 * i);
            if (i < a.iterations) acc |= (unsigned long long)code(true, i) << (2 * i);
        }
        *wu_pats = wu;
        *acc_pats = acc;
        return kg;
    }
    return 0;
}

// Launches the specialised instance when there is one (or when compiling one now is worth it).
// mode: 0 never, 1 when the work seen for this sequence passes a threshold, 2 always.
// *launched tells whether a kernel was enqueued; false means "use the precompiled kernel".
cudaError_t launch_lambda_spec(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps, int sm_count,
                               cudaStream_t st, int kind, int pixels_per_thread, int threads, size_t smem_bytes, int mode,
                               bool* launched) {
    *launched = false;
    const int jit_mode = mode & 3;
    if (mode == 0) return cudaSuccess;
    unsigned long long wu = 0, acc = 0;
    const int kg = sequence_group_period(a, &wu, &acc);
    if (kg == 0) return cudaSuccess;
    const long long tile_px = (long long)threads * pixels_per_thread;
    const long long tiles = (a.n_pixels + tile_px - 1) / tile_px;
    const long long cap = kind == 0 ? sm_count : 4LL * sm_count;   // the exact kernel's shared tables allow one CTA per SM
    const unsigned grid = (unsigned)(tiles < cap ? tiles : cap);
    char name[160];
    static const char* const kinds[4] = {"k_lambda_exact", "k_lambda_fast<FusedF64>", "k_lambda_fast<FusedF32>", "k_lambda_fast<OrbitF64>"};

    int dev = 0;
    cudaError_t ce = cudaGetDevice(&dev);
    if (ce != cudaSuccess) return ce;
    void* params[] = {const_cast<LambdaArgs*>(&a), &out64, &out32, &steps};

    if (mode & kSpecUsePrebuilt) {   // an instance compiled with the library
        for (const PrebuiltKernel& k : prebuilt_list()) {
            // a region shorter than one period never runs its straight-line block (it is walked step by step from the
            // selector words), so its patterns need not match; whether a third parameter occurs must match in any case
            const int bs = 2 * kg;
            const bool uses_c = ((wu | acc) & 0xAAAAAAAAAAAAAAAAull) != 0, k_uses_c = ((k.wu_pats | k.acc_pats) & 0xAAAAAAAAAAAAAAAAull) != 0;
            if (k.kind != kind || k.pixels_per_thread != pixels_per_thread || k.threads != threads || k.kg != kg ||
                (a.warmup >= bs && k.wu_pats != wu) || (a.iterations >= bs && k.acc_pats != acc) || uses_c != k_uses_c)
                continue;
            const Key key{dev, pixels_per_thread, kg, k.wu_pats, k.acc_pats, kind, threads, 1};
            CUfunction fn = nullptr;
            {
                std::lock_guard<std::mutex> lk(g_mu);
                Entry& e = g_cache[key];
                if (!e.fn && !e.failed && !compile_entry(key, &e, smem_bytes, &k)) e.failed = true;   // loads the embedded code
                fn = e.fn;
            }
            if (!fn) break;   // could not be loaded (lyap_jit_note says why): run-time compilation or the generic kernel
            if (tiles > 0) {
                const CUresult r = driver().launch_kernel(fn, grid, 1, 1, (unsigned)threads, 1, 1, (unsigned)smem_bytes, (CUstream)st, params, nullptr);
                if (r != CUDA_SUCCESS) {
                    std::lock_guard<std::mutex> lk(g_mu);
                    g_note = "cuLaunchKernel of the embedded kernel failed";
                    g_cache[key].fn = nullptr;
                    g_cache[key].failed = true;
                    break;
                }
            }
            snprintf(name, sizeof name, "%s_spec<%d px/thread, period %d steps> (built for the patterns of \"%s\")", kinds[kind],
                     pixels_per_thread, 2 * kg, k.sequence);
            note_lambda_kernel(name);
            *launched = true;
            return cudaSuccess;
        }
    }
    if (jit_mode == 0) return cudaSuccess;

    const Key key{dev, pixels_per_thread, kg, wu, acc, kind, threads, 0};
    CUfunction fn = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        Entry& e = g_cache[key];
        e.work_seen += (double)a.n_pixels * ((double)a.warmup + a.iterations);
        // compiling takes about a second, so it waits until that much work with these patterns has been asked for;
        // code another device of this process already compiled is only loaded, which is cheap
        const CodeKey ck{pixels_per_thread, kg, wu, acc, kind, threads, 0};
        const auto have = g_cubins.find(ck);
        const bool cubin_ready = have != g_cubins.end() && !have->second.empty();
        if (!e.fn && !e.failed) {
            if (jit_mode >= 2 || cubin_ready) {
                if (!compile_entry(key, &e, smem_bytes)) e.failed = true;   // compiles if need be, loads into this device's context
            } else if (e.work_seen >= 2e10) {
                // Compile on a background thread; launches go on with the generic kernel and switch over once the code
                // is there (loading it is quick and is done above, by whichever launch comes next).
                int& state = g_background[ck];
                if (state == 2) {
                    e.failed = true;
                } else if (state == 0) {
                    state = 1;
                    std::thread([key, ck]() {
                        std::vector<char> cubin;
                        std::string note;
                        const bool ok = compile_cubin(key, &cubin, &note);
                        std::lock_guard<std::mutex> lk2(g_mu);
                        if (ok) {
                            g_cubins[ck] = std::move(cubin);
                            g_background[ck] = 0;
                        } else {
                            g_note = note;
                            g_background[ck] = 2;
                        }
                    }).detach();
                }
            }
        }
        fn = e.fn;
    }
    if (!fn) return cudaSuccess;
    if (tiles <= 0) { *launched = true; return cudaSuccess; }
    const CUresult r = driver().launch_kernel(fn, grid, 1, 1, (unsigned)threads, 1, 1, (unsigned)smem_bytes, (CUstream)st, params, nullptr);
    if (r != CUDA_SUCCESS) {
        std::lock_guard<std::mutex> lk(g_mu);
        g_note = "cuLaunchKernel of the specialised kernel failed";
        g_cache[key].fn = nullptr;
        g_cache[key].failed = true;
        return cudaSuccess;   // not launched: the caller uses the generic kernel
    }
    snprintf(name, sizeof name, "%s_spec<%d px/thread, period %d steps> (compiled at run time)", kinds[kind], pixels_per_thread, 2 * kg);
    note_lambda_kernel(name);
    *launched = true;
    return cudaSuccess;
}

}  // namespace lyap
