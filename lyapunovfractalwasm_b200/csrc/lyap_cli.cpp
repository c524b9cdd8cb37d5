// lyap_cli.cpp -- command-line driver over the C ABI (C++23 host code, no CUDA in this file).
//
// Default arguments reproduce the page's own call (reference web/fractal_renderer.js:144-154):
// 800x800, a,b in [0,4], warm-up 100, sequence and iteration count as the form would give them
// (web/index.html:110-124; defaults "AB", 1000), palette "cosmic".  --config N selects one of the five
// benchmark configurations.  Output: one JSON line with timings; --out writes the frame (.ppm = RGB,
// .rgba = raw RGBA8, .f64 = raw normalised doubles, the array the WASM export returns).
// --config 5 --frames N renders N frames of the zoom batch, starting at --frame, dealt round-robin to the
// GPUs (lyap_multi_render_frames on a kept lyap_multi); --out name.ppm then writes name.0000.ppm, name.0001.ppm, ...; --repeat R renders the
// batch R times and reports the last pass (the first one pays for loading the run-time compiler and compiling).
#include <algorithm>
#include <charconv>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <format>
#include <fstream>
#include <iostream>
#include <string>
#include <string_view>
#include <vector>

#include "../../include/lyap_b200.h"

namespace {

struct Options {
    double min_x = 0.0, max_x = 4.0, min_y = 0.0, max_y = 4.0;
    int width = 800, height = 800, iterations = 1000, warmup = 100;
    std::string sequence = "AB", palette = "cosmic", mode = "exact", out;
    bool has_c = false;
    double c = 0.0;
    int gpus = 1, frame = 0, frames = 0, repeat = 1;
    bool glow = false;
    bool gather = false;
    bool quiet = false;   // no progress callback: the frame's lambda stage is then one kernel launch
};

[[noreturn]] void usage(const char* why) {
    std::cerr << "lyap_cli: " << why << "\n"
              << "usage: lyap_cli [--config 1..5 [--frame K] [--frames N [--repeat R]]] [--width W --height H --min-x .. --max-x .. --min-y .. --max-y ..]\n"
              << "                [--sequence S] [--iterations N] [--warmup N] [--c V] [--palette NAME]\n"
              << "                [--mode exact|fast64|fast32|orbit64] [--gpus N [--gather]] [--repeat R] [--quiet] [--glow] [--out file.ppm|.rgba|.f64]\n";
    std::exit(2);
}

void apply_config(Options& o, int n) {
    switch (n) {
        case 1: o = {2, 4, 2, 4, 512, 512, 1000, 100, "AB"}; break;
        case 2: o = {2.5, 4, 2.5, 4, 4096, 4096, 2000, 200, "AABAB"}; break;
        case 3: o = {3.4, 4.0, 2.5, 3.4, 16384, 16384, 4000, 500, "BBBBBBAAAAAA"}; break;
        case 4: o = {2, 4, 2, 4, 65536, 65536, 1000, 100, "AB"}; break;
        case 5: {
            const int k = o.frame;
            const double h = 0.5 * std::pow(0.97, k);   // zoom batch: half-width 0.5*0.97^k around (3.82, 3.45)
            o = {3.82 - h, 3.82 + h, 3.45 - h, 3.45 + h, 1920, 1080, 3000, 300, "ABC"};
            o.has_c = true;
            o.c = 3.7;
            o.frame = k;
        } break;
        default: usage("--config takes 1..5");
    }
}

std::string json_escape(std::string_view s) {
    std::string out;
    for (char ch : s) {
        if (ch == '"' || ch == '\\') out += '\\';
        out += ch;
    }
    return out;
}

double to_double(std::string_view s) {
    return std::strtod(std::string(s).c_str(), nullptr);
}

int to_int(std::string_view s) {
    int v = 0;
    auto [p, ec] = std::from_chars(s.data(), s.data() + s.size(), v);
    if (ec != std::errc() || p != s.data() + s.size()) usage("bad integer");
    return v;
}

void write_frame(const std::string& path, const uint8_t* rgba, int width, int height) {
    std::ofstream f(path, std::ios::binary);
    if (!f) { std::cerr << "lyap_cli: cannot write " << path << "\n"; std::exit(1); }
    const size_t n = static_cast<size_t>(width) * static_cast<size_t>(height);
    if (path.ends_with(".ppm")) {
        f << std::format("P6\n{} {}\n255\n", width, height);
        std::vector<uint8_t> rgb(n * 3);
        for (size_t i = 0; i < n; ++i) { rgb[3 * i] = rgba[4 * i]; rgb[3 * i + 1] = rgba[4 * i + 1]; rgb[3 * i + 2] = rgba[4 * i + 2]; }
        f.write(reinterpret_cast<const char*>(rgb.data()), static_cast<std::streamsize>(rgb.size()));
    } else {
        f.write(reinterpret_cast<const char*>(rgba), static_cast<std::streamsize>(n * 4));
    }
}

// Frames o.frame .. o.frame + o.frames - 1 of the zoom batch: window half-width 0.5*0.97^k around (3.82, 3.45),
// everything else as given (size, sequence, c, palette, mode).
int render_zoom_batch(const Options& o, const lyap_params& base) {
    const int nf = o.frames;
    std::vector<lyap_params> frames(nf, base);
    for (int i = 0; i < nf; ++i) {
        const double h = 0.5 * std::pow(0.97, o.frame + i);
        frames[i].min_x = 3.82 - h; frames[i].max_x = 3.82 + h;
        frames[i].min_y = 3.45 - h; frames[i].max_y = 3.45 + h;
    }
    const size_t bytes = static_cast<size_t>(o.width) * static_cast<size_t>(o.height) * 4;
    std::vector<uint8_t*> rgba(nf, nullptr);
    for (int i = 0; i < nf; ++i) {
        void* q = nullptr;
        if (lyap_host_alloc(&q, bytes) != LYAP_OK) {
            std::cerr << "lyap_cli: " << lyap_last_error() << "\n";
            return 1;
        }
        rgba[i] = static_cast<uint8_t*>(q);
    }
    std::vector<int32_t> devs(std::max(1, o.gpus));
    for (size_t i = 0; i < devs.size(); ++i) devs[i] = static_cast<int32_t>(i);
    std::vector<lyap_render_stats> st(nf);
    int status = LYAP_OK;
    double wall_ms = 0.0, first_pass_ms = 0.0;
    // the devices are set up once and kept for every pass (contexts, streams, two buffer sets each)
    lyap_multi* m = nullptr;
    const auto t_setup = std::chrono::steady_clock::now();
    status = lyap_multi_create(&m, static_cast<int32_t>(devs.size()), devs.data(), 0);
    const double setup_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t_setup).count();
    for (int pass = 0; pass < std::max(1, o.repeat) && status == LYAP_OK; ++pass) {
        const auto t0 = std::chrono::steady_clock::now();
        status = lyap_multi_render_frames(m, frames.data(), nf, nullptr, rgba.data(), st.data());
        wall_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        if (pass == 0) first_pass_ms = wall_ms;
    }
    lyap_multi_destroy(m);
    if (status != LYAP_OK) {
        std::cerr << "lyap_cli: " << lyap_status_string(status) << ": " << lyap_last_error() << "\n";
        return 1;
    }
    uint64_t executed = 0, nominal = 0;
    double ms_lambda = 0, ms_device = 0;
    for (const auto& s : st) {
        executed += s.executed_steps;
        nominal += s.nominal_steps;
        ms_lambda += s.ms_lambda;
        ms_device += s.ms_total_device;
    }
    if (!o.out.empty()) {
        const size_t dot = o.out.rfind('.');
        for (int i = 0; i < nf; ++i)
            write_frame(std::format("{}.{:04d}{}", o.out.substr(0, dot), o.frame + i, dot == std::string::npos ? "" : o.out.substr(dot)),
                        rgba[i], o.width, o.height);
    }
    for (uint8_t* q : rgba) lyap_host_free(q);
    std::cout << std::format(
        "{{\"frames\": {}, \"first_frame\": {}, \"width\": {}, \"height\": {}, \"sequence\": \"{}\", \"mode\": \"{}\", "
        "\"gpus\": {}, \"executed_steps\": {}, \"nominal_steps\": {}, \"ms_lambda_sum\": {:.3f}, \"ms_device_sum\": {:.3f}, "
        "\"ms_wall\": {:.3f}, \"frames_per_s_wall\": {:.2f}, \"steps_per_s_wall\": {:.4e}, \"ms_lambda_first\": {:.3f}, "
        "\"ms_lambda_last\": {:.3f}, \"passes\": {}, \"ms_wall_first_pass\": {:.3f}, \"ms_device_setup\": {:.3f}, \"jit_note\": \"{}\"}}\n",
        nf, o.frame, o.width, o.height, o.sequence, o.mode, devs.size(), executed, nominal, ms_lambda, ms_device, wall_ms,
        nf / (wall_ms * 1e-3), executed / (wall_ms * 1e-3), st.front().ms_lambda, st.back().ms_lambda, std::max(1, o.repeat), first_pass_ms, setup_ms, lyap_jit_note());
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    Options o;
    std::vector<std::string_view> args(argv + 1, argv + argc);
    // --frame has to be known before --config 5 is applied
    for (size_t i = 0; i + 1 < args.size(); ++i)
        if (args[i] == "--frame") o.frame = to_int(args[i + 1]);
    for (size_t i = 0; i < args.size(); ++i) {
        const auto a = args[i];
        auto next = [&]() -> std::string_view {
            if (i + 1 >= args.size()) usage("missing value");
            return args[++i];
        };
        if (a == "--config") { const int fr = o.frame; o.frame = fr; apply_config(o, to_int(next())); }
        else if (a == "--frame") next();
        else if (a == "--frames") o.frames = to_int(next());
        else if (a == "--repeat") o.repeat = to_int(next());
        else if (a == "--width") o.width = to_int(next());
        else if (a == "--height") o.height = to_int(next());
        else if (a == "--min-x") o.min_x = to_double(next());
        else if (a == "--max-x") o.max_x = to_double(next());
        else if (a == "--min-y") o.min_y = to_double(next());
        else if (a == "--max-y") o.max_y = to_double(next());
        else if (a == "--sequence") o.sequence = std::string(next());
        else if (a == "--iterations") o.iterations = to_int(next());
        else if (a == "--warmup") o.warmup = to_int(next());
        else if (a == "--c") { o.has_c = true; o.c = to_double(next()); }
        else if (a == "--palette") o.palette = std::string(next());
        else if (a == "--mode") o.mode = std::string(next());
        else if (a == "--gpus") o.gpus = to_int(next());
        else if (a == "--out") o.out = std::string(next());
        else if (a == "--glow") o.glow = true;
        else if (a == "--gather") o.gather = true;
        else if (a == "--quiet") o.quiet = true;
        else usage("unknown option");
    }

    lyap_params p;
    lyap_params_default(&p);
    p.min_x = o.min_x; p.max_x = o.max_x; p.min_y = o.min_y; p.max_y = o.max_y;
    p.width = o.width; p.height = o.height;
    p.sequence = o.sequence.data(); p.sequence_len = static_cast<int32_t>(o.sequence.size());
    p.iterations = o.iterations; p.warmup = o.warmup;
    p.mode = o.mode == "exact" ? LYAP_MODE_EXACT : o.mode == "fast64" ? LYAP_MODE_FAST_FP64 : o.mode == "fast32" ? LYAP_MODE_FAST_FP32
             : o.mode == "orbit64" ? LYAP_MODE_FAST_FP64_ORBIT : -1;
    if (p.mode < 0) usage("--mode takes exact, fast64, fast32 or orbit64");
    p.palette = lyap_palette_from_name(o.palette.c_str());
    p.c_enabled = o.has_c ? 1 : 0;
    p.c_value = o.c;

    if (o.frames > 0) return render_zoom_batch(o, p);

    const size_t n = static_cast<size_t>(o.width) * static_cast<size_t>(o.height);
    const bool want_f64 = o.out.ends_with(".f64");
    std::vector<double> norm(want_f64 ? n : 0);
    std::vector<uint8_t> rgba(n * 4);
    lyap_render_stats st{};
    lyap_multi_stats ms{};
    std::string multi_note;
    const auto t0 = std::chrono::steady_clock::now();
    int status;
    if (o.gpus <= 1) {
        lyap_ctx* ctx = nullptr;
        if ((status = lyap_create(&ctx, 0)) == LYAP_OK) {
            for (int pass = 0; pass < std::max(1, o.repeat) && status == LYAP_OK; ++pass)
                status = lyap_render(ctx, &p, nullptr, nullptr, want_f64 ? norm.data() : nullptr, rgba.data(),
                                     o.quiet ? nullptr : +[](double f) { std::fprintf(stderr, "\rprogress %5.1f %%", 100.0 * f); }, &st);
            if (!o.quiet) std::fprintf(stderr, "\n");
            lyap_destroy(ctx);
        }
    } else {
        // one frame as row bands over the devices; --gather collects the RGBA8 bands in device 0's memory first (NCCL
        // send/recv) and copies the frame to the host from there; --repeat renders it again on the same object
        std::vector<int32_t> devs(o.gpus);
        for (int i = 0; i < o.gpus; ++i) devs[i] = i;
        lyap_multi* m = nullptr;
        if ((status = lyap_multi_create(&m, o.gpus, devs.data(), o.gather ? 1 : 0)) == LYAP_OK) {
            for (int pass = 0; pass < std::max(1, o.repeat) && status == LYAP_OK; ++pass)
                status = lyap_multi_render(m, &p, o.gather ? LYAP_MULTI_GATHER_RGBA : 0, nullptr, nullptr,
                                           want_f64 ? norm.data() : nullptr, rgba.data(), 0.0, &ms);
            multi_note = lyap_multi_note(m);
            lyap_multi_destroy(m);
        }
        st.executed_steps = ms.executed_steps; st.nominal_steps = ms.nominal_steps;
        st.lambda_min = ms.lambda_min; st.lambda_max = ms.lambda_max;
        st.ms_lambda = ms.ms_lambda_max; st.ms_total_device = ms.ms_device_max;
    }
    if (status == LYAP_OK && o.glow) {   // the page's last step (web/fractal_renderer.js:203)
        lyap_ctx* ctx = nullptr;
        if ((status = lyap_create(&ctx, 0)) == LYAP_OK) {
            status = lyap_glow(ctx, rgba.data(), o.width, o.height, rgba.data());
            lyap_destroy(ctx);
        }
    }
    const double wall_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (status != LYAP_OK) {
        std::cerr << "lyap_cli: " << lyap_status_string(status) << ": " << lyap_last_error() << "\n";
        return 1;
    }
    if (!o.out.empty()) {
        if (want_f64) {
            std::ofstream f(o.out, std::ios::binary);
            if (!f) { std::cerr << "lyap_cli: cannot write " << o.out << "\n"; return 1; }
            f.write(reinterpret_cast<const char*>(norm.data()), static_cast<std::streamsize>(n * 8));
        } else {
            write_frame(o.out, rgba.data(), o.width, o.height);
        }
    }
    std::cout << std::format(
        "{{\"width\": {}, \"height\": {}, \"sequence\": \"{}\", \"mode\": \"{}\", \"gpus\": {}, \"executed_steps\": {}, "
        "\"nominal_steps\": {}, \"lambda_min\": {}, \"lambda_max\": {}, \"ms_lambda\": {:.3f}, \"ms_device\": {:.3f}, "
        "\"ms_wall\": {:.3f}, \"steps_per_s_wall\": {:.4e}, \"ms_render_last_pass\": {:.3f}, \"gather_ms\": {:.3f}, "
        "\"gather_bytes\": {}, \"gather_gbs\": {:.1f}, \"used_nccl\": {}, \"multi_note\": \"{}\", \"kernel\": \"{}\"}}\n",
        o.width, o.height, o.sequence, o.mode, o.gpus, st.executed_steps, st.nominal_steps, st.lambda_min, st.lambda_max,
        st.ms_lambda, st.ms_total_device, wall_ms, st.executed_steps / (wall_ms * 1e-3), ms.ms_wall, ms.ms_gather, ms.gather_bytes,
        ms.ms_gather > 0 ? ms.gather_bytes / (ms.ms_gather * 1e-3) / 1e9 : 0.0, ms.used_nccl, multi_note, json_escape(lyap_last_kernel()));
    return 0;
}
