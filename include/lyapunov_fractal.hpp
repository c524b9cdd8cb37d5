// lyapunov_fractal.hpp -- C++23 drop-in for the reference header of the same name.
//
// Code written against the reference's src/lyapunov_fractal.hpp (namespace lyapunov,
// FractalComputer::ComputationParams at :15-25, computeFractal at :27, normalizeData at :105)
// compiles against this file unchanged and runs on a B200 through liblyap_b200.so.
// Link with -llyap_b200.  There is no CPU path: failures throw std::runtime_error.
//
// Differences a caller can observe:
//   * the progress callback runs on the calling thread, in order, per finished row chunk, then 1.0
//     (the reference calls it every 10th row from OpenMP workers in any order, :88-90,97-99);
//   * an empty sequence, non-positive sizes or negative counts throw instead of being undefined
//     (:34-37 divides by zero on an empty sequence);
//   * pixel counts are 64-bit (the reference multiplies two ints, :28);
//   * log/pow/exp are the engine's own fixed definitions (last-bit differences from a given libm).
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstdlib>
#include <stdexcept>
#include <string>
#include <vector>

#include "lyap_b200.h"

namespace lyapunov {

namespace detail {
// One engine context per thread, created on first use on device LYAP_DEVICE (default 0).
struct Context {
    lyap_ctx* ctx = nullptr;
    Context() {
        int device = 0;
        if (const char* env = std::getenv("LYAP_DEVICE")) device = std::atoi(env);
        if (int st = lyap_create(&ctx, device); st != LYAP_OK)
            throw std::runtime_error(std::string("lyap_create: ") + lyap_last_error());
    }
    ~Context() { lyap_destroy(ctx); }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
};
inline lyap_ctx* context() {
    thread_local Context c;
    return c.ctx;
}
inline void check(int status, const char* what) {
    if (status != LYAP_OK) throw std::runtime_error(std::string(what) + ": " + lyap_last_error());
}
}  // namespace detail

class FractalComputer {
public:
    struct ComputationParams {
        double min_x = 0.0;
        double max_x = 4.0;
        double min_y = 0.0;
        double max_y = 4.0;
        int width = 800;
        int height = 600;
        std::string sequence = "ABABABAB";
        int iterations = 10000;
        int warmup = 100;
    };

    std::vector<double> computeFractal(const ComputationParams& params, void (*progressCallback)(double)) {
        lyap_params p;
        lyap_params_default(&p);
        p.min_x = params.min_x;
        p.max_x = params.max_x;
        p.min_y = params.min_y;
        p.max_y = params.max_y;
        p.width = params.width;
        p.height = params.height;
        p.sequence = params.sequence.data();
        p.sequence_len = static_cast<int32_t>(params.sequence.size());
        p.iterations = params.iterations;
        p.warmup = params.warmup;
        if (params.width < 1 || params.height < 1) throw std::runtime_error("computeFractal: width and height must be >= 1");
        std::vector<double> fractal_data(static_cast<std::size_t>(params.width) * static_cast<std::size_t>(params.height));
        detail::check(lyap_compute_fractal(detail::context(), &p, fractal_data.data(), progressCallback), "computeFractal");
        return fractal_data;
    }
};

inline std::vector<double> normalizeData(const std::vector<double>& fractal_data) {
    if (fractal_data.empty()) return {};
    std::vector<double> normalized(fractal_data.size());
    detail::check(lyap_normalize_data(detail::context(), fractal_data.data(), fractal_data.size(), normalized.data()),
                  "normalizeData");
    return normalized;
}

// The page-side colour stage (web/fractal_renderer.js:177-200) as a C++ call: normalised frame ->
// RGBA8 bytes with the named palette ("cosmic" when unknown, :280).
inline std::vector<std::uint8_t> renderRGBA(const std::vector<double>& normalized, int width, int height,
                                            const std::string& colorScheme = "cosmic") {
    if (width < 1 || height < 1 || normalized.size() != static_cast<std::size_t>(width) * static_cast<std::size_t>(height))
        throw std::runtime_error("renderRGBA: size mismatch");
    std::vector<std::uint8_t> rgba(normalized.size() * 4);
    detail::check(lyap_colorize(detail::context(), normalized.data(), width, height,
                                lyap_palette_from_name(colorScheme.c_str()), rgba.data()),
                  "renderRGBA");
    return rgba;
}

// The page's glow pass (web/fractal_renderer.js:313-334) on an RGBA8 frame, the engine's reading of it.
inline std::vector<std::uint8_t> applyGlow(const std::vector<std::uint8_t>& rgba, int width, int height) {
    if (width < 1 || height < 1 || rgba.size() != static_cast<std::size_t>(width) * static_cast<std::size_t>(height) * 4)
        throw std::runtime_error("applyGlow: size mismatch");
    std::vector<std::uint8_t> out(rgba.size());
    detail::check(lyap_glow(detail::context(), rgba.data(), width, height, out.data()), "applyGlow");
    return out;
}

}  // namespace lyapunov
