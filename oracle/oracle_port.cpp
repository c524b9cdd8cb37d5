// oracle_port.cpp -- CPU restatement of the reference's hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file is the checker for the CUDA engine.  Nothing in the product path may
// call, link or load it; only tests, the smoke check and the bench's CPU-baseline
// leg use it.
//
// What it restates (reference file:line, paths relative to the reference project):
//   oracle_lambda_rows      src/lyapunov_fractal.hpp:27-102  computeFractal, for a global row set
//   oracle_minmax           src/lyapunov_fractal.hpp:110-120 normalizeData pass 1
//   oracle_normalize_with   src/lyapunov_fractal.hpp:122-137 normalizeData pass 2
//   oracle_normalize        src/lyapunov_fractal.hpp:105-140 whole normalizeData
//   oracle_box3             web/fractal_renderer.js:283-311  applyPostProcessing
//   oracle_palette          web/fractal_renderer.js:207-281  getColorFunction (+ hslToRgb :26-47)
//   oracle_colorize         web/fractal_renderer.js:177-198  renderFractal up to the ImageData store
//   oracle_glow             web/fractal_renderer.js:313-334  applyGlow (browser-defined; this project's reading)
//
// Differences from the reference, on purpose:
//   * rows are addressed by their GLOBAL index (r_y = min_y + dy*y_global with the global dy), so
//     a band or a strided subset of a frame larger than the reference can allocate gives the same
//     bits the whole frame would (the reference's int pixel count overflows at 65536^2);
//   * an optional third parameter value for sequence letter 'C' (extension; off => 'C' is "not A");
//   * log/pow/exp/sin/cos are this project's own functions (lyap_math.h), not libm.  The pinning
//     of this restatement against the unmodified reference header built with the same math is
//     done in tests/test_oracle.py via oracle/_ref.
//
// Build: see oracle/Makefile (g++ -O3 -std=c++20 -ffp-contract=off -mfma -fopenmp).
#include <cmath>
#include <cstdint>
#include <cstring>
#include <limits>
#include <vector>

#include "../lyapunovfractalwasm_b200/csrc/lyap_math.h"

extern "C" {

double oracle_log(double x) { return lyap_log(x); }
double oracle_exp(double x) { return lyap_exp(x); }
double oracle_pow(double x, double y) { return lyap_pow(x, y); }
double oracle_sin(double x) { return lyap_sin(x); }
double oracle_cos(double x) { return lyap_cos(x); }

// Word-wise FNV-1a style hash over 64-bit words.
uint64_t oracle_hash64(const uint64_t* w, uint64_t n) {
    uint64_t h = 1469598103934665603ull;
    for (uint64_t i = 0; i < n; ++i) {
        h ^= w[i];
        h *= 1099511628211ull;
    }
    return h;
}

// Lyapunov exponent (bits per step) of one pixel; *steps gets the executed logistic updates.
static double pixel_lambda(double r_x, double r_y, double r_c, int has_c, const uint8_t* sel, int seq_len,
                           int warmup, int iterations, uint64_t* steps) {
    // sel[j]: 0 = A, 1 = B, 2 = C
    if (r_x <= 0.0 || r_y <= 0.0) return -5.0;               // :47-50
    const double log_2 = LYAP_LN2;                             // :32 (compile-time folded in the reference)
    double current_x = 0.5;                                    // :31,52
    double lyap = 0.0;
    int valid_terms = 0;
    uint64_t n = 0;
    int ph = 0;
    for (int i = 0; i < warmup; ++i) {                         // :56-63
        const int s = sel[ph];
        if (++ph == seq_len) ph = 0;
        const double r = s == 0 ? r_x : ((s == 2 && has_c) ? r_c : r_y);
        current_x = r * current_x * (1.0 - current_x);
        ++n;
        if (current_x <= 0.0 || current_x >= 1.0 || !std::isfinite(current_x)) break;
    }
    if (std::isfinite(current_x) && current_x > 0.0 && current_x < 1.0) {   // :65
        ph = warmup % seq_len;
        for (int i = 0; i < iterations; ++i) {                 // :66-81
            const int s = sel[ph];
            if (++ph == seq_len) ph = 0;
            const double r = s == 0 ? r_x : ((s == 2 && has_c) ? r_c : r_y);
            const double deriv = std::fabs(r * (1.0 - 2.0 * current_x));
            if (deriv > 0.0) {
                lyap += lyap_log(deriv);
                valid_terms++;
            }
            current_x = r * current_x * (1.0 - current_x);
            ++n;
            if (current_x <= 0.0 || current_x >= 1.0 || !std::isfinite(current_x)) break;
        }
    }
    *steps += n;
    return valid_terms > 0 ? lyap / (valid_terms * log_2) : -5.0;   // :84-85
}

// Rows y = y0, y0+stride, ... < y1 of the width x height frame; out holds those rows packed.
// Returns executed logistic steps.  c_enabled = 0 reproduces the reference ('C' == not 'A').
uint64_t oracle_lambda_rows(double min_x, double max_x, double min_y, double max_y, int width, int height,
                            const char* sequence, int seq_len, int iterations, int warmup, int c_enabled,
                            double c_value, int64_t y0, int64_t y1, int64_t row_stride, double* out) {
    const double dx = (max_x - min_x) / (width - 1.0);         // :29
    const double dy = (max_y - min_y) / (height - 1.0);        // :30
    std::vector<uint8_t> sel(seq_len);
    for (int j = 0; j < seq_len; ++j) sel[j] = sequence[j] == 'A' ? 0 : (sequence[j] == 'C' ? 2 : 1);   // :37
    const int64_t nrows = y1 > y0 ? (y1 - y0 + row_stride - 1) / row_stride : 0;
    uint64_t total = 0;
#pragma omp parallel for schedule(dynamic) reduction(+ : total)
    for (int64_t k = 0; k < nrows; ++k) {
        const int y = (int)(y0 + k * row_stride);
        const double r_y = min_y + dy * y;                      // :42
        uint64_t steps = 0;
        for (int x = 0; x < width; ++x) {
            const double r_x = min_x + dx * x;                  // :45
            out[k * (int64_t)width + x] =
                pixel_lambda(r_x, r_y, c_value, c_enabled, sel.data(), seq_len, warmup, iterations, &steps);
        }
        total += steps;
    }
    return total;
}

// normalizeData pass 1: min/max over finite values > -4.  Starts from +max / lowest like the reference.
void oracle_minmax(const double* v, uint64_t n, double* mn, double* mx) {
    double lo = std::numeric_limits<double>::max();
    double hi = std::numeric_limits<double>::lowest();
    for (uint64_t i = 0; i < n; ++i) {
        const double val = v[i];
        if (std::isfinite(val) && val > -4.0) {
            lo = std::fmin(lo, val);
            hi = std::fmax(hi, val);
        }
    }
    *mn = lo;
    *mx = hi;
}

// normalizeData pass 2 with a given (global) min/max.
void oracle_normalize_with(const double* v, uint64_t n, double mn, double mx, double* out) {
    if (mn >= mx) {                                            // :122
        for (uint64_t i = 0; i < n; ++i) out[i] = 0.0;
        return;
    }
    const double range = mx - mn;
    const double range_inv = 1.0 / range;                      // :124-125
#pragma omp parallel for
    for (int64_t i = 0; i < (int64_t)n; ++i) {
        const double val = v[i];
        if (std::isfinite(val) && val > -4.0) {
            const double t = (val - mn) * range_inv;
            const double s = lyap_pow(t, 1.2);
            out[i] = 1.0 / (1.0 + lyap_exp(-7.0 * (s - 0.5)));
        } else {
            out[i] = 0.0;
        }
    }
}

void oracle_normalize(const double* v, uint64_t n, double* out) {
    double mn, mx;
    oracle_minmax(v, n, &mn, &mx);
    oracle_normalize_with(v, n, mn, mx, out);
}

// 3x3 mean with image-edge clipping, fixed summation order.
void oracle_box3(const double* in, int width, int height, double* out) {
#pragma omp parallel for
    for (int y = 0; y < height; ++y) {
        for (int x = 0; x < width; ++x) {
            const int64_t idx = (int64_t)y * width + x;
            double sum = in[idx];
            int count = 1;
            for (int dy = -1; dy <= 1; ++dy) {
                for (int dx = -1; dx <= 1; ++dx) {
                    if (dx == 0 && dy == 0) continue;
                    const int nx = x + dx, ny = y + dy;
                    if (nx >= 0 && nx < width && ny >= 0 && ny < height) {
                        sum += in[(int64_t)ny * width + nx];
                        count++;
                    }
                }
            }
            out[idx] = sum / count;
        }
    }
}

static double hue2rgb(double p, double q, double t) {
    if (t < 0) t += 1;
    if (t > 1) t -= 1;
    if (t < 1.0 / 6) return p + (q - p) * 6 * t;
    if (t < 1.0 / 2) return q;
    if (t < 2.0 / 3) return p + (q - p) * (2.0 / 3 - t) * 6;
    return p;
}

// Store into a clamped unsigned byte: integers after floor, NaN -> 0.
static uint8_t clamp_u8(double v) {
    if (!(v > 0.0)) return 0;
    if (v >= 255.0) return 255;
    return (uint8_t)v;
}

// palette ids: 0 cosmic, 1 nebula, 2 aurora, 3 solarflare, 4 blackhole, 5 psychedelic, 6 rainbow
void oracle_palette(double t, int palette, uint8_t* rgb) {
    const double PI = LYAP_PI;
    const double mid = std::fabs(t - 0.5) * 2;
    const double intensity = 1 - mid;
    double r, g, b;
    switch (palette) {
        default:
        case 0: {
            const double phase = mid * PI;
            r = std::floor(255 * (intensity * 0.8 + 0.2 * lyap_sin(phase)));
            g = std::floor(255 * (intensity * 0.3));
            b = std::floor(255 * (intensity * 0.9 + 0.1 * lyap_cos(phase)));
        } break;
        case 1:
            r = std::floor(255 * (intensity * 0.9 + 0.1 * lyap_pow(t, 1.5)));
            g = std::floor(255 * (intensity * 0.5));
            b = std::floor(255 * (intensity * 0.8));
            break;
        case 2: {
            const double phase = mid * PI;
            r = std::floor(255 * (intensity * 0.6));
            g = std::floor(255 * (intensity * 0.9 + 0.1 * lyap_sin(phase)));
            b = std::floor(255 * (intensity * 0.7));
        } break;
        case 3:
            r = std::floor(255 * (intensity * 0.95));
            g = std::floor(255 * (intensity * 0.6));
            b = std::floor(255 * (intensity * 0.2));
            break;
        case 4: {
            const double phase = mid * PI;
            r = std::floor(255 * (intensity * 0.5));
            g = std::floor(255 * (intensity * 0.7));
            b = std::floor(255 * (intensity * 0.9 + 0.1 * lyap_sin(phase)));
        } break;
        case 5: {
            const double phase = t * PI * 6;
            r = std::floor(255 * (intensity * (0.5 + 0.5 * lyap_sin(phase))));
            g = std::floor(255 * (intensity * (0.5 + 0.5 * lyap_sin(phase + 2 * PI / 3))));
            b = std::floor(255 * (intensity * (0.5 + 0.5 * lyap_sin(phase + 4 * PI / 3))));
        } break;
        case 6: {
            const double hue = t * 360;
            const double h = hue / 360;
            const double q = 0.5 + 1.0 - 0.5 * 1.0;   // l + s - l*s with s = 1, l = 0.5
            const double p = 2 * 0.5 - q;
            const double cr = hue2rgb(p, q, h + 1.0 / 3);
            const double cg = hue2rgb(p, q, h);
            const double cb = hue2rgb(p, q, h - 1.0 / 3);
            r = std::floor(255 * (intensity * cr));
            g = std::floor(255 * (intensity * cg));
            b = std::floor(255 * (intensity * cb));
        } break;
    }
    rgb[0] = clamp_u8(r);
    rgb[1] = clamp_u8(g);
    rgb[2] = clamp_u8(b);
}

// box mean + palette + RGBA store (alpha 255) of a normalised frame.
void oracle_colorize(const double* norm, int width, int height, int palette, uint8_t* rgba) {
    std::vector<double> boxed((size_t)width * height);
    oracle_box3(norm, width, height, boxed.data());
#pragma omp parallel for
    for (int64_t i = 0; i < (int64_t)width * height; ++i) {
        oracle_palette(boxed[i], palette, rgba + 4 * i);
        rgba[4 * i + 3] = 255;
    }
}

// Glow: three self-draws of the canvas with 'screen' compositing (web/fractal_renderer.js:313-334):
// blur(6px) at alpha 0.3, blur(2px) at alpha 0.4, no filter at alpha 0.1.  The browser's compositor defines the
// exact arithmetic there; this is the engine's own reading of the Canvas / CSS filter rules, the same one the CUDA
// kernels follow: Gaussian of standard deviation sigma truncated at ceil(3 sigma) and normalised, transparent black
// outside the canvas, premultiplied source, opaque backdrop, so per channel
//     out = Cb + alpha * Sp * (1 - Cb),   Sp = blurred premultiplied source,
// and the canvas is rounded to 8 bits after each draw.
static void glow_weights(double sigma, std::vector<double>& w) {
    const int R = (int)std::ceil(3.0 * sigma);
    w.assign(2 * R + 1, 0.0);
    double sum = 0.0;
    for (int k = -R; k <= R; ++k) {
        w[k + R] = lyap_exp(-(double)(k * k) / (2.0 * sigma * sigma));
        sum += w[k + R];
    }
    for (double& v : w) v /= sum;
}

static void glow_pass(std::vector<uint8_t>& canvas, int width, int height, double sigma, double alpha) {
    const size_t n = (size_t)width * height;
    std::vector<double> sp(n * 3);
    if (sigma > 0.0) {
        std::vector<double> w;
        glow_weights(sigma, w);
        const int R = (int)(w.size() / 2);
        std::vector<double> tmp(n * 3);
#pragma omp parallel for
        for (int y = 0; y < height; ++y)
            for (int x = 0; x < width; ++x)
                for (int c = 0; c < 3; ++c) {
                    double s = 0.0;
                    for (int k = -R; k <= R; ++k) {
                        const int xx = x + k;
                        if (xx >= 0 && xx < width) s += w[k + R] * (canvas[((size_t)y * width + xx) * 4 + c] / 255.0);
                    }
                    tmp[((size_t)y * width + x) * 3 + c] = s;
                }
#pragma omp parallel for
        for (int y = 0; y < height; ++y)
            for (int x = 0; x < width; ++x)
                for (int c = 0; c < 3; ++c) {
                    double s = 0.0;
                    for (int k = -R; k <= R; ++k) {
                        const int yy = y + k;
                        if (yy >= 0 && yy < height) s += w[k + R] * tmp[((size_t)yy * width + x) * 3 + c];
                    }
                    sp[((size_t)y * width + x) * 3 + c] = s;
                }
    } else {
        for (size_t i = 0; i < n; ++i)
            for (int c = 0; c < 3; ++c) sp[i * 3 + c] = canvas[i * 4 + c] / 255.0;
    }
    for (size_t i = 0; i < n; ++i)
        for (int c = 0; c < 3; ++c) {
            const double cb = canvas[i * 4 + c] / 255.0;
            const double out = cb + alpha * sp[i * 3 + c] * (1.0 - cb);
            double q = std::floor(out * 255.0 + 0.5);
            canvas[i * 4 + c] = (uint8_t)(q < 0.0 ? 0.0 : (q > 255.0 ? 255.0 : q));
        }
}

void oracle_glow(const uint8_t* rgba_in, int width, int height, uint8_t* rgba_out) {
    std::vector<uint8_t> canvas(rgba_in, rgba_in + (size_t)width * height * 4);
    glow_pass(canvas, width, height, 6.0, 0.3);
    glow_pass(canvas, width, height, 2.0, 0.4);
    glow_pass(canvas, width, height, 0.0, 0.1);
    std::memcpy(rgba_out, canvas.data(), canvas.size());
}

int oracle_abi_version(void) { return 1; }

}  // extern "C"
