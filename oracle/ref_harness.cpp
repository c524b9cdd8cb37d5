// ref_harness.cpp -- C entry points around the UNMODIFIED reference header.  TEST INFRASTRUCTURE ONLY.
//
// The header (src/lyapunov_fractal.hpp of the reference project) is included from where it lies,
// never copied.  It is built twice by oracle/Makefile, outputs under oracle/_ref/:
//   libref_lyapmath.so  log/pow/exp resolved to this project's lyap_math.h (math_interpose.cpp,
//                       bound with -Bsymbolic): the bit-exact oracle for the CUDA engine.
//   libref_stock.so     log/pow/exp from the host libm: "the natively compiled reference", used
//                       as the timed CPU baseline and to report the distance between the two.
#include <limits>
#include <cstdint>
#include <cstring>
#include <lyapunov_fractal.hpp>
#ifdef _OPENMP
#include <omp.h>
#endif

extern "C" {

// computeFractal (src/lyapunov_fractal.hpp:27); out must hold width*height doubles.
int ref_compute_fractal(double min_x, double max_x, double min_y, double max_y, int width, int height,
                        const char* sequence, int iterations, int warmup, double* out) {
    lyapunov::FractalComputer::ComputationParams p;
    p.min_x = min_x; p.max_x = max_x; p.min_y = min_y; p.max_y = max_y;
    p.width = width; p.height = height; p.sequence = sequence;
    p.iterations = iterations; p.warmup = warmup;
    lyapunov::FractalComputer fc;
    std::vector<double> v = fc.computeFractal(p, nullptr);
    std::memcpy(out, v.data(), v.size() * sizeof(double));
    return (int)v.size();
}

// normalizeData (src/lyapunov_fractal.hpp:105)
int ref_normalize(const double* in, uint64_t n, double* out) {
    std::vector<double> v(in, in + n);
    std::vector<double> r = lyapunov::normalizeData(v);
    std::memcpy(out, r.data(), r.size() * sizeof(double));
    return (int)r.size();
}

// Threads the header's "#pragma omp parallel for ... if(params.height > 100)" (src/lyapunov_fractal.hpp:40) will use,
// and a way to set them (the timed CPU baseline reports a one-thread figure beside the all-threads one).
int ref_omp_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
void ref_omp_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

// struct defaults (src/lyapunov_fractal.hpp:15-25), for the boundary test
void ref_default_params(double* f4, int* i4, char* seq, int seq_cap) {
    lyapunov::FractalComputer::ComputationParams p;
    f4[0] = p.min_x; f4[1] = p.max_x; f4[2] = p.min_y; f4[3] = p.max_y;
    i4[0] = p.width; i4[1] = p.height; i4[2] = p.iterations; i4[3] = p.warmup;
    std::strncpy(seq, p.sequence.c_str(), seq_cap - 1);
    seq[seq_cap - 1] = 0;
}

}  // extern "C"
