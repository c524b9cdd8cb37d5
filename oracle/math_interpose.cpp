// math_interpose.cpp -- gives the reference header this project's log/pow/exp.  TEST INFRASTRUCTURE ONLY.
// Linked into oracle/_ref/libref_lyapmath.so with -Wl,-Bsymbolic so the header's std::log, std::pow and
// std::exp calls (src/lyapunov_fractal.hpp:72,132,133) bind here instead of to libm.
#include "../lyapunovfractalwasm_b200/csrc/lyap_math.h"
extern "C" {
double log(double x) noexcept { return lyap_log(x); }
double exp(double x) noexcept { return lyap_exp(x); }
double pow(double x, double y) noexcept { return lyap_pow(x, y); }
}
