// lyap_prebuilt.cu -- instances of the lambda kernels compiled at BUILD time for one sequence each.
//
// The specialised form of the lambda kernels (a whole period of the sequence as one straight-line block, see
// lyap_exact_kernel.cuh) needs the sequence's two-step group patterns as compile-time constants.  For any sequence
// the library can produce that form at run time (lyap_jit.cu, NVRTC); for the sequences below it is compiled here by
// nvcc from the same source, so the first frame of a process already runs it and a machine without the run-time
// compiler loses nothing.  The file is compiled once per sequence (-DLYAP_PREBUILT_SET=n), each into its own object.
//
//   set  sequence        warm-up % len   used by
//   0    AB              0               512^2 and 65536^2 frames, the page's default call ("AB", "ABABABAB", ...)
//   1    AABAB           0               4096^2 frame
//   2    BBBBBBAAAAAA    8               16384^2 frame (500 warm-up steps: accumulation starts at phase 8)
//   3    ABC (c given)   0               zoom batch with the third parameter
//   4    ABB             0               "ABC" without the third parameter ('C' is then "not A", reference :37)
//
// A launch uses an instance when its (group period, warm-up patterns, accumulation patterns) equal the instance's,
// whatever the sequence string was.
#include <cuda_runtime.h>

#include "lyap_engine.h"
#include "lyap_math.h"

#include "lyap_exact_kernel.cuh"
#include "lyap_kernels_fast.cuh"

#ifndef LYAP_PREBUILT_SET
#error "compile with -DLYAP_PREBUILT_SET=0..4"
#endif

namespace lyap {
namespace {

#if LYAP_PREBUILT_SET == 0
constexpr char kSeq[] = "AB";
constexpr bool kUseC = false;
constexpr int kAccPhase = 0;
#elif LYAP_PREBUILT_SET == 1
constexpr char kSeq[] = "AABAB";
constexpr bool kUseC = false;
constexpr int kAccPhase = 0;
#elif LYAP_PREBUILT_SET == 2
constexpr char kSeq[] = "BBBBBBAAAAAA";
constexpr bool kUseC = false;
constexpr int kAccPhase = 8;
#elif LYAP_PREBUILT_SET == 3
constexpr char kSeq[] = "ABC";
constexpr bool kUseC = true;
constexpr int kAccPhase = 0;
#elif LYAP_PREBUILT_SET == 4
constexpr char kSeq[] = "ABB";
constexpr bool kUseC = false;
constexpr int kAccPhase = 0;
#endif

constexpr int kLen = (int)sizeof(kSeq) - 1;

// selector code of step i: 'A' -> 0 (column parameter), 'C' with the extension -> 2, anything else -> 1 (row parameter)
constexpr unsigned code_at(int i) {
    const char ch = kSeq[i % kLen];
    return ch == 'A' ? 0u : ((kUseC && ch == 'C') ? 2u : 1u);
}

// smallest number of two-step groups after which the pattern repeats (what sequence_group_period finds at run time)
constexpr int min_group_period() {
    for (int kg = 1; kg <= 16; ++kg) {
        bool ok = true;
        for (int i = 0; i < 4 * kLen && ok; ++i) ok = code_at(i) == code_at(i + 2 * kg);
        if (ok) return kg;
    }
    return 0;
}
constexpr int kKG = min_group_period();
static_assert(kKG > 0, "the sequence has no group period up to 16");

constexpr unsigned long long pats_from(int first) {
    unsigned long long v = 0;
    for (int i = 0; i < 2 * kKG; ++i) v |= (unsigned long long)code_at(first + i) << (2 * i);
    return v;
}
constexpr unsigned long long kWuPats = pats_from(0), kAccPats = pats_from(kAccPhase);
constexpr int kThreads = 512;

}  // namespace

// named for what it is: k_lambda_exact_seq<pixels per thread, group period, warm-up patterns, accumulation patterns>
template <int P, int KG, unsigned long long WU, unsigned long long ACC>
__global__ void __launch_bounds__(512, 1)
k_lambda_exact_seq(const __grid_constant__ LambdaArgs a, double* __restrict__ out64, float* __restrict__ out32,
                   unsigned long long* __restrict__ steps_out) {
    lambda_exact_body<P, 512, pats_use_c(WU | ACC), 2, KG, WU, ACC>(a, out64, out32, steps_out);
}

template <typename T, int P, int KG, unsigned long long WU, unsigned long long ACC>
__global__ void __launch_bounds__(512)
k_lambda_fast_seq(const __grid_constant__ LambdaArgs a, double* __restrict__ out64, float* __restrict__ out32,
                  unsigned long long* __restrict__ steps_out) {
    lambda_fast_body<T, P, 512, KG, WU, ACC>(a, out64, out32, steps_out);
}

namespace {

struct Registrar {
    Registrar() {
        // the shapes the launchers ask for: exact 2 or 3 pixels per thread, fast fp64 4, fast fp32 2 (512 threads each)
        register_prebuilt({0, 3, kThreads, kKG, kWuPats, kAccPats,
                           reinterpret_cast<const void*>(&k_lambda_exact_seq<3, kKG, kWuPats, kAccPats>), kSeq});
        register_prebuilt({0, 2, kThreads, kKG, kWuPats, kAccPats,
                           reinterpret_cast<const void*>(&k_lambda_exact_seq<2, kKG, kWuPats, kAccPats>), kSeq});
        register_prebuilt({1, 4, kThreads, kKG, kWuPats, kAccPats,
                           reinterpret_cast<const void*>(&k_lambda_fast_seq<double, 4, kKG, kWuPats, kAccPats>), kSeq});
        register_prebuilt({2, 2, kThreads, kKG, kWuPats, kAccPats,
                           reinterpret_cast<const void*>(&k_lambda_fast_seq<float, 2, kKG, kWuPats, kAccPats>), kSeq});
    }
};
const Registrar g_registrar;

}  // namespace
}  // namespace lyap
