// lyap_args.h -- kernel parameter block of the lambda kernels (plain types only: also compiled at run time).
#pragma once

namespace lyap {

// Per-step parameter selectors, 2 bits per step (0 = A/column, 1 = B/row, 2 = C/scalar), 16 steps per
// 32-bit word.  Warm-up steps start at word 0, accumulation steps at word `acc_word0`, each region in
// its own words so both can be walked in whole 16-step chunks plus one partial chunk.  A region longer than
// its share of the table stores one period of the sequence in whole words (lcm(len, 16) steps) and repeats
// it: word w of a region is sel[word0 + w % wrap].
constexpr int kStepsPerWord = 16;
constexpr int kMaxSelWords = 896;  // 14336 distinct steps through kernel parameters (kernel parameter space is 4 KB)

struct LambdaArgs {
    double min_x, min_y, dx, dy, c_value;
    long long row_begin;   // global index of the first row of this launch
    long long n_pixels;    // rows * width
    int width;
    int warmup, iterations;
    int acc_word0;
    int fast_ok_c;         // c_value is positive, finite and of ordinary magnitude (or unused)
    int wu_wrap, acc_wrap; // words after which each region's selectors repeat (>= the region's words when it is stored whole)
    unsigned int sel[kMaxSelWords];
};

}  // namespace lyap
