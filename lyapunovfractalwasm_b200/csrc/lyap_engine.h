// lyap_engine.h -- internal interface between the C ABI (lyap_abi.cu) and the kernels (lyap_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace lyap {

// Per-step parameter selectors, 2 bits per step (0 = A/column, 1 = B/row, 2 = C/scalar), 16 steps per
// 32-bit word.  Warm-up steps start at word 0, accumulation steps at word `acc_word0`, each region in
// its own words so both can be walked in whole 16-step chunks plus one partial chunk.
constexpr int kStepsPerWord = 16;
constexpr int kMaxSelWords = 896;  // 14336 steps through kernel parameters (kernel parameter space is 4 KB)

struct LambdaArgs {
    double min_x, min_y, dx, dy, c_value;
    long long row_begin;   // global index of the first row of this launch
    long long n_pixels;    // rows * width
    int width;
    int warmup, iterations;
    int acc_word0;
    int fast_ok_c;         // c_value is positive, finite and of ordinary magnitude (or unused)
    unsigned int sel[kMaxSelWords];
};

struct LaunchInfo {
    int sm_count;
};

cudaError_t launch_lambda_exact(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                int sm_count, cudaStream_t st);
cudaError_t launch_lambda_fast64(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st);
cudaError_t launch_lambda_fast32(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st);

// scratch for the min/max reduction: 2*kMinmaxBlocks doubles + one unsigned ticket (zero before first use;
// the kernel leaves it zero again)
constexpr int kMinmaxBlocks = 1184;  // 8 per SM on 148 SMs
constexpr size_t kMinmaxScratchBytes = 2 * kMinmaxBlocks * sizeof(double) + 16;
cudaError_t launch_minmax(const double* v, unsigned long long n, double* minmax, void* scratch, cudaStream_t st);
cudaError_t launch_normalize(const double* v, unsigned long long n, const double* minmax, double* out,
                             int sm_count, cudaStream_t st);
cudaError_t launch_colorize(const double* norm, int width, long long rows, int rows_above, int rows_below,
                            int palette, unsigned char* rgba, cudaStream_t st);

// issue-rate micro-benchmarks; return thread-level instructions executed per launch
cudaError_t launch_fp64_peak(double* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st);
cudaError_t launch_fp32_peak(float* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st);

// records the calling thread's last error message (implemented beside lyap_last_error)
int set_error(int status, const char* message);

}  // namespace lyap
