// lyap_engine.h -- internal interface between the C ABI (lyap_abi.cu) and the kernels (lyap_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "lyap_args.h"

namespace lyap {

struct LaunchInfo {
    int sm_count;
};

cudaError_t launch_lambda_exact(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                int sm_count, cudaStream_t st);
cudaError_t launch_lambda_fast64(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st);
cudaError_t launch_lambda_fast32(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st);

// run-time specialised instance of a lambda kernel (lyap_jit.cu); kind: 0 exact, 1 fast fp64, 2 fast fp32.
// *launched == false means "not used, launch the precompiled kernel".  mode: 0 never, 1 once enough work with this
// sequence has been seen, 2 always.
cudaError_t launch_lambda_spec(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps, int sm_count,
                               cudaStream_t st, int kind, int pixels_per_thread, int threads, size_t smem_bytes, int mode,
                               bool* launched);
const char* jit_last_note();
// Group-pattern period of the sequence in `a` (1..16) with the two regions' patterns, or 0 when there is none.
int sequence_group_period(const LambdaArgs& a, unsigned long long* wu_pats, unsigned long long* acc_pats);

// scratch for the min/max reduction: 2*kMinmaxBlocks doubles + one unsigned ticket (zero before first use;
// the kernel leaves it zero again)
constexpr int kMinmaxBlocks = 1184;  // 8 per SM on 148 SMs
constexpr size_t kMinmaxScratchBytes = 2 * kMinmaxBlocks * sizeof(double) + 16;
cudaError_t launch_minmax(const double* v, unsigned long long n, double* minmax, void* scratch, cudaStream_t st);
cudaError_t launch_normalize(const double* v, unsigned long long n, const double* minmax, double* out,
                             int sm_count, cudaStream_t st);
cudaError_t launch_colorize(const double* norm, int width, long long rows, int rows_above, int rows_below,
                            int palette, unsigned char* rgba, cudaStream_t st);

// glow on an RGBA8 canvas in place; scratch holds width*height*3 doubles
cudaError_t launch_glow(unsigned char* canvas, int width, int height, double* scratch, cudaStream_t st);

// issue-rate micro-benchmarks; return thread-level instructions executed per launch
cudaError_t launch_fp64_peak(double* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st);
cudaError_t launch_fp32_peak(float* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st);

// records the calling thread's last error message (implemented beside lyap_last_error)
int set_error(int status, const char* message);

}  // namespace lyap
