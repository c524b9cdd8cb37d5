// lyap_engine.h -- internal interface between the C ABI (lyap_abi.cu) and the kernels (lyap_kernels.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "lyap_args.h"

struct lyap_params;

namespace lyap {

cudaError_t launch_lambda_exact(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                int sm_count, cudaStream_t st);
cudaError_t launch_lambda_fast64(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st);
cudaError_t launch_lambda_fast32(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                 int sm_count, cudaStream_t st);
cudaError_t launch_lambda_orbit64(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps,
                                  int sm_count, cudaStream_t st);

// Instance of a lambda kernel made for the sequence's patterns (lyap_jit.cu); kind: 0 exact, 1 fast fp64, 2 fast fp32, 3 fast fp64 on the exact orbit.
// *launched == false means "not used, launch the generic kernel".  mode: low two bits say when to compile at run time
// (0 never, 1 once enough work with this sequence has been seen, 2 at once); kSpecUsePrebuilt allows the instances
// compiled at build time (lyap_prebuilt.cu), which are tried first.
constexpr int kSpecUsePrebuilt = 4;
cudaError_t launch_lambda_spec(const LambdaArgs& a, double* out64, float* out32, unsigned long long* steps, int sm_count,
                               cudaStream_t st, int kind, int pixels_per_thread, int threads, size_t smem_bytes, int mode,
                               bool* launched);
const char* jit_last_note();
// Name of the lambda kernel the calling thread launched last ("" before the first launch), with how it was made:
// "... (built for this sequence)", "... (compiled at run time)", or the generic kernel's name.
const char* last_lambda_kernel();
void note_lambda_kernel(const char* text);

// A lambda kernel compiled at build time for one sequence's patterns: device code (a cubin for sm_100a) embedded in the
// library, made by build.py with the same compiler, source text and options as a run-time instance (lyap_prebuilt.cu).
// kind: 0 exact, 1 fast fp64, 2 fast fp32, 3 fast fp64 on the exact orbit.  launch_lambda_spec prefers a matching entry to compiling at run time.
struct PrebuiltKernel {
    int kind, pixels_per_thread, threads, kg;
    unsigned long long wu_pats, acc_pats;
    const unsigned char* cubin;
    size_t cubin_bytes;
    const char* sequence;
};
void register_prebuilt(const PrebuiltKernel& k);
// Group-pattern period of the sequence in `a` (1..16) with the two regions' patterns, or 0 when there is none.
int sequence_group_period(const LambdaArgs& a, unsigned long long* wu_pats, unsigned long long* acc_pats);

// scratch for the min/max reduction: 2*kMinmaxBlocks doubles + one unsigned ticket (zero before first use;
// the kernel leaves it zero again)
constexpr int kMinmaxBlocks = 1184;  // upper bound of the grid (8 blocks per SM on a 148-SM part); sizes the scratch
constexpr size_t kMinmaxScratchBytes = 2 * kMinmaxBlocks * sizeof(double) + 16;
cudaError_t launch_minmax(const double* v, unsigned long long n, double* minmax, void* scratch, int sm_count, cudaStream_t st);
cudaError_t launch_normalize(const double* v, unsigned long long n, const double* minmax, double* out,
                             int sm_count, cudaStream_t st);
cudaError_t launch_colorize(const double* norm, int width, long long rows, int rows_above, int rows_below,
                            int palette, unsigned char* rgba, int sm_count, cudaStream_t st);

// glow on an RGBA8 canvas in place; scratch holds width*height*3 doubles
cudaError_t launch_glow(unsigned char* canvas, int width, int height, double* scratch, int sm_count, cudaStream_t st);

// issue-rate micro-benchmarks; return thread-level instructions executed per launch
cudaError_t launch_fp64_peak(double* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st);
cudaError_t launch_fp32_peak(float* sink, int sm_count, int iters, unsigned long long* instr, cudaStream_t st);

// records the calling thread's last error message (implemented beside lyap_last_error)
int set_error(int status, const char* message);
// the parameter checks of the lambda entry points, for a whole frame (needs no device)
int validate_whole_frame(const ::lyap_params* p);

}  // namespace lyap
