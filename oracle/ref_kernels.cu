/*
 * C-ABI launcher shim around the REFERENCE's own CUDA kernels.  TEST
 * INFRASTRUCTURE ONLY: nothing shipped links or loads the library built
 * from this file.
 *
 * The kernels themselves are not in this repository.  The two headers are
 * included from the reference checkout where it lies (the build recipe passes
 * -I<reference>/cuda), so the object code in oracle/_ref/libexodus_ref.so is
 * the reference's lifForwardKernel / lifBackwardKernel / ... compiled for
 * sm_100a, without libtorch or pybind11.  The only thing the headers need
 * from libtorch is the AT_ERROR macro (cuda/lif_kernels.h:373-374), replaced
 * here by an error flag.
 *
 * All pointers are device pointers, tensors [N, T] row-major float32, exactly
 * the arguments cuda/bindings.cu:14-257 hands to the launchers.  As in the
 * reference, launches go to the legacy default stream; ref_sync() waits for
 * them and returns the CUDA error state.
 */
#include <cuda_runtime.h>
#include <cmath>
#include <cstdio>

static int g_ref_error = 0;
#define AT_ERROR(...) do { g_ref_error = 1; } while (0)

#include "lif_kernels.h"
#include "leaky_kernels.h"

extern "C" {

int ref_sync(void)
{
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaGetLastError();
    int flag = g_ref_error;
    g_ref_error = 0;
    return (e == cudaSuccess && !flag) ? 0 : (flag ? -1 : (int)e);
}

/* cuda/bindings.cu:14-70 */
void ref_lif_forward(float *spikes, float *vmem, const float *input, const float *v_init,
                     const float *alpha, const float *subtract, const float *theta,
                     const float *theta_low, int apply_theta_low, int max_spikes,
                     unsigned N, unsigned T)
{
    lifForwardCuda<float>(spikes, vmem, input, v_init, alpha, subtract, theta, theta_low,
                          apply_theta_low != 0, (unsigned)max_spikes, N, T);
}

/* cuda/bindings.cu:72-110 */
void ref_lif_backward(float *input_grad, const float *output_grad, const float *surr,
                      const float *not_clipped, const float *alpha, const float *subtract_scaled,
                      unsigned N, unsigned T)
{
    lifBackwardCuda<float>(input_grad, output_grad, surr, not_clipped, alpha, subtract_scaled, N, T);
}

/* cuda/bindings.cu:112-158 */
void ref_lif_backward_alpha(float *alpha_grad, const float *output_grad, const float *vmem_post,
                            const float *v_init, const float *surr, const float *not_clipped,
                            const float *alpha, const float *subtract, unsigned N, unsigned T)
{
    lifBackwardAlphaCuda<float>(alpha_grad, output_grad, vmem_post, v_init, surr, not_clipped,
                                alpha, subtract, N, T);
}

/* cuda/bindings.cu:163-193 */
void ref_leaky_forward(float *out, const float *input, const float *v_init, const float *alpha,
                       unsigned N, unsigned T)
{
    leakyForwardCuda<float>(out, input, v_init, alpha, N, T);
}

/* cuda/bindings.cu:195-221 */
void ref_leaky_backward(float *input_grad, const float *output_grad, const float *alpha,
                        unsigned N, unsigned T)
{
    leakyBackwardCuda<float>(input_grad, output_grad, alpha, N, T);
}

/* cuda/bindings.cu:223-257 */
void ref_leaky_backward_alpha(float *alpha_grad, const float *output_grad, const float *output,
                              const float *v_init, const float *alpha, unsigned N, unsigned T)
{
    leakyBackwardAlphaCuda<float>(alpha_grad, output_grad, output, v_init, alpha, N, T);
}

}  // extern "C"
