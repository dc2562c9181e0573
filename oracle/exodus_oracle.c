/*
 * CPU restatement of the sinabs-exodus neuron kernels.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is the checker the CUDA library is compared against.  It is never
 * part of the shipped path: only the test-suite, the smoke check and the
 * CPU-baseline leg of the benchmark may load it.
 *
 * Every routine follows one reference kernel, with the CUDA thread index
 * replaced by a `for` over neurons.  All tensors are [N, T] row-major
 * (index n*T + t), float32, exactly like the reference's device tensors.
 *
 * Floating-point association.  The reference is compiled by nvcc with its
 * default -fmad=true, which contracts a*b+c into one fused multiply-add.
 * This file is compiled with -ffp-contract=off and spells every contraction
 * out with fmaf(), so the CPU result has the same roundings as the reference's
 * GPU build.  Building with -DORC_NO_FMA gives the un-contracted association
 * instead (used to show which one the reference build really has).
 *
 * Parity status: pinned against outputs of the reference's own kernels
 * (compiled for sm_100a from the reference sources and run on a B200); the
 * vectors live in tests/golden/ with the script that made them.
 *
 * Reference files followed (paths inside the reference project):
 *   cuda/lif_kernels.h    : lifForwardKernel 40-93, lifBackwardKernel 122-168,
 *                           lifBackwardAlphaKernel 199-246
 *   cuda/leaky_kernels.h  : leakyForwardKernel 29-58, leakyBackwardKernel 82-110,
 *                           leakyBackwardAlphaKernel 133-165
 *   sinabs/exodus/spike.py: IntegrateAndFire.backward 229-291 (glue restated in
 *                           orc_iaf_function_backward)
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>
#include <limits.h>

#ifdef ORC_NO_FMA
static inline float orc_fma(float a, float b, float c) { volatile float p = a * b; return p + c; }
#else
static inline float orc_fma(float a, float b, float c) { return fmaf(a, b, c); }
#endif

/* float -> unsigned with the semantics of the GPU's cvt.rzi.u32.f32:
 * truncate toward zero, saturate, NaN -> 0.  (A plain C cast is undefined
 * outside the range.) */
static inline uint32_t orc_f2u_sat(float x)
{
    if (!(x > 0.0f)) return 0u;                 /* negatives, -0, NaN */
    if (x >= 4294967296.0f) return UINT32_MAX;
    return (uint32_t)x;
}

static inline uint32_t orc_min_u32(uint32_t a, uint32_t b) { return a < b ? a : b; }

/* ------------------------------------------------------------------------
 * lifForwardKernel, cuda/lif_kernels.h:58-91
 * v_init is the state AFTER the previous reset.  vmem receives the state
 * BEFORE the reset of the same step.  max_spikes = UINT32_MAX means no limit
 * (cuda/bindings.cu:50-51 turns -1 into that value).
 * ---------------------------------------------------------------------- */
void orc_lif_forward(float *spikes, float *vmem, const float *input,
                     const float *v_init, const float *alpha, const float *subtract,
                     const float *theta, const float *theta_low, int apply_theta_low,
                     uint32_t max_spikes, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float v = v_init[n];
        uint32_t act = 0;
        for (int64_t t = 0; t < T; ++t) {
            /* lif_kernels.h:63  vmemCurr -= activation * membrSubtract */
            v = orc_fma(-(float)act, subtract[n], v);
            /* lif_kernels.h:66,72  vmemCurr *= alpha; vmemCurr += input */
            v = orc_fma(v, alpha[n], input[n * T + t]);
            /* lif_kernels.h:75-77 */
            if (apply_theta_low && v < theta_low[n]) v = theta_low[n];
            /* lif_kernels.h:80-84 */
            if (v >= theta[n]) act = orc_min_u32(orc_f2u_sat(v / theta[n]), max_spikes);
            else act = 0;
            spikes[n * T + t] = (float)act;
            vmem[n * T + t] = v;
        }
    }
}

/* ------------------------------------------------------------------------
 * lifBackwardKernel, cuda/lif_kernels.h:142-166.  One (neuron, i) pair per
 * CUDA thread there; two nested loops here.  `subtract_scaled` is alpha*c as
 * the caller passes it (sinabs/exodus/spike.py:269).
 * ---------------------------------------------------------------------- */
void orc_lif_backward(float *input_grad, const float *output_grad, const float *surr,
                      const float *not_clipped, const float *alpha,
                      const float *subtract_scaled, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int64_t row = n * T;
        for (int64_t i = 0; i < T; ++i) {
            float acc = not_clipped[row + i];
            float gi = output_grad[row + i] * acc;
            for (int64_t j = i + 1; j < T && acc != 0.0f; ++j) {
                float f = orc_fma(-subtract_scaled[n], surr[row + j - 1], alpha[n]);
                acc *= (f * not_clipped[row + j]);
                gi = orc_fma(acc, output_grad[row + j], gi);
            }
            input_grad[row + i] = gi;
        }
    }
}

/* ------------------------------------------------------------------------
 * lifBackwardAlphaKernel, cuda/lif_kernels.h:219-244.  The factor
 * alpha*(1.0 - c*surr) is evaluated in double there because of the double
 * literal (line 234): c*surr is a float product, the rest is double, and the
 * product with the float accumulator is rounded back to float.
 * ---------------------------------------------------------------------- */
void orc_lif_backward_alpha(float *alpha_grad, const float *output_grad,
                            const float *vmem_post, const float *v_init,
                            const float *surr, const float *not_clipped,
                            const float *alpha, const float *subtract, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int64_t row = n * T;
        float acc = v_init[n];
        float first = not_clipped[row] * acc;
        float ag = output_grad[row] * first;
        for (int64_t j = 1; j < T; ++j) {
            volatile float cs = subtract[n] * surr[row + j - 1];
            double fac = (double)alpha[n] * (1.0 - (double)cs);
            acc = (float)((double)acc * fac);
            acc += vmem_post[row + j - 1];
            acc *= not_clipped[row + j];
            ag = orc_fma(acc, output_grad[row + j], ag);
        }
        alpha_grad[n] = ag;
    }
}

/* leakyForwardKernel, cuda/leaky_kernels.h:41-56 */
void orc_leaky_forward(float *out, const float *input, const float *v_init,
                       const float *alpha, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float v = v_init[n];
        for (int64_t t = 0; t < T; ++t) {
            v = orc_fma(v, alpha[n], input[n * T + t]);
            out[n * T + t] = v;
        }
    }
}

/* leakyBackwardKernel, cuda/leaky_kernels.h:96-108 (reverse time) */
void orc_leaky_backward(float *input_grad, const float *output_grad, const float *alpha,
                        int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float g = 0.0f;
        for (int64_t t = T - 1; t >= 0; --t) {
            g = orc_fma(g, alpha[n], output_grad[n * T + t]);
            input_grad[n * T + t] = g;
        }
    }
}

/* leakyBackwardAlphaKernel, cuda/leaky_kernels.h:150-163 */
void orc_leaky_backward_alpha(float *alpha_grad, const float *output_grad, const float *output,
                              const float *v_init, const float *alpha, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int64_t row = n * T;
        float g = v_init[n];
        float ag = g * output_grad[row];
        for (int64_t t = 1; t < T; ++t) {
            g = orc_fma(alpha[n], g, output[row + t - 1]);
            ag = orc_fma(g, output_grad[row + t], ag);
        }
        alpha_grad[n] = ag;
    }
}

/* ========================================================================
 * Double-precision ground truth.  Same equations, evaluated in double, with
 * the backward written as the reverse-time recurrence
 *     R_t = n_t * (g_t + f_t * R_{t+1}),   f_t = alpha * (1 - c * s_t)
 * which is algebraically the same sum as lifBackwardKernel's double loop and
 * the adjoint of lifBackwardAlphaKernel's forward recurrence:
 *     alphaGrad = sum_t R_t * vpost_{t-1}  (+ the first-step term below).
 * Inputs are float arrays (the values the GPU saw); outputs are double.
 * ====================================================================== */
void orc_lif_backward_f64(double *input_grad, double *alpha_grad /* nullable */,
                          const float *output_grad, const float *surr,
                          const float *not_clipped, const float *vmem_post /* nullable */,
                          const float *v_init /* nullable */, const float *alpha,
                          const float *subtract, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int64_t row = n * T;
        const double a = alpha[n], c = subtract[n];
        double R = 0.0, ag = 0.0;
        for (int64_t t = T - 1; t >= 0; --t) {
            const double f = a * (1.0 - c * (double)surr[row + t]);
            const double Rn = R;              /* R_{t+1} */
            R = (double)not_clipped[row + t] * ((double)output_grad[row + t] + f * R);
            input_grad[row + t] = R;
            if (alpha_grad) {
                const double vprev = (t > 0) ? (double)vmem_post[row + t - 1] : (double)v_init[n];
                ag += R * vprev;
                /* lif_kernels.h:219-238: the t=0 accumulator is carried into
                 * t=1 without the t=0 clip gate. */
                if (t == 0) ag += (1.0 - (double)not_clipped[row]) * (double)v_init[n] * f * Rn;
            }
        }
        if (alpha_grad) alpha_grad[n] = ag;
    }
}

void orc_leaky_forward_f64(double *out, const float *input, const float *v_init,
                           const float *alpha, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        double v = v_init[n];
        for (int64_t t = 0; t < T; ++t) {
            v = v * (double)alpha[n] + (double)input[n * T + t];
            out[n * T + t] = v;
        }
    }
}

void orc_leaky_backward_f64(double *input_grad, double *alpha_grad /* nullable */,
                            const float *output_grad, const float *input /* nullable */,
                            const float *v_init /* nullable */, const float *alpha,
                            int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int64_t row = n * T;
        double g = 0.0;
        for (int64_t t = T - 1; t >= 0; --t) {
            g = g * (double)alpha[n] + (double)output_grad[row + t];
            input_grad[row + t] = g;
        }
        if (alpha_grad) {
            /* alphaGrad = sum_t inputGrad_t * v_{t-1}, v_{-1} = v_init, with v
             * re-integrated in double from the float input. */
            double v = v_init[n], ag = 0.0;
            for (int64_t t = 0; t < T; ++t) {
                ag += input_grad[row + t] * v;
                v = v * (double)alpha[n] + (double)input[row + t];
            }
            alpha_grad[n] = ag;
        }
    }
}
