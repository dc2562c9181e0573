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

/* ========================================================================
 * Extensions beyond the reference kernels (still test infrastructure).
 *
 * orc_lif_forward_ext: lifForwardKernel (cuda/lif_kernels.h:58-91) with the two
 * options the B200 library adds to that step:
 *   in_scale  (nullable) multiplies the input per neuron; the product is rounded
 *             on its own and then enters the fused multiply-add, which is what a
 *             separate PyTorch multiplication in front of lifForward gives
 *             (sinabs/exodus/layers/lif.py:206-209);
 *   reset_to_value != 0   replaces "v -= act * subtract" (lif_kernels.h:63) by
 *             "v = subtract[n] where act > 0" -- not a reference mode: the
 *             reference layer rejects every reset but MembraneSubtract
 *             (sinabs/exodus/layers/lif.py:136-143).
 * ====================================================================== */
void orc_lif_forward_ext(float *spikes, float *vmem, const float *input,
                         const float *v_init, const float *alpha, const float *subtract,
                         const float *theta, const float *theta_low, int apply_theta_low,
                         uint32_t max_spikes, const float *in_scale /* nullable */,
                         int reset_to_value, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        float v = v_init[n];
        uint32_t act = 0;
        const float sc = in_scale ? in_scale[n] : 1.0f;
        for (int64_t t = 0; t < T; ++t) {
            if (reset_to_value) { if (act) v = subtract[n]; }
            else v = orc_fma(-(float)act, subtract[n], v);
            volatile float x = sc * input[n * T + t];
            v = orc_fma(v, alpha[n], x);
            if (apply_theta_low && v < theta_low[n]) v = theta_low[n];
            if (v >= theta[n]) act = orc_min_u32(orc_f2u_sat(v / theta[n]), max_spikes);
            else act = 0;
            spikes[n * T + t] = (float)act;
            vmem[n * T + t] = v;
        }
    }
}

/* ------------------------------------------------------------------------
 * Float64 adjoint of a LIF layer with synaptic stage, i.e. of the chain the
 * reference layer runs as leakyForward -> x*alpha -> (1-alpha)*i -> lifForward
 * (sinabs/exodus/layers/lif.py:185-258):
 *     i_t = a_s*i_{t-1} + s_s*x_t
 *     v_t = clip( a_m*post(v_{t-1}) + s_m*i_t ),  post = v - c*spikes  (or the
 *           reset value where a spike occurred when reset_to_value != 0)
 * linearised at the given v_mem / spikes / i_syn (the values the forward
 * produced), with ds/dv := surr (given, double).  Reverse sweep:
 *     g_t = surr_t*go_t + gv_t                       (spike.py:266)
 *     R_t = n_t*(g_t + f_t*R_{t+1}),  f_t = a_m*(1 - c*surr_t)   [subtract]
 *                                     f_t = a_m*[spikes_t == 0]  [reset to value]
 *     G_t = a_s*G_{t+1} + s_m*R_t + gis_t,   grad_x_t = s_s*G_t
 * A gradient on the state after the last reset enters through the last step's
 * go/gv (v_post = v - c*spikes; reset to value: passes only where no spike).
 * Parameter gradients per neuron instance: a_m: sum_t R_t*post_{t-1} (+ the
 * reference's first-step term, lif_kernels.h:219-238, subtract mode only),
 * s_m: sum_t R_t*i_t, a_s: sum_t G_t*i_{t-1}, s_s: sum_t G_t*x_t.
 * Every [N] / [N,T] argument is double; nullable ones are marked.
 * ---------------------------------------------------------------------- */
void orc_lif_syn_backward_f64(double *grad_input,
                              double *grad_alpha_mem, double *grad_scale_mem,      /* nullable */
                              double *grad_alpha_syn, double *grad_scale_syn,      /* nullable */
                              double *grad_v_init, double *grad_i_init,            /* nullable */
                              const double *grad_spikes, const double *grad_v_mem /* nullable */,
                              const double *grad_v_last /* nullable */, const double *grad_i_syn /* nullable */,
                              const double *grad_i_last /* nullable */,
                              const double *v_mem, const double *spikes, const double *i_syn,
                              const double *input, const double *surr,
                              const double *v_init, const double *i_init,
                              const double *alpha_syn, const double *scale_syn,
                              const double *scale_mem, const double *alpha_mem,
                              const double *subtract, const double *theta_low /* nullable */,
                              int reset_to_value, int64_t N, int64_t T)
{
#pragma omp parallel for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
        const int64_t row = n * T;
        const double am = alpha_mem[n], sm = scale_mem[n], as = alpha_syn[n], ss = scale_syn[n], c = subtract[n];
        double R = 0.0, G = 0.0, R1 = 0.0, f0 = 0.0;
        double gam = 0.0, gsm = 0.0, gas = 0.0, gss = 0.0;
        for (int64_t t = T - 1; t >= 0; --t) {
            const double v = v_mem[row + t], a = spikes[row + t], s = surr[row + t];
            double go = grad_spikes[row + t];
            double gv = grad_v_mem ? grad_v_mem[row + t] : 0.0;
            double gis = grad_i_syn ? grad_i_syn[row + t] : 0.0;
            if (t == T - 1) {
                if (grad_v_last) {
                    if (reset_to_value) gv += (a != 0.0) ? 0.0 : grad_v_last[n];
                    else { go -= c * grad_v_last[n]; gv += grad_v_last[n]; }
                }
                if (grad_i_last) gis += grad_i_last[n];
            }
            const double nt = (theta_low && !(v > theta_low[n])) ? 0.0 : 1.0;
            const double f = reset_to_value ? ((a != 0.0) ? 0.0 : am) : am * (1.0 - c * s);
            R1 = R;
            R = nt * (s * go + gv + f * R);
            if (t == 0) f0 = f;
            double post_prev, i_prev;
            if (t > 0) {
                const double vp = v_mem[row + t - 1], ap = spikes[row + t - 1];
                post_prev = reset_to_value ? ((ap != 0.0) ? c : vp) : vp - c * ap;
                i_prev = i_syn[row + t - 1];
            } else {
                post_prev = v_init[n];
                i_prev = i_init[n];
            }
            gam += R * post_prev;
            if (t == 0 && !reset_to_value && nt == 0.0) gam += v_init[n] * f0 * R1;
            gsm += R * i_syn[row + t];
            G = as * G + sm * R + gis;
            gas += G * i_prev;
            gss += G * input[row + t];
            grad_input[row + t] = ss * G;
        }
        if (grad_alpha_mem) grad_alpha_mem[n] = gam;
        if (grad_scale_mem) grad_scale_mem[n] = gsm;
        if (grad_alpha_syn) grad_alpha_syn[n] = gas;
        if (grad_scale_syn) grad_scale_syn[n] = gss;
        if (grad_v_init) grad_v_init[n] = am * R;
        if (grad_i_init) grad_i_init[n] = as * G;
    }
}
