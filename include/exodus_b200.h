/*
 * exodus_b200 -- C ABI of the B200 (sm_100a) neuron kernels.
 *
 * libexodus_b200.so replaces the pybind11 module `exodus_cuda` of the
 * reference (cuda/bindings.cu:362-373).  Every entry point takes raw device
 * pointers and sizes, launches on the stream it is given, allocates nothing
 * and returns an int status (0 = EXB_OK).  The only state kept between calls
 * is a device status word per kernel family (see exb_device_status) and the
 * built-in scratch array of exb_leaky_forward_scan_static.  No
 * exception crosses this boundary; exb_last_error() gives the text of the
 * calling thread's most recent failure.
 *
 * Tensors.  A problem is N = B*M independent neurons over T time steps, all
 * float32.  Neuron n = b*M + m.  Two storage layouts of a [N, T] tensor:
 *
 *   EXB_LAYOUT_NT   element (n, t) at  n*T + t            (time contiguous; the
 *                   layout of the reference's kernels and autograd Functions)
 *   EXB_LAYOUT_BTM  element (b, t, m) at (b*T + t)*M + m  (neurons contiguous,
 *                   "time-major"; a layer's own (batch, time, ...) tensor, so
 *                   every time step is one coalesced sweep over neurons)
 *
 * Per-neuron parameters (alpha, threshold, ...) are never expanded to N
 * values by the caller; each comes with a mode:
 *
 *   EXB_PARAM_SCALAR   one value                       p[0]
 *   EXB_PARAM_PER_M    M values shared over the batch  p[m]
 *   EXB_PARAM_PER_N    N values                        p[b*M + m]
 *
 * State vectors (v_init, v_post_last, grad_init, per-instance alpha grads) are
 * always N values indexed b*M + m, in both layouts.
 */
#ifndef EXODUS_B200_H
#define EXODUS_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { EXB_OK = 0, EXB_ERR_ARG = 1, EXB_ERR_ALIGN = 2, EXB_ERR_LAUNCH = 3, EXB_ERR_UNSUPPORTED = 4,
       EXB_ERR_DEVICE = 5, EXB_ERR_TIMEOUT = 6 };

enum { EXB_LAYOUT_NT = 0, EXB_LAYOUT_BTM = 1 };
enum { EXB_PARAM_SCALAR = 0, EXB_PARAM_PER_M = 1, EXB_PARAM_PER_N = 2, EXB_PARAM_SHAPE_MASK = 3 };

/* Bits that may be OR-ed into a mode to let the kernels derive the decay and the input scale of a stage from
 * what a layer actually owns, so that the small tensor operations of the reference layer around its kernels
 * (layers/lif.py:188,194-195,204-214: exp(-1/tau), 1 - alpha, x * alpha) need no launches of their own:
 *   on an alpha argument  EXB_PARAM_IS_TAU           the values are time constants; alpha = exp(-1/tau)
 *   on a scale argument   EXB_SCALE_ONE_MINUS_ALPHA  the scale is 1 - alpha of the same stage (pointer must be NULL)
 *                         EXB_SCALE_TIMES_ALPHA      the scale (given, 1 - alpha, or 1) is multiplied by alpha
 * The roundings are those of the PyTorch expressions they replace. */
enum { EXB_PARAM_IS_TAU = 0x10, EXB_SCALE_ONE_MINUS_ALPHA = 0x20, EXB_SCALE_TIMES_ALPHA = 0x40 };

/* What happens to the membrane after a step that emitted spikes.
 * SUBTRACT: v <- v - a*c       (the reference's only mode, cuda/lif_kernels.h:63)
 * TO_VALUE: v <- c where a > 0 (extension: `subtract` then holds the reset value) */
enum { EXB_RESET_SUBTRACT = 0, EXB_RESET_TO_VALUE = 1 };

/* Surrogate gradient ds/dv evaluated inside the backward kernel from the saved
 * membrane potential.  p0, p1 are the two float parameters.
 * GENERIC            : read a caller-computed tensor `surr` (any callable)
 * SINGLE_EXPONENTIAL : p1/(p0*theta) * exp(-|v-theta| / (p0*theta))     p0=grad_width p1=grad_scale
 * HEAVISIDE          : [v >= theta - p0] / theta                        p0=window
 * PERIODIC_EXPONENTIAL: u=v-theta/2; w = v<theta ? u : u-floor(u/theta);
 *                       p1 * exp(-|w-theta/2| / p0) / theta             p0=grad_width p1=grad_scale */
enum { EXB_SURR_GENERIC = 0, EXB_SURR_SINGLE_EXPONENTIAL = 1, EXB_SURR_HEAVISIDE = 2,
       EXB_SURR_PERIODIC_EXPONENTIAL = 3 };

#define EXB_MAX_SPIKES_UNLIMITED 0xFFFFFFFFu

const char *exb_version(void);
const char *exb_last_error(void);
const char *exb_status_string(int status);

/* Kernels that stage data through TMA wait on shared-memory barriers; every such
 * wait is bounded.  If one ever runs out, the kernel records it in a device
 * status word, writes NaN to the per-neuron results of the affected neurons
 * (final states, initial-state and parameter gradients, the output sum) and
 * returns normally.  exb_device_status waits for `stream`,
 * returns EXB_ERR_TIMEOUT if that happened since the last query (and clears the
 * word), EXB_OK otherwise.  No counterpart in the reference, whose kernels
 * never wait (cuda/lif_kernels.h, cuda/leaky_kernels.h). */
int exb_device_status(int device, void *stream);

/* Sets, on `device`, how many polls a bounded wait may take before it gives up (0 = the default,
 * 2^22, several seconds), and a diagnostic switch: with withhold_scan_flags != 0 the segments of
 * the time-parallel leaky scan (exb_leaky_*_scan*) do not raise their ready flags, so every
 * dependent segment's wait runs out.  That is how the give-up path can be exercised without any
 * fault: the kernel returns normally, exb_device_status reports EXB_ERR_TIMEOUT once, and the
 * per-neuron results the wait belonged to (final states, parameter gradients, output sum) are
 * NaN.  Applies to kernels launched afterwards; call it with (device, 0, 0) to restore the defaults.
 * Synchronous (a constant upload); not for the steady state.  No counterpart in the reference. */
int exb_set_wait_limit(int device, uint32_t polls, int withhold_scan_flags);

/* Forward spike scan.  Replaces lifForward (cuda/bindings.cu:14-70, kernel
 * cuda/lif_kernels.h:40-93).  Per neuron and step:
 *     v <- (v - a*c)*alpha + in_t ; v <- max(v, theta_low) ; a <- v >= theta ? min(trunc(v/theta), max_spikes) : 0
 * spikes_t = a, v_mem_t = v (before the reset).  v_init is the state after the
 * previous reset (NULL = 0).  theta_low NULL = no lower bound.  in_scale
 * (NULL = 1) multiplies in_t per neuron and fuses the layer's norm_input
 * factor (layers/lif.py:206-209).
 * Optional fused outputs (NULL to skip): v_post_last[N] = state after the
 * reset of the last step; spike_count[1] += total number of spikes (exact
 * integer; the caller zeroes it).
 * v_mem may be NULL for a forward pass that is neither differentiated nor recorded (8 instead of
 * 12 bytes per neuron-step): time-major layout, M % 4 == 0 and 16-byte aligned tensors only,
 * otherwise EXB_ERR_UNSUPPORTED.  The reference always writes it (cuda/lif_kernels.h:88). */
int exb_lif_forward(float *spikes, float *v_mem, const float *input, const float *v_init,
                    const float *in_scale, int in_scale_mode,
                    const float *alpha, int alpha_mode,
                    const float *subtract, int subtract_mode,
                    const float *theta, int theta_mode,
                    const float *theta_low, int theta_low_mode,
                    uint32_t max_spikes, int reset_mode,
                    float *v_post_last, unsigned long long *spike_count,
                    int64_t B, int64_t T, int64_t M, int layout,
                    int device, void *stream);

/* exb_lif_forward that also records the membrane potential AFTER each step's reset:
 * v_post[b,t,m] = v_mem - subtract * spikes (EXB_RESET_SUBTRACT; product rounded first, as
 * the layer's PyTorch expression layers/lif.py:256 does) or the reset value where a spike
 * occurred (EXB_RESET_TO_VALUE).  It is what a layer with record_states stores
 * (layers/lif.py:299-300); written by the same launch, 4 more bytes per neuron-step instead
 * of a read-read-write pass.  Time-major layout only (EXB_ERR_UNSUPPORTED otherwise). */
int exb_lif_forward_record(float *spikes, float *v_mem, float *v_post, const float *input, const float *v_init,
                           const float *in_scale, int in_scale_mode,
                           const float *alpha, int alpha_mode,
                           const float *subtract, int subtract_mode,
                           const float *theta, int theta_mode,
                           const float *theta_low, int theta_low_mode,
                           uint32_t max_spikes, int reset_mode,
                           float *v_post_last, unsigned long long *spike_count,
                           int64_t B, int64_t T, int64_t M, int layout,
                           int device, void *stream);

/* exb_lif_forward with the spike raster as one byte per neuron-step instead of a float32.  The reference stores
 * the count as float (cuda/lif_kernels.h:87 `static_cast<float>(activation)`) and hands that raster to the next
 * layer (layers/lif.py:296-297); a consumer that can take bytes saves 3 of the forward's 12 bytes per neuron-step.
 * Counts above 255 are stored as 255: with max_spikes > 255 (EXB_MAX_SPIKES_UNLIMITED included) the caller must say
 * that this is acceptable (saturate != 0), else EXB_ERR_ARG; the membrane always resets by the true count, and
 * spike_count receives the true total.  v_mem may be NULL: a forward pass that is neither differentiated nor
 * recorded needs only the spikes (5 bytes per neuron-step in all).  Time-major layout, M % 4 == 0 and 16-byte
 * aligned tensors only; otherwise EXB_ERR_UNSUPPORTED and the caller uses exb_lif_forward. */
int exb_lif_forward_u8(uint8_t *spikes, float *v_mem, const float *input, const float *v_init,
                       const float *in_scale, int in_scale_mode,
                       const float *alpha, int alpha_mode,
                       const float *subtract, int subtract_mode,
                       const float *theta, int theta_mode,
                       const float *theta_low, int theta_low_mode,
                       uint32_t max_spikes, int reset_mode, int saturate,
                       float *v_post_last, unsigned long long *spike_count,
                       int64_t B, int64_t T, int64_t M, int device, void *stream);

/* Fused reverse-time EXODUS backward.  Replaces lifBackward + lifBackwardAlpha
 * (cuda/bindings.cu:72-158, kernels cuda/lif_kernels.h:122-168, 199-246) and
 * the tensor glue of IntegrateAndFire.backward (sinabs/exodus/spike.py:251-289):
 * one pass over the saved v_mem computes the surrogate s_t, the clip gate
 * n_t = [v_t > theta_low], g_t = s_t*grad_spikes_t + grad_v_mem_t and
 *     R_t = n_t * (g_t + (alpha - alpha*c*s_t) * R_{t+1}),  grad_input_t = R_t.
 * grad_v_mem may be NULL (no gradient through v_mem).  grad_v_last[N] (may be
 * NULL) is a gradient w.r.t. v_post_last of the forward call.
 * grad_init[N] (may be NULL) = alpha * R_0 (spike.py:289).
 * grad_alpha[N] (may be NULL) = per-instance d/d alpha (needs v_init or NULL=0);
 * the spike counts are recomputed from v_mem, so `spikes` is not read.
 * `surr` is read only with EXB_SURR_GENERIC.  With in_scale the kernel writes
 * grad_input_t = scale*R_t, and grad_scale[N] (may be NULL) = sum_t R_t*in_t.
 * With `input` (the forward's unscaled input) given, that sum reads it.  With
 * input == NULL it is rebuilt from v_mem alone, using
 * scale*in_t = v_t - alpha*vpost_{t-1} wherever R_t != 0, at no extra memory
 * traffic; this needs every scale to be non-zero.
 * acc_decay (may be NULL; time-major TMA-eligible shapes only, else EXB_ERR_UNSUPPORTED): float64
 * accumulator with the SHAPE OF THE ALPHA ARGUMENT (1, M or B*M values), zeroed by the caller, to which
 * the kernel adds the gradient with respect to the values passed as `alpha` -- alpha or, with
 * EXB_PARAM_IS_TAU, tau -- including the part that reaches them through a scale derived from alpha
 * (EXB_SCALE_* bits).  It replaces grad_alpha / grad_scale (both must then be NULL) and the reduction
 * over the batch and the chain rule that the reference leaves to autograd (layers/lif.py:43-44,204). */
int exb_lif_backward(float *grad_input, float *grad_alpha, float *grad_init, float *grad_scale,
                     const float *grad_spikes, const float *grad_v_mem, const float *grad_v_last,
                     const float *v_mem, const float *surr, const float *v_init, const float *input,
                     const float *in_scale, int in_scale_mode,
                     const float *alpha, int alpha_mode,
                     const float *subtract, int subtract_mode,
                     const float *theta, int theta_mode,
                     const float *theta_low, int theta_low_mode,
                     uint32_t max_spikes, int reset_mode,
                     int surrogate_kind, float surr_p0, float surr_p1, double *acc_decay,
                     int64_t B, int64_t T, int64_t M, int layout,
                     int device, void *stream);

/* Forward and backward of a training step that never materialises v_mem.  No counterpart in the reference, whose
 * forward always writes v_mem and whose backward reads it (cuda/lif_kernels.h:88, sinabs/exodus/spike.py:200,246).
 * exb_lif_forward_ckpt is exb_lif_forward with, instead of v_mem, the state that enters every EXB_CKPT_EVERY-th
 * step: ckpt[b, j, m] = post-reset potential before step j * EXB_CKPT_EVERY (the initial state for j = 0), a
 * [B][ceil(T / EXB_CKPT_EVERY)][M] tensor, one eighth of v_mem.  exb_lif_backward_ckpt is exb_lif_backward with
 * (input, ckpt) in place of v_mem: for every chunk of EXB_CKPT_EVERY steps it repeats the forward recurrence from
 * the chunk's checkpoint with the forward kernel's own step arithmetic, which yields v_mem bit for bit, and then
 * runs the reverse recurrence on it, so all gradients equal those of exb_lif_backward on the v_mem that
 * exb_lif_forward writes.  The forward then moves 8.5 instead of 12 bytes per neuron-step, the backward 12.5
 * instead of 12, and 7/8 of v_mem's memory is never allocated.  Not available: a gradient arriving on v_mem, the
 * generic surrogate (both need the tensor), the [N,T] layout.  `input` is the forward's unscaled input; the scale
 * gradient is always rebuilt from the state (needs non-zero scales).  Time-major layout, M % 4 == 0 and 16-byte
 * aligned tensors only; otherwise EXB_ERR_UNSUPPORTED and the caller uses the v_mem pair. */
#define EXB_CKPT_EVERY 8
int exb_lif_forward_ckpt(float *spikes, float *ckpt, const float *input, const float *v_init,
                         const float *in_scale, int in_scale_mode,
                         const float *alpha, int alpha_mode,
                         const float *subtract, int subtract_mode,
                         const float *theta, int theta_mode,
                         const float *theta_low, int theta_low_mode,
                         uint32_t max_spikes, int reset_mode,
                         float *v_post_last, unsigned long long *spike_count,
                         int64_t B, int64_t T, int64_t M, int device, void *stream);
int exb_lif_backward_ckpt(float *grad_input, float *grad_alpha, float *grad_init, float *grad_scale,
                          const float *grad_spikes, const float *grad_v_last,
                          const float *input, const float *ckpt, const float *v_init,
                          const float *in_scale, int in_scale_mode,
                          const float *alpha, int alpha_mode,
                          const float *subtract, int subtract_mode,
                          const float *theta, int theta_mode,
                          const float *theta_low, int theta_low_mode,
                          uint32_t max_spikes, int reset_mode,
                          int surrogate_kind, float surr_p0, float surr_p1, double *acc_decay,
                          int64_t B, int64_t T, int64_t M, int device, void *stream);

/* Converts float64 accumulators that the backward entry points filled (acc_decay) to the float32 gradient
 * tensor `out` and clears them, so that the same accumulator serves the next backward pass:
 * out[i] = (float) acc[i]; acc[i] = 0, for i < n.  One small launch.  No counterpart in the reference, which
 * leaves the reduction to autograd's expand-backward (layers/lif.py:43-44). */
int exb_acc_finish(float *out, double *acc, int64_t n, int device, void *stream);

/* One-shot sum-allreduce of a small float vector between the GPUs of one node, for the time-constant
 * gradients that batch-sharded ranks exchange once per step (a few KB: launch latency, not bandwidth).
 * `buffers` and `signals` are device arrays of `world` addresses: buffers[p] is rank p's data area of
 * 2*n floats, signals[p] its signal area of 2*world uint32 (zero before the first call), both mapped into
 * this process (CUDA peer / fabric mapping, e.g. PyTorch symmetric memory).  Every rank calls with the same
 * n and the same epoch, which starts at 1 and grows by 1 per call.  One CTA: publishes `in` in the own area,
 * signals every peer, waits -- bounded, see exb_set_wait_limit -- for every peer's signal, and adds all
 * ranks' vectors in rank order with plain peer loads, so all ranks get the same bits in `out`.  If a peer
 * does not arrive in time, `out` is NaN and exb_device_status reports EXB_ERR_TIMEOUT.  No counterpart in
 * the reference (which is single-GPU); the library's default exchange is an NCCL allreduce. */
int exb_allreduce_oneshot(float *out, const float *in, const uint64_t *buffers, const uint64_t *signals,
                          int rank, int world, int64_t n, uint32_t epoch, int device, void *stream);

/* Leaky integrator forward, v_t = alpha*v_{t-1} + scale*in_t.  Replaces
 * leakyForward (cuda/bindings.cu:163-193, kernel cuda/leaky_kernels.h:29-58).
 * in_scale (NULL = 1) is a per-neuron factor on the input that fuses the
 * layer's decay_early / norm_input multiplications (layers/lif.py:194-195,
 * 206-214).  v_last[N] (may be NULL) receives v_{T-1}.  out_sum (may be NULL)
 * points at one double on the device, zeroed by the caller, to which the sum of
 * all outputs is added: the layer's `output.sum() / numel` (layers/lif.py:305)
 * without another pass over the output. */
int exb_leaky_forward(float *out, const float *input, const float *v_init,
                      const float *alpha, int alpha_mode,
                      const float *in_scale, int in_scale_mode,
                      float *v_last, double *out_sum,
                      int64_t B, int64_t T, int64_t M, int layout,
                      int device, void *stream);

/* Leaky integrator backward, G_t = alpha*G_{t+1} + grad_out_t, grad_input_t =
 * scale*G_t.  Replaces leakyBackward + leakyBackwardAlpha (cuda/bindings.cu:195-257,
 * kernels cuda/leaky_kernels.h:82-110, 133-165).  grad_v_last[N] (may be NULL)
 * is added to grad_out at t = T-1.  grad_init[N] (may be NULL) = alpha*G_0.
 * grad_alpha[N] (may be NULL) = sum_t G_t * out_{t-1}, out_{-1} = v_init; it
 * needs `out` (the forward result).  grad_scale[N] (may be NULL) =
 * sum_t G_t * in_t needs `input`.  acc_decay: as for exb_lif_backward (needs `out`, and `input` when the
 * scale is derived from alpha). */
int exb_leaky_backward(float *grad_input, float *grad_alpha, float *grad_init, float *grad_scale,
                       const float *grad_out, const float *grad_v_last,
                       const float *out, const float *input, const float *v_init,
                       const float *alpha, int alpha_mode,
                       const float *in_scale, int in_scale_mode, double *acc_decay,
                       int64_t B, int64_t T, int64_t M, int layout,
                       int device, void *stream);

/* LIF layer with synaptic stage in one kernel per direction (time-major layout only, M % 4 == 0,
 * 16-byte aligned tensors; otherwise EXB_ERR_UNSUPPORTED and the caller chains exb_leaky_* and
 * exb_lif_*).  The reference runs the two stages as separate kernels with PyTorch passes in between
 * (layers/lif.py:185-198, 200-258: leakyForward, x*alpha, (1-alpha)*i, lifForward).
 *   i_t = alpha_syn*i_{t-1} + scale_syn*in_t ;  membrane step of exb_lif_forward on scale_mem*i_t
 * Forward writes i_syn, spikes, v_mem (+ optional v_post_last[N], i_last[N], spike_count); v_mem and i_syn may
 * both be NULL for a pass that is neither differentiated nor recorded (8 instead of 16 bytes per neuron-step).
 * Backward takes gradients w.r.t. spikes and optionally v_mem, v_post_last, i_syn, i_last, and
 * writes grad_input, optional grad_v_init / grad_i_init, and -- all four or none -- the
 * per-instance gradients w.r.t. alpha_mem, scale_mem, alpha_syn, scale_syn (these need `i_syn`;
 * scale_syn must be non-zero: its gradient is rebuilt from i_t - alpha_syn*i_{t-1}).
 * acc_decay_mem / acc_decay_syn (both or neither; they replace the four per-instance outputs): float64
 * accumulators shaped like alpha_mem / alpha_syn, as acc_decay of exb_lif_backward, one per stage. */
int exb_lif_syn_forward(float *spikes, float *v_mem, float *i_syn, const float *input,
                        const float *v_init, const float *i_init,
                        const float *alpha_syn, int alpha_syn_mode, const float *scale_syn, int scale_syn_mode,
                        const float *scale_mem, int scale_mem_mode,
                        const float *alpha_mem, int alpha_mem_mode,
                        const float *subtract, int subtract_mode,
                        const float *theta, int theta_mode,
                        const float *theta_low, int theta_low_mode,
                        uint32_t max_spikes, int reset_mode,
                        float *v_post_last, float *i_last, unsigned long long *spike_count,
                        int64_t B, int64_t T, int64_t M, int device, void *stream);

/* exb_lif_syn_forward with the byte raster of exb_lif_forward_u8 (same saturation rule).  v_mem and i_syn may both
 * be NULL (inference: only the spikes and the final states are written, 5 bytes per neuron-step instead of 16). */
int exb_lif_syn_forward_u8(uint8_t *spikes, float *v_mem, float *i_syn, const float *input,
                           const float *v_init, const float *i_init,
                           const float *alpha_syn, int alpha_syn_mode, const float *scale_syn, int scale_syn_mode,
                           const float *scale_mem, int scale_mem_mode,
                           const float *alpha_mem, int alpha_mem_mode,
                           const float *subtract, int subtract_mode,
                           const float *theta, int theta_mode,
                           const float *theta_low, int theta_low_mode,
                           uint32_t max_spikes, int reset_mode, int saturate,
                           float *v_post_last, float *i_last, unsigned long long *spike_count,
                           int64_t B, int64_t T, int64_t M, int device, void *stream);

int exb_lif_syn_backward(float *grad_input,
                         float *grad_alpha_mem, float *grad_scale_mem, float *grad_alpha_syn, float *grad_scale_syn,
                         float *grad_v_init, float *grad_i_init,
                         const float *grad_spikes, const float *grad_v_mem, const float *grad_v_last,
                         const float *grad_i_syn, const float *grad_i_last,
                         const float *v_mem, const float *i_syn, const float *surr,
                         const float *v_init, const float *i_init,
                         const float *alpha_syn, int alpha_syn_mode, const float *scale_syn, int scale_syn_mode,
                         const float *scale_mem, int scale_mem_mode,
                         const float *alpha_mem, int alpha_mem_mode,
                         const float *subtract, int subtract_mode,
                         const float *theta, int theta_mode,
                         const float *theta_low, int theta_low_mode,
                         uint32_t max_spikes, int reset_mode,
                         int surrogate_kind, float surr_p0, float surr_p1,
                         double *acc_decay_mem, double *acc_decay_syn,
                         int64_t B, int64_t T, int64_t M, int device, void *stream);

/* Time-parallel variants of the leaky integrator for long sequences with few neurons
 * (time-major layout only).  The reference has one thread per neuron walking through all of
 * T (cuda/leaky_kernels.h:41-56, 96-108), which leaves the GPU empty when N is small; here
 * the time axis is cut into segments that run in different CTAs and exchange their end states
 * through `workspace`, caller-provided device scratch memory of at least
 * exb_leaky_scan_workspace_bytes(B, T, M) bytes, 16-byte aligned.  That function returns 0 when
 * splitting is not applicable (short T, M % 4 != 0); the scan entry points then return
 * EXB_ERR_UNSUPPORTED and the caller uses exb_leaky_forward / exb_leaky_backward.  Arguments
 * and results are those of the plain entry points; results agree to rounding (the carry
 * across segments is folded in a different order).
 * workspace_clean != 0: the caller guarantees that the workspace is in the state a scan call leaves it in
 * (all zero at first, and every call that ran to its end restores that), so the entry point need not clear
 * it first; with 0 the entry point clears what must start from zero on `stream` before the kernel. */
int64_t exb_leaky_scan_workspace_bytes(int64_t B, int64_t T, int64_t M);

int exb_leaky_forward_scan(float *out, const float *input, const float *v_init,
                           const float *alpha, int alpha_mode,
                           const float *in_scale, int in_scale_mode,
                           float *v_last, double *out_sum, void *workspace, int64_t workspace_bytes, int workspace_clean,
                           int64_t B, int64_t T, int64_t M, int device, void *stream);

int exb_leaky_backward_scan(float *grad_input, float *grad_alpha, float *grad_init, float *grad_scale,
                            const float *grad_out, const float *grad_v_last,
                            const float *out, const float *input, const float *v_init,
                            const float *alpha, int alpha_mode,
                            const float *in_scale, int in_scale_mode, double *acc_decay,
                            void *workspace, int64_t workspace_bytes, int workspace_clean,
                            int64_t B, int64_t T, int64_t M, int device, void *stream);

/* exb_leaky_forward_scan for callers that have no scratch memory to give.  No counterpart in
 * the reference (its kernels use no scratch memory at all).
 *
 * Who needs it: a host whose device memory was handed out once at start-up and that may not
 * allocate afterwards -- an inference or real-time service with a fixed memory budget, or code
 * running inside another framework's memory pool where a raw allocation would bypass (and can
 * exhaust or fragment) that pool and stalls the device while it happens.  Such a caller still
 * passes its input and output tensors, but the scratch the scan needs is a fixed 1 MiB array
 * that is part of the library image (EXB_STATIC_SCRATCH_BYTES; every GPU that loads the library
 * holds it until the process ends).  This entry point calls no allocating routine of any kind.
 *
 * Limits and rules:
 *  - a shape whose scratch need (exb_leaky_scan_workspace_bytes) exceeds EXB_STATIC_SCRATCH_BYTES
 *    is rejected with EXB_ERR_ARG and a message that says how much was needed; shapes the scan
 *    does not apply to give EXB_ERR_UNSUPPORTED, as with exb_leaky_forward_scan;
 *  - the first call on each device looks up the array's device address (once per device, with
 *    that device current) and, like the first call of any entry point, makes the CUDA runtime load
 *    the kernel; make that first call before any stream capture begins and before the point from
 *    which the host may no longer allocate;
 *  - all calls on a device share the one array, and it keeps what the previous call left in it.
 *    Each call clears the part that must start from zero (work ticket and ready flags) on
 *    `stream` ahead of its kernel, so calls issued one after another on a stream are fine.  Two
 *    calls that can run on the GPU at the same time (different streams, different host threads)
 *    would use the same flags and aggregates and corrupt each other: do not overlap them.
 * Arguments and results are those of exb_leaky_forward_scan without the workspace pair. */
#define EXB_STATIC_SCRATCH_BYTES (1u << 20)
/* The size the loaded library was built with (for bindings that cannot see this header). */
int64_t exb_static_scratch_bytes(void);
int exb_leaky_forward_scan_static(float *out, const float *input, const float *v_init,
                                  const float *alpha, int alpha_mode,
                                  const float *in_scale, int in_scale_mode,
                                  float *v_last,
                                  int64_t B, int64_t T, int64_t M, int device, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* EXODUS_B200_H */
