// Argument blocks and launcher prototypes shared between the kernel
// translation units and the C-ABI front end.
#pragma once

#include "exb_math.cuh"

namespace exb {

struct LifFwdArgs {
    float *spikes, *v_mem;
    const float *input, *v_init;
    NeuronParams np;
    unsigned maxs;
    float *v_post_last;
    unsigned long long *spike_count;
    float *v_post;     // optional full record of the potential after each step's reset (time-major kernels only)
    uint8_t *spikes_u8 = nullptr;   // compact raster instead of `spikes` (TMA-staged kernels only; v_mem may then be null)
    // Checkpoints instead of v_mem (TMA-staged time-major kernels only): the state entering every
    // EXB_CKPT_EVERY-th step, [B][ceil(T / EXB_CKPT_EVERY)][M]; the backward rebuilds v_mem from them and the input.
    float *ckpt = nullptr;
    int64_t B, T, M;
};

struct LifBwdArgs {
    // Parameter-shaped float64 accumulator for the gradient w.r.t. the decay values the caller passed (alpha or
    // tau), scale derived from alpha included; replaces grad_alpha / grad_scale.  TMA-staged kernels only.
    double *acc_decay = nullptr;
    float *grad_input, *grad_alpha, *grad_init, *grad_scale;
    const float *go, *gv, *g_last, *v_mem, *surr, *v_init, *input;
    const float *ckpt = nullptr;      // with `input` and without `v_mem`: v_mem is rebuilt chunk by chunk (see LifFwdArgs)
    NeuronParams np;
    unsigned maxs;
    float p0, p1;
    int64_t B, T, M;
};

struct LeakyFwdArgs {
    float *out;
    const float *input, *v_init;
    Param alpha, scale;
    float *v_last;
    double *out_sum;   // optional: receives (atomically) the sum of all outputs
    int64_t B, T, M;
};

struct LeakyBwdArgs {
    double *acc_decay = nullptr;      // as in LifBwdArgs
    float *grad_input, *grad_alpha, *grad_init, *grad_scale;
    const float *go, *g_last, *out, *input, *v_init;
    Param alpha, scale;
    int64_t B, T, M;
};

// LIF with synaptic stage, both stages in one kernel (time-major layout only).
struct LifSynFwdArgs {
    float *spikes, *v_mem, *i_syn;
    const float *input, *v_init, *i_init;
    NeuronParams np;               // membrane stage; np.scale multiplies i_syn
    Param alpha_syn, scale_syn;    // synaptic stage; scale_syn multiplies the input
    unsigned maxs;
    float *v_post_last, *i_last;
    unsigned long long *spike_count;
    uint8_t *spikes_u8 = nullptr;   // compact raster instead of `spikes`; v_mem and i_syn may then be null
    int64_t B, T, M;
};

struct LifSynBwdArgs {
    double *acc_decay_mem = nullptr, *acc_decay_syn = nullptr;      // both or neither; replace the four per-instance outputs
    float *grad_input;
    float *grad_alpha_mem, *grad_scale_mem, *grad_alpha_syn, *grad_scale_syn;   // all four or none
    float *grad_v_init, *grad_i_init;
    const float *go, *gv, *g_vlast, *g_isyn, *g_ilast;
    const float *v_mem, *i_syn, *surr, *v_init, *i_init;
    NeuronParams np;
    Param alpha_syn, scale_syn;
    unsigned maxs;
    float p0, p1;
    int64_t B, T, M;
};

cudaError_t launch_lif_syn_forward(const LifSynFwdArgs &a, int reset_mode, cudaStream_t s, bool *used);
cudaError_t launch_lif_syn_backward(const LifSynBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used);
cudaError_t read_device_status_lif_syn(cudaStream_t s, unsigned int *out);

// Each launcher returns a cudaError_t from the launch (cudaPeekAtLastError).
cudaError_t launch_lif_forward(const LifFwdArgs &a, int layout, int reset_mode, cudaStream_t s);
cudaError_t launch_lif_backward(const LifBwdArgs &a, int layout, int reset_mode, int surr_kind, cudaStream_t s);
cudaError_t launch_leaky_forward(const LeakyFwdArgs &a, int layout, cudaStream_t s);
cudaError_t launch_leaky_backward(const LeakyBwdArgs &a, int layout, cudaStream_t s);

// TMA-staged variants (time-major layout only).  `*used` tells whether the launch happened;
// when false (shape or alignment not eligible) the caller takes the plain-load kernel.
cudaError_t launch_lif_forward_tma(const LifFwdArgs &a, int reset_mode, cudaStream_t s, bool *used);
cudaError_t launch_lif_backward_tma(const LifBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used);
// The same with v_mem rebuilt from a.ckpt and a.input (a.v_mem, a.gv, a.surr must be null).
cudaError_t launch_lif_backward_ckpt_tma(const LifBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used);
// [N,T] layout through TMA boxes of one row class (T % 4 == 0, T >= 64, N a multiple of the class count, tensors
// at the same 16-byte aligned position inside a 128-byte line).
cudaError_t launch_lif_forward_nt_tma(const LifFwdArgs &a, int reset_mode, cudaStream_t s, bool *used);
cudaError_t launch_lif_backward_nt_tma(const LifBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used);
cudaError_t launch_leaky_forward_tma(const LeakyFwdArgs &a, cudaStream_t s, bool *used);
cudaError_t launch_leaky_backward_tma(const LeakyBwdArgs &a, cudaStream_t s, bool *used);
// Time-parallel leaky integrator (time-major layout): the time axis is cut into segments that
// run in different CTAs.  Needs caller-provided scratch memory of leaky_scan_workspace_bytes().
int64_t leaky_scan_workspace_bytes(int64_t B, int64_t T, int64_t M);
// `clean`: the workspace is known to be in the all-zero state a completed scan leaves it in (no memset needed).
cudaError_t launch_leaky_forward_scan(const LeakyFwdArgs &a, void *workspace, int64_t workspace_bytes, bool clean,
                                      cudaStream_t s, bool *used);
cudaError_t launch_leaky_backward_scan(const LeakyBwdArgs &a, void *workspace, int64_t workspace_bytes, bool clean,
                                       cudaStream_t s, bool *used);
// One-shot sum-allreduce of a small vector over peer-mapped memory (one CTA per rank; see exb_tma_kernels.cu).
cudaError_t launch_allreduce_oneshot(float *out, const float *in, const unsigned long long *buffers,
                                     const unsigned long long *signals, int rank, int world, int64_t n, unsigned int epoch,
                                     cudaStream_t s);
// out[i] = (float) acc[i]; acc[i] = 0.
cudaError_t launch_acc_finish(float *out, double *acc, int64_t n, cudaStream_t s);
// Forward scan on the library's own fixed scratch array (no caller workspace).
size_t leaky_scan_static_capacity();
cudaError_t launch_leaky_forward_scan_static(const LeakyFwdArgs &a, int device, cudaStream_t s, bool *used);
cudaError_t read_device_status(cudaStream_t s, unsigned int *out);
// Poll limit of the bounded waits (0 = default) on the current device, one setter per translation unit with
// such waits; the first also sets the diagnostic switch that keeps the time-parallel scan's ready flags down.
cudaError_t set_wait_limit(unsigned int polls, bool withhold_scan_flags);
cudaError_t set_wait_limit_lif_bwd(unsigned int polls);
cudaError_t set_wait_limit_lif_syn(unsigned int polls);
cudaError_t set_wait_limit_lif_nt_bwd(unsigned int polls);
cudaError_t read_device_status_lif_bwd(cudaStream_t s, unsigned int *out);
cudaError_t read_device_status_lif_nt_bwd(cudaStream_t s, unsigned int *out);
cudaError_t set_wait_limit_lif_bwd_rec(unsigned int polls);
cudaError_t read_device_status_lif_bwd_rec(cudaStream_t s, unsigned int *out);
// EXB_DISABLE_TMA=1 in the environment forces the plain-load kernels (debugging aid).
bool tma_enabled();

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long x)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
}

// Sum over the warp of per-thread partial sums, added to *dst by lane 0 (all 32 lanes must call).
__device__ __forceinline__ void warp_add_f64(double *dst, double x, int lane)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    if (lane == 0) atomicAdd(dst, x);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace exb
