// C-ABI front end: argument validation, device selection, dispatch.
// Nothing here allocates device memory.  State kept between calls: the text of the calling
// thread's last error (host); per device, the status words and the poll limit of the bounded
// waits, and the built-in scratch array of exb_leaky_forward_scan_static (all in the kernel
// translation units).
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <cstdlib>

#include "exb_kernels.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

// Makes `device` current for the duration of one entry point and restores the
// previous device afterwards (the reference calls cudaSetDevice without
// restoring, cuda/bindings.cu:45).
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int device)
    {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (device >= 0 && device != prev && cudaSetDevice(device) != cudaSuccess) ok = false;
    }
    ~DeviceGuard()
    {
        int cur = -1;
        if (prev >= 0 && cudaGetDevice(&cur) == cudaSuccess && cur != prev) cudaSetDevice(prev);
    }
};

// Shape in the low bits; the derived-parameter bits only where they mean something: IS_TAU on a decay
// argument, the SCALE bits on a scale argument.
bool mode_ok(int mode, int allowed_flags = 0)
{
    const int shape = mode & EXB_PARAM_SHAPE_MASK;
    return (mode & ~(EXB_PARAM_SHAPE_MASK | allowed_flags)) == 0 &&
           (shape == EXB_PARAM_SCALAR || shape == EXB_PARAM_PER_M || shape == EXB_PARAM_PER_N);
}
constexpr int DECAY_FLAGS = EXB_PARAM_IS_TAU;
constexpr int SCALE_FLAGS = EXB_SCALE_ONE_MINUS_ALPHA | EXB_SCALE_TIMES_ALPHA;

// A scale that is 1 - alpha has no values of its own.
bool scale_arg_ok(const float *scale, int mode)
{
    if (!scale && !(mode & SCALE_FLAGS)) return true;      // absent
    if (!mode_ok(mode, SCALE_FLAGS)) return false;
    return !((mode & EXB_SCALE_ONE_MINUS_ALPHA) && scale);
}

int check_geometry(int64_t B, int64_t T, int64_t M, int layout)
{
    if (B < 0 || T < 0 || M < 0) return fail(EXB_ERR_ARG, "negative size (B=%lld T=%lld M=%lld)", (long long)B, (long long)T, (long long)M);
    if (layout != EXB_LAYOUT_NT && layout != EXB_LAYOUT_BTM) return fail(EXB_ERR_ARG, "unknown layout %d", layout);
    // Kernel grids are 1-D in units of 128..1024 neurons; keep far away from 2^31 blocks.
    if (B > 0 && M > 0 && (double)B * (double)M > 1.0e11) return fail(EXB_ERR_ARG, "B*M too large");
    // Time steps are counted in int inside the kernels (2^31 steps of one neuron would be 8.6 GB per tensor).
    if (T > 0x7fffffffll - 64) return fail(EXB_ERR_ARG, "T too large (%lld)", (long long)T);
    return EXB_OK;
}

// Every tensor and vector is float32 (or wider, for the counters): an address that is not a multiple of 4
// cannot be one, and the kernels would fault on it.
template <typename... P>
bool all_aligned4(const P *...ptrs)
{
    return (((reinterpret_cast<uintptr_t>(static_cast<const void *>(ptrs)) & 3u) == 0) && ...);
}

int misaligned(const char *who)
{
    return fail(EXB_ERR_ALIGN, "%s: every tensor must be aligned to its element size (float32: 4 bytes; counters: 8)", who);
}

int launch_status(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return EXB_OK;
    return fail(EXB_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

}  // namespace

extern "C" {

const char *exb_version(void) { return "exodus_b200 0.1.0 (sm_100a)"; }

const char *exb_last_error(void) { return g_err; }

const char *exb_status_string(int status)
{
    switch (status) {
    case EXB_OK: return "ok";
    case EXB_ERR_ARG: return "invalid argument";
    case EXB_ERR_ALIGN: return "misaligned pointer";
    case EXB_ERR_LAUNCH: return "kernel launch failed";
    case EXB_ERR_UNSUPPORTED: return "unsupported configuration";
    case EXB_ERR_DEVICE: return "cannot select device";
    case EXB_ERR_TIMEOUT: return "device-side wait ran out";
    default: return "unknown status";
    }
}

int exb_device_status(int device, void *stream)
{
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_device_status: cannot select device %d", device);
    unsigned int code = 0, code2 = 0;
    cudaError_t e = exb::read_device_status((cudaStream_t)stream, &code);
    unsigned int code3 = 0, code4 = 0;
    if (e == cudaSuccess) e = exb::read_device_status_lif_bwd((cudaStream_t)stream, &code2);
    if (e == cudaSuccess) e = exb::read_device_status_lif_syn((cudaStream_t)stream, &code3);
    unsigned int code5 = 0;
    if (e == cudaSuccess) e = exb::read_device_status_lif_nt_bwd((cudaStream_t)stream, &code4);
    if (e == cudaSuccess) e = exb::read_device_status_lif_bwd_rec((cudaStream_t)stream, &code5);
    if (e != cudaSuccess) return fail(EXB_ERR_LAUNCH, "exb_device_status: %s", cudaGetErrorString(e));
    if (!code) code = code2 ? code2 : (code3 ? code3 : (code4 ? code4 : code5));
    if (code) return fail(EXB_ERR_TIMEOUT, "a bounded device-side wait ran out (code %u); results of the affected call are incomplete", code);
    return EXB_OK;
}

int exb_set_wait_limit(int device, uint32_t polls, int withhold_scan_flags)
{
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_set_wait_limit: cannot select device %d", device);
    cudaError_t e = exb::set_wait_limit(polls, withhold_scan_flags != 0);
    if (e == cudaSuccess) e = exb::set_wait_limit_lif_bwd(polls);
    if (e == cudaSuccess) e = exb::set_wait_limit_lif_syn(polls);
    if (e == cudaSuccess) e = exb::set_wait_limit_lif_nt_bwd(polls);
    if (e == cudaSuccess) e = exb::set_wait_limit_lif_bwd_rec(polls);
    if (e != cudaSuccess) return fail(EXB_ERR_LAUNCH, "exb_set_wait_limit: %s", cudaGetErrorString(e));
    return EXB_OK;
}

}  // extern "C"

static int lif_forward_impl(const char *who, float *spikes, uint8_t *spikes_u8, float *v_mem, float *v_post, const float *input, const float *v_init,
                    const float *in_scale, int in_scale_mode,
                    const float *alpha, int alpha_mode,
                    const float *subtract, int subtract_mode,
                    const float *theta, int theta_mode,
                    const float *theta_low, int theta_low_mode,
                    uint32_t max_spikes, int reset_mode,
                    float *v_post_last, unsigned long long *spike_count,
                    int64_t B, int64_t T, int64_t M, int layout,
                    int device, void *stream, float *ckpt = nullptr)
{
    if (int st = check_geometry(B, T, M, layout)) return st;
    if (ckpt) {
        if (!spikes || !input) return fail(EXB_ERR_ARG, "%s: spikes, ckpt and input are required", who);
    } else if (spikes_u8) {
        if (!input) return fail(EXB_ERR_ARG, "%s: spikes and input are required", who);
        if (layout != EXB_LAYOUT_BTM) return fail(EXB_ERR_UNSUPPORTED, "%s: the compact raster is written by the time-major kernels only", who);
    } else if (!spikes || !input) {
        return fail(EXB_ERR_ARG, "%s: spikes and input are required", who);
    } else if (!v_mem && (v_post || layout != EXB_LAYOUT_BTM)) {
        return fail(EXB_ERR_UNSUPPORTED, "%s: v_mem may be omitted in the time-major layout without a post-reset record only", who);
    }
    if (!alpha || !theta) return fail(EXB_ERR_ARG, "%s: alpha and theta are required", who);
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !mode_ok(theta_mode) || (subtract && !mode_ok(subtract_mode)) ||
        (theta_low && !mode_ok(theta_low_mode)) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "%s: bad parameter mode", who);
    if (reset_mode != EXB_RESET_SUBTRACT && reset_mode != EXB_RESET_TO_VALUE)
        return fail(EXB_ERR_ARG, "%s: bad reset mode %d", who, reset_mode);
    if (reset_mode == EXB_RESET_TO_VALUE && !subtract)
        return fail(EXB_ERR_ARG, "%s: reset-to-value needs the value in `subtract`", who);
    if (v_post && layout != EXB_LAYOUT_BTM)
        return fail(EXB_ERR_UNSUPPORTED, "%s: the post-reset record is written by the time-major kernels only", who);
    if (!all_aligned4(spikes, v_mem, v_post, input, v_init, in_scale, alpha, subtract, theta, theta_low, v_post_last, ckpt) ||
        (reinterpret_cast<uintptr_t>(spike_count) & 7u))
        return misaligned(who);
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "%s: cannot select device %d", who, device);

    exb::LifFwdArgs a;
    a.spikes = spikes; a.v_mem = v_mem; a.input = input; a.v_init = v_init;
    a.np.alpha = exb::make_param(alpha, alpha_mode, M);
    a.np.c = exb::make_param(subtract, subtract_mode, M);
    a.np.th = exb::make_param(theta, theta_mode, M);
    a.np.lo = exb::make_param(theta_low, theta_low_mode, M);
    a.np.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.maxs = max_spikes;
    a.v_post_last = v_post_last; a.spike_count = spike_count; a.v_post = v_post;
    a.spikes_u8 = spikes_u8;
    a.ckpt = ckpt;
    a.B = B; a.T = T; a.M = M;
    if (spikes_u8 || ckpt || !v_mem) {
        bool used = false;
        cudaError_t e = exb::tma_enabled() ? exb::launch_lif_forward_tma(a, reset_mode, (cudaStream_t)stream, &used) : cudaSuccess;
        if (e != cudaSuccess) return launch_status(e, who);
        if (!used) return fail(EXB_ERR_UNSUPPORTED, "%s: shape or alignment not eligible (needs M %% 4 == 0 and 16-byte aligned tensors)", who);
        return EXB_OK;
    }
    return launch_status(exb::launch_lif_forward(a, layout, reset_mode, (cudaStream_t)stream), who);
}

extern "C" {

int exb_lif_forward(float *spikes, float *v_mem, const float *input, const float *v_init,
                    const float *in_scale, int in_scale_mode,
                    const float *alpha, int alpha_mode,
                    const float *subtract, int subtract_mode,
                    const float *theta, int theta_mode,
                    const float *theta_low, int theta_low_mode,
                    uint32_t max_spikes, int reset_mode,
                    float *v_post_last, unsigned long long *spike_count,
                    int64_t B, int64_t T, int64_t M, int layout,
                    int device, void *stream)
{
    return lif_forward_impl("exb_lif_forward", spikes, nullptr, v_mem, nullptr, input, v_init, in_scale, in_scale_mode, alpha,
                            alpha_mode, subtract, subtract_mode, theta, theta_mode, theta_low, theta_low_mode,
                            max_spikes, reset_mode, v_post_last, spike_count, B, T, M, layout, device, stream);
}

int exb_lif_forward_record(float *spikes, float *v_mem, float *v_post, const float *input, const float *v_init,
                           const float *in_scale, int in_scale_mode,
                           const float *alpha, int alpha_mode,
                           const float *subtract, int subtract_mode,
                           const float *theta, int theta_mode,
                           const float *theta_low, int theta_low_mode,
                           uint32_t max_spikes, int reset_mode,
                           float *v_post_last, unsigned long long *spike_count,
                           int64_t B, int64_t T, int64_t M, int layout,
                           int device, void *stream)
{
    if (!v_post) return fail(EXB_ERR_ARG, "exb_lif_forward_record: v_post is required (use exb_lif_forward without it)");
    return lif_forward_impl("exb_lif_forward_record", spikes, nullptr, v_mem, v_post, input, v_init, in_scale, in_scale_mode,
                            alpha, alpha_mode, subtract, subtract_mode, theta, theta_mode, theta_low, theta_low_mode,
                            max_spikes, reset_mode, v_post_last, spike_count, B, T, M, layout, device, stream);
}

int exb_lif_forward_u8(uint8_t *spikes, float *v_mem, const float *input, const float *v_init,
                       const float *in_scale, int in_scale_mode,
                       const float *alpha, int alpha_mode,
                       const float *subtract, int subtract_mode,
                       const float *theta, int theta_mode,
                       const float *theta_low, int theta_low_mode,
                       uint32_t max_spikes, int reset_mode, int saturate,
                       float *v_post_last, unsigned long long *spike_count,
                       int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (!spikes) return fail(EXB_ERR_ARG, "exb_lif_forward_u8: spikes is required");
    if (max_spikes > 255u && !saturate)
        return fail(EXB_ERR_ARG, "exb_lif_forward_u8: more than 255 spikes per step are possible (max_spikes = %u); "
                    "pass saturate != 0 to store min(count, 255)", max_spikes);
    return lif_forward_impl("exb_lif_forward_u8", nullptr, spikes, v_mem, nullptr, input, v_init, in_scale, in_scale_mode,
                            alpha, alpha_mode, subtract, subtract_mode, theta, theta_mode, theta_low, theta_low_mode,
                            max_spikes, reset_mode, v_post_last, spike_count, B, T, M, EXB_LAYOUT_BTM, device, stream);
}

int exb_lif_forward_ckpt(float *spikes, float *ckpt, const float *input, const float *v_init,
                         const float *in_scale, int in_scale_mode,
                         const float *alpha, int alpha_mode,
                         const float *subtract, int subtract_mode,
                         const float *theta, int theta_mode,
                         const float *theta_low, int theta_low_mode,
                         uint32_t max_spikes, int reset_mode,
                         float *v_post_last, unsigned long long *spike_count,
                         int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (!ckpt) return fail(EXB_ERR_ARG, "exb_lif_forward_ckpt: ckpt is required (use exb_lif_forward without it)");
    return lif_forward_impl("exb_lif_forward_ckpt", spikes, nullptr, nullptr, nullptr, input, v_init, in_scale, in_scale_mode,
                            alpha, alpha_mode, subtract, subtract_mode, theta, theta_mode, theta_low, theta_low_mode,
                            max_spikes, reset_mode, v_post_last, spike_count, B, T, M, EXB_LAYOUT_BTM, device, stream, ckpt);
}

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
                          int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    const char *who = "exb_lif_backward_ckpt";
    if (int st = check_geometry(B, T, M, EXB_LAYOUT_BTM)) return st;
    if (!grad_input || !grad_spikes || !input || !ckpt)
        return fail(EXB_ERR_ARG, "%s: grad_input, grad_spikes, input and ckpt are required", who);
    if (!alpha || !theta) return fail(EXB_ERR_ARG, "%s: alpha and theta are required", who);
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !mode_ok(theta_mode) || (subtract && !mode_ok(subtract_mode)) ||
        (theta_low && !mode_ok(theta_low_mode)) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "%s: bad parameter mode", who);
    if (acc_decay && (grad_alpha || grad_scale))
        return fail(EXB_ERR_ARG, "%s: acc_decay replaces grad_alpha and grad_scale; pass NULL for those", who);
    if (acc_decay && (reinterpret_cast<uintptr_t>(acc_decay) & 7u)) return misaligned(who);
    if (reset_mode != EXB_RESET_SUBTRACT && reset_mode != EXB_RESET_TO_VALUE)
        return fail(EXB_ERR_ARG, "%s: bad reset mode %d", who, reset_mode);
    if (reset_mode == EXB_RESET_TO_VALUE && !subtract)
        return fail(EXB_ERR_ARG, "%s: reset-to-value needs the value in `subtract`", who);
    if (surrogate_kind <= EXB_SURR_GENERIC || surrogate_kind > EXB_SURR_PERIODIC_EXPONENTIAL)
        return fail(EXB_ERR_ARG, "%s: needs one of the built-in surrogates (kind %d given): the generic one is a function "
                    "of a v_mem tensor that this pass never materialises", who, surrogate_kind);
    const bool scale_derived = (in_scale_mode & SCALE_FLAGS) != 0;
    if (grad_scale && !in_scale && !scale_derived)
        return fail(EXB_ERR_ARG, "%s: grad_scale is rebuilt from the state and needs in_scale", who);
    if (!all_aligned4(grad_input, grad_alpha, grad_init, grad_scale, grad_spikes, grad_v_last, input, ckpt, v_init, in_scale,
                      alpha, subtract, theta, theta_low))
        return misaligned(who);
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "%s: cannot select device %d", who, device);

    exb::LifBwdArgs a;
    a.grad_input = grad_input; a.grad_alpha = grad_alpha; a.grad_init = grad_init; a.grad_scale = grad_scale;
    a.go = grad_spikes; a.gv = nullptr; a.g_last = grad_v_last; a.v_mem = nullptr; a.surr = nullptr;
    a.v_init = v_init; a.input = input; a.ckpt = ckpt;
    a.np.alpha = exb::make_param(alpha, alpha_mode, M);
    a.np.c = exb::make_param(subtract, subtract_mode, M);
    a.np.th = exb::make_param(theta, theta_mode, M);
    a.np.lo = exb::make_param(theta_low, theta_low_mode, M);
    a.np.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.maxs = max_spikes; a.p0 = surr_p0; a.p1 = surr_p1;
    a.acc_decay = acc_decay;
    a.B = B; a.T = T; a.M = M;
    bool used = false;
    cudaError_t e = exb::tma_enabled() ? exb::launch_lif_backward_ckpt_tma(a, reset_mode, surrogate_kind, (cudaStream_t)stream, &used)
                                       : cudaSuccess;
    if (e != cudaSuccess) return launch_status(e, who);
    if (!used) return fail(EXB_ERR_UNSUPPORTED, "%s: shape or alignment not eligible (needs M %% 4 == 0 and 16-byte aligned tensors)", who);
    return EXB_OK;
}

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
                     int device, void *stream)
{
    if (int st = check_geometry(B, T, M, layout)) return st;
    if (!grad_input || !grad_spikes || !v_mem)
        return fail(EXB_ERR_ARG, "exb_lif_backward: grad_input, grad_spikes and v_mem are required");
    if (!alpha || !theta) return fail(EXB_ERR_ARG, "exb_lif_backward: alpha and theta are required");
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !mode_ok(theta_mode) || (subtract && !mode_ok(subtract_mode)) ||
        (theta_low && !mode_ok(theta_low_mode)) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "exb_lif_backward: bad parameter mode");
    const bool scale_derived = (in_scale_mode & SCALE_FLAGS) != 0;
    if (acc_decay && (grad_alpha || grad_scale))
        return fail(EXB_ERR_ARG, "exb_lif_backward: acc_decay replaces grad_alpha and grad_scale; pass NULL for those");
    if (acc_decay && (reinterpret_cast<uintptr_t>(acc_decay) & 7u)) return misaligned("exb_lif_backward");
    if (reset_mode != EXB_RESET_SUBTRACT && reset_mode != EXB_RESET_TO_VALUE)
        return fail(EXB_ERR_ARG, "exb_lif_backward: bad reset mode %d", reset_mode);
    if (reset_mode == EXB_RESET_TO_VALUE && !subtract)
        return fail(EXB_ERR_ARG, "exb_lif_backward: reset-to-value needs the value in `subtract`");
    if (surrogate_kind < EXB_SURR_GENERIC || surrogate_kind > EXB_SURR_PERIODIC_EXPONENTIAL)
        return fail(EXB_ERR_ARG, "exb_lif_backward: unknown surrogate kind %d", surrogate_kind);
    if (surrogate_kind == EXB_SURR_GENERIC && !surr)
        return fail(EXB_ERR_ARG, "exb_lif_backward: the generic surrogate needs the `surr` tensor");
    if (grad_scale && !input && !in_scale && !scale_derived)
        return fail(EXB_ERR_ARG, "exb_lif_backward: grad_scale without `input` is rebuilt from v_mem and needs in_scale");
    if (!all_aligned4(grad_input, grad_alpha, grad_init, grad_scale, grad_spikes, grad_v_mem, grad_v_last, v_mem, surr,
                      v_init, input, in_scale, alpha, subtract, theta, theta_low))
        return misaligned("exb_lif_backward");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_lif_backward: cannot select device %d", device);

    exb::LifBwdArgs a;
    a.grad_input = grad_input; a.grad_alpha = grad_alpha; a.grad_init = grad_init; a.grad_scale = grad_scale;
    a.go = grad_spikes; a.gv = grad_v_mem; a.g_last = grad_v_last; a.v_mem = v_mem;
    a.surr = (surrogate_kind == EXB_SURR_GENERIC) ? surr : nullptr;
    a.v_init = v_init; a.input = input;
    a.np.alpha = exb::make_param(alpha, alpha_mode, M);
    a.np.c = exb::make_param(subtract, subtract_mode, M);
    a.np.th = exb::make_param(theta, theta_mode, M);
    a.np.lo = exb::make_param(theta_low, theta_low_mode, M);
    a.np.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.maxs = max_spikes; a.p0 = surr_p0; a.p1 = surr_p1;
    a.acc_decay = acc_decay;
    a.B = B; a.T = T; a.M = M;
    const cudaError_t e = exb::launch_lif_backward(a, layout, reset_mode, surrogate_kind, (cudaStream_t)stream);
    if (e == cudaErrorNotSupported)
        return fail(EXB_ERR_UNSUPPORTED, "exb_lif_backward: acc_decay needs a shape the TMA-staged kernels take "
                    "(time-major, M %% 4 == 0, 16-byte aligned tensors)");
    return launch_status(e, "exb_lif_backward");
}

int exb_leaky_forward(float *out, const float *input, const float *v_init,
                      const float *alpha, int alpha_mode,
                      const float *in_scale, int in_scale_mode,
                      float *v_last, double *out_sum,
                      int64_t B, int64_t T, int64_t M, int layout,
                      int device, void *stream)
{
    if (int st = check_geometry(B, T, M, layout)) return st;
    if (!out || !input || !alpha) return fail(EXB_ERR_ARG, "exb_leaky_forward: out, input and alpha are required");
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "exb_leaky_forward: bad parameter mode");
    if (!all_aligned4(out, input, v_init, alpha, in_scale, v_last) || (reinterpret_cast<uintptr_t>(out_sum) & 7u))
        return misaligned("exb_leaky_forward");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_leaky_forward: cannot select device %d", device);

    exb::LeakyFwdArgs a;
    a.out = out; a.input = input; a.v_init = v_init;
    a.alpha = exb::make_param(alpha, alpha_mode, M);
    a.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.v_last = v_last;
    a.out_sum = out_sum;
    a.B = B; a.T = T; a.M = M;
    return launch_status(exb::launch_leaky_forward(a, layout, (cudaStream_t)stream), "exb_leaky_forward");
}

int exb_leaky_backward(float *grad_input, float *grad_alpha, float *grad_init, float *grad_scale,
                       const float *grad_out, const float *grad_v_last,
                       const float *out, const float *input, const float *v_init,
                       const float *alpha, int alpha_mode,
                       const float *in_scale, int in_scale_mode, double *acc_decay,
                       int64_t B, int64_t T, int64_t M, int layout,
                       int device, void *stream)
{
    if (int st = check_geometry(B, T, M, layout)) return st;
    if (!grad_input || !grad_out || !alpha)
        return fail(EXB_ERR_ARG, "exb_leaky_backward: grad_input, grad_out and alpha are required");
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "exb_leaky_backward: bad parameter mode");
    if ((grad_alpha || acc_decay) && !out) return fail(EXB_ERR_ARG, "exb_leaky_backward: the alpha gradient needs `out`");
    if ((grad_scale || (acc_decay && (in_scale_mode & SCALE_FLAGS))) && !input)
        return fail(EXB_ERR_ARG, "exb_leaky_backward: the scale gradient needs `input`");
    if (acc_decay && (grad_alpha || grad_scale))
        return fail(EXB_ERR_ARG, "exb_leaky_backward: acc_decay replaces grad_alpha and grad_scale; pass NULL for those");
    if (acc_decay && (reinterpret_cast<uintptr_t>(acc_decay) & 7u)) return misaligned("exb_leaky_backward");
    if (!all_aligned4(grad_input, grad_alpha, grad_init, grad_scale, grad_out, grad_v_last, out, input, v_init, alpha, in_scale))
        return misaligned("exb_leaky_backward");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_leaky_backward: cannot select device %d", device);

    exb::LeakyBwdArgs a;
    a.grad_input = grad_input; a.grad_alpha = grad_alpha; a.grad_init = grad_init; a.grad_scale = grad_scale;
    a.go = grad_out; a.g_last = grad_v_last; a.out = out; a.input = input; a.v_init = v_init;
    a.alpha = exb::make_param(alpha, alpha_mode, M);
    a.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.acc_decay = acc_decay;
    a.B = B; a.T = T; a.M = M;
    const cudaError_t e = exb::launch_leaky_backward(a, layout, (cudaStream_t)stream);
    if (e == cudaErrorNotSupported)
        return fail(EXB_ERR_UNSUPPORTED, "exb_leaky_backward: acc_decay needs a shape the TMA-staged kernels take "
                    "(time-major, M %% 4 == 0, 16-byte aligned tensors)");
    return launch_status(e, "exb_leaky_backward");
}

int64_t exb_leaky_scan_workspace_bytes(int64_t B, int64_t T, int64_t M)
{
    if (B <= 0 || T <= 0 || M <= 0) return 0;
    return exb::leaky_scan_workspace_bytes(B, T, M);
}

int exb_leaky_forward_scan(float *out, const float *input, const float *v_init,
                           const float *alpha, int alpha_mode,
                           const float *in_scale, int in_scale_mode,
                           float *v_last, double *out_sum, void *workspace, int64_t workspace_bytes, int workspace_clean,
                           int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (int st = check_geometry(B, T, M, EXB_LAYOUT_BTM)) return st;
    if (!out || !input || !alpha) return fail(EXB_ERR_ARG, "exb_leaky_forward_scan: out, input and alpha are required");
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "exb_leaky_forward_scan: bad parameter mode");
    if (!workspace) return fail(EXB_ERR_ARG, "exb_leaky_forward_scan: workspace is required");
    if (!all_aligned4(out, input, v_init, alpha, in_scale, v_last) || (reinterpret_cast<uintptr_t>(out_sum) & 7u))
        return misaligned("exb_leaky_forward_scan");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_leaky_forward_scan: cannot select device %d", device);
    exb::LeakyFwdArgs a;
    a.out = out; a.input = input; a.v_init = v_init;
    a.alpha = exb::make_param(alpha, alpha_mode, M);
    a.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.v_last = v_last;
    a.out_sum = out_sum;
    a.B = B; a.T = T; a.M = M;
    bool used = false;
    cudaError_t e = exb::launch_leaky_forward_scan(a, workspace, workspace_bytes, workspace_clean != 0, (cudaStream_t)stream, &used);
    if (e != cudaSuccess) return launch_status(e, "exb_leaky_forward_scan");
    if (!used) return fail(EXB_ERR_UNSUPPORTED, "exb_leaky_forward_scan: shape, alignment or workspace not eligible");
    return EXB_OK;
}

int exb_leaky_backward_scan(float *grad_input, float *grad_alpha, float *grad_init, float *grad_scale,
                            const float *grad_out, const float *grad_v_last,
                            const float *out, const float *input, const float *v_init,
                            const float *alpha, int alpha_mode,
                            const float *in_scale, int in_scale_mode, double *acc_decay,
                            void *workspace, int64_t workspace_bytes, int workspace_clean,
                            int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (int st = check_geometry(B, T, M, EXB_LAYOUT_BTM)) return st;
    if (!grad_input || !grad_out || !alpha)
        return fail(EXB_ERR_ARG, "exb_leaky_backward_scan: grad_input, grad_out and alpha are required");
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "exb_leaky_backward_scan: bad parameter mode");
    if ((grad_alpha || acc_decay) && !out) return fail(EXB_ERR_ARG, "exb_leaky_backward_scan: the alpha gradient needs `out`");
    if ((grad_scale || (acc_decay && (in_scale_mode & SCALE_FLAGS))) && !input)
        return fail(EXB_ERR_ARG, "exb_leaky_backward_scan: the scale gradient needs `input`");
    if (acc_decay && (grad_alpha || grad_scale))
        return fail(EXB_ERR_ARG, "exb_leaky_backward_scan: acc_decay replaces grad_alpha and grad_scale; pass NULL for those");
    if (acc_decay && (reinterpret_cast<uintptr_t>(acc_decay) & 7u)) return misaligned("exb_leaky_backward_scan");
    if (!workspace) return fail(EXB_ERR_ARG, "exb_leaky_backward_scan: workspace is required");
    if (!all_aligned4(grad_input, grad_alpha, grad_init, grad_scale, grad_out, grad_v_last, out, input, v_init, alpha, in_scale))
        return misaligned("exb_leaky_backward_scan");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_leaky_backward_scan: cannot select device %d", device);
    exb::LeakyBwdArgs a;
    a.grad_input = grad_input; a.grad_alpha = grad_alpha; a.grad_init = grad_init; a.grad_scale = grad_scale;
    a.go = grad_out; a.g_last = grad_v_last; a.out = out; a.input = input; a.v_init = v_init;
    a.alpha = exb::make_param(alpha, alpha_mode, M);
    a.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.acc_decay = acc_decay;
    a.B = B; a.T = T; a.M = M;
    bool used = false;
    cudaError_t e = exb::launch_leaky_backward_scan(a, workspace, workspace_bytes, workspace_clean != 0, (cudaStream_t)stream, &used);
    if (e != cudaSuccess) return launch_status(e, "exb_leaky_backward_scan");
    if (!used) return fail(EXB_ERR_UNSUPPORTED, "exb_leaky_backward_scan: shape, alignment or workspace not eligible");
    return EXB_OK;
}

int exb_acc_finish(float *out, double *acc, int64_t n, int device, void *stream)
{
    if (n < 0) return fail(EXB_ERR_ARG, "exb_acc_finish: negative size");
    if (n == 0) return EXB_OK;
    if (!out || !acc) return fail(EXB_ERR_ARG, "exb_acc_finish: out and acc are required");
    if ((reinterpret_cast<uintptr_t>(out) & 3u) || (reinterpret_cast<uintptr_t>(acc) & 7u)) return misaligned("exb_acc_finish");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_acc_finish: cannot select device %d", device);
    return launch_status(exb::launch_acc_finish(out, acc, n, (cudaStream_t)stream), "exb_acc_finish");
}

int exb_allreduce_oneshot(float *out, const float *in, const uint64_t *buffers, const uint64_t *signals,
                          int rank, int world, int64_t n, uint32_t epoch, int device, void *stream)
{
    if (!out || !in || !buffers || !signals) return fail(EXB_ERR_ARG, "exb_allreduce_oneshot: out, in, buffers and signals are required");
    if (world < 1 || world > 16 || rank < 0 || rank >= world)
        return fail(EXB_ERR_ARG, "exb_allreduce_oneshot: rank %d of %d (at most 16 ranks)", rank, world);
    if (n <= 0 || n > (1 << 24)) return fail(EXB_ERR_ARG, "exb_allreduce_oneshot: n must be in 1 .. 2^24");
    if (epoch == 0) return fail(EXB_ERR_ARG, "exb_allreduce_oneshot: epochs start at 1 (the signal words start at 0)");
    if (!all_aligned4(out, in) || (reinterpret_cast<uintptr_t>(buffers) & 7u) || (reinterpret_cast<uintptr_t>(signals) & 7u))
        return misaligned("exb_allreduce_oneshot");
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_allreduce_oneshot: cannot select device %d", device);
    return launch_status(exb::launch_allreduce_oneshot(out, in, reinterpret_cast<const unsigned long long *>(buffers),
                                                       reinterpret_cast<const unsigned long long *>(signals), rank, world, n,
                                                       epoch, (cudaStream_t)stream), "exb_allreduce_oneshot");
}

int64_t exb_static_scratch_bytes(void) { return (int64_t)exb::leaky_scan_static_capacity(); }

// Time-parallel leaky forward for callers that cannot supply scratch memory (see the header).
// Nothing is allocated here or below: the workspace is a fixed array inside the library.
int exb_leaky_forward_scan_static(float *out, const float *input, const float *v_init,
                                  const float *alpha, int alpha_mode,
                                  const float *in_scale, int in_scale_mode,
                                  float *v_last,
                                  int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (int st = check_geometry(B, T, M, EXB_LAYOUT_BTM)) return st;
    if (!out || !input || !alpha)
        return fail(EXB_ERR_ARG, "exb_leaky_forward_scan_static: out, input and alpha are required");
    if (!mode_ok(alpha_mode, DECAY_FLAGS) || !scale_arg_ok(in_scale, in_scale_mode))
        return fail(EXB_ERR_ARG, "exb_leaky_forward_scan_static: bad parameter mode");
    if (!all_aligned4(out, input, v_init, alpha, in_scale, v_last)) return misaligned("exb_leaky_forward_scan_static");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    const int64_t need = exb::leaky_scan_workspace_bytes(B, T, M);
    if (need == 0)
        return fail(EXB_ERR_UNSUPPORTED, "exb_leaky_forward_scan_static: the time-parallel scan does not apply to "
                    "B=%lld T=%lld M=%lld (use exb_leaky_forward)", (long long)B, (long long)T, (long long)M);
    if ((size_t)need > exb::leaky_scan_static_capacity())
        return fail(EXB_ERR_ARG, "exb_leaky_forward_scan_static: this shape needs %lld bytes of scratch, the built-in "
                    "array holds %zu; use exb_leaky_forward_scan with a caller-provided workspace",
                    (long long)need, exb::leaky_scan_static_capacity());
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_leaky_forward_scan_static: cannot select device %d", device);
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess)
        return fail(EXB_ERR_DEVICE, "exb_leaky_forward_scan_static: cannot query the current device");
    exb::LeakyFwdArgs a;
    a.out = out; a.input = input; a.v_init = v_init;
    a.alpha = exb::make_param(alpha, alpha_mode, M);
    a.scale = exb::make_param(in_scale, in_scale_mode, M);
    a.v_last = v_last;
    a.out_sum = nullptr;
    a.B = B; a.T = T; a.M = M;
    bool used = false;
    cudaError_t e = exb::launch_leaky_forward_scan_static(a, current, (cudaStream_t)stream, &used);
    if (e != cudaSuccess) return launch_status(e, "exb_leaky_forward_scan_static");
    if (!used) return fail(EXB_ERR_UNSUPPORTED, "exb_leaky_forward_scan_static: shape or alignment not eligible");
    return EXB_OK;
}

}  // extern "C"

static int lif_syn_forward_impl(const char *who, float *spikes, uint8_t *spikes_u8, float *v_mem, float *i_syn, const float *input,
                        const float *v_init, const float *i_init,
                        const float *alpha_syn, int alpha_syn_mode, const float *scale_syn, int scale_syn_mode,
                        const float *scale_mem, int scale_mem_mode,
                        const float *alpha_mem, int alpha_mem_mode,
                        const float *subtract, int subtract_mode,
                        const float *theta, int theta_mode,
                        const float *theta_low, int theta_low_mode,
                        uint32_t max_spikes, int reset_mode,
                        float *v_post_last, float *i_last, unsigned long long *spike_count,
                        int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (int st = check_geometry(B, T, M, EXB_LAYOUT_BTM)) return st;
    if (spikes_u8) {
        if (!input || !alpha_syn || !alpha_mem || !theta)
            return fail(EXB_ERR_ARG, "%s: spikes, input, alpha_syn, alpha_mem and theta are required", who);
        if ((v_mem != nullptr) != (i_syn != nullptr))
            return fail(EXB_ERR_ARG, "%s: pass both v_mem and i_syn or neither", who);
    } else {
        if (!spikes || !input || !alpha_syn || !alpha_mem || !theta)
            return fail(EXB_ERR_ARG, "%s: spikes, input, alpha_syn, alpha_mem and theta are required", who);
        if ((v_mem != nullptr) != (i_syn != nullptr))
            return fail(EXB_ERR_ARG, "%s: pass both v_mem and i_syn or neither", who);
    }
    if (!mode_ok(alpha_syn_mode, DECAY_FLAGS) || !mode_ok(alpha_mem_mode, DECAY_FLAGS) || !mode_ok(theta_mode) ||
        !scale_arg_ok(scale_syn, scale_syn_mode) || !scale_arg_ok(scale_mem, scale_mem_mode) ||
        (subtract && !mode_ok(subtract_mode)) || (theta_low && !mode_ok(theta_low_mode)))
        return fail(EXB_ERR_ARG, "exb_lif_syn_forward: bad parameter mode");
    if (reset_mode != EXB_RESET_SUBTRACT && reset_mode != EXB_RESET_TO_VALUE)
        return fail(EXB_ERR_ARG, "exb_lif_syn_forward: bad reset mode %d", reset_mode);
    if (reset_mode == EXB_RESET_TO_VALUE && !subtract)
        return fail(EXB_ERR_ARG, "exb_lif_syn_forward: reset-to-value needs the value in `subtract`");
    if (!all_aligned4(spikes, v_mem, i_syn, input, v_init, i_init, alpha_syn, scale_syn, scale_mem, alpha_mem, subtract,
                      theta, theta_low, v_post_last, i_last) || (reinterpret_cast<uintptr_t>(spike_count) & 7u))
        return misaligned("exb_lif_syn_forward");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_lif_syn_forward: cannot select device %d", device);
    exb::LifSynFwdArgs a;
    a.spikes = spikes; a.v_mem = v_mem; a.i_syn = i_syn; a.input = input; a.v_init = v_init; a.i_init = i_init;
    a.np.alpha = exb::make_param(alpha_mem, alpha_mem_mode, M);
    a.np.c = exb::make_param(subtract, subtract_mode, M);
    a.np.th = exb::make_param(theta, theta_mode, M);
    a.np.lo = exb::make_param(theta_low, theta_low_mode, M);
    a.np.scale = exb::make_param(scale_mem, scale_mem_mode, M);
    a.alpha_syn = exb::make_param(alpha_syn, alpha_syn_mode, M);
    a.scale_syn = exb::make_param(scale_syn, scale_syn_mode, M);
    a.maxs = max_spikes;
    a.v_post_last = v_post_last; a.i_last = i_last; a.spike_count = spike_count;
    a.spikes_u8 = spikes_u8;
    a.B = B; a.T = T; a.M = M;
    bool used = false;
    cudaError_t e = exb::launch_lif_syn_forward(a, reset_mode, (cudaStream_t)stream, &used);
    if (e != cudaSuccess) return launch_status(e, "exb_lif_syn_forward");
    if (!used) return fail(EXB_ERR_UNSUPPORTED, "exb_lif_syn_forward: shape or alignment not eligible (needs M %% 4 == 0 and 16-byte aligned tensors)");
    return EXB_OK;
}

extern "C" {

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
                        int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    return lif_syn_forward_impl("exb_lif_syn_forward", spikes, nullptr, v_mem, i_syn, input, v_init, i_init, alpha_syn,
                                alpha_syn_mode, scale_syn, scale_syn_mode, scale_mem, scale_mem_mode, alpha_mem,
                                alpha_mem_mode, subtract, subtract_mode, theta, theta_mode, theta_low, theta_low_mode,
                                max_spikes, reset_mode, v_post_last, i_last, spike_count, B, T, M, device, stream);
}

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
                           int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (!spikes) return fail(EXB_ERR_ARG, "exb_lif_syn_forward_u8: spikes is required");
    if (max_spikes > 255u && !saturate)
        return fail(EXB_ERR_ARG, "exb_lif_syn_forward_u8: more than 255 spikes per step are possible (max_spikes = %u); "
                    "pass saturate != 0 to store min(count, 255)", max_spikes);
    return lif_syn_forward_impl("exb_lif_syn_forward_u8", nullptr, spikes, v_mem, i_syn, input, v_init, i_init, alpha_syn,
                                alpha_syn_mode, scale_syn, scale_syn_mode, scale_mem, scale_mem_mode, alpha_mem,
                                alpha_mem_mode, subtract, subtract_mode, theta, theta_mode, theta_low, theta_low_mode,
                                max_spikes, reset_mode, v_post_last, i_last, spike_count, B, T, M, device, stream);
}

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
                         int64_t B, int64_t T, int64_t M, int device, void *stream)
{
    if (int st = check_geometry(B, T, M, EXB_LAYOUT_BTM)) return st;
    if (!grad_input || !grad_spikes || !v_mem || !alpha_syn || !alpha_mem || !theta)
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: grad_input, grad_spikes, v_mem, alpha_syn, alpha_mem and theta are required");
    if (!mode_ok(alpha_syn_mode, DECAY_FLAGS) || !mode_ok(alpha_mem_mode, DECAY_FLAGS) || !mode_ok(theta_mode) ||
        !scale_arg_ok(scale_syn, scale_syn_mode) || !scale_arg_ok(scale_mem, scale_mem_mode) ||
        (subtract && !mode_ok(subtract_mode)) || (theta_low && !mode_ok(theta_low_mode)))
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: bad parameter mode");
    if (reset_mode != EXB_RESET_SUBTRACT && reset_mode != EXB_RESET_TO_VALUE)
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: bad reset mode %d", reset_mode);
    if (reset_mode == EXB_RESET_TO_VALUE && !subtract)
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: reset-to-value needs the value in `subtract`");
    if (surrogate_kind < EXB_SURR_GENERIC || surrogate_kind > EXB_SURR_PERIODIC_EXPONENTIAL)
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: unknown surrogate kind %d", surrogate_kind);
    if (surrogate_kind == EXB_SURR_GENERIC && !surr)
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: the generic surrogate needs the `surr` tensor");
    const int ngrads = (grad_alpha_mem != nullptr) + (grad_scale_mem != nullptr) + (grad_alpha_syn != nullptr) +
                       (grad_scale_syn != nullptr);
    if (ngrads != 0 && ngrads != 4)
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: pass all four parameter-gradient outputs or none");
    if ((acc_decay_mem != nullptr) != (acc_decay_syn != nullptr))
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: pass both acc_decay_mem and acc_decay_syn or neither");
    if (acc_decay_mem && ngrads != 0)
        return fail(EXB_ERR_ARG, "exb_lif_syn_backward: the accumulators replace the four per-instance outputs; pass NULL for those");
    if (acc_decay_mem && ((reinterpret_cast<uintptr_t>(acc_decay_mem) | reinterpret_cast<uintptr_t>(acc_decay_syn)) & 7u))
        return misaligned("exb_lif_syn_backward");
    if ((ngrads == 4 || acc_decay_mem) && !i_syn) return fail(EXB_ERR_ARG, "exb_lif_syn_backward: parameter gradients need `i_syn`");
    if (!all_aligned4(grad_input, grad_alpha_mem, grad_scale_mem, grad_alpha_syn, grad_scale_syn, grad_v_init, grad_i_init,
                      grad_spikes, grad_v_mem, grad_v_last, grad_i_syn, grad_i_last, v_mem, i_syn, surr, v_init, i_init,
                      alpha_syn, scale_syn, scale_mem, alpha_mem, subtract, theta, theta_low))
        return misaligned("exb_lif_syn_backward");
    if (B == 0 || M == 0 || T == 0) return EXB_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return fail(EXB_ERR_DEVICE, "exb_lif_syn_backward: cannot select device %d", device);
    exb::LifSynBwdArgs a;
    a.grad_input = grad_input;
    a.grad_alpha_mem = grad_alpha_mem; a.grad_scale_mem = grad_scale_mem;
    a.grad_alpha_syn = grad_alpha_syn; a.grad_scale_syn = grad_scale_syn;
    a.grad_v_init = grad_v_init; a.grad_i_init = grad_i_init;
    a.go = grad_spikes; a.gv = grad_v_mem; a.g_vlast = grad_v_last; a.g_isyn = grad_i_syn; a.g_ilast = grad_i_last;
    a.v_mem = v_mem; a.i_syn = i_syn; a.surr = (surrogate_kind == EXB_SURR_GENERIC) ? surr : nullptr;
    a.v_init = v_init; a.i_init = i_init;
    a.np.alpha = exb::make_param(alpha_mem, alpha_mem_mode, M);
    a.np.c = exb::make_param(subtract, subtract_mode, M);
    a.np.th = exb::make_param(theta, theta_mode, M);
    a.np.lo = exb::make_param(theta_low, theta_low_mode, M);
    a.np.scale = exb::make_param(scale_mem, scale_mem_mode, M);
    a.alpha_syn = exb::make_param(alpha_syn, alpha_syn_mode, M);
    a.scale_syn = exb::make_param(scale_syn, scale_syn_mode, M);
    a.maxs = max_spikes; a.p0 = surr_p0; a.p1 = surr_p1;
    a.acc_decay_mem = acc_decay_mem; a.acc_decay_syn = acc_decay_syn;
    a.B = B; a.T = T; a.M = M;
    bool used = false;
    cudaError_t e = exb::launch_lif_syn_backward(a, reset_mode, surrogate_kind, (cudaStream_t)stream, &used);
    if (e != cudaSuccess) return launch_status(e, "exb_lif_syn_backward");
    if (!used) return fail(EXB_ERR_UNSUPPORTED, "exb_lif_syn_backward: shape or alignment not eligible");
    return EXB_OK;
}

}  // extern "C"
