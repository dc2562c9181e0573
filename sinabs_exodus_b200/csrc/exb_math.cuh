// Per-step neuron arithmetic shared by every kernel of the library, plus the
// small vector load/store helpers.  Everything here is float32 with the
// roundings written out (__fmaf_rn, __fmul_rn, ...) so that the association is
// the same in every kernel and does not depend on compiler contraction.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <math.h>

#include "../../include/exodus_b200.h"

namespace exb {

// A per-neuron parameter that is not expanded by the caller:
// value(b, m) = p[b*sb + m*sm]; scalar (0,0), per-m (0,1), per-n (M,1).
// `flags` are the EXB_PARAM_IS_TAU / EXB_SCALE_* bits of the mode the caller passed.
struct Param {
    const float *p;
    int64_t sb, sm;
    int flags;
    __device__ __forceinline__ float get(int64_t b, int64_t m, float dflt) const
    {
        return p ? __ldg(p + b * sb + m * sm) : dflt;
    }
};

__host__ inline Param make_param(const float *p, int mode, int64_t M)
{
    Param r;
    r.p = p;
    r.flags = mode & ~EXB_PARAM_SHAPE_MASK;
    mode &= EXB_PARAM_SHAPE_MASK;
    r.sb = (mode == EXB_PARAM_PER_N) ? M : 0;
    r.sm = (mode == EXB_PARAM_SCALAR) ? 0 : 1;
    return r;
}

// Decay per step from the value the caller passed: alpha itself, or exp(-1/tau) with EXB_PARAM_IS_TAU
// (correctly rounded reciprocal, exact negation, expf: the roundings of `torch.exp(-1.0 / tau)`).
__device__ __forceinline__ float decay_of(const Param &a, int64_t b, int64_t m)
{
    const float x = a.get(b, m, 1.0f);
    return (a.flags & EXB_PARAM_IS_TAU) ? expf(-__frcp_rn(x)) : x;
}

// Input scale: the given value (1 when there is none), replaced by 1 - alpha with EXB_SCALE_ONE_MINUS_ALPHA and then
// multiplied by alpha with EXB_SCALE_TIMES_ALPHA (the layers' norm_input and decay_early factors,
// layers/lif.py:194-195,206-214 of the reference, formed with the same roundings as the PyTorch expressions there).
__device__ __forceinline__ float scale_of(const Param &s, float alpha, int64_t b, int64_t m)
{
    float v = s.get(b, m, 1.0f);
    if (s.flags & EXB_SCALE_ONE_MINUS_ALPHA) v = __fsub_rn(1.0f, alpha);
    if (s.flags & EXB_SCALE_TIMES_ALPHA) v = __fmul_rn(v, alpha);
    return v;
}

// Gradient w.r.t. the value the caller passed for the decay, from the gradient w.r.t. alpha (ga) and, when the scale
// is derived from alpha, the gradient w.r.t. the scale (gs): d scale / d alpha is -1, +1 or 1 - 2*alpha; with
// EXB_PARAM_IS_TAU the chain rule through alpha = exp(-1/tau) multiplies by alpha / tau^2.  Linear in (ga, gs), so
// partial sums may be folded one by one.
__device__ __forceinline__ float decay_param_grad(float ga, float gs, const Param &a, const Param &s, float alpha,
                                                  int64_t b, int64_t m)
{
    float g = ga;
    const bool om = (s.flags & EXB_SCALE_ONE_MINUS_ALPHA) != 0, ta = (s.flags & EXB_SCALE_TIMES_ALPHA) != 0;
    if (om && ta) g = __fmaf_rn(__fmaf_rn(-2.0f, alpha, 1.0f), gs, g);
    else if (om) g = __fsub_rn(g, gs);
    else if (ta) g = __fmaf_rn(s.get(b, m, 1.0f), gs, g);
    if (a.flags & EXB_PARAM_IS_TAU) {
        const float r = __frcp_rn(a.get(b, m, 1.0f));
        g = __fmul_rn(__fmul_rn(__fmul_rn(g, alpha), r), r);
    }
    return g;
}

// Adds one thread's V per-neuron gradient values to a float64 accumulator that has the shape of the parameter
// `p` (1, M or B*M values).  Every lane of the warp must call.  One value: warp sum and one atomic per warp; M
// values: one atomic per neuron (the batch items meet there); B*M values: nobody else writes the slot.
template <int V>
__device__ __forceinline__ void acc_param_grad(double *acc, const Param &p, const float (&val)[V], bool valid, int64_t b,
                                               int64_t m, int lane)
{
    if (p.sb == 0 && p.sm == 0) {
        double s = 0.0;
        if (valid) {
#pragma unroll
            for (int j = 0; j < V; ++j) s += (double)val[j];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) atomicAdd(acc, s);
    } else if (valid) {
#pragma unroll
        for (int j = 0; j < V; ++j) atomicAdd(acc + b * p.sb + (m + j) * p.sm, (double)val[j]);
    }
}

// Limit on the number of spikes per step, in the forms the step needs.
struct SpikeCfg {
    unsigned maxs;   // maximum count (0xFFFFFFFF = no limit)
    unsigned oneu;   // min(1, maxs)
    float onef;      // the same as float
};

__host__ __device__ inline SpikeCfg make_spike_cfg(unsigned maxs)
{
    SpikeCfg c;
    c.maxs = maxs;
    c.oneu = maxs >= 1u ? 1u : 0u;
    c.onef = maxs >= 1u ? 1.0f : 0.0f;
    return c;
}

// Constants of one neuron, loaded once before the time loop.
struct Neuron {
    float alpha;   // decay
    float c;       // subtract value (or reset value)
    float th;      // threshold
    float th2;     // potential from which the spike count needs the division (see spike_count_f)
    float lo;      // lower bound, -inf when there is none
    float scale;   // input scale, 1 when there is none
};

struct NeuronParams {
    Param alpha, c, th, lo, scale;
    // true when no parameter varies between neurons
    __host__ bool uniform() const
    {
        const Param *all[5] = {&alpha, &c, &th, &lo, &scale};
        for (const Param *q : all)
            if (q->p && (q->sb != 0 || q->sm != 0)) return false;
        return true;
    }
    __device__ __forceinline__ Neuron load(int64_t b, int64_t m, const SpikeCfg &cfg) const
    {
        Neuron q;
        q.alpha = decay_of(alpha, b, m);
        q.th = th.get(b, m, 1.0f);
        q.c = c.get(b, m, q.th);
        // For a positive threshold and th <= v < 2*th the correctly rounded quotient v/th lies in
        // [1, 2), so the count is 1 without dividing; with at most one spike allowed the division is
        // never needed.  A non-positive threshold always takes the exact path.
        q.th2 = (q.th > 0.0f) ? ((cfg.maxs <= 1u) ? INFINITY : __fadd_rn(q.th, q.th)) : q.th;
        q.lo = lo.get(b, m, -INFINITY);
        q.scale = scale_of(scale, q.alpha, b, m);
        return q;
    }
};

// Spike count as float for membrane potential v: min(trunc(v/th), maxs) where v >= th, else 0
// (cuda/lif_kernels.h:80-84 of the reference).
__device__ __forceinline__ float spike_count_f(float v, const Neuron &q, const SpikeCfg &cfg)
{
    float af = (v >= q.th) ? cfg.onef : 0.0f;
    if (v >= q.th2) af = __uint2float_rn(min(__float2uint_rz(__fdiv_rn(v, q.th)), cfg.maxs));
    return af;
}

// Exact spike total of one thread: c32 counts steps that reached the threshold, c64 collects what
// the exact path adds or takes away (modulo 2^64, so that a correction below zero cancels).
struct SpikeTotal {
    unsigned c32;
    unsigned long long c64;
    __device__ __forceinline__ unsigned long long total(const SpikeCfg &cfg) const
    {
        return c64 + (unsigned long long)c32 * cfg.oneu;
    }
};

// One forward step (cuda/lif_kernels.h:61-84): reset with the previous count `af`, decay,
// integrate, clip from below, count spikes.  The common case (0 or 1 spike) is branch-free.
template <int RESET>
__device__ __forceinline__ void lif_step(float &v, float &af, float x, const Neuron &q, const SpikeCfg &cfg,
                                         SpikeTotal &cnt)
{
    if (RESET == EXB_RESET_SUBTRACT) v = __fmaf_rn(-af, q.c, v);
    else v = (af != 0.0f) ? q.c : v;
    v = __fmaf_rn(v, q.alpha, __fmul_rn(q.scale, x));
    v = (v < q.lo) ? q.lo : v;
    const bool sp = v >= q.th;
    af = sp ? cfg.onef : 0.0f;
    cnt.c32 += sp ? 1u : 0u;
    if (v >= q.th2) {
        const unsigned a = min(__float2uint_rz(__fdiv_rn(v, q.th)), cfg.maxs);
        af = __uint2float_rn(a);
        cnt.c64 += (unsigned long long)a - (unsigned long long)cfg.oneu;
    }
}

// The same step for the V neurons of one thread, with ONE branch for the rare exact path
// instead of one per neuron.
// NQ is V (one set of constants per neuron) or 1 (all parameters are single values, so the
// thread keeps one set for its V neurons: fewer registers, nothing recomputed).
template <int RESET, int V, int NQ>
__device__ __forceinline__ void lif_step_vec(float (&v)[V], float (&af)[V], const float (&x)[V], const Neuron (&qs)[NQ],
                                             const SpikeCfg &cfg, SpikeTotal &cnt)
{
    bool exact = false;
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const Neuron &q = qs[NQ == 1 ? 0 : j];
        if (RESET == EXB_RESET_SUBTRACT) v[j] = __fmaf_rn(-af[j], q.c, v[j]);
        else v[j] = (af[j] != 0.0f) ? q.c : v[j];
        v[j] = __fmaf_rn(v[j], q.alpha, __fmul_rn(q.scale, x[j]));
        v[j] = (v[j] < q.lo) ? q.lo : v[j];
        const bool sp = v[j] >= q.th;
        af[j] = sp ? cfg.onef : 0.0f;
        cnt.c32 += sp ? 1u : 0u;
        exact |= (v[j] >= q.th2);
    }
    if (exact) {
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const Neuron &q = qs[NQ == 1 ? 0 : j];
            if (v[j] >= q.th2) {
                const unsigned a = min(__float2uint_rz(__fdiv_rn(v[j], q.th)), cfg.maxs);
                af[j] = __uint2float_rn(a);
                cnt.c64 += (unsigned long long)a - (unsigned long long)cfg.oneu;
            }
        }
    }
}

// State after the reset that follows a step with spike count `af`.
template <int RESET>
__device__ __forceinline__ float post_reset(float v, float af, const Neuron &q)
{
    if (RESET == EXB_RESET_SUBTRACT) return __fmaf_rn(-af, q.c, v);
    return (af != 0.0f) ? q.c : v;
}

// The same for the recorded potential (layers/lif.py:256 of the reference: `v_mem - subtract * spikes`,
// formed by PyTorch with a rounded product): two roundings, so that a recording equals the reference's bit for bit.
template <int RESET>
__device__ __forceinline__ float recorded_post(float v, float af, const Neuron &q)
{
    if (RESET == EXB_RESET_SUBTRACT) return __fsub_rn(v, __fmul_rn(q.c, af));
    return (af != 0.0f) ? q.c : v;
}

// Surrogate-gradient constants of one neuron.
struct SurrConst {
    float k0, k1, k2, k3;
};

// 2^x by the special-function unit (relative error at most 2^-22).
__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// The exponential surrogates evaluate exp(-d/w) as 2^(-d * log2(e)/w) with the scaled reciprocal width
// prepared once per neuron: one multiplication and one special-function instruction per step where expf
// takes about ten.  Error: 2^-22 relative from the unit plus |d/w| * 1.7e-7 relative from the two roundings
// of the exponent, i.e. below 1e-6 of the surrogate's peak everywhere (checked against the float64 forms in
// the tests at 1e-5 on the gradients).
template <int SURR>
__device__ __forceinline__ SurrConst surr_prepare(const Neuron &q, float p0, float p1)
{
    constexpr float LOG2E = 1.4426950408889634f;
    SurrConst s;
    s.k0 = s.k1 = s.k2 = s.k3 = 0.0f;
    if (SURR == EXB_SURR_SINGLE_EXPONENTIAL) {
        const float w = __fmul_rn(q.th, p0);
        s.k0 = __fdiv_rn(LOG2E, w);       // log2(e)/width
        s.k1 = __fdiv_rn(p1, w);          // amplitude
    } else if (SURR == EXB_SURR_HEAVISIDE) {
        s.k0 = __fsub_rn(q.th, p0);       // window edge
        s.k1 = __fdiv_rn(1.0f, q.th);
    } else if (SURR == EXB_SURR_PERIODIC_EXPONENTIAL) {
        s.k0 = __fdiv_rn(LOG2E, p0);
        s.k1 = __fdiv_rn(p1, q.th);
        s.k2 = __fmul_rn(q.th, 0.5f);
        s.k3 = __fdiv_rn(1.0f, q.th);
    }
    return s;
}

// floor(u / th) for th > 0 without the division: the estimate floor(u * (1/th)) is off by at most one, and the
// sign of the exact remainder u - k*th (one fused multiply-add) says in which direction.  For th <= 0 (no
// sensible threshold) the IEEE quotient is used.
__device__ __forceinline__ float floor_div(float u, float th, float rth)
{
    if (!(th > 0.0f)) return floorf(__fdiv_rn(u, th));
    float k = floorf(__fmul_rn(u, rth));
    const float r = __fmaf_rn(-k, th, u);
    k = (r < 0.0f) ? k - 1.0f : k;
    k = (r >= th) ? k + 1.0f : k;
    return k;
}

template <int SURR>
__device__ __forceinline__ float surrogate(float v, const Neuron &q, const SurrConst &s, float loaded)
{
    if (SURR == EXB_SURR_SINGLE_EXPONENTIAL) {
        return __fmul_rn(s.k1, ex2_approx(__fmul_rn(-fabsf(__fsub_rn(v, q.th)), s.k0)));
    } else if (SURR == EXB_SURR_HEAVISIDE) {
        return (v >= s.k0) ? s.k1 : 0.0f;
    } else if (SURR == EXB_SURR_PERIODIC_EXPONENTIAL) {
        const float u = __fsub_rn(v, s.k2);
        const float w = (v < q.th) ? u : __fsub_rn(u, floor_div(u, q.th, s.k3));
        return __fmul_rn(s.k1, ex2_approx(__fmul_rn(-fabsf(__fsub_rn(w, s.k2)), s.k0)));
    }
    return loaded;
}

// Running state of the reverse-time sweep of one neuron.
struct BwdState {
    float R;      // R_{t+1}: gradient w.r.t. the membrane potential one step later
    float ag;     // alpha-gradient accumulator
    float sg;     // input-scale-gradient accumulator
    float vnext;  // v_{t+1} (only for SCALE_GRAD_FROM_STATE)
};

// How the gradient w.r.t. the input scale, sum_t R_t * x_t, is formed.
//   SCALE_GRAD_FROM_INPUT  reads the forward input x_t (one more tensor to stream)
//   SCALE_GRAD_FROM_STATE  uses scale*x_t = v_t - alpha*vpost_{t-1}, which holds wherever R_t != 0
//                          (a clipped step has R_t = 0), and divides the sum by scale at the end:
//                          nothing but v_mem is read.  Needs scale != 0.
enum { SCALE_GRAD_NONE = 0, SCALE_GRAD_FROM_INPUT = 1, SCALE_GRAD_FROM_STATE = 2 };

// One reverse step.  v: saved pre-reset membrane potential; go/gv: incoming
// gradients w.r.t. spikes and v_mem at this step; sl: caller-supplied surrogate
// (generic mode); x: unscaled forward input (only when WANT_SCALE_GRAD).
// Returns R_t; on return st.R == R_t.  `f_out`, `n_out` give the step's
// propagation factor and clip gate for the caller's first-step handling.
template <int SURR, int RESET, bool WANT_ALPHA_GRAD, int WANT_SCALE_GRAD>
__device__ __forceinline__ float lif_bwd_step(BwdState &st, float v, float go, float gv, float sl, float x,
                                              const Neuron &q, const SurrConst &sc, float cp, const SpikeCfg &cfg,
                                              float &f_out, bool &n_out)
{
    const float s = surrogate<SURR>(v, q, sc, sl);
    const bool n = v > q.lo;
    const float g = __fadd_rn(__fmul_rn(s, go), gv);
    float af = 0.0f;
    if (RESET == EXB_RESET_TO_VALUE || WANT_ALPHA_GRAD || WANT_SCALE_GRAD == SCALE_GRAD_FROM_STATE)
        af = spike_count_f(v, q, cfg);
    float f;
    if (RESET == EXB_RESET_SUBTRACT) f = __fmaf_rn(-cp, s, q.alpha);   // alpha - (alpha*c)*s
    else f = (af != 0.0f) ? 0.0f : q.alpha;
    if (WANT_ALPHA_GRAD || WANT_SCALE_GRAD == SCALE_GRAD_FROM_STATE) {
        const float vpost = post_reset<RESET>(v, af, q);
        if (WANT_ALPHA_GRAD) st.ag = __fmaf_rn(st.R, vpost, st.ag);
        if (WANT_SCALE_GRAD == SCALE_GRAD_FROM_STATE) {
            st.sg = __fmaf_rn(st.R, __fmaf_rn(-q.alpha, vpost, st.vnext), st.sg);   // R_{t+1} * scale*x_{t+1}
            st.vnext = v;
        }
    }
    const float Rt = n ? __fmaf_rn(f, st.R, g) : 0.0f;
    if (WANT_SCALE_GRAD == SCALE_GRAD_FROM_INPUT) st.sg = __fmaf_rn(Rt, x, st.sg);
    st.R = Rt;
    f_out = f;
    n_out = n;
    return Rt;
}

// A gradient G w.r.t. the post-reset state of the LAST step enters the sweep
// through that step's two incoming gradients: v_post = v - c*a gives
// go += -c*G and gv += G (reset-to-value: gv += G where no spike occurred).
template <int RESET>
__device__ __forceinline__ void fold_last_state_grad(float &go, float &gv, float G, float v,
                                                     const Neuron &q, const SpikeCfg &cfg)
{
    if (RESET == EXB_RESET_SUBTRACT) {
        go = __fmaf_rn(-q.c, G, go);
        gv = __fadd_rn(gv, G);
    } else {
        gv = __fadd_rn(gv, (spike_count_f(v, q, cfg) != 0.0f) ? 0.0f : G);
    }
}

// Terms of the alpha gradient that involve the initial state, added after the
// sweep reached t = 0 (st.R == R_0).  R1 is R_1 (0 when T == 1), f0/n0 the
// factor and clip gate of step 0.  The second term reproduces
// cuda/lif_kernels.h:219-238 of the reference, where the t = 0 accumulator is
// carried into t = 1 without the t = 0 clip gate.
template <int RESET>
__device__ __forceinline__ float alpha_grad_finish(const BwdState &st, float v_init, float R1, float f0, bool n0)
{
    float ag = __fmaf_rn(st.R, v_init, st.ag);
    if (RESET == EXB_RESET_SUBTRACT && !n0) ag = __fmaf_rn(__fmul_rn(v_init, f0), R1, ag);
    return ag;
}

// Gradient w.r.t. the input scale after the sweep reached t = 0 (st.R == R_0, st.vnext == v_0).
template <int WANT_SCALE_GRAD>
__device__ __forceinline__ float scale_grad_finish(const BwdState &st, float v_init, const Neuron &q)
{
    if (WANT_SCALE_GRAD == SCALE_GRAD_FROM_STATE)
        return __fdiv_rn(__fmaf_rn(st.R, __fmaf_rn(-q.alpha, v_init, st.vnext), st.sg), q.scale);
    return st.sg;
}

// ---- small vector helpers -------------------------------------------------
template <int V>
__device__ __forceinline__ void ldv(float (&d)[V], const float *p)
{
    if (V == 4) {
        const float4 t = __ldcs(reinterpret_cast<const float4 *>(p));
        d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
    } else if (V == 2) {
        const float2 t = __ldcs(reinterpret_cast<const float2 *>(p));
        d[0] = t.x; d[1] = t.y;
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] = __ldcs(p + j);
    }
}

template <int V>
__device__ __forceinline__ void stv(float *p, const float (&d)[V])
{
    if (V == 4) {
        __stcs(reinterpret_cast<float4 *>(p), make_float4(d[0], d[1], d[2], d[3]));
    } else if (V == 2) {
        __stcs(reinterpret_cast<float2 *>(p), make_float2(d[0], d[1]));
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) __stcs(p + j, d[j]);
    }
}

// Spike counts of one thread's V adjacent neurons to the output raster: float32 as the reference stores them
// (cuda/lif_kernels.h:87), or one byte each, saturating at 255 (the compact raster; V = 4 -> one 32-bit store).
template <int V>
__device__ __forceinline__ void st_spikes(float *p, const float (&af)[V]) { stv<V>(p, af); }

template <int V>
__device__ __forceinline__ void st_spikes(uint8_t *p, const float (&af)[V])
{
    unsigned b[V];
#pragma unroll
    for (int j = 0; j < V; ++j) b[j] = min(__float2uint_rz(af[j]), 255u);
    if (V == 4) {
        __stcs(reinterpret_cast<unsigned *>(p), b[0] | (b[1] << 8) | (b[2] << 16) | (b[3] << 24));
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) __stcs(p + j, (uint8_t)b[j]);
    }
}

}  // namespace exb
