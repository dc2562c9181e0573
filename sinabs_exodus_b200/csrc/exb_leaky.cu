// Leaky-integrator kernels (ExpLeak layer and the synaptic stage of LIF):
//     forward   v_t = alpha*v_{t-1} + scale*in_t
//     backward  G_t = alpha*G_{t+1} + grad_out_t,  grad_in_t = scale*G_t
//               d/d alpha = sum_t G_t*v_{t-1},     d/d scale = sum_t G_t*in_t
//
// This file: the [N,T]-layout kernels and the launchers of both layouts.  The
// time-major (B,T,M) kernels are in exb_tma_kernels.cu (TMA-staged, incl. the
// time-parallel scan) and exb_ring.cuh (cp.async rings).
//
// [N,T]: the recurrence is linear, so one warp owns one neuron row and scans
// it 32*E time steps at a time: every lane integrates E consecutive steps,
// a warp-shuffle scan combines the 32 lane aggregates (multipliers
// alpha^(E*2^d)), and the carry of the segment moves on in a register.  Loads
// and stores are contiguous along time, no transposition is needed.
#include "exb_kernels.cuh"

namespace exb {

// ===========================================================================
// [N,T]: warp-shuffle scan over time
// ===========================================================================
constexpr int SCAN_WARPS = 8;

struct ScanPowers {
    float a;        // alpha
    float pw[5];    // alpha^(E*2^d)
    float fwd;      // alpha^(E*lane)
    float bwd;      // alpha^(E*(31-lane))
};

// The powers are formed in double and rounded once: a float power built by
// repeated squaring carries tens of ulps, which the carry chain of a long,
// slowly decaying row (alpha close to 1) would accumulate segment by segment.
template <int E>
__device__ __forceinline__ ScanPowers scan_powers(float alpha, int lane)
{
    ScanPowers p;
    p.a = alpha;
    double pw[5];
    double aE = (double)alpha;
#pragma unroll
    for (int e = 1; e < E; ++e) aE *= (double)alpha;
    pw[0] = aE;
#pragma unroll
    for (int d = 1; d < 5; ++d) pw[d] = pw[d - 1] * pw[d - 1];
    double f = 1.0, b = 1.0;
#pragma unroll
    for (int d = 0; d < 5; ++d) {
        p.pw[d] = (float)pw[d];
        if (lane & (1 << d)) f *= pw[d];
        if ((31 - lane) & (1 << d)) b *= pw[d];
    }
    p.fwd = (float)f;
    p.bwd = (float)b;
    return p;
}

template <int E>
__device__ __forceinline__ void load_seg(float (&x)[E], const float *row, int64_t t, int64_t T)
{
    if (E == 4) {
        if (t + 4 <= T) {
            ldv<4>(reinterpret_cast<float(&)[4]>(x), row + t);
        } else {
#pragma unroll
            for (int e = 0; e < E; ++e) x[e] = (t + e < T) ? __ldcs(row + t + e) : 0.0f;
        }
    } else {
#pragma unroll
        for (int e = 0; e < E; ++e) x[e] = (t + e < T) ? __ldcs(row + t + e) : 0.0f;
    }
}

template <int E>
__device__ __forceinline__ void store_seg(float *row, const float (&x)[E], int64_t t, int64_t T)
{
    if (E == 4 && t + 4 <= T) {
        stv<4>(row + t, reinterpret_cast<const float(&)[4]>(x));
    } else {
#pragma unroll
        for (int e = 0; e < E; ++e)
            if (t + e < T) __stcs(row + t + e, x[e]);
    }
}

template <int E>
__global__ void __launch_bounds__(SCAN_WARPS * 32) leaky_fwd_nt_kernel(const LeakyFwdArgs A)
{
    const int lane = threadIdx.x & 31;
    const int64_t n = blockIdx.x * (int64_t)SCAN_WARPS + (threadIdx.x >> 5);
    const int64_t N = A.B * A.M, T = A.T;
    if (n >= N) return;
    const int64_t b = n / A.M, m = n - b * A.M;
    const float alpha_nm = decay_of(A.alpha, b, m);
    const ScanPowers p = scan_powers<E>(alpha_nm, lane);
    const float sc = scale_of(A.scale, alpha_nm, b, m);
    float carry = A.v_init ? __ldg(A.v_init + n) : 0.0f;
    const float *rin = A.input + n * T;
    float *rout = A.out + n * T;

    double total = 0.0;
    float x[E], xnext[E];
    load_seg<E>(x, rin, (int64_t)lane * E, T);
    for (int64_t t0 = 0; t0 < T; t0 += 32 * E) {
        const int64_t t = t0 + (int64_t)lane * E;
        load_seg<E>(xnext, rin, t + 32 * E, T);
        float y = 0.0f;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            x[e] = __fmul_rn(sc, x[e]);
            y = __fmaf_rn(y, p.a, x[e]);
        }
#pragma unroll
        for (int d = 0; d < 5; ++d) {
            const float up = __shfl_up_sync(0xffffffffu, y, 1 << d);
            if (lane >= (1 << d)) y = __fmaf_rn(p.pw[d], up, y);
        }
        float ex = __shfl_up_sync(0xffffffffu, y, 1);
        if (lane == 0) ex = 0.0f;
        float o = __fmaf_rn(p.fwd, carry, ex);
        float res[E];
#pragma unroll
        for (int e = 0; e < E; ++e) {
            o = __fmaf_rn(o, p.a, x[e]);
            res[e] = o;
        }
        store_seg<E>(rout, res, t, T);
        if (A.v_last) {
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (t + e == T - 1) A.v_last[n] = res[e];
        }
        if (A.out_sum) {
            float part = 0.0f;
#pragma unroll
            for (int e = 0; e < E; ++e)
                if (t + e < T) part += res[e];
            total += (double)part;
        }
        carry = __shfl_sync(0xffffffffu, o, 31);
#pragma unroll
        for (int e = 0; e < E; ++e) x[e] = xnext[e];
    }
    if (A.out_sum) warp_add_f64(A.out_sum, total, lane);
}

template <int E, bool WA, bool WS>
__global__ void __launch_bounds__(SCAN_WARPS * 32) leaky_bwd_nt_kernel(const LeakyBwdArgs A)
{
    const int lane = threadIdx.x & 31;
    const int64_t n = blockIdx.x * (int64_t)SCAN_WARPS + (threadIdx.x >> 5);
    const int64_t N = A.B * A.M, T = A.T;
    if (n >= N) return;
    const int64_t b = n / A.M, m = n - b * A.M;
    const float alpha_nm = decay_of(A.alpha, b, m);
    const ScanPowers p = scan_powers<E>(alpha_nm, lane);
    const float sc = scale_of(A.scale, alpha_nm, b, m);
    const float vinit = A.v_init ? __ldg(A.v_init + n) : 0.0f;
    const float glast = A.g_last ? __ldg(A.g_last + n) : 0.0f;
    const float *rgo = A.go + n * T;
    const float *rout = WA ? A.out + n * T : nullptr;
    const float *rin = WS ? A.input + n * T : nullptr;
    float *rgi = A.grad_input + n * T;
    float carry = 0.0f, ag = 0.0f, sg = 0.0f;
    constexpr int SEG = 32 * E;

    for (int64_t t0 = ((T - 1) / SEG) * SEG; t0 >= 0; t0 -= SEG) {
        const int64_t t = t0 + (int64_t)lane * E;
        float g[E], o[E], x[E];
        load_seg<E>(g, rgo, t, T);
        if (WA) load_seg<E>(o, rout, t, T);
        if (WS) load_seg<E>(x, rin, t, T);
#pragma unroll
        for (int e = 0; e < E; ++e)
            if (t + e == T - 1) g[e] = __fadd_rn(g[e], glast);
        float y = 0.0f;
#pragma unroll
        for (int e = E - 1; e >= 0; --e) y = __fmaf_rn(y, p.a, g[e]);
#pragma unroll
        for (int d = 0; d < 5; ++d) {
            const float dn = __shfl_down_sync(0xffffffffu, y, 1 << d);
            if (lane + (1 << d) < 32) y = __fmaf_rn(p.pw[d], dn, y);
        }
        float ex = __shfl_down_sync(0xffffffffu, y, 1);
        if (lane == 31) ex = 0.0f;
        float G = __fmaf_rn(p.bwd, carry, ex);
        float res[E], Gs[E];
#pragma unroll
        for (int e = E - 1; e >= 0; --e) {
            G = __fmaf_rn(G, p.a, g[e]);
            Gs[e] = G;
            res[e] = __fmul_rn(sc, G);
            if (WS) sg = __fmaf_rn(G, x[e], sg);
        }
        store_seg<E>(rgi, res, t, T);
        if (WA) {
            // v_{t-1} for the lane's first step comes from the lane to the left;
            // lane 0 fetches it from memory (or takes v_init at t = 0).
            float prev = __shfl_up_sync(0xffffffffu, o[E - 1], 1);
            if (lane == 0) prev = (t0 > 0) ? __ldg(rout + t0 - 1) : vinit;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                if (t + e < T) ag = __fmaf_rn(Gs[e], prev, ag);
                prev = o[e];
            }
        }
        carry = __shfl_sync(0xffffffffu, G, 0);
    }
    if (A.grad_init && lane == 0) A.grad_init[n] = __fmul_rn(p.a, carry);
    if (WA) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ag += __shfl_xor_sync(0xffffffffu, ag, off);
        if (lane == 0) A.grad_alpha[n] = ag;
    }
    if (WS) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sg += __shfl_xor_sync(0xffffffffu, sg, off);
        if (lane == 0) A.grad_scale[n] = sg;
    }
}

// ===========================================================================
// launchers
// ===========================================================================
static inline bool all_aligned16(std::initializer_list<const void *> ptrs)
{
    for (const void *p : ptrs)
        if (p && !aligned16(p)) return false;
    return true;
}

}  // namespace exb
#include "exb_ring.cuh"
namespace exb {

cudaError_t launch_leaky_forward(const LeakyFwdArgs &a, int layout, cudaStream_t s)
{
    if (layout == EXB_LAYOUT_BTM && tma_enabled()) {
        bool used = false;
        cudaError_t e = launch_leaky_forward_tma(a, s, &used);
        if (e != cudaSuccess || used) return e;
    }
    if (layout == EXB_LAYOUT_BTM) {
        if (a.M % 4 == 0 && all_aligned16({a.out, a.input})) {
            cudaError_t e = launch_ring<4>(leaky_fwd_btm_ring_kernel<4>, a, 1, s);
            if (e != cudaSuccess) return e;
        } else {
            cudaError_t e = can_vec2(a.M, {a.out, a.input}) ? launch_ring<2>(leaky_fwd_btm_ring_kernel<2>, a, 1, s)
                                                            : launch_ring<1>(leaky_fwd_btm_ring_kernel<1>, a, 1, s);
            if (e != cudaSuccess) return e;
        }
    } else {
        const int64_t N = a.B * a.M;
        const unsigned grid = (unsigned)((N + SCAN_WARPS - 1) / SCAN_WARPS);
        if (a.T % 4 == 0 && all_aligned16({a.out, a.input}))
            leaky_fwd_nt_kernel<4><<<grid, SCAN_WARPS * 32, 0, s>>>(a);
        else
            leaky_fwd_nt_kernel<1><<<grid, SCAN_WARPS * 32, 0, s>>>(a);
    }
    return cudaPeekAtLastError();
}

template <bool WA, bool WS>
static cudaError_t launch_leaky_bwd_t(const LeakyBwdArgs &a, int layout, cudaStream_t s)
{
    if (layout == EXB_LAYOUT_BTM) {
        if (a.M % 4 == 0 && all_aligned16({a.grad_input, a.go, a.out, a.input})) {
            cudaError_t e = launch_ring<4>(leaky_bwd_btm_ring_kernel<4, WA, WS>, a, 1 + (WA ? 1 : 0) + (WS ? 1 : 0), s);
            if (e != cudaSuccess) return e;
        } else {
            const int nt = 1 + (WA ? 1 : 0) + (WS ? 1 : 0);
            cudaError_t e = can_vec2(a.M, {a.grad_input, a.go, a.out, a.input})
                                ? launch_ring<2>(leaky_bwd_btm_ring_kernel<2, WA, WS>, a, nt, s)
                                : launch_ring<1>(leaky_bwd_btm_ring_kernel<1, WA, WS>, a, nt, s);
            if (e != cudaSuccess) return e;
        }
    } else {
        const int64_t N = a.B * a.M;
        const unsigned grid = (unsigned)((N + SCAN_WARPS - 1) / SCAN_WARPS);
        if (a.T % 4 == 0 && all_aligned16({a.grad_input, a.go, a.out, a.input}))
            leaky_bwd_nt_kernel<4, WA, WS><<<grid, SCAN_WARPS * 32, 0, s>>>(a);
        else
            leaky_bwd_nt_kernel<1, WA, WS><<<grid, SCAN_WARPS * 32, 0, s>>>(a);
    }
    return cudaPeekAtLastError();
}

cudaError_t launch_leaky_backward(const LeakyBwdArgs &a, int layout, cudaStream_t s)
{
    if (layout == EXB_LAYOUT_BTM && tma_enabled()) {
        bool used = false;
        cudaError_t e = launch_leaky_backward_tma(a, s, &used);
        if (e != cudaSuccess || used) return e;
    }
    if (a.acc_decay) return cudaErrorNotSupported;      // only the TMA-staged kernels reduce in the kernel
    const bool wa = a.grad_alpha != nullptr, ws = a.grad_scale != nullptr;
    if (wa && ws) return launch_leaky_bwd_t<true, true>(a, layout, s);
    if (wa) return launch_leaky_bwd_t<true, false>(a, layout, s);
    if (ws) return launch_leaky_bwd_t<false, true>(a, layout, s);
    return launch_leaky_bwd_t<false, false>(a, layout, s);
}

}  // namespace exb
