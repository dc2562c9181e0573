// Time-major kernels for shapes the TMA path cannot take (M not a multiple of 4, or tensors that
// are not 16-byte aligned): thread-private software pipelines through shared memory.
//
// A TMA box needs 16-byte row pitches.  Without them a thread owns 1 neuron (or 2 when rows are
// 8-byte aligned) and walks through time; what limits such a kernel is the number of bytes it
// keeps in flight.  Holding many time steps in registers costs the occupancy that is needed for
// the same purpose (the register-buffered kernels reach 4.4 TB/s on c2-sized problems with odd M).
// Here every thread copies ITS OWN elements of the next time steps (up to 28) into its own shared-memory
// slots with cp.async (4 or 8 bytes), in commit groups of 4 steps.  No thread ever reads another
// thread's slot, so the only synchronisation is cp.async.wait_group: no barriers, no registers
// held by data in flight; a forward ring of 8 groups keeps 28 x 4 bytes x 1024 threads = 112 KB in
// flight per SM.
#pragma once

#include <initializer_list>

namespace exb {

constexpr int RING_G = 4;                    // time steps per commit group
constexpr int RING_THREADS = 256;
// Groups in a ring (ng: 8, 4 or 2; ng - 1 are in flight while one is consumed) are chosen by the
// launcher so that a CTA's rings stay within 64 KB; a ring holds RING_G * ng time steps per thread.

template <int BYTES>
__device__ __forceinline__ void ring_copy(float *dst, const float *src)
{
    static_assert(BYTES == 4 || BYTES == 8 || BYTES == 16, "cp.async sizes");
    asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src),
                 "n"(BYTES)
                 : "memory");
}

__device__ __forceinline__ void ring_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

// Wait until at most ng - 1 groups are pending (the count must be an immediate).
__device__ __forceinline__ void ring_wait(int ng)
{
    if (ng == 8) asm volatile("cp.async.wait_group 7;" ::: "memory");
    else if (ng == 4) asm volatile("cp.async.wait_group 3;" ::: "memory");
    else asm volatile("cp.async.wait_group 1;" ::: "memory");
}

// Slot of time step t for this thread: rows of RING_THREADS*V floats, one row per slot; mask = slots - 1.
template <int V>
__device__ __forceinline__ float *ring_slot(float *mine, int t, int mask)
{
    return mine + (t & mask) * (RING_THREADS * V);
}

template <int V>
__device__ __forceinline__ void lds_small(float (&d)[V], const float *p)
{
    if (V == 4) {
        const float4 t = *reinterpret_cast<const float4 *>(p);
        d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
    } else if (V == 2) {
        const float2 t = *reinterpret_cast<const float2 *>(p);
        d[0] = t.x; d[1] = t.y;
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] = p[j];
    }
}

// ===========================================================================
// forward
// ===========================================================================
template <int V, int RESET>
__global__ void __launch_bounds__(RING_THREADS, 4) lif_fwd_btm_ring_kernel(const LifFwdArgs A, const int ng)
{
    extern __shared__ __align__(16) float ring_smem[];
    const int64_t MV = A.M / V;
    const int64_t total = A.B * MV;
    int64_t gid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const bool valid = gid < total;
    if (!valid) gid = total - 1;   // keeps the warp whole for the final reduction; stores are skipped
    const int64_t b = gid / MV;
    const int64_t m = (gid - b * MV) * V;
    const int64_t n = b * A.M + m;
    const int64_t T = A.T, M = A.M;

    const SpikeCfg cfg = make_spike_cfg(A.maxs);
    Neuron q[V];
    float v[V], af[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        q[j] = A.np.load(b, m + j, cfg);
        v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
        af[j] = 0.0f;
    }
    const int64_t base = (b * T) * M + m;
    const float *in = A.input + base;
    float *sp = A.spikes + base;
    float *vm = A.v_mem + base;
    float *rec = A.v_post ? A.v_post + base : nullptr;      // optional record of the potential after each reset
    SpikeTotal cnt;
    cnt.c32 = 0u; cnt.c64 = 0ull;
    float *mine = ring_smem + threadIdx.x * V;
    const int mask = RING_G * ng - 1;

    // int time indices and pointers advanced step by step: 64-bit index arithmetic per element would
    // make the kernel instruction-bound
    const int Ti = (int)T;
    int t_issue = 0;
    const float *p_issue = in;
    auto issue = [&]() {      // a group past the end is empty but still counted
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            if (t_issue < Ti) ring_copy<4 * V>(ring_slot<V>(mine, t_issue, mask), p_issue);
            ++t_issue;
            p_issue += M;
        }
        ring_commit();
    };
    for (int g = 0; g < ng - 1; ++g) issue();
    for (int t0 = 0; t0 < Ti; t0 += RING_G) {
        issue();
        ring_wait(ng);
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            const int t = t0 + u;
            if (t < Ti) {
                float xs[V];
                lds_small<V>(xs, ring_slot<V>(mine, t, mask));
                lif_step_vec<RESET, V, V>(v, af, xs, q, cfg, cnt);
                if (valid) {
                    stv<V>(sp, af);
                    stv<V>(vm, v);
                    if (rec) {
                        float vp[V];
#pragma unroll
                        for (int j = 0; j < V; ++j) vp[j] = recorded_post<RESET>(v[j], af[j], q[j]);
                        stv<V>(rec, vp);
                    }
                }
                sp += M;
                vm += M;
                if (rec) rec += M;
            }
        }
    }
    if (A.v_post_last && valid) {
#pragma unroll
        for (int j = 0; j < V; ++j) A.v_post_last[n + j] = post_reset<RESET>(v[j], af[j], q[j]);
    }
    if (A.spike_count) {
        const unsigned long long tot = warp_sum_u64(valid ? cnt.total(cfg) : 0ull);
        if ((threadIdx.x & 31) == 0 && tot) atomicAdd(A.spike_count, tot);
    }
}

// ===========================================================================
// backward: the same pipeline from the last time step down, one ring per streamed tensor
// ===========================================================================
template <int V, int SURR, int RESET, bool WA, int WS>
__global__ void __launch_bounds__(RING_THREADS, 4) lif_bwd_btm_ring_kernel(const LifBwdArgs A, const int ng)
{
    extern __shared__ __align__(16) float ring_smem[];
    const int64_t MV = A.M / V;
    const int64_t total = A.B * MV;
    const int64_t gid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (gid >= total) return;
    const int64_t b = gid / MV;
    const int64_t m = (gid - b * MV) * V;
    const int64_t n = b * A.M + m;
    const int64_t T = A.T, M = A.M;

    const SpikeCfg cfg = make_spike_cfg(A.maxs);
    Neuron q[V];
    SurrConst sc[V];
    float cp[V];
    BwdState st[V];
    float Rprev[V], f0[V], glast[V];
    bool n0[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        q[j] = A.np.load(b, m + j, cfg);
        sc[j] = surr_prepare<SURR>(q[j], A.p0, A.p1);
        cp[j] = __fmul_rn(q[j].alpha, q[j].c);
        st[j].R = 0.0f; st[j].ag = 0.0f; st[j].sg = 0.0f; st[j].vnext = 0.0f;
        Rprev[j] = 0.0f; f0[j] = 0.0f; n0[j] = true;
        glast[j] = A.g_last ? __ldg(A.g_last + n + j) : 0.0f;
    }
    const int64_t base = (b * T) * M + m;
    const float *go = A.go + base;
    const float *vm = A.v_mem + base;
    const float *gv = A.gv ? A.gv + base : nullptr;
    const float *sl = (SURR == EXB_SURR_GENERIC) ? A.surr + base : nullptr;
    const float *xin = (WS == SCALE_GRAD_FROM_INPUT) ? A.input + base : nullptr;
    float *gi = A.grad_input + base;

    const int mask = RING_G * ng - 1;
    const int TENSOR = RING_G * ng * RING_THREADS * V;     // floats of one tensor's ring
    float *r_go = ring_smem + threadIdx.x * V;
    float *r_vm = r_go + TENSOR;
    float *r_gv = r_vm + TENSOR;                          // present only when gv is streamed
    float *r_sl = r_gv + (gv ? TENSOR : 0);
    float *r_xi = r_sl + ((SURR == EXB_SURR_GENERIC) ? TENSOR : 0);

    // processing index p = 0, 1, ... walks t = T-1, T-2, ...; slots are addressed by p.  One element
    // offset (from the tensors' common base) serves all streamed tensors.
    const int Ti = (int)T;
    int p_issue = 0;
    int64_t off_issue = (T - 1) * M;
    auto issue = [&]() {
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            if (p_issue < Ti) {
                ring_copy<4 * V>(ring_slot<V>(r_go, p_issue, mask), go + off_issue);
                ring_copy<4 * V>(ring_slot<V>(r_vm, p_issue, mask), vm + off_issue);
                if (gv) ring_copy<4 * V>(ring_slot<V>(r_gv, p_issue, mask), gv + off_issue);
                if (SURR == EXB_SURR_GENERIC) ring_copy<4 * V>(ring_slot<V>(r_sl, p_issue, mask), sl + off_issue);
                if (WS == SCALE_GRAD_FROM_INPUT) ring_copy<4 * V>(ring_slot<V>(r_xi, p_issue, mask), xin + off_issue);
            }
            ++p_issue;
            off_issue -= M;
        }
        ring_commit();
    };
    for (int g = 0; g < ng - 1; ++g) issue();
    gi += (T - 1) * M;
    for (int p0 = 0; p0 < Ti; p0 += RING_G) {
        issue();
        ring_wait(ng);
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            const int p = p0 + u;
            if (p < Ti) {
                float xgo[V], xv[V];
                float xgv[V] = {}, xsl[V] = {}, xx[V] = {};
                lds_small<V>(xgo, ring_slot<V>(r_go, p, mask));
                lds_small<V>(xv, ring_slot<V>(r_vm, p, mask));
                if (gv) lds_small<V>(xgv, ring_slot<V>(r_gv, p, mask));
                if (SURR == EXB_SURR_GENERIC) lds_small<V>(xsl, ring_slot<V>(r_sl, p, mask));
                if (WS == SCALE_GRAD_FROM_INPUT) lds_small<V>(xx, ring_slot<V>(r_xi, p, mask));
                float r[V];
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    if (p == 0 && A.g_last) fold_last_state_grad<RESET>(xgo[j], xgv[j], glast[j], xv[j], q[j], cfg);
                    Rprev[j] = st[j].R;
                    const float Rt = lif_bwd_step<SURR, RESET, WA, WS>(st[j], xv[j], xgo[j], xgv[j], xsl[j], xx[j], q[j],
                                                                      sc[j], cp[j], cfg, f0[j], n0[j]);
                    r[j] = __fmul_rn(q[j].scale, Rt);
                }
                stv<V>(gi, r);
                gi -= M;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
        if (A.grad_init) A.grad_init[n + j] = __fmul_rn(q[j].alpha, st[j].R);
        const float vi = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
        if (WA) A.grad_alpha[n + j] = alpha_grad_finish<RESET>(st[j], vi, Rprev[j], f0[j], n0[j]);
        if (WS) A.grad_scale[n + j] = scale_grad_finish<WS>(st[j], vi, q[j]);
    }
}

// ===========================================================================
// leaky integrator, same pipelines
// ===========================================================================
template <int V>
__global__ void __launch_bounds__(RING_THREADS, 4) leaky_fwd_btm_ring_kernel(const LeakyFwdArgs A, const int ng)
{
    extern __shared__ __align__(16) float ring_smem[];
    const int64_t MV = A.M / V;
    const int64_t total = A.B * MV;
    int64_t gid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    const bool valid = gid < total;
    if (!valid) gid = total - 1;   // keeps the warp whole for the final reduction; stores are skipped
    const int64_t b = gid / MV;
    const int64_t m = (gid - b * MV) * V;
    const int64_t n = b * A.M + m;
    const int64_t M = A.M;
    const int Ti = (int)A.T;
    float al[V], sc[V], v[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        al[j] = decay_of(A.alpha, b, m + j);
        sc[j] = scale_of(A.scale, al[j], b, m + j);
        v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
    }
    const int64_t base = (b * A.T) * M + m;
    float *out = A.out + base;
    float *mine = ring_smem + threadIdx.x * V;
    const int mask = RING_G * ng - 1;
    double total_out = 0.0;

    int t_issue = 0;
    const float *p_issue = A.input + base;
    auto issue = [&]() {
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            if (t_issue < Ti) ring_copy<4 * V>(ring_slot<V>(mine, t_issue, mask), p_issue);
            ++t_issue;
            p_issue += M;
        }
        ring_commit();
    };
    for (int g = 0; g < ng - 1; ++g) issue();
    for (int t0 = 0; t0 < Ti; t0 += RING_G) {
        issue();
        ring_wait(ng);
        float part = 0.0f;
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            const int t = t0 + u;
            if (t < Ti) {
                float xs[V];
                lds_small<V>(xs, ring_slot<V>(mine, t, mask));
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    v[j] = __fmaf_rn(v[j], al[j], __fmul_rn(sc[j], xs[j]));
                    part += v[j];
                }
                if (valid) stv<V>(out, v);
                out += M;
            }
        }
        total_out += (double)part;
    }
    if (A.v_last && valid) {
#pragma unroll
        for (int j = 0; j < V; ++j) A.v_last[n + j] = v[j];
    }
    if (A.out_sum) warp_add_f64(A.out_sum, valid ? total_out : 0.0, threadIdx.x & 31);
}

template <int V, bool WA, bool WS>
__global__ void __launch_bounds__(RING_THREADS, 4) leaky_bwd_btm_ring_kernel(const LeakyBwdArgs A, const int ng)
{
    extern __shared__ __align__(16) float ring_smem[];
    const int64_t MV = A.M / V;
    const int64_t gid = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (gid >= A.B * MV) return;
    const int64_t b = gid / MV;
    const int64_t m = (gid - b * MV) * V;
    const int64_t n = b * A.M + m;
    const int64_t T = A.T, M = A.M;
    const int Ti = (int)T;
    float al[V], sc[V], G[V], ag[V], sg[V], glast[V];
#pragma unroll
    for (int j = 0; j < V; ++j) {
        al[j] = decay_of(A.alpha, b, m + j);
        sc[j] = scale_of(A.scale, al[j], b, m + j);
        G[j] = 0.0f; ag[j] = 0.0f; sg[j] = 0.0f;
        glast[j] = A.g_last ? __ldg(A.g_last + n + j) : 0.0f;
    }
    const int64_t base = (b * T) * M + m;
    const float *go = A.go + base;
    const float *vo = WA ? A.out + base : nullptr;
    const float *xin = WS ? A.input + base : nullptr;
    float *gi = A.grad_input + base + (T - 1) * M;

    const int mask = RING_G * ng - 1;
    const int TENSOR = RING_G * ng * RING_THREADS * V;
    float *r_go = ring_smem + threadIdx.x * V;
    float *r_vo = r_go + TENSOR;
    float *r_xi = r_vo + (WA ? TENSOR : 0);

    int p_issue = 0;
    int64_t off_issue = (T - 1) * M;
    auto issue = [&]() {
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            if (p_issue < Ti) {
                ring_copy<4 * V>(ring_slot<V>(r_go, p_issue, mask), go + off_issue);
                if (WA) ring_copy<4 * V>(ring_slot<V>(r_vo, p_issue, mask), vo + off_issue);
                if (WS) ring_copy<4 * V>(ring_slot<V>(r_xi, p_issue, mask), xin + off_issue);
            }
            ++p_issue;
            off_issue -= M;
        }
        ring_commit();
    };
    for (int g = 0; g < ng - 1; ++g) issue();
    for (int p0 = 0; p0 < Ti; p0 += RING_G) {
        issue();
        ring_wait(ng);
#pragma unroll
        for (int u = 0; u < RING_G; ++u) {
            const int p = p0 + u;
            if (p < Ti) {
                float xgo[V];
                float xo[V] = {}, xx[V] = {};
                lds_small<V>(xgo, ring_slot<V>(r_go, p, mask));
                if (WA) lds_small<V>(xo, ring_slot<V>(r_vo, p, mask));
                if (WS) lds_small<V>(xx, ring_slot<V>(r_xi, p, mask));
                float r[V];
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    if (p == 0) xgo[j] = __fadd_rn(xgo[j], glast[j]);
                    if (WA) ag[j] = __fmaf_rn(G[j], xo[j], ag[j]);      // G_{t+1} * v_t
                    G[j] = __fmaf_rn(G[j], al[j], xgo[j]);
                    if (WS) sg[j] = __fmaf_rn(G[j], xx[j], sg[j]);
                    r[j] = __fmul_rn(sc[j], G[j]);
                }
                stv<V>(gi, r);
                gi -= M;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
        if (A.grad_init) A.grad_init[n + j] = __fmul_rn(al[j], G[j]);
        if (WA) A.grad_alpha[n + j] = __fmaf_rn(G[j], A.v_init ? __ldg(A.v_init + n + j) : 0.0f, ag[j]);
        if (WS) A.grad_scale[n + j] = sg[j];
    }
}

// Groups per ring such that the rings of `ntensors` tensors take at most 64 KB per CTA.
template <int V>
static inline int ring_groups(int ntensors)
{
    const int fit = 16 / (ntensors * V);      // 64 KB / (RING_G * RING_THREADS * 4 bytes * V * ntensors)
    return fit >= 8 ? 8 : (fit >= 4 ? 4 : 2);
}

template <int V>
static inline size_t ring_smem_bytes(int ntensors, int ng)
{
    return (size_t)ntensors * RING_G * ng * RING_THREADS * V * sizeof(float);
}

static inline bool can_vec2(int64_t M, std::initializer_list<const void *> ptrs)
{
    if (M % 2) return false;
    for (const void *p : ptrs)
        if (p && (reinterpret_cast<uintptr_t>(p) & 7u)) return false;
    return true;
}

template <int V, typename K, typename Args>
static cudaError_t launch_ring(K kern, const Args &a, int ntensors, cudaStream_t s)
{
    const int ng = ring_groups<V>(ntensors);
    const size_t sm = ring_smem_bytes<V>(ntensors, ng);
    if (sm > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
        if (e != cudaSuccess) return e;
    }
    const int64_t total = a.B * (a.M / V);
    kern<<<(unsigned)((total + RING_THREADS - 1) / RING_THREADS), RING_THREADS, sm, s>>>(a, ng);
    return cudaSuccess;
}

}  // namespace exb
