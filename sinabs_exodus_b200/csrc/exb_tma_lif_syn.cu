// LIF layer with synaptic stage as ONE kernel per direction (time-major layout, TMA-staged).
//
// forward   i_t = alpha_syn*i_{t-1} + scale_syn*x_t          (synaptic leaky integrator)
//           v_t, a_t = spike step on scale_mem*i_t            (membrane, see lif_step)
//           one read (x), three writes (i_syn, spikes, v_mem): 16 B per neuron-step instead of
//           8 + 12 for the two separate kernels (the second of which re-reads i_syn)
// backward  R_t from (grad_spikes, v_mem) exactly as lif_bwd_step does, then in the same step
//           G_t = alpha_syn*G_{t+1} + scale_mem*R_t (+ grad_i_syn_t),  grad_x_t = scale_syn*G_t
//           reads grad_spikes, v_mem (and i_syn when parameter gradients are wanted), writes grad_x.
//
// Parameter gradients (all four or none): alpha_mem and scale_mem as in the membrane kernel
// (scale_mem from the streamed i_syn), alpha_syn = sum_t G_t*i_{t-1}, and scale_syn rebuilt from
// scale_syn*x_t = i_t - alpha_syn*i_{t-1}, so x is never read again.
#include "exb_tma_common.cuh"

namespace exb {

struct TmaMaps6 {
    CUtensorMap m[6];
};

template <int RESET, int NW, int V, bool UNI>
__global__ void __launch_bounds__((NW + 1) * 32, MinBlocks<NW, V, (V == 4)>::value)
lif_syn_fwd_tma_kernel(const __grid_constant__ TmaMaps6 maps, const LifSynFwdArgs A, const int tiles_m, const PipeCfg pc)
{
    using G = TileGeom<NW, V>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    const int tensor_floats = pc.tc * G::W;
    Ring *ring = reinterpret_cast<Ring *>(smem_raw + (size_t)pc.stages * tensor_floats * sizeof(float));
    ring_init(ring, pc.stages, NW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + pc.tc - 1) / pc.tc;

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[1] = {&maps.m[0]};
            produce<NW, V>(ring, stages, mp, 1, nchunks, m0, b, pc, false);
        }
    } else {
        const int c = threadIdx.x * V;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        const SpikeCfg cfg = make_spike_cfg(A.maxs);
        constexpr int NQ = UNI ? 1 : V;
        Neuron q[NQ];
        float as[NQ], ss[NQ];
        float v[V], af[V], isyn[V];
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
            q[j] = A.np.load(b, mm + j, cfg);
            as[j] = A.alpha_syn.get(b, mm + j, 1.0f);
            ss[j] = A.scale_syn.get(b, mm + j, 1.0f);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
            isyn[j] = A.i_init ? __ldg(A.i_init + n + j) : 0.0f;
            af[j] = 0.0f;
        }
        const int64_t base = ((int64_t)b * T) * A.M + mm;
        float *sp = A.spikes + base;
        float *vm = A.v_mem + base;
        float *is = A.i_syn + base;
        const int64_t M = A.M;
        const int col = tile_col_off<NW, V>(pc.tc, c);
        SpikeTotal cnt;
        cnt.c32 = 0u; cnt.c64 = 0ull;
        bool ok = true;
        RingPos pos = {0, 0u};
        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *st = stages + (size_t)pos.s * tensor_floats + col;
            const int tmax = min(pc.tc, T - k * pc.tc);
#pragma unroll 2
            for (int tt = 0; tt < tmax; ++tt) {
                float xs[V];
                lds_vec<V>(xs, st + tt * G::BW);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const int jq = (NQ == 1) ? 0 : j;
                    isyn[j] = __fmaf_rn(isyn[j], as[jq], __fmul_rn(ss[jq], xs[j]));
                }
                lif_step_vec<RESET, V, NQ>(v, af, isyn, q, cfg, cnt);
                if (valid) {
                    stv<V>(is, isyn);
                    stv<V>(sp, af);
                    stv<V>(vm, v);
                }
                is += M;
                sp += M;
                vm += M;
            }
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        if (ok && valid) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                if (A.v_post_last) A.v_post_last[n + j] = post_reset<RESET>(v[j], af[j], q[NQ == 1 ? 0 : j]);
                if (A.i_last) A.i_last[n + j] = isyn[j];
            }
        }
        if (A.spike_count) {
            const unsigned long long tot = warp_sum_u64((valid && ok) ? cnt.total(cfg) : 0ull);
            if (lane == 0 && tot) atomicAdd(A.spike_count, tot);
        }
    }
    ring_finish(ring, pc.stages);
}

// WG: parameter gradients wanted (streams i_syn as well).
// The narrow tile with all four parameter gradients keeps about twenty values live per thread: at the
// 48 registers of 8 CTAs per SM the compiler recomputes loop invariants in every step; 7 CTAs give 56.
template <int SURR, int RESET, bool WG, int NW, int V, bool UNI>
__global__ void __launch_bounds__((NW + 1) * 32, (V == 1 && WG) ? 7 : MinBlocks<NW, V, (V == 4)>::value)
lif_syn_bwd_tma_kernel(const __grid_constant__ TmaMaps6 maps, const LifSynBwdArgs A, const int tiles_m, const int nmaps,
                       const PipeCfg pc)
{
    using G = TileGeom<NW, V>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    const int tensor_floats = pc.tc * G::W;
    const int stage_floats = nmaps * tensor_floats;
    Ring *ring = reinterpret_cast<Ring *>(smem_raw + (size_t)pc.stages * stage_floats * sizeof(float));
    ring_init(ring, pc.stages, NW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + pc.tc - 1) / pc.tc;
    // stage layout: [grad_spikes][v_mem]([grad_v_mem])([surr])([i_syn])([grad_i_syn])
    const bool has_gv = A.gv != nullptr, has_gis = A.g_isyn != nullptr;
    const int i_sl = 2 + (has_gv ? 1 : 0);
    const int i_is = i_sl + ((SURR == EXB_SURR_GENERIC) ? 1 : 0);
    const int i_gis = i_is + (WG ? 1 : 0);
    constexpr int WS = WG ? SCALE_GRAD_FROM_INPUT : SCALE_GRAD_NONE;

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[6] = {&maps.m[0], &maps.m[1], &maps.m[2], &maps.m[3], &maps.m[4], &maps.m[5]};
            produce<NW, V>(ring, stages, mp, nmaps, nchunks, m0, b, pc, true);
        }
    } else {
        const int c = threadIdx.x * V;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        const SpikeCfg cfg = make_spike_cfg(A.maxs);
        constexpr int NQ = UNI ? 1 : V;
        Neuron q[NQ];
        SurrConst sc[NQ];
        float cp[NQ], as[NQ], ss[NQ];
        float Rprev[V], f0[V], glast[V], gilast[V];
        bool n0[V];
        BwdState st[V];
        float Gs[V], ag_syn[V], sg_syn[V], inext[V];   // synaptic sweep: G_{t+1}, accumulators, i_{t+1}
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
            q[j] = A.np.load(b, mm + j, cfg);
            sc[j] = surr_prepare<SURR>(q[j], A.p0, A.p1);
            cp[j] = __fmul_rn(q[j].alpha, q[j].c);
            as[j] = A.alpha_syn.get(b, mm + j, 1.0f);
            ss[j] = A.scale_syn.get(b, mm + j, 1.0f);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            st[j].R = 0.0f; st[j].ag = 0.0f; st[j].sg = 0.0f; st[j].vnext = 0.0f;
            Rprev[j] = 0.0f; f0[j] = 0.0f; n0[j] = true;
            glast[j] = A.g_vlast ? __ldg(A.g_vlast + n + j) : 0.0f;
            gilast[j] = A.g_ilast ? __ldg(A.g_ilast + n + j) : 0.0f;
            Gs[j] = 0.0f; ag_syn[j] = 0.0f; sg_syn[j] = 0.0f; inext[j] = 0.0f;
        }
        const int64_t M = A.M;
        float *gi_base = A.grad_input + ((int64_t)b * T) * M + mm;
        const int col = tile_col_off<NW, V>(pc.tc, c);
        bool ok = true;
        RingPos pos = {0, 0u};
        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *stg = stages + (size_t)pos.s * stage_floats + col;
            const int chunk = nchunks - 1 - k;
            const int tmax = min(pc.tc, T - chunk * pc.tc);
            float *gi = gi_base + (int64_t)(chunk * pc.tc + tmax - 1) * M;
#pragma unroll 2
            for (int tt = tmax - 1; tt >= 0; --tt) {
                const float *e = stg + tt * G::BW;
                float go[V], vv[V];
                float gv[V] = {}, sl[V] = {}, is[V] = {}, gis[V] = {};
                lds_vec<V>(go, e);
                lds_vec<V>(vv, e + tensor_floats);
                if (has_gv) lds_vec<V>(gv, e + 2 * tensor_floats);
                if (SURR == EXB_SURR_GENERIC) lds_vec<V>(sl, e + i_sl * tensor_floats);
                if (WG) lds_vec<V>(is, e + i_is * tensor_floats);
                if (has_gis) lds_vec<V>(gis, e + i_gis * tensor_floats);
                const bool last = (chunk * pc.tc + tt == T - 1);
                float r[V];
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    const int jq = (NQ == 1) ? 0 : j;
                    if (last) {
                        if (A.g_vlast) fold_last_state_grad<RESET>(go[j], gv[j], glast[j], vv[j], q[jq], cfg);
                        gis[j] = __fadd_rn(gis[j], gilast[j]);
                    }
                    Rprev[j] = st[j].R;
                    const float Rt = lif_bwd_step<SURR, RESET, WG, WS>(st[j], vv[j], go[j], gv[j], sl[j], is[j], q[jq],
                                                                      sc[jq], cp[jq], cfg, f0[j], n0[j]);
                    // synaptic stage: gradient arriving at i_t, then one reverse step
                    const float h = __fmaf_rn(q[jq].scale, Rt, gis[j]);
                    if (WG) {
                        ag_syn[j] = __fmaf_rn(Gs[j], is[j], ag_syn[j]);                               // G_{t+1} * i_t
                        sg_syn[j] = __fmaf_rn(Gs[j], __fmaf_rn(-as[jq], is[j], inext[j]), sg_syn[j]);  // G_{t+1} * scale*x_{t+1}
                        inext[j] = is[j];
                    }
                    Gs[j] = __fmaf_rn(Gs[j], as[jq], h);
                    r[j] = __fmul_rn(ss[jq], Gs[j]);
                }
                if (valid) stv<V>(gi, r);
                gi -= M;
            }
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        if (ok && valid) {
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const int jq = (NQ == 1) ? 0 : j;
                const float vi = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
                const float ii = A.i_init ? __ldg(A.i_init + n + j) : 0.0f;
                if (A.grad_v_init) A.grad_v_init[n + j] = __fmul_rn(q[jq].alpha, st[j].R);
                if (A.grad_i_init) A.grad_i_init[n + j] = __fmul_rn(as[jq], Gs[j]);
                if (WG) {
                    A.grad_alpha_mem[n + j] = alpha_grad_finish<RESET>(st[j], vi, Rprev[j], f0[j], n0[j]);
                    A.grad_scale_mem[n + j] = st[j].sg;
                    A.grad_alpha_syn[n + j] = __fmaf_rn(Gs[j], ii, ag_syn[j]);
                    A.grad_scale_syn[n + j] =
                        __fdiv_rn(__fmaf_rn(Gs[j], __fmaf_rn(-as[jq], ii, inext[j]), sg_syn[j]), ss[jq]);
                }
            }
        }
    }
    ring_finish(ring, pc.stages);
}

// ===========================================================================
// host side
// ===========================================================================
static bool syn_uniform(const NeuronParams &np, const Param &a, const Param &s)
{
    auto uni = [](const Param &q) { return !q.p || (q.sb == 0 && q.sm == 0); };
    return np.uniform() && uni(a) && uni(s);
}

template <int RESET, int NW, int V, bool UNI>
static cudaError_t run_syn_fwd(const LifSynFwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    const PipeCfg pc = pipe_cfg(G::W, 1, a.B * ((a.M + G::W - 1) / G::W));
    TmaMaps6 maps;
    if (!make_btm_tensor_map(&maps.m[0], a.input, a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = 1; i < 6; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, V>(1, pc);
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = lif_syn_fwd_tma_kernel<RESET, NW, V, UNI>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, pc);
    *used = true;
    return cudaPeekAtLastError();
}

template <int RESET>
static cudaError_t pick_syn_fwd(const LifSynFwdArgs &a, cudaStream_t s, bool *used)
{
    if (!use_wide(a.B, a.M)) return run_syn_fwd<RESET, NWARPS, 1, true>(a, s, used);
    return syn_uniform(a.np, a.alpha_syn, a.scale_syn) ? run_syn_fwd<RESET, NWARPS, 4, true>(a, s, used)
                                                       : run_syn_fwd<RESET, NWARPS, 4, false>(a, s, used);
}

cudaError_t launch_lif_syn_forward(const LifSynFwdArgs &a, int reset_mode, cudaStream_t s, bool *used)
{
    *used = false;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.spikes) || !aligned16(a.v_mem) || !aligned16(a.i_syn) ||
        !aligned16(a.input))
        return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? pick_syn_fwd<EXB_RESET_SUBTRACT>(a, s, used)
                                            : pick_syn_fwd<EXB_RESET_TO_VALUE>(a, s, used);
}

template <int SURR, int RESET, bool WG, int NW, int V, bool UNI>
static cudaError_t run_syn_bwd(const LifSynBwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    TmaMaps6 maps;
    const float *ptrs[6] = {a.go, a.v_mem, nullptr, nullptr, nullptr, nullptr};
    int nmaps = 2;
    if (a.gv) ptrs[nmaps++] = a.gv;
    if (SURR == EXB_SURR_GENERIC) ptrs[nmaps++] = a.surr;
    if (WG) ptrs[nmaps++] = a.i_syn;
    if (a.g_isyn) ptrs[nmaps++] = a.g_isyn;
    const PipeCfg pc = pipe_cfg(G::W, nmaps, a.B * ((a.M + G::W - 1) / G::W));
    for (int i = 0; i < nmaps; ++i)
        if (!make_btm_tensor_map(&maps.m[i], ptrs[i], a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = nmaps; i < 6; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, V>(nmaps, pc);
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = lif_syn_bwd_tma_kernel<SURR, RESET, WG, NW, V, UNI>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, nmaps, pc);
    *used = true;
    return cudaPeekAtLastError();
}

template <int SURR, int RESET, bool WG>
static cudaError_t pick_syn_bwd(const LifSynBwdArgs &a, cudaStream_t s, bool *used)
{
    if (!use_wide(a.B, a.M)) return run_syn_bwd<SURR, RESET, WG, NWARPS, 1, true>(a, s, used);
    return syn_uniform(a.np, a.alpha_syn, a.scale_syn) ? run_syn_bwd<SURR, RESET, WG, NWARPS, 4, true>(a, s, used)
                                                       : run_syn_bwd<SURR, RESET, WG, NWARPS, 4, false>(a, s, used);
}

template <int SURR, int RESET>
static cudaError_t flags_syn_bwd(const LifSynBwdArgs &a, cudaStream_t s, bool *used)
{
    return a.grad_alpha_mem ? pick_syn_bwd<SURR, RESET, true>(a, s, used) : pick_syn_bwd<SURR, RESET, false>(a, s, used);
}

template <int RESET>
static cudaError_t surr_syn_bwd(const LifSynBwdArgs &a, int kind, cudaStream_t s, bool *used)
{
    switch (kind) {
    case EXB_SURR_GENERIC: return flags_syn_bwd<EXB_SURR_GENERIC, RESET>(a, s, used);
    case EXB_SURR_SINGLE_EXPONENTIAL: return flags_syn_bwd<EXB_SURR_SINGLE_EXPONENTIAL, RESET>(a, s, used);
    case EXB_SURR_HEAVISIDE: return flags_syn_bwd<EXB_SURR_HEAVISIDE, RESET>(a, s, used);
    default: return flags_syn_bwd<EXB_SURR_PERIODIC_EXPONENTIAL, RESET>(a, s, used);
    }
}

cudaError_t launch_lif_syn_backward(const LifSynBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used)
{
    *used = false;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.grad_input)) return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? surr_syn_bwd<EXB_RESET_SUBTRACT>(a, surr_kind, s, used)
                                            : surr_syn_bwd<EXB_RESET_TO_VALUE>(a, surr_kind, s, used);
}

cudaError_t read_device_status_lif_syn(cudaStream_t s, unsigned int *out)
{
    static const unsigned int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_exb_status, sizeof(unsigned int), 0, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return e;
    if (*out) e = cudaMemcpyToSymbolAsync(g_exb_status, &zero, sizeof(unsigned int), 0, cudaMemcpyHostToDevice, s);
    return e;
}

}  // namespace exb
