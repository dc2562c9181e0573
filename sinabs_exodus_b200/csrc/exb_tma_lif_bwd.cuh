// TMA-staged fused reverse-time EXODUS backward (time-major layout): kernel and launch templates, instantiated
// by exb_tma_lif_bwd.cu (v_mem read from memory) and exb_tma_lif_bwd_rec.cu (v_mem rebuilt from checkpoints).
#pragma once

#include "exb_tma_common.cuh"

namespace exb {

// ===========================================================================
// fused reverse-time backward
// ===========================================================================
// REC: the second streamed tensor is the forward input, not v_mem; v_mem is rebuilt chunk by chunk from the state
// that entered the chunk (A.ckpt, written by the forward kernel every EXB_CKPT_EVERY steps, which is then also the
// chunk length) with the forward kernel's own step function, in place over the input tile -- bit for bit the tensor
// the forward pass would have written.  A step then moves 4 bytes per neuron less in the forward pass.
template <int SURR, int RESET, bool WA, int WS, int NW, int V, bool UNI, bool REC>
__global__ void __launch_bounds__((NW + 1) * 32, (REC && V == 4) ? 3 : MinBlocks<NW, V, (V == 4 && (!UNI || WA || WS != 0 || SURR == EXB_SURR_PERIODIC_EXPONENTIAL))>::value)
lif_bwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LifBwdArgs A, const int tiles_m, const int nmaps,
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
    // stage layout: [grad_spikes][v_mem]([grad_v_mem])([surr])([input])
    const bool has_gv = A.gv != nullptr;
    const int i_sl = 2 + (has_gv ? 1 : 0);
    const int i_x = i_sl + ((SURR == EXB_SURR_GENERIC) ? 1 : 0);

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[5] = {&maps.m[0], &maps.m[1], &maps.m[2], &maps.m[3], &maps.m[4]};
            produce<NW, V>(ring, stages, mp, nmaps, nchunks, m0, b, pc, true);
        }
    } else {
        const int c = threadIdx.x * V;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        const SpikeCfg cfg = make_spike_cfg(A.maxs);
        constexpr int NQ = UNI ? 1 : V;       // UNI: every parameter is a single value
        Neuron q[NQ];
        SurrConst sc[NQ];
        float cp[NQ], Rprev[V], f0[V], glast[V];
        bool n0[V];
        BwdState st[V];
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
            q[j] = A.np.load(b, mm + j, cfg);
            sc[j] = surr_prepare<SURR>(q[j], A.p0, A.p1);
            cp[j] = __fmul_rn(q[j].alpha, q[j].c);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            st[j].R = 0.0f; st[j].ag = 0.0f; st[j].sg = 0.0f; st[j].vnext = 0.0f;
            Rprev[j] = 0.0f; f0[j] = 0.0f; n0[j] = true;
            glast[j] = A.g_last ? __ldg(A.g_last + n + j) : 0.0f;
        }
        const int64_t M = A.M;
        float *gi_base = A.grad_input + ((int64_t)b * T) * M + mm;
        const int col = tile_col_off<NW, V>(pc.tc, c);
        bool ok = true;
        RingPos pos = {0, 0u};
        // REC: checkpoint of the chunk about to be processed, fetched one chunk ahead
        const float *ckp = REC ? A.ckpt + ((int64_t)b * nchunks) * M + mm : nullptr;
        float ck_next[V];
#pragma unroll
        for (int j = 0; j < V; ++j) ck_next[j] = 0.0f;
        if (REC && valid) ldg_vec<V>(ck_next, ckp + (int64_t)(nchunks - 1) * M);
        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            float *stg = stages + (size_t)pos.s * stage_floats + col;
            const int chunk = nchunks - 1 - k;
            const int tmax = min(pc.tc, T - chunk * pc.tc);
            float *gi = gi_base + (int64_t)(chunk * pc.tc + tmax - 1) * M;
            if (REC) {
                float vr[V], afr[V];
#pragma unroll
                for (int j = 0; j < V; ++j) { vr[j] = ck_next[j]; afr[j] = 0.0f; }
                if (chunk > 0 && valid) ldg_vec<V>(ck_next, ckp + (int64_t)(chunk - 1) * M);
                SpikeTotal unused;
                unused.c32 = 0u; unused.c64 = 0ull;
                float *xt = stg + tensor_floats;
#pragma unroll 2
                for (int tt = 0; tt < tmax; ++tt) {
                    float xs[V];
                    lds_vec<V>(xs, xt + tt * G::BW);
                    lif_step_vec<RESET, V, NQ>(vr, afr, xs, q, cfg, unused);
                    sts_vec<V>(xt + tt * G::BW, vr);
                }
            }
#pragma unroll 2
            for (int tt = tmax - 1; tt >= 0; --tt) {
                const float *e = stg + tt * G::BW;
                float go[V], vv[V];
                float gv[V] = {}, sl[V] = {}, xx[V] = {};
                lds_vec<V>(go, e);
                lds_vec<V>(vv, e + tensor_floats);
                if (has_gv) lds_vec<V>(gv, e + 2 * tensor_floats);
                if (SURR == EXB_SURR_GENERIC) lds_vec<V>(sl, e + i_sl * tensor_floats);
                if (WS == SCALE_GRAD_FROM_INPUT) lds_vec<V>(xx, e + i_x * tensor_floats);
                if (A.g_last && chunk * pc.tc + tt == T - 1) {
#pragma unroll
                    for (int j = 0; j < V; ++j) fold_last_state_grad<RESET>(go[j], gv[j], glast[j], vv[j], q[NQ == 1 ? 0 : j], cfg);
                }
                float r[V];
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    Rprev[j] = st[j].R;
                    constexpr int NQ1 = (NQ == 1);
                    const int jq = NQ1 ? 0 : j;
                    const float Rt = lif_bwd_step<SURR, RESET, WA, WS>(st[j], vv[j], go[j], gv[j], sl[j], xx[j], q[jq], sc[jq],
                                                                      cp[jq], cfg, f0[j], n0[j]);
                    r[j] = __fmul_rn(q[jq].scale, Rt);
                }
                if (valid) stv<V>(gi, r);
                gi -= M;
            }
            if (REC) fence_proxy_async_smem();      // the tile was written by threads and will be refilled by TMA
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        float gdecay[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const Neuron &qj = q[NQ == 1 ? 0 : j];
            gdecay[j] = 0.0f;
            if (valid) {
                if (!ok) { st[j].R = NAN; st[j].ag = NAN; st[j].sg = NAN; }      // a wait ran out: poison the results
                if (A.grad_init) A.grad_init[n + j] = __fmul_rn(qj.alpha, st[j].R);
                const float vi = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
                const float ga = WA ? alpha_grad_finish<RESET>(st[j], vi, Rprev[j], f0[j], n0[j]) : 0.0f;
                const float gs = WS ? scale_grad_finish<WS>(st[j], vi, qj) : 0.0f;
                if (A.acc_decay) {
                    gdecay[j] = decay_param_grad(ga, gs, A.np.alpha, A.np.scale, qj.alpha, b, mm + j);
                } else {
                    if (WA) A.grad_alpha[n + j] = ga;
                    if (WS) A.grad_scale[n + j] = gs;
                }
            }
        }
        if (A.acc_decay) acc_param_grad<V>(A.acc_decay, A.np.alpha, gdecay, valid, b, mm, lane);
    }
    ring_finish(ring, pc.stages);
}

template <int SURR, int RESET, bool WA, int WS, int NW, int V, bool UNI, bool REC>
static cudaError_t run_lif_bwd(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    TmaMaps maps;
    const float *ptrs[5] = {a.go, REC ? a.input : a.v_mem, nullptr, nullptr, nullptr};
    int nmaps = 2;
    if (!REC) {
        if (a.gv) ptrs[nmaps++] = a.gv;
        if (SURR == EXB_SURR_GENERIC) ptrs[nmaps++] = a.surr;
        if (WS == SCALE_GRAD_FROM_INPUT) ptrs[nmaps++] = a.input;
    }
    PipeCfg pc = pipe_cfg(G::W, nmaps, a.B * ((a.M + G::W - 1) / G::W));
    if (REC) {      // a chunk starts where a checkpoint was taken; wide tiles: 2 stages of 32 KB, three CTAs per SM
        static const int env_st = env_int("EXB_REC_STAGES", 0);
        pc.tc = EXB_CKPT_EVERY;
        pc.stages = (V == 4) ? 2 : 4;
        if (env_st >= 2 && env_st <= MAX_STAGES) pc.stages = env_st;
    }
    for (int i = 0; i < nmaps; ++i)
        if (!make_btm_tensor_map(&maps.m[i], ptrs[i], a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = nmaps; i < 5; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, V>(nmaps, pc);
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = lif_bwd_tma_kernel<SURR, RESET, WA, WS, NW, V, UNI, REC>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, nmaps, pc);
    *used = true;
    return cudaPeekAtLastError();
}

template <int SURR, int RESET, bool WA, int WS, bool REC>
static cudaError_t pick_lif_bwd(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    if (!use_wide(a.B, a.M)) return run_lif_bwd<SURR, RESET, WA, WS, NWARPS, 1, true, REC>(a, s, used);
    return a.np.uniform() ? run_lif_bwd<SURR, RESET, WA, WS, NWARPS, 4, true, REC>(a, s, used)
                          : run_lif_bwd<SURR, RESET, WA, WS, NWARPS, 4, false, REC>(a, s, used);
}

template <int SURR, int RESET, bool REC>
static cudaError_t flags_lif_bwd(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    // With an accumulator the alpha gradient is always wanted, and the scale gradient when the scale derives from alpha.
    const bool derived = (a.np.scale.flags & (EXB_SCALE_ONE_MINUS_ALPHA | EXB_SCALE_TIMES_ALPHA)) != 0;
    const bool wa = a.grad_alpha != nullptr || a.acc_decay != nullptr;
    const bool want_scale = a.grad_scale != nullptr || (a.acc_decay != nullptr && derived);
    // with checkpoints the input tile becomes v_mem: the scale gradient is then always rebuilt from the state
    const int ws = want_scale ? ((a.input && !REC) ? SCALE_GRAD_FROM_INPUT : SCALE_GRAD_FROM_STATE) : SCALE_GRAD_NONE;
    if (wa) {
        if (!REC && ws == SCALE_GRAD_FROM_INPUT) return pick_lif_bwd<SURR, RESET, true, SCALE_GRAD_FROM_INPUT, REC>(a, s, used);
        if (ws == SCALE_GRAD_FROM_STATE) return pick_lif_bwd<SURR, RESET, true, SCALE_GRAD_FROM_STATE, REC>(a, s, used);
        return pick_lif_bwd<SURR, RESET, true, SCALE_GRAD_NONE, REC>(a, s, used);
    }
    if (!REC && ws == SCALE_GRAD_FROM_INPUT) return pick_lif_bwd<SURR, RESET, false, SCALE_GRAD_FROM_INPUT, REC>(a, s, used);
    if (ws == SCALE_GRAD_FROM_STATE) return pick_lif_bwd<SURR, RESET, false, SCALE_GRAD_FROM_STATE, REC>(a, s, used);
    return pick_lif_bwd<SURR, RESET, false, SCALE_GRAD_NONE, REC>(a, s, used);
}

template <int RESET, bool REC>
static cudaError_t surr_lif_bwd(const LifBwdArgs &a, int kind, cudaStream_t s, bool *used)
{
    switch (kind) {
    case EXB_SURR_GENERIC:      // needs the caller's surrogate of v_mem, which the checkpointed pass never materialises
        if constexpr (REC) return cudaSuccess;
        else return flags_lif_bwd<EXB_SURR_GENERIC, RESET, false>(a, s, used);
    case EXB_SURR_SINGLE_EXPONENTIAL: return flags_lif_bwd<EXB_SURR_SINGLE_EXPONENTIAL, RESET, REC>(a, s, used);
    case EXB_SURR_HEAVISIDE: return flags_lif_bwd<EXB_SURR_HEAVISIDE, RESET, REC>(a, s, used);
    default: return flags_lif_bwd<EXB_SURR_PERIODIC_EXPONENTIAL, RESET, REC>(a, s, used);
    }
}

}  // namespace exb
