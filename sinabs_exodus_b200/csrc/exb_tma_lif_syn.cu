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
//
// Both kernels are bound by instruction issue before they are bound by memory (one thread per
// neuron on small layers), so the time loop is written to issue as little as possible around the
// arithmetic: the time steps per pipeline stage TC and the order of the streamed tensors are
// template parameters, which makes every shared-memory address of a full chunk an immediate
// offset from one per-chunk pointer and unrolls the chunk completely; the step that takes the
// gradients of the final states (t = T-1) is peeled off in front of the sweep; what only the
// first step's epilogue needs (R_1, its factor and clip gate) is captured once per chunk, not
// once per step.  Gradients arriving on v_mem or i_syn (EXTRA) are rare and take a variant with
// a run-time stage layout.
#include "exb_tma_common.cuh"

#include <type_traits>

namespace exb {

struct TmaMaps6 {
    CUtensorMap m[6];
};

// Launch geometry known at compile time: tile, time steps per stage.
template <int NW, int V, int TC>
struct SynGeom {
    using G = TileGeom<NW, V>;
    static constexpr int TF = TC * G::W;      // floats of one tensor in one stage
};

// ST: element type of the spike raster (float, or uint8_t for the compact raster); WS: write v_mem and i_syn
// (a forward pass that nobody differentiates or records needs only the spikes).
template <int RESET, int NW, int V, bool UNI, int TC, typename ST, bool WS>
__global__ void __launch_bounds__((NW + 1) * 32, MinBlocks<NW, V, (V == 4)>::value)
lif_syn_fwd_tma_kernel(const __grid_constant__ TmaMaps6 maps, const LifSynFwdArgs A, const int tiles_m, const int nstages)
{
    using G = TileGeom<NW, V>;
    constexpr int TF = SynGeom<NW, V, TC>::TF;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    Ring *ring = reinterpret_cast<Ring *>(smem_raw + (size_t)nstages * TF * sizeof(float));
    ring_init(ring, nstages, NW);
    const PipeCfg pc = {TC, nstages};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + TC - 1) / TC;

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
            as[j] = decay_of(A.alpha_syn, b, mm + j);
            ss[j] = scale_of(A.scale_syn, as[j], b, mm + j);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
            isyn[j] = A.i_init ? __ldg(A.i_init + n + j) : 0.0f;
            af[j] = 0.0f;
        }
        // Element offsets inside one batch item fit 32 bits (the launcher checks T*M < 2^31): one 32-bit offset
        // per step serves all three outputs, each address one widening multiply-add from its base.
        const int64_t base = ((int64_t)b * T) * A.M + mm;
        float *const is_b = WS ? A.i_syn + base : nullptr;
        ST *const sp_b = (std::is_same<ST, float>::value ? reinterpret_cast<ST *>(A.spikes) : reinterpret_cast<ST *>(A.spikes_u8)) + base;
        float *const vm_b = WS ? A.v_mem + base : nullptr;
        const int Mi = (int)A.M;
        const int col = tile_col_off<NW, V>(TC, c);
        SpikeTotal cnt;
        cnt.c32 = 0u; cnt.c64 = 0ull;
        bool ok = true;
        RingPos pos = {0, 0u};

        auto step = [&](const float *e, const int o) {
            float xs[V];
            lds_vec<V>(xs, e);
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const int jq = (NQ == 1) ? 0 : j;
                isyn[j] = __fmaf_rn(isyn[j], as[jq], __fmul_rn(ss[jq], xs[j]));
            }
            lif_step_vec<RESET, V, NQ>(v, af, isyn, q, cfg, cnt);
            if (valid) {
                if (WS) stv<V>(is_b + o, isyn);
                st_spikes<V>(sp_b + o, af);
                if (WS) stv<V>(vm_b + o, v);
            }
        };

        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *st = stages + (size_t)pos.s * TF + col;
            const int o0 = k * TC * Mi;
            if (k + 1 < nchunks || T == nchunks * TC) {      // a full chunk: every shared-memory address an immediate
#pragma unroll
                for (int tt = 0; tt < TC; ++tt) step(st + tt * G::BW, o0 + tt * Mi);
            } else {
                const int tmax = T - k * TC;
                for (int tt = 0; tt < tmax; ++tt) step(st + tt * G::BW, o0 + tt * Mi);
            }
            release_chunk(ring, pos, lane);
            pos.advance(nstages);
        }
        if (valid) {      // NaN when a wait ran out: the failure must not pass for a state
#pragma unroll
            for (int j = 0; j < V; ++j) {
                if (A.v_post_last) A.v_post_last[n + j] = ok ? post_reset<RESET>(v[j], af[j], q[NQ == 1 ? 0 : j]) : NAN;
                if (A.i_last) A.i_last[n + j] = ok ? isyn[j] : NAN;
            }
        }
        if (A.spike_count) {
            const unsigned long long tot = warp_sum_u64((valid && ok) ? cnt.total(cfg) : 0ull);
            if (lane == 0 && tot) atomicAdd(A.spike_count, tot);
        }
    }
    ring_finish(ring, nstages);
}

// Where each streamed tensor sits inside a stage, in units of one tensor's floats.  Order:
// [grad_spikes][v_mem]([grad_v_mem])([surr])([i_syn])([grad_i_syn]).  Without EXTRA the optional gradient
// inputs are absent and the positions are compile-time constants.
template <int SURR, bool WG, bool EXTRA>
struct SynSlots {
    int gv, sl, is, gis;      // used only with EXTRA
    __device__ __forceinline__ int slot_sl() const { return EXTRA ? sl : 2; }
    __device__ __forceinline__ int slot_is() const { return EXTRA ? is : (2 + (SURR == EXB_SURR_GENERIC ? 1 : 0)); }
};

// Running state of one thread's V neurons in the reverse sweep.
template <int V>
struct SynBwdState {
    BwdState st[V];
    float Gs[V], ag_syn[V], sg_syn[V], inext[V];      // synaptic sweep: G_{t+1}, accumulators, i_{t+1}
};

// WG: parameter gradients wanted (streams i_syn as well).
// The narrow tile with all four parameter gradients keeps about twenty values live per thread: at the
// 48 registers of 8 CTAs per SM the compiler recomputes loop invariants in every step; 7 CTAs give 56.
// The wide tile with per-neuron parameters and parameter gradients keeps four neurons' constants and
// accumulators: 3 CTAs per SM (128 registers) instead of spilling at 96.
template <int V, bool WG, bool UNI>
struct SynBwdBlocks {
    static constexpr int value = (V == 1) ? (WG ? 7 : 8) : ((WG && !UNI) ? 3 : 4);
};

template <int SURR, int RESET, bool WG, bool EXTRA, int NW, int V, bool UNI, int TC>
__global__ void __launch_bounds__((NW + 1) * 32, SynBwdBlocks<V, WG, UNI>::value)
lif_syn_bwd_tma_kernel(const __grid_constant__ TmaMaps6 maps, const LifSynBwdArgs A, const int tiles_m, const int nmaps,
                       const int nstages)
{
    using G = TileGeom<NW, V>;
    constexpr int TF = SynGeom<NW, V, TC>::TF;
    constexpr int NMAPS_FIXED = 2 + (SURR == EXB_SURR_GENERIC ? 1 : 0) + (WG ? 1 : 0);
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    const int stage_floats = (EXTRA ? nmaps : NMAPS_FIXED) * TF;
    Ring *ring = reinterpret_cast<Ring *>(smem_raw + (size_t)nstages * stage_floats * sizeof(float));
    ring_init(ring, nstages, NW);
    const PipeCfg pc = {TC, nstages};

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + TC - 1) / TC;
    constexpr int WS = WG ? SCALE_GRAD_FROM_INPUT : SCALE_GRAD_NONE;

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[6] = {&maps.m[0], &maps.m[1], &maps.m[2], &maps.m[3], &maps.m[4], &maps.m[5]};
            produce<NW, V>(ring, stages, mp, EXTRA ? nmaps : NMAPS_FIXED, nchunks, m0, b, pc, true);
        }
    } else {
        const bool has_gv = EXTRA && A.gv != nullptr, has_gis = EXTRA && A.g_isyn != nullptr;
        SynSlots<SURR, WG, EXTRA> slots;
        slots.gv = 2;
        slots.sl = 2 + (has_gv ? 1 : 0);
        slots.is = slots.sl + ((SURR == EXB_SURR_GENERIC) ? 1 : 0);
        slots.gis = slots.is + (WG ? 1 : 0);

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
        SynBwdState<V> S;
        float R1[V], f0[V];
        bool n0[V];
#pragma unroll
        for (int j = 0; j < NQ; ++j) {
            q[j] = A.np.load(b, mm + j, cfg);
            sc[j] = surr_prepare<SURR>(q[j], A.p0, A.p1);
            cp[j] = __fmul_rn(q[j].alpha, q[j].c);
            as[j] = decay_of(A.alpha_syn, b, mm + j);
            ss[j] = scale_of(A.scale_syn, as[j], b, mm + j);
        }
#pragma unroll
        for (int j = 0; j < V; ++j) {
            S.st[j].R = 0.0f; S.st[j].ag = 0.0f; S.st[j].sg = 0.0f; S.st[j].vnext = 0.0f;
            R1[j] = 0.0f; f0[j] = 0.0f; n0[j] = true;
            S.Gs[j] = 0.0f; S.ag_syn[j] = 0.0f; S.sg_syn[j] = 0.0f; S.inext[j] = 0.0f;
        }
        const int Mi = (int)A.M;      // element offsets inside one batch item fit 32 bits (checked by the launcher)
        float *const gi_base = A.grad_input + ((int64_t)b * T) * A.M + mm;
        const int col = tile_col_off<NW, V>(TC, c);
        bool ok = true;
        RingPos pos = {0, 0u};

        // One reverse step on the operands at `e` (this thread's column, one time step of a stage); the input
        // gradient goes to `gi`.  LAST: the step at t = T-1, which also takes the gradients of the final states.
        // `fo`/`no` receive the step's propagation factor and clip gate.
        auto step = [&](const float *e, float *gi, auto last_tag, float (&fo)[V], bool (&no)[V]) {
            constexpr bool LAST = decltype(last_tag)::value;
            float go[V], vv[V];
            float gv[V] = {}, sl[V] = {}, is[V] = {}, gis[V] = {};
            lds_vec<V>(go, e);
            lds_vec<V>(vv, e + TF);
            if (has_gv) lds_vec<V>(gv, e + slots.gv * TF);
            if (SURR == EXB_SURR_GENERIC) lds_vec<V>(sl, e + slots.slot_sl() * TF);
            if (WG) lds_vec<V>(is, e + slots.slot_is() * TF);
            if (has_gis) lds_vec<V>(gis, e + slots.gis * TF);
            float r[V];
#pragma unroll
            for (int j = 0; j < V; ++j) {
                const int jq = (NQ == 1) ? 0 : j;
                if (LAST) {
                    if (A.g_vlast) fold_last_state_grad<RESET>(go[j], gv[j], __ldg(A.g_vlast + n + j), vv[j], q[jq], cfg);
                    if (A.g_ilast) gis[j] = __fadd_rn(gis[j], __ldg(A.g_ilast + n + j));
                }
                const float Rt = lif_bwd_step<SURR, RESET, WG, WS>(S.st[j], vv[j], go[j], gv[j], sl[j], is[j], q[jq],
                                                                  sc[jq], cp[jq], cfg, fo[j], no[j]);
                // synaptic stage: gradient arriving at i_t, then one reverse step
                const float h = (EXTRA || LAST) ? __fmaf_rn(q[jq].scale, Rt, gis[j]) : __fmul_rn(q[jq].scale, Rt);
                if (WG) {
                    S.ag_syn[j] = __fmaf_rn(S.Gs[j], is[j], S.ag_syn[j]);                               // G_{t+1} * i_t
                    S.sg_syn[j] = __fmaf_rn(S.Gs[j], __fmaf_rn(-as[jq], is[j], S.inext[j]), S.sg_syn[j]);  // G_{t+1} * scale*x_{t+1}
                    S.inext[j] = is[j];
                }
                S.Gs[j] = __fmaf_rn(S.Gs[j], as[jq], h);
                r[j] = __fmul_rn(ss[jq], S.Gs[j]);
            }
            if (valid) stv<V>(gi, r);
        };
        using TagLast = std::true_type;
        using TagMid = std::false_type;
        float fdump[V];
        bool ndump[V];

        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *stg = stages + (size_t)pos.s * stage_floats + col;
            const int chunk = nchunks - 1 - k;
            float *const gi0 = gi_base + chunk * TC * Mi;      // time step 0 of the chunk
            if (k > 0) {
                // every chunk but the one at the end of time is full: addresses are immediates, no loop
#pragma unroll
                for (int tt = TC - 1; tt >= 1; --tt) step(stg + tt * G::BW, gi0 + tt * Mi, TagMid{}, fdump, ndump);
            } else {
                const int tmax = T - chunk * TC;
                if (tmax > 1) {
                    step(stg + (tmax - 1) * G::BW, gi0 + (tmax - 1) * Mi, TagLast{}, fdump, ndump);
                    for (int tt = tmax - 2; tt >= 1; --tt) step(stg + tt * G::BW, gi0 + tt * Mi, TagMid{}, fdump, ndump);
                }
            }
            // time step 0 of the chunk; for the chunk at t = 0 this is the step whose factor, gate and
            // predecessor the alpha gradient's epilogue needs, so they are kept from here
#pragma unroll
            for (int j = 0; j < V; ++j) R1[j] = S.st[j].R;
            if (k == 0 && T - chunk * TC == 1) step(stg, gi0, TagLast{}, f0, n0);
            else step(stg, gi0, TagMid{}, f0, n0);
            release_chunk(ring, pos, lane);
            pos.advance(nstages);
        }
        float gd_mem[V], gd_syn[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            const int jq = (NQ == 1) ? 0 : j;
            gd_mem[j] = 0.0f; gd_syn[j] = 0.0f;
            if (valid) {
                const float vi = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
                const float ii = A.i_init ? __ldg(A.i_init + n + j) : 0.0f;
                if (!ok) {      // a wait ran out: poison the per-neuron results
                    S.st[j].R = NAN; S.st[j].ag = NAN; S.st[j].sg = NAN; S.Gs[j] = NAN; S.ag_syn[j] = NAN; S.sg_syn[j] = NAN;
                }
                if (A.grad_v_init) A.grad_v_init[n + j] = __fmul_rn(q[jq].alpha, S.st[j].R);
                if (A.grad_i_init) A.grad_i_init[n + j] = __fmul_rn(as[jq], S.Gs[j]);
                if (WG) {
                    const float ga_mem = alpha_grad_finish<RESET>(S.st[j], vi, R1[j], f0[j], n0[j]);
                    const float gs_mem = S.st[j].sg;
                    const float ga_syn = __fmaf_rn(S.Gs[j], ii, S.ag_syn[j]);
                    const float gs_syn = __fdiv_rn(__fmaf_rn(S.Gs[j], __fmaf_rn(-as[jq], ii, S.inext[j]), S.sg_syn[j]), ss[jq]);
                    if (A.acc_decay_mem) {
                        gd_mem[j] = decay_param_grad(ga_mem, gs_mem, A.np.alpha, A.np.scale, q[jq].alpha, b, mm + j);
                        gd_syn[j] = decay_param_grad(ga_syn, gs_syn, A.alpha_syn, A.scale_syn, as[jq], b, mm + j);
                    } else {
                        A.grad_alpha_mem[n + j] = ga_mem;
                        A.grad_scale_mem[n + j] = gs_mem;
                        A.grad_alpha_syn[n + j] = ga_syn;
                        A.grad_scale_syn[n + j] = gs_syn;
                    }
                }
            }
        }
        if (WG && A.acc_decay_mem) {
            acc_param_grad<V>(A.acc_decay_mem, A.np.alpha, gd_mem, valid, b, mm, lane);
            acc_param_grad<V>(A.acc_decay_syn, A.alpha_syn, gd_syn, valid, b, mm, lane);
        }
    }
    ring_finish(ring, nstages);
}

// ===========================================================================
// host side
// ===========================================================================
static bool syn_uniform(const NeuronParams &np, const Param &a, const Param &s)
{
    auto uni = [](const Param &q) { return !q.p || (q.sb == 0 && q.sm == 0); };
    return np.uniform() && uni(a) && uni(s);
}

// Stages that fit: as many as the shared memory left to one CTA allows (all CTAs of a small grid should be
// resident at once, see pipe_cfg), at least 2, at most 6.
static int syn_stages(size_t stage_bytes, int64_t ctas)
{
    static const int env_st = env_int("EXB_TMA_STAGES", 0);
    int64_t budget = 64 * 1024;
    const int64_t per_sm = (ctas + sm_count() - 1) / sm_count();
    if (per_sm >= 1 && per_sm <= 8) budget = (224 * 1024) / per_sm - 1280;
    if (budget > 96 * 1024) budget = 96 * 1024;
    int s = (int)(budget / (int64_t)stage_bytes);
    if (s > 6) s = 6;
    if (env_st > 1 && env_st <= MAX_STAGES) s = env_st;
    return s;
}

// Time steps per stage: the larger of the two compiled values whose ring still has `min_stages` stages.  The forward
// streams one tensor and likes a deep ring; the backward streams two to five and does more per chunk, and measured
// faster with twice the steps per stage on two stages than with half of them on five (synaptic layer, 128 x 500 x
// 1024: 200 us against 235 us), because the work per chunk (barrier wait, release, pointer set-up) halves.
// EXB_SYN_FWD_TC / EXB_SYN_BWD_TC (else EXB_TMA_TC) in the environment force one of them, EXB_SYN_FWD_STAGES the
// forward's stage count (tuning aids).
template <int TC_BIG, int TC_SMALL>
static int syn_pick_tc(int w, int nmaps, int64_t ctas, bool backward)
{
    const int min_stages = backward ? 2 : 4;
    static const int env_any = env_int("EXB_TMA_TC", 0);
    static const int env_fwd = env_int("EXB_SYN_FWD_TC", 0);
    static const int env_bwd = env_int("EXB_SYN_BWD_TC", 0);
    const int env_dir = backward ? env_bwd : env_fwd;
    const int env_tc = env_dir ? env_dir : env_any;
    if (env_tc == TC_BIG || env_tc == TC_SMALL) return env_tc;
    const size_t big = (size_t)TC_BIG * w * 4 * nmaps;
    if (big <= 16 * 1024 && syn_stages(big, ctas) >= min_stages) return TC_BIG;
    return TC_SMALL;
}

template <int RESET, int NW, int V, bool UNI, int TC>
static cudaError_t run_syn_fwd(const LifSynFwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t stage_bytes = (size_t)TC * G::W * 4;
    int nstages = syn_stages(stage_bytes, a.B * tiles_m);
    // With four or more CTAs resident per SM they are the parallelism; a deep ring on top only adds loads in flight
    // that compete with this kernel's stores (three tensors out for one in).  128 x 500 x 1024, whole step replayed
    // as a CUDA graph: 8 steps x 6 stages 0.3892 ms, 8 x 3 0.3827, 8 x 2 0.3782, 4 x 6 0.3880.
    if (a.B * tiles_m >= 4 * (int64_t)sm_count() && nstages > 2) nstages = 2;
    static const int env_fst = env_int("EXB_SYN_FWD_STAGES", 0);
    if (env_fst > 1 && env_fst <= MAX_STAGES) nstages = env_fst;
    if (nstages < 2) return cudaSuccess;
    TmaMaps6 maps;
    if (!make_btm_tensor_map(&maps.m[0], a.input, a.B, a.T, a.M, G::BW, TC)) return cudaSuccess;
    for (int i = 1; i < 6; ++i) maps.m[i] = maps.m[0];
    const PipeCfg pc = {TC, nstages};
    const size_t smem = tma_smem_bytes<NW, V>(1, pc);
    auto kern = a.spikes_u8 ? (a.v_mem ? lif_syn_fwd_tma_kernel<RESET, NW, V, UNI, TC, uint8_t, true>
                                       : lif_syn_fwd_tma_kernel<RESET, NW, V, UNI, TC, uint8_t, false>)
                : a.v_mem   ? lif_syn_fwd_tma_kernel<RESET, NW, V, UNI, TC, float, true>
                            : lif_syn_fwd_tma_kernel<RESET, NW, V, UNI, TC, float, false>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, nstages);
    *used = true;
    return cudaPeekAtLastError();
}

template <int RESET>
static cudaError_t pick_syn_fwd(const LifSynFwdArgs &a, cudaStream_t s, bool *used)
{
    if (!use_wide(a.B, a.M)) {
        const int tc = syn_pick_tc<16, 8>(128, 1, a.B * ((a.M + 127) / 128), false);
        return tc == 16 ? run_syn_fwd<RESET, NWARPS, 1, true, 16>(a, s, used) : run_syn_fwd<RESET, NWARPS, 1, true, 8>(a, s, used);
    }
    const int tc = syn_pick_tc<4, 2>(512, 1, a.B * ((a.M + 511) / 512), false);
    if (syn_uniform(a.np, a.alpha_syn, a.scale_syn))
        return tc == 4 ? run_syn_fwd<RESET, NWARPS, 4, true, 4>(a, s, used) : run_syn_fwd<RESET, NWARPS, 4, true, 2>(a, s, used);
    return tc == 4 ? run_syn_fwd<RESET, NWARPS, 4, false, 4>(a, s, used) : run_syn_fwd<RESET, NWARPS, 4, false, 2>(a, s, used);
}

cudaError_t launch_lif_syn_forward(const LifSynFwdArgs &a, int reset_mode, cudaStream_t s, bool *used)
{
    *used = false;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.input) || a.T * a.M >= (1ll << 31)) return cudaSuccess;
    // v_mem and i_syn are written together or not at all (a forward pass that is neither differentiated nor recorded)
    if ((a.v_mem != nullptr) != (a.i_syn != nullptr)) return cudaSuccess;
    if (a.v_mem && (!aligned16(a.v_mem) || !aligned16(a.i_syn))) return cudaSuccess;
    if (a.spikes_u8 ? !aligned16(a.spikes_u8) : !aligned16(a.spikes)) return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? pick_syn_fwd<EXB_RESET_SUBTRACT>(a, s, used)
                                            : pick_syn_fwd<EXB_RESET_TO_VALUE>(a, s, used);
}

template <int SURR, int RESET, bool WG, bool EXTRA, int NW, int V, bool UNI, int TC>
static cudaError_t run_syn_bwd(const LifSynBwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    TmaMaps6 maps;
    const float *ptrs[6] = {a.go, a.v_mem, nullptr, nullptr, nullptr, nullptr};
    int nmaps = 2;
    if (EXTRA && a.gv) ptrs[nmaps++] = a.gv;
    if (SURR == EXB_SURR_GENERIC) ptrs[nmaps++] = a.surr;
    if (WG) ptrs[nmaps++] = a.i_syn;
    if (EXTRA && a.g_isyn) ptrs[nmaps++] = a.g_isyn;
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t stage_bytes = (size_t)nmaps * TC * G::W * 4;
    const int nstages = syn_stages(stage_bytes, a.B * tiles_m);
    if (nstages < 2) return cudaSuccess;
    for (int i = 0; i < nmaps; ++i)
        if (!make_btm_tensor_map(&maps.m[i], ptrs[i], a.B, a.T, a.M, G::BW, TC)) return cudaSuccess;
    for (int i = nmaps; i < 6; ++i) maps.m[i] = maps.m[0];
    const PipeCfg pc = {TC, nstages};
    const size_t smem = tma_smem_bytes<NW, V>(nmaps, pc);
    auto kern = lif_syn_bwd_tma_kernel<SURR, RESET, WG, EXTRA, NW, V, UNI, TC>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, nmaps, nstages);
    *used = true;
    return cudaPeekAtLastError();
}

template <int SURR, int RESET, bool WG, bool EXTRA>
static cudaError_t pick_syn_bwd(const LifSynBwdArgs &a, cudaStream_t s, bool *used)
{
    const int nmaps = 2 + (SURR == EXB_SURR_GENERIC ? 1 : 0) + (WG ? 1 : 0) + (a.gv ? 1 : 0) + (a.g_isyn ? 1 : 0);
    if (!use_wide(a.B, a.M)) {
        const int tc = syn_pick_tc<8, 4>(128, nmaps, a.B * ((a.M + 127) / 128), true);
        return tc == 8 ? run_syn_bwd<SURR, RESET, WG, EXTRA, NWARPS, 1, true, 8>(a, s, used)
                       : run_syn_bwd<SURR, RESET, WG, EXTRA, NWARPS, 1, true, 4>(a, s, used);
    }
    const int tc = syn_pick_tc<4, 2>(512, nmaps, a.B * ((a.M + 511) / 512), true);
    if (syn_uniform(a.np, a.alpha_syn, a.scale_syn))
        return tc == 4 ? run_syn_bwd<SURR, RESET, WG, EXTRA, NWARPS, 4, true, 4>(a, s, used)
                       : run_syn_bwd<SURR, RESET, WG, EXTRA, NWARPS, 4, true, 2>(a, s, used);
    return tc == 4 ? run_syn_bwd<SURR, RESET, WG, EXTRA, NWARPS, 4, false, 4>(a, s, used)
                   : run_syn_bwd<SURR, RESET, WG, EXTRA, NWARPS, 4, false, 2>(a, s, used);
}

template <int SURR, int RESET>
static cudaError_t flags_syn_bwd(const LifSynBwdArgs &a, cudaStream_t s, bool *used)
{
    const bool extra = a.gv != nullptr || a.g_isyn != nullptr;
    if (a.grad_alpha_mem || a.acc_decay_mem)
        return extra ? pick_syn_bwd<SURR, RESET, true, true>(a, s, used) : pick_syn_bwd<SURR, RESET, true, false>(a, s, used);
    return extra ? pick_syn_bwd<SURR, RESET, false, true>(a, s, used) : pick_syn_bwd<SURR, RESET, false, false>(a, s, used);
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
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.grad_input) || a.T * a.M >= (1ll << 31)) return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? surr_syn_bwd<EXB_RESET_SUBTRACT>(a, surr_kind, s, used)
                                            : surr_syn_bwd<EXB_RESET_TO_VALUE>(a, surr_kind, s, used);
}

cudaError_t set_wait_limit_lif_syn(unsigned int polls) { return set_wait_limit_here(polls); }

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
