// TMA-staged time-major kernels: spike scan forward, leaky integrator forward and backward,
// the time-parallel leaky scan, and their launchers.  The fused LIF backward lives in
// exb_tma_lif_bwd.cu.  See exb_tma.cuh for the pipeline.
#include "exb_tma_common.cuh"

#include <mutex>
#include <type_traits>

namespace exb {

// ===========================================================================
// spike scan forward
// ===========================================================================
// REC: also write the potential after each step's reset (the layers' `record_states`).
// ST: element type of the spike raster (float, or uint8_t for the compact raster); WV: write v_mem (a forward
// pass that nobody differentiates or records needs only the spikes).
// CK: write the state that enters every EXB_CKPT_EVERY-th step (post-reset potential; the initial state at step 0)
// to A.ckpt, for a backward pass that rebuilds v_mem instead of reading it.
template <int RESET, int NW, int V, bool UNI, bool REC, typename ST, bool WV, bool CK = false>
__global__ void __launch_bounds__((NW + 1) * 32, MinBlocks<NW, V, (V == 4 && !UNI)>::value)
lif_fwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LifFwdArgs A, const int tiles_m, const PipeCfg pc)
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
        const int c = threadIdx.x * V;                 // column inside the tile
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;                    // M % 4 == 0 and V in {1, 4}: all V neurons or none
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        const SpikeCfg cfg = make_spike_cfg(A.maxs);
        constexpr int NQ = UNI ? 1 : V;       // UNI: every parameter is a single value
        Neuron q[NQ];
        float v[V], af[V];
#pragma unroll
        for (int j = 0; j < NQ; ++j) q[j] = A.np.load(b, mm + j, cfg);
#pragma unroll
        for (int j = 0; j < V; ++j) {
            v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
            af[j] = 0.0f;
        }
        const int64_t base = ((int64_t)b * T) * A.M + mm;
        ST *sp = (std::is_same<ST, float>::value ? reinterpret_cast<ST *>(A.spikes) : reinterpret_cast<ST *>(A.spikes_u8)) + base;
        float *vm = WV ? A.v_mem + base : nullptr;
        float *rec = REC ? A.v_post + base : nullptr;
        float *ck = CK ? A.ckpt + ((int64_t)b * ((T + EXB_CKPT_EVERY - 1) / EXB_CKPT_EVERY)) * A.M + mm : nullptr;
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
#pragma unroll 4
            for (int tt = 0; tt < tmax; ++tt) {
                float xs[V];
                lds_vec<V>(xs, st + tt * G::BW);
                if (CK && ((k * pc.tc + tt) & (EXB_CKPT_EVERY - 1)) == 0) {
                    if (valid) {
                        float vs[V];
#pragma unroll
                        for (int j = 0; j < V; ++j) vs[j] = post_reset<RESET>(v[j], af[j], q[NQ == 1 ? 0 : j]);
                        stv<V>(ck, vs);
                    }
                    ck += M;
                }
                lif_step_vec<RESET, V, NQ>(v, af, xs, q, cfg, cnt);
                if (valid) {
                    st_spikes<V>(sp, af);
                    if (WV) stv<V>(vm, v);
                    if (REC) {
                        float vp[V];
#pragma unroll
                        for (int j = 0; j < V; ++j) vp[j] = recorded_post<RESET>(v[j], af[j], q[NQ == 1 ? 0 : j]);
                        stv<V>(rec, vp);
                    }
                }
                sp += M;
                if (WV) vm += M;
                if (REC) rec += M;
            }
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        if (valid && A.v_post_last) {      // NaN when a wait ran out: the failure must not pass for a state
#pragma unroll
            for (int j = 0; j < V; ++j) A.v_post_last[n + j] = ok ? post_reset<RESET>(v[j], af[j], q[NQ == 1 ? 0 : j]) : NAN;
        }
        if (A.spike_count) {
            const unsigned long long tot = warp_sum_u64((valid && ok) ? cnt.total(cfg) : 0ull);
            if (lane == 0 && tot) atomicAdd(A.spike_count, tot);
        }
    }
    ring_finish(ring, pc.stages);
}

// ===========================================================================
// leaky integrator
// ===========================================================================
template <int NW, int V>
__global__ void __launch_bounds__((NW + 1) * 32, MinBlocks<NW, V>::value)
leaky_fwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LeakyFwdArgs A, const int tiles_m, const PipeCfg pc)
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
        float al[V], sc[V], v[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            al[j] = decay_of(A.alpha, b, mm + j);
            sc[j] = scale_of(A.scale, al[j], b, mm + j);
            v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
        }
        const int64_t M = A.M;
        float *out = A.out + ((int64_t)b * T) * M + mm;
        const int col = tile_col_off<NW, V>(pc.tc, c);
        bool ok = true;
        double total = 0.0;
        RingPos pos = {0, 0u};
        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *st = stages + (size_t)pos.s * tensor_floats + col;
            const int tmax = min(pc.tc, T - k * pc.tc);
            float part = 0.0f;
#pragma unroll 4
            for (int tt = 0; tt < tmax; ++tt) {
                float xs[V];
                lds_vec<V>(xs, st + tt * G::BW);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    v[j] = __fmaf_rn(v[j], al[j], __fmul_rn(sc[j], xs[j]));
                    part += v[j];
                }
                if (valid) stv<V>(out, v);
                out += M;
            }
            total += (double)part;
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        if (valid && A.v_last) {
#pragma unroll
            for (int j = 0; j < V; ++j) A.v_last[n + j] = ok ? v[j] : NAN;
        }
        if (A.out_sum) warp_add_f64(A.out_sum, valid ? (ok ? total : (double)NAN) : 0.0, lane);
    }
    ring_finish(ring, pc.stages);
}

template <bool WA, int WS, int NW, int V>
__global__ void __launch_bounds__((NW + 1) * 32, MinBlocks<NW, V, (WA && WS)>::value)
leaky_bwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LeakyBwdArgs A, const int tiles_m, const int nmaps,
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
    // stage layout: [grad_out]([out])([input])
    const int i_x = WA ? 2 : 1;

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
        float al[V], sc[V], G_[V], ag[V], sg[V], glast[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            al[j] = decay_of(A.alpha, b, mm + j);
            sc[j] = scale_of(A.scale, al[j], b, mm + j);
            G_[j] = 0.0f; ag[j] = 0.0f; sg[j] = 0.0f;
            glast[j] = A.g_last ? __ldg(A.g_last + n + j) : 0.0f;
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
#pragma unroll 4
            for (int tt = tmax - 1; tt >= 0; --tt) {
                const float *e = stg + tt * G::BW;
                float go[V];
                float vo[V] = {}, xx[V] = {};
                lds_vec<V>(go, e);
                if (WA) lds_vec<V>(vo, e + tensor_floats);
                if (WS) lds_vec<V>(xx, e + i_x * tensor_floats);
                const bool last = (chunk * pc.tc + tt == T - 1);
                float r[V];
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    if (last) go[j] = __fadd_rn(go[j], glast[j]);
                    if (WA) ag[j] = __fmaf_rn(G_[j], vo[j], ag[j]);
                    G_[j] = __fmaf_rn(G_[j], al[j], go[j]);
                    if (WS) sg[j] = __fmaf_rn(G_[j], xx[j], sg[j]);
                    r[j] = __fmul_rn(sc[j], G_[j]);
                }
                if (valid) stv<V>(gi, r);
                gi -= M;
            }
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        float gdecay[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            gdecay[j] = 0.0f;
            if (valid) {
                if (!ok) { G_[j] = NAN; ag[j] = NAN; sg[j] = NAN; }      // a wait ran out: poison the results
                if (A.grad_init) A.grad_init[n + j] = __fmul_rn(al[j], G_[j]);
                const float ga = WA ? __fmaf_rn(G_[j], A.v_init ? __ldg(A.v_init + n + j) : 0.0f, ag[j]) : 0.0f;
                if (A.acc_decay) {
                    gdecay[j] = decay_param_grad(ga, sg[j], A.alpha, A.scale, al[j], b, mm + j);
                } else {
                    if (WA) A.grad_alpha[n + j] = ga;
                    if (WS) A.grad_scale[n + j] = sg[j];
                }
            }
        }
        if (A.acc_decay) acc_param_grad<V>(A.acc_decay, A.alpha, gdecay, valid, b, mm, lane);
    }
    ring_finish(ring, pc.stages);
}

}  // namespace exb
#include "exb_leaky_scan.cuh"
#include "exb_lif_nt_tma.cuh"
namespace exb {

template <int RESET, int NW, int V, bool UNI>
static cudaError_t run_lif_fwd(const LifFwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    const int64_t ctas = a.B * ((a.M + G::W - 1) / G::W);
    PipeCfg pc = pipe_cfg(G::W, 1, ctas);
    // The pipeline shape follows what the variant writes per float it reads (wide tiles on many waves; measured on
    // 8 x 500 x 262144).  Two or three float tensors (spikes + v_mem [+ record]): long stages, one CTA per SM, see
    // long_stages_for_wide_forward.  About one float tensor (spikes alone; spikes + checkpoints; bytes + v_mem):
    // two CTAs per SM -- checkpoint variant 1.372 ms with 16 x 3, 1.374 with 16 x 2, 1.387 with 8 x 4, 1.498 with
    // 32 x 2, 1.567 with 16 x 4.  The byte raster alone (a quarter of a tensor out) is a read stream and keeps the
    // short default stages with many CTAs: 0.812 ms with 4 x 4, 0.832 with 16 x 2, 1.063 with 16 x 3, 1.806 with 32 x 2.
    const int float_tensors_out = a.spikes_u8 ? (a.v_mem ? 1 : 0) : (1 + (a.v_mem ? 1 : 0) + (a.v_post ? 1 : 0));
    if (float_tensors_out >= 1) {
        long_stages_for_wide_forward(pc, V, ctas, a.T);
        if (float_tensors_out == 1 && pc.tc == 32 && pc.stages == 2) { pc.tc = 16; pc.stages = 3; }
    }
    static const int env_tc = env_int("EXB_LIF_FWD_TC", 0), env_st = env_int("EXB_LIF_FWD_STAGES", 0);
    if (env_tc > 0 && env_tc <= 256) pc.tc = env_tc;
    if (env_st > 1 && env_st <= MAX_STAGES) pc.stages = env_st;
    TmaMaps maps;
    if (!make_btm_tensor_map(&maps.m[0], a.input, a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = 1; i < 5; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, V>(1, pc);
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = a.spikes_u8 ? (a.v_mem ? lif_fwd_tma_kernel<RESET, NW, V, UNI, false, uint8_t, true>
                                       : lif_fwd_tma_kernel<RESET, NW, V, UNI, false, uint8_t, false>)
                : a.ckpt    ? lif_fwd_tma_kernel<RESET, NW, V, UNI, false, float, false, true>
                : !a.v_mem  ? lif_fwd_tma_kernel<RESET, NW, V, UNI, false, float, false>
                : a.v_post  ? lif_fwd_tma_kernel<RESET, NW, V, UNI, true, float, true>
                            : lif_fwd_tma_kernel<RESET, NW, V, UNI, false, float, true>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, pc);
    *used = true;
    return cudaPeekAtLastError();
}

cudaError_t launch_lif_forward_tma(const LifFwdArgs &a, int reset_mode, cudaStream_t s, bool *used)
{
    *used = false;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.input) || (a.v_post && !aligned16(a.v_post))) return cudaSuccess;
    if (a.spikes_u8) {      // compact raster: no float raster, v_mem optional, no post-reset record
        if (!aligned16(a.spikes_u8) || (a.v_mem && !aligned16(a.v_mem)) || a.v_post || a.ckpt) return cudaSuccess;
    } else if (a.ckpt) {    // checkpoints instead of v_mem
        if (!aligned16(a.spikes) || !aligned16(a.ckpt) || a.v_mem || a.v_post) return cudaSuccess;
    } else if (!a.v_mem) {  // spikes only: a forward pass that is neither differentiated nor recorded
        if (!aligned16(a.spikes) || a.v_post) return cudaSuccess;
    } else if (!aligned16(a.spikes) || !aligned16(a.v_mem)) {
        return cudaSuccess;
    }
    const bool wide = use_wide(a.B, a.M);
    const bool uni = a.np.uniform();
    if (reset_mode == EXB_RESET_SUBTRACT) {
        if (!wide) return run_lif_fwd<EXB_RESET_SUBTRACT, NWARPS, 1, true>(a, s, used);
        return uni ? run_lif_fwd<EXB_RESET_SUBTRACT, NWARPS, 4, true>(a, s, used)
                   : run_lif_fwd<EXB_RESET_SUBTRACT, NWARPS, 4, false>(a, s, used);
    }
    if (!wide) return run_lif_fwd<EXB_RESET_TO_VALUE, NWARPS, 1, true>(a, s, used);
    return uni ? run_lif_fwd<EXB_RESET_TO_VALUE, NWARPS, 4, true>(a, s, used)
               : run_lif_fwd<EXB_RESET_TO_VALUE, NWARPS, 4, false>(a, s, used);
}

template <int NW, int V>
static cudaError_t run_leaky_fwd(const LeakyFwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    const int64_t ctas = a.B * ((a.M + G::W - 1) / G::W);
    PipeCfg pc = pipe_cfg(G::W, 1, ctas);
    long_stages_for_wide_forward(pc, V, ctas, a.T);      // 8 x 500 x 262144: 1.301 -> 1.262 ms
    TmaMaps maps;
    if (!make_btm_tensor_map(&maps.m[0], a.input, a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = 1; i < 5; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, V>(1, pc);
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = leaky_fwd_tma_kernel<NW, V>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, pc);
    *used = true;
    return cudaPeekAtLastError();
}

cudaError_t launch_leaky_forward_tma(const LeakyFwdArgs &a, cudaStream_t s, bool *used)
{
    *used = false;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.out) || !aligned16(a.input)) return cudaSuccess;
    return use_wide(a.B, a.M) ? run_leaky_fwd<NWARPS, 4>(a, s, used) : run_leaky_fwd<NWARPS, 1>(a, s, used);
}

template <bool WA, int WS, int NW, int V>
static cudaError_t run_leaky_bwd(const LeakyBwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW, V>;
    TmaMaps maps;
    const float *ptrs[5] = {a.go, nullptr, nullptr, nullptr, nullptr};
    int nmaps = 1;
    if (WA) ptrs[nmaps++] = a.out;
    if (WS) ptrs[nmaps++] = a.input;
    const PipeCfg pc = pipe_cfg(G::W, nmaps, a.B * ((a.M + G::W - 1) / G::W));
    for (int i = 0; i < nmaps; ++i)
        if (!make_btm_tensor_map(&maps.m[i], ptrs[i], a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = nmaps; i < 5; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, V>(nmaps, pc);
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = leaky_bwd_tma_kernel<WA, WS, NW, V>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, nmaps, pc);
    *used = true;
    return cudaPeekAtLastError();
}

template <bool WA, int WS>
static cudaError_t pick_leaky_bwd(const LeakyBwdArgs &a, cudaStream_t s, bool *used)
{
    return use_wide(a.B, a.M) ? run_leaky_bwd<WA, WS, NWARPS, 4>(a, s, used) : run_leaky_bwd<WA, WS, NWARPS, 1>(a, s, used);
}

cudaError_t launch_leaky_backward_tma(const LeakyBwdArgs &a, cudaStream_t s, bool *used)
{
    *used = false;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.grad_input)) return cudaSuccess;
    const bool derived = (a.scale.flags & (EXB_SCALE_ONE_MINUS_ALPHA | EXB_SCALE_TIMES_ALPHA)) != 0;
    const bool wa = a.grad_alpha != nullptr || a.acc_decay != nullptr;
    const bool ws = a.grad_scale != nullptr || (a.acc_decay != nullptr && derived);
    if (wa && ws) return pick_leaky_bwd<true, true>(a, s, used);
    if (wa) return pick_leaky_bwd<true, false>(a, s, used);
    if (ws) return pick_leaky_bwd<false, true>(a, s, used);
    return pick_leaky_bwd<false, false>(a, s, used);
}

// ---- time-parallel leaky scan ----------------------------------------------------------
constexpr int SCAN_V = 1;       // one neuron per thread: most CTAs for few neurons

// Splits T into segments so that about 8 CTAs per SM exist; false when splitting is pointless.
// The segment length is a multiple of 16 steps whatever the number of streamed tensors, so that
// forward and backward (which stream 1 to 3 tensors) agree on the scratch size; the pipeline
// chunk is the power of two <= 16 that keeps a stage near 8 KB.
constexpr int SCAN_ALIGN = 16;

static bool scan_geometry(int64_t B, int64_t T, int64_t M, int nmaps, PipeCfg *pc, ScanGeom *sg, int *tiles_m)
{
    using G = TileGeom<NWARPS, SCAN_V>;
    if (!eligible(B, T, M)) return false;
    pc->stages = 4;
    pc->tc = SCAN_ALIGN;
    while (pc->tc > 2 && pc->tc * G::W * 4 * nmaps > 8 * 1024) pc->tc /= 2;
    *tiles_m = (int)((M + G::W - 1) / G::W);
    const int64_t ntiles = B * *tiles_m;
    if (ntiles > (1 << 24)) return false;
    const int64_t want = (8 * 148 + ntiles - 1) / ntiles;
    const int64_t max_by_len = T / (4 * SCAN_ALIGN);
    int64_t nseg = want < max_by_len ? want : max_by_len;
    if (nseg > SCAN_MAX_SEGMENTS) nseg = SCAN_MAX_SEGMENTS;
    if (nseg < 2) return false;
    int64_t L = (T + nseg - 1) / nseg;
    L = (L + SCAN_ALIGN - 1) / SCAN_ALIGN * SCAN_ALIGN;
    nseg = (T + L - 1) / L;
    if (nseg < 2) return false;
    sg->nseg = (int)nseg;
    sg->L = (int)L;
    sg->ntiles = (int)ntiles;
    return true;
}

int64_t leaky_scan_workspace_bytes(int64_t B, int64_t T, int64_t M)
{
    PipeCfg pc;
    ScanGeom sg;
    int tiles_m;
    if (!scan_geometry(B, T, M, 1, &pc, &sg, &tiles_m)) return 0;
    return (int64_t)(scan_ws_words(sg.ntiles, sg.nseg, TileGeom<NWARPS, SCAN_V>::W) * 4);
}

static bool scan_workspace(void *workspace, int64_t bytes, const ScanGeom &sg, ScanWs *ws, size_t *zero_bytes)
{
    const int W = TileGeom<NWARPS, SCAN_V>::W;
    const size_t words = scan_ws_words(sg.ntiles, sg.nseg, W);
    if (!workspace || bytes < (int64_t)(words * 4) || (reinterpret_cast<uintptr_t>(workspace) & 15u)) return false;
    unsigned int *w = static_cast<unsigned int *>(workspace);
    const size_t flags = ((size_t)sg.ntiles * sg.nseg + 15) / 16 * 16;
    ws->ticket = w;
    ws->flags = w + 16;
    ws->agg = reinterpret_cast<float *>(w + 16 + flags);
    *zero_bytes = (16 + flags) * 4;
    return true;
}

cudaError_t launch_leaky_forward_scan(const LeakyFwdArgs &a, void *workspace, int64_t workspace_bytes, bool clean,
                                      cudaStream_t s, bool *used)
{
    using G = TileGeom<NWARPS, SCAN_V>;
    *used = false;
    PipeCfg pc;
    ScanGeom sg;
    int tiles_m;
    if (!aligned16(a.out) || !aligned16(a.input)) return cudaSuccess;
    if (!scan_geometry(a.B, a.T, a.M, 1, &pc, &sg, &tiles_m)) return cudaSuccess;
    ScanWs ws;
    size_t zero_bytes;
    if (!scan_workspace(workspace, workspace_bytes, sg, &ws, &zero_bytes)) return cudaSuccess;
    TmaMaps maps;
    if (!make_btm_tensor_map(&maps.m[0], a.input, a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = 1; i < 5; ++i) maps.m[i] = maps.m[0];
    const size_t smem = tma_smem_bytes<NWARPS, SCAN_V>(1, pc);
    auto kern = leaky_fwd_scan_kernel<NWARPS, SCAN_V>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    if (!clean) e = cudaMemsetAsync(workspace, 0, zero_bytes, s);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)((int64_t)sg.ntiles * sg.nseg), (NWARPS + 1) * 32, smem, s>>>(maps, a, tiles_m, pc, sg, ws);
    *used = true;
    return cudaPeekAtLastError();
}

cudaError_t launch_leaky_backward_scan(const LeakyBwdArgs &a, void *workspace, int64_t workspace_bytes, bool clean,
                                       cudaStream_t s, bool *used)
{
    using G = TileGeom<NWARPS, SCAN_V>;
    *used = false;
    if (!aligned16(a.grad_input)) return cudaSuccess;
    const bool derived = (a.scale.flags & (EXB_SCALE_ONE_MINUS_ALPHA | EXB_SCALE_TIMES_ALPHA)) != 0;
    const bool wa = a.grad_alpha != nullptr || a.acc_decay != nullptr;
    const bool ws_ = a.grad_scale != nullptr || (a.acc_decay != nullptr && derived);
    const float *ptrs[5] = {a.go, nullptr, nullptr, nullptr, nullptr};
    int nmaps = 1;
    if (wa) ptrs[nmaps++] = a.out;
    if (ws_) ptrs[nmaps++] = a.input;
    PipeCfg pc;
    ScanGeom sg;
    int tiles_m;
    if (!scan_geometry(a.B, a.T, a.M, nmaps, &pc, &sg, &tiles_m)) return cudaSuccess;
    ScanWs ws;
    size_t zero_bytes;
    if (!scan_workspace(workspace, workspace_bytes, sg, &ws, &zero_bytes)) return cudaSuccess;
    TmaMaps maps;
    for (int i = 0; i < nmaps; ++i)
        if (!make_btm_tensor_map(&maps.m[i], ptrs[i], a.B, a.T, a.M, G::BW, pc.tc)) return cudaSuccess;
    for (int i = nmaps; i < 5; ++i) maps.m[i] = maps.m[0];
    const size_t smem = tma_smem_bytes<NWARPS, SCAN_V>(nmaps, pc);
    auto kern = leaky_bwd_scan_kernel<NWARPS, SCAN_V>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    if (!clean) e = cudaMemsetAsync(workspace, 0, zero_bytes, s);
    const size_t nbytes = (size_t)(a.B * a.M) * sizeof(float);
    if (e == cudaSuccess && a.grad_alpha) e = cudaMemsetAsync(a.grad_alpha, 0, nbytes, s);
    if (e == cudaSuccess && a.grad_scale) e = cudaMemsetAsync(a.grad_scale, 0, nbytes, s);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)((int64_t)sg.ntiles * sg.nseg), (NWARPS + 1) * 32, smem, s>>>(maps, a, tiles_m, nmaps, pc, sg, ws, wa, ws_);
    *used = true;
    return cudaPeekAtLastError();
}

// ---- time-parallel leaky forward on library-owned scratch -------------------------------
// Some hosts cannot hand the library a scratch buffer: an inference server or embedded runtime
// whose whole device-memory budget was carved up at start-up, or a plug-in that lives inside
// another framework's memory pool, has nowhere to get one from once it is running, and
// allocating behind the owner's back (cudaMalloc synchronises the device and can fail or
// fragment a nearly full GPU) is exactly what such hosts forbid.  For them the scan's scratch
// lives in this fixed array, part of the library image: every GPU that loads the library
// holds these bytes until the process exits.
// EXB_STATIC_SCRATCH_BYTES (1 MiB, set in the public header) covers every shape with up to ~1300 (tile, segment) pairs.
static __device__ __align__(256) unsigned char g_static_scratch[EXB_STATIC_SCRATCH_BYTES];
static_assert(sizeof(g_static_scratch) == EXB_STATIC_SCRATCH_BYTES, "the array is what the header promises");

// Device address of the array on `device`, which must be the current device.  In host code the
// array's name is only a handle; the address a kernel can use comes from cudaGetSymbolAddress.
// Looked up once per device and remembered.
static cudaError_t static_scratch_address(int device, void **out)
{
    constexpr int MAX_DEVICES = 64;
    static void *cached[MAX_DEVICES] = {};
    static std::mutex mu;
    if (device < 0 || device >= MAX_DEVICES) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(mu);
    if (!cached[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        cached[device] = p;
    }
    *out = cached[device];
    return cudaSuccess;
}

size_t leaky_scan_static_capacity() { return sizeof(g_static_scratch); }

// Same launch as launch_leaky_forward_scan, with the library's own array as the workspace.
// `device` is the current device.  The launcher clears the ticket and the ready flags at the
// head of the array on the stream before the kernel, so whatever the previous call left there
// does not matter; the aggregates behind them are written before they are read.
cudaError_t launch_leaky_forward_scan_static(const LeakyFwdArgs &a, int device, cudaStream_t s, bool *used)
{
    *used = false;
    void *scratch = nullptr;
    cudaError_t e = static_scratch_address(device, &scratch);
    if (e != cudaSuccess) return e;
    return launch_leaky_forward_scan(a, scratch, (int64_t)sizeof(g_static_scratch), false, s, used);
}

// out[i] = (float) acc[i]; acc[i] = 0
__global__ void acc_finish_kernel(float *out, double *acc, int64_t n)
{
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        out[i] = (float)acc[i];
        acc[i] = 0.0;
    }
}

cudaError_t launch_acc_finish(float *out, double *acc, int64_t n, cudaStream_t s)
{
    if (n <= 0) return cudaSuccess;
    acc_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(out, acc, n);
    return cudaPeekAtLastError();
}

// ---- one-shot sum-allreduce of a small vector over peer memory --------------------------------------------
// For the few KB of time-constant gradients that batch-sharded ranks exchange once per step.  Every rank owns a
// slot pair (two parities) in a buffer that all ranks of the node have mapped (NVLink peer access), and a row of
// signal words per parity.  One CTA per rank: copy the local partial into the own slot, make it visible
// system-wide, store the call's epoch into every peer's signal row, wait (bounded) for every peer's epoch, then
// read all ranks' slots with plain peer loads and add them in rank order, so that every rank obtains the same
// bits.  Two parities are enough: a rank can only enter call k+2, which reuses the slots of call k, after every
// peer has signalled call k+1, which a peer does after it finished reading call k.  No multimem, no TMA.
__device__ __forceinline__ void st_release_sys(unsigned int *p, unsigned int v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ float ld_relaxed_sys(const float *p)
{
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}

constexpr int ONESHOT_MAX_RANKS = 16;

__global__ void __launch_bounds__(256) allreduce_oneshot_kernel(float *out, const float *in, const unsigned long long *buffers,
                                                                const unsigned long long *signals, int rank, int world,
                                                                int n, unsigned int epoch)
{
    __shared__ int s_ok;
    const int parity = (int)(epoch & 1u);
    float *mine = reinterpret_cast<float *>(buffers[rank]) + (size_t)parity * n;
    for (int i = threadIdx.x; i < n; i += blockDim.x) mine[i] = in[i];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        const int p = threadIdx.x;
        // announce: "rank `rank` has published call `epoch`" in peer p's row
        st_release_sys(reinterpret_cast<unsigned int *>(signals[p]) + parity * world + rank, epoch);
        // and wait for p's announcement in the own row
        const unsigned int *flag = reinterpret_cast<const unsigned int *>(signals[rank]) + parity * world + p;
        bool arrived = ld_acquire_sys(flag) == epoch;
        const uint32_t limit = c_exb_wait_limit;
        for (uint32_t i = 1; !arrived && i < limit; ++i) {
            __nanosleep(100);
            arrived = ld_acquire_sys(flag) == epoch;
        }
        if (!arrived) {
            report_timeout(EXB_STATUS_PEER_WAIT);
            s_ok = 0;
        }
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float acc = 0.0f;
        if (ok) {
            for (int p = 0; p < world; ++p)
                acc = __fadd_rn(acc, ld_relaxed_sys(reinterpret_cast<const float *>(buffers[p]) + (size_t)parity * n + i));
        } else {
            acc = NAN;      // a peer never arrived: the sum is not known
        }
        out[i] = acc;
    }
}

cudaError_t launch_allreduce_oneshot(float *out, const float *in, const unsigned long long *buffers,
                                     const unsigned long long *signals, int rank, int world, int64_t n, unsigned int epoch,
                                     cudaStream_t s)
{
    if (world < 1 || world > ONESHOT_MAX_RANKS || rank < 0 || rank >= world || n <= 0 || n > (1 << 24))
        return cudaErrorInvalidValue;
    allreduce_oneshot_kernel<<<1, 256, 0, s>>>(out, in, buffers, signals, rank, world, (int)n, epoch);
    return cudaPeekAtLastError();
}

bool tma_enabled()
{
    static const bool on = []() {
        const char *v = getenv("EXB_DISABLE_TMA");
        return !(v && v[0] == '1');
    }();
    return on;
}

// Sets the poll limit of the bounded waits of this translation unit on the current device (0 = default) and
// the diagnostic switch that keeps the scan's ready flags down.
cudaError_t set_wait_limit(unsigned int polls, bool withhold_scan_flags)
{
    cudaError_t e = set_wait_limit_here(polls);
    if (e != cudaSuccess) return e;
    const unsigned int w = withhold_scan_flags ? 1u : 0u;
    return cudaMemcpyToSymbol(c_exb_scan_withhold_flags, &w, sizeof(w));
}

// Reads and clears the status word of the current device (synchronises `stream`).
cudaError_t read_device_status(cudaStream_t s, unsigned int *out)
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
