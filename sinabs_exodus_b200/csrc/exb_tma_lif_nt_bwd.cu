// [N,T] layout, TMA-staged fused reverse-time EXODUS backward.
//
// Same shape as the TMA-staged [N,T] forward (exb_lif_nt_tma.cuh): a CTA owns 128 rows of one row class, a producer
// warp streams boxes of [32 steps x 32 rows] of every input tensor (grad_spikes, v_mem and, when present,
// grad_v_mem, the surrogate values and the forward input) through a ring of stages, walking time backwards; the four
// consumer warps -- one thread per row -- run the reverse recurrence over the 32 steps of a stage (the chunk code the
// cp.async kernels use, exb_lif_nt_chunk.cuh), overwrite the grad_spikes tile with the input gradient and hand it
// to a TMA store.  The chunk that holds a class's first steps when its rows start inside a 128-byte line (negative
// time coordinate) is stored by the warps themselves.  Per-row results (initial-state, alpha and scale gradients)
// are written per row; the in-kernel reduction into an accumulator is a feature of the time-major kernels only.
//
// Shared memory: a stage is 16 KB per streamed tensor.  Two tensors: 3 stages (96 KB, two CTAs per SM); three:
// 2 stages (96 KB); four or five: 2 stages (128-160 KB, one CTA per SM).
#include "exb_tma_common.cuh"
#include "exb_nt_tma_common.cuh"
#include "exb_lif_nt_chunk.cuh"

namespace exb {

struct NtbMaps {
    CUtensorMap in[5];     // stage order: grad_spikes, v_mem, [grad_v_mem], [surr], [input]
    CUtensorMap out;       // grad_input
};

template <int SURR, int RESET, bool WA, int WS>
__global__ void __launch_bounds__((NTT_WARPS + 1) * 32, 2)
lif_bwd_nt_tma_kernel(const __grid_constant__ NtbMaps maps, const LifBwdArgs A, const int nstages, const int ntiles,
                      const int lp, const int a_base)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the swizzle works on 1 KB atoms: every box must start on one
    float *stages = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    const int stage_floats = ntiles * NTT_STAGE;
    Ring *ring = reinterpret_cast<Ring *>(stages + (size_t)nstages * stage_floats);
    ring_init(ring, nstages, NTT_WARPS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = A.B * A.M;
    const int T = (int)A.T;
    const int cls = (int)(blockIdx.x & ((1u << lp) - 1u));        // this CTA's class
    const int blk = (int)(blockIdx.x >> lp);                      // its block of 128 rows of that class
    const int a = (a_base + cls * (T & 31)) & 31;                 // where the rows of the class start inside a line
    const int r0 = blk * NTT_ROWS;                                // first row, counted inside the class
    const int nchunks = (T + a + NTT_BOX_T - 1) / NTT_BOX_T;
    const int i_gv = A.gv ? 2 : -1;
    const int i_sl = (SURR == EXB_SURR_GENERIC) ? (2 + (A.gv ? 1 : 0)) : -1;
    const int i_xi = (WS == SCALE_GRAD_FROM_INPUT) ? (ntiles - 1) : -1;

    if (warp == NTT_WARPS) {
        if (lane == 0) {
            int s = 0;
            uint32_t par = 0u;
            int kk = 0;
            for (; kk < nchunks; ++kk) {
                const int k = nchunks - 1 - kk;
                if (kk >= nstages && !mbar_wait(smem_u32(&ring->empty[s]), par ^ 1u)) {
                    report_timeout(EXB_STATUS_EMPTY_WAIT);
                    ring->aborted = 1;
                    break;
                }
                const uint32_t bar = smem_u32(&ring->full[s]);
                mbar_arrive_expect_tx(bar, (uint32_t)(stage_floats * sizeof(float)));
                float *dst = stages + (size_t)s * stage_floats;
                // boxes (or parts) outside the tensor are filled with zeros and still count as bytes
                for (int i = 0; i < ntiles; ++i)
#pragma unroll
                    for (int w = 0; w < NTT_WARPS; ++w)
                        tma_load_3d(smem_u32(dst + i * NTT_STAGE + w * 32 * NTT_BOX_T), &maps.in[i], k * NTT_BOX_T - a, cls,
                                    r0 + w * 32, bar);
                if (++s == nstages) { s = 0; par ^= 1u; }
            }
            ring->issued = kk;
        }
    } else {
        const int64_t row = (int64_t)r0 + warp * 32 + lane;            // inside the class
        const int64_t n = cls + (row << lp);
        const bool valid = n < N;
        const int64_t nn = valid ? n : 0;
        const int64_t b = nn / A.M, m = nn - b * A.M;
        const SpikeCfg cfg = make_spike_cfg(A.maxs);
        const Neuron q = A.np.load(b, m, cfg);
        const SurrConst sc = surr_prepare<SURR>(q, A.p0, A.p1);
        const float cp = __fmul_rn(q.alpha, q.c);
        BwdState st;
        st.R = 0.0f; st.ag = 0.0f; st.sg = 0.0f; st.vnext = 0.0f;
        float Rprev = 0.0f, f0 = 0.0f;
        bool nc0 = true;
        const float glast = (A.g_last && valid) ? __ldg(A.g_last + nn) : 0.0f;
        const bool fold_last = A.g_last != nullptr;
        const int wtile = warp * 32 * NTT_BOX_T;       // this warp's quarter of a tile
        bool ok = true;
        RingPos pos = {0, 0u};
        for (int kk = 0; kk < nchunks; ++kk) {
            const int k = nchunks - 1 - kk;
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            float *set = stages + (size_t)pos.s * stage_floats + wtile;
            float *tg = set;
            const float *tv = set + NTT_STAGE;
            const float *tgv = i_gv >= 0 ? set + i_gv * NTT_STAGE : nullptr;
            const float *tsl = i_sl >= 0 ? set + i_sl * NTT_STAGE : nullptr;
            const float *txi = i_xi >= 0 ? set + i_xi * NTT_STAGE : nullptr;
            const int tb = k * NTT_BOX_T - a;          // time step of column 0 (the same for the whole CTA)
            if (tb >= 0 && tb + NTT_BOX_T < T)         // strictly inside: no guards, and not the last time step
                ntv_bwd_chunk<SURR, RESET, WA, WS, false>(tg, tv, tgv, tsl, txi, lane, tb, T, false, glast, st, Rprev, f0,
                                                          nc0, q, sc, cp, cfg);
            else
                ntv_bwd_chunk<SURR, RESET, WA, WS, true>(tg, tv, tgv, tsl, txi, lane, tb, T, fold_last, glast, st, Rprev,
                                                         f0, nc0, q, sc, cp, cfg);
            if (tb < 0) {
                // A TMA store may not start at a negative coordinate: the warp stores the granules of this chunk
                // itself, a quarter-warp per row (lane -> row it*4 + lane/8, granule lane%8).
                __syncwarp();
                const int g = lane & 7, q4 = lane >> 3;
                if (g >= (a >> 2)) {
#pragma unroll 1
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 4 + q4;
                        const int64_t gn = cls + (((int64_t)r0 + warp * 32 + r) << lp);
                        if (gn < N)
                            __stcs(reinterpret_cast<float4 *>(A.grad_input + gn * T + tb + 4 * g),
                                   *reinterpret_cast<const float4 *>(tg + ntv_off(r, g)));
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ring->empty[pos.s]));
            } else {
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_3d(&maps.out, tb, cls, r0 + warp * 32, smem_u32(tg));
                    tma_store_commit();
                    tma_store_wait_read();      // the stage may be overwritten from here on
                    mbar_arrive(smem_u32(&ring->empty[pos.s]));
                }
                __syncwarp();
            }
            pos.advance(nstages);
        }
        if (lane == 0) tma_store_wait_all();
        if (valid) {
            if (!ok) { st.R = NAN; st.ag = NAN; st.sg = NAN; }      // a wait ran out: poison the results
            if (A.grad_init) A.grad_init[n] = __fmul_rn(q.alpha, st.R);
            const float vi = A.v_init ? __ldg(A.v_init + n) : 0.0f;
            if (WA) A.grad_alpha[n] = alpha_grad_finish<RESET>(st, vi, Rprev, f0, nc0);
            if (WS) A.grad_scale[n] = scale_grad_finish<WS>(st, vi, q);
        }
    }
    ring_finish(ring, nstages);
}

template <int SURR, int RESET, bool WA, int WS>
static cudaError_t run_lif_bwd_nt(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    const int64_t N = a.B * a.M;
    const int lp = nt_class_log2(a.T);
    if (lp < 0) return cudaSuccess;
    const float *ptrs[5] = {a.go, a.v_mem, nullptr, nullptr, nullptr};
    int ntiles = 2;
    if (a.gv) ptrs[ntiles++] = a.gv;
    if (SURR == EXB_SURR_GENERIC) ptrs[ntiles++] = a.surr;
    if (WS == SCALE_GRAD_FROM_INPUT) ptrs[ntiles++] = a.input;
    // all tensors must agree on where a row starts inside its line
    const uintptr_t pos = reinterpret_cast<uintptr_t>(a.grad_input) & 127u;
    for (int i = 0; i < ntiles; ++i)
        if (!ptrs[i] || (reinterpret_cast<uintptr_t>(ptrs[i]) & 127u) != pos) return cudaSuccess;
    NtbMaps maps;
    for (int i = 0; i < ntiles; ++i)
        if (!make_nt_tensor_map(&maps.in[i], ptrs[i], N, a.T, lp)) return cudaSuccess;
    for (int i = ntiles; i < 5; ++i) maps.in[i] = maps.in[0];
    if (!make_nt_tensor_map(&maps.out, a.grad_input, N, a.T, lp)) return cudaSuccess;
    // one class per CTA: p classes x blocks of 128 rows of a class (the class index varies fastest)
    const int64_t ctas = (((N >> lp) + NTT_ROWS - 1) / NTT_ROWS) << lp;
    if (ctas > 0x7fffffffll) return cudaSuccess;
    static const int env_st = env_int("EXB_NT_TMA_BWD_STAGES", 0);
    const int nstages = (env_st >= 2 && env_st <= 6) ? env_st : (ntiles == 2 ? 3 : 2);
    const size_t smem = (size_t)nstages * ntiles * NTT_STAGE * sizeof(float) + sizeof(Ring) + 1024 + 128;
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = lif_bwd_nt_tma_kernel<SURR, RESET, WA, WS>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)ctas, (NTT_WARPS + 1) * 32, smem, s>>>(maps, a, nstages, ntiles, lp, (int)(pos >> 2));
    *used = true;
    return cudaPeekAtLastError();
}

template <int SURR, int RESET>
static cudaError_t flags_lif_bwd_nt(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    const bool wa = a.grad_alpha != nullptr;
    const int ws = a.grad_scale ? (a.input ? SCALE_GRAD_FROM_INPUT : SCALE_GRAD_FROM_STATE) : SCALE_GRAD_NONE;
    if (wa) {
        if (ws == SCALE_GRAD_FROM_INPUT) return run_lif_bwd_nt<SURR, RESET, true, SCALE_GRAD_FROM_INPUT>(a, s, used);
        if (ws == SCALE_GRAD_FROM_STATE) return run_lif_bwd_nt<SURR, RESET, true, SCALE_GRAD_FROM_STATE>(a, s, used);
        return run_lif_bwd_nt<SURR, RESET, true, SCALE_GRAD_NONE>(a, s, used);
    }
    if (ws == SCALE_GRAD_FROM_INPUT) return run_lif_bwd_nt<SURR, RESET, false, SCALE_GRAD_FROM_INPUT>(a, s, used);
    if (ws == SCALE_GRAD_FROM_STATE) return run_lif_bwd_nt<SURR, RESET, false, SCALE_GRAD_FROM_STATE>(a, s, used);
    return run_lif_bwd_nt<SURR, RESET, false, SCALE_GRAD_NONE>(a, s, used);
}

template <int RESET>
static cudaError_t surr_lif_bwd_nt(const LifBwdArgs &a, int kind, cudaStream_t s, bool *used)
{
    switch (kind) {
    case EXB_SURR_GENERIC: return flags_lif_bwd_nt<EXB_SURR_GENERIC, RESET>(a, s, used);
    case EXB_SURR_SINGLE_EXPONENTIAL: return flags_lif_bwd_nt<EXB_SURR_SINGLE_EXPONENTIAL, RESET>(a, s, used);
    case EXB_SURR_HEAVISIDE: return flags_lif_bwd_nt<EXB_SURR_HEAVISIDE, RESET>(a, s, used);
    default: return flags_lif_bwd_nt<EXB_SURR_PERIODIC_EXPONENTIAL, RESET>(a, s, used);
    }
}

cudaError_t launch_lif_backward_nt_tma(const LifBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used)
{
    *used = false;
    static const bool off = env_int("EXB_DISABLE_NT_TMA", 0) == 1;
    if (off || a.acc_decay) return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? surr_lif_bwd_nt<EXB_RESET_SUBTRACT>(a, surr_kind, s, used)
                                            : surr_lif_bwd_nt<EXB_RESET_TO_VALUE>(a, surr_kind, s, used);
}

cudaError_t set_wait_limit_lif_nt_bwd(unsigned int polls) { return set_wait_limit_here(polls); }

// Status word of this translation unit (see read_device_status).
cudaError_t read_device_status_lif_nt_bwd(cudaStream_t s, unsigned int *out)
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
