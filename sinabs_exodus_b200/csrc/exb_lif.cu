// Spiking-neuron kernels: forward spike scan and fused reverse-time EXODUS
// backward.  This file holds the [N,T]-layout kernels and the launchers of both
// layouts; the time-major (B,T,M) kernels are in exb_tma_*.cu (TMA-staged) and
// exb_ring.cuh (cp.async rings, for shapes a TMA box cannot describe).
//
// In every kernel one thread owns a neuron (or a few adjacent ones) and walks
// through time; the membrane state, spike count and all gradient accumulators
// live in registers for the whole sweep.
//
// [N,T] kernels: one warp owns 32 neurons; 32x32 tiles are moved between
// global memory (coalesced along time) and shared memory (read along neurons),
// so the same per-thread sweep runs on a transposed tile.
#include "exb_kernels.cuh"
#include "exb_lif_nt_chunk.cuh"

namespace exb {

// ===========================================================================
// [N,T] layout: warp-private tiles of 32 rows (neurons) x 32 time steps, padded to 33 columns
// ===========================================================================
// A row of this layout starts wherever n*T*4 bytes falls, in general not on a 128-byte line.
// Chunks cut at fixed time steps would then straddle lines: every 128-byte piece of a row would
// touch five 32-byte sectors instead of four and write two of them partially (measured on B200:
// 2.2 TB/s for T = 300 against 4.8 TB/s for line-aligned pieces).  So every row gets its own
// chunk boundaries, on the 128-byte lines of the output tensor: with `a` the position of the
// row's first element inside its line (in floats), chunk k of that row covers the time steps
// [32k - a, 32k - a + 32) that fall inside [0, T).  The lanes of a warp own one row each during
// the recurrence, which is sequential per row anyway, so the rows need not be in step.
constexpr int TSTR = 33;
constexpr int TILE_FLOATS = TILE * TSTR;
constexpr int NT_WARPS = 4;

// Position (in floats) of element (n, 0) of an [N,T] tensor inside its 128-byte line.
__device__ __forceinline__ int line_pos(const void *base, int64_t n, int64_t T)
{
    return (int)(((reinterpret_cast<uintptr_t>(base) >> 2) + (uint64_t)(n * T)) & (TILE - 1));
}

__device__ __forceinline__ int nt_chunks(int64_t T) { return (int)((T + 2 * TILE - 2) / TILE); }

// Chunk k of the 32 rows from row n0 on: lane j moves element j of every row's chunk.  `a0` is
// line_pos of row n0; `src` points at element (n0, 0).
__device__ __forceinline__ void tile_prefetch(float *tile, const float *src, int64_t T, int rows, int k, int a0, int lane)
{
    const unsigned dst = (unsigned)__cvta_generic_to_shared(tile + lane);
    const int step = (int)(T & (TILE - 1));
    int a = a0;
#pragma unroll 8
    for (int r = 0; r < rows; ++r) {
        const int64_t t = (int64_t)k * TILE - a + lane;
        if (t >= 0 && t < T)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + r * TSTR * 4), "l"(src + r * T + t) : "memory");
        a = (a + step) & (TILE - 1);
    }
}

__device__ __forceinline__ void prefetch_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

template <int PENDING>
__device__ __forceinline__ void prefetch_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory");
}

__device__ __forceinline__ void tile_store(float *dst, const float *tile, int64_t T, int rows, int k, int a0, int lane)
{
    const int step = (int)(T & (TILE - 1));
    int a = a0;
#pragma unroll 8
    for (int r = 0; r < rows; ++r) {
        const int64_t t = (int64_t)k * TILE - a + lane;
        if (t >= 0 && t < T) __stcs(dst + r * T + t, tile[r * TSTR + lane]);
        a = (a + step) & (TILE - 1);
    }
}

template <int RESET>
__global__ void __launch_bounds__(NT_WARPS * 32) lif_fwd_nt_kernel(const LifFwdArgs A)
{
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = A.B * A.M, T = A.T;
    const int64_t n0 = (blockIdx.x * (int64_t)NT_WARPS + warp) * TILE;
    if (n0 >= N) return;   // whole warp leaves together
    float *tbuf = smem + warp * (3 * TILE_FLOATS);     // two input tiles (double buffer) + one spike tile
    float *ts = tbuf + 2 * TILE_FLOATS;
    const int rows = (int)min((int64_t)TILE, N - n0);
    const bool valid = lane < rows;
    const int64_t n = valid ? n0 + lane : n0;
    const int64_t b = n / A.M, m = n - b * A.M;
    const SpikeCfg cfg = make_spike_cfg(A.maxs);
    const Neuron q = A.np.load(b, m, cfg);
    float v = A.v_init ? __ldg(A.v_init + n) : 0.0f;
    float af = 0.0f;
    SpikeTotal cnt;
    cnt.c32 = 0u; cnt.c64 = 0ull;

    const int a0 = line_pos(A.spikes, n0, T);          // chunk boundaries follow the outputs' lines
    const int a = line_pos(A.spikes, n, T);            // this lane's own row
    const int nchunks = nt_chunks(T);
    const float *src = A.input + n0 * T;
    tile_prefetch(tbuf, src, T, rows, 0, a0, lane);
    prefetch_commit();
    int cur = 0;
    for (int k = 0; k < nchunks; ++k, cur ^= 1) {
        float *tx = tbuf + cur * TILE_FLOATS;
        if (k + 1 < nchunks) {
            tile_prefetch(tbuf + (cur ^ 1) * TILE_FLOATS, src, T, rows, k + 1, a0, lane);
            prefetch_commit();
            prefetch_wait<1>();
        } else {
            prefetch_wait<0>();
        }
        __syncwarp();
        if (valid) {
            const int64_t tb = (int64_t)k * TILE - a;   // time step of column 0
            const int j_lo = tb < 0 ? (int)-tb : 0;
            const int j_hi = (int)min((int64_t)TILE, T - tb);
            for (int j = j_lo; j < j_hi; ++j) {
                lif_step<RESET>(v, af, tx[lane * TSTR + j], q, cfg, cnt);
                ts[lane * TSTR + j] = af;
                tx[lane * TSTR + j] = v;
            }
        }
        __syncwarp();
        tile_store(A.spikes + n0 * T, ts, T, rows, k, a0, lane);
        tile_store(A.v_mem + n0 * T, tx, T, rows, k, a0, lane);
        __syncwarp();
    }
    if (A.v_post_last && valid) A.v_post_last[n] = post_reset<RESET>(v, af, q);
    if (A.spike_count) {
        const unsigned long long tot = warp_sum_u64(valid ? cnt.total(cfg) : 0ull);
        if (lane == 0 && tot) atomicAdd(A.spike_count, tot);
    }
}

template <int SURR, int RESET, bool WA, int WS>
__global__ void __launch_bounds__(NT_WARPS * 32) lif_bwd_nt_kernel(const LifBwdArgs A, int ntiles)
{
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = A.B * A.M, T = A.T;
    const int64_t n0 = (blockIdx.x * (int64_t)NT_WARPS + warp) * TILE;
    if (n0 >= N) return;
    // per warp: two sets (double buffer) of `ntiles` input tiles; grad_input overwrites grad_spikes in place
    float *wbase = smem + warp * (2 * ntiles * TILE_FLOATS);
    const int i_gv = A.gv ? 2 : -1;
    const int i_sl = (SURR == EXB_SURR_GENERIC) ? (2 + (A.gv ? 1 : 0)) : -1;
    const int i_xi = (WS == SCALE_GRAD_FROM_INPUT) ? (ntiles - 1) : -1;

    const int rows = (int)min((int64_t)TILE, N - n0);
    const bool valid = lane < rows;
    const int64_t n = valid ? n0 + lane : n0;
    const int64_t b = n / A.M, m = n - b * A.M;
    const SpikeCfg cfg = make_spike_cfg(A.maxs);
    const Neuron q = A.np.load(b, m, cfg);
    const SurrConst sc = surr_prepare<SURR>(q, A.p0, A.p1);
    const float cp = __fmul_rn(q.alpha, q.c);
    BwdState st;
    st.R = 0.0f; st.ag = 0.0f; st.sg = 0.0f; st.vnext = 0.0f;
    float Rprev = 0.0f, f0 = 0.0f;
    bool nc0 = true;
    const float glast = (A.g_last && valid) ? __ldg(A.g_last + n) : 0.0f;

    const int a0 = line_pos(A.grad_input, n0, T);      // chunk boundaries follow the output's lines
    const int a = line_pos(A.grad_input, n, T);        // this lane's own row
    const int nchunks = nt_chunks(T);
    const int64_t off = n0 * T;

    // one commit group per set of tiles: the waits below count sets
    auto prefetch_set = [&](float *set, int k) {
        const float *srcs[5] = {A.go + off, A.v_mem + off, i_gv >= 0 ? A.gv + off : nullptr,
                                i_sl >= 0 ? A.surr + off : nullptr, i_xi >= 0 ? A.input + off : nullptr};
        const int slots[5] = {0, 1, i_gv, i_sl, i_xi};
#pragma unroll
        for (int i = 0; i < 5; ++i) {
            if (slots[i] < 0) continue;
            tile_prefetch(set + slots[i] * TILE_FLOATS, srcs[i], T, rows, k, a0, lane);
        }
        prefetch_commit();
    };

    prefetch_set(wbase, nchunks - 1);
    int cur = 0;
    for (int k = nchunks - 1; k >= 0; --k, cur ^= 1) {
        float *set = wbase + cur * (ntiles * TILE_FLOATS);
        float *tg = set, *tv = set + TILE_FLOATS;
        const float *tgv = i_gv >= 0 ? set + i_gv * TILE_FLOATS : nullptr;
        const float *tsl = i_sl >= 0 ? set + i_sl * TILE_FLOATS : nullptr;
        const float *txi = i_xi >= 0 ? set + i_xi * TILE_FLOATS : nullptr;
        if (k > 0) {
            prefetch_set(wbase + (cur ^ 1) * (ntiles * TILE_FLOATS), k - 1);
            prefetch_wait<1>();
        } else {
            prefetch_wait<0>();
        }
        __syncwarp();
        if (valid) {
            const int64_t tb = (int64_t)k * TILE - a;   // time step of column 0
            const int j_lo = tb < 0 ? (int)-tb : 0;
            const int j_hi = (int)min((int64_t)TILE, T - tb);
            for (int j = j_hi - 1; j >= j_lo; --j) {
                const int i = lane * TSTR + j;
                float go = tg[i], gv = tgv ? tgv[i] : 0.0f;
                const float v = tv[i];
                if (A.g_last && tb + j == T - 1) fold_last_state_grad<RESET>(go, gv, glast, v, q, cfg);
                Rprev = st.R;
                const float Rt = lif_bwd_step<SURR, RESET, WA, WS>(st, v, go, gv, (SURR == EXB_SURR_GENERIC) ? tsl[i] : 0.0f,
                                                                  (WS == SCALE_GRAD_FROM_INPUT) ? txi[i] : 0.0f, q, sc, cp, cfg, f0, nc0);
                tg[i] = __fmul_rn(q.scale, Rt);
            }
        }
        __syncwarp();
        tile_store(A.grad_input + off, tg, T, rows, k, a0, lane);
        __syncwarp();
    }
    if (valid) {
        if (A.grad_init) A.grad_init[n] = __fmul_rn(q.alpha, st.R);
        const float vi = A.v_init ? __ldg(A.v_init + n) : 0.0f;
        if (WA) A.grad_alpha[n] = alpha_grad_finish<RESET>(st, vi, Rprev, f0, nc0);
        if (WS) A.grad_scale[n] = scale_grad_finish<WS>(st, vi, q);
    }
}

}  // namespace exb
#include "exb_lif_nt.cuh"
#include "exb_ring.cuh"
namespace exb {

// ===========================================================================
// launchers
// ===========================================================================
static inline bool can_vec4(int64_t M, std::initializer_list<const void *> ptrs)
{
    if (M % 4) return false;
    for (const void *p : ptrs)
        if (p && !aligned16(p)) return false;
    return true;
}

template <int RESET>
static cudaError_t launch_fwd_t(const LifFwdArgs &a, int layout, cudaStream_t s)
{
    if (layout == EXB_LAYOUT_BTM) {
        if (can_vec4(a.M, {a.spikes, a.v_mem, a.input, a.v_post})) {
            cudaError_t e = launch_ring<4>(lif_fwd_btm_ring_kernel<4, RESET>, a, 1, s);
            if (e != cudaSuccess) return e;
        } else if (can_vec2(a.M, {a.spikes, a.v_mem, a.input, a.v_post})) {
            cudaError_t e = launch_ring<2>(lif_fwd_btm_ring_kernel<2, RESET>, a, 1, s);
            if (e != cudaSuccess) return e;
        } else {
            cudaError_t e = launch_ring<1>(lif_fwd_btm_ring_kernel<1, RESET>, a, 1, s);
            if (e != cudaSuccess) return e;
        }
    } else {
        const int64_t N = a.B * a.M;
        const int64_t warps = (N + TILE - 1) / TILE;
        const unsigned grid = (unsigned)((warps + NT_WARPS - 1) / NT_WARPS);
        const bool vec = ntv_eligible(a.T, a.spikes, {a.v_mem, a.input});
        const size_t sm = (size_t)NT_WARPS * 3 * (vec ? NTV_TILE_FLOATS : TILE_FLOATS) * sizeof(float);
        auto kern = vec ? lif_fwd_ntv_kernel<RESET> : lif_fwd_nt_kernel<RESET>;
        if (sm > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            if (e != cudaSuccess) return e;
        }
        kern<<<grid, NT_WARPS * 32, sm, s>>>(a);
    }
    return cudaPeekAtLastError();
}

cudaError_t launch_lif_forward(const LifFwdArgs &a, int layout, int reset_mode, cudaStream_t s)
{
    if (layout == EXB_LAYOUT_BTM && tma_enabled()) {
        bool used = false;
        cudaError_t e = launch_lif_forward_tma(a, reset_mode, s, &used);
        if (e != cudaSuccess || used) return e;
    }
    if (layout == EXB_LAYOUT_NT && tma_enabled()) {
        bool used = false;
        cudaError_t e = launch_lif_forward_nt_tma(a, reset_mode, s, &used);
        if (e != cudaSuccess || used) return e;
    }
    return reset_mode == EXB_RESET_SUBTRACT ? launch_fwd_t<EXB_RESET_SUBTRACT>(a, layout, s)
                                            : launch_fwd_t<EXB_RESET_TO_VALUE>(a, layout, s);
}

template <int SURR, int RESET, bool WA, int WS>
static cudaError_t launch_bwd_t(const LifBwdArgs &a, int layout, cudaStream_t s)
{
    if (layout == EXB_LAYOUT_BTM) {
        if (can_vec4(a.M, {a.grad_input, a.go, a.gv, a.v_mem, a.surr, a.input})) {
            const int nt4 = 2 + (a.gv ? 1 : 0) + (SURR == EXB_SURR_GENERIC ? 1 : 0) + (WS == SCALE_GRAD_FROM_INPUT ? 1 : 0);
            cudaError_t e = launch_ring<4>(lif_bwd_btm_ring_kernel<4, SURR, RESET, WA, WS>, a, nt4, s);
            if (e != cudaSuccess) return e;
        } else {
            const int nt = 2 + (a.gv ? 1 : 0) + (SURR == EXB_SURR_GENERIC ? 1 : 0) + (WS == SCALE_GRAD_FROM_INPUT ? 1 : 0);
            cudaError_t e = can_vec2(a.M, {a.grad_input, a.go, a.gv, a.v_mem, a.surr, a.input})
                                ? launch_ring<2>(lif_bwd_btm_ring_kernel<2, SURR, RESET, WA, WS>, a, nt, s)
                                : launch_ring<1>(lif_bwd_btm_ring_kernel<1, SURR, RESET, WA, WS>, a, nt, s);
            if (e != cudaSuccess) return e;
        }
    } else {
        const int64_t N = a.B * a.M;
        const int64_t warps = (N + TILE - 1) / TILE;
        const int ntiles = 2 + (a.gv ? 1 : 0) + (SURR == EXB_SURR_GENERIC ? 1 : 0) + (WS == SCALE_GRAD_FROM_INPUT ? 1 : 0);
        const bool vec = ntv_eligible(a.T, a.grad_input, {a.go, a.v_mem, a.gv, a.surr, a.input});
        const size_t sm = (size_t)NT_WARPS * 2 * ntiles * (vec ? NTV_TILE_FLOATS : TILE_FLOATS) * sizeof(float);
        auto kern = vec ? lif_bwd_ntv_kernel<SURR, RESET, WA, WS> : lif_bwd_nt_kernel<SURR, RESET, WA, WS>;
        if (sm > 48 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
            if (e != cudaSuccess) return e;
        }
        kern<<<(unsigned)((warps + NT_WARPS - 1) / NT_WARPS), NT_WARPS * 32, sm, s>>>(a, ntiles);
    }
    return cudaPeekAtLastError();
}

template <int SURR, int RESET>
static cudaError_t launch_bwd_flags(const LifBwdArgs &a, int layout, cudaStream_t s)
{
    const bool wa = a.grad_alpha != nullptr;
    const int ws = a.grad_scale ? (a.input ? SCALE_GRAD_FROM_INPUT : SCALE_GRAD_FROM_STATE) : SCALE_GRAD_NONE;
    if (wa) {
        if (ws == SCALE_GRAD_FROM_INPUT) return launch_bwd_t<SURR, RESET, true, SCALE_GRAD_FROM_INPUT>(a, layout, s);
        if (ws == SCALE_GRAD_FROM_STATE) return launch_bwd_t<SURR, RESET, true, SCALE_GRAD_FROM_STATE>(a, layout, s);
        return launch_bwd_t<SURR, RESET, true, SCALE_GRAD_NONE>(a, layout, s);
    }
    if (ws == SCALE_GRAD_FROM_INPUT) return launch_bwd_t<SURR, RESET, false, SCALE_GRAD_FROM_INPUT>(a, layout, s);
    if (ws == SCALE_GRAD_FROM_STATE) return launch_bwd_t<SURR, RESET, false, SCALE_GRAD_FROM_STATE>(a, layout, s);
    return launch_bwd_t<SURR, RESET, false, SCALE_GRAD_NONE>(a, layout, s);
}

template <int RESET>
static cudaError_t launch_bwd_surr(const LifBwdArgs &a, int layout, int surr_kind, cudaStream_t s)
{
    switch (surr_kind) {
    case EXB_SURR_GENERIC: return launch_bwd_flags<EXB_SURR_GENERIC, RESET>(a, layout, s);
    case EXB_SURR_SINGLE_EXPONENTIAL: return launch_bwd_flags<EXB_SURR_SINGLE_EXPONENTIAL, RESET>(a, layout, s);
    case EXB_SURR_HEAVISIDE: return launch_bwd_flags<EXB_SURR_HEAVISIDE, RESET>(a, layout, s);
    default: return launch_bwd_flags<EXB_SURR_PERIODIC_EXPONENTIAL, RESET>(a, layout, s);
    }
}

cudaError_t launch_lif_backward(const LifBwdArgs &a, int layout, int reset_mode, int surr_kind, cudaStream_t s)
{
    if (layout == EXB_LAYOUT_BTM && tma_enabled()) {
        bool used = false;
        cudaError_t e = launch_lif_backward_tma(a, reset_mode, surr_kind, s, &used);
        if (e != cudaSuccess || used) return e;
    }
    if (a.acc_decay) return cudaErrorNotSupported;      // only the time-major TMA-staged kernels reduce in the kernel
    if (layout == EXB_LAYOUT_NT && tma_enabled()) {
        bool used = false;
        cudaError_t e = launch_lif_backward_nt_tma(a, reset_mode, surr_kind, s, &used);
        if (e != cudaSuccess || used) return e;
    }
    return reset_mode == EXB_RESET_SUBTRACT ? launch_bwd_surr<EXB_RESET_SUBTRACT>(a, layout, surr_kind, s)
                                            : launch_bwd_surr<EXB_RESET_TO_VALUE>(a, layout, surr_kind, s);
}

}  // namespace exb
