// [N,T] layout, fast variant: 16-byte pieces between global and shared memory.
//
// A warp owns 32 rows (neurons) and walks time in chunks of 32 steps.  The chunk boundaries of
// every row lie on the 128-byte lines of the output tensor (see line_pos in exb_lif.cu), so a
// row's chunk is exactly one aligned line: eight 16-byte granules.  One warp instruction moves
// four such lines (lane -> row it*4 + lane/8, granule lane%8), a quarter of the instructions
// of the 4-byte variant, which was bound by instruction issue.
//
// Shared-memory tile: 32 rows x 32 floats, unpadded; granule g of row r is stored at granule
// position g ^ (r & 7).  Both access patterns are then free of bank conflicts with 16-byte
// accesses: the copy phases touch the eight granules of one row per quarter-warp, the
// recurrence touches the same granule of eight consecutive rows per quarter-warp.
//
// Row heads and tails (time steps outside [0,T) inside a line belong to the neighbouring rows)
// are moved element by element.  Needs every tensor's base address congruent to the output's
// modulo 16 bytes and T <= 2^25; the launcher falls back to the 4-byte variant otherwise.
#pragma once

namespace exb {

constexpr int NTV_TILE_FLOATS = TILE * TILE;   // unpadded


// What one lane moves in the copy phases: granule lane%8 of rows it*4 + lane/8, it = 0..7.
// Everything that does not depend on the chunk is kept here, so a copy costs a handful of
// instructions per granule: with kb = 32*k, the granule's first time step is kb + c[it] and its
// element offset from the warp's first row is kb + off[it].
struct NtvLane {
    int c[8];      // 4*g - (position of the row's first element in its line); far negative for rows past the end
    int off[8];    // r*T + c
    int sm0, sm1;  // tile offset (floats) of this lane's granule for even / odd `it`, without the it*128 term
};

__device__ __forceinline__ NtvLane ntv_lane(int lane, int a0, int T, int rows)
{
    NtvLane L;
    const int step = T & (TILE - 1);
    const int q = lane >> 3, g = lane & 7;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int r = it * 4 + q;
        const int ar = (a0 + r * step) & (TILE - 1);
        L.c[it] = (r < rows) ? 4 * g - ar : -(1 << 30);
        L.off[it] = r * T + 4 * g - ar;
    }
    L.sm0 = q * TILE + ((g ^ q) << 2);
    L.sm1 = q * TILE + ((g ^ (q | 4)) << 2);
    return L;
}

__device__ __forceinline__ void ntv_prefetch(float *tile, const float *src, int T, int kb, const NtvLane &L)
{
    const unsigned base = (unsigned)__cvta_generic_to_shared(tile);
    const unsigned tm3 = (unsigned)max(T - 3, 0);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int t0 = kb + L.c[it];
        const float *gp = src + (kb + L.off[it]);
        const unsigned dst = base + 4u * (unsigned)(((it & 1) ? L.sm1 : L.sm0) + it * 4 * TILE);
        if ((unsigned)t0 < tm3) {
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gp) : "memory");
        } else if (t0 > -4 && t0 < T) {
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if ((unsigned)(t0 + e) < (unsigned)T)
                    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 4u * e), "l"(gp + e) : "memory");
        }
    }
}

__device__ __forceinline__ void ntv_store(float *dst, const float *tile, int T, int kb, const NtvLane &L)
{
    const unsigned tm3 = (unsigned)max(T - 3, 0);
    float4 val[8];
#pragma unroll
    for (int it = 0; it < 8; ++it)
        val[it] = *reinterpret_cast<const float4 *>(tile + ((it & 1) ? L.sm1 : L.sm0) + it * 4 * TILE);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int t0 = kb + L.c[it];
        float *gp = dst + (kb + L.off[it]);
        if ((unsigned)t0 < tm3) {
            __stcs(reinterpret_cast<float4 *>(gp), val[it]);
        } else if (t0 > -4 && t0 < T) {
            const float e4[4] = {val[it].x, val[it].y, val[it].z, val[it].w};
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if ((unsigned)(t0 + e) < (unsigned)T) __stcs(gp + e, e4[e]);
        }
    }
}

// Forward recurrence of one lane's row over one chunk.  GUARD: the chunk holds time steps
// outside [0,T) for this row (first and last chunk only).
template <int RESET, bool GUARD>
__device__ __forceinline__ void ntv_fwd_chunk(float *tx, float *ts, int lane, int tb, int T, float &v, float &af,
                                              const Neuron &q, const SpikeCfg &cfg, SpikeTotal &cnt)
{
    // the next granule is read before this one's results are written: the compiler cannot tell that
    // the two do not alias and would otherwise serialise a shared-memory round trip per granule
    float4 xn = *reinterpret_cast<const float4 *>(tx + ntv_off(lane, 0));
#pragma unroll(GUARD ? 1 : 8)   // the guarded variant runs twice per row: keep its code small
    for (int g = 0; g < 8; ++g) {
        const int o = ntv_off(lane, g);
        const float4 x4 = xn;
        if (g < 7) xn = *reinterpret_cast<const float4 *>(tx + ntv_off(lane, g + 1));
        float x[4] = {x4.x, x4.y, x4.z, x4.w};
        float s[4], u[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (!GUARD || (unsigned)(tb + 4 * g + e) < (unsigned)T) lif_step<RESET>(v, af, x[e], q, cfg, cnt);
            s[e] = af;
            u[e] = v;
        }
        *reinterpret_cast<float4 *>(ts + o) = make_float4(s[0], s[1], s[2], s[3]);
        *reinterpret_cast<float4 *>(tx + o) = make_float4(u[0], u[1], u[2], u[3]);
    }
}

template <int RESET>
__global__ void __launch_bounds__(NT_WARPS * 32) lif_fwd_ntv_kernel(const LifFwdArgs A)
{
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = A.B * A.M;
    const int T = (int)A.T;
    const int64_t n0 = (blockIdx.x * (int64_t)NT_WARPS + warp) * TILE;
    if (n0 >= N) return;   // whole warp leaves together
    float *tbuf = smem + warp * (3 * NTV_TILE_FLOATS);   // two input tiles (double buffer) + one spike tile
    float *ts = tbuf + 2 * NTV_TILE_FLOATS;
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

    const int a0 = line_pos(A.spikes, n0, A.T);
    const int a = line_pos(A.spikes, n, A.T);
    const NtvLane L = ntv_lane(lane, a0, T, rows);
    const int nchunks = nt_chunks(A.T);
    const float *src = A.input + n0 * A.T;
    ntv_prefetch(tbuf, src, T, 0, L);
    prefetch_commit();
    int cur = 0;
    for (int k = 0; k < nchunks; ++k, cur ^= 1) {
        float *tx = tbuf + cur * NTV_TILE_FLOATS;
        if (k + 1 < nchunks) {
            ntv_prefetch(tbuf + (cur ^ 1) * NTV_TILE_FLOATS, src, T, (k + 1) * TILE, L);
            prefetch_commit();
            prefetch_wait<1>();
        } else {
            prefetch_wait<0>();
        }
        __syncwarp();
        if (valid) {
            const int tb = k * TILE - a;   // time step of column 0
            if (tb >= 0 && tb + TILE <= T) ntv_fwd_chunk<RESET, false>(tx, ts, lane, tb, T, v, af, q, cfg, cnt);
            else ntv_fwd_chunk<RESET, true>(tx, ts, lane, tb, T, v, af, q, cfg, cnt);
        }
        __syncwarp();
        ntv_store(A.spikes + n0 * A.T, ts, T, k * TILE, L);
        ntv_store(A.v_mem + n0 * A.T, tx, T, k * TILE, L);
        __syncwarp();
    }
    if (A.v_post_last && valid) A.v_post_last[n] = post_reset<RESET>(v, af, q);
    if (A.spike_count) {
        const unsigned long long tot = warp_sum_u64(valid ? cnt.total(cfg) : 0ull);
        if (lane == 0 && tot) atomicAdd(A.spike_count, tot);
    }
}

template <int SURR, int RESET, bool WA, int WS>
__global__ void __launch_bounds__(NT_WARPS * 32) lif_bwd_ntv_kernel(const LifBwdArgs A, int ntiles)
{
    extern __shared__ __align__(16) float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = A.B * A.M;
    const int T = (int)A.T;
    const int64_t n0 = (blockIdx.x * (int64_t)NT_WARPS + warp) * TILE;
    if (n0 >= N) return;
    // per warp: two sets (double buffer) of `ntiles` tiles
    float *wbase = smem + warp * (2 * ntiles * NTV_TILE_FLOATS);
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
    const bool fold_last = A.g_last != nullptr;

    const int a0 = line_pos(A.grad_input, n0, A.T);
    const int a = line_pos(A.grad_input, n, A.T);
    const NtvLane L = ntv_lane(lane, a0, T, rows);
    const int nchunks = nt_chunks(A.T);
    const int64_t off = n0 * A.T;

    auto prefetch_set = [&](float *set, int k) {
        const int kb = k * TILE;
        ntv_prefetch(set, A.go + off, T, kb, L);
        ntv_prefetch(set + NTV_TILE_FLOATS, A.v_mem + off, T, kb, L);
        if (i_gv >= 0) ntv_prefetch(set + i_gv * NTV_TILE_FLOATS, A.gv + off, T, kb, L);
        if (i_sl >= 0) ntv_prefetch(set + i_sl * NTV_TILE_FLOATS, A.surr + off, T, kb, L);
        if (i_xi >= 0) ntv_prefetch(set + i_xi * NTV_TILE_FLOATS, A.input + off, T, kb, L);
        prefetch_commit();
    };

    prefetch_set(wbase, nchunks - 1);
    int cur = 0;
    for (int k = nchunks - 1; k >= 0; --k, cur ^= 1) {
        float *set = wbase + cur * (ntiles * NTV_TILE_FLOATS);
        float *tg = set;
        const float *tv = set + NTV_TILE_FLOATS;
        const float *tgv = i_gv >= 0 ? set + i_gv * NTV_TILE_FLOATS : nullptr;
        const float *tsl = i_sl >= 0 ? set + i_sl * NTV_TILE_FLOATS : nullptr;
        const float *txi = i_xi >= 0 ? set + i_xi * NTV_TILE_FLOATS : nullptr;
        if (k > 0) {
            prefetch_set(wbase + (cur ^ 1) * (ntiles * NTV_TILE_FLOATS), k - 1);
            prefetch_wait<1>();
        } else {
            prefetch_wait<0>();
        }
        __syncwarp();
        if (valid) {
            const int tb = k * TILE - a;   // time step of column 0
            if (tb >= 0 && tb + TILE < T)  // strictly inside: no guards, and not the last time step
                ntv_bwd_chunk<SURR, RESET, WA, WS, false>(tg, tv, tgv, tsl, txi, lane, tb, T, false, glast, st, Rprev, f0,
                                                          nc0, q, sc, cp, cfg);
            else
                ntv_bwd_chunk<SURR, RESET, WA, WS, true>(tg, tv, tgv, tsl, txi, lane, tb, T, fold_last, glast, st, Rprev,
                                                         f0, nc0, q, sc, cp, cfg);
        }
        __syncwarp();
        ntv_store(A.grad_input + off, tg, T, k * TILE, L);
        __syncwarp();
    }
    if (valid) {
        if (A.grad_init) A.grad_init[n] = __fmul_rn(q.alpha, st.R);
        const float vi = A.v_init ? __ldg(A.v_init + n) : 0.0f;
        if (WA) A.grad_alpha[n] = alpha_grad_finish<RESET>(st, vi, Rprev, f0, nc0);
        if (WS) A.grad_scale[n] = scale_grad_finish<WS>(st, vi, q);
    }
}

// All tensors share the output's position inside a 16-byte granule, and T fits the int arithmetic.
static inline bool ntv_eligible(int64_t T, const void *ref, std::initializer_list<const void *> others)
{
    if (T > (1ll << 25)) return false;   // 32 rows of T floats are addressed with int offsets
    const uintptr_t r = reinterpret_cast<uintptr_t>(ref) & 15u;
    for (const void *p : others)
        if (p && (reinterpret_cast<uintptr_t>(p) & 15u) != r) return false;
    return true;
}

}  // namespace exb
