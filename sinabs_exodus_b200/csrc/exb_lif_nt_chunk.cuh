// [N,T] layout: what the cp.async kernels (exb_lif_nt.cuh) and the TMA-staged kernels share -- the swizzled
// 32 x 32 tile of one warp and the reverse recurrence over one chunk of it.
//
// Tile: 32 rows x 32 floats, unpadded; the 16-byte granule g of row r is stored at granule position g ^ (r & 7).
// This is the placement of TMA's 128-byte swizzle for tiles that start on 1 KB boundaries, and it keeps both access
// patterns free of bank conflicts with 16-byte accesses: copies touch the eight granules of one row per
// quarter-warp, the recurrence touches the same granule of eight consecutive rows per quarter-warp.
#pragma once

#include "exb_kernels.cuh"

namespace exb {

constexpr int TILE = 32;

__device__ __forceinline__ int ntv_off(int r, int g) { return r * TILE + ((g ^ (r & 7)) << 2); }

// Reverse recurrence of one lane's row over one chunk; grad_input overwrites grad_spikes in place.
template <int SURR, int RESET, bool WA, int WS, bool GUARD>
__device__ __forceinline__ void ntv_bwd_chunk(float *tg, const float *tv, const float *tgv, const float *tsl,
                                              const float *txi, int lane, int tb, int T, bool fold_last, float glast,
                                              BwdState &st, float &Rprev, float &f0, bool &nc0, const Neuron &q,
                                              const SurrConst &sc, float cp, const SpikeCfg &cfg)
{
    // one granule ahead, for the same reason as in the forward chunk
    float4 go_n = *reinterpret_cast<const float4 *>(tg + ntv_off(lane, 7));
    float4 v_n = *reinterpret_cast<const float4 *>(tv + ntv_off(lane, 7));
#pragma unroll
    for (int g = 7; g >= 0; --g) {
        const int o = ntv_off(lane, g);
        const float4 go4 = go_n, v4 = v_n;
        float4 gv4 = make_float4(0.f, 0.f, 0.f, 0.f), sl4 = gv4, xi4 = gv4;
        if (tgv) gv4 = *reinterpret_cast<const float4 *>(tgv + o);
        if (SURR == EXB_SURR_GENERIC) sl4 = *reinterpret_cast<const float4 *>(tsl + o);
        if (WS == SCALE_GRAD_FROM_INPUT) xi4 = *reinterpret_cast<const float4 *>(txi + o);
        if (g > 0) {
            go_n = *reinterpret_cast<const float4 *>(tg + ntv_off(lane, g - 1));
            v_n = *reinterpret_cast<const float4 *>(tv + ntv_off(lane, g - 1));
        }
        float go[4] = {go4.x, go4.y, go4.z, go4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
        float gv[4] = {gv4.x, gv4.y, gv4.z, gv4.w}, sl[4] = {sl4.x, sl4.y, sl4.z, sl4.w};
        float xi[4] = {xi4.x, xi4.y, xi4.z, xi4.w};
        float r[4];
#pragma unroll
        for (int e = 3; e >= 0; --e) {
            const int t = tb + 4 * g + e;
            r[e] = 0.0f;
            if (GUARD && (unsigned)t >= (unsigned)T) continue;
            if (fold_last && t == T - 1) fold_last_state_grad<RESET>(go[e], gv[e], glast, vv[e], q, cfg);
            Rprev = st.R;
            const float Rt = lif_bwd_step<SURR, RESET, WA, WS>(st, vv[e], go[e], gv[e], sl[e], xi[e], q, sc, cp, cfg, f0, nc0);
            r[e] = __fmul_rn(q.scale, Rt);
        }
        *reinterpret_cast<float4 *>(tg + o) = make_float4(r[0], r[1], r[2], r[3]);
    }
}

}  // namespace exb
